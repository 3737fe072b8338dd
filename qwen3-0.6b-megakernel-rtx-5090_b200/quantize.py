"""Weight quantisation for the FP8-E4M3 variant of the decode engine.

Scheme (the one BASELINE.json's FP8 configuration names): per output row, ``scale = max|w_row| / 448`` in
fp32, ``q = round_to_nearest_even(w / scale)`` as e4m3; activations, accumulation and the KV cache stay as they
are.  The engine's row format packs each row as ``in`` e4m3 bytes + a 16-byte trailer whose first four bytes
are the fp32 scale (``include/qwen_megakernel.h``, ``qmk_set_weight_format``), so a row and its scale travel
through the same bulk copy.  Norm vectors are left in fp16.
"""

from __future__ import annotations

import torch

E4M3_MAX = 448.0
TRAILER = 16
FIELDS_PER_LAYER = 11


def quantize_rows_fp8(w: torch.Tensor):
    """fp16/fp32 matrix ``[out, in]`` -> (e4m3 tensor ``[out, in]``, fp32 scales ``[out]``)."""
    wf = w.detach().to(torch.float32)
    scale = wf.abs().amax(dim=1) / E4M3_MAX
    scale = torch.where(scale > 0, scale, torch.ones_like(scale))
    q = (wf / scale[:, None]).to(torch.float8_e4m3fn)
    return q, scale


def dequantize_rows_fp8(q: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """The fp32 matrix the engine effectively multiplies with."""
    return q.to(torch.float32) * scale.to(torch.float32)[:, None]


def pack_rows_fp8(q: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """uint8 ``[out, in + 16]`` in the engine's row format."""
    rows, k = q.shape
    out = torch.zeros(rows, k + TRAILER, dtype=torch.uint8, device=q.device)
    out[:, :k] = q.view(torch.uint8)
    out[:, k:k + 4] = scale.to(torch.float32).contiguous().view(torch.uint8).view(rows, 4)
    return out.contiguous()


def quantize_weights_fp8(weights: dict):
    """Reference-layout fp16 weight dict -> (engine dict with packed fp8 matrices, oracle dict with the
    dequantised fp32 matrices).  Both keep the embedding / LM-head tie."""
    def both(w):
        q, s = quantize_rows_fp8(w)
        return pack_rows_fp8(q, s), dequantize_rows_fp8(q, s)

    e_embed, o_embed = both(weights["embed_weight"])
    e_layers, o_layers = [], []
    for t in weights["layer_weights"]:
        if t.dim() == 2:
            p, d = both(t)
            e_layers.append(p)
            o_layers.append(d)
        else:                       # norm vectors stay fp16
            e_layers.append(t)
            o_layers.append(t)
    common = dict(final_norm_weight=weights["final_norm_weight"], cos_table=weights["cos_table"],
                  sin_table=weights["sin_table"])
    engine = dict(embed_weight=e_embed, lm_head_weight=e_embed, layer_weights=e_layers, **common)
    oracle = dict(embed_weight=o_embed, lm_head_weight=o_embed, layer_weights=o_layers, **common)
    return engine, oracle


def weight_bytes_fp8(num_layers: int = 28, vocab_size: int = 151936) -> int:
    """Bytes one decode step reads with fp8 rows: matrices at 1 byte + 16-byte trailers, fp16 norm vectors."""
    rows_k = [(2048, 1024), (1024, 1024), (1024, 1024), (1024, 2048), (3072, 1024), (3072, 1024), (1024, 3072)]
    per_layer = sum(r * (k + TRAILER) for r, k in rows_k) + (1024 + 1024 + 128 + 128) * 2
    return num_layers * per_layer + vocab_size * (1024 + TRAILER) + 1024 * 2 + (1024 + TRAILER)
