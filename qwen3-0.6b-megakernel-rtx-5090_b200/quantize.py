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


# ----------------------------------------------------------------------------- NVFP4 (e2m1 values, block-16 scales)
E2M1_GRID = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)
E2M1_MAX = 6.0
NVFP4_BLOCK = 16


def round_to_e2m1(x: torch.Tensor) -> torch.Tensor:
    """Nearest e2m1 value (sign-magnitude, magnitudes 0, .5, 1, 1.5, 2, 3, 4, 6); ties go to the even code."""
    grid = torch.tensor(E2M1_GRID, dtype=torch.float32, device=x.device)
    mag = x.abs().clamp(max=E2M1_MAX)
    dist = (mag[..., None] - grid).abs()
    # among equally near grid points prefer the even index: subtract a tiny bonus from even codes' distance
    bonus = torch.tensor([1e-7 if i % 2 == 0 else 0.0 for i in range(8)], dtype=torch.float32, device=x.device)
    idx = (dist - bonus).argmin(dim=-1)
    return torch.sign(x) * grid[idx]


def quantize_blocks_nvfp4(w: torch.Tensor):
    """fp16/fp32 matrix ``[out, in]`` (``in`` a multiple of 16) -> (e2m1 values as fp32 ``[out, in]``,
    e4m3 block scales ``[out, in / 16]``, fp32 tensor scale).  ``w ~= tensor_scale * block_scale * value``:
    the tensor scale maps the largest block maximum onto the e4m3 range, each block scale maps its block's
    maximum onto 6 (the e2m1 maximum)."""
    wf = w.detach().to(torch.float32)
    rows, k = wf.shape
    assert k % NVFP4_BLOCK == 0
    blocks = wf.view(rows, k // NVFP4_BLOCK, NVFP4_BLOCK)
    amax = blocks.abs().amax(dim=2)
    tensor_scale = float(amax.max()) / (E2M1_MAX * E4M3_MAX)
    if tensor_scale == 0.0:
        tensor_scale = 1.0
    sb = (amax / E2M1_MAX / tensor_scale).to(torch.float8_e4m3fn)
    sbf = sb.to(torch.float32)
    denom = torch.where(sbf > 0, sbf * tensor_scale, torch.ones_like(sbf))
    vals = round_to_e2m1(blocks / denom[..., None])
    vals = torch.where(sbf[..., None] > 0, vals, torch.zeros_like(vals))
    return vals.view(rows, k), sb, tensor_scale


def dequantize_nvfp4(vals: torch.Tensor, block_scales: torch.Tensor, tensor_scale: float) -> torch.Tensor:
    rows, k = vals.shape
    sbf = block_scales.to(torch.float32)
    return (vals.view(rows, k // NVFP4_BLOCK, NVFP4_BLOCK) * (sbf * tensor_scale)[..., None]).view(rows, k)


def nvfp4_row_bytes(k: int) -> int:
    return k // 2 + k // NVFP4_BLOCK + TRAILER


def pack_rows_nvfp4(vals: torch.Tensor, block_scales: torch.Tensor, tensor_scale: float) -> torch.Tensor:
    """uint8 ``[out, in/2 + in/16 + 16]`` in the engine's NVFP4 row format: e2m1 codes two per byte (element 2i in
    the low nibble), the row's e4m3 block scales, a 16-byte trailer whose first four bytes are the fp32 tensor
    scale (``include/qwen_megakernel.h``, ``qmk_set_weight_format``)."""
    rows, k = vals.shape
    grid = torch.tensor(E2M1_GRID, dtype=torch.float32, device=vals.device)
    code = torch.searchsorted(grid, vals.abs().contiguous()).to(torch.uint8)       # exact grid values -> their index
    code = code | ((vals < 0) | ((vals == 0) & (torch.signbit(vals)))).to(torch.uint8) * 8
    out = torch.zeros(rows, nvfp4_row_bytes(k), dtype=torch.uint8, device=vals.device)
    out[:, :k // 2] = code[:, 0::2] | (code[:, 1::2] << 4)
    out[:, k // 2:k // 2 + k // NVFP4_BLOCK] = block_scales.contiguous().view(torch.uint8)
    ts = torch.tensor([tensor_scale], dtype=torch.float32, device=vals.device).view(torch.uint8)
    out[:, k // 2 + k // NVFP4_BLOCK:k // 2 + k // NVFP4_BLOCK + 4] = ts
    return out.contiguous()


def quantize_weights_nvfp4(weights: dict):
    """Reference-layout fp16 weight dict -> (engine dict with PACKED NVFP4 matrices, oracle dict with the
    dequantised fp32 matrices), embedding / LM-head tie kept - the packed counterpart of ``expand_weights_nvfp4``."""
    def both(w):
        vals, sb, ts = quantize_blocks_nvfp4(w)
        return pack_rows_nvfp4(vals, sb, ts), dequantize_nvfp4(vals, sb, ts)

    e_embed, o_embed = both(weights["embed_weight"])
    e_layers, o_layers = [], []
    for t in weights["layer_weights"]:
        if t.dim() == 2:
            p, d = both(t)
            e_layers.append(p)
            o_layers.append(d)
        else:
            e_layers.append(t)
            o_layers.append(t)
    common = dict(final_norm_weight=weights["final_norm_weight"], cos_table=weights["cos_table"],
                  sin_table=weights["sin_table"])
    return (dict(embed_weight=e_embed, lm_head_weight=e_embed, layer_weights=e_layers, **common),
            dict(embed_weight=o_embed, lm_head_weight=o_embed, layer_weights=o_layers, **common))


def _quantised_dicts(weights: dict, requant):
    """(fp16 dict holding the dequantised matrices, fp32 oracle dict) with the embedding tie kept."""
    deq_embed = requant(weights["embed_weight"])
    e_layers, o_layers = [], []
    for t in weights["layer_weights"]:
        if t.dim() == 2:
            d = requant(t)
            e_layers.append(d.to(torch.float16))
            o_layers.append(d)
        else:
            e_layers.append(t)
            o_layers.append(t)
    common = dict(final_norm_weight=weights["final_norm_weight"], cos_table=weights["cos_table"],
                  sin_table=weights["sin_table"])
    e16 = deq_embed.to(torch.float16)
    return (dict(embed_weight=e16, lm_head_weight=e16, layer_weights=e_layers, **common),
            dict(embed_weight=deq_embed, lm_head_weight=deq_embed, layer_weights=o_layers, **common))


def expand_weights_fp8(weights: dict):
    """FP8-E4M3 row-quantised weights EXPANDED to fp16 for engines without a packed-fp8 path (the tensor-core
    batched decode): same quantisation as ``quantize_weights_fp8``, stored as fp16(q * scale).  Keeps the
    numerics of the quantised model, not its memory footprint.  Returns (engine dict, oracle dict)."""
    return _quantised_dicts(weights, lambda w: dequantize_rows_fp8(*quantize_rows_fp8(w)))


def expand_weights_nvfp4(weights: dict):
    """NVFP4 (e2m1 + e4m3 block-16 scales + fp32 tensor scale) quantised weights expanded to fp16, as above."""
    return _quantised_dicts(weights, lambda w: dequantize_nvfp4(*quantize_blocks_nvfp4(w)))


def weight_bytes_nvfp4(num_layers: int = 28, vocab_size: int = 151936) -> int:
    """Bytes a packed NVFP4 model streams per decode step: 4-bit values + one e4m3 scale per 16 (norms fp16)."""
    elems = num_layers * 15_728_640 + vocab_size * 1024
    return elems // 2 + elems // 16 + num_layers * 2304 * 2 + 1024 * 2 + 4 * (7 * num_layers + 1)
