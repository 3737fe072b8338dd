"""CPU fp32 oracle for the Qwen3-0.6B greedy decode path.  TEST INFRASTRUCTURE ONLY.

This file is the checker, never the product: only ``tests/``,
``__graft_entry__.smoke()`` and ``bench.py``'s CPU-baseline / ``--impl reference``
legs may import it.  The CUDA engine never routes through it.

PARITY UNPINNED: the reference project ships no tests, golden vectors or
known-answer fixtures for this path, and its own ``Decoder`` contains no
arithmetic (it only forwards to CUDA ops and cannot be imported without them,
``Model/Qwen06B_architecture.py:92-93``).  This file therefore restates, in plain
fp32 torch on the CPU, the arithmetic of the reference CUDA source
``Tools/megakernel/megakernel_5090.cu`` (cited per function below as ``MK:line``)
and is cross-checked against ``transformers.Qwen3ForCausalLM`` in
``tests/test_oracle.py``.  Every golden file under ``tests/golden/`` was produced
by this module (see ``tests/golden/make_golden.py``).

Semantics kept from the reference: RMSNorm eps 1e-6 everywhere (MK:84,368,418);
per-head QK-RMSNorm *before* RoPE; rotate-half RoPE with theta 1e6 sharing one
table row between element ``i`` and ``i+64`` (MK:380-393); scores scaled by
``attn_scale`` (``1/sqrt(128)``, ``Model/Qwen06B_architecture.py:212``); causal
attention over ``position+1`` cache rows (MK:893); GQA ``kv_head = q_head // 2``
(MK:490); residual adds after O-proj and down-proj; tied LM head; greedy argmax;
the EOS token is logged and generation stops after it (MK:770-788).

Rounding: the KV cache is fp16 storage in the reference (MK:392, 396-397) and in
the benchmark configuration, so the oracle rounds K (after RoPE) and V to fp16 at
the cache write and reads them back, exactly there and nowhere else
(``kv_dtype=torch.float16``, the default).  The reference additionally rounds the
residual stream, q/k/v, the attention output, the SiLU argument and the RoPE
tables to fp16 between phases; those are incidental to its kernel, and the oracle
keeps them in fp32 (weights are the fp16-rounded values, upcast), which makes it
the precision ceiling an engine is measured against.  ``kv_dtype=torch.float32``
removes the cache rounding too (used to state the size of that one effect).
"""

from __future__ import annotations

import math
from typing import List, Optional, Sequence

import torch
import torch.nn.functional as F

HIDDEN_SIZE = 1024
INTERMEDIATE_SIZE = 3072
NUM_Q_HEADS = 16
NUM_KV_HEADS = 8
HEAD_DIM = 128
Q_SIZE = NUM_Q_HEADS * HEAD_DIM
KV_SIZE = NUM_KV_HEADS * HEAD_DIM
ROPE_THETA = 1_000_000.0
RMS_EPS = 1e-6
FIELDS_PER_LAYER = 11
(IN_LN, WQ, WK, WV, Q_NORM, K_NORM, WO, POST_LN, W_GATE, W_UP, W_DOWN) = range(FIELDS_PER_LAYER)


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float = RMS_EPS) -> torch.Tensor:
    """``x * rsqrt(mean(x^2) + eps) * w`` over the last dim (MK:839-878, 625-650, 921-947)."""
    var = x.pow(2).mean(dim=-1, keepdim=True)
    return x * torch.rsqrt(var + eps) * w


def rope_angles(positions: torch.Tensor, theta: float = ROPE_THETA) -> torch.Tensor:
    """fp32 angles ``pos * theta^(-2i/128)``, i = 0..63 (Model/Qwen06B_architecture.py:126-130)."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, HEAD_DIM, 2, dtype=torch.float32) / HEAD_DIM))
    return torch.outer(positions.to(torch.float32), inv_freq)


def apply_rope(x: torch.Tensor, ang: torch.Tensor) -> torch.Tensor:
    """Rotate-half RoPE (MK:380-393).  ``x``: [T, heads, 128]; ``ang``: [T, 64]."""
    c = torch.cos(ang)[:, None, :]
    s = torch.sin(ang)[:, None, :]
    lo, hi = x[..., : HEAD_DIM // 2], x[..., HEAD_DIM // 2:]
    return torch.cat((lo * c - hi * s, lo * s + hi * c), dim=-1)


class Decoder:
    """Stateful fp32 decoder with the reference ``Decoder`` API
    (``Model/Qwen06B_architecture.py:188-448``): ``step``, ``reset``, ``position``,
    ``generate``; plus ``prefill``/``generate_ids``/``last_logits``/``trace`` for tests.
    """

    def __init__(self, weights: dict, tokenizer=None, max_seq_len: int = 2048,
                 kv_dtype: torch.dtype = torch.float16, rope_from_tables: bool = False,
                 num_threads: Optional[int] = None):
        if num_threads:
            torch.set_num_threads(num_threads)
        self.tokenizer = tokenizer
        self.max_seq_len = int(max_seq_len)
        self.kv_dtype = kv_dtype
        self.rope_from_tables = rope_from_tables
        f32 = lambda t: t.detach().to("cpu", torch.float32).contiguous()
        self.embed = f32(weights["embed_weight"])            # [V, 1024]; tied LM head
        self.final_norm = f32(weights["final_norm_weight"])
        flat = weights["layer_weights"]
        assert len(flat) % FIELDS_PER_LAYER == 0
        self.num_layers = len(flat) // FIELDS_PER_LAYER
        self.layers = []
        for li in range(self.num_layers):
            t = [f32(flat[li * FIELDS_PER_LAYER + j]) for j in range(FIELDS_PER_LAYER)]
            # fused QKV rows in the order q, k, v (MK:261-281)
            self.layers.append(dict(
                in_ln=t[IN_LN], wqkv=torch.cat((t[WQ], t[WK], t[WV]), dim=0),
                q_norm=t[Q_NORM], k_norm=t[K_NORM], wo=t[WO], post_ln=t[POST_LN],
                wgu=torch.cat((t[W_GATE], t[W_UP]), dim=0), wd=t[W_DOWN]))
        self.vocab_size = self.embed.shape[0]
        self.attn_scale = 1.0 / math.sqrt(HEAD_DIM)
        if rope_from_tables:
            self._cos = weights["cos_table"].to("cpu", torch.float32)[:, : HEAD_DIM // 2]
            self._sin = weights["sin_table"].to("cpu", torch.float32)[:, : HEAD_DIM // 2]
        self.k_cache = torch.zeros(self.num_layers, NUM_KV_HEADS, self.max_seq_len, HEAD_DIM, dtype=kv_dtype)
        self.v_cache = torch.zeros_like(self.k_cache)
        self._position = 0
        self.last_logits: Optional[torch.Tensor] = None
        self.last_normed: Optional[torch.Tensor] = None
        self.trace: Optional[dict] = None   # filled when step(..., trace=True)

    # ------------------------------------------------------------------ core
    def _rope(self, x: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        if self.rope_from_tables:
            c = self._cos[positions][:, None, :]
            s = self._sin[positions][:, None, :]
            lo, hi = x[..., : HEAD_DIM // 2], x[..., HEAD_DIM // 2:]
            return torch.cat((lo * c - hi * s, lo * s + hi * c), dim=-1)
        return apply_rope(x, rope_angles(positions))

    def _forward(self, ids: Sequence[int], want_logits: bool, trace: bool = False) -> Optional[torch.Tensor]:
        """Run ``len(ids)`` consecutive tokens starting at ``self._position``.

        One token is the reference's ``ldg_decode_body`` (MK:796-948); several
        tokens at once is the same arithmetic with a causal mask (used for
        prompts, where the reference loops token by token, MK:1324-1350).
        """
        T = len(ids)
        p0 = self._position
        if p0 + T > self.max_seq_len:
            raise ValueError(f"position {p0}+{T} exceeds max_seq_len {self.max_seq_len}")
        pos = torch.arange(p0, p0 + T)
        x = self.embed[torch.as_tensor(list(ids), dtype=torch.long)]           # MK:825-830
        tr = {} if trace else None
        for li, lw in enumerate(self.layers):
            h = rmsnorm(x, lw["in_ln"])                                        # MK:839-878
            qkv = h @ lw["wqkv"].T                                             # MK:251-302
            q = qkv[:, :Q_SIZE].view(T, NUM_Q_HEADS, HEAD_DIM)
            k = qkv[:, Q_SIZE:Q_SIZE + KV_SIZE].view(T, NUM_KV_HEADS, HEAD_DIM)
            v = qkv[:, Q_SIZE + KV_SIZE:].view(T, NUM_KV_HEADS, HEAD_DIM)
            q = self._rope(rmsnorm(q, lw["q_norm"]), pos)                      # MK:403-442
            k = self._rope(rmsnorm(k, lw["k_norm"]), pos)                      # MK:355-393
            self.k_cache[li, :, p0:p0 + T] = k.transpose(0, 1).to(self.kv_dtype)   # MK:392
            self.v_cache[li, :, p0:p0 + T] = v.transpose(0, 1).to(self.kv_dtype)   # MK:396-397
            L = p0 + T
            kc = self.k_cache[li, :, :L].to(torch.float32)                     # [8, L, 128]
            vc = self.v_cache[li, :, :L].to(torch.float32)
            qh = q.transpose(0, 1).reshape(NUM_KV_HEADS, 2 * T, HEAD_DIM)      # q heads 2g, 2g+1 share kv g (MK:490)
            scores = torch.bmm(qh, kc.transpose(1, 2)) * self.attn_scale       # MK:500-505
            if T > 1:
                row_pos = pos.repeat(2)                                        # query position of each row
                mask = torch.arange(L)[None, :] > row_pos[:, None]
                scores = scores.masked_fill(mask[None], float("-inf"))
            probs = torch.softmax(scores, dim=-1)                              # MK:507-556
            att = torch.bmm(probs, vc).view(NUM_KV_HEADS, 2, T, HEAD_DIM)
            att = att.permute(2, 0, 1, 3).reshape(T, Q_SIZE)
            x1 = att @ lw["wo"].T + x                                          # MK:596-620
            h2 = rmsnorm(x1, lw["post_ln"])                                    # MK:625-650
            gu = h2 @ lw["wgu"].T
            inter = F.silu(gu[:, :INTERMEDIATE_SIZE]) * gu[:, INTERMEDIATE_SIZE:]   # MK:653-685
            x = inter @ lw["wd"].T + x1                                        # MK:690-715
            if tr is not None:
                tr[li] = dict(qkv=qkv.clone(), q_rot=q.reshape(T, Q_SIZE).clone(),
                              k_rot=k.reshape(T, KV_SIZE).clone(), attn=att.clone(),
                              x1=x1.clone(), inter=inter.clone(), x2=x.clone())
        self._position += T
        if tr is not None:
            self.trace = tr
        if not want_logits:
            return None
        normed = rmsnorm(x[-1], self.final_norm)                               # MK:921-947
        self.last_normed = normed
        self.last_logits = self.embed @ normed                                 # MK:1024-1094
        return self.last_logits

    # ------------------------------------------------------------- reference API
    @property
    def position(self) -> int:
        return self._position

    def reset(self) -> None:
        """Position back to 0 (Model/Qwen06B_architecture.py:384-390)."""
        self._position = 0
        self.k_cache.zero_()
        self.v_cache.zero_()

    @torch.no_grad()
    def step(self, input_token_id: int, trace: bool = False) -> int:
        """One decode step; returns the greedy token (lowest index on ties)."""
        logits = self._forward([int(input_token_id)], want_logits=True, trace=trace)
        return int(torch.argmax(logits).item())

    @torch.no_grad()
    def prefill(self, ids: Sequence[int], chunk: int = 256) -> None:
        """Fill the KV cache for ``ids`` without producing tokens (MK:1276-1355)."""
        ids = list(ids)
        for i in range(0, len(ids), chunk):
            self._forward(ids[i:i + chunk], want_logits=False)

    @torch.no_grad()
    def generate_ids(self, prompt_ids: Sequence[int], max_tokens: int, eos_token_id: int = -1,
                     keep_logits: bool = False):
        """Request semantics of ``Decoder.generate`` (Model/Qwen06B_architecture.py:398-448) on IDs:
        reset, prefill ``ids[:-1]``, decode from ``ids[-1]``; the EOS token ends the loop and is
        dropped from the returned list.  Returns ``(tokens, logits_per_step | None)``.
        """
        ids = list(prompt_ids)
        self.reset()
        if len(ids) > 1:
            self.prefill(ids[:-1])
        out: List[int] = []
        logs = []
        cur = ids[-1]
        for _ in range(max_tokens):
            cur = self.step(cur)
            if keep_logits:
                logs.append(self.last_logits.clone())
            if cur == eos_token_id:
                break
            out.append(cur)
        return out, (torch.stack(logs) if keep_logits and logs else None)

    def generate(self, prompt: str, max_tokens: int = 100):
        ids = self.tokenizer.encode(prompt, add_special_tokens=False)
        eos = getattr(self.tokenizer, "eos_token_id", -1)
        out, _ = self.generate_ids(ids, max_tokens, eos_token_id=-1 if eos is None else eos)
        return self.tokenizer.decode(out, skip_special_tokens=True), len(ids), len(out)
