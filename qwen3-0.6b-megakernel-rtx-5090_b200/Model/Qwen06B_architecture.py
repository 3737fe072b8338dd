"""Host side of the B200 Qwen3-0.6B decode engine: weight layout and the ``Decoder`` API.

Mirrors the public surface of the reference module of the same name
(``Model/Qwen06B_architecture.py``): module constants, ``load_weights``,
``_pack_layer_weights``, ``Decoder`` (``step`` / ``reset`` / ``position`` /
``generate``) and the module-level ``generate``.  A program written against the
reference imports this file unchanged.  What differs underneath:

* the ops come from the sm_100a C-ABI library through ``qwen_megakernel_C`` and a
  whole request (all decode steps, LM head, argmax, token feedback) is one launch;
* ``max_seq_len`` is a constructor argument (the reference fixes 2048,
  ``Model/Qwen06B_architecture.py:21``); RoPE angles are computed in the kernel in
  fp32 for any position, the fp16 tables are still built and passed for
  signature compatibility (and are used when ``rope_from_table=True``);
* the scratch tensors of the reference signature are allocated at their reference
  sizes but only ``hidden``, ``norm_out`` and the argmax partials are written;
* ``prefill_ids`` / ``generate_ids`` expose the token-ID level under ``generate``.
"""

from __future__ import annotations

import contextlib
import math
import os
from typing import List, Optional, Sequence, Tuple

import torch

try:  # same lookup order as the reference (Model/Qwen06B_architecture.py:7-10, 31-38)
    import qwen_megakernel_C
except ImportError:  # pragma: no cover - exercised only without a built library
    qwen_megakernel_C = None

EXTENSION_ABI_VERSION = 2

NUM_LAYERS = 28
NUM_KV_HEADS = 8
HEAD_DIM = 128
HIDDEN_SIZE = 1024
INTERMEDIATE_SIZE = 3072
Q_SIZE = 16 * HEAD_DIM
KV_SIZE = 8 * HEAD_DIM
MAX_SEQ_LEN = 2048
VOCAB_SIZE = 151936
# Size of the caller-side argmax partial buffers in the reference signature
# (Model/Qwen06B_architecture.py:26); this engine fills one entry per CTA (<= 256).
LDG_LM_NUM_BLOCKS = 680
ROPE_THETA = 1_000_000.0
FIELDS_PER_LAYER = 11
_FIELD_NAMES = ("input_layernorm", "q_proj", "k_proj", "v_proj", "q_norm", "k_norm", "o_proj",
                "post_attn_norm", "gate_proj", "up_proj", "down_proj")


def _require_megakernel_op(op_name: str):
    """The named op, or ``RuntimeError`` saying the native library is not loaded."""
    if qwen_megakernel_C is not None and hasattr(qwen_megakernel_C, op_name):
        return getattr(qwen_megakernel_C, op_name)
    ns = getattr(torch.ops, "qwen_megakernel_C", None)
    if ns is not None and hasattr(ns, op_name):
        return getattr(ns, op_name)
    have = [n for n in ("decode", "generate_nosync", "prefill")
            if qwen_megakernel_C is not None and hasattr(qwen_megakernel_C, n)]
    raise RuntimeError(
        f"qwen_megakernel_C op '{op_name}' is unavailable. The CUDA library is not built/loaded "
        f"(run build.py; torch {torch.__version__}). Available ops: {', '.join(have) or 'none'}.")


def _assert_extension_compatibility() -> None:
    """ABI handshake with the native library (reference: Model/Qwen06B_architecture.py:62-89)."""
    if qwen_megakernel_C is None:
        return
    try:
        got = int(qwen_megakernel_C.abi_version())
    except Exception:
        got = None
    if got != EXTENSION_ABI_VERSION:
        raise RuntimeError(
            f"Incompatible qwen_megakernel_C binary: expected ABI {EXTENSION_ABI_VERSION}, got {got}. "
            "The packed layer-pointer layout of Python and CUDA sides must match; rebuild the library.")


_assert_extension_compatibility()
_decode = _require_megakernel_op("decode")


def rope_inv_freq(theta: float = ROPE_THETA) -> torch.Tensor:
    return 1.0 / (theta ** (torch.arange(0, HEAD_DIM, 2, dtype=torch.float32) / HEAD_DIM))


def build_rope_tables(max_seq_len: int, device="cuda", theta: float = ROPE_THETA):
    """fp16 ``[max_seq_len, 128]`` cos/sin tables with duplicated halves
    (layout of Model/Qwen06B_architecture.py:126-132)."""
    ang = torch.outer(torch.arange(max_seq_len, dtype=torch.float32), rope_inv_freq(theta))
    cos = torch.cos(ang).repeat(1, 2).to(torch.float16).to(device).contiguous()
    sin = torch.sin(ang).repeat(1, 2).to(torch.float16).to(device).contiguous()
    return cos, sin


def load_weights(model_name: str = "Qwen/Qwen3-0.6B", verbose: bool = True, max_seq_len: int = MAX_SEQ_LEN,
                 device: str = "cuda"):
    """HF checkpoint -> (weights dict, tokenizer) in the reference layout
    (Model/Qwen06B_architecture.py:96-163).  Needs the checkpoint on disk or a network.  ``device`` is where the
    tensors end up (the reference always loads to "cuda"; "cpu" serves tests of the layout)."""
    if not verbose:
        os.environ.setdefault("HF_HUB_DISABLE_PROGRESS_BARS", "1")
        os.environ.setdefault("TRANSFORMERS_NO_ADVISORY_WARNINGS", "1")
    from transformers import AutoModelForCausalLM, AutoTokenizer

    if verbose:
        print(f"Loading {model_name}...")
    # (no device_map: it needs the accelerate package; load on the host, then move)
    model = AutoModelForCausalLM.from_pretrained(model_name, dtype=torch.float16).to(device)
    tokenizer = AutoTokenizer.from_pretrained(model_name)
    sd = model.state_dict()
    hf_names = ("input_layernorm", "self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj",
                "self_attn.q_norm", "self_attn.k_norm", "self_attn.o_proj", "post_attention_layernorm",
                "mlp.gate_proj", "mlp.up_proj", "mlp.down_proj")
    n_layers = model.config.num_hidden_layers
    layer_weights = [sd[f"model.layers.{li}.{n}.weight"].contiguous() for li in range(n_layers) for n in hf_names]
    embed = sd["model.embed_tokens.weight"].contiguous()
    cos, sin = build_rope_tables(max_seq_len, device=device)
    weights = dict(embed_weight=embed, layer_weights=layer_weights,
                   final_norm_weight=sd["model.norm.weight"].contiguous(), lm_head_weight=embed,
                   cos_table=cos, sin_table=sin)
    del model
    if torch.cuda.is_available():
        torch.cuda.empty_cache()
    return weights, tokenizer


def _pack_layer_weights(layer_weights: Sequence[torch.Tensor]) -> torch.Tensor:
    """int64 device table, 12 pointers per layer (11 + zero pad), 16-byte aligned
    (layout of Model/Qwen06B_architecture.py:166-185 / megakernel_5090.cu:91-104)."""
    n_layers, rem = divmod(len(layer_weights), FIELDS_PER_LAYER)
    assert rem == 0, "layer_weights must hold 11 tensors per layer"
    table = torch.zeros(n_layers, FIELDS_PER_LAYER + 1, dtype=torch.int64)
    for li in range(n_layers):
        for j in range(FIELDS_PER_LAYER):
            table[li, j] = layer_weights[li * FIELDS_PER_LAYER + j].data_ptr()
    device = layer_weights[0].device
    raw = torch.zeros(table.numel() + 2, dtype=torch.int64, device=device)
    shift = ((16 - raw.data_ptr() % 16) % 16) // 8
    view = raw[shift:shift + table.numel()]
    view.copy_(table.flatten())
    assert view.data_ptr() % 16 == 0
    return view


class Decoder:
    """Stateful greedy decoder on one B200 (API of Model/Qwen06B_architecture.py:188-448)."""

    def __init__(self, weights=None, tokenizer=None, model_name: str = "Qwen/Qwen3-0.6B", verbose: bool = True,
                 max_seq_len: int = MAX_SEQ_LEN, rope_from_table: bool = False, device: str = "cuda",
                 weight_format: str = "fp16", prefill_mode: str = "serial"):
        if not torch.cuda.is_available():
            raise RuntimeError("Decoder needs a CUDA device (sm_100a); there is no CPU path")
        if weights is None:
            weights, tokenizer = load_weights(model_name, verbose=verbose, max_seq_len=max_seq_len, device=device)
        self.tokenizer = tokenizer
        self.max_seq_len = int(max_seq_len)
        self._position = 0
        self._weights = weights
        self._embed_weight = weights["embed_weight"]
        self._final_norm_weight = weights["final_norm_weight"]
        self._lm_head_weight = weights["lm_head_weight"]
        dev = self._embed_weight.device
        self.num_layers = len(weights["layer_weights"]) // FIELDS_PER_LAYER
        self.vocab_size = int(self._embed_weight.shape[0])
        # "fp16"; "fp8" (matrices packed by quantize.quantize_weights_fp8); "nvfp4" (quantize.quantize_weights_nvfp4:
        # read by the tensor-core ops only - tensor prefill, BatchDecoder(engine="gemm"))
        if weight_format not in ("fp16", "fp8", "nvfp4"):
            raise ValueError("weight_format must be 'fp16', 'fp8' or 'nvfp4'")
        self.weight_format = weight_format
        # "serial": the reference's token-by-token prefill (fp32 activations, bit-identical to decoding the
        # prompt); "tensor": chunked prefill on the tensor cores (fp16 GEMM operands; packed matrices are expanded
        # inside the GEMMs)
        if prefill_mode not in ("serial", "tensor"):
            raise ValueError("prefill_mode must be 'serial' or 'tensor'")
        if prefill_mode == "serial" and weight_format == "nvfp4":
            raise ValueError("NVFP4 weights need prefill_mode='tensor' (the persistent kernels do not read them)")
        self.prefill_mode = prefill_mode
        cos, sin = weights.get("cos_table"), weights.get("sin_table")
        if cos is None or cos.shape[0] < self.max_seq_len or cos.device != dev:
            cos, sin = build_rope_tables(self.max_seq_len, device=dev)
        self._cos_table, self._sin_table = cos, sin
        self._layer_weights_packed = _pack_layer_weights(weights["layer_weights"])
        self._check_weight_alignment(weights["layer_weights"], verbose)
        self._attn_scale = 1.0 / math.sqrt(HEAD_DIM)

        self._k_cache = torch.zeros(self.num_layers, NUM_KV_HEADS, self.max_seq_len, HEAD_DIM,
                                    dtype=torch.float16, device=dev)
        self._v_cache = torch.zeros_like(self._k_cache)
        self._kv_high_water = 0

        f16 = dict(dtype=torch.float16, device=dev)
        f32 = dict(dtype=torch.float32, device=dev)
        self._hidden = torch.zeros(HIDDEN_SIZE, **f16)
        self._act = torch.zeros(HIDDEN_SIZE, **f32)
        self._res = torch.zeros(HIDDEN_SIZE, **f32)
        self._q = torch.zeros(Q_SIZE, **f16)
        self._k = torch.zeros(KV_SIZE, **f16)
        self._v = torch.zeros(KV_SIZE, **f16)
        self._attn_out = torch.zeros(Q_SIZE, **f16)
        self._mlp_inter = torch.zeros(INTERMEDIATE_SIZE, **f32)
        self._norm_out = torch.zeros(HIDDEN_SIZE, **f32)
        self._fmax_vals = torch.zeros(LDG_LM_NUM_BLOCKS, **f32)
        self._fmax_idxs = torch.zeros(LDG_LM_NUM_BLOCKS, dtype=torch.int32, device=dev)
        # token log: device tensor for the kernel, pinned host twin for the single DtoH copy
        self._output_log = torch.full((self.max_seq_len,), -1, dtype=torch.int32, device=dev)
        self._output_log_cpu = torch.empty(self.max_seq_len, dtype=torch.int32).pin_memory()

        self._rope_from_table = int(bool(rope_from_table))
        self._inv_freq = rope_inv_freq()
        # An engine handle of the library carries this decoder's options and applies them with every op; the
        # reference's pybind module (free functions only) has none, and the module-level ops are used instead.
        self._engine = None
        if qwen_megakernel_C is not None and hasattr(qwen_megakernel_C, "Engine"):
            self._engine = qwen_megakernel_C.Engine(
                device=dev, vocab_size=self.vocab_size, weight_format=weight_format,
                rope_from_table=self._rope_from_table, inv_freq=self._inv_freq)
            self._decode_op = self._engine.decode
            self._gen = self._engine.generate_nosync
            self._prefill_op = self._engine.prefill
        else:
            self._decode_op = _decode
            self._gen = _require_megakernel_op("generate_nosync")
            self._prefill_op = _require_megakernel_op("prefill")
        row_bytes = {"fp16": 2 * HIDDEN_SIZE, "fp8": HIDDEN_SIZE + 16,
                     "nvfp4": HIDDEN_SIZE // 2 + HIDDEN_SIZE // 16 + 16}[weight_format]
        if self._embed_weight.numel() * self._embed_weight.element_size() != self.vocab_size * row_bytes:
            raise RuntimeError(f"embedding tensor does not have {self.vocab_size} rows of {row_bytes} bytes: "
                               f"weight_format={weight_format!r} does not match the weights")
        self.apply_options()

    def apply_options(self) -> None:
        """The library keeps vocabulary size, weight format, RoPE mode and frequencies per DEVICE, not per decoder.
        Every op of this decoder re-applies its own values first (host-side and cheap: unchanged values are
        recognised), so decoders with different vocabularies or weight formats can live on one GPU."""
        if self._engine is not None:
            self._engine.apply()
        elif qwen_megakernel_C is not None and hasattr(qwen_megakernel_C, "configure"):
            qwen_megakernel_C.configure(vocab_size=self.vocab_size, rope_from_table=self._rope_from_table)
            qwen_megakernel_C.set_weight_format(self.weight_format)
            qwen_megakernel_C.set_inv_freq(self._inv_freq)

    # ------------------------------------------------------------------ argument packing
    def _common(self):
        return (self._embed_weight, self._layer_weights_packed, self._final_norm_weight, self._lm_head_weight,
                self._cos_table, self._sin_table, self._k_cache, self._v_cache, self._hidden, self._act,
                self._res, self._q, self._k, self._v, self._attn_out, self._mlp_inter, self._norm_out,
                self._fmax_vals, self._fmax_idxs)

    def _eos(self) -> int:
        eos = getattr(self.tokenizer, "eos_token_id", None)
        return -1 if eos is None else int(eos)

    def _check_weight_alignment(self, layer_weights, verbose=True) -> None:
        bad = [f"layer {i // FIELDS_PER_LAYER} [{_FIELD_NAMES[i % FIELDS_PER_LAYER]}]"
               for i, t in enumerate(layer_weights) if t.data_ptr() % 16]
        if bad:
            raise RuntimeError("weight tensors not 16-byte aligned: " + ", ".join(bad[:8]))
        if verbose:
            print("All weight pointers 16-byte aligned OK")

    # ------------------------------------------------------------------ reference API
    @property
    def position(self) -> int:
        return self._position

    def reset(self) -> None:
        """Back to position 0.  Cache rows are not cleared: every row below the current
        length is rewritten before it is read."""
        self._position = 0
        self._kv_high_water = 0

    def step(self, input_token_id: int) -> int:
        """One decode step through the ``decode`` op (Model/Qwen06B_architecture.py:351-380)."""
        self.apply_options()
        out = self._decode_op(int(input_token_id), *self._common(), self.num_layers, self._position,
                      self.max_seq_len, self._attn_scale)
        tok = int(out.item())
        self._position += 1
        self._kv_high_water = max(self._kv_high_water, self._position)
        return tok

    def prefill_ids(self, ids: Sequence[int]) -> None:
        """KV cache for ``ids`` at the current position through the ``prefill`` op."""
        if len(ids) == 0:
            return
        self.apply_options()
        t = torch.tensor(list(ids), dtype=torch.int32)
        if self.prefill_mode == "tensor":
            _require_megakernel_op("prefill_chunked")(
                t, self._embed_weight, self._layer_weights_packed, self._cos_table, self._sin_table,
                self._k_cache, self._v_cache, self.num_layers, self._position, self.max_seq_len, self._attn_scale)
        else:
            self._prefill_op(t, *self._common(), self.num_layers, self._position, self.max_seq_len,
                             self._attn_scale)
        self._position += len(ids)
        self._kv_high_water = max(self._kv_high_water, self._position)

    def generate_ids(self, prompt_ids: Sequence[int], max_tokens: int, reset: bool = True) -> List[int]:
        """Token-ID form of ``generate``: prefill ``ids[:-1]``, decode from ``ids[-1]``, one DtoH copy
        of the token log, trim at the first unwritten entry or EOS."""
        ids = list(prompt_ids)
        if not ids:
            raise ValueError("empty prompt")
        if reset:
            self.reset()
        self.prefill_ids(ids[:-1])
        max_tokens = int(max_tokens)
        if max_tokens <= 0:
            return []
        log = self._output_log[:max_tokens]
        log.fill_(-1)
        eos = self._eos()
        self.apply_options()
        self._gen(ids[-1], max_tokens, *self._common(), log, self.num_layers, self._position,
                  self.max_seq_len, self._attn_scale, eos)
        host = self._output_log_cpu[:max_tokens]
        host.copy_(log)                       # stream is idle: the op synchronised
        out: List[int] = []
        for tok in host.tolist():
            if tok == -1 or tok == eos:
                break
            out.append(tok)
        self._position += len(out)
        self._kv_high_water = max(self._kv_high_water, self._position)
        return out

    def generate(self, prompt: str, max_tokens: int = 100) -> Tuple[str, int, int]:
        """``(text, n_prompt_tokens, n_output_tokens)`` (Model/Qwen06B_architecture.py:398-448)."""
        ids = self.tokenizer.encode(prompt, add_special_tokens=False)
        out = self.generate_ids(ids, max_tokens)
        return self.tokenizer.decode(out, skip_special_tokens=True), len(ids), len(out)


class BatchDecoder:
    """Greedy decode of up to four independent sequences per launch.

    The reference decodes one sequence per persistent launch
    (Model/Qwen06B_architecture.py:398-448); this wraps the multi-sequence form of the same kernel
    (``generate_batch`` op): weights are streamed once per step and shared by all sequences, each
    sequence has its own KV cache and position.  Prompts are prefilled one after the other through
    the ``prefill`` op, then all sequences decode together.
    """

    MAX_SEQUENCES = 4            # per persistent launch
    MAX_GEMM_SEQUENCES = 128     # per call of the tensor-core batched decode

    def __init__(self, weights=None, tokenizer=None, num_sequences: int = 4, max_seq_len: int = MAX_SEQ_LEN,
                 verbose: bool = False, engine: str = "auto", **decoder_kw):
        """``engine``: "persistent" (one megakernel launch, <= 4 sequences, fp32 activations), "gemm" (tcgen05
        GEMMs per step, <= 128 sequences, fp16 GEMM operands; packed FP8 / NVFP4 matrices are expanded inside the
        GEMMs) or "auto": persistent up to 3 sequences, gemm above (NVFP4: always gemm) -
        measured at 1024-token contexts, 4 sequences: 2060 tok/s persistent, 2566 tok/s gemm; 2 sequences: 1519
        against 1321."""
        n = int(num_sequences)
        if engine == "auto":
            engine = "persistent" if n <= 3 and decoder_kw.get("weight_format", "fp16") != "nvfp4" else "gemm"
        if engine not in ("persistent", "gemm"):
            raise ValueError("engine must be 'auto', 'persistent' or 'gemm'")
        limit = self.MAX_SEQUENCES if engine == "persistent" else self.MAX_GEMM_SEQUENCES
        if not 1 <= n <= limit:
            raise ValueError(f"num_sequences must be 1..{limit} for the {engine} engine")
        self.engine = engine
        self.num_sequences = n
        # slot 0 owns the weights, tables and the first cache; the other slots only add caches
        self._base = Decoder(weights=weights, tokenizer=tokenizer, max_seq_len=max_seq_len, verbose=verbose,
                             **decoder_kw)
        self.tokenizer = self._base.tokenizer
        self.max_seq_len = self._base.max_seq_len
        dev = self._base._embed_weight.device
        self._k_caches = [self._base._k_cache] + [torch.zeros_like(self._base._k_cache)
                                                   for _ in range(self.num_sequences - 1)]
        self._v_caches = [self._base._v_cache] + [torch.zeros_like(self._base._v_cache)
                                                   for _ in range(self.num_sequences - 1)]
        self._logs = [torch.full((self.max_seq_len,), -1, dtype=torch.int32, device=dev)
                      for _ in range(self.num_sequences)]
        self._logs_cpu = torch.empty(self.num_sequences, self.max_seq_len, dtype=torch.int32).pin_memory()
        self.positions = [0] * self.num_sequences
        self._gen_batch = _require_megakernel_op("generate_batch" if engine == "persistent" else "decode_batched")
        # The tensor-core prefill and the tensor-core batched decode use separate workspaces and locks in the
        # library: a scheduler may prefill one slot (on its own stream) while other slots decode.  The persistent
        # engine and the token-serial prefill share the megakernel's exchange area and must not overlap.
        self.supports_overlap = engine == "gemm" and self._base.prefill_mode == "tensor"
        self._prefill_stream = torch.cuda.Stream(device=dev) if self.supports_overlap else None
        # Decode rounds of an overlapping scheduler must stay off the legacy default stream: work queued there
        # (this op's event wait lasts a whole round) orders itself against every blocking stream of the process.
        self._decode_stream = torch.cuda.Stream(device=dev) if self.supports_overlap else None

    def prefill_slot(self, b: int, ids: Sequence[int]) -> None:
        """Fill slot ``b``'s KV cache with ``ids`` from position 0 (the ``prefill`` op)."""
        if not 0 <= b < self.num_sequences:
            raise ValueError("slot out of range")
        if len(ids) > self.max_seq_len:
            raise ValueError("prompt exceeds max_seq_len")
        base = self._base
        base._k_cache, base._v_cache = self._k_caches[b], self._v_caches[b]
        try:
            base._position = 0
            if self._prefill_stream is not None:
                with torch.cuda.stream(self._prefill_stream):   # the op blocks until its stream is idle
                    base.prefill_ids(ids)
            else:
                base.prefill_ids(ids)
        finally:
            base._k_cache, base._v_cache = self._k_caches[0], self._v_caches[0]
        self.positions[b] = len(ids)

    _prefill_slot = prefill_slot

    @property
    def packed_prefill_rows(self) -> int:
        """Rows one ``prefill_slots`` pass may hold (each prompt padded to a multiple of 128); 0: no packed prefill."""
        base = self._base
        return 4096 if base.prefill_mode == "tensor" else 0

    def prefill_many(self, slots: Sequence[int], prompts: Sequence[Sequence[int]]) -> None:
        """Prefill any number of slots: in packed passes of up to ``packed_prefill_rows`` rows where the engine has
        them, a prompt longer than that (or any prompt of an engine without packed prefill) through ``prefill_slot``."""
        budget = self.packed_prefill_rows
        group, rows = [], 0

        def flush():
            nonlocal group, rows
            if len(group) == 1:
                self.prefill_slot(*group[0])
            elif group:
                self.prefill_slots([b for b, _ in group], [ids for _, ids in group])
            group, rows = [], 0
        for b, ids in zip(slots, prompts):
            need = (max(len(ids), 1) + 127) // 128 * 128
            if budget <= 0 or need > budget:
                self.prefill_slot(b, ids)
                continue
            if group and (rows + need > budget or len(group) == 64):
                flush()
            group.append((b, list(ids)))
            rows += need
        flush()

    def prefill_slots(self, slots: Sequence[int], prompts: Sequence[Sequence[int]]) -> None:
        """Fill the caches of several slots in ONE tensor-core pass (``qmk_prefill_packed``): weights are read once for all
        of them and a pass's ~200 launches are shared.  Empty prompts are skipped (their slot starts at position 0)."""
        slots = [int(b) for b in slots]
        if len(slots) != len(prompts) or len(set(slots)) != len(slots) or not all(0 <= b < self.num_sequences for b in slots):
            raise ValueError("slots must be distinct, in range, one per prompt")
        base = self._base
        if base.prefill_mode != "tensor":
            raise RuntimeError("prefill_slots needs prefill_mode='tensor'")
        todo = [(b, list(ids)) for b, ids in zip(slots, prompts) if len(ids) > 0]
        for _, ids in todo:
            if len(ids) > self.max_seq_len:
                raise ValueError("prompt exceeds max_seq_len")
        if todo:
            base.apply_options()
            args = ([ids for _, ids in todo], base._embed_weight, base._layer_weights_packed, base._cos_table, base._sin_table,
                    [self._k_caches[b] for b, _ in todo], [self._v_caches[b] for b, _ in todo], base.num_layers, self.max_seq_len,
                    base._attn_scale)
            op = _require_megakernel_op("prefill_packed")
            if self._prefill_stream is not None:
                with torch.cuda.stream(self._prefill_stream):   # the op blocks until its stream is idle
                    op(*args)
            else:
                op(*args)
        for b, ids in zip(slots, prompts):
            self.positions[b] = len(ids)


    def decode_slots(self, slots: Sequence[int], first_tokens: Sequence[int], steps: int) -> List[List[int]]:
        """One launch: ``steps`` greedy tokens for every slot in ``slots`` (any subset, each from its own
        position and ``first_tokens`` entry).  Returns the raw token lists (no EOS cut) and advances
        the slots' positions by ``steps``."""
        slots = [int(b) for b in slots]
        steps = int(steps)
        if len(set(slots)) != len(slots) or not all(0 <= b < self.num_sequences for b in slots):
            raise ValueError("slots must be distinct and in range")
        if steps <= 0 or not slots:
            return [[] for _ in slots]
        for b in slots:
            if self.positions[b] + steps > self.max_seq_len:
                raise ValueError(f"slot {b}: position + steps exceeds max_seq_len")
        base = self._base
        logs = [self._logs[b][:steps] for b in slots]
        ctx = torch.cuda.stream(self._decode_stream) if self._decode_stream is not None else contextlib.nullcontext()
        out = []
        base.apply_options()
        with ctx:
            self._gen_batch(list(first_tokens), [self.positions[b] for b in slots], steps, base._embed_weight,
                            base._layer_weights_packed, base._final_norm_weight, base._lm_head_weight,
                            base._cos_table, base._sin_table, [self._k_caches[b] for b in slots],
                            [self._v_caches[b] for b in slots], logs, base.num_layers, self.max_seq_len,
                            base._attn_scale)
            for i, b in enumerate(slots):
                host = self._logs_cpu[b, :steps]
                host.copy_(logs[i], non_blocking=True)
            torch.cuda.current_stream().synchronize()
        for b in slots:
            out.append(self._logs_cpu[b, :steps].tolist())
            self.positions[b] += steps
        return out

    def generate_ids(self, prompts: Sequence[Sequence[int]], max_tokens: int) -> List[List[int]]:
        """One list of new token IDs per prompt (cut at EOS, which is not returned).  ``len(prompts)``
        may be below ``num_sequences``; the launch then carries fewer sequences."""
        n = len(prompts)
        if not 1 <= n <= self.num_sequences:
            raise ValueError(f"between 1 and {self.num_sequences} prompts per call")
        max_tokens = int(max_tokens)
        firsts = []
        heads = []
        for b, ids in enumerate(prompts):
            ids = list(ids)
            if not ids:
                raise ValueError("empty prompt")
            if len(ids) - 1 + max_tokens > self.max_seq_len:
                raise ValueError("prompt + max_tokens exceeds max_seq_len")
            heads.append(ids[:-1])
            firsts.append(ids[-1])
        self.prefill_many(list(range(n)), heads)
        if max_tokens <= 0:
            return [[] for _ in range(n)]
        base = self._base
        logs = [self._logs[b][:max_tokens] for b in range(n)]
        for log in logs:
            log.fill_(-1)
        base.apply_options()
        self._gen_batch(firsts, self.positions[:n], max_tokens, base._embed_weight, base._layer_weights_packed,
                        base._final_norm_weight, base._lm_head_weight, base._cos_table, base._sin_table,
                        self._k_caches[:n], self._v_caches[:n], logs, base.num_layers, self.max_seq_len,
                        base._attn_scale)
        eos = base._eos()
        outs: List[List[int]] = []
        for b in range(n):
            host = self._logs_cpu[b, :max_tokens]
            host.copy_(logs[b])
            out: List[int] = []
            for tok in host.tolist():
                if tok == -1 or tok == eos:
                    break
                out.append(tok)
            outs.append(out)
            # cache rows past an EOS were written but are never read: the position counts what was returned
            self.positions[b] += len(out)
        return outs


def generate(prompt: str, max_tokens: int = 50, verbose: bool = True) -> str:
    """Load the model, generate once, return the text."""
    text, _, _ = Decoder(verbose=verbose).generate(prompt, max_tokens)
    return text
