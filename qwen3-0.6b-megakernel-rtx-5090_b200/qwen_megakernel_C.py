"""Op surface ``qwen_megakernel_C`` over the sm_100a C-ABI library (ctypes, no libtorch).

Same module name, op names, argument order and error behaviour as the reference's
pybind module (``Tools/megakernel/qwen_ops.cpp:46-267``): ``decode``,
``generate_nosync``, ``prefill``, ``abi_version``.  Argument checks that the
reference does with ``TORCH_CHECK`` raise ``RuntimeError`` here too.  Tensors are
only unwrapped to raw pointers; all arithmetic happens in the CUDA library.

There is no CPU fallback: importing this module without the built library raises
``ImportError``, and calling an op without a CUDA device raises ``RuntimeError``.

Additions with no counterpart in the reference are grouped at the bottom
(``configure``, ``set_inv_freq``, ``set_logits_dump``, ``sync_status``, ...).
"""

from __future__ import annotations

import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIBRARY_PATH = os.environ.get("QWEN_MEGAKERNEL_LIB", os.path.join(_HERE, "libqwen_megakernel.so"))

if not os.path.exists(LIBRARY_PATH):
    raise ImportError(
        f"qwen_megakernel_C: {LIBRARY_PATH} is not built. Run `python build.py` in {_HERE} "
        "(nvcc, sm_100a). There is no CPU or PyTorch fallback for the decode ops.")

_lib = ctypes.CDLL(LIBRARY_PATH)

_P, _I, _F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
_PTRS19 = [_P] * 19  # embed .. block_max_idxs, in the reference's order (qwen_ops.cpp:9-17)

_lib.launch_ldg_decode_direct.argtypes = [_I, _P, *_PTRS19, _I, _I, _I, _F, _P]
_lib.launch_ldg_decode_direct.restype = None
_lib.launch_ldg_decode_persistent.argtypes = [_I, _P, *_PTRS19, _I, _I, _I, _F, _P]
_lib.launch_ldg_decode_persistent.restype = None
_lib.launch_ldg_generate_nosync.argtypes = [_I, _I, *_PTRS19, _P, _I, _I, _I, _F, _I, _P]
_lib.launch_ldg_generate_nosync.restype = None
_lib.launch_ldg_prefill.argtypes = [_P, _I, *_PTRS19, _I, _I, _I, _F, _P]
_lib.launch_ldg_prefill.restype = None
_lib.qmk_abi_version.restype = _I
_lib.qmk_configure.argtypes = [_I, _I, _I, _I, _I]
_lib.qmk_configure.restype = _I
_lib.qmk_set_inv_freq.argtypes = [_P]
_lib.qmk_set_inv_freq.restype = _I
_lib.qmk_set_logits_dump.argtypes = [_P]
_lib.qmk_set_logits_dump.restype = _I
_lib.qmk_set_tuning.argtypes = [_I, _I]
_lib.qmk_set_tuning.restype = _I
_lib.qmk_set_weight_format.argtypes = [_I]
_lib.qmk_set_weight_format.restype = _I
_lib.qmk_set_tuning2.argtypes = [_I, _I]
_lib.qmk_set_tuning2.restype = _I
_lib.qmk_set_profile_buffer.argtypes = [_P]
_lib.qmk_set_profile_buffer.restype = _I
_lib.qmk_set_prefill_attention.argtypes = [_I]
_lib.qmk_set_prefill_attention.restype = _I
_lib.qmk_set_decode_attention.argtypes = [_I]
_lib.qmk_set_decode_attention.restype = _I
_lib.qmk_set_step_overlap.argtypes = [_I]
_lib.qmk_set_step_overlap.restype = _I
_lib.qmk_set_fused.argtypes = [_I, _I]
_lib.qmk_set_fused.restype = _I
_lib.qmk_invalidate_weights.restype = _I
_lib.qmk_release_weights.argtypes = [_P]
_lib.qmk_release_weights.restype = _I
_lib.qmk_decode.argtypes = [_I, _P, *([_P] * 12), _I, _I, _I, _F, _P]
_lib.qmk_decode.restype = _I
_lib.qmk_generate.argtypes = [_I, _I, *([_P] * 12), _P, _I, _I, _I, _F, _I, _I, _P]
_lib.qmk_generate.restype = _I
_lib.qmk_prefill.argtypes = [_P, _I, *([_P] * 7), _I, _I, _I, _F, _P]
_lib.qmk_prefill.restype = _I
_lib.qmk_generate_static.argtypes = [_I, _I, *([_P] * 7), _P, _I, _I, _I, _F, _I, _P]
_lib.qmk_generate_static.restype = _I
_lib.qmk_generate_batch.argtypes = [_I, _P, _P, _I, *([_P] * 6), _P, _P, _P, _I, _I, _F, _I, _P]
_lib.qmk_generate_batch.restype = _I
_lib.qmk_decode_batched.argtypes = [_I, _P, _P, _I, *([_P] * 6), _P, _P, _P, _I, _I, _F, _P]
_lib.qmk_decode_batched.restype = _I
_lib.qmk_prefill_chunked.argtypes = [_P, _I, _P, _P, _P, _P, _P, _P, _I, _I, _I, _F, _P]
_lib.qmk_prefill_chunked.restype = _I
_lib.qmk_prefill_packed.argtypes = [_P, _I, _P, _P, _P, _P, _P, _P, _P, _I, _I, _F, _P]
_lib.qmk_prefill_packed.restype = _I
_lib.qmk_gemm_f16_tn.argtypes = [_P, _P, _P, _I, _I, _I, _P]
_lib.qmk_gemm_f16_tn.restype = _I
_lib.qmk_gemm_packed_tn.argtypes = [_P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P]
_lib.qmk_gemm_packed_tn.restype = _I


class _EngineConfig(ctypes.Structure):
    _fields_ = [("device", _I), ("vocab_size", _I), ("weight_format", _I), ("rope_from_table", _I),
                ("split_len", _I), ("max_ctas", _I), ("timeout_ms", _I), ("fused", _I), ("inv_freq64", _P)]


_lib.qmk_engine_create.argtypes = [ctypes.POINTER(_EngineConfig), ctypes.POINTER(_P)]
_lib.qmk_engine_create.restype = _I
_lib.qmk_engine_destroy.argtypes = [_P]
_lib.qmk_engine_destroy.restype = _I
_lib.qmk_engine_apply.argtypes = [_P]
_lib.qmk_engine_apply.restype = _I
_lib.qmk_engine_decode.argtypes = [_P] + _lib.qmk_decode.argtypes
_lib.qmk_engine_decode.restype = _I
_lib.qmk_engine_generate.argtypes = [_P] + _lib.qmk_generate.argtypes
_lib.qmk_engine_generate.restype = _I
_lib.qmk_engine_prefill.argtypes = [_P] + _lib.qmk_prefill.argtypes
_lib.qmk_engine_prefill.restype = _I
_lib.qmk_sync_status.restype = _I
_lib.qmk_last_error.restype = ctypes.c_char_p
_lib.qmk_num_ctas.restype = _I
_lib.qmk_scratch_bytes.restype = ctypes.c_longlong
_lib.qmk_selftest_wait_timeout.argtypes = [_I]
_lib.qmk_selftest_wait_timeout.restype = _I
_lib.qmk_selftest_gemm_wait_timeout.argtypes = [_I]
_lib.qmk_selftest_gemm_wait_timeout.restype = _I

EXPORTED_SYMBOLS = (
    "launch_ldg_decode_direct", "launch_ldg_decode_persistent", "launch_ldg_generate_nosync",
    "launch_ldg_prefill", "qmk_abi_version", "qmk_configure", "qmk_set_inv_freq", "qmk_set_logits_dump",
    "qmk_set_weight_format", "qmk_set_tuning", "qmk_set_tuning2", "qmk_set_profile_buffer", "qmk_set_fused", "qmk_set_step_overlap", "qmk_set_prefill_attention", "qmk_set_decode_attention", "qmk_invalidate_weights", "qmk_release_weights", "qmk_decode", "qmk_generate", "qmk_generate_static", "qmk_generate_batch", "qmk_gemm_f16_tn", "qmk_gemm_packed_tn", "qmk_decode_batched", "qmk_prefill_chunked", "qmk_prefill_packed", "qmk_prefill", "qmk_engine_create", "qmk_engine_destroy", "qmk_engine_apply", "qmk_engine_decode", "qmk_engine_generate", "qmk_engine_prefill", "qmk_sync_status", "qmk_last_error", "qmk_num_ctas",
    "qmk_scratch_bytes", "qmk_selftest_wait_timeout", "qmk_selftest_gemm_wait_timeout",
)


def _check(cond: bool, msg: str) -> None:
    if not cond:
        raise RuntimeError(msg)


def _require_cuda() -> None:
    _check(torch.cuda.is_available(),
           "qwen_megakernel_C: no CUDA device; the decode ops have no CPU fallback")


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t) -> int:
    return 0 if t is None else t.data_ptr()


def _check_table(layer_weights_packed: torch.Tensor, who: str) -> None:
    # qwen_ops.cpp:75-78, 155-157, 226-228
    _check(layer_weights_packed.data_ptr() % 16 == 0,
           f"{who}: layer_weights_packed must be 16-byte aligned "
           f"(address ends in {layer_weights_packed.data_ptr() % 16})")


def _raise_if_failed(who: str) -> None:
    msg = _lib.qmk_last_error().decode()
    if msg:
        raise RuntimeError(f"{who}: {msg}")


def abi_version() -> int:
    """Layout version of the packed layer table (qwen_ops.cpp:42-44)."""
    return int(_lib.qmk_abi_version())


def decode(input_token_id, embed_weight, layer_weights_packed, final_norm_weight, lm_head_weight,
           cos_table, sin_table, k_cache, v_cache, hidden, act, res, q, k, v, attn_out, mlp_inter,
           norm_out, bmax_vals, bmax_idxs, num_layers, position, max_seq_len, attn_scale):
    """One greedy step; returns an int32[1] CUDA tensor, does not synchronise (qwen_ops.cpp:46-110)."""
    _require_cuda()
    _check_table(layer_weights_packed, "decode")
    out = torch.zeros(1, dtype=torch.int32, device=embed_weight.device)
    _lib.launch_ldg_decode_direct(
        int(input_token_id), out.data_ptr(), _ptr(embed_weight), _ptr(layer_weights_packed),
        _ptr(final_norm_weight), _ptr(lm_head_weight), _ptr(cos_table), _ptr(sin_table), _ptr(k_cache),
        _ptr(v_cache), _ptr(hidden), _ptr(act), _ptr(res), _ptr(q), _ptr(k), _ptr(v), _ptr(attn_out),
        _ptr(mlp_inter), _ptr(norm_out), _ptr(bmax_vals), _ptr(bmax_idxs),
        int(num_layers), int(position), int(max_seq_len), float(attn_scale), _stream())
    _raise_if_failed("decode")
    return out


def generate_nosync(first_token_id, num_steps, embed_weight, layer_weights_packed, final_norm_weight,
                    lm_head_weight, cos_table, sin_table, k_cache, v_cache, hidden, act, res, q, k, v,
                    attn_out, mlp_inter, norm_out, bmax_vals, bmax_idxs, output_log, num_layers,
                    start_position, max_seq_len, attn_scale, eos_token_id=151645):
    """``num_steps`` greedy tokens into ``output_log``; blocks; returns ``output_log`` (qwen_ops.cpp:112-191)."""
    _require_cuda()
    _check(output_log.dtype == torch.int32,
           f"generate_nosync: output_log must be dtype int32, got {output_log.dtype}")
    _check(output_log.is_cuda, "generate_nosync: output_log must be on CUDA")
    _check(output_log.is_contiguous(), "generate_nosync: output_log must be contiguous")
    _check(output_log.numel() >= num_steps,
           f"generate_nosync: output_log.numel() ({output_log.numel()}) < num_steps ({num_steps})")
    _check_table(layer_weights_packed, "generate_nosync")
    _lib.launch_ldg_generate_nosync(
        int(first_token_id), int(num_steps), _ptr(embed_weight), _ptr(layer_weights_packed),
        _ptr(final_norm_weight), _ptr(lm_head_weight), _ptr(cos_table), _ptr(sin_table), _ptr(k_cache),
        _ptr(v_cache), _ptr(hidden), _ptr(act), _ptr(res), _ptr(q), _ptr(k), _ptr(v), _ptr(attn_out),
        _ptr(mlp_inter), _ptr(norm_out), _ptr(bmax_vals), _ptr(bmax_idxs), output_log.data_ptr(),
        int(num_layers), int(start_position), int(max_seq_len), float(attn_scale),
        -1 if eos_token_id is None else int(eos_token_id), _stream())
    _raise_if_failed("generate_nosync")
    return output_log


def prefill(token_ids, embed_weight, layer_weights_packed, final_norm_weight, lm_head_weight, cos_table,
            sin_table, k_cache, v_cache, hidden, act, res, q, k, v, attn_out, mlp_inter, norm_out,
            bmax_vals, bmax_idxs, num_layers, start_position, max_seq_len, attn_scale):
    """Fills the KV cache for a CPU int32 token tensor; blocks (qwen_ops.cpp:193-260)."""
    _check(token_ids.dtype == torch.int32, "token_ids must be int32")
    _check(token_ids.device.type == "cpu", "token_ids must be on CPU")
    _check(token_ids.is_contiguous(), "token_ids must be contiguous")
    n = int(token_ids.shape[0])
    if n == 0:
        return None
    _require_cuda()
    _check_table(layer_weights_packed, "prefill")
    _lib.launch_ldg_prefill(
        token_ids.data_ptr(), n, _ptr(embed_weight), _ptr(layer_weights_packed), _ptr(final_norm_weight),
        _ptr(lm_head_weight), _ptr(cos_table), _ptr(sin_table), _ptr(k_cache), _ptr(v_cache), _ptr(hidden),
        _ptr(act), _ptr(res), _ptr(q), _ptr(k), _ptr(v), _ptr(attn_out), _ptr(mlp_inter), _ptr(norm_out),
        _ptr(bmax_vals), _ptr(bmax_idxs), int(num_layers), int(start_position), int(max_seq_len),
        float(attn_scale), _stream())
    _raise_if_failed("prefill")
    return None


# ---------------------------------------------------------------- additions
class Engine:
    """One client's view of a GPU: an engine handle of the library (``qmk_engine_create``) that carries the
    client's options - vocabulary size, weight format, RoPE mode and frequencies, grid cap, time-out - and offers
    ``decode`` / ``generate_nosync`` / ``prefill`` with the arguments of the module-level ops.  Each call applies the
    options and runs the op under one hold of the library's lock, so engines with different options can share a GPU."""

    def __init__(self, device=None, vocab_size=151936, weight_format="fp16", rope_from_table=False, inv_freq=None,
                 split_len=-1, max_ctas=-1, timeout_ms=-1, fused=-1):
        _require_cuda()
        if device is None:
            device = torch.cuda.current_device()
        index = torch.device(device).index if not isinstance(device, int) else device
        fmt = {"fp16": 0, "fp8": 1, "nvfp4": 2, 0: 0, 1: 1, 2: 2}.get(weight_format)
        _check(fmt is not None, f"Engine: unknown weight_format {weight_format!r}")
        freq = None
        if inv_freq is not None:
            freq = inv_freq.detach().to(dtype=torch.float32, device="cpu").contiguous()
            _check(freq.numel() == 64, "Engine: inv_freq must hold 64 values")
        cfg = _EngineConfig(int(index if index is not None else torch.cuda.current_device()), int(vocab_size), fmt,
                            int(bool(rope_from_table)), int(split_len), int(max_ctas), int(timeout_ms), int(fused),
                            freq.data_ptr() if freq is not None else None)
        handle = _P()
        rc = _lib.qmk_engine_create(ctypes.byref(cfg), ctypes.byref(handle))
        if rc != 0:
            raise RuntimeError(f"Engine: qmk_engine_create failed (status {rc})")
        self._handle = handle
        self.device = cfg.device

    def close(self) -> None:
        handle, self._handle = getattr(self, "_handle", None), None
        if handle and _lib is not None:       # (module globals are gone when the interpreter shuts down)
            _lib.qmk_engine_destroy(handle)

    __del__ = close

    def _live(self):
        _check(bool(self._handle), "Engine: used after close()")
        return self._handle

    def _done(self, who: str, rc: int) -> None:
        if rc != 0:
            raise RuntimeError(f"{who}: {_lib.qmk_last_error().decode()} (status {rc})")

    def apply(self) -> None:
        """Makes this engine's options the device's current ones, for the entry points that take no handle
        (``generate_batch``, ``decode_batched``, ``prefill_chunked``, ``generate_static``)."""
        self._done("Engine.apply", _lib.qmk_engine_apply(self._live()))

    def decode(self, input_token_id, embed_weight, layer_weights_packed, final_norm_weight, lm_head_weight,
               cos_table, sin_table, k_cache, v_cache, hidden, act, res, q, k, v, attn_out, mlp_inter,
               norm_out, bmax_vals, bmax_idxs, num_layers, position, max_seq_len, attn_scale):
        """``decode`` of the module (same arguments and result) with this engine's options."""
        _check_table(layer_weights_packed, "decode")
        out = torch.zeros(1, dtype=torch.int32, device=embed_weight.device)
        self._done("decode", _lib.qmk_engine_decode(
            self._live(), int(input_token_id), out.data_ptr(), _ptr(embed_weight), _ptr(layer_weights_packed),
            _ptr(final_norm_weight), _ptr(lm_head_weight), _ptr(cos_table), _ptr(sin_table), _ptr(k_cache),
            _ptr(v_cache), _ptr(hidden), _ptr(norm_out), _ptr(bmax_vals), _ptr(bmax_idxs), int(num_layers),
            int(position), int(max_seq_len), float(attn_scale), _stream()))
        return out

    def generate_nosync(self, first_token_id, num_steps, embed_weight, layer_weights_packed, final_norm_weight,
                        lm_head_weight, cos_table, sin_table, k_cache, v_cache, hidden, act, res, q, k, v,
                        attn_out, mlp_inter, norm_out, bmax_vals, bmax_idxs, output_log, num_layers,
                        start_position, max_seq_len, attn_scale, eos_token_id=151645):
        """``generate_nosync`` of the module (same arguments and result) with this engine's options."""
        _check(output_log.dtype == torch.int32 and output_log.is_cuda and output_log.is_contiguous(),
               "generate_nosync: output_log must be a contiguous int32 CUDA tensor")
        _check(output_log.numel() >= num_steps,
               f"generate_nosync: output_log.numel() ({output_log.numel()}) < num_steps ({num_steps})")
        _check_table(layer_weights_packed, "generate_nosync")
        self._done("generate_nosync", _lib.qmk_engine_generate(
            self._live(), int(first_token_id), int(num_steps), _ptr(embed_weight), _ptr(layer_weights_packed),
            _ptr(final_norm_weight), _ptr(lm_head_weight), _ptr(cos_table), _ptr(sin_table), _ptr(k_cache),
            _ptr(v_cache), _ptr(hidden), _ptr(norm_out), _ptr(bmax_vals), _ptr(bmax_idxs), output_log.data_ptr(),
            int(num_layers), int(start_position), int(max_seq_len), float(attn_scale),
            -1 if eos_token_id is None else int(eos_token_id), 1, _stream()))
        return output_log

    def prefill(self, token_ids, embed_weight, layer_weights_packed, final_norm_weight, lm_head_weight, cos_table,
                sin_table, k_cache, v_cache, hidden, act, res, q, k, v, attn_out, mlp_inter, norm_out,
                bmax_vals, bmax_idxs, num_layers, start_position, max_seq_len, attn_scale):
        """``prefill`` of the module (same arguments) with this engine's options."""
        _check(token_ids.dtype == torch.int32, "token_ids must be int32")
        _check(not token_ids.is_cuda, "prefill: token_ids must be a CPU tensor")
        _check(token_ids.is_contiguous(), "prefill: token_ids must be contiguous")
        if token_ids.numel() == 0:
            return None
        _check_table(layer_weights_packed, "prefill")
        self._done("prefill", _lib.qmk_engine_prefill(
            self._live(), token_ids.data_ptr(), int(token_ids.numel()), _ptr(embed_weight), _ptr(layer_weights_packed),
            _ptr(final_norm_weight), _ptr(cos_table), _ptr(sin_table), _ptr(k_cache), _ptr(v_cache),
            int(num_layers), int(start_position), int(max_seq_len), float(attn_scale), _stream()))


def configure(vocab_size=-1, rope_from_table=-1, split_len=-1, max_ctas=-1, timeout_ms=-1) -> None:
    """Engine options of the current device; negative keeps the present value."""
    rc = _lib.qmk_configure(int(vocab_size), int(rope_from_table), int(split_len), int(max_ctas), int(timeout_ms))
    _check(rc == 0, f"configure failed with status {rc}")


def set_inv_freq(inv_freq: torch.Tensor) -> None:
    """64 fp32 RoPE inverse frequencies (CPU tensor) used for in-kernel angles."""
    _require_cuda()
    t = inv_freq.detach().to("cpu", torch.float32).contiguous()
    _check(t.numel() == 64, "inv_freq must have 64 elements")
    rc = _lib.qmk_set_inv_freq(t.data_ptr())
    _check(rc == 0, f"set_inv_freq failed with status {rc}")


def set_logits_dump(buf) -> None:
    """fp32 CUDA tensor ``[steps, vocab]`` that decode steps fill with all logits, or None."""
    if buf is not None:
        _check(buf.is_cuda and buf.dtype == torch.float32 and buf.is_contiguous(),
               "logits dump must be a contiguous fp32 CUDA tensor")
    _lib.qmk_set_logits_dump(_ptr(buf))


def set_tuning(spin_sleep_ns=-1, l2_evict_first=-1, repl=-1, stream_inflight=-1) -> None:
    """Performance knobs (see include/qwen_megakernel.h); negative keeps a value."""
    _check(_lib.qmk_set_tuning(int(spin_sleep_ns), int(l2_evict_first)) == 0, "set_tuning failed")
    _check(_lib.qmk_set_tuning2(int(repl), int(stream_inflight)) == 0, "set_tuning failed")


WEIGHT_FORMATS = {"fp16": 0, "fp8": 1, "nvfp4": 2}


def set_weight_format(fmt) -> None:
    """"fp16" (default), "fp8" (e4m3 rows with a 16-byte scale trailer) or "nvfp4" (e2m1 pairs + e4m3 block scales +
    trailer; tensor-core entry points only); see include/qwen_megakernel.h."""
    code = WEIGHT_FORMATS[fmt] if isinstance(fmt, str) else int(fmt)
    _check(_lib.qmk_set_weight_format(code) == 0, f"set_weight_format({fmt!r}) failed")


PROFILE_STRIDE = 768


def set_fused(fused=-1, red_copies=-1) -> None:
    """Single-sequence kernel choice: fused (default) or unfused; accumulator copies of the fused kernel's sums."""
    _require_cuda()
    if _lib.qmk_set_fused(int(fused), int(red_copies)) != 0:
        _raise_if_failed("set_fused")


def set_prefill_attention(tensor_core: bool) -> None:
    """Chunked prefill: causal attention on tcgen05 (default) or on the mma.sync kernel."""
    _check(_lib.qmk_set_prefill_attention(int(bool(tensor_core))) == 0, "set_prefill_attention failed")


def set_decode_attention(tensor_core: bool) -> None:
    """Batched decode: per-sequence attention on mma.sync tiles (default) or on the CUDA-core kernel."""
    _check(_lib.qmk_set_decode_attention(int(bool(tensor_core))) == 0, "set_decode_attention failed")


def set_step_overlap(enabled: bool) -> None:
    """Batched decode: launch the kernels of a step as programmatic dependents of one another (default on)."""
    _check(_lib.qmk_set_step_overlap(int(bool(enabled))) == 0, "set_step_overlap failed")


def invalidate_weights() -> None:
    """After editing W_o / W_down in place: the fused kernel's K-major copies are rebuilt at the next call."""
    _require_cuda()
    if _lib.qmk_invalidate_weights() != 0:
        _raise_if_failed("invalidate_weights")


def release_weights(layer_weights_packed=None) -> None:
    """Frees the K-major copies made for this layer table (None: for all tables) on the current device."""
    _require_cuda()
    if _lib.qmk_release_weights(_ptr(layer_weights_packed)) != 0:
        _raise_if_failed("release_weights")


def set_profile_buffer(buf) -> None:
    """int64 CUDA tensor ``[grid, 768]`` receiving per-CTA phase timestamps (ns) of the last step
    of each launch (slot map: include/qwen_megakernel.h), or None."""
    if buf is not None:
        _check(buf.is_cuda and buf.dtype == torch.int64 and buf.is_contiguous(),
               "profile buffer must be a contiguous int64 CUDA tensor")
    _lib.qmk_set_profile_buffer(_ptr(buf))


def generate_static(first_token_id, num_steps, embed_weight, layer_weights_packed, final_norm_weight,
                    lm_head_weight, k_cache, v_cache, norm_out, output_log, num_layers, start_position,
                    max_seq_len, attn_scale, eos_token_id=-1):
    """``generate_nosync`` for callers that cannot allocate device memory while running (a server whose
    cache pool already owns all free HBM, a loop that cannot take cudaMalloc's device-wide sync): same
    kernel, same tokens, scratch in a fixed array inside the library.  ``max_seq_len`` <= 2048.
    Blocks; raises ``RuntimeError`` on any reported error; returns ``output_log``."""
    _require_cuda()
    _check(output_log.dtype == torch.int32 and output_log.is_cuda and output_log.is_contiguous(),
           "generate_static: output_log must be a contiguous int32 CUDA tensor")
    _check(output_log.numel() >= num_steps, "generate_static: output_log is shorter than num_steps")
    _check_table(layer_weights_packed, "generate_static")
    rc = _lib.qmk_generate_static(
        int(first_token_id), int(num_steps), _ptr(embed_weight), _ptr(layer_weights_packed),
        _ptr(final_norm_weight), _ptr(lm_head_weight), _ptr(k_cache), _ptr(v_cache), _ptr(norm_out),
        output_log.data_ptr(), int(num_layers), int(start_position), int(max_seq_len), float(attn_scale),
        -1 if eos_token_id is None else int(eos_token_id), _stream())
    if rc != 0:
        raise RuntimeError(f"generate_static: {_lib.qmk_last_error().decode()} (status {rc})")
    return output_log


MAX_BATCH_SEQUENCES = 4


def generate_batch(first_token_ids, start_positions, num_steps, embed_weight, layer_weights_packed,
                   final_norm_weight, lm_head_weight, cos_table, sin_table, k_caches, v_caches, output_logs,
                   num_layers, max_seq_len, attn_scale, synchronize=True):
    """Greedy decode of 1..4 independent sequences in one persistent launch (weights are streamed once
    per step for all of them).  ``first_token_ids`` / ``start_positions``: one int per sequence;
    ``k_caches`` / ``v_caches``: one fp16 cache tensor pair per sequence (filled by ``prefill``);
    ``output_logs``: one int32 CUDA tensor of >= ``num_steps`` entries per sequence.  All sequences run
    ``num_steps`` steps (no EOS stop).  Raises ``RuntimeError`` on any reported error."""
    _require_cuda()
    n = len(first_token_ids)
    _check(1 <= n <= MAX_BATCH_SEQUENCES, "generate_batch: 1 to 4 sequences per launch")
    _check(len(start_positions) == n and len(k_caches) == n and len(v_caches) == n and len(output_logs) == n,
           "generate_batch: per-sequence lists differ in length")
    for log in output_logs:
        _check(log.dtype == torch.int32 and log.is_cuda and log.is_contiguous() and log.numel() >= num_steps,
               "generate_batch: each output_log must be a contiguous int32 CUDA tensor of >= num_steps entries")
    _check_table(layer_weights_packed, "generate_batch")
    ints = ctypes.c_int * n
    ptrs = ctypes.c_void_p * n
    rc = _lib.qmk_generate_batch(
        n, ints(*[int(t) for t in first_token_ids]), ints(*[int(p) for p in start_positions]), int(num_steps),
        _ptr(embed_weight), _ptr(layer_weights_packed), _ptr(final_norm_weight), _ptr(lm_head_weight),
        _ptr(cos_table), _ptr(sin_table), ptrs(*[_ptr(t) for t in k_caches]), ptrs(*[_ptr(t) for t in v_caches]),
        ptrs(*[_ptr(t) for t in output_logs]), int(num_layers), int(max_seq_len), float(attn_scale),
        1 if synchronize else 0, _stream())
    if rc != 0:
        raise RuntimeError(f"generate_batch: {_lib.qmk_last_error().decode()} (status {rc})")
    return output_logs


MAX_GEMM_BATCH_SEQUENCES = 128


def decode_batched(first_token_ids, start_positions, num_steps, embed_weight, layer_weights_packed,
                   final_norm_weight, lm_head_weight, cos_table, sin_table, k_caches, v_caches, output_logs,
                   num_layers, max_seq_len, attn_scale):
    """``generate_batch`` for up to 128 sequences on the tensor-core path (tcgen05 GEMMs per step instead of
    one persistent kernel; fp16 weights only).  Same arguments and result."""
    _require_cuda()
    n = len(first_token_ids)
    _check(1 <= n <= MAX_GEMM_BATCH_SEQUENCES, "decode_batched: 1 to 128 sequences per call")
    _check(len(start_positions) == n and len(k_caches) == n and len(v_caches) == n and len(output_logs) == n,
           "decode_batched: per-sequence lists differ in length")
    for log in output_logs:
        _check(log.dtype == torch.int32 and log.is_cuda and log.is_contiguous() and log.numel() >= num_steps,
               "decode_batched: each output_log must be a contiguous int32 CUDA tensor of >= num_steps entries")
    _check_table(layer_weights_packed, "decode_batched")
    ints = ctypes.c_int * n
    ptrs = ctypes.c_void_p * n
    rc = _lib.qmk_decode_batched(
        n, ints(*[int(t) for t in first_token_ids]), ints(*[int(p) for p in start_positions]), int(num_steps),
        _ptr(embed_weight), _ptr(layer_weights_packed), _ptr(final_norm_weight), _ptr(lm_head_weight),
        _ptr(cos_table), _ptr(sin_table), ptrs(*[_ptr(t) for t in k_caches]), ptrs(*[_ptr(t) for t in v_caches]),
        ptrs(*[_ptr(t) for t in output_logs]), int(num_layers), int(max_seq_len), float(attn_scale), _stream())
    if rc != 0:
        raise RuntimeError(f"decode_batched: {_lib.qmk_last_error().decode()} (status {rc})")
    return output_logs


def prefill_chunked(token_ids, embed_weight, layer_weights_packed, cos_table, sin_table, k_cache, v_cache,
                    num_layers, start_position, max_seq_len, attn_scale):
    """``prefill`` on the tensor cores (chunks of up to 4096 tokens, tcgen05 GEMMs; fp16 weights only).
    ``token_ids``: CPU int32 tensor.  Blocks; raises ``RuntimeError`` on any reported error."""
    _require_cuda()
    _check((not token_ids.is_cuda) and token_ids.dtype == torch.int32 and token_ids.is_contiguous(),
           "prefill_chunked: token_ids must be a contiguous CPU int32 tensor")
    _check_table(layer_weights_packed, "prefill_chunked")
    rc = _lib.qmk_prefill_chunked(
        token_ids.data_ptr(), int(token_ids.numel()), _ptr(embed_weight), _ptr(layer_weights_packed),
        _ptr(cos_table), _ptr(sin_table), _ptr(k_cache), _ptr(v_cache), int(num_layers), int(start_position),
        int(max_seq_len), float(attn_scale), _stream())
    if rc != 0:
        raise RuntimeError(f"prefill_chunked: {_lib.qmk_last_error().decode()} (status {rc})")
    return None


def prefill_packed(token_lists, embed_weight, layer_weights_packed, cos_table, sin_table, k_caches, v_caches,
                   num_layers, max_seq_len, attn_scale):
    """Several prompts in one tensor-core prefill pass: ``token_lists[s]`` (ints) fills ``k_caches[s]`` / ``v_caches[s]``
    from position 0.  At most 64 sequences and 4096 rows after padding each prompt to a multiple of 128.  Blocks;
    raises ``RuntimeError`` on any reported error."""
    _require_cuda()
    n = len(token_lists)
    _check(n >= 1 and n == len(k_caches) == len(v_caches), "prefill_packed: one cache pair per prompt")
    _check_table(layer_weights_packed, "prefill_packed")
    flat = [int(t) for ids in token_lists for t in ids]
    tok = (ctypes.c_int * max(len(flat), 1))(*flat)
    lens = (ctypes.c_int * n)(*[len(ids) for ids in token_lists])
    kp = (ctypes.c_void_p * n)(*[_ptr(c) for c in k_caches])
    vp = (ctypes.c_void_p * n)(*[_ptr(c) for c in v_caches])
    rc = _lib.qmk_prefill_packed(tok, n, lens, _ptr(embed_weight), _ptr(layer_weights_packed), _ptr(cos_table), _ptr(sin_table),
                                 kp, vp, int(num_layers), int(max_seq_len), float(attn_scale), _stream())
    if rc != 0:
        raise RuntimeError(f"prefill_packed: {_lib.qmk_last_error().decode()} (status {rc})")
    return None


def gemm_f16_tn(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor = None) -> torch.Tensor:
    """``a @ b.T`` in fp32 for fp16 CUDA matrices ``a [m, k]`` and ``b [n, k]`` on the tcgen05 tensor cores
    (m, n multiples of 128; k a multiple of 64)."""
    _require_cuda()
    _check(a.is_cuda and b.is_cuda and a.dtype == torch.float16 and b.dtype == torch.float16 and
           a.is_contiguous() and b.is_contiguous() and a.dim() == 2 and b.dim() == 2 and a.shape[1] == b.shape[1],
           "gemm_f16_tn: contiguous fp16 CUDA matrices [m, k] and [n, k] expected")
    m, k = a.shape
    n = b.shape[0]
    if out is None:
        out = torch.empty(m, n, dtype=torch.float32, device=a.device)
    _check(out.is_cuda and out.dtype == torch.float32 and out.is_contiguous() and tuple(out.shape) == (m, n),
           "gemm_f16_tn: out must be a contiguous fp32 CUDA matrix [m, n]")
    rc = _lib.qmk_gemm_f16_tn(_ptr(a), _ptr(b), _ptr(out), int(m), int(n), int(k), _stream())
    if rc != 0:
        raise RuntimeError(f"gemm_f16_tn failed with status {rc}")
    return out


def gemm_packed_tn(a: torch.Tensor, b: torch.Tensor, weight_format, b2: torch.Tensor = None, mode: str = "plain",
                   box_n: int = 0) -> torch.Tensor:
    """``a @ dequantised(b).T`` with ``b`` kept packed on the device (uint8 ``[n, row_bytes]``: ``"fp8"`` or ``"nvfp4"``
    rows, see ``quantize.pack_rows_fp8`` / ``pack_rows_nvfp4``).  ``mode``: ``"plain"`` -> fp32 ``[m, n]``; ``"splitk"`` ->
    fp32 ``[4, m, n]`` partial matrices; ``"swiglu"`` (``b`` gate, ``b2`` up) -> fp16 ``[m, n]``."""
    _require_cuda()
    fmt = WEIGHT_FORMATS[weight_format] if isinstance(weight_format, str) else int(weight_format)
    code = {"plain": 0, "splitk": 1, "swiglu": 2}[mode]
    _check(a.is_cuda and a.dtype == torch.float16 and a.is_contiguous() and a.dim() == 2,
           "gemm_packed_tn: a must be a contiguous fp16 CUDA matrix [m, k]")
    m, k = a.shape
    row_bytes = {1: k + 16, 2: k // 2 + k // 16 + 16}[fmt]
    for t in (b,) if b2 is None else (b, b2):
        _check(t.is_cuda and t.dtype == torch.uint8 and t.is_contiguous() and t.dim() == 2 and t.shape[1] == row_bytes,
               f"gemm_packed_tn: packed matrices must be contiguous uint8 CUDA tensors [n, {row_bytes}]")
    n = b.shape[0]
    if code == 2:
        out = torch.empty(m, n, dtype=torch.float16, device=a.device)
    else:
        out = torch.empty((4, m, n) if code == 1 else (m, n), dtype=torch.float32, device=a.device)
    rc = _lib.qmk_gemm_packed_tn(_ptr(a), _ptr(b), _ptr(b2), _ptr(out), int(m), int(n), int(k), fmt, code, int(box_n),
                                 _stream())
    if rc != 0:
        raise RuntimeError(f"gemm_packed_tn failed with status {rc}")
    return out


def sync_status() -> int:
    return int(_lib.qmk_sync_status())


def last_error() -> str:
    return _lib.qmk_last_error().decode()


def num_ctas() -> int:
    _require_cuda()
    return int(_lib.qmk_num_ctas())


def scratch_bytes() -> int:
    return int(_lib.qmk_scratch_bytes())


def selftest_wait_timeout(budget_us: int = 200) -> int:
    _require_cuda()
    return int(_lib.qmk_selftest_wait_timeout(int(budget_us)))


def selftest_gemm_wait_timeout(budget_us: int = 300) -> int:
    """Runs the tcgen05 GEMM's bounded wait dry (its loads are never issued); 4 = gave up as designed."""
    _require_cuda()
    return int(_lib.qmk_selftest_gemm_wait_timeout(int(budget_us)))
