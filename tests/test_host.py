"""CPU tests of the boundary: the C-ABI library builds, loads and exports every symbol the header
declares; the op module validates arguments like the reference binding; nothing computes here."""

import ctypes
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol(built_library):
    header = open(os.path.join(ROOT, "include", "qwen_megakernel.h")).read()
    declared = set(re.findall(r"\b((?:launch_ldg|qmk)_\w+)\s*\(", header))
    assert {"launch_ldg_decode_direct", "launch_ldg_decode_persistent", "launch_ldg_generate_nosync",
            "launch_ldg_prefill"} <= declared
    lib = ctypes.CDLL(built_library)
    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} declared in the header but not exported"
    import qwen_megakernel_C as C
    assert declared == set(C.EXPORTED_SYMBOLS)


def test_engine_handle_argument_checks(built_library):
    """qmk_engine_create refuses null pointers and unknown weight formats before touching a GPU; destroying a null
    handle is a no-op."""
    import qwen_megakernel_C as C
    lib = C._lib
    handle = ctypes.c_void_p()
    assert lib.qmk_engine_create(None, ctypes.byref(handle)) != 0
    cfg = C._EngineConfig(0, 151936, 5, 0, -1, -1, -1, -1, None)
    assert lib.qmk_engine_create(ctypes.byref(cfg), ctypes.byref(handle)) != 0 and not handle
    assert lib.qmk_engine_destroy(None) == 0
    assert lib.qmk_engine_apply(None) != 0


def test_abi_version_handshake(built_library):
    import qwen_megakernel_C as C
    from Model import Qwen06B_architecture as A
    assert C.abi_version() == 2 == A.EXTENSION_ABI_VERSION
    assert C.scratch_bytes() < 8 << 20   # 4 copies x 4 sequences of the exchange area


def test_reference_constants_and_surface(built_library):
    from Model import Qwen06B_architecture as A
    assert (A.NUM_LAYERS, A.NUM_KV_HEADS, A.HEAD_DIM, A.HIDDEN_SIZE, A.INTERMEDIATE_SIZE) == (28, 8, 128, 1024, 3072)
    assert (A.Q_SIZE, A.KV_SIZE, A.MAX_SEQ_LEN, A.VOCAB_SIZE, A.ROPE_THETA) == (2048, 1024, 2048, 151936, 1e6)
    for name in ("load_weights", "_pack_layer_weights", "Decoder", "generate", "_require_megakernel_op"):
        assert hasattr(A, name)
    for name in ("step", "reset", "position", "generate"):
        assert hasattr(A.Decoder, name)
    with pytest.raises(RuntimeError, match="unavailable"):
        A._require_megakernel_op("no_such_op")


def test_pack_layer_weights_layout(built_library):
    from Model.Qwen06B_architecture import _pack_layer_weights
    import synthetic as S
    w = S.make_weights(seed=1, num_layers=2, vocab_size=64)
    t = _pack_layer_weights(w["layer_weights"])
    assert t.dtype == torch.int64 and t.numel() == 2 * 12 and t.data_ptr() % 16 == 0
    tab = t.view(2, 12)
    for li in range(2):
        for j in range(11):
            assert tab[li, j].item() == w["layer_weights"][li * 11 + j].data_ptr()
        assert tab[li, 11].item() == 0


def test_argument_validation_matches_reference_binding(built_library):
    """dtype / device / contiguity / size checks raise RuntimeError before any launch
    (reference: qwen_ops.cpp:142-150, 219-221)."""
    import qwen_megakernel_C as C
    dummy = [torch.zeros(4)] * 19
    with pytest.raises(RuntimeError, match="int32"):
        C.prefill(torch.zeros(3, dtype=torch.int64), *dummy, 1, 0, 16, 0.1)
    with pytest.raises(RuntimeError, match="contiguous"):
        C.prefill(torch.zeros(6, dtype=torch.int32)[::2], *dummy, 1, 0, 16, 0.1)
    assert C.prefill(torch.zeros(0, dtype=torch.int32), *dummy, 1, 0, 16, 0.1) is None
    if not torch.cuda.is_available():
        with pytest.raises(RuntimeError, match="no CUDA device"):
            C.generate_nosync(1, 2, *dummy, torch.zeros(4, dtype=torch.int32), 1, 0, 16, 0.1)
        with pytest.raises(RuntimeError, match="no CUDA device"):
            C.decode(1, *dummy, 1, 0, 16, 0.1)
        with pytest.raises(RuntimeError, match="CUDA device"):
            from Model.Qwen06B_architecture import Decoder
            Decoder(weights={})


def test_stub_tokenizer_roundtrip():
    import synthetic as S
    tok = S.StubTokenizer(eos_token_id=7, vocab_size=100)
    assert tok.encode("5 17 230") == [5, 17, 30]
    assert tok.decode([5, 17]) == "5 17"
    assert tok.apply_chat_template([{"role": "user", "content": "1 2"}]) == "1 2"


def test_build_rejects_a_stack_frame_in_a_decode_megakernel():
    """build.py reads ptxas' report: a decode megakernel with a per-thread stack frame must fail the build."""
    import build
    ok = ("ptxas info    : Function properties for _ZN3qmk23qwen3_decode_megakernelEN4qmkp6ParamsE\n"
          "    8 bytes stack frame, 4 bytes spill stores, 4 bytes spill loads\n"
          "ptxas info    : Function properties for _ZN3qmk17rope_table_kernelEPfi\n"
          "    400 bytes stack frame, 0 bytes spill stores, 0 bytes spill loads\n")
    build.check_stack_frames(ok)          # small frame; other kernels are not held to the limit
    bad = ok.replace("    8 bytes stack frame", "    408 bytes stack frame")
    with pytest.raises(RuntimeError, match="stack frame"):
        build.check_stack_frames(bad)
