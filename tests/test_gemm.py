"""The tcgen05 GEMM (TMA tiles -> tcgen05.mma -> TMEM -> global) against torch on the same fp16 operands.
Products of fp16 values are exact in fp32 and both sides accumulate in fp32, so the only difference is
summation order: tolerance 1e-3 relative to the row/column magnitudes, far below any layout error."""

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def C(built_library):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import qwen_megakernel_C
    return qwen_megakernel_C


@pytest.mark.parametrize("m,n,k", [(128, 128, 64), (128, 128, 256), (256, 1024, 1024), (512, 3072, 1024), (128, 1024, 3072),
                                   (1024, 2048, 512), (512, 2048, 256)])   # N tiles of 32, 32, 32, 128, 32, 128 and 64 columns on 148 SMs
def test_matches_torch(C, m, n, k):
    g = torch.Generator("cpu").manual_seed(m + n + k)
    a = torch.randn(m, k, generator=g).to(torch.float16).cuda()
    b = torch.randn(n, k, generator=g).to(torch.float16).cuda()
    got = C.gemm_f16_tn(a, b)
    want = a.float() @ b.float().T
    err = float((got - want).abs().max())
    print(f"gemm {m}x{n}x{k}: max abs err {err:.3e} (|want| max {float(want.abs().max()):.1f})")
    assert err < 1e-3 * (k ** 0.5) * 4


def test_every_element_lands_in_its_place(C):
    """Operands that make every output element distinct: A row i = one-hot at column i (scaled), so C row i is
    a scaled copy of B's column i; any swizzle or tile mix-up moves values."""
    m = n = 256
    k = 256
    a = torch.zeros(m, k, dtype=torch.float16)
    a[torch.arange(m), torch.arange(m) % k] = 1.0
    b = (torch.arange(n * k, dtype=torch.float32).reshape(n, k) % 2039).to(torch.float16)
    got = C.gemm_f16_tn(a.cuda(), b.cuda()).cpu()
    want = a.float() @ b.float().T
    assert torch.equal(got, want)


def _packed(fmt, w):
    """(packed uint8 matrix on the GPU, the fp32 matrix it stands for)"""
    import quantize as Q
    if fmt == "fp8":
        q, sc = Q.quantize_rows_fp8(w)
        return Q.pack_rows_fp8(q, sc).cuda(), Q.dequantize_rows_fp8(q, sc)
    vals, sb, ts = Q.quantize_blocks_nvfp4(w)
    return Q.pack_rows_nvfp4(vals, sb, ts).cuda(), Q.dequantize_nvfp4(vals, sb, ts)


@pytest.mark.parametrize("fmt", ["fp8", "nvfp4"])
@pytest.mark.parametrize("m,n,k,box", [(128, 128, 256, 0), (128, 1024, 1024, 32), (256, 2048, 1024, 64), (256, 1024, 3072, 128),
                                       (128, 3072, 2048, 0)])
def test_packed_weights_match_torch(C, fmt, m, n, k, box):
    """B kept packed in device memory (FP8-E4M3 rows / NVFP4 rows) and expanded to fp16 tiles inside the kernel: the
    result must be A times the DEQUANTISED matrix - e4m3 values and e2m1 x block-scale products are exact in fp16,
    accumulation is fp32, the row / tensor scale multiplies the fp32 sum - so only summation order and one fp32
    rounding of the scale separate it from torch: 1e-5 relative to the largest output."""
    g = torch.Generator("cpu").manual_seed(m + n + k)
    a = torch.randn(m, k, generator=g).to(torch.float16)
    packed, deq = _packed(fmt, torch.randn(n, k, generator=g) * 0.05)
    want = a.float() @ deq.T
    got = C.gemm_packed_tn(a.cuda(), packed, fmt, box_n=box).cpu()
    err = float((got - want).abs().max())
    print(f"packed {fmt} gemm {m}x{n}x{k} box {box}: max abs err {err:.3e} (|want| max {float(want.abs().max()):.2f})")
    assert err < 1e-5 * float(want.abs().max()) + 1e-6


@pytest.mark.parametrize("fmt", ["fp8", "nvfp4"])
def test_packed_split_k_and_swiglu_forms(C, fmt):
    """The two other forms a decode step uses: split-K partial matrices (their sum is the product) and the fused
    gate/up pair with the SwiGLU epilogue (fp16 output)."""
    g = torch.Generator("cpu").manual_seed(5)
    m, n, k = 128, 1024, 2048
    a = torch.randn(m, k, generator=g).to(torch.float16)
    packed, deq = _packed(fmt, torch.randn(n, k, generator=g) * 0.05)
    parts = C.gemm_packed_tn(a.cuda(), packed, fmt, mode="splitk").cpu()
    want = a.float() @ deq.T
    assert float((parts.sum(0) - want).abs().max()) < 1e-5 * float(want.abs().max()) + 1e-6
    for z in range(4):     # every part is the product over its own quarter of K
        wz = a[:, z * 512:(z + 1) * 512].float() @ deq[:, z * 512:(z + 1) * 512].T
        assert float((parts[z] - wz).abs().max()) < 1e-5 * float(wz.abs().max()) + 1e-6
    k = 1024
    a = torch.randn(m, k, generator=g).to(torch.float16)
    gate_p, gate = _packed(fmt, torch.randn(n, k, generator=g) * 0.05)
    up_p, up = _packed(fmt, torch.randn(n, k, generator=g) * 0.05)
    for box in (32, 64):
        act = C.gemm_packed_tn(a.cuda(), gate_p, fmt, b2=up_p, mode="swiglu", box_n=box).cpu().float()
        gv, uv = a.float() @ gate.T, a.float() @ up.T
        want = torch.nn.functional.silu(gv) * uv
        assert float((act - want).abs().max()) < 2e-3 * float(want.abs().max()) + 1e-4    # fp16 output rounding


@pytest.mark.parametrize("fmt", ["fp8", "nvfp4"])
def test_packed_elements_land_in_their_places(C, fmt):
    """One-hot rows of A pick single columns of the packed matrix: every output element is one dequantised weight,
    so a wrong nibble order, swizzle segment, block scale or row scale shows up as a wrong VALUE, not as noise."""
    m, n, k = 256, 256, 256
    a = torch.zeros(m, k, dtype=torch.float16)
    a[torch.arange(m), torch.arange(m) % k] = 1.0
    g = torch.Generator("cpu").manual_seed(9)
    w = torch.randn(n, k, generator=g) * torch.linspace(0.01, 1.0, n)[:, None]      # rows (and blocks) of different scale
    packed, deq = _packed(fmt, w)
    got = C.gemm_packed_tn(a.cuda(), packed, fmt).cpu()
    want = a.float() @ deq.T
    assert torch.allclose(got, want, rtol=3e-7, atol=0.0)


def test_bad_shapes_are_refused(C):
    a = torch.zeros(100, 64, dtype=torch.float16, device="cuda")
    b = torch.zeros(128, 64, dtype=torch.float16, device="cuda")
    with pytest.raises(RuntimeError):
        C.gemm_f16_tn(a, b)


def test_bounded_wait_reports_timeout_and_frees_tmem(C):
    """Loads that never come: the kernel's waits give up after their budget, report status 4, release TMEM and
    return; the context stays usable and the next GEMM (which needs TMEM on the same SM) is exact."""
    for _ in range(3):
        assert C.selftest_gemm_wait_timeout(300) == 4
    a = torch.ones(128, 64, dtype=torch.float16, device="cuda")
    assert torch.equal(C.gemm_f16_tn(a, a), torch.full((128, 128), 64.0, device="cuda"))
