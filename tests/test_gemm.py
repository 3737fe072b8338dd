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
