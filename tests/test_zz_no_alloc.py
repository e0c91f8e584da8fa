"""The allocation-free decode GEMM must agree with the regular entry point.

`b2_nvfp4_gemm_small_m_noalloc` exists for hosts that may not allocate device memory from inside a
plugin call (a serving loop that owns all of HBM, a latency-critical section, a sandbox); its scratch
is an array built into the library and shared by every call.  Two calls in a row, on different
operands, are compared with `b2_nvfp4_gemm` on the same operands: the second call shows that the
contents the first one left in the shared array do no harm.  The file name sorts last so that a run
stopping at the first failure has already run every other test.
"""

import pytest
import torch

pytestmark = pytest.mark.gpu

TOLERANCE = 2e-3  # relative Frobenius error, the GEMM's stated bar


def _operands(M, N, K, seed):
    from tirx_kernels.basic import nvfp4_gemm as gemm

    g = torch.Generator().manual_seed(seed)
    a = torch.randn(M, K, generator=g).to(torch.bfloat16).cuda()
    b = torch.randn(N, K, generator=g).to(torch.bfloat16).cuda()
    ga, gb = 2688.0 / a.float().abs().max(), 2688.0 / b.float().abs().max()
    A_fp4, A_sf = gemm.quantize_operand(a, ga)
    B_fp4, B_sf = gemm.quantize_operand(b, gb)
    alpha = (1.0 / (ga * gb)).reshape(1).float().cuda()
    return A_fp4, B_fp4, A_sf, B_sf, alpha


def test_matches_the_allocating_entry_point_on_two_calls_in_a_row(native):
    from tirx_kernels.basic import nvfp4_gemm as gemm

    for seed, (M, N, K) in enumerate([(16, 8192, 8192), (100, 2048, 4096)]):
        A_fp4, B_fp4, A_sf, B_sf, alpha = _operands(M, N, K, seed)
        want = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
        got = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
        native.nvfp4_gemm(A_fp4, B_fp4, A_sf, B_sf, alpha, want, M, N, K)
        native.nvfp4_gemm_small_m_noalloc(A_fp4, B_fp4, A_sf, B_sf, alpha, got, M, N, K)
        torch.cuda.synchronize()
        native.nvfp4_gemm_status()
        assert torch.isfinite(got.float()).all()
        assert gemm.relative_frobenius_error(got, want) <= TOLERANCE


def test_rejects_what_does_not_fit_the_built_in_scratch(native):
    z = torch.zeros(1 << 20, dtype=torch.uint8, device="cuda")
    one = torch.ones(1, device="cuda")
    d = torch.empty(1 << 20, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ValueError, match="1 <= M <= 128"):
        native.nvfp4_gemm_small_m_noalloc(z, z, z, z, one, d, 256, 1024, 1024)
    # 128 x 2048 in 8 K ranges would need 8 MiB of partial sums
    with pytest.raises(ValueError, match="built-in scratch"):
        native.nvfp4_gemm_small_m_noalloc(z, z, z, z, one, d, 128, 2048, 16384)
