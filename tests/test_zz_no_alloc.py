"""The allocation-free decode GEMM: right answers, nothing allocated, its limit enforced.

`b2_nvfp4_gemm_small_m_noalloc` exists for hosts that may not allocate device memory from inside a
plugin call (a serving loop that owns all of HBM, a latency-critical section, a sandbox); its scratch
is an array built into the library and shared by every call.  Two calls in a row, on different
operands, are compared with the CPU oracle and with `b2_nvfp4_gemm` on the same operands: the second
call shows that the contents the first one left in the shared array do no harm.  The file name sorts
last so that a run stopping at the first failure has already run every other test.
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


# the decode shape; a shape whose partial sums fill the 4 MiB array exactly (8 K ranges x 128 x 1024 x 4 B);
# one that takes the 128-row ring
SHAPES = [(16, 8192, 8192), (128, 1024, 8192), (100, 2048, 4096)]


def test_two_calls_in_a_row_match_the_oracle_and_the_allocating_entry_point(native):
    import oracle_provider
    from tirx_kernels.basic import nvfp4_gemm as gemm

    for seed, (M, N, K) in enumerate(SHAPES):
        A_fp4, B_fp4, A_sf, B_sf, alpha = _operands(M, N, K, seed)
        peer = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
        got = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
        native.nvfp4_gemm(A_fp4, B_fp4, A_sf, B_sf, alpha, peer, M, N, K)
        native.nvfp4_gemm_small_m_noalloc(A_fp4, B_fp4, A_sf, B_sf, alpha, got, M, N, K)
        torch.cuda.synchronize()
        native.nvfp4_gemm_status()
        native.nvfp4_gemm_small_m_noalloc_status()
        assert torch.isfinite(got.float()).all()
        want = oracle_provider.gemm_expected(dict(A_fp4=A_fp4, B_fp4=B_fp4, A_sf=A_sf, B_sf=B_sf,
                                                  alpha=float(alpha.item())))
        assert gemm.relative_frobenius_error(got.cpu(), want) <= TOLERANCE
        # same kernel variant and K ranges as the allocating entry point: the same bits
        assert torch.equal(got, peer)


def test_device_memory_does_not_move_across_a_call(native):
    """What the entry point exists for.  The kernels' modules are loaded by a first round of calls (CUDA
    loads a module lazily, on the first launch of any of its kernels, and that moves the figure once);
    from then on the free device memory is the same before and after every call."""
    M, N, K = 16, 8192, 8192
    A_fp4, B_fp4, A_sf, B_sf, alpha = _operands(M, N, K, 7)
    got = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    native.nvfp4_gemm_small_m_noalloc(A_fp4, B_fp4, A_sf, B_sf, alpha, got, M, N, K)
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for _ in range(3):
        native.nvfp4_gemm_small_m_noalloc(A_fp4, B_fp4, A_sf, B_sf, alpha, got, M, N, K)
    torch.cuda.synchronize()
    native.nvfp4_gemm_small_m_noalloc_status()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before


def test_rejects_what_does_not_fit_the_built_in_scratch(native):
    z = torch.zeros(1 << 21, dtype=torch.uint8, device="cuda")
    one = torch.ones(1, device="cuda")
    d = torch.empty(1 << 20, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ValueError, match="1 <= M <= 128"):
        native.nvfp4_gemm_small_m_noalloc(z, z, z, z, one, d, 256, 1024, 1024)
    # 128 x 4608 is 72 tiles of 64 columns; cut into two K ranges (144 CTAs) it would need 4.5 MiB of partial sums
    with pytest.raises(ValueError, match="built-in scratch"):
        native.nvfp4_gemm_small_m_noalloc(z, z, z, z, one, d, 128, 4608, 2048)
