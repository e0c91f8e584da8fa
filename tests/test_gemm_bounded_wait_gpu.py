"""One bounded wait of the GEMM kernel is made to run out, without a fault, a trap or an endless loop.

Every device-side wait of `nvfp4_gemm` has a budget; when it runs out the kernel records which role
gave up, the other roles drain, tensor memory is released and the kernel returns.  The test hook
`b2_nvfp4_gemm_inject_test_fault(1)` makes the next launch announce 16 bytes more for its first K slab
than the copies deliver: all copies land and nothing stays in flight, the slab's barrier just never
completes.  With the budget shortened to a few milliseconds the launch must come back by itself,
`b2_nvfp4_gemm_status` must name the MMA role's wait, and the next ordinary launch must be correct.
"""

import time

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture()
def short_waits(native):
    native.nvfp4_gemm_set_wait_budget_ms(5)
    yield native
    native.nvfp4_gemm_inject_test_fault(0)
    native.nvfp4_gemm_set_wait_budget_ms(0)
    native.nvfp4_gemm_set_variant(-1)


@pytest.mark.parametrize("which,M,N,K", [(0, 128, 128, 256), (2, 256, 256, 512), (4, 16, 512, 2048)])
def test_an_expired_wait_ends_the_kernel_and_is_reported(which, M, N, K, short_waits):
    import oracle_provider
    from tirx_kernels.basic import nvfp4_gemm as mod

    native = short_waits
    A_fp4, B_fp4, A_sf, B_sf, alpha, _ = mod.prepare_data(M, N, K)
    alpha_t = torch.tensor([float(alpha)], device="cuda")
    out = torch.zeros(M, N, dtype=torch.bfloat16, device="cuda")
    native.nvfp4_gemm_set_variant(which)
    native.nvfp4_gemm(A_fp4, B_fp4, A_sf, B_sf, alpha_t, out, M, N, K)  # a clean launch first
    torch.cuda.synchronize()
    native.nvfp4_gemm_status()

    native.nvfp4_gemm_inject_test_fault(1)
    began = time.perf_counter()
    native.nvfp4_gemm(A_fp4, B_fp4, A_sf, B_sf, alpha_t, out, M, N, K)
    torch.cuda.synchronize()
    elapsed = time.perf_counter() - began
    assert elapsed < 2.0, f"the kernel took {elapsed:.2f} s to give up with a 5 ms budget"
    with pytest.raises(RuntimeError, match="bounded wait expired .MMA waiting for loaded operands"):
        native.nvfp4_gemm_status()
    native.nvfp4_gemm_status()  # reading cleared the word

    # the fault was for one launch only: the same problem now runs to the right answer
    out.fill_(float("nan"))
    native.nvfp4_gemm(A_fp4, B_fp4, A_sf, B_sf, alpha_t, out, M, N, K)
    torch.cuda.synchronize()
    native.nvfp4_gemm_status()
    want = oracle_provider.gemm_expected(dict(A_fp4=A_fp4, B_fp4=B_fp4, A_sf=A_sf, B_sf=B_sf,
                                              alpha=float(alpha_t.item())))
    assert mod.relative_frobenius_error(out.cpu(), want) <= 2e-3
