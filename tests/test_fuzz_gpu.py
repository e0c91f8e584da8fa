"""Seeded random shapes beyond the reference's own config lists, each checked bit for bit against the CPU
oracle through the kernel modules' `run_test` (quantizers) or within the stated tolerance (GEMM).

The reference's lists pin round row lengths; these cases walk the dispatch boundaries in between: row
lengths that are odd multiples of the block size, row counts around the 128-row padding of the swizzled
layouts, lengths on both sides of every kernel-selection threshold (flat / row kernel, register-resident /
shared-memory / cluster RMSNorm, short-A GEMM ring, K ranges)."""

import random

import pytest
import torch

pytestmark = pytest.mark.gpu

DTYPES = ("float16", "bfloat16")


def _quantize_cases():
    rng = random.Random(1234)
    cases = []
    for _ in range(28):
        m = rng.choice([1, 2, 7, 31, 127, 128, 129, 255, 300, 1023, 1024, 1025, 2050])
        k = 16 * rng.choice([1, 2, 3, 5, 8, 17, 64, 127, 128, 129, 448, 515, 1024, 1025])
        cases.append((rng.choice(DTYPES), m, k, rng.choice(["linear", "128x4", "8x4"]), rng.random() < 0.3,
                      rng.random() < 0.2))
    return cases


@pytest.mark.parametrize("dtype,m,k,layout,silu,pdl", _quantize_cases())
def test_quantize_random_shapes(dtype, m, k, layout, silu, pdl, oracle_expected):
    from tirx_kernels.flashinfer.quantization import nvfp4_quantize

    nvfp4_quantize.run_test(dtype=dtype, m=m, k=k, sf_layout=layout, fuse_silu=silu, enable_pdl=pdl)


def _per_token_cases():
    rng = random.Random(99)
    cases = []
    for _ in range(14):
        m = rng.choice([1, 3, 64, 127, 129, 500, 1024, 1500])
        k = 16 * rng.choice([1, 4, 9, 64, 128, 200, 448, 1024, 1100, 2048])
        cases.append((rng.choice(DTYPES), m, k, rng.choice(["linear", "128x4", "8x4"]), rng.random() < 0.3))
    return cases


@pytest.mark.parametrize("dtype,m,k,layout,zero_row", _per_token_cases())
def test_per_token_random_shapes(dtype, m, k, layout, zero_row, oracle_expected):
    from tirx_kernels.flashinfer.quantization import nvfp4_quantize_per_token

    nvfp4_quantize_per_token.run_test(dtype=dtype, m=m, k=k, sf_layout=layout, zero_row=zero_row)


def _norm_cases(seed, count):
    rng = random.Random(seed)
    cases = []
    for _ in range(count):
        block = rng.choice([16, 16, 32])
        scale_format = "e4m3" if block == 16 else "ue8m0"
        H = block * rng.choice([4, 5, 8, 13, 32, 63, 64, 100, 128, 224, 255, 256, 448, 512, 640, 1024])
        if block == 16 and H < 64:
            H = 64
        M = rng.choice([1, 2, 5, 33, 127, 128, 130, 513])
        cases.append(dict(dtype=rng.choice(DTYPES), H=H, M=M, block_size=block, scale_format=scale_format,
                          swizzled=rng.random() < 0.5, enable_pdl=rng.random() < 0.2,
                          eps=rng.choice([1e-4, 1e-5, 1e-6])))
    return cases


@pytest.mark.parametrize("case", _norm_cases(7, 28), ids=lambda c: f"{c['dtype'][:2]}_m{c['M']}_h{c['H']}_b{c['block_size']}")
def test_rmsnorm_random_shapes(case, oracle_expected):
    from tirx_kernels.flashinfer.norm import rmsnorm_fp4quant as mod

    case = dict(case)
    rng = random.Random(case["H"] * 31 + case["M"])
    mode = rng.choice(["computed", "one", "nonunit"]) if case["scale_format"] == "e4m3" else "none"
    cfg = mod._cfg("fuzz", case.pop("dtype"), case.pop("H"), global_scale_mode=mode, **case)
    mod.run_test(**cfg)


@pytest.mark.parametrize("case", _norm_cases(11, 24), ids=lambda c: f"{c['dtype'][:2]}_m{c['M']}_h{c['H']}_b{c['block_size']}")
def test_add_rmsnorm_random_shapes(case, oracle_expected):
    from tirx_kernels.flashinfer.norm import add_rmsnorm_fp4quant as mod

    case = dict(case)
    rng = random.Random(case["H"] * 17 + case["M"])
    mode = rng.choice(["none", "one", "nonunit"]) if case["scale_format"] == "e4m3" else "none"
    cfg = mod._cfg("fuzz", case.pop("dtype"), case.pop("H"), global_scale_mode=mode,
                   output_both_sf_layouts=rng.random() < 0.4, output_norm=rng.random() < 0.4, **case)
    mod.run_test(**cfg)


def _gemm_cases():
    rng = random.Random(5)
    cases = []
    for _ in range(12):
        M = rng.choice([1, 5, 16, 32, 33, 100, 128, 129, 300, 513])
        N = 128 * rng.choice([1, 2, 3, 5, 8, 11, 16])
        K = 256 * rng.choice([1, 2, 3, 8, 9, 16, 32])
        cases.append((M, N, K))
    return cases


@pytest.mark.parametrize("M,N,K", _gemm_cases())
def test_gemm_random_shapes(M, N, K, native):
    import oracle_provider
    from tirx_kernels.basic import nvfp4_gemm as mod

    A_fp4, B_fp4, A_sf, B_sf, alpha, _ = mod.prepare_data(M, N, K)
    alpha_t = torch.tensor([float(alpha)], device="cuda")
    out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    native.nvfp4_gemm(A_fp4, B_fp4, A_sf, B_sf, alpha_t, out, M, N, K)
    torch.cuda.synchronize()
    native.nvfp4_gemm_status()
    want = oracle_provider.gemm_expected(dict(A_fp4=A_fp4, B_fp4=B_fp4, A_sf=A_sf, B_sf=B_sf,
                                              alpha=float(alpha_t.item())))
    assert torch.isfinite(out.float()).all()
    assert mod.relative_frobenius_error(out.cpu(), want) <= 2e-3  # the workload definition's bar
