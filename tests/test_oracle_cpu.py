"""CPU checks of the oracle itself: format conversions, layouts, the two restatements against
each other, and the self-contained checks the reference carries for this path."""

import numpy as np
import pytest
import torch

from oracle import c_oracle
from oracle import nvfp4_oracle as o


def _bits(t):
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def test_e4m3_encode_matches_torch_cast_and_saturates():
    rng = np.random.default_rng(0)
    v = np.concatenate([np.linspace(0, 448, 100001, dtype=np.float32),
                        rng.uniform(0, 448, 100000).astype(np.float32),
                        rng.uniform(0, 2.0**-5, 20000).astype(np.float32), o.E4M3_VALUES[:127]])
    expected = torch.from_numpy(v).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    assert np.array_equal(o.e4m3_encode(v), expected)
    # torch's cast yields NaN above 464; the PTX conversion saturates to 448 (0x7E)
    assert list(o.e4m3_encode(np.array([449.0, 465.0, 1e9, np.inf], dtype=np.float32))) == [0x7E] * 4
    assert o.e4m3_encode(np.array([np.nan], dtype=np.float32))[0] == 0x7F


def test_e4m3_and_e2m1_round_trip_every_code():
    assert np.array_equal(o.e4m3_encode(o.E4M3_VALUES[:127]), np.arange(127))
    assert np.array_equal(o.e4m3_encode(o.E4M3_VALUES[128:255]), np.arange(128, 255))
    assert np.array_equal(o.e2m1_encode(o.E2M1_VALUES), np.arange(16))


def test_e2m1_ties_go_to_even_and_saturate():
    ties = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.5, 1e9], dtype=np.float32)
    assert [o.E2M1_VALUES[c] for c in o.e2m1_encode(ties)] == [0, 1, 1, 2, 2, 4, 4, 6, 6]
    assert list(o.e2m1_encode(-ties)) == [c | 8 for c in o.e2m1_encode(ties)]
    assert o.e2m1_encode(np.array([-0.0], dtype=np.float32))[0] == 0x8


@pytest.mark.parametrize("layout", ["128x4", "8x4"])
@pytest.mark.parametrize("m,cols", [(1, 1), (13, 65), (120, 64), (129, 5), (256, 516)])
def test_swizzled_offsets_are_a_bijection_into_the_padded_buffer(layout, m, cols):
    pad = o.padded_sf_cols(cols)
    tile = 8 if layout == "8x4" else 128
    rows_padded = -(-m // tile) * tile
    off = o.sf_offsets(layout, np.arange(rows_padded)[:, None], np.arange(pad)[None, :], pad).reshape(-1)
    assert np.array_equal(np.sort(off), np.arange(rows_padded * pad))
    assert o.sf_buffer_size(m, cols, layout) == rows_padded * pad


def test_bf16_and_f16_products_round_once():
    rng = np.random.default_rng(1)
    a = rng.integers(0, 1 << 16, 200000).astype(np.uint16)
    b = rng.integers(0, 1 << 16, 200000).astype(np.uint16)
    for dtype, tdt in ((o.BF16, torch.bfloat16), (o.F16, torch.float16)):
        ta = torch.from_numpy(a.view(np.int16)).view(tdt)
        tb = torch.from_numpy(b.view(np.int16)).view(tdt)
        want = (ta.double() * tb.double()).to(tdt).float().numpy()
        got = o.mul_16bit(a, b, dtype)
        ok = np.isnan(want) | (want == got)
        assert ok.all()


@pytest.mark.parametrize("dtype,tdt", [(o.BF16, torch.bfloat16), (o.F16, torch.float16)])
@pytest.mark.parametrize("m,k,layout", [(1, 16, "linear"), (13, 1040, "linear"), (120, 1024, "128x4"),
                                        (128, 1040, "128x4"), (13, 1024, "8x4"), (64, 8208, "128x4")])
def test_c_and_numpy_quantizers_agree(dtype, tdt, m, k, layout):
    g = torch.Generator().manual_seed(7)
    bits = _bits(torch.randn(m, k, generator=g).to(tdt))
    a = o.nvfp4_quantize(bits, dtype, 0.83, layout)
    b = c_oracle.nvfp4_quantize(bits, dtype, 0.83, layout)
    assert np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1])


@pytest.mark.parametrize("dtype,tdt", [(o.BF16, torch.bfloat16), (o.F16, torch.float16)])
@pytest.mark.parametrize("M,H,swizzled", [(17, 64, False), (129, 80, True), (3, 3072, False), (3, 3088, True),
                                          (3, 6160, False), (5, 7168, True), (3, 16400, False), (2, 32768, False)])
def test_c_and_numpy_rmsnorm_agree(dtype, tdt, M, H, swizzled):
    g = torch.Generator().manual_seed(9)
    x = _bits(torch.randn(M, H, generator=g).to(tdt))
    w = _bits(torch.randn(H, generator=g).to(tdt))
    a = o.rmsnorm_fp4quant(x, w, dtype, 21.0, 1e-6, swizzled=swizzled, sf_fill=0xA5)
    b = c_oracle.rmsnorm_fp4quant(x, w, dtype, 21.0, 1e-6, swizzled=swizzled, sf_fill=0xA5)
    assert np.array_equal(a[0], b[0]) and np.array_equal(a[1].reshape(-1), b[1].reshape(-1))


def test_quantizer_output_decodes_close_to_the_input():
    g = torch.Generator().manual_seed(42)
    x = torch.randn(256, 2048, generator=g).to(torch.bfloat16)
    gs = np.float32(2688.0 / x.float().abs().max().item())
    packed, sf = o.nvfp4_quantize(_bits(x), o.BF16, gs, "128x4")
    deq = o.dequantize_nvfp4(packed, sf, "128x4", gs)
    ref = x.float().numpy()
    assert np.linalg.norm(deq - ref) / np.linalg.norm(ref) < 0.12
    assert np.array_equal(deq, c_oracle.dequantize_nvfp4(packed, sf, "128x4", gs))


@pytest.mark.parametrize("block_size,scale_format", [(16, "e4m3"), (32, "ue8m0"), (32, "e4m3")])
def test_rmsnorm_oracle_passes_the_reference_math_check(block_size, scale_format):
    """rtol 0.5 / atol 2.0 against an fp32 RMSNorm: rmsnorm_fp4quant.py _assert_math :1334-1344."""
    g = torch.Generator().manual_seed(3)
    x = torch.randn(33, 4096, generator=g).to(torch.float16)
    w = torch.randn(4096, generator=g).to(torch.float16)
    gs = 3.25
    packed, sf = o.rmsnorm_fp4quant(_bits(x), _bits(w), o.F16, gs, 1e-6, block_size, scale_format)
    if block_size == 16 or scale_format == "e4m3":
        deq = o.dequantize_nvfp4(packed, sf, "linear", gs, block_size)
    else:
        deq = o.dequantize_mxfp4(packed, sf, "linear", block_size)
    ref = o.rmsnorm_reference_f32(_bits(x), _bits(w), o.F16, 1e-6)
    assert np.isfinite(deq).all()
    assert np.all(np.abs(deq - ref) <= 2.0 + 0.5 * np.abs(ref))


def test_zero_global_scale_gives_signed_zero_values_and_zero_scales():
    """rmsnorm_fp4quant.py :1325-1332."""
    g = torch.Generator().manual_seed(4)
    x = torch.randn(3, 4096, generator=g).to(torch.float16)
    w = torch.randn(4096, generator=g).to(torch.float16)
    packed, sf = o.rmsnorm_fp4quant(_bits(x), _bits(w), o.F16, 0.0, 1e-6)
    assert not np.any(packed & 0x77) and not np.any(sf)


def test_cluster_reduction_tree_is_restated():
    cfg = o.source_config(65536)
    assert (cfg["cluster_n"], cfg["tpr"], cfg["vec_blocks"]) == (2, 256, 16)
    assert o.source_config(1048576)["cluster_n"] == 16
    g = torch.Generator().manual_seed(5)
    x = _bits(torch.randn(2, 65536, generator=g).to(torch.bfloat16))
    s = o.rmsnorm_sum_of_squares(x, o.BF16)
    ref = (o.bits_to_f32(x, o.BF16).astype(np.float64) ** 2).sum(-1)
    assert np.allclose(s, ref, rtol=1e-6)


def test_add_rmsnorm_configuration_follows_the_reference_thresholds():
    """_source_config of add_rmsnorm_fp4quant.py :354-363: four row tiles in one CTA, two per cluster CTA."""
    assert o.add_source_config(16384)["cluster_n"] == 1
    assert o.add_source_config(16400)["cluster_n"] == 1 and o.add_source_config(16400)["tpr"] == 256
    for h, n in ((32768, 2), (131072, 4), (262144, 8), (524288, 16)):
        assert o.add_source_config(h)["cluster_n"] == n
    assert o.add_source_config(32768)["tpr"] == 128  # the cluster CTAs of this row use 128 threads


def test_add_rmsnorm_restatement_is_self_consistent():
    rng = np.random.default_rng(5)
    M, H = 5, 512
    x = o.f32_to_bits(rng.standard_normal((M, H)).astype(np.float32), "bfloat16")
    r = o.f32_to_bits(rng.standard_normal((M, H)).astype(np.float32), "bfloat16")
    w = o.f32_to_bits((1 + 0.1 * rng.standard_normal(H)).astype(np.float32), "bfloat16")
    out = o.add_rmsnorm_fp4quant(x, r, w, "bfloat16", 1.0, 1e-6, swizzled=True)
    h = o.bits_to_f32(x, "bfloat16") + o.bits_to_f32(r, "bfloat16")
    assert np.array_equal(out["residual"], o.f32_to_bits(h.astype(np.float32), "bfloat16"))
    hr = o.bits_to_f32(out["residual"], "bfloat16")
    want = hr / np.sqrt((h * h).mean(axis=-1, keepdims=True) + 1e-6) * o.bits_to_f32(w, "bfloat16")
    deq = o.unpack_e2m1(out["y"]).reshape(M, -1, 16) * o.e4m3_decode(out["scale"])[..., None]
    assert np.abs(deq.reshape(M, H) - want).max() <= 0.5 * np.abs(want).max()
    assert np.allclose(o.bits_to_f32(out["y_norm"], "bfloat16"), want, rtol=2e-2, atol=2e-2)
    # the swizzled buffer holds exactly the logical codes
    assert np.array_equal(o.logical_scales(out["scale_buffer"], M, H // 16, "128x4"), out["scale"])
    # zero residual and unit weight reduce to the plain block recipe on x * rstd
    zeros = np.zeros_like(x)
    ones = o.f32_to_bits(np.ones(H, dtype=np.float32), "bfloat16")
    plain = o.add_rmsnorm_fp4quant(x, zeros, ones, "bfloat16", 1.0, 1e-6)
    assert np.array_equal(plain["residual"], x)


def test_per_token_restatement_properties():
    rng = np.random.default_rng(9)
    m, k = 7, 1040
    x = rng.standard_normal((m, k)).astype(np.float32)
    x[0] = 0.0
    bits = o.f32_to_bits(x, "float16")
    packed, sf, token = o.nvfp4_quantize_per_token(bits, "float16", 1.0 / 2688.0, "128x4")
    assert token[0] == 0.0 and not packed[0].any()
    amax = np.abs(o.bits_to_f32(bits, "float16")).max(axis=-1)
    assert np.array_equal(token[1:], (amax[1:] * np.float32(1.0 / 2688.0)).astype(np.float32))
    # scaling a row by two doubles its token scale and leaves its codes unchanged
    bits2 = o.f32_to_bits(2.0 * o.bits_to_f32(bits, "float16"), "float16")
    packed2, sf2, token2 = o.nvfp4_quantize_per_token(bits2, "float16", 1.0 / 2688.0, "128x4")
    assert np.array_equal(token2, 2.0 * token)
    same = np.mean(packed2 == packed)
    assert same > 0.99  # rcp.approx of the doubled scale may move a handful of codes by one step
    # padding columns (65 -> 68) and padding rows (7 -> 128) of the swizzled buffer are zero
    logical = o.logical_scales(sf, m, k // 16, "128x4")
    assert sf.sum() == logical.sum()


def _random_gemm_operands(M, N, K, seed):
    rng = np.random.default_rng(seed)
    pad = lambda rows: -(-rows // 128) * 128
    a = rng.integers(0, 256, size=(M, K // 2), dtype=np.uint8)
    b = rng.integers(0, 256, size=(N, K // 2), dtype=np.uint8)
    a_sf = rng.integers(0x20, 0x60, size=pad(M) * K // 16, dtype=np.uint8)  # finite, moderate E4M3 codes
    b_sf = rng.integers(0x20, 0x60, size=pad(N) * K // 16, dtype=np.uint8)
    return a, b, a_sf, b_sf


def test_gemm_oracle_on_sampled_rows_equals_those_rows_of_the_full_product():
    a, b, a_sf, b_sf = _random_gemm_operands(200, 128, 512, seed=3)
    full = o.nvfp4_gemm(a, b, a_sf, b_sf, 2.0 ** -9)
    rows = np.array([0, 7, 31, 32, 127, 128, 199])
    assert np.array_equal(o.nvfp4_gemm(a, b, a_sf, b_sf, 2.0 ** -9, rows=rows), full[rows])


def test_torch_side_gemm_checker_agrees_with_the_oracle():
    """`_checks.dequantized_matmul_fp32` is what run_test holds the GEMM to at full size; here it runs on
    the CPU, on the oracle's own operands."""
    import torch

    from tirx_kernels import _checks

    a, b, a_sf, b_sf = _random_gemm_operands(256, 384, 1024, seed=4)
    want = o.nvfp4_gemm(a, b, a_sf, b_sf, 2.0 ** -9)
    got = _checks.dequantized_matmul_fp32(torch.from_numpy(a), torch.from_numpy(b), torch.from_numpy(a_sf),
                                          torch.from_numpy(b_sf), 2.0 ** -9, row_chunk=100)
    want_t = torch.from_numpy(want.view(np.int16)).view(torch.bfloat16).float()
    assert float((got.float() - want_t).norm() / want_t.norm()) <= 2e-4
