"""GPU parity of `nvfp4_quantize`: packed bytes and the whole scale buffer must equal the CPU
oracle's, through the C-ABI, on the reference's correctness matrix and at the full benchmark sizes."""

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _module():
    from tirx_kernels.flashinfer.quantization import nvfp4_quantize

    return nvfp4_quantize


def _labels():
    return [c["label"] for c in _module().CONFIGS]


@pytest.mark.parametrize("label", _labels())
def test_reference_config_matrix_is_bit_exact(label, oracle_expected):
    from tirx_kernels.registry import discover_kernels
    from tirx_kernels.runner import run_kernel_test

    kernels = discover_kernels()
    config = next(c for c in kernels["nvfp4_quantize"].CONFIGS if c["label"] == label)
    run_kernel_test("nvfp4_quantize", config, registry=kernels)


def _baseline_input(m, k, outliers):
    """Seeded N(0,1) activations; with `outliers`, 0.1 % of the entries (seeded positions) x 50."""
    g = torch.Generator().manual_seed(42)
    x = torch.randn(m, k, generator=g, dtype=torch.float32)
    if outliers:
        n = -(-m * k // 1000)
        pos = torch.randperm(m * k, generator=g)[:n]
        x.view(-1)[pos] *= 50.0
    x = x.to(torch.bfloat16)
    gs = torch.tensor([2688.0], dtype=torch.float32) / x.float().abs().max()
    return x, gs


@pytest.mark.parametrize("m,k,layout,outliers", [(4096, 7168, "linear", False), (16384, 7168, "128x4", True)])
def test_baseline_shapes_are_bit_exact_at_full_size(m, k, layout, outliers, native):
    import oracle_provider
    from oracle import c_oracle

    x, gs = _baseline_input(m, k, outliers)
    xd, gsd = x.cuda(), gs.cuda()
    out = torch.empty(m, k // 2, dtype=torch.uint8, device="cuda")
    sf = torch.full((native.lib().b2_nvfp4_sf_bytes(m, k, native.SF_LAYOUT_CODES[layout]),), 0xA5,
                    dtype=torch.uint8, device="cuda")
    native.nvfp4_quantize(xd, out, sf, gsd, m, k, "bfloat16", layout)
    torch.cuda.synchronize()
    want_packed, want_sf = c_oracle.nvfp4_quantize(oracle_provider.to_bits(x), "bfloat16", float(gs.item()),
                                                   layout, oracle_provider.probe_mufu(native))
    assert np.array_equal(out.cpu().numpy(), want_packed)
    assert np.array_equal(sf.cpu().numpy(), want_sf)
    # size-independent property: a second launch over the same input is idempotent
    out2, sf2 = torch.empty_like(out), torch.empty_like(sf)
    native.nvfp4_quantize(xd, out2, sf2, gsd, m, k, "bfloat16", layout)
    assert torch.equal(out, out2) and torch.equal(sf, sf2)


def test_row_shards_concatenate_to_the_full_result(native):
    """Quantization shards by rows with no exchange: any 128-row-aligned split gives the same bytes."""
    m, k = 1024, 2048
    x, gs = _baseline_input(m, k, True)
    xd, gsd = x.cuda(), gs.cuda()
    full_out = torch.empty(m, k // 2, dtype=torch.uint8, device="cuda")
    full_sf = torch.empty(m * k // 16, dtype=torch.uint8, device="cuda")
    native.nvfp4_quantize(xd, full_out, full_sf, gsd, m, k, "bfloat16", "128x4")
    parts_out, parts_sf = [], []
    for r0 in range(0, m, 256):
        o = torch.empty(256, k // 2, dtype=torch.uint8, device="cuda")
        s = torch.empty(256 * k // 16, dtype=torch.uint8, device="cuda")
        native.nvfp4_quantize(xd[r0:r0 + 256], o, s, gsd, 256, k, "bfloat16", "128x4")
        parts_out.append(o)
        parts_sf.append(s)
    assert torch.equal(torch.cat(parts_out), full_out) and torch.equal(torch.cat(parts_sf), full_sf)


def test_invalid_arguments_are_rejected_before_launch(native):
    mod = _module()
    with pytest.raises(ValueError):
        mod.get_kernel(dtype="float16", m=4, k=24)
    with pytest.raises(ValueError):
        mod.get_kernel(dtype="float32", m=4, k=32)
    x = torch.zeros(4, 32, dtype=torch.float16, device="cuda")
    gs = torch.ones(1, device="cuda")
    out = torch.empty(4, 16, dtype=torch.uint8, device="cuda")
    sf = torch.empty(8, dtype=torch.uint8, device="cuda")
    with pytest.raises(ValueError, match="k=24"):
        native.nvfp4_quantize(x, out, sf, gs, 4, 24, "float16", "linear")
    with pytest.raises(ValueError, match="m=0"):
        native.nvfp4_quantize(x, out, sf, gs, 0, 32, "float16", "linear")


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_silu_fast_division_equals_div_rn_on_every_input(dtype, native):
    """The SiLU-fused quantizer divides with packed FMAs where that is exact and with div.rn.f32 elsewhere.
    A gate is a 16-bit value, so the whole input domain is 65536 values per dtype: all of them, NaNs,
    infinities, zeros of both signs and subnormals included, must give div.rn.f32's bits, and those must
    be the oracle's (mul.f32, ex2.approx.ftz from the device, add.f32, IEEE division)."""
    import oracle_provider
    from oracle import nvfp4_oracle

    bits = torch.arange(65536, dtype=torch.int32).to(torch.int16)
    gates = bits.view(dtype).float().numpy()
    fast = native.mufu_probe("silu", gates)
    exact = native.mufu_probe("silu_div_rn", gates)
    assert np.array_equal(fast.view(np.uint32), exact.view(np.uint32))
    mufu = oracle_provider.probe_mufu(native)
    finite = np.isfinite(gates)
    with np.errstate(all="ignore"):
        want = nvfp4_oracle.silu_f32(gates[finite], mufu)
    assert np.array_equal(exact[finite].view(np.uint32), np.asarray(want, dtype=np.float32).view(np.uint32))
