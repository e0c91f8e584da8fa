"""Live differential against flashinfer's own GPU kernels at the benchmarked shapes.

The reference takes its expected bytes from flashinfer at test time, on the same inputs, for every
configuration: `flashinfer.quantization.nvfp4_quantize(backend="cute-dsl")`
(tirx_kernels/flashinfer/quantization/nvfp4_quantize.py:418-438, compared at :479-481),
`flashinfer.norm.rmsnorm_fp4quant` (tirx_kernels/flashinfer/norm/rmsnorm_fp4quant.py:1187-1215, :1405)
and, for the GEMM's operands, `flashinfer.nvfp4_quantize(..., sfLayout=layout_128x4, do_shuffle=False)`
(tirx_kernels/basic/nvfp4_gemm.py:49-61).  These tests do the same with the flashinfer build that is
installed beside this package, byte for byte and at full size: the 4096 x 7168 linear and the
16384 x 7168 swizzled quantization with outliers, the 8192 x 7168 RMSNorm + quantization, and both
operands of the 8192^3 GEMM.  Where flashinfer cannot be imported, or cannot build its kernel on a
machine without network access, the test is skipped with that reason.
"""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _flashinfer():
    try:
        import flashinfer  # noqa: F401
        from flashinfer import SfLayout
        from flashinfer.quantization import nvfp4_quantize
    except Exception as error:  # not installed, or its import needs something this machine lacks
        pytest.skip(f"flashinfer is not importable here: {type(error).__name__}: {error}")
    return SfLayout, nvfp4_quantize


def _flashinfer_quantize(a, gs, layout: str):
    """(packed bytes, flat scale bytes) of flashinfer's quantizer; the back-end the reference names first."""
    SfLayout, nvfp4_quantize = _flashinfer()
    enum = {"linear": SfLayout.layout_linear, "128x4": SfLayout.layout_128x4, "8x4": SfLayout.layout_8x4}[layout]
    failures = []
    for backend in ("cute-dsl", "cuda"):
        try:
            out, sf = nvfp4_quantize(a, gs.reshape(1).float(), sfLayout=enum, backend=backend)
            torch.cuda.synchronize()
            return out.view(torch.uint8), sf.view(torch.uint8).reshape(-1), backend
        except Exception as error:
            failures.append(f"{backend}: {type(error).__name__}: {str(error)[:200]}")
    pytest.skip("flashinfer could not build or run nvfp4_quantize here: " + " | ".join(failures))


def _baseline_input(m, k, outliers):
    g = torch.Generator().manual_seed(42)
    x = torch.randn(m, k, generator=g, dtype=torch.float32)
    if outliers:
        pos = torch.randperm(m * k, generator=g)[: -(-m * k // 1000)]
        x.view(-1)[pos] *= 50.0
    x = x.to(torch.bfloat16)
    gs = torch.tensor([2688.0], dtype=torch.float32) / x.float().abs().max()
    return x.cuda(), gs.cuda()


def _assert_same_bytes(got, want, what):
    got, want = got.reshape(-1), want.reshape(-1)
    assert got.numel() == want.numel(), f"{what}: {got.numel()} bytes against flashinfer's {want.numel()}"
    differing = int((got != want).sum())
    assert differing == 0, f"{what}: {differing} of {got.numel()} bytes differ from flashinfer"


@pytest.mark.parametrize("m,k,layout,outliers", [(4096, 7168, "linear", False), (16384, 7168, "128x4", True)])
def test_nvfp4_quantize_equals_flashinfer_at_the_benchmarked_shapes(m, k, layout, outliers, native):
    x, gs = _baseline_input(m, k, outliers)
    want_packed, want_sf, backend = _flashinfer_quantize(x, gs, layout)
    out = torch.empty(m, k // 2, dtype=torch.uint8, device="cuda")
    sf = torch.full((native.lib().b2_nvfp4_sf_bytes(m, k, native.SF_LAYOUT_CODES[layout]),), 0xA5,
                    dtype=torch.uint8, device="cuda")
    native.nvfp4_quantize(x, out, sf, gs, m, k, "bfloat16", layout)
    torch.cuda.synchronize()
    print(f"flashinfer back-end: {backend}")
    _assert_same_bytes(out, want_packed, "packed E2M1")
    _assert_same_bytes(sf, want_sf, "scale buffer (padding included)")


def test_rmsnorm_fp4quant_equals_flashinfer_at_the_benchmarked_shape(native):
    """8192 x 7168 bf16, gamma = 1 + 0.1 N(0,1), eps 1e-6, swizzled E4M3 scales: run_test's own launch
    compared with flashinfer through the expected-value hook the module offers."""
    _flashinfer()
    try:
        from flashinfer.norm import rmsnorm_fp4quant as fi_rmsnorm_fp4quant
    except Exception as error:
        pytest.skip(f"flashinfer.norm.rmsnorm_fp4quant is not importable here: {type(error).__name__}: {error}")
    from tirx_kernels import _checks, runner
    from tirx_kernels.flashinfer.norm import rmsnorm_fp4quant as rms

    config = next(c for c in rms.BENCH_CONFIGS if c["case"] == "bench_nv_swizzled_large")
    calls = []

    def provider(kernel, **kw):
        assert kernel == "flashinfer_rmsnorm_fp4quant"
        cfg = kw["config"]
        try:
            y, scales = fi_rmsnorm_fp4quant(kw["x"].contiguous(), kw["weight"].contiguous(),
                                            global_scale=kw["global_scale"].reshape(1).float(), eps=float(cfg["eps"]),
                                            block_size=int(cfg["block_size"]), scale_format=str(cfg["scale_format"]),
                                            is_sf_swizzled_layout=bool(cfg["swizzled"]))
            torch.cuda.synchronize()
        except Exception as error:
            pytest.skip(f"flashinfer could not build or run rmsnorm_fp4quant here: {type(error).__name__}: "
                        f"{str(error)[:300]}")
        M, H = int(cfg["M"]), int(cfg["H"])
        layout = "128x4" if cfg["swizzled"] else "linear"
        logical = _checks.logical_scale_bytes(scales.view(torch.uint8), M, H // int(cfg["block_size"]), layout)
        calls.append((M, H))
        return y.view(torch.uint8).cpu(), logical.cpu()

    runner.set_reference_provider(provider)
    try:
        runner.run_kernel_test("flashinfer_rmsnorm_fp4quant", config)
    finally:
        runner.set_reference_provider(None)
    assert calls == [(8192, 7168)]


def test_gemm_operand_bytes_equal_flashinfer(native):
    """`prepare_data(8192, 8192, 8192)` quantizes A and B with this package's kernel where the reference
    calls flashinfer: the bytes the GEMM consumes must be the ones the reference's GEMM would consume."""
    from tirx_kernels.basic import nvfp4_gemm as gemm

    M = N = K = 8192
    A_fp4, B_fp4, A_sf, B_sf, alpha, _, A_origin, B_origin = gemm.prepare_data(M, N, K, return_origin=True)
    for name, origin, packed, sf in (("A", A_origin, A_fp4, A_sf), ("B", B_origin, B_fp4, B_sf)):
        gs = (448 * 6 / origin.float().abs().nan_to_num().max()).reshape(1)
        want_packed, want_sf, _ = _flashinfer_quantize(origin, gs, "128x4")
        _assert_same_bytes(packed, want_packed, f"{name}: packed E2M1")
        _assert_same_bytes(sf, want_sf, f"{name}: swizzled scales")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_silu_fused_quantizer_against_flashinfer_composition(dtype, native):
    """The SiLU-fused quantizer has no fused counterpart in the flashinfer build beside this package (the
    reference compares with `silu_and_mul_nvfp4_quantize`, nvfp4_quantize.py:418-438).  What that build does
    have is the composition the fused kernel is defined to equal: `silu_and_mul` (gate|up -> the input
    dtype) followed by `nvfp4_quantize`.  Two comparisons: this package's plain quantizer on flashinfer's
    SiLU output must equal flashinfer's quantizer byte for byte (the quantizer stage alone), and the fused
    kernel must agree with the composition up to the rare element where the two SiLU implementations round
    an fp32 intermediate differently (each such element can move one packed byte by one E2M1 step or, at a
    block maximum, one scale byte): the differing count is printed and bounded.  Measured on a B200: bf16
    0 of 7,340,032 packed bytes and 0 of 917,504 scale bytes; fp16 2 packed bytes and 0 scale bytes."""
    _flashinfer()
    try:
        from flashinfer.activation import silu_and_mul
    except Exception as error:
        pytest.skip(f"flashinfer.activation.silu_and_mul is not importable here: {type(error).__name__}: {error}")
    m, k, layout = 4096, 3584, "128x4"
    name = {torch.bfloat16: "bfloat16", torch.float16: "float16"}[dtype]
    g = torch.Generator().manual_seed(42)
    x = torch.randn(m, 2 * k, generator=g, dtype=torch.float32).to(dtype).cuda()
    gs = torch.tensor([1.25], device="cuda")
    try:
        activated = silu_and_mul(x)
        torch.cuda.synchronize()
    except Exception as error:
        pytest.skip(f"flashinfer could not build or run silu_and_mul here: {type(error).__name__}: {str(error)[:200]}")
    want_packed, want_sf, backend = _flashinfer_quantize(activated, gs, layout)
    sf_bytes = native.lib().b2_nvfp4_sf_bytes(m, k, native.SF_LAYOUT_CODES[layout])
    # stage 2 alone: the plain quantizer on flashinfer's activated tensor
    out = torch.empty(m, k // 2, dtype=torch.uint8, device="cuda")
    sf = torch.empty(sf_bytes, dtype=torch.uint8, device="cuda")
    native.nvfp4_quantize(activated.contiguous(), out, sf, gs, m, k, name, layout)
    torch.cuda.synchronize()
    _assert_same_bytes(out, want_packed, "quantizer stage: packed E2M1")
    _assert_same_bytes(sf, want_sf, "quantizer stage: scale buffer")
    # the fused kernel against the composition
    fused_out = torch.empty_like(out)
    fused_sf = torch.empty_like(sf)
    native.nvfp4_quantize(x, fused_out, fused_sf, gs, m, k, name, layout, fuse_silu=True)
    torch.cuda.synchronize()
    packed_diff = int((fused_out.reshape(-1) != want_packed.reshape(-1)).sum())
    sf_diff = int((fused_sf.reshape(-1) != want_sf.reshape(-1)).sum())
    print(f"{name}: {packed_diff} of {fused_out.numel()} packed bytes and {sf_diff} of {fused_sf.numel()} scale bytes "
          f"differ from silu_and_mul + nvfp4_quantize ({backend})")
    assert packed_diff <= fused_out.numel() * 1e-5
    assert sf_diff <= fused_sf.numel() * 1e-5
