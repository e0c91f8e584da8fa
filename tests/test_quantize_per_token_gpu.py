"""GPU parity of `nvfp4_quantize_per_token`: packed bytes, the whole scale buffer (padding
included) and the per-row scales bit-exact against the CPU oracle on every reference config."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _module():
    from tirx_kernels.flashinfer.quantization import nvfp4_quantize_per_token

    return nvfp4_quantize_per_token


@pytest.mark.parametrize("config", _module().CONFIGS, ids=lambda c: c["label"])
def test_reference_config_is_bit_exact(config, oracle_expected):
    from tirx_kernels.registry import discover_kernels
    from tirx_kernels.runner import run_kernel_test

    run_kernel_test("nvfp4_quantize_per_token", config, registry=discover_kernels())


@pytest.mark.parametrize("dtype,m,k,layout", [("bfloat16", 300, 7168, "128x4"), ("float16", 9, 16384, "linear"), ("bfloat16", 3, 32768, "128x4"),
                                             ("bfloat16", 5, 32, "8x4"), ("float16", 129, 4112, "128x4")])
def test_shapes_beyond_the_reference_list(dtype, m, k, layout, oracle_expected):
    """The hidden size of the throughput benchmark, a row too long for the register-resident path,
    the smallest swizzled shape, and ragged rows and columns together."""
    _module().run_test(dtype=dtype, m=m, k=k, sf_layout=layout)


def test_rejects_what_the_reference_rejects(native):
    mod = _module()
    for kwargs, message in ((dict(dtype="float32", m=4, k=64), "Unsupported dtype"),
                            (dict(dtype="float16", m=4, k=64, sf_layout="4x4"), "Unsupported sf_layout"),
                            (dict(dtype="float16", m=0, k=64), "must be >= 1"),
                            (dict(dtype="float16", m=4, k=24), "k % 16 != 0")):
        with pytest.raises(ValueError, match=message):
            mod.get_kernel(**kwargs)


def test_full_size_round_trip(native):
    """16384 x 7168 (the reference's largest bench shape): decode(e2m1 * e4m3) * token scale stays
    within the format's error bound of the input, and padding scales are zero."""
    mod = _module()
    m, k = 16384, 7168
    a, gs_inv = mod.prepare_data("bfloat16", m, k, "128x4")
    out, sf, pts = mod._alloc_outputs(m, k, "128x4")
    ex = mod.get_kernel("bfloat16", m, k, "128x4").config["launcher"]
    ex(a.view(-1), out.view(-1), sf, pts, m, gs_inv)
    torch.cuda.synchronize()
    mod._self_check(a, gs_inv, out, sf, pts, m, k, "128x4")
