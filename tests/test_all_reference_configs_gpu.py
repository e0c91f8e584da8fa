"""Exhaustive sweep: EVERY configuration the reference lists for the four quantizer kernels (2308 in
all) against the CPU oracle, bit for bit.  It takes about eight minutes on a B200 (the oracle is the slow
side), so it only runs when B2_ALL_CONFIGS=1; the default GPU suite samples the same lists.

    B2_ALL_CONFIGS=1 python -m pytest tests/test_all_reference_configs_gpu.py -m gpu -q
"""

import os

import pytest

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(os.environ.get("B2_ALL_CONFIGS") != "1", reason="set B2_ALL_CONFIGS=1 for the full sweep")]

KERNELS = {"nvfp4_quantize": 21, "nvfp4_quantize_per_token": 17, "flashinfer_rmsnorm_fp4quant": 1025,
           "flashinfer_add_rmsnorm_fp4quant": 1245}


@pytest.mark.parametrize("kernel", sorted(KERNELS))
def test_every_reference_config_is_bit_exact(kernel, oracle_expected):
    from tirx_kernels.registry import discover_kernels
    from tirx_kernels.runner import run_kernel_test

    kernels = discover_kernels()
    configs = kernels[kernel].CONFIGS
    assert len(configs) == KERNELS[kernel]
    failures = []
    for config in configs:
        try:
            run_kernel_test(kernel, config, registry=kernels)
        except Exception as error:  # collect, so that one report lists them all
            failures.append(f"{config['label']}: {type(error).__name__}: {str(error)[:160]}")
    assert not failures, f"{len(failures)} of {len(configs)} configs failed:\n" + "\n".join(failures[:20])
