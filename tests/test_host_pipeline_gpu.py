"""The host-buffer pipeline produces the bytes of a single whole-batch launch."""

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype,m,k,layout,chunks", [("bfloat16", 1000, 2048, "128x4", 4), ("float16", 640, 1040, "linear", 3),
                                                    ("bfloat16", 4096, 7168, "128x4", 8), ("float16", 50, 512, "8x4", 2)])
def test_pipeline_matches_one_launch(dtype, m, k, layout, chunks, native):
    from tirx_kernels.flashinfer.quantization import nvfp4_quantize as quant
    from tirx_kernels.flashinfer.quantization.host_pipeline import HostQuantizePipeline

    a, gs = quant.prepare_data(dtype, m, k, layout)
    out, sf = quant._alloc_outputs(m, k, layout)
    ex = quant.get_kernel(dtype, m, k, layout).config["launcher"]
    quant._run_launch(ex, a, gs, out, sf, m, k, layout)
    x_pin = a.cpu().pin_memory()
    out_pin = torch.empty(m, k // 2, dtype=torch.uint8).pin_memory()
    sf_pin = torch.full((sf.numel(),), 0xA5, dtype=torch.uint8).pin_memory()
    pipeline = HostQuantizePipeline(dtype, m, k, layout, chunks=chunks)
    pipeline(x_pin, gs, out_pin, sf_pin)
    pipeline(x_pin, gs, out_pin, sf_pin)
    torch.cuda.synchronize()
    assert torch.equal(out_pin, out.cpu())
    assert torch.equal(sf_pin, sf.cpu())
