"""Generates golden vectors for the quantizers by running flashinfer's own GPU kernels.

    python tests/golden/make_flashinfer_golden.py [out_dir]      (needs a B200)

The reference's tests take their expected bytes from flashinfer at test time
(`flashinfer.quantization.nvfp4_quantize(backend="cute-dsl")`,
tirx_kernels/flashinfer/quantization/nvfp4_quantize.py:418-438, and
`flashinfer.cute_dsl.rmsnorm_fp4quant`, tirx_kernels/flashinfer/norm/rmsnorm_fp4quant.py:1187-1215)
and store none.  This script runs the flashinfer build installed in this image (0.6.11, not the
revision the reference pins) on seeded inputs drawn on the CPU and stores inputs and outputs as
small .npz files, which tests/test_golden_cpu.py replays against the CPU oracle.  Each case is
attempted independently; failures are recorded in MANIFEST.json instead of aborting.
"""

import json
import sys
import traceback
from pathlib import Path

import numpy as np
import torch


def bits(t):
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def u8(t):
    return t.detach().cpu().contiguous().view(torch.uint8).numpy()


QUANT_CASES = [
    # (dtype, m, k, layout, fuse_silu, global_scale)
    ("bfloat16", 128, 1024, "128x4", False, 0.8125),
    ("float16", 13, 1040, "linear", False, 1.37),
    ("float16", 120, 1024, "128x4", False, 0.61),
    ("bfloat16", 128, 1024, "8x4", False, 1.05),
    ("float16", 64, 8208, "128x4", False, 0.93),
    ("bfloat16", 256, 2048, "128x4", False, None),  # None: 448*6/amax, the GEMM's data contract
    ("float16", 128, 1024, "128x4", True, 0.77),
]
RMS_CASES = [
    # (dtype, M, H, block, scale_format, swizzled, global_scale)
    ("bfloat16", 5, 7168, 16, "e4m3", True, None),
    ("float16", 33, 4096, 16, "e4m3", False, None),
    ("bfloat16", 129, 80, 16, "e4m3", True, None),
    ("bfloat16", 16, 2048, 32, "ue8m0", False, None),
    ("float16", 3, 3088, 16, "e4m3", False, 3.25),
]
TORCH_DTYPE = {"float16": torch.float16, "bfloat16": torch.bfloat16}


def quant_case(case, backend):
    from flashinfer import SfLayout
    from flashinfer.quantization import nvfp4_quantize

    dtype, m, k, layout, silu, gs = case
    g = torch.Generator().manual_seed(42)
    a = torch.randn(m, k * (2 if silu else 1), generator=g).to(TORCH_DTYPE[dtype])
    if gs is None:
        gs = float(448.0 * 6.0 / a.float().abs().max())
    gs_t = torch.tensor([gs], dtype=torch.float32, device="cuda")
    enum = {"linear": SfLayout.layout_linear, "128x4": SfLayout.layout_128x4, "8x4": SfLayout.layout_8x4}[layout]
    if silu:
        from flashinfer.quantization import silu_and_mul_nvfp4_quantize

        out, sf = silu_and_mul_nvfp4_quantize(a.cuda(), gs_t, is_sf_swizzled_layout=layout != "linear",
                                              is_sf_8x4_layout=layout == "8x4")
    else:
        out, sf = nvfp4_quantize(a.cuda(), gs_t, sfLayout=enum, backend=backend)
    torch.cuda.synchronize()
    return {"a_bits": bits(a), "global_scale": np.float32(gs_t.item()), "packed": u8(out), "sf": u8(sf).reshape(-1)}


def rms_case(case):
    from flashinfer.norm import rmsnorm_fp4quant

    dtype, M, H, block, fmt, swizzled, gs = case
    g = torch.Generator().manual_seed(42)
    x = torch.randn(M, H, generator=g).to(TORCH_DTYPE[dtype])
    w = torch.randn(H, generator=g).to(TORCH_DTYPE[dtype])
    gs_t = None if gs is None else torch.tensor([gs], dtype=torch.float32, device="cuda")
    y, scales = rmsnorm_fp4quant(x.cuda(), w.cuda(), global_scale=gs_t, eps=1e-6, block_size=block,
                                 scale_format=fmt, is_sf_swizzled_layout=swizzled)
    torch.cuda.synchronize()
    return {"x_bits": bits(x), "w_bits": bits(w), "global_scale": np.float32(1.0 if gs is None else gs),
            "packed": u8(y), "sf": u8(scales).reshape(-1)}


def main():
    out_dir = Path(sys.argv[1] if len(sys.argv) > 1 else "gpurun_out/golden")
    out_dir.mkdir(parents=True, exist_ok=True)
    import flashinfer

    manifest = {"flashinfer_version": getattr(flashinfer, "__version__", "?"),
                "gpu": torch.cuda.get_device_name(0), "cases": []}
    for i, case in enumerate(QUANT_CASES):
        for backend in ("cute-dsl", "cuda"):
            if case[4] and backend == "cuda":
                continue
            name = f"quant_{i}_{backend.replace('-', '')}"
            entry = {"name": name, "kind": "nvfp4_quantize", "backend": backend, "case": list(case)}
            try:
                np.savez_compressed(out_dir / f"{name}.npz", **quant_case(case, backend))
                entry["status"] = "ok"
            except Exception as error:
                entry.update(status="failed", error=f"{type(error).__name__}: {error}",
                             trace=traceback.format_exc()[-1500:])
            manifest["cases"].append(entry)
    for i, case in enumerate(RMS_CASES):
        name = f"rms_{i}"
        entry = {"name": name, "kind": "rmsnorm_fp4quant", "case": list(case)}
        try:
            np.savez_compressed(out_dir / f"{name}.npz", **rms_case(case))
            entry["status"] = "ok"
        except Exception as error:
            entry.update(status="failed", error=f"{type(error).__name__}: {error}",
                         trace=traceback.format_exc()[-1500:])
        manifest["cases"].append(entry)
    (out_dir / "MANIFEST.json").write_text(json.dumps(manifest, indent=1))
    print(json.dumps({c["name"]: c["status"] for c in manifest["cases"]}))


if __name__ == "__main__":
    main()
