"""Generates golden vectors for the quantizers by running flashinfer's own GPU kernels.

    python tests/golden/make_flashinfer_golden.py [out_dir]      (needs a B200)

The reference's tests take their expected bytes from flashinfer at test time
(`flashinfer.quantization.nvfp4_quantize(backend="cute-dsl")`,
tirx_kernels/flashinfer/quantization/nvfp4_quantize.py:418-438, and
`flashinfer.cute_dsl.rmsnorm_fp4quant`, tirx_kernels/flashinfer/norm/rmsnorm_fp4quant.py:1187-1215,
`flashinfer.norm.add_rmsnorm_fp4quant`, tirx_kernels/flashinfer/norm/add_rmsnorm_fp4quant.py:1508-1555,
`nvfp4_quantize(..., per_token_activation=True)`, .../quantization/nvfp4_quantize_per_token.py:278-291)
and store none.  This script runs the flashinfer build installed in this image (0.6.11, not the
revision the reference pins) on seeded inputs drawn on the CPU and stores its OUTPUTS as small
.npz files (inputs are regenerated from the seed by `quant_inputs` / `rms_inputs`; their SHA-256
is stored to detect generator drift).  It also records the values the B200 returned for every
hardware-approximate instruction the CPU oracle needs on these cases (mufu_tables.npz), so that
tests/test_golden_cpu.py can replay the oracle bit for bit on a machine without a GPU.
Each case is attempted independently; failures are recorded in MANIFEST.json.
"""

import hashlib
import json
import sys
import traceback
from pathlib import Path

import numpy as np
import torch

REPO = Path(__file__).resolve().parents[2]
for entry in (REPO, REPO / "tirx-kernels_b200"):
    if str(entry) not in sys.path:
        sys.path.insert(0, str(entry))

TORCH_DTYPE = {"float16": torch.float16, "bfloat16": torch.bfloat16}

QUANT_CASES = [
    # (dtype, m, k, layout, global_scale)   None: 448*6/amax, the GEMM's data contract
    ("bfloat16", 32, 512, "128x4", 0.8125),
    ("float16", 13, 1040, "linear", 1.37),
    ("float16", 40, 256, "128x4", 0.61),
    ("bfloat16", 24, 512, "8x4", 1.05),
    ("float16", 8, 8208, "128x4", 0.93),
    ("bfloat16", 64, 1024, "128x4", None),
]
RMS_CASES = [
    # (dtype, M, H, block, scale_format, swizzled, global_scale)
    ("bfloat16", 3, 7168, 16, "e4m3", True, None),
    ("float16", 9, 4096, 16, "e4m3", False, None),
    ("bfloat16", 129, 80, 16, "e4m3", True, None),
    ("bfloat16", 8, 2048, 32, "ue8m0", False, None),
    ("float16", 3, 3088, 16, "e4m3", False, 3.25),
]
PER_TOKEN_CASES = [
    # (dtype, m, k, layout, zero_row); the inverse global scale is 1 / (448 * 6)
    ("float16", 13, 1040, "linear", False),
    ("bfloat16", 40, 1024, "128x4", True),
    ("float16", 13, 1024, "8x4", False),
    ("bfloat16", 6, 8256, "128x4", False),
]
ADD_CASES = [
    # (dtype, M, H, block, scale_format, swizzled, both_layouts, global_scale)
    ("bfloat16", 5, 4096, 16, "e4m3", True, False, None),
    ("float16", 7, 1536, 16, "e4m3", False, True, 3.25),
    ("bfloat16", 4, 2048, 32, "ue8m0", False, False, None),
    ("bfloat16", 1, 32768, 16, "e4m3", False, False, None),   # the reference spreads this row over two CTAs
    ("bfloat16", 3, 7168, 16, "e4m3", True, False, None),
    ("float16", 17, 64, 16, "e4m3", False, False, None),
]


def bits(t):
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def u8(t):
    return t.detach().cpu().contiguous().view(torch.uint8).numpy()


def digest(*arrays) -> str:
    h = hashlib.sha256()
    for a in arrays:
        h.update(np.ascontiguousarray(a).tobytes())
    return h.hexdigest()


def quant_inputs(case):
    dtype, m, k, layout, gs = case
    g = torch.Generator().manual_seed(42)
    a = torch.randn(m, k, generator=g).to(TORCH_DTYPE[dtype])
    if gs is None:
        gs = float(448.0 * 6.0 / a.float().abs().max())
    return a, float(np.float32(gs))


def rms_inputs(case):
    dtype, M, H, block, fmt, swizzled, gs = case
    g = torch.Generator().manual_seed(42)
    x = torch.randn(M, H, generator=g).to(TORCH_DTYPE[dtype])
    w = torch.randn(H, generator=g).to(TORCH_DTYPE[dtype])
    return x, w, float(1.0 if gs is None else gs)


def per_token_inputs(case):
    dtype, m, k, layout, zero_row = case
    g = torch.Generator().manual_seed(42)
    a = torch.randn(m, k, generator=g).to(TORCH_DTYPE[dtype])
    if zero_row:
        a[0].zero_()
    return a, float(np.float32(1.0 / (448.0 * 6.0)))


def run_per_token(case):
    from flashinfer import SfLayout
    from flashinfer.quantization import nvfp4_quantize

    a, gs_inv = per_token_inputs(case)
    gs_t = torch.tensor([gs_inv], dtype=torch.float32, device="cuda")
    enum = {"linear": SfLayout.layout_linear, "128x4": SfLayout.layout_128x4, "8x4": SfLayout.layout_8x4}[case[3]]
    out, sf, pts = nvfp4_quantize(a.cuda(), gs_t, sfLayout=enum, backend="cuda", per_token_activation=True)
    torch.cuda.synchronize()
    return u8(out), u8(sf).reshape(-1), pts.detach().cpu().float().numpy().reshape(-1)


def add_inputs(case):
    dtype, M, H, block, fmt, swizzled, both, gs = case
    g = torch.Generator().manual_seed(42)
    x = torch.randn(M, H, generator=g).to(TORCH_DTYPE[dtype])
    r = torch.randn(M, H, generator=g).to(TORCH_DTYPE[dtype])
    w = torch.randn(H, generator=g).to(TORCH_DTYPE[dtype])
    return x, r, w, float(1.0 if gs is None else gs)


def run_add(case):
    from flashinfer.norm import add_rmsnorm_fp4quant

    dtype, M, H, block, fmt, swizzled, both, gs = case
    x, r, w, _ = add_inputs(case)
    gs_t = None if gs is None else torch.tensor([gs], dtype=torch.float32, device="cuda")
    residual = r.cuda()
    result = add_rmsnorm_fp4quant(x.cuda(), residual, w.cuda(), global_scale=gs_t, eps=1e-6, block_size=block,
                                  scale_format=fmt, is_sf_swizzled_layout=swizzled, output_both_sf_layouts=both)
    torch.cuda.synchronize()
    out = {"packed": u8(result[0]), "sf": u8(result[1]).reshape(-1), "residual": bits(residual)}
    if both:
        out["sf_unswizzled"] = u8(result[2]).reshape(-1)
    return out


def run_quant(case, backend):
    from flashinfer import SfLayout
    from flashinfer.quantization import nvfp4_quantize

    a, gs = quant_inputs(case)
    gs_t = torch.tensor([gs], dtype=torch.float32, device="cuda")
    enum = {"linear": SfLayout.layout_linear, "128x4": SfLayout.layout_128x4, "8x4": SfLayout.layout_8x4}[case[3]]
    out, sf = nvfp4_quantize(a.cuda(), gs_t, sfLayout=enum, backend=backend)
    torch.cuda.synchronize()
    return u8(out), u8(sf).reshape(-1)


def run_rms(case):
    from flashinfer.norm import rmsnorm_fp4quant

    dtype, M, H, block, fmt, swizzled, gs = case
    x, w, _ = rms_inputs(case)
    gs_t = None if gs is None else torch.tensor([gs], dtype=torch.float32, device="cuda")
    y, scales = rmsnorm_fp4quant(x.cuda(), w.cuda(), global_scale=gs_t, eps=1e-6, block_size=block,
                                 scale_format=fmt, is_sf_swizzled_layout=swizzled)
    torch.cuda.synchronize()
    return u8(y), u8(scales).reshape(-1)


def record_mufu_tables(out_dir: Path) -> None:
    """Runs the CPU oracle on every case with the device probe behind it and stores what it asked for."""
    from oracle import c_oracle
    from oracle import nvfp4_oracle as o
    from tirx_kernels import _native

    recorder = o.RecordingMufu(o.ProbeMufu(_native.mufu_probe))
    for case in QUANT_CASES:  # both restatements: the C one asks for whole per-code tables
        a, gs = quant_inputs(case)
        o.nvfp4_quantize(bits(a), case[0], gs, case[3], False, recorder)
        c_oracle.nvfp4_quantize(bits(a), case[0], gs, case[3], recorder)
    for case in RMS_CASES:
        x, w, gs = rms_inputs(case)
        o.rmsnorm_fp4quant(bits(x), bits(w), case[0], gs, 1e-6, case[3], case[4], case[5], recorder)
        if case[3] == 16:
            c_oracle.rmsnorm_fp4quant(bits(x), bits(w), case[0], gs, 1e-6, case[5], recorder)
    for case in PER_TOKEN_CASES:
        a, gs_inv = per_token_inputs(case)
        o.nvfp4_quantize_per_token(bits(a), case[0], gs_inv, case[3], recorder)
    for case in ADD_CASES:
        x, r, w, gs = add_inputs(case)
        o.add_rmsnorm_fp4quant(bits(x), bits(r), bits(w), case[0], gs, 1e-6, case[3], case[4], case[5], recorder)
    np.savez_compressed(out_dir / "mufu_tables.npz", **recorder.arrays())


def main():
    out_dir = Path(sys.argv[1] if len(sys.argv) > 1 else "golden_out")
    out_dir.mkdir(parents=True, exist_ok=True)
    import flashinfer

    manifest = {"flashinfer_version": getattr(flashinfer, "__version__", "?"),
                "gpu": torch.cuda.get_device_name(0), "torch": torch.__version__, "cases": []}
    for i, case in enumerate(QUANT_CASES):
        entry = {"name": f"quant_{i}", "kind": "nvfp4_quantize", "case": list(case)}
        try:
            a, gs = quant_inputs(case)
            packed, sf = run_quant(case, "cute-dsl")
            packed_cuda, sf_cuda = run_quant(case, "cuda")
            entry["cuda_backend_identical"] = bool(np.array_equal(packed, packed_cuda) and np.array_equal(sf, sf_cuda))
            entry["input_sha256"] = digest(bits(a), np.float32(gs))
            np.savez_compressed(out_dir / f"quant_{i}.npz", packed=packed, sf=sf, global_scale=np.float32(gs))
            entry["status"] = "ok"
        except Exception as error:
            entry.update(status="failed", error=f"{type(error).__name__}: {error}", trace=traceback.format_exc()[-1200:])
        manifest["cases"].append(entry)
    for i, case in enumerate(RMS_CASES):
        entry = {"name": f"rms_{i}", "kind": "rmsnorm_fp4quant", "case": list(case)}
        try:
            x, w, gs = rms_inputs(case)
            packed, sf = run_rms(case)
            entry["input_sha256"] = digest(bits(x), bits(w), np.float32(gs))
            np.savez_compressed(out_dir / f"rms_{i}.npz", packed=packed, sf=sf, global_scale=np.float32(gs))
            entry["status"] = "ok"
        except Exception as error:
            entry.update(status="failed", error=f"{type(error).__name__}: {error}", trace=traceback.format_exc()[-1200:])
        manifest["cases"].append(entry)
    for i, case in enumerate(PER_TOKEN_CASES):
        entry = {"name": f"pertoken_{i}", "kind": "nvfp4_quantize_per_token", "case": list(case)}
        try:
            a, gs_inv = per_token_inputs(case)
            packed, sf, pts = run_per_token(case)
            entry["input_sha256"] = digest(bits(a), np.float32(gs_inv))
            np.savez_compressed(out_dir / f"pertoken_{i}.npz", packed=packed, sf=sf, token_scale=pts,
                                gs_inv=np.float32(gs_inv))
            entry["status"] = "ok"
        except Exception as error:
            entry.update(status="failed", error=f"{type(error).__name__}: {error}", trace=traceback.format_exc()[-1200:])
        manifest["cases"].append(entry)
    for i, case in enumerate(ADD_CASES):
        entry = {"name": f"add_{i}", "kind": "add_rmsnorm_fp4quant", "case": list(case)}
        try:
            x, r, w, gs = add_inputs(case)
            out = run_add(case)
            entry["input_sha256"] = digest(bits(x), bits(r), bits(w), np.float32(gs))
            np.savez_compressed(out_dir / f"add_{i}.npz", global_scale=np.float32(gs), **out)
            entry["status"] = "ok"
        except Exception as error:
            entry.update(status="failed", error=f"{type(error).__name__}: {error}", trace=traceback.format_exc()[-1200:])
        manifest["cases"].append(entry)
    try:
        record_mufu_tables(out_dir)
        manifest["mufu_tables"] = "ok"
    except Exception as error:
        manifest["mufu_tables"] = f"failed: {type(error).__name__}: {error}"
    (out_dir / "MANIFEST.json").write_text(json.dumps(manifest, indent=1))
    print(json.dumps({c["name"]: c["status"] for c in manifest["cases"]}), manifest["mufu_tables"])


if __name__ == "__main__":
    main()
