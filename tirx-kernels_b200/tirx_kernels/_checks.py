"""Torch-side helpers shared by the kernel modules' ``run_test`` / ``run_gpu``.

Byte-format decoding (packed E2M1, E4M3 / UE8M0 block scales, the three scale-factor
layouts), guard regions, and the roofline annotation of benchmark records.  Everything
here runs on whatever device its tensors live on; none of it is on the launch path.
"""

from __future__ import annotations

import json
import os
from pathlib import Path

E2M1_TABLE = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0]
GUARD_ELEMENTS = 128
GUARD_BYTE = 0xA5


def ceil_div(a: int, b: int) -> int:
    return -(-a // b)


def padded_sf_cols(sf_cols: int) -> int:
    return ceil_div(sf_cols, 4) * 4


def sf_numel(m: int, sf_cols: int, layout: str) -> int:
    if layout == "linear":
        return m * sf_cols
    tile = 8 if layout == "8x4" else 128
    return ceil_div(m, tile) * tile * padded_sf_cols(sf_cols)


def sf_offsets(layout: str, m: int, sf_cols: int, device):
    """int64 [m, sf_cols] byte offsets of the logical scale (r, c) inside a layout's buffer."""
    import torch

    rows = torch.arange(m, device=device, dtype=torch.int64)[:, None]
    cols = torch.arange(sf_cols, device=device, dtype=torch.int64)[None, :]
    pad = padded_sf_cols(sf_cols)
    if layout == "linear":
        return rows * sf_cols + cols
    if layout == "128x4":
        return (rows // 128) * (128 * pad) + (cols // 4) * 512 + (rows % 32) * 16 + ((rows % 128) // 32) * 4 + cols % 4
    if layout == "8x4":
        return (rows // 8) * (ceil_div(pad, 4) * 32) + (cols // 4) * 32 + (rows % 8) * 4 + cols % 4
    raise ValueError(f"unknown sf layout {layout!r}")


def logical_scale_bytes(sf, m: int, sf_cols: int, layout: str):
    return sf.reshape(-1)[sf_offsets(layout, m, sf_cols, sf.device)]


def unpack_e2m1(packed):
    """uint8 [m, k/2] -> float32 [m, k]; the low nibble holds the even element."""
    import torch

    m = packed.shape[0]
    nibbles = torch.stack((packed & 0x0F, packed >> 4), dim=-1).reshape(m, -1).long()
    table = torch.tensor(E2M1_TABLE, device=packed.device, dtype=torch.float32)
    return table[nibbles]


def dequantize(packed, sf, layout: str, *, block_size: int = 16, scale_format: str = "e4m3", global_scale=1.0):
    """value = e2m1 * scale (E4M3 scale divided by the global encode scale, or 2**(UE8M0 - 127))."""
    import torch

    values = unpack_e2m1(packed)
    m, k = values.shape
    raw = logical_scale_bytes(sf, m, k // block_size, layout)
    if scale_format == "e4m3":
        scales = raw.view(torch.float8_e4m3fn).float() / float(global_scale)
    else:
        scales = torch.pow(2.0, raw.int() - 127)
    return (values.view(m, -1, block_size) * scales[..., None]).reshape(m, k)


def dequantized_matmul_fp32(A_fp4, B_fp4, A_sf, B_sf, alpha: float, *, row_chunk: int = 2048):
    """bf16 [M, N] of alpha * dequantize(A) @ dequantize(B)^T in fp32 with TF32 off, on the device of
    the operands: the checker the GEMM is held to at sizes a CPU oracle cannot afford in full.  A is
    decoded in row chunks so that the temporaries stay small beside the operands."""
    import torch

    M, N = A_fp4.shape[0], B_fp4.shape[0]
    k = A_fp4.shape[1] * 2
    tf32 = torch.backends.cuda.matmul.allow_tf32
    precision = torch.get_float32_matmul_precision()
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.set_float32_matmul_precision("highest")
    try:
        b = torch.empty(N, k, dtype=torch.float32, device=B_fp4.device)
        sf_b = logical_scale_bytes(B_sf, N, k // 16, "128x4").view(torch.float8_e4m3fn)
        for r0 in range(0, N, row_chunk):
            r1 = min(N, r0 + row_chunk)
            b[r0:r1] = (unpack_e2m1(B_fp4[r0:r1]).view(r1 - r0, -1, 16) * sf_b[r0:r1].float()[..., None]).reshape(r1 - r0, k)
        out = torch.empty(M, N, dtype=torch.bfloat16, device=A_fp4.device)
        sf_a = logical_scale_bytes(A_sf, M, k // 16, "128x4").view(torch.float8_e4m3fn)
        for r0 in range(0, M, row_chunk):
            r1 = min(M, r0 + row_chunk)
            a = (unpack_e2m1(A_fp4[r0:r1]).view(r1 - r0, -1, 16) * sf_a[r0:r1].float()[..., None]).reshape(r1 - r0, k)
            out[r0:r1] = (torch.mm(a, b.t()) * float(alpha)).to(torch.bfloat16)
        return out
    finally:
        torch.backends.cuda.matmul.allow_tf32 = tf32
        torch.set_float32_matmul_precision(precision)


def padding_mask(m: int, sf_cols: int, layout: str, device):
    """bool mask over a swizzled buffer: True where no logical (row < m, col < sf_cols) scale lives."""
    import torch

    mask = torch.ones(sf_numel(m, sf_cols, layout), dtype=torch.bool, device=device)
    mask[sf_offsets(layout, m, sf_cols, device).reshape(-1)] = False
    return mask


def with_guard(numel: int, dtype, device, fill):
    """A tensor of `numel` elements followed by GUARD_ELEMENTS guard elements set to `fill`."""
    import torch

    backing = torch.empty(numel + GUARD_ELEMENTS, dtype=dtype, device=device)
    backing[numel:].fill_(fill)
    return backing, backing[:numel]


# ---- roofline annotation ---------------------------------------------------------------------
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
NOMINAL_NVFP4_TFLOPS = 9000.0  # dense; 4x the dense bf16 rate of the same tensor cores


def measured_peaks() -> tuple[dict, str]:
    """(peaks, "measured" | "fallback"): the pool's measured copy bandwidth and bf16 GEMM rate."""
    candidates = [os.environ.get("B200_MEASURED_PEAKS")] if os.environ.get("B200_MEASURED_PEAKS") else []
    here = Path(__file__).resolve()
    candidates += [str(parent / "MEASURED_PEAKS.json") for parent in here.parents[:4]]
    for candidate in candidates:
        try:
            with open(candidate) as handle:
                data = json.load(handle)
            if "hbm_gbs" in data:
                return data, "measured"
        except (OSError, ValueError):
            continue
    return dict(FALLBACK_PEAKS), "fallback"


def roofline_hbm(algorithmic_bytes: int, microseconds: float) -> dict:
    peaks, source = measured_peaks()
    achieved = algorithmic_bytes / (microseconds * 1e-6) / 1e9
    return {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
            "frac": achieved / peaks["hbm_gbs"], "peak_source": source, "algorithmic_bytes": algorithmic_bytes}


def roofline_nvfp4(flops: int, microseconds: float) -> dict:
    """Tensor roofline of the block-scaled FP4 GEMM.

    The pool measures a dense bf16 GEMM; the dense NVFP4 rate of the same tensor cores is 4x
    the bf16 rate, so the denominator is 4 x the measured bf16 burst figure.  The fraction of
    the nominal 9 PFLOP/s is reported beside it.
    """
    peaks, source = measured_peaks()
    achieved = flops / (microseconds * 1e-6) / 1e12
    peak = 4.0 * peaks["bf16_tflops"]
    return {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
            "frac": achieved / peak, "peak_source": f"4 x {source} bf16 burst",
            "frac_of_nominal_9pf": achieved / NOMINAL_NVFP4_TFLOPS, "flops": flops}
