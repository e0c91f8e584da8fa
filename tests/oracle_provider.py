"""Bridges the CPU oracle into `tirx_kernels.runner.set_reference_provider` for the tests.

The oracle computes every byte on the host; the only thing taken from the device is the value
of each hardware-approximate instruction, one instruction per element, through b2_mufu_probe.
"""

import numpy as np
import torch

from oracle import c_oracle, nvfp4_oracle


def to_bits(tensor: torch.Tensor) -> np.ndarray:
    """fp16/bf16 tensor (any device) -> uint16 numpy storage."""
    return tensor.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def probe_mufu(native) -> nvfp4_oracle.ProbeMufu:
    return nvfp4_oracle.ProbeMufu(native.mufu_probe)


def make_provider(native, *, prefer_c: bool = True):
    mufu = probe_mufu(native)

    def provider(kernel: str, **kw):
        if kernel == "nvfp4_quantize":
            bits = to_bits(kw["a"])
            gs = float(kw["global_scale"].item())
            if prefer_c and not kw["fuse_silu"]:
                packed, sf = c_oracle.nvfp4_quantize(bits, kw["dtype"], gs, kw["sf_layout"], mufu)
            else:
                packed, sf = nvfp4_oracle.nvfp4_quantize(bits, kw["dtype"], gs, kw["sf_layout"],
                                                         kw["fuse_silu"], mufu)
            return torch.from_numpy(packed), torch.from_numpy(sf)
        if kernel == "nvfp4_quantize_per_token":
            packed, sf, pts = nvfp4_oracle.nvfp4_quantize_per_token(
                to_bits(kw["a"]), kw["dtype"], float(kw["gs_inv"].item()), kw["sf_layout"], mufu)
            return torch.from_numpy(packed), torch.from_numpy(sf), torch.from_numpy(pts)
        if kernel == "flashinfer_rmsnorm_fp4quant":
            cfg = kw["config"]
            packed, sf = nvfp4_oracle.rmsnorm_fp4quant(
                to_bits(kw["x"]), to_bits(kw["weight"]), cfg["input_dtype"], float(kw["global_scale"].item()),
                float(cfg["eps"]), int(cfg["block_size"]), str(cfg["scale_format"]), bool(cfg["swizzled"]), mufu)
            M, H = int(cfg["M"]), int(cfg["H"])
            cols = H // int(cfg["block_size"])
            layout = "128x4" if cfg["swizzled"] else "linear"
            logical = nvfp4_oracle.logical_scales(sf, M, cols, layout)
            return torch.from_numpy(packed), torch.from_numpy(np.ascontiguousarray(logical))
        if kernel == "flashinfer_add_rmsnorm_fp4quant":
            cfg = kw["config"]
            dtype = cfg["input_dtype"]
            out = nvfp4_oracle.add_rmsnorm_fp4quant(
                to_bits(kw["x"]), to_bits(kw["residual"]), to_bits(kw["weight"]), dtype,
                float(kw["global_scale"].item()), float(cfg["eps"]), int(cfg["block_size"]),
                str(cfg["scale_format"]), False, mufu)
            tdtype = {"float16": torch.float16, "bfloat16": torch.bfloat16}[dtype]
            as_tensor = lambda bits: torch.from_numpy(bits.view(np.int16).copy()).view(tdtype)
            return {"y": torch.from_numpy(out["y"]), "scale": torch.from_numpy(out["scale"]),
                    "y_norm": as_tensor(out["y_norm"]), "residual": as_tensor(out["residual"])}
        if kernel == "nvfp4_gemm":
            return gemm_expected(kw)
        raise KeyError(kernel)

    return provider


def gemm_expected(kw) -> torch.Tensor:
    """bf16 D of dequantize-then-fp32-matmul on the very bytes the kernel consumed; with
    kw["rows"] (row indices of A) only those rows of D."""
    rows = kw.get("rows")
    if rows is not None:
        rows = np.asarray(torch.as_tensor(rows).cpu().numpy(), dtype=np.int64)
    bits = nvfp4_oracle.nvfp4_gemm(kw["A_fp4"].cpu().numpy(), kw["B_fp4"].cpu().numpy(),
                                   kw["A_sf"].cpu().numpy(), kw["B_sf"].cpu().numpy(), kw["alpha"], rows=rows)
    return torch.from_numpy(bits.view(np.int16)).view(torch.bfloat16)
