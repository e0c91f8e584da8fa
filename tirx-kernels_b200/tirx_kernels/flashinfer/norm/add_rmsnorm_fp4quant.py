"""``flashinfer_add_rmsnorm_fp4quant``: residual add + RMSNorm + FP4 block quantization (CUDA, sm_100a).

Drop-in for tirx_kernels/flashinfer/norm/add_rmsnorm_fp4quant.py of the reference: same
``KERNEL_META`` (:49-53), config keys and labels (``_cfg`` :366-428; the 1222 upstream-mirroring and 23
structural cases of ``CONFIGS`` :430-746; ``BENCH_CONFIGS`` :748-774), the positional executable
signature ``ex(x, residual, weight, y, scale, scale_unswizzled, y_norm, global_scale, M, eps)``
(:1210-1221, :1457-1470), caller-owned outputs, in-place residual update and ``ValueError`` on bad
shapes (:777-785).

``output_both_sf_layouts`` writes the scale bytes 128x4-swizzled into ``scale`` and linearly into
``scale_unswizzled``; ``output_norm`` also writes the normalized, weighted row in the input dtype.
The kernel is ``b2_add_rmsnorm_fp4quant`` in the C-ABI library.
"""

from __future__ import annotations

from typing import Any

from tirx_kernels import _checks, _native
from tirx_kernels._protocol import KernelHandle
from tirx_kernels.runner import bench

KERNEL_META = {
    "name": "flashinfer_add_rmsnorm_fp4quant",
    "category": "flashinfer",
    "compute_capability": 10,
}

_DTYPES = ("float16", "bfloat16")
_DEFAULT_EPS = 1e-6
_GUARD_ELEMENTS = _checks.GUARD_ELEMENTS
_GUARD_BYTE = _checks.GUARD_BYTE


def _torch_input_dtype(dtype: str):
    import torch

    return {"float16": torch.float16, "bfloat16": torch.bfloat16}[dtype]


def _validate(config: dict[str, Any]) -> None:
    if config["input_dtype"] not in _DTYPES:
        raise ValueError(f"unsupported input_dtype={config['input_dtype']!r}")
    if int(config["block_size"]) not in (16, 32):
        raise ValueError("block_size must be 16 or 32")
    if int(config["H"]) < 64 or int(config["H"]) % int(config["block_size"]):
        raise ValueError("H must be >=64 and divisible by block_size")
    if config["scale_format"] not in ("e4m3", "ue8m0"):
        raise ValueError("scale_format must be e4m3 or ue8m0")


def _effective_scale_format(config: dict[str, Any]) -> str:
    return "e4m3" if int(config["block_size"]) == 16 or str(config["scale_format"]) == "e4m3" else "ue8m0"


def _primary_swizzled(config: dict[str, Any]) -> bool:
    return bool(config["swizzled"]) or bool(config["output_both_sf_layouts"])


def cluster_size(H: int) -> int:
    """CTAs per row the reference uses for this H (``_source_config`` :354-363); it fixes the order of
    the fp32 sum and, above 1, the arithmetic of the quantization pass."""
    for candidate in (1, 2, 4, 8, 16):
        hpc = H // candidate
        tpr = next(t for limit, t in ((64, 8), (128, 16), (3072, 32), (6144, 64), (16384, 128), (1 << 62, 256))
                   if hpc <= limit)
        threads = 128 if hpc <= 16384 else 256
        rows, wpr = threads // tpr, max(tpr // 32, 1)
        vb = max(1, _checks.ceil_div(hpc // 8, tpr))
        tile, red = rows * 8 * vb * tpr * 2, rows * wpr * 4
        estimate = 4 * tile + red if candidate == 1 else 2 * tile + red * candidate + 8
        if H % candidate == 0 and estimate <= 232448:
            return candidate
    return 16


def algorithmic_bytes(M: int, H: int, block_size: int, both: bool, norm: bool) -> int:
    """x and residual read, residual written, weight, packed output, scale bytes, optional outputs."""
    columns = H // block_size
    return M * H * 2 * 3 + H * 2 + M * H // 2 + M * columns * (2 if both else 1) + (M * H * 2 if norm else 0) + 4


class _Executable:
    """Launchable with the reference executable's positional signature; returns None."""

    def __init__(self, config: dict[str, Any]):
        self.config = dict(config)

    def __call__(self, x, residual, weight, y, scale, scale_unswizzled, y_norm, global_scale, M: int,
                 eps: float) -> None:
        c = self.config
        H = int(c["H"])
        if x.numel() != M * H or residual.numel() != M * H or weight.numel() != H or y.numel() != M * (H // 2):
            raise ValueError("tensor sizes do not match (M, H)")
        _native.add_rmsnorm_fp4quant(x, residual, weight, y, scale, scale_unswizzled, y_norm, global_scale, M, H,
                                     eps, str(c["input_dtype"]), int(c["block_size"]), str(c["scale_format"]),
                                     bool(c["swizzled"]), bool(c["output_both_sf_layouts"]),
                                     bool(c["output_norm"]), bool(c["enable_pdl"]))


def get_kernel(**config: Any) -> KernelHandle:
    """Handle for one (dtype, H, block, format, layout, optional outputs, pdl) specialization."""
    config.setdefault("swizzled", False)
    config.setdefault("output_both_sf_layouts", False)
    config.setdefault("output_norm", False)
    config.setdefault("enable_pdl", False)
    _validate(config)
    keys = ("input_dtype", "H", "block_size", "scale_format", "swizzled", "output_both_sf_layouts", "output_norm",
            "enable_pdl")
    spec = {k: config[k] for k in keys}
    return KernelHandle("b2_add_rmsnorm_fp4quant", {"launcher": _Executable(spec), **spec})


# ---- data -----------------------------------------------------------------------------------------
def _logical_shape(config: dict[str, Any]) -> tuple[int, ...]:
    H = int(config["H"])
    if int(config.get("input_ndim", 2)) == 3:
        return int(config["B"]), int(config["S"]), H
    return int(config["M"]), H


def _prepare_tensors(config: dict[str, Any]) -> dict[str, Any]:
    """Seeded x, residual and weight with guard regions (reference :1330-1384).

    Values are drawn on the CPU (seed 42) and copied over, so a host oracle sees the same bits.
    ``weight_mode="gamma"`` draws 1 + 0.1*N(0,1) instead of the reference's N(0,1).
    """
    import torch

    M, H = int(config["M"]), int(config["H"])
    dtype = _torch_input_dtype(str(config["input_dtype"]))
    generator = torch.Generator().manual_seed(42)
    if str(config.get("data_mode", "random")) == "zero":
        x_host = torch.zeros(M, H, dtype=dtype)
        r_host = torch.zeros(M, H, dtype=dtype)
    elif H >= 65536:
        columns = torch.arange(H)
        x_host = torch.where(columns % 2 == 0, 0.75, -0.5).to(dtype).expand(M, H).contiguous()
        r_host = torch.where(columns % 3 == 0, -0.25, 0.5).to(dtype).expand(M, H).contiguous()
    else:
        x_host = torch.randn(M, H, generator=generator, dtype=torch.float32).to(dtype)
        r_host = torch.randn(M, H, generator=generator, dtype=torch.float32).to(dtype)
    w_host = torch.randn(H, generator=generator, dtype=torch.float32)
    if config.get("weight_mode") == "gamma":
        w_host = 1.0 + 0.1 * w_host
    w_host = w_host.to(dtype)

    x_backing, x_arg = _checks.with_guard(M * H, dtype, "cuda", 1.0)
    x_arg.copy_(x_host.view(-1))
    residual_backing, residual_arg = _checks.with_guard(M * H, dtype, "cuda", 1.0)
    residual_arg.copy_(r_host.view(-1))
    weight_backing, weight = _checks.with_guard(H, dtype, "cuda", 1.0)
    weight.copy_(w_host)

    mode = str(config.get("global_scale_mode", "none"))
    if mode in ("none", "one"):
        scale_value = 1.0
    elif mode == "nonunit":
        scale_value = 3.25
    elif mode == "zero":
        scale_value = 0.0
    elif mode == "computed":
        h = (x_host.float() + r_host.float()).to(dtype).float()
        normed = h * torch.rsqrt(h.square().mean(dim=-1, keepdim=True) + float(config["eps"])) * w_host.float()
        scale_value = 448.0 * 6.0 / float(normed.abs().amax().clamp_min(torch.finfo(torch.float32).tiny))
    else:
        raise ValueError(f"unsupported global_scale_mode={mode!r}")
    global_scale = torch.tensor([scale_value], dtype=torch.float32, device="cuda")
    shape = _logical_shape(config)
    return {"x": x_arg.view(shape), "x2d": x_arg.view(M, H), "x_arg": x_arg, "x_backing": x_backing,
            "residual": residual_arg.view(shape), "residual2d": residual_arg.view(M, H),
            "residual_arg": residual_arg, "residual_backing": residual_backing,
            "weight": weight, "weight_backing": weight_backing, "global_scale": global_scale}


def _scale_storage_size(config: dict[str, Any]) -> int:
    M, H = int(config["M"]), int(config["H"])
    columns = H // int(config["block_size"])
    if _primary_swizzled(config):
        return _checks.ceil_div(M, 128) * _checks.ceil_div(columns, 4) * 512
    return M * columns


def _prepare_output(config: dict[str, Any]) -> dict[str, Any]:
    """Caller-owned outputs, all four always present as in the fixed ABI (reference :1395-1454)."""
    import torch

    M, H = int(config["M"]), int(config["H"])
    columns = H // int(config["block_size"])
    dtype = _torch_input_dtype(str(config["input_dtype"]))
    sizes = {"y": M * (H // 2), "scale": _scale_storage_size(config), "scale_unswizzled": M * columns,
             "y_norm": M * H}
    out: dict[str, Any] = {"sizes": sizes}
    for name in ("y", "scale", "scale_unswizzled"):
        backing, arg = _checks.with_guard(sizes[name], torch.uint8, "cuda", _GUARD_BYTE)
        arg.fill_(_GUARD_BYTE)
        out[name + "_backing"], out[name + "_arg"] = backing, arg
    backing, arg = _checks.with_guard(sizes["y_norm"], dtype, "cuda", 1.0)
    arg.fill_(1.0)
    out["y_norm_backing"], out["y_norm_arg"] = backing, arg
    out["y"] = out["y_arg"].view(M, H // 2)
    out["scale"] = out["scale_arg"] if _primary_swizzled(config) else out["scale_arg"].view(M, columns)
    out["scale_unswizzled"] = out["scale_unswizzled_arg"].view(M, columns)
    out["y_norm"] = out["y_norm_arg"].view(M, H)
    names = ("y", "scale", "scale_unswizzled", "y_norm")
    out["pointers"] = {n: out[n].data_ptr() for n in names}
    out["strides"] = {n: out[n].stride() for n in names}
    return out


def prepare_data(**config: Any):
    """Deterministic inputs and caller-owned fixed-ABI outputs (reference :1296-1311)."""
    config = dict(config)
    data, output = _prepare_tensors(config), _prepare_output(config)
    return (data["x_arg"], data["residual_arg"], data["weight"], output["y_arg"], output["scale_arg"],
            output["scale_unswizzled_arg"], output["y_norm_arg"], data["global_scale"])


def _launch(executable, data, output, config: dict[str, Any]):
    return executable(data["x_arg"], data["residual_arg"], data["weight"], output["y_arg"], output["scale_arg"],
                      output["scale_unswizzled_arg"], output["y_norm_arg"], data["global_scale"],
                      int(config["M"]), float(config["eps"]))


# ---- checks ------------------------------------------------------------------------------------------
def _layout(config) -> str:
    return "128x4" if _primary_swizzled(config) else "linear"


def _logical_scale_bytes(output, config: dict[str, Any]):
    M, H = int(config["M"]), int(config["H"])
    return _checks.logical_scale_bytes(output["scale_arg"], M, H // int(config["block_size"]), _layout(config))


def _math_oracle(snapshot, config: dict[str, Any]):
    """The reference's independent fp32 oracle (:1704-1715)."""
    M, H = int(config["M"]), int(config["H"])
    dtype = _torch_input_dtype(str(config["input_dtype"]))
    h = snapshot["x"].view(M, H).float() + snapshot["residual"].view(M, H).float()
    rstd = (h.square().mean(dim=-1, keepdim=True) + float(config["eps"])).rsqrt()
    narrow = h.to(dtype)
    if cluster_size(H) == 1:
        return narrow.float() * rstd * snapshot["weight"].float()
    return (narrow * snapshot["weight"]).to(dtype).float() * rstd


def _assert_math(output, data, snapshot, config: dict[str, Any]) -> None:
    import torch

    fmt = _effective_scale_format(config)
    if fmt == "e4m3" and float(data["global_scale"].item()) == 0.0:
        if torch.count_nonzero(output["y"] & 0x77) or torch.count_nonzero(_logical_scale_bytes(output, config)):
            raise AssertionError("zero global scale must produce signed-zero FP4 and scales")
        return
    oracle = _math_oracle(snapshot, config)
    deq = _checks.dequantize(output["y"], output["scale_arg"], _layout(config), block_size=int(config["block_size"]),
                             scale_format=fmt, global_scale=float(data["global_scale"].item()))
    if not torch.isfinite(deq).all():
        raise AssertionError("dequantized output contains non-finite values")
    torch.testing.assert_close(deq, oracle, rtol=0.5, atol=2.0,
                               msg=lambda m: f"independent FP32 add/RMSNorm oracle: {m}")
    if bool(config["output_norm"]):
        torch.testing.assert_close(output["y_norm"], oracle.to(_torch_input_dtype(str(config["input_dtype"]))),
                                   rtol=1e-2, atol=1e-2, msg=lambda m: f"optional y_norm oracle: {m}")


def _assert_inputs_and_residual(data, snapshot, config: dict[str, Any]) -> None:
    """Inputs untouched, residual = x + residual rounded once, guards intact (reference :1567-1591)."""
    import torch

    for name in ("x", "weight", "global_scale"):
        if not torch.equal(data[name], snapshot[name]):
            raise AssertionError(f"{name} tensor was modified")
    expected = (snapshot["x"].float() + snapshot["residual"].float()).to(_torch_input_dtype(str(config["input_dtype"])))
    if not torch.equal(data["residual"], expected):
        count = int((data["residual"] != expected).sum().item())
        raise AssertionError(f"{count} residual values differ from in-place add")
    M, H = int(config["M"]), int(config["H"])
    for name, size in (("x", M * H), ("residual", M * H), ("weight", H)):
        if not torch.all(data[name + "_backing"][size:] == 1):
            raise AssertionError(f"{name} guard was modified")


def _assert_output_integrity(output, config: dict[str, Any]) -> None:
    """Identity, guards, and outputs that were not requested keep their fill (reference :1629-1658)."""
    import torch

    for name in ("y", "scale", "scale_unswizzled", "y_norm"):
        if output[name].data_ptr() != output["pointers"][name] or output[name].stride() != output["strides"][name]:
            raise AssertionError(f"{name} identity changed")
        fill = 1 if name == "y_norm" else _GUARD_BYTE
        if not torch.all(output[name + "_backing"][output["sizes"][name]:] == fill):
            raise AssertionError(f"{name} guard was modified")
    if not bool(config["output_both_sf_layouts"]) and not torch.all(output["scale_unswizzled_arg"] == _GUARD_BYTE):
        raise AssertionError("scale_unswizzled was written although not requested")
    if not bool(config["output_norm"]) and not torch.all(output["y_norm_arg"] == 1):
        raise AssertionError("y_norm was written although not requested")
    if _primary_swizzled(config):
        M, H = int(config["M"]), int(config["H"])
        mask = _checks.padding_mask(M, H // int(config["block_size"]), "128x4", "cuda")
        if not torch.all(output["scale_arg"][mask] == _GUARD_BYTE):
            raise AssertionError("swizzled padding positions were written")


def run_test(**config: Any) -> None:
    """Launch one config and validate it.

    Exact comparison against an installed expected-value provider (packed bytes, logical scale
    bytes, linear scale copy, normalized row, residual; the reference compares raw bytes with its
    own oracle library, :1810-1815), then the reference's self-contained checks.
    """
    import torch

    from tirx_kernels.runner import compile_kernel, reference_provider

    config = dict(config)
    config.setdefault("input_ndim", 2)
    _validate(config)
    data = _prepare_tensors(config)
    snapshot = {name: data[name].clone() for name in ("x", "residual", "weight", "global_scale")}
    output = _prepare_output(config)
    executable = compile_kernel(get_kernel(**config))
    if _launch(executable, data, output, config) is not None:
        raise AssertionError("AddRMSNormFP4Quant ABI must return None")
    torch.cuda.synchronize()
    provider = reference_provider()
    if provider is not None:
        M, H = int(config["M"]), int(config["H"])
        want = provider("flashinfer_add_rmsnorm_fp4quant", x=snapshot["x"].view(M, H),
                        residual=snapshot["residual"].view(M, H), weight=snapshot["weight"],
                        global_scale=data["global_scale"], config=config)

        def same(name, got, expected):
            got, expected = got.cpu(), expected.reshape(got.shape)
            if not torch.equal(got, expected):
                raise AssertionError(f"{int((got != expected).sum())} {name} differ from the oracle")

        same("packed FP4 bytes", output["y"], want["y"])
        same("logical scale bytes", _logical_scale_bytes(output, config), want["scale"])
        same("residual values", data["residual2d"].view(torch.int16), want["residual"].view(torch.int16))
        if bool(config["output_both_sf_layouts"]):
            same("linear scale bytes", output["scale_unswizzled"], want["scale"])
        if bool(config["output_norm"]):
            same("y_norm values", output["y_norm"].view(torch.int16), want["y_norm"].view(torch.int16))
    _assert_inputs_and_residual(data, snapshot, config)
    _assert_math(output, data, snapshot, config)
    _assert_output_integrity(output, config)


def prepare_bench(**config: Any):
    from tirx_kernels.runner import compile_kernel, prepared_gpu_benchmark

    config.setdefault("input_ndim", 2)
    state = {"config": dict(config), "executable": compile_kernel(get_kernel(**config))}
    return prepared_gpu_benchmark(run_gpu, state)


def run_gpu(prepared, *, warmup=None, repeat=None, timer=None, rounds=1, cooldown_s=1.0, **kwargs: Any):
    """Kernel-only timing of one config; the record carries its HBM roofline."""
    import torch

    config = {**prepared["config"], **kwargs}
    data, output = _prepare_tensors(config), _prepare_output(config)
    executable = prepared["executable"]

    def tirx_launch():
        return _launch(executable, data, output, config)

    if tirx_launch() is not None:
        raise AssertionError("benchmark closure must return None")
    torch.cuda.synchronize()
    result = bench({"tirx": tirx_launch}, warmup=warmup, repeat=repeat, timer=timer, rounds=rounds,
                   cooldown_s=cooldown_s)
    result["roofline"] = _checks.roofline_hbm(
        algorithmic_bytes(int(config["M"]), int(config["H"]), int(config["block_size"]),
                          bool(config["output_both_sf_layouts"]), bool(config["output_norm"])),
        result["impls"]["tirx"])
    return result


def run_bench(*, warmup=None, repeat=None, timer=None, rounds=1, cooldown_s=1.0, **config: Any):
    return prepare_bench(**config).run_gpu(warmup=warmup, repeat=repeat, timer=timer, rounds=rounds,
                                           cooldown_s=cooldown_s)


# ---- config matrix (labels identical to the reference's) ------------------------------------------------
def _cfg(case: str, dtype: str, H: int, *, M: int | None = None, B: int | None = None, S: int | None = None,
         block_size: int = 16, scale_format: str = "e4m3", swizzled: bool = False,
         output_both_sf_layouts: bool = False, output_norm: bool = False, enable_pdl: bool = False,
         eps: float = _DEFAULT_EPS, global_scale_mode: str = "none", allocation: str = "preallocated",
         data_mode: str = "random", **extra: Any) -> dict[str, Any]:
    if M is None:
        if B is None or S is None:
            raise ValueError("either M or both B/S must be provided")
        M, shape, ndim = B * S, f"b{B}_s{S}", 3
    else:
        if B is not None or S is not None:
            raise ValueError("M and B/S are mutually exclusive")
        shape, ndim = f"m{M}", 2
    short = {"float16": "fp16", "bfloat16": "bf16"}[dtype]
    eps_code = {1e-4: "1e4", 1e-5: "1e5", 1e-6: "1e6"}[eps]
    label = (f"{case}_{short}_{shape}_h{H}_b{block_size}_{scale_format}_sw{int(swizzled)}_"
             f"both{int(output_both_sf_layouts)}_yn{int(output_norm)}_pdl{int(enable_pdl)}_eps{eps_code}_"
             f"gs{global_scale_mode}_{allocation}_{data_mode}")
    return {"label": label, "case": case, "input_dtype": dtype, "input_ndim": ndim, "M": M, "B": B, "S": S, "H": H,
            "block_size": block_size, "scale_format": scale_format, "swizzled": swizzled,
            "output_both_sf_layouts": output_both_sf_layouts, "output_norm": output_norm,
            "enable_pdl": enable_pdl, "eps": eps, "global_scale_mode": global_scale_mode,
            "allocation": allocation, "data_mode": data_mode, **extra}


_MX = {"block_size": 32, "scale_format": "ue8m0"}
_BOTH = {"output_both_sf_layouts": True}

_NV2D = [_cfg("nv2d", d, H, M=M, eps=e) for M in (1, 4, 16, 32, 7, 13, 128, 512, 1000, 8192, 16384)
         for H in (64, 128, 256, 512, 1024, 1536, 2048, 4096, 8192) for d in _DTYPES for e in (1e-5, 1e-6)]
_NV3D = [_cfg("nv3d", d, H, B=B, S=S, eps=1e-5) for B in (1, 4, 3, 7, 128) for S in (16, 64, 128, 37)
         for H in (128, 256, 1536, 4096, 8192) for d in _DTYPES]
_LARGE_BATCH = [_cfg("large_batch", "float16", H, M=M) for M, H in ((512, 4096), (1024, 4096))]
_MX_BASIC = [_cfg("mx_basic", d, H, M=M, **_MX) for M in (1, 4, 16, 7, 128, 8192)
             for H in (128, 256, 512, 1536, 2048, 4096) for d in _DTYPES]
_CROSS = [
    *[_cfg("fused_vs_separate", "float16", H, M=M) for M in (4, 16, 128, 512) for H in (256, 512, 1024, 4096, 8192)],
    *[_cfg("nv_matches_separate", d, H, M=M) for M in (1, 4, 16, 128) for H in (64, 256, 512, 1024, 2048, 4096)
      for d in _DTYPES],
    *[_cfg("mx_matches_separate", d, H, M=M, **_MX) for M in (1, 4, 16, 128)
      for H in (128, 256, 512, 1024, 2048, 4096) for d in _DTYPES],
    *[_cfg("global_scale_consistency", "float16", H, M=M, global_scale_mode="nonunit") for M in (1, 16, 64)
      for H in (256, 1024, 4096)],
]
_LARGE_H = [
    *[_cfg("large_h_nv", d, H, M=M) for M in (1, 16, 128, 1024) for H in (16384, 32768) for d in _DTYPES],
    *[_cfg("large_h_mx", d, H, M=M, **_MX) for M in (1, 16, 128, 1024) for H in (16384, 32768) for d in _DTYPES],
]
_SWIZZLED = [
    *[_cfg("swizzled_nv", d, H, M=M, swizzled=True) for M in (1, 16, 128, 256) for H in (512, 1024, 2048, 4096)
      for d in _DTYPES],
    *[_cfg("swizzled_mx", d, H, M=M, swizzled=True, **_MX) for M in (1, 16, 128, 256)
      for H in (512, 1024, 2048, 4096) for d in _DTYPES],
]
_ALLOCATION = [
    *[_cfg("auto2d_nv", d, H, M=M, allocation="auto") for M in (1, 16, 128) for H in (256, 1024, 4096) for d in _DTYPES],
    *[_cfg("auto3d_nv", "float16", H, B=B, S=S, allocation="auto") for B in (1, 4, 16) for S in (16, 64)
      for H in (256, 1024)],
    *[_cfg("auto_mx", "float16", H, M=M, allocation="auto", **_MX) for M in (1, 16, 128) for H in (256, 1024)],
    *[_cfg("auto_swizzled", "float16", H, M=M, swizzled=True, allocation="auto") for M in (16, 128) for H in (512, 1024)],
    *[_cfg("auto_matches_preallocated", "float16", H, M=M, allocation="compare") for M in (16, 128) for H in (512, 1024)],
]
_RESIDUAL = [
    *[_cfg("residual2d", d, H, M=M) for M in (1, 4, 16, 128, 512) for H in (256, 512, 1024, 4096) for d in _DTYPES],
    *[_cfg("residual3d", d, H, B=B, S=S) for B in (1, 4, 16) for S in (16, 64, 128) for H in (256, 1024, 4096)
      for d in _DTYPES],
    *[_cfg("residual_mx", d, H, M=M, **_MX) for M in (1, 16, 128) for H in (256, 1024, 2048) for d in _DTYPES],
    *[_cfg("residual_large_h", d, H, M=M) for M in (1, 16, 128) for H in (16384, 32768) for d in _DTYPES],
    *[_cfg("residual_used_for_norm", "float16", H, M=M) for M in (16, 128) for H in (512, 1024)],
    *[_cfg("residual_preallocated", "float16", H, M=M) for M in (16, 128) for H in (512, 1024)],
    *[_cfg("residual_swizzled", "float16", H, M=M, swizzled=True) for M in (16, 128) for H in (512, 1024)],
    _cfg("residual_not_aliased", "float16", 512, M=16),
]
_BOTH_CONFIGS = [
    *[_cfg("both_nv", d, H, M=M, **_BOTH) for M in (1, 16, 128, 256) for H in (256, 512, 1024, 4096) for d in _DTYPES],
    *[_cfg("both_mx", d, H, M=M, **_MX, **_BOTH) for M in (1, 16, 128, 256) for H in (256, 512, 1024, 4096)
      for d in _DTYPES],
    *[_cfg("both_consistency", "float16", H, M=M, **_BOTH) for M in (1, 16, 128) for H in (512, 1024, 4096)],
    *[_cfg("both3d", "float16", H, B=B, S=S, **_BOTH) for B in (1, 4, 8) for S in (16, 64, 128) for H in (256, 1024)],
    *[_cfg("both_global", "float16", H, M=M, global_scale_mode="nonunit", **_BOTH) for M in (16, 128)
      for H in (512, 1024)],
    *[_cfg("both_preallocated", "float16", H, M=M, **_BOTH) for M in (16, 128) for H in (512, 1024)],
    *[_cfg("both_large_h", d, H, M=M, **_BOTH) for M in (1, 16, 128) for H in (16384, 32768) for d in _DTYPES],
    *[_cfg("both_residual", "float16", H, M=M, **_BOTH) for M in (16, 128) for H in (512, 1024)],
    _cfg("both_ignores_swizzle", "float16", 1024, M=64, swizzled=True, **_BOTH),
]
_YOUT = [
    *[_cfg("yout_reference", d, H, M=M, output_norm=True) for M in (1, 64) for H in (256, 4096) for d in _DTYPES],
    *[_cfg("yout_quant_unchanged", d, H, M=M, output_norm=True, global_scale_mode="nonunit") for M in (1, 64)
      for H in (256, 2048) for d in _DTYPES],
    *[_cfg("yout_both", "bfloat16", H, M=M, output_norm=True, **_BOTH) for M in (1, 16, 128) for H in (512, 2048)],
    *[_cfg("yout3d", "bfloat16", H, B=B, S=37, output_norm=True) for B in (1, 4) for H in (256, 2048)],
    *[_cfg("yout_not_global_scaled", d, 2048, M=M, output_norm=True, global_scale_mode="nonunit") for M in (1, 64)
      for d in _DTYPES],
    *[_cfg("yout_mx", d, 2048, M=M, output_norm=True, **_MX) for M in (1, 64) for d in _DTYPES],
]
_UPSTREAM = [*_NV2D, *_NV3D, *_LARGE_BATCH, *_MX_BASIC, *_CROSS, *_LARGE_H, *_SWIZZLED, *_ALLOCATION, *_RESIDUAL,
             *_BOTH_CONFIGS, *_YOUT]

_STRUCTURE = [
    _cfg("guard_subwarp_row_tail", "float16", 64, M=17),
    _cfg("guard_nv_column_tail", "bfloat16", 80, M=129, swizzled=True),
    _cfg("guard_mx_column_tail", "float16", 160, M=3, **_MX),
    *[_cfg("guard_threshold", "bfloat16", H, M=3) for H in (3072, 3088, 6144, 6160, 14336, 16384, 16400)],
    *[_cfg(f"guard_cluster{c}", "bfloat16", H, M=1) for c, H in ((2, 32768), (4, 131072), (8, 262144), (16, 524288))],
    _cfg("guard_pdl", "bfloat16", 4096, M=3, enable_pdl=True),
    _cfg("guard_block32_e4m3", "float16", 4096, M=3, block_size=32, scale_format="e4m3", global_scale_mode="nonunit"),
    _cfg("guard_block16_requested_ue8", "float16", 4096, M=3, scale_format="ue8m0"),
    _cfg("guard_zero_data", "bfloat16", 4096, M=3, data_mode="zero"),
    _cfg("guard_zero_global", "float16", 4096, M=3, global_scale_mode="zero"),
    _cfg("guard_both_column_tail", "bfloat16", 80, M=129, **_BOTH),
    _cfg("guard_cluster16_both", "bfloat16", 524288, M=1, **_BOTH),
    _cfg("guard_cluster16_yout", "bfloat16", 524288, M=1, output_norm=True),
    _cfg("guard_pdl_both_yout", "bfloat16", 4096, M=3, output_norm=True, enable_pdl=True, **_BOTH),
]

CONFIGS = [*_UPSTREAM, *_STRUCTURE]

assert len(_UPSTREAM) == 1222 and len(_STRUCTURE) == 23
assert len({config["label"] for config in CONFIGS}) == len(CONFIGS)

# The reference's ten latency-bound shapes, then the throughput shape this build is measured on
# (8192 tokens x hidden 7168, gamma = 1 + 0.1*N(0,1), swizzled NVFP4 scales under a computed global scale).
BENCH_CONFIGS = [
    _cfg("bench_nv", "bfloat16", 4096, M=32),
    _cfg("bench_nv_large", "bfloat16", 8192, M=64),
    _cfg("bench_nv_global", "bfloat16", 4096, M=32, global_scale_mode="one"),
    _cfg("bench_nv_swizzled", "bfloat16", 4096, M=32, swizzled=True),
    _cfg("bench_mx", "bfloat16", 4096, M=32, **_MX),
    _cfg("bench_nv_3d", "bfloat16", 128, B=32, S=32),
    _cfg("bench_nv_both", "bfloat16", 4096, M=32, **_BOTH),
    _cfg("bench_nv_both_large", "bfloat16", 8192, M=64, **_BOTH),
    _cfg("bench_nv_both_global", "bfloat16", 4096, M=32, global_scale_mode="one", **_BOTH),
    _cfg("bench_mx_both", "bfloat16", 4096, M=32, **_MX, **_BOTH),
    _cfg("bench_nv_swizzled_large", "bfloat16", 7168, M=8192, swizzled=True, global_scale_mode="computed",
         weight_mode="gamma"),
]

__all__ = ["BENCH_CONFIGS", "CONFIGS", "KERNEL_META", "get_kernel", "prepare_bench", "prepare_data",
           "run_bench", "run_gpu", "run_test"]
