"""``flashinfer_rmsnorm_fp4quant``: RMSNorm fused with FP4 block quantization (CUDA, sm_100a).

Drop-in for tirx_kernels/flashinfer/norm/rmsnorm_fp4quant.py of the reference: same
``KERNEL_META`` (:29-33), config keys and labels (``_cfg`` :411-461; the 1007 upstream-mirroring
and 18 structural cases of ``CONFIGS`` :464-663; ``BENCH_CONFIGS`` :676-691), the positional
executable signature ``ex(x_flat, weight, y_flat, scales_flat, global_scale, M, eps)``
(:983-991, :1156-1165), caller-owned outputs and ``ValueError`` on bad shapes (:694-704).

Block 16 always uses E4M3 scales under the fp32 global scale (NVFP4); block 32 uses UE8M0
(MXFP4) unless ``scale_format="e4m3"``.  Scales are linear ``[M, H/block]`` or 128x4-swizzled
(padding positions untouched).  The kernel is ``b2_rmsnorm_fp4quant`` in the C-ABI library.
"""

from __future__ import annotations

import itertools
from typing import Any

from tirx_kernels import _checks, _native
from tirx_kernels._protocol import KernelHandle
from tirx_kernels.runner import bench

KERNEL_META = {
    "name": "flashinfer_rmsnorm_fp4quant",
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


def _validate(input_dtype: str, H: int, block_size: int, scale_format: str, M: int) -> None:
    if input_dtype not in _DTYPES:
        raise ValueError(f"unsupported input_dtype={input_dtype!r}")
    if block_size not in (16, 32):
        raise ValueError(f"unsupported block_size={block_size}")
    if H < 64 or H % block_size != 0:
        raise ValueError(f"H={H} must be >=64 and divisible by block_size={block_size}")
    if scale_format not in ("e4m3", "ue8m0"):
        raise ValueError(f"unsupported scale_format={scale_format!r}")
    if M <= 0:
        raise ValueError(f"M must be positive, got {M}")


def _effective_scale_format(block_size: int, scale_format: str) -> str:
    return "e4m3" if block_size == 16 or scale_format == "e4m3" else "ue8m0"


def _scale_storage_size(config: dict[str, Any]) -> int:
    M, H = int(config["M"]), int(config["H"])
    columns = H // int(config["block_size"])
    if bool(config["swizzled"]):
        return _checks.ceil_div(M, 128) * _checks.ceil_div(columns, 4) * 512
    return M * columns


def algorithmic_bytes(M: int, H: int, block_size: int, swizzled: bool) -> int:
    """x once + weight + packed output + the scale bytes written + the global scale."""
    return M * H * 2 + H * 2 + M * H // 2 + M * (H // block_size) + 4


class _Executable:
    """Launchable with the reference executable's positional signature; returns None."""

    def __init__(self, input_dtype, H, block_size, scale_format, swizzled, enable_pdl):
        self.input_dtype, self.H, self.block_size = input_dtype, H, block_size
        self.scale_format, self.swizzled, self.enable_pdl = scale_format, swizzled, enable_pdl

    def __call__(self, x_flat, weight, y_flat, scales_flat, global_scale, M: int, eps: float) -> None:
        H = self.H
        if x_flat.numel() != M * H or weight.numel() != H or y_flat.numel() != M * (H // 2):
            raise ValueError("tensor sizes do not match (M, H)")
        _native.rmsnorm_fp4quant(x_flat, weight, y_flat, scales_flat, global_scale, M, H, eps,
                                 self.input_dtype, self.block_size, self.scale_format, self.swizzled,
                                 self.enable_pdl)


def get_kernel(input_dtype: str, M: int, H: int, block_size: int, scale_format: str, swizzled: bool,
               enable_pdl: bool, **kwargs: Any) -> KernelHandle:
    """Handle for one (dtype, H, block_size, scale_format, swizzled, pdl) specialization."""
    _validate(input_dtype, H, block_size, scale_format, M)
    launcher = _Executable(input_dtype, H, block_size, scale_format, swizzled, enable_pdl)
    return KernelHandle("b2_rmsnorm_fp4quant", {"launcher": launcher, "input_dtype": input_dtype, "H": H,
                                                "block_size": block_size, "scale_format": scale_format,
                                                "swizzled": swizzled, "enable_pdl": enable_pdl})


# ---- data -----------------------------------------------------------------------------------------
def _logical_shape(config: dict[str, Any]) -> tuple[int, ...]:
    H = int(config["H"])
    if int(config.get("input_ndim", 2)) == 3:
        return int(config["B"]), int(config["S"]), H
    return int(config["M"]), H


def _prepare_tensors(config: dict[str, Any]) -> dict[str, Any]:
    """Seeded inputs with guard regions after x and weight (reference :1060-1110).

    Values are drawn on the CPU (seed 42) and copied over, so a host oracle sees the same bits;
    ``weight_mode="gamma"`` draws 1 + 0.1*N(0,1) instead of the reference's N(0,1).
    """
    import torch

    M, H = int(config["M"]), int(config["H"])
    dtype = _torch_input_dtype(str(config["input_dtype"]))
    generator = torch.Generator().manual_seed(42)
    if config.get("data_mode") == "zero":
        x_host = torch.zeros(M, H, dtype=dtype)
    elif H >= 65536:
        columns = torch.arange(H)
        magnitude = torch.where(columns % 257 < 128, 0.5, 1.0)
        x_host = torch.where(columns % 2 == 0, magnitude, -magnitude).to(dtype).expand(M, H).contiguous()
    else:
        x_host = torch.randn(M, H, generator=generator, dtype=torch.float32).to(dtype)
    w_host = torch.randn(H, generator=generator, dtype=torch.float32)
    if config.get("weight_mode") == "gamma":
        w_host = 1.0 + 0.1 * w_host
    w_host = w_host.to(dtype)

    x_backing, x_arg = _checks.with_guard(M * H, dtype, "cuda", 1.0)
    x_arg.copy_(x_host.view(-1))
    weight_backing, weight = _checks.with_guard(H, dtype, "cuda", 1.0)
    weight.copy_(w_host)

    mode = str(config.get("global_scale_mode", "computed"))
    if mode == "computed":
        x_f32 = x_host.float()
        rms = x_f32 * torch.rsqrt(x_f32.square().mean(dim=-1, keepdim=True) + float(config["eps"]))
        rms = (rms * w_host.float()).to(dtype)
        max_abs = rms.float().abs().amax().clamp_min(torch.finfo(torch.float32).tiny)
        scale_value = 448.0 * 6.0 / float(max_abs.item())
    elif mode in ("none", "one"):
        scale_value = 1.0
    elif mode == "nonunit":
        scale_value = 3.25
    elif mode == "zero":
        scale_value = 0.0
    else:
        raise ValueError(f"unsupported global_scale_mode={mode!r}")
    global_scale = torch.tensor([scale_value], dtype=torch.float32, device="cuda")
    return {"x": x_arg.view(_logical_shape(config)), "x2d": x_arg.view(M, H), "x_arg": x_arg,
            "x_backing": x_backing, "weight": weight, "weight_backing": weight_backing,
            "global_scale": global_scale}


def _prepare_output(config: dict[str, Any], *, initialize: bool) -> dict[str, Any]:
    import torch

    M, H = int(config["M"]), int(config["H"])
    y_size, scale_size = M * (H // 2), _scale_storage_size(config)
    y_backing, y_arg = _checks.with_guard(y_size, torch.uint8, "cuda", _GUARD_BYTE)
    scale_backing, scale_arg = _checks.with_guard(scale_size, torch.uint8, "cuda", _GUARD_BYTE)
    if initialize:
        y_arg.fill_(_GUARD_BYTE)
        scale_arg.fill_(_GUARD_BYTE)
    y = y_arg.view(M, H // 2)
    scale = scale_arg if bool(config["swizzled"]) else scale_arg.view(M, H // int(config["block_size"]))
    return {"y": y, "scale": scale, "y_arg": y_arg, "scale_arg": scale_arg, "y_backing": y_backing,
            "scale_backing": scale_backing, "y_size": y_size, "scale_size": scale_size,
            "y_ptr": y.data_ptr(), "scale_ptr": scale.data_ptr(), "y_stride": y.stride(),
            "scale_stride": scale.stride()}


def prepare_data(**config: Any):
    """Deterministic inputs and caller-owned packed outputs."""
    data = _prepare_tensors(dict(config))
    output = _prepare_output(dict(config), initialize=True)
    return data["x"], data["weight"], output["y"], output["scale"], data["global_scale"]


def _launch(executable, data, output, config: dict[str, Any]):
    return executable(data["x_arg"], data["weight"], output["y_arg"], output["scale_arg"],
                      data["global_scale"], int(config["M"]), float(config["eps"]))


# ---- checks ------------------------------------------------------------------------------------------
def _layout(config) -> str:
    return "128x4" if bool(config["swizzled"]) else "linear"


def _logical_scale_bytes(output, config: dict[str, Any]):
    M, H = int(config["M"]), int(config["H"])
    return _checks.logical_scale_bytes(output["scale_arg"], M, H // int(config["block_size"]), _layout(config))


def _assert_math(output, data, config: dict[str, Any]) -> None:
    """The reference's independent fp32 check (:1322-1344) and its zero-global-scale invariant."""
    import torch

    fmt = _effective_scale_format(int(config["block_size"]), str(config["scale_format"]))
    if fmt == "e4m3" and float(data["global_scale"].item()) == 0.0:
        if torch.count_nonzero(output["y"] & 0x77) or torch.count_nonzero(_logical_scale_bytes(output, config)):
            raise AssertionError("zero global scale must produce signed-zero FP4 values and scales")
        return
    deq = _checks.dequantize(output["y"], output["scale_arg"], _layout(config),
                             block_size=int(config["block_size"]), scale_format=fmt,
                             global_scale=float(data["global_scale"].item()))
    x = data["x2d"].float()
    normalized = x * (x.square().mean(dim=-1, keepdim=True) + float(config["eps"])).rsqrt()
    oracle = (normalized * data["weight"].float()).to(_torch_input_dtype(config["input_dtype"])).float()
    if not torch.isfinite(deq).all():
        raise AssertionError("dequantized output contains non-finite values")
    torch.testing.assert_close(deq, oracle, rtol=0.5, atol=2.0,
                               msg=lambda m: f"independent FP32 RMSNorm oracle: {m}")


def _assert_inputs_unchanged(data, snapshot, config) -> None:
    import torch

    M, H = int(config["M"]), int(config["H"])
    for name in ("x", "weight", "global_scale"):
        if not torch.equal(data[name], snapshot[name]):
            raise AssertionError(f"{name} tensor was modified")
    if not torch.all(data["x_backing"][M * H:] == 1) or not torch.all(data["weight_backing"][H:] == 1):
        raise AssertionError("input guard was modified")


def _assert_output_integrity(output) -> None:
    import torch

    if output["y"].data_ptr() != output["y_ptr"] or output["y"].stride() != output["y_stride"]:
        raise AssertionError("packed-output identity changed")
    if output["scale"].data_ptr() != output["scale_ptr"] or output["scale"].stride() != output["scale_stride"]:
        raise AssertionError("scale-output identity changed")
    if not torch.all(output["y_backing"][output["y_size"]:] == _GUARD_BYTE):
        raise AssertionError("packed-output guard was modified")
    if not torch.all(output["scale_backing"][output["scale_size"]:] == _GUARD_BYTE):
        raise AssertionError("scale-output guard was modified")


def run_test(**config: Any) -> None:
    """Launch one config and validate it.

    Exact byte comparison against an installed expected-value provider (packed bytes and the
    logical scale bytes, as the reference compares with its own oracle, :1309-1319), then the
    reference's self-contained checks: fp32 RMSNorm within rtol 0.5 / atol 2.0, inputs and guard
    regions untouched, output identity, and ``None`` returned by the executable.
    """
    import torch

    from tirx_kernels.runner import compile_kernel, reference_provider

    config = dict(config)
    config.setdefault("input_ndim", 2)
    _validate(str(config["input_dtype"]), int(config["H"]), int(config["block_size"]),
              str(config["scale_format"]), int(config["M"]))
    data = _prepare_tensors(config)
    snapshot = {name: data[name].clone() for name in ("x", "weight", "global_scale")}
    output = _prepare_output(config, initialize=True)
    executable = compile_kernel(get_kernel(
        input_dtype=str(config["input_dtype"]), M=1, H=int(config["H"]), block_size=int(config["block_size"]),
        scale_format=str(config["scale_format"]), swizzled=bool(config["swizzled"]),
        enable_pdl=bool(config["enable_pdl"])))
    if _launch(executable, data, output, config) is not None:
        raise AssertionError("RMSNormFP4Quant ABI must return None")
    torch.cuda.synchronize()
    provider = reference_provider()
    if provider is not None:
        ref_y, ref_scales = provider("flashinfer_rmsnorm_fp4quant", x=data["x2d"], weight=data["weight"],
                                     global_scale=data["global_scale"], config=config)
        if not torch.equal(output["y"].cpu(), ref_y.reshape(output["y"].shape)):
            count = int((output["y"].cpu() != ref_y.reshape(output["y"].shape)).sum())
            raise AssertionError(f"{count} packed FP4 bytes differ from the oracle")
        got = _logical_scale_bytes(output, config).cpu()
        if not torch.equal(got, ref_scales.reshape(got.shape)):
            count = int((got != ref_scales.reshape(got.shape)).sum())
            raise AssertionError(f"{count} logical scale bytes differ from the oracle")
    _assert_math(output, data, config)
    _assert_inputs_unchanged(data, snapshot, config)
    _assert_output_integrity(output)
    if bool(config["swizzled"]):  # positions holding no logical scale must keep their fill
        M, H = int(config["M"]), int(config["H"])
        mask = _checks.padding_mask(M, H // int(config["block_size"]), "128x4", "cuda")
        if not torch.all(output["scale_arg"][mask] == _GUARD_BYTE):
            raise AssertionError("swizzled padding positions were written")


def prepare_bench(**config: Any):
    from tirx_kernels.runner import compile_kernel, prepared_gpu_benchmark

    config.setdefault("input_ndim", 2)
    state = {"config": dict(config), "executable": compile_kernel(get_kernel(**config))}
    return prepared_gpu_benchmark(run_gpu, state)


def run_gpu(prepared, *, warmup=None, repeat=None, timer=None, rounds=1, cooldown_s=1.0, **kwargs: Any):
    """Kernel-only timing of one config; the record carries its HBM roofline."""
    import torch

    config = {**prepared["config"], **kwargs}
    data = _prepare_tensors(config)
    output = _prepare_output(config, initialize=False)
    executable = prepared["executable"]

    def tirx_launch():
        return _launch(executable, data, output, config)

    if tirx_launch() is not None:
        raise AssertionError("benchmark closure must return None")
    torch.cuda.synchronize()
    result = bench({"tirx": tirx_launch}, warmup=warmup, repeat=repeat, timer=timer, rounds=rounds,
                   cooldown_s=cooldown_s)
    result["roofline"] = _checks.roofline_hbm(
        algorithmic_bytes(int(config["M"]), int(config["H"]), int(config["block_size"]), bool(config["swizzled"])),
        result["impls"]["tirx"])
    return result


def run_bench(*, warmup=None, repeat=None, timer=None, rounds=1, cooldown_s=1.0, **config: Any):
    return prepare_bench(**config).run_gpu(warmup=warmup, repeat=repeat, timer=timer, rounds=rounds,
                                           cooldown_s=cooldown_s)


# ---- config matrix (labels identical to the reference's) ------------------------------------------------
def _cfg(case: str, dtype: str, H: int, *, M: int | None = None, B: int | None = None, S: int | None = None,
         block_size: int = 16, scale_format: str = "e4m3", swizzled: bool = False, enable_pdl: bool = False,
         eps: float = _DEFAULT_EPS, global_scale_mode: str = "computed", allocation: str = "preallocated",
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
             f"pdl{int(enable_pdl)}_eps{eps_code}_gs{global_scale_mode}_{allocation}_{data_mode}")
    return {"label": label, "case": case, "input_dtype": dtype, "input_ndim": ndim, "M": M, "B": B, "S": S,
            "H": H, "block_size": block_size, "scale_format": scale_format, "swizzled": swizzled,
            "enable_pdl": enable_pdl, "eps": eps, "global_scale_mode": global_scale_mode,
            "allocation": allocation, "data_mode": data_mode, **extra}


_MX = {"block_size": 32, "scale_format": "ue8m0", "global_scale_mode": "none"}
_prod = itertools.product

_NV2D = [_cfg("nv2d", d, H, M=M, eps=e)
         for M, H, d, e in _prod((1, 4, 16, 32, 7, 13, 33, 100, 128, 8192, 16384),
                                 (64, 128, 256, 512, 1024, 1536, 2048, 4096, 8192), _DTYPES, (1e-5, 1e-6))]
_NV3D = [_cfg("nv3d", d, H, B=B, S=S, eps=1e-5)
         for B, S, H, d in _prod((1, 4, 3, 7, 128), (16, 64, 128, 37, 99), (128, 256, 1536, 4096, 8192), _DTYPES)]
_LARGE_BATCH = [_cfg("large_batch", "float16", 4096, M=M) for M in (512, 1024)]
_MX_BASIC = [_cfg("mx_basic", d, H, M=M, **_MX)
             for M, H, d in _prod((1, 4, 16, 7, 25, 128, 8192), (128, 256, 512, 1536, 2048, 4096), _DTYPES)]
_CROSS = (
    [_cfg("fused_vs_separate", "float16", H, M=M)
     for M, H in _prod((4, 16, 128, 512, 8192), (256, 512, 1024, 1536, 4096, 8192))]
    + [_cfg("nv_matches_separate", d, H, M=M)
       for M, H, d in _prod((1, 4, 16, 128), (64, 256, 512, 1024, 2048, 4096), _DTYPES)]
    + [_cfg("mx_matches_separate", d, H, M=M, **_MX)
       for M, H, d in _prod((1, 4, 16, 128), (128, 256, 512, 1024, 2048, 4096), _DTYPES)]
    + [_cfg("global_scale_consistency", "float16", H, M=M, global_scale_mode="nonunit")
       for M, H in _prod((1, 16, 64), (256, 1024, 4096))]
)
_LARGE_H = (
    [_cfg("large_h_nv", d, H, M=M) for M, H, d in _prod((1, 16, 128, 1024), (16384, 32768), _DTYPES)]
    + [_cfg("large_h_mx", d, H, M=M, **_MX) for M, H, d in _prod((1, 16, 128, 1024), (16384, 32768), _DTYPES)]
)
_SWIZZLED = (
    [_cfg("swizzled_nv", d, H, M=M, swizzled=True)
     for M, H, d in _prod((1, 16, 128, 256), (512, 1024, 2048, 4096), _DTYPES)]
    + [_cfg("swizzled_mx", d, H, M=M, swizzled=True, **_MX)
       for M, H, d in _prod((1, 16, 128, 256), (512, 1024, 2048, 4096), _DTYPES)]
)
_ALLOCATION = (
    [_cfg("auto2d_nv", d, H, M=M, allocation="auto") for M, H, d in _prod((1, 16, 128), (256, 1024, 4096), _DTYPES)]
    + [_cfg("auto3d_nv", "float16", H, B=B, S=S, allocation="auto")
       for B, S, H in _prod((1, 4, 16), (16, 64), (256, 1024))]
    + [_cfg("auto_mx", "float16", H, M=M, allocation="auto", **_MX) for M, H in _prod((1, 16, 128), (256, 1024))]
    + [_cfg("auto_swizzled", "float16", H, M=M, swizzled=True, allocation="auto")
       for M, H in _prod((16, 128), (512, 1024))]
    + [_cfg("auto_matches_preallocated", "float16", H, M=M, allocation="compare")
       for M, H in _prod((16, 128), (512, 1024))]
)
_UPSTREAM = [*_NV2D, *_NV3D, *_LARGE_BATCH, *_MX_BASIC, *_CROSS, *_LARGE_H, *_SWIZZLED, *_ALLOCATION]

_STRUCTURE = [
    _cfg("subwarp_rows_tail", "float16", 64, M=17),
    _cfg("subwarp_mx", "bfloat16", 64, M=17, **_MX),
    _cfg("column_tail_nv", "bfloat16", 80, M=129, swizzled=True),
    _cfg("column_tail_mx", "float16", 160, M=3, **_MX),
    *[_cfg("thread_threshold", "bfloat16", H, M=3) for H in (3072, 3088, 6144, 6160, 14336, 16384, 16400)],
    _cfg("cluster2", "bfloat16", 65536, M=1),
    _cfg("cluster16", "bfloat16", 1048576, M=1, enable_pdl=True),
    _cfg("pdl", "bfloat16", 4096, M=3, enable_pdl=True),
    _cfg("block32_e4m3", "float16", 4096, M=3, block_size=32, scale_format="e4m3", global_scale_mode="nonunit"),
    _cfg("block16_requested_ue8", "float16", 4096, M=3, block_size=16, scale_format="ue8m0"),
    _cfg("zero_input", "bfloat16", 4096, M=3, data_mode="zero"),
    _cfg("zero_global_scale", "float16", 4096, M=3, global_scale_mode="zero"),
]

CONFIGS = [*_UPSTREAM, *_STRUCTURE]

assert len(_UPSTREAM) == 1007 and len(_STRUCTURE) == 18
assert len({config["label"] for config in CONFIGS}) == len(CONFIGS)

# The reference's six latency-bound shapes, then the throughput shape this build is measured on
# (8192 tokens x hidden 7168, gamma = 1 + 0.1*N(0,1), swizzled NVFP4 scales).
BENCH_CONFIGS = [
    _cfg("bench_nv", "bfloat16", 4096, M=32, global_scale_mode="none"),
    _cfg("bench_nv_large", "bfloat16", 8192, M=64, global_scale_mode="none"),
    _cfg("bench_nv_global", "bfloat16", 4096, M=32, global_scale_mode="one"),
    _cfg("bench_nv_swizzled", "bfloat16", 4096, M=32, swizzled=True, global_scale_mode="none"),
    _cfg("bench_mx", "bfloat16", 4096, M=32, **_MX),
    _cfg("bench_nv_3d", "bfloat16", 128, B=32, S=32, global_scale_mode="none"),
    _cfg("bench_nv_swizzled_large", "bfloat16", 7168, M=8192, swizzled=True, weight_mode="gamma"),
]

__all__ = ["BENCH_CONFIGS", "CONFIGS", "KERNEL_META", "get_kernel", "prepare_bench", "prepare_data",
           "run_bench", "run_gpu", "run_test"]
