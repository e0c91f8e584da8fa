"""``nvfp4_quantize_per_token``: NVFP4 block quantizer with one scale per token row (CUDA, sm_100a).

Drop-in for tirx_kernels/flashinfer/quantization/nvfp4_quantize_per_token.py of the reference:
same ``KERNEL_META`` (:77-81), config keys and labels (``_cfg`` :409-421, ``CONFIGS`` :429-447,
``BENCH_CONFIGS`` :450-461), the positional executable signature
``ex(a_flat, out_flat, sf, pts, m, gs_inv)`` (:145-152, :321) and ``ValueError`` for shapes outside
the dispatch domain (:102-110).

``pts[r] = amax(row r) * gs_inv`` is the scale a consumer multiplies back in; the row's blocks are
quantized with its reciprocal in place of the global scale.  The kernel is
``b2_nvfp4_quantize_per_token`` in the C-ABI library; it also zero-fills the padding rows of the
swizzled layouts, which the reference leaves to a zero-initialised buffer.
"""

from __future__ import annotations

from typing import Any

from tirx_kernels import _checks, _native
from tirx_kernels._protocol import KernelHandle
from tirx_kernels.runner import bench

KERNEL_META = {
    "name": "nvfp4_quantize_per_token",
    "category": "flashinfer",
    "compute_capability": 10,
}

_DTYPES = ("float16", "bfloat16")
_SF_LAYOUTS = ("linear", "128x4", "8x4")
NVFP4_SF_VEC_SIZE = 16


def _torch_dtype(dtype: str):
    import torch

    return {"float16": torch.float16, "bfloat16": torch.bfloat16}[dtype]


def _validate(dtype: str, m: int, k: int, sf_layout: str) -> None:
    if dtype not in _DTYPES:
        raise ValueError(f"Unsupported dtype: {dtype}")
    if sf_layout not in _SF_LAYOUTS:
        raise ValueError(f"Unsupported sf_layout: {sf_layout}")
    if m < 1:
        raise ValueError(f"m={m} must be >= 1")
    if k <= 0 or k % NVFP4_SF_VEC_SIZE != 0:
        raise ValueError(f"k={k} outside the source dispatch domain (k % 16 != 0)")


def _padded_m(m: int, sf_layout: str) -> int:
    if sf_layout == "linear":
        return m
    tile = 8 if sf_layout == "8x4" else 128
    return _checks.ceil_div(m, tile) * tile


def _padded_sf_cols(k: int, sf_layout: str) -> int:
    cols = k // NVFP4_SF_VEC_SIZE
    return cols if sf_layout == "linear" else _checks.ceil_div(cols, 4) * 4


def _sf_numel(m: int, k: int, sf_layout: str) -> int:
    return _padded_m(m, sf_layout) * _padded_sf_cols(k, sf_layout)


def algorithmic_bytes(m: int, k: int, sf_layout: str) -> int:
    """Input once + packed output + the scale buffer + one fp32 scale per row + the inverse global scale."""
    return m * k * 2 + m * k // 2 + _sf_numel(m, k, sf_layout) + m * 4 + 4


class _Executable:
    """Launchable with the reference executable's positional signature; returns None."""

    def __init__(self, dtype: str, k: int, sf_layout: str, enable_pdl: bool):
        self.dtype, self.k, self.sf_layout, self.enable_pdl = dtype, k, sf_layout, enable_pdl

    def __call__(self, a_flat, out_flat, sf, pts, m: int, gs_inv) -> None:
        k = self.k
        if a_flat.numel() != m * k or out_flat.numel() != m * (k // 2) or pts.numel() != m:
            raise ValueError("tensor sizes do not match (m, k)")
        if sf.numel() != _sf_numel(m, k, self.sf_layout):
            raise ValueError("scale buffer size does not match the layout")
        _native.nvfp4_quantize_per_token(a_flat, out_flat, sf, pts, gs_inv, m, k, self.dtype, self.sf_layout,
                                         self.enable_pdl)


def get_kernel(dtype: str, m: int, k: int, sf_layout: str = "128x4", enable_pdl: bool = False,
               **kwargs) -> KernelHandle:
    """Handle for one (dtype, k, sf_layout) specialization."""
    _validate(dtype, m, k, sf_layout)
    launcher = _Executable(dtype, k, sf_layout, enable_pdl)
    return KernelHandle("b2_nvfp4_quantize_per_token", {"launcher": launcher, "dtype": dtype, "m": m, "k": k,
                                                        "sf_layout": sf_layout, "enable_pdl": enable_pdl})


def prepare_data(dtype: str, m: int, k: int, sf_layout: str = "128x4", enable_pdl: bool = False,
                 zero_row: bool = False, **kwargs):
    """A seeded ``[m, k]`` input and the ``[1]`` fp32 inverse global scale 1 / (448 * 6) (:235-256).

    Drawn on the CPU (generator seed 42) so that a host-side oracle sees the same bits;
    ``zero_row`` blanks row 0 to reach the all-zero-row path.
    """
    import torch

    _validate(dtype, m, k, sf_layout)
    generator = torch.Generator().manual_seed(42)
    a = torch.randn(m, k, generator=generator, dtype=torch.float32).to(_torch_dtype(dtype))
    if zero_row:
        a[0].zero_()
    gs_inv = torch.tensor([1.0 / (448.0 * 6.0)], dtype=torch.float32)
    return a.cuda(), gs_inv.cuda()


def _alloc_outputs(m: int, k: int, sf_layout: str):
    import torch

    out = torch.empty(m, k // 2, dtype=torch.uint8, device="cuda")
    sf = torch.empty(_sf_numel(m, k, sf_layout), dtype=torch.uint8, device="cuda")
    pts = torch.empty(m, dtype=torch.float32, device="cuda")
    return out, sf, pts


def _self_check(a, gs_inv, out, sf, pts, m, k, sf_layout) -> None:
    """Checks that need no second implementation: token scales, decode error bound, zeroed padding."""
    import torch

    x = a.float()
    want_pts = x.abs().amax(dim=-1) * float(gs_inv.item())
    torch.testing.assert_close(pts, want_pts, rtol=1e-6, atol=0.0)
    # value = e2m1 * e4m3 * token_scale: decode with a unit global scale, then apply the row scale
    deq = _checks.dequantize(out, sf, sf_layout, global_scale=1.0) * pts[:, None]
    if not torch.isfinite(deq).all():
        raise AssertionError("dequantized output contains non-finite values")
    block_amax = x.view(m, -1, 16).abs().amax(dim=-1, keepdim=True).expand(-1, -1, 16).reshape(m, k)
    bound = block_amax * (1.0 / 6.0 + 1.0 / 8.0) + 1e-6
    worst = ((deq - x).abs() - bound).max().item()
    if worst > 0:
        raise AssertionError(f"dequantized value off by more than the format allows (excess {worst:.4g})")
    if sf_layout != "linear":
        mask = _checks.padding_mask(m, k // 16, sf_layout, sf.device)
        if torch.count_nonzero(sf[mask]):
            raise AssertionError("padding scale factors are not zero")


def run_test(dtype: str, m: int, k: int, sf_layout: str = "128x4", enable_pdl: bool = False,
             zero_row: bool = False, **kwargs) -> None:
    """Launch one config and validate it: packed bytes, the whole scale buffer and the token scales
    must equal an installed expected-value provider bit for bit (the reference demands the same of
    its own oracle, :324-327); the self-contained checks run in every case."""
    import torch

    from tirx_kernels.runner import compile_kernel, reference_provider

    a, gs_inv = prepare_data(dtype=dtype, m=m, k=k, sf_layout=sf_layout, zero_row=zero_row)
    ex = compile_kernel(get_kernel(dtype=dtype, m=m, k=k, sf_layout=sf_layout, enable_pdl=enable_pdl))
    out, sf, pts = _alloc_outputs(m, k, sf_layout)
    sf.fill_(_checks.GUARD_BYTE)
    snapshot = a.clone()
    if ex(a.view(-1), out.view(-1), sf, pts, m, gs_inv) is not None:
        raise AssertionError("executable must return None")
    torch.cuda.synchronize()
    if not torch.equal(a, snapshot):
        raise AssertionError("input tensor was modified")
    provider = reference_provider()
    if provider is not None:
        ref_fp4, ref_sf, ref_pts = provider("nvfp4_quantize_per_token", a=a, gs_inv=gs_inv, dtype=dtype,
                                            sf_layout=sf_layout)
        torch.testing.assert_close(out.cpu(), ref_fp4.reshape(out.shape), rtol=0, atol=0)
        torch.testing.assert_close(sf.cpu(), ref_sf.reshape(-1), rtol=0, atol=0)
        torch.testing.assert_close(pts.cpu(), ref_pts.reshape(-1), rtol=0, atol=0)
    _self_check(a, gs_inv, out, sf, pts, m, k, sf_layout)


def prepare_bench(**kwargs: Any):
    from tirx_kernels.runner import compile_kernel, prepared_gpu_benchmark

    state = {"config": dict(kwargs), "executable": compile_kernel(get_kernel(**kwargs))}
    return prepared_gpu_benchmark(run_gpu, state)


def run_gpu(prepared, *, warmup=None, repeat=None, timer=None, rounds=1, cooldown_s=1.0, **kwargs):
    """Kernel-only timing of one config; the record carries its HBM roofline."""
    config = {**prepared["config"], **kwargs}
    dtype, m, k = config["dtype"], config["m"], config["k"]
    sf_layout = config.get("sf_layout", "128x4")
    ex = prepared["executable"]
    a, gs_inv = prepare_data(dtype=dtype, m=m, k=k, sf_layout=sf_layout, zero_row=config.get("zero_row", False))
    out, sf, pts = _alloc_outputs(m, k, sf_layout)

    def tirx_launch():
        ex(a.view(-1), out.view(-1), sf, pts, m, gs_inv)

    result = bench({"tirx": tirx_launch}, warmup=warmup, repeat=repeat, timer=timer, rounds=rounds,
                   cooldown_s=cooldown_s)
    result["roofline"] = _checks.roofline_hbm(algorithmic_bytes(m, k, sf_layout), result["impls"]["tirx"])
    return result


def run_bench(dtype: str, m: int, k: int, sf_layout: str = "128x4", enable_pdl: bool = False,
              zero_row: bool = False, *, warmup=None, repeat=None, timer=None, rounds=1, cooldown_s=1.0,
              **kwargs):
    prepared = prepare_bench(dtype=dtype, m=m, k=k, sf_layout=sf_layout, enable_pdl=enable_pdl,
                             zero_row=zero_row, **kwargs)
    return prepared.run_gpu(warmup=warmup, repeat=repeat, timer=timer, rounds=rounds, cooldown_s=cooldown_s)


def _cfg(dtype, m, k, sf_layout="128x4", enable_pdl=False, zero_row=False):
    dt = {"float16": "fp16", "bfloat16": "bf16"}[dtype]
    label = f"{dt}_{sf_layout}_m{m}_k{k}{'_zerorow' if zero_row else ''}{'_pdl' if enable_pdl else ''}"
    return {"label": label, "dtype": dtype, "m": m, "k": k, "sf_layout": sf_layout, "enable_pdl": enable_pdl,
            "zero_row": zero_row}


# Both dtypes; the three scale layouts; an all-zero row; swizzled row and column padding; rows with
# more than 128 scale blocks; the smallest shape; the PDL variant.
CONFIGS = [
    _cfg("float16", 1, 16, "linear"),
    _cfg("float16", 128, 1024, "linear"),
    _cfg("bfloat16", 128, 1024, "linear"),
    _cfg("float16", 512, 4096, "linear"),
    _cfg("bfloat16", 512, 4096, "linear"),
    _cfg("float16", 13, 1040, "linear"),
    _cfg("float16", 128, 1024, "linear", False, True),
    _cfg("float16", 128, 1024, "128x4"),
    _cfg("bfloat16", 128, 1024, "128x4"),
    _cfg("float16", 120, 1024, "128x4"),
    _cfg("float16", 128, 1040, "128x4"),
    _cfg("float16", 512, 4096, "128x4"),
    _cfg("bfloat16", 512, 4096, "128x4"),
    _cfg("float16", 64, 8256, "128x4"),
    _cfg("float16", 13, 1024, "8x4"),
    _cfg("bfloat16", 128, 1024, "8x4"),
    _cfg("float16", 512, 4096, "128x4", True),
]

BENCH_CONFIGS = [
    _cfg("float16", 4096, 4096, "linear"),
    _cfg("bfloat16", 4096, 4096, "linear"),
    _cfg("float16", 4096, 4096, "128x4"),
    _cfg("bfloat16", 4096, 4096, "128x4"),
    _cfg("float16", 16384, 7168, "linear"),
    _cfg("float16", 16384, 7168, "128x4"),
    _cfg("float16", 1024, 2048, "linear"),
    _cfg("float16", 1024, 2048, "128x4"),
    _cfg("float16", 128, 1024, "linear"),
    _cfg("float16", 128, 1024, "128x4"),
]

__all__ = ["BENCH_CONFIGS", "CONFIGS", "KERNEL_META", "get_kernel", "prepare_bench", "prepare_data",
           "run_bench", "run_gpu", "run_test"]
