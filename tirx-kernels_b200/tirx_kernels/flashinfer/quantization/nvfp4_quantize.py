"""``nvfp4_quantize``: NVFP4 block quantizer, hand-written CUDA behind the reference interface.

Drop-in for tirx_kernels/flashinfer/quantization/nvfp4_quantize.py of the reference: same
``KERNEL_META``, config keys and labels (``_cfg`` :577-589, ``CONFIGS`` :597-619,
``BENCH_CONFIGS`` :622-635), the same positional executable signature
(``ex(in_flat, out_flat, sf, m, total_sf | padded_m, global_scale)``, :214-221 / :259-266),
caller-owned outputs, ``ValueError`` on shapes outside the dispatch domain (:90-98).

One 16-element block yields one E4M3 scale byte and eight packed E2M1 bytes; scale factors are
written in the linear, 128x4-swizzled or 8x4-swizzled layout (padding zero-filled); the
``fuse_silu`` variant quantizes SiLU(gate)*up of a ``[m, 2k]`` input.  The kernel is
``b2_nvfp4_quantize`` in the C-ABI library.
"""

from __future__ import annotations

from typing import Any

from tirx_kernels import _checks, _native
from tirx_kernels._protocol import KernelHandle
from tirx_kernels.runner import bench

KERNEL_META = {"name": "nvfp4_quantize", "category": "flashinfer", "compute_capability": 10}

_DTYPES = ("float16", "bfloat16")
_SF_LAYOUTS = ("linear", "128x4", "8x4")
NVFP4_SF_VEC_SIZE = 16


def _torch_dtype(dtype: str):
    import torch

    return {"float16": torch.float16, "bfloat16": torch.bfloat16}[dtype]


def _validate(dtype: str, m: int, k: int, sf_layout: str, fuse_silu: bool) -> None:
    if dtype not in _DTYPES:
        raise ValueError(f"Unsupported dtype: {dtype}")
    if sf_layout not in _SF_LAYOUTS:
        raise ValueError(f"Unsupported sf_layout: {sf_layout}")
    if m < 1:
        raise ValueError(f"m={m} must be >= 1")
    if k <= 0 or k % NVFP4_SF_VEC_SIZE != 0:
        raise ValueError(f"k={k} outside the source dispatch domain (k % 16 != 0)")


def _padded_m(m: int, sf_layout: str) -> int:
    tile = 8 if sf_layout == "8x4" else 128
    return _checks.ceil_div(m, tile) * tile


def _padded_sf_cols(k: int) -> int:
    return _checks.padded_sf_cols(k // NVFP4_SF_VEC_SIZE)


def _sf_numel(m: int, k: int, sf_layout: str) -> int:
    return _checks.sf_numel(m, k // NVFP4_SF_VEC_SIZE, sf_layout)


def algorithmic_bytes(m: int, k: int, sf_layout: str, fuse_silu: bool = False) -> int:
    """Bytes one launch must move: input + packed output + scale buffer + the global scale."""
    return m * k * 2 * (2 if fuse_silu else 1) + m * k // 2 + _sf_numel(m, k, sf_layout) + 4


class _Executable:
    """Launchable with the reference executable's positional signature."""

    def __init__(self, dtype: str, m: int, k: int, sf_layout: str, fuse_silu: bool, enable_pdl: bool):
        self.dtype, self.m, self.k = dtype, m, k
        self.sf_layout, self.fuse_silu, self.enable_pdl = sf_layout, fuse_silu, enable_pdl

    def __call__(self, in_flat, out_flat, sf, m_rows: int, total_sf_or_padded_m: int, global_scale) -> None:
        expected = (m_rows * (self.k // NVFP4_SF_VEC_SIZE) if self.sf_layout == "linear"
                    else _padded_m(m_rows, self.sf_layout))
        if total_sf_or_padded_m != expected:
            raise ValueError(f"inconsistent launch argument {total_sf_or_padded_m}, expected {expected}")
        if in_flat.numel() != m_rows * self.k * (2 if self.fuse_silu else 1):
            raise ValueError("input element count does not match (m, k)")
        if out_flat.numel() != m_rows * self.k // 2 or sf.numel() != _sf_numel(m_rows, self.k, self.sf_layout):
            raise ValueError("output buffers do not match (m, k, sf_layout)")
        _native.nvfp4_quantize(in_flat, out_flat, sf, global_scale, m_rows, self.k, self.dtype,
                               self.sf_layout, self.fuse_silu, self.enable_pdl)


def get_kernel(dtype: str, m: int, k: int, sf_layout: str = "128x4", fuse_silu: bool = False,
               enable_pdl: bool = False, **kwargs) -> KernelHandle:
    """Handle for one (dtype, m, k, sf_layout, fuse_silu) specialization."""
    _validate(dtype, m, k, sf_layout, fuse_silu)
    launcher = _Executable(dtype, m, k, sf_layout, fuse_silu, enable_pdl)
    return KernelHandle("b2_nvfp4_quantize", {"launcher": launcher, "dtype": dtype, "m": m, "k": k,
                                              "sf_layout": sf_layout, "fuse_silu": fuse_silu,
                                              "enable_pdl": enable_pdl})


def prepare_data(dtype: str, m: int, k: int, sf_layout: str = "128x4", fuse_silu: bool = False,
                 enable_pdl: bool = False, **kwargs):
    """A seeded ``[m, k]`` (``[m, 2k]`` with fuse_silu) input and a ``[1]`` fp32 global scale.

    Drawn on the CPU (generator seed 42) and copied to the device so that a host-side oracle
    sees the same bits; the reference seeds the CUDA generator instead (:394-396).
    """
    import torch

    _validate(dtype, m, k, sf_layout, fuse_silu)
    generator = torch.Generator().manual_seed(42)
    a = torch.randn(m, k * (2 if fuse_silu else 1), generator=generator, dtype=torch.float32)
    global_scale = torch.rand(1, generator=generator, dtype=torch.float32) + 0.5
    return a.to(_torch_dtype(dtype)).cuda(), global_scale.cuda()


def _alloc_outputs(m: int, k: int, sf_layout: str):
    import torch

    out = torch.empty(m, k // 2, dtype=torch.uint8, device="cuda")
    sf = torch.empty(_sf_numel(m, k, sf_layout), dtype=torch.uint8, device="cuda")
    return out, sf


def _run_launch(ex, a, gs, out, sf, m, k, sf_layout):
    if sf_layout == "linear":
        ex(a.view(-1), out.view(-1), sf, m, m * (k // NVFP4_SF_VEC_SIZE), gs)
    else:
        ex(a.view(-1), out.view(-1), sf, m, _padded_m(m, sf_layout), gs)


def _self_check(a, gs, out, sf, dtype, m, k, sf_layout, fuse_silu) -> None:
    """Checks that need no second implementation: decode error bound and zeroed padding."""
    import torch

    x = a.float()
    if fuse_silu:
        x = (torch.nn.functional.silu(x[:, :k]) * x[:, k:]).to(_torch_dtype(dtype)).float()
    deq = _checks.dequantize(out, sf, sf_layout, global_scale=float(gs.item()))
    if not torch.isfinite(deq).all():
        raise AssertionError("dequantized output contains non-finite values")
    block_amax = x.view(m, -1, 16).abs().amax(dim=-1, keepdim=True).expand(-1, -1, 16).reshape(m, k)
    # E2M1 spacing is at most 2/6 of the block maximum; the E4M3 scale adds at most 1/16 relative.
    bound = block_amax * (1.0 / 6.0 + 1.0 / 8.0) + 1e-6
    worst = ((deq - x).abs() - bound).max().item()
    if worst > 0:
        raise AssertionError(f"dequantized value off by more than the format allows (excess {worst:.4g})")
    if sf_layout != "linear":
        mask = _checks.padding_mask(m, k // 16, sf_layout, sf.device)
        if torch.count_nonzero(sf[mask]):
            raise AssertionError("padding scale factors are not zero")


def run_test(dtype: str, m: int, k: int, sf_layout: str = "128x4", fuse_silu: bool = False,
             enable_pdl: bool = False, **kwargs) -> None:
    """Launch one config and validate it.

    With an expected-value provider installed (``runner.set_reference_provider``) the packed
    bytes and the whole scale buffer must match it exactly, as the reference demands of its
    own oracle (:479-481); the self-contained checks run in every case.
    """
    import torch

    from tirx_kernels.runner import compile_kernel, reference_provider

    a, gs = prepare_data(dtype=dtype, m=m, k=k, sf_layout=sf_layout, fuse_silu=fuse_silu)
    ex = compile_kernel(get_kernel(dtype=dtype, m=m, k=k, sf_layout=sf_layout, fuse_silu=fuse_silu,
                                   enable_pdl=enable_pdl))
    out, sf = _alloc_outputs(m, k, sf_layout)
    sf.fill_(_checks.GUARD_BYTE)
    snapshot = a.clone()
    _run_launch(ex, a, gs, out, sf, m, k, sf_layout)
    torch.cuda.synchronize()
    if not torch.equal(a, snapshot):
        raise AssertionError("input tensor was modified")
    provider = reference_provider()
    if provider is not None:
        ref_fp4, ref_sf = provider("nvfp4_quantize", a=a, global_scale=gs, dtype=dtype,
                                   sf_layout=sf_layout, fuse_silu=fuse_silu)
        torch.testing.assert_close(out.cpu(), ref_fp4.reshape(out.shape), rtol=0, atol=0)
        torch.testing.assert_close(sf.cpu(), ref_sf.reshape(-1), rtol=0, atol=0)
    _self_check(a, gs, out, sf, dtype, m, k, sf_layout, fuse_silu)


def prepare_bench(**kwargs: Any):
    """Bind the executable before the workload touches a GPU."""
    from tirx_kernels.runner import compile_kernel, prepared_gpu_benchmark

    state = {"config": dict(kwargs), "executable": compile_kernel(get_kernel(**kwargs))}
    return prepared_gpu_benchmark(run_gpu, state)


def run_gpu(prepared, *, warmup=None, repeat=None, timer=None, rounds=1, cooldown_s=1.0, **kwargs):
    """Kernel-only timing of one config; the record carries its HBM roofline."""
    config = {**prepared["config"], **kwargs}
    dtype, m, k = config["dtype"], config["m"], config["k"]
    sf_layout = config.get("sf_layout", "128x4")
    fuse_silu = config.get("fuse_silu", False)
    ex = prepared["executable"]
    a, gs = prepare_data(dtype=dtype, m=m, k=k, sf_layout=sf_layout, fuse_silu=fuse_silu)
    out, sf = _alloc_outputs(m, k, sf_layout)

    def tirx_launch():
        _run_launch(ex, a, gs, out, sf, m, k, sf_layout)

    result = bench({"tirx": tirx_launch}, warmup=warmup, repeat=repeat, timer=timer, rounds=rounds,
                   cooldown_s=cooldown_s)
    result["roofline"] = _checks.roofline_hbm(algorithmic_bytes(m, k, sf_layout, fuse_silu),
                                              result["impls"]["tirx"])
    return result


def run_bench(dtype: str, m: int, k: int, sf_layout: str = "128x4", fuse_silu: bool = False,
              enable_pdl: bool = False, *, warmup=None, repeat=None, timer=None, rounds=1,
              cooldown_s=1.0, **kwargs):
    prepared = prepare_bench(dtype=dtype, m=m, k=k, sf_layout=sf_layout, fuse_silu=fuse_silu,
                             enable_pdl=enable_pdl, **kwargs)
    return prepared.run_gpu(warmup=warmup, repeat=repeat, timer=timer, rounds=rounds, cooldown_s=cooldown_s)


def _cfg(dtype, m, k, sf_layout="128x4", fuse_silu=False, enable_pdl=False):
    short = {"float16": "fp16", "bfloat16": "bf16"}[dtype]
    label = f"{short}_{sf_layout}_m{m}_k{k}" + ("_silu" if fuse_silu else "") + ("_pdl" if enable_pdl else "")
    return {"label": label, "dtype": dtype, "m": m, "k": k, "sf_layout": sf_layout,
            "fuse_silu": fuse_silu, "enable_pdl": enable_pdl}


# The reference's correctness matrix (same labels): both dtypes; the three layouts; SiLU fusion;
# row padding (120 -> 128, 13 -> 16), column padding (65 -> 68, 513 -> 516), rows wider than
# 512 scale blocks; the minimal 1x16 shape; the PDL variant.
CONFIGS = [
    _cfg("float16", 1, 16, "linear"),
    _cfg("float16", 128, 1024, "linear"),
    _cfg("bfloat16", 128, 1024, "linear"),
    _cfg("float16", 512, 4096, "linear"),
    _cfg("bfloat16", 512, 4096, "linear"),
    _cfg("float16", 13, 1040, "linear"),
    _cfg("float16", 128, 1024, "128x4"),
    _cfg("bfloat16", 128, 1024, "128x4"),
    _cfg("float16", 120, 1024, "128x4"),
    _cfg("float16", 128, 1040, "128x4"),
    _cfg("float16", 512, 4096, "128x4"),
    _cfg("bfloat16", 512, 4096, "128x4"),
    _cfg("float16", 64, 8256, "128x4"),
    _cfg("float16", 64, 8208, "128x4"),
    _cfg("float16", 13, 1024, "8x4"),
    _cfg("bfloat16", 128, 1024, "8x4"),
    _cfg("float16", 128, 1024, "linear", True),
    _cfg("float16", 128, 1024, "128x4", True),
    _cfg("bfloat16", 512, 4096, "128x4", True),
    _cfg("float16", 64, 8256, "128x4", True),
    _cfg("float16", 512, 4096, "linear", False, True),
]

# The reference's sweep, then the two shapes this build is measured on.
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
    _cfg("float16", 4096, 3584, "128x4", True),
    _cfg("bfloat16", 4096, 3584, "128x4", True),
    _cfg("bfloat16", 4096, 7168, "linear"),
    _cfg("bfloat16", 16384, 7168, "128x4"),
]
