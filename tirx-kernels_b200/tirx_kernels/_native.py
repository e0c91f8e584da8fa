"""ctypes binding of the C-ABI library (include/b200_nvfp4.h).

The library is the product: if it is missing or a symbol cannot be resolved, import of a
kernel module fails loudly.  Nothing here falls back to PyTorch or CPU code.
"""

from __future__ import annotations

import ctypes
import os
from pathlib import Path

DTYPE_CODES = {"float16": 0, "bfloat16": 1}
SF_LAYOUT_CODES = {"linear": 0, "128x4": 1, "8x4": 2}
SCALE_FORMAT_CODES = {"e4m3": 0, "ue8m0": 1}
MUFU_OPS = {"rcp_ftz": 0, "rsqrt_ftz": 1, "lg2": 2, "ex2": 3, "ex2_ftz": 4,
            # the quantizer's SiLU as its kernel computes it / with div.rn.f32 throughout
            "silu": 5, "silu_div_rn": 6}

OK, ERR_INVALID_ARGUMENT, ERR_CUDA, ERR_DEVICE_TIMEOUT, ERR_UNSUPPORTED = range(5)

_LIB_DIR = Path(__file__).resolve().parent.parent / "lib"
_MAIN = None
_CUBLASLT = None

_vp, _i, _f, _i64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_int64

# symbol -> (restype, argtypes); every name include/b200_nvfp4.h declares for the main library
MAIN_SIGNATURES = {
    "b2_last_error": (ctypes.c_char_p, []),
    "b2_abi_version": (_i, []),
    "b2_nvfp4_quantize": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp]),
    "b2_nvfp4_quantize_per_token": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp]),
    "b2_nvfp4_sf_bytes": (_i64, [_i, _i, _i]),
    "b2_rmsnorm_fp4quant": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _f, _i, _i, _i, _i, _i, _vp]),
    "b2_add_rmsnorm_fp4quant": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _f, _i, _i, _i, _i, _i, _i, _i, _vp]),
    "b2_nvfp4_gemm": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp]),
    "b2_rmsnorm_fp4quant_timeline": (_i, [_vp]),
    "b2_nvfp4_gemm_small_m_noalloc": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp]),
    "b2_nvfp4_gemm_status": (_i, [_vp]),
    "b2_nvfp4_gemm_small_m_noalloc_status": (_i, [_vp]),
    "b2_nvfp4_gemm_set_wait_budget_ms": (_i, [_i]),
    "b2_nvfp4_gemm_inject_test_fault": (_i, [_i]),
    "b2_nvfp4_gemm_set_variant": (_i, [_i]),
    "b2_nvfp4_gemm_role_timers": (_i, [_i, _vp, _vp]),
    "b2_mufu_probe": (_i, [_i, _vp, _vp, _i, _vp]),
    "b2_peer_alloc": (_i, [ctypes.POINTER(ctypes.c_void_p), _i64]),
    "b2_peer_free": (_i, [_vp]),
    "b2_peer_export": (_i, [_vp, ctypes.c_char_p]),
    "b2_peer_open": (_i, [ctypes.c_char_p, ctypes.POINTER(ctypes.c_void_p)]),
    "b2_peer_close": (_i, [_vp]),
    "b2_nvfp4_gemm_allgather": (_i, [_vp, _vp, _vp, _vp, _vp, ctypes.POINTER(ctypes.c_void_p), _i, _i, _i, _i, _i, _vp]),
}
CUBLASLT_SIGNATURES = {
    "b2_nvfp4_gemm_cublaslt": (_i, [_vp, _vp, _vp, _vp, _f, _vp, _i, _i, _i, _vp]),
}


class NativeLibraryError(RuntimeError):
    """The CUDA extension is absent or incomplete; there is no fallback path."""


def library_path(name: str = "libb200nvfp4.so") -> Path:
    override = os.environ.get("B200_NVFP4_LIB_DIR")
    return (Path(override) if override else _LIB_DIR) / name


def _load(name: str, signatures: dict) -> ctypes.CDLL:
    path = library_path(name)
    if not path.exists():
        raise NativeLibraryError(
            f"{path} not found: build it with `python tirx-kernels_b200/build.py` "
            "(nvcc, sm_100a). This package has no CPU or PyTorch fallback."
        )
    lib = ctypes.CDLL(str(path))
    for symbol, (restype, argtypes) in signatures.items():
        try:
            fn = getattr(lib, symbol)
        except AttributeError as exc:
            raise NativeLibraryError(f"{path} does not export {symbol}") from exc
        fn.restype = restype
        fn.argtypes = argtypes
    return lib


def lib() -> ctypes.CDLL:
    global _MAIN
    if _MAIN is None:
        _MAIN = _load("libb200nvfp4.so", MAIN_SIGNATURES)
    return _MAIN


def cublaslt_lib() -> ctypes.CDLL:
    global _CUBLASLT
    if _CUBLASLT is None:
        _preload_torch_cublaslt()
        _CUBLASLT = _load("libb200nvfp4_cublaslt.so", CUBLASLT_SIGNATURES)
    return _CUBLASLT


def _preload_torch_cublaslt() -> None:
    """Load the cuBLASLt build PyTorch ships before ours resolves its `libcublasLt.so.12`.

    PyTorch links against its own cuBLAS / cuBLASLt pair; if a different cuBLASLt with the same
    soname is mapped first, torch's cuBLAS later binds to it and fails with INVALID_VALUE.
    """
    try:
        import nvidia.cublas as _pkg

        for root in _pkg.__path__:
            candidate = Path(root) / "lib" / "libcublasLt.so.12"
            if candidate.exists():
                ctypes.CDLL(str(candidate), mode=ctypes.RTLD_GLOBAL)
                return
    except ImportError:
        pass


def last_error() -> str:
    return (lib().b2_last_error() or b"").decode(errors="replace")


def check(status: int, what: str) -> None:
    """Map a C status to the exception the reference raises at the same point."""
    if status == OK:
        return
    message = f"{what}: {last_error()}"
    if status in (ERR_INVALID_ARGUMENT, ERR_UNSUPPORTED):
        raise ValueError(message)
    raise RuntimeError(message)


def current_stream_ptr() -> int:
    import torch

    return int(torch.cuda.current_stream().cuda_stream)


def _ptr(tensor) -> int:
    return int(tensor.data_ptr())


def _require_cuda(*tensors) -> None:
    for t in tensors:
        if not t.is_cuda:
            raise ValueError("all tensors must be CUDA tensors")
        if not t.is_contiguous():
            raise ValueError("all tensors must be contiguous")


# ---- thin typed wrappers (torch tensors in, None out, asynchronous on the current stream) ----
def nvfp4_quantize(inp, out, sf, global_scale, m: int, k: int, dtype: str, sf_layout: str,
                   fuse_silu: bool = False, enable_pdl: bool = False) -> None:
    _require_cuda(inp, out, sf, global_scale)
    check(
        lib().b2_nvfp4_quantize(_ptr(inp), _ptr(out), _ptr(sf), _ptr(global_scale), m, k,
                                DTYPE_CODES[dtype], SF_LAYOUT_CODES[sf_layout], int(fuse_silu),
                                int(enable_pdl), current_stream_ptr()),
        "b2_nvfp4_quantize",
    )


def nvfp4_quantize_per_token(inp, out, sf, token_scale, gs_inv, m: int, k: int, dtype: str, sf_layout: str,
                             enable_pdl: bool = False) -> None:
    _require_cuda(inp, out, sf, token_scale, gs_inv)
    check(
        lib().b2_nvfp4_quantize_per_token(_ptr(inp), _ptr(out), _ptr(sf), _ptr(token_scale), _ptr(gs_inv), m, k,
                                          DTYPE_CODES[dtype], SF_LAYOUT_CODES[sf_layout], int(enable_pdl),
                                          current_stream_ptr()),
        "b2_nvfp4_quantize_per_token",
    )


def rmsnorm_fp4quant(x, weight, y, scales, global_scale, M: int, H: int, eps: float, dtype: str,
                     block_size: int, scale_format: str, swizzled: bool, enable_pdl: bool) -> None:
    _require_cuda(x, weight, y, scales, global_scale)
    check(
        lib().b2_rmsnorm_fp4quant(_ptr(x), _ptr(weight), _ptr(y), _ptr(scales), _ptr(global_scale),
                                  M, H, float(eps), DTYPE_CODES[dtype], block_size,
                                  SCALE_FORMAT_CODES[scale_format], int(swizzled), int(enable_pdl),
                                  current_stream_ptr()),
        "b2_rmsnorm_fp4quant",
    )


def add_rmsnorm_fp4quant(x, residual, weight, y, scales, scales_unswizzled, y_norm, global_scale, M: int, H: int,
                         eps: float, dtype: str, block_size: int, scale_format: str, swizzled: bool,
                         output_both_sf_layouts: bool, output_norm: bool, enable_pdl: bool) -> None:
    _require_cuda(x, residual, weight, y, scales, scales_unswizzled, y_norm, global_scale)
    check(
        lib().b2_add_rmsnorm_fp4quant(_ptr(x), _ptr(residual), _ptr(weight), _ptr(y), _ptr(scales),
                                      _ptr(scales_unswizzled), _ptr(y_norm), _ptr(global_scale), M, H, float(eps),
                                      DTYPE_CODES[dtype], block_size, SCALE_FORMAT_CODES[scale_format],
                                      int(swizzled), int(output_both_sf_layouts), int(output_norm),
                                      int(enable_pdl), current_stream_ptr()),
        "b2_add_rmsnorm_fp4quant",
    )


def nvfp4_gemm(A, B, SFA, SFB, alpha, D, M: int, N: int, K: int) -> None:
    _require_cuda(A, B, SFA, SFB, alpha, D)
    check(
        lib().b2_nvfp4_gemm(_ptr(A), _ptr(B), _ptr(SFA), _ptr(SFB), _ptr(alpha), _ptr(D), M, N, K,
                            current_stream_ptr()),
        "b2_nvfp4_gemm",
    )


def nvfp4_gemm_small_m_noalloc(A, B, SFA, SFB, alpha, D, M: int, N: int, K: int) -> None:
    """Decode-sized GEMM whose scratch is built into the library: for callers that may not allocate."""
    _require_cuda(A, B, SFA, SFB, alpha, D)
    check(
        lib().b2_nvfp4_gemm_small_m_noalloc(_ptr(A), _ptr(B), _ptr(SFA), _ptr(SFB), _ptr(alpha), _ptr(D),
                                            M, N, K, current_stream_ptr()),
        "b2_nvfp4_gemm_small_m_noalloc",
    )


def peer_alloc(nbytes: int) -> int:
    """Device allocation that can be exported to the other processes of the box; returns its address."""
    ptr = ctypes.c_void_p()
    check(lib().b2_peer_alloc(ctypes.byref(ptr), int(nbytes)), "b2_peer_alloc")
    return int(ptr.value)


def peer_free(ptr: int) -> None:
    check(lib().b2_peer_free(ptr), "b2_peer_free")


def peer_export(ptr: int) -> bytes:
    handle = ctypes.create_string_buffer(64)
    check(lib().b2_peer_export(ptr, handle), "b2_peer_export")
    return handle.raw


def peer_open(handle: bytes) -> int:
    if len(handle) != 64:
        raise ValueError("a peer handle is 64 bytes")
    ptr = ctypes.c_void_p()
    check(lib().b2_peer_open(handle, ctypes.byref(ptr)), "b2_peer_open")
    return int(ptr.value)


def peer_close(ptr: int) -> None:
    check(lib().b2_peer_close(ptr), "b2_peer_close")


def nvfp4_gemm_allgather(A, B, SFA, SFB, alpha, buffers, rank: int, M: int, N: int, K: int) -> None:
    """GEMM by this rank's weight slab; tiles land in columns [rank*N, (rank+1)*N) of every buffer.

    `buffers` are this process's addresses of all ranks' [M, world*N] bf16 buffers, in rank order.
    """
    _require_cuda(A, B, SFA, SFB, alpha)
    world = len(buffers)
    array = (ctypes.c_void_p * world)(*[int(b) for b in buffers])
    check(
        lib().b2_nvfp4_gemm_allgather(_ptr(A), _ptr(B), _ptr(SFA), _ptr(SFB), _ptr(alpha), array, world,
                                      int(rank), M, N, K, current_stream_ptr()),
        "b2_nvfp4_gemm_allgather",
    )


def nvfp4_gemm_set_variant(variant: int) -> None:
    check(lib().b2_nvfp4_gemm_set_variant(int(variant)), "b2_nvfp4_gemm_set_variant")


def nvfp4_gemm_status() -> None:
    check(lib().b2_nvfp4_gemm_status(current_stream_ptr()), "b2_nvfp4_gemm_status")


def nvfp4_gemm_small_m_noalloc_status() -> None:
    check(lib().b2_nvfp4_gemm_small_m_noalloc_status(current_stream_ptr()), "b2_nvfp4_gemm_small_m_noalloc_status")


def nvfp4_gemm_set_wait_budget_ms(milliseconds: int) -> None:
    """Test hook: budget of the kernels' bounded waits (0 = the default, one second)."""
    check(lib().b2_nvfp4_gemm_set_wait_budget_ms(int(milliseconds)), "b2_nvfp4_gemm_set_wait_budget_ms")


def nvfp4_gemm_inject_test_fault(fault: int) -> None:
    """Test hook: 1 = the next launch's first K slab never completes its barrier (no fault, no hang)."""
    check(lib().b2_nvfp4_gemm_inject_test_fault(int(fault)), "b2_nvfp4_gemm_inject_test_fault")


def nvfp4_gemm_cublaslt(A, B, SFA, SFB, alpha: float, D, M: int, N: int, K: int) -> None:
    _require_cuda(A, B, SFA, SFB, D)
    status = cublaslt_lib().b2_nvfp4_gemm_cublaslt(_ptr(A), _ptr(B), _ptr(SFA), _ptr(SFB),
                                                   float(alpha), _ptr(D), M, N, K,
                                                   current_stream_ptr())
    if status != OK:
        raise RuntimeError(f"b2_nvfp4_gemm_cublaslt failed with status {status}")


def mufu_probe(op: str, values):
    """Evaluate one MUFU instruction per element on the current device (numpy in, numpy out)."""
    import numpy as np
    import torch

    host = np.ascontiguousarray(values, dtype=np.float32)
    if host.size == 0:
        return host.copy()
    dev_in = torch.from_numpy(host.reshape(-1)).cuda()
    dev_out = torch.empty_like(dev_in)
    check(
        lib().b2_mufu_probe(MUFU_OPS[op], _ptr(dev_in), _ptr(dev_out), dev_in.numel(),
                            current_stream_ptr()),
        "b2_mufu_probe",
    )
    return dev_out.cpu().numpy().reshape(host.shape)
