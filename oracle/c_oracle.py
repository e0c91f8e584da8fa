"""ctypes wrapper of the C restatement (TEST INFRASTRUCTURE - never on the product path).

Takes the hardware-approximate values from the same `mufu` providers as nvfp4_oracle.py and
feeds them to the C code as small tables, so full-size inputs are checked bit for bit in
seconds and the same code can be timed as the CPU baseline.
"""

from __future__ import annotations

import ctypes
import os

import numpy as np

from . import build as _build
from . import nvfp4_oracle as _np_oracle

_LIB = None
LAYOUT_CODES = {"linear": 0, "128x4": 1, "8x4": 2}


def lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        path = _build.LIBRARY if _build.LIBRARY.exists() else _build.build()
        _LIB = ctypes.CDLL(str(path))
        _LIB.oracle_sf_bytes.restype = ctypes.c_int64
        _LIB.oracle_rmsnorm_shifted_mean.restype = ctypes.c_int
    return _LIB


def _gomp():
    lib()  # the oracle library pulls the OpenMP runtime in
    return ctypes.CDLL("libgomp.so.1")


def threads() -> int:
    """Threads the next parallel region will use."""
    try:
        return int(_gomp().omp_get_max_threads())
    except OSError:
        return int(os.environ.get("OMP_NUM_THREADS", os.cpu_count() or 1))


def use_all_host_threads() -> int:
    """Undo a launcher's OMP_NUM_THREADS=1 (torchrun sets it for every rank): one thread per core this
    process may run on.  Returns the thread count now in force."""
    count = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    try:
        _gomp().omp_set_num_threads(int(count))
    except OSError:
        pass
    return threads()


def _p(array: np.ndarray):
    return array.ctypes.data_as(ctypes.c_void_p)


def _codes_f32() -> np.ndarray:
    return _np_oracle.E4M3_VALUES.copy()


def quantize_tables(global_scale, mufu):
    """(rcp(6), per-E4M3-code output scale) for nvfp4_quantize (fp_quant.py :383-401)."""
    gs = np.float32(global_scale)
    rcp6 = mufu.rcp_ftz(np.array([6.0], dtype=np.float32))[0]
    rcp_gs = mufu.rcp_ftz(np.array([gs], dtype=np.float32))[0]
    d = _codes_f32()
    with np.errstate(over="ignore", invalid="ignore"):
        prod = (d * rcp_gs).astype(np.float32)
    valid = np.isfinite(d) & (d > 0)
    table = np.zeros(256, dtype=np.float32)
    table[valid] = mufu.rcp_ftz(prod[valid])
    return np.float32(rcp6), table


def nvfp4_quantize(x_bits: np.ndarray, dtype: str, global_scale, sf_layout: str = "128x4", mufu=None):
    mufu = mufu or _np_oracle.ExactMufu()
    x_bits = np.ascontiguousarray(x_bits, dtype=np.uint16)
    m, k = x_bits.shape
    rcp6, table = quantize_tables(global_scale, mufu)
    packed = np.empty((m, k // 2), dtype=np.uint8)
    sf = np.empty(_np_oracle.sf_buffer_size(m, k // 16, sf_layout), dtype=np.uint8)
    lib().oracle_nvfp4_quantize(_p(x_bits), ctypes.c_int(dtype == _np_oracle.BF16), ctypes.c_int(m),
                                ctypes.c_int(k), ctypes.c_float(np.float32(global_scale)),
                                ctypes.c_float(rcp6), _p(table), ctypes.c_int(LAYOUT_CODES[sf_layout]),
                                _p(packed), _p(sf))
    return packed, sf


def rmsnorm_fp4quant(x_bits, w_bits, dtype: str, global_scale, eps: float, swizzled: bool = False,
                     mufu=None, sf_fill: int = 0):
    """Block 16 / E4M3 only (the NVFP4 path); other variants live in nvfp4_oracle.py."""
    mufu = mufu or _np_oracle.ExactMufu()
    x_bits = np.ascontiguousarray(x_bits, dtype=np.uint16)
    w_bits = np.ascontiguousarray(w_bits, dtype=np.uint16)
    M, H = x_bits.shape
    is_bf16 = ctypes.c_int(dtype == _np_oracle.BF16)
    shifted = np.empty(M, dtype=np.float32)
    if lib().oracle_rmsnorm_shifted_mean(_p(x_bits), is_bf16, ctypes.c_int(M), ctypes.c_int(H),
                                         ctypes.c_float(np.float32(eps)), _p(shifted)) != 0:
        raise ValueError(f"H={H} needs the cluster reduction tree, which only nvfp4_oracle.py restates")
    rstd = np.ascontiguousarray(mufu.rsqrt_ftz(shifted), dtype=np.float32)
    rcp6 = mufu.rcp_ftz(np.array([6.0], dtype=np.float32))[0]
    d = _codes_f32()
    valid = np.isfinite(d) & (d > 0)
    table = np.zeros(256, dtype=np.float32)
    table[valid] = mufu.rcp_ftz(d[valid])
    y = np.empty((M, H // 2), dtype=np.uint8)
    nblk = H // 16
    size = (-(-M // 128) * 128 * _np_oracle.padded_sf_cols(nblk)) if swizzled else M * nblk
    sf = np.full(size, sf_fill, dtype=np.uint8)
    lib().oracle_rmsnorm_quant(_p(x_bits), _p(w_bits), is_bf16, ctypes.c_int(M), ctypes.c_int(H), _p(rstd),
                               ctypes.c_float(np.float32(global_scale)), ctypes.c_float(np.float32(rcp6)),
                               _p(table), ctypes.c_int(bool(swizzled)), _p(y), _p(sf))
    return y, (sf if swizzled else sf.reshape(M, nblk))


def dequantize_nvfp4(packed, sf, layout: str, global_scale=1.0) -> np.ndarray:
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    sf = np.ascontiguousarray(sf, dtype=np.uint8)
    m, half = packed.shape
    out = np.empty((m, half * 2), dtype=np.float32)
    lib().oracle_dequantize_nvfp4(_p(packed), _p(sf), ctypes.c_int(m), ctypes.c_int(half * 2),
                                  ctypes.c_int(LAYOUT_CODES[layout]), ctypes.c_float(np.float32(global_scale)),
                                  _p(out))
    return out
