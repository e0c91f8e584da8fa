"""CPU oracle for the NVFP4 hot path (TEST INFRASTRUCTURE - never on the product path).

A vectorised numpy restatement of the arithmetic the mlc-ai/TIRx-kernels reference
performs on the GPU for three registry entries.  Every function cites the reference
file:line it follows.  Only tests/, the smoke check and the benchmark's CPU-baseline
leg may import this module; the shipped package never does.

Pinning status.  The reference holds no golden vectors for this path: its own tests
compare against a third-party GPU kernel (flashinfer, pinned at git f2e04400,
reference-dependencies.json:31-36) at test time.  This oracle is therefore pinned
against (a) fixtures under tests/golden/ produced by running the flashinfer build
that ships in this image on a B200 (tests/golden/make_flashinfer_golden.py), when those
exist, and (b) the self-contained checks the reference carries (dequantise-vs-fp32
tolerances, zero-scale invariants, torch's float8_e4m3fn cast).  Where neither applies,
parity is unpinned and the tests say so.

Hardware-approximate instructions.  rcp.approx.ftz, rsqrt.approx.ftz, lg2.approx and
ex2.approx are not specified bit for bit, so they enter through a `mufu` provider:
`ExactMufu` rounds the true value correctly (usable without a GPU), `ProbeMufu`
evaluates the single instruction on the device through b2_mufu_probe and nothing else.
"""

from __future__ import annotations

import numpy as np

F16 = "float16"
BF16 = "bfloat16"
E2M1_VALUES = np.array(
    [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0],
    dtype=np.float32,
)
_F32_TINY = np.float32(2.0**-126)


# --------------------------------------------------------------------------------------
# MUFU providers
# --------------------------------------------------------------------------------------
def _ftz(x: np.ndarray) -> np.ndarray:
    x = np.asarray(x, dtype=np.float32)
    return np.where(np.abs(x) < _F32_TINY, np.copysign(np.float32(0.0), x), x).astype(np.float32)


class ExactMufu:
    """Correctly rounded stand-ins (with the .ftz behaviour where the instruction has it)."""

    name = "exact"

    def rcp_ftz(self, x):
        with np.errstate(divide="ignore", over="ignore", invalid="ignore"):
            return _ftz(np.float32(1.0) / _ftz(x))

    def rsqrt_ftz(self, x):
        with np.errstate(divide="ignore", invalid="ignore"):
            r = 1.0 / np.sqrt(_ftz(x).astype(np.float64))
        return _ftz(r.astype(np.float32))

    def lg2(self, x):
        with np.errstate(divide="ignore", invalid="ignore"):
            return np.log2(np.asarray(x, dtype=np.float32).astype(np.float64)).astype(np.float32)

    def ex2(self, x):
        with np.errstate(over="ignore", under="ignore"):
            return np.exp2(np.asarray(x, dtype=np.float32).astype(np.float64)).astype(np.float32)

    def ex2_ftz(self, x):
        with np.errstate(over="ignore", under="ignore"):
            return _ftz(np.exp2(_ftz(x).astype(np.float64)).astype(np.float32))


class ProbeMufu:
    """Takes each approximate instruction's value from the hardware.

    `probe(op_name, float32 array) -> float32 array` evaluates exactly one instruction per
    element (ops: "rcp_ftz", "rsqrt_ftz", "lg2", "ex2", "ex2_ftz").
    """

    name = "probe"

    def __init__(self, probe):
        self._probe = probe

    def _run(self, op, x):
        x = np.ascontiguousarray(x, dtype=np.float32)
        flat = x.reshape(-1)
        uniq, inverse = np.unique(flat.view(np.uint32), return_inverse=True)
        out = np.asarray(self._probe(op, uniq.view(np.float32)), dtype=np.float32)
        return out[inverse].reshape(x.shape)

    def rcp_ftz(self, x):
        return self._run("rcp_ftz", x)

    def rsqrt_ftz(self, x):
        return self._run("rsqrt_ftz", x)

    def lg2(self, x):
        return self._run("lg2", x)

    def ex2(self, x):
        return self._run("ex2", x)

    def ex2_ftz(self, x):
        return self._run("ex2_ftz", x)


# --------------------------------------------------------------------------------------
# 16-bit input types
# --------------------------------------------------------------------------------------
def bits_to_f32(bits: np.ndarray, dtype: str) -> np.ndarray:
    """uint16 storage -> exact float32 value (fp_quant.py unpack_lo/hi_f32 :78-97)."""
    bits = np.asarray(bits, dtype=np.uint16)
    if dtype == BF16:
        return (bits.astype(np.uint32) << np.uint32(16)).view(np.float32)
    return bits.view(np.float16).astype(np.float32)


def _round_f64_to_16bit(v: np.ndarray, dtype: str) -> np.ndarray:
    """Round-to-nearest-even of exact float64 values to bf16/fp16, returned as float32."""
    v = np.asarray(v, dtype=np.float64)
    mant_bits, min_quantum_exp, max_finite = (7, -133, None) if dtype == BF16 else (10, -24, 65504.0)
    _, e = np.frexp(v)  # |v| = m * 2**e with m in [0.5, 1)
    qexp = np.maximum(e - 1 - mant_bits, min_quantum_exp)
    with np.errstate(over="ignore", invalid="ignore"):
        q = np.ldexp(np.rint(np.ldexp(v, -qexp)), qexp)
    q = np.where(np.isfinite(v), q, v)
    if max_finite is not None:
        q = np.where(np.abs(q) > max_finite, np.copysign(np.inf, q), q)
    with np.errstate(over="ignore"):
        return q.astype(np.float32)  # bf16 overflow (>= 2**128) becomes inf here


def f32_to_bits(v: np.ndarray, dtype: str) -> np.ndarray:
    """float32 -> uint16 storage with cvt.rn semantics (fp_quant.py cvt_f32x2_to_packed :347-360)."""
    v = np.asarray(v, dtype=np.float32)
    if dtype == F16:
        with np.errstate(over="ignore"):
            return v.astype(np.float16).view(np.uint16)
    r = _round_f64_to_16bit(v.astype(np.float64), BF16)
    bits = (r.view(np.uint32) >> np.uint32(16)).astype(np.uint16)
    return np.where(np.isnan(v), np.uint16(0x7FFF), bits)


def mul_16bit(a_bits: np.ndarray, b_bits: np.ndarray, dtype: str) -> np.ndarray:
    """mul.bf16x2 / mul.f16x2 lane: exact product, one rounding to the 16-bit type.

    Returns the product as float32 (exactly representable).  rmsnorm_fp4quant.py
    _multiply_8_pairs :203-208.
    """
    prod = bits_to_f32(a_bits, dtype).astype(np.float64) * bits_to_f32(b_bits, dtype).astype(np.float64)
    return _round_f64_to_16bit(prod, dtype)


# --------------------------------------------------------------------------------------
# E4M3 / E2M1 conversions
# --------------------------------------------------------------------------------------
def _e4m3_table() -> np.ndarray:
    codes = np.arange(256, dtype=np.uint32)
    sign = np.where(codes & 0x80, -1.0, 1.0)
    exp = (codes >> 3) & 0xF
    man = codes & 0x7
    val = np.where(exp == 0, man / 8.0 * 2.0**-6, (1.0 + man / 8.0) * 2.0 ** (exp.astype(np.float64) - 7))
    val = np.where((codes & 0x7F) == 0x7F, np.nan, val)
    return (sign * val).astype(np.float32)


E4M3_VALUES = _e4m3_table()


def e4m3_decode(codes: np.ndarray) -> np.ndarray:
    """cvt.rn.f16x2.e4m3x2 then cvt.f32.f16: exact (fp_quant.py :387-394)."""
    return E4M3_VALUES[np.asarray(codes, dtype=np.uint8)]


def e4m3_encode(v: np.ndarray) -> np.ndarray:
    """cvt.rn.satfinite.e4m3x2.f32 on one lane: RNE, |v| > 448 -> 448, NaN -> 0x7F
    (fp_quant.py cvt_f32_to_e4m3 :375-380)."""
    v = np.asarray(v, dtype=np.float32)
    a = np.abs(v).astype(np.float64)
    _, e = np.frexp(a)
    qexp = np.maximum(e - 1 - 3, -9)  # 3 mantissa bits; subnormal quantum 2**-9
    with np.errstate(over="ignore", invalid="ignore"):
        q = np.ldexp(np.rint(np.ldexp(a, -qexp)), qexp)
    q = np.where(np.isnan(a), 0.0, np.minimum(q, 448.0))
    # encode the (exactly representable) magnitude
    _, e2 = np.frexp(q)
    exp_field = np.clip(e2 - 1 + 7, 0, 15)
    normal = q >= 2.0**-6
    man_norm = np.rint(np.ldexp(q, -(e2 - 1)) * 8.0 - 8.0)
    man_sub = np.rint(q * 2.0**9)
    code = np.where(normal, exp_field * 8 + man_norm, man_sub).astype(np.int64)
    code = np.where(np.isnan(v), 0x7F, code)
    sign = np.where(np.signbit(v) & ~np.isnan(v), 0x80, 0)
    return (code | sign).astype(np.uint8)


def e2m1_encode(v: np.ndarray) -> np.ndarray:
    """cvt.rn.satfinite.e2m1x2.f32 on one lane -> 4-bit code (fp_quant.py cvt_e2m1x8 :291-306).

    Grid {0,.5,1,1.5,2,3,4,6}; ties go to the code with an even mantissa bit; |v| > 6 -> 6;
    the sign bit is kept (-0 -> 0x8); NaN -> +6 (the type has no NaN).
    """
    v = np.asarray(v, dtype=np.float32)
    a = np.abs(v)
    code = (
        (a > 0.25).astype(np.uint8)
        + (a >= 0.75)
        + (a > 1.25)
        + (a >= 1.75)
        + (a > 2.5)
        + (a >= 3.5)
        + (a > 5.0)
    ).astype(np.uint8)
    code = np.where(np.isnan(v), np.uint8(7), code)
    sign = np.where(np.signbit(v) & ~np.isnan(v), np.uint8(8), np.uint8(0))
    return (code | sign).astype(np.uint8)


def pack_nibbles(codes: np.ndarray) -> np.ndarray:
    """[..., 2n] 4-bit codes -> [..., n] bytes, even element in the low nibble."""
    codes = np.asarray(codes, dtype=np.uint8)
    return (codes[..., 0::2] | (codes[..., 1::2] << np.uint8(4))).astype(np.uint8)


# --------------------------------------------------------------------------------------
# scale-factor layouts (fp_quant.py sf_offset_128x4 :250-258, sf_offset_8x4 :261-269)
# --------------------------------------------------------------------------------------
def padded_sf_cols(cols: int) -> int:
    return (cols + 3) // 4 * 4


def sf_offsets(layout: str, rows: np.ndarray, cols: np.ndarray, padded_cols: int) -> np.ndarray:
    rows = np.asarray(rows, dtype=np.int64)
    cols = np.asarray(cols, dtype=np.int64)
    if layout == "linear":
        return rows * padded_cols + cols
    if layout == "128x4":
        return (
            cols % 4
            + (cols // 4) * 512
            + (rows % 32) * 16
            + ((rows % 128) // 32) * 4
            + (rows // 128) * (128 * padded_cols)
        )
    if layout == "8x4":
        k_tiles = (padded_cols + 3) // 4
        return (rows // 8) * (k_tiles * 32) + (cols // 4) * 32 + (rows % 8) * 4 + cols % 4
    raise ValueError(f"unknown sf layout {layout!r}")


def sf_buffer_size(m: int, sf_cols: int, layout: str) -> int:
    """nvfp4_quantize.py _sf_numel :126-129."""
    if layout == "linear":
        return m * sf_cols
    tile = 8 if layout == "8x4" else 128
    return (m + tile - 1) // tile * tile * padded_sf_cols(sf_cols)


# --------------------------------------------------------------------------------------
# nvfp4_quantize  (tirx_kernels/flashinfer/quantization/nvfp4_quantize.py)
# --------------------------------------------------------------------------------------
def silu_f32(g: np.ndarray, mufu) -> np.ndarray:
    """fp_quant.py silu_f32 :340-344: mul.f32 by -log2(e), ex2.approx.ftz.f32, add.f32 of 1.0, div.rn.f32."""
    g = np.asarray(g, dtype=np.float32)
    e = mufu.ex2_ftz(g * np.float32(-1.4426950408889634))
    with np.errstate(over="ignore", invalid="ignore", divide="ignore"):
        return (g / (e + np.float32(1.0))).astype(np.float32)


def silu_and_mul(gate_bits, up_bits, dtype: str, mufu) -> np.ndarray:
    """fp_quant.py silu_and_mul_pair :363-372; returns uint16 storage."""
    u = bits_to_f32(up_bits, dtype)
    s = silu_f32(bits_to_f32(gate_bits, dtype), mufu)
    with np.errstate(over="ignore", invalid="ignore"):
        return f32_to_bits((s * u).astype(np.float32), dtype)


def nvfp4_quantize(x_bits, dtype: str, global_scale, sf_layout: str = "128x4", fuse_silu: bool = False,
                   mufu=None):
    """Block quantizer: _process_block :152-183; SF placement and zero fill :237-247, :279-364.

    x_bits: uint16 [m, k] (or [m, 2k] = [gate | up] with fuse_silu).  Returns
    (packed uint8 [m, k/2], sf uint8 [sf_buffer_size]).
    """
    mufu = mufu or ExactMufu()
    x_bits = np.asarray(x_bits, dtype=np.uint16)
    m, in_cols = x_bits.shape
    k = in_cols // 2 if fuse_silu else in_cols
    if k <= 0 or k % 16:
        raise ValueError(f"k={k} outside the source dispatch domain (k % 16 != 0)")
    if fuse_silu:
        x_bits = silu_and_mul(x_bits[:, :k], x_bits[:, k:], dtype, mufu)
    gs = np.float32(global_scale)
    x = bits_to_f32(x_bits, dtype)
    nsb = k // 16
    blocks = x.reshape(m, nsb, 16)
    with np.errstate(invalid="ignore"):
        amax = np.fmax.reduce(np.abs(blocks), axis=-1).astype(np.float32)  # max.* drop NaNs
    rcp6 = mufu.rcp_ftz(np.array([6.0], dtype=np.float32))[0]
    with np.errstate(over="ignore", invalid="ignore"):
        scale = (gs * (amax * rcp6).astype(np.float32)).astype(np.float32)
    sf_code = e4m3_encode(scale)
    sf_f32 = e4m3_decode(sf_code)
    rcp_gs = mufu.rcp_ftz(np.array([gs], dtype=np.float32))[0]
    with np.errstate(over="ignore", invalid="ignore"):
        prod = (sf_f32 * rcp_gs).astype(np.float32)
    inv = mufu.rcp_ftz(prod)
    out_scale = np.where(sf_f32 == 0.0, np.float32(0.0), inv).astype(np.float32)
    with np.errstate(over="ignore", invalid="ignore"):
        scaled = (blocks * out_scale[..., None]).astype(np.float32)
    packed = pack_nibbles(e2m1_encode(scaled).reshape(m, k))

    if sf_layout == "linear":
        return packed, sf_code.reshape(-1).copy()
    pad_cols = padded_sf_cols(nsb)
    sf = np.zeros(sf_buffer_size(m, nsb, sf_layout), dtype=np.uint8)
    rows = np.arange(m)[:, None]
    cols = np.arange(nsb)[None, :]
    sf[sf_offsets(sf_layout, rows, cols, pad_cols)] = sf_code
    return packed, sf


FLOAT32_MAX = np.float32(3.4028234663852886e38)


def nvfp4_quantize_per_token(x_bits, dtype: str, gs_inv, sf_layout: str = "128x4", mufu=None):
    """tirx_kernels/flashinfer/quantization/nvfp4_quantize_per_token.py: row scales :195-211, block
    recipe _process_block_pt :56-74 (nvfp4_compute_output_scale, fp_quant_kern.py:377-394), SF
    placement and column padding :216-229; padding rows are zero (host-initialised buffer, :262-264).

    Returns (packed uint8 [m, k/2], sf uint8 [sf_buffer_size], token_scale float32 [m]).

    PARITY UNPINNED: the reference takes its expected bytes from flashinfer's CuTe-DSL per-token
    kernel, which the flashinfer build available here (0.6.11) does not contain; that build's CUDA
    per-token path is a different implementation and agrees with this restatement on > 99.5 % of the
    bytes (tests/test_golden_cpu.py bounds the distance).  The block recipe itself is the pinned
    one of nvfp4_quantize with the row's encode scale in place of the global scale.
    """
    mufu = mufu or ExactMufu()
    x_bits = np.asarray(x_bits, dtype=np.uint16)
    m, k = x_bits.shape
    if k <= 0 or k % 16:
        raise ValueError(f"k={k} outside the source dispatch domain (k % 16 != 0)")
    x = bits_to_f32(x_bits, dtype)
    nsb = k // 16
    blocks = x.reshape(m, nsb, 16)
    with np.errstate(invalid="ignore"):
        amax = np.fmax.reduce(np.abs(blocks), axis=-1).astype(np.float32)
        row_amax = np.fmax.reduce(amax, axis=-1).astype(np.float32)
    zero = row_amax == 0.0
    with np.errstate(over="ignore", invalid="ignore"):
        token = np.where(zero, np.float32(0.0), (row_amax * np.float32(gs_inv)).astype(np.float32)).astype(np.float32)
    encode = np.where(zero, FLOAT32_MAX, mufu.rcp_ftz(np.where(zero, np.float32(1.0), token))).astype(np.float32)
    rcp6 = mufu.rcp_ftz(np.array([6.0], dtype=np.float32))[0]
    with np.errstate(over="ignore", invalid="ignore"):
        scale = (encode[:, None] * (amax * rcp6).astype(np.float32)).astype(np.float32)
    sf_code = e4m3_encode(scale)
    sf_f32 = e4m3_decode(sf_code)
    rcp_enc = mufu.rcp_ftz(encode)
    with np.errstate(over="ignore", invalid="ignore"):
        prod = (sf_f32 * rcp_enc[:, None]).astype(np.float32)
    inv = mufu.rcp_ftz(prod)
    out_scale = np.where(sf_f32 == 0.0, np.float32(0.0), inv).astype(np.float32)
    with np.errstate(over="ignore", invalid="ignore"):
        scaled = (blocks * out_scale[..., None]).astype(np.float32)
    packed = pack_nibbles(e2m1_encode(scaled).reshape(m, k))
    if sf_layout == "linear":
        return packed, sf_code.reshape(-1).copy(), token
    pad_cols = padded_sf_cols(nsb)
    sf = np.zeros(sf_buffer_size(m, nsb, sf_layout), dtype=np.uint8)
    sf[sf_offsets(sf_layout, np.arange(m)[:, None], np.arange(nsb)[None, :], pad_cols)] = sf_code
    return packed, sf, token


# --------------------------------------------------------------------------------------
# flashinfer_rmsnorm_fp4quant  (tirx_kernels/flashinfer/norm/rmsnorm_fp4quant.py)
# --------------------------------------------------------------------------------------
def threads_per_row(h_per_cta: int) -> int:
    """_threads_per_row :344-355."""
    for limit, tpr in ((64, 8), (128, 16), (3072, 32), (6144, 64), (16384, 128)):
        if h_per_cta <= limit:
            return tpr
    return 256


def source_config(H: int) -> dict:
    """_derived_config / _estimate_smem / _source_config :358-400."""

    def derived(cluster_n):
        hpc = H // cluster_n
        tpr = threads_per_row(hpc)
        threads = 128 if hpc <= 16384 else 256
        rows = threads // tpr
        wpr = max(tpr // 32, 1)
        vb = max(1, -(-(hpc // 8) // tpr))
        cols = 8 * vb * tpr
        return dict(tpr=tpr, threads=threads, rows=rows, warps_per_row=wpr, vec_blocks=vb, cols=cols,
                    tile_bytes=rows * cols * 2)

    cluster_n = 16
    for cand in (1, 2, 4, 8, 16):
        c = derived(cand)
        red = c["rows"] * c["warps_per_row"] * 4
        est = 2 * c["tile_bytes"] + red if cand == 1 else c["tile_bytes"] + red * cand + 8
        if H % cand == 0 and est <= 232448:
            cluster_n = cand
            break
    cfg = derived(cluster_n)
    cfg["cluster_n"] = cluster_n
    return cfg


def _butterfly(v: np.ndarray, xors) -> np.ndarray:
    """XOR butterfly over the last axis (lanes), fp32 adds: _butterfly_sum_f32 :101-104."""
    lanes = np.arange(v.shape[-1])
    for x in xors:
        v = (v + v[..., lanes ^ x]).astype(np.float32)
    return v


def rmsnorm_sum_of_squares(x_bits, dtype: str) -> np.ndarray:
    """The reference's fp32 reduction tree, kernel_body :786-893; returns [M] float32."""
    x = bits_to_f32(x_bits, dtype)
    return sum_of_squares_tree(x, source_config(x.shape[1]))


def sum_of_squares_tree(x: np.ndarray, cfg: dict) -> np.ndarray:
    """Sum of x*x over the rows of fp32 `x` [M, H] in the order a launch configuration fixes."""
    M, H = x.shape
    tpr, vb, cols, cn = cfg["tpr"], cfg["vec_blocks"], cfg["cols"], cfg["cluster_n"]
    wpr = cfg["warps_per_row"]
    padded = np.zeros((M, cn * cols), dtype=np.float32)
    padded[:, :H] = x  # CTA c of a cluster owns columns [c*cols, (c+1)*cols) (:787-789)
    sq = (padded * padded).astype(np.float32).reshape(M, cn, vb, tpr, 8)
    local = np.zeros((M, cn, tpr), dtype=np.float32)
    for b in range(vb):  # b-major, element order (:832-834)
        for i in range(8):
            local = (local + sq[:, :, b, :, i]).astype(np.float32)
    row_xors = [s for s in (1, 2, 4, 8, 16) if s < min(tpr, 32)]
    if tpr <= 32:
        assert cn == 1
        return _butterfly(local[:, 0, :], row_xors)[:, 0]
    warp = _butterfly(local.reshape(M, cn, wpr, 32), row_xors)[..., 0]  # [M, cn, wpr]
    full = (1, 2, 4, 8, 16)
    if cn == 1:  # :839-856
        lanes = np.zeros((M, 32), dtype=np.float32)
        lanes[:, :wpr] = warp[:, 0, :]
        return _butterfly(lanes, full)[:, 0]
    # cluster path :857-891: partial index = cta * wpr + warp; lane sums partials lane, lane+32, ...
    partials = warp.reshape(M, cn * wpr)
    total = cn * wpr
    lanes = np.zeros((M, 32), dtype=np.float32)
    for it in range(-(-total // 32)):
        idx = np.arange(32) + it * 32
        ok = idx < total
        add = np.zeros((M, 32), dtype=np.float32)
        add[:, ok] = partials[:, idx[ok]]
        lanes = np.where(ok[None, :], (lanes + add).astype(np.float32), lanes)
    return _butterfly(lanes, full)[:, 0]


def rmsnorm_shifted_mean(sum_sq: np.ndarray, H: int, eps: float) -> np.ndarray:
    """mean + eps, :895-899: one fma for power-of-two H, div.rn then add otherwise."""
    eps32 = np.float32(eps)
    if H & (H - 1) == 0:
        wide = sum_sq.astype(np.longdouble) * np.longdouble(np.float32(1.0 / H)) + np.longdouble(eps32)
        return wide.astype(np.float32)
    return ((sum_sq / np.float32(H)).astype(np.float32) + eps32).astype(np.float32)


def rmsnorm_fp4quant(x_bits, w_bits, dtype: str, global_scale, eps: float, block_size: int = 16,
                     scale_format: str = "e4m3", swizzled: bool = False, mufu=None, sf_fill: int = 0):
    """kernel_body :745-980 with _process_scale_block :266-337.

    Returns (packed uint8 [M, H/2], sf uint8 buffer).  Positions of a swizzled buffer that the
    kernel never writes keep `sf_fill` (the reference leaves them untouched).
    """
    mufu = mufu or ExactMufu()
    x_bits = np.asarray(x_bits, dtype=np.uint16)
    w_bits = np.asarray(w_bits, dtype=np.uint16)
    M, H = x_bits.shape
    use_e4m3 = block_size == 16 or scale_format == "e4m3"
    sum_sq = rmsnorm_sum_of_squares(x_bits, dtype)
    rstd = mufu.rsqrt_ftz(rmsnorm_shifted_mean(sum_sq, H, eps))[:, None, None]
    nblk = H // block_size
    prod = mul_16bit(x_bits, w_bits[None, :], dtype).reshape(M, nblk, block_size)
    with np.errstate(invalid="ignore"):
        max_xw = np.fmax.reduce(np.abs(prod), axis=-1).astype(np.float32)[..., None]
    with np.errstate(over="ignore", invalid="ignore"):
        values = (prod * rstd).astype(np.float32)
        max_abs = (max_xw * rstd).astype(np.float32)
    rcp6 = mufu.rcp_ftz(np.array([6.0], dtype=np.float32))[0]
    if use_e4m3:
        gs = np.float32(global_scale)
        with np.errstate(over="ignore", invalid="ignore"):
            s = ((gs * max_abs).astype(np.float32) * rcp6).astype(np.float32)
        s = np.fmin(s, np.float32(448.0))  # min.f32: a NaN operand yields the other one
        code = e4m3_encode(s)
        d = e4m3_decode(code)
        r = np.where(d == 0.0, np.float32(0.0), mufu.rcp_ftz(d)).astype(np.float32)
        with np.errstate(over="ignore", invalid="ignore"):
            out_scale = (r * gs).astype(np.float32)
    else:  # UE8M0: _cvt_f32_to_ue8m0 :155-171, _ue8m0_to_output_scale :174-185
        with np.errstate(over="ignore", invalid="ignore"):
            v = (max_abs * rcp6).astype(np.float32)
        lg = mufu.lg2(np.where(v > 0, v, np.float32(1.0)))
        e = np.ceil(lg.astype(np.float64)).astype(np.int64) + 127
        code = np.where(v <= 0, 0, np.clip(e, 0, 255)).astype(np.uint8)
        cand = mufu.ex2((127 - code.astype(np.int32)).astype(np.float32))
        out_scale = np.where(code == 0, np.float32(0.0), cand).astype(np.float32)
    with np.errstate(over="ignore", invalid="ignore"):
        scaled = (values * out_scale).astype(np.float32)
    packed = pack_nibbles(e2m1_encode(scaled).reshape(M, H))
    code = code.reshape(M, nblk)
    if not swizzled:
        return packed, code.copy()
    pad_cols = padded_sf_cols(nblk)
    sf = np.full(-(-M // 128) * 128 * pad_cols, sf_fill, dtype=np.uint8)
    sf[sf_offsets("128x4", np.arange(M)[:, None], np.arange(nblk)[None, :], pad_cols)] = code
    return packed, sf


# --------------------------------------------------------------------------------------
# flashinfer_add_rmsnorm_fp4quant  (tirx_kernels/flashinfer/norm/add_rmsnorm_fp4quant.py)
# --------------------------------------------------------------------------------------
def add_source_config(H: int) -> dict:
    """_derived_config / _estimate_smem / _source_config :325-363: as `source_config`, but the
    one-CTA form keeps four row tiles (x, residual, weight, h) and the cluster form two."""

    def derived(cluster_n):
        hpc = H // cluster_n
        tpr = threads_per_row(hpc)
        threads = 128 if hpc <= 16384 else 256
        rows = threads // tpr
        wpr = max(tpr // 32, 1)
        vb = max(1, -(-(hpc // 8) // tpr))
        cols = 8 * vb * tpr
        return dict(tpr=tpr, threads=threads, rows=rows, warps_per_row=wpr, vec_blocks=vb, cols=cols,
                    tile_bytes=rows * cols * 2)

    cluster_n = 16
    for cand in (1, 2, 4, 8, 16):
        c = derived(cand)
        red = c["rows"] * c["warps_per_row"] * 4
        est = 4 * c["tile_bytes"] + red if cand == 1 else 2 * c["tile_bytes"] + red * cand + 8
        if H % cand == 0 and est <= 232448:
            cluster_n = cand
            break
    cfg = derived(cluster_n)
    cfg["cluster_n"] = cluster_n
    return cfg


def add_rmsnorm_fp4quant(x_bits, r_bits, w_bits, dtype: str, global_scale, eps: float, block_size: int = 16,
                         scale_format: str = "e4m3", swizzled: bool = False, mufu=None, sf_fill: int = 0):
    """kernel_body :825-1206 with _process_add_scale_block :156-314.

    h = x + residual in fp32 (add.f32x2 :951-958); the squares of the UNROUNDED sums are added in the
    usual tree order (:960-983); h rounded to the input dtype replaces the residual (:1052-1071).
    One CTA per row (:177-229): value = (h * rstd) * w in fp32 on the rounded h, block maximum of
    |value| in fp32.  Cluster rows (:230-258): the rmsnorm_fp4quant recipe on the rounded h
    (16-bit product h*w, maximum times rstd).  Scale and output scale as in rmsnorm_fp4quant.

    Returns dict(y, scale (linear [M, nblk] codes), scale_buffer (layout of `swizzled`), y_norm bits
    (the values before the output scale, rounded to the input dtype :134-153), residual bits).
    """
    mufu = mufu or ExactMufu()
    x_bits = np.asarray(x_bits, dtype=np.uint16)
    r_bits = np.asarray(r_bits, dtype=np.uint16)
    w_bits = np.asarray(w_bits, dtype=np.uint16)
    M, H = x_bits.shape
    use_e4m3 = block_size == 16 or scale_format == "e4m3"
    cfg = add_source_config(H)
    with np.errstate(over="ignore", invalid="ignore"):
        h32 = (bits_to_f32(x_bits, dtype) + bits_to_f32(r_bits, dtype)).astype(np.float32)
    h_bits = f32_to_bits(h32, dtype)
    sum_sq = sum_of_squares_tree(h32, cfg)
    rstd = mufu.rsqrt_ftz(rmsnorm_shifted_mean(sum_sq, H, eps))[:, None, None]
    nblk = H // block_size
    if cfg["cluster_n"] == 1:
        h = bits_to_f32(h_bits, dtype).reshape(M, nblk, block_size)
        w = bits_to_f32(w_bits, dtype).reshape(1, nblk, block_size)
        with np.errstate(over="ignore", invalid="ignore"):
            values = ((h * rstd).astype(np.float32) * w).astype(np.float32)
            max_abs = np.fmax.reduce(np.abs(values), axis=-1).astype(np.float32)[..., None]
    else:
        prod = mul_16bit(h_bits, w_bits[None, :], dtype).reshape(M, nblk, block_size)
        with np.errstate(over="ignore", invalid="ignore"):
            max_xw = np.fmax.reduce(np.abs(prod), axis=-1).astype(np.float32)[..., None]
            values = (prod * rstd).astype(np.float32)
            max_abs = (max_xw * rstd).astype(np.float32)
    rcp6 = mufu.rcp_ftz(np.array([6.0], dtype=np.float32))[0]
    if use_e4m3:
        gs = np.float32(global_scale)
        with np.errstate(over="ignore", invalid="ignore"):
            sc = ((gs * max_abs).astype(np.float32) * rcp6).astype(np.float32)
        sc = np.fmin(sc, np.float32(448.0))
        code = e4m3_encode(sc)
        d = e4m3_decode(code)
        r = np.where(d == 0.0, np.float32(0.0), mufu.rcp_ftz(d)).astype(np.float32)
        with np.errstate(over="ignore", invalid="ignore"):
            out_scale = (r * gs).astype(np.float32)
    else:
        with np.errstate(over="ignore", invalid="ignore"):
            v = (max_abs * rcp6).astype(np.float32)
        lg = mufu.lg2(np.where(v > 0, v, np.float32(1.0)))
        e = np.ceil(lg.astype(np.float64)).astype(np.int64) + 127
        code = np.where(v <= 0, 0, np.clip(e, 0, 255)).astype(np.uint8)
        cand = mufu.ex2((127 - code.astype(np.int32)).astype(np.float32))
        out_scale = np.where(code == 0, np.float32(0.0), cand).astype(np.float32)
    with np.errstate(over="ignore", invalid="ignore"):
        scaled = (values * out_scale).astype(np.float32)
    packed = pack_nibbles(e2m1_encode(scaled).reshape(M, H))
    code = code.reshape(M, nblk)
    if swizzled:
        pad_cols = padded_sf_cols(nblk)
        buf = np.full(-(-M // 128) * 128 * pad_cols, sf_fill, dtype=np.uint8)
        buf[sf_offsets("128x4", np.arange(M)[:, None], np.arange(nblk)[None, :], pad_cols)] = code
    else:
        buf = code.copy()
    return {"y": packed, "scale": code.copy(), "scale_buffer": buf,
            "y_norm": f32_to_bits(values.reshape(M, H), dtype), "residual": h_bits}


# --------------------------------------------------------------------------------------
# decoding and the GEMM oracle
# --------------------------------------------------------------------------------------
def unpack_e2m1(packed: np.ndarray) -> np.ndarray:
    """uint8 [m, k/2] -> float32 [m, k]; low nibble first (rmsnorm_fp4quant.py _dequantize :1277-1290)."""
    packed = np.asarray(packed, dtype=np.uint8)
    m = packed.shape[0]
    nib = np.stack((packed & 0xF, packed >> 4), axis=-1).reshape(m, -1)
    return E2M1_VALUES[nib]


def logical_scales(sf: np.ndarray, m: int, sf_cols: int, layout: str) -> np.ndarray:
    """Gathers the [m, sf_cols] scale bytes out of a layout (_logical_scale_bytes :1258-1274)."""
    pad = sf_cols if layout == "linear" else padded_sf_cols(sf_cols)
    off = sf_offsets(layout, np.arange(m)[:, None], np.arange(sf_cols)[None, :], pad)
    return np.asarray(sf, dtype=np.uint8).reshape(-1)[off]


def dequantize_nvfp4(packed, sf, layout: str, global_scale=1.0, block_size: int = 16) -> np.ndarray:
    """value = e2m1 * e4m3 / global_scale (_dequantize :1291-1297)."""
    vals = unpack_e2m1(packed)
    m, k = vals.shape
    scales = e4m3_decode(logical_scales(sf, m, k // block_size, layout)) / np.float32(global_scale)
    return (vals.reshape(m, -1, block_size) * scales[..., None]).reshape(m, k).astype(np.float32)


def dequantize_mxfp4(packed, sf, layout: str, block_size: int = 32) -> np.ndarray:
    vals = unpack_e2m1(packed)
    m, k = vals.shape
    scales = np.exp2(logical_scales(sf, m, k // block_size, layout).astype(np.float32) - 127.0)
    return (vals.reshape(m, -1, block_size) * scales[..., None]).reshape(m, k).astype(np.float32)


def dequantize_nvfp4_rows(packed, sf, rows, block_size: int = 16) -> np.ndarray:
    """Rows `rows` of dequantize_nvfp4(packed, sf, "128x4"): only those rows are decoded."""
    rows = np.asarray(rows, dtype=np.int64)
    vals = unpack_e2m1(np.asarray(packed, dtype=np.uint8)[rows])
    k = vals.shape[1]
    sf_cols = k // block_size
    off = sf_offsets("128x4", rows[:, None], np.arange(sf_cols)[None, :], padded_sf_cols(sf_cols))
    scales = e4m3_decode(np.asarray(sf, dtype=np.uint8).reshape(-1)[off])
    return (vals.reshape(len(rows), -1, block_size) * scales[..., None]).reshape(len(rows), k).astype(np.float32)


def nvfp4_gemm(a_packed, b_packed, a_sf, b_sf, alpha, rows=None) -> np.ndarray:
    """D = bf16(alpha * A_deq @ B_deq^T) with fp32 accumulation; returns bf16 storage (uint16).

    Semantics of tirx_kernels/basic/nvfp4_gemm.py: block-scaled operands :694-719, alpha then
    bf16 in the epilogue :795-800; data contract prepare_data :47-66.  With `rows` (indices into
    A) only those output rows are computed, which keeps problems of 8192^3 and beyond within
    seconds of CPU time while every sampled row is still a full-length dot product.
    """
    import torch

    if rows is None:
        a = torch.from_numpy(dequantize_nvfp4(a_packed, a_sf, "128x4"))
    else:
        a = torch.from_numpy(dequantize_nvfp4_rows(a_packed, a_sf, rows))
    b = torch.from_numpy(dequantize_nvfp4(b_packed, b_sf, "128x4"))
    d = torch.mm(a, b.t()) * float(np.float32(alpha))
    return d.to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)


def rmsnorm_reference_f32(x_bits, w_bits, dtype: str, eps: float) -> np.ndarray:
    """The reference's independent fp32 oracle, _math_oracle :1300-1306."""
    x = bits_to_f32(x_bits, dtype).astype(np.float32)
    w = bits_to_f32(w_bits, dtype).astype(np.float32)
    normalized = x * (1.0 / np.sqrt((x * x).mean(axis=-1, keepdims=True) + np.float32(eps)))
    return bits_to_f32(f32_to_bits((normalized * w).astype(np.float32), dtype), dtype)


# --------------------------------------------------------------------------------------
# recorded MUFU values: lets a machine without a GPU replay what the hardware returned
# --------------------------------------------------------------------------------------
MUFU_OPS = ("rcp_ftz", "rsqrt_ftz", "lg2", "ex2", "ex2_ftz")


class RecordingMufu:
    """Wraps a provider and remembers every (op, input bits) -> output bits pair it served."""

    name = "recording"

    def __init__(self, inner):
        self._inner = inner
        self.tables = {op: {} for op in MUFU_OPS}

    def _wrap(self, op, x):
        x = np.ascontiguousarray(x, dtype=np.float32)
        out = np.asarray(getattr(self._inner, op)(x), dtype=np.float32)
        keys = x.reshape(-1).view(np.uint32)
        vals = out.reshape(-1).view(np.uint32)
        uniq, first = np.unique(keys, return_index=True)
        self.tables[op].update(zip(uniq.tolist(), vals[first].tolist()))
        return out

    def rcp_ftz(self, x):
        return self._wrap("rcp_ftz", x)

    def rsqrt_ftz(self, x):
        return self._wrap("rsqrt_ftz", x)

    def lg2(self, x):
        return self._wrap("lg2", x)

    def ex2(self, x):
        return self._wrap("ex2", x)

    def ex2_ftz(self, x):
        return self._wrap("ex2_ftz", x)

    def arrays(self) -> dict:
        out = {}
        for op, table in self.tables.items():
            keys = np.array(sorted(table), dtype=np.uint32)
            out[f"{op}_in"] = keys
            out[f"{op}_out"] = np.array([table[k] for k in keys.tolist()], dtype=np.uint32)
        return out


class TableMufu:
    """Replays recorded hardware values; an input that was never recorded is an error."""

    name = "table"

    def __init__(self, arrays):
        self._tables = {op: (np.asarray(arrays[f"{op}_in"], dtype=np.uint32),
                             np.asarray(arrays[f"{op}_out"], dtype=np.uint32)) for op in MUFU_OPS}

    def _lookup(self, op, x):
        x = np.ascontiguousarray(x, dtype=np.float32)
        keys, vals = self._tables[op]
        bits = x.reshape(-1).view(np.uint32)
        pos = np.searchsorted(keys, bits)
        pos = np.minimum(pos, max(len(keys) - 1, 0))
        if len(keys) == 0 or not np.array_equal(keys[pos], bits):
            raise KeyError(f"{op}: input not in the recorded table")
        return vals[pos].view(np.float32).reshape(x.shape)

    def rcp_ftz(self, x):
        return self._lookup("rcp_ftz", x)

    def rsqrt_ftz(self, x):
        return self._lookup("rsqrt_ftz", x)

    def lg2(self, x):
        return self._lookup("lg2", x)

    def ex2(self, x):
        return self._lookup("ex2", x)

    def ex2_ftz(self, x):
        return self._lookup("ex2_ftz", x)
