/*
 * Scalar C restatement of the NVFP4 quantizer arithmetic (TEST INFRASTRUCTURE - never on
 * the product path).  It exists so that full-size inputs can be checked bit for bit in
 * seconds and to serve as the timed CPU baseline; oracle/nvfp4_oracle.py is the
 * vectorised statement of the same arithmetic and the two are cross-checked in tests/.
 *
 * Reference followed (paths inside mlc-ai/TIRx-kernels):
 *   tirx_kernels/flashinfer/quantization/nvfp4_quantize.py:152-183   _process_block
 *   tirx_kernels/flashinfer/utils/fp_quant.py:60-69,100-103,250-269,291-311,375-401
 *   tirx_kernels/flashinfer/norm/rmsnorm_fp4quant.py:266-337,786-900
 *
 * Values of the hardware-approximate instructions (rcp.approx.ftz, rsqrt.approx.ftz) are
 * inputs: the caller passes rcp(6), per-E4M3-code tables and per-row rstd, taken either
 * from correct rounding (no GPU) or from the device probe.
 *
 * Build:  gcc -O2 -fopenmp -ffp-contract=off -fno-fast-math -shared -fPIC (see oracle/build.py)
 */
#include <math.h>
#include <stdint.h>
#include <string.h>

static inline float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static inline uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }

static inline float load16(uint16_t bits, int is_bf16) {
  if (is_bf16) return u2f((uint32_t)bits << 16);
  _Float16 h; memcpy(&h, &bits, 2); return (float)h;
}

/* cvt.rn.satfinite.e4m3x2.f32, one lane */
static uint8_t e4m3_encode(float v) {
  if (isnan(v)) return 0x7F;
  uint8_t sign = signbit(v) ? 0x80 : 0;
  float a = fabsf(v);
  if (isinf(a)) return sign | 0x7E;
  int e; frexpf(a, &e);
  int qexp = e - 1 - 3; if (qexp < -9) qexp = -9;
  float q = ldexpf(nearbyintf(ldexpf(a, -qexp)), qexp);
  if (q > 448.0f) q = 448.0f;
  if (q < 0.015625f) return sign | (uint8_t)(q * 512.0f);
  int e2; frexpf(q, &e2);
  int man = (int)(ldexpf(q, -(e2 - 1)) * 8.0f - 8.0f);
  return sign | (uint8_t)((e2 - 1 + 7) * 8 + man);
}

static float e4m3_decode(uint8_t c) {
  int exp = (c >> 3) & 0xF, man = c & 7;
  float v = exp == 0 ? ldexpf((float)man, -9) : ldexpf(1.0f + man / 8.0f, exp - 7);
  if ((c & 0x7F) == 0x7F) v = NAN;
  return (c & 0x80) ? -v : v;
}

/* cvt.rn.satfinite.e2m1x2.f32, one lane */
static inline uint8_t e2m1_encode(float v) {
  if (isnan(v)) return 7;
  float a = fabsf(v);
  uint8_t code = (uint8_t)((a > 0.25f) + (a >= 0.75f) + (a > 1.25f) + (a >= 1.75f) + (a > 2.5f) +
                           (a >= 3.5f) + (a > 5.0f));
  return code | (signbit(v) ? 8 : 0);
}

static inline int64_t sf_offset(int layout, int64_t r, int64_t c, int64_t pad_cols, int64_t lin_cols) {
  if (layout == 0) return r * lin_cols + c;
  if (layout == 1)
    return (c & 3) + (c >> 2) * 512 + (r & 31) * 16 + ((r & 127) >> 5) * 4 + (r >> 7) * (128 * pad_cols);
  return (r >> 3) * (((pad_cols + 3) / 4) * 32) + (c >> 2) * 32 + (r & 7) * 4 + (c & 3);
}

/* E4M3 codes of every positive finite scale, for building the per-code tables on the host. */
void oracle_e4m3_decode_table(float* out256) {
  for (int c = 0; c < 256; ++c) out256[c] = e4m3_decode((uint8_t)c);
}

int64_t oracle_sf_bytes(int m, int sf_cols, int layout) {
  if (layout == 0) return (int64_t)m * sf_cols;
  int64_t tile = layout == 2 ? 8 : 128;
  return (m + tile - 1) / tile * tile * (((int64_t)sf_cols + 3) / 4 * 4);
}

/*
 * nvfp4_quantize without SiLU fusion.
 *   out_scale_by_code[c] = 0 if decode(c) == 0 else rcp.approx.ftz(decode(c) * rcp.approx.ftz(gs))
 * The scale buffer is zero-filled first for swizzled layouts (the reference zero-fills padding).
 */
void oracle_nvfp4_quantize(const uint16_t* x, int is_bf16, int m, int k, float gs, float rcp6,
                           const float* out_scale_by_code, int layout, uint8_t* packed, uint8_t* sf) {
  const int nsb = k / 16;
  const int64_t pad_cols = ((int64_t)nsb + 3) / 4 * 4;
  if (layout != 0) memset(sf, 0, (size_t)oracle_sf_bytes(m, nsb, layout));
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < m; ++r) {
    for (int c = 0; c < nsb; ++c) {
      const uint16_t* blk = x + r * k + c * 16;
      float v[16], amax = 0.0f;
      for (int i = 0; i < 16; ++i) {
        v[i] = load16(blk[i], is_bf16);
        float a = fabsf(v[i]);
        if (a > amax) amax = a; /* NaNs are dropped, as max.f16x2/max.bf16x2 do */
      }
      float scale = gs * (amax * rcp6);
      uint8_t code = e4m3_encode(scale);
      float out_scale = out_scale_by_code[code];
      sf[sf_offset(layout, r, c, pad_cols, nsb)] = code;
      uint8_t* dst = packed + r * (k / 2) + c * 8;
      for (int i = 0; i < 8; ++i) {
        uint8_t lo = e2m1_encode(v[2 * i] * out_scale);
        uint8_t hi = e2m1_encode(v[2 * i + 1] * out_scale);
        dst[i] = (uint8_t)(lo | (hi << 4));
      }
    }
  }
}

/* ---- RMSNorm + quantize, block 16 / E4M3 ------------------------------------------------ */
static int threads_per_row(int h) {
  if (h <= 64) return 8;
  if (h <= 128) return 16;
  if (h <= 3072) return 32;
  if (h <= 6144) return 64;
  if (h <= 16384) return 128;
  return 256;
}

/* The reference's fp32 summation tree for rows a single CTA holds (cluster_n == 1), then
 * mean + eps.  Returns -1 when H needs the cluster path (not restated in C). */
int oracle_rmsnorm_shifted_mean(const uint16_t* x, int is_bf16, int M, int H, float eps, float* out) {
  const int tpr = threads_per_row(H);
  const int nchunks = H / 8;
  int vb = (nchunks + tpr - 1) / tpr; if (vb < 1) vb = 1;
  const int rows = (tpr == 256 ? 256 : 128) / tpr;
  if (2LL * rows * vb * tpr * 16 + 64 > 232448) return -1;
  const int lanes = tpr < 32 ? tpr : 32;
  const int wpr = tpr >= 32 ? tpr / 32 : 1;
  const int pow2 = (H & (H - 1)) == 0;
  const float inv_h = 1.0f / (float)H;
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < M; ++r) {
    float local[256];
    for (int t = 0; t < tpr; ++t) {
      float acc = 0.0f;
      for (int b = 0; b < vb; ++b) {
        int chunk = t + b * tpr;
        if (chunk >= nchunks) continue;
        const uint16_t* p = x + r * H + (int64_t)chunk * 8;
        for (int i = 0; i < 8; ++i) { float f = load16(p[i], is_bf16); acc = acc + f * f; }
      }
      local[t] = acc;
    }
    float warp_sum[8];
    for (int w = 0; w < wpr; ++w) {
      float lane[32];
      for (int l = 0; l < lanes; ++l) lane[l] = local[w * 32 + l];
      for (int s = 1; s < lanes; s <<= 1) {
        float nxt[32];
        for (int l = 0; l < lanes; ++l) nxt[l] = lane[l] + lane[l ^ s];
        memcpy(lane, nxt, sizeof(float) * lanes);
      }
      warp_sum[w] = lane[0];
    }
    float sum = warp_sum[0];
    if (wpr > 1) {
      float lane[32];
      for (int l = 0; l < 32; ++l) lane[l] = l < wpr ? warp_sum[l] : 0.0f;
      for (int s = 1; s < 32; s <<= 1) {
        float nxt[32];
        for (int l = 0; l < 32; ++l) nxt[l] = lane[l] + lane[l ^ s];
        memcpy(lane, nxt, sizeof(lane));
      }
      sum = lane[0];
    }
    out[r] = pow2 ? fmaf(sum, inv_h, eps) : (sum / (float)H) + eps;
  }
  return 0;
}

/* mul.bf16x2 / mul.f16x2 lane: exact product rounded once to the 16-bit type, as fp32 */
static inline float mul16(uint16_t a, uint16_t b, int is_bf16) {
  if (!is_bf16) {
    _Float16 ha, hb; memcpy(&ha, &a, 2); memcpy(&hb, &b, 2);
    return (float)(_Float16)((float)ha * (float)hb);
  }
  double p = (double)u2f((uint32_t)a << 16) * (double)u2f((uint32_t)b << 16);
  if (isnan(p) || isinf(p)) return (float)p;
  int e; frexp(p, &e);
  int qexp = e - 1 - 7; if (qexp < -133) qexp = -133;
  return (float)ldexp(nearbyint(ldexp(p, -qexp)), qexp);
}

/*
 * Pass 2 of flashinfer_rmsnorm_fp4quant (block 16, E4M3):  rcp_by_code[c] = 0 if decode(c) == 0
 * else rcp.approx.ftz(decode(c)).  Scale positions that hold no logical scale are not written.
 */
void oracle_rmsnorm_quant(const uint16_t* x, const uint16_t* w, int is_bf16, int M, int H,
                          const float* rstd, float gs, float rcp6, const float* rcp_by_code,
                          int swizzled, uint8_t* y, uint8_t* sf) {
  const int nblk = H / 16;
  const int64_t pad_cols = ((int64_t)nblk + 3) / 4 * 4;
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < M; ++r) {
    const float rs = rstd[r];
    for (int c = 0; c < nblk; ++c) {
      float p[16], amax = 0.0f;
      for (int i = 0; i < 16; ++i) {
        p[i] = mul16(x[r * H + c * 16 + i], w[c * 16 + i], is_bf16);
        float a = fabsf(p[i]);
        if (a > amax) amax = a;
      }
      float max_abs = amax * rs;
      float s = (gs * max_abs) * rcp6;
      if (!(s <= 448.0f)) s = 448.0f; /* min.f32: a NaN operand yields the other one */
      uint8_t code = e4m3_encode(s);
      float out_scale = rcp_by_code[code] * gs;
      sf[sf_offset(swizzled ? 1 : 0, r, c, pad_cols, nblk)] = code;
      uint8_t* dst = y + r * (H / 2) + c * 8;
      for (int i = 0; i < 8; ++i) {
        uint8_t lo = e2m1_encode((p[2 * i] * rs) * out_scale);
        uint8_t hi = e2m1_encode((p[2 * i + 1] * rs) * out_scale);
        dst[i] = (uint8_t)(lo | (hi << 4));
      }
    }
  }
}

/* D = bf16(alpha * dequant(A) . dequant(B)^T) for a tile of rows, fp32 accumulation. */
static const float kE2M1[16] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f,
                                -0.0f, -0.5f, -1.0f, -1.5f, -2.0f, -3.0f, -4.0f, -6.0f};

void oracle_dequantize_nvfp4(const uint8_t* packed, const uint8_t* sf, int m, int k, int layout,
                             float global_scale, float* out) {
  const int nsb = k / 16;
  const int64_t pad_cols = ((int64_t)nsb + 3) / 4 * 4;
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < m; ++r) {
    for (int c = 0; c < nsb; ++c) {
      float s = e4m3_decode(sf[sf_offset(layout, r, c, pad_cols, nsb)]) / global_scale;
      for (int i = 0; i < 8; ++i) {
        uint8_t b = packed[r * (k / 2) + c * 8 + i];
        out[r * k + c * 16 + 2 * i] = kE2M1[b & 0xF] * s;
        out[r * k + c * 16 + 2 * i + 1] = kE2M1[b >> 4] * s;
      }
    }
  }
}
