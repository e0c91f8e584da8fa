// NVFP4 block quantizers for sm_100a.
//
// Arithmetic follows tirx_kernels/flashinfer/quantization/nvfp4_quantize.py:152-183
// (_process_block) and the instruction helpers of tirx_kernels/flashinfer/utils/fp_quant.py;
// the launch geometry does not.  Two kernels:
//   * flat slot kernel: the input is one flat array of 32-byte blocks, consecutive threads own
//     consecutive 16-element blocks, each fetched with a single 256-bit streaming load, several
//     loads issued per thread before the first is consumed.  Any shape, SiLU fusion, zero fill of
//     padding slots.
//   * row kernel: one CTA of 128 threads per row, thread t holds blocks t, t + 128, ... of the
//     row in registers.  It is the per-token quantizer (row maximum between load and quantize)
//     and, without that step, the faster plain quantizer for tall activations (m >= 1024, rows of
//     128..1024 blocks): 16384 CTAs of 48 registers keep more bytes in flight per SM than the
//     persistent flat grid and reach the measured copy bandwidth.
#include <algorithm>
#include <cstdlib>

#include "common.cuh"

namespace b2 {
namespace {

struct QuantParams {
  const uint8_t* in;   // [m, in_cols] 16-bit elements
  uint8_t* out;        // [m, k/2]
  uint8_t* sf;         // scale factors in the requested layout
  const float* gs;     // device scalar
  int m;               // data rows
  int k;               // quantized columns
  int nsb;             // k / 16: scale blocks per row
  int slot_cols;       // nsb (linear) or nsb rounded up to 4 (swizzled): slots per row
  int64_t in_row_bytes;  // bytes between input rows (2k, or 4k with SiLU fusion)
  uint32_t total_slots;  // slot rows * slot_cols
  uint64_t div_magic;    // floor(2^div_shift / slot_cols) + 1
  int div_shift;
  int enable_pdl;
};

// SiLU(gate) * up on one packed pair, re-rounded to the input type
// (fp_quant.py silu_f32 :340-344, silu_and_mul_pair :363-372).
template <typename Tag>
__device__ __forceinline__ uint32_t silu_and_mul_pair(uint32_t gate, uint32_t up) {
  // The reference unpacks with a multiply by 1.0, which changes no bit of a finite value.
  const float2 s = mul_f32x2(silu_f32x2(unpack2<Tag>(gate)), unpack2<Tag>(up));
  return pack_from_f32<Tag>(s.x, s.y);
}

// One 16-element block held as 8 packed words -> (E4M3 scale byte, 64 packed E2M1 bits).
template <typename Tag>
__device__ __forceinline__ void quantize_block(const uint32_t (&w)[8], float gs, float rcp_gs,
                                               float rcp6, uint32_t& sf_byte, uint2& packed) {
  const uint32_t lo4[4] = {w[0], w[1], w[2], w[3]};
  const uint32_t hi4[4] = {w[4], w[5], w[6], w[7]};
  const uint32_t m2 = hmax2<Tag>(absmax_4<Tag>(lo4), absmax_4<Tag>(hi4));
  const float amax = pair_max_to_f32<Tag>(m2);
  // scale = gs * (amax * rcp(6)), two roundings, inner product first.
  const float scale = mul_f32(gs, mul_f32(amax, rcp6));
  sf_byte = cvt_f32_to_e4m3(scale) & 0xFFu;
  const float sf_f32 = e4m3_to_f32(sf_byte);
  // out_scale = rcp(sf * rcp(gs)), zero when the stored scale is zero.
  const float inv = rcp_approx_ftz(mul_f32(sf_f32, rcp_gs));
  const float out_scale = (sf_f32 == 0.0f) ? 0.0f : inv;
  // x * out_scale, two elements per mul.f32x2 (each half rounds like mul.f32)
  const float2 s2 = make_float2(out_scale, out_scale);
  float v[8];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 q = mul_f32x2(unpack2<Tag>(w[i]), s2);
    v[2 * i] = q.x;
    v[2 * i + 1] = q.y;
  }
  packed.x = cvt_e2m1x8(v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 q = mul_f32x2(unpack2<Tag>(w[4 + i]), s2);
    v[2 * i] = q.x;
    v[2 * i + 1] = q.y;
  }
  packed.y = cvt_e2m1x8(v);
}

template <bool V8>
__device__ __forceinline__ void load_block(const uint8_t* p, uint32_t (&w)[8]) {
  if constexpr (V8) {
    ld_stream_256(p, w);
  } else {
    uint32_t a[4], b[4];
    ld_stream_128(p, a);
    ld_stream_128(p + 16, b);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      w[i] = a[i];
      w[4 + i] = b[i];
    }
  }
}

template <typename Tag, int LAYOUT, bool SILU, bool V8, int UNROLL>
__global__ void __launch_bounds__(256)
    nvfp4_quantize_kernel(const __grid_constant__ QuantParams p) {
  if (p.enable_pdl) pdl_wait();
  const float gs = *p.gs;
  const float rcp_gs = rcp_approx_ftz(gs);
  const float rcp6 = rcp_approx_ftz(6.0f);
  const uint32_t stride = gridDim.x * blockDim.x;
  const int out_row_bytes = p.k >> 1;

  for (uint32_t base = blockIdx.x * blockDim.x + threadIdx.x; base < p.total_slots;
       base += stride * UNROLL) {
    uint32_t w[UNROLL][8];
    uint32_t u[SILU ? UNROLL : 1][8];
    int row[UNROLL], col[UNROLL];
    bool live[UNROLL], data[UNROLL];
    // Phase 1: decode the slots and issue every load of this iteration.
#pragma unroll
    for (int j = 0; j < UNROLL; ++j) {
      const uint32_t s = base + j * stride;
      live[j] = s < p.total_slots;
      const uint32_t r = static_cast<uint32_t>((static_cast<uint64_t>(s) * p.div_magic) >> p.div_shift);
      row[j] = static_cast<int>(r);
      col[j] = static_cast<int>(s - r * static_cast<uint32_t>(p.slot_cols));
      data[j] = live[j] && row[j] < p.m && col[j] < p.nsb;
      if (data[j]) {
        const uint8_t* src = p.in + static_cast<int64_t>(row[j]) * p.in_row_bytes + col[j] * 32;
        load_block<V8>(src, w[j]);
        if constexpr (SILU) load_block<V8>(src + 2 * p.k, u[j]);
      }
    }
    // Phase 2: quantize and store.
#pragma unroll
    for (int j = 0; j < UNROLL; ++j) {
      if (!live[j]) continue;
      int64_t sf_off;
      if constexpr (LAYOUT == B2_SF_LINEAR) {
        sf_off = static_cast<int64_t>(row[j]) * p.nsb + col[j];
      } else if constexpr (LAYOUT == B2_SF_128x4) {
        sf_off = sf_offset_128x4(row[j], col[j], p.slot_cols);
      } else {
        sf_off = sf_offset_8x4(row[j], col[j], p.slot_cols);
      }
      if (!data[j]) {  // padding row or padding column of a swizzled layout
        p.sf[sf_off] = 0;
        continue;
      }
      if constexpr (SILU) {
#pragma unroll
        for (int i = 0; i < 8; ++i) w[j][i] = silu_and_mul_pair<Tag>(w[j][i], u[j][i]);
      }
      uint32_t sf_byte;
      uint2 packed;
      quantize_block<Tag>(w[j], gs, rcp_gs, rcp6, sf_byte, packed);
      p.sf[sf_off] = static_cast<uint8_t>(sf_byte);
      *reinterpret_cast<uint2*>(p.out + static_cast<int64_t>(row[j]) * out_row_bytes + col[j] * 8) =
          packed;
    }
  }
  if (p.enable_pdl) pdl_launch_dependents();
}

template <typename Tag, int LAYOUT, bool SILU, bool V8>
int launch(const QuantParams& p, cudaStream_t stream) {
  // SiLU fusion is bound by the math pipes, not by loads in flight: one slot per iteration keeps the
  // kernel at 45 registers and five CTAs per SM.
  constexpr int kUnroll = SILU ? 1 : 4;
  constexpr int kThreads = 256;
  auto kernel = nvfp4_quantize_kernel<Tag, LAYOUT, SILU, V8, kUnroll>;
  const int sms = device_sm_count();
  if (sms <= 0) return B2_ERR_CUDA;
  const int64_t per_block = static_cast<int64_t>(kThreads) * kUnroll;
  const int64_t want = (static_cast<int64_t>(p.total_slots) + per_block - 1) / per_block;
  const int grid = static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(want, sms * 8LL)));

  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  if (p.enable_pdl) {
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
  }
  B2_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, p));
  return B2_OK;
}

template <typename Tag, int LAYOUT>
int dispatch_flags(const QuantParams& p, bool silu, bool v8, cudaStream_t stream) {
  if (silu) return v8 ? launch<Tag, LAYOUT, true, true>(p, stream) : launch<Tag, LAYOUT, true, false>(p, stream);
  return v8 ? launch<Tag, LAYOUT, false, true>(p, stream) : launch<Tag, LAYOUT, false, false>(p, stream);
}

template <typename Tag>
int dispatch_layout(const QuantParams& p, int layout, bool silu, bool v8, cudaStream_t stream) {
  switch (layout) {
    case B2_SF_LINEAR: return dispatch_flags<Tag, B2_SF_LINEAR>(p, silu, v8, stream);
    case B2_SF_128x4: return dispatch_flags<Tag, B2_SF_128x4>(p, silu, v8, stream);
    default: return dispatch_flags<Tag, B2_SF_8x4>(p, silu, v8, stream);
  }
}

// ---- per-token variant (tirx_kernels/flashinfer/quantization/nvfp4_quantize_per_token.py) -------
// One CTA of 128 threads per row, as in the reference (:142-232): row maximum, token scale
// = amax * gs_inv, encode scale = rcp(token scale) (FLT_MAX for an all-zero row, :203-211), then
// the ordinary block recipe with the row's encode scale in place of the global scale (:56-74).
// Unlike the reference, which reads the row twice, the blocks a thread owns (t, t + 128, ...)
// stay in registers between the two passes when the row has at most 128 * NB blocks, and rows
// past m (padding rows of the swizzled layouts) are zero-filled by extra CTAs instead of the host.
struct PerTokenParams {
  const uint8_t* in;
  uint8_t* out;
  uint8_t* sf;
  float* token_scale;  // [m]
  const float* gs_inv;
  int m;
  int k;
  int nsb;
  int pad_cols;
  int enable_pdl;
};

template <int LAYOUT>
__device__ __forceinline__ int64_t sf_offset_any(int row, int col, int nsb, int pad_cols) {
  if constexpr (LAYOUT == B2_SF_LINEAR) return static_cast<int64_t>(row) * nsb + col;
  else if constexpr (LAYOUT == B2_SF_128x4) return sf_offset_128x4(row, col, pad_cols);
  else return sf_offset_8x4(row, col, pad_cols);
}

template <typename Tag>
__device__ __forceinline__ float block_amax(const uint32_t (&w)[8]) {
  const uint32_t lo4[4] = {w[0], w[1], w[2], w[3]};
  const uint32_t hi4[4] = {w[4], w[5], w[6], w[7]};
  return pair_max_to_f32<Tag>(hmax2<Tag>(absmax_4<Tag>(lo4), absmax_4<Tag>(hi4)));
}

// PER_TOKEN = false turns the same one-CTA-per-row structure into the plain quantizer (one global
// scale read from `gs_inv`, no row maximum, no token scales): for tall activations it keeps more
// bytes in flight per SM than the flat slot kernel above.
template <typename Tag, int LAYOUT, bool V8, int NB, bool PER_TOKEN = true>
__global__ void __launch_bounds__(128) nvfp4_quantize_row_kernel(const __grid_constant__ PerTokenParams p) {
  constexpr int kThreads = 128;
  __shared__ float red[4];
  const int row = blockIdx.x;
  const int t = threadIdx.x;
  if (p.enable_pdl) pdl_wait();
  if (row >= p.m) {  // padding row of a swizzled layout
    for (int c = t; c < p.pad_cols; c += kThreads) p.sf[sf_offset_any<LAYOUT>(row, c, p.nsb, p.pad_cols)] = 0;
    return;
  }
  const uint8_t* in_row = p.in + static_cast<int64_t>(row) * p.k * 2;
  uint8_t* out_row = p.out + static_cast<int64_t>(row) * (p.k >> 1);

  uint32_t w[NB > 0 ? NB : 1][8];
  float local = 0.0f;
  if constexpr (NB > 0) {
#pragma unroll
    for (int j = 0; j < NB; ++j) {
      const int col = t + j * kThreads;
      if (col < p.nsb) load_block<V8>(in_row + col * 32, w[j]);
    }
    if constexpr (PER_TOKEN) {
#pragma unroll
      for (int j = 0; j < NB; ++j)
        if (t + j * kThreads < p.nsb) local = max_f32(local, block_amax<Tag>(w[j]));
    }
  } else if constexpr (PER_TOKEN) {
    for (int col = t; col < p.nsb; col += kThreads) {
      load_block<V8>(in_row + col * 32, w[0]);
      local = max_f32(local, block_amax<Tag>(w[0]));
    }
  }
  float encode;
  if constexpr (PER_TOKEN) {
#pragma unroll
    for (int x = 1; x < 32; x <<= 1) local = max_f32(local, __shfl_xor_sync(0xFFFFFFFFu, local, x));
    if ((t & 31) == 0) red[t >> 5] = local;
    __syncthreads();
    float row_amax = (t & 31) < 4 ? red[t & 31] : 0.0f;
#pragma unroll
    for (int x = 1; x < 32; x <<= 1) row_amax = max_f32(row_amax, __shfl_xor_sync(0xFFFFFFFFu, row_amax, x));
    const float gs_inv = *p.gs_inv;
    float token = 0.0f;
    encode = 3.4028234663852886e38f;
    if (row_amax != 0.0f) {
      token = mul_f32(row_amax, gs_inv);
      encode = rcp_approx_ftz(token);
    }
    if (t == 0) p.token_scale[row] = token;
  } else {
    encode = *p.gs_inv;  // the plain quantizer's global scale
  }
  const float rcp_enc = rcp_approx_ftz(encode);
  const float rcp6 = rcp_approx_ftz(6.0f);

  auto emit = [&](const uint32_t(&blk)[8], int col) {
    uint32_t sf_byte;
    uint2 packed;
    quantize_block<Tag>(blk, encode, rcp_enc, rcp6, sf_byte, packed);
    p.sf[sf_offset_any<LAYOUT>(row, col, p.nsb, p.pad_cols)] = static_cast<uint8_t>(sf_byte);
    *reinterpret_cast<uint2*>(out_row + col * 8) = packed;
  };
  if constexpr (NB > 0) {
#pragma unroll
    for (int j = 0; j < NB; ++j)
      if (t + j * kThreads < p.nsb) emit(w[j], t + j * kThreads);
  } else {
    for (int col = t; col < p.nsb; col += kThreads) {
      load_block<V8>(in_row + col * 32, w[0]);  // second read of the row: served by L2
      emit(w[0], col);
    }
  }
  if constexpr (LAYOUT != B2_SF_LINEAR) {
    for (int c = p.nsb + t; c < p.pad_cols; c += kThreads) p.sf[sf_offset_any<LAYOUT>(row, c, p.nsb, p.pad_cols)] = 0;
  }
  if (p.enable_pdl) pdl_launch_dependents();
}

template <typename Tag, int LAYOUT, bool V8>
int launch_per_token(const PerTokenParams& p, int rows, cudaStream_t stream) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(rows);
  cfg.blockDim = dim3(128);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  if (p.enable_pdl) {
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
  }
  if (p.nsb <= 128) {
    B2_CUDA_TRY(cudaLaunchKernelEx(&cfg, nvfp4_quantize_row_kernel<Tag, LAYOUT, V8, 1>, p));
  } else if (p.nsb <= 256) {
    B2_CUDA_TRY(cudaLaunchKernelEx(&cfg, nvfp4_quantize_row_kernel<Tag, LAYOUT, V8, 2>, p));
  } else if (p.nsb <= 512) {
    B2_CUDA_TRY(cudaLaunchKernelEx(&cfg, nvfp4_quantize_row_kernel<Tag, LAYOUT, V8, 4>, p));
  } else if (p.nsb <= 1024) {
    B2_CUDA_TRY(cudaLaunchKernelEx(&cfg, nvfp4_quantize_row_kernel<Tag, LAYOUT, V8, 8>, p));
  } else {
    B2_CUDA_TRY(cudaLaunchKernelEx(&cfg, nvfp4_quantize_row_kernel<Tag, LAYOUT, V8, 0>, p));
  }
  return B2_OK;
}

// Plain quantizer through the row kernel (register-resident sizes only).
template <typename Tag, int LAYOUT, bool V8>
int launch_rows(const PerTokenParams& p, int rows, cudaStream_t stream) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(rows);
  cfg.blockDim = dim3(128);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  if (p.enable_pdl) {
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
  }
  if (p.nsb <= 128) {
    B2_CUDA_TRY(cudaLaunchKernelEx(&cfg, nvfp4_quantize_row_kernel<Tag, LAYOUT, V8, 1, false>, p));
  } else if (p.nsb <= 256) {
    B2_CUDA_TRY(cudaLaunchKernelEx(&cfg, nvfp4_quantize_row_kernel<Tag, LAYOUT, V8, 2, false>, p));
  } else if (p.nsb <= 512) {
    B2_CUDA_TRY(cudaLaunchKernelEx(&cfg, nvfp4_quantize_row_kernel<Tag, LAYOUT, V8, 4, false>, p));
  } else {
    B2_CUDA_TRY(cudaLaunchKernelEx(&cfg, nvfp4_quantize_row_kernel<Tag, LAYOUT, V8, 8, false>, p));
  }
  return B2_OK;
}

template <typename Tag>
int dispatch_rows(const PerTokenParams& p, int layout, bool v8, int rows, cudaStream_t stream) {
  switch (layout) {
    case B2_SF_LINEAR:
      return v8 ? launch_rows<Tag, B2_SF_LINEAR, true>(p, rows, stream) : launch_rows<Tag, B2_SF_LINEAR, false>(p, rows, stream);
    case B2_SF_128x4:
      return v8 ? launch_rows<Tag, B2_SF_128x4, true>(p, rows, stream) : launch_rows<Tag, B2_SF_128x4, false>(p, rows, stream);
    default:
      return v8 ? launch_rows<Tag, B2_SF_8x4, true>(p, rows, stream) : launch_rows<Tag, B2_SF_8x4, false>(p, rows, stream);
  }
}

template <typename Tag>
int dispatch_per_token(const PerTokenParams& p, int layout, bool v8, int rows, cudaStream_t stream) {
  switch (layout) {
    case B2_SF_LINEAR:
      return v8 ? launch_per_token<Tag, B2_SF_LINEAR, true>(p, rows, stream)
                : launch_per_token<Tag, B2_SF_LINEAR, false>(p, rows, stream);
    case B2_SF_128x4:
      return v8 ? launch_per_token<Tag, B2_SF_128x4, true>(p, rows, stream)
                : launch_per_token<Tag, B2_SF_128x4, false>(p, rows, stream);
    default:
      return v8 ? launch_per_token<Tag, B2_SF_8x4, true>(p, rows, stream)
                : launch_per_token<Tag, B2_SF_8x4, false>(p, rows, stream);
  }
}

// 0: flat slot kernel always; 1: row kernel for tall activations (default); 2: row kernel whenever
// the row fits in registers.  Read once from B2_QUANT_ROW_KERNEL (a tuning and test knob).
int g_row_kernel_mode = [] {
  const char* v = getenv("B2_QUANT_ROW_KERNEL");
  return v ? atoi(v) : 1;
}();

}  // namespace
}  // namespace b2

extern "C" int64_t b2_nvfp4_sf_bytes(int m, int k, int sf_layout) {
  if (m < 1 || k <= 0 || k % 16 != 0) return -1;
  const int64_t nsb = k / 16;
  if (sf_layout == B2_SF_LINEAR) return static_cast<int64_t>(m) * nsb;
  const int64_t tile = sf_layout == B2_SF_8x4 ? 8 : 128;
  if (sf_layout != B2_SF_8x4 && sf_layout != B2_SF_128x4) return -1;
  return (m + tile - 1) / tile * tile * ((nsb + 3) / 4 * 4);
}

extern "C" int b2_nvfp4_quantize(const void* in, void* out, void* sf, const float* gs_dev, int m,
                                 int k, int in_dtype, int sf_layout, int fuse_silu, int enable_pdl,
                                 void* stream) {
  using namespace b2;
  if (in_dtype != B2_DTYPE_F16 && in_dtype != B2_DTYPE_BF16) {
    set_error("b2_nvfp4_quantize: unsupported in_dtype %d", in_dtype);
    return B2_ERR_INVALID_ARGUMENT;
  }
  if (sf_layout != B2_SF_LINEAR && sf_layout != B2_SF_128x4 && sf_layout != B2_SF_8x4) {
    set_error("b2_nvfp4_quantize: unsupported sf_layout %d", sf_layout);
    return B2_ERR_INVALID_ARGUMENT;
  }
  if (m < 1) {
    set_error("b2_nvfp4_quantize: m=%d must be >= 1", m);
    return B2_ERR_INVALID_ARGUMENT;
  }
  if (k <= 0 || k % 16 != 0) {
    set_error("b2_nvfp4_quantize: k=%d outside the dispatch domain (k %% 16 != 0)", k);
    return B2_ERR_INVALID_ARGUMENT;
  }
  if (!in || !out || !sf || !gs_dev) {
    set_error("b2_nvfp4_quantize: null pointer argument");
    return B2_ERR_INVALID_ARGUMENT;
  }
  if ((reinterpret_cast<uintptr_t>(in) & 15) || (reinterpret_cast<uintptr_t>(out) & 7)) {
    set_error("b2_nvfp4_quantize: `in` must be 16-byte and `out` 8-byte aligned");
    return B2_ERR_INVALID_ARGUMENT;
  }
  QuantParams p;
  p.in = static_cast<const uint8_t*>(in);
  p.out = static_cast<uint8_t*>(out);
  p.sf = static_cast<uint8_t*>(sf);
  p.gs = gs_dev;
  p.m = m;
  p.k = k;
  p.nsb = k / 16;
  p.in_row_bytes = static_cast<int64_t>(k) * (fuse_silu ? 4 : 2);
  p.enable_pdl = enable_pdl ? 1 : 0;
  int64_t slot_rows = m;
  p.slot_cols = p.nsb;
  if (sf_layout != B2_SF_LINEAR) {
    const int tile = sf_layout == B2_SF_8x4 ? 8 : 128;
    slot_rows = (static_cast<int64_t>(m) + tile - 1) / tile * tile;
    p.slot_cols = (p.nsb + 3) / 4 * 4;
  }
  const int64_t total = slot_rows * p.slot_cols;
  if (total >= (1LL << 31)) {
    set_error("b2_nvfp4_quantize: %lld scale blocks exceed the 2^31 limit", (long long)total);
    return B2_ERR_INVALID_ARGUMENT;
  }
  p.total_slots = static_cast<uint32_t>(total);
  int l = 0;
  while ((1LL << l) < p.slot_cols) ++l;
  p.div_shift = 32 + l;
  p.div_magic = (1ULL << p.div_shift) / static_cast<uint64_t>(p.slot_cols) + 1;
  const bool v8 = (reinterpret_cast<uintptr_t>(in) & 31) == 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (!fuse_silu && g_row_kernel_mode != 0 && p.nsb <= 1024 &&
      (g_row_kernel_mode == 2 || (m >= 1024 && p.nsb >= 128))) {
    // tall activation: one CTA per row, blocks held in registers
    PerTokenParams r;
    r.in = p.in;
    r.out = p.out;
    r.sf = p.sf;
    r.token_scale = nullptr;
    r.gs_inv = gs_dev;
    r.m = m;
    r.k = k;
    r.nsb = p.nsb;
    r.pad_cols = p.slot_cols;
    r.enable_pdl = p.enable_pdl;
    if (in_dtype == B2_DTYPE_F16) return dispatch_rows<F16Tag>(r, sf_layout, v8, static_cast<int>(slot_rows), s);
    return dispatch_rows<BF16Tag>(r, sf_layout, v8, static_cast<int>(slot_rows), s);
  }
  if (in_dtype == B2_DTYPE_F16) return dispatch_layout<F16Tag>(p, sf_layout, fuse_silu != 0, v8, s);
  return dispatch_layout<BF16Tag>(p, sf_layout, fuse_silu != 0, v8, s);
}

extern "C" int b2_nvfp4_quantize_per_token(const void* in, void* out, void* sf, float* token_scale,
                                           const float* gs_inv_dev, int m, int k, int in_dtype, int sf_layout,
                                           int enable_pdl, void* stream) {
  using namespace b2;
  if (in_dtype != B2_DTYPE_F16 && in_dtype != B2_DTYPE_BF16) {
    set_error("b2_nvfp4_quantize_per_token: Unsupported dtype: %d", in_dtype);
    return B2_ERR_INVALID_ARGUMENT;
  }
  if (sf_layout != B2_SF_LINEAR && sf_layout != B2_SF_128x4 && sf_layout != B2_SF_8x4) {
    set_error("b2_nvfp4_quantize_per_token: Unsupported sf_layout: %d", sf_layout);
    return B2_ERR_INVALID_ARGUMENT;
  }
  if (m < 1) {
    set_error("b2_nvfp4_quantize_per_token: m=%d must be >= 1", m);
    return B2_ERR_INVALID_ARGUMENT;
  }
  if (k <= 0 || k % 16 != 0) {
    set_error("b2_nvfp4_quantize_per_token: k=%d outside the source dispatch domain (k %% 16 != 0)", k);
    return B2_ERR_INVALID_ARGUMENT;
  }
  if (!in || !out || !sf || !token_scale || !gs_inv_dev) {
    set_error("b2_nvfp4_quantize_per_token: null pointer argument");
    return B2_ERR_INVALID_ARGUMENT;
  }
  if ((reinterpret_cast<uintptr_t>(in) & 15) || (reinterpret_cast<uintptr_t>(out) & 7)) {
    set_error("b2_nvfp4_quantize_per_token: `in` must be 16-byte and `out` 8-byte aligned");
    return B2_ERR_INVALID_ARGUMENT;
  }
  PerTokenParams p;
  p.in = static_cast<const uint8_t*>(in);
  p.out = static_cast<uint8_t*>(out);
  p.sf = static_cast<uint8_t*>(sf);
  p.token_scale = token_scale;
  p.gs_inv = gs_inv_dev;
  p.m = m;
  p.k = k;
  p.nsb = k / 16;
  p.pad_cols = p.nsb;
  int64_t rows = m;
  if (sf_layout != B2_SF_LINEAR) {
    const int tile = sf_layout == B2_SF_8x4 ? 8 : 128;
    rows = (static_cast<int64_t>(m) + tile - 1) / tile * tile;
    p.pad_cols = (p.nsb + 3) / 4 * 4;
  }
  if (rows > 2147483647ll) {
    set_error("b2_nvfp4_quantize_per_token: m=%d exceeds the grid limit", m);
    return B2_ERR_INVALID_ARGUMENT;
  }
  p.enable_pdl = enable_pdl ? 1 : 0;
  const bool v8 = (reinterpret_cast<uintptr_t>(in) & 31) == 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (in_dtype == B2_DTYPE_F16) return dispatch_per_token<F16Tag>(p, sf_layout, v8, static_cast<int>(rows), s);
  return dispatch_per_token<BF16Tag>(p, sf_layout, v8, static_cast<int>(rows), s);
}
