// Residual add + RMSNorm + FP4 block quantization for sm_100a.
//
// Arithmetic follows tirx_kernels/flashinfer/norm/add_rmsnorm_fp4quant.py of the reference:
//   h = x + residual in fp32 (kernel_body :951-958); the squares of the UNROUNDED sums are added
//   one by one by virtual thread t over its chunks t, t+tpr, ... (:960-983), then the usual
//   butterflies; h rounded to the input dtype replaces the residual in place (:1052-1071).
//   Rows one CTA holds (:177-229): value = (h * rstd) * w in fp32 on the rounded h, block
//   maximum of |value| in fp32.  Rows spread over a cluster (:230-258): 16-bit product h * w,
//   its maximum times rstd, value = product * rstd.  Scale byte and output scale as in
//   rmsnorm_fp4quant (:260-272), optional second copy of the scale bytes in the linear layout
//   (:274-290) and optional normalized row in the input dtype (:134-153, :309-314).
// The launch configuration (threads per row, cluster size) only fixes the summation order here;
// data movement is this file's own: x and the residual are read once, the rounded h is parked in
// shared memory, and the quantization pass reads it from there with one thread per scale block.
#include <algorithm>
#include <cstdlib>

#include "common.cuh"
#include "norm_quant.cuh"

namespace b2 {
namespace {

struct AddRmsParams {
  const uint8_t* x;
  uint8_t* residual;   // in: residual, out: x + residual rounded to the input dtype
  const uint8_t* w;
  uint8_t* y;
  uint8_t* sf;         // primary scale buffer (swizzled when `sf_swizzled`)
  uint8_t* sf_linear;  // second, linear copy (both layouts requested), else unused
  uint8_t* y_norm;     // normalized row in the input dtype, else unused
  const float* gs;
  int M;
  int H;
  int vb;
  int block_size;
  int use_e4m3;
  int sf_swizzled;
  int both;
  int norm;
  int sf_cols;
  int sf_pad_cols;
  int pow2;
  float eps;
  float inv_h;
  int enable_pdl;
  int stagger_ns;   // start offset between the CTAs that share an SM at launch (0 = none)
  int first_ctas;   // CTAs resident at launch
  int sm_count;
};

__device__ __forceinline__ void ld_global_128(const void* p, uint32_t (&r)[4]) {
  asm volatile("ld.global.L1::no_allocate.v4.b32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "l"(p));
}

// One chunk of 8 values: h = x + r (fp32), acc += h*h element by element (separate multiply and
// add: the square of an fp32 sum is not exact), returns h rounded to the input dtype.
template <typename Tag>
__device__ __forceinline__ uint4 add_chunk(const uint32_t (&xw)[4], const uint32_t (&rw)[4], float& acc) {
  uint32_t out[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float lo = add_f32(unpack_lo<Tag>(xw[i]), unpack_lo<Tag>(rw[i]));
    const float hi = add_f32(unpack_hi<Tag>(xw[i]), unpack_hi<Tag>(rw[i]));
    acc = add_f32(acc, mul_f32(lo, lo));
    acc = add_f32(acc, mul_f32(hi, hi));
    out[i] = pack_from_f32<Tag>(lo, hi);
  }
  return make_uint4(out[0], out[1], out[2], out[3]);
}

struct BlockScale {
  uint32_t code;
  float out_scale;
};
__device__ __forceinline__ BlockScale block_scale(float max_abs, float gs, float rcp6, bool use_e4m3) {
  BlockScale s;
  if (use_e4m3) {
    const float v = min_f32(mul_f32(mul_f32(gs, max_abs), rcp6), 448.0f);
    s.code = cvt_f32_to_e4m3(v) & 0xFFu;
    const float d = e4m3_to_f32(s.code);
    const float r = rcp_approx_ftz(d);
    s.out_scale = mul_f32(d == 0.0f ? 0.0f : r, gs);
  } else {
    s.code = cvt_f32_to_ue8m0(mul_f32(max_abs, rcp6));
    s.out_scale = ue8m0_to_output_scale(s.code);
  }
  return s;
}

// Quantizes one scale block whose rounded h sits in shared memory (`hblk`: BLOCK/8 chunks) and
// writes every output of the block.  CLUSTER selects the arithmetic of the cluster rows.
template <typename Tag, int BLOCK, bool CLUSTER>
__device__ __forceinline__ void quantize_block(const AddRmsParams& p, const uint4* hblk, int row, int j, float rstd,
                                               float gs, float rcp6) {
  constexpr int kChunks = BLOCK / 8;
  const uint4* wrow = reinterpret_cast<const uint4*>(p.w);
  float v[kChunks][8];
  float max_abs;
  if constexpr (CLUSTER) {
    uint32_t m2 = 0u;
#pragma unroll
    for (int c = 0; c < kChunks; ++c) {
      const uint4 hc = hblk[c];
      const uint4 wc = __ldg(wrow + j * kChunks + c);
      const uint32_t prod[4] = {hmul2<Tag>(hc.x, wc.x), hmul2<Tag>(hc.y, wc.y), hmul2<Tag>(hc.z, wc.z),
                                hmul2<Tag>(hc.w, wc.w)};
      const uint32_t m = absmax_4<Tag>(prod);
      m2 = c == 0 ? m : hmax2<Tag>(m2, m);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        v[c][2 * i] = mul_f32(unpack_lo<Tag>(prod[i]), rstd);
        v[c][2 * i + 1] = mul_f32(unpack_hi<Tag>(prod[i]), rstd);
      }
    }
    max_abs = mul_f32(pair_max_to_f32<Tag>(m2), rstd);
  } else {
    max_abs = 0.0f;
#pragma unroll
    for (int c = 0; c < kChunks; ++c) {
      const uint4 hc = hblk[c];
      const uint4 wc = __ldg(wrow + j * kChunks + c);
      const uint32_t hw[4] = {hc.x, hc.y, hc.z, hc.w};
      const uint32_t ww[4] = {wc.x, wc.y, wc.z, wc.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        v[c][2 * i] = mul_f32(mul_f32(unpack_lo<Tag>(hw[i]), rstd), unpack_lo<Tag>(ww[i]));
        v[c][2 * i + 1] = mul_f32(mul_f32(unpack_hi<Tag>(hw[i]), rstd), unpack_hi<Tag>(ww[i]));
        max_abs = max_f32(max_abs, fabsf(v[c][2 * i]));
        max_abs = max_f32(max_abs, fabsf(v[c][2 * i + 1]));
      }
    }
  }
  const BlockScale s = block_scale(max_abs, gs, rcp6, p.use_e4m3 != 0);

  const int64_t primary = p.sf_swizzled ? sf_offset_128x4(row, j, p.sf_pad_cols)
                                        : static_cast<int64_t>(row) * p.sf_cols + j;
  p.sf[primary] = static_cast<uint8_t>(s.code);
  if (p.both) p.sf_linear[static_cast<int64_t>(row) * p.sf_cols + j] = static_cast<uint8_t>(s.code);

  uint32_t q[kChunks];
  const float2 o2 = make_float2(s.out_scale, s.out_scale);
#pragma unroll
  for (int c = 0; c < kChunks; ++c) {
    float scaled[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 t = mul_f32x2(make_float2(v[c][2 * i], v[c][2 * i + 1]), o2);
      scaled[2 * i] = t.x;
      scaled[2 * i + 1] = t.y;
    }
    q[c] = cvt_e2m1x8(scaled);
  }
  uint8_t* yrow = p.y + static_cast<int64_t>(row) * (p.H >> 1);
  if constexpr (kChunks == 2) {
    *reinterpret_cast<uint2*>(yrow + j * 8) = make_uint2(q[0], q[1]);
  } else {
    *reinterpret_cast<uint4*>(yrow + j * 16) = make_uint4(q[0], q[1], q[2], q[3]);
  }
  if (p.norm) {
    uint4* nrow = reinterpret_cast<uint4*>(p.y_norm + (static_cast<int64_t>(row) * p.H + static_cast<int64_t>(j) * BLOCK) * 2);
#pragma unroll
    for (int c = 0; c < kChunks; ++c)
      nrow[c] = make_uint4(pack_from_f32<Tag>(v[c][0], v[c][1]), pack_from_f32<Tag>(v[c][2], v[c][3]),
                           pack_from_f32<Tag>(v[c][4], v[c][5]), pack_from_f32<Tag>(v[c][6], v[c][7]));
  }
}

// ---- rows one CTA holds -----------------------------------------------------------------------------
template <typename Tag, int TPR, int BLOCK>
__global__ void __launch_bounds__(TPR == 256 ? 256 : 128)
    add_rmsnorm_fp4quant_kernel(const __grid_constant__ AddRmsParams p) {
  constexpr int kThreads = TPR == 256 ? 256 : 128;
  constexpr int kRows = kThreads / TPR;
  constexpr int kWarpsPerRow = TPR >= 32 ? TPR / 32 : 1;
  constexpr int kChunksPerBlock = BLOCK / 8;
  extern __shared__ __align__(16) uint8_t smem[];
  uint4* tile = reinterpret_cast<uint4*>(smem);  // rounded h: [kRows][vb * TPR] chunks
  float* red = reinterpret_cast<float*>(smem + static_cast<size_t>(kRows) * p.vb * TPR * 16);

  const int tid = threadIdx.x;
  const int row_in_cta = tid / TPR;
  const int t = tid % TPR;
  const int row = blockIdx.x * kRows + row_in_cta;
  const bool row_valid = row < p.M;
  const int nchunks = p.H >> 3;
  const int lane = tid & 31;
  const int warp = tid >> 5;

  if (p.enable_pdl) pdl_wait();
  // The CTAs resident at launch would all stream their rows in at once and then all quantize at once; the
  // k-th CTA of an SM starts k * stagger_ns late (a fixed number of short sleeps).
  if (p.stagger_ns > 0 && static_cast<int>(blockIdx.x) < p.first_ctas) {
    const unsigned long long wait_ns = static_cast<unsigned long long>(blockIdx.x / p.sm_count) * p.stagger_ns;
    unsigned long long t0, now;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    for (unsigned long long i = 0; i < wait_ns / 32 + 8; ++i) {  // timed, and bounded by a count of short sleeps
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
      if (now - t0 >= wait_ns) break;
      __nanosleep(64);
    }
  }
  const float rcp6 = rcp_approx_ftz(6.0f);
  const uint4* xrow = reinterpret_cast<const uint4*>(p.x + static_cast<int64_t>(row) * p.H * 2);
  uint4* rrow = reinterpret_cast<uint4*>(p.residual + static_cast<int64_t>(row) * p.H * 2);
  uint4* my_row = tile + static_cast<size_t>(row_in_cta) * p.vb * TPR;

  float sum = 0.0f;
  for (int b0 = 0; b0 < p.vb; b0 += 2) {
    uint32_t xc[2][4], rc[2][4];
    bool ok[2];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int chunk = t + (b0 + j) * TPR;
      ok[j] = row_valid && (b0 + j) < p.vb && chunk < nchunks;
      if (ok[j]) {
        ld_stream_128(xrow + chunk, xc[j]);
        ld_global_128(rrow + chunk, rc[j]);
      }
    }
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      if (ok[j]) {
        const int chunk = t + (b0 + j) * TPR;
        const uint4 h = add_chunk<Tag>(xc[j], rc[j], sum);
        my_row[chunk] = h;
        rrow[chunk] = h;
      }
    }
  }
#pragma unroll
  for (int x = 1; x < (TPR < 32 ? TPR : 32); x <<= 1) sum = add_f32(sum, __shfl_xor_sync(0xFFFFFFFFu, sum, x));
  if constexpr (kWarpsPerRow > 1) {
    const int row_warp = warp / kWarpsPerRow;
    const int warp_in_row = warp % kWarpsPerRow;
    if (lane == 0) red[row_warp + warp_in_row * kRows] = sum;
    __syncthreads();
    float part = lane < kWarpsPerRow ? red[row_warp + lane * kRows] : 0.0f;
#pragma unroll
    for (int x = 1; x < 32; x <<= 1) part = add_f32(part, __shfl_xor_sync(0xFFFFFFFFu, part, x));
    sum = part;
  } else {
    __syncthreads();
  }
  const float shifted =
      p.pow2 ? __fmaf_rn(sum, p.inv_h, p.eps) : add_f32(__fdiv_rn(sum, static_cast<float>(p.H)), p.eps);
  const float rstd = rsqrt_approx_ftz(shifted);
  const float gs = p.use_e4m3 ? *p.gs : 0.0f;
  if (!row_valid) return;
  for (int j = t; j < p.sf_cols; j += TPR)
    quantize_block<Tag, BLOCK, false>(p, my_row + j * kChunksPerBlock, row, j, rstd, gs, rcp6);
  if (p.enable_pdl) pdl_launch_dependents();
}

// ---- rows spread over a thread-block cluster -----------------------------------------------------------
template <typename Tag, int TPR, int BLOCK>
__global__ void __launch_bounds__(TPR) add_rmsnorm_fp4quant_cluster_kernel(const __grid_constant__ AddRmsParams p,
                                                                            int cluster_n) {
  constexpr int kWarps = TPR / 32;
  constexpr int kChunksPerBlock = BLOCK / 8;
  extern __shared__ __align__(16) uint8_t smem[];
  uint4* tile = reinterpret_cast<uint4*>(smem);
  float* partials = reinterpret_cast<float*>(smem + static_cast<size_t>(p.vb) * TPR * 16);  // [cluster_n * kWarps]

  const int t = threadIdx.x;
  const int lane = t & 31, warp = t >> 5;
  const int cta = static_cast<int>(cluster_rank());
  const int row = blockIdx.x / cluster_n;
  const int nchunks = p.H >> 3;
  const int chunk0 = cta * p.vb * TPR;

  if (p.enable_pdl) pdl_wait();
  const float rcp6 = rcp_approx_ftz(6.0f);
  const uint4* xrow = reinterpret_cast<const uint4*>(p.x + static_cast<int64_t>(row) * p.H * 2);
  uint4* rrow = reinterpret_cast<uint4*>(p.residual + static_cast<int64_t>(row) * p.H * 2);

  float sum = 0.0f;
  for (int b0 = 0; b0 < p.vb; b0 += 2) {
    uint32_t xc[2][4], rc[2][4];
    bool ok[2];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int local = t + (b0 + j) * TPR;
      ok[j] = (b0 + j) < p.vb && chunk0 + local < nchunks;
      if (ok[j]) {
        ld_stream_128(xrow + chunk0 + local, xc[j]);
        ld_global_128(rrow + chunk0 + local, rc[j]);
      }
    }
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      if (ok[j]) {
        const int local = t + (b0 + j) * TPR;
        const uint4 h = add_chunk<Tag>(xc[j], rc[j], sum);
        tile[local] = h;
        rrow[chunk0 + local] = h;
      }
    }
  }
#pragma unroll
  for (int x = 1; x < 32; x <<= 1) sum = add_f32(sum, __shfl_xor_sync(0xFFFFFFFFu, sum, x));
  if (lane < cluster_n) st_cluster_f32(partials + cta * kWarps + warp, static_cast<uint32_t>(lane), sum);
  cluster_barrier();
  const int total = cluster_n * kWarps;
  float part = 0.0f;
  for (int i = lane; i < total; i += 32) part = add_f32(part, partials[i]);
#pragma unroll
  for (int x = 1; x < 32; x <<= 1) part = add_f32(part, __shfl_xor_sync(0xFFFFFFFFu, part, x));
  const float shifted =
      p.pow2 ? __fmaf_rn(part, p.inv_h, p.eps) : add_f32(__fdiv_rn(part, static_cast<float>(p.H)), p.eps);
  const float rstd = rsqrt_approx_ftz(shifted);
  const float gs = p.use_e4m3 ? *p.gs : 0.0f;

  const int blocks_here = p.vb * TPR / kChunksPerBlock;
  const int block0 = chunk0 / kChunksPerBlock;
  for (int jl = t; jl < blocks_here; jl += TPR) {
    const int j = block0 + jl;
    if (j >= p.sf_cols) break;
    quantize_block<Tag, BLOCK, true>(p, tile + jl * kChunksPerBlock, row, j, rstd, gs, rcp6);
  }
  if (p.enable_pdl) pdl_launch_dependents();
}

// add_rmsnorm_fp4quant.py _derived_config / _estimate_smem / _source_config :325-363
int add_source_cluster_n(int H) {
  for (int cand = 1; cand <= 16; cand *= 2) {
    const int hpc = H / cand;
    const int tpr = threads_per_row(hpc);
    const int threads = hpc <= 16384 ? 128 : 256;
    const int rows = threads / tpr;
    const int wpr = std::max(tpr / 32, 1);
    const int64_t vb = std::max(1, ((hpc / 8) + tpr - 1) / tpr);
    const int64_t tile = static_cast<int64_t>(rows) * 8 * vb * tpr * 2;
    const int64_t red = static_cast<int64_t>(rows) * wpr * 4;
    const int64_t est = cand == 1 ? 4 * tile + red : 2 * tile + red * cand + 8;
    if (H % cand == 0 && est <= 232448) return cand;
  }
  return 16;
}

void set_launch_attrs(cudaLaunchConfig_t& cfg, cudaLaunchAttribute* attr, int cluster_n, bool pdl) {
  int n = 0;
  if (cluster_n > 1) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = cluster_n;
    attr[n].val.clusterDim.y = 1;
    attr[n].val.clusterDim.z = 1;
    ++n;
  }
  if (pdl) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
}

template <typename Tag, int TPR, int BLOCK>
int launch(const AddRmsParams& p, cudaStream_t stream) {
  constexpr int kThreads = TPR == 256 ? 256 : 128;
  constexpr int kRows = kThreads / TPR;
  constexpr int kWarpsPerRow = TPR >= 32 ? TPR / 32 : 1;
  auto kernel = add_rmsnorm_fp4quant_kernel<Tag, TPR, BLOCK>;
  const size_t smem = static_cast<size_t>(kRows) * p.vb * TPR * 16 + kRows * kWarpsPerRow * 4;
  if (smem > 48 * 1024)
    B2_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((p.M + kRows - 1) / kRows);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  set_launch_attrs(cfg, attr, 1, p.enable_pdl != 0);
  AddRmsParams q = p;
  // B2_ADDRMS_STAGGER_NS: start offset between the CTAs that share an SM at launch, for launches of two
  // generations of CTAs or more (default 300; 8192 x 7168: none 66.3 us, 100 ns 66.3, 200 ns 65.8, 300 ns 65.3).
  static const int stagger = [] { const char* v = getenv("B2_ADDRMS_STAGGER_NS"); return v ? atoi(v) : 300; }();
  if (stagger > 0) {
    int per_sm = 0;
    B2_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kThreads, smem));
    q.sm_count = std::max(device_sm_count(), 1);
    q.first_ctas = per_sm * q.sm_count;
    q.stagger_ns = static_cast<int>(cfg.gridDim.x) >= 2 * q.first_ctas ? stagger : 0;
  }
  B2_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, q));
  return B2_OK;
}

template <typename Tag, int TPR, int BLOCK>
int launch_cluster(const AddRmsParams& p, int cluster_n, cudaStream_t stream) {
  auto kernel = add_rmsnorm_fp4quant_cluster_kernel<Tag, TPR, BLOCK>;
  const size_t smem = static_cast<size_t>(p.vb) * TPR * 16 + static_cast<size_t>(cluster_n) * (TPR / 32) * 4;
  B2_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
  if (cluster_n > 8) B2_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(p.M) * cluster_n);
  cfg.blockDim = dim3(TPR);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  set_launch_attrs(cfg, attr, cluster_n, p.enable_pdl != 0);
  B2_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, p, cluster_n));
  return B2_OK;
}

template <typename Tag, int BLOCK>
int dispatch(const AddRmsParams& p, int tpr, int cluster_n, cudaStream_t stream) {
  if (cluster_n > 1) {
    if (tpr == 128) return launch_cluster<Tag, 128, BLOCK>(p, cluster_n, stream);
    return launch_cluster<Tag, 256, BLOCK>(p, cluster_n, stream);
  }
  switch (tpr) {
    case 8: return launch<Tag, 8, BLOCK>(p, stream);
    case 16: return launch<Tag, 16, BLOCK>(p, stream);
    case 32: return launch<Tag, 32, BLOCK>(p, stream);
    case 64: return launch<Tag, 64, BLOCK>(p, stream);
    case 128: return launch<Tag, 128, BLOCK>(p, stream);
    default: return launch<Tag, 256, BLOCK>(p, stream);
  }
}

}  // namespace
}  // namespace b2

extern "C" int b2_add_rmsnorm_fp4quant(const void* x, void* residual, const void* w, void* y, void* sf,
                                       void* sf_unswizzled, void* y_norm, const float* gs_dev, int M, int H,
                                       float eps, int in_dtype, int block_size, int scale_format, int swizzled,
                                       int output_both_sf_layouts, int output_norm, int enable_pdl, void* stream) {
  using namespace b2;
  if (in_dtype != B2_DTYPE_F16 && in_dtype != B2_DTYPE_BF16) {
    set_error("b2_add_rmsnorm_fp4quant: unsupported input_dtype %d", in_dtype);
    return B2_ERR_INVALID_ARGUMENT;
  }
  if (block_size != 16 && block_size != 32) {
    set_error("b2_add_rmsnorm_fp4quant: block_size must be 16 or 32");
    return B2_ERR_INVALID_ARGUMENT;
  }
  if (H < 64 || H % block_size != 0) {
    set_error("b2_add_rmsnorm_fp4quant: H must be >=64 and divisible by block_size");
    return B2_ERR_INVALID_ARGUMENT;
  }
  if (scale_format != B2_SCALE_E4M3 && scale_format != B2_SCALE_UE8M0) {
    set_error("b2_add_rmsnorm_fp4quant: scale_format must be e4m3 or ue8m0");
    return B2_ERR_INVALID_ARGUMENT;
  }
  if (M <= 0) {
    set_error("b2_add_rmsnorm_fp4quant: M must be positive, got %d", M);
    return B2_ERR_INVALID_ARGUMENT;
  }
  const bool use_e4m3 = block_size == 16 || scale_format == B2_SCALE_E4M3;
  if (!x || !residual || !w || !y || !sf || (use_e4m3 && !gs_dev) || (output_both_sf_layouts && !sf_unswizzled) ||
      (output_norm && !y_norm)) {
    set_error("b2_add_rmsnorm_fp4quant: null pointer argument");
    return B2_ERR_INVALID_ARGUMENT;
  }
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(residual) & 15) ||
      (reinterpret_cast<uintptr_t>(w) & 15) || (reinterpret_cast<uintptr_t>(y) & 7) ||
      (output_norm && (reinterpret_cast<uintptr_t>(y_norm) & 15))) {
    set_error("b2_add_rmsnorm_fp4quant: x, residual, w and y_norm must be 16-byte aligned, y 8-byte aligned");
    return B2_ERR_INVALID_ARGUMENT;
  }
  const int cluster_n = add_source_cluster_n(H);
  const int hpc = H / cluster_n;
  const int tpr = threads_per_row(hpc);
  if (cluster_n > 1 && tpr != 128 && tpr != 256) {
    set_error("b2_add_rmsnorm_fp4quant: H=%d: unexpected cluster configuration", H);
    return B2_ERR_UNSUPPORTED;
  }
  AddRmsParams p;
  p.x = static_cast<const uint8_t*>(x);
  p.residual = static_cast<uint8_t*>(residual);
  p.w = static_cast<const uint8_t*>(w);
  p.y = static_cast<uint8_t*>(y);
  p.sf = static_cast<uint8_t*>(sf);
  p.sf_linear = static_cast<uint8_t*>(sf_unswizzled);
  p.y_norm = static_cast<uint8_t*>(y_norm);
  p.gs = gs_dev;
  p.M = M;
  p.H = H;
  p.vb = std::max(1, ((hpc / 8) + tpr - 1) / tpr);
  p.block_size = block_size;
  p.use_e4m3 = use_e4m3 ? 1 : 0;
  p.sf_swizzled = (swizzled || output_both_sf_layouts) ? 1 : 0;
  p.both = output_both_sf_layouts ? 1 : 0;
  p.norm = output_norm ? 1 : 0;
  p.sf_cols = H / block_size;
  p.sf_pad_cols = (p.sf_cols + 3) / 4 * 4;
  p.pow2 = (H & (H - 1)) == 0;
  p.eps = eps;
  p.inv_h = 1.0f / static_cast<float>(H);
  p.enable_pdl = enable_pdl ? 1 : 0;
  p.stagger_ns = 0;
  p.first_ctas = 0;
  p.sm_count = 1;
  if (static_cast<int64_t>(M) * cluster_n > 2147483647ll) {
    set_error("b2_add_rmsnorm_fp4quant: M=%d x cluster %d exceeds the grid limit", M, cluster_n);
    return B2_ERR_UNSUPPORTED;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (in_dtype == B2_DTYPE_F16)
    return block_size == 16 ? dispatch<F16Tag, 16>(p, tpr, cluster_n, s) : dispatch<F16Tag, 32>(p, tpr, cluster_n, s);
  return block_size == 16 ? dispatch<BF16Tag, 16>(p, tpr, cluster_n, s) : dispatch<BF16Tag, 32>(p, tpr, cluster_n, s);
}
