// RMSNorm fused with FP4 block quantization for sm_100a.
//
// Bit parity with tirx_kernels/flashinfer/norm/rmsnorm_fp4quant.py requires the fp32
// sum of squares to be accumulated in exactly the reference's order (kernel_body
// :786-900): with tpr = threads_per_row(H) (:344-355), virtual thread t owns the
// 8-element chunks t, t+tpr, t+2*tpr, ... of its row and adds their squares one by
// one; partial sums are combined by an XOR butterfly inside the warp and, for rows
// wider than a warp, by a second butterfly over the per-warp partials.  This kernel
// keeps that tree and changes the data movement: the row is read from HBM exactly
// once with 128-bit loads and parked in shared memory; the quantization pass reads it
// back from there with one thread per scale block (no shuffles, the scale computed
// once per block) and writes packed output as coalesced 64-bit words.  The kernel is
// bound by instruction issue as much as by HBM, so squares are accumulated with FMA
// (bit-identical here, the squares being exact in fp32) and the scaling multiplies
// use the two-wide mul.f32x2.
#include <algorithm>
#include <atomic>
#include <cstdlib>

#include "common.cuh"
#include "norm_quant.cuh"

namespace b2 {
namespace {

struct RmsParams {
  const uint8_t* x;
  const uint8_t* w;
  uint8_t* y;
  uint8_t* sf;
  const float* gs;
  int M;
  int H;
  int vb;            // chunks of 8 values per virtual thread
  int block_size;    // 16 or 32
  int use_e4m3;      // E4M3 scales under a global scale, else UE8M0
  int swizzled;
  int sf_cols;       // H / block_size
  int sf_pad_cols;   // sf_cols rounded up to 4
  int pow2;          // H is a power of two
  float eps;
  float inv_h;       // 1.0f / H (exact when pow2)
  int enable_pdl;
  int prefetch_ctas;  // block-owner kernel: look-ahead distance in CTAs (0 = no prefetch)
  int stagger_ns;     // block-owner kernel: start offset between the CTAs that share an SM at launch (0 = none)
  int first_ctas;     // CTAs resident at launch (they are the ones that get an offset)
  int sm_count;
  int stagger_free;   // CTAs per SM that start at once
  int stagger_first;  // offset of the first delayed CTA of an SM (-1: same as stagger_ns)
  unsigned long long* timeline;  // block-owner kernel: per CTA {start, rows reduced, end} in ns and the SM id; null = off
};

__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// acc + x*x for eight values in element order.  The square of a bf16/fp16 value is exact in fp32,
// so one FMA per element rounds exactly like the reference's mul.f32 followed by add.f32.
template <typename Tag>
__device__ __forceinline__ float sum_sq_8(float acc, const uint4& c) {
  const uint32_t w[4] = {c.x, c.y, c.z, c.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float lo = unpack_lo<Tag>(w[i]), hi = unpack_hi<Tag>(w[i]);
    acc = __fmaf_rn(lo, lo, acc);
    acc = __fmaf_rn(hi, hi, acc);
  }
  return acc;
}

// Eight products p (packed pairs) -> eight E2M1 nibbles of (p * rstd) * out_scale.
template <typename Tag>
__device__ __forceinline__ uint32_t quantize_8(const uint32_t (&prod)[4], float rstd, float out_scale) {
  const float2 r2 = make_float2(rstd, rstd), o2 = make_float2(out_scale, out_scale);
  float v[8];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 q = mul_f32x2(mul_f32x2(unpack2<Tag>(prod[i]), r2), o2);
    v[2 * i] = q.x;
    v[2 * i + 1] = q.y;
  }
  return cvt_e2m1x8(v);
}

template <typename Tag, int TPR, int BLOCK>
__global__ void __launch_bounds__(TPR == 256 ? 256 : 128)
    rmsnorm_fp4quant_kernel(const __grid_constant__ RmsParams p) {
  constexpr int kThreads = TPR == 256 ? 256 : 128;
  constexpr int kRows = kThreads / TPR;
  constexpr int kWarpsPerRow = TPR >= 32 ? TPR / 32 : 1;
  constexpr int kChunksPerBlock = BLOCK / 8;  // 16-byte chunks per scale block
  extern __shared__ __align__(16) uint8_t smem[];
  uint4* tile = reinterpret_cast<uint4*>(smem);  // [kRows][vb * TPR] chunks of 8 values, row-contiguous
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

  const float rcp6 = rcp_approx_ftz(6.0f);
  const uint4* xrow = reinterpret_cast<const uint4*>(p.x + static_cast<int64_t>(row) * p.H * 2);
  uint4* my_row = tile + static_cast<size_t>(row_in_cta) * p.vb * TPR;

  // ---- pass 1: one HBM read of the row; virtual thread t adds chunks t, t+TPR, ... in order ----
  float sum = 0.0f;
  for (int b0 = 0; b0 < p.vb; b0 += 4) {
    uint4 c[4];
    bool ok[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int chunk = t + (b0 + j) * TPR;
      ok[j] = row_valid && (b0 + j) < p.vb && chunk < nchunks;
      if (ok[j]) {
        uint32_t r[4];
        ld_stream_128(xrow + chunk, r);
        c[j] = make_uint4(r[0], r[1], r[2], r[3]);
      }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (ok[j]) {
        my_row[t + (b0 + j) * TPR] = c[j];
        sum = sum_sq_8<Tag>(sum, c[j]);
      }
    }
  }
#pragma unroll
  for (int x = 1; x < (TPR < 32 ? TPR : 32); x <<= 1) {
    sum = add_f32(sum, __shfl_xor_sync(0xFFFFFFFFu, sum, x));
  }
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
    __syncthreads();  // pass 2 reads chunks other threads of the row parked
  }
  const float shifted =
      p.pow2 ? __fmaf_rn(sum, p.inv_h, p.eps) : add_f32(__fdiv_rn(sum, static_cast<float>(p.H)), p.eps);
  const float rstd = rsqrt_approx_ftz(shifted);
  const float gs = p.use_e4m3 ? *p.gs : 0.0f;
  if (!row_valid) return;

  // ---- pass 2: one thread per scale block, from the shared-memory copy ----
  const uint4* wrow = reinterpret_cast<const uint4*>(p.w);
  uint8_t* yrow = p.y + static_cast<int64_t>(row) * (p.H >> 1);
  // byte offset of scale (row, 0); scale (row, j) lives at + j (linear) or + (j >> 2) * 512 + (j & 3)
  const int64_t sf_row = p.swizzled ? sf_offset_128x4(row, 0, p.sf_pad_cols) : static_cast<int64_t>(row) * p.sf_cols;
  uint8_t* sf_base = p.sf + sf_row;
  for (int j = t; j < p.sf_cols; j += TPR) {
    uint32_t prod[kChunksPerBlock][4];
#pragma unroll
    for (int c = 0; c < kChunksPerBlock; ++c) {
      const uint4 xc = my_row[j * kChunksPerBlock + c];
      const uint4 wc = __ldg(wrow + j * kChunksPerBlock + c);
      prod[c][0] = hmul2<Tag>(xc.x, wc.x);
      prod[c][1] = hmul2<Tag>(xc.y, wc.y);
      prod[c][2] = hmul2<Tag>(xc.z, wc.z);
      prod[c][3] = hmul2<Tag>(xc.w, wc.w);
    }
    uint32_t m2 = absmax_4<Tag>(prod[0]);
#pragma unroll
    for (int c = 1; c < kChunksPerBlock; ++c) m2 = hmax2<Tag>(m2, absmax_4<Tag>(prod[c]));
    const float max_abs = mul_f32(pair_max_to_f32<Tag>(m2), rstd);
    uint32_t code;
    float out_scale;
    if (p.use_e4m3) {
      const float s = min_f32(mul_f32(mul_f32(gs, max_abs), rcp6), 448.0f);
      code = cvt_f32_to_e4m3(s) & 0xFFu;
      const float d = e4m3_to_f32(code);
      const float r = rcp_approx_ftz(d);
      out_scale = mul_f32(d == 0.0f ? 0.0f : r, gs);
    } else {
      code = cvt_f32_to_ue8m0(mul_f32(max_abs, rcp6));
      out_scale = ue8m0_to_output_scale(code);
    }
    uint32_t q[kChunksPerBlock];
#pragma unroll
    for (int c = 0; c < kChunksPerBlock; ++c) q[c] = quantize_8<Tag>(prod[c], rstd, out_scale);
    if constexpr (kChunksPerBlock == 2) {
      *reinterpret_cast<uint2*>(yrow + j * 8) = make_uint2(q[0], q[1]);
    } else {
      *reinterpret_cast<uint4*>(yrow + j * 16) = make_uint4(q[0], q[1], q[2], q[3]);
    }
    sf_base[p.swizzled ? ((j >> 2) * 512 + (j & 3)) : j] = static_cast<uint8_t>(code);
  }
  if (p.enable_pdl) pdl_launch_dependents();
}

// Register-resident variant for rows that split evenly over the virtual threads
// (H / 8 == vb * TPR, vb <= VBMAX, TPR >= 32): thread t keeps its chunks t, t + TPR, ... in
// registers from the single HBM read, adds their squares in the reference's order, and later
// quantizes the very same chunks, so the row never visits shared memory.  A scale block is 2 (or
// 4) consecutive chunks, which sit in adjacent lanes: the block maximum is combined with one (two)
// XOR shuffles of the packed pair maximum, each lane derives the same scale and quantizes its own
// eight values to one 32-bit word, and the first lane of a block stores the scale byte.
template <typename Tag, int TPR, int BLOCK, int VBMAX>
__global__ void __launch_bounds__(TPR == 256 ? 256 : 128)
    rmsnorm_fp4quant_reg_kernel(const __grid_constant__ RmsParams p) {
  constexpr int kThreads = TPR == 256 ? 256 : 128;
  constexpr int kRows = kThreads / TPR;
  constexpr int kWarpsPerRow = TPR / 32;
  constexpr int kLanesPerBlock = BLOCK / 8;
  __shared__ float red[kRows * kWarpsPerRow];

  const int tid = threadIdx.x;
  const int row_in_cta = tid / TPR;
  const int t = tid % TPR;
  const int row = blockIdx.x * kRows + row_in_cta;
  const bool row_valid = row < p.M;  // uniform within a warp: a warp never spans two rows
  const int lane = tid & 31;
  const int warp = tid >> 5;

  if (p.enable_pdl) pdl_wait();

  const float rcp6 = rcp_approx_ftz(6.0f);
  const uint4* xrow = reinterpret_cast<const uint4*>(p.x + static_cast<int64_t>(row) * p.H * 2);
  uint4 c[VBMAX];
#pragma unroll
  for (int b = 0; b < VBMAX; ++b) {
    if (row_valid && b < p.vb) {
      uint32_t r[4];
      ld_stream_128(xrow + t + b * TPR, r);
      c[b] = make_uint4(r[0], r[1], r[2], r[3]);
    } else {
      c[b] = make_uint4(0u, 0u, 0u, 0u);
    }
  }
  float sum = 0.0f;
#pragma unroll
  for (int b = 0; b < VBMAX; ++b)
    if (b < p.vb) sum = sum_sq_8<Tag>(sum, c[b]);
#pragma unroll
  for (int x = 1; x < 32; x <<= 1) sum = add_f32(sum, __shfl_xor_sync(0xFFFFFFFFu, sum, x));
  if constexpr (kWarpsPerRow > 1) {
    const int row_warp = warp / kWarpsPerRow;
    const int warp_in_row = warp % kWarpsPerRow;
    if (lane == 0) red[row_warp + warp_in_row * kRows] = sum;
    __syncthreads();
    float part = lane < kWarpsPerRow ? red[row_warp + lane * kRows] : 0.0f;
#pragma unroll
    for (int x = 1; x < 32; x <<= 1) part = add_f32(part, __shfl_xor_sync(0xFFFFFFFFu, part, x));
    sum = part;
  }
  if (!row_valid) return;
  const float shifted =
      p.pow2 ? __fmaf_rn(sum, p.inv_h, p.eps) : add_f32(__fdiv_rn(sum, static_cast<float>(p.H)), p.eps);
  const float rstd = rsqrt_approx_ftz(shifted);
  const float gs = p.use_e4m3 ? *p.gs : 0.0f;

  const uint4* wrow = reinterpret_cast<const uint4*>(p.w);
  uint32_t* yrow = reinterpret_cast<uint32_t*>(p.y + static_cast<int64_t>(row) * (p.H >> 1));
  const int64_t sf_row = p.swizzled ? sf_offset_128x4(row, 0, p.sf_pad_cols) : static_cast<int64_t>(row) * p.sf_cols;
  uint8_t* sf_base = p.sf + sf_row;
#pragma unroll
  for (int b = 0; b < VBMAX; ++b) {
    if (b < p.vb) {
      const int chunk = t + b * TPR;
      const uint4 wc = __ldg(wrow + chunk);
      uint32_t prod[4];
      prod[0] = hmul2<Tag>(c[b].x, wc.x);
      prod[1] = hmul2<Tag>(c[b].y, wc.y);
      prod[2] = hmul2<Tag>(c[b].z, wc.z);
      prod[3] = hmul2<Tag>(c[b].w, wc.w);
      uint32_t m2 = absmax_4<Tag>(prod);
      m2 = hmax2<Tag>(m2, __shfl_xor_sync(0xFFFFFFFFu, m2, 1));
      if constexpr (kLanesPerBlock == 4) m2 = hmax2<Tag>(m2, __shfl_xor_sync(0xFFFFFFFFu, m2, 2));
      const float max_abs = mul_f32(pair_max_to_f32<Tag>(m2), rstd);
      uint32_t code;
      float out_scale;
      if (p.use_e4m3) {
        const float s = min_f32(mul_f32(mul_f32(gs, max_abs), rcp6), 448.0f);
        code = cvt_f32_to_e4m3(s) & 0xFFu;
        const float d = e4m3_to_f32(code);
        const float r = rcp_approx_ftz(d);
        out_scale = mul_f32(d == 0.0f ? 0.0f : r, gs);
      } else {
        code = cvt_f32_to_ue8m0(mul_f32(max_abs, rcp6));
        out_scale = ue8m0_to_output_scale(code);
      }
      yrow[chunk] = quantize_8<Tag>(prod, rstd, out_scale);
      if ((t & (kLanesPerBlock - 1)) == 0) {
        const int j = chunk / kLanesPerBlock;
        sf_base[p.swizzled ? ((j >> 2) * 512 + (j & 3)) : j] = static_cast<uint8_t>(code);
      }
    }
  }
  if (p.enable_pdl) pdl_launch_dependents();
}

// Block-owner variant of the register-resident kernel: one physical thread plays V = BLOCK / 8
// adjacent virtual threads (v = V*q + i), so the chunks it owns for a given b, V*q + i + b*TPR, are
// the V consecutive chunks of ONE scale block.  It keeps V running sums, combines them as the
// first log2(V) butterfly steps would (lane l and l^1 both end up with s_l + s_(l^1)), and continues
// the butterfly over the remaining lane bits with shuffles among the 32 / V physical lanes that
// stand for one virtual warp.  The quantization pass then needs no shuffle at all: every thread
// scales and packs whole blocks (one 256-bit load, one 64-bit store, one scale byte each).
// Requires H / 8 == vb * TPR, V * vb <= 16, TPR >= 32.
template <typename Tag, int TPR, int BLOCK, int VBMAX>
__global__ void __launch_bounds__(128) rmsnorm_fp4quant_block_kernel(const __grid_constant__ RmsParams p) {
  constexpr int V = BLOCK / 8;
  // The 7- and 8-block instantiations are only launched for rows of exactly that many blocks per
  // thread: without the per-block predicate the compiler interleaves the blocks (80 registers instead
  // of 72 at seven blocks, six CTAs per SM instead of seven) and the kernel still gains 6 %.
  constexpr bool kExact = V == 2 && (VBMAX == 7 || VBMAX == 8);
  constexpr int kThreads = 128;
  constexpr int P = TPR / V;                   // physical threads per row
  constexpr int kRows = kThreads / P;          // rows per CTA
  constexpr int kVWarpsPerRow = TPR / 32;      // virtual warps per row
  constexpr int kLanesPerVWarp = 32 / V;       // physical lanes standing for one virtual warp
  __shared__ float red[kRows * kVWarpsPerRow];

  const int tid = threadIdx.x;
  const int row_in_cta = tid / P;
  const int q = tid % P;
  const int row = blockIdx.x * kRows + row_in_cta;
  const bool row_valid = row < p.M;
  const int lane = tid & 31;

  if (p.timeline && tid == 0) {
    unsigned int sm;
    asm volatile("mov.u32 %0, %%smid;" : "=r"(sm));
    p.timeline[blockIdx.x * 4 + 0] = global_timer_ns();
    p.timeline[blockIdx.x * 4 + 3] = sm;
  }
  if (p.enable_pdl) pdl_wait();
  // The CTAs that become resident at launch would all load for the same few microseconds and then all
  // compute, with HBM idle meanwhile.  Later CTAs start whenever an earlier one leaves and are spread out
  // by themselves; the first ones are spread out here: the k-th CTA of an SM starts k * stagger_ns late.
  if (p.stagger_ns > 0 && static_cast<int>(blockIdx.x) < p.first_ctas) {
    const int slot = static_cast<int>(blockIdx.x) / p.sm_count;
    unsigned long long wait_ns = slot < p.stagger_free ? 0ull : static_cast<unsigned long long>(slot - p.stagger_free + 1) * p.stagger_ns;
    if (p.stagger_first >= 0 && slot >= p.stagger_free) wait_ns = p.stagger_first + static_cast<unsigned long long>(slot - p.stagger_free) * p.stagger_ns;
    // timed by the global timer, and bounded by a count of short sleeps whatever that timer does
    const unsigned long long t0 = global_timer_ns();
    for (unsigned long long i = 0; i < wait_ns / 32 + 8 && global_timer_ns() - t0 < wait_ns; ++i) __nanosleep(64);
  }
  const float rcp6 = rcp_approx_ftz(6.0f);
  const uint8_t* xrow = p.x + static_cast<int64_t>(row) * p.H * 2;
  uint32_t c[VBMAX][V * 4];  // block b of this thread: chunks V*q + i + b*TPR, i < V
#pragma unroll
  for (int b = 0; b < VBMAX; ++b) {
    if (row_valid && (kExact || b < p.vb)) {
      const uint8_t* src = xrow + static_cast<int64_t>(V * q + b * TPR) * 16;
      if constexpr (V == 2) {
        uint32_t r[8];
        ld_stream_256(src, r);
#pragma unroll
        for (int i = 0; i < 8; ++i) c[b][i] = r[i];
      } else {
        uint32_t r0[8], r1[8];
        ld_stream_256(src, r0);
        ld_stream_256(src + 32, r1);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          c[b][i] = r0[i];
          c[b][8 + i] = r1[i];
        }
      }
    } else {
#pragma unroll
      for (int i = 0; i < V * 4; ++i) c[b][i] = 0u;
    }
  }
  // The weights are needed only after the reduction; asking L2 for them now takes a cold miss off the
  // critical path of a small launch (32 x 4096 with cold caches: 7.4 -> 5.3 us).  Only where all CTAs run at
  // once: thousands of CTAs asking for the same 14 KB cost a large launch 25 %.
  if (static_cast<int>(gridDim.x) <= p.first_ctas) {
#pragma unroll
    for (int b = 0; b < VBMAX; ++b) {
      if (kExact || b < p.vb)
        asm volatile("prefetch.global.L2 [%0];" ::"l"(p.w + static_cast<int64_t>(q + b * P) * V * 16));
    }
  }
  // Look-ahead: ask L2 for the rows of a CTA that starts about half a generation of resident CTAs
  // later.  Its own loads then find their lines in L2 (or on their way) instead of waiting a full
  // DRAM round trip with 56 registers per thread tied up.
  if (p.prefetch_ctas > 0) {
    const int64_t cta_bytes = static_cast<int64_t>(kRows) * p.H * 2;
    const int64_t first = (static_cast<int64_t>(blockIdx.x) + p.prefetch_ctas) * cta_bytes;
    const int64_t end = static_cast<int64_t>(p.M) * p.H * 2;
    for (int64_t off = first + static_cast<int64_t>(tid) * 128; off < first + cta_bytes && off < end;
         off += kThreads * 128)
      asm volatile("prefetch.global.L2 [%0];" ::"l"(p.x + off));
  }
  // The V running sums advance in lock step, two per fma.rn.f32x2: the same chain of roundings per sum as
  // one fma.rn.f32 per element, at half the instructions.
  float acc[V];
#pragma unroll
  for (int i = 0; i < V; ++i) acc[i] = 0.0f;
#pragma unroll
  for (int b = 0; b < VBMAX; ++b) {
    if (kExact || b < p.vb) {
#pragma unroll
      for (int pair = 0; pair < V; pair += 2) {
        float2 a2 = make_float2(acc[pair], acc[pair + 1]);
#pragma unroll
        for (int wi = 0; wi < 4; ++wi) {
          const uint32_t w0 = c[b][4 * pair + wi], w1 = c[b][4 * (pair + 1) + wi];
          const float2 lo = make_float2(unpack_lo<Tag>(w0), unpack_lo<Tag>(w1));
          a2 = fma_f32x2(lo, lo, a2);
          const float2 hi = make_float2(unpack_hi<Tag>(w0), unpack_hi<Tag>(w1));
          a2 = fma_f32x2(hi, hi, a2);
        }
        acc[pair] = a2.x;
        acc[pair + 1] = a2.y;
      }
    }
  }
  float sum = add_f32(acc[0], acc[1]);
  if constexpr (V == 4) sum = add_f32(sum, add_f32(acc[2], acc[3]));
#pragma unroll
  for (int x = 1; x < kLanesPerVWarp; x <<= 1) sum = add_f32(sum, __shfl_xor_sync(0xFFFFFFFFu, sum, x));
  if constexpr (kVWarpsPerRow > 1) {
    // virtual warp w of the row = physical lanes [w * kLanesPerVWarp, ...) of the row's threads
    const int vwarp = q / kLanesPerVWarp;
    if (q % kLanesPerVWarp == 0) red[row_in_cta * kVWarpsPerRow + vwarp] = sum;
    __syncthreads();
    float part = lane < kVWarpsPerRow ? red[row_in_cta * kVWarpsPerRow + lane] : 0.0f;
    if constexpr (P < 32) {
      // several rows share this physical warp: every lane reads its own row's partials
      part = (lane % P) < kVWarpsPerRow ? red[row_in_cta * kVWarpsPerRow + (lane % P)] : 0.0f;
    }
#pragma unroll
    for (int x = 1; x < 32; x <<= 1) {
      if (P >= 32 || x < P) part = add_f32(part, __shfl_xor_sync(0xFFFFFFFFu, part, x));
      else part = add_f32(part, 0.0f);  // lanes past the row's partials hold zero in the reference
    }
    sum = part;
  }
  const float shifted =
      p.pow2 ? __fmaf_rn(sum, p.inv_h, p.eps) : add_f32(__fdiv_rn(sum, static_cast<float>(p.H)), p.eps);
  const float rstd = rsqrt_approx_ftz(shifted);
  const float gs = p.use_e4m3 ? *p.gs : 0.0f;
  if (p.timeline && tid == 0) p.timeline[blockIdx.x * 4 + 1] = global_timer_ns();
  if (!row_valid) return;

  const uint8_t* wbase = p.w;
  uint8_t* yrow = p.y + static_cast<int64_t>(row) * (p.H >> 1);
  const int64_t sf_row = p.swizzled ? sf_offset_128x4(row, 0, p.sf_pad_cols) : static_cast<int64_t>(row) * p.sf_cols;
  uint8_t* sf_base = p.sf + sf_row;
#pragma unroll
  for (int b = 0; b < VBMAX; ++b) {
    if (kExact || b < p.vb) {
      const int j = q + b * P;  // scale block index in the row
      uint32_t prod[V][4];
#pragma unroll
      for (int i = 0; i < V; ++i) {
        const uint4 wc = __ldg(reinterpret_cast<const uint4*>(wbase) + j * V + i);
        prod[i][0] = hmul2<Tag>(c[b][4 * i], wc.x);
        prod[i][1] = hmul2<Tag>(c[b][4 * i + 1], wc.y);
        prod[i][2] = hmul2<Tag>(c[b][4 * i + 2], wc.z);
        prod[i][3] = hmul2<Tag>(c[b][4 * i + 3], wc.w);
      }
      uint32_t m2 = absmax_4<Tag>(prod[0]);
#pragma unroll
      for (int i = 1; i < V; ++i) m2 = hmax2<Tag>(m2, absmax_4<Tag>(prod[i]));
      const float max_abs = mul_f32(pair_max_to_f32<Tag>(m2), rstd);
      uint32_t code;
      float out_scale;
      if (p.use_e4m3) {
        const float sc = min_f32(mul_f32(mul_f32(gs, max_abs), rcp6), 448.0f);
        code = cvt_f32_to_e4m3(sc) & 0xFFu;
        const float d = e4m3_to_f32(code);
        const float r = rcp_approx_ftz(d);
        out_scale = mul_f32(d == 0.0f ? 0.0f : r, gs);
      } else {
        code = cvt_f32_to_ue8m0(mul_f32(max_abs, rcp6));
        out_scale = ue8m0_to_output_scale(code);
      }
      uint32_t qv[V];
#pragma unroll
      for (int i = 0; i < V; ++i) qv[i] = quantize_8<Tag>(prod[i], rstd, out_scale);
      if constexpr (V == 2) {
        *reinterpret_cast<uint2*>(yrow + j * 8) = make_uint2(qv[0], qv[1]);
      } else {
        *reinterpret_cast<uint4*>(yrow + j * 16) = make_uint4(qv[0], qv[1], qv[2], qv[3]);
      }
      sf_base[p.swizzled ? ((j >> 2) * 512 + (j & 3)) : j] = static_cast<uint8_t>(code);
    }
  }
  if (p.enable_pdl) pdl_launch_dependents();
  if (p.timeline && tid == 0) p.timeline[blockIdx.x * 4 + 2] = global_timer_ns();
}

// ---- rows spread over a thread-block cluster (rmsnorm_fp4quant.py kernel_body :857-891) ----------
// When one CTA cannot hold a row, the reference gives CTA c of a cluster the columns
// [c * cols, (c + 1) * cols), lets every warp of every CTA publish its partial sum at index
// c * warps_per_row + warp in all CTAs of the cluster, and has each lane add partials lane,
// lane + 32, ... before the final butterfly.  Same here: 256 threads per CTA, one row per cluster,
// partials written into every CTA's shared memory through distributed shared memory, one
// hardware cluster barrier, then the quantization pass over this CTA's own columns.
template <typename Tag, int BLOCK>
__global__ void __launch_bounds__(256) rmsnorm_fp4quant_cluster_kernel(const __grid_constant__ RmsParams p, int cluster_n) {
  constexpr int kTpr = 256, kWarps = 8;
  constexpr int kChunksPerBlock = BLOCK / 8;
  extern __shared__ __align__(16) uint8_t smem[];
  uint4* tile = reinterpret_cast<uint4*>(smem);  // this CTA's vb * 256 chunks
  float* partials = reinterpret_cast<float*>(smem + static_cast<size_t>(p.vb) * kTpr * 16);  // [cluster_n * 8]

  const int t = threadIdx.x;
  const int lane = t & 31, warp = t >> 5;
  const int cta = static_cast<int>(cluster_rank());
  const int row = blockIdx.x / cluster_n;  // < M by construction of the grid
  const int nchunks = p.H >> 3;
  const int chunk0 = cta * p.vb * kTpr;  // first chunk of this CTA's column range

  if (p.enable_pdl) pdl_wait();
  const float rcp6 = rcp_approx_ftz(6.0f);
  const uint4* xrow = reinterpret_cast<const uint4*>(p.x + static_cast<int64_t>(row) * p.H * 2);

  float sum = 0.0f;
  for (int b0 = 0; b0 < p.vb; b0 += 4) {
    uint4 c[4];
    bool ok[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int local = t + (b0 + j) * kTpr;
      ok[j] = (b0 + j) < p.vb && chunk0 + local < nchunks;
      if (ok[j]) {
        uint32_t r[4];
        ld_stream_128(xrow + chunk0 + local, r);
        c[j] = make_uint4(r[0], r[1], r[2], r[3]);
      }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (ok[j]) {
        tile[t + (b0 + j) * kTpr] = c[j];
        sum = sum_sq_8<Tag>(sum, c[j]);
      }
    }
  }
#pragma unroll
  for (int x = 1; x < 32; x <<= 1) sum = add_f32(sum, __shfl_xor_sync(0xFFFFFFFFu, sum, x));
  if (lane < cluster_n) st_cluster_f32(partials + cta * kWarps + warp, static_cast<uint32_t>(lane), sum);
  cluster_barrier();  // every partial of the row is in this CTA's shared memory; also orders `tile`
  const int total = cluster_n * kWarps;
  float part = 0.0f;
  for (int i = lane; i < total; i += 32) part = add_f32(part, partials[i]);
#pragma unroll
  for (int x = 1; x < 32; x <<= 1) part = add_f32(part, __shfl_xor_sync(0xFFFFFFFFu, part, x));
  const float shifted =
      p.pow2 ? __fmaf_rn(part, p.inv_h, p.eps) : add_f32(__fdiv_rn(part, static_cast<float>(p.H)), p.eps);
  const float rstd = rsqrt_approx_ftz(shifted);
  const float gs = p.use_e4m3 ? *p.gs : 0.0f;

  const uint4* wrow = reinterpret_cast<const uint4*>(p.w);
  uint8_t* yrow = p.y + static_cast<int64_t>(row) * (p.H >> 1);
  const int64_t sf_row = p.swizzled ? sf_offset_128x4(row, 0, p.sf_pad_cols) : static_cast<int64_t>(row) * p.sf_cols;
  uint8_t* sf_base = p.sf + sf_row;
  const int blocks_here = p.vb * kTpr / kChunksPerBlock;
  const int block0 = chunk0 / kChunksPerBlock;
  for (int jl = t; jl < blocks_here; jl += kTpr) {
    const int j = block0 + jl;
    if (j >= p.sf_cols) break;
    uint32_t prod[kChunksPerBlock][4];
#pragma unroll
    for (int c = 0; c < kChunksPerBlock; ++c) {
      const uint4 xc = tile[jl * kChunksPerBlock + c];
      const uint4 wc = __ldg(wrow + j * kChunksPerBlock + c);
      prod[c][0] = hmul2<Tag>(xc.x, wc.x);
      prod[c][1] = hmul2<Tag>(xc.y, wc.y);
      prod[c][2] = hmul2<Tag>(xc.z, wc.z);
      prod[c][3] = hmul2<Tag>(xc.w, wc.w);
    }
    uint32_t m2 = absmax_4<Tag>(prod[0]);
#pragma unroll
    for (int c = 1; c < kChunksPerBlock; ++c) m2 = hmax2<Tag>(m2, absmax_4<Tag>(prod[c]));
    const float max_abs = mul_f32(pair_max_to_f32<Tag>(m2), rstd);
    uint32_t code;
    float out_scale;
    if (p.use_e4m3) {
      const float sc = min_f32(mul_f32(mul_f32(gs, max_abs), rcp6), 448.0f);
      code = cvt_f32_to_e4m3(sc) & 0xFFu;
      const float d = e4m3_to_f32(code);
      const float r = rcp_approx_ftz(d);
      out_scale = mul_f32(d == 0.0f ? 0.0f : r, gs);
    } else {
      code = cvt_f32_to_ue8m0(mul_f32(max_abs, rcp6));
      out_scale = ue8m0_to_output_scale(code);
    }
    uint32_t q[kChunksPerBlock];
#pragma unroll
    for (int c = 0; c < kChunksPerBlock; ++c) q[c] = quantize_8<Tag>(prod[c], rstd, out_scale);
    if constexpr (kChunksPerBlock == 2) {
      *reinterpret_cast<uint2*>(yrow + j * 8) = make_uint2(q[0], q[1]);
    } else {
      *reinterpret_cast<uint4*>(yrow + j * 16) = make_uint4(q[0], q[1], q[2], q[3]);
    }
    sf_base[p.swizzled ? ((j >> 2) * 512 + (j & 3)) : j] = static_cast<uint8_t>(code);
  }
  if (p.enable_pdl) pdl_launch_dependents();
}

template <typename Tag, int BLOCK>
int launch_cluster(const RmsParams& p, int cluster_n, cudaStream_t stream) {
  auto kernel = rmsnorm_fp4quant_cluster_kernel<Tag, BLOCK>;
  const size_t smem = static_cast<size_t>(p.vb) * 256 * 16 + static_cast<size_t>(cluster_n) * 8 * 4;
  B2_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
  if (cluster_n > 8) B2_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(p.M) * cluster_n);
  cfg.blockDim = dim3(256);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cluster_n;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.numAttrs = 1;
  if (p.enable_pdl) {
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.numAttrs = 2;
  }
  cfg.attrs = attr;
  B2_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, p, cluster_n));
  return B2_OK;
}

// rmsnorm_fp4quant.py _derived_config / _estimate_smem / _source_config :358-400: the smallest
// cluster size whose per-CTA row tile fits in shared memory.
int source_cluster_n(int H) {
  for (int cand = 1; cand <= 16; cand *= 2) {
    const int hpc = H / cand;
    const int tpr = threads_per_row(hpc);
    const int threads = hpc <= 16384 ? 128 : 256;
    const int rows = threads / tpr;
    const int wpr = std::max(tpr / 32, 1);
    const int64_t vb = std::max(1, ((hpc / 8) + tpr - 1) / tpr);
    const int64_t tile = static_cast<int64_t>(rows) * 8 * vb * tpr * 2;
    const int64_t red = static_cast<int64_t>(rows) * wpr * 4;
    const int64_t est = cand == 1 ? 2 * tile + red : tile + red * cand + 8;
    if (H % cand == 0 && est <= 232448) return cand;
  }
  return 16;
}

// Tuning and test knob: B2_RMSNORM_BLOCK_OWNER=0 falls back to the per-chunk register kernel.
int g_block_owner = [] {
  const char* v = getenv("B2_RMSNORM_BLOCK_OWNER");
  return v ? atoi(v) : 1;
}();

// Tuning knob: B2_RMSNORM_PREFETCH = 0 switches the block-owner kernel's look-ahead prefetch off, N > 0
// sets its distance to N CTAs; default: half the CTAs resident on the device at once (measured at
// 8192 x 7168 with cold inputs: off 35.2 us, a quarter or half a generation 33.4-33.8 us, a whole one 36.0 us),
// a third for the rows that also get the start offset below (29.6 against 29.7 us, 34.8 against 35.2 at 8192 x 8192).
int g_prefetch = [] {
  const char* v = getenv("B2_RMSNORM_PREFETCH");
  return v ? atoi(v) : -1;
}();

// Tuning knobs: B2_RMSNORM_STAGGER_FIRST_NS / B2_RMSNORM_STAGGER_NS = when the CTAs that share an SM at launch
// start (block-owner kernel): the first at once, the second after FIRST ns, every further one NS ns later
// (NS = 0: all start together; FIRST = -1: FIRST = NS).  Default for rows of 7 or 8 scale blocks per thread in
// launches of two generations of CTAs or more: 3500 / 800, none otherwise.  Measured at 8192 x 7168 with cold
// inputs: the CTAs resident at launch all wait ~6 us for their rows (888 CTAs ask for 25 MB at once), then all
// quantize for ~4 us with HBM idle; spread out, the steady mix of loading and quantizing CTAs is reached
// earlier: 31.5 us with no offsets; a uniform offset of 800 ns 31.4, 1200 30.4, 1500 29.5, 2000 30.8; first
// 2500-3500 then 800-1000: 29.1-29.3 (letting two or three CTAs per SM start at once: no gain at any offset).
// Rows of 4096 values lose 3 % with it.
int g_stagger_ns = [] {
  const char* v = getenv("B2_RMSNORM_STAGGER_NS");
  return v ? atoi(v) : -1;
}();
int g_stagger_first_ns = [] {
  const char* v = getenv("B2_RMSNORM_STAGGER_FIRST_NS");
  return v ? atoi(v) : -2;  // -2: default
}();

// Device buffer of the per-CTA timeline (b2_rmsnorm_fp4quant_timeline); null = not recording.
std::atomic<unsigned long long*> g_timeline{nullptr};

// B2_RMSNORM_STAGGER_FREE = CTAs per SM that start without an offset (default 1).
int g_stagger_free = [] {
  const char* v = getenv("B2_RMSNORM_STAGGER_FREE");
  return v ? atoi(v) : 1;
}();

template <typename Kernel>
int launch_config(Kernel kernel, const RmsParams& p, int rows_per_cta, int threads, size_t smem, cudaStream_t stream) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((p.M + rows_per_cta - 1) / rows_per_cta);
  cfg.blockDim = dim3(threads);
  cfg.dynamicSmemBytes = smem;
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

template <typename Kernel>
int launch_block_owner(Kernel kernel, RmsParams p, int rows_per_cta, cudaStream_t stream, bool long_rows = false) {
  static int resident = 0;  // per instantiation
  if (resident == 0) {
    int per_sm = 0;
    B2_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, 128, 0));
    const int sms = device_sm_count();
    resident = std::max(2, per_sm * std::max(sms, 1));
  }
  p.prefetch_ctas = g_prefetch < 0 ? (long_rows ? resident / 3 : resident / 2) : g_prefetch;
  // (only where at least two generations of CTAs follow one another: a launch that fits the GPU at once
  // would merely start late)
  const int grid = (p.M + rows_per_cta - 1) / rows_per_cta;
  p.stagger_ns = g_stagger_ns < 0 ? (long_rows && grid >= 2 * resident ? 800 : 0) : g_stagger_ns;
  p.first_ctas = resident;
  p.stagger_free = g_stagger_free;
  p.stagger_first = g_stagger_first_ns < -1 ? (p.stagger_ns > 0 && g_stagger_ns < 0 ? 3500 : -1) : g_stagger_first_ns;
  p.timeline = g_timeline.load(std::memory_order_relaxed);
  p.sm_count = std::max(device_sm_count(), 1);
  return launch_config(kernel, p, rows_per_cta, 128, 0, stream);
}

template <typename Tag, int TPR, int BLOCK>
int launch(const RmsParams& p, cudaStream_t stream) {
  constexpr int kThreads = TPR == 256 ? 256 : 128;
  constexpr int kRows = kThreads / TPR;
  constexpr int kWarpsPerRow = TPR >= 32 ? TPR / 32 : 1;
  if constexpr (TPR >= 32) {
    constexpr int kV = BLOCK / 8;
    constexpr int kBlockVb = 16 / kV;  // blocks a thread of the block-owner kernel can hold
    if (g_block_owner && (p.H >> 3) == p.vb * TPR && p.vb <= kBlockVb &&
        (reinterpret_cast<uintptr_t>(p.x) & 31) == 0 && (p.H % 16) == 0) {
      constexpr int kP = TPR / kV;
      // the kernel is instantiated for a few block counts per thread: registers (and with them the CTAs
      // per SM) follow the row length instead of the maximum
      if constexpr (kV == 2) {
        if (p.vb <= 4) return launch_block_owner(rmsnorm_fp4quant_block_kernel<Tag, TPR, BLOCK, 4>, p, 128 / kP, stream);
        if (p.vb <= 6) return launch_block_owner(rmsnorm_fp4quant_block_kernel<Tag, TPR, BLOCK, 6>, p, 128 / kP, stream);
        if (p.vb == 7) return launch_block_owner(rmsnorm_fp4quant_block_kernel<Tag, TPR, BLOCK, 7>, p, 128 / kP, stream, TPR >= 128);
      } else {
        if (p.vb <= 2) return launch_block_owner(rmsnorm_fp4quant_block_kernel<Tag, TPR, BLOCK, 2>, p, 128 / kP, stream);
      }
      return launch_block_owner(rmsnorm_fp4quant_block_kernel<Tag, TPR, BLOCK, kBlockVb>, p, 128 / kP, stream,
                                kV == 2 && TPR >= 128 && p.vb == 8);
    }
    if ((p.H >> 3) == p.vb * TPR && p.vb <= 16) {
      if (p.vb <= 8) return launch_config(rmsnorm_fp4quant_reg_kernel<Tag, TPR, BLOCK, 8>, p, kRows, kThreads, 0, stream);
      return launch_config(rmsnorm_fp4quant_reg_kernel<Tag, TPR, BLOCK, 16>, p, kRows, kThreads, 0, stream);
    }
  }
  auto kernel = rmsnorm_fp4quant_kernel<Tag, TPR, BLOCK>;
  const size_t smem = static_cast<size_t>(kRows) * p.vb * TPR * 16 + kRows * kWarpsPerRow * 4;
  if (smem > 48 * 1024) {
    B2_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     static_cast<int>(smem)));
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((p.M + kRows - 1) / kRows);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem;
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

template <typename Tag, int BLOCK>
int dispatch_tpr(const RmsParams& p, int tpr, cudaStream_t stream) {
  switch (tpr) {
    case 8: return launch<Tag, 8, BLOCK>(p, stream);
    case 16: return launch<Tag, 16, BLOCK>(p, stream);
    case 32: return launch<Tag, 32, BLOCK>(p, stream);
    case 64: return launch<Tag, 64, BLOCK>(p, stream);
    case 128: return launch<Tag, 128, BLOCK>(p, stream);
    default: return launch<Tag, 256, BLOCK>(p, stream);
  }
}

template <typename Tag>
int dispatch_block(const RmsParams& p, int tpr, cudaStream_t stream) {
  return p.block_size == 16 ? dispatch_tpr<Tag, 16>(p, tpr, stream) : dispatch_tpr<Tag, 32>(p, tpr, stream);
}

}  // namespace
}  // namespace b2

extern "C" int b2_rmsnorm_fp4quant(const void* x, const void* w, void* y, void* sf,
                                   const float* gs_dev, int M, int H, float eps, int in_dtype,
                                   int block_size, int scale_format, int swizzled, int enable_pdl,
                                   void* stream) {
  using namespace b2;
  if (in_dtype != B2_DTYPE_F16 && in_dtype != B2_DTYPE_BF16) {
    set_error("b2_rmsnorm_fp4quant: unsupported input_dtype %d", in_dtype);
    return B2_ERR_INVALID_ARGUMENT;
  }
  if (block_size != 16 && block_size != 32) {
    set_error("b2_rmsnorm_fp4quant: unsupported block_size=%d", block_size);
    return B2_ERR_INVALID_ARGUMENT;
  }
  if (H < 64 || H % block_size != 0) {
    set_error("b2_rmsnorm_fp4quant: H=%d must be >=64 and divisible by block_size=%d", H, block_size);
    return B2_ERR_INVALID_ARGUMENT;
  }
  if (scale_format != B2_SCALE_E4M3 && scale_format != B2_SCALE_UE8M0) {
    set_error("b2_rmsnorm_fp4quant: unsupported scale_format %d", scale_format);
    return B2_ERR_INVALID_ARGUMENT;
  }
  if (M <= 0) {
    set_error("b2_rmsnorm_fp4quant: M must be positive, got %d", M);
    return B2_ERR_INVALID_ARGUMENT;
  }
  const bool use_e4m3 = block_size == 16 || scale_format == B2_SCALE_E4M3;
  if (!x || !w || !y || !sf || (use_e4m3 && !gs_dev)) {
    set_error("b2_rmsnorm_fp4quant: null pointer argument");
    return B2_ERR_INVALID_ARGUMENT;
  }
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(w) & 15) ||
      (reinterpret_cast<uintptr_t>(y) & 3)) {
    set_error("b2_rmsnorm_fp4quant: x and w must be 16-byte aligned, y 4-byte aligned");
    return B2_ERR_INVALID_ARGUMENT;
  }
  const int tpr = threads_per_row(H);
  RmsParams p;
  p.x = static_cast<const uint8_t*>(x);
  p.w = static_cast<const uint8_t*>(w);
  p.y = static_cast<uint8_t*>(y);
  p.sf = static_cast<uint8_t*>(sf);
  p.gs = gs_dev;
  p.M = M;
  p.H = H;
  p.vb = std::max(1, ((H / 8) + tpr - 1) / tpr);
  p.block_size = block_size;
  p.use_e4m3 = use_e4m3 ? 1 : 0;
  p.swizzled = swizzled ? 1 : 0;
  p.sf_cols = H / block_size;
  p.sf_pad_cols = (p.sf_cols + 3) / 4 * 4;
  p.pow2 = (H & (H - 1)) == 0;
  p.eps = eps;
  p.inv_h = 1.0f / static_cast<float>(H);
  p.enable_pdl = enable_pdl ? 1 : 0;
  p.prefetch_ctas = 0;
  p.stagger_ns = 0;
  p.first_ctas = 0;
  p.sm_count = 1;
  p.stagger_free = 1;
  p.stagger_first = -1;
  p.timeline = nullptr;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int cluster_n = source_cluster_n(H);
  if (cluster_n > 1) {
    // one CTA cannot hold the row: spread it over a cluster, as the reference does
    const int hpc = H / cluster_n;
    if (threads_per_row(hpc) != 256) {
      set_error("b2_rmsnorm_fp4quant: H=%d: unexpected cluster configuration", H);
      return B2_ERR_UNSUPPORTED;
    }
    p.vb = std::max(1, ((hpc / 8) + 255) / 256);
    if (static_cast<size_t>(p.vb) * 256 * 16 + 1024 > 232448 || static_cast<int64_t>(M) * cluster_n > 2147483647ll) {
      set_error("b2_rmsnorm_fp4quant: H=%d does not fit a cluster of 16 CTAs", H);
      return B2_ERR_UNSUPPORTED;
    }
    if (in_dtype == B2_DTYPE_F16)
      return block_size == 16 ? launch_cluster<F16Tag, 16>(p, cluster_n, s) : launch_cluster<F16Tag, 32>(p, cluster_n, s);
    return block_size == 16 ? launch_cluster<BF16Tag, 16>(p, cluster_n, s) : launch_cluster<BF16Tag, 32>(p, cluster_n, s);
  }
  if (in_dtype == B2_DTYPE_F16) return dispatch_block<F16Tag>(p, tpr, s);
  return dispatch_block<BF16Tag>(p, tpr, s);
}

// Observability: while `device_buf` is non-null, launches of the register-resident (block-owner) kernel
// record, per CTA, four 64-bit words at device_buf[4 * cta]: start, row sums reduced, end (nanoseconds of
// the GPU's global timer) and the SM the CTA ran on.  The buffer must hold 4 * ceil(M / rows per CTA)
// words (4 * M is always enough); pass null to stop recording.
extern "C" int b2_rmsnorm_fp4quant_timeline(unsigned long long* device_buf) {
  b2::g_timeline.store(device_buf, std::memory_order_relaxed);
  return B2_OK;
}
