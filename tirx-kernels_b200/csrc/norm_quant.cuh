// Device and host helpers shared by the RMSNorm-with-FP4-quantization kernels
// (rmsnorm_fp4quant.cu, add_rmsnorm_fp4quant.cu).
#pragma once

#include "common.cuh"

namespace b2 {

// rmsnorm_fp4quant.py _cvt_f32_to_ue8m0 :155-171
__device__ __forceinline__ uint32_t cvt_f32_to_ue8m0(float v) {
  const bool is_zero = v <= 0.0f;
  int r = __float2int_ru(lg2_approx(v)) + 127;
  r = r < 0 ? 0 : r;
  r = r > 255 ? 255 : r;
  return is_zero ? 0u : static_cast<uint32_t>(r);
}
// rmsnorm_fp4quant.py _ue8m0_to_output_scale :174-185
__device__ __forceinline__ float ue8m0_to_output_scale(uint32_t code) {
  const float cand = ex2_approx(__int2float_rn(127 - static_cast<int>(code)));
  return code == 0u ? 0.0f : cand;
}

// ---- thread-block cluster primitives (distributed shared memory, hardware cluster barrier) ----
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void st_cluster_f32(const float* local, uint32_t target_cta, float v) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;"
               : "=r"(remote)
               : "r"(static_cast<uint32_t>(__cvta_generic_to_shared(local))), "r"(target_cta));
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(v) : "memory");
}
__device__ __forceinline__ void cluster_barrier() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// rmsnorm_fp4quant.py _threads_per_row :344-355
inline int threads_per_row(int h) {
  if (h <= 64) return 8;
  if (h <= 128) return 16;
  if (h <= 3072) return 32;
  if (h <= 6144) return 64;
  if (h <= 16384) return 128;
  return 256;
}

}  // namespace b2
