// Host-side plumbing shared by every entry point: the thread-local error string,
// the per-device SM-count cache, and the MUFU probe used by the test oracle.
#include <cstdarg>
#include <cstdio>
#include <mutex>

#include "common.cuh"

namespace b2 {

namespace {
thread_local char g_error[512] = "";
}

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

int cuda_fail(cudaError_t err, const char* what) {
  set_error("CUDA error %d (%s) in %s", static_cast<int>(err), cudaGetErrorString(err), what);
  return B2_ERR_CUDA;
}

int device_sm_count() {
  static std::mutex mu;
  static int cache[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    set_error("cudaGetDevice failed");
    return -1;
  }
  std::lock_guard<std::mutex> lock(mu);
  if (cache[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) {
      set_error("cudaDeviceGetAttribute(MultiProcessorCount) failed");
      return -1;
    }
    cache[dev] = n;
  }
  return cache[dev];
}

namespace {
__global__ void mufu_probe_kernel(int op, const float* __restrict__ in, float* __restrict__ out,
                                  int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float x = in[i];
  float r;
  switch (op) {
    case B2_MUFU_RCP_FTZ: r = rcp_approx_ftz(x); break;
    case B2_MUFU_RSQRT_FTZ: r = rsqrt_approx_ftz(x); break;
    case B2_MUFU_LG2: r = lg2_approx(x); break;
    case B2_MUFU_EX2: r = ex2_approx(x); break;
    case B2_PROBE_SILU: r = silu_f32x2<false>(make_float2(x, x)).x; break;
    case B2_PROBE_SILU_DIV_RN: r = silu_f32x2<true>(make_float2(x, x)).x; break;
    default: r = ex2_approx_ftz(x); break;
  }
  out[i] = r;
}
}  // namespace

}  // namespace b2

extern "C" const char* b2_last_error(void) { return b2::g_error; }

extern "C" int b2_abi_version(void) { return 1; }

extern "C" int b2_mufu_probe(int op, const float* in_dev, float* out_dev, int n, void* stream) {
  using namespace b2;
  if (op < B2_MUFU_RCP_FTZ || op > B2_PROBE_SILU_DIV_RN) {
    set_error("b2_mufu_probe: unknown op %d", op);
    return B2_ERR_INVALID_ARGUMENT;
  }
  if (n < 0 || (n > 0 && (!in_dev || !out_dev))) {
    set_error("b2_mufu_probe: bad buffer arguments");
    return B2_ERR_INVALID_ARGUMENT;
  }
  if (n == 0) return B2_OK;
  mufu_probe_kernel<<<(n + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(op, in_dev,
                                                                                    out_dev, n);
  B2_CUDA_TRY(cudaGetLastError());
  return B2_OK;
}
