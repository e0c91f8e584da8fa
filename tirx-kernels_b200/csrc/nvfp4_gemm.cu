// placeholder until the tcgen05 kernel lands
#include "common.cuh"
extern "C" int b2_nvfp4_gemm(const void*, const void*, const void*, const void*, const float*, void*,
                             int, int, int, void*) {
  b2::set_error("b2_nvfp4_gemm: not built yet");
  return B2_ERR_UNSUPPORTED;
}
extern "C" int b2_nvfp4_gemm_status(void*) { return B2_OK; }
