// cuBLASLt NVFP4 matmul: the NVIDIA-library peer the reference times beside its own GEMM
// (nvfp4_cublaslt, tirx_kernels/basic/nvfp4_gemm.py:113-239).  Benchmark-only; built into its
// own shared object so the product library has no cuBLAS dependency.
//
// cuBLASLt wants column-major operands, so the row-major problem D = A * B^T is posed as
// D^T (N x M, ld N) = B (op T, K x N storage) * A (op N, K x M storage), with 16-element
// UE4M3 block scales for both operands and an fp32 host alpha.
#include <cublasLt.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <map>
#include <memory>
#include <mutex>
#include <tuple>

#include "../../include/b200_nvfp4.h"

namespace {

struct Plan {
  cublasLtHandle_t handle = nullptr;
  cublasLtMatmulDesc_t op = nullptr;
  cublasLtMatrixLayout_t lay_b = nullptr, lay_a = nullptr, lay_d = nullptr;
  cublasLtMatmulPreference_t pref = nullptr;
  cublasLtMatmulHeuristicResult_t choice{};
  void* workspace = nullptr;
  size_t workspace_bytes = 128u << 20;
  bool ok = false;

  Plan(int M, int N, int K) {
    if (cublasLtCreate(&handle) != CUBLAS_STATUS_SUCCESS) return;
    if (cublasLtMatmulDescCreate(&op, CUBLAS_COMPUTE_32F, CUDA_R_32F) != CUBLAS_STATUS_SUCCESS) return;
    const cublasOperation_t tr = CUBLAS_OP_T, no = CUBLAS_OP_N;
    const cublasLtMatmulMatrixScale_t vec16 = CUBLASLT_MATMUL_MATRIX_SCALE_VEC16_UE4M3;
    bool good = true;
    good &= cublasLtMatmulDescSetAttribute(op, CUBLASLT_MATMUL_DESC_TRANSA, &tr, sizeof(tr)) == CUBLAS_STATUS_SUCCESS;
    good &= cublasLtMatmulDescSetAttribute(op, CUBLASLT_MATMUL_DESC_TRANSB, &no, sizeof(no)) == CUBLAS_STATUS_SUCCESS;
    good &= cublasLtMatmulDescSetAttribute(op, CUBLASLT_MATMUL_DESC_A_SCALE_MODE, &vec16, sizeof(vec16)) == CUBLAS_STATUS_SUCCESS;
    good &= cublasLtMatmulDescSetAttribute(op, CUBLASLT_MATMUL_DESC_B_SCALE_MODE, &vec16, sizeof(vec16)) == CUBLAS_STATUS_SUCCESS;
    good &= cublasLtMatrixLayoutCreate(&lay_b, CUDA_R_4F_E2M1, K, N, K) == CUBLAS_STATUS_SUCCESS;
    good &= cublasLtMatrixLayoutCreate(&lay_a, CUDA_R_4F_E2M1, K, M, K) == CUBLAS_STATUS_SUCCESS;
    good &= cublasLtMatrixLayoutCreate(&lay_d, CUDA_R_16BF, N, M, N) == CUBLAS_STATUS_SUCCESS;
    if (!good) return;
    if (cudaMalloc(&workspace, workspace_bytes) != cudaSuccess) return;
    // the heuristic needs non-null scale pointers to accept the block-scaled descriptor
    good &= cublasLtMatmulDescSetAttribute(op, CUBLASLT_MATMUL_DESC_A_SCALE_POINTER, &workspace, sizeof(workspace)) == CUBLAS_STATUS_SUCCESS;
    good &= cublasLtMatmulDescSetAttribute(op, CUBLASLT_MATMUL_DESC_B_SCALE_POINTER, &workspace, sizeof(workspace)) == CUBLAS_STATUS_SUCCESS;
    good &= cublasLtMatmulPreferenceCreate(&pref) == CUBLAS_STATUS_SUCCESS;
    good &= cublasLtMatmulPreferenceSetAttribute(pref, CUBLASLT_MATMUL_PREF_MAX_WORKSPACE_BYTES, &workspace_bytes,
                                                 sizeof(workspace_bytes)) == CUBLAS_STATUS_SUCCESS;
    if (!good) return;
    int found = 0;
    if (cublasLtMatmulAlgoGetHeuristic(handle, op, lay_b, lay_a, lay_d, lay_d, pref, 1, &choice, &found) !=
            CUBLAS_STATUS_SUCCESS || found == 0)
      return;
    ok = true;
  }
  ~Plan() {
    if (workspace) cudaFree(workspace);
    if (pref) cublasLtMatmulPreferenceDestroy(pref);
    if (lay_b) cublasLtMatrixLayoutDestroy(lay_b);
    if (lay_a) cublasLtMatrixLayoutDestroy(lay_a);
    if (lay_d) cublasLtMatrixLayoutDestroy(lay_d);
    if (op) cublasLtMatmulDescDestroy(op);
    if (handle) cublasLtDestroy(handle);
  }
};

std::mutex g_mu;
// Plans live until the process exits and are deliberately never destroyed: a static destructor would call
// into cuBLASLt and the CUDA runtime while those (and any attached profiler) are being torn down.
auto& g_plans = *new std::map<std::tuple<int, int, int, int>, std::unique_ptr<Plan>>();

}  // namespace

extern "C" int b2_nvfp4_gemm_cublaslt(const void* A, const void* B, const void* SFA, const void* SFB,
                                      float alpha, void* D, int M, int N, int K, void* stream) {
  if (!A || !B || !SFA || !SFB || !D || M < 1 || N < 1 || K < 1) return B2_ERR_INVALID_ARGUMENT;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return B2_ERR_CUDA;
  Plan* plan;
  {
    std::lock_guard<std::mutex> lock(g_mu);
    auto& slot = g_plans[std::make_tuple(dev, M, N, K)];
    if (!slot) slot = std::make_unique<Plan>(M, N, K);
    plan = slot.get();
  }
  if (!plan->ok) return B2_ERR_UNSUPPORTED;
  // cuBLAS "A" is the logical B operand and vice versa (see the header comment).
  if (cublasLtMatmulDescSetAttribute(plan->op, CUBLASLT_MATMUL_DESC_A_SCALE_POINTER, &SFB, sizeof(SFB)) != CUBLAS_STATUS_SUCCESS ||
      cublasLtMatmulDescSetAttribute(plan->op, CUBLASLT_MATMUL_DESC_B_SCALE_POINTER, &SFA, sizeof(SFA)) != CUBLAS_STATUS_SUCCESS)
    return B2_ERR_CUDA;
  const float beta = 0.0f;
  const cublasStatus_t st = cublasLtMatmul(plan->handle, plan->op, &alpha, B, plan->lay_b, A, plan->lay_a, &beta, D,
                                           plan->lay_d, D, plan->lay_d, &plan->choice.algo, plan->workspace,
                                           plan->workspace_bytes, static_cast<cudaStream_t>(stream));
  return st == CUBLAS_STATUS_SUCCESS ? B2_OK : B2_ERR_CUDA;
}
