// bfloat16 matrix product through cuBLASLt: y[N, O] = x[N, K] . w[O, K]^T, float32 accumulation.
//
// The output is bfloat16, or float32; a float32 output may be accumulated into (y += x . w^T), which
// is how a product adds itself to the float32 residual stream without a rounding in between.
// Row-major x and w are, to a column-major library, w^T and x^T: D[O, N] = op_T(w)[O, K] . x[K, N].
//
// The handle, the chosen algorithm per shape and nothing else are kept here; the caller passes the
// workspace. Everything is created on the first call of a shape, so a first call per shape must
// come before stream capture.
#include <cublasLt.h>

#include <map>
#include <mutex>
#include <tuple>

#include "common.cuh"

namespace {

struct Plan {
  cublasLtMatmulDesc_t op = nullptr;
  cublasLtMatrixLayout_t a = nullptr, b = nullptr, c = nullptr;
  cublasLtMatmulAlgo_t algo;
  bool ok = false;
};

cublasLtHandle_t g_handle = nullptr;
std::mutex g_mutex;
std::map<std::tuple<int, int, int, int, size_t>, Plan> g_plans;

int make_plan(Plan& plan, int N, int O, int K, int out_f32, size_t workspace_bytes) {
  cublasStatus_t st;
  if ((st = cublasLtMatmulDescCreate(&plan.op, CUBLAS_COMPUTE_32F, CUDA_R_32F)) != CUBLAS_STATUS_SUCCESS) return 1000 + st;
  const cublasOperation_t ta = CUBLAS_OP_T, tb = CUBLAS_OP_N;
  cublasLtMatmulDescSetAttribute(plan.op, CUBLASLT_MATMUL_DESC_TRANSA, &ta, sizeof(ta));
  cublasLtMatmulDescSetAttribute(plan.op, CUBLASLT_MATMUL_DESC_TRANSB, &tb, sizeof(tb));
  const cudaDataType_t out = out_f32 ? CUDA_R_32F : CUDA_R_16BF;
  if ((st = cublasLtMatrixLayoutCreate(&plan.a, CUDA_R_16BF, K, O, K)) != CUBLAS_STATUS_SUCCESS) return 1000 + st;
  if ((st = cublasLtMatrixLayoutCreate(&plan.b, CUDA_R_16BF, K, N, K)) != CUBLAS_STATUS_SUCCESS) return 1000 + st;
  if ((st = cublasLtMatrixLayoutCreate(&plan.c, out, O, N, O)) != CUBLAS_STATUS_SUCCESS) return 1000 + st;
  cublasLtMatmulPreference_t pref;
  cublasLtMatmulPreferenceCreate(&pref);
  cublasLtMatmulPreferenceSetAttribute(pref, CUBLASLT_MATMUL_PREF_MAX_WORKSPACE_BYTES, &workspace_bytes,
                                       sizeof(workspace_bytes));
  cublasLtMatmulHeuristicResult_t result;
  int found = 0;
  st = cublasLtMatmulAlgoGetHeuristic(g_handle, plan.op, plan.a, plan.b, plan.c, plan.c, pref, 1, &result, &found);
  cublasLtMatmulPreferenceDestroy(pref);
  if (st != CUBLAS_STATUS_SUCCESS || found == 0) return 2000 + (int)st;
  plan.algo = result.algo;
  plan.ok = true;
  return 0;
}

}  // namespace

// Returns 0, a CUDA error code (< 1000), 1000 + a cuBLAS status, or 2000 + status when no algorithm fits.
AKAS_API int akas_gemm_bf16(const void* x, const void* w, void* y, int N, int O, int K, int out_f32, int accumulate,
                            void* workspace, long long workspace_bytes, cudaStream_t stream) {
  if (N <= 0 || O <= 0) return 0;
  if (K <= 0 || (accumulate && !out_f32)) return (int)cudaErrorInvalidValue;
  Plan* plan;
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    if (g_handle == nullptr) {
      const cublasStatus_t st = cublasLtCreate(&g_handle);
      if (st != CUBLAS_STATUS_SUCCESS) return 1000 + (int)st;
    }
    // The library's choice of algorithm is looked up once per shape. A serving step brings any number of tokens, so
    // beyond 256 tokens the choice is made for the count rounded up to a multiple of 256 and reused for every count
    // in that range (the look-up costs about as much as a short product runs).
    const int planned = N <= 256 ? N : (N + 255) / 256 * 256;
    const auto key = std::make_tuple(planned, O, K, out_f32, (size_t)workspace_bytes);
    auto it = g_plans.find(key);
    if (it == g_plans.end()) {
      Plan fresh;
      const int err = make_plan(fresh, planned, O, K, out_f32, (size_t)workspace_bytes);
      if (err) return err;
      it = g_plans.emplace(key, fresh).first;
    }
    plan = &it->second;
  }
  const float alpha = 1.f, beta = accumulate ? 1.f : 0.f;
  cublasLtMatrixLayout_t b = plan->b, c = plan->c;
  const bool other_count = N > 256 && N % 256 != 0;  // the plan's layouts are for the rounded count
  if (other_count) {
    if (cublasLtMatrixLayoutCreate(&b, CUDA_R_16BF, K, N, K) != CUBLAS_STATUS_SUCCESS) return 1000;
    if (cublasLtMatrixLayoutCreate(&c, out_f32 ? CUDA_R_32F : CUDA_R_16BF, O, N, O) != CUBLAS_STATUS_SUCCESS) {
      cublasLtMatrixLayoutDestroy(b);
      return 1000;
    }
  }
  cublasStatus_t st = cublasLtMatmul(g_handle, plan->op, &alpha, w, plan->a, x, b, &beta, y, c, y, c, &plan->algo, workspace,
                                     (size_t)workspace_bytes, stream);
  if (other_count) {
    cublasLtMatrixLayoutDestroy(b);
    cublasLtMatrixLayoutDestroy(c);
    if (st != CUBLAS_STATUS_SUCCESS) {  // the algorithm does not take this count after all: look it up exactly
      Plan exact;
      const int err = make_plan(exact, N, O, K, out_f32, (size_t)workspace_bytes);
      if (err) return err;
      st = cublasLtMatmul(g_handle, exact.op, &alpha, w, exact.a, x, exact.b, &beta, y, exact.c, y, exact.c, &exact.algo,
                          workspace, (size_t)workspace_bytes, stream);
      cublasLtMatrixLayoutDestroy(exact.a);
      cublasLtMatrixLayoutDestroy(exact.b);
      cublasLtMatrixLayoutDestroy(exact.c);
      cublasLtMatmulDescDestroy(exact.op);
    }
  }
  if (st != CUBLAS_STATUS_SUCCESS) return 1000 + (int)st;
  return 0;
}
