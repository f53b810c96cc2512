// W8A8 linear layer around the fused quantisation kernels: cuBLASLt INT8 GEMM (int32 accumulation)
// + this library's dequantising epilogue, with an entry for activations that are already quantised.
// Layouts and call follow the reference's Matmul (src/kernels/matmul.cu:36-56, 140-155): cuBLASLt is
// column major, each row-major buffer reads as its transpose, the call computes y^T = W . x^T with
// mapped dims M = n, N = m, K = k, operation T on the weight and N on the activations.
#include <cublasLt.h>

#include <map>
#include <mutex>
#include <tuple>

#include "rh_common.cuh"
#include "rh_linear.h"

namespace rh {
namespace {

struct Plan {
    cublasLtMatmulDesc_t desc = nullptr;
    cublasLtMatrixLayout_t w = nullptr, x = nullptr, y = nullptr;
    cublasLtMatmulAlgo_t algo;
};
using PlanKey = std::tuple<void*, int, int, int, size_t>;   // handle, m, n, k, workspace bytes

std::mutex& plan_mutex() { static std::mutex m; return m; }
std::map<PlanKey, Plan>& plans() { static std::map<PlanKey, Plan> p; return p; }

void destroy(Plan& p) {
    if (p.w) cublasLtMatrixLayoutDestroy(p.w);
    if (p.x) cublasLtMatrixLayoutDestroy(p.x);
    if (p.y) cublasLtMatrixLayoutDestroy(p.y);
    if (p.desc) cublasLtMatmulDescDestroy(p.desc);
    p = Plan{};
}

#define RH_LT(expr, what)                                                                              \
    do {                                                                                               \
        const cublasStatus_t st_ = (expr);                                                             \
        if (st_ != CUBLAS_STATUS_SUCCESS) {                                                            \
            destroy(plan);                                                                             \
            return host::fail(RH_ERR_CUDA, "rh_linear_w8a8: %s: %s", what, cublasLtGetStatusString(st_)); \
        }                                                                                              \
    } while (0)

// Finds or builds the plan; *out stays valid until rh_linear_release / destroy of the handle.
int get_plan(cublasLtHandle_t handle, int m, int n, int k, size_t workspace_bytes, const Plan** out) {
    const PlanKey key{handle, m, n, k, workspace_bytes};
    std::lock_guard<std::mutex> lock(plan_mutex());
    auto& table = plans();
    if (const auto it = table.find(key); it != table.end()) {
        *out = &it->second;
        return RH_OK;
    }
    Plan plan;
    const int64_t lt_m = n, lt_n = m, lt_k = k;
    RH_LT(cublasLtMatmulDescCreate(&plan.desc, CUBLAS_COMPUTE_32I, CUDA_R_32I), "matmul descriptor");
    const cublasOperation_t ta = CUBLAS_OP_T, tb = CUBLAS_OP_N;
    RH_LT(cublasLtMatmulDescSetAttribute(plan.desc, CUBLASLT_MATMUL_DESC_TRANSA, &ta, sizeof(ta)), "transa");
    RH_LT(cublasLtMatmulDescSetAttribute(plan.desc, CUBLASLT_MATMUL_DESC_TRANSB, &tb, sizeof(tb)), "transb");
    RH_LT(cublasLtMatrixLayoutCreate(&plan.w, CUDA_R_8I, lt_k, lt_m, lt_k), "weight layout");
    RH_LT(cublasLtMatrixLayoutCreate(&plan.x, CUDA_R_8I, lt_k, lt_n, lt_k), "activation layout");
    RH_LT(cublasLtMatrixLayoutCreate(&plan.y, CUDA_R_32I, lt_m, lt_n, lt_m), "accumulator layout");
    cublasLtMatmulPreference_t pref = nullptr;
    RH_LT(cublasLtMatmulPreferenceCreate(&pref), "preference");
    cublasStatus_t st = cublasLtMatmulPreferenceSetAttribute(pref, CUBLASLT_MATMUL_PREF_MAX_WORKSPACE_BYTES,
                                                             &workspace_bytes, sizeof(workspace_bytes));
    cublasLtMatmulHeuristicResult_t heuristic{};
    int returned = 0;
    if (st == CUBLAS_STATUS_SUCCESS)
        st = cublasLtMatmulAlgoGetHeuristic(handle, plan.desc, plan.w, plan.x, plan.y, plan.y, pref, 1, &heuristic, &returned);
    cublasLtMatmulPreferenceDestroy(pref);
    RH_LT(st, "algorithm heuristic");
    if (returned <= 0) {
        destroy(plan);
        return host::fail(RH_ERR_UNSUPPORTED_DIM, "rh_linear_w8a8: no cuBLASLt algorithm for m=%d n=%d k=%d", m, n, k);
    }
    plan.algo = heuristic.algo;
    *out = &table.emplace(key, plan).first->second;
    return RH_OK;
}
#undef RH_LT

void release(void* handle) {
    std::lock_guard<std::mutex> lock(plan_mutex());
    auto& table = plans();
    for (auto it = table.begin(); it != table.end();) {
        if (std::get<0>(it->first) == handle) {
            destroy(it->second);
            it = table.erase(it);
        } else {
            ++it;
        }
    }
}

}  // namespace
}  // namespace rh

using namespace rh;

extern "C" int rh_linear_w8a8_prequantized(void* y, const int8_t* q, const float* x_scale, const int8_t* weight,
                                           const void* w_scale, int32_t* acc, int m, int n, int k, void* lt_handle,
                                           void* workspace, size_t workspace_bytes, void* stream) {
    RH_REQUIRE(y && q && x_scale && weight && w_scale && acc && lt_handle, RH_ERR_INVALID_ARG,
               "rh_linear_w8a8_prequantized: null pointer");
    RH_REQUIRE(m >= 1 && n >= 1 && k >= 1, RH_ERR_INVALID_ARG, "rh_linear_w8a8_prequantized: matmul dims must be positive");
    RH_REQUIRE(k % 4 == 0, RH_ERR_UNSUPPORTED_DIM, "rh_linear_w8a8_prequantized: int8 gemm requires k divisible by 4 (got %d)", k);
    RH_REQUIRE(workspace != nullptr || workspace_bytes == 0, RH_ERR_INVALID_ARG,
               "rh_linear_w8a8_prequantized: workspace_bytes given without a workspace");
    const Plan* plan = nullptr;
    if (int e = get_plan(static_cast<cublasLtHandle_t>(lt_handle), m, n, k, workspace_bytes, &plan)) return e;
    const int32_t alpha = 1, beta = 0;
    const cublasStatus_t st = cublasLtMatmul(static_cast<cublasLtHandle_t>(lt_handle), plan->desc, &alpha, weight, plan->w,
                                             q, plan->x, &beta, acc, plan->y, acc, plan->y, &plan->algo, workspace,
                                             workspace_bytes, static_cast<cudaStream_t>(stream));
    if (st != CUBLAS_STATUS_SUCCESS)
        return host::fail(RH_ERR_LAUNCH, "rh_linear_w8a8_prequantized: cublasLtMatmul: %s", cublasLtGetStatusString(st));
    return rh_dequantize_w8a8(y, acc, x_scale, w_scale, m, n, stream);
}

extern "C" int rh_linear_w8a8(void* y, const void* x, const int8_t* weight, const void* w_scale, int8_t* q,
                              float* x_scale, int32_t* acc, int m, int n, int k, void* lt_handle, void* workspace,
                              size_t workspace_bytes, void* stream) {
    RH_REQUIRE(x != nullptr && q != nullptr && x_scale != nullptr, RH_ERR_INVALID_ARG, "rh_linear_w8a8: null pointer");
    RH_REQUIRE(m >= 1 && n >= 1 && k >= 1, RH_ERR_INVALID_ARG, "rh_linear_w8a8: matmul dims must be positive");
    RH_REQUIRE(k % 4 == 0, RH_ERR_UNSUPPORTED_DIM, "rh_linear_w8a8: int8 gemm requires k divisible by 4 (got %d)", k);
    if (int e = rh_quantize_per_token_int8(q, x_scale, x, m, k, stream)) return e;
    return rh_linear_w8a8_prequantized(y, q, x_scale, weight, w_scale, acc, m, n, k, lt_handle, workspace,
                                       workspace_bytes, stream);
}

extern "C" int rh_linear_create_handle(void** lt_handle_out) {
    RH_REQUIRE(lt_handle_out != nullptr, RH_ERR_INVALID_ARG, "rh_linear_create_handle: null pointer");
    cublasLtHandle_t h = nullptr;
    const cublasStatus_t st = cublasLtCreate(&h);
    if (st != CUBLAS_STATUS_SUCCESS) return host::fail(RH_ERR_CUDA, "rh_linear_create_handle: %s", cublasLtGetStatusString(st));
    *lt_handle_out = h;
    return RH_OK;
}

extern "C" int rh_linear_release(void* lt_handle) {
    RH_REQUIRE(lt_handle != nullptr, RH_ERR_INVALID_ARG, "rh_linear_release: null handle");
    release(lt_handle);
    return RH_OK;
}

extern "C" int rh_linear_destroy_handle(void* lt_handle) {
    RH_REQUIRE(lt_handle != nullptr, RH_ERR_INVALID_ARG, "rh_linear_destroy_handle: null handle");
    release(lt_handle);
    const cublasStatus_t st = cublasLtDestroy(static_cast<cublasLtHandle_t>(lt_handle));
    if (st != CUBLAS_STATUS_SUCCESS) return host::fail(RH_ERR_CUDA, "rh_linear_destroy_handle: %s", cublasLtGetStatusString(st));
    return RH_OK;
}
