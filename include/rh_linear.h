/*
 * rh_linear.h — C ABI of librh_linear.so: the W8A8 linear layer around this library's fused
 * quantisation kernels.  The GEMM itself stays cuBLASLt, exactly as in the reference; what this adds is
 * an entry that takes ALREADY QUANTISED activations, so the INT8 codes and per-token scales written by
 * rh_rmsnorm_add_quant_int8 / rh_swiglu_quant_int8 (rh_kernels.h) feed the GEMM directly instead of
 * being re-quantised inside every linear layer.
 *
 * librh_linear.so links librh_kernels.so and libcublasLt.so.12; librh_kernels.so itself has no cuBLAS
 * dependency.  Conventions as in rh_kernels.h: device pointers, `stream` is a cudaStream_t passed as
 * void*, status-code returns, rh_last_error_string() for the reason.  `lt_handle` is a
 * cublasLtHandle_t passed as void*; the caller owns it and the workspace.
 *
 * Per (handle, m, n, k, workspace size) the matmul descriptor, the three layouts and the algorithm the
 * heuristic picks are built on first use and kept (the reference's Matmul::get_or_build_plan does the
 * same in its plan_cache_, src/kernels/matmul.cu:21-93); building a plan is host work only, so a first
 * call inside stream capture is allowed.  rh_linear_release() drops the plans of a handle.
 */
#ifndef RH_LINEAR_H
#define RH_LINEAR_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* y[m,n] = bf16((q[m,k] . weight[n,k]^T) * x_scale[row] * w_scale[col]): the INT8 GEMM (int32
 * accumulation into acc[m,n]) followed by the dequantising epilogue rh_dequantize_w8a8.
 * This is Matmul::linear_w8a8 (include/runtherder/kernels/matmul.cuh:63-71, src/kernels/matmul.cu:126-158)
 * without its first step, the quantize_per_token_int8 call at matmul.cu:138; the cublasLtMatmul call and
 * its layouts are those of matmul.cu:36-56,140-155 (weight read as its transpose, plain column-major
 * int32 output).  k must be a multiple of 4 (matmul.cu:136).  No counterpart entry exists in the
 * reference: it is the hand-off that lets a caller quantise once per distinct input. */
int rh_linear_w8a8_prequantized(void* y, const int8_t* q, const float* x_scale, const int8_t* weight,
                                const void* w_scale, int32_t* acc, int m, int n, int k, void* lt_handle,
                                void* workspace, size_t workspace_bytes, void* stream);

/* The reference's call as it stands: quantise x[m,k] (bf16) per token into q / x_scale, then the above.
 * Replaces Matmul::linear_w8a8 (matmul.cu:126-158); q, x_scale and acc are the W8A8Buffer members
 * (matmul.cuh:22-29). */
int rh_linear_w8a8(void* y, const void* x, const int8_t* weight, const void* w_scale, int8_t* q,
                   float* x_scale, int32_t* acc, int m, int n, int k, void* lt_handle, void* workspace,
                   size_t workspace_bytes, void* stream);

/* Convenience for hosts without their own cuBLASLt set-up (tests, Python): create / destroy a handle
 * (cublasLtCreate / cublasLtDestroy; Matmul::Matmul, matmul.cu:14-19).  Destroy also releases its plans. */
int rh_linear_create_handle(void** lt_handle_out);
int rh_linear_destroy_handle(void* lt_handle);

/* Drops every cached plan of `lt_handle` (call before destroying a handle created elsewhere). */
int rh_linear_release(void* lt_handle);

#ifdef __cplusplus
}
#endif
#endif /* RH_LINEAR_H */
