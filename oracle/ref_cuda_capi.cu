// C-linkage entry points onto the reference's own CUDA kernels
// (src/kernels/{rmsnorm,quantization,rope,activation,embedding,attention,flash_decode,flash_prefill}.cu), which the
// Makefile compiles for sm_100a from where they lie and links with this file
// into _ref/libref_cuda.so.  It is the GPU-side oracle (identical intrinsics
// and operation order) and the CUDA baseline the benchmark times beside the
// new kernels.  Test and benchmark infrastructure only.
#include <cstdint>

#include <runtherder/kernels/activation.cuh>
#include <runtherder/kernels/attention.cuh>
#include <runtherder/kernels/flash_decode.cuh>
#include <runtherder/kernels/flash_prefill.cuh>
#include <runtherder/kernels/embedding.cuh>
#include <runtherder/kernels/quantization.cuh>
#include <runtherder/kernels/rmsnorm.cuh>
#include <runtherder/kernels/rope.cuh>

namespace rk = runtherder::kernels;
using bf16 = __nv_bfloat16;

extern "C" {

void refcuda_rmsnorm(void* y, const void* x, const void* g, int num_tokens, int hidden_dim, float eps,
                     void* stream) {
    rk::rmsnorm_bf16_forward(static_cast<bf16*>(y), static_cast<const bf16*>(x),
                             static_cast<const bf16*>(g), num_tokens, hidden_dim, eps,
                             static_cast<cudaStream_t>(stream));
}

void refcuda_rmsnorm_add(void* y, void* h_out, const void* x, const void* residual, const void* g,
                         int num_tokens, int hidden_dim, float eps, void* stream) {
    rk::rmsnorm_add_bf16_forward(static_cast<bf16*>(y), static_cast<bf16*>(h_out),
                                 static_cast<const bf16*>(x), static_cast<const bf16*>(residual),
                                 static_cast<const bf16*>(g), num_tokens, hidden_dim, eps,
                                 static_cast<cudaStream_t>(stream));
}

void refcuda_quantize_per_token_int8(std::int8_t* q, float* x_scale, const void* x, int num_tokens,
                                     int dim, void* stream) {
    rk::quantize_per_token_int8(q, x_scale, static_cast<const bf16*>(x), num_tokens, dim,
                                static_cast<cudaStream_t>(stream));
}

void refcuda_dequantize_w8a8(void* y, const std::int32_t* acc, const float* x_scale, const void* w_scale,
                             int m, int n, void* stream) {
    rk::dequantize_w8a8(static_cast<bf16*>(y), acc, x_scale, static_cast<const bf16*>(w_scale), m, n,
                        static_cast<cudaStream_t>(stream));
}

void refcuda_quantize_kv_fp8(void* q, float* scale, const void* x, const int* at_pos, int rows_per_pos,
                             int num_rows, int head_dim, void* stream) {
    rk::quantize_kv_fp8(static_cast<__nv_fp8_e4m3*>(q), scale, static_cast<const bf16*>(x), at_pos,
                        rows_per_pos, num_rows, head_dim, static_cast<cudaStream_t>(stream));
}

void refcuda_swiglu(void* y, const void* gate, const void* up, int n, void* stream) {
    rk::swiglu_bf16_forward(static_cast<bf16*>(y), static_cast<const bf16*>(gate),
                            static_cast<const bf16*>(up), n, static_cast<cudaStream_t>(stream));
}

void refcuda_rope(void* q, void* k, const int* positions, const float* inv_freq, int seq_len,
                  int num_q_heads, int num_kv_heads, int head_dim, void* stream) {
    rk::rope_bf16(static_cast<bf16*>(q), static_cast<bf16*>(k), positions, inv_freq, seq_len,
                  num_q_heads, num_kv_heads, head_dim, static_cast<cudaStream_t>(stream));
}

void refcuda_embedding_lookup(void* out, const void* table, const int* ids, int num_tokens,
                              int hidden_dim, void* stream) {
    rk::embedding_lookup_bf16_forward(static_cast<bf16*>(out), static_cast<const bf16*>(table), ids,
                                      num_tokens, hidden_dim, static_cast<cudaStream_t>(stream));
}

// The naive causal attention the reference's flash tests use as their oracle.
void refcuda_attention_causal(void* out, const void* q, const void* k, const void* v, const float* k_scale,
                              const float* v_scale, int n_new, const int* cache_len, int num_q_heads,
                              int num_kv_heads, int head_dim, float scale, void* stream) {
    rk::attention_causal_bf16(static_cast<bf16*>(out), static_cast<const bf16*>(q),
                              static_cast<const __nv_fp8_e4m3*>(k), static_cast<const __nv_fp8_e4m3*>(v), k_scale,
                              v_scale, n_new, cache_len, num_q_heads, num_kv_heads, head_dim, scale,
                              static_cast<cudaStream_t>(stream));
}

void refcuda_flash_decode_split(void* out, const void* q, const void* k, const void* v, const float* k_scale,
                                const float* v_scale, float* partial, int num_splits, const int* cache_len,
                                int num_q_heads, int num_kv_heads, int head_dim, float scale, void* stream) {
    rk::flash_decode_split_bf16(static_cast<bf16*>(out), static_cast<const bf16*>(q),
                                static_cast<const __nv_fp8_e4m3*>(k), static_cast<const __nv_fp8_e4m3*>(v), k_scale,
                                v_scale, partial, num_splits, cache_len, num_q_heads, num_kv_heads, head_dim, scale,
                                static_cast<cudaStream_t>(stream));
}

void refcuda_flash_prefill(void* out, const void* q, const void* k, const void* v, const float* k_scale,
                           const float* v_scale, int n_new, const int* cache_len, int num_q_heads, int num_kv_heads,
                           int head_dim, float scale, void* stream) {
    rk::flash_prefill_bf16(static_cast<bf16*>(out), static_cast<const bf16*>(q), static_cast<const __nv_fp8_e4m3*>(k),
                           static_cast<const __nv_fp8_e4m3*>(v), k_scale, v_scale, n_new, cache_len, num_q_heads,
                           num_kv_heads, head_dim, scale, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
