// C++ entry points with the exact signatures of runtherder's kernel API
// (namespace runtherder::kernels), exported by librh_kernels.so.  runtherder's
// layer composition (src/model/supported/llama/{llama3,qwen3,qwen2}.cu), its
// KVCache::append (include/runtherder/engine/kv_cache.h:74-77), Matmul::linear_w8a8
// (src/kernels/matmul.cu:138,157) and its kernel tests keep including their own
// headers and simply link against this library instead of runtherder_kernels.
//
// Behaviour on error matches the reference (include/runtherder/check.h:8-23,
// include/runtherder/device/check.cuh:11-26): a message on stderr, then
// std::exit(EXIT_FAILURE).  Each function forwards to the C entry point of the same
// name in rh_kernels.h, which documents the arithmetic.
//
// The default `stream = nullptr` of the reference's headers lives in those headers;
// it is repeated here so this header can also be used on its own.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include <cstdint>

namespace runtherder::kernels {

// include/runtherder/kernels/rmsnorm.cuh:15-22
void rmsnorm_bf16_forward(__nv_bfloat16* y, const __nv_bfloat16* x, const __nv_bfloat16* g,
                          int num_tokens, int hidden_dim, float eps, cudaStream_t stream = nullptr);

// include/runtherder/kernels/rmsnorm.cuh:36-45
void rmsnorm_add_bf16_forward(__nv_bfloat16* y, __nv_bfloat16* h_out, const __nv_bfloat16* x,
                              const __nv_bfloat16* residual, const __nv_bfloat16* g, int num_tokens,
                              int hidden_dim, float eps, cudaStream_t stream = nullptr);

// include/runtherder/kernels/quantization.cuh:17-22
void quantize_per_token_int8(std::int8_t* q, float* x_scale, const __nv_bfloat16* x, int num_tokens,
                             int dim, cudaStream_t stream = nullptr);

// include/runtherder/kernels/quantization.cuh:31-37
void dequantize_w8a8(__nv_bfloat16* y, const std::int32_t* acc, const float* x_scale,
                     const __nv_bfloat16* w_scale, int m, int n, cudaStream_t stream = nullptr);

// include/runtherder/kernels/quantization.cuh:50-57
void quantize_kv_fp8(__nv_fp8_e4m3* q, float* scale, const __nv_bfloat16* x, const int* at_pos,
                     int rows_per_pos, int num_rows, int head_dim, cudaStream_t stream = nullptr);

// include/runtherder/kernels/activation.cuh:16-21
void swiglu_bf16_forward(__nv_bfloat16* y, const __nv_bfloat16* gate, const __nv_bfloat16* up, int n,
                         cudaStream_t stream = nullptr);

// include/runtherder/kernels/rope.cuh:16-25
void rope_bf16(__nv_bfloat16* q, __nv_bfloat16* k, const int* positions, const float* inv_freq,
               int seq_len, int num_q_heads, int num_kv_heads, int head_dim,
               cudaStream_t stream = nullptr);

// include/runtherder/kernels/embedding.cuh:14-20
void embedding_lookup_bf16_forward(__nv_bfloat16* out, const __nv_bfloat16* embedding_table,
                                   const int* token_ids, int num_tokens, int hidden_dim,
                                   cudaStream_t stream = nullptr);

// include/runtherder/kernels/bias.cuh:20-30
void qkv_bias_add_bf16_forward(__nv_bfloat16* q, __nv_bfloat16* k, __nv_bfloat16* v, const __nv_bfloat16* q_bias,
                               const __nv_bfloat16* k_bias, const __nv_bfloat16* v_bias, int n, int q_dim,
                               int kv_dim, cudaStream_t stream = nullptr);

// include/runtherder/kernels/flash_decode.cuh:27-62 (the scratch size stays the reference's constexpr
// flash_split_scratch_floats, same layout; rh_flash_split_scratch_floats is its C twin)
void flash_decode_split_bf16(__nv_bfloat16* out, const __nv_bfloat16* q, const __nv_fp8_e4m3* k,
                             const __nv_fp8_e4m3* v, const float* k_scale, const float* v_scale, float* partial,
                             int num_splits, const int* cache_len, int num_q_heads, int num_kv_heads,
                             int head_dim, float scale, cudaStream_t stream = nullptr);

// include/runtherder/kernels/flash_prefill.cuh:27-40
void flash_prefill_bf16(__nv_bfloat16* out, const __nv_bfloat16* q, const __nv_fp8_e4m3* k, const __nv_fp8_e4m3* v,
                        const float* k_scale, const float* v_scale, int n_new, const int* cache_len, int num_q_heads,
                        int num_kv_heads, int head_dim, float scale, cudaStream_t stream = nullptr);

}  // namespace runtherder::kernels
