// Link-time drop-in for runtherder's kernel library: the reference's C++ signatures,
// forwarding to the C ABI and keeping its fatal-error convention.
#include <cstdio>
#include <cstdlib>

#include "rh_dropin.hpp"
#include "rh_kernels.h"

namespace {

void die_on_error(int status, const char* fn) {
    if (status == RH_OK) return;
    std::fprintf(stderr, "runtherder check failed in %s\n  status:    %s\n  reason:    %s\n", fn,
                 rh_status_string(status), rh_last_error_string());
    std::exit(EXIT_FAILURE);
}

}  // namespace

namespace runtherder::kernels {

void rmsnorm_bf16_forward(__nv_bfloat16* y, const __nv_bfloat16* x, const __nv_bfloat16* g,
                          int num_tokens, int hidden_dim, float eps, cudaStream_t stream) {
    die_on_error(rh_rmsnorm_bf16(y, x, g, num_tokens, hidden_dim, eps, stream), "rmsnorm_bf16_forward");
}

void rmsnorm_add_bf16_forward(__nv_bfloat16* y, __nv_bfloat16* h_out, const __nv_bfloat16* x,
                              const __nv_bfloat16* residual, const __nv_bfloat16* g, int num_tokens,
                              int hidden_dim, float eps, cudaStream_t stream) {
    die_on_error(rh_rmsnorm_add_bf16(y, h_out, x, residual, g, num_tokens, hidden_dim, eps, stream),
                 "rmsnorm_add_bf16_forward");
}

void quantize_per_token_int8(std::int8_t* q, float* x_scale, const __nv_bfloat16* x, int num_tokens,
                             int dim, cudaStream_t stream) {
    die_on_error(rh_quantize_per_token_int8(q, x_scale, x, num_tokens, dim, stream), "quantize_per_token_int8");
}

void dequantize_w8a8(__nv_bfloat16* y, const std::int32_t* acc, const float* x_scale,
                     const __nv_bfloat16* w_scale, int m, int n, cudaStream_t stream) {
    die_on_error(rh_dequantize_w8a8(y, acc, x_scale, w_scale, m, n, stream), "dequantize_w8a8");
}

void quantize_kv_fp8(__nv_fp8_e4m3* q, float* scale, const __nv_bfloat16* x, const int* at_pos,
                     int rows_per_pos, int num_rows, int head_dim, cudaStream_t stream) {
    die_on_error(rh_quantize_kv_fp8(reinterpret_cast<std::uint8_t*>(q), scale, x, at_pos, rows_per_pos,
                                    num_rows, head_dim, stream),
                 "quantize_kv_fp8");
}

void swiglu_bf16_forward(__nv_bfloat16* y, const __nv_bfloat16* gate, const __nv_bfloat16* up, int n,
                         cudaStream_t stream) {
    die_on_error(rh_swiglu_bf16(y, gate, up, n, stream), "swiglu_bf16_forward");
}

void rope_bf16(__nv_bfloat16* q, __nv_bfloat16* k, const int* positions, const float* inv_freq,
               int seq_len, int num_q_heads, int num_kv_heads, int head_dim, cudaStream_t stream) {
    die_on_error(rh_rope_bf16(q, k, positions, inv_freq, seq_len, num_q_heads, num_kv_heads, head_dim, stream),
                 "rope_bf16");
}

void embedding_lookup_bf16_forward(__nv_bfloat16* out, const __nv_bfloat16* embedding_table,
                                   const int* token_ids, int num_tokens, int hidden_dim,
                                   cudaStream_t stream) {
    die_on_error(rh_embedding_lookup_bf16(out, embedding_table, token_ids, num_tokens, hidden_dim, stream),
                 "embedding_lookup_bf16_forward");
}

void qkv_bias_add_bf16_forward(__nv_bfloat16* q, __nv_bfloat16* k, __nv_bfloat16* v, const __nv_bfloat16* q_bias,
                               const __nv_bfloat16* k_bias, const __nv_bfloat16* v_bias, int n, int q_dim,
                               int kv_dim, cudaStream_t stream) {
    die_on_error(rh_qkv_bias_add_bf16(q, k, v, q_bias, k_bias, v_bias, n, q_dim, kv_dim, stream),
                 "qkv_bias_add_bf16_forward");
}

void flash_decode_split_bf16(__nv_bfloat16* out, const __nv_bfloat16* q, const __nv_fp8_e4m3* k,
                             const __nv_fp8_e4m3* v, const float* k_scale, const float* v_scale, float* partial,
                             int num_splits, const int* cache_len, int num_q_heads, int num_kv_heads,
                             int head_dim, float scale, cudaStream_t stream) {
    die_on_error(rh_flash_decode_split_bf16(out, q, reinterpret_cast<const std::uint8_t*>(k),
                                            reinterpret_cast<const std::uint8_t*>(v), k_scale, v_scale, partial,
                                            num_splits, cache_len, num_q_heads, num_kv_heads, head_dim, scale,
                                            stream),
                 "flash_decode_split_bf16");
}

void flash_prefill_bf16(__nv_bfloat16* out, const __nv_bfloat16* q, const __nv_fp8_e4m3* k, const __nv_fp8_e4m3* v,
                        const float* k_scale, const float* v_scale, int n_new, const int* cache_len, int num_q_heads,
                        int num_kv_heads, int head_dim, float scale, cudaStream_t stream) {
    die_on_error(rh_flash_prefill_bf16(out, q, reinterpret_cast<const std::uint8_t*>(k),
                                       reinterpret_cast<const std::uint8_t*>(v), k_scale, v_scale, n_new, cache_len,
                                       num_q_heads, num_kv_heads, head_dim, scale, stream),
                 "flash_prefill_bf16");
}

}  // namespace runtherder::kernels
