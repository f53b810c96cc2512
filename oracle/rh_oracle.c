/*
 * CPU oracle for the row-wise layer kernels.  TEST INFRASTRUCTURE ONLY: this
 * file is the checker the CUDA library is compared against.  Nothing in the
 * shipped library links, loads or calls it.
 *
 * Every function restates, in plain C on bf16/fp8 bit patterns, the arithmetic
 * of one piece of dev08math/runtherder; the citation beside each function is
 * the reference file and lines it follows (paths relative to the reference's
 * project root).  Where the reference has a host implementation (the
 * anonymous-namespace helpers inside its tests/kernels sources) that host code
 * is what is restated; where it has none, the CUDA kernel's arithmetic is.
 *
 * Parity status: PINNED.  The bf16 and E4M3 conversions are checked
 * exhaustively, and every restated function is checked bit for bit, against
 * the reference's own host helpers compiled unmodified (libref_host.so, built
 * by this directory's Makefile) and against golden vectors generated from
 * them.  Functions with no host counterpart in the reference
 * (quantize_per_token_int8, embedding gather, llama3 inv_freq scaling, cache
 * slot addressing) are pinned on the GPU against the reference's CUDA kernels
 * built for sm_100a (libref_cuda.so).
 *
 * Build: gcc -O2 -std=c11 -ffp-contract=off -fPIC -shared rh_oracle.c -lm
 * (-ffp-contract=off: no fused multiply-add may be introduced on the host).
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <string.h>

#define ORC_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------------ */
/* Number formats                                                           */
/* ------------------------------------------------------------------------ */

static inline uint32_t f32_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float bits_f32(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

/* bf16 -> fp32 is exact: the 16 bits are the top half of the fp32 pattern. */
ORC_API float orc_bf16_to_f32(uint16_t h) { return bits_f32((uint32_t)h << 16); }

/* fp32 -> bf16, round to nearest even; NaN becomes 0x7FFF (the value CUDA's
 * host and device __float2bfloat16 produce). */
ORC_API uint16_t orc_f32_to_bf16(float f) {
    uint32_t u = f32_bits(f);
    if ((u & 0x7fffffffu) > 0x7f800000u) return 0x7fffu;
    uint32_t lsb = (u >> 16) & 1u;
    u += 0x7fffu + lsb;
    return (uint16_t)(u >> 16);
}

/* fp32 -> FP8 E4M3 (1-4-3, bias 7, no infinities, max finite 448), round to
 * nearest even, saturate-to-finite; NaN becomes 0x7F.  This is the conversion
 * __nv_fp8_e4m3(float) performs (reference: src/kernels/quantization.cu:249-250,
 * tests/kernels/test_quantization.cpp:58). */
ORC_API uint8_t orc_f32_to_e4m3(float f) {
    uint32_t u = f32_bits(f);
    uint8_t sign = (uint8_t)((u >> 24) & 0x80u);
    if ((u & 0x7fffffffu) > 0x7f800000u) return 0x7fu;   /* NaN: sign dropped, as CUDA does */
    double a = fabs((double)f);
    if (a == 0.0) return sign;
    if (isinf(a)) return (uint8_t)(sign | 0x7eu);
    int e2;
    (void)frexp(a, &e2);               /* a = m * 2^e2, m in [0.5,1) -> floor(log2 a) = e2-1 */
    int E = e2 - 1;
    double step = (E < -6) ? ldexp(1.0, -9) : ldexp(1.0, E - 3);
    double r = nearbyint(a / step) * step;   /* default mode: ties to even */
    if (r > 448.0) r = 448.0;
    if (r == 0.0) return sign;
    if (r < ldexp(1.0, -6)) return (uint8_t)(sign | (uint8_t)(r / ldexp(1.0, -9)));
    (void)frexp(r, &e2);
    E = e2 - 1;
    int mant = (int)((r / ldexp(1.0, E) - 1.0) * 8.0);
    return (uint8_t)(sign | (uint8_t)(((E + 7) << 3) | mant));
}

/* FP8 E4M3 -> fp32 (exact). */
ORC_API float orc_e4m3_to_f32(uint8_t b) {
    int s = b >> 7, e = (b >> 3) & 15, m = b & 7;
    float v;
    if (e == 15 && m == 7) v = NAN;
    else if (e == 0) v = (float)ldexp((double)m, -9);
    else v = (float)ldexp(1.0 + m / 8.0, e - 7);
    return s ? -v : v;
}

/* Read side of the KV cache: include/runtherder/kernels/quantization.cuh:63-66. */
ORC_API float orc_dequantize_kv_fp8(uint8_t q, float scale) { return orc_e4m3_to_f32(q) * scale; }

/* ------------------------------------------------------------------------ */
/* RMSNorm: tests/kernels/test_rmsnorm.cpp:39-61 (host reference of           */
/* src/kernels/rmsnorm.cu:214-224).  Sum of squares in double, narrowed to   */
/* float, rrms = 1/sqrtf(ss/H + eps), y = bf16((x*rrms)*g).                  */
/* ------------------------------------------------------------------------ */
ORC_API void orc_rmsnorm(uint16_t* y, const uint16_t* x, const uint16_t* g,
                         long num_tokens, int hidden_dim, float eps) {
    for (long row = 0; row < num_tokens; ++row) {
        const uint16_t* xr = x + (size_t)row * hidden_dim;
        uint16_t* yr = y + (size_t)row * hidden_dim;
        double ss = 0.0;
        for (int j = 0; j < hidden_dim; ++j) {
            float xv = orc_bf16_to_f32(xr[j]);
            ss += (double)xv * (double)xv;
        }
        float rrms = 1.0f / sqrtf((float)(ss / hidden_dim) + eps);
        for (int j = 0; j < hidden_dim; ++j) {
            float xv = orc_bf16_to_f32(xr[j]);
            float gv = orc_bf16_to_f32(g[j]);
            yr[j] = orc_f32_to_bf16(xv * rrms * gv);
        }
    }
}

/* Residual add + RMSNorm: tests/kernels/test_rmsnorm.cpp:68-97 (host reference
 * of src/kernels/rmsnorm.cu:226-238).  h = x + residual in fp32; h_out is the
 * bf16 rounding of h, while the sum of squares and y use the unrounded h.
 * h_out may alias residual (each element is read before it is written). */
ORC_API void orc_rmsnorm_add(uint16_t* y, uint16_t* h_out, const uint16_t* x,
                             const uint16_t* residual, const uint16_t* g,
                             long num_tokens, int hidden_dim, float eps, float* h_tmp) {
    for (long row = 0; row < num_tokens; ++row) {
        size_t off = (size_t)row * hidden_dim;
        double ss = 0.0;
        for (int j = 0; j < hidden_dim; ++j) {
            float xv = orc_bf16_to_f32(x[off + j]);
            float rv = orc_bf16_to_f32(residual[off + j]);
            h_tmp[j] = xv + rv;
            h_out[off + j] = orc_f32_to_bf16(h_tmp[j]);
            ss += (double)h_tmp[j] * (double)h_tmp[j];
        }
        float rrms = 1.0f / sqrtf((float)(ss / hidden_dim) + eps);
        for (int j = 0; j < hidden_dim; ++j) {
            float gv = orc_bf16_to_f32(g[j]);
            y[off + j] = orc_f32_to_bf16(h_tmp[j] * rrms * gv);
        }
    }
}

/* ------------------------------------------------------------------------ */
/* Per-token symmetric INT8 quantisation.  The reference has no host code    */
/* for it; this restates the kernel, src/kernels/quantization.cu:63-96:      */
/* amax starts at 0; x_scale = amax/127; inv = amax>0 ? 127/amax : 0;        */
/* q = clamp(round_half_even(x*inv), -127, 127).  All IEEE fp32.             */
/* ------------------------------------------------------------------------ */
/* clamp(__float2int_rn(p), -127, 127).  The device conversion rounds half to even, maps NaN to 0
 * and saturates out-of-range values (so +-Inf end at +-127 after the clamp). */
static inline int int8_code(float p) {
    if (isnan(p)) return 0;
    if (p >= 127.5f) return 127;
    if (p <= -127.5f) return -127;
    long qi = lrintf(p);                 /* default mode: ties to even */
    if (qi > 127) qi = 127;
    if (qi < -127) qi = -127;
    return (int)qi;
}

ORC_API void orc_quantize_per_token_int8(int8_t* q, float* x_scale, const uint16_t* x,
                                         long num_tokens, int dim) {
    for (long row = 0; row < num_tokens; ++row) {
        const uint16_t* xr = x + (size_t)row * dim;
        int8_t* qr = q + (size_t)row * dim;
        float amax = 0.0f;
        for (int j = 0; j < dim; ++j) amax = fmaxf(amax, fabsf(orc_bf16_to_f32(xr[j])));
        x_scale[row] = amax / 127.0f;
        float inv = (amax > 0.0f) ? (127.0f / amax) : 0.0f;
        for (int j = 0; j < dim; ++j) {
            qr[j] = (int8_t)int8_code(orc_bf16_to_f32(xr[j]) * inv);
        }
    }
}

/* W8A8 GEMM epilogue: src/kernels/quantization.cu:153-171.
 * y = bf16((float(acc) * x_scale[row]) * float(w_scale[col])). */
ORC_API void orc_dequantize_w8a8(uint16_t* y, const int32_t* acc, const float* x_scale,
                                 const uint16_t* w_scale, long m, int n) {
    for (long r = 0; r < m; ++r)
        for (int c = 0; c < n; ++c) {
            float ws = orc_bf16_to_f32(w_scale[c]);
            float v = (float)acc[(size_t)r * n + c] * x_scale[r] * ws;
            y[(size_t)r * n + c] = orc_f32_to_bf16(v);
        }
}

/* ------------------------------------------------------------------------ */
/* FP8 KV quantisation: tests/kernels/test_quantization.cpp:42-62 for the    */
/* arithmetic (scale = amax/448, inv = amax>0 ? 448/amax : 0,                */
/* q = e4m3(x*inv)), src/kernels/quantization.cu:210-211 for the slot        */
/* addressing dst_row = row + at_pos*rows_per_pos (source rows count from 0).*/
/* ------------------------------------------------------------------------ */
ORC_API void orc_quantize_kv_fp8(uint8_t* q, float* scale, const uint16_t* x, int at_pos,
                                 int rows_per_pos, long num_rows, int head_dim) {
    for (long row = 0; row < num_rows; ++row) {
        const uint16_t* xr = x + (size_t)row * head_dim;
        size_t dst = (size_t)row + (size_t)at_pos * (size_t)rows_per_pos;
        float amax = 0.0f;
        for (int j = 0; j < head_dim; ++j) amax = fmaxf(amax, fabsf(orc_bf16_to_f32(xr[j])));
        float inv = (amax > 0.0f) ? (448.0f / amax) : 0.0f;
        scale[dst] = amax / 448.0f;
        for (int j = 0; j < head_dim; ++j)
            q[dst * head_dim + j] = orc_f32_to_e4m3(orc_bf16_to_f32(xr[j]) * inv);
    }
}

/* ------------------------------------------------------------------------ */
/* SwiGLU: tests/kernels/test_activation.cpp:33-44 (host reference of        */
/* src/kernels/activation.cu:15-41).  s = 1/(1+exp(-g)) in double,           */
/* y = bf16(float(g*s*u)).                                                    */
/* ------------------------------------------------------------------------ */
ORC_API void orc_swiglu(uint16_t* y, const uint16_t* gate, const uint16_t* up, size_t n) {
    for (size_t i = 0; i < n; ++i) {
        double g = orc_bf16_to_f32(gate[i]);
        double u = orc_bf16_to_f32(up[i]);
        double s = 1.0 / (1.0 + exp(-g));
        y[i] = orc_f32_to_bf16((float)(g * s * u));
    }
}

/* ------------------------------------------------------------------------ */
/* RoPE, rotate-half pairs (i, i+D/2), in place.                              */
/* orc_rope_theta follows tests/kernels/test_rope.cpp:41-75 exactly: the     */
/* frequency theta_base^(-2i/D) is evaluated in double for every element.    */
/* ------------------------------------------------------------------------ */
ORC_API void orc_rope_theta(uint16_t* tensor, int start_pos, long seq_len, int num_heads,
                            int head_dim, float theta_base) {
    int half = head_dim / 2;
    for (long t = 0; t < seq_len; ++t) {
        int pos = start_pos + (int)t;
        for (int h = 0; h < num_heads; ++h) {
            size_t off = ((size_t)t * num_heads + h) * head_dim;
            for (int i = 0; i < half; ++i) {
                double exponent = -2.0 * (double)i / (double)head_dim;
                double freq = pow((double)theta_base, exponent);
                double th = (double)pos * freq;
                double c = cos(th), s = sin(th);
                double a = orc_bf16_to_f32(tensor[off + i]);
                double b = orc_bf16_to_f32(tensor[off + i + half]);
                tensor[off + i] = orc_f32_to_bf16((float)(a * c - b * s));
                tensor[off + i + half] = orc_f32_to_bf16((float)(a * s + b * c));
            }
        }
    }
}

/* The same loop fed from a caller-supplied frequency table and per-token
 * positions, which is how the kernel is called (src/kernels/rope.cu:31-54:
 * theta = float(pos) * inv_freq[i] as an fp32 product).  The rotation itself
 * is carried out in double like the test's host reference. */
ORC_API void orc_rope_table(uint16_t* tensor, const int32_t* positions, const float* inv_freq,
                            long seq_len, int num_heads, int head_dim) {
    int half = head_dim / 2;
    for (long t = 0; t < seq_len; ++t) {
        for (int h = 0; h < num_heads; ++h) {
            size_t off = ((size_t)t * num_heads + h) * head_dim;
            for (int i = 0; i < half; ++i) {
                float thf = (float)positions[t] * inv_freq[i];
                double c = cos((double)thf), s = sin((double)thf);
                double a = orc_bf16_to_f32(tensor[off + i]);
                double b = orc_bf16_to_f32(tensor[off + i + half]);
                tensor[off + i] = orc_f32_to_bf16((float)(a * c - b * s));
                tensor[off + i + half] = orc_f32_to_bf16((float)(a * s + b * c));
            }
        }
    }
}

/* ------------------------------------------------------------------------ */
/* Frequency tables (host, load time).                                        */
/* Plain: src/model/supported/llama/llama.cu:128-143.                        */
/* Llama-3 rescaling: src/model/supported/llama/llama3.cu:26-60.             */
/* ------------------------------------------------------------------------ */
ORC_API void orc_rope_inv_freq_plain(float* out, int head_dim, float theta_base) {
    int half = head_dim / 2;
    for (int i = 0; i < half; ++i) {
        double exponent = -2.0 * (double)i / (double)head_dim;
        out[i] = (float)pow((double)theta_base, exponent);
    }
}

ORC_API void orc_rope_inv_freq_llama3(float* out, int head_dim, float theta_base, float factor_f,
                                      float low_freq_factor_f, float high_freq_factor_f,
                                      int original_max_position_embeddings) {
    orc_rope_inv_freq_plain(out, head_dim, theta_base);
    double factor = factor_f, low = low_freq_factor_f, high = high_freq_factor_f;
    double old_len = (double)original_max_position_embeddings;
    double low_wavelen = old_len / low, high_wavelen = old_len / high;
    const double two_pi = 2.0 * 3.14159265358979323846;
    for (int i = 0; i < head_dim / 2; ++i) {
        double f = (double)out[i];
        double wavelen = two_pi / f;
        double scaled = f;
        if (wavelen > low_wavelen) {
            scaled = f / factor;
        } else if (wavelen >= high_wavelen) {
            double smooth = (old_len / wavelen - low) / (high - low);
            scaled = (1.0 - smooth) * (f / factor) + smooth * f;
        }
        out[i] = (float)scaled;
    }
}

/* ------------------------------------------------------------------------ */
/* Embedding gather: src/kernels/embedding.cu:25-35 (row copy, ids unchecked).*/
/* ------------------------------------------------------------------------ */
ORC_API void orc_embedding_lookup(uint16_t* out, const uint16_t* table, const int32_t* ids,
                                  long num_tokens, int hidden_dim) {
    for (long i = 0; i < num_tokens; ++i)
        memcpy(out + (size_t)i * hidden_dim, table + (size_t)ids[i] * hidden_dim,
               (size_t)hidden_dim * 2);
}

/* ------------------------------------------------------------------------ */
/* Row-broadcast bias add (Qwen2 q/k/v projections):                         */
/* tests/kernels/test_bias.cpp:33-45 (host reference of src/kernels/bias.cu:15-28). */
/* out = bf16(float(x) + float(bias[c])); may run in place.                  */
/* ------------------------------------------------------------------------ */
ORC_API void orc_add_rows(uint16_t* out, const uint16_t* x, const uint16_t* bias, long n, int dim) {
    for (long r = 0; r < n; ++r)
        for (int c = 0; c < dim; ++c) {
            size_t i = (size_t)r * dim + c;
            out[i] = orc_f32_to_bf16(orc_bf16_to_f32(x[i]) + orc_bf16_to_f32(bias[c]));
        }
}

/* ------------------------------------------------------------------------ */
/* Decode attention over the FP8 cache: the formula of the reference's naive  */
/* kernel (src/kernels/attention.cu:31-86 at n_new == 1, which its own        */
/* tests/kernels/test_flash_decode.cpp:117-126 uses as the oracle of          */
/* flash_decode_split_bf16): scores q . (code * k_scale) * scale over keys     */
/* 0..cache_len, softmax, weighted sum of code * v_scale, bf16 output.  The   */
/* reference evaluates it in fp32 in a kernel-specific order and documents    */
/* that orders differ "in the last bits, not in value"                        */
/* (include/runtherder/kernels/flash_decode.cuh:45-46); this restatement       */
/* evaluates it in double, so it is the value every order approximates.       */
/* out_f32 (optional) receives the unrounded result.  No host counterpart in  */
/* the reference: pinned on the GPU, within one bf16 ulp, to the reference's  */
/* naive and split kernels built for sm_100a.                                 */
/* ------------------------------------------------------------------------ */
ORC_API void orc_attention_decode_fp8(uint16_t* out, float* out_f32, const uint16_t* q, const uint8_t* k,
                                      const uint8_t* v, const float* k_scale, const float* v_scale,
                                      int cache_len, int num_q_heads, int num_kv_heads, int head_dim,
                                      float scale, double* score_buf /* cache_len + 1 doubles */) {
    const int n_keys = cache_len + 1;
    const int group = num_q_heads / num_kv_heads;
    for (int qh = 0; qh < num_q_heads; ++qh) {
        const int kvh = qh / group;
        const uint16_t* q_row = q + (size_t)qh * head_dim;
        double m = -INFINITY;
        for (int j = 0; j < n_keys; ++j) {
            const size_t row = (size_t)j * num_kv_heads + kvh;
            double s = 0.0;
            for (int d = 0; d < head_dim; ++d)
                s += (double)orc_bf16_to_f32(q_row[d]) *
                     ((double)orc_e4m3_to_f32(k[row * head_dim + d]) * (double)k_scale[row]);
            s *= (double)scale;
            score_buf[j] = s;
            if (s > m) m = s;
        }
        double denom = 0.0;
        for (int j = 0; j < n_keys; ++j) {
            score_buf[j] = exp(score_buf[j] - m);
            denom += score_buf[j];
        }
        for (int d = 0; d < head_dim; ++d) {
            double acc = 0.0;
            for (int j = 0; j < n_keys; ++j) {
                const size_t row = (size_t)j * num_kv_heads + kvh;
                acc += score_buf[j] * ((double)orc_e4m3_to_f32(v[row * head_dim + d]) * (double)v_scale[row]);
            }
            const float r = (float)(acc / denom);
            if (out_f32) out_f32[(size_t)qh * head_dim + d] = r;
            out[(size_t)qh * head_dim + d] = orc_f32_to_bf16(r);
        }
    }
}

/* The same for n_new query tokens (prefill / chunked prefill): token t attends */
/* keys 0..cache_len + t (src/kernels/attention.cu:45-49).  q, out: [n_new, Hq, D]. */
ORC_API void orc_attention_causal_fp8(uint16_t* out, float* out_f32, const uint16_t* q, const uint8_t* k,
                                      const uint8_t* v, const float* k_scale, const float* v_scale, int n_new,
                                      int cache_len, int num_q_heads, int num_kv_heads, int head_dim, float scale,
                                      double* score_buf /* cache_len + n_new doubles */) {
    const size_t row = (size_t)num_q_heads * head_dim;
    for (int t = 0; t < n_new; ++t)
        orc_attention_decode_fp8(out + t * row, out_f32 ? out_f32 + t * row : NULL, q + t * row, k, v, k_scale,
                                 v_scale, cache_len + t, num_q_heads, num_kv_heads, head_dim, scale, score_buf);
}

/* ------------------------------------------------------------------------ */
/* Chains, as the reference's layer composition issues them.  Each stage     */
/* rounds to bf16 exactly where the reference stores a bf16 tensor.          */
/* ------------------------------------------------------------------------ */

/* residual add + RMSNorm, then INT8 quantisation of the stored bf16 result:
 * src/model/supported/llama/llama3.cu:216-226 calling src/kernels/matmul.cu:138.
 * residual == NULL selects the plain norm (layer 0, llama3.cu:211-214). */
ORC_API void orc_rmsnorm_add_quant_int8(int8_t* q, float* x_scale, uint16_t* h_out, uint16_t* y,
                                        const uint16_t* x, const uint16_t* residual,
                                        const uint16_t* g, long num_tokens, int hidden_dim,
                                        float eps, float* h_tmp) {
    if (residual) orc_rmsnorm_add(y, h_out, x, residual, g, num_tokens, hidden_dim, eps, h_tmp);
    else orc_rmsnorm(y, x, g, num_tokens, hidden_dim, eps);
    orc_quantize_per_token_int8(q, x_scale, y, num_tokens, hidden_dim);
}

/* SwiGLU into the gate buffer, then INT8 quantisation inside the down
 * projection: llama3.cu:248-251 + matmul.cu:138. */
ORC_API void orc_swiglu_quant_int8(int8_t* q, float* x_scale, uint16_t* y, const uint16_t* gate,
                                   const uint16_t* up, long num_tokens, int inter_dim) {
    orc_swiglu(y, gate, up, (size_t)num_tokens * inter_dim);
    orc_quantize_per_token_int8(q, x_scale, y, num_tokens, inter_dim);
}

/* [Qwen3: per-head RMSNorm of q and k in place, qwen3.cu:189-194] -> RoPE in
 * place (llama3.cu:228-230) -> KVCache::append = FP8 quantisation of the
 * rotated k and of v at slot at_pos (include/runtherder/engine/kv_cache.h:62-78).
 * q and k are updated in place; q_norm/k_norm may be NULL. */
ORC_API void orc_rope_kv_fp8(uint16_t* q, uint16_t* k, const uint16_t* v, const uint16_t* q_norm,
                             const uint16_t* k_norm, float eps, const int32_t* positions,
                             const float* inv_freq, uint8_t* k_cache, float* k_scale,
                             uint8_t* v_cache, float* v_scale, int at_pos, long seq_len,
                             int num_q_heads, int num_kv_heads, int head_dim) {
    if (q_norm) orc_rmsnorm(q, q, q_norm, seq_len * num_q_heads, head_dim, eps);
    if (k_norm) orc_rmsnorm(k, k, k_norm, seq_len * num_kv_heads, head_dim, eps);
    orc_rope_table(q, positions, inv_freq, seq_len, num_q_heads, head_dim);
    orc_rope_table(k, positions, inv_freq, seq_len, num_kv_heads, head_dim);
    orc_quantize_kv_fp8(k_cache, k_scale, k, at_pos, num_kv_heads, seq_len * num_kv_heads, head_dim);
    orc_quantize_kv_fp8(v_cache, v_scale, v, at_pos, num_kv_heads, seq_len * num_kv_heads, head_dim);
}

/* ------------------------------------------------------------------------ */
/* Synthetic inputs.  A counter-based generator that the CUDA library        */
/* implements identically on the device, so any slice of a multi-gigabyte    */
/* benchmark tensor can be regenerated here.  Not derived from the reference.*/
/* ------------------------------------------------------------------------ */
static inline uint64_t mix64(uint64_t z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
static inline uint64_t stream_key(uint64_t seed, uint64_t tensor_id) {
    return mix64(mix64(seed + 0x9E3779B97F4A7C15ull) ^ (tensor_id * 0xD1B54A32D192ED03ull + 0x632BE59BD9B4E019ull));
}
static inline uint64_t draw64(uint64_t key, uint64_t counter) {
    return mix64(key + (counter + 1) * 0x9E3779B97F4A7C15ull);
}

/* Irwin-Hall(12) of 16-bit uniforms: mean 0, variance 1, exact in fp32. */
static inline float synth_normal(uint64_t key, uint64_t idx) {
    uint32_t s = 0;
    for (int k = 0; k < 3; ++k) {
        uint64_t r = draw64(key, 3 * idx + k);
        s += (uint32_t)(r & 0xffff) + (uint32_t)((r >> 16) & 0xffff) +
             (uint32_t)((r >> 32) & 0xffff) + (uint32_t)(r >> 48);
    }
    return (float)((int32_t)s - 6 * 65535) * (1.0f / 65536.0f);
}

/* out[i] = bf16(normal(start+i) * std * chan_scale[(start+i) % ncols]) */
ORC_API void orc_synth_normal_bf16(uint16_t* out, size_t count, uint64_t seed, uint64_t tensor_id,
                                   uint64_t start, float std, const float* chan_scale, int ncols) {
    uint64_t key = stream_key(seed, tensor_id);
    for (size_t i = 0; i < count; ++i) {
        uint64_t idx = start + i;
        float v = synth_normal(key, idx) * std;
        if (chan_scale) v = v * chan_scale[idx % (uint64_t)ncols];
        out[i] = orc_f32_to_bf16(v);
    }
}

/* out[i] = bf16(lo + (hi-lo) * u), u = 24 random bits * 2^-24 */
ORC_API void orc_synth_uniform_bf16(uint16_t* out, size_t count, uint64_t seed, uint64_t tensor_id,
                                    uint64_t start, float lo, float hi) {
    uint64_t key = stream_key(seed, tensor_id);
    for (size_t i = 0; i < count; ++i) {
        float u = (float)(uint32_t)(draw64(key, start + i) >> 40) * (1.0f / 16777216.0f);
        float w = (hi - lo) * u;
        out[i] = orc_f32_to_bf16(lo + w);
    }
}

/* out[i] = 64 random bits mod modulus */
ORC_API void orc_synth_ids_i32(int32_t* out, size_t count, uint64_t seed, uint64_t tensor_id,
                               uint64_t start, int32_t modulus) {
    uint64_t key = stream_key(seed, tensor_id);
    for (size_t i = 0; i < count; ++i)
        out[i] = (int32_t)(draw64(key, start + i) % (uint64_t)modulus);
}
