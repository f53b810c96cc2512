/*
 * rh_kernels.h — C ABI of librh_kernels.so: B200 (sm_100a) implementations of
 * runtherder's row-wise decoder-layer kernels.
 *
 * Conventions
 *  - Every pointer is a DEVICE pointer unless the parameter is documented as host.
 *    bf16 tensors are passed as void* (16-bit patterns), FP8 E4M3 as uint8_t*.
 *  - `stream` is a cudaStream_t passed as void* (NULL = legacy default stream).
 *  - All work is enqueued on `stream`; no kernel entry point synchronises, allocates or
 *    keeps a pointer, so every such call may be recorded into a CUDA graph.  positions /
 *    at_pos / token ids are read on the device at execution time.  The exceptions are the
 *    diagnostics, each documented where it is declared: rh_selftest, rh_selftest_static,
 *    rh_device_error, rh_selfcheck_bounded_wait and rh_selfcheck_role_wait synchronise (the
 *    first and the last two also allocate), and rh_init is host-side set-up.
 *  - Row starts must be 16-byte aligned (bf16 row length a multiple of 8).
 *  - Return value: RH_OK or an rh_status error; rh_last_error_string() gives the
 *    reason for the last failure on the calling thread.  Nothing is launched
 *    when an error is returned.  There is no CPU fallback of any kind.
 *
 * The reference has no C ABI: its boundary is a set of C++ free functions in
 * namespace runtherder::kernels.  Each entry point below names the reference
 * declaration it stands in for (paths relative to the reference's root); the
 * C++ functions with the reference's exact signatures are exported by the same
 * library (see rh_dropin.hpp) and forward to these.
 */
#ifndef RH_KERNELS_H
#define RH_KERNELS_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum rh_status {
    RH_OK = 0,
    RH_ERR_INVALID_ARG = 1,     /* null pointer, non-positive count, eps <= 0, forbidden aliasing */
    RH_ERR_UNSUPPORTED_DIM = 2, /* row length not a multiple of 8 / beyond the supported maximum */
    RH_ERR_MISALIGNED = 3,      /* a pointer is not 16-byte aligned */
    RH_ERR_LAUNCH = 4,          /* the CUDA runtime rejected the launch */
    RH_ERR_CUDA = 5             /* another CUDA runtime call failed (host-buffer helpers only) */
} rh_status;

#define RH_MAX_ROW_DIM 16384 /* longest row of the CTA-per-row kernels (reference: rmsnorm.cu:205-208) */
#define RH_MAX_HEAD_DIM 256  /* reference: rope.cu:12 */

int rh_version(void);

/* Optional one-time preparation of `device` (host-side; may be called from any thread, any number of
 * times): loads the code of every kernel of this library onto the device, opts the kernels that need it
 * in to their dynamic shared memory, caches the occupancy figures their grids are sized with, the SM
 * count and the address of the device error word.  After it, no launch on that device has first-use work
 * left, so even the very first call of an entry point may happen inside stream capture.  Without it each
 * kernel does the same work on its first launch per device (harmless outside capture: the reference runs
 * its first decode step eagerly, src/engine/generator.cu:54-58).  The current device is left unchanged.
 * No counterpart in the reference (its kernels need no set-up). */
int rh_init(int device);
const char* rh_status_string(int status);
const char* rh_last_error_string(void);

/* ---- Drop-in entry points (one per reference kernel) ------------------------------------ */

/* y = (x / rms(x)) * g per row; y may alias x.
 * Replaces runtherder::kernels::rmsnorm_bf16_forward
 * (include/runtherder/kernels/rmsnorm.cuh:15-22, src/kernels/rmsnorm.cu:214-224). */
int rh_rmsnorm_bf16(void* y, const void* x, const void* g, int num_tokens, int hidden_dim, float eps,
                    void* stream);

/* h_out = bf16(x + residual); y = (h / rms(h)) * g with the unrounded fp32 h.
 * h_out may alias residual; y must differ from h_out.
 * Replaces rmsnorm_add_bf16_forward (rmsnorm.cuh:36-45, rmsnorm.cu:226-238). */
int rh_rmsnorm_add_bf16(void* y, void* h_out, const void* x, const void* residual, const void* g,
                        int num_tokens, int hidden_dim, float eps, void* stream);

/* The forward pass's final norm when only the last token feeds lm_head: y_last[hidden_dim] is row
 * num_tokens-1 of what rh_rmsnorm_add_bf16 would write to y for x, residual [num_tokens, hidden_dim];
 * no other row is read, nothing else is written.  Stands in for the rmsnorm_add_bf16_forward call plus
 * the `normed + (n-1) * hidden_dim` slice at src/model/supported/llama/llama3.cu:254-263 (and the same
 * lines of qwen2.cu / qwen3.cu), which normalise all n rows and rewrite the residual stream although
 * nothing reads either again: 8 * hidden_dim * (n-1) bytes per forward at prefill. */
int rh_rmsnorm_add_last_row_bf16(void* y_last, const void* x, const void* residual, const void* g,
                                 int num_tokens, int hidden_dim, float eps, void* stream);

/* Per-token symmetric INT8: x_scale = amax/127, q = clamp(rn(x * (127/amax)), -127, 127);
 * a zero row gives scale 0 and codes 0.
 * Replaces quantize_per_token_int8 (include/runtherder/kernels/quantization.cuh:17-22,
 * src/kernels/quantization.cu:116-149). */
int rh_quantize_per_token_int8(int8_t* q, float* x_scale, const void* x, int num_tokens, int dim,
                               void* stream);

/* y[m,n] = bf16(acc * x_scale[row] * w_scale[col]) — the W8A8 GEMM epilogue.
 * Replaces dequantize_w8a8 (quantization.cuh:31-37, quantization.cu:175-191). */
int rh_dequantize_w8a8(void* y, const int32_t* acc, const float* x_scale, const void* w_scale, int m,
                       int n, void* stream);

/* Per-row FP8 E4M3: scale = amax/448, q = e4m3_satfinite(x * (448/amax)), written at
 * destination row (row + *at_pos * rows_per_pos); *at_pos is read on the device.
 * Replaces quantize_kv_fp8 (quantization.cuh:50-57, quantization.cu:272-309). */
int rh_quantize_kv_fp8(uint8_t* q, float* scale, const void* x, const int* at_pos, int rows_per_pos,
                       int num_rows, int head_dim, void* stream);

/* y = silu(gate) * up over n elements; y may alias gate or up.
 * Replaces swiglu_bf16_forward (include/runtherder/kernels/activation.cuh:16-21,
 * src/kernels/activation.cu:45-58).  n is 64-bit here; the C++ shim keeps the int. */
int rh_swiglu_bf16(void* y, const void* gate, const void* up, long long n, void* stream);

/* In-place rotate-half RoPE on q [T,Hq,D] and k [T,Hkv,D] from a frequency table.
 * Replaces rope_bf16 (include/runtherder/kernels/rope.cuh:16-25, src/kernels/rope.cu:59-81). */
int rh_rope_bf16(void* q, void* k, const int* positions, const float* inv_freq, int seq_len,
                 int num_q_heads, int num_kv_heads, int head_dim, void* stream);

/* out[i,:] = table[ids[i],:].
 * Replaces embedding_lookup_bf16_forward (include/runtherder/kernels/embedding.cuh:14-20,
 * src/kernels/embedding.cu:40-54). */
int rh_embedding_lookup_bf16(void* out, const void* table, const int* token_ids, int num_tokens,
                             int hidden_dim, void* stream);

/* q[r,:] += q_bias, k[r,:] += k_bias, v[r,:] += v_bias in place (Qwen2's projection biases); every
 * output is bf16(float(x) + float(b)).
 * Replaces qkv_bias_add_bf16_forward (include/runtherder/kernels/bias.cuh:20-30,
 * src/kernels/bias.cu:64-90 — a file that does not compile as shipped: line 1 carries a stray token). */
int rh_qkv_bias_add_bf16(void* q, void* k, void* v, const void* q_bias, const void* k_bias,
                         const void* v_bias, int n, int q_dim, int kv_dim, void* stream);

/* Floats of scratch that rh_flash_decode_split_bf16 needs for `max_splits` splits: [Hq, splits] m,
 * then l, then [Hq, splits, head_dim] acc in one slab (0 for non-positive arguments).
 * Replaces flash_split_scratch_floats (include/runtherder/kernels/flash_decode.cuh:11-25). */
size_t rh_flash_split_scratch_floats(int num_q_heads, int head_dim, int max_splits);

/* Split-KV flash decode of one query token over the FP8 cache: out[h,:] = softmax_j(scale * q[h] .
 * K[j,kvh]) V[j,kvh] over keys j = 0 .. *cache_len, K/V = E4M3 code * per-(token, kv head) scale
 * (layout: include/runtherder/attention/kv_view.h:8-19); *cache_len is read on the device.
 * `partial` is caller-owned scratch of rh_flash_split_scratch_floats(Hq, D, num_splits) floats;
 * any num_splits >= 1 is correct at any *cache_len.  head_dim in {32, 64, 128, 256, 512} (512 takes a plain CUDA-core form).  The result
 * differs from a serial fp32 evaluation by float reassociation only (at most 1 bf16 ulp).
 * Replaces flash_decode_split_bf16 (include/runtherder/kernels/flash_decode.cuh:27-62,
 * src/kernels/flash_decode.cu:271-325; called from src/attention/adaptive.cu:30-33). */
int rh_flash_decode_split_bf16(void* out, const void* q, const uint8_t* k, const uint8_t* v,
                               const float* k_scale, const float* v_scale, float* partial, int num_splits,
                               const int* cache_len, int num_q_heads, int num_kv_heads, int head_dim,
                               float scale, void* stream);

/* Causal attention of n_new query tokens over the FP8 cache (prefill, chunked prefill): token t
 * attends keys 0 .. *cache_len + t.  out, q: [n_new, Hq, head_dim] bf16; k, v: [*cache_len + n_new,
 * Hkv, head_dim] E4M3 with per-(token, kv head) scales; *cache_len is read on the device.
 * head_dim must be 128 (as in the reference).  Operands narrow to f16 before the tensor-core
 * products as in the reference (q magnitudes must lie in f16's range); accumulation and softmax
 * are fp32.  Results are within one bf16 ulp of the exact value (tests/test_gpu_flash_prefill.py).
 * The default form runs on tcgen05.mma (one CTA per SM holding 256 or all 512 of its tensor-memory columns for
 * its lifetime; out 16-byte aligned); an out that is only 4-byte aligned takes an mma.sync form.
 * Replaces flash_prefill_bf16 (include/runtherder/kernels/flash_prefill.cuh:27-40,
 * src/kernels/flash_prefill.cu:213-241; called from src/attention/adaptive.cu:37-40). */
int rh_flash_prefill_bf16(void* out, const void* q, const uint8_t* k, const uint8_t* v, const float* k_scale,
                          const float* v_scale, int n_new, const int* cache_len, int num_q_heads,
                          int num_kv_heads, int head_dim, float scale, void* stream);

/* ---- Fused entry points (new; each equals a chain of the reference's calls) --------------- */

/* [residual add +] RMSNorm + per-token INT8 quantisation in one pass over the row.
 * Equals rmsnorm_add_bf16_forward (or rmsnorm_bf16_forward when residual == NULL) followed by
 * quantize_per_token_int8 of the stored bf16 result — the sequence
 * src/model/supported/llama/llama3.cu:211-226 + src/kernels/matmul.cu:138 issues.
 * h_out is written only when residual != NULL (may alias residual); y is optional (NULL skips
 * the bf16 store). */
int rh_rmsnorm_add_quant_int8(int8_t* q, float* x_scale, void* h_out, void* y_or_null, const void* x,
                              const void* residual_or_null, const void* g, int num_tokens,
                              int hidden_dim, float eps, void* stream);

/* SwiGLU + per-token INT8 quantisation of the bf16-rounded product, one pass per row.
 * Equals swiglu_bf16_forward + quantize_per_token_int8 (llama3.cu:248-251 + matmul.cu:138).
 * y is optional and may alias gate or up. */
int rh_swiglu_quant_int8(int8_t* q, float* x_scale, void* y_or_null, const void* gate, const void* up,
                         int num_tokens, int inter_dim, void* stream);

/* [per-head RMSNorm of q and k] + RoPE + FP8 KV-cache append, one launch.
 * Equals (qwen3.cu:189-194 when q_norm/k_norm are given) rmsnorm_bf16_forward on q and k rows,
 * rope_bf16 (llama3.cu:228-230), then KVCache::append = quantize_kv_fp8 of the rotated k and of v
 * (include/runtherder/engine/kv_cache.h:62-78).  q is rotated in place; the rotated bf16 k is
 * written to k_out when it is not NULL (k_out may alias k_in).  k_cache/v_cache/k_scale/v_scale are
 * the layer's slabs ([max_seq, Hkv, D] E4M3 and [max_seq, Hkv] fp32); slot = *at_pos + token.
 * head_dim must be one of 16, 32, 64, 128, 256 (other even head_dims: rh_rope_bf16 followed by
 * rh_quantize_kv_fp8). */
int rh_rope_kv_fp8(void* q, void* k_out_or_null, const void* k_in, const void* v_in,
                   const void* q_norm_or_null, const void* k_norm_or_null, float eps,
                   const int* positions, const float* inv_freq, uint8_t* k_cache, float* k_scale,
                   uint8_t* v_cache, float* v_scale, const int* at_pos, int seq_len, int num_q_heads,
                   int num_kv_heads, int head_dim, void* stream);

/* The same with Qwen2's projection biases folded in (no QK-norm): every q/k/v row is first
 * bf16(float(x) + float(bias)) — q_bias [Hq*D], k_bias and v_bias [Hkv*D] — then rotated / appended.
 * Equals qkv_bias_add_bf16_forward followed by rope_bf16 and KVCache::append
 * (src/model/supported/llama/qwen2.cu:183-191; src/kernels/bias.cu:64-90), one launch and one pass over
 * q/k/v instead of two; q, k_out and both caches are bit-identical to that sequence.  v_in is read
 * only (the separate bias kernel rewrites it in place; nothing reads it afterwards). */
int rh_bias_rope_kv_fp8(void* q, void* k_out_or_null, const void* k_in, const void* v_in, const void* q_bias,
                        const void* k_bias, const void* v_bias, const int* positions, const float* inv_freq,
                        uint8_t* k_cache, float* k_scale, uint8_t* v_cache, float* v_scale, const int* at_pos,
                        int seq_len, int num_q_heads, int num_kv_heads, int head_dim, void* stream);

/* ---- Decode-loop glue on the device ------------------------------------------------------- */

/* positions[i] = start_pos + i for i < n, *decode_pos = start_pos: what LlamaModel::stage
 * (src/model/supported/llama/llama.cu:266-274) and EngineContext::set_decode_pos
 * (include/runtherder/engine/context.h:41-45) do with a host iota and two synchronous copies.
 * start_pos is passed by value: inside a captured graph use rh_decode_advance instead. */
int rh_stage_positions(int* positions, int* decode_pos_or_null, int start_pos, int n, void* stream);

/* End-of-step update for a graph-captured decode loop: *token_slot = *next_token (the sampled id, when
 * both are given), *position += step, *decode_pos += step — all device-resident, so the next replay
 * sees the next position without any host copy. */
int rh_decode_advance(int* token_slot_or_null, int* position_or_null, int* decode_pos_or_null,
                      const int* next_token_or_null, int step, void* stream);

/* ---- Host-side tables (HOST pointers, no GPU involved) ----------------------------------- */

/* out[i] = (float) pow((double)theta, -2i/D), i < D/2.
 * Replaces rope_inv_freq_plain (src/model/supported/llama/llama.cu:128-143). */
int rh_rope_inv_freq_plain(float* out_host, int head_dim, float theta_base);

/* Llama-3 long-context rescaling of the plain table.
 * Replaces rope_inv_freq_llama3 (src/model/supported/llama/llama3.cu:26-60). */
int rh_rope_inv_freq_llama3(float* out_host, int head_dim, float theta_base, float factor,
                            float low_freq_factor, float high_freq_factor,
                            int original_max_position_embeddings);

/* ---- Synthetic benchmark inputs (device generators, counter-based, reproducible) --------- */

/* out[i] = bf16(N(0,1)(start+i) * std * chan_scale[(start+i) % ncols]); chan_scale may be NULL. */
int rh_synth_normal_bf16(void* out, size_t count, uint64_t seed, uint64_t tensor_id, uint64_t start,
                         float std, const float* chan_scale, int ncols, void* stream);
/* out[i] = bf16(U[lo,hi)) */
int rh_synth_uniform_bf16(void* out, size_t count, uint64_t seed, uint64_t tensor_id, uint64_t start,
                          float lo, float hi, void* stream);
/* out[i] = U{0..modulus-1} */
int rh_synth_ids_i32(int32_t* out, size_t count, uint64_t seed, uint64_t tensor_id, uint64_t start,
                     int32_t modulus, void* stream);

/* ---- Self-check ------------------------------------------------------------------------------ */

/* The kernels replace three IEEE divisions of the reference (amax/qmax, qmax/amax, 1/(1+e)) by
 * refined reciprocals.  This runs, on the current device, an exhaustive comparison of those sequences
 * with IEEE division over every operand they can meet and writes mismatch counts to
 * mismatches_host[0..7] (HOST pointer): [0] sigmoid reciprocal with one refinement step (the default), [1] with two, [2],[3] 127/amax and 448/amax, [4],[5] amax/127 and amax/448, [6],[7] unused.
 * Everything the library uses by default must read 0.  Diagnostic: allocates, synchronises. */
int rh_selftest(unsigned int* mismatches_host);

/* rh_selftest without any allocation.  This entry point has no counterpart in the reference; it exists
 * for hosts that cannot call cudaMalloc once they are running — an engine that, like the reference's,
 * hands all device memory to its weight slab, scratch arena and KV cache at start-up, where a later
 * cudaMalloc may fail and in any case stalls the device.  The mismatch counters live in a fixed
 * array inside the library image (RH_SELFTEST_MAX_COUNTERS counters, held on every GPU that loads
 * the library until the process exits).  Writes the first `num_counters` counts of rh_selftest's
 * layout to mismatches_host (HOST pointer); num_counters > RH_SELFTEST_MAX_COUNTERS is rejected with
 * RH_ERR_UNSUPPORTED_DIM.  Work is enqueued on `stream` and the call returns after the stream has
 * drained.  The array is shared by all calls on a device: it is zeroed at the start of each call, and
 * calls whose GPU work overlaps race on it — serialise them.  The first call on a device resolves the
 * array's device address; make it before any stream capture starts. */
#define RH_SELFTEST_MAX_COUNTERS 8
int rh_selftest_static(unsigned int* mismatches_host, int num_counters, void* stream);

/* The staged kernels wait on shared-memory barriers with a poll limit instead of spinning forever.
 * A wait that ran out records (source line << 8 | 1) in a sticky per-device word and the kernel
 * returns early; this reads that word into *error_host (HOST pointer; 0 = no error so far).
 * Synchronises the device. */
int rh_device_error(int* error_host);

/* Failure-detection self-check: one warp waits, with a limit of `polls` (1..65536) polls of up to 20 us
 * each, on a barrier that nothing completes.  The wait must run out: *gave_up_host becomes 1, *error_host
 * the error word the probe recorded (non-zero; a private word — the sticky device error word is not
 * touched), the kernel returns normally and the context stays usable.  Diagnostic: allocates, synchronises. */
int rh_selfcheck_bounded_wait(int polls, int* gave_up_host, int* error_host);

/* The same for the waits between the warp roles of the prefill attention kernel
 * (runtherder_b200/csrc/flash_prefill_ws.cu): warp 0 waits with a limit of `tries` (16..65536) on a barrier
 * that nothing completes and must give up, raising the CTA-wide flag; warp 1, waiting with the kernel's own
 * limit (2^20) on another such barrier, must be released by that flag.  result_host (HOST, 4 ints): [0] 1 if
 * warp 0's wait claimed success (0 expected), [1] the flag (1 expected), [2] the error word the probe recorded
 * (source line << 8 | 1; a private word), [3] the tries warp 1 used (far below 2^20 expected).  The kernel
 * returns normally and the context stays usable.  Diagnostic: allocates, synchronises. */
int rh_selfcheck_role_wait(int tries, int* result_host);

/* ---- Tuning knobs (process-wide; for experiments, defaults are the tuned values) --------- */

/* key: "rows_ctas_per_sm", "swiglu_ctas_per_sm", "rope_warps_per_cta", "embed_ctas_per_sm",
 * "swiglu_rcp_steps" (stand-alone SwiGLU: 1|2 refinement steps, 3 = IEEE division), "swiglu_stages"
 * (depth of the bulk-copy staging ring of the fused SwiGLU kernel, 1 = direct loads), "rows_prefetch"
 * (rows a row kernel keeps in flight through its cp.async ring, 1..3; 4 = plain loads), "rows_smem_h"
 * (1 = keep the fp32 row in registers instead of shared memory), "no_pdl" (1 = launch
 * without the programmatic-dependent-launch attribute; by default each kernel may be scheduled
 * while the previous kernel of its stream drains and orders itself on the device before its first
 * memory access, so stream semantics are unchanged), "prefill_tiles" (1|2: the mma.sync forms of the prefill
 * attention kernel with one or two 16-row tiles per warp; default: the tcgen05 forms with S and O in tensor
 * memory), "prefill_parts" (which tcgen05 form: default the role-split one, with 5 | 6 forcing one | two row
 * blocks per CTA; 1|2|4 = the single-role form with that many threads per score row, 3 = the single-role form
 * with the scores read in accumulator-fragment shape); value <= 0 restores
 * the default.  Returns RH_ERR_INVALID_ARG for an unknown key. */
int rh_tune(const char* key, int value);

#ifdef __cplusplus
}
#endif
#endif /* RH_KERNELS_H */
