// Token-embedding gather: out[i, :] = table[ids[i], :], a pure row copy
// (reference: src/kernels/embedding.cu:17-36; ids are not validated there either).
//
// Rows of the table are scattered, so each row is one contiguous burst of
// hidden_dim*2 bytes.  A CTA of 128 threads copies a row with up to four 128-bit
// loads in flight per thread, and walks rows blockIdx.x, +gridDim.x, ... with the
// next row's id fetched one iteration ahead so the id -> row dependency is off the
// critical path.
#include "rh_common.cuh"

namespace rh {

namespace {

constexpr int kEmbThreads = 128;
constexpr int kEmbUnroll = 4;

__global__ void __launch_bounds__(kEmbThreads) embedding_kernel(uint4* __restrict__ out,
                                                                const uint4* __restrict__ table,
                                                                const int* __restrict__ ids,
                                                                long long num_tokens, int n_vecs) {
    long long row = blockIdx.x;
    pdl_enter();
    if (row >= num_tokens) return;
    int id = __ldg(ids + row);
    while (row < num_tokens) {
        const long long next = row + gridDim.x;
        int id_next = 0;
        if (next < num_tokens) id_next = __ldg(ids + next);
        const uint4* src = table + static_cast<size_t>(id) * n_vecs;
        uint4* dst = out + static_cast<size_t>(row) * n_vecs;
        for (int base = threadIdx.x; base < n_vecs; base += kEmbThreads * kEmbUnroll) {
            uint4 v[kEmbUnroll];
#pragma unroll
            for (int k = 0; k < kEmbUnroll; ++k) {
                const int i = base + k * kEmbThreads;
                if (i < n_vecs) v[k] = ld_stream_ro(src + i);
            }
#pragma unroll
            for (int k = 0; k < kEmbUnroll; ++k) {
                const int i = base + k * kEmbThreads;
                if (i < n_vecs) st_vec(dst + i, v[k]);
            }
        }
        row = next;
        id = id_next;
    }
}

// y[m,n] = bf16((float(acc) * x_scale[row]) * float(w_scale[col])): the epilogue of the
// W8A8 GEMM (reference: src/kernels/quantization.cu:153-171), four columns per thread when
// n allows 16-byte accumulator loads.
template <bool kVec4>
__global__ void __launch_bounds__(256) dequant_w8a8_kernel(__nv_bfloat16* __restrict__ y,
                                                           const int32_t* __restrict__ acc,
                                                           const float* __restrict__ x_scale,
                                                           const __nv_bfloat16* __restrict__ w_scale,
                                                           long long m, int n) {
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    pdl_enter();
    if constexpr (kVec4) {
        const int n4 = n >> 2;
        const long long total = m * n4;
        for (long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total; idx += stride) {
            const long long row = idx / n4;
            const int c4 = static_cast<int>(idx - row * n4);
            const int4 a = *reinterpret_cast<const int4*>(acc + row * n + 4 * c4);
            const uint2 w = __ldg(reinterpret_cast<const uint2*>(w_scale) + c4);
            const float xs = __ldg(x_scale + row);
            const float v0 = static_cast<float>(a.x) * xs * bf_lo(w.x);
            const float v1 = static_cast<float>(a.y) * xs * bf_hi(w.x);
            const float v2 = static_cast<float>(a.z) * xs * bf_lo(w.y);
            const float v3 = static_cast<float>(a.w) * xs * bf_hi(w.y);
            *reinterpret_cast<uint2*>(y + row * n + 4 * c4) = make_uint2(pack_bf16x2(v0, v1), pack_bf16x2(v2, v3));
        }
    } else {
        const long long total = m * n;
        for (long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total; idx += stride) {
            const long long row = idx / n;
            const int col = static_cast<int>(idx - row * n);
            const float v = static_cast<float>(acc[idx]) * x_scale[row] * __bfloat162float(w_scale[col]);
            y[idx] = __float2bfloat16(v);
        }
    }
}

// q[r,:] += q_bias, k[r,:] += k_bias, v[r,:] += v_bias in place, each output bf16(float(x) + float(b))
// (reference: src/kernels/bias.cu:15-60, Qwen2's projections).  One 128-bit vector per thread over the
// concatenated [n, q_vecs + 2*kv_vecs] index space; the fp32 adds are issued in pairs.
__global__ void __launch_bounds__(256) qkv_bias_add_kernel(uint4* __restrict__ q, uint4* __restrict__ k,
                                                           uint4* __restrict__ v, const uint4* __restrict__ qb,
                                                           const uint4* __restrict__ kb, const uint4* __restrict__ vb,
                                                           long long total, int q_vecs, int kv_vecs) {
    const int row_vecs = q_vecs + 2 * kv_vecs;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    pdl_enter();
    for (long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total; idx += stride) {
        const long long row = idx / row_vecs;
        int col = static_cast<int>(idx - row * row_vecs);
        uint4* x;
        const uint4* b;
        if (col < q_vecs) {
            x = q + row * q_vecs + col; b = qb + col;
        } else if ((col -= q_vecs) < kv_vecs) {
            x = k + row * kv_vecs + col; b = kb + col;
        } else {
            col -= kv_vecs;
            x = v + row * kv_vecs + col; b = vb + col;
        }
        const uint4 xv = ld_stream(x), bv = ld_weight(b);
        const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w}, bw[4] = {bv.x, bv.y, bv.z, bv.w};
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 r = add2_rn(bf2_to_f2(xw[j]), bf2_to_f2(bw[j]));
            o[j] = pack_bf16x2(r.x, r.y);
        }
        st_vec(x, make_uint4(o[0], o[1], o[2], o[3]));
    }
}

// Device-side replacements for the per-step host work of the decode loop (reference:
// LlamaModel::stage, src/model/supported/llama/llama.cu:266-274, and EngineContext::set_decode_pos,
// include/runtherder/engine/context.h:41-45 — three synchronous cudaMemcpy per generated token).
__global__ void stage_positions_kernel(int* __restrict__ positions, int* __restrict__ decode_pos, int start_pos, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    pdl_enter();
    if (i < n) positions[i] = start_pos + i;            // std::iota(positions, start_pos)
    if (i == 0 && decode_pos != nullptr) *decode_pos = start_pos;
}
__global__ void decode_advance_kernel(int* __restrict__ token_slot, int* __restrict__ position, int* __restrict__ decode_pos,
                                      const int* __restrict__ next_token, int step) {
    pdl_enter();
    if (threadIdx.x == 0 && blockIdx.x == 0) {
        if (token_slot != nullptr && next_token != nullptr) *token_slot = *next_token;
        if (position != nullptr) *position += step;
        if (decode_pos != nullptr) *decode_pos += step;
    }
}

}  // namespace

}  // namespace rh

using namespace rh;

extern "C" int rh_stage_positions(int* positions, int* decode_pos_or_null, int start_pos, int n, void* stream) {
    RH_REQUIRE(positions != nullptr, RH_ERR_INVALID_ARG, "rh_stage_positions: null pointer");
    RH_REQUIRE(n >= 1, RH_ERR_INVALID_ARG, "rh_stage_positions: stage needs at least one token");
    RH_REQUIRE(start_pos >= 0, RH_ERR_INVALID_ARG, "rh_stage_positions: start_pos must be >= 0");
    host::launch<stage_positions_kernel>(dim3((n + 255) / 256), dim3(256), 0, static_cast<cudaStream_t>(stream), positions, decode_pos_or_null, start_pos, n);
    return host::check_launch("stage_positions_kernel");
}

extern "C" int rh_decode_advance(int* token_slot_or_null, int* position_or_null, int* decode_pos_or_null,
                                 const int* next_token_or_null, int step, void* stream) {
    RH_REQUIRE(position_or_null || decode_pos_or_null || token_slot_or_null, RH_ERR_INVALID_ARG,
               "rh_decode_advance: nothing to advance");
    RH_REQUIRE(step >= 0, RH_ERR_INVALID_ARG, "rh_decode_advance: step must be >= 0");
    host::launch<decode_advance_kernel>(dim3(1), dim3(32), 0, static_cast<cudaStream_t>(stream), token_slot_or_null, position_or_null,
                                                                         decode_pos_or_null, next_token_or_null, step);
    return host::check_launch("decode_advance_kernel");
}

extern "C" int rh_qkv_bias_add_bf16(void* q, void* k, void* v, const void* q_bias, const void* k_bias,
                                    const void* v_bias, int n, int q_dim, int kv_dim, void* stream) {
    RH_REQUIRE(q && k && v && q_bias && k_bias && v_bias, RH_ERR_INVALID_ARG, "rh_qkv_bias_add_bf16: null pointer");
    RH_REQUIRE(n >= 1, RH_ERR_INVALID_ARG, "rh_qkv_bias_add_bf16: n must be >= 1");
    RH_REQUIRE(q_dim >= kVec && kv_dim >= kVec, RH_ERR_UNSUPPORTED_DIM, "rh_qkv_bias_add_bf16: q_dim and kv_dim must be >= 8");
    RH_REQUIRE(q_dim % kVec == 0 && kv_dim % kVec == 0, RH_ERR_UNSUPPORTED_DIM,
               "rh_qkv_bias_add_bf16: q_dim and kv_dim must be multiples of 8");
    RH_REQUIRE(host::aligned16(q) && host::aligned16(k) && host::aligned16(v) && host::aligned16(q_bias) &&
                   host::aligned16(k_bias) && host::aligned16(v_bias),
               RH_ERR_MISALIGNED, "rh_qkv_bias_add_bf16: pointers must be 16-byte aligned");
    const int q_vecs = q_dim / kVec, kv_vecs = kv_dim / kVec;
    const long long total = static_cast<long long>(n) * (q_vecs + 2 * kv_vecs);
    long long grid = (total + 255) / 256;
    const long long cap = static_cast<long long>(host::num_sms()) * 16;
    if (grid > cap) grid = cap;
    host::launch<qkv_bias_add_kernel>(dim3(static_cast<unsigned>(grid)), dim3(256), 0, static_cast<cudaStream_t>(stream), 
        static_cast<uint4*>(q), static_cast<uint4*>(k), static_cast<uint4*>(v), static_cast<const uint4*>(q_bias),
        static_cast<const uint4*>(k_bias), static_cast<const uint4*>(v_bias), total, q_vecs, kv_vecs);
    return host::check_launch("qkv_bias_add_kernel");
}

extern "C" int rh_embedding_lookup_bf16(void* out, const void* table, const int* token_ids,
                                        int num_tokens, int hidden_dim, void* stream) {
    RH_REQUIRE(out && table && token_ids, RH_ERR_INVALID_ARG, "rh_embedding_lookup_bf16: null pointer");
    RH_REQUIRE(num_tokens >= 1, RH_ERR_INVALID_ARG, "rh_embedding_lookup_bf16: num_tokens must be >= 1");
    RH_REQUIRE(hidden_dim >= kVec && hidden_dim % kVec == 0, RH_ERR_UNSUPPORTED_DIM,
               "rh_embedding_lookup_bf16: hidden_dim must be a positive multiple of 8 (got %d)", hidden_dim);
    RH_REQUIRE(host::aligned16(out) && host::aligned16(table), RH_ERR_MISALIGNED,
               "rh_embedding_lookup_bf16: pointers must be 16-byte aligned");
    int per_sm = host::tuning(host::kEmbedCtasPerSm);
    if (per_sm <= 0) per_sm = 64;   // pure copy: resident CTAs = bytes in flight
    const long long cap = static_cast<long long>(host::num_sms()) * per_sm;
    const int grid = static_cast<int>(num_tokens < cap ? num_tokens : cap);
    host::launch<embedding_kernel>(dim3(grid), dim3(kEmbThreads), 0, static_cast<cudaStream_t>(stream), 
        static_cast<uint4*>(out), static_cast<const uint4*>(table), token_ids, num_tokens, hidden_dim / kVec);
    return host::check_launch("embedding_kernel");
}

extern "C" int rh_dequantize_w8a8(void* y, const int32_t* acc, const float* x_scale, const void* w_scale,
                                  int m, int n, void* stream) {
    RH_REQUIRE(y && acc && x_scale && w_scale, RH_ERR_INVALID_ARG, "rh_dequantize_w8a8: null pointer");
    RH_REQUIRE(m >= 1, RH_ERR_INVALID_ARG, "rh_dequantize_w8a8: m must be >= 1");
    RH_REQUIRE(n >= 1, RH_ERR_INVALID_ARG, "rh_dequantize_w8a8: n must be >= 1");
    const bool vec4 = (n % 4 == 0) && host::aligned16(acc) && (reinterpret_cast<uintptr_t>(y) & 7u) == 0 &&
                      (reinterpret_cast<uintptr_t>(w_scale) & 7u) == 0;
    const long long work = vec4 ? static_cast<long long>(m) * (n / 4) : static_cast<long long>(m) * n;
    long long grid = (work + 255) / 256;
    const long long cap = static_cast<long long>(host::num_sms()) * 16;
    if (grid > cap) grid = cap;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (vec4)
        host::launch<dequant_w8a8_kernel<true>>(dim3(static_cast<unsigned>(grid)), dim3(256), 0, s, 
            static_cast<__nv_bfloat16*>(y), acc, x_scale, static_cast<const __nv_bfloat16*>(w_scale), m, n);
    else
        host::launch<dequant_w8a8_kernel<false>>(dim3(static_cast<unsigned>(grid)), dim3(256), 0, s, 
            static_cast<__nv_bfloat16*>(y), acc, x_scale, static_cast<const __nv_bfloat16*>(w_scale), m, n);
    return host::check_launch("dequant_w8a8_kernel");
}
