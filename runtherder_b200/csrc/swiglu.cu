// SwiGLU, stand-alone and fused with per-token INT8 quantisation.
//
// Arithmetic per element, exactly as the reference kernel (src/kernels/activation.cu:33-37):
//   s = 1.0f / (1.0f + __expf(-g));  y = bf16_rn((g * s) * u)
// The fused kernel keeps the bf16-rounded products of one token row in registers
// (packed, 4 registers per 8 values), takes the row amax, and emits INT8 codes
// — gate and up are read once, the bf16 product never travels to HBM unless the
// caller asks for it.
#include "rh_common.cuh"

namespace rh {

namespace {

__device__ __forceinline__ float silu_mul(float g, float u) {
    const float s = 1.0f / (1.0f + __expf(-g));
    return g * s * u;
}

__device__ __forceinline__ uint4 swiglu8(const uint4& gv, const uint4& uv) {
    float g[8], u[8], y[8];
    unpack8(gv, g);
    unpack8(uv, u);
#pragma unroll
    for (int j = 0; j < 8; ++j) y[j] = silu_mul(g[j], u[j]);
    return pack8(y);
}

constexpr int kElemThreads = 256;
constexpr int kElemUnroll = 4;

// Flat elementwise kernel: each CTA covers kElemThreads*kElemUnroll consecutive vectors,
// all loads of a thread issued before its first store.
__global__ void __launch_bounds__(kElemThreads) swiglu_kernel(uint4* __restrict__ y, const uint4* gate,
                                                              const uint4* up, long long n_vec) {
    const long long base = static_cast<long long>(blockIdx.x) * (kElemThreads * kElemUnroll) + threadIdx.x;
    uint4 gv[kElemUnroll], uv[kElemUnroll];
#pragma unroll
    for (int k = 0; k < kElemUnroll; ++k) {
        const long long i = base + k * kElemThreads;
        if (i < n_vec) {
            gv[k] = ld_stream(gate + i);
            uv[k] = ld_stream(up + i);
        }
    }
#pragma unroll
    for (int k = 0; k < kElemUnroll; ++k) {
        const long long i = base + k * kElemThreads;
        if (i < n_vec) st_vec(y + i, swiglu8(gv[k], uv[k]));
    }
}

template <int kThreads, int VPT, bool kStoreY>
__global__ void __launch_bounds__(kThreads, (kThreads == 512 ? 2 : 4))
swiglu_quant_kernel(int8_t* __restrict__ q, float* __restrict__ x_scale, void* y, const void* gate,
                    const void* up, long long num_tokens, int inter_dim) {
    constexpr int kWarps = kThreads / 32;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int n_vecs = inter_dim / kVec;
    __shared__ float s_mx[2][kWarps];

    int parity = 0;
    for (long long row = blockIdx.x; row < num_tokens; row += gridDim.x, parity ^= 1) {
        const size_t row_off = static_cast<size_t>(row) * n_vecs;
        const uint4* g_row = static_cast<const uint4*>(gate) + row_off;
        const uint4* u_row = static_cast<const uint4*>(up) + row_off;

        // Two slots (four 128-bit loads) are in flight per thread at a time; the products are
        // kept packed, so a 14336-wide row costs 16 registers per thread at 512 threads.
        uint4 yw[VPT];
        uint32_t m2 = 0u;
#pragma unroll
        for (int s0 = 0; s0 < VPT; s0 += 2) {
            uint4 gv[2], uv[2];
#pragma unroll
            for (int k = 0; k < 2; ++k) {
                const int i = tid + (s0 + k) * kThreads;
                if (s0 + k < VPT && i < n_vecs) {
                    gv[k] = ld_stream(g_row + i);
                    uv[k] = ld_stream(u_row + i);
                }
            }
#pragma unroll
            for (int k = 0; k < 2; ++k) {
                const int s = s0 + k;
                const int i = tid + s * kThreads;
                if (s < VPT && i < n_vecs) {
                    yw[s] = swiglu8(gv[k], uv[k]);
                    if constexpr (kStoreY) st_vec(static_cast<uint4*>(y) + row_off + i, yw[s]);
                    m2 = max_nan_bf16x2(m2, abs_bf16x2(yw[s].x));
                    m2 = max_nan_bf16x2(m2, abs_bf16x2(yw[s].y));
                    m2 = max_nan_bf16x2(m2, abs_bf16x2(yw[s].z));
                    m2 = max_nan_bf16x2(m2, abs_bf16x2(yw[s].w));
                }
            }
            asm volatile("" ::: "memory");  // keep the next pair's loads behind this pair's math
        }
        // The reference's amax (fmaxf) skips NaN; redo this thread's share that way if it holds
        // a non-finite value, and let those elements take the exact conversion path below.
        const float m_lo = bf_lo(m2), m_hi = bf_hi(m2);
        const bool finite = (m_lo <= 3.0e38f) && (m_hi <= 3.0e38f);
        float amax = fmaxf(m_lo, m_hi);
        if (!finite) {
            amax = 0.0f;
#pragma unroll
            for (int s = 0; s < VPT; ++s) {
                const int i = tid + s * kThreads;
                if (i < n_vecs) {
                    float f[8];
                    unpack8(yw[s], f);
#pragma unroll
                    for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(f[j]));
                }
            }
        }
        amax = group_max<32>(amax);
        if (lane == 0) s_mx[parity][warp] = amax;
        __syncthreads();
        amax = group_max<kWarps>(s_mx[parity][lane & (kWarps - 1)]);

        const float inv = (amax > 0.0f) ? (127.0f / amax) : 0.0f;
        if (tid == 0) x_scale[row] = amax / 127.0f;
        const bool fast = finite && inv <= 3.0e38f;
        uint2* q_row = reinterpret_cast<uint2*>(q) + row_off;
#pragma unroll
        for (int s = 0; s < VPT; ++s) {
            const int i = tid + s * kThreads;
            if (i < n_vecs) {
                if (fast) {
                    st_vec8(q_row + i, pack_int8x8_fast(yw[s], inv));
                } else {
                    float f[8];
                    unpack8(yw[s], f);
                    st_vec8(q_row + i, pack_int8x8(f, inv));
                }
            }
        }
    }
}

template <int kThreads, int VPT>
int launch_swiglu_quant(int8_t* q, float* x_scale, void* y, const void* gate, const void* up,
                        long long num_tokens, int inter_dim, cudaStream_t stream) {
    static const int resident_y = host::resident_ctas(
        reinterpret_cast<const void*>(&swiglu_quant_kernel<kThreads, VPT, true>), kThreads);
    static const int resident_n = host::resident_ctas(
        reinterpret_cast<const void*>(&swiglu_quant_kernel<kThreads, VPT, false>), kThreads);
    const int tuned = host::tuning(host::kSwigluCtasPerSm);
    const long long cap =
        static_cast<long long>(host::num_sms()) * (tuned > 0 ? tuned : (y ? resident_y : resident_n));
    const int grid = static_cast<int>(num_tokens < cap ? num_tokens : cap);
    if (y) swiglu_quant_kernel<kThreads, VPT, true><<<grid, kThreads, 0, stream>>>(q, x_scale, y, gate, up, num_tokens, inter_dim);
    else swiglu_quant_kernel<kThreads, VPT, false><<<grid, kThreads, 0, stream>>>(q, x_scale, y, gate, up, num_tokens, inter_dim);
    return host::check_launch("swiglu_quant_kernel");
}

}  // namespace

}  // namespace rh

using namespace rh;

extern "C" int rh_swiglu_bf16(void* y, const void* gate, const void* up, long long n, void* stream) {
    RH_REQUIRE(y && gate && up, RH_ERR_INVALID_ARG, "rh_swiglu_bf16: null pointer");
    RH_REQUIRE(n >= kVec, RH_ERR_UNSUPPORTED_DIM, "rh_swiglu_bf16: n must be >= 8 (got %lld)", n);
    RH_REQUIRE(n % kVec == 0, RH_ERR_UNSUPPORTED_DIM, "rh_swiglu_bf16: n must be a multiple of 8 (got %lld)", n);
    RH_REQUIRE(host::aligned16(y) && host::aligned16(gate) && host::aligned16(up), RH_ERR_MISALIGNED,
               "rh_swiglu_bf16: pointers must be 16-byte aligned");
    const long long n_vec = n / kVec;
    const long long per_cta = kElemThreads * kElemUnroll;
    const long long grid = (n_vec + per_cta - 1) / per_cta;
    RH_REQUIRE(grid <= 0x7fffffffLL, RH_ERR_UNSUPPORTED_DIM, "rh_swiglu_bf16: n too large");
    swiglu_kernel<<<static_cast<unsigned>(grid), kElemThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<uint4*>(y), static_cast<const uint4*>(gate), static_cast<const uint4*>(up), n_vec);
    return host::check_launch("swiglu_kernel");
}

extern "C" int rh_swiglu_quant_int8(int8_t* q, float* x_scale, void* y_or_null, const void* gate,
                                    const void* up, int num_tokens, int inter_dim, void* stream) {
    RH_REQUIRE(q && x_scale && gate && up, RH_ERR_INVALID_ARG, "rh_swiglu_quant_int8: null pointer");
    RH_REQUIRE(num_tokens >= 1, RH_ERR_INVALID_ARG, "rh_swiglu_quant_int8: num_tokens must be >= 1");
    RH_REQUIRE(inter_dim >= kVec && inter_dim % kVec == 0, RH_ERR_UNSUPPORTED_DIM,
               "rh_swiglu_quant_int8: inter_dim must be a positive multiple of 8 (got %d)", inter_dim);
    RH_REQUIRE(inter_dim <= RH_MAX_ROW_DIM, RH_ERR_UNSUPPORTED_DIM,
               "rh_swiglu_quant_int8: inter_dim %d exceeds %d", inter_dim, RH_MAX_ROW_DIM);
    RH_REQUIRE(host::aligned16(gate) && host::aligned16(up) && host::aligned16(y_or_null) &&
                   (reinterpret_cast<uintptr_t>(q) & 7u) == 0,
               RH_ERR_MISALIGNED, "rh_swiglu_quant_int8: pointers must be 16-byte aligned (q: 8)");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int n_vecs = inter_dim / kVec;
    if (n_vecs <= 256) return launch_swiglu_quant<256, 1>(q, x_scale, y_or_null, gate, up, num_tokens, inter_dim, s);
    if (n_vecs <= 512) return launch_swiglu_quant<256, 2>(q, x_scale, y_or_null, gate, up, num_tokens, inter_dim, s);
    if (n_vecs <= 1024) return launch_swiglu_quant<512, 2>(q, x_scale, y_or_null, gate, up, num_tokens, inter_dim, s);
    if (n_vecs <= 1536) return launch_swiglu_quant<512, 3>(q, x_scale, y_or_null, gate, up, num_tokens, inter_dim, s);
    return launch_swiglu_quant<512, 4>(q, x_scale, y_or_null, gate, up, num_tokens, inter_dim, s);
}
