// SwiGLU, stand-alone and fused with per-token INT8 quantisation.
//
// Arithmetic per element, exactly as the reference kernel (src/kernels/activation.cu:33-37):
//   s = 1.0f / (1.0f + __expf(-g));  y = bf16_rn((g * s) * u)
// The fused kernel keeps the bf16-rounded products of one token row in registers
// (packed, 4 registers per 8 values), takes the row amax, and emits INT8 codes
// — gate and up are read once, the bf16 product never travels to HBM unless the
// caller asks for it.
#include "rh_common.cuh"
#include "rh_pipeline.cuh"

namespace rh {

namespace {

// Eight products y = bf16((g * s) * u).  kSteps = 0 evaluates the reference's expression verbatim;
// kSteps = 1, 2 use the refined reciprocal on register pairs, and drop to the verbatim expression
// for a vector holding a gate below kGateExactBelow (never the case for real activations).
template <int kSteps>
__device__ __forceinline__ uint4 swiglu8(const uint4& gv, const uint4& uv) {
    const uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w}, uw[4] = {uv.x, uv.y, uv.z, uv.w};
    uint32_t out[4];
    bool exact = (kSteps == 0);
    if (kSteps != 0) {
        const __nv_bfloat162 m = __hmin2(__hmin2(*reinterpret_cast<const __nv_bfloat162*>(&gw[0]),
                                                 *reinterpret_cast<const __nv_bfloat162*>(&gw[1])),
                                         __hmin2(*reinterpret_cast<const __nv_bfloat162*>(&gw[2]),
                                                 *reinterpret_cast<const __nv_bfloat162*>(&gw[3])));
        const uint32_t mw = *reinterpret_cast<const uint32_t*>(&m);
        exact = fminf(bf_lo(mw), bf_hi(mw)) < kGateExactBelow;
    }
    if (exact) {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float2 g = bf2_to_f2(gw[k]), u = bf2_to_f2(uw[k]);
            out[k] = pack_bf16x2(g.x * sigmoid_reference(g.x) * u.x, g.y * sigmoid_reference(g.y) * u.y);
        }
    } else {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float2 g = bf2_to_f2(gw[k]), u = bf2_to_f2(uw[k]);
            const float2 y = mul2_rn(mul2_rn(g, sigmoid2<(kSteps == 0 ? 2 : kSteps)>(g)), u);
            out[k] = pack_bf16x2(y.x, y.y);
        }
    }
    return make_uint4(out[0], out[1], out[2], out[3]);
}

// Fused kernels hoist the range check out of the per-vector path: they always take the refined
// reciprocal, track the smallest gate a thread has seen (one packed min per word), and only a thread
// that met a gate below kGateExactBelow recomputes its vectors with the verbatim expression.
template <int kSteps>
__device__ __forceinline__ uint4 swiglu8_unchecked(const uint4& gv, const uint4& uv) {
    if constexpr (kSteps == 0) return swiglu8<0>(gv, uv);
    const uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w}, uw[4] = {uv.x, uv.y, uv.z, uv.w};
    uint32_t out[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const float2 g = bf2_to_f2(gw[k]), u = bf2_to_f2(uw[k]);
        const float2 y = mul2_rn(mul2_rn(g, sigmoid2<(kSteps == 0 ? 1 : kSteps)>(g)), u);
        out[k] = pack_bf16x2(y.x, y.y);
    }
    return make_uint4(out[0], out[1], out[2], out[3]);
}
constexpr uint32_t kGateMinInit = 0x7f807f80u;   // +Inf, +Inf
__device__ __forceinline__ uint32_t gate_min_acc(uint32_t m, const uint4& gv) {
    __nv_bfloat162 r = *reinterpret_cast<__nv_bfloat162*>(&m);
    r = __hmin2(r, *reinterpret_cast<const __nv_bfloat162*>(&gv.x));
    r = __hmin2(r, *reinterpret_cast<const __nv_bfloat162*>(&gv.y));
    r = __hmin2(r, *reinterpret_cast<const __nv_bfloat162*>(&gv.z));
    r = __hmin2(r, *reinterpret_cast<const __nv_bfloat162*>(&gv.w));
    return *reinterpret_cast<uint32_t*>(&r);
}
__device__ __forceinline__ bool gate_min_needs_exact(uint32_t m) {
    return fminf(bf_lo(m), bf_hi(m)) < kGateExactBelow;
}

constexpr int kElemThreads = 256;
constexpr int kElemUnroll = 4;

// Flat elementwise kernel: each CTA covers kElemThreads*kElemUnroll consecutive vectors,
// all loads of a thread issued before its first store.
template <int kSteps>
__global__ void __launch_bounds__(kElemThreads) swiglu_kernel(uint4* __restrict__ y, const uint4* gate,
                                                              const uint4* up, long long n_vec) {
    const long long base = static_cast<long long>(blockIdx.x) * (kElemThreads * kElemUnroll) + threadIdx.x;
    pdl_enter();
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
        if (i < n_vec) st_vec(y + i, swiglu8<kSteps>(gv[k], uv[k]));
    }
}

template <int kThreads, int VPT, bool kStoreY, int kSteps>
__global__ void __launch_bounds__(kThreads, (kThreads == 512 ? 2 : 4))
swiglu_quant_kernel(int8_t* __restrict__ q, float* __restrict__ x_scale, void* y, const void* gate,
                    const void* up, long long num_tokens, int inter_dim) {
    constexpr int kWarps = kThreads / 32;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int n_vecs = inter_dim / kVec;
    __shared__ float s_mx[2][kWarps];
    pdl_wait();

    int parity = 0;
    for (long long row = blockIdx.x; row < num_tokens; row += gridDim.x, parity ^= 1) {
        if (row + gridDim.x >= num_tokens) pdl_trigger();   // last row of this CTA
        const size_t row_off = static_cast<size_t>(row) * n_vecs;
        const uint4* g_row = static_cast<const uint4*>(gate) + row_off;
        const uint4* u_row = static_cast<const uint4*>(up) + row_off;

        // Two slots (four 128-bit loads) are in flight per thread at a time; the products are
        // kept packed, so a 14336-wide row costs 16 registers per thread at 512 threads.
        uint4 yw[VPT];
        uint32_t m2 = 0u, gmin = kGateMinInit;
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
                    gmin = gate_min_acc(gmin, gv[k]);
                    yw[s] = swiglu8_unchecked<kSteps>(gv[k], uv[k]);
                    if constexpr (kStoreY) st_vec(static_cast<uint4*>(y) + row_off + i, yw[s]);
                    m2 = amax_acc_bf16x2(m2, yw[s].x);
                    m2 = amax_acc_bf16x2(m2, yw[s].y);
                    m2 = amax_acc_bf16x2(m2, yw[s].z);
                    m2 = amax_acc_bf16x2(m2, yw[s].w);
                }
            }
            asm volatile("" ::: "memory");  // keep the next pair's loads behind this pair's math
        }
        if (kSteps != 0 && gate_min_needs_exact(gmin)) {   // a gate below -85: redo this thread's share verbatim
            m2 = 0u;
#pragma unroll
            for (int s = 0; s < VPT; ++s) {
                const int i = tid + s * kThreads;
                if (i < n_vecs) {
                    yw[s] = swiglu8<0>(ld_stream(g_row + i), ld_stream(u_row + i));
                    if constexpr (kStoreY) st_vec(static_cast<uint4*>(y) + row_off + i, yw[s]);
                    m2 = amax_acc_bf16x2(m2, yw[s].x);
                    m2 = amax_acc_bf16x2(m2, yw[s].y);
                    m2 = amax_acc_bf16x2(m2, yw[s].z);
                    m2 = amax_acc_bf16x2(m2, yw[s].w);
                }
            }
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
        amax = warp_max_nonneg(amax);
        if (lane == 0) s_mx[parity][warp] = amax;
        __syncthreads();
        amax = warp_max_nonneg(s_mx[parity][lane & (kWarps - 1)]);

        const float inv = quant_inv_scale<127>(amax);
        if (tid == 0) x_scale[row] = quant_scale<127>(amax);
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

// Staged variant (256 consumer threads + one producer warp).  The producer streams 4 KB slots of gate
// and up through a shared-memory ring with bulk copies, so the bytes in flight no longer depend on how
// many loads a consumer can hold in registers while it is busy with ex2/rcp; consumers take one slot
// at a time.  Same element-to-thread mapping and arithmetic as swiglu_quant_kernel<256, VPT>.
constexpr int kSwiSlotBytes = 256 * 16;

template <int VPT, bool kStoreY, int kSteps>
__global__ void __launch_bounds__(256 + 32, 4)
swiglu_quant_staged_kernel(int8_t* __restrict__ q, float* __restrict__ x_scale, void* y, const void* gate,
                           const void* up, long long num_tokens, int inter_dim, const int stages, int* error_word) {
    constexpr int kThreads = 256, kWarps = 8;
    extern __shared__ __align__(128) unsigned char ring[];
    uint64_t* full = reinterpret_cast<uint64_t*>(ring + static_cast<size_t>(stages) * 2 * kSwiSlotBytes);
    uint64_t* empty = full + stages;
    __shared__ float s_mx[2][kWarps];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int n_vecs = inter_dim / kVec;
    const int slots_per_row = (n_vecs + kThreads - 1) / kThreads;
    if (tid == 0) {
        for (int s = 0; s < stages; ++s) {
            pipe::mbar_init(full + s, 1);
            pipe::mbar_init(empty + s, kWarps);
        }
        pipe::mbar_init_fence();
    }
    __syncthreads();
    pdl_wait();

    if (tid >= kThreads) {
        if (tid == kThreads) {
            int s = 0;
            uint32_t round = 0;
            for (long long row = blockIdx.x; row < num_tokens; row += gridDim.x) {
                const size_t row_off = static_cast<size_t>(row) * n_vecs;
                for (int sl = 0; sl < slots_per_row; ++sl) {
                    if (round > 0 && !pipe::mbar_wait(empty + s, (round - 1) & 1, __LINE__, error_word)) return;
                    const int vec0 = sl * kThreads;
                    const uint32_t bytes = static_cast<uint32_t>(min(kThreads, n_vecs - vec0)) * 16u;
                    unsigned char* dst = ring + static_cast<size_t>(s) * 2 * kSwiSlotBytes;
                    pipe::mbar_expect_tx(full + s, 2 * bytes);
                    pipe::bulk_load(dst, static_cast<const uint4*>(gate) + row_off + vec0, bytes, full + s);
                    pipe::bulk_load(dst + kSwiSlotBytes, static_cast<const uint4*>(up) + row_off + vec0, bytes, full + s);
                    if (++s == stages) { s = 0; ++round; }
                }
            }
        }
        return;
    }

    int parity = 0, s = 0;
    uint32_t phase = 0;
    for (long long row = blockIdx.x; row < num_tokens; row += gridDim.x, parity ^= 1) {
        if (row + gridDim.x >= num_tokens) pdl_trigger();   // last row of this CTA
        const size_t row_off = static_cast<size_t>(row) * n_vecs;
        uint4 yw[VPT];
        uint32_t m2 = 0u, gmin = kGateMinInit;
#pragma unroll
        for (int sl = 0; sl < VPT; ++sl) {
            if (sl < slots_per_row) {
                if (!pipe::mbar_wait(full + s, phase, __LINE__, error_word)) return;
                const unsigned char* src = ring + static_cast<size_t>(s) * 2 * kSwiSlotBytes + tid * 16;
                const int i = tid + sl * kThreads;
                uint4 gv = make_uint4(0, 0, 0, 0), uv = make_uint4(0, 0, 0, 0);
                if (i < n_vecs) {
                    gv = *reinterpret_cast<const uint4*>(src);
                    uv = *reinterpret_cast<const uint4*>(src + kSwiSlotBytes);
                }
                __syncwarp();
                if (lane == 0) pipe::mbar_arrive(empty + s);
                if (++s == stages) { s = 0; phase ^= 1; }
                if (i < n_vecs) {
                    gmin = gate_min_acc(gmin, gv);
                    yw[sl] = swiglu8_unchecked<kSteps>(gv, uv);
                    if constexpr (kStoreY) st_vec(static_cast<uint4*>(y) + row_off + i, yw[sl]);
                    m2 = amax_acc_bf16x2(m2, yw[sl].x);
                    m2 = amax_acc_bf16x2(m2, yw[sl].y);
                    m2 = amax_acc_bf16x2(m2, yw[sl].z);
                    m2 = amax_acc_bf16x2(m2, yw[sl].w);
                }
            }
        }
        if (gate_min_needs_exact(gmin)) {   // a gate below -85: redo this thread's share verbatim, from global memory
            m2 = 0u;
#pragma unroll
            for (int sl = 0; sl < VPT; ++sl) {
                const int i = tid + sl * kThreads;
                if (i < n_vecs) {
                    yw[sl] = swiglu8<0>(ld_stream(static_cast<const uint4*>(gate) + row_off + i),
                                        ld_stream(static_cast<const uint4*>(up) + row_off + i));
                    if constexpr (kStoreY) st_vec(static_cast<uint4*>(y) + row_off + i, yw[sl]);
                    m2 = amax_acc_bf16x2(m2, yw[sl].x);
                    m2 = amax_acc_bf16x2(m2, yw[sl].y);
                    m2 = amax_acc_bf16x2(m2, yw[sl].z);
                    m2 = amax_acc_bf16x2(m2, yw[sl].w);
                }
            }
        }
        const float m_lo = bf_lo(m2), m_hi = bf_hi(m2);
        const bool finite = (m_lo <= 3.0e38f) && (m_hi <= 3.0e38f);
        float amax = fmaxf(m_lo, m_hi);
        if (!finite) {
            amax = 0.0f;
#pragma unroll
            for (int sl = 0; sl < VPT; ++sl) {
                if (tid + sl * kThreads < n_vecs) {
                    float f[8];
                    unpack8(yw[sl], f);
#pragma unroll
                    for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(f[j]));
                }
            }
        }
        amax = warp_max_nonneg(amax);
        if (lane == 0) s_mx[parity][warp] = amax;
        pipe::consumer_sync(kThreads);
        amax = warp_max_nonneg(s_mx[parity][lane & (kWarps - 1)]);

        const float inv = quant_inv_scale<127>(amax);
        if (tid == 0) x_scale[row] = quant_scale<127>(amax);
        const bool fast = finite && inv <= 3.0e38f;
        uint2* q_row = reinterpret_cast<uint2*>(q) + row_off;
#pragma unroll
        for (int sl = 0; sl < VPT; ++sl) {
            const int i = tid + sl * kThreads;
            if (i < n_vecs) {
                if (fast) {
                    st_vec8(q_row + i, pack_int8x8_fast(yw[sl], inv));
                } else {
                    float f[8];
                    unpack8(yw[sl], f);
                    st_vec8(q_row + i, pack_int8x8(f, inv));
                }
            }
        }
    }
}

template <int VPT, bool kStoreY, int kSteps>
int launch_swiglu_quant_staged(int8_t* q, float* x_scale, void* y, const void* gate, const void* up,
                               long long num_tokens, int inter_dim, int stages, cudaStream_t stream) {
    const size_t smem = static_cast<size_t>(stages) * 2 * kSwiSlotBytes + 2 * stages * sizeof(uint64_t);
    static int configured_stages = 0;
    static int resident = 1;
    if (configured_stages != stages) {
        const void* fn = reinterpret_cast<const void*>(&swiglu_quant_staged_kernel<VPT, kStoreY, kSteps>);
        cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        resident = host::resident_ctas(fn, 256 + 32, smem);
        configured_stages = stages;
    }
    const int tuned = host::tuning(host::kSwigluCtasPerSm);
    const long long cap = static_cast<long long>(host::num_sms()) * (tuned > 0 ? tuned : resident);
    const int grid = static_cast<int>(num_tokens < cap ? num_tokens : cap);
    host::launch(swiglu_quant_staged_kernel<VPT, kStoreY, kSteps>, dim3(grid), dim3(256 + 32), smem, stream, q, x_scale, y, gate, up, num_tokens,
                                                                                       inter_dim, stages, host::device_error_word());
    return host::check_launch("swiglu_quant_staged_kernel");
}

// Prefetch-ring variant (256 threads, no producer warp, no barriers for the data): each thread keeps
// the gate/up vectors of its next kDepth slots on their way into private shared-memory slots with
// cp.async and reads back only what it copied itself.  Same mapping and arithmetic as the kernels above.
template <int VPT, bool kStoreY, int kSteps, int kDepth>
__global__ void __launch_bounds__(256, 4)
swiglu_quant_prefetch_kernel(int8_t* __restrict__ q, float* __restrict__ x_scale, void* y, const void* gate,
                             const void* up, long long num_tokens, int inter_dim) {
    constexpr int kThreads = 256, kWarps = 8;
    extern __shared__ uint4 pre[];   // [kDepth][gate|up][256]
    __shared__ float s_mx[2][kWarps];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int n_vecs = inter_dim / kVec;
    const int slots_per_row = (n_vecs + kThreads - 1) / kThreads;
    pdl_wait();

    // producer cursor: the next (row, slot-in-row) to fetch
    long long p_row = blockIdx.x;
    int p_sl = 0;
    auto fetch_next = [&](int ring_slot, uint32_t after) {
        if (p_row < num_tokens) {
            const int i = tid + p_sl * kThreads;
            if (i < n_vecs) {
                const size_t off = static_cast<size_t>(p_row) * n_vecs + i;
                cp_async16(pre + (ring_slot * 2 + 0) * kThreads + tid, static_cast<const uint4*>(gate) + off, after);
                cp_async16(pre + (ring_slot * 2 + 1) * kThreads + tid, static_cast<const uint4*>(up) + off, after);
            }
            if (++p_sl == slots_per_row) { p_sl = 0; p_row += gridDim.x; }
        }
        cp_async_commit();
    };
#pragma unroll
    for (int d = 0; d < kDepth; ++d) fetch_next(d, 0u);

    int parity = 0, ring = 0;
    for (long long row = blockIdx.x; row < num_tokens; row += gridDim.x, parity ^= 1) {
        if (row + gridDim.x >= num_tokens) pdl_trigger();   // last row of this CTA
        const size_t row_off = static_cast<size_t>(row) * n_vecs;
        uint4 yw[VPT];
        uint32_t m2 = 0u, gmin = kGateMinInit;
#pragma unroll
        for (int sl = 0; sl < VPT; ++sl) {
            if (sl < slots_per_row) {
                cp_async_wait<kDepth - 1>();
                const int i = tid + sl * kThreads;
                uint4 gv = make_uint4(0, 0, 0, 0), uv = make_uint4(0, 0, 0, 0);
                if (i < n_vecs) {
                    gv = pre[(ring * 2 + 0) * kThreads + tid];
                    uv = pre[(ring * 2 + 1) * kThreads + tid];
                }
                fetch_next(ring, gv.x ^ uv.w);     // refill the slot just drained, behind the reads above
                ring = (ring + 1 == kDepth) ? 0 : ring + 1;
                if (i < n_vecs) {
                    gmin = gate_min_acc(gmin, gv);
                    yw[sl] = swiglu8_unchecked<kSteps>(gv, uv);
                    if constexpr (kStoreY) st_vec(static_cast<uint4*>(y) + row_off + i, yw[sl]);
                    m2 = amax_acc_bf16x2(m2, yw[sl].x);
                    m2 = amax_acc_bf16x2(m2, yw[sl].y);
                    m2 = amax_acc_bf16x2(m2, yw[sl].z);
                    m2 = amax_acc_bf16x2(m2, yw[sl].w);
                }
            }
        }
        if (kSteps != 0 && gate_min_needs_exact(gmin)) {   // a gate below -85: redo this thread's share verbatim
            m2 = 0u;
#pragma unroll
            for (int sl = 0; sl < VPT; ++sl) {
                const int i = tid + sl * kThreads;
                if (i < n_vecs) {
                    yw[sl] = swiglu8<0>(ld_stream(static_cast<const uint4*>(gate) + row_off + i),
                                        ld_stream(static_cast<const uint4*>(up) + row_off + i));
                    if constexpr (kStoreY) st_vec(static_cast<uint4*>(y) + row_off + i, yw[sl]);
                    m2 = amax_acc_bf16x2(m2, yw[sl].x);
                    m2 = amax_acc_bf16x2(m2, yw[sl].y);
                    m2 = amax_acc_bf16x2(m2, yw[sl].z);
                    m2 = amax_acc_bf16x2(m2, yw[sl].w);
                }
            }
        }
        const float m_lo = bf_lo(m2), m_hi = bf_hi(m2);
        const bool finite = (m_lo <= 3.0e38f) && (m_hi <= 3.0e38f);
        float amax = fmaxf(m_lo, m_hi);
        if (!finite) {
            amax = 0.0f;
#pragma unroll
            for (int sl = 0; sl < VPT; ++sl) {
                if (tid + sl * kThreads < n_vecs) {
                    float f[8];
                    unpack8(yw[sl], f);
#pragma unroll
                    for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(f[j]));
                }
            }
        }
        amax = warp_max_nonneg(amax);
        if (lane == 0) s_mx[parity][warp] = amax;
        __syncthreads();
        amax = warp_max_nonneg(s_mx[parity][lane & (kWarps - 1)]);

        const float inv = quant_inv_scale<127>(amax);
        if (tid == 0) x_scale[row] = quant_scale<127>(amax);
        const bool fast = finite && inv <= 3.0e38f;
        uint2* q_row = reinterpret_cast<uint2*>(q) + row_off;
#pragma unroll
        for (int sl = 0; sl < VPT; ++sl) {
            const int i = tid + sl * kThreads;
            if (i < n_vecs) {
                if (fast) {
                    st_vec8(q_row + i, pack_int8x8_fast(yw[sl], inv));
                } else {
                    float f[8];
                    unpack8(yw[sl], f);
                    st_vec8(q_row + i, pack_int8x8(f, inv));
                }
            }
        }
    }
    cp_async_wait<0>();
}

template <int VPT, bool kStoreY, int kDepth>
int launch_swiglu_quant_prefetch(int8_t* q, float* x_scale, void* y, const void* gate, const void* up,
                                 long long num_tokens, int inter_dim, cudaStream_t stream) {
    constexpr size_t smem = static_cast<size_t>(kDepth) * 2 * 256 * sizeof(uint4);
    static int resident = 0;
    const void* fn = reinterpret_cast<const void*>(&swiglu_quant_prefetch_kernel<VPT, kStoreY, 1, kDepth>);
    if (resident == 0) {
        cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        resident = host::resident_ctas(fn, 256, smem);
    }
    const int tuned = host::tuning(host::kSwigluCtasPerSm);
    const long long cap = static_cast<long long>(host::num_sms()) * (tuned > 0 ? tuned : resident);
    const int grid = static_cast<int>(num_tokens < cap ? num_tokens : cap);
    host::launch(swiglu_quant_prefetch_kernel<VPT, kStoreY, 1, kDepth>, dim3(grid), dim3(256), smem, stream, q, x_scale, y, gate, up, num_tokens, inter_dim);
    return host::check_launch("swiglu_quant_prefetch_kernel");
}

template <int kThreads, int VPT, int kSteps>
int launch_swiglu_quant_steps(int8_t* q, float* x_scale, void* y, const void* gate, const void* up,
                              long long num_tokens, int inter_dim, cudaStream_t stream) {
    static const int resident_y = host::resident_ctas(
        reinterpret_cast<const void*>(&swiglu_quant_kernel<kThreads, VPT, true, kSteps>), kThreads);
    static const int resident_n = host::resident_ctas(
        reinterpret_cast<const void*>(&swiglu_quant_kernel<kThreads, VPT, false, kSteps>), kThreads);
    const int tuned = host::tuning(host::kSwigluCtasPerSm);
    const long long cap =
        static_cast<long long>(host::num_sms()) * (tuned > 0 ? tuned : (y ? resident_y : resident_n));
    const int grid = static_cast<int>(num_tokens < cap ? num_tokens : cap);
    if (y) host::launch(swiglu_quant_kernel<kThreads, VPT, true, kSteps>, dim3(grid), dim3(kThreads), 0, stream, q, x_scale, y, gate, up, num_tokens, inter_dim);
    else host::launch(swiglu_quant_kernel<kThreads, VPT, false, kSteps>, dim3(grid), dim3(kThreads), 0, stream, q, x_scale, y, gate, up, num_tokens, inter_dim);
    return host::check_launch("swiglu_quant_kernel");
}

// Reciprocal refinement steps: 1 by default (exhaustively exact, see rh_selftest);
// rh_tune("swiglu_rcp_steps", 2) adds a second step, 3 selects the IEEE division.
int rcp_steps() {
    const int t = host::tuning(host::kSwigluRcpSteps);
    return t == 2 ? 2 : (t >= 3 ? 0 : 1);
}

template <int kThreads, int VPT>
int launch_swiglu_quant(int8_t* q, float* x_scale, void* y, const void* gate, const void* up,
                        long long num_tokens, int inter_dim, cudaStream_t stream) {
    if constexpr (kThreads == 256 && VPT >= 2) {
        // rh_tune("swiglu_prefetch", d): cp.async prefetch ring of d slots (2, 4 or 6) instead of the bulk-copy ring.
        const int pf = host::tuning(host::kSwigluPrefetch);
        if (pf >= 2 && rcp_steps() == 1 && num_tokens >= 4LL * host::num_sms()) {
            if (pf >= 6) return y ? launch_swiglu_quant_prefetch<VPT, true, 6>(q, x_scale, y, gate, up, num_tokens, inter_dim, stream)
                                  : launch_swiglu_quant_prefetch<VPT, false, 6>(q, x_scale, y, gate, up, num_tokens, inter_dim, stream);
            if (pf >= 4) return y ? launch_swiglu_quant_prefetch<VPT, true, 4>(q, x_scale, y, gate, up, num_tokens, inter_dim, stream)
                                  : launch_swiglu_quant_prefetch<VPT, false, 4>(q, x_scale, y, gate, up, num_tokens, inter_dim, stream);
            return y ? launch_swiglu_quant_prefetch<VPT, true, 2>(q, x_scale, y, gate, up, num_tokens, inter_dim, stream)
                     : launch_swiglu_quant_prefetch<VPT, false, 2>(q, x_scale, y, gate, up, num_tokens, inter_dim, stream);
        }
        // With plenty of rows the bulk-copy staging ring wins (measured on B200 at I = 14336: 0.80 ms vs
        // 0.85 ms for 65536 rows): three slots by default, rh_tune("swiglu_stages", n) sets the depth
        // and n = 1 selects the direct-load kernel.  Few rows are latency-bound: direct loads.
        int stages = host::tuning(host::kSwigluStages);
        if (stages == 0) stages = 3;
        if (stages >= 2 && rcp_steps() == 1 && num_tokens >= 4LL * host::num_sms()) {
            return y ? launch_swiglu_quant_staged<VPT, true, 1>(q, x_scale, y, gate, up, num_tokens, inter_dim, stages, stream)
                     : launch_swiglu_quant_staged<VPT, false, 1>(q, x_scale, y, gate, up, num_tokens, inter_dim, stages, stream);
        }
    }
    switch (rcp_steps()) {
        case 0: return launch_swiglu_quant_steps<kThreads, VPT, 0>(q, x_scale, y, gate, up, num_tokens, inter_dim, stream);
        case 1: return launch_swiglu_quant_steps<kThreads, VPT, 1>(q, x_scale, y, gate, up, num_tokens, inter_dim, stream);
        default: return launch_swiglu_quant_steps<kThreads, VPT, 2>(q, x_scale, y, gate, up, num_tokens, inter_dim, stream);
    }
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
    const unsigned g = static_cast<unsigned>(grid);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    uint4* yp = static_cast<uint4*>(y);
    const uint4 *gp = static_cast<const uint4*>(gate), *up_ = static_cast<const uint4*>(up);
    switch (rcp_steps()) {
        case 0: host::launch(swiglu_kernel<0>, dim3(g), dim3(kElemThreads), 0, s, yp, gp, up_, n_vec); break;
        case 1: host::launch(swiglu_kernel<1>, dim3(g), dim3(kElemThreads), 0, s, yp, gp, up_, n_vec); break;
        default: host::launch(swiglu_kernel<2>, dim3(g), dim3(kElemThreads), 0, s, yp, gp, up_, n_vec); break;
    }
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
    // 256 threads x up to 8 vectors each (7 x 256 = 14336/8 exactly), or 512 x up to 4 on request.
    const bool wide = host::tuning(host::kSwigluThreads) == 512 && n_vecs > 512;
#define RH_SWIGLU(T, V) return launch_swiglu_quant<T, V>(q, x_scale, y_or_null, gate, up, num_tokens, inter_dim, s)
    if (wide) {
        if (n_vecs <= 1024) RH_SWIGLU(512, 2);
        if (n_vecs <= 1536) RH_SWIGLU(512, 3);
        RH_SWIGLU(512, 4);
    }
    switch ((n_vecs + 255) / 256) {
        case 1: RH_SWIGLU(256, 1);
        case 2: RH_SWIGLU(256, 2);
        case 3: RH_SWIGLU(256, 3);
        case 4: RH_SWIGLU(256, 4);
        case 5: RH_SWIGLU(256, 5);
        case 6: RH_SWIGLU(256, 6);
        case 7: RH_SWIGLU(256, 7);
        default: RH_SWIGLU(256, 8);
    }
#undef RH_SWIGLU
}
