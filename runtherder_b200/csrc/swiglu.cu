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

// ---- fused SwiGLU + per-token INT8 ----------------------------------------------------------------
//
// The fused kernels use the negated sigmoid (neg_sigmoid).  The default form, which does not store y,
// carries the products NEGATED: a thread's packed bf16 words hold -y, the amax is sign-blind, and the
// codes are taken with the negated inverse scale ((-y) * (-inv) is bit for bit y * inv).  Its range
// check of the refined reciprocal is hoisted out of the per-vector path: a thread tracks the smallest
// gate it has seen (one packed min per word) and only a thread that met a gate below the fast range
// (or a NaN) recomputes its share with the reference's expression verbatim.  The form that stores y
// computes +y (two sign flips per pair) and makes the range check per vector, before the store, so that
// y may alias gate or up: nothing is re-read after it has been overwritten.
constexpr uint32_t kSignBits = 0x80008000u;
__device__ __forceinline__ uint4 flip_signs(const uint4& v) {
    return make_uint4(v.x ^ kSignBits, v.y ^ kSignBits, v.z ^ kSignBits, v.w ^ kSignBits);
}
// Eight products through the negated sigmoid.  kNegated: the words hold -y (no extra instruction);
// otherwise the gate is negated for the product, which costs two sign flips per pair and gives +y.
template <bool kNegated>
__device__ __forceinline__ uint4 fast_swiglu8(const uint4& gv, const uint4& uv) {
    const uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w}, uw[4] = {uv.x, uv.y, uv.z, uv.w};
    uint32_t out[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const float2 g = bf2_to_f2(gw[k]);
        const float2 y = mul2_rn(mul2_rn(kNegated ? g : neg2(g), neg_sigmoid2(g)), bf2_to_f2(uw[k]));
        out[k] = pack_bf16x2(y.x, y.y);
    }
    return make_uint4(out[0], out[1], out[2], out[3]);
}
constexpr uint32_t kGateMinInit = 0x7f807f80u;   // +Inf, +Inf
__device__ __forceinline__ uint32_t gate_min_acc(uint32_t m, const uint4& gv) {
    __nv_bfloat162 r = *reinterpret_cast<__nv_bfloat162*>(&m);
    r = __hmin2_nan(r, *reinterpret_cast<const __nv_bfloat162*>(&gv.x));   // a NaN gate must surface: it would
    r = __hmin2_nan(r, *reinterpret_cast<const __nv_bfloat162*>(&gv.y));   // poison the gates it shares a
    r = __hmin2_nan(r, *reinterpret_cast<const __nv_bfloat162*>(&gv.z));   // reciprocal with
    r = __hmin2_nan(r, *reinterpret_cast<const __nv_bfloat162*>(&gv.w));
    return *reinterpret_cast<uint32_t*>(&r);
}
__device__ __forceinline__ bool gate_min_needs_exact(uint32_t m) {
    return !(bf_lo(m) >= kGateExactBelow && bf_hi(m) >= kGateExactBelow);   // true for NaN as well
}
// +y of one vector with the range check made here (the variant that stores y).
__device__ __forceinline__ uint4 swiglu8_range_checked(const uint4& gv, const uint4& uv) {
    if (gate_min_needs_exact(gate_min_acc(kGateMinInit, gv))) return swiglu8<0>(gv, uv);
    return fast_swiglu8<false>(gv, uv);
}
__device__ __forceinline__ uint32_t amax_acc4(uint32_t m2, const uint4& w) {
    m2 = amax_acc_bf16x2(m2, w.x);
    m2 = amax_acc_bf16x2(m2, w.y);
    m2 = amax_acc_bf16x2(m2, w.z);
    return amax_acc_bf16x2(m2, w.w);
}

constexpr int kSwiThreads = 256, kSwiWarps = 8;

// One vector of a row: products (+y when y is stored, -y otherwise), optional y store, running amax / gate min.
template <bool kStoreY>
__device__ __forceinline__ uint4 swiglu_slot(const uint4& gv, const uint4& uv, uint4* y_dst, uint32_t& m2, uint32_t& gmin) {
    uint4 w;
    if constexpr (kStoreY) {
        w = swiglu8_range_checked(gv, uv);
        st_vec(y_dst, w);
    } else {
        gmin = gate_min_acc(gmin, gv);
        w = fast_swiglu8<true>(gv, uv);
    }
    m2 = amax_acc4(m2, w);
    return w;
}

// A thread whose gates left the fast range recomputes its vectors verbatim from global memory (only in
// the variant that does not store y, so gate and up still hold the inputs).
template <int VPT, bool kFull, int kCT = kSwiThreads>
__device__ __forceinline__ void redo_exact(uint4 (&yw)[VPT], uint32_t& m2, const uint4* g_row, const uint4* u_row, int tid, int n_vecs) {
    m2 = 0u;
#pragma unroll
    for (int s = 0; s < VPT; ++s) {
        const int i = tid + s * kCT;
        if (kFull || i < n_vecs) {
            yw[s] = flip_signs(swiglu8<0>(ld_stream(g_row + i), ld_stream(u_row + i)));
            m2 = amax_acc4(m2, yw[s]);
        }
    }
}

// Row amax -> scale -> codes, from the packed products (kNegated: -y) of the CTA's kCT consumer threads.  `sync` is the
// barrier among those threads.  kFull: the row is exactly VPT * kCT vectors, no tail predicate anywhere.
template <int VPT, bool kFull, bool kNegated, int kCT = kSwiThreads, typename Sync>
__device__ __forceinline__ void quantise_row(const uint4 (&yw)[VPT], uint32_t m2, int tid, int n_vecs, float* s_mx,
                                             int8_t* q, float* x_scale, long long row, Sync sync) {
    const int lane = tid & 31, warp = tid >> 5;
    // The reference's amax (fmaxf) skips NaN; the packed NaN-propagating max reveals a non-finite value,
    // and a thread that holds one redoes its share that way and converts its elements on the exact path.
    const float m_lo = bf_lo(m2), m_hi = bf_hi(m2);
    const bool finite = (m_lo <= 3.0e38f) && (m_hi <= 3.0e38f);
    float amax = fmaxf(m_lo, m_hi);
    if (!finite) {
        amax = 0.0f;
#pragma unroll
        for (int s = 0; s < VPT; ++s) {
            if (kFull || tid + s * kCT < n_vecs) {
                float f[8];
                unpack8(yw[s], f);
#pragma unroll
                for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(f[j]));
            }
        }
    }
    amax = warp_max_nonneg(amax);
    if (lane == 0) s_mx[warp] = amax;
    sync();
    amax = warp_max_nonneg(lane < kCT / 32 ? s_mx[lane] : 0.0f);

    const float inv = quant_inv_scale<127>(amax);
    if (tid == 0) x_scale[row] = quant_scale<127>(amax);
    uint2* q_row = reinterpret_cast<uint2*>(q) + static_cast<size_t>(row) * n_vecs;
    if (finite && inv <= kFastInvMax) {
        const float2 ninv4 = splat2(inv * (kNegated ? -4.0f : 4.0f));
#pragma unroll
        for (int s = 0; s < VPT; ++s) {
            const int i = tid + s * kCT;
            if (kFull || i < n_vecs) st_vec8(q_row + i, pack_int8x8_fast4(yw[s], ninv4));
        }
    } else {
#pragma unroll
        for (int s = 0; s < VPT; ++s) {
            const int i = tid + s * kCT;
            if (kFull || i < n_vecs) {
                float f[8];
                unpack8(yw[s], f);
                st_vec8(q_row + i, pack_int8x8(f, kNegated ? -inv : inv));
            }
        }
    }
}

// Direct-load kernel (few rows: latency-bound): a CTA of 256 threads per row, two slots (four 128-bit
// loads) in flight per thread, products kept packed (4 registers per 8 values).
template <int VPT, bool kStoreY, bool kFull>
__global__ void __launch_bounds__(kSwiThreads, 4)
swiglu_quant_kernel(int8_t* __restrict__ q, float* __restrict__ x_scale, void* y, const void* gate,
                    const void* up, long long num_tokens, int inter_dim) {
    const int tid = threadIdx.x;
    const int n_vecs = inter_dim / kVec;
    __shared__ float s_mx[2][kSwiWarps];
    pdl_wait();

    int parity = 0;
    for (long long row = blockIdx.x; row < num_tokens; row += gridDim.x, parity ^= 1) {
        if (row + gridDim.x >= num_tokens) pdl_trigger();   // last row of this CTA
        const size_t row_off = static_cast<size_t>(row) * n_vecs;
        const uint4* g_row = static_cast<const uint4*>(gate) + row_off;
        const uint4* u_row = static_cast<const uint4*>(up) + row_off;
        uint4* y_row = static_cast<uint4*>(y) + row_off;

        uint4 yw[VPT];
        uint32_t m2 = 0u, gmin = kGateMinInit;
#pragma unroll
        for (int s0 = 0; s0 < VPT; s0 += 2) {
            uint4 gv[2], uv[2];
#pragma unroll
            for (int k = 0; k < 2; ++k) {
                const int i = tid + (s0 + k) * kSwiThreads;
                if (s0 + k < VPT && (kFull || i < n_vecs)) {
                    gv[k] = ld_stream(g_row + i);
                    uv[k] = ld_stream(u_row + i);
                }
            }
#pragma unroll
            for (int k = 0; k < 2; ++k) {
                const int i = tid + (s0 + k) * kSwiThreads;
                if (s0 + k < VPT && (kFull || i < n_vecs))
                    yw[s0 + k] = swiglu_slot<kStoreY>(gv[k], uv[k], y_row + i, m2, gmin);
            }
            asm volatile("" ::: "memory");  // keep the next pair's loads behind this pair's math
        }
        if constexpr (!kStoreY) {
            if (gate_min_needs_exact(gmin)) redo_exact<VPT, kFull>(yw, m2, g_row, u_row, tid, n_vecs);
        }
        quantise_row<VPT, kFull, !kStoreY>(yw, m2, tid, n_vecs, s_mx[parity], q, x_scale, row, [] { __syncthreads(); });
    }
}

// Staged kernel (256 consumer threads + one producer warp), the default when there are rows to stream.
// The producer moves 4 KB slots of gate and up through a shared-memory ring with bulk copies, so the
// bytes in flight do not depend on how many loads a consumer can hold in registers while it is busy
// with ex2/rcp; consumers take one slot at a time.  Same element-to-thread mapping and arithmetic as
// the direct kernel.  A wait that runs out is recorded in the device error word and in a CTA-wide
// flag; every consumer tests the flag behind the row barrier, so the CTA leaves together.
constexpr int kSwiSlotBytes = kSwiThreads * 16;

template <int VPT, bool kStoreY, bool kFull>
__global__ void __launch_bounds__(kSwiThreads + 32, 4)
swiglu_quant_staged_kernel(int8_t* __restrict__ q, float* __restrict__ x_scale, void* y, const void* gate,
                           const void* up, long long num_tokens, int inter_dim, const int stages, int* error_word) {
    extern __shared__ __align__(128) unsigned char ring[];
    uint64_t* full = reinterpret_cast<uint64_t*>(ring + static_cast<size_t>(stages) * 2 * kSwiSlotBytes);
    uint64_t* empty = full + stages;
    __shared__ float s_mx[2][kSwiWarps];
    __shared__ int s_gave_up;

    const int tid = threadIdx.x, lane = tid & 31;
    const int n_vecs = inter_dim / kVec;
    const int slots_per_row = kFull ? VPT : (n_vecs + kSwiThreads - 1) / kSwiThreads;
    if (tid == 0) {
        for (int s = 0; s < stages; ++s) {
            pipe::mbar_init(full + s, 1);
            pipe::mbar_init(empty + s, kSwiWarps);
        }
        s_gave_up = 0;
        pipe::mbar_init_fence();
    }
    __syncthreads();
    pdl_wait();

    if (tid >= kSwiThreads) {
        if (tid == kSwiThreads) {
            int s = 0;
            uint32_t round = 0;
            for (long long row = blockIdx.x; row < num_tokens; row += gridDim.x) {
                const size_t row_off = static_cast<size_t>(row) * n_vecs;
                for (int sl = 0; sl < slots_per_row; ++sl) {
                    if (round > 0 && !pipe::mbar_wait(empty + s, (round - 1) & 1, __LINE__, error_word)) return;
                    const int vec0 = sl * kSwiThreads;
                    const uint32_t bytes = kFull ? kSwiSlotBytes : static_cast<uint32_t>(min(kSwiThreads, n_vecs - vec0)) * 16u;
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
        uint4* y_row = static_cast<uint4*>(y) + row_off;
        uint4 yw[VPT];
        uint32_t m2 = 0u, gmin = kGateMinInit;
#pragma unroll
        for (int sl = 0; sl < VPT; ++sl) {
            if (kFull || sl < slots_per_row) {
                if (!pipe::mbar_wait(full + s, phase, __LINE__, error_word)) {
                    s_gave_up = 1;
                    break;
                }
                const unsigned char* src = ring + static_cast<size_t>(s) * 2 * kSwiSlotBytes + tid * 16;
                const int i = tid + sl * kSwiThreads;
                const bool live = kFull || i < n_vecs;
                uint4 gv = make_uint4(0, 0, 0, 0), uv = make_uint4(0, 0, 0, 0);
                if (live) {
                    gv = *reinterpret_cast<const uint4*>(src);
                    uv = *reinterpret_cast<const uint4*>(src + kSwiSlotBytes);
                }
                __syncwarp();
                if (lane == 0) pipe::mbar_arrive(empty + s);
                if (++s == stages) { s = 0; phase ^= 1; }
                if (live) yw[sl] = swiglu_slot<kStoreY>(gv, uv, y_row + i, m2, gmin);
            }
        }
        if constexpr (!kStoreY) {
            if (gate_min_needs_exact(gmin))
                redo_exact<VPT, kFull>(yw, m2, static_cast<const uint4*>(gate) + row_off, static_cast<const uint4*>(up) + row_off, tid, n_vecs);
        }
        bool gave_up = false;
        quantise_row<VPT, kFull, !kStoreY>(yw, m2, tid, n_vecs, s_mx[parity], q, x_scale, row, [&] {
            pipe::consumer_sync(kSwiThreads);
            gave_up = *reinterpret_cast<volatile int*>(&s_gave_up) != 0;
        });
        if (gave_up) return;   // every consumer reads the same flag behind the same barrier
    }
}

template <int VPT, bool kStoreY, bool kFull>
int launch_swiglu_quant_staged(int8_t* q, float* x_scale, void* y, const void* gate, const void* up,
                               long long num_tokens, int inter_dim, int stages, cudaStream_t stream) {
    constexpr auto kernel = &swiglu_quant_staged_kernel<VPT, kStoreY, kFull>;
    constexpr size_t kDefaultSmem = 3 * 2 * kSwiSlotBytes + 2 * 3 * sizeof(uint64_t);
    const size_t smem = static_cast<size_t>(stages) * 2 * kSwiSlotBytes + 2 * stages * sizeof(uint64_t);
    (void)host::KernelAtLoad<kernel, kSwiThreads + 32, kDefaultSmem>::token;
    const int resident = host::kernel_setup(reinterpret_cast<const void*>(kernel), kSwiThreads + 32, smem);
    const int tuned = host::tuning(host::kSwigluCtasPerSm);
    const long long cap = static_cast<long long>(host::num_sms()) * (tuned > 0 ? tuned : resident);
    const int grid = static_cast<int>(num_tokens < cap ? num_tokens : cap);
    host::launch<kernel>(dim3(grid), dim3(kSwiThreads + 32), smem, stream, q, x_scale, y, gate, up, num_tokens,
                 inter_dim, stages, host::device_error_word());
    return host::check_launch("swiglu_quant_staged_kernel");
}

// Ring kernel: the staged kernel for rows that divide evenly — kCT consumer threads x VPT vectors is the
// whole row and VPT is a multiple of the kStages ring slots — so that every slot index, shared-memory offset
// and barrier address is a compile-time constant and a slot's wait parity depends at most on the row's
// parity: no ring cursor, no wrap test, no address arithmetic per slot.  SwiGLU + INT8 has no ordered
// reduction, so the element-to-thread mapping is free: a 14336-wide row (1792 vectors) runs as 224 threads
// x 8 vectors over 4 slots, 8192 as 256 x 4 over 4, 12288 as 256 x 6 over 3.  Codes only (y is not stored).
template <int VPT, int kCT, int kStages>
__global__ void __launch_bounds__(kCT + 32, 4)
swiglu_quant_ring_kernel(int8_t* __restrict__ q, float* __restrict__ x_scale, const void* gate, const void* up,
                         long long num_tokens, int* error_word) {
    static_assert(VPT % kStages == 0 && kCT % 32 == 0, "shape");
    constexpr int kWarps = kCT / 32, kUses = VPT / kStages;     // uses of a slot per row
    constexpr int kVecBytes = kCT * 16, kStageBytes = 2 * kVecBytes;
    constexpr int n_vecs = VPT * kCT;
    __shared__ __align__(128) unsigned char ring[kStages * kStageBytes];
    __shared__ uint64_t full[kStages], empty[kStages];
    __shared__ float s_mx[2][kWarps];
    __shared__ int s_gave_up;

    const int tid = threadIdx.x, lane = tid & 31;
    if (tid == 0) {
#pragma unroll
        for (int s = 0; s < kStages; ++s) {
            pipe::mbar_init(full + s, 1);
            pipe::mbar_init(empty + s, kWarps);
        }
        s_gave_up = 0;
        pipe::mbar_init_fence();
    }
    __syncthreads();
    pdl_wait();

    if (tid >= kCT) {
        if (tid == kCT) {
            uint32_t n_row = 0;                                   // rows this CTA has issued
            for (long long row = blockIdx.x; row < num_tokens; row += gridDim.x, ++n_row) {
                const uint4* g_row = static_cast<const uint4*>(gate) + static_cast<size_t>(row) * n_vecs;
                const uint4* u_row = static_cast<const uint4*>(up) + static_cast<size_t>(row) * n_vecs;
#pragma unroll
                for (int sl = 0; sl < VPT; ++sl) {
                    const int s = sl % kStages;
                    const uint32_t use = n_row * kUses + sl / kStages;   // how often slot s has been filled before
                    if (use > 0 && !pipe::mbar_wait(empty + s, (use - 1) & 1, __LINE__, error_word)) return;
                    unsigned char* dst = ring + s * kStageBytes;
                    pipe::mbar_expect_tx(full + s, kStageBytes);
                    pipe::bulk_load(dst, g_row + sl * kCT, kVecBytes, full + s);
                    pipe::bulk_load(dst + kVecBytes, u_row + sl * kCT, kVecBytes, full + s);
                }
            }
        }
        return;
    }

    int parity = 0;
    uint32_t row_bit = 0;                                         // (rows processed) & 1
    for (long long row = blockIdx.x; row < num_tokens; row += gridDim.x, parity ^= 1, row_bit ^= 1) {
        if (row + gridDim.x >= num_tokens) pdl_trigger();   // last row of this CTA
        uint4 yw[VPT];
        uint32_t m2 = 0u, gmin = kGateMinInit;
#pragma unroll
        for (int sl = 0; sl < VPT; ++sl) {
            const int s = sl % kStages;
            // use number of slot s = rows * kUses + sl / kStages: its parity needs the row only when kUses is odd
            const uint32_t phase = ((kUses & 1) ? row_bit : 0u) ^ ((sl / kStages) & 1);
            if (!pipe::mbar_wait(full + s, phase, __LINE__, error_word)) {
                s_gave_up = 1;
                break;
            }
            const unsigned char* src = ring + s * kStageBytes + tid * 16;
            const uint4 gv = *reinterpret_cast<const uint4*>(src);
            const uint4 uv = *reinterpret_cast<const uint4*>(src + kVecBytes);
            __syncwarp();
            if (lane == 0) pipe::mbar_arrive(empty + s);
            yw[sl] = swiglu_slot<false>(gv, uv, nullptr, m2, gmin);
        }
        if (gate_min_needs_exact(gmin))
            redo_exact<VPT, true, kCT>(yw, m2, static_cast<const uint4*>(gate) + static_cast<size_t>(row) * n_vecs,
                                       static_cast<const uint4*>(up) + static_cast<size_t>(row) * n_vecs, tid, n_vecs);
        bool gave_up = false;
        quantise_row<VPT, true, true, kCT>(yw, m2, tid, n_vecs, s_mx[parity], q, x_scale, row, [&] {
            pipe::consumer_sync(kCT);
            gave_up = *reinterpret_cast<volatile int*>(&s_gave_up) != 0;
        });
        if (gave_up) return;   // every consumer reads the same flag behind the same barrier
    }
}

template <int VPT, int kCT, int kStages>
int launch_swiglu_quant_ring(int8_t* q, float* x_scale, const void* gate, const void* up, long long num_tokens,
                             cudaStream_t stream) {
    constexpr auto kernel = &swiglu_quant_ring_kernel<VPT, kCT, kStages>;
    const int resident = host::setup<kernel, kCT + 32>();
    const int tuned = host::tuning(host::kSwigluCtasPerSm);
    const long long cap = static_cast<long long>(host::num_sms()) * (tuned > 0 ? tuned : resident);
    const int grid = static_cast<int>(num_tokens < cap ? num_tokens : cap);
    // Launched WITHOUT the programmatic-dependent-launch attribute.  Four of these CTAs take an SM's whole
    // register file (64 x 256 x 4), and a launch that carries the attribute gets only three per SM (measured:
    // the fourth CTA of every SM then runs as a second wave on its own, 0.72 -> 0.96 ms at 65536 rows), which a
    // persistent grid with a fixed row assignment cannot absorb.  The kernel still orders itself with
    // griddepcontrol.wait (a no-op here) and still releases its own dependents early.
    host::launch_plain<kernel>(dim3(grid), dim3(kCT + 32), 0, stream, q, x_scale, gate, up, num_tokens, host::device_error_word());
    return host::check_launch("swiglu_quant_ring_kernel");
}

template <int VPT, bool kStoreY, bool kFull>
int launch_swiglu_quant_direct(int8_t* q, float* x_scale, void* y, const void* gate, const void* up,
                               long long num_tokens, int inter_dim, cudaStream_t stream) {
    constexpr auto kernel = &swiglu_quant_kernel<VPT, kStoreY, kFull>;
    const int resident = host::setup<kernel, kSwiThreads>();
    const int tuned = host::tuning(host::kSwigluCtasPerSm);
    const long long cap = static_cast<long long>(host::num_sms()) * (tuned > 0 ? tuned : resident);
    const int grid = static_cast<int>(num_tokens < cap ? num_tokens : cap);
    host::launch<kernel>(dim3(grid), dim3(kSwiThreads), 0, stream, q, x_scale, y, gate, up, num_tokens, inter_dim);
    return host::check_launch("swiglu_quant_kernel");
}

template <int VPT>
int launch_swiglu_quant(int8_t* q, float* x_scale, void* y, const void* gate, const void* up,
                        long long num_tokens, int inter_dim, cudaStream_t stream) {
    const bool full = inter_dim == VPT * kSwiThreads * kVec;
    // With plenty of rows the bulk-copy staging ring wins (three slots by default; rh_tune("swiglu_stages", n)
    // sets the depth, n = 1 selects the direct-load kernel).  Few rows are latency-bound: direct loads.
    int stages = host::tuning(host::kSwigluStages);
    if (stages == 0) stages = 3;
    const bool staged = stages >= 2 && num_tokens >= 4LL * host::num_sms();
#define RH_GO(Y, F)                                                                                                   \
    return staged ? launch_swiglu_quant_staged<VPT, Y, F>(q, x_scale, y, gate, up, num_tokens, inter_dim, stages, stream) \
                  : launch_swiglu_quant_direct<VPT, Y, F>(q, x_scale, y, gate, up, num_tokens, inter_dim, stream)
    if (y) { if (full) RH_GO(true, true); RH_GO(true, false); }
    if (full) RH_GO(false, true);
    RH_GO(false, false);
#undef RH_GO
}

// Reciprocal refinement steps of the stand-alone kernel: 1 by default (exhaustively exact, see
// rh_selftest); rh_tune("swiglu_rcp_steps", 2) adds a second step, 3 selects the IEEE division.
int rcp_steps() {
    const int t = host::tuning(host::kSwigluRcpSteps);
    return t == 2 ? 2 : (t >= 3 ? 0 : 1);
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
        case 0: host::launch<swiglu_kernel<0>>(dim3(g), dim3(kElemThreads), 0, s, yp, gp, up_, n_vec); break;
        case 1: host::launch<swiglu_kernel<1>>(dim3(g), dim3(kElemThreads), 0, s, yp, gp, up_, n_vec); break;
        default: host::launch<swiglu_kernel<2>>(dim3(g), dim3(kElemThreads), 0, s, yp, gp, up_, n_vec); break;
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
    // Rows that divide evenly into a static ring (see swiglu_quant_ring_kernel), when there are rows to stream
    // and y is not wanted; rh_tune("swiglu_ring", 1) turns it off.
    if (y_or_null == nullptr && num_tokens >= 4LL * host::num_sms() && host::tuning(host::kSwigluRingOff) != 1 &&
        host::tuning(host::kSwigluStages) == 0) {
        if (inter_dim == 14336) return launch_swiglu_quant_ring<8, 224, 4>(q, x_scale, gate, up, num_tokens, s);
        if (inter_dim == 8192) return launch_swiglu_quant_ring<4, 256, 4>(q, x_scale, gate, up, num_tokens, s);
        if (inter_dim == 12288) return launch_swiglu_quant_ring<6, 256, 3>(q, x_scale, gate, up, num_tokens, s);
    }
    // 256 threads x up to 8 vectors each (7 x 256 = 14336 / 8 exactly).
#define RH_SWIGLU(V) return launch_swiglu_quant<V>(q, x_scale, y_or_null, gate, up, num_tokens, inter_dim, s)
    switch ((n_vecs + 255) / 256) {
        case 1: RH_SWIGLU(1);
        case 2: RH_SWIGLU(2);
        case 3: RH_SWIGLU(3);
        case 4: RH_SWIGLU(4);
        case 5: RH_SWIGLU(5);
        case 6: RH_SWIGLU(6);
        case 7: RH_SWIGLU(7);
        default: RH_SWIGLU(8);
    }
#undef RH_SWIGLU
}
