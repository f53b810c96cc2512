// CTA-per-row kernels: [residual add +] RMSNorm [+ per-token INT8 quantisation],
// stand-alone per-token INT8 quantisation, and per-row FP8 quantisation of long rows.
//
// Layout.  A row of `dim` bf16 values is `dim/8` 128-bit vectors.  A CTA of 256
// threads owns one row at a time; thread t holds vectors t, t+256, ... (at most
// eight) in registers, so the row is read from HBM exactly once and every output
// (h_out, y, codes, scale) is produced from that single read.  The grid is sized
// to the machine and each CTA walks rows blockIdx.x, blockIdx.x+gridDim.x, ...,
// keeping the norm gains in registers across rows.
//
// Numerics.  The sum of squares follows the reference kernel's fp32 order exactly
// (src/kernels/rmsnorm.cu:77-113: per-thread fused multiply-add chain over its
// vectors in order, shuffle tree per warp, then the same tree over the eight warp
// partials), so rrms — and with it every bf16 output and every INT8 code — is
// bit-identical to the reference's CUDA kernel.  amax reductions are exact in any
// order.
#include <type_traits>

#include "rh_common.cuh"

namespace rh {

namespace {

constexpr int kRowThreads = 256;
constexpr int kRowWarps = kRowThreads / 32;

enum : unsigned {
    kFNorm = 1u,    // RMS-normalise (else the row is quantised as it is)
    kFAdd = 2u,     // h = x + residual, h_out written
    kFStoreY = 4u,  // write the bf16 normalised row
    kFInt8 = 8u,    // write INT8 codes + amax/127
    kFFp8 = 16u,    // write E4M3 codes + amax/448 at the at_pos-relative destination row
    kFSkipH = 32u,  // with kFAdd: h is formed but not written (nobody reads the residual stream afterwards)
};

struct RowArgs {
    void* y;
    void* h_out;
    const void* x;
    const void* residual;
    const void* g;
    void* codes;
    float* scale;
    const int* at_pos;
    int rows_per_pos;
    long long num_rows;
    int dim;
    float eps;
};

// Per-thread view of a launch: which vectors of a row this thread owns and where they live.
// kFull: the row is exactly VPT * 256 vectors, so no tail predicate exists and every per-row offset
// is a compile-time constant.
template <int VPT, bool kFull>
struct RowCtx {
    int tid, lane, warp, n_vecs_rt;
    float dim_f, inv_dim;
    bool dim_pow2;
    __device__ __forceinline__ int n_vecs() const { return kFull ? VPT * kRowThreads : n_vecs_rt; }
    __device__ __forceinline__ bool live(int s) const { return kFull || tid + s * kRowThreads < n_vecs_rt; }
};

template <int VPT, bool kFull>
__device__ __forceinline__ RowCtx<VPT, kFull> make_ctx(const RowArgs& a) {
    RowCtx<VPT, kFull> c;
    c.tid = threadIdx.x; c.lane = c.tid & 31; c.warp = c.tid >> 5;
    c.n_vecs_rt = a.dim / kVec;
    c.dim_f = static_cast<float>(a.dim);
    c.dim_pow2 = (a.dim & (a.dim - 1)) == 0;  // then ss/dim is an exact scaling
    c.inv_dim = 1.0f / c.dim_f;
    return c;
}

// This thread's pointers into the current row (vector tid of the row; vector s is 256 further on).
// They advance by one grid stride per row, so no per-row 64-bit multiply is left in the loop.
struct RowPtrs {
    const uint4* x;
    const uint4* r;
    uint4* h_out;
    uint4* y;
    uint2* codes;
    float* scale;   // of the current destination row
};

// Everything that happens to one row once its vectors sit in registers (xv, rv): h, h_out, the
// sum of squares and rrms, y, amax, codes and scale.
// kSmemH: the fp32 row h is parked in shared memory between the two passes instead of in 8*VPT
// registers per thread (layout [slot][half][thread] float4: conflict-free), which buys a resident CTA.
template <int VPT, unsigned F, bool kSmemH, bool kFull>
__device__ __forceinline__ void process_row(const RowArgs& a, const RowCtx<VPT, kFull>& c, const RowPtrs& p,
                                            const uint4 (&xv)[VPT], const uint4 (&rv)[VPT], const uint4 (&gw)[VPT],
                                            float* s_ss, float* s_mx, float4* s_h) {
    constexpr bool kNorm = (F & kFNorm) != 0, kAdd = (F & kFAdd) != 0, kStoreY = (F & kFStoreY) != 0;
    constexpr bool kInt8 = (F & kFInt8) != 0, kFp8 = (F & kFFp8) != 0, kQuant = kInt8 || kFp8;
    const int tid = c.tid, lane = c.lane, warp = c.warp;

    uint4 yw[VPT];  // the row as the next kernel would read it back: packed bf16

    if constexpr (kNorm) {
        float h[kSmemH ? 1 : VPT][8];
        float ss = 0.0f;
#pragma unroll
        for (int s0 = 0; s0 < VPT; ++s0) {
            const int s = kSmemH ? 0 : s0;           // register slot
            if (c.live(s0)) {
                if constexpr (kAdd) {
                    const uint32_t xw[4] = {xv[s0].x, xv[s0].y, xv[s0].z, xv[s0].w};
                    const uint32_t rw[4] = {rv[s0].x, rv[s0].y, rv[s0].z, rv[s0].w};
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const float2 hh = add2_rn(bf2_to_f2(xw[k]), bf2_to_f2(rw[k]));
                        h[s][2 * k] = hh.x;
                        h[s][2 * k + 1] = hh.y;
                    }
                    if constexpr ((F & kFSkipH) == 0) st_vec(p.h_out + s0 * kRowThreads, pack8(h[s]));
                } else {
                    unpack8(xv[s0], h[s]);
                }
#pragma unroll
                for (int j = 0; j < 8; ++j) ss = __fmaf_rn(h[s][j], h[s][j], ss);
                if constexpr (kSmemH) {
                    s_h[(s0 * 2 + 0) * kRowThreads + tid] = make_float4(h[0][0], h[0][1], h[0][2], h[0][3]);
                    s_h[(s0 * 2 + 1) * kRowThreads + tid] = make_float4(h[0][4], h[0][5], h[0][6], h[0][7]);
                }
            }
        }
        ss = group_sum<32>(ss);
        if (lane == 0) s_ss[warp] = ss;
        __syncthreads();
        const float total = group_sum<kRowWarps>(s_ss[lane & (kRowWarps - 1)]);
        const float rrms = rsqrtf((c.dim_pow2 ? total * c.inv_dim : total / c.dim_f) + a.eps);
        const float2 rrms2 = splat2(rrms);
#pragma unroll
        for (int s = 0; s < VPT; ++s) {
            if (c.live(s)) {
                const uint32_t gws[4] = {gw[s].x, gw[s].y, gw[s].z, gw[s].w};
                float hv[8];
                if constexpr (kSmemH) {   // each thread reads back exactly what it wrote: no barrier needed
                    const float4 lo = s_h[(s * 2 + 0) * kRowThreads + tid], hi = s_h[(s * 2 + 1) * kRowThreads + tid];
                    hv[0] = lo.x; hv[1] = lo.y; hv[2] = lo.z; hv[3] = lo.w;
                    hv[4] = hi.x; hv[5] = hi.y; hv[6] = hi.z; hv[7] = hi.w;
                } else {
#pragma unroll
                    for (int j = 0; j < 8; ++j) hv[j] = h[s][j];
                }
                uint32_t w[4];
#pragma unroll
                for (int k = 0; k < 4; ++k) {   // y = (h * rrms) * g, two elements per instruction
                    const float2 yf = mul2_rn(mul2_rn(make_float2(hv[2 * k], hv[2 * k + 1]), rrms2), bf2_to_f2(gws[k]));
                    w[k] = pack_bf16x2(yf.x, yf.y);
                }
                yw[s] = make_uint4(w[0], w[1], w[2], w[3]);
                if constexpr (kStoreY) st_vec(p.y + s * kRowThreads, yw[s]);
            }
        }
    } else {
#pragma unroll
        for (int s = 0; s < VPT; ++s) yw[s] = xv[s];
    }

    if constexpr (kQuant) {
        // Row amax of the bf16 values.  The packed NaN-propagating max tells, for free,
        // whether this thread holds a non-finite value; the reference's fmaxf skips NaN.
        uint32_t m2 = 0u;
#pragma unroll
        for (int s = 0; s < VPT; ++s) {
            if (c.live(s)) {
                m2 = amax_acc_bf16x2(m2, yw[s].x);
                m2 = amax_acc_bf16x2(m2, yw[s].y);
                m2 = amax_acc_bf16x2(m2, yw[s].z);
                m2 = amax_acc_bf16x2(m2, yw[s].w);
            }
        }
        const float m_lo = bf_lo(m2), m_hi = bf_hi(m2);
        const bool finite = (m_lo <= 3.0e38f) && (m_hi <= 3.0e38f);  // false for Inf and NaN
        float amax = fmaxf(m_lo, m_hi);
        if (!finite) {
            amax = 0.0f;
#pragma unroll
            for (int s = 0; s < VPT; ++s) {
                if (c.live(s)) {
                    float f[8];
                    unpack8(yw[s], f);
#pragma unroll
                    for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(f[j]));
                }
            }
        }
        amax = warp_max_nonneg(amax);
        if (lane == 0) s_mx[warp] = amax;
        __syncthreads();
        amax = warp_max_nonneg(s_mx[lane & (kRowWarps - 1)]);

        constexpr int kQMax = kInt8 ? 127 : 448;
        const float inv = quant_inv_scale<kQMax>(amax);
        if (tid == 0) *p.scale = quant_scale<kQMax>(amax);
        if (kInt8 && finite && inv <= kFastInvMax) {  // a huge inverse (tiny amax) takes the exact path
            const float2 inv4 = splat2(inv * 4.0f);
#pragma unroll
            for (int s = 0; s < VPT; ++s)
                if (c.live(s)) st_vec8(p.codes + s * kRowThreads, pack_int8x8_fast4(yw[s], inv4));
        } else {
#pragma unroll
            for (int s = 0; s < VPT; ++s) {
                if (c.live(s)) {
                    float yf[8];
                    unpack8(yw[s], yf);
                    st_vec8(p.codes + s * kRowThreads, kInt8 ? pack_int8x8(yf, inv) : pack_e4m3x8(yf, inv));
                }
            }
        }
    }
}

// A CTA of 256 threads walks rows blockIdx.x, blockIdx.x + gridDim.x, ...  kDepth = 0: each thread loads
// its vectors of the row straight into registers.  kDepth >= 1: each thread keeps the vectors of its next
// kDepth rows on their way into private shared-memory slots (cp.async), so the global-load latency of a
// row is paid while the previous rows are being reduced and quantised.
template <int VPT, unsigned F, bool kSmemH, int kDepth, bool kFull>
__global__ void __launch_bounds__(kRowThreads, (kSmemH ? 4 : ((F & kFNorm) == 0 ? (VPT <= 2 ? 6 : 2) : (VPT <= 2 ? 3 : 1))))
rows_kernel(const RowArgs a) {
    constexpr bool kNorm = (F & kFNorm) != 0, kAdd = (F & kFAdd) != 0, kStoreY = (F & kFStoreY) != 0;
    constexpr bool kQuant = (F & (kFInt8 | kFFp8)) != 0;
    constexpr int kOps = kAdd ? 2 : 1;
    __shared__ float s_ss[2][kRowWarps];
    __shared__ float s_mx[2][kRowWarps];
    __shared__ float4 s_h[kSmemH ? VPT * 2 * kRowThreads : 1];
    extern __shared__ uint4 pre[];   // [kDepth][kOps][VPT][256], thread-private columns
    pdl_wait();
    const RowCtx<VPT, kFull> c = make_ctx<VPT, kFull>(a);
    const int n_vecs = c.n_vecs();
    uint4 gw[VPT];
    if constexpr (kNorm) {
#pragma unroll
        for (int s = 0; s < VPT; ++s)
            if (c.live(s)) gw[s] = ld_weight(static_cast<const uint4*>(a.g) + c.tid + s * kRowThreads);
    }

    // Pointers of this thread into its current row; one grid stride further per row.
    const size_t first = static_cast<size_t>(blockIdx.x) * n_vecs + c.tid;
    const size_t stride = static_cast<size_t>(gridDim.x) * n_vecs;
    RowPtrs p;
    p.x = static_cast<const uint4*>(a.x) + first;
    p.r = kAdd ? static_cast<const uint4*>(a.residual) + first : nullptr;
    p.h_out = (kAdd && (F & kFSkipH) == 0) ? static_cast<uint4*>(a.h_out) + first : nullptr;
    p.y = kStoreY ? static_cast<uint4*>(a.y) + first : nullptr;
    p.codes = nullptr;
    p.scale = nullptr;
    if constexpr (kQuant) {
        long long slot_base = 0;
        if constexpr ((F & kFFp8) != 0) slot_base = static_cast<long long>(*a.at_pos) * a.rows_per_pos;
        p.codes = static_cast<uint2*>(a.codes) + static_cast<size_t>(slot_base) * n_vecs + first;
        p.scale = a.scale + slot_base + blockIdx.x;
    }

    // The prefetch cursor runs kDepth rows ahead of the row being processed.
    const uint4* fx = p.x;
    const uint4* fr = p.r;
    long long frow = blockIdx.x;
    auto fetch = [&](int slot, uint32_t after) {
        if (frow < a.num_rows) {
#pragma unroll
            for (int s = 0; s < VPT; ++s) {
                if (c.live(s)) {
                    cp_async16(pre + ((slot * kOps + 0) * VPT + s) * kRowThreads + c.tid, fx + s * kRowThreads, after);
                    if constexpr (kAdd)
                        cp_async16(pre + ((slot * kOps + 1) * VPT + s) * kRowThreads + c.tid, fr + s * kRowThreads, after);
                }
            }
        }
        cp_async_commit();
        frow += gridDim.x;
        fx += stride;
        if constexpr (kAdd) fr += stride;
    };
    if constexpr (kDepth > 0) {
#pragma unroll
        for (int d = 0; d < kDepth; ++d) fetch(d, 0u);
    }

    int parity = 0, slot = 0;
    for (long long row = blockIdx.x; row < a.num_rows; row += gridDim.x, parity ^= 1) {
        if (row + gridDim.x >= a.num_rows) pdl_trigger();   // last row of this CTA
        uint4 xv[VPT], rv[VPT];
        if constexpr (kDepth > 0) {
            cp_async_wait<kDepth - 1>();
            uint32_t tie = 0u;
#pragma unroll
            for (int s = 0; s < VPT; ++s) {
                if (c.live(s)) {
                    xv[s] = pre[((slot * kOps + 0) * VPT + s) * kRowThreads + c.tid];
                    tie ^= xv[s].x;
                    if constexpr (kAdd) {
                        rv[s] = pre[((slot * kOps + 1) * VPT + s) * kRowThreads + c.tid];
                        tie ^= rv[s].w;
                    }
                }
            }
            fetch(slot, tie);   // refill the slot just drained, behind the reads above
            if constexpr (kDepth > 1) slot = (slot + 1 == kDepth) ? 0 : slot + 1;
        } else {
#pragma unroll
            for (int s = 0; s < VPT; ++s) {
                if (c.live(s)) {
                    xv[s] = ld_stream(p.x + s * kRowThreads);
                    if constexpr (kAdd) rv[s] = ld_stream(p.r + s * kRowThreads);
                }
            }
        }
        process_row<VPT, F, kSmemH, kFull>(a, c, p, xv, rv, gw, s_ss[parity], s_mx[parity], s_h);
        p.x += stride;
        if constexpr (kAdd) {
            p.r += stride;
            if constexpr ((F & kFSkipH) == 0) p.h_out += stride;
        }
        if constexpr (kStoreY) p.y += stride;
        if constexpr (kQuant) { p.codes += stride; p.scale += gridDim.x; }
    }
    if constexpr (kDepth > 0) cp_async_wait<0>();
}

// Short rows (dim <= 256): kLanes = next power of two >= dim/8 lanes own one row, one
// vector each, so a warp carries 32/kLanes rows and no lane idles.  The reference
// runs these with one 256-thread CTA per row (16 threads busy at dim 128); its
// summation tree over the first kLanes lanes is what group_sum<kLanes> reproduces.
template <int kLanes, unsigned F>
__global__ void __launch_bounds__(kRowThreads) short_rows_kernel(const RowArgs a) {
    constexpr bool kNorm = (F & kFNorm) != 0, kAdd = (F & kFAdd) != 0, kStoreY = (F & kFStoreY) != 0;
    constexpr bool kInt8 = (F & kFInt8) != 0, kFp8 = (F & kFFp8) != 0, kQuant = kInt8 || kFp8;
    constexpr int kRowsPerCta = kRowThreads / kLanes;

    const int n_vecs = a.dim / kVec;
    const int sub = threadIdx.x % kLanes;
    const bool active = sub < n_vecs;
    const float dim_f = static_cast<float>(a.dim);

    pdl_enter();
    uint4 gw = make_uint4(0, 0, 0, 0);
    if (kNorm && active) gw = ld_weight(static_cast<const uint4*>(a.g) + sub);
    long long slot_base = 0;
    if constexpr (kFp8) slot_base = static_cast<long long>(*a.at_pos) * a.rows_per_pos;

    const long long stride = static_cast<long long>(gridDim.x) * kRowsPerCta;
    // All lanes of a warp run the same number of iterations (shuffles need the full warp).
    const long long first = static_cast<long long>(blockIdx.x) * kRowsPerCta;
    for (long long base = first; base < a.num_rows; base += stride) {
        const long long row = base + threadIdx.x / kLanes;
        const bool live = active && row < a.num_rows;
        const size_t off = static_cast<size_t>(row) * n_vecs + sub;

        uint4 xv = make_uint4(0, 0, 0, 0), rv = make_uint4(0, 0, 0, 0);
        if (live) {
            xv = ld_stream(static_cast<const uint4*>(a.x) + off);
            if constexpr (kAdd) rv = ld_stream(static_cast<const uint4*>(a.residual) + off);
        }

        uint4 yv = xv;
        if constexpr (kNorm) {
            float h[8], g[8], yf[8];
            unpack8(xv, h);
            if constexpr (kAdd) {
                float r[8];
                unpack8(rv, r);
#pragma unroll
                for (int j = 0; j < 8; ++j) h[j] += r[j];
                if (live) st_vec(static_cast<uint4*>(a.h_out) + off, pack8(h));
            }
            float ss = 0.0f;
#pragma unroll
            for (int j = 0; j < 8; ++j) ss = __fmaf_rn(h[j], h[j], ss);
            const float total = group_sum<kLanes>(ss);
            const float rrms = rsqrtf(total / dim_f + a.eps);
            unpack8(gw, g);
#pragma unroll
            for (int j = 0; j < 8; ++j) yf[j] = h[j] * rrms * g[j];
            yv = pack8(yf);
            if (kStoreY && live) st_vec(static_cast<uint4*>(a.y) + off, yv);
        }
        if constexpr (kQuant) {
            float yf[8];
            unpack8(yv, yf);
            float amax = 0.0f;
#pragma unroll
            for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(yf[j]));
            amax = group_max<kLanes>(amax);
            constexpr float kQMax = kInt8 ? 127.0f : 448.0f;
            const float inv = (amax > 0.0f) ? (kQMax / amax) : 0.0f;
            const long long dst_row = row + slot_base;
            if (live) {
                if (sub == 0) a.scale[dst_row] = amax / kQMax;
                st_vec8(static_cast<uint2*>(a.codes) + static_cast<size_t>(dst_row) * n_vecs + sub,
                        kInt8 ? pack_int8x8(yf, inv) : pack_e4m3x8(yf, inv));
            }
        }
    }
}

// Grid = CTAs of this instantiation that fit on the whole device (set up once per device), capped at
// three per SM for the prefetching forms, so each CTA keeps its gains in registers and walks its share of
// the rows.
template <int VPT, unsigned F, bool kSmemH, int kDepth, bool kFull>
void launch_form(const RowArgs& a, cudaStream_t stream, int per_sm_cap) {
    constexpr int kOps = (F & kFAdd) ? 2 : 1;
    constexpr size_t smem = static_cast<size_t>(kDepth) * kOps * VPT * kRowThreads * sizeof(uint4);
    constexpr auto kernel = &rows_kernel<VPT, F, kSmemH, kDepth, kFull>;
    const int resident = host::setup<kernel, kRowThreads, smem>();
    const int tuned = host::tuning(host::kRowsCtasPerSm);
    const int per_sm = tuned > 0 ? tuned : (per_sm_cap > 0 && resident > per_sm_cap ? per_sm_cap : resident);
    const long long cap = static_cast<long long>(host::num_sms()) * per_sm;
    const int grid = static_cast<int>(a.num_rows < cap ? a.num_rows : cap);
    host::launch<kernel>(dim3(grid), dim3(kRowThreads), smem, stream, a);
}

template <int VPT, unsigned F, bool kFull>
void launch_long(const RowArgs& a, cudaStream_t stream) {
    if constexpr (VPT <= 2) {
        // Plenty of rows: cp.async prefetch ring, rh_tune("rows_prefetch", depth 1..3; 4 = off).  Defaults
        // from measurements at 65536 x 4096 on B200: norm + INT8 one row ahead (295 us vs 322 us), plain
        // quantisation two rows ahead (120 us vs 131 us), both with three CTAs per SM; the bf16-output norm
        // is store-bound and loses with a ring (370 us vs 332 us), so it keeps the plain loads.
        constexpr bool kQuantOut = (F & (kFInt8 | kFFp8)) != 0;
        constexpr bool kSm = (F & kFNorm) != 0;
        int depth = host::tuning(host::kRowsPrefetch);
        if (depth == 0) depth = !kQuantOut ? 4 : ((F & kFNorm) != 0 ? 1 : 2);
        if (depth <= 3 && a.num_rows >= 4LL * host::num_sms() && host::tuning(host::kRowsSmemH) != 1) {
            if (depth == 1) launch_form<VPT, F, kSm, 1, kFull>(a, stream, 3);
            else if (depth == 2) launch_form<VPT, F, kSm, 2, kFull>(a, stream, 3);
            else launch_form<VPT, F, kSm, 3, kFull>(a, stream, 3);
            return;
        }
    }
    if constexpr ((F & kFNorm) != 0 && VPT <= 4) {   // 8 KB of shared memory per slot: up to 32 KB static
        if (host::tuning(host::kRowsSmemH) != 1) {   // rh_tune("rows_smem_h", 1) keeps h in registers
            launch_form<VPT, F, true, 0, kFull>(a, stream, 0);
            return;
        }
    }
    launch_form<VPT, F, false, 0, kFull>(a, stream, 0);
}

template <unsigned F>
int launch_rows(const RowArgs& a, cudaStream_t stream) {
    const int n_vecs = a.dim / kVec;
    if (n_vecs <= 32) {
        int lanes = 1;
        while (lanes < n_vecs) lanes <<= 1;
        const long long rows_per_cta = kRowThreads / lanes;
        const long long want = (a.num_rows + rows_per_cta - 1) / rows_per_cta;
        const long long cap = static_cast<long long>(host::num_sms()) * 8;
        const int grid = static_cast<int>(want < cap ? want : cap);
        switch (lanes) {
            case 1: host::launch<short_rows_kernel<1, F>>(dim3(grid), dim3(kRowThreads), 0, stream, a); break;
            case 2: host::launch<short_rows_kernel<2, F>>(dim3(grid), dim3(kRowThreads), 0, stream, a); break;
            case 4: host::launch<short_rows_kernel<4, F>>(dim3(grid), dim3(kRowThreads), 0, stream, a); break;
            case 8: host::launch<short_rows_kernel<8, F>>(dim3(grid), dim3(kRowThreads), 0, stream, a); break;
            case 16: host::launch<short_rows_kernel<16, F>>(dim3(grid), dim3(kRowThreads), 0, stream, a); break;
            default: host::launch<short_rows_kernel<32, F>>(dim3(grid), dim3(kRowThreads), 0, stream, a); break;
        }
        return host::check_launch("short_rows_kernel");
    }
    const int vpt = (n_vecs + kRowThreads - 1) / kRowThreads;
    // Rows of exactly 2 x 256 or 4 x 256 vectors (4096 and 8192 wide) take the form without tail predicates.
    if (vpt <= 1) launch_long<1, F, false>(a, stream);
    else if (vpt <= 2) { if (n_vecs == 2 * kRowThreads) launch_long<2, F, true>(a, stream); else launch_long<2, F, false>(a, stream); }
    else if (vpt <= 4) { if (n_vecs == 4 * kRowThreads) launch_long<4, F, true>(a, stream); else launch_long<4, F, false>(a, stream); }
    else launch_long<8, F, false>(a, stream);
    return host::check_launch("rows_kernel");
}

int check_rows(const char* who, long long num_rows, int dim) {
    RH_REQUIRE(num_rows >= 1, RH_ERR_INVALID_ARG, "%s: row count must be >= 1 (got %lld)", who, num_rows);
    RH_REQUIRE(dim >= kVec, RH_ERR_UNSUPPORTED_DIM, "%s: row length must be >= 8 (got %d)", who, dim);
    RH_REQUIRE(dim % kVec == 0, RH_ERR_UNSUPPORTED_DIM, "%s: row length must be divisible by 8 (got %d)", who, dim);
    RH_REQUIRE(dim <= RH_MAX_ROW_DIM, RH_ERR_UNSUPPORTED_DIM, "%s: row length %d exceeds %d", who, dim,
               RH_MAX_ROW_DIM);
    return RH_OK;
}

}  // namespace

}  // namespace rh

using namespace rh;

extern "C" int rh_rmsnorm_bf16(void* y, const void* x, const void* g, int num_tokens, int hidden_dim,
                               float eps, void* stream) {
    if (int e = check_rows("rh_rmsnorm_bf16", num_tokens, hidden_dim)) return e;
    RH_REQUIRE(y && x && g, RH_ERR_INVALID_ARG, "rh_rmsnorm_bf16: null pointer");
    RH_REQUIRE(eps > 0.0f, RH_ERR_INVALID_ARG, "rh_rmsnorm_bf16: eps must be > 0");
    RH_REQUIRE(host::aligned16(y) && host::aligned16(x) && host::aligned16(g), RH_ERR_MISALIGNED,
               "rh_rmsnorm_bf16: pointers must be 16-byte aligned");
    RowArgs a{y, nullptr, x, nullptr, g, nullptr, nullptr, nullptr, 0, num_tokens, hidden_dim, eps};
    return launch_rows<kFNorm | kFStoreY>(a, static_cast<cudaStream_t>(stream));
}

extern "C" int rh_rmsnorm_add_bf16(void* y, void* h_out, const void* x, const void* residual,
                                   const void* g, int num_tokens, int hidden_dim, float eps,
                                   void* stream) {
    if (int e = check_rows("rh_rmsnorm_add_bf16", num_tokens, hidden_dim)) return e;
    RH_REQUIRE(y && h_out && x && residual && g, RH_ERR_INVALID_ARG, "rh_rmsnorm_add_bf16: null pointer");
    RH_REQUIRE(eps > 0.0f, RH_ERR_INVALID_ARG, "rh_rmsnorm_add_bf16: eps must be > 0");
    RH_REQUIRE(y != h_out, RH_ERR_INVALID_ARG, "rh_rmsnorm_add_bf16: y and h_out must be distinct buffers");
    RH_REQUIRE(host::aligned16(y) && host::aligned16(h_out) && host::aligned16(x) &&
                   host::aligned16(residual) && host::aligned16(g),
               RH_ERR_MISALIGNED, "rh_rmsnorm_add_bf16: pointers must be 16-byte aligned");
    RowArgs a{y, h_out, x, residual, g, nullptr, nullptr, nullptr, 0, num_tokens, hidden_dim, eps};
    return launch_rows<kFNorm | kFAdd | kFStoreY>(a, static_cast<cudaStream_t>(stream));
}

extern "C" int rh_rmsnorm_add_last_row_bf16(void* y_last, const void* x, const void* residual, const void* g,
                                            int num_tokens, int hidden_dim, float eps, void* stream) {
    if (int e = check_rows("rh_rmsnorm_add_last_row_bf16", num_tokens, hidden_dim)) return e;
    RH_REQUIRE(y_last && x && residual && g, RH_ERR_INVALID_ARG, "rh_rmsnorm_add_last_row_bf16: null pointer");
    RH_REQUIRE(eps > 0.0f, RH_ERR_INVALID_ARG, "rh_rmsnorm_add_last_row_bf16: eps must be > 0");
    RH_REQUIRE(host::aligned16(y_last) && host::aligned16(x) && host::aligned16(residual) && host::aligned16(g),
               RH_ERR_MISALIGNED, "rh_rmsnorm_add_last_row_bf16: pointers must be 16-byte aligned");
    const size_t last = static_cast<size_t>(num_tokens - 1) * static_cast<size_t>(hidden_dim) * sizeof(__nv_bfloat16);
    RowArgs a{y_last, nullptr, static_cast<const char*>(x) + last, static_cast<const char*>(residual) + last, g,
              nullptr, nullptr, nullptr, 0, 1, hidden_dim, eps};
    return launch_rows<kFNorm | kFAdd | kFStoreY | kFSkipH>(a, static_cast<cudaStream_t>(stream));
}

extern "C" int rh_quantize_per_token_int8(int8_t* q, float* x_scale, const void* x, int num_tokens,
                                          int dim, void* stream) {
    if (int e = check_rows("rh_quantize_per_token_int8", num_tokens, dim)) return e;
    RH_REQUIRE(q && x_scale && x, RH_ERR_INVALID_ARG, "rh_quantize_per_token_int8: null pointer");
    RH_REQUIRE(host::aligned16(x) && (reinterpret_cast<uintptr_t>(q) & 7u) == 0, RH_ERR_MISALIGNED,
               "rh_quantize_per_token_int8: x must be 16-byte and q 8-byte aligned");
    RowArgs a{nullptr, nullptr, x, nullptr, nullptr, q, x_scale, nullptr, 0, num_tokens, dim, 0.0f};
    return launch_rows<kFInt8>(a, static_cast<cudaStream_t>(stream));
}

extern "C" int rh_quantize_kv_fp8(uint8_t* q, float* scale, const void* x, const int* at_pos,
                                  int rows_per_pos, int num_rows, int head_dim, void* stream) {
    if (int e = check_rows("rh_quantize_kv_fp8", num_rows, head_dim)) return e;
    RH_REQUIRE(q && scale && x, RH_ERR_INVALID_ARG, "rh_quantize_kv_fp8: null pointer");
    RH_REQUIRE(at_pos != nullptr, RH_ERR_INVALID_ARG, "rh_quantize_kv_fp8: at_pos must not be null");
    RH_REQUIRE(rows_per_pos >= 1, RH_ERR_INVALID_ARG, "rh_quantize_kv_fp8: rows_per_pos must be >= 1");
    RH_REQUIRE(host::aligned16(x) && (reinterpret_cast<uintptr_t>(q) & 7u) == 0, RH_ERR_MISALIGNED,
               "rh_quantize_kv_fp8: x must be 16-byte and q 8-byte aligned");
    RowArgs a{nullptr, nullptr, x, nullptr, nullptr, q, scale, at_pos, rows_per_pos, num_rows, head_dim, 0.0f};
    return launch_rows<kFFp8>(a, static_cast<cudaStream_t>(stream));
}

extern "C" int rh_rmsnorm_add_quant_int8(int8_t* q, float* x_scale, void* h_out, void* y_or_null,
                                         const void* x, const void* residual_or_null, const void* g,
                                         int num_tokens, int hidden_dim, float eps, void* stream) {
    if (int e = check_rows("rh_rmsnorm_add_quant_int8", num_tokens, hidden_dim)) return e;
    RH_REQUIRE(q && x_scale && x && g, RH_ERR_INVALID_ARG, "rh_rmsnorm_add_quant_int8: null pointer");
    RH_REQUIRE(eps > 0.0f, RH_ERR_INVALID_ARG, "rh_rmsnorm_add_quant_int8: eps must be > 0");
    RH_REQUIRE(residual_or_null == nullptr || h_out != nullptr, RH_ERR_INVALID_ARG,
               "rh_rmsnorm_add_quant_int8: h_out is required when a residual is given");
    RH_REQUIRE(y_or_null == nullptr || y_or_null != h_out, RH_ERR_INVALID_ARG,
               "rh_rmsnorm_add_quant_int8: y and h_out must be distinct buffers");
    RH_REQUIRE(host::aligned16(x) && host::aligned16(g) && host::aligned16(h_out) &&
                   host::aligned16(y_or_null) && host::aligned16(residual_or_null) &&
                   (reinterpret_cast<uintptr_t>(q) & 7u) == 0,
               RH_ERR_MISALIGNED, "rh_rmsnorm_add_quant_int8: pointers must be 16-byte aligned (q: 8)");
    RowArgs a{y_or_null, h_out, x, residual_or_null, g, q, x_scale, nullptr, 0, num_tokens, hidden_dim, eps};
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (residual_or_null) {
        return y_or_null ? launch_rows<kFNorm | kFAdd | kFStoreY | kFInt8>(a, s)
                         : launch_rows<kFNorm | kFAdd | kFInt8>(a, s);
    }
    return y_or_null ? launch_rows<kFNorm | kFStoreY | kFInt8>(a, s) : launch_rows<kFNorm | kFInt8>(a, s);
}
