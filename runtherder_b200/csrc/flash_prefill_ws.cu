// Causal prefill attention over the FP8-E4M3 KV cache, tcgen05 form with the work of a CTA split by role.
// Same contract as flash_prefill.cu (runtherder::kernels::flash_prefill_bf16,
// include/runtherder/kernels/flash_prefill.cuh:27-40); same tile geometry, operand layouts and arithmetic as
// the fragment form in flash_prefill_tc.cu (row blocks of 128 query rows of one kv head, key tiles of 64, scores
// read in the accumulator-fragment shape, weights in tensor memory), except that all of Q sits in shared memory
// and the tensor-memory columns that frees hold a second buffer for the weights.
//
// What differs is who does what.  In flash_prefill_tc.cu every thread walks through every phase of a tile
// and the CTA meets at two barriers per tile, so the phases add up: switching any one of them off
// (conversion, products, loads) shortens the kernel by that phase's share.  Here the warps take three roles
// and hand tiles to one another through mbarriers, so that the phases of neighbouring tiles overlap (one row
// block per CTA shown; with two, warps 0-15 are the softmax warps of blocks 0 and 1, warps 16-17 their product
// warps and warps 18-21 the conversion warps, whose tiles both blocks share):
//
//   warps 0-7   softmax      wait S_j  -> load scores, release S -> scale, mask, maximum, weights
//                            -> store W_j (two buffers) -> only if a row maximum moved: wait for
//                            O += W_{j-1} V_{j-1}, rescale O -> W ready
//   warp  8     products     S_0;  per tile: [S_j read, K_{j+1} ready] S_{j+1} = Q K_{j+1}^T
//                                            [W_j ready, V_j ready]     O += W_j V_j
//   warps 9-11  conversion   raw E4M3 rows (cp.async, one tile ahead) -> f16 operand tiles (two buffers each) and
//                            the per-key constants; K_j once S_{j-2} is complete, V_j once O += W_{j-2} V_{j-2} is
//
// S_{j+1} is computed while the softmax warps still work on the scores of tile j, which they hold in
// registers; the conversion of the next tiles runs beside both.  Barriers that serve a double-buffered
// resource exist once per buffer, so that no waiter can be overtaken by two phases.
// Every wait is bounded; a wait that gives up raises a CTA-wide flag that ends every other wait within one
// polling interval, records where it happened, and the CTA leaves through the common exit, which releases the
// tensor memory.
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include "flash_prefill_tc.cuh"
#include "rh_kernels.h"

namespace rh {
namespace ws {

using namespace tc;

constexpr int kChunks = kKeys * 8;                       // 16-byte chunks per raw tile
constexpr int kCstRing = 4;        // constants of tile j are read while those of tiles j+1, j+2 are written
constexpr int kTileBytes = 2 * kKeys * 128;              // an f16 operand tile: [2 dim blocks][64 keys][128 B]   16 KB

// A CTA carries kBlocks row blocks of 128 query rows (consecutive token ranges of the same kv head and head
// chunk) that share the converted K and V tiles; one CTA per SM either way (shared memory).  Two blocks: a tile
// is converted once for twice the rows; one block: for prompts whose grid does not exceed the SM count anyway.
template <int kBlocks>
struct Geo {
    static constexpr int kSoftmaxWarps = 8 * kBlocks;
    static constexpr int kIssuerWarp0 = kSoftmaxWarps;               // one product warp per row block
    static constexpr int kConvWarp0 = kSoftmaxWarps + kBlocks;
    static constexpr int kConvWarps = kBlocks == 1 ? 3 : 4;
    static constexpr int kConvThreads = 32 * kConvWarps;
    static constexpr int kThreads = 32 * (kConvWarp0 + kConvWarps);  // 384 or 704
    static constexpr int kPerConv = (kChunks + kConvThreads - 1) / kConvThreads;
    static constexpr int kTmem = kTmemCols * kBlocks;
    static constexpr int kQBytes = 2 * kRows * 128;
    // shared-memory map, relative to a 1024-byte aligned base
    static constexpr int kSQ = 0;                                    // per block [2 dim blocks][128 rows][128 B]: Q
    static constexpr int kSK = kSQ + kBlocks * kQBytes;              // two K tiles                               32 KB
    static constexpr int kSV = kSK + 2 * kTileBytes;                 // two V tiles                               32 KB
    static constexpr int kSRawK = kSV + 2 * kTileBytes;              // raw K rows                                 8 KB
    static constexpr int kSRawV = kSRawK + kKeys * kD;               // raw V rows                                 8 KB
    static constexpr int kSRawS = kSRawV + kKeys * kD;               // 64 K scales, 64 V scales
    static constexpr int kSCst = kSRawS + 2 * kKeys * 4;             // ring of {ksl[64], lgv[64], rvs[64]}
    static constexpr int kSBar = kSCst + kCstRing * 3 * kKeys * 4;   // mbarriers, tensor-memory base, give-up flag
    static constexpr int kSmemBytes = kSBar + 256 + 1024;
    // mbarriers: per row block {S complete x2, O += W V complete x2, S read, W ready}, then K ready x2, V ready x2;
    // tile j uses entry j % 2 of the paired ones, in that entry's phase j / 2
    static constexpr int kBarsPerBlock = 6;
    static constexpr int kBarKReady = kBarsPerBlock * kBlocks;
    static constexpr int kBarVReady = kBarKReady + 2;
    static constexpr int kNumBars = kBarVReady + 2;
};
enum BlockBar { kBarQK = 0, kBarPV = 2, kBarSRead = 4, kBarWReady = 5 };

constexpr int kTries = 1 << 20;
constexpr int kLazyNs = 100;      // pause between polls of the product and conversion warps

// Bounded wait that also ends when another thread of the CTA has given up.  kBackoffNs > 0 sleeps between
// tries: for the roles whose reaction time is not on the critical path (a poll is a shared-memory access and
// an issue slot taken from the softmax warps).
template <int kBackoffNs = 0>
__device__ __forceinline__ bool wait_phase(uint64_t* bar, uint32_t parity, volatile int* gave_up, int where, int* error_word,
                                           int tries = kTries, int* tries_used = nullptr) {
    const uint32_t addr = pipe::smem_u32(bar);
    for (int i = 0; i < tries; ++i) {       // a try blocks for a while in hardware before it reports failure
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(addr), "r"(parity)
            : "memory");
        if (ok != 0) return true;
        if ((i & 15) == 15 && *gave_up != 0) {                 // looked at now and then: a poll is a shared-memory access
            if (tries_used != nullptr) *tries_used = i + 1;
            return false;
        }
        if constexpr (kBackoffNs > 0) __nanosleep(kBackoffNs);
    }
    *gave_up = 1;
    if (error_word != nullptr) atomicCAS(error_word, 0, (where << 8) | 1);
    if (tries_used != nullptr) *tries_used = tries;
    return false;
}

// Probe of the give-up path of wait_phase (rh_selfcheck_role_wait): warp 0 waits with a limit of `tries` on a
// barrier that nothing completes and must give up; warp 1 waits with the kernels' own limit on another such
// barrier and must be released by warp 0's flag long before that limit.  out: [0] warp 0's wait returned true (0
// expected), [1] the give-up flag, [2] the error word the probe recorded (a private word), [3] tries warp 1 used.
__global__ void role_wait_probe_kernel(int tries, int* out) {
    __shared__ uint64_t bars[2];
    __shared__ int flag[2];
    if (threadIdx.x == 0) {
        pipe::mbar_init(&bars[0], 1);
        pipe::mbar_init(&bars[1], 1);
        flag[0] = 0;
        pipe::mbar_init_fence();
    }
    __syncthreads();
    volatile int* const gave_up = flag;
    if (threadIdx.x < 32) {
        const bool ok = wait_phase(&bars[0], 0, gave_up, __LINE__, out + 2, tries);
        if (threadIdx.x == 0) out[0] = ok ? 1 : 0;
    } else {
        int used = 0;
        (void)wait_phase(&bars[1], 0, gave_up, __LINE__, nullptr, kTries, &used);
        if (threadIdx.x == 32) out[3] = used;
    }
    __syncthreads();
    if (threadIdx.x == 0) out[1] = flag[0];
}

// Barrier among the `count` threads that use named barrier `id`, returning the OR of their predicates.
__device__ __forceinline__ bool group_or(int id, int count, bool pred) {
    uint32_t out;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\tsetp.ne.b32 q, %3, 0;\n\t"
        "bar.red.or.pred p, %1, %2, q;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(out)
        : "r"(id), "r"(count), "r"(static_cast<uint32_t>(pred))
        : "memory");
    return out != 0;
}

// the key whose K row becomes row r of the K operand tile (S column 16a + 8h + 2c + e holds key 16a + 4c + 2h + e)
__device__ __forceinline__ int key_of_k_row(int r) { return (r & 48) | ((r & 6) << 1) | ((r & 8) >> 2) | (r & 1); }

// grid (token tiles of kBlocks * tokens_per_cta tokens, num_kv_heads * head_chunks)
template <int kBlocks>
__global__ void __launch_bounds__(Geo<kBlocks>::kThreads, 1) flash_prefill_ws_kernel(const Args p) {
    using G = Geo<kBlocks>;
    extern __shared__ unsigned char raw_smem[];
    const uint32_t base = (pipe::smem_u32(raw_smem) + 1023u) & ~1023u;          // shared-space address, 1 KB aligned
    unsigned char* const sm = raw_smem + (base - pipe::smem_u32(raw_smem));     // the same place, generic pointer
    uint64_t* const bars = reinterpret_cast<uint64_t*>(sm + G::kSBar);
    uint32_t* const tmem_slot = reinterpret_cast<uint32_t*>(sm + G::kSBar + 8 * G::kNumBars);
    volatile int* const gave_up = reinterpret_cast<volatile int*>(sm + G::kSBar + 8 * G::kNumBars + 8);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int kvh = blockIdx.y / p.head_chunks;
    const int chunk = blockIdx.y - kvh * p.head_chunks;
    const int tile = gridDim.x - 1 - blockIdx.x;            // long (late) token tiles first
    const int cta_tok0 = tile * (kBlocks * p.tokens_per_cta);

    if (tid == 0) {
#pragma unroll
        for (int g = 0; g < kBlocks; ++g) {
            uint64_t* const bb = bars + g * G::kBarsPerBlock;
            pipe::mbar_init(&bb[kBarQK], 1);
            pipe::mbar_init(&bb[kBarQK + 1], 1);
            pipe::mbar_init(&bb[kBarPV], 1);
            pipe::mbar_init(&bb[kBarPV + 1], 1);
            pipe::mbar_init(&bb[kBarSRead], 8);
            pipe::mbar_init(&bb[kBarWReady], 8);
        }
        pipe::mbar_init(&bars[G::kBarKReady], G::kConvThreads);
        pipe::mbar_init(&bars[G::kBarKReady + 1], G::kConvThreads);
        pipe::mbar_init(&bars[G::kBarVReady], G::kConvThreads);
        pipe::mbar_init(&bars[G::kBarVReady + 1], G::kConvThreads);
        *gave_up = 0;
        pipe::mbar_init_fence();
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(pipe::smem_u32(tmem_slot)), "r"(G::kTmem) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    pdl_enter();
    const int clen = *p.cache_len;
    const int total_keys = clen + p.n_new;
    const int last_tok = min(cta_tok0 + kBlocks * p.tokens_per_cta, p.n_new) - 1;
    // every row block walks the tiles the CTA's last token needs (an earlier block finds its last tile masked)
    const int n_tiles = min((total_keys + kKeys - 1) / kKeys, (clen + last_tok) / kKeys + 1);

    // this warp's row block (softmax and product warps) and that block's tensor memory: S 64 columns, O 128,
    // two W buffers (f16 pairs) of 32.  With two W buffers the softmax warps need not wait for the previous
    // O += W V before they store the next weights.
    const int blk = warp < G::kSoftmaxWarps ? warp >> 3 : (warp < G::kConvWarp0 ? warp - G::kIssuerWarp0 : 0);
    const int wb = warp & 7;                                 // warp within the block's softmax warps
    const int tok0 = cta_tok0 + blk * p.tokens_per_cta;
    uint64_t* const bb = bars + blk * G::kBarsPerBlock;
    const uint32_t tmem_s = tmem + blk * kTmemCols, tmem_o = tmem_s + kKeys, tmem_w = tmem_o + kD;
    const int q_off = G::kSQ + blk * G::kQBytes;

    // ---- Q (softmax warps): row of the block, bf16 -> f16 into shared memory ([dim block][row][128 bytes, swizzled]);
    //      dims 0..63 by the block's first four warps, dims 64..127 by the other four ----
    if (warp < G::kSoftmaxWarps) {
        const int row = 32 * (wb & 3) + lane, part = wb >> 2;
        const int head_slot = row / p.tokens_per_cta;
        const int tok = tok0 + (row - head_slot * p.tokens_per_cta);
        const int head_in_group = chunk * p.heads_per_cta + head_slot;
        const bool row_valid = head_slot < p.heads_per_cta && head_in_group < p.group && tok < p.n_new;   // rows past the block's head slots idle
        const int qh = kvh * p.group + head_in_group;
        const __nv_bfloat16* src = p.q + (static_cast<size_t>(row_valid ? tok : 0) * p.num_q_heads + (row_valid ? qh : 0)) * kD;
        auto load_chunk = [&](int cidx) {
            uint4 w = make_uint4(0u, 0u, 0u, 0u);
            if (row_valid) w = *reinterpret_cast<const uint4*>(src + cidx * 8);
            uint4 h;
            h.x = pack_f16x2(bf_lo(w.x), bf_hi(w.x));
            h.y = pack_f16x2(bf_lo(w.y), bf_hi(w.y));
            h.z = pack_f16x2(bf_lo(w.z), bf_hi(w.z));
            h.w = pack_f16x2(bf_lo(w.w), bf_hi(w.w));
            return h;
        };
#pragma unroll
        for (int c = 0; c < 8; ++c)
            *reinterpret_cast<uint4*>(sm + q_off + part * (kRows * 128) + swz128(row, c)) = load_chunk(8 * part + c);
    }
    // Q is in place for the product warps once the softmax warps have stored it; the conversion warps do not
    // touch it and go straight to their first copies, which then overlap the loading of Q.
    fence_async_smem();
    tc_fence_before();
    if (warp < G::kConvWarp0) named_sync(3, 32 * G::kConvWarp0);
    tc_fence_after();

    if (warp < G::kSoftmaxWarps) {
        // =============================== softmax ===============================
        // this thread's two rows (lanes 16 (wb / 4) + lane / 4 and + 8 of the warp's quarter); its keys are
        // 16 a + 4 (lane % 4) + i, a and i in 0..3
        const int c2 = lane & 3;
        const int row_a = 32 * (wb & 3) + 16 * (wb >> 2) + (lane >> 2), row_b = row_a + 8;
        const uint32_t my_lanes16 = static_cast<uint32_t>(32 * (wb & 3) + 16 * (wb >> 2)) << 16;
        const int slot_a = row_a / p.tokens_per_cta, slot_b = row_b / p.tokens_per_cta;
        const int tok_a = tok0 + (row_a - slot_a * p.tokens_per_cta), tok_b = tok0 + (row_b - slot_b * p.tokens_per_cta);
        const int qpos_a = clen + tok_a, qpos_b = clen + tok_b;
        const int qpos_min = min(qpos_a, qpos_b);
        float m_a = kMInit, m_b = kMInit, l_a = 0.0f, l_b = 0.0f;
        bool ok = true;
        for (int j = 0; j < n_tiles && ok; ++j) {
            ok = wait_phase(&bb[kBarQK + (j & 1)], (j >> 1) & 1, gave_up, __LINE__, p.error_word);
            if (!ok) break;
            tc_fence_after();
            uint32_t sr[32];
            tmem_ld_frag_x8(sr, tmem_s + my_lanes16);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) pipe::mbar_arrive(&bb[kBarSRead]);            // S may be overwritten by the next product

            const float* const cst = reinterpret_cast<const float*>(sm + G::kSCst) + (j & (kCstRing - 1)) * 3 * kKeys + 4 * c2;
            // pair 2 (2 a + h): row a, keys 16 a + 4 c2 + 2 h + {0, 1}; pair 2 (2 a + h) + 1: the same keys of row b.
            // Paired fp32 instructions (two IEEE operations per issue slot) carry the scaling, the shift by the
            // maximum, the denominators and the rescale of O.
            float2 sv[16];
#pragma unroll
            for (int a = 0; a < 4; ++a) {
                const float4 kk = *reinterpret_cast<const float4*>(cst + 16 * a);
                const float4 lg = *reinterpret_cast<const float4*>(cst + kKeys + 16 * a);
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int r = 4 * (2 * a + h);
                    const float2 k2 = h ? make_float2(kk.z, kk.w) : make_float2(kk.x, kk.y);
                    const float2 l2 = h ? make_float2(lg.z, lg.w) : make_float2(lg.x, lg.y);
                    sv[r / 2] = fma2_rn(make_float2(__uint_as_float(sr[r]), __uint_as_float(sr[r + 1])), k2, l2);
                    sv[r / 2 + 1] = fma2_rn(make_float2(__uint_as_float(sr[r + 2]), __uint_as_float(sr[r + 3])), k2, l2);
                }
            }
            if (j * kKeys + kKeys - 1 > qpos_min) {                     // tiles that reach past a row's diagonal
#pragma unroll
                for (int g = 0; g < 8; ++g) {
                    const int key = j * kKeys + 16 * (g >> 1) + 4 * c2 + 2 * (g & 1);
                    if (key > qpos_a) sv[2 * g].x = -INFINITY;
                    if (key + 1 > qpos_a) sv[2 * g].y = -INFINITY;
                    if (key > qpos_b) sv[2 * g + 1].x = -INFINITY;
                    if (key + 1 > qpos_b) sv[2 * g + 1].y = -INFINITY;
                }
            }
            float mx_a = -INFINITY, mx_b = -INFINITY;
#pragma unroll
            for (int g = 0; g < 8; ++g) {
                mx_a = fmaxf(mx_a, fmaxf(sv[2 * g].x, sv[2 * g].y));
                mx_b = fmaxf(mx_b, fmaxf(sv[2 * g + 1].x, sv[2 * g + 1].y));
            }
            mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
            mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
            mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
            mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
            // The maximum is followed exactly: the largest weight of a row is then exactly 1 in f16, so a row
            // dominated by one key keeps its weight-to-sum ratio free of f16 rounding.
            const float mn_a = fmaxf(m_a, mx_a), mn_b = fmaxf(m_b, mx_b);
            const float corr_a = ex2f(m_a - mn_a), corr_b = ex2f(m_b - mn_b);
            m_a = mn_a;
            m_b = mn_b;
            const float2 neg_a = splat2(-mn_a), neg_b = splat2(-mn_b);
            float2 sum_a = make_float2(0.0f, 0.0f), sum_b = make_float2(0.0f, 0.0f);
            uint32_t wv[16];                 // word 4 a + h: row a, keys 16 a + 4 c2 + 2 h + {0, 1}; 4 a + 2 + h: row b
#pragma unroll
            for (int a = 0; a < 4; ++a) {
                const float4 rv = *reinterpret_cast<const float4*>(cst + 2 * kKeys + 16 * a);
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int g = 2 * a + h;
                    const float2 r2 = h ? make_float2(rv.z, rv.w) : make_float2(rv.x, rv.y);
                    const float2 xa = add2_rn(sv[2 * g], neg_a), xb = add2_rn(sv[2 * g + 1], neg_b);
                    const float2 ea = make_float2(ex2f(xa.x), ex2f(xa.y)), eb = make_float2(ex2f(xb.x), ex2f(xb.y));
                    sum_a = fma2_rn(ea, r2, sum_a);
                    sum_b = fma2_rn(eb, r2, sum_b);
                    wv[4 * a + h] = pack_f16x2(ea.x, ea.y);
                    wv[4 * a + 2 + h] = pack_f16x2(eb.x, eb.y);
                }
            }
            l_a = fmaf(l_a, corr_a, sum_a.x + sum_a.y);
            l_b = fmaf(l_b, corr_b, sum_b.x + sum_b.y);
            const bool moved = j > 0 && __any_sync(0xffffffffu, corr_a != 1.0f || corr_b != 1.0f);
            // W buffer j % 2 is free: O += W_{j-2} V_{j-2} was issued before S_j by the same thread, and the commit
            // that completed the barrier of S_j covers every product issued before it.  O may only be touched
            // once O += W_{j-1} V_{j-1} has completed, which is waited for only when a maximum moved.  Skipping
            // that wait on other tiles is safe for the parity test: no product of a later tile can complete
            // before this warp has signalled "W ready" for it.
            if (moved) {
                ok = wait_phase(&bb[kBarPV + ((j - 1) & 1)], ((j - 1) >> 1) & 1, gave_up, __LINE__, p.error_word);
                if (!ok) break;
                tc_fence_after();
            }
            tmem_st_frag_x4(tmem_w + (j & 1) * (kKeys / 2) + my_lanes16, wv);
            if (moved) {
                const float2 ca = splat2(corr_a), cb2 = splat2(corr_b);
#pragma unroll 1
                for (int cb = 0; cb < kD; cb += 64) {        // two round trips through tensor memory
                    uint32_t ov[32];
                    tmem_ld_frag_x8(ov, tmem_o + my_lanes16 + cb);
#pragma unroll
                    for (int g = 0; g < 8; ++g) {
                        const float2 oa = mul2_rn(make_float2(__uint_as_float(ov[4 * g]), __uint_as_float(ov[4 * g + 1])), ca);
                        const float2 ob = mul2_rn(make_float2(__uint_as_float(ov[4 * g + 2]), __uint_as_float(ov[4 * g + 3])), cb2);
                        ov[4 * g] = __float_as_uint(oa.x);
                        ov[4 * g + 1] = __float_as_uint(oa.y);
                        ov[4 * g + 2] = __float_as_uint(ob.x);
                        ov[4 * g + 3] = __float_as_uint(ob.y);
                    }
                    tmem_st_frag_x8(tmem_o + my_lanes16 + cb, ov);
                }
            }
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            tc_fence_before();
            __syncwarp();
            if (lane == 0) pipe::mbar_arrive(&bb[kBarWReady]);
        }
        // ---- epilogue: normalise and store this thread's two rows ----
        if (ok && n_tiles > 0)
            ok = wait_phase(&bb[kBarPV + ((n_tiles - 1) & 1)], ((n_tiles - 1) >> 1) & 1, gave_up, __LINE__, p.error_word);
        if (ok && n_tiles > 0) {
            tc_fence_after();
            l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
            l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
            l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
            l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
            const float inv_a = 1.0f / l_a, inv_b = 1.0f / l_b;
            const int hig_a = chunk * p.heads_per_cta + slot_a, hig_b = chunk * p.heads_per_cta + slot_b;
            const bool valid_a = slot_a < p.heads_per_cta && hig_a < p.group && tok_a < p.n_new;
            const bool valid_b = slot_b < p.heads_per_cta && hig_b < p.group && tok_b < p.n_new;
            __nv_bfloat16* const dst_a = p.out + (static_cast<size_t>(valid_a ? tok_a : 0) * p.num_q_heads + (valid_a ? kvh * p.group + hig_a : 0)) * kD + 2 * c2;
            __nv_bfloat16* const dst_b = p.out + (static_cast<size_t>(valid_b ? tok_b : 0) * p.num_q_heads + (valid_b ? kvh * p.group + hig_b : 0)) * kD + 2 * c2;
#pragma unroll 1
            for (int cb = 0; cb < kD; cb += 32) {
                uint32_t ov[16];
                tmem_ld_frag_x4(ov, tmem_o + my_lanes16 + cb);
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    if (valid_a)
                        *reinterpret_cast<__nv_bfloat162*>(dst_a + cb + 8 * g) =
                            __floats2bfloat162_rn(__uint_as_float(ov[4 * g]) * inv_a, __uint_as_float(ov[4 * g + 1]) * inv_a);
                    if (valid_b)
                        *reinterpret_cast<__nv_bfloat162*>(dst_b + cb + 8 * g) =
                            __floats2bfloat162_rn(__uint_as_float(ov[4 * g + 2]) * inv_b, __uint_as_float(ov[4 * g + 3]) * inv_b);
                }
            }
        }
    } else if (warp < G::kConvWarp0) {
        // =============================== products of row block `blk` ===============================
        constexpr uint32_t kIdescQK = instr_desc(kKeys, false);
        constexpr uint32_t kIdescPV = instr_desc(kD, true);
        auto issue_qk = [&](int tile_j) {                     // S = Q K^T: eight products of depth 16
            tc_fence_after();
            if (lane == 0) {
                const uint32_t k_base = base + G::kSK + (tile_j & 1) * kTileBytes;
#pragma unroll
                for (int s = 0; s < 4; ++s)       // dims 0..63: both operands from shared memory
                    umma_f16(tmem_s, smem_desc(base + q_off + s * 32, 16), smem_desc(k_base + s * 32, 16), kIdescQK, s > 0);
#pragma unroll
                for (int s = 0; s < 4; ++s)       // dims 64..127
                    umma_f16(tmem_s, smem_desc(base + q_off + kRows * 128 + s * 32, 16), smem_desc(k_base + kKeys * 128 + s * 32, 16), kIdescQK, true);
                umma_commit(&bb[kBarQK + (tile_j & 1)]);
            }
            __syncwarp();
        };
        bool ok = wait_phase<kLazyNs>(&bars[G::kBarKReady], 0, gave_up, __LINE__, p.error_word);
        if (ok) issue_qk(0);
        for (int j = 0; j < n_tiles && ok; ++j) {
            if (j + 1 < n_tiles) {
                ok = wait_phase<kLazyNs>(&bb[kBarSRead], j & 1, gave_up, __LINE__, p.error_word) &&
                     wait_phase<kLazyNs>(&bars[G::kBarKReady + ((j + 1) & 1)], ((j + 1) >> 1) & 1, gave_up, __LINE__, p.error_word);
                if (!ok) break;
                issue_qk(j + 1);
            }
            ok = wait_phase<kLazyNs>(&bb[kBarWReady], j & 1, gave_up, __LINE__, p.error_word) &&
                 wait_phase<kLazyNs>(&bars[G::kBarVReady + (j & 1)], (j >> 1) & 1, gave_up, __LINE__, p.error_word);
            if (!ok) break;
            tc_fence_after();
            if (lane == 0) {
                const uint32_t v_base = base + G::kSV + (j & 1) * kTileBytes;
#pragma unroll
                for (int s = 0; s < kKeys / 16; ++s)
                    umma_f16_ts(tmem_o, tmem_w + (j & 1) * (kKeys / 2) + s * 8, smem_desc(v_base + s * 2048, kKeys * 128), kIdescPV, j > 0 || s > 0);
                umma_commit(&bb[kBarPV + (j & 1)]);
            }
            __syncwarp();
        }
    } else {
        // =============================== conversion ===============================
        constexpr int kPerConv = G::kPerConv;
        const int t = tid - 32 * G::kConvWarp0;
        const uint32_t row_stride = static_cast<uint32_t>(p.num_kv_heads) * kD;
        // A raw tile holds the rows in operand order, [row][128 bytes, swizzled].  It is copied with eight
        // consecutive threads on the eight 16-byte pieces of one row (whole 128-byte lines of the cache) and
        // converted with eight consecutive threads on the same piece of eight consecutive rows (conflict-free
        // in the raw tile and in the operand tile); the conversion group meets at a named barrier in between.
        // All offsets are fixed per thread; the global pointers advance by one tile per step.
        uint32_t copy_off[kPerConv], raw_off[kPerConv], dst_off[kPerConv], gk_off[kPerConv], gv_off[kPerConv];
        int k_key[kPerConv], v_key[kPerConv];
#pragma unroll
        for (int i = 0; i < kPerConv; ++i) {
            const int c = t + G::kConvThreads * i;
            const int cr = (c >> 3) & (kKeys - 1), cch = c & 7;             // the copy's row and piece
            copy_off[i] = swz128(cr, cch);
            k_key[i] = key_of_k_row(cr);
            v_key[i] = cr;
            gk_off[i] = static_cast<uint32_t>(k_key[i]) * row_stride + cch * 16;
            gv_off[i] = static_cast<uint32_t>(v_key[i]) * row_stride + cch * 16;
            const int r = c & (kKeys - 1), ch = (c >> 6) & 7;               // the conversion's row and piece
            raw_off[i] = swz128(r, ch);
            dst_off[i] = (ch >> 2) * (kKeys * 128) + swz128(r, 2 * (ch & 3));       // the second half sits at ^ 16
        }
        const bool has_last = t + G::kConvThreads * (kPerConv - 1) < kChunks;      // the last chunk may exist in the first warps only
        const size_t tile_bytes = static_cast<size_t>(kKeys) * row_stride;
        const uint8_t* gk = p.k + static_cast<size_t>(kvh) * kD;
        const uint8_t* gv = p.v + static_cast<size_t>(kvh) * kD;
        const float* gks = p.k_scale + static_cast<size_t>(t & (kKeys - 1)) * p.num_kv_heads + kvh;
        const float* gvs = p.v_scale + static_cast<size_t>(t & (kKeys - 1)) * p.num_kv_heads + kvh;
        const size_t tile_scales = static_cast<size_t>(kKeys) * p.num_kv_heads;
        int next_k0 = 0, next_v0 = 0;                       // first key of the tile the next issue fetches
        auto issue_k = [&]() {
            const int room = total_keys - next_k0;          // keys of the tile that exist (the rest is zero-filled)
#pragma unroll
            for (int i = 0; i < kPerConv; ++i) {
                if (i + 1 < kPerConv || has_last) {
                    const bool live = k_key[i] < room;
                    cp16_zfill(base + G::kSRawK + copy_off[i], live ? gk + gk_off[i] : p.k, live);
                }
            }
            if (t < kKeys) {                                  // the scales stay in key order
                const bool live = t < room;
                cp4_zfill(base + G::kSRawS + t * 4, live ? gks : p.k_scale, live);
                cp4_zfill(base + G::kSRawS + kKeys * 4 + t * 4, live ? gvs : p.v_scale, live);
            }
            cp_async_commit();
            gk += tile_bytes;
            gks += tile_scales;
            gvs += tile_scales;
            next_k0 += kKeys;
        };
        auto issue_v = [&]() {
            const int room = total_keys - next_v0;
#pragma unroll
            for (int i = 0; i < kPerConv; ++i) {
                if (i + 1 < kPerConv || has_last) {
                    const bool live = v_key[i] < room;
                    cp16_zfill(base + G::kSRawV + copy_off[i], live ? gv + gv_off[i] : p.v, live);
                }
            }
            cp_async_commit();
            gv += tile_bytes;
            next_v0 += kKeys;
        };
        // E4M3 -> f16 into an operand tile: [dim block of 64][row][128 bytes, swizzled]; K and V share the form
        // (K is consumed K-major: a row is a key; V MN-major: the 128 bytes of a row are 64 consecutive dims)
        auto convert_rows = [&](int raw_base, int dst_base) {
#pragma unroll
            for (int i = 0; i < kPerConv; ++i) {
                if (i + 1 < kPerConv || has_last) {
                    const uint4 w = *reinterpret_cast<const uint4*>(sm + raw_base + raw_off[i]);
                    uint4 h0, h1;
                    e4m3x4_to_f16x2x2(w.x, h0.x, h0.y);
                    e4m3x4_to_f16x2x2(w.y, h0.z, h0.w);
                    e4m3x4_to_f16x2x2(w.z, h1.x, h1.y);
                    e4m3x4_to_f16x2x2(w.w, h1.z, h1.w);
                    unsigned char* const dst = sm + dst_base + dst_off[i];
                    *reinterpret_cast<uint4*>(dst) = h0;
                    *reinterpret_cast<uint4*>(reinterpret_cast<uintptr_t>(dst) ^ 16) = h1;
                }
            }
        };
        // a tile buffer is free once every row block's product that read it has completed
        auto wait_blocks = [&](int which, int buf, uint32_t parity, int where) {
            bool all = true;
#pragma unroll
            for (int g = 0; g < kBlocks; ++g)
                all = all && wait_phase<kLazyNs>(&bars[g * G::kBarsPerBlock + which + buf], parity, gave_up, where, p.error_word);
            return all;
        };
        issue_k();
        issue_v();
        bool ok = true;
        for (int j = 0; j < n_tiles && ok; ++j) {
            const int buf = j & 1;
            const uint32_t freed = ((j - 2) >> 1) & 1;       // phase in which tile j - 2 released buffer `buf`
            // K of tile j, once S_{j-2} is complete
            if (j >= 2) ok = wait_blocks(kBarQK, buf, freed, __LINE__);
            cp_async_wait<1>();                                          // this thread's K pieces and scales of tile j
            if (group_or(1, G::kConvThreads, !ok)) { ok = false; break; }    // everyone's pieces have landed
            convert_rows(G::kSRawK, G::kSK + buf * kTileBytes);
            if (t < kKeys) {      // K scale x softmax scale x log2(e), log2 of the V scale, its inverse
                const float* const sc = reinterpret_cast<const float*>(sm + G::kSRawS);
                float* const cst = reinterpret_cast<float*>(sm + G::kSCst) + (j & (kCstRing - 1)) * 3 * kKeys;
                const float lg = fmaxf(lg2f(sc[kKeys + t]), kLgFloor);
                cst[t] = sc[t] * p.scale_log2e;
                cst[kKeys + t] = lg;
                cst[2 * kKeys + t] = ex2f(-lg);
            }
            fence_async_smem();
            pipe::mbar_arrive(&bars[G::kBarKReady + buf]);
            named_sync(2, G::kConvThreads);                  // the raw K tile has been read by all
            issue_k();                                                   // tile j + 1 (all zeros past the last one)
            // V of tile j, once O += W_{j-2} V_{j-2} is complete
            if (j >= 2) ok = wait_blocks(kBarPV, buf, freed, __LINE__);
            cp_async_wait<1>();                                          // this thread's V pieces of tile j
            if (group_or(1, G::kConvThreads, !ok)) { ok = false; break; }
            convert_rows(G::kSRawV, G::kSV + buf * kTileBytes);
            fence_async_smem();
            pipe::mbar_arrive(&bars[G::kBarVReady + buf]);
            named_sync(2, G::kConvThreads);
            issue_v();
        }
        cp_async_wait<0>();
    }

    // ---- common exit: every role arrives here, then the tensor memory is released ----
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(G::kTmem) : "memory");
    }
}

}  // namespace ws

extern "C" int rh_selfcheck_role_wait(int tries, int* result_host) {
    RH_REQUIRE(result_host != nullptr, RH_ERR_INVALID_ARG, "rh_selfcheck_role_wait: null pointer");
    RH_REQUIRE(tries >= 16 && tries <= (1 << 16), RH_ERR_INVALID_ARG, "rh_selfcheck_role_wait: tries must be in 16..65536");
    int* scratch = nullptr;
    if (cudaMalloc(&scratch, 4 * sizeof(int)) != cudaSuccess) return host::fail(RH_ERR_CUDA, "rh_selfcheck_role_wait: cudaMalloc failed");
    cudaMemset(scratch, 0, 4 * sizeof(int));
    ws::role_wait_probe_kernel<<<1, 64>>>(tries, scratch);
    if (int e = host::check_launch("role_wait_probe_kernel")) {
        cudaFree(scratch);
        return e;
    }
    const cudaError_t err = cudaMemcpy(result_host, scratch, 4 * sizeof(int), cudaMemcpyDeviceToHost);
    cudaFree(scratch);
    if (err != cudaSuccess) return host::fail(RH_ERR_CUDA, "rh_selfcheck_role_wait: %s", cudaGetErrorString(err));
    return RH_OK;
}

// Launcher of the role-split forms; `a` is filled in by launch_flash_prefill_tc (tokens_per_cta per row block).
// blocks: row blocks per CTA (the caller picks two once the one-block grid exceeds the SM count).
int launch_flash_prefill_ws(const tc::Args& a, int blocks, cudaStream_t stream, const char* fn) {
    const unsigned grid_y = static_cast<unsigned>(a.num_kv_heads * a.head_chunks);
    if (blocks == 2) {
        using G = ws::Geo<2>;
        const dim3 grid(static_cast<unsigned>((a.n_new + 2 * a.tokens_per_cta - 1) / (2 * a.tokens_per_cta)), grid_y);
        (void)host::setup<&ws::flash_prefill_ws_kernel<2>, G::kThreads, G::kSmemBytes>();
        host::launch<ws::flash_prefill_ws_kernel<2>>(grid, dim3(G::kThreads), static_cast<size_t>(G::kSmemBytes), stream, a);
    } else {
        using G = ws::Geo<1>;
        const dim3 grid(static_cast<unsigned>((a.n_new + a.tokens_per_cta - 1) / a.tokens_per_cta), grid_y);
        (void)host::setup<&ws::flash_prefill_ws_kernel<1>, G::kThreads, G::kSmemBytes>();
        host::launch<ws::flash_prefill_ws_kernel<1>>(grid, dim3(G::kThreads), static_cast<size_t>(G::kSmemBytes), stream, a);
    }
    return host::check_launch(fn);
}

}  // namespace rh
