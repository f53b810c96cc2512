// Causal prefill attention over the FP8-E4M3 KV cache on the 5th-generation tensor cores
// (tcgen05.mma, accumulators in tensor memory).  Same contract as flash_prefill.cu
// (runtherder::kernels::flash_prefill_bf16, include/runtherder/kernels/flash_prefill.cuh:27-40).
//
// A CTA owns 128 query rows of one kv head — four query heads x 32 consecutive tokens (three x 42, two x 64, one x 128) —
// and walks the causal key tiles of 64 keys with 128 x kParts threads (kParts threads share a row: each
// takes 64 / kParts keys of the row's scores and 128 / kParts columns of its output):
//   raw E4M3 rows of the tile (cp.async, each thread its own chunks)
//     -> f16 operand tiles in shared memory in the canonical 128-byte-swizzled layouts (exact conversion)
//     -> S[128 x 64] = Q K^T: eight tcgen05.mma (M=128, N=64, K=16), fp32 in tensor memory
//     -> the threads of row r load their part of S row r (tcgen05.ld 32x32b), apply the K scale, the V scale
//        in the exponent and the causal mask, agree on the row maximum through shared memory (a named
//        barrier per 32-row quarter), store their weights as f16 pairs into tensor memory (tcgen05.st) and
//        rescale their columns of O in tensor memory when the running maximum moved
//     -> O[128 x 128] += W V: four tcgen05.mma (M=128, N=128, K=16) with W read from tensor memory and V
//        read MN-major from shared memory exactly as the cache stores it.
// The default form (kFrag) reads the scores in the tensor core's accumulator-fragment shape instead
// (tcgen05.ld 16x256b): a warp owns 16 rows and all 64 keys of the tile, a thread two rows and sixteen keys —
// four runs of four consecutive keys — so a row's maximum is two shuffles away, no value crosses a warp, and a
// thread reads 48 per-key constants per tile instead of 96.  For the weights to land where the A operand of
// O += W V expects them, the K rows of the tile are laid out in the order that makes S column
// 16a + 8h + 2c + e hold key 16a + 4c + 2h + e.
// One elected thread issues the products; completion comes back through mbarriers (tcgen05.commit).
// Every mbarrier wait is bounded and agreed on by the whole CTA (__syncthreads_or), and every path out
// of the kernel releases the tensor memory it allocated.
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include <atomic>

#include "flash_prefill_tc.cuh"
#include "rh_kernels.h"

namespace rh {
namespace tc {

// grid (token tiles, num_kv_heads * head_chunks), 128 * kParts threads.
template <int kParts, bool kFrag = false>
__global__ void __launch_bounds__(128 * kParts, 2) flash_prefill_tc_kernel(const Args p) {
    static_assert(!kFrag || kParts == 2, "the fragment form is written for eight warps");
    constexpr int kThreads = 128 * kParts;
    constexpr int kC = kKeys / kParts;       // score columns per thread
    constexpr int kOC = kD / kParts;         // output columns per thread
    extern __shared__ unsigned char raw_smem[];
    const uint32_t base = (pipe::smem_u32(raw_smem) + 1023u) & ~1023u;          // shared-space address, 1 KB aligned
    unsigned char* const sm = raw_smem + (base - pipe::smem_u32(raw_smem));     // the same place, generic pointer
    uint64_t* const bar_s = reinterpret_cast<uint64_t*>(sm + kOffBar);
    uint64_t* const bar_o = bar_s + 1;
    uint32_t* const tmem_slot = reinterpret_cast<uint32_t*>(sm + kOffBar + 16);
    float* const xch = reinterpret_cast<float*>(sm + kOffXch);

    const int tid = threadIdx.x, warp = tid >> 5;
    const int row = tid & (kRows - 1), part = tid >> 7;     // warp w reaches tensor-memory lanes 32 (w % 4) ..
    const int kvh = blockIdx.y / p.head_chunks;
    const int chunk = blockIdx.y - kvh * p.head_chunks;
    const int tile = gridDim.x - 1 - blockIdx.x;            // long (late) token tiles first
    const int tok0 = tile * p.tokens_per_cta;
    // row = (head slot row / tokens_per_cta, token row % tokens_per_cta)
    const int head_slot = row / p.tokens_per_cta;
    const int tok = tok0 + (row - head_slot * p.tokens_per_cta);
    const int head_in_group = chunk * p.heads_per_cta + head_slot;
    const bool row_valid = head_slot < p.heads_per_cta && head_in_group < p.group && tok < p.n_new;   // rows past the block's head slots idle
    const int qh = kvh * p.group + head_in_group;

    // ---- one-time set-up: barriers, tensor memory ----
    if (tid == 0) {
        pipe::mbar_init(bar_s, 1);
        pipe::mbar_init(bar_o, 1);
        pipe::mbar_init_fence();
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(pipe::smem_u32(tmem_slot)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    const uint32_t tmem_s = tmem, tmem_o = tmem + kKeys, tmem_w = tmem + kKeys + kD;   // column offsets
    const uint32_t tmem_q = tmem_w + kKeys / 2;
    const uint32_t my_lane = static_cast<uint32_t>(32 * (warp & 3)) << 16;     // this warp's quarter of the 128 lanes

    pdl_enter();
    const int clen = *p.cache_len;
    const int total_keys = clen + p.n_new;
    const int last_tok = min(tok0 + p.tokens_per_cta, p.n_new) - 1;
    const int n_tiles = min((total_keys + kKeys - 1) / kKeys, (clen + last_tok) / kKeys + 1);
    const int qpos = clen + tok;

    // ---- raw tile copies and conversion: thread t owns key t % 64 and the 16-byte chunks c0, c0 + kStep, ...
    //      of its K row and of its V row (eight consecutive keys per quarter-warp: conflict-free both ways).
    //      Every shared-memory offset is fixed per thread; the global pointers advance by one tile per step.
    constexpr uint32_t kIdescQK = instr_desc(kKeys, false);
    constexpr uint32_t kIdescPV = instr_desc(kD, true);
    constexpr int kStep = kThreads / 64;     // chunk stride between this thread's chunks of a row
    constexpr int kNch = 8 / kStep;          // chunks per row and matrix
    const int key_l = tid & 63, c0 = tid >> 6;
    // the key whose K row becomes row key_l of the K operand tile (the fragment form's column order, see the top)
    const int kkey = kFrag ? ((key_l & 48) | ((key_l & 6) << 1) | ((key_l & 8) >> 2) | (key_l & 1)) : key_l;
    const size_t row_stride = static_cast<size_t>(p.num_kv_heads) * kD;
    const size_t head_off = static_cast<size_t>(kvh) * kD + c0 * 16;
    const uint8_t* gk = p.k + static_cast<size_t>(kkey) * row_stride + head_off;
    const uint8_t* gv = p.v + static_cast<size_t>(key_l) * row_stride + head_off;
    const size_t tile_bytes = static_cast<size_t>(kKeys) * row_stride;
    const float* gks = p.k_scale + static_cast<size_t>(key_l) * p.num_kv_heads + kvh;
    const float* gvs = p.v_scale + static_cast<size_t>(key_l) * p.num_kv_heads + kvh;
    const size_t tile_scales = static_cast<size_t>(kKeys) * p.num_kv_heads;
    uint32_t raw_off[kNch], dst_off[kNch];
#pragma unroll
    for (int t = 0; t < kNch; ++t) {
        const int ch = c0 + t * kStep;
        raw_off[t] = kOffRaw + swz128(key_l, ch);
        dst_off[t] = (ch >> 2) * (kKeys * 128) + swz128(key_l, 2 * (ch & 3));      // the second half sits at ^ 16
    }
    // K rows (with both scale vectors) and V rows travel as separate cp.async groups, issued in the order
    // K0 V0 K1 V1 ...: a wait that leaves one group pending always covers the tile part needed next.
    int next_key_k = kkey, next_key_v = key_l;           // this thread's key in the tile the next issue fetches
    auto issue_k = [&]() {
        const bool live = next_key_k < total_keys;
#pragma unroll
        for (int t = 0; t < kNch; ++t) cp16_zfill(base + raw_off[t], live ? gk + t * kStep * 16 : p.k, live);
        if (tid < kKeys) {                                // the scales stay in key order
            const bool live_s = next_key_k - kkey + tid < total_keys;
            cp4_zfill(base + kOffRaw + 2 * kKeys * kD + tid * 4, live_s ? gks : p.k_scale, live_s);
            cp4_zfill(base + kOffRaw + 2 * kKeys * kD + kKeys * 4 + tid * 4, live_s ? gvs : p.v_scale, live_s);
        }
        cp_async_commit();
        gk += tile_bytes;
        gks += tile_scales;
        gvs += tile_scales;
        next_key_k += kKeys;
    };
    auto issue_v = [&]() {
        const bool live = next_key_v < total_keys;
#pragma unroll
        for (int t = 0; t < kNch; ++t) cp16_zfill(base + raw_off[t] + kKeys * kD, live ? gv + t * kStep * 16 : p.v, live);
        cp_async_commit();
        gv += tile_bytes;
        next_key_v += kKeys;
    };
    // E4M3 -> f16 into the operand tiles: [dim block of 64][key][128 bytes, swizzled]; K and V share the form
    // (K is consumed K-major: a row is a key; V MN-major: the 128 bytes of a row are 64 consecutive dims)
    auto convert_rows = [&](int which) {
#pragma unroll
        for (int t = 0; t < kNch; ++t) {
            const uint4 w = *reinterpret_cast<const uint4*>(sm + raw_off[t] + which * (kKeys * kD));
            uint4 h0, h1;
            e4m3x4_to_f16x2x2(w.x, h0.x, h0.y);
            e4m3x4_to_f16x2x2(w.y, h0.z, h0.w);
            e4m3x4_to_f16x2x2(w.z, h1.x, h1.y);
            e4m3x4_to_f16x2x2(w.w, h1.z, h1.w);
            unsigned char* const dst = sm + (which ? kOffV : kOffK) + dst_off[t];
            *reinterpret_cast<uint4*>(dst) = h0;
            *reinterpret_cast<uint4*>(reinterpret_cast<uintptr_t>(dst) ^ 16) = h1;
        }
    };
    // K rows plus the per-key constants of the tile: K scale x softmax scale x log2(e), log2 of the V scale, its inverse
    auto convert_k = [&]() {
        convert_rows(0);
        if (tid < kKeys) {
            const float* const sc = reinterpret_cast<const float*>(sm + kOffRaw + 2 * kKeys * kD);
            float* const cst = reinterpret_cast<float*>(sm + kOffCst);
            const float lg = fmaxf(lg2f(sc[kKeys + tid]), kLgFloor);
            cst[tid] = sc[tid] * p.scale_log2e;
            cst[kKeys + tid] = lg;
            cst[2 * kKeys + tid] = ex2f(-lg);
        }
    };
    auto issue_qk = [&]() {                               // S = Q K^T: eight products of depth 16
        tc_fence_after();
#pragma unroll
        for (int s = 0; s < 4; ++s)       // dims 0..63: both operands from shared memory
            umma_f16(tmem_s, smem_desc(base + kOffQ + s * 32, 16), smem_desc(base + kOffK + s * 32, 16), kIdescQK, s > 0);
#pragma unroll
        for (int s = 0; s < 4; ++s)       // dims 64..127: Q from tensor memory
            umma_f16_ts(tmem_s, tmem_q + s * 8, smem_desc(base + kOffK + kKeys * 128 + s * 32, 16), kIdescQK, true);
        umma_commit(bar_s);
    };
    issue_k();
    issue_v();

    // ---- Q: row `row`, bf16 -> f16.  Dims 0..63 go to shared memory ([row][128 bytes, swizzled]), dims 64..127 to
    //      tensor memory (row = lane, two f16 per column) as the A operand of the second half of S = Q K^T.
    //      kParts threads share the row's 16 chunks of 8 dims; `part` is uniform in a warp. ----
    {
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
        constexpr int kPer = kParts == 1 ? 8 : 16 / kParts;     // chunks per thread and half
        if (kParts == 1 || part < kParts / 2) {
#pragma unroll
            for (int c = 0; c < kPer; ++c) {
                const int cidx = (kParts == 1 ? 0 : part * kPer) + c;
                *reinterpret_cast<uint4*>(sm + kOffQ + swz128(row, cidx)) = load_chunk(cidx);
            }
        }
        if (kParts == 1 || part >= kParts / 2) {
            uint32_t qw[4 * kPer];
            const int first = kParts == 1 ? 0 : (part - kParts / 2) * kPer;     // chunk within the upper half
#pragma unroll
            for (int c = 0; c < kPer; ++c) {
                const uint4 h = load_chunk(8 + first + c);
                qw[4 * c] = h.x;
                qw[4 * c + 1] = h.y;
                qw[4 * c + 2] = h.z;
                qw[4 * c + 3] = h.w;
            }
            tmem_st_words<4 * kPer>(tmem_q + my_lane + 4 * first, qw);
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        }
    }

    float m_run = kMInit, l_run = 0.0f;      // m_run is the same in all threads of a row; l_run is this thread's part
    bool failed = false;
    // fragment form: this thread's two rows (lanes 16 (warp / 4) + lane / 4 and + 8 of the warp's quarter) and
    // their state; its keys are 16 a + 4 (lane % 4) + i, a and i in 0..3
    const int lane = tid & 31;
    const int c2 = lane & 3;
    const int row_a = 32 * (warp & 3) + 16 * (warp >> 2) + (lane >> 2), row_b = row_a + 8;
    const uint32_t my_lanes16 = static_cast<uint32_t>(32 * (warp & 3) + 16 * (warp >> 2)) << 16;
    const int slot_a = row_a / p.tokens_per_cta, slot_b = row_b / p.tokens_per_cta;
    const int tok_a = tok0 + (row_a - slot_a * p.tokens_per_cta), tok_b = tok0 + (row_b - slot_b * p.tokens_per_cta);
    const int qpos_a = clen + tok_a, qpos_b = clen + tok_b;
    float m_a = kMInit, m_b = kMInit, l_a = 0.0f, l_b = 0.0f;

    // ---- prologue: K of tile 0 converted, S_0 = Q K_0^T under way, V of tile 0 converted meanwhile ----
    cp_async_wait<1>();                                          // K rows and scales of tile 0 (V rows may be pending)
    convert_k();
    issue_k();                                                   // tile 1 (an empty group past the last tile)
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    if (tid == 0) issue_qk();
    cp_async_wait<1>();                                          // V rows of tile 0
    convert_rows(1);
    issue_v();

    // Steady state of tile j.  The tensor core works on O += W_j V_j while the threads convert K of tile j+1,
    // and on S_{j+1} while they convert V of tile j+1; the threads' softmax of tile j follows the wait for S_j.
    for (int j = 0; j < n_tiles; ++j) {          // leaves early only through the CTA-wide votes below
        {
            const bool ok = mbar_wait_quiet(bar_s, j & 1, __LINE__, p.error_word);
            tc_fence_after();
            if (!ok) failed = true;
        }

        if constexpr (kFrag) {
            // ---- two rows x sixteen keys per thread: scales, mask, maxima (two shuffles), weights, sums ----
            const float* const cst = reinterpret_cast<const float*>(sm + kOffCst) + 4 * c2;
            uint32_t sr[32];
            tmem_ld_frag_x8(sr, tmem_s + my_lanes16);
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
            if (j * kKeys + kKeys - 1 > min(qpos_a, qpos_b)) {       // tiles that reach past a row's diagonal
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
            // the maximum is followed exactly (see the other form below)
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
            tmem_st_frag_x4(tmem_w + my_lanes16, wv);
            l_a = fmaf(l_a, corr_a, sum_a.x + sum_a.y);
            l_b = fmaf(l_b, corr_b, sum_b.x + sum_b.y);
            if (j > 0 && __any_sync(0xffffffffu, corr_a != 1.0f || corr_b != 1.0f)) {
                const float2 ca = splat2(corr_a), cb2 = splat2(corr_b);
#pragma unroll 1
                for (int cb = 0; cb < kD; cb += 32) {
                    uint32_t ov[16];
                    tmem_ld_frag_x4(ov, tmem_o + my_lanes16 + cb);
#pragma unroll
                    for (int g = 0; g < 4; ++g) {
                        const float2 oa = mul2_rn(make_float2(__uint_as_float(ov[4 * g]), __uint_as_float(ov[4 * g + 1])), ca);
                        const float2 ob = mul2_rn(make_float2(__uint_as_float(ov[4 * g + 2]), __uint_as_float(ov[4 * g + 3])), cb2);
                        ov[4 * g] = __float_as_uint(oa.x);
                        ov[4 * g + 1] = __float_as_uint(oa.y);
                        ov[4 * g + 2] = __float_as_uint(ob.x);
                        ov[4 * g + 3] = __float_as_uint(ob.y);
                    }
                    tmem_st_frag_x4(tmem_o + my_lanes16 + cb, ov);
                }
            }
        } else {
        // ---- this thread's kC scores of its row: scales, mask, maximum ----
        const float* const cst = reinterpret_cast<const float*>(sm + kOffCst) + part * kC;
        const int key0 = j * kKeys + part * kC;
        const bool diag = j * kKeys + kKeys - 1 > qpos;
        float sv[kC];
        tmem_ld<kC>(sv, tmem_s + my_lane + part * kC);
        float mx = -INFINITY;
#pragma unroll
        for (int i = 0; i < kC; i += 4) {
            const float4 kk = *reinterpret_cast<const float4*>(cst + i);
            const float4 lg = *reinterpret_cast<const float4*>(cst + kKeys + i);
            sv[i] = fmaf(sv[i], kk.x, lg.x);
            sv[i + 1] = fmaf(sv[i + 1], kk.y, lg.y);
            sv[i + 2] = fmaf(sv[i + 2], kk.z, lg.z);
            sv[i + 3] = fmaf(sv[i + 3], kk.w, lg.w);
        }
        if (diag) {                          // the one or two tiles that straddle the diagonal
#pragma unroll
            for (int i = 0; i < kC; ++i)
                if (key0 + i > qpos) sv[i] = -INFINITY;
        }
#pragma unroll
        for (int i = 0; i < kC; i += 4) mx = fmaxf(mx, fmaxf(fmaxf(sv[i], sv[i + 1]), fmaxf(sv[i + 2], sv[i + 3])));
        if constexpr (kParts > 1) {          // the row's threads sit in warps w, w + 4, ...: one named barrier per quarter
            xch[part * kRows + row] = mx;
            named_sync(1 + (warp & 3), 32 * kParts);
#pragma unroll
            for (int q = 0; q < kParts; ++q) mx = fmaxf(mx, xch[q * kRows + row]);
        }
        // The reference follows the maximum exactly: the largest weight of a row is then exactly 1 in f16,
        // so a row dominated by one key keeps its weight-to-sum ratio free of f16 rounding.  (A reference
        // that lags the maximum by a threshold saves most rescales of O but rounds the dominant weight:
        // measured, two-ulp outputs on inputs with widely spread V scales.)
        const float m_new = fmaxf(m_run, mx);
        const float corr = ex2f(m_run - m_new);
        m_run = m_new;
        float sum4[4] = {0.0f, 0.0f, 0.0f, 0.0f};      // independent chains
        uint32_t wv[kC / 2];                           // this thread's weights, two f16 per word
#pragma unroll
        for (int i = 0; i < kC; i += 8) {
            float e[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) e[u] = ex2f(sv[i + u] - m_new);
            const float4 r0 = *reinterpret_cast<const float4*>(cst + 2 * kKeys + i);
            const float4 r1 = *reinterpret_cast<const float4*>(cst + 2 * kKeys + i + 4);
            sum4[0] = fmaf(e[0], r0.x, fmaf(e[4], r1.x, sum4[0]));
            sum4[1] = fmaf(e[1], r0.y, fmaf(e[5], r1.y, sum4[1]));
            sum4[2] = fmaf(e[2], r0.z, fmaf(e[6], r1.z, sum4[2]));
            sum4[3] = fmaf(e[3], r0.w, fmaf(e[7], r1.w, sum4[3]));
            wv[i / 2] = pack_f16x2(e[0], e[1]);
            wv[i / 2 + 1] = pack_f16x2(e[2], e[3]);
            wv[i / 2 + 2] = pack_f16x2(e[4], e[5]);
            wv[i / 2 + 3] = pack_f16x2(e[6], e[7]);
        }
        // W stays in tensor memory as the A operand of O += W V (O += W_{j-1} V_{j-1} has completed: see below)
        tmem_st_words<kC / 2>(tmem_w + my_lane + part * (kC / 2), wv);
        l_run = fmaf(l_run, corr, (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));
        // this thread's columns of the O row (O += W_{j-1} V_{j-1} completed before V of this tile was converted)
        if (j > 0 && __any_sync(0xffffffffu, corr != 1.0f)) {
#pragma unroll 1
            for (int cb = 0; cb < kOC; cb += 32) {
                float ov[32];
                tmem_ld32(ov, tmem_o + my_lane + part * kOC + cb);
#pragma unroll
                for (int i = 0; i < 32; ++i) ov[i] *= corr;
                tmem_st32(tmem_o + my_lane + part * kOC + cb, ov);
            }
        }
        }   // !kFrag
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        fence_async_smem();
        tc_fence_before();
        if (__syncthreads_or(failed)) { failed = true; break; }

        // ---- O += W_j V_j ----
        if (tid == 0) {
            tc_fence_after();
#pragma unroll
            for (int s = 0; s < kKeys / 16; ++s)
                umma_f16_ts(tmem_o, tmem_w + s * 8, smem_desc(base + kOffV + s * 2048, kKeys * 128), kIdescPV, j > 0 || s > 0);
            umma_commit(bar_o);
        }
        if (j + 1 < n_tiles) {
            // K of tile j+1: the K tile is free (S_j is complete), the product above runs meanwhile
            cp_async_wait<1>();
            convert_k();
            issue_k();
            fence_async_smem();
            tc_fence_before();
            if (__syncthreads_or(failed)) { failed = true; break; }
            if (tid == 0) issue_qk();                            // every thread has read S_j: its columns are free
            // V of tile j+1 once O += W_j V_j is complete; S_{j+1} runs meanwhile
            const bool ok = mbar_wait_quiet(bar_o, j & 1, __LINE__, p.error_word);
            tc_fence_after();
            if (!ok) failed = true;
            cp_async_wait<1>();
            convert_rows(1);
            issue_v();
        }
    }

    // ---- epilogue: normalise, store; every path releases the tensor memory ----
    if (!failed && n_tiles > 0) {
        const bool ok = mbar_wait_quiet(bar_o, (n_tiles - 1) & 1, __LINE__, p.error_word);
        tc_fence_after();
        if (!ok) failed = true;
    }
    if constexpr (kFrag) {
        if (!__syncthreads_or(failed) && n_tiles > 0) {
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
    } else {
    if constexpr (kParts > 1) xch[part * kRows + row] = l_run;     // last read of xch was before the loop's final barrier
    if (!__syncthreads_or(failed) && n_tiles > 0) {
        float l_row = l_run;
        if constexpr (kParts > 1) {
            l_row = 0.0f;
#pragma unroll
            for (int q = 0; q < kParts; ++q) l_row += xch[q * kRows + row];
        }
        const float inv = 1.0f / l_row;
        __nv_bfloat16* const dst = p.out + (static_cast<size_t>(row_valid ? tok : 0) * p.num_q_heads + (row_valid ? qh : 0)) * kD + part * kOC;
#pragma unroll 1
        for (int cb = 0; cb < kOC; cb += 32) {
            float ov[32];
            tmem_ld32(ov, tmem_o + my_lane + part * kOC + cb);
            if (row_valid) {
#pragma unroll
                for (int i = 0; i < 32; i += 8) {
                    uint4 w;
                    __nv_bfloat162 t;
                    t = __floats2bfloat162_rn(ov[i] * inv, ov[i + 1] * inv); w.x = *reinterpret_cast<uint32_t*>(&t);
                    t = __floats2bfloat162_rn(ov[i + 2] * inv, ov[i + 3] * inv); w.y = *reinterpret_cast<uint32_t*>(&t);
                    t = __floats2bfloat162_rn(ov[i + 4] * inv, ov[i + 5] * inv); w.z = *reinterpret_cast<uint32_t*>(&t);
                    t = __floats2bfloat162_rn(ov[i + 6] * inv, ov[i + 7] * inv); w.w = *reinterpret_cast<uint32_t*>(&t);
                    *reinterpret_cast<uint4*>(dst + cb + i) = w;
                }
            }
        }
    }
    }   // !kFrag
    cp_async_wait<0>();
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
    }
}

}  // namespace tc

int launch_flash_prefill_ws(const tc::Args& a, int blocks, cudaStream_t stream, const char* fn);   // flash_prefill_ws.cu

// Launcher used by rh_flash_prefill_bf16 when the tensor-memory form is selected.
int launch_flash_prefill_tc(void* out, const void* q, const uint8_t* k, const uint8_t* v, const float* k_scale,
                            const float* v_scale, int n_new, const int* cache_len, int num_q_heads, int num_kv_heads,
                            float scale, cudaStream_t stream, const char* fn) {
    tc::Args a;
    a.out = static_cast<__nv_bfloat16*>(out);
    a.q = static_cast<const __nv_bfloat16*>(q);
    a.k = k;
    a.v = v;
    a.k_scale = k_scale;
    a.v_scale = v_scale;
    a.cache_len = cache_len;
    a.error_word = host::device_error_word();
    a.n_new = n_new;
    a.num_q_heads = num_q_heads;
    a.num_kv_heads = num_kv_heads;
    a.group = num_q_heads / num_kv_heads;
    // The query heads of a kv head are dealt evenly over as few row blocks as hold them at four heads each
    // (3 -> 3, 5 -> 3 + 2, 6 -> 3 + 3, 7 -> 4 + 3), and a block takes as many tokens as fit its 128 rows (three
    // heads: 42 tokens, two rows idle), so no head slot of a block stays empty.
    a.head_chunks = (a.group + 3) / 4;
    a.heads_per_cta = (a.group + a.head_chunks - 1) / a.head_chunks;
    a.tokens_per_cta = tc::kRows / a.heads_per_cta;
    a.scale_log2e = scale * tc::kLog2e;
    const dim3 grid(static_cast<unsigned>((n_new + a.tokens_per_cta - 1) / a.tokens_per_cta),
                    static_cast<unsigned>(num_kv_heads * a.head_chunks));
    RH_REQUIRE(grid.y <= 65535u, RH_ERR_UNSUPPORTED_DIM, "%s: too many kv heads", fn);
    // +20 pads the shared-memory request of this file's forms so that one CTA fits per SM (a measuring aid)
    const int knob = host::tuning(host::kPrefillParts);
    const int parts = knob >= 20 ? knob - 20 : knob;
    const size_t smem = knob >= 20 ? 120u * 1024u : static_cast<size_t>(tc::kSmemBytes);
    constexpr size_t kOptIn = 120u * 1024u;   // the padded request is the largest one
    // Default: the role-split form (flash_prefill_ws.cu), with two row blocks per CTA once the one-block grid
    // would put more than one CTA on an SM anyway.  "prefill_parts" 5 | 6 force one | two blocks; 3 selects the
    // fragment form of this file and 1 | 2 | 4 its forms with that many threads per score row.
    if (parts <= 0 || parts == 5 || parts == 6) {
        const long long ctas_one = static_cast<long long>(grid.x) * grid.y;
        const int blocks = parts == 5 ? 1 : (parts == 6 ? 2 : (ctas_one > host::num_sms() ? 2 : 1));
        return launch_flash_prefill_ws(a, blocks, stream, fn);
    }
    if (parts == 3) {
        (void)host::setup<&tc::flash_prefill_tc_kernel<2, true>, 256, kOptIn>();
        host::launch<tc::flash_prefill_tc_kernel<2, true>>(grid, dim3(256), smem, stream, a);
    } else if (parts == 1) {
        (void)host::setup<&tc::flash_prefill_tc_kernel<1>, 128, kOptIn>();
        host::launch<tc::flash_prefill_tc_kernel<1>>(grid, dim3(128), smem, stream, a);
    } else if (parts == 4) {
        (void)host::setup<&tc::flash_prefill_tc_kernel<4>, 512, kOptIn>();
        host::launch<tc::flash_prefill_tc_kernel<4>>(grid, dim3(512), smem, stream, a);
    } else {
        (void)host::setup<&tc::flash_prefill_tc_kernel<2>, 256, kOptIn>();
        host::launch<tc::flash_prefill_tc_kernel<2>>(grid, dim3(256), smem, stream, a);
    }
    return host::check_launch(fn);
}

}  // namespace rh
