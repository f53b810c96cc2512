// Split-KV flash decode over the FP8-E4M3 KV cache: one query token, all query heads, keys
// 0 .. *cache_len, K/V dequantised by their per-(token, kv head) scales.
// Replaces runtherder::kernels::flash_decode_split_bf16
// (include/runtherder/kernels/flash_decode.cuh:27-62, src/kernels/flash_decode.cu:119-325), which
// runs one 128-thread CTA per (query head, split), re-reads a kv head's rows once per query head of
// its group and spends ~30 warp instructions per key and query head on scalar dequantise + FMA.
//
// Here a CTA owns (kv head, split) and serves every query head of the group from one pass over the
// rows, so the cache is read once.  The two contractions run on the tensor cores as
// mma.sync.m16n8k16 (f16 inputs, fp32 accumulate): the query heads are rows 0..7 of the 16-row tile
// (the op is bound by HBM and by instruction issue, not by tensor throughput, and a decode step has
// no 64-row tile to give a tcgen05 instruction); rows 8..15 carry the low halves of the softmax
// weights in the second product, so weights enter with 22 bits.  E4M3 converts to f16 exactly with
// one cvt per pair of codes, and the per-key scales never touch the operands:
//   score_j  = (q . Kcodes_j) * ks_j * scale            -> applied to the fp32 accumulator
//   O        = sum_j 2^(score_j + lg2 vs_j - m) Vcodes_j -> the V scale rides in the exponent
//   l        = sum_j 2^(score_j - m)                     -> m = running max of score_j + lg2 vs_j
// so the weights handed to the second mma lie in (0, 1] whatever the scales are.  q is scaled by a
// power of two per head into f16's normal range (exact), the weights by 2^10 to keep small ones out
// of the f16 subnormals; both factors are divided out again in fp32.
//
// Layout tricks that keep the key loop free of barriers and cross-lane traffic: the dot product over
// head_dim is order-free, so lane (r, c) of a warp takes a quarter of a K row (every fourth 16-byte
// chunk) and consumes it 4 bytes per k-step; the sum over keys is order-free too, so lane (r, c)
// takes keys 4c..4c+3 of a 16-key tile for the PV product and transposes their bytes into key pairs
// with four prmt per 16 bytes.  Each lane stages exactly the bytes it consumes through its own slots
// of a cp.async ring, several tiles ahead.
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include <atomic>

#include "rh_common.cuh"
#include "rh_kernels.h"

namespace rh {
namespace {

constexpr int kFdWarps = 4;
constexpr int kFdThreads = kFdWarps * 32;
constexpr int kFdTileKeys = 16;        // keys per warp iteration = one k16 step of the PV product
constexpr int kFdRows = 8;             // query heads per CTA (rows 0..7 of the m16 tile)
constexpr float kFdLog2e = 1.4426950408889634f;
constexpr float kFdMInit = -1.0e30f;   // running max before any key (finite: differences stay defined)
constexpr float kFdLgFloor = -100.0f;  // floor of lg2(v_scale): a zero scale must not give -inf - -inf
constexpr float kFdWeightShift = 10.0f;  // PV weights are 2^10 * softmax weight in f16

struct FdArgs {
    const __nv_bfloat16* q;
    const uint8_t* k;
    const uint8_t* v;
    const float* k_scale;
    const float* v_scale;
    float* partial;
    const int* cache_len;
    int num_splits;
    int num_q_heads;
    int num_kv_heads;
    int group;          // query heads per kv head
    int row_chunks;     // ceil(group / 8): CTAs per (kv head, split)
    float scale_log2e;  // softmax scale * log2(e)
};

__device__ __forceinline__ uint32_t e4m3x2_to_f16x2(uint32_t two_codes) {
    const __half2_raw h = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(two_codes), __NV_E4M3);
    return static_cast<uint32_t>(h.x) | (static_cast<uint32_t>(h.y) << 16);
}

__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
}

// D(16x8, fp32) += A(16x16, f16, row) * B(16x8, f16, col); rows 8..15 of A are zero here.
__device__ __forceinline__ void mma_rows8(float (&d)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
    const uint32_t zero = 0u;
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(zero), "r"(a2), "r"(zero), "r"(b0), "r"(b1));
}

// Same with all 16 rows of A in use: rows 8..15 carry the low halves of the weights.
__device__ __forceinline__ void mma_rows16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                           uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// w = hi + lo with hi = f16(w), lo = f16(w - hi): 22 significant bits across the two halves.
__device__ __forceinline__ void split_f16x2(float w0, float w1, uint32_t& hi, uint32_t& lo) {
    const __half2 h = __floats2half2_rn(w0, w1);
    const float2 back = __half22float2(h);
    hi = *reinterpret_cast<const uint32_t*>(&h);
    lo = pack_f16x2(w0 - back.x, w1 - back.y);
}

__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float lg2_approx(float x) {
    float y;
    asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// cp.async of kBytes (4, 8 or 16) from global to shared memory; an invalid source zero-fills.
template <int kBytes>
__device__ __forceinline__ void fd_cp_async(void* smem_dst, const void* gmem_src, bool valid) {
    const uint32_t dst = static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst));
    const int src_bytes = valid ? kBytes : 0;
    if constexpr (kBytes == 16) {
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(gmem_src), "r"(src_bytes) : "memory");
    } else {
        asm volatile("cp.async.ca.shared.global [%0], [%1], %2, %3;" ::"r"(dst), "l"(gmem_src), "n"(kBytes), "r"(src_bytes)
                     : "memory");
    }
}

// Reads one staged chunk of kBytes (4, 8 or 16) into 32-bit words.
template <int kBytes>
__device__ __forceinline__ void fd_lds(uint32_t* dst, const unsigned char* src) {
    if constexpr (kBytes == 16) {
        const uint4 t = *reinterpret_cast<const uint4*>(src);
        dst[0] = t.x; dst[1] = t.y; dst[2] = t.z; dst[3] = t.w;
    } else if constexpr (kBytes == 8) {
        const uint2 t = *reinterpret_cast<const uint2*>(src);
        dst[0] = t.x; dst[1] = t.y;
    } else {
        dst[0] = *reinterpret_cast<const uint32_t*>(src);
    }
}

// Geometry of the per-warp staging ring.  A stage holds one 16-key tile exactly as the lanes consume
// it: every lane copies (cp.async) the bytes it will itself read back, so a stage needs no barrier,
// only the lane's own wait_group.  [2 K blocks][chunks][32 lanes] + [4 V keys][chunks][32 lanes] + 32 scales.
template <int D>
struct FdRing {
    static constexpr int kKChunk = (D / 4 >= 16) ? 16 : D / 4;   // bytes per cp.async of a K quarter-row
    static constexpr int kKChunks = (D / 4) / kKChunk;
    static constexpr int kVChunk = (D / 8 >= 16) ? 16 : D / 8;   // bytes per cp.async of a V eighth-row
    static constexpr int kVChunks = (D / 8) / kVChunk;
    static constexpr int kKBytes = 2 * (D / 4) * 32;
    static constexpr int kVBytes = 4 * (D / 8) * 32;
    static constexpr int kStageBytes = kKBytes + kVBytes + 32 * 4;
    static constexpr int kStages = (D <= 128) ? 4 : 3;
    static constexpr int kRingBytes = kFdWarps * kStages * kStageBytes;
    static constexpr int kOPitch = 66;   // see the merge below
    static constexpr int kMergeBytes = kFdWarps * (D / 8) * kOPitch * 4 + 2 * kFdWarps * kFdRows * 4;
    static constexpr int kSmemBytes = kRingBytes > kMergeBytes ? kRingBytes : kMergeBytes;
};

// One 16-key tile as a warp holds it: lane (r, c) has the c-th quarter of the K rows of columns r of
// the two 8-key blocks, and 1/8 of the V rows of keys 4c..4c+3.
template <int D>
struct FdTile {
    uint32_t kw[2][D / 16];
    uint32_t vw[4][D / 32];
    float sc;   // lanes 0..15: k scale of key lane; lanes 16..31: v scale of key lane-16
};

// Partial kernel: grid (num_kv_heads * row_chunks, num_splits), 4 warps.  The 16-key tiles of the
// history are dealt evenly to the splits; warp w of a CTA folds tiles w, w+4, ... of its split into
// its own online-softmax state, with the next three tiles on their way into its staging ring while
// the current one is computed (at the reference's 32 splits and depth 8196 that is a warp's whole
// share, in flight at once).  The four states are merged through shared memory (reusing the ring)
// and written to the scratch slab as (m, l, acc[D]) per query head.
template <int D>
__global__ void __launch_bounds__(kFdThreads, (D <= 128 ? 3 : 1)) flash_decode_partial_kernel(const FdArgs p) {
    using Ring = FdRing<D>;
    constexpr int kKWords = D / 16;   // 32-bit words of a K row per lane (= k-steps of the QK product)
    constexpr int kVWords = D / 32;   // 32-bit words of a V row per lane
    constexpr int kNB = D / 8;        // 8-wide output blocks of the PV product
    static_assert(D == 32 || D == 64 || D == 128 || D == 256, "head_dim");

    extern __shared__ __align__(16) unsigned char fd_smem[];
    // After the key loop the ring is reused for the merge.  Per warp and output block: 8 rows x 8
    // columns of the accumulator tile, padded to 66 floats so that the 8-byte stores of a block and
    // the reads across blocks both spread over all banks.
    constexpr int kOPitch = Ring::kOPitch;
    float* const s_o = reinterpret_cast<float*>(fd_smem);                       // [warp][nb][kOPitch]
    float* const s_m = s_o + kFdWarps * kNB * kOPitch;                          // [warp][row]
    float* const s_l = s_m + kFdWarps * kFdRows;                                // [warp][row]

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int r = lane >> 2, c = lane & 3;
    const int kvh = blockIdx.x / p.row_chunks;
    const int chunk = blockIdx.x - kvh * p.row_chunks;
    const int split = blockIdx.y;
    const int head_in_group = chunk * kFdRows + r;
    const bool row_valid = head_in_group < p.group;
    const int qh = kvh * p.group + head_in_group;

    pdl_enter();

    // ---- key range of this split: whole tiles, dealt evenly ----
    const int n_keys = *p.cache_len + 1;
    const long long total_tiles = (static_cast<long long>(n_keys) + kFdTileKeys - 1) / kFdTileKeys;
    const int tile_lo = static_cast<int>(total_tiles * split / p.num_splits);
    const int tile_hi = static_cast<int>(total_tiles * (split + 1) / p.num_splits);
    const int n_tiles = tile_hi - tile_lo;
    const int start = tile_lo * kFdTileKeys;
    const int end = min(tile_hi * kFdTileKeys, n_keys);

    const size_t row_stride = static_cast<size_t>(p.num_kv_heads) * D;   // bytes between keys
    // Lane c takes chunk c of every group of four kKChunk-byte chunks of a K row (not one contiguous
    // quarter): the four lanes of a row then cover whole 32-byte sectors with each copy instruction.
    const uint8_t* k_lane = p.k + static_cast<size_t>(kvh) * D + c * Ring::kKChunk;
    const uint8_t* v_lane = p.v + static_cast<size_t>(kvh) * D + r * (D / 8);

    const int my_tiles = n_tiles > warp ? (n_tiles - warp + kFdWarps - 1) / kFdWarps : 0;
    unsigned char* const ring = fd_smem + static_cast<size_t>(warp) * Ring::kStages * Ring::kStageBytes;

    // issue the copies of this warp's i-th tile (or nothing) and close the group
    auto issue_tile = [&](int i) {
        if (i < my_tiles) {
            const int kb = start + (warp + i * kFdWarps) * kFdTileKeys;
            unsigned char* const st = ring + (i % Ring::kStages) * Ring::kStageBytes;
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int key = kb + 4 * (r >> 1) + 2 * j + (r & 1);   // column r of 8-key block j
                const bool live = key < end;
                const uint8_t* src = live ? k_lane + static_cast<size_t>(key) * row_stride : p.k;
#pragma unroll
                for (int ch = 0; ch < Ring::kKChunks; ++ch)
                    fd_cp_async<Ring::kKChunk>(st + ((j * Ring::kKChunks + ch) * 32 + lane) * Ring::kKChunk,
                                               src + ch * 4 * Ring::kKChunk, live);
            }
#pragma unroll
            for (int i4 = 0; i4 < 4; ++i4) {
                const int key = kb + 4 * c + i4;
                const bool live = key < end;
                const uint8_t* src = live ? v_lane + static_cast<size_t>(key) * row_stride : p.v;
#pragma unroll
                for (int ch = 0; ch < Ring::kVChunks; ++ch)
                    fd_cp_async<Ring::kVChunk>(st + Ring::kKBytes + ((i4 * Ring::kVChunks + ch) * 32 + lane) * Ring::kVChunk,
                                               src + ch * Ring::kVChunk, live);
            }
            const int key = kb + (lane & 15);
            const bool live = key < end;
            const float* src = (lane >= 16 ? p.v_scale : p.k_scale) + (live ? static_cast<size_t>(key) * p.num_kv_heads + kvh : 0);
            fd_cp_async<4>(st + Ring::kKBytes + Ring::kVBytes + lane * 4, src, live);
        }
        cp_async_commit();
    };
    // read back what this lane copied for its i-th tile
    auto read_tile = [&](FdTile<D>& tl, int i) {
        const unsigned char* const st = ring + (i % Ring::kStages) * Ring::kStageBytes;
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int ch = 0; ch < Ring::kKChunks; ++ch)
                fd_lds<Ring::kKChunk>(&tl.kw[j][ch * (Ring::kKChunk / 4)],
                                      st + ((j * Ring::kKChunks + ch) * 32 + lane) * Ring::kKChunk);
#pragma unroll
        for (int i4 = 0; i4 < 4; ++i4)
#pragma unroll
            for (int ch = 0; ch < Ring::kVChunks; ++ch)
                fd_lds<Ring::kVChunk>(&tl.vw[i4][ch * (Ring::kVChunk / 4)],
                                      st + Ring::kKBytes + ((i4 * Ring::kVChunks + ch) * 32 + lane) * Ring::kVChunk);
        tl.sc = *reinterpret_cast<const float*>(st + Ring::kKBytes + Ring::kVBytes + lane * 4);
    };

#pragma unroll
    for (int i = 0; i < Ring::kStages - 1; ++i) issue_tile(i);   // in flight while q is prepared

    // ---- q fragment: head r, the lane's quarter of the dims, scaled by a power of two into (-2, 2) ----
    uint32_t qa0[kKWords], qa2[kKWords];
    float row_factor = 0.0f;   // scale * log2e * 2^e: turns the raw accumulator into log2-domain scores
    {
        float qf[D / 4];
        if (row_valid) {
            const __nv_bfloat16* src = p.q + static_cast<size_t>(qh) * D + c * Ring::kKChunk;   // same dims as k_lane
#pragma unroll
            for (int i = 0; i < D / 4; i += 2) {
                const int dim = (i / Ring::kKChunk) * 4 * Ring::kKChunk + i % Ring::kKChunk;
                const __nv_bfloat162 two = *reinterpret_cast<const __nv_bfloat162*>(src + dim);
                qf[i] = __low2float(two);
                qf[i + 1] = __high2float(two);
            }
        } else {
#pragma unroll
            for (int i = 0; i < D / 4; ++i) qf[i] = 0.0f;
        }
        float amax = 0.0f;
#pragma unroll
        for (int i = 0; i < D / 4; ++i) amax = fmaxf(amax, fabsf(qf[i]));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
        int e = ((__float_as_int(amax) >> 23) & 0xff) - 127;   // floor(log2(amax)) for normal amax
        e = amax > 0.0f ? max(-100, min(100, e)) : 0;
        const float down = __int_as_float((127 - e) << 23);   // 2^-e
        const float up = __int_as_float((127 + e) << 23);     // 2^e
        row_factor = p.scale_log2e * up;
#pragma unroll
        for (int s = 0; s < kKWords; ++s) {
            qa0[s] = pack_f16x2(qf[4 * s] * down, qf[4 * s + 1] * down);
            qa2[s] = pack_f16x2(qf[4 * s + 2] * down, qf[4 * s + 3] * down);
        }
    }

    float o[kNB][4];
#pragma unroll
    for (int nb = 0; nb < kNB; ++nb) o[nb][0] = o[nb][1] = o[nb][2] = o[nb][3] = 0.0f;
    float m_run = kFdMInit, l_run = 0.0f;

    auto fold_tile = [&](const FdTile<D>& tl, int t) {
        const int kb = start + t * kFdTileKeys;
        // ---- S = Q K^T: two blocks of 8 keys, kKWords k-steps each ----
        // (even and odd k-steps accumulate separately: four dependent chains instead of two)
        float s0[4] = {0.0f, 0.0f, 0.0f, 0.0f}, s1[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        float s2[4] = {0.0f, 0.0f, 0.0f, 0.0f}, s3[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
        for (int s = 0; s < kKWords; s += 2) {
            mma_rows8(s0, qa0[s], qa2[s], e4m3x2_to_f16x2(tl.kw[0][s] & 0xffffu), e4m3x2_to_f16x2(tl.kw[0][s] >> 16));
            mma_rows8(s1, qa0[s], qa2[s], e4m3x2_to_f16x2(tl.kw[1][s] & 0xffffu), e4m3x2_to_f16x2(tl.kw[1][s] >> 16));
            mma_rows8(s2, qa0[s + 1], qa2[s + 1], e4m3x2_to_f16x2(tl.kw[0][s + 1] & 0xffffu), e4m3x2_to_f16x2(tl.kw[0][s + 1] >> 16));
            mma_rows8(s3, qa0[s + 1], qa2[s + 1], e4m3x2_to_f16x2(tl.kw[1][s + 1] & 0xffffu), e4m3x2_to_f16x2(tl.kw[1][s + 1] >> 16));
        }

        // ---- scores of keys kb+4c+{0,1,2,3} for head r, in the log2 domain ----
        const float lg = fmaxf(lg2_approx(tl.sc), kFdLgFloor);   // meaningful in lanes 16..31 (v scales)
        float score[4], shifted[4];
        const float raw[4] = {s0[0] + s2[0], s0[1] + s2[1], s1[0] + s3[0], s1[1] + s3[1]};
        float tile_max = -INFINITY;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float ks = __shfl_sync(0xffffffffu, tl.sc, 4 * c + i);
            const float lgv = __shfl_sync(0xffffffffu, lg, 16 + 4 * c + i);
            const bool live = kb + 4 * c + i < end;
            score[i] = live ? raw[i] * (ks * row_factor) : -INFINITY;
            shifted[i] = score[i] + lgv;
            tile_max = fmaxf(tile_max, shifted[i]);
        }
        tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, 1));
        tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, 2));
        const float m_new = fmaxf(m_run, tile_max);
        const float corr = ex2_approx(m_run - m_new);
        m_run = m_new;
        float w[4], psum = 0.0f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            w[i] = ex2_approx(shifted[i] - m_new + kFdWeightShift);
            psum += ex2_approx(score[i] - m_new);
        }
        l_run = l_run * corr + psum;
        if (__any_sync(0xffffffffu, corr != 1.0f)) {
#pragma unroll
            for (int nb = 0; nb < kNB; ++nb) {
                o[nb][0] *= corr;
                o[nb][1] *= corr;
                o[nb][2] *= corr;
                o[nb][3] *= corr;
            }
        }

        // ---- O += W V: weights of the 16 keys as the A fragment, V bytes transposed to key pairs ----
        // Rows 8..15 of the tile, idle otherwise, carry the weights' low halves: the f16 rounding of a
        // weight (2^-12) would show in the bf16 result where the sum over keys cancels.
        uint32_t wa0, wa1, wa2, wa3;
        split_f16x2(w[0], w[1], wa0, wa1);
        split_f16x2(w[2], w[3], wa2, wa3);
#pragma unroll
        for (int wc = 0; wc < kVWords; ++wc) {
            const uint32_t t01 = __byte_perm(tl.vw[0][wc], tl.vw[1][wc], 0x5140);   // k0.b0 k1.b0 k0.b1 k1.b1
            const uint32_t t23 = __byte_perm(tl.vw[2][wc], tl.vw[3][wc], 0x5140);
            const uint32_t u01 = __byte_perm(tl.vw[0][wc], tl.vw[1][wc], 0x7362);   // k0.b2 k1.b2 k0.b3 k1.b3
            const uint32_t u23 = __byte_perm(tl.vw[2][wc], tl.vw[3][wc], 0x7362);
            mma_rows16(o[4 * wc + 0], wa0, wa1, wa2, wa3, e4m3x2_to_f16x2(t01 & 0xffffu), e4m3x2_to_f16x2(t23 & 0xffffu));
            mma_rows16(o[4 * wc + 1], wa0, wa1, wa2, wa3, e4m3x2_to_f16x2(t01 >> 16), e4m3x2_to_f16x2(t23 >> 16));
            mma_rows16(o[4 * wc + 2], wa0, wa1, wa2, wa3, e4m3x2_to_f16x2(u01 & 0xffffu), e4m3x2_to_f16x2(u23 & 0xffffu));
            mma_rows16(o[4 * wc + 3], wa0, wa1, wa2, wa3, e4m3x2_to_f16x2(u01 >> 16), e4m3x2_to_f16x2(u23 >> 16));
        }
    };

    for (int i = 0; i < my_tiles; ++i) {
        issue_tile(i + Ring::kStages - 1);          // into the stage read one trip ago
        cp_async_wait<Ring::kStages - 1>();         // tile i has landed (this lane's own copies)
        FdTile<D> tl;
        read_tile(tl, i);
        fold_tile(tl, warp + i * kFdWarps);
    }
    cp_async_wait<0>();
    __syncthreads();   // every warp is done with its ring: the merge may overwrite it

    // ---- merge the four warps ----
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
    if (c == 0) {
        s_m[warp * kFdRows + r] = m_run;
        s_l[warp * kFdRows + r] = l_run;
    }
#pragma unroll
    for (int nb = 0; nb < kNB; ++nb)
        *reinterpret_cast<float2*>(&s_o[(warp * kNB + nb) * kOPitch + r * 8 + 2 * c]) =
            make_float2(o[nb][0] + o[nb][2], o[nb][1] + o[nb][3]);
    __syncthreads();

    const long long hs = static_cast<long long>(p.num_q_heads) * p.num_splits;
    const int rows_here = min(kFdRows, p.group - chunk * kFdRows);
    const float unshift = ex2_approx(-kFdWeightShift);
    for (int idx = threadIdx.x; idx < rows_here * D; idx += kFdThreads) {
        const int row = idx / D, d = idx - row * D;
        float big = s_m[row];
#pragma unroll
        for (int wv = 1; wv < kFdWarps; ++wv) big = fmaxf(big, s_m[wv * kFdRows + row]);
        const int at = (d % kNB) * kOPitch + row * 8 + d / kNB;   // column `col` of output block nb is dim col*D/8 + nb
        float a = 0.0f;
#pragma unroll
        for (int wv = 0; wv < kFdWarps; ++wv)
            a += s_o[wv * kNB * kOPitch + at] * ex2_approx(s_m[wv * kFdRows + row] - big);
        const long long slot = static_cast<long long>(kvh * p.group + chunk * kFdRows + row) * p.num_splits + split;
        p.partial[2 * hs + slot * D + d] = a * unshift;
        if (d == 0) {
            float l = 0.0f;
#pragma unroll
            for (int wv = 0; wv < kFdWarps; ++wv) l += s_l[wv * kFdRows + row] * ex2_approx(s_m[wv * kFdRows + row] - big);
            p.partial[slot] = big;
            p.partial[hs + slot] = l;
        }
    }
}

// Reduce kernel: one CTA of 256 threads per query head merges the splits' states (reference:
// src/kernels/flash_decode.cu:233-257, one thread per element walking the splits one after the
// other).  Here thread (g, j) owns four output elements j and the splits g, g+G, ...: every load of
// the CTA is in flight at once, each thread folds its splits online, and the G running states are
// merged through shared memory.  m is a log2-domain maximum.
constexpr int kFdReduceThreads = 256;

template <int D>
__global__ void __launch_bounds__(kFdReduceThreads) flash_decode_reduce_kernel(__nv_bfloat16* __restrict__ out,
                                                                              const float* __restrict__ partial,
                                                                              int num_splits, int num_q_heads) {
    constexpr int kVecs = D / 4;                      // float4 columns of a row
    constexpr int kGroups = kFdReduceThreads / kVecs;  // splits walked in parallel
    __shared__ float4 s_acc[kGroups][kVecs];
    __shared__ float s_m[kGroups], s_l[kGroups];

    const int qh = blockIdx.x;
    const int j = threadIdx.x % kVecs, g = threadIdx.x / kVecs;
    const long long hs = static_cast<long long>(num_q_heads) * num_splits;
    const float* m_row = partial + static_cast<long long>(qh) * num_splits;
    const float* l_row = m_row + hs;
    const float4* acc_row = reinterpret_cast<const float4*>(partial + 2 * hs + static_cast<long long>(qh) * num_splits * D);
    pdl_enter();

    float m = kFdMInit, l = 0.0f;
    float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll 4
    for (int i = g; i < num_splits; i += kGroups) {
        const float mi = m_row[i], li = l_row[i];
        const float4 a = acc_row[static_cast<size_t>(i) * kVecs + j];
        const float m_new = fmaxf(m, mi);
        const float c_old = ex2_approx(m - m_new), c_new = ex2_approx(mi - m_new);
        l = l * c_old + li * c_new;
        acc.x = acc.x * c_old + a.x * c_new;
        acc.y = acc.y * c_old + a.y * c_new;
        acc.z = acc.z * c_old + a.z * c_new;
        acc.w = acc.w * c_old + a.w * c_new;
        m = m_new;
    }
    s_acc[g][j] = acc;
    if (j == 0) {
        s_m[g] = m;
        s_l[g] = l;
    }
    __syncthreads();
    if (g == 0) {
        float big = s_m[0];
#pragma unroll
        for (int i = 1; i < kGroups; ++i) big = fmaxf(big, s_m[i]);
        float l_all = 0.0f;
        float4 sum = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
        for (int i = 0; i < kGroups; ++i) {
            const float w = ex2_approx(s_m[i] - big);
            const float4 a = s_acc[i][j];
            l_all += s_l[i] * w;
            sum.x += a.x * w;
            sum.y += a.y * w;
            sum.z += a.z * w;
            sum.w += a.w * w;
        }
        const float inv = 1.0f / l_all;
        __nv_bfloat162 lo = __floats2bfloat162_rn(sum.x * inv, sum.y * inv);
        __nv_bfloat162 hi = __floats2bfloat162_rn(sum.z * inv, sum.w * inv);
        uint2 packed;
        packed.x = *reinterpret_cast<const uint32_t*>(&lo);
        packed.y = *reinterpret_cast<const uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(out + static_cast<size_t>(qh) * D + 4 * j) = packed;
    }
}

template <int D>
void launch_partial(const FdArgs& a, cudaStream_t stream) {
    const dim3 grid(static_cast<unsigned>(a.num_kv_heads * a.row_chunks), static_cast<unsigned>(a.num_splits));
    constexpr int smem = FdRing<D>::kSmemBytes;
    if constexpr (smem > 48 * 1024) {   // opt in once per device; the attribute is per device and idempotent
        static std::atomic<unsigned> configured{0};
        int dev = 0;
        cudaGetDevice(&dev);
        const unsigned bit = 1u << (dev & 31);
        if ((configured.load(std::memory_order_relaxed) & bit) == 0) {
            cudaFuncSetAttribute(reinterpret_cast<const void*>(&flash_decode_partial_kernel<D>),
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
            configured.fetch_or(bit, std::memory_order_relaxed);
        }
    }
    host::launch(flash_decode_partial_kernel<D>, grid, dim3(kFdThreads), static_cast<size_t>(smem), stream, a);
}

}  // namespace
}  // namespace rh

using namespace rh;

extern "C" size_t rh_flash_split_scratch_floats(int num_q_heads, int head_dim, int max_splits) {
    if (num_q_heads < 1 || head_dim < 1 || max_splits < 1) return 0;
    const size_t slots = static_cast<size_t>(num_q_heads) * static_cast<size_t>(max_splits);
    return slots * 2 + slots * static_cast<size_t>(head_dim);
}

extern "C" int rh_flash_decode_split_bf16(void* out, const void* q, const uint8_t* k, const uint8_t* v,
                                          const float* k_scale, const float* v_scale, float* partial,
                                          int num_splits, const int* cache_len, int num_q_heads,
                                          int num_kv_heads, int head_dim, float scale, void* stream) {
    const char* const fn = "rh_flash_decode_split_bf16";
    RH_REQUIRE(out && q && k && v && k_scale && v_scale && partial, RH_ERR_INVALID_ARG, "%s: null pointer", fn);
    RH_REQUIRE(cache_len != nullptr, RH_ERR_INVALID_ARG, "%s: cache_len must not be null", fn);
    RH_REQUIRE(num_splits >= 1 && num_splits <= 65535, RH_ERR_INVALID_ARG, "%s: num_splits must be in 1..65535", fn);
    RH_REQUIRE(num_q_heads >= 1, RH_ERR_INVALID_ARG, "%s: num_q_heads must be >= 1", fn);
    RH_REQUIRE(num_kv_heads >= 1, RH_ERR_INVALID_ARG, "%s: num_kv_heads must be >= 1", fn);
    RH_REQUIRE(num_q_heads % num_kv_heads == 0, RH_ERR_INVALID_ARG,
               "%s: num_q_heads must be divisible by num_kv_heads", fn);
    RH_REQUIRE(head_dim == 32 || head_dim == 64 || head_dim == 128 || head_dim == 256, RH_ERR_UNSUPPORTED_DIM,
               "%s: head_dim must be one of 32, 64, 128, 256", fn);
    RH_REQUIRE(host::aligned16(q) && host::aligned16(k) && host::aligned16(v) && host::aligned16(partial),
               RH_ERR_MISALIGNED, "%s: q, k, v and partial must be 16-byte aligned", fn);
    RH_REQUIRE((reinterpret_cast<uintptr_t>(out) & 7u) == 0, RH_ERR_MISALIGNED, "%s: out must be 8-byte aligned", fn);

    FdArgs a;
    a.q = static_cast<const __nv_bfloat16*>(q);
    a.k = k;
    a.v = v;
    a.k_scale = k_scale;
    a.v_scale = v_scale;
    a.partial = partial;
    a.cache_len = cache_len;
    a.num_splits = num_splits;
    a.num_q_heads = num_q_heads;
    a.num_kv_heads = num_kv_heads;
    a.group = num_q_heads / num_kv_heads;
    a.row_chunks = (a.group + kFdRows - 1) / kFdRows;
    a.scale_log2e = scale * kFdLog2e;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (head_dim) {
        case 32: launch_partial<32>(a, s); break;
        case 64: launch_partial<64>(a, s); break;
        case 128: launch_partial<128>(a, s); break;
        default: launch_partial<256>(a, s); break;
    }
    if (const int st = host::check_launch(fn)) return st;
    const dim3 rgrid(static_cast<unsigned>(num_q_heads)), rblock(kFdReduceThreads);
    __nv_bfloat16* o = static_cast<__nv_bfloat16*>(out);
    const float* part = partial;
    switch (head_dim) {
        case 32: host::launch(flash_decode_reduce_kernel<32>, rgrid, rblock, 0, s, o, part, num_splits, num_q_heads); break;
        case 64: host::launch(flash_decode_reduce_kernel<64>, rgrid, rblock, 0, s, o, part, num_splits, num_q_heads); break;
        case 128: host::launch(flash_decode_reduce_kernel<128>, rgrid, rblock, 0, s, o, part, num_splits, num_q_heads); break;
        default: host::launch(flash_decode_reduce_kernel<256>, rgrid, rblock, 0, s, o, part, num_splits, num_q_heads); break;
    }
    return host::check_launch(fn);
}
