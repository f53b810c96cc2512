// Split-KV flash decode over the FP8-E4M3 KV cache: one query token, all query heads, keys
// 0 .. *cache_len, K/V dequantised by their per-(token, kv head) scales.
// Replaces runtherder::kernels::flash_decode_split_bf16
// (include/runtherder/kernels/flash_decode.cuh:27-62, src/kernels/flash_decode.cu:119-325), which
// runs one 128-thread CTA per (query head, split), re-reads a kv head's rows once per query head of
// its group and spends ~30 warp instructions per key and query head on scalar dequantise + FMA.
//
// Here a CTA owns (kv head, split) and serves every query head of the group from one pass over the
// rows, so the cache is read once.  Both contractions run on the tensor cores as mma.sync.m16n8k16
// (f16 inputs, fp32 accumulate) in the form that fills the 16-row operand with cache data and puts
// the few query heads on the 8-wide side — the op is bound by HBM and by instruction issue, and a
// decode step has no 64-row tile to give a tcgen05 instruction:
//   S^T[16 keys x 8 cols]  = K[16 keys x 16 dims]    . q^T[16 dims x 8 cols]   per k-step
//   O^T[16 dims x 8 cols] += V^T[16 dims x 16 keys]  . W^T[16 keys x 8 cols]   per 16-dim block
// E4M3 converts to f16 exactly, two codes per cvt, and the per-key scales never touch the operands:
//   score_j  = (q . Kcodes_j) * ks_j * scale             -> applied to the fp32 accumulator
//   O        = sum_j 2^(score_j + lg2 vs_j - m) Vcodes_j  -> the V scale rides in the exponent
//   l        = sum_j 2^(score_j - m)                      -> m = running max of score_j + lg2 vs_j
// so the weights handed to the second mma lie in (0, 1] whatever the scales are.  q is scaled by a
// power of two per head into f16's normal range (exact), the weights by 2^10 to keep small ones out
// of the f16 subnormals; both factors are divided out again in fp32.  A weight enters as hi + lo
// (two f16, 22 bits): with at most four query heads per kv head the lo halves ride in the four idle
// columns of the same mma, wider groups issue a second one.
//
// Layout tricks that keep the key loop free of barriers: the dot product over head_dim is
// order-free, so lane (r, c) of a warp takes a quarter of the K rows of keys r and r+8 of a tile
// (every fourth 16-byte chunk) and consumes it 4 bytes per k-step; the sum over keys is order-free
// too, so lane (r, c) takes keys 4c..4c+3 for the second product and transposes their bytes into key
// pairs with four prmt per 16 bytes; the weights change from "row = key" to "row = column" with one
// movmatrix per 8 keys.  A warp stages its tiles through its own cp.async ring, several tiles ahead:
// V bytes and scales by the lane that consumes them, K rows as whole rows (full 128-byte lines per
// request) read back across lanes after a __syncwarp — no CTA barrier in the key loop.
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include <atomic>

#include "rh_common.cuh"
#include "rh_kernels.h"

namespace rh {
namespace {

constexpr int kFdWarps = 4;
constexpr int kFdThreads = kFdWarps * 32;
constexpr int kFdSubKeys = 16;         // one k16 step of the second product
constexpr int kFdSubs = 1;              // sub-tiles folded together per trip (2 = two independent instruction
                                        // streams per warp: measured no faster, 20 more registers)
constexpr int kFdTileKeys = kFdSubs * kFdSubKeys;   // keys per warp iteration
constexpr int kFdCols = 8;             // the 8-wide side of both products
constexpr float kFdLog2e = 1.4426950408889634f;
constexpr float kFdMInit = -1.0e30f;   // running max before any key (finite: differences stay defined)
constexpr float kFdLgFloor = -100.0f;  // floor of lg2(v_scale): a zero scale must not give -inf - -inf
constexpr float kFdWeightShift = 10.0f;  // weights enter the second product as 2^10 * softmax weight

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
    int heads_per_cta;  // 4 (hi and lo halves of the weights share one mma) or 8
    int row_chunks;     // ceil(group / heads_per_cta): CTAs per (kv head, split)
    float scale_log2e;  // softmax scale * log2(e)
};

// Four E4M3 codes of a 32-bit word -> two f16x2 (codes 0,1 and codes 2,3).
__device__ __forceinline__ void e4m3x4_to_f16x2x2(uint32_t word, uint32_t& lo, uint32_t& hi) {
    asm("{\n\t.reg .b16 l, h;\n\tmov.b32 {l, h}, %2;\n\tcvt.rn.f16x2.e4m3x2 %0, l;\n\tcvt.rn.f16x2.e4m3x2 %1, h;\n\t}"
        : "=r"(lo), "=r"(hi)
        : "r"(word));
}

__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
}

// D(16x8, fp32) += A(16x16, f16, row) * B(16x8, f16, col)
__device__ __forceinline__ void mma_16x8x16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                            uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// 8x8 transpose of 16-bit elements across the warp: lane (r, c) gives elements (r, 2c), (r, 2c+1)
// and receives (2c, r), (2c+1, r).
__device__ __forceinline__ uint32_t transpose_8x8_b16(uint32_t x) {
    uint32_t y;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(y) : "r"(x));
    return y;
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

// cp.async of kBytes (4, 8 or 16) from global to shared memory.
template <int kBytes>
__device__ __forceinline__ void fd_cp_async(void* smem_dst, const void* gmem_src) {
    const uint32_t dst = static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst));
    if constexpr (kBytes == 16) {
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(gmem_src) : "memory");
    } else {
        asm volatile("cp.async.ca.shared.global [%0], [%1], %2;" ::"r"(dst), "l"(gmem_src), "n"(kBytes) : "memory");
    }
}
// The same with a validity flag: an invalid source is not read and the destination is zero-filled.
template <int kBytes>
__device__ __forceinline__ void fd_cp_async_zfill(void* smem_dst, const void* gmem_src, bool valid) {
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

// Geometry of the per-warp staging ring.  A stage holds one 16-key tile: the 16 K rows (row-major,
// odd rows rotated by four chunks; for head_dim 32 per consuming lane instead), the V bytes as
// [4 keys][chunks][32 lanes] and 32 scales, each V byte and scale copied by the lane that reads it
// back, so a stage needs the lane's own wait_group and a __syncwarp for the K rows.
template <int D>
struct FdRing {
    static constexpr int kKChunk = (D / 4 >= 16) ? 16 : D / 4;   // bytes per cp.async of a K quarter-row
    static constexpr int kKChunks = (D / 4) / kKChunk;
    static constexpr int kVChunk = (D / 8 >= 16) ? 16 : D / 8;   // bytes per cp.async of a V eighth-row
    static constexpr int kVChunks = (D / 8) / kVChunk;
    static constexpr int kKBytes = 2 * (D / 4) * 32;
    static constexpr int kVBytes = 4 * (D / 8) * 32;
    static constexpr int kSubBytes = kKBytes + kVBytes + 32 * 4;   // one 16-key sub-tile
    static constexpr int kStageBytes = kFdSubs * kSubBytes;
    static constexpr int kStages = 4;
    static constexpr int kRingBytes = kFdWarps * kStages * kStageBytes;
    // merge buffers: per warp the accumulators as the lanes hold them, then m and l per column
    static constexpr int kMergeBytes = kFdWarps * (D / 16) * 32 * 16 + 2 * kFdWarps * kFdCols * 4;
    static constexpr int kSmemBytes = kRingBytes > kMergeBytes ? kRingBytes : kMergeBytes;
};

// One 16-key tile as a warp holds it: lane (r, c) has its quarter of the K rows of (tile-local) keys
// ka = 4*(r/2) + r%2 and kb = ka + 2, and its eighth of the V rows of keys 4c..4c+3.
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
// kWide: more than four query heads per CTA — the eight columns are eight heads and the weights'
// low halves take a second mma; otherwise columns 4..7 repeat heads 0..3 and carry the low halves.
template <int D, bool kWide>
__global__ void __launch_bounds__(kFdThreads, (D <= 128 ? 2 : 1)) flash_decode_partial_kernel(const FdArgs p) {
    using Ring = FdRing<D>;
    constexpr int kKWords = D / 16;   // 32-bit words of a K row per lane (= k-steps of the first product)
    constexpr int kVWords = D / 32;   // 32-bit words of a V row per lane
    constexpr int kMB = D / 16;       // 16-dim blocks of the second product
    constexpr int kHeads = kWide ? 8 : 4;
    static_assert(D == 32 || D == 64 || D == 128 || D == 256, "head_dim");

    extern __shared__ __align__(16) unsigned char fd_smem[];

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int r = lane >> 2, c = lane & 3;
    const int kvh = blockIdx.x / p.row_chunks;
    const int chunk = blockIdx.x - kvh * p.row_chunks;
    const int split = blockIdx.y;
    const int head_in_group = chunk * kHeads + (kWide ? r : (r & 3));   // the head of column r
    const bool col_valid = head_in_group < p.group;
    const int qh = kvh * p.group + head_in_group;

    pdl_enter();

    // ---- q first: its loads do not depend on the history length and are in flight while the key range is
    //      worked out and the first tiles are requested.  The lane's dims are those of k_lane below: runs of
    //      kKChunk dims, 4 kKChunk apart. ----
    constexpr int kQVecs = D / 32;                        // 16-byte pieces of q per lane
    constexpr int kQVecsPerRun = Ring::kKChunk / 8;
    uint4 qraw[kQVecs];
    {
        const __nv_bfloat16* const src = p.q + static_cast<size_t>(col_valid ? qh : 0) * D + c * Ring::kKChunk;
#pragma unroll
        for (int v = 0; v < kQVecs; ++v) {
            qraw[v] = make_uint4(0u, 0u, 0u, 0u);
            if (col_valid) qraw[v] = *reinterpret_cast<const uint4*>(src + (v / kQVecsPerRun) * 4 * Ring::kKChunk + (v % kQVecsPerRun) * 8);
        }
    }

    // ---- key range of this split: whole tiles, dealt evenly ----
    const int n_keys = *p.cache_len + 1;
    const long long total_tiles = (static_cast<long long>(n_keys) + kFdTileKeys - 1) / kFdTileKeys;
    int tile_lo, tile_hi;
    if (total_tiles * (p.num_splits + 1) < (1LL << 31)) {            // the usual case: 32-bit divisions
        const unsigned tt = static_cast<unsigned>(total_tiles), ns = static_cast<unsigned>(p.num_splits);
        tile_lo = static_cast<int>(tt * static_cast<unsigned>(split) / ns);
        tile_hi = static_cast<int>(tt * static_cast<unsigned>(split + 1) / ns);
    } else {
        tile_lo = static_cast<int>(total_tiles * split / p.num_splits);
        tile_hi = static_cast<int>(total_tiles * (split + 1) / p.num_splits);
    }
    const int n_tiles = tile_hi - tile_lo;
    const int start = tile_lo * kFdTileKeys;
    const int end = min(tile_hi * kFdTileKeys, n_keys);

    const size_t row_stride = static_cast<size_t>(p.num_kv_heads) * D;   // bytes between keys
    const int key_a = 4 * (r >> 1) + (r & 1);                            // tile-local key of row r (row r+8: +2)
    // Lane c takes chunk c of every group of four kKChunk-byte chunks of a K row (not one contiguous
    // quarter): the four lanes of a row then cover whole 32-byte sectors with each copy instruction.
    const uint8_t* const k_lane = p.k + static_cast<size_t>(kvh) * D + c * Ring::kKChunk + key_a * row_stride;
    const uint8_t* const k_lane_b = k_lane + 2 * row_stride;   // row r+8 of the tile
    const uint8_t* const v_lane = p.v + static_cast<size_t>(kvh) * D + r * (D / 8) + (4 * c) * row_stride;
    const uint8_t* const v_lane1 = v_lane + row_stride;
    const uint8_t* const v_lane2 = v_lane1 + row_stride;
    const uint8_t* const v_lane3 = v_lane2 + row_stride;
    const float* const s_lane = (lane >= 16 ? p.v_scale : p.k_scale) + static_cast<size_t>(lane & 15) * p.num_kv_heads + kvh;

    // K rows are staged as whole rows (a request covers full 128-byte lines: 8 lanes per row) and read back
    // across lanes; odd rows keep their chunks rotated by four so the reads stay conflict-free.
    constexpr bool kRowCopies = Ring::kKChunk == 16;
    constexpr int kCPR = D / 16;                     // 16-byte chunks per K row
    constexpr int kKCopies = kRowCopies ? 16 * kCPR / 32 : 0;
    const int row_l = lane / (kCPR < 32 ? kCPR : 32), chunk_l = lane % (kCPR < 32 ? kCPR : 32);
    auto k_swz = [](int row) { return kCPR >= 8 ? ((row & 1) << 2) : 0; };
    const uint8_t* const k_row_lane = p.k + static_cast<size_t>(kvh) * D + chunk_l * 16 + row_l * row_stride;
    const int my_tiles = n_tiles > warp ? (n_tiles - warp + kFdWarps - 1) / kFdWarps : 0;
    unsigned char* const ring = fd_smem + static_cast<size_t>(warp) * Ring::kStages * Ring::kStageBytes;

    // issue the copies of this warp's i-th tile (or nothing) and close the group
    auto issue_tile = [&](int i) {
        if (i < my_tiles) {
#pragma unroll
            for (int u = 0; u < kFdSubs; ++u) {
                const int kb = start + (warp + i * kFdWarps) * kFdTileKeys + u * kFdSubKeys;
                unsigned char* const st = ring + (i % Ring::kStages) * Ring::kStageBytes + u * Ring::kSubBytes;
                const size_t off = static_cast<size_t>(kb) * row_stride;
                const float* const s_src = s_lane + static_cast<size_t>(kb) * p.num_kv_heads;
                if (kb + kFdSubKeys <= end) {   // every sub-tile but the last of the history
                    if constexpr (kRowCopies) {   // whole 128-byte lines per request: 32 / kCPR rows per instruction
#pragma unroll
                        for (int i2 = 0; i2 < kKCopies; ++i2) {
                            const int row = i2 * (32 / kCPR) + row_l;
                            fd_cp_async<16>(st + row * D + ((chunk_l ^ k_swz(row)) << 4), k_row_lane + off + i2 * (32 / kCPR) * row_stride);
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 2; ++j)
#pragma unroll
                            for (int ch = 0; ch < Ring::kKChunks; ++ch)
                                fd_cp_async<Ring::kKChunk>(st + ((j * Ring::kKChunks + ch) * 32 + lane) * Ring::kKChunk,
                                                           (j == 0 ? k_lane : k_lane_b) + off + ch * 4 * Ring::kKChunk);
                    }
#pragma unroll
                    for (int i4 = 0; i4 < 4; ++i4)
#pragma unroll
                        for (int ch = 0; ch < Ring::kVChunks; ++ch)
                            fd_cp_async<Ring::kVChunk>(st + Ring::kKBytes + ((i4 * Ring::kVChunks + ch) * 32 + lane) * Ring::kVChunk,
                                                       (i4 == 0 ? v_lane : i4 == 1 ? v_lane1 : i4 == 2 ? v_lane2 : v_lane3) + off + ch * Ring::kVChunk);
                    fd_cp_async<4>(st + Ring::kKBytes + Ring::kVBytes + lane * 4, s_src);
                } else {
                    if constexpr (kRowCopies) {
#pragma unroll
                        for (int i2 = 0; i2 < kKCopies; ++i2) {
                            const int row = i2 * (32 / kCPR) + row_l;
                            const bool live = kb + row < end;
                            fd_cp_async_zfill<16>(st + row * D + ((chunk_l ^ k_swz(row)) << 4),
                                                  live ? k_row_lane + off + i2 * (32 / kCPR) * row_stride : p.k, live);
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 2; ++j) {
                            const bool live = kb + key_a + 2 * j < end;
#pragma unroll
                            for (int ch = 0; ch < Ring::kKChunks; ++ch)
                                fd_cp_async_zfill<Ring::kKChunk>(st + ((j * Ring::kKChunks + ch) * 32 + lane) * Ring::kKChunk,
                                                                 live ? k_lane + off + (2 * j) * row_stride + ch * 4 * Ring::kKChunk : p.k, live);
                        }
                    }
#pragma unroll
                    for (int i4 = 0; i4 < 4; ++i4) {
                        const bool live = kb + 4 * c + i4 < end;
#pragma unroll
                        for (int ch = 0; ch < Ring::kVChunks; ++ch)
                            fd_cp_async_zfill<Ring::kVChunk>(st + Ring::kKBytes + ((i4 * Ring::kVChunks + ch) * 32 + lane) * Ring::kVChunk,
                                                             live ? v_lane + off + i4 * row_stride + ch * Ring::kVChunk : p.v, live);
                    }
                    const bool live = kb + (lane & 15) < end;
                    fd_cp_async_zfill<4>(st + Ring::kKBytes + Ring::kVBytes + lane * 4, live ? s_src : p.k_scale, live);
                }
            }
        }
        cp_async_commit();
    };
    // read back what this lane copied for sub-tile u of its i-th tile
    auto read_tile = [&](FdTile<D>& tl, int i, int u) {
        const unsigned char* const st = ring + (i % Ring::kStages) * Ring::kStageBytes + u * Ring::kSubBytes;
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int ch = 0; ch < Ring::kKChunks; ++ch) {
                if constexpr (kRowCopies) {   // row key_a + 2j, chunk 4*ch + c of it (copied by other lanes)
                    const int row = key_a + 2 * j;
                    fd_lds<16>(&tl.kw[j][ch * 4], st + row * D + (((4 * ch + c) ^ k_swz(row)) << 4));
                } else {
                    fd_lds<Ring::kKChunk>(&tl.kw[j][ch * (Ring::kKChunk / 4)],
                                          st + ((j * Ring::kKChunks + ch) * 32 + lane) * Ring::kKChunk);
                }
            }
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

    // ---- q as the B operand: column r, the lane's quarter of the dims, scaled by a power of two
    //      into (-2, 2); word s holds the four dims of k-step s ----
    uint32_t qb0[kKWords], qb1[kKWords];
    float factor0, factor1;   // scale * log2e * 2^e of the heads of columns 2c and 2c+1
    {
        float qf[D / 4];     // the lane's dims in order: element i sits in word i / 2 of the pieces loaded above
#pragma unroll
        for (int v = 0; v < kQVecs; ++v) {
            const uint32_t w[4] = {qraw[v].x, qraw[v].y, qraw[v].z, qraw[v].w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                qf[8 * v + 2 * e] = bf_lo(w[e]);
                qf[8 * v + 2 * e + 1] = bf_hi(w[e]);
            }
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
        const float factor = p.scale_log2e * up;               // of column r
        factor0 = __shfl_sync(0xffffffffu, factor, 4 * (2 * c));
        factor1 = __shfl_sync(0xffffffffu, factor, 4 * (2 * c + 1));
#pragma unroll
        for (int s = 0; s < kKWords; ++s) {
            qb0[s] = pack_f16x2(qf[4 * s] * down, qf[4 * s + 1] * down);
            qb1[s] = pack_f16x2(qf[4 * s + 2] * down, qf[4 * s + 3] * down);
        }
    }

    // accumulator of block mb: [dim 16r+2mb][col 2c], [same][col 2c+1], [dim 16r+2mb+1][col 2c], [same][col 2c+1]
    float o[kMB][4];
#pragma unroll
    for (int mb = 0; mb < kMB; ++mb) o[mb][0] = o[mb][1] = o[mb][2] = o[mb][3] = 0.0f;
    float m0 = kFdMInit, m1 = kFdMInit, l0 = 0.0f, l1 = 0.0f;   // columns 2c and 2c+1

    auto fold_tile = [&](const FdTile<D> (&tl)[kFdSubs], int t) {
        // ---- S^T = K q^T per sub-tile: rows = keys (r -> key_a, r+8 -> key_a+2), columns = heads ----
        float score[kFdSubs][4], shifted[kFdSubs][4];   // [key a, col 0], [key a, col 1], [key b, col 0], [key b, col 1]
        float t0 = -INFINITY, t1 = -INFINITY;
#pragma unroll
        for (int u = 0; u < kFdSubs; ++u) {
            const int kb = start + t * kFdTileKeys + u * kFdSubKeys;
            float sa[4] = {0.0f, 0.0f, 0.0f, 0.0f}, sb[4] = {0.0f, 0.0f, 0.0f, 0.0f};   // two chains
#pragma unroll
            for (int s = 0; s < kKWords; s += 2) {
                uint32_t a0, a1, a2, a3;
                e4m3x4_to_f16x2x2(tl[u].kw[0][s], a0, a2);
                e4m3x4_to_f16x2x2(tl[u].kw[1][s], a1, a3);
                mma_16x8x16(sa, a0, a1, a2, a3, qb0[s], qb1[s]);
                e4m3x4_to_f16x2x2(tl[u].kw[0][s + 1], a0, a2);
                e4m3x4_to_f16x2x2(tl[u].kw[1][s + 1], a1, a3);
                mma_16x8x16(sb, a0, a1, a2, a3, qb0[s + 1], qb1[s + 1]);
            }
            // scores in the log2 domain
            const float lg = fmaxf(lg2_approx(tl[u].sc), kFdLgFloor);   // meaningful in lanes 16..31 (v scales)
            const float ks_a = __shfl_sync(0xffffffffu, tl[u].sc, key_a), ks_b = __shfl_sync(0xffffffffu, tl[u].sc, key_a + 2);
            const float lg_a = __shfl_sync(0xffffffffu, lg, 16 + key_a), lg_b = __shfl_sync(0xffffffffu, lg, 18 + key_a);
            const bool live_a = kb + key_a < end, live_b = kb + key_a + 2 < end;
            score[u][0] = live_a ? (sa[0] + sb[0]) * (ks_a * factor0) : -INFINITY;
            score[u][1] = live_a ? (sa[1] + sb[1]) * (ks_a * factor1) : -INFINITY;
            score[u][2] = live_b ? (sa[2] + sb[2]) * (ks_b * factor0) : -INFINITY;
            score[u][3] = live_b ? (sa[3] + sb[3]) * (ks_b * factor1) : -INFINITY;
            shifted[u][0] = score[u][0] + lg_a;
            shifted[u][1] = score[u][1] + lg_a;
            shifted[u][2] = score[u][2] + lg_b;
            shifted[u][3] = score[u][3] + lg_b;
            t0 = fmaxf(t0, fmaxf(shifted[u][0], shifted[u][2]));
            t1 = fmaxf(t1, fmaxf(shifted[u][1], shifted[u][3]));
        }
#pragma unroll
        for (int off = 4; off < 32; off <<= 1) {   // over the 8 key rows
            t0 = fmaxf(t0, __shfl_xor_sync(0xffffffffu, t0, off));
            t1 = fmaxf(t1, __shfl_xor_sync(0xffffffffu, t1, off));
        }
        const float n0 = fmaxf(m0, t0), n1 = fmaxf(m1, t1);
        const float corr0 = ex2_approx(m0 - n0), corr1 = ex2_approx(m1 - n1);
        m0 = n0;
        m1 = n1;
        if (__any_sync(0xffffffffu, corr0 != 1.0f || corr1 != 1.0f)) {
#pragma unroll
            for (int mb = 0; mb < kMB; ++mb) {
                o[mb][0] *= corr0;
                o[mb][1] *= corr1;
                o[mb][2] *= corr0;
                o[mb][3] *= corr1;
            }
        }
        const float ns0 = n0 - kFdWeightShift, ns1 = n1 - kFdWeightShift;
        float p0 = 0.0f, p1 = 0.0f;
#pragma unroll
        for (int u = 0; u < kFdSubs; ++u) {
            const float w0 = ex2_approx(shifted[u][0] - ns0), w1 = ex2_approx(shifted[u][1] - ns1);
            const float w2 = ex2_approx(shifted[u][2] - ns0), w3 = ex2_approx(shifted[u][3] - ns1);
            p0 += ex2_approx(score[u][0] - n0) + ex2_approx(score[u][2] - n0);
            p1 += ex2_approx(score[u][1] - n1) + ex2_approx(score[u][3] - n1);

            // ---- weights as the B operand: [key][col] -> [col][key pairs] by an 8x8 transpose per 8 keys.
            //      The f16 rounding of a weight (2^-12) would show in the bf16 result where the sum over
            //      keys cancels, so the low halves go in as well. ----
            uint32_t hi_a, lo_a, hi_b, lo_b;
            split_f16x2(w0, w1, hi_a, lo_a);   // key a, columns 2c, 2c+1
            split_f16x2(w2, w3, hi_b, lo_b);   // key b
            uint32_t b0, b1;
            [[maybe_unused]] uint32_t b0_lo = 0u, b1_lo = 0u;
            if constexpr (kWide) {
                b0 = transpose_8x8_b16(hi_a);
                b1 = transpose_8x8_b16(hi_b);
                b0_lo = transpose_8x8_b16(lo_a);
                b1_lo = transpose_8x8_b16(lo_b);
            } else {   // columns 4..7 (lanes c >= 2) repeat heads 0..3: they carry the low halves
                b0 = transpose_8x8_b16(c >= 2 ? lo_a : hi_a);
                b1 = transpose_8x8_b16(c >= 2 ? lo_b : hi_b);
            }

            // ---- O^T += V^T W^T: V bytes of keys 4c..4c+3 transposed into key pairs ----
#pragma unroll
            for (int wc = 0; wc < kVWords; ++wc) {
                const uint32_t t01 = __byte_perm(tl[u].vw[0][wc], tl[u].vw[1][wc], 0x5140);   // k0.b0 k1.b0 k0.b1 k1.b1
                const uint32_t t23 = __byte_perm(tl[u].vw[2][wc], tl[u].vw[3][wc], 0x5140);
                const uint32_t u01 = __byte_perm(tl[u].vw[0][wc], tl[u].vw[1][wc], 0x7362);   // k0.b2 k1.b2 k0.b3 k1.b3
                const uint32_t u23 = __byte_perm(tl[u].vw[2][wc], tl[u].vw[3][wc], 0x7362);
                uint32_t a0, a1, a2, a3;
                e4m3x4_to_f16x2x2(t01, a0, a1);   // dim 4wc (rows r) and dim 4wc+1 (rows r+8), keys 4c, 4c+1
                e4m3x4_to_f16x2x2(t23, a2, a3);   // the same dims, keys 4c+2, 4c+3
                mma_16x8x16(o[2 * wc], a0, a1, a2, a3, b0, b1);
                if constexpr (kWide) mma_16x8x16(o[2 * wc], a0, a1, a2, a3, b0_lo, b1_lo);
                e4m3x4_to_f16x2x2(u01, a0, a1);   // dims 4wc+2, 4wc+3
                e4m3x4_to_f16x2x2(u23, a2, a3);
                mma_16x8x16(o[2 * wc + 1], a0, a1, a2, a3, b0, b1);
                if constexpr (kWide) mma_16x8x16(o[2 * wc + 1], a0, a1, a2, a3, b0_lo, b1_lo);
            }
        }
        l0 = l0 * corr0 + p0;
        l1 = l1 * corr1 + p1;
    };

    for (int i = 0; i < my_tiles; ++i) {
        if constexpr (kRowCopies) __syncwarp();     // every lane has read the stage that is refilled next
        issue_tile(i + Ring::kStages - 1);          // into the stage read one trip ago
        cp_async_wait<Ring::kStages - 1>();         // this lane's copies of tile i have landed
        if constexpr (kRowCopies) __syncwarp();     // ... and the other lanes' K rows
        FdTile<D> tl[kFdSubs];
#pragma unroll
        for (int u = 0; u < kFdSubs; ++u) read_tile(tl[u], i, u);
        fold_tile(tl, warp + i * kFdWarps);
    }
    cp_async_wait<0>();
    __syncthreads();   // every warp is done with its ring: the merge may overwrite it

    // ---- merge the warps: accumulators as the lanes hold them, m and l per column ----
    float4* const s_o = reinterpret_cast<float4*>(fd_smem);                          // [warp][mb][lane]
    float* const s_m = reinterpret_cast<float*>(s_o + kFdWarps * kMB * 32);          // [warp][col]
    float* const s_l = s_m + kFdWarps * kFdCols;                                     // [warp][col]
#pragma unroll
    for (int off = 4; off < 32; off <<= 1) {
        l0 += __shfl_xor_sync(0xffffffffu, l0, off);
        l1 += __shfl_xor_sync(0xffffffffu, l1, off);
    }
    if (r == 0) {
        s_m[warp * kFdCols + 2 * c] = m0;
        s_m[warp * kFdCols + 2 * c + 1] = m1;
        s_l[warp * kFdCols + 2 * c] = l0;
        s_l[warp * kFdCols + 2 * c + 1] = l1;
    }
#pragma unroll
    for (int mb = 0; mb < kMB; ++mb) s_o[(warp * kMB + mb) * 32 + lane] = make_float4(o[mb][0], o[mb][1], o[mb][2], o[mb][3]);
    __syncthreads();

    const long long hs = static_cast<long long>(p.num_q_heads) * p.num_splits;
    const int heads_here = min(kHeads, p.group - chunk * kHeads);
    const float unshift = ex2_approx(-kFdWeightShift);
    const float* const s_of = reinterpret_cast<const float*>(s_o);
    for (int idx = threadIdx.x; idx < heads_here * D; idx += kFdThreads) {
        const int h = idx / D, d = idx - h * D;
        // dim d sits in lane row d/(D/8), block (d % (D/8)) / 2, odd dims in elements 2, 3; column h in
        // lane c = h/2, element h%2
        const int lane_r = d / (D / 8), within = d % (D / 8);
        const int at = ((within >> 1) * 32 + lane_r * 4 + (h >> 1)) * 4 + (h & 1) + 2 * (within & 1);
        float big = s_m[h];
#pragma unroll
        for (int wv = 1; wv < kFdWarps; ++wv) big = fmaxf(big, s_m[wv * kFdCols + h]);
        float a = 0.0f;
#pragma unroll
        for (int wv = 0; wv < kFdWarps; ++wv) {
            float part = s_of[wv * kMB * 128 + at];
            if constexpr (!kWide) part += s_of[wv * kMB * 128 + at + 8];   // column h+4: lane c+2, the low halves
            a += part * ex2_approx(s_m[wv * kFdCols + h] - big);
        }
        const long long slot = static_cast<long long>(kvh * p.group + chunk * kHeads + h) * p.num_splits + split;
        p.partial[2 * hs + slot * D + d] = a * unshift;
        if (d == 0) {
            float l = 0.0f;
#pragma unroll
            for (int wv = 0; wv < kFdWarps; ++wv) l += s_l[wv * kFdCols + h] * ex2_approx(s_m[wv * kFdCols + h] - big);
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

// head_dim 512 (the reference accepts it, src/kernels/flash_decode.cu:313-314; none of its models uses it):
// a plain form of the same split — a CTA per (query head, split), warp w takes keys w, w+4, ... of the
// split, a lane owns 16 of the 512 dims (one 128-bit load of K codes and one of V codes per key), the
// score is a shuffle-reduced dot product, the online-softmax state (m, l, acc) is fp32 — and writes the
// scratch slab in the layout the reduce kernel reads.  The tensor-core form above would need 256
// registers of tile and accumulator per lane at this width.
constexpr int kFdWideDim = 512;

__device__ __forceinline__ void e4m3x16_to_f32(const uint4& w, float (&f)[16]) {
    const uint32_t words[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        uint32_t lo, hi;
        e4m3x4_to_f16x2x2(words[i], lo, hi);
        const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&lo));
        const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&hi));
        f[4 * i] = a.x; f[4 * i + 1] = a.y; f[4 * i + 2] = b.x; f[4 * i + 3] = b.y;
    }
}

__global__ void __launch_bounds__(kFdThreads) flash_decode_partial_wide_kernel(const FdArgs p) {
    constexpr int D = kFdWideDim;
    __shared__ float s_acc[kFdWarps][D];
    __shared__ float s_m[kFdWarps], s_l[kFdWarps];
    const int qh = blockIdx.x, split = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kvh = qh / p.group;
    pdl_enter();
    const int n_keys = *p.cache_len + 1;
    const int per = (n_keys + p.num_splits - 1) / p.num_splits;
    const int begin = split * per, end = min(n_keys, begin + per);

    float qf[16];
    {
        const uint4* qp = reinterpret_cast<const uint4*>(p.q + static_cast<size_t>(qh) * D + lane * 16);
        float lo[8], hi[8];
        unpack8(qp[0], lo);
        unpack8(qp[1], hi);
#pragma unroll
        for (int i = 0; i < 8; ++i) { qf[i] = lo[i] * p.scale_log2e; qf[8 + i] = hi[i] * p.scale_log2e; }
    }
    float m = kFdMInit, l = 0.0f, acc[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) acc[i] = 0.0f;
    for (int key = begin + warp; key < end; key += kFdWarps) {
        const size_t row = static_cast<size_t>(key) * p.num_kv_heads + kvh;
        const uint4 kc = *reinterpret_cast<const uint4*>(p.k + row * D + lane * 16);
        const uint4 vc = *reinterpret_cast<const uint4*>(p.v + row * D + lane * 16);
        const float ks = p.k_scale[row], vs = p.v_scale[row];
        float kf[16], vf[16];
        e4m3x16_to_f32(kc, kf);
        float dot = 0.0f;
#pragma unroll
        for (int i = 0; i < 16; ++i) dot = fmaf(qf[i], kf[i], dot);
        dot = group_sum<32>(dot) * ks;
        const float m_new = fmaxf(m, dot);
        const float corr = ex2_approx(m - m_new), w = ex2_approx(dot - m_new);
        l = l * corr + w;
        e4m3x16_to_f32(vc, vf);
        const float wv = w * vs;
#pragma unroll
        for (int i = 0; i < 16; ++i) acc[i] = fmaf(wv, vf[i], acc[i] * corr);
        m = m_new;
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) s_acc[warp][lane * 16 + i] = acc[i];
    if (lane == 0) { s_m[warp] = m; s_l[warp] = l; }
    __syncthreads();
    float big = s_m[0];
#pragma unroll
    for (int wv = 1; wv < kFdWarps; ++wv) big = fmaxf(big, s_m[wv]);
    const long long hs = static_cast<long long>(p.num_q_heads) * p.num_splits;
    const long long slot = static_cast<long long>(qh) * p.num_splits + split;
    for (int d = threadIdx.x; d < D; d += kFdThreads) {
        float a = 0.0f;
#pragma unroll
        for (int wv = 0; wv < kFdWarps; ++wv) a += s_acc[wv][d] * ex2_approx(s_m[wv] - big);
        p.partial[2 * hs + slot * D + d] = a;
    }
    if (threadIdx.x == 0) {
        float lsum = 0.0f;
#pragma unroll
        for (int wv = 0; wv < kFdWarps; ++wv) lsum += s_l[wv] * ex2_approx(s_m[wv] - big);
        p.partial[slot] = big;
        p.partial[hs + slot] = lsum;
    }
}

template <int D, bool kWide>
void launch_partial_as(const FdArgs& a, cudaStream_t stream) {
    const dim3 grid(static_cast<unsigned>(a.num_kv_heads * a.row_chunks), static_cast<unsigned>(a.num_splits));
    constexpr int smem = FdRing<D>::kSmemBytes;
    (void)host::setup<&flash_decode_partial_kernel<D, kWide>, kFdThreads, static_cast<size_t>(smem)>();   // shared-memory opt-in, once per device
    host::launch<flash_decode_partial_kernel<D, kWide>>(grid, dim3(kFdThreads), static_cast<size_t>(smem), stream, a);
}

template <int D>
void launch_partial(const FdArgs& a, cudaStream_t stream) {
    if (a.heads_per_cta > 4) launch_partial_as<D, true>(a, stream);
    else launch_partial_as<D, false>(a, stream);
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
    RH_REQUIRE(head_dim == 32 || head_dim == 64 || head_dim == 128 || head_dim == 256 || head_dim == 512, RH_ERR_UNSUPPORTED_DIM,
               "%s: head_dim must be one of 32, 64, 128, 256, 512", fn);
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
    a.heads_per_cta = a.group > 4 ? 8 : 4;
    a.row_chunks = (a.group + a.heads_per_cta - 1) / a.heads_per_cta;
    a.scale_log2e = scale * kFdLog2e;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (head_dim) {
        case 32: launch_partial<32>(a, s); break;
        case 64: launch_partial<64>(a, s); break;
        case 128: launch_partial<128>(a, s); break;
        case 256: launch_partial<256>(a, s); break;
        default:
            host::launch<flash_decode_partial_wide_kernel>(dim3(static_cast<unsigned>(num_q_heads), static_cast<unsigned>(num_splits)),
                                                           dim3(kFdThreads), 0, s, a);
            break;
    }
    if (const int st = host::check_launch(fn)) return st;
    const dim3 rgrid(static_cast<unsigned>(num_q_heads)), rblock(kFdReduceThreads);
    __nv_bfloat16* o = static_cast<__nv_bfloat16*>(out);
    const float* part = partial;
    switch (head_dim) {
        case 32: host::launch<flash_decode_reduce_kernel<32>>(rgrid, rblock, 0, s, o, part, num_splits, num_q_heads); break;
        case 64: host::launch<flash_decode_reduce_kernel<64>>(rgrid, rblock, 0, s, o, part, num_splits, num_q_heads); break;
        case 128: host::launch<flash_decode_reduce_kernel<128>>(rgrid, rblock, 0, s, o, part, num_splits, num_q_heads); break;
        case 256: host::launch<flash_decode_reduce_kernel<256>>(rgrid, rblock, 0, s, o, part, num_splits, num_q_heads); break;
        default: host::launch<flash_decode_reduce_kernel<512>>(rgrid, rblock, 0, s, o, part, num_splits, num_q_heads); break;
    }
    return host::check_launch(fn);
}
