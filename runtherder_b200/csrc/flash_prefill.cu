// Causal attention of n_new query tokens over the FP8-E4M3 KV cache (prefill and chunked prefill).
// Replaces runtherder::kernels::flash_prefill_bf16
// (include/runtherder/kernels/flash_prefill.cuh:27-40, src/kernels/flash_prefill.cu:34-241).
//
// The reference runs one CTA of 4 warps per (64-token tile, query head): every query head of a group
// converts the same K/V tile again, one byte per thread and iteration, and the tile is loaded, converted
// and consumed strictly one after the other.  Here a CTA serves ALL query heads of a kv head for its
// token tile (warp = 16 tokens of one head, up to 8 warps), so a K/V tile is fetched and converted once
// per group: cp.async brings the raw E4M3 rows of the next tile in while the current one is converted
// (16 codes per thread and step, two codes per cvt) and multiplied.  The contractions are
// mma.sync.m16n8k16 (f16 operands, fp32 accumulate) fed by ldmatrix from XOR-swizzled shared memory.
// As in the decode kernel the per-key scales never touch the operands: the K scale multiplies the fp32
// score, the V scale rides in the exponent of the weight (w = 2^(s + lg2 vs - m), at most 1) and the
// softmax denominator accumulates w / vs, so V enters the second product as exact E4M3 values.
//
// Shared memory feeds the tensor cores here: with 16 query rows per warp every K/V fragment read serves one
// product and the kernel is bound by shared-memory bandwidth (76 % of peak, tensor pipe 45 %), so for
// prompts that fill the GPU a warp owns 32 rows and every fragment serves two.
// Not a tcgen05 kernel: that is the next step for this op (a 128-row UMMA tile per CTA reads the K/V
// operands from shared memory once per CTA instead of once per warp).
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include <atomic>

#include "rh_common.cuh"
#include "rh_kernels.h"

namespace rh {
namespace {

constexpr int kPfD = 128;        // head_dim (the reference supports 128 only: flash_prefill.cu:227)
constexpr int kPfKeys = 64;      // keys per tile
constexpr int kPfMaxWarps = 8;
constexpr int kPfRowBytes = kPfD * 2;   // one f16 row in shared memory
constexpr float kPfLog2e = 1.4426950408889634f;
constexpr float kPfMInit = -1.0e30f;
constexpr float kPfLgFloor = -100.0f;

// shared-memory map (bytes); kMT = 16-row tiles per warp (1 or 2), which also is the number of f16
// K/V tile buffers (the 2-tile form runs one CTA per SM and can afford to convert a tile ahead)
constexpr int kPfTileF16 = kPfKeys * kPfRowBytes;                  // 16 KB: a converted K or V tile
constexpr int kPfRawTile = kPfKeys * kPfD;                         // 8 KB: a raw E4M3 K or V tile
constexpr int kPfRawStage = 2 * kPfRawTile + 2 * kPfKeys * 4;      // K, V, k scales, v scales
constexpr int kPfCstBytes = 3 * kPfKeys * 4;                       // ksl[64], lgv[64], rvs[64]
template <int kMT>
struct PfSmem {
    static constexpr int kBufs = kMT;
    static constexpr int kOffKV = 0;                                        // [buf][K, V] f16 tiles
    static constexpr int kOffRaw = kOffKV + kBufs * 2 * kPfTileF16;         // [2] raw stages
    static constexpr int kOffCst = kOffRaw + 2 * kPfRawStage;               // [buf] per-key constants
    static constexpr int kOffQ = kOffCst + kBufs * kPfCstBytes;             // [warps][16 * kMT rows][128] f16
    static constexpr int bytes(int warps) { return kOffQ + warps * 16 * kMT * kPfRowBytes; }
};

struct PfArgs {
    __nv_bfloat16* out;
    const __nv_bfloat16* q;
    const uint8_t* k;
    const uint8_t* v;
    const float* k_scale;
    const float* v_scale;
    const int* cache_len;
    int n_new;
    int num_q_heads;
    int num_kv_heads;
    int group;           // query heads per kv head
    int heads_per_cta;   // min(group, 8)
    int subs;            // token sub-tiles (one warp each) per CTA: max(1, 8 / heads_per_cta)
    int head_chunks;     // ceil(group / heads_per_cta)
    float scale_log2e;
};

__device__ __forceinline__ void pf_e4m3x4_to_f16x2x2(uint32_t word, uint32_t& lo, uint32_t& hi) {
    asm("{\n\t.reg .b16 l, h;\n\tmov.b32 {l, h}, %2;\n\tcvt.rn.f16x2.e4m3x2 %0, l;\n\tcvt.rn.f16x2.e4m3x2 %1, h;\n\t}"
        : "=r"(lo), "=r"(hi)
        : "r"(word));
}
__device__ __forceinline__ uint32_t pf_pack_f16x2(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
}
__device__ __forceinline__ void pf_mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void pf_ldsm_x4(uint32_t (&r)[4], uint32_t smem_addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(smem_addr));
}
__device__ __forceinline__ void pf_ldsm_x4_trans(uint32_t (&r)[4], uint32_t smem_addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(smem_addr));
}
__device__ __forceinline__ float pf_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float pf_lg2(float x) {
    float y;
    asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ void pf_cp_async16_zfill(uint32_t smem_addr, const void* gmem, bool valid) {
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_addr), "l"(gmem), "r"(bytes) : "memory");
}
__device__ __forceinline__ void pf_cp_async4_zfill(uint32_t smem_addr, const void* gmem, bool valid) {
    const int bytes = valid ? 4 : 0;
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(smem_addr), "l"(gmem), "r"(bytes) : "memory");
}
// byte offset of 16-byte chunk `chunk` (0..15) of row `row` in an f16 tile: chunks are XORed with the
// row so that the eight rows an ldmatrix reads, and the rows a conversion step writes, spread over banks
__device__ __forceinline__ int pf_swz(int row, int chunk) { return row * kPfRowBytes + ((chunk ^ (row & 7)) << 4); }
// the same for the 8 chunks of a raw 128-byte row
__device__ __forceinline__ int pf_swz_raw(int row, int chunk) { return row * kPfD + ((chunk ^ (row & 7)) << 4); }

// grid (token tiles, num_kv_heads * head_chunks); block = 32 * heads_here * subs threads; a warp owns
// 16 * kMT consecutive tokens of one query head.
template <int kMT>
__global__ void __launch_bounds__(kPfMaxWarps * 32, (kMT == 1 ? 2 : 1)) flash_prefill_kernel(const PfArgs p) {
    using L = PfSmem<kMT>;
    constexpr int kRows = 16 * kMT;   // tokens per warp
    extern __shared__ __align__(128) unsigned char pf_smem[];
    const uint32_t smem_base = static_cast<uint32_t>(__cvta_generic_to_shared(pf_smem));
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int n_threads = blockDim.x;
    const int r = lane >> 2, c = lane & 3;

    const int kvh = blockIdx.y / p.head_chunks;
    const int chunk = blockIdx.y - kvh * p.head_chunks;
    const int heads_here = min(p.heads_per_cta, p.group - chunk * p.heads_per_cta);
    const int sub = warp / heads_here;                      // token sub-tile of this warp
    const int head = warp - sub * heads_here;               // its query head within the chunk
    const bool warp_active = sub < p.subs;                  // blockDim is sized for the widest chunk
    const int qh = kvh * p.group + chunk * p.heads_per_cta + head;
    const int tile = gridDim.x - 1 - blockIdx.x;            // long (late) token tiles first
    const int tok0_cta = tile * kRows * p.subs;
    const int tok0 = tok0_cta + kRows * sub;                // first token of this warp

    pdl_enter();
    const int clen = *p.cache_len;
    const int total_keys = clen + p.n_new;
    const int last_tok_cta = min(tok0_cta + kRows * p.subs, p.n_new) - 1;
    const int n_tiles = min((total_keys + kPfKeys - 1) / kPfKeys, (clen + last_tok_cta) / kPfKeys + 1);
    const int last_tok_warp = min(tok0 + kRows, p.n_new) - 1;
    const int warp_last_tile = (warp_active && last_tok_warp >= tok0) ? (clen + last_tok_warp) / kPfKeys : -1;

    // ---- raw tile copies (all threads): 64 K rows + 64 V rows of 128 bytes (chunks swizzled), 2 x 64 scales ----
    const size_t row_stride = static_cast<size_t>(p.num_kv_heads) * kPfD;
    auto issue_raw = [&](int j) {
        const uint32_t st = smem_base + L::kOffRaw + (j & 1) * kPfRawStage;
        for (int id = tid; id < 2 * kPfKeys * 8; id += n_threads) {
            const int which = id >> 9, row = (id >> 3) & 63, ch = id & 7;
            const int key = j * kPfKeys + row;
            const bool live = key < total_keys;
            const uint8_t* src = (which ? p.v : p.k) + (live ? static_cast<size_t>(key) * row_stride + static_cast<size_t>(kvh) * kPfD + ch * 16 : 0);
            pf_cp_async16_zfill(st + which * kPfRawTile + pf_swz_raw(row, ch), src, live);
        }
        for (int id = tid; id < 2 * kPfKeys; id += n_threads) {
            const int which = id >> 6, row = id & 63;
            const int key = j * kPfKeys + row;
            const bool live = key < total_keys;
            const float* src = (which ? p.v_scale : p.k_scale) + (live ? static_cast<size_t>(key) * p.num_kv_heads + kvh : 0);
            pf_cp_async4_zfill(st + 2 * kPfRawTile + which * kPfKeys * 4 + row * 4, src, live);
        }
        cp_async_commit();
    };
    // ---- convert raw tile j into f16 buffer j % kBufs: 16 codes per step, 8 cvt, two swizzled 16-byte
    //      stores; a quarter-warp works on eight consecutive rows of one chunk column, so the swizzles make
    //      both the read and the stores conflict-free ----
    auto convert = [&](int j) {
        const unsigned char* const raw = pf_smem + L::kOffRaw + (j & 1) * kPfRawStage;
        unsigned char* const kv = pf_smem + L::kOffKV + (j % L::kBufs) * 2 * kPfTileF16;
        for (int id = tid; id < 2 * kPfKeys * 8; id += n_threads) {
            const int which = id >> 9, ch = (id >> 6) & 7, row = id & 63;
            const uint4 w = *reinterpret_cast<const uint4*>(raw + which * kPfRawTile + pf_swz_raw(row, ch));
            uint4 h0, h1;
            pf_e4m3x4_to_f16x2x2(w.x, h0.x, h0.y);
            pf_e4m3x4_to_f16x2x2(w.y, h0.z, h0.w);
            pf_e4m3x4_to_f16x2x2(w.z, h1.x, h1.y);
            pf_e4m3x4_to_f16x2x2(w.w, h1.z, h1.w);
            unsigned char* const dst = kv + which * kPfTileF16;
            *reinterpret_cast<uint4*>(dst + pf_swz(row, 2 * ch)) = h0;
            *reinterpret_cast<uint4*>(dst + pf_swz(row, 2 * ch + 1)) = h1;
        }
        float* const cst = reinterpret_cast<float*>(pf_smem + L::kOffCst + (j % L::kBufs) * kPfCstBytes);
        for (int id = tid; id < kPfKeys; id += n_threads) {
            const float* const sc = reinterpret_cast<const float*>(raw + 2 * kPfRawTile);
            const float lg = fmaxf(pf_lg2(sc[kPfKeys + id]), kPfLgFloor);
            cst[id] = sc[id] * p.scale_log2e;
            cst[kPfKeys + id] = lg;
            cst[2 * kPfKeys + id] = pf_ex2(-lg);
        }
    };
    issue_raw(0);

    // ---- Q: this warp's rows, bf16 -> f16, swizzled (operands narrow to f16 as in the reference) ----
    const int q_off = L::kOffQ + warp * kRows * kPfRowBytes;
    const uint32_t q_s = smem_base + q_off;
    if (warp_active) {
#pragma unroll
        for (int i = 0; i < 8 * kMT; ++i) {
            const int id = lane + 32 * i, row = id >> 4, ch = id & 15;
            const int tok = tok0 + row;
            uint4 w = make_uint4(0u, 0u, 0u, 0u);
            if (tok < p.n_new)
                w = *reinterpret_cast<const uint4*>(p.q + (static_cast<size_t>(tok) * p.num_q_heads + qh) * kPfD + ch * 8);
            uint4 h;
            h.x = pf_pack_f16x2(bf_lo(w.x), bf_hi(w.x));
            h.y = pf_pack_f16x2(bf_lo(w.y), bf_hi(w.y));
            h.z = pf_pack_f16x2(bf_lo(w.z), bf_hi(w.z));
            h.w = pf_pack_f16x2(bf_lo(w.w), bf_hi(w.w));
            *reinterpret_cast<uint4*>(pf_smem + q_off + pf_swz(row, ch)) = h;
        }
    }

    float o[kMT][16][4];
    float m_run[kMT][2], l_run[kMT][2];   // rows r and r+8 of each 16-row tile
#pragma unroll
    for (int t = 0; t < kMT; ++t) {
#pragma unroll
        for (int n = 0; n < 16; ++n) o[t][n][0] = o[t][n][1] = o[t][n][2] = o[t][n][3] = 0.0f;
        m_run[t][0] = m_run[t][1] = kPfMInit;
        l_run[t][0] = l_run[t][1] = 0.0f;
    }

    // per-lane ldmatrix row/chunk selectors
    const int a_row = (lane & 7) + 8 * ((lane >> 3) & 1), a_ch = lane >> 4;          // Q: A operand
    const int k_row = (lane & 7) + 8 * (lane >> 4), k_ch = (lane >> 3) & 1;          // K: B operand of Q K^T
    const int v_row = (lane & 7) + 8 * ((lane >> 3) & 1), v_ch = lane >> 4;          // V: B operand of P V (transposed)

    if constexpr (kMT == 2) {   // two f16 buffers: tile 0 is converted ahead of the loop
        cp_async_wait<0>();
        __syncthreads();
        if (1 < n_tiles) issue_raw(1);
        convert(0);
    }

    for (int j = 0; j < n_tiles; ++j) {
        if constexpr (kMT == 1) {
            cp_async_wait<0>();
            __syncthreads();   // raw tile j has landed for every thread; everybody is done with the f16 tiles of j-1
            if (j + 1 < n_tiles) issue_raw(j + 1);
            convert(j);
            __syncthreads();
        } else {
            cp_async_wait<0>();
            __syncthreads();   // f16 tile j is complete, raw tile j+1 has landed, f16 buffer (j+1)%2 is free again
            if (j + 2 < n_tiles) issue_raw(j + 2);
            if (j + 1 < n_tiles) convert(j + 1);   // other warps' products overlap this
        }
        if (j > warp_last_tile) continue;   // every key of this tile is in this warp's future

        const uint32_t k_s = smem_base + L::kOffKV + (j % L::kBufs) * 2 * kPfTileF16, v_s = k_s + kPfTileF16;
        const float* const cst = reinterpret_cast<const float*>(pf_smem + L::kOffCst + (j % L::kBufs) * kPfCstBytes);
        const float2* const ksl2 = reinterpret_cast<const float2*>(cst);
        const float2* const lgv2 = reinterpret_cast<const float2*>(cst + kPfKeys);
        const float2* const rvs2 = reinterpret_cast<const float2*>(cst + 2 * kPfKeys);

        // ---- S = Q K^T (16 * kMT x 64 per warp): every K fragment feeds kMT products ----
        float s[kMT][8][4];
#pragma unroll
        for (int t = 0; t < kMT; ++t)
#pragma unroll
            for (int n = 0; n < 8; ++n) s[t][n][0] = s[t][n][1] = s[t][n][2] = s[t][n][3] = 0.0f;
#pragma unroll
        for (int kk = 0; kk < kPfD / 16; ++kk) {
            uint32_t a[kMT][4];
#pragma unroll
            for (int t = 0; t < kMT; ++t) pf_ldsm_x4(a[t], q_s + pf_swz(16 * t + a_row, 2 * kk + a_ch));
#pragma unroll
            for (int nn = 0; nn < 4; ++nn) {
                uint32_t b[4];
                pf_ldsm_x4(b, k_s + pf_swz(16 * nn + k_row, 2 * kk + k_ch));
#pragma unroll
                for (int t = 0; t < kMT; ++t) {
                    pf_mma(s[t][2 * nn], a[t], b[0], b[1]);
                    pf_mma(s[t][2 * nn + 1], a[t], b[2], b[3]);
                }
            }
        }

        // ---- log2-domain scores with the V scale in the exponent, causal mask, online softmax ----
        const bool diag = j * kPfKeys + kPfKeys - 1 > clen + tok0;   // some key of the tile is masked for some row
#pragma unroll
        for (int t = 0; t < kMT; ++t) {
            const int qpos_lo = clen + tok0 + 16 * t + r, qpos_hi = qpos_lo + 8;
            float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
            for (int n = 0; n < 8; ++n) {
                const float2 kk = ksl2[n * 4 + c], lg = lgv2[n * 4 + c];
                s[t][n][0] = fmaf(s[t][n][0], kk.x, lg.x);
                s[t][n][1] = fmaf(s[t][n][1], kk.y, lg.y);
                s[t][n][2] = fmaf(s[t][n][2], kk.x, lg.x);
                s[t][n][3] = fmaf(s[t][n][3], kk.y, lg.y);
                if (diag) {
                    const int kpos = j * kPfKeys + 8 * n + 2 * c;
                    if (kpos > qpos_lo) s[t][n][0] = -INFINITY;
                    if (kpos + 1 > qpos_lo) s[t][n][1] = -INFINITY;
                    if (kpos > qpos_hi) s[t][n][2] = -INFINITY;
                    if (kpos + 1 > qpos_hi) s[t][n][3] = -INFINITY;
                }
                mx_lo = fmaxf(mx_lo, fmaxf(s[t][n][0], s[t][n][1]));
                mx_hi = fmaxf(mx_hi, fmaxf(s[t][n][2], s[t][n][3]));
            }
            mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
            mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
            mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
            mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
            const float n_lo = fmaxf(m_run[t][0], mx_lo), n_hi = fmaxf(m_run[t][1], mx_hi);
            const float corr_lo = pf_ex2(m_run[t][0] - n_lo), corr_hi = pf_ex2(m_run[t][1] - n_hi);
            m_run[t][0] = n_lo;
            m_run[t][1] = n_hi;
            float sum_lo = 0.0f, sum_hi = 0.0f;
#pragma unroll
            for (int n = 0; n < 8; ++n) {
                const float2 rv = rvs2[n * 4 + c];
                s[t][n][0] = pf_ex2(s[t][n][0] - n_lo);
                s[t][n][1] = pf_ex2(s[t][n][1] - n_lo);
                s[t][n][2] = pf_ex2(s[t][n][2] - n_hi);
                s[t][n][3] = pf_ex2(s[t][n][3] - n_hi);
                sum_lo = fmaf(s[t][n][0], rv.x, fmaf(s[t][n][1], rv.y, sum_lo));
                sum_hi = fmaf(s[t][n][2], rv.x, fmaf(s[t][n][3], rv.y, sum_hi));
            }
            l_run[t][0] = fmaf(l_run[t][0], corr_lo, sum_lo);
            l_run[t][1] = fmaf(l_run[t][1], corr_hi, sum_hi);
            if (__any_sync(0xffffffffu, corr_lo != 1.0f || corr_hi != 1.0f)) {
#pragma unroll
                for (int n = 0; n < 16; ++n) {
                    o[t][n][0] *= corr_lo;
                    o[t][n][1] *= corr_lo;
                    o[t][n][2] *= corr_hi;
                    o[t][n][3] *= corr_hi;
                }
            }
        }

        // ---- O += W V (V as exact E4M3 values; four 16-key steps; every V fragment feeds kMT products) ----
#pragma unroll
        for (int kc = 0; kc < kPfKeys / 16; ++kc) {
            uint32_t a[kMT][4];
#pragma unroll
            for (int t = 0; t < kMT; ++t) {
                a[t][0] = pf_pack_f16x2(s[t][2 * kc][0], s[t][2 * kc][1]);
                a[t][1] = pf_pack_f16x2(s[t][2 * kc][2], s[t][2 * kc][3]);
                a[t][2] = pf_pack_f16x2(s[t][2 * kc + 1][0], s[t][2 * kc + 1][1]);
                a[t][3] = pf_pack_f16x2(s[t][2 * kc + 1][2], s[t][2 * kc + 1][3]);
            }
#pragma unroll
            for (int nn = 0; nn < kPfD / 16; ++nn) {
                uint32_t b[4];
                pf_ldsm_x4_trans(b, v_s + pf_swz(16 * kc + v_row, 2 * nn + v_ch));
#pragma unroll
                for (int t = 0; t < kMT; ++t) {
                    pf_mma(o[t][2 * nn], a[t], b[0], b[1]);
                    pf_mma(o[t][2 * nn + 1], a[t], b[2], b[3]);
                }
            }
        }
    }

    // ---- normalise and store ----
    if (!warp_active) return;
#pragma unroll
    for (int t = 0; t < kMT; ++t) {
        float l_lo = l_run[t][0], l_hi = l_run[t][1];
        l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
        l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
        l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
        l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
        const float inv_lo = 1.0f / l_lo, inv_hi = 1.0f / l_hi;
        const int tok_lo = tok0 + 16 * t + r, tok_hi = tok_lo + 8;
        __nv_bfloat16* const out_lo = p.out + (static_cast<size_t>(tok_lo) * p.num_q_heads + qh) * kPfD + 2 * c;
        __nv_bfloat16* const out_hi = p.out + (static_cast<size_t>(tok_hi) * p.num_q_heads + qh) * kPfD + 2 * c;
#pragma unroll
        for (int n = 0; n < 16; ++n) {
            if (tok_lo < p.n_new)
                *reinterpret_cast<__nv_bfloat162*>(out_lo + 8 * n) = __floats2bfloat162_rn(o[t][n][0] * inv_lo, o[t][n][1] * inv_lo);
            if (tok_hi < p.n_new)
                *reinterpret_cast<__nv_bfloat162*>(out_hi + 8 * n) = __floats2bfloat162_rn(o[t][n][2] * inv_hi, o[t][n][3] * inv_hi);
        }
    }
}

template <int kMT>
int launch_prefill(PfArgs a, cudaStream_t stream, const char* fn) {
    const int warps = a.heads_per_cta * a.subs;
    const int tokens_per_cta = 16 * kMT * a.subs;
    const int smem = PfSmem<kMT>::bytes(warps);
    // opt in to the largest shared-memory request of this form, once per device
    (void)host::setup<&flash_prefill_kernel<kMT>, kPfMaxWarps * 32, static_cast<size_t>(PfSmem<kMT>::bytes(kPfMaxWarps))>();
    const dim3 grid(static_cast<unsigned>((a.n_new + tokens_per_cta - 1) / tokens_per_cta),
                    static_cast<unsigned>(a.num_kv_heads * a.head_chunks));
    RH_REQUIRE(grid.y <= 65535u, RH_ERR_UNSUPPORTED_DIM, "%s: too many kv heads", fn);
    host::launch<flash_prefill_kernel<kMT>>(grid, dim3(static_cast<unsigned>(warps * 32)), static_cast<size_t>(smem), stream, a);
    return host::check_launch(fn);
}

}  // namespace
}  // namespace rh

using namespace rh;

namespace rh {
// flash_prefill_tc.cu: the same product on the 5th-generation tensor cores (tcgen05.mma, tensor memory)
int launch_flash_prefill_tc(void* out, const void* q, const uint8_t* k, const uint8_t* v, const float* k_scale,
                            const float* v_scale, int n_new, const int* cache_len, int num_q_heads, int num_kv_heads,
                            float scale, cudaStream_t stream, const char* fn);
}  // namespace rh

extern "C" int rh_flash_prefill_bf16(void* out, const void* q, const uint8_t* k, const uint8_t* v, const float* k_scale,
                                     const float* v_scale, int n_new, const int* cache_len, int num_q_heads,
                                     int num_kv_heads, int head_dim, float scale, void* stream) {
    const char* const fn = "rh_flash_prefill_bf16";
    RH_REQUIRE(out && q && k && v && k_scale && v_scale, RH_ERR_INVALID_ARG, "%s: null pointer", fn);
    RH_REQUIRE(cache_len != nullptr, RH_ERR_INVALID_ARG, "%s: cache_len must not be null", fn);
    RH_REQUIRE(n_new >= 1, RH_ERR_INVALID_ARG, "%s: n_new must be >= 1", fn);
    RH_REQUIRE(num_q_heads >= 1 && num_kv_heads >= 1, RH_ERR_INVALID_ARG, "%s: head counts must be >= 1", fn);
    RH_REQUIRE(num_q_heads % num_kv_heads == 0, RH_ERR_INVALID_ARG,
               "%s: num_q_heads must be a multiple of num_kv_heads", fn);
    RH_REQUIRE(head_dim == kPfD, RH_ERR_UNSUPPORTED_DIM, "%s: supports head_dim 128 only", fn);
    RH_REQUIRE(host::aligned16(q) && host::aligned16(k) && host::aligned16(v), RH_ERR_MISALIGNED,
               "%s: q, k and v must be 16-byte aligned", fn);
    RH_REQUIRE((reinterpret_cast<uintptr_t>(out) & 3u) == 0, RH_ERR_MISALIGNED, "%s: out must be 4-byte aligned", fn);

    PfArgs a;
    a.out = static_cast<__nv_bfloat16*>(out);
    a.q = static_cast<const __nv_bfloat16*>(q);
    a.k = k;
    a.v = v;
    a.k_scale = k_scale;
    a.v_scale = v_scale;
    a.cache_len = cache_len;
    a.n_new = n_new;
    a.num_q_heads = num_q_heads;
    a.num_kv_heads = num_kv_heads;
    a.group = num_q_heads / num_kv_heads;
    a.heads_per_cta = a.group < kPfMaxWarps ? a.group : kPfMaxWarps;
    a.subs = kPfMaxWarps / a.heads_per_cta;
    a.head_chunks = (a.group + a.heads_per_cta - 1) / a.heads_per_cta;
    a.scale_log2e = scale * kPfLog2e;
    // Two 16-row tiles per warp halve the shared-memory reads per product (one CTA per SM, 255 registers);
    // short prompts do not fill the GPU with such CTAs and take the one-tile form (two CTAs per SM).
    const long long ctas_wide = static_cast<long long>((n_new + 32 * a.subs - 1) / (32 * a.subs)) * num_kv_heads * a.head_chunks;
    // Default: the tcgen05 form (flash_prefill_tc.cu; it stores 16-byte pieces of `out`).  "prefill_tiles" 1 or 2,
    // or an `out` that is only 4-byte aligned, selects the mma.sync forms below.
    const int pick = host::tuning(host::kPrefillTiles);
    if (pick != 1 && pick != 2 && host::aligned16(out))
        return launch_flash_prefill_tc(out, q, k, v, k_scale, v_scale, n_new, cache_len, num_q_heads, num_kv_heads, scale,
                                       static_cast<cudaStream_t>(stream), fn);
    const bool wide = pick == 2 || (pick != 1 && ctas_wide >= 2LL * host::num_sms());
    return wide ? launch_prefill<2>(a, static_cast<cudaStream_t>(stream), fn)
                : launch_prefill<1>(a, static_cast<cudaStream_t>(stream), fn);
}
