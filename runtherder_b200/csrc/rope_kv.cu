// RoPE on Q and K, optionally preceded by Qwen3's per-head RMSNorm and followed by
// the FP8 E4M3 KV-cache append of the rotated K and of V — one launch for what the
// reference issues as rmsnorm x2, rope, quantize_kv_fp8 x2.
//
// Layout.  A head row of D bf16 values is D/8 vectors; the rotate-half pairs are
// (i, i+D/2), i.e. vector v of the lower half pairs with vector v + D/16 of the
// upper half.  D/16 lanes own one head row: lane `sub` holds lower vector `sub` and
// upper vector `sub + D/16`, so both members of every pair, the head's sum of squares
// and its amax live inside one lane group and need only shuffles.  A warp carries
// 32/(D/16) head rows at a time ("a group": 4 rows at D = 128) and walks a chunk of
// consecutive groups of ONE token, so cos/sin of the token's 8 angles per lane are
// computed once and reused for every head of the chunk (the reference recomputes
// them for each of the Hq+Hkv heads).
//
// Numerics follow the reference kernels operation for operation:
//   norm  (src/kernels/rmsnorm.cu:77-135 at hidden_dim = D): per-vector FMA chain, then
//          the shuffle tree — lower+upper vector first (the tree's offset-D/16 level),
//          then offsets D/32 ... 1; y = bf16((h*rrms)*g)
//   rope  (src/kernels/rope.cu:35-54): theta = float(pos)*inv_freq[i]; __sincosf;
//          bf16(a*c - b*s), bf16(a*s + b*c) on the bf16-rounded inputs
//   fp8   (src/kernels/quantization.cu:210-250): amax of the bf16 row; scale = amax/448;
//          e4m3(x * (448/amax)); destination row = token*Hkv + head + at_pos*Hkv
#include "rh_common.cuh"

namespace rh {

namespace {

struct RopeArgs {
    void* q;
    void* k_out;
    const void* k_in;
    const void* v_in;
    const void* q_norm;
    const void* k_norm;
    float eps;
    const int* positions;
    const float* inv_freq;
    uint8_t* k_cache;
    float* k_scale;
    uint8_t* v_cache;
    float* v_scale;
    const int* at_pos;
    int seq_len;
    int num_q_heads;
    int num_kv_heads;
    int groups_per_item;  // head groups one warp handles for its token
    int items_per_token;
    // Qwen2's projection biases (src/kernels/bias.cu:64-90), [Hq*D], [Hkv*D], [Hkv*D]; all three or none.
    // x = bf16(float(x) + float(bias)) is applied to a row as it is loaded, before norm / rotation / append.
    const void* q_bias;
    const void* k_bias;
    const void* v_bias;
};

// row + bias on packed bf16 words: every element bf16(float(x) + float(b)) (src/kernels/bias.cu:15-28)
__device__ __forceinline__ uint4 add_bias_row(const uint4& x, const uint4& b) {
    const uint32_t xw[4] = {x.x, x.y, x.z, x.w}, bw[4] = {b.x, b.y, b.z, b.w};
    uint32_t o[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const float2 t = add2_rn(bf2_to_f2(xw[k]), bf2_to_f2(bw[k]));
        o[k] = pack_bf16x2(t.x, t.y);
    }
    return make_uint4(o[0], o[1], o[2], o[3]);
}

// The rotation.  The reference writes `a*c - b*s` and `a*s + b*c` (src/kernels/rope.cu:53-54) and
// nvcc contracts each into one product plus a fused multiply-add on the FIRST product; the
// contraction is spelled out here because it is part of the result's bits and the compiler picks
// a different one when the expression is inlined into a larger body.
__device__ __forceinline__ void rotate(float a, float b, float c, float s, float& lo, float& hi) {
    const float2 t = mul2_rn(splat2(b), make_float2(s, c));                    // {b*s, b*c}
    const float2 r = fma2_rn(splat2(a), make_float2(c, s), make_float2(-t.x, t.y));
    lo = r.x;
    hi = r.y;
}

template <int D, bool kNorm, bool kKV>
__global__ void __launch_bounds__(256) rope_kv_generic_kernel(const RopeArgs p) {
    constexpr int kLanesPerHead = D / 16;
    constexpr int kHeadsPerGroup = 32 / kLanesPerHead;
    constexpr int kVecsPerRow = D / 8;

    const int lane = threadIdx.x & 31;
    const int sub = lane % kLanesPerHead;
    const int hslot = lane / kLanesPerHead;
    const int warps_per_cta = blockDim.x >> 5;
    const long long item = static_cast<long long>(blockIdx.x) * warps_per_cta + (threadIdx.x >> 5);
    const long long num_items = static_cast<long long>(p.seq_len) * p.items_per_token;
    pdl_enter();
    if (item >= num_items) return;  // whole warps only: shuffles below stay convergent

    const int token = static_cast<int>(item / p.items_per_token);
    const int chunk = static_cast<int>(item % p.items_per_token);
    const int Hq = p.num_q_heads, Hkv = p.num_kv_heads;
    const int rows = Hq + (kKV ? 2 * Hkv : Hkv);
    const int groups = (rows + kHeadsPerGroup - 1) / kHeadsPerGroup;
    const int g_begin = chunk * p.groups_per_item;
    const int g_end = min(groups, g_begin + p.groups_per_item);

    // cos/sin of this lane's eight angles
    float cs[8], sn[8];
    {
        const float pos = static_cast<float>(p.positions[token]);
        const float4 f0 = __ldg(reinterpret_cast<const float4*>(p.inv_freq) + 2 * sub);
        const float4 f1 = __ldg(reinterpret_cast<const float4*>(p.inv_freq) + 2 * sub + 1);
        const float fr[8] = {f0.x, f0.y, f0.z, f0.w, f1.x, f1.y, f1.z, f1.w};
#pragma unroll
        for (int j = 0; j < 8; ++j) __sincosf(pos * fr[j], &sn[j], &cs[j]);
    }
    long long slot_base = 0;
    if constexpr (kKV) slot_base = static_cast<long long>(*p.at_pos) * Hkv;

    // role of head row r: 0 = Q, 1 = K, 2 = V, 3 = none
    auto row_src = [&](int r, int& role) -> const uint4* {
        if (r < Hq) {
            role = 0;
            return static_cast<const uint4*>(p.q) + (static_cast<size_t>(token) * Hq + r) * kVecsPerRow;
        }
        if (r < Hq + Hkv) {
            role = 1;
            return static_cast<const uint4*>(p.k_in) + (static_cast<size_t>(token) * Hkv + (r - Hq)) * kVecsPerRow;
        }
        if (kKV && r < rows) {
            role = 2;
            return static_cast<const uint4*>(p.v_in) + (static_cast<size_t>(token) * Hkv + (r - Hq - Hkv)) * kVecsPerRow;
        }
        role = 3;
        return nullptr;
    };

    int role_next;
    const uint4* src_next = row_src(g_begin * kHeadsPerGroup + hslot, role_next);
    uint4 lo_next = make_uint4(0, 0, 0, 0), hi_next = make_uint4(0, 0, 0, 0);
    if (role_next != 3) {
        lo_next = ld_stream(src_next + sub);
        hi_next = ld_stream(src_next + sub + kLanesPerHead);
    }

    for (int g = g_begin; g < g_end; ++g) {
        const int r = g * kHeadsPerGroup + hslot;
        const int role = role_next;
        uint4 lo_v = lo_next, hi_v = hi_next;
        if (p.q_bias != nullptr && role != 3) {
            const int head = role == 0 ? r : (role == 1 ? r - Hq : r - Hq - Hkv);
            const uint4* bias = static_cast<const uint4*>(role == 0 ? p.q_bias : (role == 1 ? p.k_bias : p.v_bias)) +
                                static_cast<size_t>(head) * kVecsPerRow;
            lo_v = add_bias_row(lo_v, ld_weight(bias + sub));
            hi_v = add_bias_row(hi_v, ld_weight(bias + sub + kLanesPerHead));
        }
        if (g + 1 < g_end) {  // prefetch the next group's rows while this one is processed
            src_next = row_src(r + kHeadsPerGroup, role_next);
            if (role_next != 3) {
                lo_next = ld_stream(src_next + sub);
                hi_next = ld_stream(src_next + sub + kLanesPerHead);
            }
        }

        float a[8], b[8];
        unpack8(lo_v, a);
        unpack8(hi_v, b);

        if constexpr (kNorm) {
            // every lane runs the shuffles; only Q and K rows keep the result
            float ss_lo = 0.0f, ss_hi = 0.0f;
#pragma unroll
            for (int j = 0; j < 8; ++j) ss_lo = __fmaf_rn(a[j], a[j], ss_lo);
#pragma unroll
            for (int j = 0; j < 8; ++j) ss_hi = __fmaf_rn(b[j], b[j], ss_hi);
            const float total = group_sum<kLanesPerHead>(ss_lo + ss_hi);
            const float rrms = rsqrtf(total / static_cast<float>(D) + p.eps);
            if (role <= 1) {
                const uint4* w = static_cast<const uint4*>(role == 0 ? p.q_norm : p.k_norm);
                float gl[8], gh[8];
                unpack8(ld_weight(w + sub), gl);
                unpack8(ld_weight(w + sub + kLanesPerHead), gh);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    a[j] = round_bf16(a[j] * rrms * gl[j]);
                    b[j] = round_bf16(b[j] * rrms * gh[j]);
                }
            }
        }

        uint4 out_lo = lo_v, out_hi = hi_v;
        if (role <= 1) {
            float ol[8], oh[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) rotate(a[j], b[j], cs[j], sn[j], ol[j], oh[j]);
            out_lo = pack8(ol);
            out_hi = pack8(oh);
        }
        if (role == 0 || (role == 1 && p.k_out != nullptr)) {
            uint4* dst = (role == 0)
                             ? static_cast<uint4*>(p.q) + (static_cast<size_t>(token) * Hq + r) * kVecsPerRow
                             : static_cast<uint4*>(p.k_out) + (static_cast<size_t>(token) * Hkv + (r - Hq)) * kVecsPerRow;
            st_vec(dst + sub, out_lo);
            st_vec(dst + sub + kLanesPerHead, out_hi);
        }

        if constexpr (kKV) {
            float fl[8], fh[8];
            unpack8(out_lo, fl);
            unpack8(out_hi, fh);
            float amax = 0.0f;
#pragma unroll
            for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fmaxf(fabsf(fl[j]), fabsf(fh[j])));
            amax = group_max<kLanesPerHead>(amax);
            const float inv = (amax > 0.0f) ? (448.0f / amax) : 0.0f;
            if (role == 1 || role == 2) {
                const int kv_head = (role == 1) ? (r - Hq) : (r - Hq - Hkv);
                const long long dst_row = static_cast<long long>(token) * Hkv + kv_head + slot_base;
                uint8_t* cache = (role == 1) ? p.k_cache : p.v_cache;
                float* scale = (role == 1) ? p.k_scale : p.v_scale;
                if (sub == 0) scale[dst_row] = amax / 448.0f;
                uint2* c = reinterpret_cast<uint2*>(cache + static_cast<size_t>(dst_row) * D);
                st_vec8(c + sub, pack_e4m3x8(fl, inv));
                st_vec8(c + sub + kLanesPerHead, pack_e4m3x8(fh, inv));
            }
        }
    }
}

constexpr int kRopeDepth = 4;   // groups in flight per warp in the fast kernel (1 KB each at D = 128)

// Fast path for head counts that are multiples of the heads a warp carries (4 at D = 128): every
// group of a warp is then all-Q, all-K or all-V, so the three roles become three straight loops with
// no per-row role logic, row pointers advance by a constant, and the rotation works on the register
// pairs a packed bf16 word unpacks into:
//   lo2 = fma2(a2, c2, b2 * (-s2)),  hi2 = fma2(a2, s2, b2 * c2)
// — the same two roundings per output as fma(a, c, -(b*s)) and fma(a, s, b*c).
template <int D, bool kNorm, bool kKV>
__global__ void __launch_bounds__(256) rope_kv_kernel(const RopeArgs p) {
    constexpr int kLanesPerHead = D / 16;
    constexpr int kHeadsPerGroup = 32 / kLanesPerHead;
    constexpr int kVecsPerRow = D / 8;

    const int lane = threadIdx.x & 31;
    const int sub = lane % kLanesPerHead;
    const int hslot = lane / kLanesPerHead;
    const int warps_per_cta = blockDim.x >> 5;
    const long long item = static_cast<long long>(blockIdx.x) * warps_per_cta + (threadIdx.x >> 5);
    const long long num_items = static_cast<long long>(p.seq_len) * p.items_per_token;
    pdl_enter();
    if (item >= num_items) return;  // whole warps only

    const int token = static_cast<int>(item / p.items_per_token);
    const int chunk = static_cast<int>(item % p.items_per_token);
    const int Hq = p.num_q_heads, Hkv = p.num_kv_heads;
    const int gq = Hq / kHeadsPerGroup, gk = Hkv / kHeadsPerGroup;
    const int groups = gq + gk + (kKV ? gk : 0);
    const int g_begin = chunk * p.groups_per_item;
    const int g_end = min(groups, g_begin + p.groups_per_item);

    float2 c2[4], s2[4], ns2[4];   // cos, sin, -sin of this lane's eight angles, as pairs
    if (g_begin < gq + gk) {
        const float pos = static_cast<float>(p.positions[token]);
        const float4 f0 = __ldg(reinterpret_cast<const float4*>(p.inv_freq) + 2 * sub);
        const float4 f1 = __ldg(reinterpret_cast<const float4*>(p.inv_freq) + 2 * sub + 1);
        const float fr[8] = {f0.x, f0.y, f0.z, f0.w, f1.x, f1.y, f1.z, f1.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            __sincosf(pos * fr[2 * k], &s2[k].x, &c2[k].x);
            __sincosf(pos * fr[2 * k + 1], &s2[k].y, &c2[k].y);
            ns2[k] = neg2(s2[k]);
        }
    }
    long long slot_base = 0;
    if constexpr (kKV) slot_base = static_cast<long long>(*p.at_pos) * Hkv;

    // [per-head RMSNorm +] rotation of one head row held as (lo, hi) vectors; returns the rotated words.
    auto norm_rotate = [&](const uint4& lo_v, const uint4& hi_v, const void* norm_w, uint4& out_lo, uint4& out_hi) {
        const uint32_t lw[4] = {lo_v.x, lo_v.y, lo_v.z, lo_v.w}, hw[4] = {hi_v.x, hi_v.y, hi_v.z, hi_v.w};
        float2 a2[4], b2[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            a2[k] = bf2_to_f2(lw[k]);
            b2[k] = bf2_to_f2(hw[k]);
        }
        if constexpr (kNorm) {
            float ss_lo = 0.0f, ss_hi = 0.0f;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                ss_lo = __fmaf_rn(a2[k].x, a2[k].x, ss_lo);
                ss_lo = __fmaf_rn(a2[k].y, a2[k].y, ss_lo);
            }
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                ss_hi = __fmaf_rn(b2[k].x, b2[k].x, ss_hi);
                ss_hi = __fmaf_rn(b2[k].y, b2[k].y, ss_hi);
            }
            const float total = group_sum<kLanesPerHead>(ss_lo + ss_hi);
            const float2 rrms = splat2(rsqrtf(total / static_cast<float>(D) + p.eps));
            const uint4 gl = ld_weight(static_cast<const uint4*>(norm_w) + sub);
            const uint4 gh = ld_weight(static_cast<const uint4*>(norm_w) + sub + kLanesPerHead);
            const uint32_t glw[4] = {gl.x, gl.y, gl.z, gl.w}, ghw[4] = {gh.x, gh.y, gh.z, gh.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {   // bf16((h * rrms) * g), as the stored tensor the rotation reads
                const float2 ya = mul2_rn(mul2_rn(a2[k], rrms), bf2_to_f2(glw[k]));
                const float2 yb = mul2_rn(mul2_rn(b2[k], rrms), bf2_to_f2(ghw[k]));
                a2[k] = bf2_to_f2(pack_bf16x2(ya.x, ya.y));
                b2[k] = bf2_to_f2(pack_bf16x2(yb.x, yb.y));
            }
        }
        uint32_t ol[4], oh[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float2 lo2 = fma2_rn(a2[k], c2[k], mul2_rn(b2[k], ns2[k]));
            const float2 hi2 = fma2_rn(a2[k], s2[k], mul2_rn(b2[k], c2[k]));
            ol[k] = pack_bf16x2(lo2.x, lo2.y);
            oh[k] = pack_bf16x2(hi2.x, hi2.y);
        }
        out_lo = make_uint4(ol[0], ol[1], ol[2], ol[3]);
        out_hi = make_uint4(oh[0], oh[1], oh[2], oh[3]);
    };

    // FP8 append of one head row (packed bf16 words) at destination row dst_row.
    auto append_fp8 = [&](const uint4& lo_v, const uint4& hi_v, uint8_t* cache, float* scale, long long dst_row) {
        const uint32_t w[8] = {lo_v.x, lo_v.y, lo_v.z, lo_v.w, hi_v.x, hi_v.y, hi_v.z, hi_v.w};
        __nv_bfloat162 m = __habs2(*reinterpret_cast<const __nv_bfloat162*>(&w[0]));
#pragma unroll
        for (int k = 1; k < 8; ++k) m = __hmax2(m, __habs2(*reinterpret_cast<const __nv_bfloat162*>(&w[k])));   // skips NaN like fmaxf
        const uint32_t mw = *reinterpret_cast<const uint32_t*>(&m);
        float amax = fmaxf(fmaxf(bf_lo(mw), bf_hi(mw)), 0.0f);
        amax = group_max<kLanesPerHead>(amax);
        const float2 inv2 = splat2(quant_inv_scale<448>(amax));
        if (sub == 0) scale[dst_row] = quant_scale<448>(amax);
        uint32_t c[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float2 p0 = mul2_rn(bf2_to_f2(w[2 * k]), inv2), p1 = mul2_rn(bf2_to_f2(w[2 * k + 1]), inv2);
            c[k] = static_cast<uint32_t>(__nv_cvt_float2_to_fp8x2(p0, __NV_SATFINITE, __NV_E4M3)) |
                   (static_cast<uint32_t>(__nv_cvt_float2_to_fp8x2(p1, __NV_SATFINITE, __NV_E4M3)) << 16);
        }
        uint2* dst = reinterpret_cast<uint2*>(cache + static_cast<size_t>(dst_row) * D);
        st_vec8(dst + sub, make_uint2(c[0], c[1]));
        st_vec8(dst + sub + kLanesPerHead, make_uint2(c[2], c[3]));
    };

    // One loop over the chunk's groups; the role of a group is warp-uniform.  The rows of the next
    // kDepth groups are always on their way into this warp's slice of shared memory (cp.async, 16 bytes
    // per lane and vector, L2 only), so a warp keeps kDepth KB in flight without holding them in
    // registers; every lane reads back only what it copied itself, so no barrier is involved.
    auto group_src = [&](int g) -> const uint4* {
        const int h = hslot;
        if (g < gq) return static_cast<const uint4*>(p.q) + (static_cast<size_t>(token) * Hq + g * kHeadsPerGroup + h) * kVecsPerRow;
        if (g < gq + gk)
            return static_cast<const uint4*>(p.k_in) + (static_cast<size_t>(token) * Hkv + (g - gq) * kHeadsPerGroup + h) * kVecsPerRow;
        return static_cast<const uint4*>(p.v_in) + (static_cast<size_t>(token) * Hkv + (g - gq - gk) * kHeadsPerGroup + h) * kVecsPerRow;
    };
    extern __shared__ uint4 rope_stage[];                    // [warps][kDepth][lo|hi][32 lanes]
    uint4* mine = rope_stage + static_cast<size_t>(threadIdx.x >> 5) * (kRopeDepth * 64) + lane;
    auto fetch = [&](int g, int slot, uint32_t after) {      // `after`: a value the copy must wait for
        const uint4* src = group_src(g);
        cp_async16(mine + slot * 64, src + sub, after);
        cp_async16(mine + slot * 64 + 32, src + sub + kLanesPerHead, after);
    };
#pragma unroll
    for (int d = 0; d < kRopeDepth; ++d) {
        if (g_begin + d < g_end) fetch(g_begin + d, d, 0u);
        cp_async_commit();
    }
    int slot = 0;
    for (int g = g_begin; g < g_end; ++g) {
        cp_async_wait<kRopeDepth - 1>();
        uint4 lo_v = mine[slot * 64], hi_v = mine[slot * 64 + 32];
        // refill this slot with the group kDepth ahead; the copy is tied to the values just read so it
        // cannot be issued before they have left shared memory
        if (g + kRopeDepth < g_end) fetch(g + kRopeDepth, slot, lo_v.x ^ hi_v.w);
        cp_async_commit();
        slot = (slot + 1 == kRopeDepth) ? 0 : slot + 1;
        if (p.q_bias != nullptr) {               // warp-uniform: the group's role picks the bias tensor
            const uint4* bias = g < gq ? static_cast<const uint4*>(p.q_bias) + static_cast<size_t>(g * kHeadsPerGroup + hslot) * kVecsPerRow
                                : g < gq + gk ? static_cast<const uint4*>(p.k_bias) + static_cast<size_t>((g - gq) * kHeadsPerGroup + hslot) * kVecsPerRow
                                              : static_cast<const uint4*>(p.v_bias) + static_cast<size_t>((g - gq - gk) * kHeadsPerGroup + hslot) * kVecsPerRow;
            lo_v = add_bias_row(lo_v, ld_weight(bias + sub));
            hi_v = add_bias_row(hi_v, ld_weight(bias + sub + kLanesPerHead));
        }

        if (g < gq) {                            // Q: rotate in place
            uint4* rowp = static_cast<uint4*>(p.q) + (static_cast<size_t>(token) * Hq + g * kHeadsPerGroup + hslot) * kVecsPerRow;
            uint4 out_lo, out_hi;
            norm_rotate(lo_v, hi_v, p.q_norm, out_lo, out_hi);
            st_vec(rowp + sub, out_lo);
            st_vec(rowp + sub + kLanesPerHead, out_hi);
        } else if (g < gq + gk) {                // K: rotate, optional bf16 write-back, FP8 append
            const size_t row = static_cast<size_t>(token) * Hkv + (g - gq) * kHeadsPerGroup + hslot;
            uint4 out_lo, out_hi;
            norm_rotate(lo_v, hi_v, p.k_norm, out_lo, out_hi);
            if (p.k_out != nullptr) {
                uint4* dst = static_cast<uint4*>(p.k_out) + row * kVecsPerRow;
                st_vec(dst + sub, out_lo);
                st_vec(dst + sub + kLanesPerHead, out_hi);
            }
            if constexpr (kKV) append_fp8(out_lo, out_hi, p.k_cache, p.k_scale, static_cast<long long>(row) + slot_base);
        } else if constexpr (kKV) {              // V: FP8 append only
            const size_t row = static_cast<size_t>(token) * Hkv + (g - gq - gk) * kHeadsPerGroup + hslot;
            append_fp8(lo_v, hi_v, p.v_cache, p.v_scale, static_cast<long long>(row) + slot_base);
        }
    }
    cp_async_wait<0>();
}

// Any even head_dim <= 256 that is not a multiple of 16: one thread per rotation pair.
__global__ void rope_generic_kernel(__nv_bfloat16* q, __nv_bfloat16* k, const int* positions,
                                    const float* inv_freq, long long total_pairs, int num_q_heads,
                                    int num_kv_heads, int head_dim) {
    const int half = head_dim >> 1;
    const int heads = num_q_heads + num_kv_heads;
    pdl_enter();
    for (long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total_pairs;
         idx += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int i = static_cast<int>(idx % half);
        const long long th = idx / half;
        const int head = static_cast<int>(th % heads);
        const long long token = th / heads;
        float s, c;
        __sincosf(static_cast<float>(positions[token]) * inv_freq[i], &s, &c);
        __nv_bfloat16* row = (head < num_q_heads)
                                 ? q + (token * num_q_heads + head) * head_dim
                                 : k + (token * num_kv_heads + (head - num_q_heads)) * head_dim;
        const float a = __bfloat162float(row[i]);
        const float b = __bfloat162float(row[i + half]);
        float lo, hi;
        rotate(a, b, c, s, lo, hi);
        row[i] = __float2bfloat16(lo);
        row[i + half] = __float2bfloat16(hi);
    }
}

template <int D>
int launch_rope(RopeArgs p, bool norm, bool kv, cudaStream_t stream) {
    constexpr int kHeadsPerGroup = 32 / (D / 16);
    const int rows = p.num_q_heads + (kv ? 2 : 1) * p.num_kv_heads;
    const int groups = (rows + kHeadsPerGroup - 1) / kHeadsPerGroup;
    // Enough warps to fill the machine first; beyond that, fewer and longer warps so the
    // cos/sin of a token are shared by more of its heads.
    const long long target_items = static_cast<long long>(host::num_sms()) * 32;
    long long gpi = (static_cast<long long>(p.seq_len) * groups) / target_items;
    if (gpi < 1) gpi = 1;
    if (gpi > groups) gpi = groups;
    p.groups_per_item = static_cast<int>(gpi);
    p.items_per_token = (groups + p.groups_per_item - 1) / p.groups_per_item;
    const long long items = static_cast<long long>(p.seq_len) * p.items_per_token;
    int warps = host::tuning(host::kRopeWarpsPerCta);
    if (warps <= 0) warps = 4;
    if (warps > 8) warps = 8;
    const long long grid = (items + warps - 1) / warps;
    RH_REQUIRE(grid <= 0x7fffffffLL, RH_ERR_UNSUPPORTED_DIM, "rope: too many rows for one launch");
    const unsigned g = static_cast<unsigned>(grid), b = static_cast<unsigned>(warps * 32);
    const bool aligned = p.num_q_heads % kHeadsPerGroup == 0 && p.num_kv_heads % kHeadsPerGroup == 0;
    if (aligned) {
        const size_t smem = static_cast<size_t>(warps) * kRopeDepth * 64 * sizeof(uint4);   // <= 32 KB
        if (kv) {
            if (norm) host::launch<rope_kv_kernel<D, true, true>>(dim3(g), dim3(b), smem, stream, p);
            else host::launch<rope_kv_kernel<D, false, true>>(dim3(g), dim3(b), smem, stream, p);
        } else {
            if (norm) host::launch<rope_kv_kernel<D, true, false>>(dim3(g), dim3(b), smem, stream, p);
            else host::launch<rope_kv_kernel<D, false, false>>(dim3(g), dim3(b), smem, stream, p);
        }
    } else {
        if (kv) {
            if (norm) host::launch<rope_kv_generic_kernel<D, true, true>>(dim3(g), dim3(b), 0, stream, p);
            else host::launch<rope_kv_generic_kernel<D, false, true>>(dim3(g), dim3(b), 0, stream, p);
        } else {
            if (norm) host::launch<rope_kv_generic_kernel<D, true, false>>(dim3(g), dim3(b), 0, stream, p);
            else host::launch<rope_kv_generic_kernel<D, false, false>>(dim3(g), dim3(b), 0, stream, p);
        }
    }
    return host::check_launch("rope_kv_kernel");
}

int dispatch_rope(const RopeArgs& p, int head_dim, bool norm, bool kv, cudaStream_t stream) {
    switch (head_dim) {
        case 16: return launch_rope<16>(p, norm, kv, stream);
        case 32: return launch_rope<32>(p, norm, kv, stream);
        case 64: return launch_rope<64>(p, norm, kv, stream);
        case 128: return launch_rope<128>(p, norm, kv, stream);
        case 256: return launch_rope<256>(p, norm, kv, stream);
        default: return -1;
    }
}

int check_rope(const char* who, int seq_len, int hq, int hkv, int d) {
    RH_REQUIRE(seq_len >= 1, RH_ERR_INVALID_ARG, "%s: seq_len must be >= 1", who);
    RH_REQUIRE(hq >= 1, RH_ERR_INVALID_ARG, "%s: num_q_heads must be >= 1", who);
    RH_REQUIRE(hkv >= 1, RH_ERR_INVALID_ARG, "%s: num_kv_heads must be >= 1", who);
    RH_REQUIRE(d >= 2, RH_ERR_UNSUPPORTED_DIM, "%s: head_dim must be >= 2", who);
    RH_REQUIRE(d % 2 == 0, RH_ERR_UNSUPPORTED_DIM, "%s: head_dim must be even", who);
    RH_REQUIRE(d <= RH_MAX_HEAD_DIM, RH_ERR_UNSUPPORTED_DIM, "%s: head_dim exceeds %d", who, RH_MAX_HEAD_DIM);
    return RH_OK;
}

}  // namespace

}  // namespace rh

using namespace rh;

extern "C" int rh_rope_bf16(void* q, void* k, const int* positions, const float* inv_freq, int seq_len,
                            int num_q_heads, int num_kv_heads, int head_dim, void* stream) {
    if (int e = check_rope("rh_rope_bf16", seq_len, num_q_heads, num_kv_heads, head_dim)) return e;
    RH_REQUIRE(q && k && positions && inv_freq, RH_ERR_INVALID_ARG, "rh_rope_bf16: null pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool fast = (head_dim == 16 || head_dim == 32 || head_dim == 64 || head_dim == 128 || head_dim == 256) &&
                      host::aligned16(q) && host::aligned16(k) && host::aligned16(inv_freq);
    if (fast) {
        RopeArgs p{};
        p.q = q; p.k_out = k; p.k_in = k; p.positions = positions; p.inv_freq = inv_freq;
        p.seq_len = seq_len; p.num_q_heads = num_q_heads; p.num_kv_heads = num_kv_heads;
        return dispatch_rope(p, head_dim, false, false, s);
    }
    const long long pairs = static_cast<long long>(seq_len) * (num_q_heads + num_kv_heads) * (head_dim / 2);
    long long grid = (pairs + 255) / 256;
    const long long cap = static_cast<long long>(host::num_sms()) * 16;
    if (grid > cap) grid = cap;
    host::launch<rope_generic_kernel>(dim3(static_cast<unsigned>(grid)), dim3(256), 0, s, 
        static_cast<__nv_bfloat16*>(q), static_cast<__nv_bfloat16*>(k), positions, inv_freq, pairs,
        num_q_heads, num_kv_heads, head_dim);
    return host::check_launch("rope_generic_kernel");
}

extern "C" int rh_rope_kv_fp8(void* q, void* k_out_or_null, const void* k_in, const void* v_in,
                              const void* q_norm_or_null, const void* k_norm_or_null, float eps,
                              const int* positions, const float* inv_freq, uint8_t* k_cache,
                              float* k_scale, uint8_t* v_cache, float* v_scale, const int* at_pos,
                              int seq_len, int num_q_heads, int num_kv_heads, int head_dim,
                              void* stream) {
    if (int e = check_rope("rh_rope_kv_fp8", seq_len, num_q_heads, num_kv_heads, head_dim)) return e;
    RH_REQUIRE(q && k_in && v_in && positions && inv_freq && k_cache && k_scale && v_cache && v_scale,
               RH_ERR_INVALID_ARG, "rh_rope_kv_fp8: null pointer");
    RH_REQUIRE(at_pos != nullptr, RH_ERR_INVALID_ARG, "rh_rope_kv_fp8: at_pos must not be null");
    const bool norm = q_norm_or_null != nullptr || k_norm_or_null != nullptr;
    RH_REQUIRE(!norm || (q_norm_or_null && k_norm_or_null), RH_ERR_INVALID_ARG,
               "rh_rope_kv_fp8: q_norm and k_norm must be given together");
    RH_REQUIRE(!norm || eps > 0.0f, RH_ERR_INVALID_ARG, "rh_rope_kv_fp8: eps must be > 0");
    RH_REQUIRE(head_dim == 16 || head_dim == 32 || head_dim == 64 || head_dim == 128 || head_dim == 256,
               RH_ERR_UNSUPPORTED_DIM, "rh_rope_kv_fp8: head_dim must be 16, 32, 64, 128 or 256 (got %d)", head_dim);
    RH_REQUIRE(host::aligned16(q) && host::aligned16(k_out_or_null) && host::aligned16(k_in) &&
                   host::aligned16(v_in) && host::aligned16(q_norm_or_null) && host::aligned16(k_norm_or_null) &&
                   host::aligned16(inv_freq) && (reinterpret_cast<uintptr_t>(k_cache) & 7u) == 0 &&
                   (reinterpret_cast<uintptr_t>(v_cache) & 7u) == 0,
               RH_ERR_MISALIGNED, "rh_rope_kv_fp8: pointers must be 16-byte aligned (caches: 8)");
    RopeArgs p{q, k_out_or_null, k_in, v_in, q_norm_or_null, k_norm_or_null, eps, positions, inv_freq,
               k_cache, k_scale, v_cache, v_scale, at_pos, seq_len, num_q_heads, num_kv_heads, 0, 0,
               nullptr, nullptr, nullptr};
    return dispatch_rope(p, head_dim, norm, true, static_cast<cudaStream_t>(stream));
}

extern "C" int rh_bias_rope_kv_fp8(void* q, void* k_out_or_null, const void* k_in, const void* v_in, const void* q_bias,
                                   const void* k_bias, const void* v_bias, const int* positions, const float* inv_freq,
                                   uint8_t* k_cache, float* k_scale, uint8_t* v_cache, float* v_scale,
                                   const int* at_pos, int seq_len, int num_q_heads, int num_kv_heads, int head_dim,
                                   void* stream) {
    const char* const fn = "rh_bias_rope_kv_fp8";
    if (int e = check_rope(fn, seq_len, num_q_heads, num_kv_heads, head_dim)) return e;
    RH_REQUIRE(q && k_in && v_in && positions && inv_freq && k_cache && k_scale && v_cache && v_scale,
               RH_ERR_INVALID_ARG, "%s: null pointer", fn);
    RH_REQUIRE(q_bias && k_bias && v_bias, RH_ERR_INVALID_ARG, "%s: the three biases must be given", fn);
    RH_REQUIRE(at_pos != nullptr, RH_ERR_INVALID_ARG, "%s: at_pos must not be null", fn);
    RH_REQUIRE(head_dim == 16 || head_dim == 32 || head_dim == 64 || head_dim == 128 || head_dim == 256,
               RH_ERR_UNSUPPORTED_DIM, "%s: head_dim must be 16, 32, 64, 128 or 256 (got %d)", fn, head_dim);
    RH_REQUIRE(host::aligned16(q) && host::aligned16(k_out_or_null) && host::aligned16(k_in) && host::aligned16(v_in) &&
                   host::aligned16(q_bias) && host::aligned16(k_bias) && host::aligned16(v_bias) &&
                   host::aligned16(inv_freq) && (reinterpret_cast<uintptr_t>(k_cache) & 7u) == 0 &&
                   (reinterpret_cast<uintptr_t>(v_cache) & 7u) == 0,
               RH_ERR_MISALIGNED, "%s: pointers must be 16-byte aligned (caches: 8)", fn);
    RopeArgs p{q, k_out_or_null, k_in, v_in, nullptr, nullptr, 1.0f, positions, inv_freq,
               k_cache, k_scale, v_cache, v_scale, at_pos, seq_len, num_q_heads, num_kv_heads, 0, 0,
               q_bias, k_bias, v_bias};
    return dispatch_rope(p, head_dim, false, true, static_cast<cudaStream_t>(stream));
}
