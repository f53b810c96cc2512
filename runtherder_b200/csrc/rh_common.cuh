// Shared device helpers for the row-wise kernels: 128-bit streaming loads and
// stores, bf16 packing, the reduction trees, and the host-side error plumbing.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "rh_kernels.h"

namespace rh {

constexpr int kVec = 8;       // bf16 elements per 128-bit access
constexpr int kNumSMs = 148;  // B200; only used to size grids (the actual count is queried)

// ---- memory access ---------------------------------------------------------------------

// Activations are read once: keep them out of L1.  A plain (coherent) load is
// used rather than the read-only path because several ops run in place.
__device__ __forceinline__ uint4 ld_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
// Read-only data that is touched once (gathered embedding rows): non-coherent path, no L1 line.
__device__ __forceinline__ uint4 ld_stream_ro(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
// Weights (norm gains, frequency table) are re-read by every row: read-only path.
__device__ __forceinline__ uint4 ld_weight(const void* p) {
    return __ldg(reinterpret_cast<const uint4*>(p));
}
__device__ __forceinline__ void st_vec(void* p, uint4 v) { *reinterpret_cast<uint4*>(p) = v; }
__device__ __forceinline__ void st_vec8(void* p, uint2 v) { *reinterpret_cast<uint2*>(p) = v; }

// ---- bf16 <-> fp32 -------------------------------------------------------------------------

__device__ __forceinline__ float bf_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
    f[0] = bf_lo(v.x); f[1] = bf_hi(v.x);
    f[2] = bf_lo(v.y); f[3] = bf_hi(v.y);
    f[4] = bf_lo(v.z); f[5] = bf_hi(v.z);
    f[6] = bf_lo(v.w); f[7] = bf_hi(v.w);
}

// Round-to-nearest-even fp32 -> bf16 of two values, packed (lo in bits 0..15).
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
    return make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]), pack_bf16x2(f[4], f[5]),
                      pack_bf16x2(f[6], f[7]));
}
// The fp32 value of bf16_rn(x): what a later kernel would read back from a stored bf16 tensor.
__device__ __forceinline__ float round_bf16(float x) { return __bfloat162float(__float2bfloat16(x)); }

// ---- quantisation codes ------------------------------------------------------------------

// clamp(round_half_even(p), -127, 127), as the reference's INT8 kernel computes it.
__device__ __forceinline__ int int8_code(float p) { return max(-127, min(127, __float2int_rn(p))); }

__device__ __forceinline__ uint2 pack_int8x8(const float (&y)[8], float inv) {
    uint32_t w[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const uint32_t b0 = static_cast<uint32_t>(int8_code(y[4 * h + 0] * inv)) & 0xffu;
        const uint32_t b1 = static_cast<uint32_t>(int8_code(y[4 * h + 1] * inv)) & 0xffu;
        const uint32_t b2 = static_cast<uint32_t>(int8_code(y[4 * h + 2] * inv)) & 0xffu;
        const uint32_t b3 = static_cast<uint32_t>(int8_code(y[4 * h + 3] * inv)) & 0xffu;
        w[h] = b0 | (b1 << 8) | (b2 << 16) | (b3 << 24);
    }
    return make_uint2(w[0], w[1]);
}

// Packed bf16x2 helpers for the row amax.  The NaN-propagating max reveals, at no extra
// cost, whether a thread holds a non-finite value (the reference's fmaxf skips NaN).
__device__ __forceinline__ uint32_t abs_bf16x2(uint32_t w) { return w & 0x7fff7fffu; }
__device__ __forceinline__ uint32_t max_nan_bf16x2(uint32_t a, uint32_t b) {
    __nv_bfloat162 r = __hmax2_nan(*reinterpret_cast<__nv_bfloat162*>(&a), *reinterpret_cast<__nv_bfloat162*>(&b));
    return *reinterpret_cast<uint32_t*>(&r);
}

// INT8 code of p = y*inv without the conversion unit: adding 1.5*2^23 leaves
// round_half_even(p) in the low mantissa byte (two's complement).  |p| <= 127.0001 for a
// finite row, so the reference's clamp never engages; valid only for finite p.
__device__ __forceinline__ uint32_t int8_code_fast(float y, float inv) {
    return __float_as_uint(__fadd_rn(__fmul_rn(y, inv), 12582912.0f));
}
__device__ __forceinline__ uint2 pack_int8x8_fast(const uint4& w, float inv) {
    const uint32_t c0 = int8_code_fast(bf_lo(w.x), inv), c1 = int8_code_fast(bf_hi(w.x), inv);
    const uint32_t c2 = int8_code_fast(bf_lo(w.y), inv), c3 = int8_code_fast(bf_hi(w.y), inv);
    const uint32_t c4 = int8_code_fast(bf_lo(w.z), inv), c5 = int8_code_fast(bf_hi(w.z), inv);
    const uint32_t c6 = int8_code_fast(bf_lo(w.w), inv), c7 = int8_code_fast(bf_hi(w.w), inv);
    const uint32_t lo = __byte_perm(__byte_perm(c0, c1, 0x0040), __byte_perm(c2, c3, 0x0040), 0x5410);
    const uint32_t hi = __byte_perm(__byte_perm(c4, c5, 0x0040), __byte_perm(c6, c7, 0x0040), 0x5410);
    return make_uint2(lo, hi);
}

// Eight E4M3 codes (round-to-nearest-even, saturate to +-448), the conversion __nv_fp8_e4m3(float) does.
__device__ __forceinline__ uint2 pack_e4m3x8(const float (&y)[8], float inv) {
    uint32_t w[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const uint32_t p0 = __nv_cvt_float2_to_fp8x2(make_float2(y[4 * h + 0] * inv, y[4 * h + 1] * inv),
                                                     __NV_SATFINITE, __NV_E4M3);
        const uint32_t p1 = __nv_cvt_float2_to_fp8x2(make_float2(y[4 * h + 2] * inv, y[4 * h + 3] * inv),
                                                     __NV_SATFINITE, __NV_E4M3);
        w[h] = p0 | (p1 << 16);
    }
    return make_uint2(w[0], w[1]);
}

// ---- reductions ----------------------------------------------------------------------------
//
// The sum-of-squares must reproduce the reference kernel's fp32 summation tree
// bit for bit (rmsnorm.cu:17-42): a shuffle-down tree 16,8,4,2,1 inside each
// warp, then the same tree over the eight warp partials.  A butterfly (xor)
// exchange pairs the same lanes at every level, and fp32 addition commutes, so
// every lane ends with exactly the value the reference's lane 0 holds.

template <int kLanes>
__device__ __forceinline__ float group_sum(float v) {
#pragma unroll
    for (int o = kLanes / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
template <int kLanes>
__device__ __forceinline__ float group_max(float v) {
#pragma unroll
    for (int o = kLanes / 2; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

}  // namespace rh

// ---- host side -----------------------------------------------------------------------------

namespace rh::host {

int fail(int status, const char* fmt, ...);  // records the message for rh_last_error_string
int check_launch(const char* what);           // cudaGetLastError -> RH_ERR_LAUNCH
int num_sms();                                // SM count of the current device (cached per device)
int tuning(int slot);                         // rh_tune value, 0 = use the default
int resident_ctas(const void* kernel, int threads, size_t dyn_smem = 0);  // CTAs per SM (>= 1)

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

enum TuneSlot { kRowsCtasPerSm = 0, kSwigluCtasPerSm, kRopeWarpsPerCta, kEmbedCtasPerSm, kElemCtasPerSm, kTuneSlots };

}  // namespace rh::host

#define RH_REQUIRE(cond, status, ...)                                 \
    do {                                                              \
        if (!(cond)) return ::rh::host::fail((status), __VA_ARGS__);  \
    } while (0)
