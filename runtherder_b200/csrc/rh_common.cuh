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

// Prefetch rings: each thread streams the vectors it will need into its own shared-memory slots with
// cp.async and reads back only what it copied itself, so no barrier is involved and the bytes in
// flight are set by the ring depth, not by registers.
// 16-byte asynchronous global -> shared copy (L2 only).  `after` is an unused input that orders the
// copy behind the instruction that produced it.
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src, uint32_t after) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst))),
                 "l"(gmem_src), "r"(after)
                 : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int kPending>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(kPending) : "memory");
}

// ---- bf16 <-> fp32 -------------------------------------------------------------------------

__device__ __forceinline__ float bf_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
    f[0] = bf_lo(v.x); f[1] = bf_hi(v.x);
    f[2] = bf_lo(v.y); f[3] = bf_hi(v.y);
    f[4] = bf_lo(v.z); f[5] = bf_hi(v.z);
    f[6] = bf_lo(v.w); f[7] = bf_hi(v.w);
}

// Blackwell issues two independent IEEE fp32 operations per instruction on a register pair
// (FMUL2 / FADD2 / FFMA2); each half rounds exactly like the scalar instruction, so results do
// not change — only the number of issue slots does.  A packed bf16 word maps onto one pair.
// They are issued through PTX with an explicit .rn.  Beware: a paired multiply feeding a paired add
// is merged into a paired fused multiply-add regardless (intrinsics and PTX alike), so no code here
// lets a mul2_rn result flow straight into an add2_rn where the double rounding matters.
// The register pairs are formed inside the asm block (mov.b64 of two 32-bit registers), which costs no
// instruction; building the 64-bit operand with shifts and ors in C++ leaves it to the optimiser.
__device__ __forceinline__ float2 mul2_rn(float2 a, float2 b) {
    float2 d;
    asm("{\n\t.reg .b64 ra, rb, rd;\n\t"
        "mov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\t"
        "mul.rn.f32x2 rd, ra, rb;\n\t"
        "mov.b64 {%0, %1}, rd;\n\t}"
        : "=f"(d.x), "=f"(d.y)
        : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
    return d;
}
__device__ __forceinline__ float2 add2_rn(float2 a, float2 b) {
    float2 d;
    asm("{\n\t.reg .b64 ra, rb, rd;\n\t"
        "mov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\t"
        "add.rn.f32x2 rd, ra, rb;\n\t"
        "mov.b64 {%0, %1}, rd;\n\t}"
        : "=f"(d.x), "=f"(d.y)
        : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
    return d;
}
__device__ __forceinline__ float2 fma2_rn(float2 a, float2 b, float2 c) {
    float2 d;
    asm("{\n\t.reg .b64 ra, rb, rc, rd;\n\t"
        "mov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\tmov.b64 rc, {%6, %7};\n\t"
        "fma.rn.f32x2 rd, ra, rb, rc;\n\t"
        "mov.b64 {%0, %1}, rd;\n\t}"
        : "=f"(d.x), "=f"(d.y)
        : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y), "f"(c.x), "f"(c.y));
    return d;
}
__device__ __forceinline__ float2 bf2_to_f2(uint32_t w) { return make_float2(bf_lo(w), bf_hi(w)); }
__device__ __forceinline__ float2 splat2(float v) { return make_float2(v, v); }
__device__ __forceinline__ float2 neg2(float2 v) { return make_float2(-v.x, -v.y); }

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
// m = max(m, |w|) on both halves, NaN-propagating; written with the intrinsics so the absolute value
// can ride on the max instruction as an operand modifier.
__device__ __forceinline__ uint32_t amax_acc_bf16x2(uint32_t m, uint32_t w) {
    __nv_bfloat162 r = __hmax2_nan(*reinterpret_cast<__nv_bfloat162*>(&m), __habs2(*reinterpret_cast<__nv_bfloat162*>(&w)));
    return *reinterpret_cast<uint32_t*>(&r);
}

// INT8 code of p = y*inv without the conversion unit: adding 1.5*2^23 leaves
// round_half_even(p) in the low mantissa byte (two's complement).  |p| <= 127.0001 for a
// finite row, so the reference's clamp never engages; valid only for finite p.
// The reference rounds twice (the product, then the conversion), so the addition must see the ROUNDED
// product: a paired add directly behind a paired multiply gets merged into one fused multiply-add
// (even with explicit .rn on both), whose single rounding breaks exact .5 ties (y = amax/2 gives 63.5
// -> must round to 64, not 63).  The sequence below keeps both roundings and stays paired: the product
// is taken with 4*inv (an exact scaling, so it rounds like y*inv), and the addition is a fused
// multiply-add by 0.25 (exact) — a multiply cannot be merged into another multiply's operand.
// `inv4` is 4*inv; callers check that it did not overflow.
__device__ __forceinline__ float2 int8_code_fast2(uint32_t w, float2 inv4) {
    return fma2_rn(mul2_rn(bf2_to_f2(w), inv4), splat2(0.25f), splat2(12582912.0f));
}
__device__ __forceinline__ uint2 pack_int8x8_fast4(const uint4& w, float2 inv4) {
    const float2 c0 = int8_code_fast2(w.x, inv4), c1 = int8_code_fast2(w.y, inv4);
    const float2 c2 = int8_code_fast2(w.z, inv4), c3 = int8_code_fast2(w.w, inv4);
    const uint32_t lo = __byte_perm(__byte_perm(__float_as_uint(c0.x), __float_as_uint(c0.y), 0x0040),
                                    __byte_perm(__float_as_uint(c1.x), __float_as_uint(c1.y), 0x0040), 0x5410);
    const uint32_t hi = __byte_perm(__byte_perm(__float_as_uint(c2.x), __float_as_uint(c2.y), 0x0040),
                                    __byte_perm(__float_as_uint(c3.x), __float_as_uint(c3.y), 0x0040), 0x5410);
    return make_uint2(lo, hi);
}
// Largest inverse scale the paired sequence takes (4*inv must stay finite).
constexpr float kFastInvMax = 8.0e37f;
__device__ __forceinline__ uint2 pack_int8x8_fast(const uint4& w, float inv) {
    return pack_int8x8_fast4(w, splat2(inv * 4.0f));
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

// ---- correctly rounded divisions without the division subroutine ------------------------------
//
// The reference computes scale = amax / qmax and inv = qmax / amax with IEEE division, and the
// sigmoid as 1.0f / (1.0f + e).  nvcc's division is a reciprocal approximation, refinement steps,
// a range check and a branch to a slow path.  The sequences below give the same correctly rounded
// results for the operand ranges that occur (amax is a bf16 value, qmax is 127 or 448; d = 1 + e >= 1)
// — rh_selftest() proves it exhaustively on the device it runs on — and fall back to `/` outside.

__device__ __forceinline__ float rcp_approx(float x) {
    float r;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}
// a / b from an approximate reciprocal r of b: quotient, exact remainder, correction (twice).
__device__ __forceinline__ float div_refine(float a, float b, float r) {
    float q = a * r;
    q = __fmaf_rn(__fmaf_rn(-b, q, a), r, q);
    q = __fmaf_rn(__fmaf_rn(-b, q, a), r, q);
    return q;
}
template <int kQMax>
__device__ __forceinline__ float quant_inv_scale(float amax) {   // kQMax / amax, 0 for a zero row
    constexpr float qmax = static_cast<float>(kQMax);
    if (amax >= 1.0e-30f && amax <= 1.0e30f) return div_refine(qmax, amax, rcp_approx(amax));
    return (amax > 0.0f) ? (qmax / amax) : 0.0f;
}
template <int kQMax>
__device__ __forceinline__ float quant_scale(float amax) {       // amax / kQMax
    constexpr float qmax = static_cast<float>(kQMax);
    if (amax >= 1.0e-30f && amax <= 1.0e30f) return div_refine(amax, qmax, 1.0f / qmax);
    return amax / qmax;
}
// sigmoid of two gates, s = 1 / (1 + e), e = __expf(-g) = ex2.approx.ftz(-g * log2(e)), with the
// reciprocal refined kSteps times.  Valid for g >= kGateExactBelow (1 + e stays far below the range
// where its reciprocal turns subnormal); callers send smaller gates down the IEEE-division path.
constexpr float kGateExactBelow = -85.0f;
__device__ __forceinline__ float ex2_approx(float x) {
    float r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}
template <int kSteps>
__device__ __forceinline__ float2 sigmoid2(float2 g) {
    const float2 t = mul2_rn(g, splat2(-1.4426950408889634f));
    const float2 e = make_float2(ex2_approx(t.x), ex2_approx(t.y));
    const float2 d = add2_rn(e, splat2(1.0f));
    const float2 nd = fma2_rn(e, splat2(-1.0f), splat2(-1.0f));   // -(e + 1): one paired op instead of two negations
    float2 r = make_float2(rcp_approx(d.x), rcp_approx(d.y));
    r = fma2_rn(r, fma2_rn(nd, r, splat2(1.0f)), r);
    if (kSteps >= 2) r = fma2_rn(fma2_rn(nd, r, splat2(1.0f)), r, r);
    return r;
}
// The fused kernels use the NEGATED sigmoid: the reciprocal is taken of -(1 + e) (the sign rides on the
// instruction's operand), which makes the refinement r' = r + r * (1 - d * r) two paired fused
// multiply-adds on (d, -r) with no negated copy of d.  Every step is sign-symmetric, so the result is
// exactly -sigmoid2<1>(g); rh_selftest checks it for every gate.  Same validity range as sigmoid2.
// (Letting two or four gates share one reciprocal — seed = reciprocal of the product times the other
// members — was measured too: no faster at full clock, and not exact: over all 3.6e9 ordered pairs of bf16
// gates the pair-shared sigmoid misrounds 306 264 of 7.2e9 halves, which the bf16 rounding of the product
// hides from almost every test.)
__device__ __forceinline__ float2 neg_sigmoid2(float2 g) {
    const float2 t = mul2_rn(g, splat2(-1.4426950408889634f));
    const float2 d = add2_rn(make_float2(ex2_approx(t.x), ex2_approx(t.y)), splat2(1.0f));
    const float2 rn = make_float2(rcp_approx(-d.x), rcp_approx(-d.y));
    return fma2_rn(rn, fma2_rn(d, rn, splat2(1.0f)), rn);
}
// The reference's expression, verbatim (src/kernels/activation.cu:36).
__device__ __forceinline__ float sigmoid_reference(float g) { return 1.0f / (1.0f + __expf(-g)); }

// Exhaustive check of the division-free sequences above against IEEE division, over every operand they
// can meet; `bits` runs over 0..65535 (one thread each) and count(slot) is called per mismatch.
//   0, 1  sigmoid2<1>, sigmoid2<2> against the reference's expression, every bf16 gate >= kGateExactBelow
//   2..5  kQMax/amax and amax/kQMax for 127 and 448, every non-negative bf16 amax
//   6     neg_sigmoid2 (what the fused kernels use) against the negated reference expression
template <typename Count>
__device__ __forceinline__ void selftest_checks(unsigned int bits, Count count) {
    const float g = __uint_as_float(bits << 16);
    if (g >= kGateExactBelow) {   // the range the kernels send down the refined-reciprocal path (NaN excluded)
        const unsigned int want = __float_as_uint(sigmoid_reference(g));
        if (__float_as_uint(sigmoid2<1>(splat2(g)).x) != want) count(0);
        if (__float_as_uint(sigmoid2<2>(splat2(g)).y) != want) count(1);
        const float2 ns = neg_sigmoid2(splat2(g));
        if (__float_as_uint(ns.x) != (want ^ 0x80000000u) || __float_as_uint(ns.y) != (want ^ 0x80000000u)) count(6);
    }
    if (bits <= 0x7f80u) {                                             // +0 .. +Inf
        const float amax = g;
        const float inv127 = (amax > 0.0f) ? (127.0f / amax) : 0.0f, inv448 = (amax > 0.0f) ? (448.0f / amax) : 0.0f;
        if (__float_as_uint(quant_inv_scale<127>(amax)) != __float_as_uint(inv127)) count(2);
        if (__float_as_uint(quant_inv_scale<448>(amax)) != __float_as_uint(inv448)) count(3);
        if (__float_as_uint(quant_scale<127>(amax)) != __float_as_uint(amax / 127.0f)) count(4);
        if (__float_as_uint(quant_scale<448>(amax)) != __float_as_uint(amax / 448.0f)) count(5);
    }
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
// Max of non-negative, non-NaN floats over the warp: their bit patterns order like unsigned
// integers, so one integer warp reduction replaces the five-step shuffle tree.
__device__ __forceinline__ float warp_max_nonneg(float v) {
    return __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(v)));
}
template <int kLanes>
__device__ __forceinline__ float group_max(float v) {
#pragma unroll
    for (int o = kLanes / 2; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Programmatic dependent launch.  Every kernel of this library calls pdl_wait() before its first
// access to global memory: it returns once the preceding kernel of the stream has completed and its
// writes are visible (at once when the launch carried no programmatic attribute).  pdl_trigger()
// lets the following kernel's CTAs be placed on SMs as soon as every CTA of this grid has called it
// or exited; those CTAs then block in their own pdl_wait().  Row-persistent kernels trigger when a
// CTA starts its last row, so that dependents arrive while the tail drains and do not sit on the
// SMs for the whole kernel; one-shot kernels trigger straight after the wait (pdl_enter).
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_enter() {
    pdl_wait();
    pdl_trigger();
}

}  // namespace rh

// ---- host side -----------------------------------------------------------------------------

namespace rh::host {

int fail(int status, const char* fmt, ...);  // records the message for rh_last_error_string
int check_launch(const char* what);           // cudaGetLastError -> RH_ERR_LAUNCH
int num_sms();                                // SM count of the current device (cached per device)
int tuning(int slot);                         // rh_tune value, 0 = use the default
int resident_ctas(const void* kernel, int threads, size_t dyn_smem = 0);  // CTAs per SM (>= 1), uncached query

// One-time set-up of a kernel on the CURRENT device: opts in to `dyn_smem` bytes of dynamic shared memory
// when that exceeds the 48 KB default, and asks how many CTAs of `threads` threads fit on an SM (>= 1).
// The answer is cached per (kernel, device, dyn_smem) behind a mutex, so any host thread may call it for
// any device; after the first call it is a table lookup.  rh_init() makes that first call for every kernel
// the library registered, so that no launch has set-up left to do.
int kernel_setup(const void* kernel, int threads, size_t dyn_smem = 0);
int register_kernel(const void* kernel, int threads, size_t dyn_smem);   // adds to rh_init()'s list; returns 0
int setup_all_registered();                                              // what rh_init() runs on the current device
// Naming KernelAtLoad<&kernel, threads, smem>::token in a launcher registers that instantiation while the
// library is being loaded (a static data member of a class template is initialised at load time once used).
template <auto kKernel, int kThreads, size_t kSmem = 0>
struct KernelAtLoad {
    static inline const int token = register_kernel(reinterpret_cast<const void*>(kKernel), kThreads, kSmem);
};
// The usual launcher prologue: register at load, set up (or look up) on this device.
template <auto kKernel, int kThreads, size_t kSmem = 0>
inline int setup() {
    (void)KernelAtLoad<kKernel, kThreads, kSmem>::token;
    return kernel_setup(reinterpret_cast<const void*>(kKernel), kThreads, kSmem);
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

enum TuneSlot { kRowsCtasPerSm = 0, kSwigluCtasPerSm, kRopeWarpsPerCta, kEmbedCtasPerSm, kElemCtasPerSm, kSwigluRingOff,
                kSwigluRcpSteps, kUnusedB, kSwigluStages, kRowsSmemH, kRowsPrefetch,
                kRowTickets, kNoPdl, kPrefillTiles, kPrefillParts, kTuneSlots };

// Launches kKernel with the programmatic-stream-serialization attribute (unless rh_tune("no_pdl", 1)):
// the kernel may be scheduled while the previous kernel of `stream` drains; it orders itself with
// pdl_enter().  Inside stream capture the edge becomes a programmatic dependency of the graph.
// A failure is left in the runtime's last-error slot for check_launch().  Every kernel launched this
// way is on rh_init()'s list (registered while the library loads), so its code can be made resident
// on a device before the first launch.
template <typename... P, typename... A>
inline void launch_pointer(bool dependent, void (*kernel)(P...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, A&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr = {};
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = (!dependent || tuning(kNoPdl) != 0) ? 0 : 1;
    (void)cudaLaunchKernelEx(&cfg, kernel, static_cast<P>(args)...);
}
template <auto kKernel, typename... A>
inline void launch(dim3 grid, dim3 block, size_t smem, cudaStream_t stream, A&&... args) {
    (void)KernelAtLoad<kKernel, 0, 0>::token;   // threads 0: nothing to set up, only to load
    launch_pointer(true, kKernel, grid, block, smem, stream, static_cast<A&&>(args)...);
}
// The same without the attribute: the kernel starts only when its predecessor in the stream has completed.
template <auto kKernel, typename... A>
inline void launch_plain(dim3 grid, dim3 block, size_t smem, cudaStream_t stream, A&&... args) {
    (void)KernelAtLoad<kKernel, 0, 0>::token;
    launch_pointer(false, kKernel, grid, block, smem, stream, static_cast<A&&>(args)...);
}

}  // namespace rh::host

#define RH_REQUIRE(cond, status, ...)                                 \
    do {                                                              \
        if (!(cond)) return ::rh::host::fail((status), __VA_ARGS__);  \
    } while (0)
