// Exposes, with C linkage, the host-side reference helpers that live in the
// anonymous namespace of the reference's tests/kernels/test_rmsnorm.cpp
// (rmsnorm_cpu_reference :39-61, rmsnorm_add_cpu_reference :68-97,
// make_bf16_random :19-29).  The reference source is compiled where it lies;
// nothing is copied.  Test infrastructure only.
#include <tests/kernels/test_rmsnorm.cpp>

#include <chrono>
#include <cstring>

#include <cuda_fp8.h>

namespace {
std::vector<__nv_bfloat16> to_vec(const std::uint16_t* p, std::size_t n) {
    std::vector<__nv_bfloat16> v(n);
    std::memcpy(v.data(), p, n * 2);
    return v;
}
double now_s() {
    return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count();
}
}  // namespace

extern "C" {

// returns seconds spent inside the reference function itself
double refhost_rmsnorm(std::uint16_t* y, const std::uint16_t* x, const std::uint16_t* g,
                       int num_tokens, int hidden_dim, float eps) {
    const std::size_t n = static_cast<std::size_t>(num_tokens) * hidden_dim;
    const auto xv = to_vec(x, n);
    const auto gv = to_vec(g, hidden_dim);
    const double t0 = now_s();
    const auto out = rmsnorm_cpu_reference(xv, gv, num_tokens, hidden_dim, eps);
    const double t1 = now_s();
    std::memcpy(y, out.data(), n * 2);
    return t1 - t0;
}

double refhost_rmsnorm_add(std::uint16_t* y, std::uint16_t* h_out, const std::uint16_t* x,
                           const std::uint16_t* residual, const std::uint16_t* g, int num_tokens,
                           int hidden_dim, float eps) {
    const std::size_t n = static_cast<std::size_t>(num_tokens) * hidden_dim;
    const auto xv = to_vec(x, n);
    const auto rv = to_vec(residual, n);
    const auto gv = to_vec(g, hidden_dim);
    const double t0 = now_s();
    const auto out = rmsnorm_add_cpu_reference(xv, rv, gv, num_tokens, hidden_dim, eps);
    const double t1 = now_s();
    std::memcpy(y, out.y.data(), n * 2);
    std::memcpy(h_out, out.h_out.data(), n * 2);
    return t1 - t0;
}

// the tests' input generator: mt19937(seed) + uniform_real_distribution(-scale, scale) -> bf16
void refhost_make_bf16_random(std::uint16_t* out, std::size_t count, float scale, std::uint32_t seed) {
    const auto v = make_bf16_random(count, scale, seed);
    std::memcpy(out, v.data(), count * 2);
}

// CUDA's own host conversions, for pinning the oracle's number formats
std::uint16_t refhost_f32_to_bf16(float f) {
    const __nv_bfloat16 h = __float2bfloat16(f);
    std::uint16_t u;
    std::memcpy(&u, &h, 2);
    return u;
}
float refhost_bf16_to_f32(std::uint16_t u) {
    __nv_bfloat16 h;
    std::memcpy(&h, &u, 2);
    return __bfloat162float(h);
}
std::uint8_t refhost_f32_to_e4m3(float f) {
    const __nv_fp8_e4m3 q(f);
    std::uint8_t u;
    std::memcpy(&u, &q, 1);
    return u;
}
float refhost_e4m3_to_f32(std::uint8_t u) {
    __nv_fp8_e4m3 q;
    std::memcpy(&q, &u, 1);
    return static_cast<float>(q);
}

}  // extern "C"
