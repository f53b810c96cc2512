// C-linkage access to swiglu_cpu_reference (tests/kernels/test_activation.cpp:33-44),
// compiled from the reference's source where it lies.  Test infrastructure only.
#include <tests/kernels/test_activation.cpp>

#include <chrono>
#include <cstring>

extern "C" double refhost_swiglu(std::uint16_t* y, const std::uint16_t* gate, const std::uint16_t* up,
                                 std::size_t n) {
    std::vector<__nv_bfloat16> g(n), u(n);
    std::memcpy(g.data(), gate, n * 2);
    std::memcpy(u.data(), up, n * 2);
    const auto t0 = std::chrono::steady_clock::now();
    const auto out = swiglu_cpu_reference(g, u);
    const auto t1 = std::chrono::steady_clock::now();
    std::memcpy(y, out.data(), n * 2);
    return std::chrono::duration<double>(t1 - t0).count();
}
