// C-linkage access to rope_cpu_reference (tests/kernels/test_rope.cpp:41-75),
// compiled from the reference's source where it lies.  Test infrastructure only.
#include <tests/kernels/test_rope.cpp>

#include <chrono>
#include <cstring>

extern "C" double refhost_rope(std::uint16_t* tensor, int start_pos, int seq_len, int num_heads,
                               int head_dim, float theta_base) {
    const std::size_t n = static_cast<std::size_t>(seq_len) * num_heads * head_dim;
    std::vector<__nv_bfloat16> t(n);
    std::memcpy(t.data(), tensor, n * 2);
    const auto t0 = std::chrono::steady_clock::now();
    rope_cpu_reference(t, start_pos, seq_len, num_heads, head_dim, theta_base);
    const auto t1 = std::chrono::steady_clock::now();
    std::memcpy(tensor, t.data(), n * 2);
    return std::chrono::duration<double>(t1 - t0).count();
}
