// C-linkage access to quantize_kv_reference (tests/kernels/test_quantization.cpp:42-62)
// and dequantize_kv_fp8 (include/runtherder/kernels/quantization.cuh:63-66),
// compiled from the reference's sources where they lie.  Test infrastructure only.
#include <tests/kernels/test_quantization.cpp>

#include <chrono>
#include <cstring>

extern "C" {

double refhost_quantize_kv(std::uint8_t* q, float* scale, const std::uint16_t* x, int num_rows,
                           int head_dim) {
    const std::size_t n = static_cast<std::size_t>(num_rows) * head_dim;
    std::vector<__nv_bfloat16> xv(n);
    std::memcpy(xv.data(), x, n * 2);
    const auto t0 = std::chrono::steady_clock::now();
    const KvRef ref = quantize_kv_reference(xv, num_rows, head_dim);
    const auto t1 = std::chrono::steady_clock::now();
    std::memcpy(q, ref.q.data(), n);
    std::memcpy(scale, ref.scale.data(), static_cast<std::size_t>(num_rows) * sizeof(float));
    return std::chrono::duration<double>(t1 - t0).count();
}

float refhost_dequantize_kv_fp8(std::uint8_t qb, float scale) {
    __nv_fp8_e4m3 q;
    std::memcpy(&q, &qb, 1);
    return dequantize_kv_fp8(q, scale);
}

}  // extern "C"
