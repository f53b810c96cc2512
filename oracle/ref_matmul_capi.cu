// C-linkage entry point onto the reference's own W8A8 linear layer (src/kernels/matmul.cu, compiled
// from where it lies together with src/kernels/quantization.cu into _ref/libref_matmul.so, linked with
// cuBLASLt).  It is the GPU-side oracle for rh_linear_w8a8 / rh_linear_w8a8_prequantized.  Test
// infrastructure only.
#include <cstdint>
#include <memory>

#include <runtherder/kernels/matmul.cuh>

namespace rk = runtherder::kernels;

extern "C" void refmatmul_linear_w8a8(void* y, const void* x, const std::int8_t* weight, const void* w_scale,
                                      std::int8_t* q, float* x_scale, std::int32_t* acc, int m, int n, int k,
                                      void* stream) {
    static std::unique_ptr<rk::Matmul> matmul;   // a cuBLASLt handle and the 32 MiB workspace, built on first use
    if (!matmul) matmul = std::make_unique<rk::Matmul>();
    const rk::W8A8Buffer scratch{q, x_scale, acc};
    matmul->linear_w8a8(static_cast<__nv_bfloat16*>(y), static_cast<const __nv_bfloat16*>(x), weight,
                        static_cast<const __nv_bfloat16*>(w_scale), scratch, m, n, k,
                        static_cast<cudaStream_t>(stream));
}
