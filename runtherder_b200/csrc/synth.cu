// Device generators for synthetic benchmark and test inputs.  Counter-based: the
// value of element i of tensor (seed, tensor_id) depends on nothing else, so any
// slice can be regenerated on the host bit for bit (integer hashing, then fp32
// arithmetic made of single IEEE operations).
#include "rh_common.cuh"

namespace rh {

namespace {

__host__ __device__ __forceinline__ uint64_t mix64(uint64_t z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
__host__ __device__ __forceinline__ uint64_t stream_key(uint64_t seed, uint64_t tensor_id) {
    return mix64(mix64(seed + 0x9E3779B97F4A7C15ull) ^ (tensor_id * 0xD1B54A32D192ED03ull + 0x632BE59BD9B4E019ull));
}
__device__ __forceinline__ uint64_t draw64(uint64_t key, uint64_t counter) {
    return mix64(key + (counter + 1) * 0x9E3779B97F4A7C15ull);
}

// Irwin-Hall sum of twelve 16-bit uniforms: mean 0, variance 1, exactly representable.
__device__ __forceinline__ float synth_normal(uint64_t key, uint64_t idx) {
    uint32_t s = 0;
#pragma unroll
    for (int k = 0; k < 3; ++k) {
        const uint64_t r = draw64(key, 3 * idx + k);
        s += static_cast<uint32_t>(r & 0xffff) + static_cast<uint32_t>((r >> 16) & 0xffff) +
             static_cast<uint32_t>((r >> 32) & 0xffff) + static_cast<uint32_t>(r >> 48);
    }
    return __fmul_rn(static_cast<float>(static_cast<int32_t>(s) - 6 * 65535), 1.0f / 65536.0f);
}

__global__ void synth_normal_kernel(__nv_bfloat16* out, size_t count, uint64_t key, uint64_t start, float std,
                                    const float* chan_scale, int ncols) {
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < count; i += stride) {
        const uint64_t idx = start + i;
        float v = __fmul_rn(synth_normal(key, idx), std);
        if (chan_scale) v = __fmul_rn(v, chan_scale[idx % static_cast<uint64_t>(ncols)]);
        out[i] = __float2bfloat16(v);
    }
}

__global__ void synth_uniform_kernel(__nv_bfloat16* out, size_t count, uint64_t key, uint64_t start, float lo,
                                     float hi) {
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < count; i += stride) {
        const float u = __fmul_rn(static_cast<float>(static_cast<uint32_t>(draw64(key, start + i) >> 40)),
                                  1.0f / 16777216.0f);
        const float w = __fmul_rn(__fsub_rn(hi, lo), u);
        out[i] = __float2bfloat16(__fadd_rn(lo, w));
    }
}

__global__ void synth_ids_kernel(int32_t* out, size_t count, uint64_t key, uint64_t start, int32_t modulus) {
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < count; i += stride)
        out[i] = static_cast<int32_t>(draw64(key, start + i) % static_cast<uint64_t>(modulus));
}

unsigned synth_grid(size_t count) {
    size_t g = (count + 255) / 256;
    const size_t cap = static_cast<size_t>(host::num_sms()) * 16;
    return static_cast<unsigned>(g < cap ? (g ? g : 1) : cap);
}

}  // namespace

}  // namespace rh

using namespace rh;

extern "C" int rh_synth_normal_bf16(void* out, size_t count, uint64_t seed, uint64_t tensor_id,
                                    uint64_t start, float std, const float* chan_scale, int ncols,
                                    void* stream) {
    RH_REQUIRE(out != nullptr, RH_ERR_INVALID_ARG, "rh_synth_normal_bf16: null pointer");
    RH_REQUIRE(chan_scale == nullptr || ncols >= 1, RH_ERR_INVALID_ARG, "rh_synth_normal_bf16: ncols must be >= 1");
    if (count == 0) return RH_OK;
    synth_normal_kernel<<<synth_grid(count), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<__nv_bfloat16*>(out), count, stream_key(seed, tensor_id), start, std, chan_scale, ncols);
    return host::check_launch("synth_normal_kernel");
}

extern "C" int rh_synth_uniform_bf16(void* out, size_t count, uint64_t seed, uint64_t tensor_id,
                                     uint64_t start, float lo, float hi, void* stream) {
    RH_REQUIRE(out != nullptr, RH_ERR_INVALID_ARG, "rh_synth_uniform_bf16: null pointer");
    if (count == 0) return RH_OK;
    synth_uniform_kernel<<<synth_grid(count), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<__nv_bfloat16*>(out), count, stream_key(seed, tensor_id), start, lo, hi);
    return host::check_launch("synth_uniform_kernel");
}

extern "C" int rh_synth_ids_i32(int32_t* out, size_t count, uint64_t seed, uint64_t tensor_id,
                                uint64_t start, int32_t modulus, void* stream) {
    RH_REQUIRE(out != nullptr, RH_ERR_INVALID_ARG, "rh_synth_ids_i32: null pointer");
    RH_REQUIRE(modulus >= 1, RH_ERR_INVALID_ARG, "rh_synth_ids_i32: modulus must be >= 1");
    if (count == 0) return RH_OK;
    synth_ids_kernel<<<synth_grid(count), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        out, count, stream_key(seed, tensor_id), start, modulus);
    return host::check_launch("synth_ids_kernel");
}
