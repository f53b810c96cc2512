// Host-side plumbing of the C ABI: status strings, the per-thread error message,
// device queries used to size grids, tuning knobs, and the load-time RoPE frequency
// tables (host arithmetic, no GPU).
#include <atomic>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstring>

#include "rh_common.cuh"

#include "rh_pipeline.cuh"

namespace rh {
namespace {
__device__ int g_rh_device_error = 0;
}
}  // namespace rh

namespace rh::host {

namespace {
thread_local char g_last_error[512] = "";
std::atomic<int> g_tuning[kTuneSlots];
constexpr int kMaxDevices = 64;
std::atomic<int> g_sm_count[kMaxDevices];
}  // namespace

int fail(int status, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    std::vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
    va_end(ap);
    return status;
}

int check_launch(const char* what) {
    const cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) return fail(RH_ERR_LAUNCH, "%s: launch failed: %s", what, cudaGetErrorString(err));
    return RH_OK;
}

int num_sms() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return kNumSMs;
    int n = g_sm_count[dev].load(std::memory_order_relaxed);
    if (n > 0) return n;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = kNumSMs;
    g_sm_count[dev].store(n, std::memory_order_relaxed);
    return n;
}

int resident_ctas(const void* kernel, int threads, size_t dyn_smem) {
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, threads, dyn_smem) != cudaSuccess || n < 1) {
        (void)cudaGetLastError();
        n = 1;
    }
    return n;
}

int tuning(int slot) { return g_tuning[slot].load(std::memory_order_relaxed); }

int* device_error_word() {
    static std::atomic<int*> cache[kMaxDevices];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
    int* p = cache[dev].load(std::memory_order_acquire);
    if (p == nullptr) {
        if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_rh_device_error) != cudaSuccess) return nullptr;
        cache[dev].store(p, std::memory_order_release);
    }
    return p;
}

}  // namespace rh::host

namespace rh {
namespace {

// Exhaustive check of the division-free sequences in rh_common.cuh against IEEE division, over every
// operand they can meet: all 65536 bf16 gate values for the sigmoid reciprocal, all non-NaN
// non-negative bf16 values for the quantisation scale and inverse scale.
__global__ void selftest_kernel(unsigned int* mismatches) {
    const unsigned int bits = blockIdx.x * blockDim.x + threadIdx.x;   // 0 .. 65535
    const float g = __uint_as_float(bits << 16);
    if (g >= kGateExactBelow) {   // the range the kernels send down the refined-reciprocal path (NaN excluded)
        const unsigned int want = __float_as_uint(sigmoid_reference(g));
        if (__float_as_uint(sigmoid2<1>(splat2(g)).x) != want) atomicAdd(&mismatches[0], 1u);
        if (__float_as_uint(sigmoid2<2>(splat2(g)).y) != want) atomicAdd(&mismatches[1], 1u);
    }
    if (bits <= 0x7f80u) {                                             // +0 .. +Inf
        const float amax = g;
        const float inv127 = (amax > 0.0f) ? (127.0f / amax) : 0.0f, inv448 = (amax > 0.0f) ? (448.0f / amax) : 0.0f;
        if (__float_as_uint(quant_inv_scale<127>(amax)) != __float_as_uint(inv127)) atomicAdd(&mismatches[2], 1u);
        if (__float_as_uint(quant_inv_scale<448>(amax)) != __float_as_uint(inv448)) atomicAdd(&mismatches[3], 1u);
        if (__float_as_uint(quant_scale<127>(amax)) != __float_as_uint(amax / 127.0f)) atomicAdd(&mismatches[4], 1u);
        if (__float_as_uint(quant_scale<448>(amax)) != __float_as_uint(amax / 448.0f)) atomicAdd(&mismatches[5], 1u);
    }
}

}  // namespace
}  // namespace rh

using namespace rh;

extern "C" int rh_selftest(unsigned int* mismatches_host) {
    RH_REQUIRE(mismatches_host != nullptr, RH_ERR_INVALID_ARG, "rh_selftest: null pointer");
    unsigned int* dev = nullptr;
    if (cudaMalloc(&dev, 8 * sizeof(unsigned int)) != cudaSuccess) return host::fail(RH_ERR_CUDA, "rh_selftest: cudaMalloc failed");
    cudaMemset(dev, 0, 8 * sizeof(unsigned int));
    selftest_kernel<<<256, 256>>>(dev);
    const cudaError_t err = cudaMemcpy(mismatches_host, dev, 8 * sizeof(unsigned int), cudaMemcpyDeviceToHost);
    cudaFree(dev);
    if (err != cudaSuccess) return host::fail(RH_ERR_CUDA, "rh_selftest: %s", cudaGetErrorString(err));
    return RH_OK;
}

namespace rh {
namespace {
// One warp waits on a barrier that nothing will ever complete; the bounded wait must give up, record
// the error and let the kernel return normally.
__global__ void bounded_wait_probe_kernel(int polls, int* error_word, int* gave_up) {
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        pipe::mbar_init(&bar, 1);
        pipe::mbar_init_fence();
    }
    __syncthreads();
    const bool ok = pipe::mbar_wait(&bar, 0, __LINE__, error_word, polls);
    if (threadIdx.x == 0) *gave_up = ok ? 0 : 1;
}
}  // namespace
}  // namespace rh

extern "C" int rh_selfcheck_bounded_wait(int polls, int* gave_up_host, int* error_host) {
    RH_REQUIRE(gave_up_host && error_host, RH_ERR_INVALID_ARG, "rh_selfcheck_bounded_wait: null pointer");
    RH_REQUIRE(polls >= 1 && polls <= (1 << 16), RH_ERR_INVALID_ARG, "rh_selfcheck_bounded_wait: polls must be in 1..65536");
    int* word = host::device_error_word();
    RH_REQUIRE(word != nullptr, RH_ERR_CUDA, "rh_selfcheck_bounded_wait: error word unavailable");
    int* flag = nullptr;
    if (cudaMalloc(&flag, sizeof(int)) != cudaSuccess) return host::fail(RH_ERR_CUDA, "rh_selfcheck_bounded_wait: cudaMalloc failed");
    int saved = 0;
    cudaMemcpy(&saved, word, sizeof(int), cudaMemcpyDeviceToHost);
    cudaMemset(word, 0, sizeof(int));
    cudaMemset(flag, 0, sizeof(int));
    bounded_wait_probe_kernel<<<1, 32>>>(polls, word, flag);
    cudaError_t err = cudaMemcpy(gave_up_host, flag, sizeof(int), cudaMemcpyDeviceToHost);
    if (err == cudaSuccess) err = cudaMemcpy(error_host, word, sizeof(int), cudaMemcpyDeviceToHost);
    cudaMemcpy(word, &saved, sizeof(int), cudaMemcpyHostToDevice);   // the probe leaves the sticky word as it found it
    cudaFree(flag);
    if (err != cudaSuccess) return host::fail(RH_ERR_CUDA, "rh_selfcheck_bounded_wait: %s", cudaGetErrorString(err));
    return RH_OK;
}

extern "C" int rh_device_error(int* error_host) {
    RH_REQUIRE(error_host != nullptr, RH_ERR_INVALID_ARG, "rh_device_error: null pointer");
    int* word = host::device_error_word();
    RH_REQUIRE(word != nullptr, RH_ERR_CUDA, "rh_device_error: error word unavailable");
    const cudaError_t err = cudaMemcpy(error_host, word, sizeof(int), cudaMemcpyDeviceToHost);
    if (err != cudaSuccess) return host::fail(RH_ERR_CUDA, "rh_device_error: %s", cudaGetErrorString(err));
    return RH_OK;
}

extern "C" int rh_version(void) { return 100; }

extern "C" const char* rh_status_string(int status) {
    switch (status) {
        case RH_OK: return "ok";
        case RH_ERR_INVALID_ARG: return "invalid argument";
        case RH_ERR_UNSUPPORTED_DIM: return "unsupported dimension";
        case RH_ERR_MISALIGNED: return "misaligned pointer";
        case RH_ERR_LAUNCH: return "kernel launch failed";
        case RH_ERR_CUDA: return "CUDA runtime call failed";
        default: return "unknown status";
    }
}

extern "C" const char* rh_last_error_string(void) { return host::g_last_error; }

extern "C" int rh_tune(const char* key, int value) {
    static const char* const kNames[host::kTuneSlots] = {"rows_ctas_per_sm", "swiglu_ctas_per_sm",
                                                         "rope_warps_per_cta", "embed_ctas_per_sm",
                                                         "elem_ctas_per_sm", "swiglu_threads",
                                                         "swiglu_rcp_steps", "rows_stages", "swiglu_stages",
                                                         "rows_smem_h", "rows_prefetch", "swiglu_prefetch", "no_pdl", "prefill_tiles", "prefill_parts"};
    RH_REQUIRE(key != nullptr, RH_ERR_INVALID_ARG, "rh_tune: null key");
    for (int i = 0; i < host::kTuneSlots; ++i) {
        if (std::strcmp(key, kNames[i]) == 0) {
            host::g_tuning[i].store(value > 0 ? value : 0, std::memory_order_relaxed);
            return RH_OK;
        }
    }
    return host::fail(RH_ERR_INVALID_ARG, "rh_tune: unknown key '%s'", key);
}

// theta^(-2i/D) evaluated in double and narrowed to float
// (reference: src/model/supported/llama/llama.cu:128-143).
extern "C" int rh_rope_inv_freq_plain(float* out_host, int head_dim, float theta_base) {
    RH_REQUIRE(out_host != nullptr, RH_ERR_INVALID_ARG, "rh_rope_inv_freq_plain: null pointer");
    RH_REQUIRE(head_dim >= 2, RH_ERR_UNSUPPORTED_DIM, "rh_rope_inv_freq_plain: head_dim must be >= 2");
    RH_REQUIRE(head_dim % 2 == 0, RH_ERR_UNSUPPORTED_DIM, "rh_rope_inv_freq_plain: head_dim must be even");
    RH_REQUIRE(theta_base > 0.0f, RH_ERR_INVALID_ARG, "rh_rope_inv_freq_plain: theta_base must be > 0");
    const int half = head_dim / 2;
    for (int i = 0; i < half; ++i) {
        const double exponent = -2.0 * static_cast<double>(i) / static_cast<double>(head_dim);
        out_host[i] = static_cast<float>(std::pow(static_cast<double>(theta_base), exponent));
    }
    return RH_OK;
}

// Llama-3 rescaling: wavelengths longer than orig/low are divided by `factor`, shorter than
// orig/high are kept, the band between is blended (reference:
// src/model/supported/llama/llama3.cu:26-60, all in double on the float table).
extern "C" int rh_rope_inv_freq_llama3(float* out_host, int head_dim, float theta_base, float factor,
                                       float low_freq_factor, float high_freq_factor,
                                       int original_max_position_embeddings) {
    if (int e = rh_rope_inv_freq_plain(out_host, head_dim, theta_base)) return e;
    RH_REQUIRE(high_freq_factor != low_freq_factor, RH_ERR_INVALID_ARG,
               "rh_rope_inv_freq_llama3: high_freq_factor must differ from low_freq_factor");
    const double f_div = static_cast<double>(factor);
    const double low = static_cast<double>(low_freq_factor), high = static_cast<double>(high_freq_factor);
    const double old_len = static_cast<double>(original_max_position_embeddings);
    const double low_wavelen = old_len / low, high_wavelen = old_len / high;
    constexpr double two_pi = 2.0 * 3.14159265358979323846;
    for (int i = 0; i < head_dim / 2; ++i) {
        const double f = static_cast<double>(out_host[i]);
        const double wavelen = two_pi / f;
        double scaled = f;
        if (wavelen > low_wavelen) {
            scaled = f / f_div;
        } else if (wavelen >= high_wavelen) {
            const double smooth = (old_len / wavelen - low) / (high - low);
            scaled = (1.0 - smooth) * (f / f_div) + smooth * f;
        }
        out_host[i] = static_cast<float>(scaled);
    }
    return RH_OK;
}
