// Host-side plumbing of the C ABI: status strings, the per-thread error message,
// device queries used to size grids, tuning knobs, and the load-time RoPE frequency
// tables (host arithmetic, no GPU).
#include <atomic>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <map>
#include <mutex>
#include <tuple>
#include <utility>
#include <vector>

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

namespace {
struct SetupKey {
    const void* kernel;
    int device;
    size_t smem;
    bool operator<(const SetupKey& o) const { return std::tie(kernel, device, smem) < std::tie(o.kernel, o.device, o.smem); }
};
struct Registered {
    const void* kernel;
    int threads;
    size_t smem;
};
std::mutex& setup_mutex() { static std::mutex m; return m; }
std::map<SetupKey, int>& setup_table() { static std::map<SetupKey, int> t; return t; }
std::vector<Registered>& registry() { static std::vector<Registered> r; return r; }
}  // namespace

int kernel_setup(const void* kernel, int threads, size_t dyn_smem) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 1;
    const SetupKey key{kernel, dev, dyn_smem};
    std::lock_guard<std::mutex> lock(setup_mutex());
    auto& table = setup_table();
    const auto it = table.find(key);
    if (it != table.end()) return it->second;
    // Dynamic plus static shared memory beyond 48 KB needs the opt-in.  The attribute is a ceiling on the
    // dynamic part, so it is only ever raised: never below the 48 KB every kernel starts with, never below
    // what an earlier request for this kernel on this device asked for.
    if (dyn_smem > 0) {
        static std::map<std::pair<const void*, int>, size_t> ceiling;
        size_t& have = ceiling[{kernel, dev}];
        const size_t want = dyn_smem > 48 * 1024 ? dyn_smem : 48 * 1024;
        if (want > have) {
            if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(want)) == cudaSuccess)
                have = want;
            else
                (void)cudaGetLastError();
        }
    }
    const int resident = resident_ctas(kernel, threads, dyn_smem);
    table.emplace(key, resident);
    return resident;
}

int register_kernel(const void* kernel, int threads, size_t dyn_smem) {
    std::lock_guard<std::mutex> lock(setup_mutex());
    registry().push_back(Registered{kernel, threads, dyn_smem});
    return 0;
}

int setup_all_registered() {
    std::vector<Registered> list;
    {
        std::lock_guard<std::mutex> lock(setup_mutex());
        list = registry();
    }
    for (const Registered& r : list) {
        if (r.threads > 0) {
            (void)kernel_setup(r.kernel, r.threads, r.smem);
        } else {   // no set-up of its own: asking for its attributes makes the runtime load its code
            cudaFuncAttributes attrs;
            if (cudaFuncGetAttributes(&attrs, r.kernel) != cudaSuccess) (void)cudaGetLastError();
        }
    }
    return static_cast<int>(list.size());
}

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
    selftest_checks(blockIdx.x * blockDim.x + threadIdx.x, [&](int slot) { atomicAdd(&mismatches[slot], 1u); });
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
    if (int e = host::check_launch("selftest_kernel")) {
        cudaFree(dev);
        return e;
    }
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
    // The probe records into a private word, not the sticky per-device one, so an error that a kernel on
    // another stream reports meanwhile is neither lost nor mistaken for the probe's.
    int* scratch = nullptr;   // [0] gave-up flag, [1] the probe's error word
    if (cudaMalloc(&scratch, 2 * sizeof(int)) != cudaSuccess) return host::fail(RH_ERR_CUDA, "rh_selfcheck_bounded_wait: cudaMalloc failed");
    cudaMemset(scratch, 0, 2 * sizeof(int));
    bounded_wait_probe_kernel<<<1, 32>>>(polls, scratch + 1, scratch);
    if (int e = host::check_launch("bounded_wait_probe_kernel")) {
        cudaFree(scratch);
        return e;
    }
    int result[2] = {0, 0};
    const cudaError_t err = cudaMemcpy(result, scratch, sizeof(result), cudaMemcpyDeviceToHost);
    cudaFree(scratch);
    if (err != cudaSuccess) return host::fail(RH_ERR_CUDA, "rh_selfcheck_bounded_wait: %s", cudaGetErrorString(err));
    *gave_up_host = result[0];
    *error_host = result[1];
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

extern "C" int rh_init(int device) {
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess) return host::fail(RH_ERR_CUDA, "rh_init: no CUDA device");
    RH_REQUIRE(device >= 0 && device < count, RH_ERR_INVALID_ARG, "rh_init: device %d out of range (0..%d)", device, count - 1);
    int previous = 0;
    if (cudaGetDevice(&previous) != cudaSuccess) return host::fail(RH_ERR_CUDA, "rh_init: cudaGetDevice failed");
    if (cudaSetDevice(device) != cudaSuccess) return host::fail(RH_ERR_CUDA, "rh_init: cudaSetDevice(%d) failed", device);
    (void)host::num_sms();
    const bool word_ok = host::device_error_word() != nullptr;
    (void)host::setup_all_registered();
    (void)cudaGetLastError();
    (void)cudaSetDevice(previous);
    if (!word_ok) return host::fail(RH_ERR_CUDA, "rh_init: the device error word is unavailable on device %d", device);
    return RH_OK;
}

extern "C" int rh_version(void) { return 101; }

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
                                                         "elem_ctas_per_sm", "swiglu_ring",
                                                         "swiglu_rcp_steps", "(unused)", "swiglu_stages",
                                                         "rows_smem_h", "rows_prefetch", "row_tickets", "no_pdl", "prefill_tiles", "prefill_parts"};
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
