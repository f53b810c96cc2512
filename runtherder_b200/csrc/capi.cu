// Host-side plumbing of the C ABI: status strings, the per-thread error message,
// device queries used to size grids, tuning knobs, and the load-time RoPE frequency
// tables (host arithmetic, no GPU).
#include <atomic>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstring>

#include "rh_common.cuh"

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

}  // namespace rh::host

using namespace rh;

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
                                                         "elem_ctas_per_sm"};
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
