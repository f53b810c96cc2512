// rh_selftest_static: the exhaustive self-check of rh_selftest for callers that must not touch the
// device allocator.
//
// Who that is: an inference engine of the reference's kind sizes its weight slab, scratch arena and
// KV cache once at start-up and then owns (nearly) all of the GPU's memory; from then on a cudaMalloc
// — which rh_selftest needs for its eight mismatch counters — can fail outright, and when it succeeds
// it stalls the whole device while the driver updates its page tables.  A health probe that such an
// engine runs between requests therefore wants the check without an allocation.  Here the counters
// live in a fixed array that is part of the library image itself.
//
// Consequences of that choice, all of which the caller has to know:
//  * the array costs RH_SELFTEST_MAX_COUNTERS * 4 bytes (rounded up to 256) of device memory on every
//    GPU that loads the library, from load until the process exits;
//  * it is one array per device, shared by every call: it still holds the previous call's counts,
//    so each call zeroes it on `stream` before the kernel runs, and two calls whose GPU work overlaps
//    (different streams, different threads) write the same counters and corrupt each other's result —
//    serialise them;
//  * the first call on each device looks the array's device address up (cudaGetSymbolAddress) and
//    keeps it; make that first call during start-up, before any stream capture begins.
#include <atomic>
#include <mutex>

#include "rh_common.cuh"

namespace rh {
namespace {

// Scratch: one counter per checked sequence.  In host code this name is only a handle for the
// runtime's symbol lookup — it is never passed to a kernel as a pointer.
static __device__ __align__(256) unsigned int g_selftest_counters[RH_SELFTEST_MAX_COUNTERS];

// Same checks as the allocating self-test's kernel (selftest_checks: every bf16 gate through the refined
// sigmoid reciprocals, every non-negative bf16 amax through the four scale divisions).
__global__ void selftest_static_kernel(unsigned int* counters, int num_counters) {
    selftest_checks(blockIdx.x * blockDim.x + threadIdx.x, [&](int slot) {
        if (slot < num_counters) atomicAdd(&counters[slot], 1u);
    });
}

constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
unsigned int* g_counters_dev[kMaxDevices] = {};   // device address of g_selftest_counters, per device

// Device address of the scratch array on the current device, looked up on first use.
int scratch_address(unsigned int** out) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices)
        return host::fail(RH_ERR_CUDA, "rh_selftest_static: no usable current device");
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (g_counters_dev[dev] == nullptr) {
        unsigned int* ptr = nullptr;
        const cudaError_t err = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_selftest_counters);
        if (err != cudaSuccess || ptr == nullptr)
            return host::fail(RH_ERR_CUDA, "rh_selftest_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(err));
        g_counters_dev[dev] = ptr;
    }
    *out = g_counters_dev[dev];
    return RH_OK;
}

}  // namespace
}  // namespace rh

using namespace rh;

extern "C" int rh_selftest_static(unsigned int* mismatches_host, int num_counters, void* stream) {
    RH_REQUIRE(mismatches_host != nullptr, RH_ERR_INVALID_ARG, "rh_selftest_static: null pointer");
    RH_REQUIRE(num_counters >= 1, RH_ERR_INVALID_ARG, "rh_selftest_static: num_counters must be >= 1 (got %d)", num_counters);
    RH_REQUIRE(num_counters <= RH_SELFTEST_MAX_COUNTERS, RH_ERR_UNSUPPORTED_DIM,
               "rh_selftest_static: num_counters %d exceeds the fixed scratch of %d counters", num_counters,
               RH_SELFTEST_MAX_COUNTERS);
    unsigned int* counters = nullptr;
    if (int e = scratch_address(&counters)) return e;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const size_t bytes = static_cast<size_t>(num_counters) * sizeof(unsigned int);
    cudaError_t err = cudaMemsetAsync(counters, 0, bytes, s);   // the array still holds the last call's counts
    if (err != cudaSuccess) return host::fail(RH_ERR_CUDA, "rh_selftest_static: memset: %s", cudaGetErrorString(err));
    selftest_static_kernel<<<256, 256, 0, s>>>(counters, num_counters);
    if (int e = host::check_launch("selftest_static_kernel")) return e;
    err = cudaMemcpyAsync(mismatches_host, counters, bytes, cudaMemcpyDeviceToHost, s);
    if (err == cudaSuccess) err = cudaStreamSynchronize(s);
    if (err != cudaSuccess) return host::fail(RH_ERR_CUDA, "rh_selftest_static: %s", cudaGetErrorString(err));
    return RH_OK;
}
