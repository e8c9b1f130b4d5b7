#include "common.cuh"

#include <atomic>

namespace pamk {

static thread_local int g_last_cuda_error = 0;
static std::atomic<long long> g_launches{0};

void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

int record_cuda_error(cudaError_t err) {
    g_last_cuda_error = (int)err;
    return PAMK_ERR_CUDA;
}

int sm_count() {
    static thread_local int cached_device = -1, cached = 148;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return cached;
    if (dev != cached_device) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0) cached = n;
        cached_device = dev;
    }
    return cached;
}

}  // namespace pamk

extern "C" {

const char* pamk_status_string(int status) {
    switch (status) {
        case PAMK_OK: return "ok";
        case PAMK_ERR_ARG: return "invalid argument (null pointer, negative size or unknown enum)";
        case PAMK_ERR_SIZE: return "dimension too large for this kernel";
        case PAMK_ERR_LAYOUT: return "matrix operand has no unit stride";
        case PAMK_ERR_WORKSPACE: return "workspace missing, misaligned or too small";
        case PAMK_ERR_CUDA: return "CUDA error (see pamk_last_cuda_error)";
        default: return "unknown status";
    }
}

int pamk_last_cuda_error(void) { return pamk::g_last_cuda_error; }

int pamk_abi_version(void) { return 1; }

long long pamk_launch_count(void) { return pamk::g_launches.load(std::memory_order_relaxed); }

}
