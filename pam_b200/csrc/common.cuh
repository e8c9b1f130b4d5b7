// Shared host-side plumbing of the C ABI: status codes, launch checks, grid sizing.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/pam_b200.h"

namespace pamk {

// B200: 148 SMs.  Grid sizes for the memory-bound kernels are multiples of the SM count so the
// last wave is full; the count is read once per device.
int sm_count();

// Records a failed CUDA call for pamk_last_cuda_error() and returns PAMK_ERR_CUDA.
int record_cuda_error(cudaError_t err);

// Counts kernel launches made by this library (read by pamk_launch_count()).
void count_launch();

inline int check_launch() {
    const cudaError_t err = cudaGetLastError();
    count_launch();
    return err == cudaSuccess ? PAMK_OK : record_cuda_error(err);
}

__host__ __device__ inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

#if defined(__CUDACC__)
// Asks the L2 for the `count` floats at p (a row this group of `group` threads will load in its next
// pass), one request per 128-byte line, so that the DRAM reads of the next row are in flight while the
// current one is computed; nothing is held in registers.
__device__ __forceinline__ void prefetch_row_l2(const float* p, int count, int t, int group) {
    for (int c = t * 32; c < count; c += group * 32) asm volatile("prefetch.global.L2 [%0];" ::"l"(p + c));
}
#endif

}  // namespace pamk
