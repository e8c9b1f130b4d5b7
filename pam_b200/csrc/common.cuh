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

}  // namespace pamk
