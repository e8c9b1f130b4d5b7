// Column sums of a row-major matrix: out[c] = sum_r X[r][c], ordinary fp32 adds.
//
// This is the bias gradient of a linear layer (the reference leaves it to autograd's sum over the
// token dimension).  Deterministic two-pass reduction: CTAs own a tile of 128 columns and a
// contiguous chunk of rows, their 8 warps walk the chunk with a stride of 8 rows and are added in
// warp order; a second kernel adds the chunks (32 interleaved subsets, then those in order).
// HBM-bound: the matrix is read once.
#include "common.cuh"
#include "pam_scalar.cuh"

namespace pamk {
namespace {

constexpr int kColWarps = 8;
constexpr int kColsPerCta = 128;      // 32 lanes x 4 columns

// partial[chunk][c] = sum over the chunk's rows of X[r][c]
template <bool VEC>
__global__ void __launch_bounds__(kColWarps * 32) column_partial_kernel(const float* __restrict__ X,
                                                                        float* __restrict__ partial, int64_t rows,
                                                                        int cols, int64_t rows_per_chunk) {
    __shared__ float stage[kColWarps][kColsPerCta];
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int c0 = blockIdx.x * kColsPerCta + lane * 4;
    const int64_t r0 = (int64_t)blockIdx.y * rows_per_chunk;
    const int64_t r1 = r0 + rows_per_chunk < rows ? r0 + rows_per_chunk : rows;
    float s[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    for (int64_t r = r0 + wid; r < r1; r += kColWarps) {
        const float* p = X + r * cols + c0;
        if (VEC) {
            if (c0 < cols) {
                const float4 v = __ldg(reinterpret_cast<const float4*>(p));
                s[0] = fadd(s[0], v.x); s[1] = fadd(s[1], v.y); s[2] = fadd(s[2], v.z); s[3] = fadd(s[3], v.w);
            }
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (c0 + j < cols) s[j] = fadd(s[j], __ldg(p + j));
        }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) stage[wid][lane * 4 + j] = s[j];
    __syncthreads();
    if (threadIdx.x < kColsPerCta) {
        const int c = blockIdx.x * kColsPerCta + threadIdx.x;
        float t = stage[0][threadIdx.x];
#pragma unroll
        for (int k = 1; k < kColWarps; ++k) t = fadd(t, stage[k][threadIdx.x]);
        if (c < cols) partial[(int64_t)blockIdx.y * cols + c] = t;
    }
}

// out[c] = sum over chunks of partial[chunk][c].  One CTA per 32 columns; warp j adds the chunks
// j, j + 32, j + 64, ... in that order, then the 32 warp sums are added in warp order.
constexpr int kFinalWarps = 32;
__global__ void __launch_bounds__(kFinalWarps * 32) column_final_kernel(const float* __restrict__ partial,
                                                                        float* __restrict__ out, int chunks, int cols) {
    __shared__ float stage[kFinalWarps][32];
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int c = blockIdx.x * 32 + lane;
    float t = 0.0f;
    if (c < cols) {
#pragma unroll 4
        for (int k = wid; k < chunks; k += kFinalWarps) t = fadd(t, __ldg(partial + (int64_t)k * cols + c));
    }
    stage[wid][lane] = t;
    __syncthreads();
    if (wid == 0 && c < cols) {
        t = stage[0][lane];
#pragma unroll
        for (int k = 1; k < kFinalWarps; ++k) t = fadd(t, stage[k][lane]);
        out[c] = t;
    }
}

// Row chunks: enough CTAs for about four per SM, at least 64 rows each.
int chunks_for(int64_t rows, int64_t cols) {
    const int64_t tiles = (cols + kColsPerCta - 1) / kColsPerCta;
    int64_t want = ((int64_t)sm_count() * 4 + tiles - 1) / tiles;
    const int64_t most = (rows + 63) / 64;
    if (want > most) want = most;
    if (want > 65535) want = 65535;
    return (int)(want < 1 ? 1 : want);
}

}  // namespace
}  // namespace pamk

using namespace pamk;

extern "C" {

size_t pamk_column_sum_workspace_bytes(int64_t rows, int64_t cols) {
    if (rows <= 0 || cols <= 0) return 0;
    return (size_t)chunks_for(rows, cols) * (size_t)cols * sizeof(float);
}

int pamk_column_sum(const float* X, float* out, int64_t rows, int64_t cols, void* workspace, size_t workspace_bytes,
                    void* stream) {
    if (rows < 0 || cols < 0) return PAMK_ERR_ARG;
    if (cols == 0) return PAMK_OK;
    if (out == nullptr || (rows > 0 && X == nullptr)) return PAMK_ERR_ARG;
    if (cols > 0x7fffffff - kColsPerCta) return PAMK_ERR_SIZE;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (rows == 0) {
        const cudaError_t e = cudaMemsetAsync(out, 0, (size_t)cols * sizeof(float), st);
        return e == cudaSuccess ? PAMK_OK : record_cuda_error(e);
    }
    const int chunks = chunks_for(rows, cols);
    if (workspace == nullptr || (reinterpret_cast<uintptr_t>(workspace) & 15u) != 0 ||
        workspace_bytes < (size_t)chunks * (size_t)cols * sizeof(float))
        return PAMK_ERR_WORKSPACE;
    float* partial = static_cast<float*>(workspace);
    const int64_t rows_per_chunk = (rows + chunks - 1) / chunks;
    const dim3 grid((unsigned)((cols + kColsPerCta - 1) / kColsPerCta), (unsigned)chunks);
    if ((cols & 3) == 0 && aligned16(X))
        column_partial_kernel<true><<<grid, kColWarps * 32, 0, st>>>(X, partial, rows, (int)cols, rows_per_chunk);
    else
        column_partial_kernel<false><<<grid, kColWarps * 32, 0, st>>>(X, partial, rows, (int)cols, rows_per_chunk);
    int rc = check_launch();
    if (rc != PAMK_OK) return rc;
    column_final_kernel<<<(unsigned)((cols + 31) / 32), kFinalWarps * 32, 0, st>>>(partial, out, chunks, (int)cols);
    return check_launch();
}

}
