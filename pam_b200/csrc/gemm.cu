// PAM matrix products for sm_100a.
//
//   C[z][i][j] = sum_k MUL(A[z][i][k], B[z][k][j])
//
// A PAM product is an integer add of the two fp32 bit patterns (minus the exponent bias), so the
// contraction cannot run on the tensor pipes; this is a CUDA-core kernel bounded by instruction
// issue.  The algorithmic cost per multiply-accumulate is one INT32 add and one FP32 add, and the
// kernel is organised so that the common case issues little more than those two:
//
//   * 128x128 output tile per CTA, 256 threads, 8x8 register micro-tile per thread: the operand
//     fetch is four 128-bit shared-memory loads per 64 products;
//   * operands are staged global -> registers -> shared one K-slab (16) ahead of the arithmetic
//     (double-buffered shared memory, one barrier per slab); while they pass through registers
//     the A side is pre-biased (bits - (0x3f800000 - offset)) so that the product is a single
//     add, both sides are laid out [k][row] whatever their layout in global memory (the four
//     row-/column-major combinations of the reference become two loader variants per side), and
//     the exponent range of the slab is recorded;
//   * the reference's per-product range rule (flush below 1e-37, NaN above 1e37 or for
//     inf/NaN; epfml/pam pam/cuda_kernels.cu:24-37) is hoisted: when the recorded exponent ranges
//     prove that every product of the slab is in range, the slab runs the two-instruction loop;
//     otherwise it runs a loop that evaluates the true fp32 product and applies the rule
//     exactly.  Either way every product equals the reference's bit for bit;
//   * each output is summed by one thread, strictly in k order, from +0.0f — the same order as
//     the reference's kernel (cuda_kernels.cu:608-629), so without split-K the sums are
//     bit-identical too.
//
// The same skeleton serves true-multiply products (standard_matmul) and the exact-gradient
// product (pam_matmul_bwd_kernel, cuda_kernels.cu:729-832).
#include "common.cuh"
#include "pam_scalar.cuh"

namespace pamk {
namespace {

constexpr int BM = 128, BN = 128, BK = 16, kThreads = 256;

enum Mode { kPam = 0, kStd = 1, kBwdL = 2, kBwdR = 3 };

// One matrix operand: element (r, k) of batch z lives at p[z*sb + r*sr + k*sk], where r is the
// non-contracted index (row of A / column of B).
struct MatArg {
    const float* p;
    int64_t sb, sr, sk;
};

struct GemmParams {
    MatArg A, B;
    const float* D;           // exact-gradient product only: the operand the slope depends on
    int64_t sDb, sDm, sDn;
    float* C;                 // [batch][M][N], or [split][batch][M][N] partials when splits > 1
    int M, N, K, batch;
    int splits, k_chunk;      // K is cut into `splits` ranges of k_chunk (a multiple of BK)
    int32_t bias_sub;         // 0x3f800000 - offset_bits
    int32_t off;              // offset_bits
};

// Shared-memory column swizzle: rows k and k+8 of a slab are offset by 16 columns so that the
// transposing stores of a K-contiguous operand (a warp writes 16 rows x 2 k-halves) hit 32
// distinct banks.  Groups of four columns stay contiguous for the 128-bit fragment loads.
__device__ __forceinline__ int swz(int col, int k) { return col ^ ((k & 8) << 1); }

// ---- loaders: global -> registers ---------------------------------------------------------------
// KC = operand is contiguous along k (row-major A, or B given as W[N,K]): thread t takes row
// t/2 and eight consecutive k.  Otherwise the operand is contiguous along its row index: thread t
// takes k = t/16 and two groups of four consecutive rows, 64 apart.
// Rows beyond the matrix are clamped to the last valid row (their products land in outputs that
// are never stored); k beyond the range reads as 0.0f, which the range rule turns into +0.
template <bool KC, bool VEC>
__device__ __forceinline__ void load_slab(float (&r)[8], const MatArg& m, const float* base,
                                          int row0, int rows, int k0, int k_end, int tid) {
    if (KC) {
        int row = row0 + (tid >> 1);
        row = row < rows ? row : rows - 1;
        const int k = k0 + (tid & 1) * 8;
        const float* src = base + (int64_t)row * m.sr + k;
        if (VEC) {   // k_end - k0 and K are multiples of 4, pointers 16-byte aligned
            const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
            const float4 v0 = k < k_end ? __ldg(reinterpret_cast<const float4*>(src)) : z;
            const float4 v1 = k + 4 < k_end ? __ldg(reinterpret_cast<const float4*>(src + 4)) : z;
            r[0] = v0.x; r[1] = v0.y; r[2] = v0.z; r[3] = v0.w;
            r[4] = v1.x; r[5] = v1.y; r[6] = v1.z; r[7] = v1.w;
        } else {
#pragma unroll
            for (int c = 0; c < 8; ++c) r[c] = k + c < k_end ? __ldg(src + c) : 0.0f;
        }
    } else {
        const int k = k0 + (tid >> 4);
        const int c0 = row0 + (tid & 15) * 4;
        const bool live = k < k_end;
        const float* src = base + (int64_t)k * m.sk;
        if (VEC) {   // rows % 4 == 0: a group of four is entirely inside or entirely outside
            const int g0 = c0 < rows ? c0 : rows - 4;
            const int g1 = c0 + 64 < rows ? c0 + 64 : rows - 4;
            const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
            const float4 v0 = live ? __ldg(reinterpret_cast<const float4*>(src + g0)) : z;
            const float4 v1 = live ? __ldg(reinterpret_cast<const float4*>(src + g1)) : z;
            r[0] = v0.x; r[1] = v0.y; r[2] = v0.z; r[3] = v0.w;
            r[4] = v1.x; r[5] = v1.y; r[6] = v1.z; r[7] = v1.w;
        } else {
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                int col = c0 + (c & 3) + (c >> 2) * 64;
                col = col < rows ? col : rows - 1;
                r[c] = live ? __ldg(src + col) : 0.0f;
            }
        }
    }
}

// ---- registers -> shared, laid out [k][row] -----------------------------------------------------
template <bool KC>
__device__ __forceinline__ void store_slab(float* s, const float (&r)[8], int tid) {
    if (KC) {
        const int row = tid >> 1, kh = (tid & 1) * 8;
#pragma unroll
        for (int c = 0; c < 8; ++c) s[(kh + c) * BM + swz(row, kh)] = r[c];
    } else {
        const int k = tid >> 4, c0 = (tid & 15) * 4;
        *reinterpret_cast<float4*>(s + k * BM + swz(c0, k)) = make_float4(r[0], r[1], r[2], r[3]);
        *reinterpret_cast<float4*>(s + k * BM + swz(c0 + 64, k)) = make_float4(r[4], r[5], r[6], r[7]);
    }
}

__device__ __forceinline__ void minmax_bits(const float (&r)[8], int& lo, int& hi) {
    lo = 0x7fffffff;
    hi = 0;
#pragma unroll
    for (int c = 0; c < 8; ++c) {
        const int m = f2i(r[c]) & 0x7fffffff;
        lo = min(lo, m);
        hi = max(hi, m);
    }
}

// Which loop a slab may run, from the biased-exponent ranges of its two operands.
//   products of normal finite numbers satisfy 2^(ea+eb-254) <= |a*b| <= 2^(ea+eb-252), so
//   ea+eb >= 132 puts every product above 1e-37 and ea+eb <= 374 keeps it below 1e37.
enum Path { kFast = 0, kChecked = 1 };

__device__ __forceinline__ int classify(int minA, int maxA, int minB, int maxB) {
    const int ea0 = minA >> 23, ea1 = maxA >> 23, eb0 = minB >> 23, eb1 = maxB >> 23;
    const bool fast = ea0 >= 1 && eb0 >= 1 && ea1 <= 254 && eb1 <= 254 && ea0 + eb0 >= 132 && ea1 + eb1 <= 374;
    return fast ? kFast : kChecked;
}

template <int MODE, bool A_KC, bool B_KC, bool VEC>
__global__ void __launch_bounds__(kThreads, MODE == kPam || MODE == kStd ? 2 : 1)
gemm_kernel(const GemmParams p) {
    __shared__ __align__(16) float As[2][BK * BM];
    __shared__ __align__(16) float Bs[2][BK * BN];
    __shared__ int stats[3][4];   // per slab: min/max magnitude bits of A and of B

    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int z = blockIdx.z / p.splits, sp = blockIdx.z - z * p.splits;
    const int k_begin = sp * p.k_chunk;
    const int k_end = min(p.K, k_begin + p.k_chunk);
    const int slabs = (k_end - k_begin + BK - 1) / BK;

    const float* Ab = p.A.p + (int64_t)z * p.A.sb;
    const float* Bb = p.B.p + (int64_t)z * p.B.sb;

    float acc[8][8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = 0.0f;

    // exact-gradient product: per-output constant (mantissa of D + offset) that the slope adds to
    // the other operand's bits (pam_scalar.cuh mul_slope).
    int32_t dm[MODE >= kBwdL ? 8 : 1][MODE >= kBwdL ? 8 : 1];
    if constexpr (MODE >= kBwdL) {
        const float* Db = p.D + (int64_t)z * p.sDb;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            int row = m0 + ty * 4 + (i & 3) + (i >> 2) * 64;
            row = row < p.M ? row : p.M - 1;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                int col = n0 + tx * 4 + (j & 3) + (j >> 2) * 64;
                col = col < p.N ? col : p.N - 1;
                dm[i][j] = iadd(kMant & f2i(__ldg(Db + (int64_t)row * p.sDm + (int64_t)col * p.sDn)), p.off);
            }
        }
    }

    if (MODE == kPam && tid < 12) {
        stats[tid >> 2][tid & 3] = (tid & 1) ? 0 : 0x7fffffff;   // [min, max, min, max]
    }

    float ra[8], rb[8];
    auto stage_store = [&](int buf, int slot) {
        if (MODE == kPam) {
            int lo_a, hi_a, lo_b, hi_b;
            minmax_bits(ra, lo_a, hi_a);
            minmax_bits(rb, lo_b, hi_b);
            lo_a = __reduce_min_sync(0xffffffffu, lo_a);
            hi_a = __reduce_max_sync(0xffffffffu, hi_a);
            lo_b = __reduce_min_sync(0xffffffffu, lo_b);
            hi_b = __reduce_max_sync(0xffffffffu, hi_b);
            if ((tid & 31) == 0) {
                atomicMin(&stats[slot][0], lo_a);
                atomicMax(&stats[slot][1], hi_a);
                atomicMin(&stats[slot][2], lo_b);
                atomicMax(&stats[slot][3], hi_b);
            }
#pragma unroll
            for (int c = 0; c < 8; ++c) ra[c] = i2f(isub(f2i(ra[c]), p.bias_sub));
        }
        store_slab<A_KC>(As[buf], ra, tid);
        store_slab<B_KC>(Bs[buf], rb, tid);
    };

    if (slabs > 0) {
        load_slab<A_KC, VEC>(ra, p.A, Ab, m0, p.M, k_begin, k_end, tid);
        load_slab<B_KC, VEC>(rb, p.B, Bb, n0, p.N, k_begin, k_end, tid);
    }
    __syncthreads();               // stats initialised
    if (slabs > 0) stage_store(0, 0);
    __syncthreads();

    for (int s = 0; s < slabs; ++s) {
        const int buf = s & 1;
        const bool more = s + 1 < slabs;
        if (more) {
            load_slab<A_KC, VEC>(ra, p.A, Ab, m0, p.M, k_begin + (s + 1) * BK, k_end, tid);
            load_slab<B_KC, VEC>(rb, p.B, Bb, n0, p.N, k_begin + (s + 1) * BK, k_end, tid);
        }
        int path = kFast;
        if (MODE == kPam) {
            const int slot = s % 3;
            path = classify(stats[slot][0], stats[slot][1], stats[slot][2], stats[slot][3]);
            // the slot two slabs ahead was last read before the previous barrier: reset it now
            if (tid < 4) stats[(s + 2) % 3][tid] = (tid & 1) ? 0 : 0x7fffffff;
        }
        const float* as = As[buf];
        const float* bs = Bs[buf];

        if (MODE == kPam && path == kFast) {   // (path is kFast for the other modes, which skip this)
#pragma unroll
            for (int kk = 0; kk < BK; ++kk) {
                const int4 a0 = *reinterpret_cast<const int4*>(as + kk * BM + swz(ty * 4, kk));
                const int4 a1 = *reinterpret_cast<const int4*>(as + kk * BM + swz(ty * 4 + 64, kk));
                const int4 b0 = *reinterpret_cast<const int4*>(bs + kk * BN + swz(tx * 4, kk));
                const int4 b1 = *reinterpret_cast<const int4*>(bs + kk * BN + swz(tx * 4 + 64, kk));
                const int a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
                const int b[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
                for (int i = 0; i < 8; ++i)
#pragma unroll
                    for (int j = 0; j < 8; ++j) acc[i][j] = fadd(acc[i][j], i2f(iadd(a[i], b[j])));
            }
        } else {
#pragma unroll 2
            for (int kk = 0; kk < BK; ++kk) {
                const int4 a0 = *reinterpret_cast<const int4*>(as + kk * BM + swz(ty * 4, kk));
                const int4 a1 = *reinterpret_cast<const int4*>(as + kk * BM + swz(ty * 4 + 64, kk));
                const int4 b0 = *reinterpret_cast<const int4*>(bs + kk * BN + swz(tx * 4, kk));
                const int4 b1 = *reinterpret_cast<const int4*>(bs + kk * BN + swz(tx * 4 + 64, kk));
                const int a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
                const int b[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
                if constexpr (MODE == kPam) {
                    // exact range rule on the true product; a[] holds pre-biased patterns
                    float araw[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) araw[i] = i2f(iadd(a[i], p.bias_sub));
#pragma unroll
                    for (int i = 0; i < 8; ++i)
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            const float mag = fabsf(fmul(araw[i], i2f(b[j])));
                            const float prod = mag <= i2f(kPassBits) ? i2f(iadd(a[i], b[j])) : quiet_nan();
                            if (!(mag <= i2f(kFlushBits))) acc[i][j] = fadd(acc[i][j], prod);
                        }
                } else if constexpr (MODE == kStd) {
#pragma unroll
                    for (int i = 0; i < 8; ++i)
#pragma unroll
                        for (int j = 0; j < 8; ++j) acc[i][j] = __fmaf_rn(i2f(a[i]), i2f(b[j]), acc[i][j]);
                } else {
                    // acc += delta * 2^slope, slope from the non-delta operand and D
#pragma unroll
                    for (int i = 0; i < 8; ++i)
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            const int other = MODE == kBwdL ? b[j] : a[i];
                            const float delta = i2f(MODE == kBwdL ? a[i] : b[j]);
                            acc[i][j] = __fmaf_rn(delta, i2f(kSignExp & iadd(other, dm[i][j])), acc[i][j]);
                        }
                }
            }
        }

        if (more) stage_store(buf ^ 1, (s + 1) % 3);
        __syncthreads();
    }

    // ---- epilogue ----------------------------------------------------------------------------
    float* Cz = p.C + ((int64_t)sp * p.batch + z) * ((int64_t)p.M * p.N);
    const bool vec_out = (p.N & 3) == 0 && aligned16(p.C);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int row = m0 + ty * 4 + (i & 3) + (i >> 2) * 64;
        if (row >= p.M) continue;
        float* crow = Cz + (int64_t)row * p.N;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int col = n0 + tx * 4 + h * 64;
            if (vec_out) {
                if (col < p.N)
                    *reinterpret_cast<float4*>(crow + col) =
                        make_float4(acc[i][h * 4], acc[i][h * 4 + 1], acc[i][h * 4 + 2], acc[i][h * 4 + 3]);
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    if (col + j < p.N) crow[col + j] = acc[i][h * 4 + j];
            }
        }
    }
}

// Adds the split-K partials in split order: C = ((P0 + P1) + P2) + ...
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const float* __restrict__ part, float* __restrict__ C,
                                                            int64_t count, int splits) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += stride) {
        float v = part[i];
        for (int s = 1; s < splits; ++s) v = fadd(v, part[(int64_t)s * count + i]);
        C[i] = v;
    }
}

template <int MODE>
int dispatch(const GemmParams& p, bool a_kc, bool b_kc, bool vec, dim3 grid, cudaStream_t st) {
#define PAMK_LAUNCH(AK, BKC, V) gemm_kernel<MODE, AK, BKC, V><<<grid, kThreads, 0, st>>>(p)
    if (vec) {
        if (a_kc) { if (b_kc) PAMK_LAUNCH(true, true, true); else PAMK_LAUNCH(true, false, true); }
        else      { if (b_kc) PAMK_LAUNCH(false, true, true); else PAMK_LAUNCH(false, false, true); }
    } else {
        if (a_kc) { if (b_kc) PAMK_LAUNCH(true, true, false); else PAMK_LAUNCH(true, false, false); }
        else      { if (b_kc) PAMK_LAUNCH(false, true, false); else PAMK_LAUNCH(false, false, false); }
    }
#undef PAMK_LAUNCH
    return check_launch();
}

// An operand can use 128-bit loads when its base and both non-unit strides keep every group of
// four elements 16-byte aligned and its contiguous extent is a multiple of four.
bool vectorisable(const MatArg& m, bool kc, int rows, int K) {
    if (!aligned16(m.p) || (m.sb & 3)) return false;
    return kc ? ((m.sr & 3) == 0 && (K & 3) == 0) : ((m.sk & 3) == 0 && (rows & 3) == 0);
}

int auto_split(int64_t batch, int64_t M, int64_t N, int64_t K) {
    const int64_t tiles = batch * ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
    const int64_t slots = (int64_t)sm_count() * 2;       // two resident CTAs per SM
    if (tiles * 2 > slots || K < 8 * BK) return 1;         // at least half a wave already
    int64_t s = slots / tiles;
    const int64_t max_by_k = K / (4 * BK);                 // keep >= 4 slabs per range
    if (s > max_by_k) s = max_by_k;
    if (s > 64) s = 64;
    return s < 2 ? 1 : (int)s;
}

int run(int mode, GemmParams p, bool a_kc, bool b_kc, int split_k, void* workspace, size_t workspace_bytes,
        cudaStream_t st) {
    if (p.M == 0 || p.N == 0 || p.batch == 0) return PAMK_OK;
    const int64_t count = (int64_t)p.batch * p.M * p.N;
    if (p.K == 0) {
        const cudaError_t e = cudaMemsetAsync(p.C, 0, count * sizeof(float), st);
        return e == cudaSuccess ? PAMK_OK : record_cuda_error(e);
    }
    int splits = split_k;
    if (splits == 0) {
        splits = auto_split(p.batch, p.M, p.N, p.K);
        if (splits > 1 && (workspace == nullptr || workspace_bytes < (size_t)splits * count * sizeof(float) ||
                           (reinterpret_cast<uintptr_t>(workspace) & 255u)))
            splits = 1;
    }
    if (splits < 1) return PAMK_ERR_ARG;
    const int slabs_total = (p.K + BK - 1) / BK;
    if (splits > slabs_total) splits = slabs_total;
    float* out = p.C;
    if (splits > 1) {
        if (workspace == nullptr || (reinterpret_cast<uintptr_t>(workspace) & 255u) ||
            workspace_bytes < (size_t)splits * count * sizeof(float))
            return PAMK_ERR_WORKSPACE;
        p.C = static_cast<float*>(workspace);
    }
    p.splits = splits;
    p.k_chunk = ((slabs_total + splits - 1) / splits) * BK;
    // ranges that would start beyond K are dropped (can happen after rounding k_chunk up)
    while (p.splits > 1 && (int64_t)(p.splits - 1) * p.k_chunk >= p.K) --p.splits;
    splits = p.splits;
    if (splits == 1) p.C = out;

    const int64_t gx = (p.N + BN - 1) / BN, gy = (p.M + BM - 1) / BM, gz = (int64_t)p.batch * splits;
    if (gy > 65535 || gz > 65535) return PAMK_ERR_SIZE;
    const dim3 grid((unsigned)gx, (unsigned)gy, (unsigned)gz);
    const bool vec = vectorisable(p.A, a_kc, p.M, p.K) && vectorisable(p.B, b_kc, p.N, p.K);
    int rc;
    switch (mode) {
        case kPam: rc = dispatch<kPam>(p, a_kc, b_kc, vec, grid, st); break;
        case kStd: rc = dispatch<kStd>(p, a_kc, b_kc, vec, grid, st); break;
        case kBwdL: rc = dispatch<kBwdL>(p, a_kc, b_kc, vec, grid, st); break;
        default: rc = dispatch<kBwdR>(p, a_kc, b_kc, vec, grid, st); break;
    }
    if (rc != PAMK_OK || splits == 1) return rc;
    const int64_t blocks = (count + 255) / 256;
    const int64_t cap = (int64_t)sm_count() * 8;
    splitk_reduce_kernel<<<(unsigned)(blocks < cap ? blocks : cap), 256, 0, st>>>(
        static_cast<const float*>(workspace), out, count, splits);
    return check_launch();
}

// Validates one operand and reports whether it is contiguous along k.
int operand_layout(const float* ptr, int64_t s_row, int64_t s_k, int rows, int K, bool* kc) {
    if (ptr == nullptr) return PAMK_ERR_ARG;
    if (s_k == 1 || K == 1) { *kc = true; return PAMK_OK; }
    if (s_row == 1 || rows == 1) { *kc = false; return PAMK_OK; }
    return PAMK_ERR_LAYOUT;
}

bool dims_ok(int64_t batch, int64_t M, int64_t N, int64_t K) {
    const int64_t lim = 0x7fffffff - 256;
    return batch >= 0 && M >= 0 && N >= 0 && K >= 0 && batch <= lim && M <= lim && N <= lim && K <= lim;
}

}  // namespace
}  // namespace pamk

using namespace pamk;

extern "C" {

size_t pamk_matmul_workspace_bytes(int64_t batch, int64_t M, int64_t N, int split_k) {
    if (split_k <= 1 || batch <= 0 || M <= 0 || N <= 0) return 0;
    return (size_t)split_k * (size_t)batch * (size_t)M * (size_t)N * sizeof(float);
}

int pamk_matmul_auto_split(int64_t batch, int64_t M, int64_t N, int64_t K) {
    if (batch <= 0 || M <= 0 || N <= 0 || K <= 0) return 1;
    return auto_split(batch, M, N, K);
}

int pamk_matmul(int mul_kind, const float* A, const float* B, float* C,
                int64_t batch, int64_t M, int64_t N, int64_t K,
                int64_t sAb, int64_t sAm, int64_t sAk,
                int64_t sBb, int64_t sBk, int64_t sBn,
                float offset, int split_k, void* workspace, size_t workspace_bytes, void* stream) {
    if (mul_kind != PAMK_MUL_PAM && mul_kind != PAMK_MUL_STANDARD) return PAMK_ERR_ARG;
    if (!dims_ok(batch, M, N, K)) return batch < 0 || M < 0 || N < 0 || K < 0 ? PAMK_ERR_ARG : PAMK_ERR_SIZE;
    if (split_k < 0) return PAMK_ERR_ARG;
    if (batch == 0 || M == 0 || N == 0) return PAMK_OK;
    if (C == nullptr) return PAMK_ERR_ARG;
    GemmParams p{};
    bool a_kc = true, b_kc = true;
    if (K > 0) {
        int rc = operand_layout(A, sAm, sAk, (int)M, (int)K, &a_kc);
        if (rc != PAMK_OK) return rc;
        rc = operand_layout(B, sBn, sBk, (int)N, (int)K, &b_kc);
        if (rc != PAMK_OK) return rc;
    }
    p.A = {A, sAb, sAm, sAk};
    p.B = {B, sBb, sBn, sBk};
    p.C = C;
    p.M = (int)M; p.N = (int)N; p.K = (int)K; p.batch = (int)batch;
    p.off = offset_bits(offset);
    p.bias_sub = isub(kBias, p.off);
    return run(mul_kind == PAMK_MUL_PAM ? kPam : kStd, p, a_kc, b_kc, split_k, workspace, workspace_bytes,
               static_cast<cudaStream_t>(stream));
}

int pamk_matmul_bwd(const float* L, const float* R, const float* D, float* out,
                    int64_t batch, int64_t M, int64_t N, int64_t K,
                    int64_t sLb, int64_t sLm, int64_t sLk,
                    int64_t sRb, int64_t sRk, int64_t sRn,
                    int64_t sDb, int64_t sDm, int64_t sDn,
                    int delta_l, float offset, void* stream) {
    if (!dims_ok(batch, M, N, K)) return batch < 0 || M < 0 || N < 0 || K < 0 ? PAMK_ERR_ARG : PAMK_ERR_SIZE;
    if (batch == 0 || M == 0 || N == 0) return PAMK_OK;
    if (out == nullptr || D == nullptr) return PAMK_ERR_ARG;
    GemmParams p{};
    bool l_kc = true, r_kc = true;
    if (K > 0) {
        int rc = operand_layout(L, sLm, sLk, (int)M, (int)K, &l_kc);
        if (rc != PAMK_OK) return rc;
        rc = operand_layout(R, sRn, sRk, (int)N, (int)K, &r_kc);
        if (rc != PAMK_OK) return rc;
    }
    p.A = {L, sLb, sLm, sLk};
    p.B = {R, sRb, sRn, sRk};
    p.D = D; p.sDb = sDb; p.sDm = sDm; p.sDn = sDn;
    p.C = out;
    p.M = (int)M; p.N = (int)N; p.K = (int)K; p.batch = (int)batch;
    p.off = offset_bits(offset);
    p.bias_sub = isub(kBias, p.off);
    return run(delta_l ? kBwdL : kBwdR, p, l_kc, r_kc, 1, nullptr, 0, static_cast<cudaStream_t>(stream));
}

}
