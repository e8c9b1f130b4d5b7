// PAM matrix products for sm_100a.
//
//   C[z][i][j] = sum_k MUL(A[z][i][k], B[z][k][j])
//
// A PAM product is an integer add of the two fp32 bit patterns (minus the exponent bias), so the
// contraction cannot run on the tensor pipes; this is a CUDA-core kernel bounded by instruction
// issue.  The algorithmic cost per multiply-accumulate is one INT32 add and one FP32 add, and the
// kernel is organised so that the common case issues little more than those two:
//
//   * 8x8 register micro-tile per thread, 128x128 (256 threads) or 64x64 (64 threads) output
//     tile per CTA chosen per problem so that the tiles spread evenly over the 148 SMs: the
//     operand fetch is four 128-bit shared-memory loads per 64 products;
//   * operands are staged global -> registers -> shared one K-slab (16) ahead of the arithmetic
//     (double-buffered shared memory, one barrier per slab); while they pass through registers
//     the A side is pre-biased (bits - (0x3f800000 - offset)) so that the product is a single
//     add, both sides are laid out [k][row] whatever their layout in global memory (the four
//     row-/column-major combinations of the reference become two loader variants per side), and
//     every element's exponent is tested against the safe band;
//   * the reference's per-product range rule (flush below 1e-37, NaN above 1e37 or for
//     inf/NaN; epfml/pam pam/cuda_kernels.cu:24-37) is hoisted.  A slab whose elements all have their
//     exponent in a band that keeps every product in range runs the two-instruction loop.  In any other
//     slab the choice is made per k line: a line without out-of-band elements still costs two
//     instructions per product; a line whose largest magnitudes cannot multiply beyond the pass range
//     evaluates the true product only to decide "flush or add" (four instructions); only a line
//     that could overflow, or holds an inf / NaN, applies the full three-way rule.  Either way every
//     product equals the reference's bit for bit;
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

enum Mode { kPam = 0, kStd = 1, kBwdL = 2, kBwdR = 3 };

// One matrix operand: element (r, k) of batch z lives at p[(z / inner)*sb + z*sb2 + r*sr + k*sk], where r
// is the non-contracted index (row of A / column of B) and `inner` (GemmParams) is the size of the inner
// batch dimension (1 for a plain batch: the heads of an attention product otherwise).  run() derives
// this form from the caller's (outer stride, inner stride): sb = outer - inner * inner_stride,
// sb2 = inner_stride; with inner = 1, sb = 0 and sb2 = the batch stride.
struct MatArg {
    const float* p;
    int64_t sb, sr, sk;
    int64_t sb2;
};

struct GemmParams {
    MatArg A, B;
    const float* D;           // exact-gradient product only: the operand the slope depends on
    int64_t sDb, sDm, sDn;
    float* C;                 // output, or [split][batch][M][N] partials when splits > 1
    int64_t ldc, sCb, sCb2;   // output row stride and batch strides (outer, inner); columns are contiguous
    int64_t sCsplit;          // distance between the partials of two K ranges
    const float* bias;        // optional [N]: added (ordinary fp32 add) to every output row after its sum
    int post;                 // multiply every finished sum by post_scale (PAM product) before it is stored
    float post_scale;
    int inner;                // size of the inner batch dimension (>= 1)
    unsigned inner_magic;     // floor(2^32 / inner) + 1 (0 when inner = 1): z / inner = umulhi(z, inner_magic)
    int M, N, K, batch;
    int splits, k_chunk;      // K is cut into `splits` ranges of k_chunk (a multiple of the slab)
    int32_t bias_sub;         // 0x3f800000 - offset_bits
    int32_t off;              // offset_bits
};

// Tile shapes.  Every thread owns a square register micro-tile (8x8 unless said otherwise).
//   128x128x16, 256 threads, 2 CTAs/SM: least staging overhead, for large outputs;
//   64x64x8,     64 threads, 8 CTAs/SM: four times as many CTAs, for outputs that would leave a
//                                       large tile grid with a ragged last wave (e.g. 12608 x 192).
template <int BM_, int BN_, int BK_, int CPS_, int MT_ = 8>
struct Tile {
    // every thread owns an MT x MT micro-tile (8, or 4 for the tile meant for very small outputs)
    static constexpr int BM = BM_, BN = BN_, BK = BK_, MT = MT_, kCtasPerSm = CPS_;
    static constexpr int kThreads = (BM_ / MT_) * (BN_ / MT_);
    static constexpr int TX = BN_ / MT_;
    // float4 tasks per thread when staging one operand slab
    static constexpr int kTasksA = BM_ * BK_ / 4 / kThreads, kTasksB = BN_ * BK_ / 4 / kThreads;
    // rows that one warp of the K-contiguous loader covers
    static constexpr int kRowsPerWarp = 32 / (BK_ / 4);
};
using TileLarge = Tile<128, 128, 16, 2>;
using TileSmall = Tile<64, 64, 8, 8>;
// 32x32x8 with a 4x4 micro-tile, 64 threads: batched products whose matrices are a fraction of a
// 64x64 tile (attention over 32 tokens) would otherwise spend three quarters of their adds on
// rows and columns that do not exist.
using TileTiny = Tile<32, 32, 8, 12, 4>;

// Shared-memory layout of a slab: [k][row], rows of R floats padded by four.  The padding spreads
// the transposing stores of a K-contiguous operand (a warp writes kRowsPerWarp rows x BK/4
// k-groups) over the banks, and keeps every fragment address a constant offset from one base so
// that the arithmetic loops carry no address computation (an XOR swizzle measured the same speed
// with more instructions and a few spilled registers).
__host__ __device__ constexpr int row_stride(int R) { return R + 4; }

// ---- loaders: global -> registers ---------------------------------------------------------------
// A slab is R rows x BK k, staged as float4 "tasks"; thread t takes tasks t, t + kThreads, ...
//   KC (operand contiguous along k: row-major A, or B given as W[N,K]):
//       task id -> row id / (BK/4), k-group id % (BK/4): a warp reads kRowsPerWarp rows x 4*BK bytes;
//   otherwise (contiguous along the row index): task id -> k = id / (R/4), four rows (id % (R/4))*4:
//       a warp reads 512 contiguous bytes of one k.
// Rows beyond the matrix are clamped to the last valid row (their products land in outputs that
// are never stored); k beyond the range reads as 0.0f, which the range rule turns into +0.
template <class T, int R, int NT, bool KC, bool VEC>
__device__ __forceinline__ void load_slab(float (&r)[NT * 4], const MatArg& m, const float* base,
                                          int row0, int rows, int k0, int k_end, int tid) {
#pragma unroll
    for (int t = 0; t < NT; ++t) {
        const int id = tid + t * T::kThreads;
        if (KC) {
            int row = row0 + id / (T::BK / 4);
            row = row < rows ? row : rows - 1;
            const int k = k0 + (id % (T::BK / 4)) * 4;
            const float* src = base + (int64_t)row * m.sr + k;
            if (VEC) {   // K and the split ranges are multiples of 4, pointers 16-byte aligned
                const float4 v = k < k_end ? __ldg(reinterpret_cast<const float4*>(src)) : make_float4(0.f, 0.f, 0.f, 0.f);
                r[t * 4] = v.x; r[t * 4 + 1] = v.y; r[t * 4 + 2] = v.z; r[t * 4 + 3] = v.w;
            } else {
#pragma unroll
                for (int c = 0; c < 4; ++c) r[t * 4 + c] = k + c < k_end ? __ldg(src + c) : 0.0f;
            }
        } else {
            const int k = k0 + id / (R / 4);
            const int c0 = row0 + (id % (R / 4)) * 4;
            const bool on = k < k_end;
            const float* src = base + (int64_t)k * m.sk;
            if (VEC) {   // rows % 4 == 0: a group of four is entirely inside or entirely outside
                const int g = c0 < rows ? c0 : rows - 4;
                const float4 v = on ? __ldg(reinterpret_cast<const float4*>(src + g)) : make_float4(0.f, 0.f, 0.f, 0.f);
                r[t * 4] = v.x; r[t * 4 + 1] = v.y; r[t * 4 + 2] = v.z; r[t * 4 + 3] = v.w;
            } else {
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const int col = c0 + c < rows ? c0 + c : rows - 1;
                    r[t * 4 + c] = on ? __ldg(src + col) : 0.0f;
                }
            }
        }
    }
}

// Vectorised loads keep one pointer per task that walks along K, so the per-slab work is the load,
// the range predicate and one pointer increment; the row clamp and the 64-bit address arithmetic
// are done once per kernel.
template <class T, int R, int NT, bool KC>
struct SlabWalker {
    const float* ptr[NT];
    int64_t step;                                    // elements to advance per slab

    __device__ __forceinline__ void init(const MatArg& m, const float* base, int row0, int rows, int k_begin, int tid) {
        step = KC ? (int64_t)T::BK : (int64_t)T::BK * m.sk;
#pragma unroll
        for (int t = 0; t < NT; ++t) {
            const int id = tid + t * T::kThreads;
            if (KC) {
                int row = row0 + id / (T::BK / 4);
                row = row < rows ? row : rows - 1;
                ptr[t] = base + (int64_t)row * m.sr + k_begin + (id % (T::BK / 4)) * 4;
            } else {
                const int c0 = row0 + (id % (R / 4)) * 4;
                ptr[t] = base + (int64_t)(k_begin + id / (R / 4)) * m.sk + (c0 < rows ? c0 : rows - 4);
            }
        }
    }

    __device__ __forceinline__ void load(float (&r)[NT * 4], int k0, int k_end, int tid) {
#pragma unroll
        for (int t = 0; t < NT; ++t) {
            const int id = tid + t * T::kThreads;
            const int k = KC ? k0 + (id % (T::BK / 4)) * 4 : k0 + id / (R / 4);
            const float4 v = k < k_end ? __ldg(reinterpret_cast<const float4*>(ptr[t])) : make_float4(0.f, 0.f, 0.f, 0.f);
            r[t * 4] = v.x; r[t * 4 + 1] = v.y; r[t * 4 + 2] = v.z; r[t * 4 + 3] = v.w;
            ptr[t] += step;
        }
    }
};

// ---- registers -> shared, laid out [k][row] -----------------------------------------------------
template <class T, int R, int NT, bool KC>
__device__ __forceinline__ void store_slab(float* s, const float (&r)[NT * 4], int tid) {
#pragma unroll
    for (int t = 0; t < NT; ++t) {
        const int id = tid + t * T::kThreads;
        if (KC) {
            const int row = id / (T::BK / 4), kg = (id % (T::BK / 4)) * 4;
#pragma unroll
            for (int c = 0; c < 4; ++c) s[(kg + c) * row_stride(R) + row] = r[t * 4 + c];
        } else {
            const int k = id / (R / 4), c0 = (id % (R / 4)) * 4;
            *reinterpret_cast<float4*>(s + k * row_stride(R) + c0) = make_float4(r[t * 4], r[t * 4 + 1], r[t * 4 + 2], r[t * 4 + 3]);
        }
    }
}

// ---- which loop a slab, and each of its k lines, may run ---------------------------------------------
// Products of normal finite numbers satisfy 2^(ea+eb-254) <= |a*b| <= 2^(ea+eb-252) (ea, eb the
// biased exponents), so if both factors have their exponent field in the band [66, 187] the product
// lies in [2^-122, 2^122], inside the reference's pass range (1e-37, 1e37), and the range rule
// (cuda_kernels.cu:24-37) returns the integer sum.  The band test is one three-input add and one
// unsigned max per element: 2 * bits drops the sign, minus twice the band's lower bound makes "below"
// wrap around to huge values.
//   * A slab whose elements are all in the band runs the two-instruction loop.
//   * Otherwise the staging threads that hold out-of-band elements record, per k line, that the line
//     is dirty and whether it holds an element above the band.  A clean line of a dirty slab still
//     costs two instructions per product.
//   * A dirty line evaluates the true fp32 product.  It can skip the overflow test when the largest
//     magnitudes of its two operand lines cannot multiply beyond 1e37 and neither holds an inf / NaN
//     (|a * b| rounded grows with |a| and |b|, so the two maxima bound every product of the line):
//     four instructions per product, "flush or add".  Only the remaining lines apply the full rule.
enum Path { kFast = 0, kFlush = 1, kFull = 2 };

constexpr uint32_t kBandLo2 = 2u * (66u << 23);                // 2 * smallest in-band magnitude
constexpr uint32_t kBandSpan2 = 2u * ((188u - 66u) << 23);     // in band iff 2*bits - kBandLo2 < span
constexpr uint32_t kBandHi2 = 2u * (188u << 23);               // 2 * smallest magnitude above the band

template <int N>
__device__ __forceinline__ uint32_t band_excess(const float (&r)[N], uint32_t vmax) {
#pragma unroll
    for (int c = 0; c < N; ++c) {
        const uint32_t b = (uint32_t)f2i(r[c]);
        vmax = max(vmax, b + b - kBandLo2);
    }
    return vmax;
}

// Position of element c of staging task `id` inside the slab: its k line.
template <class T, int R, bool KC>
__device__ __forceinline__ int slab_line(int id, int c) {
    return KC ? (id % (T::BK / 4)) * 4 + c : id / (R / 4);
}

// k lines of this thread's staged elements that hold an out-of-band element (low 16 bits) and an
// element above the band (bits 16..31).
template <class T, int R, int NT, bool KC>
__device__ __forceinline__ unsigned dirty_lines(const float (&r)[NT * 4], int tid) {
    unsigned lines = 0;
#pragma unroll
    for (int t = 0; t < NT; ++t)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const uint32_t b = (uint32_t)f2i(r[t * 4 + c]);
            const uint32_t m2 = b + b;
            if (m2 - kBandLo2 >= kBandSpan2) {
                const unsigned bit = 1u << slab_line<T, R, KC>(tid + t * T::kThreads, c);
                lines |= bit | (m2 >= kBandHi2 ? bit << 16 : 0u);
            }
        }
    return lines;
}

template <int MODE, class T, bool A_KC, bool B_KC, bool VEC>
__global__ void __launch_bounds__(T::kThreads, MODE == kPam || MODE == kStd ? T::kCtasPerSm : T::kCtasPerSm / 2)
gemm_kernel(const GemmParams p) {
    constexpr int BM = T::BM, BN = T::BN, BK = T::BK, MT = T::MT;
    // (the variant with both operands contiguous along their row index spills registers at 8)
    constexpr int kFastUnroll = (!A_KC && !B_KC) || 8 > BK ? BK : 8;
    __shared__ __align__(16) float As[2][BK * row_stride(BM)];
    __shared__ __align__(16) float Bs[2][BK * row_stride(BN)];
    __shared__ unsigned lines[3];   // per slab: bit k = k line holds an out-of-band element, bit 16 + k = one above the band
    __shared__ unsigned overflow_lines;   // bit k = some product of k line may leave the pass range

    const int tid = threadIdx.x;
    const int tx = tid % T::TX, ty = tid / T::TX;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int z = blockIdx.z / p.splits, sp = blockIdx.z - z * p.splits;
    const int k_begin = sp * p.k_chunk;
    const int k_end = min(p.K, k_begin + p.k_chunk);
    const int slabs = (k_end - k_begin + BK - 1) / BK;

    // batch z = outer * inner + (index in the inner dimension); outer = z / inner by a multiply-high with
    // the reciprocal prepared on the host (exact for z < 65536, the grid limit); the strides arrive
    // rearranged so that the offset is outer * sb + z * sb2
    const unsigned zo = __umulhi((unsigned)z, p.inner_magic);
    const float* Ab = p.A.p + (int64_t)zo * p.A.sb + (int64_t)z * p.A.sb2;
    const float* Bb = p.B.p + (int64_t)zo * p.B.sb + (int64_t)z * p.B.sb2;

    float acc[MT][MT];
#pragma unroll
    for (int i = 0; i < MT; ++i)
#pragma unroll
        for (int j = 0; j < MT; ++j) acc[i][j] = 0.0f;

    // exact-gradient product: per-output constant (mantissa of D + offset) that the slope adds to
    // the other operand's bits (pam_scalar.cuh mul_slope).
    int32_t dm[MODE >= kBwdL ? MT : 1][MODE >= kBwdL ? MT : 1];
    if constexpr (MODE >= kBwdL) {
        const float* Db = p.D + (int64_t)z * p.sDb;
#pragma unroll
        for (int i = 0; i < MT; ++i) {
            int row = m0 + ty * 4 + (i & 3) + (i >> 2) * (BM / 2);
            row = row < p.M ? row : p.M - 1;
#pragma unroll
            for (int j = 0; j < MT; ++j) {
                int col = n0 + tx * 4 + (j & 3) + (j >> 2) * (BN / 2);
                col = col < p.N ? col : p.N - 1;
                dm[i][j] = iadd(kMant & f2i(__ldg(Db + (int64_t)row * p.sDm + (int64_t)col * p.sDn)), p.off);
            }
        }
    }

    if (MODE == kPam && tid < 3) lines[tid] = 0;

    float ra[T::kTasksA * 4], rb[T::kTasksB * 4];
    SlabWalker<T, BM, T::kTasksA, A_KC> walk_a;
    SlabWalker<T, BN, T::kTasksB, B_KC> walk_b;
    if constexpr (VEC) {
        walk_a.init(p.A, Ab, m0, p.M, k_begin, tid);
        walk_b.init(p.B, Bb, n0, p.N, k_begin, tid);
    }
    auto stage_load = [&](int k0) {
        if constexpr (VEC) {
            walk_a.load(ra, k0, k_end, tid);
            walk_b.load(rb, k0, k_end, tid);
        } else {
            load_slab<T, BM, T::kTasksA, A_KC, false>(ra, p.A, Ab, m0, p.M, k0, k_end, tid);
            load_slab<T, BN, T::kTasksB, B_KC, false>(rb, p.B, Bb, n0, p.N, k0, k_end, tid);
        }
    };
    auto stage_store = [&](int buf, int slot) {
        if (MODE == kPam) {
            // clean warps (the common case) pay the band test and one vote; only a warp that holds
            // an out-of-band element locates it and reports its k line to the slab's word
            const bool out = band_excess(rb, band_excess(ra, 0u)) >= kBandSpan2;
            if (__any_sync(0xffffffffu, out)) {
                unsigned f = out ? (dirty_lines<T, BM, T::kTasksA, A_KC>(ra, tid) | dirty_lines<T, BN, T::kTasksB, B_KC>(rb, tid)) : 0u;
                f = __reduce_or_sync(0xffffffffu, f);
                if ((tid & 31) == 0) atomicOr(&lines[slot], f);
            }
            // the A side is pre-biased (bits - (0x3f800000 - offset)) so that a product is a two-input add
#pragma unroll
            for (int c = 0; c < T::kTasksA * 4; ++c) ra[c] = i2f(isub(f2i(ra[c]), p.bias_sub));
        }
        store_slab<T, BM, T::kTasksA, A_KC>(As[buf], ra, tid);
        store_slab<T, BN, T::kTasksB, B_KC>(Bs[buf], rb, tid);
    };

    if (slabs > 0) stage_load(k_begin);
    __syncthreads();               // flag words initialised
    if (slabs > 0) stage_store(0, 0);
    __syncthreads();

    // One slab.  (Written as a lambda called from the loop below: in this form the compiler's register
    // allocation of the 128x128 kernels needs no spills, which the same statements placed directly in
    // the loop body do.)
    auto slab_iteration = [&](int s) {
        const int buf = s & 1;
        const bool more = s + 1 < slabs;
        if (more) stage_load(k_begin + (s + 1) * BK);
        unsigned dirty = 0;
        if (MODE == kPam) {
            dirty = lines[s % 3];
            // the word two slabs ahead was last read before the previous barrier: reset it now
            if (tid == 0) lines[(s + 2) % 3] = 0;
        }
        const float* as = As[buf];
        const float* bs = Bs[buf];

#define PAMK_FRAGMENTS(kk)                                                                              \
        const int4 a0 = *reinterpret_cast<const int4*>(as + (kk) * row_stride(BM) + ty * 4);           \
        const int4 a1 = MT == 8 ? *reinterpret_cast<const int4*>(as + (kk) * row_stride(BM) + ty * 4 + BM / 2) : a0; \
        const int4 b0 = *reinterpret_cast<const int4*>(bs + (kk) * row_stride(BN) + tx * 4);           \
        const int4 b1 = MT == 8 ? *reinterpret_cast<const int4*>(bs + (kk) * row_stride(BN) + tx * 4 + BN / 2) : b0; \
        const int a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};                              \
        const int b[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};

        if (MODE == kPam && dirty == 0) {
#pragma unroll kFastUnroll
            for (int kk = 0; kk < BK; ++kk) {
                PAMK_FRAGMENTS(kk)
#pragma unroll
                for (int i = 0; i < MT; ++i)
#pragma unroll
                    for (int j = 0; j < MT; ++j) acc[i][j] = fadd(acc[i][j], i2f(iadd(a[i], b[j])));
            }
        } else if constexpr (MODE == kPam) {
            // lines that hold an element above the band: can a product leave the pass range?
            unsigned full = 0;
            if (dirty >> 16) {                                  // (uniform: read from shared memory after a barrier)
                constexpr int kLanes = T::kThreads / BK;        // threads that share one k line
                const int line = tid / kLanes, lane = tid % kLanes;
                if (tid == 0) overflow_lines = 0;
                __syncthreads();
                // (every thread takes part, whatever its line: the shuffles below name all 32 lanes)
                uint32_t hi_a = 0, hi_b = 0;                    // magnitudes compare like their bit patterns; inf / NaN are largest
                for (int q = lane; q < BM; q += kLanes) {
                    hi_a = max(hi_a, (uint32_t)iadd(f2i(as[line * row_stride(BM) + q]), p.bias_sub) & 0x7fffffffu);
                    hi_b = max(hi_b, (uint32_t)f2i(bs[line * row_stride(BN) + q]) & 0x7fffffffu);
                }
#pragma unroll
                for (int d = 1; d < kLanes; d <<= 1) {
                    hi_a = max(hi_a, __shfl_xor_sync(0xffffffffu, hi_a, d));
                    hi_b = max(hi_b, __shfl_xor_sync(0xffffffffu, hi_b, d));
                }
                // (an inf or NaN maximum makes the product inf or NaN: not <= the pass bound)
                if (lane == 0 && !(fmul(i2f((int32_t)hi_a), i2f((int32_t)hi_b)) <= i2f(kPassBits))) atomicOr(&overflow_lines, 1u << line);
                __syncthreads();
                full = overflow_lines;
            }
            const unsigned all_lines = (1u << BK) - 1u;
            if (__popc(dirty & all_lines) * 4 >= BK * 3 && full == 0) {
                // most lines dirty, none can overflow (e.g. an operand that is half zeros): "flush or add"
                // for the whole slab in one unrolled loop (it is exact for clean lines too)
#pragma unroll 2
                for (int kk = 0; kk < BK; ++kk) {
                    PAMK_FRAGMENTS(kk)
                    float araw[MT];          // a[] holds pre-biased patterns; the rule needs the values
#pragma unroll
                    for (int i = 0; i < MT; ++i) araw[i] = i2f(iadd(a[i], p.bias_sub));
#pragma unroll
                    for (int i = 0; i < MT; ++i)
#pragma unroll
                        for (int j = 0; j < MT; ++j) {
                            const float mag = fabsf(fmul(araw[i], i2f(b[j])));
                            if (mag > i2f(kFlushBits)) acc[i][j] = fadd(acc[i][j], i2f(iadd(a[i], b[j])));
                        }
                }
            } else {
                // The lines are walked in runs of one kind, each run by a loop of its own with one copy of
                // its body (with the three bodies side by side in one loop the schedule cost 12 %).
                const unsigned flush = dirty & ~full & all_lines;
                int kk = 0;
                while (kk < BK) {
                    const unsigned here = 1u << kk;
                    if (full & here) {
                        PAMK_FRAGMENTS(kk)
                        float araw[MT];
#pragma unroll
                        for (int i = 0; i < MT; ++i) araw[i] = i2f(iadd(a[i], p.bias_sub));
#pragma unroll
                        for (int i = 0; i < MT; ++i)
#pragma unroll
                            for (int j = 0; j < MT; ++j) {
                                const float mag = fabsf(fmul(araw[i], i2f(b[j])));
                                const float prod = mag <= i2f(kPassBits) ? i2f(iadd(a[i], b[j])) : quiet_nan();
                                if (!(mag <= i2f(kFlushBits))) acc[i][j] = fadd(acc[i][j], prod);
                            }
                        ++kk;
                    } else if (flush & here) {
                        const unsigned others = ~flush >> kk;
                        const int end = min(BK, kk + __ffs((int)others) - 1);
#pragma unroll 1
                        for (; kk < end; ++kk) {
                            PAMK_FRAGMENTS(kk)
                            float araw[MT];
#pragma unroll
                            for (int i = 0; i < MT; ++i) araw[i] = i2f(iadd(a[i], p.bias_sub));
#pragma unroll
                            for (int i = 0; i < MT; ++i)
#pragma unroll
                                for (int j = 0; j < MT; ++j) {
                                    const float mag = fabsf(fmul(araw[i], i2f(b[j])));
                                    if (mag > i2f(kFlushBits)) acc[i][j] = fadd(acc[i][j], i2f(iadd(a[i], b[j])));
                                }
                        }
                    } else {
                        const unsigned others = (dirty & all_lines) >> kk;
                        const int end = others ? kk + __ffs((int)others) - 1 : BK;
#pragma unroll 1
                        for (; kk < end; ++kk) {
                            PAMK_FRAGMENTS(kk)
#pragma unroll
                            for (int i = 0; i < MT; ++i)
#pragma unroll
                                for (int j = 0; j < MT; ++j) acc[i][j] = fadd(acc[i][j], i2f(iadd(a[i], b[j])));
                        }
                    }
                }
            }
        } else if constexpr (MODE != kPam) {
#pragma unroll 2
            for (int kk = 0; kk < BK; ++kk) {
                PAMK_FRAGMENTS(kk)
                if constexpr (MODE == kStd) {
#pragma unroll
                    for (int i = 0; i < MT; ++i)
#pragma unroll
                        for (int j = 0; j < MT; ++j) acc[i][j] = __fmaf_rn(i2f(a[i]), i2f(b[j]), acc[i][j]);
                } else {
                    // acc += delta * 2^slope, slope from the non-delta operand and D
#pragma unroll
                    for (int i = 0; i < MT; ++i)
#pragma unroll
                        for (int j = 0; j < MT; ++j) {
                            const int other = MODE == kBwdL ? b[j] : a[i];
                            const float delta = i2f(MODE == kBwdL ? a[i] : b[j]);
                            acc[i][j] = __fmaf_rn(delta, i2f(kSignExp & iadd(other, dm[i][j])), acc[i][j]);
                        }
                }
            }
        }
#undef PAMK_FRAGMENTS

        if (more) stage_store(buf ^ 1, (s + 1) % 3);
        __syncthreads();
    };
    for (int s = 0; s < slabs; ++s) slab_iteration(s);

    // ---- epilogue ----------------------------------------------------------------------------
    float* Cz = p.C + (int64_t)sp * p.sCsplit + (int64_t)__umulhi((unsigned)z, p.inner_magic) * p.sCb + (int64_t)z * p.sCb2;
    const bool vec_out = ((p.N | p.ldc | p.sCb | p.sCb2 | p.sCsplit) & 3) == 0 && aligned16(p.C);
    const bool post = p.post != 0 && p.splits == 1;             // (with split-K the reduction pass applies it)
    const bool add_bias = p.bias != nullptr && p.splits == 1;   // (with split-K the reduction pass adds it)
    if constexpr (MODE != kPam) {
        // The reference walks K in zero-filled tiles of 32 (cuda_kernels.cu:526-571, 608-629): when K
        // is not a multiple of 32 it also adds products of zeros, which turns a sum of -0 into +0.
        // (A PAM sum is never -0: flushed products are +0.)
        // In the exact-gradient kernel a padded term is pam_bwd(D, 0, 0) = 0 * slope(D, 0)
        // (cuda_kernels.cu:49-57, 795-809): with an offset below one and a small mantissa of D the
        // slope's bit pattern is -inf and the term is NaN.
        if (p.K & 31) {
#pragma unroll
            for (int i = 0; i < MT; ++i)
#pragma unroll
                for (int j = 0; j < MT; ++j) {
                    if constexpr (MODE == kStd) acc[i][j] = fadd(acc[i][j], 0.0f);
                    else acc[i][j] = __fmaf_rn(0.0f, i2f(kSignExp & dm[i][j]), acc[i][j]);
                }
        }
    }
#pragma unroll
    for (int i = 0; i < MT; ++i) {
        const int row = m0 + ty * 4 + (i & 3) + (i >> 2) * (BM / 2);
        if (row >= p.M) continue;
        float* crow = Cz + (int64_t)row * p.ldc;
#pragma unroll
        for (int h = 0; h < MT / 4; ++h) {
            const int col = n0 + tx * 4 + h * (BN / 2);
            if (add_bias) {                            // the bias row is re-read per output row (it stays in L1)
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    if (col + j < p.N) acc[i][h * 4 + j] = fadd(acc[i][h * 4 + j], __ldg(p.bias + col + j));
            }
            if (post) {
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][h * 4 + j] = mul(acc[i][h * 4 + j], p.post_scale, p.off);
            }
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

// Where the finished sums of a split-K product go: a plain [batch][M][N] array, or the strided output
// of the call (row stride and two batch strides).
struct OutArg {
    float* C;
    int64_t ldc, sCb, sCb2;
    int M, N, inner;
    int contiguous;
};

// Adds the split-K partials in split order: C = ((P0 + P1) + P2) + ... (+ bias[column] last; then the
// PAM product with post_scale, if asked for)
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const float* __restrict__ part, const OutArg o,
                                                            int64_t count, int splits,
                                                            const float* __restrict__ bias, int post,
                                                            float post_scale, int32_t off) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += stride) {
        float v = part[i];
        for (int s = 1; s < splits; ++s) v = fadd(v, part[(int64_t)s * count + i]);
        if (bias != nullptr) v = fadd(v, __ldg(bias + (int)(i % o.N)));
        if (post) v = mul(v, post_scale, off);
        if (o.contiguous) {
            o.C[i] = v;
        } else {
            const int64_t r = i / o.N;
            const int col = (int)(i - r * o.N);
            const int64_t z = r / o.M;
            const int row = (int)(r - z * o.M);
            const int64_t zo = z / o.inner;
            o.C[zo * o.sCb + (z - zo * o.inner) * o.sCb2 + (int64_t)row * o.ldc + col] = v;
        }
    }
}

template <int MODE, class T>
int dispatch(const GemmParams& p, bool a_kc, bool b_kc, bool vec, dim3 grid, cudaStream_t st) {
#define PAMK_LAUNCH(AK, BKC, V) gemm_kernel<MODE, T, AK, BKC, V><<<grid, T::kThreads, 0, st>>>(p)
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
    if (!aligned16(m.p) || (m.sb & 3) || (m.sb2 & 3)) return false;   // (either form of the batch strides)
    return kc ? ((m.sr & 3) == 0 && (K & 3) == 0) : ((m.sk & 3) == 0 && (rows & 3) == 0);
}

// ---- planning: tile shape and split-K ---------------------------------------------------------------
// The kernel is issue-bound, so the time of a launch is (the largest number of tiles any SM ends up
// with) x (work per tile), inflated when an SM holds too few warps to keep its schedulers busy,
// which is also the state of the SMs that run the last, partly filled wave of a larger launch.
enum TileKind { kTileLarge = 0, kTileSmall = 1, kTileTiny = 2 };

struct Plan {
    int tile;        // TileKind
    int splits;
    double cost;
};

template <class T>
Plan plan_for(int mode, int64_t batch, int64_t M, int64_t N, int64_t K, int split_request) {
    // the exact-gradient kernels hold a second 8x8 block of per-output constants in registers, so
    // half as many of their CTAs fit on an SM
    const int ctas_per_sm = mode == kBwdL || mode == kBwdR ? T::kCtasPerSm / 2 : T::kCtasPerSm;
    const int64_t sms = sm_count();
    const int64_t tiles = batch * ((M + T::BM - 1) / T::BM) * ((N + T::BN - 1) / T::BN);
    const int64_t slabs = (K + T::BK - 1) / T::BK;
    const int64_t slots = sms * ctas_per_sm;
    // cost of cutting K into s ranges, in multiply-accumulates per SM at full issue rate
    auto cost_of = [&](int64_t s, int64_t* actual) {
        if (s > slabs) s = slabs;
        const int64_t chunk_slabs = (slabs + s - 1) / s;
        s = (slabs + chunk_slabs - 1) / chunk_slabs;         // drop ranges that would be empty
        *actual = s;
        // measured: 16 resident warps per SM saturate the issue slots, 14 reach about 86 % of that,
        // 8 about 74 %
        auto util = [](int64_t ctas) {
            const double warps = (double)ctas * (T::kThreads / 32);
            return warps >= 16.0 ? 1.0 : (warps >= 8.0 ? 0.58 + 0.02 * warps : warps / 10.8);
        };
        // the smaller the tile, the more bytes are staged (and fragments loaded) per MAC
        const double staging = T::BM >= 128 ? 1.0 : (T::BM >= 64 ? 1.06 : 1.25);
        // every CTA also pays a prologue (first loads exposed) and an epilogue worth about 16 k-steps
        const double per_cta = (double)T::BM * T::BN * ((double)(chunk_slabs * T::BK) + 16.0);
        const int64_t ctas = tiles * s;
        // CTAs spread evenly over the SMs ...
        const int64_t per_sm = (ctas + sms - 1) / sms;
        double cost = (double)per_sm * per_cta / util(per_sm < ctas_per_sm ? per_sm : ctas_per_sm);
        // ... and CTAs that run as full waves over all slots plus a last, partly filled one whose SMs
        // hold few warps.  The hardware refills slots one by one, which lies between the two: a sweep
        // of tile x split over products of 1 to 9 waves fits 0.62 / 0.38 (a vocabulary-sized weight
        // gradient of 1.07 waves loses 24 % to its tail without a split).
        const int64_t full = ctas / slots, rest = (ctas - full * slots + sms - 1) / sms;
        if (full >= 1) {
            const double waves = (double)(full * ctas_per_sm) * per_cta / util(ctas_per_sm) + (rest ? (double)rest * per_cta / util(rest) : 0.0);
            cost = 0.62 * cost + 0.38 * waves;
        }
        return cost * staging + (s > 1 ? 1.1e6 : 0.0);        // the reduction pass and its launch (~12 us)
    };
    Plan pl;
    pl.tile = T::BM >= 128 ? kTileLarge : (T::BM >= 64 ? kTileSmall : kTileTiny);
    int64_t s = split_request > 0 ? split_request : 1, actual = 1;
    pl.cost = cost_of(s, &actual);
    pl.splits = (int)actual;
    if (split_request == 0 && tiles < 8 * slots && slabs >= 8) {  // automatic: fill the SMs, shorten the tail
        int64_t limit = 8 * slots / tiles;                   // up to eight full waves of CTAs
        if (limit < 2) limit = 2;
        if (limit > slabs / 4) limit = slabs / 4;            // keep at least four slabs per range
        if (limit > 64) limit = 64;
        // a fixed ladder plus the splits that fill exactly one and two waves
        const int64_t ladder[] = {2, 3, 4, 6, 8, 12, 16, 24, 32, 48, 64, slots / tiles, 2 * slots / tiles};
        for (int64_t cand : ladder) {
            if (cand < 2 || cand > limit) continue;
            int64_t got = 1;
            const double c = cost_of(cand, &got);
            // a split has to promise 5 % before it replaces the unsplit product (which also keeps
            // the reference's summation order)
            if (c < (pl.splits == 1 ? 0.95 * pl.cost : pl.cost)) { pl.cost = c; pl.splits = (int)got; }
        }
    }
    return pl;
}

// 0: choose by cost; 1: always the large tile; 2: the 64x64 tile wherever it exists; 3: the 32x32
// tile wherever it exists (PAM products), else the 64x64 tile.
int g_tile_policy = 0;

Plan make_plan(int mode, int64_t batch, int64_t M, int64_t N, int64_t K, int split_request) {
    const Plan large = plan_for<TileLarge>(mode, batch, M, N, K, split_request);
    if (mode == kStd || g_tile_policy == 1) return large;    // the true-multiply product uses the large tile
    const Plan small = plan_for<TileSmall>(mode, batch, M, N, K, split_request);
    if (g_tile_policy == 2 || (g_tile_policy == 3 && mode != kPam)) return small;
    Plan best = small.cost < large.cost ? small : large;
    // The 32x32 tile wins where the 64x64 tile pads much (192 x 197x197x64: 256x256 against 224x224
    // outputs) or leaves most SMs empty.  Its modelled cost has to be lower by a margin that sweeps of
    // tile x split fitted: 10 % for launches of at least two waves of 64x64 tiles, where only throughput
    // counts (120 products: median -12 %, worst +6 %), and for matrices no larger than one tile in a
    // dimension; 20 % for smaller launches, where the model overrates the tile (106 products with that
    // margin: median -22 %, one slower, by 0.3 %; of 34 with 10 to 20 %, 13 were slower).
    if (mode == kPam) {
        const int64_t small_tiles = batch * ((M + TileSmall::BM - 1) / TileSmall::BM) * ((N + TileSmall::BN - 1) / TileSmall::BN);
        const bool throughput_bound = small_tiles >= 2 * (int64_t)sm_count() * TileSmall::kCtasPerSm;
        const double margin = throughput_bound || M <= TileTiny::BM || N <= TileTiny::BN ? 0.9 : 0.8;
        const Plan tiny = plan_for<TileTiny>(mode, batch, M, N, K, split_request);
        if (g_tile_policy == 3 || tiny.cost < margin * best.cost) best = tiny;
    }
    return best;
}

bool workspace_ok(const void* ws, size_t bytes, int splits, int64_t count) {
    return ws != nullptr && (reinterpret_cast<uintptr_t>(ws) & 255u) == 0 &&
           bytes >= (size_t)splits * (size_t)count * sizeof(float);
}

int run(int mode, GemmParams p, bool a_kc, bool b_kc, int split_k, void* workspace, size_t workspace_bytes,
        cudaStream_t st) {
    if (p.M == 0 || p.N == 0 || p.batch == 0) return PAMK_OK;
    const int64_t count = (int64_t)p.batch * p.M * p.N;
    if (p.K == 0 && p.bias == nullptr && p.ldc == 0) {
        const cudaError_t e = cudaMemsetAsync(p.C, 0, count * sizeof(float), st);
        return e == cudaSuccess ? PAMK_OK : record_cuda_error(e);
    }
    if (split_k < 0) return PAMK_ERR_ARG;
    Plan pl = p.K == 0 ? Plan{kTileSmall, 1, 0.0} : make_plan(mode, p.batch, p.M, p.N, p.K, split_k);   // K = 0: rows of bias
    if (pl.splits > 1 && !workspace_ok(workspace, workspace_bytes, pl.splits, count)) {
        if (split_k != 0) return PAMK_ERR_WORKSPACE;         // an explicit split needs its scratch
        pl = make_plan(mode, p.batch, p.M, p.N, p.K, 1);     // automatic: fall back to no split
    }
    // the M tiles ride on grid.y (at most 65535): a very tall product planned with a small tile moves to
    // the 128x128 tile, which reaches 8.3 M rows
    if (pl.tile != kTileLarge && (p.M + (pl.tile == kTileTiny ? TileTiny::BM : TileSmall::BM) - 1) /
                                         (pl.tile == kTileTiny ? TileTiny::BM : TileSmall::BM) > 65535) {
        const int splits = pl.splits;
        pl = plan_for<TileLarge>(mode, p.batch, p.M, p.N, p.K, splits);
    }
    const int bm = pl.tile == kTileTiny ? TileTiny::BM : (pl.tile == kTileSmall ? TileSmall::BM : TileLarge::BM);
    const int bn = pl.tile == kTileTiny ? TileTiny::BN : (pl.tile == kTileSmall ? TileSmall::BN : TileLarge::BN);
    const int bk = pl.tile == kTileTiny ? TileTiny::BK : (pl.tile == kTileSmall ? TileSmall::BK : TileLarge::BK);
    if (p.inner < 1) p.inner = 1;
    if (p.ldc == 0) {                                        // plain output: [batch][M][N]
        p.ldc = p.N;
        p.sCb = (int64_t)p.inner * p.M * p.N;
        p.sCb2 = (int64_t)p.M * p.N;
    }
    OutArg out{p.C, p.ldc, p.sCb, p.sCb2, p.M, p.N, p.inner,
               p.ldc == p.N && p.sCb2 == (int64_t)p.M * p.N && p.sCb == (int64_t)p.inner * p.M * p.N};
    if (pl.splits > 1) {                                     // partials: [split][batch][M][N] in the scratch
        p.C = static_cast<float*>(workspace);
        p.ldc = p.N;
        p.sCb = (int64_t)p.inner * p.M * p.N;
        p.sCb2 = (int64_t)p.M * p.N;
        p.sCsplit = count;
    }
    // batch strides into the kernel's form (see MatArg)
    const bool vec = vectorisable(p.A, a_kc, p.M, p.K) && vectorisable(p.B, b_kc, p.N, p.K);
    auto kernel_form = [&](int64_t& outer, int64_t& inner_stride) {
        if (p.inner == 1) { inner_stride = outer; outer = 0; }
        else outer -= (int64_t)p.inner * inner_stride;
    };
    kernel_form(p.A.sb, p.A.sb2);
    kernel_form(p.B.sb, p.B.sb2);
    kernel_form(p.sCb, p.sCb2);
    p.inner_magic = p.inner == 1 ? 0u : (unsigned)((uint64_t(1) << 32) / (uint64_t)p.inner) + 1u;
    const int slabs_total = (p.K + bk - 1) / bk;
    p.splits = pl.splits;
    p.k_chunk = ((slabs_total + pl.splits - 1) / pl.splits) * bk;

    const int64_t gx = (p.N + bn - 1) / bn, gy = (p.M + bm - 1) / bm, gz = (int64_t)p.batch * pl.splits;
    if (gy > 65535 || gz > 65535) return PAMK_ERR_SIZE;
    const dim3 grid((unsigned)gx, (unsigned)gy, (unsigned)gz);
    int rc;
    switch (mode) {
        case kPam:
            rc = pl.tile == kTileTiny    ? dispatch<kPam, TileTiny>(p, a_kc, b_kc, vec, grid, st)
                 : pl.tile == kTileSmall ? dispatch<kPam, TileSmall>(p, a_kc, b_kc, vec, grid, st)
                                         : dispatch<kPam, TileLarge>(p, a_kc, b_kc, vec, grid, st);
            break;
        case kStd: rc = dispatch<kStd, TileLarge>(p, a_kc, b_kc, vec, grid, st); break;
        case kBwdL:
            rc = pl.tile == kTileSmall ? dispatch<kBwdL, TileSmall>(p, a_kc, b_kc, vec, grid, st)
                                       : dispatch<kBwdL, TileLarge>(p, a_kc, b_kc, vec, grid, st);
            break;
        default:
            rc = pl.tile == kTileSmall ? dispatch<kBwdR, TileSmall>(p, a_kc, b_kc, vec, grid, st)
                                       : dispatch<kBwdR, TileLarge>(p, a_kc, b_kc, vec, grid, st);
            break;
    }
    if (rc != PAMK_OK || pl.splits == 1) return rc;
    const int64_t blocks = (count + 255) / 256;
    const int64_t cap = (int64_t)sm_count() * 8;
    splitk_reduce_kernel<<<(unsigned)(blocks < cap ? blocks : cap), 256, 0, st>>>(
        static_cast<const float*>(workspace), out, count, pl.splits, p.bias, p.post, p.post_scale, p.off);
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

// ---- allocation-free split-K --------------------------------------------------------------------
// Scratch for pamk_matmul_static_scratch: lives in the library image, so every GPU that loads the
// library holds these 32 MiB from load until exit, and no allocation is ever needed for it.
constexpr size_t kStaticScratchFloats = size_t(8) << 20;
static __device__ __align__(256) float g_splitk_scratch[kStaticScratchFloats];

// In host code `g_splitk_scratch` is only a handle for the symbol; the device address has to be
// asked for, per device, with that device current.
constexpr int kMaxDevices = 64;
float* g_scratch_addr[kMaxDevices] = {};

int static_scratch(float** out) {
    int dev = -1;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return record_cuda_error(err);
    if (dev < 0 || dev >= kMaxDevices) return PAMK_ERR_SIZE;
    if (g_scratch_addr[dev] == nullptr) {
        void* ptr = nullptr;
        err = cudaGetSymbolAddress(&ptr, g_splitk_scratch);
        if (err != cudaSuccess) return record_cuda_error(err);
        g_scratch_addr[dev] = static_cast<float*>(ptr);
    }
    *out = g_scratch_addr[dev];
    return PAMK_OK;
}

}  // namespace
}  // namespace pamk

using namespace pamk;

extern "C" {

size_t pamk_matmul_workspace_bytes(int64_t batch, int64_t M, int64_t N, int split_k) {
    if (split_k <= 1 || batch <= 0 || M <= 0 || N <= 0) return 0;
    return (size_t)split_k * (size_t)batch * (size_t)M * (size_t)N * sizeof(float);
}

int pamk_test_set_tile_policy(int policy) {
    if (policy < 0 || policy > 3) return PAMK_ERR_ARG;
    g_tile_policy = policy;
    return PAMK_OK;
}

int pamk_test_planned_tile(int64_t batch, int64_t M, int64_t N, int64_t K) {
    if (batch <= 0 || M <= 0 || N <= 0 || K <= 0) return PAMK_ERR_ARG;
    const int tile = make_plan(kPam, batch, M, N, K, 0).tile;
    return tile == kTileLarge ? 128 : (tile == kTileSmall ? 64 : 32);
}

int pamk_matmul_auto_split(int64_t batch, int64_t M, int64_t N, int64_t K) {
    if (batch <= 0 || M <= 0 || N <= 0 || K <= 0) return 1;
    return make_plan(kPam, batch, M, N, K, 0).splits;
}

int pamk_matmul_bwd_auto_split(int64_t batch, int64_t M, int64_t N, int64_t K) {
    if (batch <= 0 || M <= 0 || N <= 0 || K <= 0) return 1;
    return make_plan(kBwdL, batch, M, N, K, 0).splits;
}

int pamk_matmul_bias(int mul_kind, const float* A, const float* B, const float* bias, float* C,
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
    p.bias = bias;
    p.M = (int)M; p.N = (int)N; p.K = (int)K; p.batch = (int)batch;
    p.off = offset_bits(offset);
    p.bias_sub = isub(kBias, p.off);
    return run(mul_kind == PAMK_MUL_PAM ? kPam : kStd, p, a_kc, b_kc, split_k, workspace, workspace_bytes,
               static_cast<cudaStream_t>(stream));
}

int pamk_matmul(int mul_kind, const float* A, const float* B, float* C,
                int64_t batch, int64_t M, int64_t N, int64_t K,
                int64_t sAb, int64_t sAm, int64_t sAk,
                int64_t sBb, int64_t sBk, int64_t sBn,
                float offset, int split_k, void* workspace, size_t workspace_bytes, void* stream) {
    return pamk_matmul_bias(mul_kind, A, B, nullptr, C, batch, M, N, K, sAb, sAm, sAk, sBb, sBk, sBn, offset, split_k,
                            workspace, workspace_bytes, stream);
}

int pamk_matmul_strided(const float* A, const float* B, float* C,
                        int64_t batch_outer, int64_t batch_inner, int64_t M, int64_t N, int64_t K,
                        int64_t sAo, int64_t sAi, int64_t sAm, int64_t sAk,
                        int64_t sBo, int64_t sBi, int64_t sBk, int64_t sBn,
                        int64_t sCo, int64_t sCi, int64_t sCm,
                        float offset, int has_post_scale, float post_scale,
                        int split_k, void* workspace, size_t workspace_bytes, void* stream) {
    if (batch_outer < 0 || batch_inner < 0) return PAMK_ERR_ARG;
    if (batch_inner > 0 && batch_outer > (0x7fffffff - 256) / batch_inner) return PAMK_ERR_SIZE;
    const int64_t batch = batch_outer * batch_inner;
    if (!dims_ok(batch, M, N, K)) return M < 0 || N < 0 || K < 0 ? PAMK_ERR_ARG : PAMK_ERR_SIZE;
    if (split_k < 0) return PAMK_ERR_ARG;
    if (batch == 0 || M == 0 || N == 0) return PAMK_OK;
    if (C == nullptr || sCm < N) return PAMK_ERR_ARG;
    GemmParams p{};
    bool a_kc = true, b_kc = true;
    if (K > 0) {
        int rc = operand_layout(A, sAm, sAk, (int)M, (int)K, &a_kc);
        if (rc != PAMK_OK) return rc;
        rc = operand_layout(B, sBn, sBk, (int)N, (int)K, &b_kc);
        if (rc != PAMK_OK) return rc;
    }
    p.A = {A, sAo, sAm, sAk, sAi};
    p.B = {B, sBo, sBn, sBk, sBi};
    p.C = C;
    p.ldc = sCm; p.sCb = sCo; p.sCb2 = sCi;
    p.inner = (int)batch_inner;
    p.post = has_post_scale != 0;
    p.post_scale = post_scale;
    p.M = (int)M; p.N = (int)N; p.K = (int)K; p.batch = (int)batch;
    p.off = offset_bits(offset);
    p.bias_sub = isub(kBias, p.off);
    return run(kPam, p, a_kc, b_kc, split_k, workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
}

size_t pamk_matmul_static_scratch_bytes(void) { return kStaticScratchFloats * sizeof(float); }

int pamk_matmul_static_scratch(const float* A, const float* B, float* C,
                               int64_t batch, int64_t M, int64_t N, int64_t K,
                               int64_t sAb, int64_t sAm, int64_t sAk,
                               int64_t sBb, int64_t sBk, int64_t sBn,
                               float offset, int split_k, void* stream) {
    if (!dims_ok(batch, M, N, K)) return batch < 0 || M < 0 || N < 0 || K < 0 ? PAMK_ERR_ARG : PAMK_ERR_SIZE;
    if (split_k < 1) return PAMK_ERR_ARG;
    if (batch == 0 || M == 0 || N == 0) return PAMK_OK;
    if (C == nullptr) return PAMK_ERR_ARG;
    // every partial sum must fit in the fixed array
    if ((double)split_k * (double)batch * (double)M * (double)N > (double)kStaticScratchFloats) return PAMK_ERR_SIZE;
    GemmParams p{};
    bool a_kc = true, b_kc = true;
    if (K > 0) {
        int rc = operand_layout(A, sAm, sAk, (int)M, (int)K, &a_kc);
        if (rc != PAMK_OK) return rc;
        rc = operand_layout(B, sBn, sBk, (int)N, (int)K, &b_kc);
        if (rc != PAMK_OK) return rc;
    }
    float* scratch = nullptr;
    const int rc = static_scratch(&scratch);
    if (rc != PAMK_OK) return rc;
    p.A = {A, sAb, sAm, sAk};
    p.B = {B, sBb, sBn, sBk};
    p.C = C;
    p.M = (int)M; p.N = (int)N; p.K = (int)K; p.batch = (int)batch;
    p.off = offset_bits(offset);
    p.bias_sub = isub(kBias, p.off);
    return run(kPam, p, a_kc, b_kc, split_k, scratch, kStaticScratchFloats * sizeof(float),
               static_cast<cudaStream_t>(stream));
}

int pamk_matmul_bwd(const float* L, const float* R, const float* D, float* out,
                    int64_t batch, int64_t M, int64_t N, int64_t K,
                    int64_t sLb, int64_t sLm, int64_t sLk,
                    int64_t sRb, int64_t sRk, int64_t sRn,
                    int64_t sDb, int64_t sDm, int64_t sDn,
                    int delta_l, float offset, int split_k, void* workspace, size_t workspace_bytes, void* stream) {
    if (!dims_ok(batch, M, N, K)) return batch < 0 || M < 0 || N < 0 || K < 0 ? PAMK_ERR_ARG : PAMK_ERR_SIZE;
    if (split_k < 0) return PAMK_ERR_ARG;
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
    return run(delta_l ? kBwdL : kBwdR, p, l_kc, r_kc, split_k, workspace, workspace_bytes,
               static_cast<cudaStream_t>(stream));
}

}
