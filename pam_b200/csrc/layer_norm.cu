// pam_ln: fused PAM layer normalisation, forward and backward.
//
// The reference evaluates layer_norm as a chain of about 15 elementwise launches forward and 40
// backward (epfml/pam pam/pam_ops.py:350-378 through autograd), each a full read and write of the
// activation, with every intermediate rounded to fp32.  Here one warp owns a row: the row stays
// in registers, the two (forward) or four (backward) row sums are warp-shuffle reductions, and
// every primitive of the chain is evaluated by the same scalar function the elementwise kernels
// use, rounding where the reference rounds.  Traffic is the algorithmic minimum: read x, write y
// (8 B/element) forward; read x and dy, write dx (12 B/element) backward.
//
// The chain, per row of width n (nf = float(n), "op" = PAM primitive, +,- = ordinary fp32):
//   mu = pad(sum x, nf);  c = x - mu;  var = pad(sum pam(c, c), nf);  v = var + eps
//   denom = (v == 0) ? 0 : exp2_op(pam(log2_op(v), 0.5))          [pam_ops.pow, :70-79]
//   y = pam(pad(c, denom), w) + b
// The backward pass recomputes the forward chain from x and applies, primitive by primitive, the
// gradient pairing of pam/cuda_bindings.py (approximate: gradients are PAM products with the
// other operand; exact: the piecewise-affine slopes).
#include "common.cuh"
#include "pam_scalar.cuh"

namespace pamk {
namespace {

constexpr int kWarpsPerCta = 4;
constexpr int kThreads = kWarpsPerCta * 32;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) v = fadd(v, __shfl_xor_sync(0xffffffffu, v, d));
    return v;
}

// Divisors shared by every row of a launch: the row width n (both means) and log2f(2) = 1 (the
// base-2 log kernel divides by it).  Prepared once per thread.
struct Shared {
    Divisor by_n, by_lb2;
    float lb2;
};

__device__ __forceinline__ Shared make_shared(float nf, int32_t off) {
    Shared s;
    s.lb2 = log2f(2.0f);                            // the base-2 kernels scale by log2f(2) = 1
    s.by_n = make_divisor(nf, off);
    s.by_lb2 = make_divisor(s.lb2, off);
    return s;
}

struct LnArgs {
    const float* x;
    const float* w;      // may be null
    const float* b;      // may be null
    const float* dy;     // backward only
    float* out;          // y (forward) or dx (backward)
    float* partials;     // backward with w/b: [gridDim.x][2][width] per-CTA sums for dw, db
    int64_t rows;
    int width;
    float nf, eps;
    int32_t off;
    float* stats;        // [rows][8] row scalars of the forward chain: written by the forward pass when not
                         // null, read by the backward pass that works from them (kStat* below)
};

// What the forward pass keeps per row for the backward pass that does not recompute it.
enum { kStatMu = 0, kStatV, kStatE, kStatFlushMax, kStatPassMax, kStatSub, kStatRecip, kStatDenom, kStatCount };

// Row-level scalars of the forward chain.
struct RowStats {
    float s1, mu, s2, v, l, m, e, denom;
};

__device__ __forceinline__ void finish_stats(RowStats& r, const LnArgs& a, const Shared& sh) {
    const float var = div_by(r.s2, sh.by_n);
    r.v = fadd(var, a.eps);
    r.l = div_by(log2(r.v), sh.by_lb2);             // log_base(v, log2f(2), off)
    r.m = mul(r.l, 0.5f, a.off);
    r.e = exp_base(r.m, sh.lb2, a.off);
    r.denom = r.v == 0.0f ? 0.0f : r.e;
}

// A lane holds NCH chunks of VEC consecutive columns: chunk q of lane L starts at column
// (q * 32 + L) * VEC.  With VEC = 4 every access of a warp is a contiguous 512-byte run.
template <int VEC, int NCH>
struct RowRegs {
    float v[NCH * VEC];
};

template <int VEC, int NCH, bool FULL>
__device__ __forceinline__ void load_row(RowRegs<VEC, NCH>& r, const float* p, int width, int lane, float fill) {
#pragma unroll
    for (int q = 0; q < NCH; ++q) {
        const int col = (q * 32 + lane) * VEC;
        if (FULL || col < width) {
            if (VEC == 4) {
                const float4 t = __ldg(reinterpret_cast<const float4*>(p + col));
                r.v[q * 4] = t.x; r.v[q * 4 + 1] = t.y; r.v[q * 4 + 2] = t.z; r.v[q * 4 + 3] = t.w;
            } else if (VEC == 2) {
                const float2 t = __ldg(reinterpret_cast<const float2*>(p + col));
                r.v[q * 2] = t.x; r.v[q * 2 + 1] = t.y;
            } else {
                r.v[q] = __ldg(p + col);
            }
        } else {
#pragma unroll
            for (int j = 0; j < VEC; ++j) r.v[q * VEC + j] = fill;
        }
    }
}

template <int VEC, int NCH, bool FULL>
__device__ __forceinline__ void store_row(const RowRegs<VEC, NCH>& r, float* p, int width, int lane) {
#pragma unroll
    for (int q = 0; q < NCH; ++q) {
        const int col = (q * 32 + lane) * VEC;
        if (FULL || col < width) {
            if (VEC == 4)
                *reinterpret_cast<float4*>(p + col) = make_float4(r.v[q * 4], r.v[q * 4 + 1], r.v[q * 4 + 2], r.v[q * 4 + 3]);
            else if (VEC == 2)
                *reinterpret_cast<float2*>(p + col) = make_float2(r.v[q * 2], r.v[q * 2 + 1]);
            else
                p[col] = r.v[q];
        }
    }
}

// FULL: the row fills every register slot of the layout (width == 32 * VEC * NCH: 128, 192, 256,
// 512, 768, 1024), so no column needs a bounds test.
template <int VEC, int NCH, bool FULL>
__device__ __forceinline__ bool live(int i, int width, int lane) {
    return FULL || ((i / VEC) * 32 + lane) * VEC + (i % VEC) < width;
}

// Forward chain up to the centred row and the row scalars.  Padding lanes hold 0 in `c` so that
// pam(0, 0) = +0 leaves the sums untouched.
template <int VEC, int NCH, bool FULL>
__device__ __forceinline__ void centre_and_stats(RowRegs<VEC, NCH>& c, RowStats& st, const LnArgs& a,
                                                 const Shared& sh, int lane) {
    float s = 0.0f;
#pragma unroll
    for (int i = 0; i < NCH * VEC; ++i) s = fadd(s, c.v[i]);
    st.s1 = warp_sum(s);
    st.mu = div_by(st.s1, sh.by_n);
    s = 0.0f;
#pragma unroll
    for (int i = 0; i < NCH * VEC; ++i) {
        c.v[i] = live<VEC, NCH, FULL>(i, a.width, lane) ? fadd(c.v[i], -st.mu) : 0.0f;
        s = fadd(s, mul(c.v[i], c.v[i], a.off));
    }
    st.s2 = warp_sum(s);
    finish_stats(st, a, sh);
}

// Minimum resident CTAs asked of the compiler: narrow layouts need few registers, and the more warps
// an SM holds the more loads it has in flight.
constexpr int min_ctas(int slots, bool backward) {
    return slots <= 8 ? (backward ? 6 : 10) : (slots <= 16 ? (backward ? 4 : 6) : 1);
}

// Rows one warp handles together.  The per-row scalar chain (variance -> log2 -> half -> exp2 ->
// exact divisor thresholds) costs more instructions than the elementwise work of a narrow row; with
// several rows in flight lane L evaluates the chain of row L % kRows only, so the warp pays for one
// chain per group instead of one per row, and the results travel back by shuffle.  Every row is
// still summed and evaluated exactly as if it were alone.
__host__ __device__ constexpr int rows_per_warp(int slots) { return slots <= 8 ? 4 : (slots <= 16 ? 2 : 1); }

template <int VEC, int NCH, bool FULL, bool SAVE = false>
__global__ void __launch_bounds__(kThreads, VEC * NCH <= 16 ? 6 : 1) ln_fwd_kernel(const LnArgs a) {
    constexpr int kRows = rows_per_warp(VEC * NCH);
    const int lane = threadIdx.x & 31;
    const int64_t warp = (int64_t)blockIdx.x * kWarpsPerCta + (threadIdx.x >> 5);
    const int64_t nwarps = (int64_t)gridDim.x * kWarpsPerCta;
    const Shared sh = make_shared(a.nf, a.off);
    for (int64_t row0 = warp * kRows; row0 < a.rows; row0 += nwarps * kRows) {
        RowRegs<VEC, NCH> c[kRows];
        float s1[kRows], s2[kRows];
#pragma unroll
        for (int r = 0; r < kRows; ++r) {
            // (a row beyond the end is computed on the last row's data and not stored)
            const int64_t row = row0 + r < a.rows ? row0 + r : a.rows - 1;
            load_row<VEC, NCH, FULL>(c[r], a.x + row * a.width, a.width, lane, 0.0f);
        }
#pragma unroll
        for (int r = 0; r < kRows; ++r) {
            float s = 0.0f;
#pragma unroll
            for (int i = 0; i < NCH * VEC; ++i) s = fadd(s, c[r].v[i]);
            s1[r] = warp_sum(s);
            const float mu = div_by(s1[r], sh.by_n);
            if (SAVE) s1[r] = mu;                          // (the sum itself is not needed again here)
            s = 0.0f;
#pragma unroll
            for (int i = 0; i < NCH * VEC; ++i) {
                c[r].v[i] = live<VEC, NCH, FULL>(i, a.width, lane) ? fadd(c[r].v[i], -mu) : 0.0f;
                s = fadd(s, mul(c[r].v[i], c[r].v[i], a.off));
            }
            s2[r] = warp_sum(s);
        }
        // the scalar chain of row (lane % kRows), then every row's divisor to every lane
        RowStats mine;
        mine.s2 = s2[0];
        if (SAVE) mine.mu = s1[0];
#pragma unroll
        for (int r = 1; r < kRows; ++r) {
            mine.s2 = (lane % kRows) == r ? s2[r] : mine.s2;
            if (SAVE) mine.mu = (lane % kRows) == r ? s1[r] : mine.mu;
        }
        finish_stats(mine, a, sh);
        const Divisor my_divisor = make_divisor(mine.denom, a.off);
        if (SAVE && lane < kRows && row0 + lane < a.rows) {         // lane r holds the chain of row r
            float4* out = reinterpret_cast<float4*>(a.stats + (row0 + lane) * kStatCount);
            out[0] = make_float4(mine.mu, mine.v, mine.e, my_divisor.flush_max);
            out[1] = make_float4(my_divisor.pass_max, i2f(my_divisor.sub), div_by(1.0f, my_divisor), mine.denom);
        }
        // weight and bias are re-read per row group (they stay in L1) rather than held in registers
        // for the whole kernel: the registers buy more resident warps
        RowRegs<VEC, NCH> p;
        if (a.w) load_row<VEC, NCH, FULL>(p, a.w, a.width, lane, 1.0f);
#pragma unroll
        for (int r = 0; r < kRows; ++r) {
            Divisor by_denom;
            by_denom.flush_max = __shfl_sync(0xffffffffu, my_divisor.flush_max, r);
            by_denom.pass_max = __shfl_sync(0xffffffffu, my_divisor.pass_max, r);
            by_denom.sub = __shfl_sync(0xffffffffu, my_divisor.sub, r);
#pragma unroll
            for (int i = 0; i < NCH * VEC; ++i) {
                const float y = div_by(c[r].v[i], by_denom);
                c[r].v[i] = a.w ? mul(y, p.v[i], a.off) : y;
            }
        }
        if (a.b) {
            load_row<VEC, NCH, FULL>(p, a.b, a.width, lane, 0.0f);
#pragma unroll
            for (int r = 0; r < kRows; ++r)
#pragma unroll
                for (int i = 0; i < NCH * VEC; ++i) c[r].v[i] = fadd(c[r].v[i], p.v[i]);
        }
#pragma unroll
        for (int r = 0; r < kRows; ++r)
            if (row0 + r < a.rows) store_row<VEC, NCH, FULL>(c[r], a.out + (row0 + r) * a.width, a.width, lane);
    }
}

// (four rows of a narrow layout need 158 registers and run 12 warps per SM; two rows at 96 registers
// and 20 warps measured 5 % slower)
__host__ __device__ constexpr int rows_per_warp_bwd(int slots) { return slots <= 8 ? 4 : (slots <= 16 ? 2 : 1); }

// SAVED: the row scalars come from the forward pass (LnArgs::stats) instead of being recomputed from x:
// no first two row sums and no forward scalar chain, so a warp no longer needs several rows in flight to
// share that chain, needs fewer registers and more warps fit on an SM (approximate gradients only).
// (Requesting the next rows from the L2 ahead of time measured 8 % slower here, as in the recomputing form.)
#ifndef PAMK_LN_SAVED_ROWS
#define PAMK_LN_SAVED_ROWS 2
#endif
template <int VEC, int NCH, bool APPROX, bool FULL, bool SAVED = false>
__global__ void __launch_bounds__(kThreads, VEC * NCH <= 16 ? (SAVED ? 5 : 3) : 1) ln_bwd_kernel(const LnArgs a) {
    constexpr int kRows = SAVED ? (VEC * NCH <= 8 ? PAMK_LN_SAVED_ROWS : 1) : rows_per_warp_bwd(VEC * NCH);
    static_assert(!SAVED || APPROX, "the exact gradients need the forward intermediates recomputed");
    __shared__ float stage[kWarpsPerCta][NCH * VEC][32];
    const int lane = threadIdx.x & 31;
    const int wid = threadIdx.x >> 5;
    const int64_t warp = (int64_t)blockIdx.x * kWarpsPerCta + wid;
    const int64_t nwarps = (int64_t)gridDim.x * kWarpsPerCta;
    const float ln2 = 0.693147180559945309417f;      // float(math.log(2.0)), cuda_bindings.py:232,271
    const Shared sh = make_shared(a.nf, a.off);
    const float recip_n = div_by(1.0f, sh.by_n);
    RowRegs<VEC, NCH> w, dw, db;
    if (a.w) load_row<VEC, NCH, FULL>(w, a.w, a.width, lane, 1.0f);
#pragma unroll
    for (int i = 0; i < NCH * VEC; ++i) dw.v[i] = db.v[i] = 0.0f;

    // kRows rows per pass: lane L evaluates the two scalar chains of row L % kRows only (see
    // rows_per_warp); rows are accumulated into dw / db in row order, as a one-row-per-pass walk would.
    for (int64_t row0 = warp * kRows; row0 < a.rows; row0 += nwarps * kRows) {
        RowRegs<VEC, NCH> c[kRows], g[kRows];
        float s1[kRows], s2[kRows];
#pragma unroll
        for (int r = 0; r < kRows; ++r) {
            const int64_t row = row0 + r < a.rows ? row0 + r : a.rows - 1;     // (beyond the end: computed, not stored)
            load_row<VEC, NCH, FULL>(c[r], a.x + row * a.width, a.width, lane, 0.0f);
            load_row<VEC, NCH, FULL>(g[r], a.dy + row * a.width, a.width, lane, 0.0f);
        }
        const int my_row = lane % kRows;
        RowStats st;
        Divisor my_divisor;
        float my_recip;
        if constexpr (SAVED) {
            // lane L reads the scalars of row L % kRows; the centred rows need every row's mean
            const int64_t mine = row0 + my_row < a.rows ? row0 + my_row : a.rows - 1;
            const float4* in = reinterpret_cast<const float4*>(a.stats + mine * kStatCount);
            const float4 s0 = __ldg(in), s1v = __ldg(in + 1);
            st.v = s0.y;
            st.e = s0.z;
            my_divisor.flush_max = s0.w;
            my_divisor.pass_max = s1v.x;
            my_divisor.sub = f2i(s1v.y);
            my_recip = s1v.z;
            st.denom = s1v.w;
#pragma unroll
            for (int r = 0; r < kRows; ++r) {
                const float mu = __shfl_sync(0xffffffffu, s0.x, r);
#pragma unroll
                for (int i = 0; i < NCH * VEC; ++i)
                    c[r].v[i] = live<VEC, NCH, FULL>(i, a.width, lane) ? fadd(c[r].v[i], -mu) : 0.0f;
            }
        } else {
#pragma unroll
            for (int r = 0; r < kRows; ++r) {
                float s = 0.0f;
#pragma unroll
                for (int i = 0; i < NCH * VEC; ++i) s = fadd(s, c[r].v[i]);
                s1[r] = warp_sum(s);
                const float mu = div_by(s1[r], sh.by_n);
                s = 0.0f;
#pragma unroll
                for (int i = 0; i < NCH * VEC; ++i) {
                    c[r].v[i] = live<VEC, NCH, FULL>(i, a.width, lane) ? fadd(c[r].v[i], -mu) : 0.0f;
                    s = fadd(s, mul(c[r].v[i], c[r].v[i], a.off));
                }
                s2[r] = warp_sum(s);
            }
            st.s2 = s2[0];
            st.s1 = s1[0];
#pragma unroll
            for (int r = 1; r < kRows; ++r) {
                st.s2 = my_row == r ? s2[r] : st.s2;
                st.s1 = my_row == r ? s1[r] : st.s1;
            }
            finish_stats(st, a, sh);
            my_divisor = make_divisor(st.denom, a.off);
            my_recip = div_by(1.0f, my_divisor);
        }

        // d(out)/d(xn), the division's two gradients; g is overwritten by d_c1
        float d_denom[kRows], recip[kRows];
#pragma unroll
        for (int r = 0; r < kRows; ++r) {
            Divisor by_denom;
            by_denom.flush_max = __shfl_sync(0xffffffffu, my_divisor.flush_max, r);
            by_denom.pass_max = __shfl_sync(0xffffffffu, my_divisor.pass_max, r);
            by_denom.sub = __shfl_sync(0xffffffffu, my_divisor.sub, r);
            recip[r] = __shfl_sync(0xffffffffu, my_recip, r);
            const float denom = __shfl_sync(0xffffffffu, st.denom, r);
            const bool row_on = row0 + r < a.rows;
            float sum_dden = 0.0f;
#pragma unroll
            for (int i = 0; i < NCH * VEC; ++i) {
                const bool on = live<VEC, NCH, FULL>(i, a.width, lane) && row_on;
                const float xn = div_by(c[r].v[i], by_denom);
                float dxn = g[r].v[i];
                if (a.w) {
                    if (on) {
                        dw.v[i] = fadd(dw.v[i], APPROX ? mul(g[r].v[i], xn, a.off) : mul_bwd(w.v[i], xn, g[r].v[i], a.off));
                        db.v[i] = fadd(db.v[i], g[r].v[i]);
                    }
                    dxn = APPROX ? mul(g[r].v[i], w.v[i], a.off) : mul_bwd(xn, w.v[i], g[r].v[i], a.off);
                } else if (a.partials && on) {
                    db.v[i] = fadd(db.v[i], g[r].v[i]);
                }
                const float dden = APPROX ? -mul(div_by(xn, by_denom), dxn, a.off)
                                          : div_bwd(c[r].v[i], denom, dxn, a.off);
                if (live<VEC, NCH, FULL>(i, a.width, lane)) sum_dden = fadd(sum_dden, dden);
                g[r].v[i] = APPROX ? mul(recip[r], dxn, a.off) : mul_bwd(c[r].v[i], recip[r], dxn, 0);
            }
            d_denom[r] = warp_sum(sum_dden);
        }

        // scalar chain back through pow(v, 0.5) and the variance, for row lane % kRows
        float my_d_denom = d_denom[0];
#pragma unroll
        for (int r = 1; r < kRows; ++r) my_d_denom = my_row == r ? d_denom[r] : my_d_denom;
        const float d_e = st.v == 0.0f ? 0.0f : my_d_denom;
        const float d_m = APPROX ? mul(mul(st.e, ln2, a.off), d_e, a.off) : exp_base_bwd(st.m, d_e, sh.lb2, a.off);
        const float d_l = APPROX ? mul(d_m, 0.5f, a.off) : mul_bwd(st.l, 0.5f, d_m, a.off);
        const float d_v = APPROX ? div(div(d_l, st.v, a.off), ln2, a.off) : log_base_bwd(st.v, d_l, sh.lb2, a.off);
        const float my_d_s2 = APPROX ? mul(recip_n, d_v, a.off) : mul_bwd(st.s2, recip_n, d_v, 0);

        // c feeds the division and both operands of pam(c, c)
#pragma unroll
        for (int r = 0; r < kRows; ++r) {
            const float d_s2 = __shfl_sync(0xffffffffu, my_d_s2, r);
            float sum_dc = 0.0f;
#pragma unroll
            for (int i = 0; i < NCH * VEC; ++i) {
                const float dsq = APPROX ? mul(d_s2, c[r].v[i], a.off) : mul_bwd(c[r].v[i], c[r].v[i], d_s2, a.off);
                g[r].v[i] = fadd(fadd(g[r].v[i], dsq), dsq);
                if (live<VEC, NCH, FULL>(i, a.width, lane)) sum_dc = fadd(sum_dc, g[r].v[i]);
            }
            const float d_mu = -warp_sum(sum_dc);
            const float d_s1 = APPROX ? mul(recip_n, d_mu, a.off) : mul_bwd(s1[r], recip_n, d_mu, 0);
#pragma unroll
            for (int i = 0; i < NCH * VEC; ++i) g[r].v[i] = fadd(g[r].v[i], d_s1);
            if (row0 + r < a.rows) store_row<VEC, NCH, FULL>(g[r], a.out + (row0 + r) * a.width, a.width, lane);
        }
    }

    // per-CTA column sums for dw / db: warps are added in warp order, CTAs by the second kernel
    if (a.partials) {
        float* slot = a.partials + (int64_t)blockIdx.x * 2 * a.width;
#pragma unroll
        for (int which = 0; which < 2; ++which) {
            __syncthreads();
#pragma unroll
            for (int i = 0; i < NCH * VEC; ++i) stage[wid][i][lane] = which == 0 ? dw.v[i] : db.v[i];
            __syncthreads();
            if (wid == 0) {
#pragma unroll
                for (int i = 0; i < NCH * VEC; ++i) {
                    const int col = ((i / VEC) * 32 + lane) * VEC + (i % VEC);
                    float t = stage[0][i][lane];
#pragma unroll
                    for (int k = 1; k < kWarpsPerCta; ++k) t = fadd(t, stage[k][i][lane]);
                    if (col < a.width) slot[which * a.width + col] = t;
                }
            }
        }
    }
}

// dw[c] = sum over CTAs of partials[cta][0][c], db likewise.  One CTA per 32 columns; warp j adds
// the partials of CTAs j, j + 32, j + 64, ... in that order, then the 32 warp sums are added in
// warp order.
constexpr int kGradWarps = 32;
__global__ void __launch_bounds__(kGradWarps * 32) ln_param_grad_kernel(const float* __restrict__ partials,
                                                                       float* __restrict__ dw, float* __restrict__ db,
                                                                       int ctas, int width) {
    __shared__ float stage[2][kGradWarps][32];
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int col = blockIdx.x * 32 + lane;
    float sw = 0.0f, sb = 0.0f;
    if (col < width) {
#pragma unroll 4
        for (int k = wid; k < ctas; k += kGradWarps) {
            sw = fadd(sw, __ldg(partials + ((int64_t)k * 2) * width + col));
            sb = fadd(sb, __ldg(partials + ((int64_t)k * 2 + 1) * width + col));
        }
    }
    stage[0][wid][lane] = sw;
    stage[1][wid][lane] = sb;
    __syncthreads();
    if (wid == 0 && col < width) {
        sw = stage[0][0][lane];
        sb = stage[1][0][lane];
#pragma unroll
        for (int k = 1; k < kGradWarps; ++k) {
            sw = fadd(sw, stage[0][k][lane]);
            sb = fadd(sb, stage[1][k][lane]);
        }
        if (dw) dw[col] = sw;
        if (db) db[col] = sb;
    }
}

// Enough CTAs to fill the resident-warp slots of every SM (the backward kernel needs more registers,
// so fewer of its CTAs fit); warps walk the rows with a grid stride.
int pick_grid(int64_t rows, bool backward) {
    const int64_t want = (rows + kWarpsPerCta - 1) / kWarpsPerCta;
    const int64_t cap = (int64_t)sm_count() * (backward ? 12 : 16);
    return (int)(want < cap ? want : cap);
}

template <bool BWD, bool APPROX, bool SAVED = false>
int launch(const LnArgs& a, int grid, cudaStream_t st) {
    // register layout: VEC consecutive columns per chunk, NCH chunks per lane; the first layout
    // that holds the row with the fewest register slots wins (192 columns: 3 chunks of 2)
    const uintptr_t bits = reinterpret_cast<uintptr_t>(a.x) | reinterpret_cast<uintptr_t>(a.out) |
                           reinterpret_cast<uintptr_t>(a.w) | reinterpret_cast<uintptr_t>(a.b) |
                           reinterpret_cast<uintptr_t>(a.dy);
    const bool v4 = (a.width & 3) == 0 && (bits & 15u) == 0;
    const bool v2 = (a.width & 1) == 0 && (bits & 7u) == 0;
#define PAMK_LN(V, N)                                                                   \
    do {                                                                                \
        if (a.width == 32 * (V) * (N)) {                                                \
            if constexpr (BWD) ln_bwd_kernel<V, N, APPROX, true, SAVED><<<grid, kThreads, 0, st>>>(a); \
            else ln_fwd_kernel<V, N, true, SAVED><<<grid, kThreads, 0, st>>>(a);        \
        } else {                                                                        \
            if constexpr (BWD) ln_bwd_kernel<V, N, APPROX, false, SAVED><<<grid, kThreads, 0, st>>>(a); \
            else ln_fwd_kernel<V, N, false, SAVED><<<grid, kThreads, 0, st>>>(a);       \
        }                                                                               \
        return check_launch();                                                          \
    } while (0)
    if (v4 && a.width <= 128) PAMK_LN(4, 1);
    if (v2 && a.width <= 192) PAMK_LN(2, 3);
    if (v4 && a.width <= 256) PAMK_LN(4, 2);
    if (v4 && a.width <= 512) PAMK_LN(4, 4);
    if (v4 && a.width <= 768) PAMK_LN(4, 6);
    if (v4 && a.width <= 1024) PAMK_LN(4, 8);
    if (a.width <= 256) PAMK_LN(1, 8);
    if (a.width <= 1024) PAMK_LN(1, 32);
#undef PAMK_LN
    return PAMK_ERR_SIZE;
}

}  // namespace
}  // namespace pamk

using namespace pamk;

extern "C" {

int pamk_layer_norm_max_width(void) { return 1024; }

int pamk_layer_norm_fwd(const float* x, const float* weight, const float* bias, float* y,
                        int64_t rows, int64_t width, float eps, float offset, void* stream) {
    if (rows < 0 || width <= 0) return PAMK_ERR_ARG;
    if (width > 1024) return PAMK_ERR_SIZE;
    if (rows == 0) return PAMK_OK;
    if (!x || !y) return PAMK_ERR_ARG;
    LnArgs a{x, weight, bias, nullptr, y, nullptr, rows, (int)width, (float)width, eps, offset_bits(offset)};
    return launch<false, false>(a, pick_grid(rows, false), static_cast<cudaStream_t>(stream));
}

int pamk_layer_norm_stats_per_row(void) { return kStatCount; }

int pamk_layer_norm_fwd_save(const float* x, const float* weight, const float* bias, float* y, float* stats,
                             int64_t rows, int64_t width, float eps, float offset, void* stream) {
    if (rows < 0 || width <= 0) return PAMK_ERR_ARG;
    if (width > 1024) return PAMK_ERR_SIZE;
    if (rows == 0) return PAMK_OK;
    if (!x || !y || !stats || (reinterpret_cast<uintptr_t>(stats) & 15u)) return PAMK_ERR_ARG;
    LnArgs a{x, weight, bias, nullptr, y, nullptr, rows, (int)width, (float)width, eps, offset_bits(offset), stats};
    return launch<false, false, true>(a, pick_grid(rows, false), static_cast<cudaStream_t>(stream));
}

int pamk_layer_norm_bwd_saved(const float* x, const float* weight, const float* dy, const float* stats, float* dx,
                              float* dweight, float* dbias, int64_t rows, int64_t width, float offset,
                              void* workspace, size_t workspace_bytes, void* stream) {
    if (rows < 0 || width <= 0) return PAMK_ERR_ARG;
    if (width > 1024) return PAMK_ERR_SIZE;
    if (dweight && !weight) return PAMK_ERR_ARG;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (rows == 0) {
        if (dweight) cudaMemsetAsync(dweight, 0, width * sizeof(float), st);
        if (dbias) cudaMemsetAsync(dbias, 0, width * sizeof(float), st);
        return PAMK_OK;
    }
    if (!x || !dy || !dx || !stats || (reinterpret_cast<uintptr_t>(stats) & 15u)) return PAMK_ERR_ARG;
    const int grid = pick_grid(rows, true);
    const bool params = dweight || dbias;
    if (params && (!workspace || workspace_bytes < pamk_layer_norm_bwd_workspace_bytes(rows, width) ||
                   (reinterpret_cast<uintptr_t>(workspace) & 15u)))
        return PAMK_ERR_WORKSPACE;
    LnArgs a{x, weight, nullptr, dy, dx, params ? static_cast<float*>(workspace) : nullptr,
             rows, (int)width, (float)width, 0.0f, offset_bits(offset), const_cast<float*>(stats)};
    const int rc = launch<true, true, true>(a, grid, st);
    if (rc != PAMK_OK || !params) return rc;
    ln_param_grad_kernel<<<(unsigned)((width + 31) / 32), kGradWarps * 32, 0, st>>>(
        static_cast<const float*>(workspace), dweight, dbias, grid, (int)width);
    return check_launch();
}

size_t pamk_layer_norm_bwd_workspace_bytes(int64_t rows, int64_t width) {
    if (rows <= 0 || width <= 0) return 0;
    return (size_t)pick_grid(rows, true) * 2 * (size_t)width * sizeof(float);
}

int pamk_layer_norm_bwd(const float* x, const float* weight, const float* dy, float* dx,
                        float* dweight, float* dbias, int64_t rows, int64_t width, float eps, float offset,
                        int approx_bwd, void* workspace, size_t workspace_bytes, void* stream) {
    if (rows < 0 || width <= 0) return PAMK_ERR_ARG;
    if (width > 1024) return PAMK_ERR_SIZE;
    if (dweight && !weight) return PAMK_ERR_ARG;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (rows == 0) {
        if (dweight) cudaMemsetAsync(dweight, 0, width * sizeof(float), st);
        if (dbias) cudaMemsetAsync(dbias, 0, width * sizeof(float), st);
        return PAMK_OK;
    }
    if (!x || !dy || !dx) return PAMK_ERR_ARG;
    const int grid = pick_grid(rows, true);
    const bool params = dweight || dbias;
    if (params && (!workspace || workspace_bytes < pamk_layer_norm_bwd_workspace_bytes(rows, width) ||
                   (reinterpret_cast<uintptr_t>(workspace) & 15u)))
        return PAMK_ERR_WORKSPACE;
    LnArgs a{x, weight, nullptr, dy, dx, params ? static_cast<float*>(workspace) : nullptr,
             rows, (int)width, (float)width, eps, offset_bits(offset)};
    const int rc = approx_bwd ? launch<true, true>(a, grid, st) : launch<true, false>(a, grid, st);
    if (rc != PAMK_OK || !params) return rc;
    ln_param_grad_kernel<<<(unsigned)((width + 31) / 32), kGradWarps * 32, 0, st>>>(
        static_cast<const float*>(workspace), dweight, dbias, grid, (int)width);
    return check_launch();
}

}
