// Fused PAM softmax and logsumexp over the last dimension, forward and backward.
//
// The reference builds both from primitives (epfml/pam pam/pam_ops.py:305-342): x*log2(e) by PAM,
// a shift by floor(max) of the WHOLE tensor, the piecewise affine exp2, an ordinary row sum and a
// PAM division (softmax) or log2 and a PAM division (logsumexp) — about ten launches each way.
// Here: one kernel finds the whole-tensor maximum of the scaled input (per-CTA maxima in scratch),
// and one row kernel does the rest with the row held in registers; every primitive goes through
// the same scalar functions as the elementwise kernels and rounds where the reference rounds.
// Traffic: 4 B/element for the maximum pass, then 8 B/element forward and 12 B/element backward.
//
// A row is owned by one warp (up to 1024 columns) or by a CTA of eight warps (up to 12288 columns,
// e.g. a 10000-word vocabulary).  -inf inputs (attention masks) get probability 0 as in the
// reference; NaN or +inf anywhere makes the shift, and with it every output, NaN as there.
#include "common.cuh"
#include "pam_scalar.cuh"

namespace pamk {
namespace {

constexpr float kLog2e = 1.44269504088896340736f;   // float(math.log2(math.e)), pam_ops.py:309
constexpr float kLn2 = 0.693147180559945309417f;    // float(math.log(2.0)), cuda_bindings.py:232

// scaled input of one element: -inf stays -inf (the reference masks it back after the PAM)
__device__ __forceinline__ float scaled_of(float x, int32_t off) {
    return x == -INFINITY ? -INFINITY : mul(x, kLog2e, off);
}

// ---- whole-tensor maximum ------------------------------------------------------------------------
// NaN is sticky, as in torch.max.  One float per CTA is written to `partials`.
__device__ __forceinline__ float nan_max(float a, float b) { return (a != a || b != b) ? quiet_nan() : fmaxf(a, b); }

__global__ void __launch_bounds__(256) scaled_max_kernel(const float* __restrict__ x, int64_t n, int32_t off,
                                                         float* __restrict__ partials) {
    __shared__ float red[8];
    float m = -INFINITY;
    const int64_t stride = (int64_t)gridDim.x * 256;
    const bool vec = aligned16(x);
    if (vec) {
        const int64_t n4 = n >> 2;
        for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < n4; i += stride) {
            const float4 v = __ldg(reinterpret_cast<const float4*>(x) + i);
            m = nan_max(m, nan_max(nan_max(scaled_of(v.x, off), scaled_of(v.y, off)),
                                   nan_max(scaled_of(v.z, off), scaled_of(v.w, off))));
        }
        for (int64_t i = (n4 << 2) + (int64_t)blockIdx.x * 256 + threadIdx.x; i < n; i += stride)
            m = nan_max(m, scaled_of(__ldg(x + i), off));
    } else {
        for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < n; i += stride)
            m = nan_max(m, scaled_of(__ldg(x + i), off));
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) m = nan_max(m, __shfl_xor_sync(0xffffffffu, m, d));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int k = 1; k < 8; ++k) m = nan_max(m, red[k]);
        partials[blockIdx.x] = m;
    }
}

// shift = floor(max over the per-CTA maxima); every thread of the row kernel computes it itself
__device__ __forceinline__ float load_shift(const float* __restrict__ partials, int count) {
    float m = -INFINITY;
    for (int k = threadIdx.x & 31; k < count; k += 32) m = nan_max(m, __ldg(partials + k));
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) m = nan_max(m, __shfl_xor_sync(0xffffffffu, m, d));
    return floorf(m);
}

// ---- rows in registers ---------------------------------------------------------------------------
struct RowArgs {
    const float* x;
    const float* g;          // backward: incoming gradient ([rows, len] softmax, [rows] logsumexp, one value for the losses)
    float* out;              // forward result or dx
    const float* partials;
    int partial_count;
    int64_t rows;
    int len;
    int32_t off;
    // loss kernels only
    const long long* target; // [rows] class index of every row
    const float* weight;     // optional per-class weights (cross-entropy gradient)
    long long ignore;        // rows whose target equals this contribute nothing (when has_ignore)
    int has_ignore;
    float c0, c1, c2;        // cross-entropy gradient: hot / cold target probability, row count (0 = no mean)
    float* aux;              // softmax forward: optional second output, the exponentials e (-0.0f where the
                             // input was -inf) for kSoftmaxBwdSaved, which takes them as x
    int post;                // softmax backward: multiply dx by post_scale (PAM product) before it is stored,
    float post_scale;        // the gradient of a PAM scaling of the scores by a constant (approx_bwd form)
};

// Thread t of a group of WARPS*32 threads holds NCH chunks of VEC consecutive columns: chunk q
// starts at column (q * WARPS*32 + t) * VEC.
template <int VEC, int NCH, int WARPS>
struct Row {
    float v[NCH * VEC];
    __device__ __forceinline__ static int col(int i, int t) { return ((i / VEC) * WARPS * 32 + t) * VEC + (i % VEC); }
    __device__ __forceinline__ void load(const float* p, int len, int t, float fill) {
#pragma unroll
        for (int q = 0; q < NCH; ++q) {
            const int c = (q * WARPS * 32 + t) * VEC;
            if (VEC == 4) {
                if (c < len) {
                    const float4 w = __ldg(reinterpret_cast<const float4*>(p + c));
                    v[q * 4] = w.x; v[q * 4 + 1] = w.y; v[q * 4 + 2] = w.z; v[q * 4 + 3] = w.w;
                } else {
                    v[q * 4] = v[q * 4 + 1] = v[q * 4 + 2] = v[q * 4 + 3] = fill;
                }
            } else {
                v[q] = c < len ? __ldg(p + c) : fill;
            }
        }
    }
    __device__ __forceinline__ void store(float* p, int len, int t) const {
#pragma unroll
        for (int q = 0; q < NCH; ++q) {
            const int c = (q * WARPS * 32 + t) * VEC;
            if (c < len) {
                if (VEC == 4) *reinterpret_cast<float4*>(p + c) = make_float4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
                else p[c] = v[q];
            }
        }
    }
};

// Sum over the group: per-thread running sum (done by the caller), butterfly over the lanes, then
// (WARPS > 1) the warp sums in warp order through shared memory.
template <int WARPS>
__device__ __forceinline__ float group_sum(float s, float* scratch) {
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) s = fadd(s, __shfl_xor_sync(0xffffffffu, s, d));
    if (WARPS == 1) return s;
    __syncthreads();
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = s;
    __syncthreads();
    float t = scratch[0];
#pragma unroll
    for (int k = 1; k < WARPS; ++k) t = fadd(t, scratch[k]);
    return t;
}

// kLossFwd / kLossBwd: label-smoothed negative log-likelihood straight from the logits (log-softmax,
// gather and row sum of fairseq's label_smoothed_nll_loss fused into the logsumexp row pass).
// kCeBwd: the gradient of pam_opt.cross_entropy (softmax - target distribution, PAM-scaled).
// kSoftmaxBwdSaved: the approximate softmax backward from the exponentials the forward pass saved
// (RowArgs::aux) instead of the input: no maximum pass and no exp2 chain.
enum Op { kSoftmaxFwd, kSoftmaxBwd, kLseFwd, kLseBwd, kLossFwd, kLossBwd, kCeBwd, kSoftmaxBwdSaved };

template <int OP, bool APPROX, int VEC, int NCH, int WARPS>
// (the backward pass from the saved exponentials on the widest one-warp layouts: capped at 128 registers for
// four CTAs per SM instead of three at 146, measured 12 % faster; a cap of 96 registers spills)
__global__ void __launch_bounds__(WARPS == 1 ? 128 : WARPS * 32, (OP == kSoftmaxBwdSaved && WARPS == 1 && VEC * NCH >= 24) ? 4 : 0)
row_kernel(const RowArgs a) {
    __shared__ float scratch[8];
    constexpr int kRowsPerCta = WARPS == 1 ? 4 : 1;
    const int t = WARPS == 1 ? (threadIdx.x & 31) : threadIdx.x;
    const int sub = WARPS == 1 ? (threadIdx.x >> 5) : 0;
    const float shift = OP == kSoftmaxBwdSaved ? 0.0f : load_shift(a.partials, a.partial_count);
    const float lb2 = log2f(2.0f);
    const int32_t off = a.off;
    using R = Row<VEC, NCH, WARPS>;

    for (int64_t row = (int64_t)blockIdx.x * kRowsPerCta + sub; row < a.rows; row += (int64_t)gridDim.x * kRowsPerCta) {
        R x, e;
        if constexpr (OP == kSoftmaxBwdSaved) {
            // the saved exponentials; -0.0f marks a masked entry (and the padding) and acts as +0 in every
            // step below: flushed products and quotients are +0, and x + (-0) = x
            e.load(a.x + row * a.len, a.len, t, -0.0f);
            const int64_t next = row + (int64_t)gridDim.x * kRowsPerCta;
            if (next < a.rows) {                               // (this kernel waits on its loads: 12 warps per SM)
                prefetch_row_l2(a.x + next * a.len, a.len, t, WARPS * 32);
                prefetch_row_l2(a.g + next * a.len, a.len, t, WARPS * 32);
            }
        } else {
            x.load(a.x + row * a.len, a.len, t, -INFINITY);   // padding behaves like a masked entry
        }
        // forward kernels: this group's next row towards the L2 while the current one is computed (measured
        // on 1024-long rows: forward 169 -> 156 us per 2^26 elements; the backward kernels, which hold three
        // rows in registers at 12 warps per SM, lose a little with it)
        if (OP == kSoftmaxFwd || OP == kLseFwd || OP == kLossFwd) {
            const int64_t next = row + (int64_t)gridDim.x * kRowsPerCta;
            if (next < a.rows) prefetch_row_l2(a.x + next * a.len, a.len, t, WARPS * 32);
        }
        float part = 0.0f;
        if constexpr (OP == kSoftmaxBwdSaved) {
#pragma unroll
            for (int i = 0; i < NCH * VEC; ++i)
                if (R::col(i, t) < a.len) part = fadd(part, e.v[i]);
        } else
#pragma unroll
        for (int i = 0; i < NCH * VEC; ++i) {
            const bool masked = x.v[i] == -INFINITY;
            const float adj = fadd(scaled_of(x.v[i], off), -shift);
            // (forward kernels and the exact backward measured faster with the compact form, the
            // approximate backward kernels with the inlined one)
            constexpr bool kCompact = OP == kSoftmaxFwd || OP == kLseFwd || OP == kLossFwd || (OP == kSoftmaxBwd && !APPROX);
            const float big = kCompact ? exp2_compact(mul(adj, lb2, off)) : exp_base(adj, lb2, off);
            e.v[i] = (OP == kSoftmaxFwd || OP == kSoftmaxBwd || OP == kCeBwd) && masked ? 0.0f : big;
            if (R::col(i, t) < a.len) part = fadd(part, e.v[i]);
        }
        const float total = group_sum<WARPS>(part, scratch);

        if (OP == kSoftmaxFwd) {
            if (a.aux) {                                       // e for the backward pass, masked entries as -0.0f
                R keep;
#pragma unroll
                for (int i = 0; i < NCH * VEC; ++i) keep.v[i] = x.v[i] == -INFINITY ? -0.0f : e.v[i];
                keep.store(a.aux + row * a.len, a.len, t);
            }
            const Divisor by_total = make_divisor(total, off);
#pragma unroll
            for (int i = 0; i < NCH * VEC; ++i) e.v[i] = div_by(e.v[i], by_total);
            e.store(a.out + row * a.len, a.len, t);
        } else if (OP == kCeBwd) {
            // pam/pam_opt.py:27-51: (softmax(x) - target distribution), PAM-scaled by the class weight,
            // the row count (reduction = mean) and the incoming gradient
            const Divisor by_total = make_divisor(total, off);
            const long long tgt = a.target[row];
            const bool ignored = a.has_ignore && tgt == a.ignore;
            const int hot = ignored ? 0 : (int)tgt;                      // ignored rows use class 0, then times 0
            const float wt = a.weight ? __ldg(a.weight + hot) : 0.0f;
            const Divisor by_rows = make_divisor(a.c2, off);
            const float gout = __ldg(a.g);
#pragma unroll
            for (int i = 0; i < NCH * VEC; ++i) {
                const int col = R::col(i, t);
                float d = fadd(div_by(e.v[i], by_total), -(col == hot ? a.c0 : a.c1));
                if (a.weight) d = mul(d, wt, off);
                if (a.has_ignore) d = fmul(d, ignored ? 0.0f : 1.0f);
                if (a.c2 > 0.0f) d = div_by(d, by_rows);
                e.v[i] = mul(d, gout, off);
            }
            e.store(a.out + row * a.len, a.len, t);
        } else if (OP == kLossFwd) {
            // lprobs = x - logsumexp(x); nll = -lprobs[target]; smooth = -(row sum of lprobs)
            const float lse = div(fadd(shift, log_base(total, lb2, 0)), kLog2e, off);
            const long long tgt = a.target[row];
            const bool ignored = a.has_ignore && tgt == a.ignore;
            float neg_sum = 0.0f, picked = 0.0f;
#pragma unroll
            for (int i = 0; i < NCH * VEC; ++i) {
                const int col = R::col(i, t);
                const float neg_lp = fadd(lse, -x.v[i]);                  // -(x - lse), exactly
                if (col < a.len) neg_sum = fadd(neg_sum, neg_lp);
                if (col == (int)tgt) picked = neg_lp;
            }
            const float smooth = group_sum<WARPS>(neg_sum, scratch);
            const float nll = group_sum<WARPS>(picked, scratch);          // one thread holds it, the others add +0
            if (t == 0) {
                a.out[row * 3] = lse;
                a.out[row * 3 + 1] = ignored ? 0.0f : nll;
                a.out[row * 3 + 2] = ignored ? 0.0f : smooth;
            }
        } else if (OP == kLossBwd) {
            // d lprobs = -(d smooth) - (d nll at the target); d lse = -(row sum of d lprobs); then the
            // logsumexp gradient chain, and x receives both contributions
            const long long tgt = a.target[row];
            const bool ignored = a.has_ignore && tgt == a.ignore;
            const float d_nll = __ldg(a.g), d_smooth = __ldg(a.g + 1);
            const float d_all = ignored ? 0.0f : -d_smooth, d_hot = ignored ? 0.0f : fadd(-d_nll, -d_smooth);
            float part_d = 0.0f;
#pragma unroll
            for (int i = 0; i < NCH * VEC; ++i) {
                const int col = R::col(i, t);
                if (col < a.len) part_d = fadd(part_d, col == (int)tgt ? d_hot : d_all);
            }
            const float gr = -group_sum<WARPS>(part_d, scratch);
            const float u = fadd(shift, log_base(total, lb2, 0));
            const float recip = div(1.0f, kLog2e, off);
            const float d_u = APPROX ? mul(recip, gr, off) : mul_bwd(u, recip, gr, 0);
            const float d_total = log_base_bwd(total, d_u, lb2, 0);
#pragma unroll
            for (int i = 0; i < NCH * VEC; ++i) {
                const int col = R::col(i, t);
                const float adj = fadd(scaled_of(x.v[i], off), -shift);
                const float d_adj = APPROX ? mul(mul(e.v[i], kLn2, off), d_total, off)
                                           : exp_base_bwd(adj, d_total, lb2, off);
                const float via_lse = APPROX ? mul(d_adj, kLog2e, off) : mul_bwd(x.v[i], kLog2e, d_adj, off);
                e.v[i] = fadd(col == (int)tgt ? d_hot : d_all, via_lse);
            }
            e.store(a.out + row * a.len, a.len, t);
        } else if (OP == kLseFwd) {
            // log2 of the row sum runs with offset 0 whatever the call's offset (pam_ops.py:341)
            const float res = div(fadd(shift, log_base(total, lb2, 0)), kLog2e, off);
            if (t == 0) a.out[row] = res;
        } else if (OP == kSoftmaxBwd || OP == kSoftmaxBwdSaved) {
            R g;
            g.load(a.g + row * a.len, a.len, t, 0.0f);
            const Divisor by_total = make_divisor(total, off);
            const float recip = div_by(1.0f, by_total);
            float dsum = 0.0f;
#pragma unroll
            for (int i = 0; i < NCH * VEC; ++i) {
                const float dden = APPROX ? -mul(div_by(div_by(e.v[i], by_total), by_total), g.v[i], off)
                                          : div_bwd(e.v[i], total, g.v[i], off);
                if (R::col(i, t) < a.len) dsum = fadd(dsum, dden);
                g.v[i] = APPROX ? mul(recip, g.v[i], off) : mul_bwd(e.v[i], recip, g.v[i], 0);
            }
            const float d_total = group_sum<WARPS>(dsum, scratch);
#pragma unroll
            for (int i = 0; i < NCH * VEC; ++i) {
                const bool masked = OP == kSoftmaxBwdSaved ? f2i(e.v[i]) == (int32_t)0x80000000 : x.v[i] == -INFINITY;
                const float adj = OP == kSoftmaxBwdSaved ? 0.0f : fadd(scaled_of(x.v[i], off), -shift);
                const float d_big = masked ? 0.0f : fadd(g.v[i], d_total);
                const float d_adj = APPROX ? mul(mul(e.v[i], kLn2, off), d_big, off)
                                           : exp_base_bwd(adj, d_big, lb2, off);
                const float d_s = masked ? 0.0f : d_adj;
                g.v[i] = APPROX ? mul(d_s, kLog2e, off) : mul_bwd(x.v[i], kLog2e, d_s, off);
                if (a.post) g.v[i] = mul(g.v[i], a.post_scale, off);
            }
            g.store(a.out + row * a.len, a.len, t);
        } else {
            const float gr = __ldg(a.g + row);
            const float u = fadd(shift, log_base(total, lb2, 0));
            const float recip = div(1.0f, kLog2e, off);
            const float d_u = APPROX ? mul(recip, gr, off) : mul_bwd(u, recip, gr, 0);
            const float d_total = log_base_bwd(total, d_u, lb2, 0);
#pragma unroll
            for (int i = 0; i < NCH * VEC; ++i) {
                const float adj = fadd(scaled_of(x.v[i], off), -shift);
                const float d_adj = APPROX ? mul(mul(e.v[i], kLn2, off), d_total, off)
                                           : exp_base_bwd(adj, d_total, lb2, off);
                e.v[i] = APPROX ? mul(d_adj, kLog2e, off) : mul_bwd(x.v[i], kLog2e, d_adj, off);
            }
            e.store(a.out + row * a.len, a.len, t);
        }
    }
}

constexpr int kMaxLen = 12288;

template <int OP, bool APPROX>
int launch_rows(const RowArgs& a, cudaStream_t st) {
    const bool vec = (a.len & 3) == 0 && aligned16(a.x) && (OP == kLseFwd || OP == kLossFwd || aligned16(a.out)) &&
                     ((OP != kSoftmaxBwd && OP != kSoftmaxBwdSaved) || aligned16(a.g)) && (a.aux == nullptr || aligned16(a.aux));
    const int64_t sms = sm_count();
#define PAMK_ROWS(V, N, W)                                                                              \
    do {                                                                                                \
        const int64_t per = (W) == 1 ? 4 : 1;                                                           \
        const int64_t want = (a.rows + per - 1) / per, cap = sms * ((W) == 1 ? 8 : 4);                  \
        row_kernel<OP, APPROX, V, N, W><<<(unsigned)(want < cap ? want : cap), (W) == 1 ? 128 : (W) * 32, 0, st>>>(a); \
        return check_launch();                                                                          \
    } while (0)
    // (the number of chunks per thread only sets how many register slots a row may fill: a shorter layout
    // for a shorter row leaves fewer idle slots and changes no sum, every thread adds its columns in the
    // same order either way)
    if (vec) {
        if (a.len <= 128) PAMK_ROWS(4, 1, 1);
        if (a.len <= 256) PAMK_ROWS(4, 2, 1);
        if (a.len <= 512) PAMK_ROWS(4, 4, 1);
        if (a.len <= 768) PAMK_ROWS(4, 6, 1);
        if (a.len <= 1024) PAMK_ROWS(4, 8, 1);
        if (a.len <= 4096) PAMK_ROWS(4, 4, 8);
        if (a.len <= kMaxLen) PAMK_ROWS(4, 12, 8);
    } else {
        if (a.len <= 64) PAMK_ROWS(1, 2, 1);
        if (a.len <= 128) PAMK_ROWS(1, 4, 1);
        if (a.len <= 224) PAMK_ROWS(1, 7, 1);
        if (a.len <= 256) PAMK_ROWS(1, 8, 1);
        if (a.len <= 1024) PAMK_ROWS(1, 32, 1);
        if (a.len <= kMaxLen) PAMK_ROWS(1, 48, 8);
    }
#undef PAMK_ROWS
    return PAMK_ERR_SIZE;
}

int max_grid(int64_t n) {
    const int64_t want = (n + 4 * 256 - 1) / (4 * 256);
    const int64_t cap = (int64_t)sm_count() * 8;
    return (int)(want < 1 ? 1 : (want < cap ? want : cap));
}

int run_rows(int op, bool approx, RowArgs a, int64_t len, float offset, void* workspace, size_t workspace_bytes, void* stream) {
    const int64_t rows = a.rows;
    if (rows < 0 || len <= 0) return PAMK_ERR_ARG;
    if (len > kMaxLen) return PAMK_ERR_SIZE;
    if (rows == 0) return PAMK_OK;
    if (!a.x || !a.out || ((op == kSoftmaxBwd || op == kSoftmaxBwdSaved || op == kLseBwd || op == kCeBwd || op == kLossBwd) && !a.g))
        return PAMK_ERR_ARG;
    if ((op == kLossFwd || op == kLossBwd || op == kCeBwd) && !a.target) return PAMK_ERR_ARG;
    const int64_t n = rows * len;
    const int grid = max_grid(n);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int32_t off = offset_bits(offset);
    if (op == kSoftmaxBwdSaved) {                     // works from the saved exponentials: no maximum pass
        a.len = (int)len;
        a.off = off;
        return launch_rows<kSoftmaxBwdSaved, true>(a, st);
    }
    if (!workspace || workspace_bytes < (size_t)grid * sizeof(float) || (reinterpret_cast<uintptr_t>(workspace) & 15u))
        return PAMK_ERR_WORKSPACE;
    float* partials = static_cast<float*>(workspace);
    scaled_max_kernel<<<grid, 256, 0, st>>>(a.x, n, off, partials);
    int rc = check_launch();
    if (rc != PAMK_OK) return rc;
    a.partials = partials;
    a.partial_count = grid;
    a.len = (int)len;
    a.off = off;
    switch (op) {
        case kSoftmaxFwd: return launch_rows<kSoftmaxFwd, false>(a, st);
        case kLseFwd: return launch_rows<kLseFwd, false>(a, st);
        case kLossFwd: return launch_rows<kLossFwd, false>(a, st);
        case kCeBwd: return launch_rows<kCeBwd, false>(a, st);
        case kSoftmaxBwd: return approx ? launch_rows<kSoftmaxBwd, true>(a, st) : launch_rows<kSoftmaxBwd, false>(a, st);
        case kLossBwd: return approx ? launch_rows<kLossBwd, true>(a, st) : launch_rows<kLossBwd, false>(a, st);
        default: return approx ? launch_rows<kLseBwd, true>(a, st) : launch_rows<kLseBwd, false>(a, st);
    }
}

RowArgs plain_rows(const float* x, const float* g, float* out, int64_t rows) {
    RowArgs a{};
    a.x = x; a.g = g; a.out = out; a.rows = rows;
    return a;
}

}  // namespace
}  // namespace pamk

using namespace pamk;

extern "C" {

int pamk_softmax_max_len(void) { return kMaxLen; }

size_t pamk_softmax_workspace_bytes(int64_t rows, int64_t len) {
    if (rows <= 0 || len <= 0) return 0;
    return (size_t)max_grid(rows * len) * sizeof(float);
}

int pamk_softmax_fwd(const float* x, float* y, int64_t rows, int64_t len, float offset,
                     void* workspace, size_t workspace_bytes, void* stream) {
    return run_rows(kSoftmaxFwd, false, plain_rows(x, nullptr, y, rows), len, offset, workspace, workspace_bytes, stream);
}

int pamk_softmax_bwd(const float* x, const float* dy, float* dx, int64_t rows, int64_t len, float offset,
                     int approx_bwd, void* workspace, size_t workspace_bytes, void* stream) {
    return run_rows(kSoftmaxBwd, approx_bwd != 0, plain_rows(x, dy, dx, rows), len, offset, workspace, workspace_bytes, stream);
}

int pamk_softmax_fwd_save(const float* x, float* y, float* e, int64_t rows, int64_t len, float offset,
                          void* workspace, size_t workspace_bytes, void* stream) {
    if (!e) return PAMK_ERR_ARG;
    RowArgs a = plain_rows(x, nullptr, y, rows);
    a.aux = e;
    return run_rows(kSoftmaxFwd, false, a, len, offset, workspace, workspace_bytes, stream);
}

int pamk_softmax_bwd_saved(const float* e, const float* dy, float* dx, int64_t rows, int64_t len, float offset,
                           int has_post_scale, float post_scale, void* stream) {
    RowArgs a = plain_rows(e, dy, dx, rows);
    a.post = has_post_scale != 0;
    a.post_scale = post_scale;
    return run_rows(kSoftmaxBwdSaved, true, a, len, offset, nullptr, 0, stream);
}

int pamk_softmax_bwd_scaled(const float* x, const float* dy, float* dx, int64_t rows, int64_t len, float offset,
                            int approx_bwd, float post_scale, void* workspace, size_t workspace_bytes, void* stream) {
    RowArgs a = plain_rows(x, dy, dx, rows);
    a.post = 1; a.post_scale = post_scale;
    return run_rows(kSoftmaxBwd, approx_bwd != 0, a, len, offset, workspace, workspace_bytes, stream);
}

int pamk_logsumexp_fwd(const float* x, float* y, int64_t rows, int64_t len, float offset,
                       void* workspace, size_t workspace_bytes, void* stream) {
    return run_rows(kLseFwd, false, plain_rows(x, nullptr, y, rows), len, offset, workspace, workspace_bytes, stream);
}

int pamk_logsumexp_bwd(const float* x, const float* dy, float* dx, int64_t rows, int64_t len, float offset,
                       int approx_bwd, void* workspace, size_t workspace_bytes, void* stream) {
    return run_rows(kLseBwd, approx_bwd != 0, plain_rows(x, dy, dx, rows), len, offset, workspace, workspace_bytes, stream);
}

int pamk_ls_loss_fwd(const float* logits, const long long* target, float* rows_out, int64_t rows, int64_t len,
                     int has_ignore, long long ignore_index, float offset,
                     void* workspace, size_t workspace_bytes, void* stream) {
    RowArgs a = plain_rows(logits, nullptr, rows_out, rows);
    a.target = target; a.has_ignore = has_ignore; a.ignore = ignore_index;
    return run_rows(kLossFwd, false, a, len, offset, workspace, workspace_bytes, stream);
}

int pamk_ls_loss_bwd(const float* logits, const long long* target, const float* grads, float* dlogits,
                     int64_t rows, int64_t len, int has_ignore, long long ignore_index, float offset, int approx_bwd,
                     void* workspace, size_t workspace_bytes, void* stream) {
    RowArgs a = plain_rows(logits, grads, dlogits, rows);
    a.target = target; a.has_ignore = has_ignore; a.ignore = ignore_index;
    return run_rows(kLossBwd, approx_bwd != 0, a, len, offset, workspace, workspace_bytes, stream);
}

int pamk_cross_entropy_bwd(const float* logits, const long long* target, const float* class_weight, const float* grad_out,
                           float* dlogits, int64_t rows, int64_t len, float hot_prob, float cold_prob, float mean_rows,
                           int has_ignore, long long ignore_index, float offset,
                           void* workspace, size_t workspace_bytes, void* stream) {
    RowArgs a = plain_rows(logits, grad_out, dlogits, rows);
    a.target = target; a.weight = class_weight; a.has_ignore = has_ignore; a.ignore = ignore_index;
    a.c0 = hot_prob; a.c1 = cold_prob; a.c2 = mean_rows;
    return run_rows(kCeBwd, false, a, len, offset, workspace, workspace_bytes, stream);
}

}
