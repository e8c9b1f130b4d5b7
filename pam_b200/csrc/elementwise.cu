// Elementwise PAM kernels: pam / pad forward and exact backward, base^x and log_base(x).
//
// HBM-bound (8-16 bytes per element), so the design is about bytes in flight: 128-bit loads and
// stores, two independent vectors per operand per thread, full occupancy, and broadcast operands (scalars, row vectors, per-row values) read in place
// instead of being expanded to full size as the reference does
// (epfml/pam pam/cuda_kernels.cu:141-516, one thread per element over .flatten()ed inputs).
#include "common.cuh"
#include "pam_scalar.cuh"

namespace pamk {
namespace {

struct Operand {
    const float* p;
    int kind;
    float imm;
};

struct Shape {
    int64_t n;        // output elements
    int64_t inner;    // length of the last dimension for PAMK_ROW / PAMK_COL operands
};

__device__ __forceinline__ float load1(const Operand& o, int64_t i, const Shape& s, float splat) {
    switch (o.kind) {
        case PAMK_FULL: return o.p[i];
        case PAMK_ROW: return o.p[s.n <= 0x7fffffff ? (int64_t)((uint32_t)i % (uint32_t)s.inner) : i % s.inner];
        case PAMK_COL: return o.p[s.n <= 0x7fffffff ? (int64_t)((uint32_t)i / (uint32_t)s.inner) : i / s.inner];
        default: return splat;
    }
}

// Vector form; the launcher guarantees i % 4 == 0, 16-byte aligned pointers and inner % 4 == 0
// whenever a ROW / COL operand is present, so the four lanes never straddle a row.
__device__ __forceinline__ float4 load4(const Operand& o, int64_t i, const Shape& s, float splat) {
    switch (o.kind) {
        case PAMK_FULL: return __ldg(reinterpret_cast<const float4*>(o.p + i));
        case PAMK_ROW: {
            const int64_t j = s.n <= 0x7fffffff ? (int64_t)((uint32_t)i % (uint32_t)s.inner) : i % s.inner;
            return __ldg(reinterpret_cast<const float4*>(o.p + j));
        }
        case PAMK_COL: {
            const int64_t r = s.n <= 0x7fffffff ? (int64_t)((uint32_t)i / (uint32_t)s.inner) : i / s.inner;
            const float v = __ldg(o.p + r);
            return make_float4(v, v, v, v);
        }
        default: return make_float4(splat, splat, splat, splat);
    }
}

__device__ __forceinline__ float splat_value(const Operand& o) {
    return o.kind == PAMK_SCALAR ? __ldg(o.p) : o.imm;
}

struct PamFwd {
    int32_t off;
    __device__ void prepare() {}
    __device__ float operator()(float a, float b, float) const { return mul(a, b, off); }
};
struct PadFwd {
    int32_t off;
    __device__ void prepare() {}
    __device__ float operator()(float a, float b, float) const { return div(a, b, off); }
};
struct PamBwd {
    int32_t off;
    __device__ void prepare() {}
    __device__ float operator()(float a, float b, float dc) const { return mul_bwd(a, b, dc, off); }
};
struct PadBwd {
    int32_t off;
    __device__ void prepare() {}
    __device__ float operator()(float a, float b, float dc) const { return div_bwd(a, b, dc, off); }
};
// Unary ops take x in slot 0 and, for the backward forms, dy in slot 1.
struct ExpFwd {
    int32_t off; float base;
    __device__ void prepare() {}
    __device__ float operator()(float x, float, float) const { return exp_base(x, log2f(base), off); }
};
struct ExpBwd {
    int32_t off; float base;
    __device__ void prepare() {}
    __device__ float operator()(float x, float dy, float) const { return exp_base_bwd(x, dy, log2f(base), off); }
};
// log_base(x) = pad(log2 x, log2f(base)): the divisor is the same for every element, so its two
// range thresholds are prepared once per thread (pam_scalar.cuh make_divisor) instead of dividing
// per element.  prepare() runs once per thread before the first element.
struct LogFwd {
    int32_t off; float base;
    Divisor by_lb;
    __device__ void prepare() { by_lb = make_divisor(log2f(base), off); }
    __device__ float operator()(float x, float, float) const { return div_by(log2(x), by_lb); }
};
struct LogBwd {
    int32_t off; float base;
    float inv_lb;                                   // pad(1, log2f(base))
    __device__ void prepare() { inv_lb = div(1.0f, log2f(base), off); }
    __device__ float operator()(float x, float dy, float) const {
        return log2_bwd(x, mul_bwd(log2(x), inv_lb, dy, 0));
    }
};

constexpr int kThreads = 256;
constexpr int kPerThread = 8;                       // two 128-bit vectors per operand per thread
constexpr int kPerBlock = kThreads * kPerThread;

// One CTA covers 2048 consecutive outputs: thread t takes the four at 4t and the four at
// 1024 + 4t, so each 128-bit access of a warp is one contiguous 512-byte run.  All loads of a
// thread are issued before its first use.  The grid is sized to the data (no persistent loop),
// with 32 registers or fewer per thread so that every SM holds its full 2048 threads.
template <class Op, int NIN, bool VEC>
__global__ void __launch_bounds__(kThreads, NIN > 2 ? 6 : 8) ew_kernel(Op op, Operand o0, Operand o1, Operand o2,
                                                         float* __restrict__ out, Shape s) {
    op.prepare();
    const float s0 = splat_value(o0);
    const float s1 = NIN > 1 ? splat_value(o1) : 0.0f;
    const float s2 = NIN > 2 ? splat_value(o2) : 0.0f;
    const int64_t base = (int64_t)blockIdx.x * kPerBlock;
    if (VEC) {
        const int64_t n4 = s.n & ~(int64_t)3;
        const int64_t i = base + threadIdx.x * 4, j = i + kThreads * 4;
        const bool one = i < n4, two = j < n4;
        if (one) {
            const float4 a0 = load4(o0, i, s, s0);
            const float4 b0 = NIN > 1 ? load4(o1, i, s, s1) : a0;
            const float4 c0 = NIN > 2 ? load4(o2, i, s, s2) : a0;
            float4 a1 = a0, b1 = b0, c1 = c0;
            if (two) {
                a1 = load4(o0, j, s, s0);
                if (NIN > 1) b1 = load4(o1, j, s, s1);
                if (NIN > 2) c1 = load4(o2, j, s, s2);
            }
            float4 r;
            r.x = op(a0.x, b0.x, c0.x); r.y = op(a0.y, b0.y, c0.y);
            r.z = op(a0.z, b0.z, c0.z); r.w = op(a0.w, b0.w, c0.w);
            *reinterpret_cast<float4*>(out + i) = r;
            if (two) {
                r.x = op(a1.x, b1.x, c1.x); r.y = op(a1.y, b1.y, c1.y);
                r.z = op(a1.z, b1.z, c1.z); r.w = op(a1.w, b1.w, c1.w);
                *reinterpret_cast<float4*>(out + j) = r;
            }
        }
        // ragged tail (fewer than four elements), done by the last CTA
        if (blockIdx.x == gridDim.x - 1) {
            const int64_t t = n4 + threadIdx.x;
            if (t < s.n)
                out[t] = op(load1(o0, t, s, s0), NIN > 1 ? load1(o1, t, s, s1) : 0.0f,
                            NIN > 2 ? load1(o2, t, s, s2) : 0.0f);
        }
    } else {
#pragma unroll
        for (int u = 0; u < kPerThread; ++u) {
            const int64_t i = base + threadIdx.x + u * kThreads;
            if (i < s.n)
                out[i] = op(load1(o0, i, s, s0), NIN > 1 ? load1(o1, i, s, s1) : 0.0f,
                            NIN > 2 ? load1(o2, i, s, s2) : 0.0f);
        }
    }
}

// An empty launch (n == 0) may carry null pointers: an empty tensor has no storage.
bool operand_ok(const Operand& o, int64_t n) {
    if (o.kind < PAMK_FULL || o.kind > PAMK_IMM) return false;
    return o.kind == PAMK_IMM || o.p != nullptr || n == 0;
}

bool operand_vectorisable(const Operand& o, int64_t inner) {
    switch (o.kind) {
        case PAMK_FULL: return aligned16(o.p);
        case PAMK_ROW: return aligned16(o.p) && inner % 4 == 0;
        case PAMK_COL: return inner % 4 == 0;
        default: return true;
    }
}

template <class Op, int NIN>
int launch(Op op, Operand o0, Operand o1, Operand o2, float* out, int64_t n, int64_t inner, void* stream) {
    if (n < 0 || (out == nullptr && n > 0)) return PAMK_ERR_ARG;
    if (!operand_ok(o0, n) || (NIN > 1 && !operand_ok(o1, n)) || (NIN > 2 && !operand_ok(o2, n))) return PAMK_ERR_ARG;
    const bool needs_inner = o0.kind == PAMK_ROW || o0.kind == PAMK_COL ||
                             (NIN > 1 && (o1.kind == PAMK_ROW || o1.kind == PAMK_COL)) ||
                             (NIN > 2 && (o2.kind == PAMK_ROW || o2.kind == PAMK_COL));
    if (needs_inner && (inner <= 0 || n % inner != 0)) return PAMK_ERR_ARG;
    if (n == 0) return PAMK_OK;
    if (inner <= 0) inner = n;
    const bool vec = aligned16(out) && operand_vectorisable(o0, inner) &&
                     (NIN < 2 || operand_vectorisable(o1, inner)) && (NIN < 3 || operand_vectorisable(o2, inner));
    const Shape s{n, inner};
    const int64_t blocks = (n + kPerBlock - 1) / kPerBlock;
    if (blocks > 0x7fffffff) return PAMK_ERR_SIZE;
    const unsigned grid = (unsigned)blocks;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (vec) ew_kernel<Op, NIN, true><<<grid, kThreads, 0, st>>>(op, o0, o1, o2, out, s);
    else ew_kernel<Op, NIN, false><<<grid, kThreads, 0, st>>>(op, o0, o1, o2, out, s);
    return check_launch();
}

const Operand kNone{nullptr, PAMK_IMM, 0.0f};

}  // namespace
}  // namespace pamk

using namespace pamk;

extern "C" {

int pamk_pam_fwd(const float* a, int a_kind, float a_imm, const float* b, int b_kind, float b_imm,
                 float* out, int64_t n, int64_t inner, float offset, void* stream) {
    return launch<PamFwd, 2>(PamFwd{offset_bits(offset)}, {a, a_kind, a_imm}, {b, b_kind, b_imm}, kNone,
                             out, n, inner, stream);
}

int pamk_pad_fwd(const float* a, int a_kind, float a_imm, const float* b, int b_kind, float b_imm,
                 float* out, int64_t n, int64_t inner, float offset, void* stream) {
    return launch<PadFwd, 2>(PadFwd{offset_bits(offset)}, {a, a_kind, a_imm}, {b, b_kind, b_imm}, kNone,
                             out, n, inner, stream);
}

int pamk_pam_bwd(const float* a, int a_kind, float a_imm, const float* b, int b_kind, float b_imm,
                 const float* dc, int dc_kind, float dc_imm,
                 float* out, int64_t n, int64_t inner, float offset, void* stream) {
    return launch<PamBwd, 3>(PamBwd{offset_bits(offset)}, {a, a_kind, a_imm}, {b, b_kind, b_imm},
                             {dc, dc_kind, dc_imm}, out, n, inner, stream);
}

int pamk_pad_bwd(const float* a, int a_kind, float a_imm, const float* b, int b_kind, float b_imm,
                 const float* dc, int dc_kind, float dc_imm,
                 float* out, int64_t n, int64_t inner, float offset, void* stream) {
    return launch<PadBwd, 3>(PadBwd{offset_bits(offset)}, {a, a_kind, a_imm}, {b, b_kind, b_imm},
                             {dc, dc_kind, dc_imm}, out, n, inner, stream);
}

int pamk_pa_exp_fwd(const float* x, float* y, int64_t n, float base, float offset, void* stream) {
    return launch<ExpFwd, 1>(ExpFwd{offset_bits(offset), base}, {x, PAMK_FULL, 0.f}, kNone, kNone, y, n, 0, stream);
}

int pamk_pa_exp_bwd(const float* x, const float* dy, float* dx, int64_t n, float base, float offset,
                    void* stream) {
    return launch<ExpBwd, 2>(ExpBwd{offset_bits(offset), base}, {x, PAMK_FULL, 0.f}, {dy, PAMK_FULL, 0.f}, kNone,
                             dx, n, 0, stream);
}

int pamk_pa_log_fwd(const float* x, float* y, int64_t n, float base, float offset, void* stream) {
    return launch<LogFwd, 1>(LogFwd{offset_bits(offset), base}, {x, PAMK_FULL, 0.f}, kNone, kNone, y, n, 0, stream);
}

int pamk_pa_log_bwd(const float* x, const float* dy, float* dx, int64_t n, float base, float offset,
                    void* stream) {
    return launch<LogBwd, 2>(LogBwd{offset_bits(offset), base}, {x, PAMK_FULL, 0.f}, {dy, PAMK_FULL, 0.f}, kNone,
                             dx, n, 0, stream);
}

}
