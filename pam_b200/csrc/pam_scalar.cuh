// Scalar PAM primitives: the bit-level definition of every piecewise affine operation.
//
// Each function reproduces, bit for bit, the result of the reference's device function of the
// same role in epfml/pam pam/cuda_kernels.cu (lines cited per function), but is written for how
// sm_100a executes it: the reference's comparisons against double literals become fp32 bit-pattern
// thresholds, and its double-precision pow() calls become exponent-field arithmetic with a double
// fallback only where the fp32 form would round twice.
//
// The header also compiles as plain C++ (tests build it for the host to check these formulas
// against the CPU oracle without a GPU), hence the PAM_HD shims below.
#pragma once

#include <math.h>
#include <stdint.h>

#if defined(__CUDACC__)
#define PAM_HD __host__ __device__ __forceinline__
#else
#define PAM_HD inline
#endif

namespace pamk {

constexpr int32_t kBias = 0x3f800000;       // bit pattern of 1.0f
constexpr int32_t kMant = 0x007fffff;
constexpr int32_t kSignExp = (int32_t)0xff800000u;
// |t| < 1e-37 (double literal) holds exactly for fp32 patterns <= kFlushBits, and |t| < 1e37 for
// patterns <= kPassBits (the two doubles fall strictly between neighbouring floats).
constexpr int32_t kFlushBits = 0x02081cea;
constexpr int32_t kPassBits = 0x7cf0bdc2;

#if defined(__CUDA_ARCH__)
PAM_HD int32_t f2i(float x) { return __float_as_int(x); }
PAM_HD float i2f(int32_t i) { return __int_as_float(i); }
PAM_HD float fmul(float a, float b) { return __fmul_rn(a, b); }   // never contracted into an FMA
PAM_HD float fadd(float a, float b) { return __fadd_rn(a, b); }
PAM_HD float fdiv(float a, float b) { return __fdiv_rn(a, b); }
// The reference returns the NAN macro, which nvcc folds to 0x7fc00000 in device code too.  The
// payload matters: a later pam_bwd may do integer arithmetic on these bits.
PAM_HD float quiet_nan() { return __int_as_float(0x7fc00000); }
#else
PAM_HD int32_t f2i(float x) { int32_t i; __builtin_memcpy(&i, &x, 4); return i; }
PAM_HD float i2f(int32_t i) { float x; __builtin_memcpy(&x, &i, 4); return x; }
PAM_HD float fmul(float a, float b) { volatile float r = a * b; return r; }
PAM_HD float fadd(float a, float b) { volatile float r = a + b; return r; }
PAM_HD float fdiv(float a, float b) { volatile float r = a / b; return r; }
PAM_HD float quiet_nan() { return i2f(0x7fc00000); }
#endif

// wrap-around integer add on bit patterns
PAM_HD int32_t iadd(int32_t a, int32_t b) { return (int32_t)((uint32_t)a + (uint32_t)b); }
PAM_HD int32_t isub(int32_t a, int32_t b) { return (int32_t)((uint32_t)a - (uint32_t)b); }
PAM_HD int32_t iadd3(int32_t a, int32_t b, int32_t c) { return (int32_t)((uint32_t)a + (uint32_t)b + (uint32_t)c); }

// float offset -> integer added to the result's bit pattern (cuda_kernels.cu:168)
PAM_HD int32_t offset_bits(float offset) { return isub(f2i(offset), kBias); }

// Range rule shared by pam and pad (cuda_kernels.cu:24-37, 69-82): `t` is the true fp32
// product/quotient; tiny -> +0.0f (sign dropped), in range -> the integer-arithmetic result,
// otherwise (overflow, inf, NaN) -> NaN.
PAM_HD float range_rule(float t, int32_t candidate) {
    const float mag = fabsf(t);                       // two compares and two selects, no branch
    const float kept = mag <= i2f(kPassBits) ? i2f(candidate) : quiet_nan();
    return mag <= i2f(kFlushBits) ? 0.0f : kept;
}

// cuda_kernels.cu:15-38
PAM_HD float mul(float a, float b, int32_t off) {
    return range_rule(fmul(a, b), isub(iadd(f2i(a), f2i(b)), kBias - off));
}

// Power-of-two slope of pam(a, b) w.r.t. a (sign of b included): cuda_kernels.cu:49-53
PAM_HD float mul_slope(float a, float b, int32_t off) {
    return i2f(kSignExp & iadd(iadd(f2i(b), kMant & f2i(a)), off));
}

// cuda_kernels.cu:40-58
PAM_HD float mul_bwd(float a, float b, float dc, int32_t off) { return fmul(dc, mul_slope(a, b, off)); }

// cuda_kernels.cu:60-83
PAM_HD float div(float a, float b, int32_t off) {
    return range_rule(fdiv(a, b), iadd(isub(f2i(a), f2i(b)), kBias - off));
}

// cuda_kernels.cu:85-108 (derivative w.r.t. the divisor)
PAM_HD float div_bwd(float a, float b, float dc, int32_t off) {
    const float q = i2f(f2i(div(a, b, off)) & kSignExp);
    const float bp = i2f(f2i(b) & 0x7f800000);
    return fmul(-fdiv(q, bp), dc);
}

// ---- division by a divisor that many dividends share ---------------------------------------------
// pad(a, d) needs the true quotient only to classify it (flush / pass / NaN); the result itself is
// integer arithmetic.  For a fixed divisor the classification is a pair of thresholds on |a|:
//     |a| <= flush_max  ->  +0.0f        (exactly the a with  fl(|a| / |d|) <= 0x02081cea)
//     |a| <= pass_max   ->  bits(a) - bits(d) + (0x3f800000 - off)
//     otherwise         ->  NaN          (also for NaN a: both comparisons are false)
// so a row that divides by one value pays one IEEE division per threshold instead of one per
// element.  make_divisor finds the two largest qualifying magnitudes exactly by correcting the
// rounded product F * |d| with a few trial divisions.
struct Divisor {
    float flush_max, pass_max;   // -1 when no magnitude qualifies
    int32_t sub;                 // bits(d) - (0x3f800000 - off)
};

// Largest finite m >= 0 with fl(m / d) <= bound, for finite d > 0 and a finite bound > 0 whose
// last mantissa bit is 0 (true of both thresholds).  Under round-to-nearest-even fl(q) <= bound
// holds exactly for q <= mid, the midpoint between bound and the next float (a tie goes to the
// even neighbour, which is bound).  So m qualifies iff m <= d * mid; that product is exact in
// double (24 x 25 significant bits) and is rounded toward zero to fp32.
PAM_HD float largest_dividend(float d, float bound) {
    const double mid = 0.5 * ((double)bound + (double)i2f(f2i(bound) + 1));
    const double limit = (double)d * mid;
#if defined(__CUDA_ARCH__)
    return __double2float_rz(limit);
#else
    const float fmax = i2f(0x7f7fffff);
    if (limit >= (double)fmax) return fmax;
    float m = (float)limit;                          // round to nearest, then step down if it went up
    if ((double)m > limit) m = i2f(f2i(m) - 1);
    return m;
#endif
}

PAM_HD Divisor make_divisor(float d, int32_t off) {
    Divisor r;
    r.sub = isub(f2i(d), kBias - off);
    const float ad = fabsf(d);
    if (ad > 0.0f && ad <= i2f(0x7f7fffff)) {        // finite, non-zero
        r.flush_max = largest_dividend(ad, i2f(kFlushBits));
        r.pass_max = largest_dividend(ad, i2f(kPassBits));
    } else if (ad > 0.0f) {                          // +-inf: finite / inf = 0 flushes, inf / inf = NaN
        r.flush_max = r.pass_max = i2f(0x7f7fffff);
    } else {                                         // zero (a / 0 = inf or NaN) or NaN: all NaN
        r.flush_max = r.pass_max = -1.0f;
    }
    return r;
}

// pad(a, d) for the divisor prepared by make_divisor(d, off): same bits as div(a, d, off)
PAM_HD float div_by(float a, const Divisor& d) {
    const float mag = fabsf(a);
    const float kept = mag <= d.pass_max ? i2f(isub(f2i(a), d.sub)) : quiet_nan();
    return mag <= d.flush_max ? 0.0f : kept;
}

// 2^e for an integer-valued float e, as an exact double (0 / inf outside double's range)
PAM_HD double exp2_int_d(float e) {
    if (!(e >= -1100.0f)) return e != e ? (double)e : 0.0;
    if (e > 1100.0f) return (double)INFINITY;
    return ldexp(1.0, (int)e);
}

// cuda_kernels.cu:110-113: pow(2, floor(x)) * (1 + (x - floor(x))), the bracket in fp32, the
// product in double, rounded to fp32 once.  For floor(x) in [-126, 127] the product of a value in
// [1, 2] with 2^floor(x) is exact in fp32, so a single fp32 multiply gives the same bits.
PAM_HD float exp2(float x) {
    const float fl = floorf(x);
    const float lin = fadd(1.0f, fadd(x, -fl));
    if (fl >= -126.0f && fl <= 127.0f) return fmul(lin, i2f(((int32_t)fl + 127) << 23));
    return (float)(exp2_int_d(fl) * (double)lin);
}

#if defined(__CUDACC__)
// exp2 with the double-precision form (exponents outside fp32's normal range) kept out of line, for
// kernels that unroll it over many elements per thread: 32 inlined copies of the rarely taken path were
// most of the softmax forward kernel's code, whose profile was led by instruction-fetch stalls
// (1024-long rows: 169 -> 126 us per 2^26 elements).  Same value as exp2.
static __device__ __noinline__ float exp2_wide(float fl, float lin) { return (float)(exp2_int_d(fl) * (double)lin); }
__device__ __forceinline__ float exp2_compact(float x) {
    const float fl = floorf(x);
    const float lin = fadd(1.0f, fadd(x, -fl));
    if (fl >= -126.0f && fl <= 127.0f) return fmul(lin, i2f(((int32_t)fl + 127) << 23));
    return exp2_wide(fl, lin);
}
#endif

// cuda_kernels.cu:115-123
PAM_HD float exp2_bwd(float x, float dy) { return fmul(i2f(f2i(exp2(x)) & kSignExp), dy); }

// cuda_kernels.cu:125-130: E = floor(log2f(x)); E + (x - 2^E) / 2^E evaluated in double and
// rounded once.  x - 2^E and the division by a power of two are exact in fp32 as well, so for
// E in [-126, 126] fp32 arithmetic (one rounding, in the final add) gives the same bits.
PAM_HD float log2(float x) {
    const float e = floorf(log2f(x));
    if (e >= -126.0f && e <= 126.0f) {
        const int32_t ei = (int32_t)e;
        const float p = i2f((ei + 127) << 23), pinv = i2f((127 - ei) << 23);
        return fadd(e, fmul(fadd(x, -p), pinv));
    }
    const double p = exp2_int_d(e);
    return (float)((double)e + ((double)x - p) / p);
}

// cuda_kernels.cu:132-136
PAM_HD float log2_bwd(float x, float dy) {
    const float e = floorf(log2f(x));
    if (e >= -126.0f && e <= 126.0f) return fmul(i2f((127 - (int32_t)e) << 23), dy);
    return (float)(exp2_int_d(-e) * (double)dy);
}

// Kernel-level compositions (cuda_kernels.cu:343, 385-390, 438, 480-483); lb = log2f(base).
PAM_HD float exp_base(float x, float lb, int32_t off) { return exp2(mul(x, lb, off)); }
PAM_HD float exp_base_bwd(float x, float dy, float lb, int32_t off) {
    return mul_bwd(x, lb, exp2_bwd(mul(x, lb, off), dy), off);
}
PAM_HD float log_base(float x, float lb, int32_t off) { return div(log2(x), lb, off); }
PAM_HD float log_base_bwd(float x, float dy, float lb, int32_t off) {
    return log2_bwd(x, mul_bwd(log2(x), div(1.0f, lb, off), dy, 0));
}

}  // namespace pamk
