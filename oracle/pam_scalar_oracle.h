/*
 * TEST INFRASTRUCTURE — CPU oracle for the PAM (piecewise affine multiplication) primitives.
 *
 * A plain-C restatement of the bit-level semantics of the reference's scalar device functions
 * (epfml/pam, pam/cuda_kernels.cu:15-136).  Nothing in the shipped package may include, link or
 * call this file; only the test-suite, the smoke check and the benchmark's CPU-baseline leg do.
 *
 * Parity status: pinned.  The 15 known-answer triples and 6 inf/NaN pairs of the reference's
 * pam/test_pam.py:13-29,36-43 are checked against these functions, and every function here is
 * compared bit-for-bit with the reference's own scalar functions compiled for the host
 * (oracle/_ref/libpam_ref.so, built by oracle/build.py from pam/cuda_kernels.cu where it lies).
 *
 * Arithmetic notes that matter for bit-exactness:
 *   - integer adds wrap around (done in uint32_t here; the reference relies on int overflow);
 *   - the range tests compare an fp32 magnitude with the *double* literals 1e-37 / 1e37;
 *   - fp32 products/quotients are IEEE round-to-nearest with denormals honoured (build this
 *     file without -ffast-math and without flush-to-zero);
 *   - pow(2, float) and the surrounding expression are evaluated in double in the reference
 *     (C++ promotion of pow(int,float)), and rounded to fp32 once at the return.
 */
#ifndef PAM_SCALAR_ORACLE_H
#define PAM_SCALAR_ORACLE_H

#include <math.h>
#include <stdint.h>
#include <string.h>

#define ORC_BIAS 0x3f800000u
#define ORC_MANT 0x007fffffu

static inline uint32_t orc_bits(float x) { uint32_t u; memcpy(&u, &x, 4); return u; }
static inline float orc_float(uint32_t u) { float x; memcpy(&x, &u, 4); return x; }

/* Three-way range rule shared by pam and pad: |t| < 1e-37 -> +0, < 1e37 -> candidate, else NaN.
 * pam/cuda_kernels.cu:24-37 and :69-82. */
static inline float orc_range_rule(float t, uint32_t candidate) {
    float mag = t < 0 ? -t : t;
    if ((double)mag < 1e-37) return 0.0f;
    if ((double)mag < 1e37) return orc_float(candidate);
    return NAN;
}

/* pam/cuda_kernels.cu:15-38 */
static inline float pam(float a, float b, int offset) {
    uint32_t ci = orc_bits(a) + orc_bits(b) - (ORC_BIAS - (uint32_t)offset);
    return orc_range_rule(a * b, ci);
}

/* pam/cuda_kernels.cu:40-58 — derivative w.r.t. a, times delta_c */
static inline float pam_bwd(float a, float b, float delta_c, int offset) {
    uint32_t si = ~ORC_MANT & (orc_bits(b) + (ORC_MANT & orc_bits(a)) + (uint32_t)offset);
    return delta_c * orc_float(si);
}

/* pam/cuda_kernels.cu:60-83 */
static inline float pad(float a, float b, int offset) {
    uint32_t ci = orc_bits(a) - orc_bits(b) + (ORC_BIAS - (uint32_t)offset);
    return orc_range_rule(a / b, ci);
}

/* pam/cuda_kernels.cu:85-108 — derivative w.r.t. b, times delta_c */
static inline float pad_bwd(float a, float b, float delta_c, int offset) {
    float q = pad(a, b, offset);
    float q_pow2 = orc_float(orc_bits(q) & ~ORC_MANT);      /* keeps the sign */
    float b_pow2 = orc_float(orc_bits(b) & 0x7f800000u);    /* 2^E_b */
    return -(q_pow2 / b_pow2) * delta_c;
}

/* pam/cuda_kernels.cu:110-113 */
static inline float pa_exp2(float x) {
    float fl = floorf(x);
    float lin = 1 + (x - fl);                                /* fp32 */
    return (float)(pow(2.0, (double)fl) * (double)lin);      /* double product, one rounding */
}

/* pam/cuda_kernels.cu:115-123 */
static inline float pa_exp2_bwd(float x, float dy) {
    float slope = orc_float(orc_bits(pa_exp2(x)) & ~ORC_MANT);
    return slope * dy;
}

/* pam/cuda_kernels.cu:125-130 */
static inline float pa_log2(float x) {
    float e = floorf(log2f(x));
    double p = pow(2.0, (double)e);
    double frac = ((double)x - p) / p;
    return (float)((double)e + frac);
}

/* pam/cuda_kernels.cu:132-136 */
static inline float pa_log2_bwd(float x, float dy) {
    float e = floorf(log2f(x));
    return (float)(pow(2.0, (double)(-e)) * (double)dy);
}

#endif
