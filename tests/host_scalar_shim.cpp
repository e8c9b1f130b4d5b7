// Test-only: builds the shipped scalar header (pam_b200/csrc/pam_scalar.cuh) for the HOST and
// wraps it in the oracle's array loops, so that the formulas the CUDA kernels use can be compared
// with the CPU oracle bit for bit on a machine without a GPU.  Only what differs between host and
// device libm (log2f) is left for the GPU tests.
#include "../pam_b200/csrc/pam_scalar.cuh"

static inline float pam(float a, float b, int off) { return pamk::mul(a, b, off); }
static inline float pam_bwd(float a, float b, float dc, int off) { return pamk::mul_bwd(a, b, dc, off); }
static inline float pad(float a, float b, int off) { return pamk::div(a, b, off); }
static inline float pad_bwd(float a, float b, float dc, int off) { return pamk::div_bwd(a, b, dc, off); }
static inline float pa_exp2(float x) { return pamk::exp2(x); }
static inline float pa_exp2_bwd(float x, float dy) { return pamk::exp2_bwd(x, dy); }
static inline float pa_log2(float x) { return pamk::log2(x); }
static inline float pa_log2_bwd(float x, float dy) { return pamk::log2_bwd(x, dy); }

#include "../oracle/array_loops.inc"

// pad(a, d) through the shared-divisor form, one divisor per call (for tests/test_scalar_header_host.py)
extern "C" void host_div_by(const float* a, float d, float* c, int64_t n, int offset) {
    const pamk::Divisor prepared = pamk::make_divisor(d, offset);
    #pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) c[i] = pamk::div_by(a[i], prepared);
}
