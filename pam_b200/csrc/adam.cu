// Fused PAM Adam update.
//
// The reference (epfml/pam submodules/fairseq/fairseq/optim/adam.py:226-252) updates every parameter
// tensor with about a dozen elementwise launches plus host-to-device copies of each scalar:
//     m  = pam(m, b1) + pam(g, 1-b1)
//     v  = pam(v, b2);  v += pam(pam(g, g), 1-b2)
//     den = pow(v, 0.5) + eps              pow(a, .5) = (a == 0) ? 0 : exp2_op(pam(log2_op(a), .5))
//     p -= pam(p, wd*lr)                   (only when weight decay is on)
//     p -= pam(pad(m, den), step_size)
// with ordinary fp32 adds/subtractions between the PAM primitives.  Here the whole rule is one pass
// per element (read p, g, m, v; write p, m, v: 28 bytes per parameter, the algorithmic minimum)
// and one launch covers a table of tensors.  Each primitive is evaluated by the same scalar
// function as the elementwise kernels and every intermediate is rounded to fp32 exactly where the
// reference materialises a tensor, so p, m and v come out bit-identical to the reference's.
#include "common.cuh"
#include "pam_scalar.cuh"

namespace pamk {
namespace {

constexpr int kTensorsPerLaunch = 256;     // (an 11 KB kernel argument: within the 32 KB that sm_70 and later take)
constexpr int kThreads = 256;
constexpr int kPerBlock = kThreads * 4;

struct AdamTable {
    float* p[kTensorsPerLaunch];
    const float* g[kTensorsPerLaunch];
    float* m[kTensorsPerLaunch];
    float* v[kTensorsPerLaunch];
    int64_t n[kTensorsPerLaunch];
    // blocks [first[k], first[k + 1]) of the launch's one-dimensional grid belong to tensor k, so that a
    // table that mixes an embedding matrix with bias vectors launches no block without work
    unsigned first[kTensorsPerLaunch + 1];
    int used;
};

struct AdamScalars {
    float b1, one_minus_b1, b2, one_minus_b2, eps, decay, step_size;
    int32_t off;
};

__device__ __forceinline__ void adam_one(float& p, float g, float& m, float& v, const AdamScalars& s, float lb2) {
    const float m1 = fadd(mul(m, s.b1, s.off), mul(g, s.one_minus_b1, s.off));
    const float v1 = fadd(mul(v, s.b2, s.off), mul(mul(g, g, s.off), s.one_minus_b2, s.off));
    const float root = v1 == 0.0f ? 0.0f
                                  : exp_base(mul(log_base(v1, lb2, s.off), 0.5f, s.off), lb2, s.off);
    const float den = fadd(root, s.eps);
    float q = p;
    if (s.decay != 0.0f) q = fadd(q, -mul(q, s.decay, s.off));
    q = fadd(q, -mul(div(m1, den, s.off), s.step_size, s.off));
    p = q;
    m = m1;
    v = v1;
}

__global__ void __launch_bounds__(kThreads) adam_kernel(const AdamTable t, const AdamScalars s) {
    int which = 0, hi = t.used;                    // largest k with first[k] <= blockIdx.x (the same for the whole CTA)
    while (hi - which > 1) {
        const int mid = (which + hi) >> 1;
        if (blockIdx.x >= t.first[mid]) which = mid; else hi = mid;
    }
    const int64_t n = t.n[which];
    const int64_t base = (int64_t)(blockIdx.x - t.first[which]) * kPerBlock;
    if (base >= n) return;
    float* __restrict__ p = t.p[which];
    const float* __restrict__ g = t.g[which];
    float* __restrict__ m = t.m[which];
    float* __restrict__ v = t.v[which];
    const float lb2 = log2f(2.0f);
    const bool vec = ((reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(g) |
                       reinterpret_cast<uintptr_t>(m) | reinterpret_cast<uintptr_t>(v)) & 15u) == 0;
    const int64_t i = base + threadIdx.x * 4;
    if (vec && i + 3 < n) {
        float4 p4 = *reinterpret_cast<const float4*>(p + i);
        const float4 g4 = __ldg(reinterpret_cast<const float4*>(g + i));
        float4 m4 = *reinterpret_cast<const float4*>(m + i);
        float4 v4 = *reinterpret_cast<const float4*>(v + i);
        adam_one(p4.x, g4.x, m4.x, v4.x, s, lb2);
        adam_one(p4.y, g4.y, m4.y, v4.y, s, lb2);
        adam_one(p4.z, g4.z, m4.z, v4.z, s, lb2);
        adam_one(p4.w, g4.w, m4.w, v4.w, s, lb2);
        *reinterpret_cast<float4*>(p + i) = p4;
        *reinterpret_cast<float4*>(m + i) = m4;
        *reinterpret_cast<float4*>(v + i) = v4;
    } else {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            if (i + c < n) {
                float pp = p[i + c], mm = m[i + c], vv = v[i + c];
                adam_one(pp, g[i + c], mm, vv, s, lb2);
                p[i + c] = pp;
                m[i + c] = mm;
                v[i + c] = vv;
            }
        }
    }
}

}  // namespace
}  // namespace pamk

using namespace pamk;

extern "C" {

int pamk_adam_step(float* const* p, const float* const* g, float* const* m, float* const* v,
                   const int64_t* n, int count,
                   float beta1, float one_minus_beta1, float beta2, float one_minus_beta2,
                   float eps, float decay, float step_size, float offset, void* stream) {
    if (count < 0) return PAMK_ERR_ARG;
    if (count == 0) return PAMK_OK;
    if (!p || !g || !m || !v || !n) return PAMK_ERR_ARG;
    const AdamScalars s{beta1, one_minus_beta1, beta2, one_minus_beta2, eps, decay, step_size, offset_bits(offset)};
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    for (int k = 0; k < count;) {
        AdamTable t{};
        int used = 0;
        int64_t blocks = 0;
        for (; k < count && used < kTensorsPerLaunch; ++k) {     // k carries on where the last table ended
            if (n[k] < 0) return PAMK_ERR_ARG;
            if (n[k] == 0) continue;
            if (!p[k] || !g[k] || !m[k] || !v[k]) return PAMK_ERR_ARG;
            const int64_t mine = (n[k] + kPerBlock - 1) / kPerBlock;
            if (blocks + mine > 0x7fffffff) {                    // this tensor starts the next table
                if (used == 0) return PAMK_ERR_SIZE;
                break;
            }
            t.p[used] = p[k]; t.g[used] = g[k]; t.m[used] = m[k]; t.v[used] = v[k]; t.n[used] = n[k];
            t.first[used] = (unsigned)blocks;
            blocks += mine;
            ++used;
        }
        if (used == 0) continue;
        t.first[used] = (unsigned)blocks;
        t.used = used;
        adam_kernel<<<(unsigned)blocks, kThreads, 0, st>>>(t, s);
        const int rc = check_launch();
        if (rc != PAMK_OK) return rc;
    }
    return PAMK_OK;
}

}
