// Integer-bit tracking of the WRAP-mode quantizers in training: i <- max(i - decay, fewest integer bits that hold the
// abs-max statistic), one launch per quantizer instead of a chain of a dozen element-wise launches on bitwidth-shaped
// tensors (these chains, not the activation kernels, set the step time of small models).
//
// Stands in for the training branch of FixedPointQuantizerKIF.call / FixedPointQuantizerKBI.call
// (src/hgq/quantizer/internal/fixed_point_quantizer.py:401-411, 277-288) with minimal_i_given_xf / minimal_i_given_xb
// (:25-31, :16-22).  Every step is an explicit fp32 operation in the reference's order (log2f, ceilf, IEEE division), so
// the integer bits come out identical to the element-wise formulation.
#include <cuda_runtime.h>

#include "hgq_common.cuh"

namespace hgq {

constexpr float kKerasEps = 1e-7f;

// torch.maximum: a NaN on either side propagates (fmaxf would drop it)
__device__ __forceinline__ float max_nan(float a, float b) { return (a != a || b != b) ? __fadd_rn(a, b) : fmaxf(a, b); }

// absmax >= 0 by construction, so the reference's branch for negative statistics is never selected
__global__ void __launch_bounds__(kThreads) k_track_kif(const float *__restrict__ absmax, const float *__restrict__ f_raw,
                                                       float *__restrict__ i_state, const float *__restrict__ decay, int64_t n) {
    const int64_t e = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    if (e >= n) return;
    const float f = rintf(__ldg(f_raw + e));                       // round_conv(f)
    const float x = __ldg(absmax + e);
    const float need = ceilf(log2f(__fadd_rn(x, exp2f(-f))));      // symmetric or not: |x| = x here
    i_state[e] = max_nan(__fsub_rn(i_state[e], __ldg(decay)), need);
}

__global__ void __launch_bounds__(kThreads) k_track_kbi(const float *__restrict__ absmax, const float *__restrict__ b_raw,
                                                       float *__restrict__ i_state, const float *__restrict__ decay, float lo,
                                                       float hi, int64_t n) {
    const int64_t e = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    if (e >= n) return;
    const float b = rintf(__ldg(b_raw + e));                       // round_conv(b)
    const float x = __ldg(absmax + e);
    const float den = __fadd_rn(__fsub_rn(1.f, exp2f(-b)), kKerasEps);
    float need = ceilf(log2f(__fdiv_rn(__fadd_rn(x, kKerasEps), den)));
    if (!(b > 0.f)) need = 32.f;                                   // no bits at all: the reference parks i at 32 (symmetric: as computed)
    float v = max_nan(__fsub_rn(i_state[e], __ldg(decay)), need);
    if (v == v) v = fminf(fmaxf(v, lo), hi);                       // the variable's MinMax constraint (+-inf: none); NaN stays
    i_state[e] = v;
}

__global__ void __launch_bounds__(kThreads) k_track_kbi_sym(const float *__restrict__ absmax, const float *__restrict__ b_raw,
                                                           float *__restrict__ i_state, const float *__restrict__ decay, float lo,
                                                           float hi, int64_t n) {
    const int64_t e = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    if (e >= n) return;
    const float b = rintf(__ldg(b_raw + e));
    const float x = __ldg(absmax + e);
    const float den = __fadd_rn(__fsub_rn(1.f, exp2f(-b)), kKerasEps);
    const float need = ceilf(log2f(__fdiv_rn(__fadd_rn(x, kKerasEps), den)));
    float v = max_nan(__fsub_rn(i_state[e], __ldg(decay)), need);
    if (v == v) v = fminf(fmaxf(v, lo), hi);
    i_state[e] = v;
}

}  // namespace hgq

using namespace hgq;

extern "C" int hgq_track_kif(const float *absmax, const float *f_raw, float *i_state, const float *decay, int64_t n, void *stream) {
    if (absmax == nullptr || f_raw == nullptr || i_state == nullptr || decay == nullptr) return HGQ_ERR_NULL;
    if (n <= 0) return HGQ_ERR_SIZE;
    k_track_kif<<<(unsigned)((n + kThreads - 1) / kThreads), kThreads, 0, (cudaStream_t)stream>>>(absmax, f_raw, i_state, decay, n);
    return check_launch();
}

extern "C" int hgq_track_kbi(const float *absmax, const float *b_raw, float *i_state, const float *decay, int symmetric, float lo,
                             float hi, int64_t n, void *stream) {
    if (absmax == nullptr || b_raw == nullptr || i_state == nullptr || decay == nullptr) return HGQ_ERR_NULL;
    if (n <= 0) return HGQ_ERR_SIZE;
    const unsigned grid = (unsigned)((n + kThreads - 1) / kThreads);
    if (symmetric)
        k_track_kbi_sym<<<grid, kThreads, 0, (cudaStream_t)stream>>>(absmax, b_raw, i_state, decay, lo, hi, n);
    else
        k_track_kbi<<<grid, kThreads, 0, (cudaStream_t)stream>>>(absmax, b_raw, i_state, decay, lo, hi, n);
    return check_launch();
}
