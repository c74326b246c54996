// Batched parameter-side kernels of a QAT step: everything that touches only bitwidth-shaped tensors and weights, for
// ALL quantizers and ALL layers of a model in one launch each, driven by descriptor tables in device memory.
//
// The reference does this work as several hundred eager element-wise launches per step on tensors of a few hundred
// elements (round_conv of every b / i / f, f = b - i, b = relu(i + f), bits = b (+ k), the weight and bias quantizer
// calls, the integer-bit tracking of every WRAP quantizer, and the autograd backward of all of it):
//   src/hgq/quantizer/internal/fixed_point_quantizer.py:92-97,244-307,401-449 (properties, KBI.call, KIF.call),
//   src/hgq/quantizer/internal/base.py:19-28 (round_conv, straight-through), src/hgq/layers/core/dense.py:93-102
//   (qkernel / qbias).
// Here a step runs five launches:
//   tables_forward    I = rint(i), F = rint(f) or rint(b) - rint(i)                               (before the forward pass)
//   weights_forward   quantised kernel and bias of every layer; WRAP quantizers of weights / biases track their integer
//                     bits in the same pass                                                       (before the forward pass)
//   tables_track_bits i <- max(i - decay, fewest bits that hold the abs-max statistic) for every tracked activation
//                     quantizer, then BITS = relu(I + F) or rint(b), (+ k for SAT)                (after the forward pass)
//   weights_backward  dL/dWq -> dL/dW, and the surrogate gradients to the weight quantizers' tables
//   tables_backward   gradients w.r.t. the derived tables (dI, dF, dBITS, written by the layer kernels and the EBOPs
//                     kernels) -> gradients of the raw variables, straight into the flat gradient bucket
// Grid = (ceil(max_n / 256), number of descriptors); a block whose descriptor has fewer entries exits at once.
// Latency-bound (10^3..10^5 elements in total): what is being removed is launches, not bytes.
#include <cuda_runtime.h>

#include "hgq_common.cuh"
#include "hgq_math.cuh"

namespace hgq {

constexpr float kKerasEpsP = 1e-7f;

__device__ __forceinline__ float max_nan_p(float a, float b) { return (a != a || b != b) ? __fadd_rn(a, b) : fmaxf(a, b); }

// fewest integer bits that hold x >= 0 with f fractional bits / with b bits in total: the op sequences of track.cu
__device__ __forceinline__ float minimal_i_xf(float x, float f) { return ceilf(log2f(__fadd_rn(x, exp2f(-f)))); }
__device__ __forceinline__ float minimal_i_xb(float x, float b, bool symmetric) {
    const float den = __fadd_rn(__fsub_rn(1.f, exp2f(-b)), kKerasEpsP);
    float need = ceilf(log2f(__fdiv_rn(__fadd_rn(x, kKerasEpsP), den)));
    if (!symmetric && !(b > 0.f)) need = 32.f;
    return need;
}

__global__ void __launch_bounds__(kThreads) k_tables_forward(const hgq_slot_desc *__restrict__ slots) {
    const hgq_slot_desc &s = slots[blockIdx.y];
    const int64_t e = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    if (e >= s.n) return;
    const float I = rintf(s.i_raw[e]);
    const float a = rintf(s.a_raw[e]);
    s.I[e] = I;
    s.F[e] = (s.kind == HGQ_SLOT_KBI) ? __fsub_rn(a, I) : a;
}

__global__ void __launch_bounds__(kThreads) k_tables_track_bits(const hgq_slot_desc *__restrict__ slots) {
    const hgq_slot_desc &s = slots[blockIdx.y];
    const int64_t e = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    if (e >= s.n) return;
    float I = s.I[e];
    if (s.absmax != nullptr) {  // a tracked activation quantizer (KIF): the statistic is max |round(x, f)|
        const float v = max_nan_p(__fsub_rn(s.i_raw[e], *s.decay), minimal_i_xf(s.absmax[e], s.F[e]));
        s.i_raw[e] = v;
        I = rintf(v);
        s.I[e] = I;
    } else if (s.tracked_weight) {  // the weights pass moved i
        I = rintf(s.i_raw[e]);
        s.I[e] = I;
    }
    float b;
    if (s.kind == HGQ_SLOT_KBI) b = rintf(s.a_raw[e]);
    else b = fmaxf(__fadd_rn(I, s.F[e]), 0.f);
    if (s.om == OM_SAT) b = __fadd_rn(b, (float)s.k[e]);
    s.BITS[e] = b;
}

__global__ void __launch_bounds__(kThreads) k_tables_backward(const hgq_slot_desc *__restrict__ slots) {
    const hgq_slot_desc &s = slots[blockIdx.y];
    const int64_t e = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    if (e >= s.n) return;
    const float dI = s.dI[e], dF = s.dF[e], dB = s.dBITS[e];
    if (s.kind == HGQ_SLOT_KBI) {  // f = b - i, bits = b (+ k)
        if (s.g_a) s.g_a[e] = __fadd_rn(dF, dB);
        if (s.g_i) s.g_i[e] = __fsub_rn(dI, dF);
    } else {                       // bits = relu(i + f) (+ k)
        const float m = (__fadd_rn(s.I[e], s.F[e]) > 0.f) ? dB : 0.f;
        if (s.g_a) s.g_a[e] = __fadd_rn(dF, m);
        if (s.g_i) s.g_i[e] = __fadd_rn(dI, m);
    }
}

__global__ void __launch_bounds__(kThreads) k_weights_forward(const hgq_weight_desc *__restrict__ ws,
                                                             const hgq_slot_desc *__restrict__ slots) {
    const hgq_weight_desc &w = ws[blockIdx.y];
    const int64_t e = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    if (e >= w.n) return;
    const hgq_slot_desc &s = slots[w.slot];
    const float x = w.w_raw[e];
    const float kf = (float)s.k[e];
    float rounded;
    if (w.mode == HGQ_WEIGHT_QUANTIZE) {
        w.wq[e] = quantize_rt(x, kf, s.I[e], s.F[e], s.rm, s.om, false, rounded);
    } else if (w.mode == HGQ_WEIGHT_ROUND) {
        w.wq[e] = quantize_rt(x, kf, 0.f, s.F[e], s.rm, OM_NONE, false, rounded);
    } else if (s.kind == HGQ_SLOT_KBI) {
        // WRAP in training, (k, b, i) parametrisation: the integer bits follow |x| first, then f = b - i rounds
        const float b = rintf(s.a_raw[e]);
        float v = max_nan_p(__fsub_rn(s.i_raw[e], *s.decay), minimal_i_xb(fabsf(x), b, s.symmetric != 0));
        if (v == v) v = fminf(fmaxf(v, s.i_lo), s.i_hi);
        s.i_raw[e] = v;
        const float I = rintf(v), F = __fsub_rn(b, I);
        s.I[e] = I;
        s.F[e] = F;
        w.wq[e] = quantize_rt(x, kf, 0.f, F, s.rm, OM_NONE, false, rounded);
    } else {
        // WRAP in training, (k, i, f) parametrisation: round, then the integer bits follow |round(x)|
        const float F = s.F[e];
        const float y = quantize_rt(x, kf, 0.f, F, s.rm, OM_NONE, false, rounded);
        w.wq[e] = y;
        const float v = max_nan_p(__fsub_rn(s.i_raw[e], *s.decay), minimal_i_xf(fabsf(y), F));
        s.i_raw[e] = v;
        s.I[e] = rintf(v);
    }
}

__global__ void __launch_bounds__(kThreads) k_weights_backward(const hgq_weight_desc *__restrict__ ws,
                                                              const hgq_slot_desc *__restrict__ slots) {
    const hgq_weight_desc &w = ws[blockIdx.y];
    const int64_t e = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    if (e >= w.n) return;
    const hgq_slot_desc &s = slots[w.slot];
    const int om = (w.mode == HGQ_WEIGHT_QUANTIZE) ? s.om : OM_NONE;
    float dx, di, df;
    quantize_grad_rt(w.dwq[e], w.w_raw[e], (float)s.k[e], (om == OM_NONE) ? 0.f : s.I[e], s.F[e], s.rm, om, dx, di, df);
    if (w.g_w) w.g_w[e] = dx;
    s.dI[e] = di;
    s.dF[e] = df;
}

template <typename D>
static int launch_over(void (*kern)(const D *), const D *descs, int count, int64_t max_n, cudaStream_t st) {
    if (descs == nullptr) return HGQ_ERR_NULL;
    if (count < 0 || max_n < 0 || count > 65535) return HGQ_ERR_SIZE;
    if (count == 0 || max_n == 0) return HGQ_OK;
    dim3 grid((unsigned)((max_n + kThreads - 1) / kThreads), (unsigned)count);
    kern<<<grid, kThreads, 0, st>>>(descs);
    return check_launch();
}

}  // namespace hgq

using namespace hgq;

extern "C" int hgq_tables_forward(const hgq_slot_desc *slots, int n_slots, int64_t max_n, void *stream) {
    return launch_over<hgq_slot_desc>(k_tables_forward, slots, n_slots, max_n, (cudaStream_t)stream);
}

extern "C" int hgq_tables_track_bits(const hgq_slot_desc *slots, int n_slots, int64_t max_n, void *stream) {
    return launch_over<hgq_slot_desc>(k_tables_track_bits, slots, n_slots, max_n, (cudaStream_t)stream);
}

extern "C" int hgq_tables_backward(const hgq_slot_desc *slots, int n_slots, int64_t max_n, void *stream) {
    return launch_over<hgq_slot_desc>(k_tables_backward, slots, n_slots, max_n, (cudaStream_t)stream);
}

extern "C" int hgq_weights_forward(const hgq_weight_desc *weights, int n_weights, int64_t max_n, const hgq_slot_desc *slots,
                                   void *stream) {
    if (weights == nullptr || slots == nullptr) return HGQ_ERR_NULL;
    if (n_weights < 0 || max_n < 0 || n_weights > 65535) return HGQ_ERR_SIZE;
    if (n_weights == 0 || max_n == 0) return HGQ_OK;
    dim3 grid((unsigned)((max_n + kThreads - 1) / kThreads), (unsigned)n_weights);
    k_weights_forward<<<grid, kThreads, 0, (cudaStream_t)stream>>>(weights, slots);
    return check_launch();
}

extern "C" int hgq_weights_backward(const hgq_weight_desc *weights, int n_weights, int64_t max_n, const hgq_slot_desc *slots,
                                    void *stream) {
    if (weights == nullptr || slots == nullptr) return HGQ_ERR_NULL;
    if (n_weights < 0 || max_n < 0 || n_weights > 65535) return HGQ_ERR_SIZE;
    if (n_weights == 0 || max_n == 0) return HGQ_OK;
    dim3 grid((unsigned)((max_n + kThreads - 1) / kThreads), (unsigned)n_weights);
    k_weights_backward<<<grid, kThreads, 0, (cudaStream_t)stream>>>(weights, slots);
    return check_launch();
}
