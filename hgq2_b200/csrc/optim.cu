// Fused parameter update of the QAT step: Adam over one flat fp32 bucket that holds every trainable
// variable of the model (weights, biases and bitwidths), with the pieces Keras' trainer applies
// around the optimizer folded into the same pass:
//   - the MonoL1 bitwidth regulariser l1 * sum(x) (src/hgq/regularizers/__init__.py:8-17) enters
//     as the constant l1 added to the gradient of the elements it covers;
//   - the MinMax / Min / Max / Constant constraints (src/hgq/constraints/__init__.py:11-69) that
//     Keras applies to a variable after its update are a per-element clamp to [lo, hi].
// The update rule is Keras' Adam: m = b1 m + (1-b1) g;  v = b2 v + (1-b2) g^2;
//   alpha = lr sqrt(1 - b2^t) / (1 - b1^t);  w -= alpha m / (sqrt(v) + eps).
// The step counter lives on the device so that a captured CUDA graph advances it.
// Streaming kernel, 28 B read + 12 B written per element; the buckets of the target models hold
// 10^4..10^5 elements, so the launch is latency-bound.
#include <cuda_runtime.h>

#include "hgq_common.cuh"

namespace hgq {

__global__ void __launch_bounds__(kThreads) k_adam(float *__restrict__ w, const float *__restrict__ g,
                                                   float *__restrict__ m, float *__restrict__ v,
                                                   const float *__restrict__ lo, const float *__restrict__ hi,
                                                   const float *__restrict__ l1, int64_t n, float lr, float b1, float b2,
                                                   float eps, float grad_scale, long long *__restrict__ step) {
    const long long t = *step + 1;
    const float c1 = 1.f - powf(b1, (float)t);
    const float c2 = 1.f - powf(b2, (float)t);
    const float alpha = lr * sqrtf(c2) / c1;
    for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (int64_t)gridDim.x * blockDim.x) {
        float ge = g[e] * grad_scale;
        if (l1) ge += l1[e];
        const float me = b1 * m[e] + (1.f - b1) * ge;
        const float ve = b2 * v[e] + (1.f - b2) * ge * ge;
        float we = w[e] - alpha * me / (sqrtf(ve) + eps);
        if (lo) we = fmaxf(we, lo[e]);
        if (hi) we = fminf(we, hi[e]);
        m[e] = me;
        v[e] = ve;
        w[e] = we;
    }
}

__global__ void k_step_inc(long long *step) { *step += 1; }

}  // namespace hgq

using namespace hgq;

extern "C" int hgq_adam_step(float *w, const float *g, float *m, float *v, const float *lo, const float *hi,
                             const float *l1, int64_t n, float lr, float beta1, float beta2, float eps,
                             float grad_scale, long long *step, void *stream) {
    if (n < 0) return HGQ_ERR_SIZE;
    if (n == 0) return HGQ_OK;
    if (!w || !g || !m || !v || !step) return HGQ_ERR_NULL;
    int64_t blocks = (n + kThreads - 1) / kThreads;
    if (blocks > (int64_t)num_sms() * 8) blocks = (int64_t)num_sms() * 8;
    cudaStream_t st = (cudaStream_t)stream;
    k_adam<<<(unsigned)blocks, kThreads, 0, st>>>(w, g, m, v, lo, hi, l1, n, lr, beta1, beta2, eps, grad_scale, step);
    if (int e = check_launch()) return e;
    k_step_inc<<<1, 1, 0, st>>>(step);
    return check_launch();
}
