// Softmax cross-entropy from logits with integer labels, mean over the batch: loss and d loss / d logits in one pass.
//
// The task loss of the QAT steps (keras.losses.SparseCategoricalCrossentropy(from_logits=True), which the reference's
// models are compiled with; the loss itself lives in Keras, outside the HGQ2 tree).  One thread per row (class counts are
// small: 5 or 10), the gradient (softmax - onehot) / B written alongside, per-CTA partial sums reduced in a fixed order by
// a second, single-block kernel -- instead of four library launches two of which run on one block.
#include <cuda_runtime.h>

#include "hgq_common.cuh"

namespace hgq {

constexpr int kXentMaxClasses = 64;

__global__ void __launch_bounds__(kThreads) k_xent_rows(const float *__restrict__ logits, const int64_t *__restrict__ labels,
                                                       float *__restrict__ dlogits, float *__restrict__ part, int64_t B, int C,
                                                       float inv_b) {
    __shared__ float red[kThreads / 32];
    const int64_t row = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    float loss = 0.f;
    if (row < B) {
        const float *z = logits + row * C;
        float v[kXentMaxClasses];
        float m = -INFINITY;
        for (int c = 0; c < C; ++c) {
            v[c] = __ldg(z + c);
            m = fmaxf(m, v[c]);
        }
        float s = 0.f;
        for (int c = 0; c < C; ++c) {
            v[c] = expf(v[c] - m);
            s += v[c];
        }
        const int64_t y = __ldg(labels + row);
        const float inv_s = 1.f / s;
        loss = (y >= 0 && y < C) ? (logf(s) - (__ldg(z + y) - m)) : 0.f;
        float *g = dlogits + row * C;
        for (int c = 0; c < C; ++c) g[c] = (v[c] * inv_s - (c == y ? 1.f : 0.f)) * inv_b;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) loss += __shfl_xor_sync(0xffffffffu, loss, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = loss;
    __syncthreads();
    if (threadIdx.x == 0) {
        float a = 0.f;
        for (int w = 0; w < kThreads / 32; ++w) a += red[w];
        part[blockIdx.x] = a;
    }
}

__global__ void __launch_bounds__(kThreads) k_xent_mean(const float *__restrict__ part, int n, float inv_b, float *__restrict__ loss) {
    __shared__ double red[kThreads];
    double a = 0.0;
    for (int i = threadIdx.x; i < n; i += kThreads) a += (double)part[i];
    red[threadIdx.x] = a;
    __syncthreads();
    for (int o = kThreads / 2; o > 0; o >>= 1) {
        if (threadIdx.x < o) red[threadIdx.x] += red[threadIdx.x + o];
        __syncthreads();
    }
    if (threadIdx.x == 0) *loss = (float)(red[0] * (double)inv_b);
}

}  // namespace hgq

using namespace hgq;

extern "C" size_t hgq_softmax_xent_workspace(int64_t B) { return B > 0 ? (size_t)((B + kThreads - 1) / kThreads) * sizeof(float) : 0; }

extern "C" int hgq_softmax_xent(const float *logits, const int64_t *labels, float *loss, float *dlogits, int64_t B, int C,
                                void *workspace, size_t workspace_bytes, void *stream) {
    if (logits == nullptr || labels == nullptr || loss == nullptr || dlogits == nullptr) return HGQ_ERR_NULL;
    if (B <= 0 || C <= 0 || C > kXentMaxClasses) return HGQ_ERR_SIZE;
    const int64_t nblk = (B + kThreads - 1) / kThreads;
    if (workspace == nullptr || workspace_bytes < (size_t)nblk * sizeof(float)) return HGQ_ERR_WORKSPACE;
    cudaStream_t st = (cudaStream_t)stream;
    const float inv_b = 1.f / (float)B;
    k_xent_rows<<<(unsigned)nblk, kThreads, 0, st>>>(logits, labels, dlogits, (float *)workspace, B, C, inv_b);
    if (int e = check_launch()) return e;
    k_xent_mean<<<1, kThreads, 0, st>>>((const float *)workspace, (int)nblk, inv_b, loss);
    return check_launch();
}
