// K3: per-layer EBOPs (effective bit operations) reduction and its gradient.
//
// Stands in for _compute_ebops of the quantised layers and the loss term the layer wrapper adds:
//   dense / einsum-dense   sum(matmul(bw_inp, bw_ker)) + mean(bw_bias) * out_size
//                          (src/hgq/layers/core/dense.py:70-80, einsum_dense.py:85-93)
//   conv2d                 sum(conv(bw_inp, bw_ker)) + mean(bw_bias) * out_size
//                          (src/hgq/layers/conv.py:91-102)
//   wrapper                _ebops.assign(cast(ebops, uint32)); add_loss(ebops * beta)
//                          (src/hgq/layers/core/base.py:95-104)
//
// Bitwidths are small non-negative integers stored as fp32.  The contraction factorises:
//   sum_{p,k,n} in[p,k] w[k,n] = sum_k (sum_p in[p,k]) (sum_n w[k,n]) = sum_k A[k] B[k]
// (for a convolution A[kh,kw,c] is the sum of the input bits over the output positions that the
// tap (kh,kw) visits).  A and B are accumulated as 64-bit integers with warp shuffles, so the
// result is the exact integer, independent of summation order; the reference accumulates the
// same products in fp32.  The data are tiny (the batch axis is 1), so one CTA does the whole
// layer: the launch is latency-bound and no roofline applies.
#include <cuda_runtime.h>

#include "hgq_common.cuh"

namespace hgq {

constexpr int kEbThreads = 1024;
constexpr int kEbMaxK = 10240;  // contraction length held in shared memory (2 x 8 B each)

__device__ __forceinline__ long long warp_sum(long long v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ long long block_sum(long long v, long long *scratch) {
    v = warp_sum(v);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        long long t = (lane < (blockDim.x >> 5)) ? scratch[lane] : 0;
        t = warp_sum(t);
        if (lane == 0) scratch[0] = t;
    }
    __syncthreads();
    const long long r = scratch[0];
    __syncthreads();
    return r;
}

struct EbopsOut {
    unsigned *ebops;   // uint32 scalar (the layer's `ebops` variable)
    float *ebops_f;    // fp32 scalar: EBOPs before the integer cast
    float *loss;       // fp32 scalar: ebops_f * beta
    float *d_in;       // gradient of loss w.r.t. bw_in  (may be NULL)
    float *d_w;        // gradient of loss w.r.t. bw_w   (may be NULL)
    float *d_bias;     // gradient of loss w.r.t. bw_bias (may be NULL)
};

__device__ void finish(long long total, const float *bw_bias, int64_t n_bias, double out_size, double scale_main,
                       double scale_bias, float beta, const EbopsOut &o, long long *scratch) {
    long long bsum = 0;
    for (int64_t j = threadIdx.x; j < n_bias; j += blockDim.x) bsum += __float2ll_rn(bw_bias[j]);
    bsum = block_sum(bsum, scratch);
    if (threadIdx.x == 0) {
        double e = (double)total * scale_main;
        if (n_bias > 0) e += ((double)bsum / (double)n_bias) * out_size * scale_bias;
        const float ef = (float)e;
        if (o.ebops) *o.ebops = (e <= 0.0) ? 0u : (e >= 4294967295.0 ? 4294967295u : (unsigned)e);
        if (o.ebops_f) *o.ebops_f = ef;
        if (o.loss) *o.loss = ef * beta;
    }
    if (o.d_bias != nullptr && n_bias > 0) {
        const float gb = (float)((double)beta * scale_bias * out_size / (double)n_bias);
        for (int64_t j = threadIdx.x; j < n_bias; j += blockDim.x) o.d_bias[j] = gb;
    }
}

// bw_in [P, K], bw_w [K, N]
__device__ __forceinline__ void ebops_dense_body(const float *__restrict__ bw_in, int64_t P, int64_t K, const float *__restrict__ bw_w,
                                                 int64_t N, const float *__restrict__ bw_bias, int64_t n_bias, double out_size,
                                                 double scale, const float *__restrict__ beta_p, const EbopsOut &o) {
    const float beta = *beta_p;
    extern __shared__ long long sm[];
    long long *A = sm, *B = sm + K, *scratch = sm + 2 * K;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    for (int64_t k = warp; k < K; k += nwarp) {  // B[k] = sum_n w[k, n]: one warp per row
        long long s = 0;
        for (int64_t n = lane; n < N; n += 32) s += __float2ll_rn(bw_w[k * N + n]);
        s = warp_sum(s);
        if (lane == 0) B[k] = s;
    }
    for (int64_t k = threadIdx.x; k < K; k += blockDim.x) {  // A[k] = sum_p in[p, k]: coalesced over k
        long long s = 0;
        for (int64_t p = 0; p < P; ++p) s += __float2ll_rn(bw_in[p * K + k]);
        A[k] = s;
    }
    __syncthreads();
    long long part = 0;
    for (int64_t k = threadIdx.x; k < K; k += blockDim.x) part += A[k] * B[k];
    const long long total = block_sum(part, scratch);
    const float gs = (float)((double)beta * scale);
    if (o.d_in)
        for (int64_t e = threadIdx.x; e < P * K; e += blockDim.x) o.d_in[e] = gs * (float)B[e % K];
    if (o.d_w)
        for (int64_t e = threadIdx.x; e < K * N; e += blockDim.x) o.d_w[e] = gs * (float)A[e / N];
    finish(total, bw_bias, n_bias, out_size, scale, scale, beta, o, scratch);
}

__global__ void __launch_bounds__(kEbThreads) k_ebops_dense(const float *__restrict__ bw_in, int64_t P, int64_t K,
                                                            const float *__restrict__ bw_w, int64_t N,
                                                            const float *__restrict__ bw_bias, int64_t n_bias,
                                                            double out_size, double scale, const float *__restrict__ beta_p, EbopsOut o) {
    ebops_dense_body(bw_in, P, K, bw_w, N, bw_bias, n_bias, out_size, scale, beta_p, o);
}

// Several dense layers in one launch: block b takes layer b (the layers are independent and each is one block's work, so a
// step's EBOPs terms cost one launch latency instead of one per layer).
struct EbBatch {
    hgq_ebops_dense_desc d[HGQ_EBOPS_BATCH_MAX];
};
__global__ void __launch_bounds__(kEbThreads) k_ebops_dense_batch(const EbBatch B) {
    const hgq_ebops_dense_desc &d = B.d[blockIdx.x];
    EbopsOut o{d.ebops, d.ebops_f, d.loss, d.d_bw_in, d.d_bw_w, d.d_bw_bias};
    ebops_dense_body(d.bw_in, d.P, d.K, d.bw_w, d.N, d.bw_bias, d.n_bias, d.out_size, d.scale, d.beta, o);
}

// bw_in [H, W, C] (channels last), bw_w [KH, KW, C, N]; output position (oh, ow) reads input
// (oh*sh + kh*dh - pt, ow*sw + kw*dw - pl); positions outside the input contribute nothing.
__global__ void __launch_bounds__(kEbThreads) k_ebops_conv2d(const float *__restrict__ bw_in, int H, int W, int C,
                                                             const float *__restrict__ bw_w, int KH, int KW, int N,
                                                             int OH, int OW, int sh, int sw, int dh, int dw, int pt,
                                                             int pl, const float *__restrict__ bw_bias,
                                                             int64_t n_bias, double out_size, double scale_main,
                                                             double scale_bias, const float *__restrict__ beta_p, EbopsOut o) {
    const float beta = *beta_p;
    extern __shared__ long long sm[];
    const int64_t K = (int64_t)KH * KW * C;
    long long *A = sm, *B = sm + K, *scratch = sm + 2 * K;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    for (int64_t k = warp; k < K; k += nwarp) {
        long long s = 0;
        for (int n = lane; n < N; n += 32) s += __float2ll_rn(bw_w[k * N + n]);
        s = warp_sum(s);
        if (lane == 0) B[k] = s;
    }
    for (int64_t k = warp; k < K; k += nwarp) {  // A[kh,kw,c]: one warp per tap, lanes over output positions
        const int c = (int)(k % C), kw = (int)((k / C) % KW), kh = (int)(k / ((int64_t)C * KW));
        long long s = 0;
        for (int op = lane; op < OH * OW; op += 32) {
            const int ih = (op / OW) * sh + kh * dh - pt, iw = (op % OW) * sw + kw * dw - pl;
            if (ih >= 0 && ih < H && iw >= 0 && iw < W) s += __float2ll_rn(bw_in[((int64_t)ih * W + iw) * C + c]);
        }
        s = warp_sum(s);
        if (lane == 0) A[k] = s;
    }
    __syncthreads();
    long long part = 0;
    for (int64_t k = threadIdx.x; k < K; k += blockDim.x) part += A[k] * B[k];
    const long long total = block_sum(part, scratch);
    const float gs = (float)((double)beta * scale_main);
    if (o.d_w)
        for (int64_t e = threadIdx.x; e < K * N; e += blockDim.x) o.d_w[e] = gs * (float)A[e / N];
    if (o.d_in) {
        // d in[h,w,c] = sum over taps (kh,kw) whose output position (oh,ow) exists of B[kh,kw,c]
        for (int64_t e = threadIdx.x; e < (int64_t)H * W * C; e += blockDim.x) {
            const int c = (int)(e % C), w = (int)((e / C) % W), h = (int)(e / ((int64_t)C * W));
            long long s = 0;
            for (int kh = 0; kh < KH; ++kh) {
                const int nh = h + pt - kh * dh;
                if (nh < 0 || nh % sh != 0 || nh / sh >= OH) continue;
                for (int kw = 0; kw < KW; ++kw) {
                    const int nw = w + pl - kw * dw;
                    if (nw < 0 || nw % sw != 0 || nw / sw >= OW) continue;
                    s += B[((int64_t)kh * KW + kw) * C + c];
                }
            }
            o.d_in[e] = gs * (float)s;
        }
    }
    finish(total, bw_bias, n_bias, out_size, scale_main, scale_bias, beta, o, scratch);
}

}  // namespace hgq

using namespace hgq;

extern "C" int hgq_ebops_dense(const float *bw_in, int64_t P, int64_t K, const float *bw_w, int64_t N,
                               const float *bw_bias, int64_t n_bias, double out_size, double scale, const float *beta,
                               uint32_t *ebops, float *ebops_f, float *loss, float *d_bw_in, float *d_bw_w,
                               float *d_bw_bias, void *stream) {
    if (P <= 0 || K <= 0 || N <= 0 || n_bias < 0) return HGQ_ERR_SIZE;
    if (K > kEbMaxK) return HGQ_ERR_SIZE;
    if (bw_in == nullptr || bw_w == nullptr || beta == nullptr || (n_bias > 0 && bw_bias == nullptr)) return HGQ_ERR_NULL;
    EbopsOut o{ebops, ebops_f, loss, d_bw_in, d_bw_w, d_bw_bias};
    const size_t smem = (size_t)(2 * K + 32) * sizeof(long long);
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(k_ebops_dense, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)((2 * kEbMaxK + 32) * sizeof(long long)));
        if (e != cudaSuccess) return (int)e;
    }
    k_ebops_dense<<<1, kEbThreads, smem, (cudaStream_t)stream>>>(bw_in, P, K, bw_w, N, bw_bias, n_bias, out_size, scale,
                                                                 beta, o);
    return check_launch();
}

extern "C" int hgq_ebops_dense_batch(const hgq_ebops_dense_desc *descs, int n, void *stream) {
    if (descs == nullptr) return HGQ_ERR_NULL;
    if (n < 1 || n > HGQ_EBOPS_BATCH_MAX) return HGQ_ERR_SIZE;
    EbBatch b;
    int64_t kmax = 0;
    for (int i = 0; i < n; ++i) {
        const hgq_ebops_dense_desc &d = descs[i];
        if (d.P <= 0 || d.K <= 0 || d.N <= 0 || d.n_bias < 0 || d.K > kEbMaxK) return HGQ_ERR_SIZE;
        if (d.bw_in == nullptr || d.bw_w == nullptr || d.beta == nullptr || (d.n_bias > 0 && d.bw_bias == nullptr)) return HGQ_ERR_NULL;
        b.d[i] = d;
        if (d.K > kmax) kmax = d.K;
    }
    const size_t smem = (size_t)(2 * kmax + 32) * sizeof(long long);
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(k_ebops_dense_batch, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)((2 * kEbMaxK + 32) * sizeof(long long)));
        if (e != cudaSuccess) return (int)e;
    }
    k_ebops_dense_batch<<<n, kEbThreads, smem, (cudaStream_t)stream>>>(b);
    return check_launch();
}

extern "C" int hgq_ebops_conv2d(const float *bw_in, int H, int W, int C, const float *bw_w, int KH, int KW, int N,
                                int OH, int OW, int stride_h, int stride_w, int dil_h, int dil_w, int pad_top,
                                int pad_left, const float *bw_bias, int64_t n_bias, double out_size, double scale_main,
                                double scale_bias, const float *beta, uint32_t *ebops, float *ebops_f, float *loss,
                                float *d_bw_in, float *d_bw_w, float *d_bw_bias, void *stream) {
    if (H <= 0 || W <= 0 || C <= 0 || KH <= 0 || KW <= 0 || N <= 0 || OH <= 0 || OW <= 0 || n_bias < 0) return HGQ_ERR_SIZE;
    if (stride_h <= 0 || stride_w <= 0 || dil_h <= 0 || dil_w <= 0 || pad_top < 0 || pad_left < 0) return HGQ_ERR_SIZE;
    const int64_t K = (int64_t)KH * KW * C;
    if (K > kEbMaxK) return HGQ_ERR_SIZE;
    if (bw_in == nullptr || bw_w == nullptr || beta == nullptr || (n_bias > 0 && bw_bias == nullptr)) return HGQ_ERR_NULL;
    EbopsOut o{ebops, ebops_f, loss, d_bw_in, d_bw_w, d_bw_bias};
    const size_t smem = (size_t)(2 * K + 32) * sizeof(long long);
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(k_ebops_conv2d, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)((2 * kEbMaxK + 32) * sizeof(long long)));
        if (e != cudaSuccess) return (int)e;
    }
    k_ebops_conv2d<<<1, kEbThreads, smem, (cudaStream_t)stream>>>(bw_in, H, W, C, bw_w, KH, KW, N, OH, OW, stride_h,
                                                                  stride_w, dil_h, dil_w, pad_top, pad_left, bw_bias,
                                                                  n_bias, out_size, scale_main, scale_bias, beta, o);
    return check_launch();
}
