// K5 (channels-last 2-D max pooling, 'valid' padding): forward with the arg-max kept as one byte per output element,
// backward as a gather over the windows that cover an input pixel.
//
// Stands in for the keras MaxPooling2D layers between the QConv2D layers of the reference's convolutional models
// (QMaxPooling2D without input quantizer, src/hgq/layers/pooling.py:146-167, delegates to the same keras op).  Ties go
// to the first element in (row, column) scan order, the rule of the torch kernels the oracle runs.
// HBM-bound: forward 4 (PH PW + 1) + 1 bytes per output element at stride = pool size, backward the mirror image.
#include <cuda_runtime.h>

#include "hgq_common.cuh"

namespace hgq {

struct PoolParams {
    int64_t B;
    int H, W, C, OH, OW, PH, PW, SH, SW;
};

template <int VEC>
__global__ void __launch_bounds__(kThreads) k_maxpool_fwd(const float *__restrict__ x, float *__restrict__ y,
                                                         unsigned char *__restrict__ idx, const PoolParams P, int64_t n_units,
                                                         const FastDiv div_cv, const FastDiv div_ow, const FastDiv div_oh) {
    const int CV = P.C / VEC;
    for (int64_t u = (int64_t)blockIdx.x * kThreads + threadIdx.x; u < n_units; u += (int64_t)gridDim.x * kThreads) {
        const uint32_t r0 = fastdiv((uint32_t)u, div_cv);  // n_units < 2^31 (checked on the host)
        const int cv = (int)((uint32_t)u - r0 * (uint32_t)CV);
        const uint32_t r1 = fastdiv(r0, div_ow);
        const int ow = (int)(r0 - r1 * (uint32_t)P.OW);
        const int64_t b = fastdiv(r1, div_oh);
        const int oh = (int)(r1 - (uint32_t)b * (uint32_t)P.OH);
        const float *src = x + ((b * P.H + (int64_t)oh * P.SH) * P.W + (int64_t)ow * P.SW) * P.C + cv * VEC;
        float best[VEC];
        unsigned char arg[VEC];
#pragma unroll
        for (int j = 0; j < VEC; ++j) {
            best[j] = -INFINITY;
            arg[j] = 0;
        }
        for (int ph = 0; ph < P.PH; ++ph)
            for (int pw = 0; pw < P.PW; ++pw) {
                float v[VEC];
                const float *p = src + ((int64_t)ph * P.W + pw) * P.C;
                if (VEC == 4) {
                    const float4 t = __ldcs(reinterpret_cast<const float4 *>(p));
                    v[0] = t.x; v[1 % VEC] = t.y; v[2 % VEC] = t.z; v[3 % VEC] = t.w;
                } else {
                    v[0] = __ldcs(p);
                }
                const unsigned char code = (unsigned char)(ph * P.PW + pw);
#pragma unroll
                for (int j = 0; j < VEC; ++j)
                    if (v[j] > best[j] || v[j] != v[j]) {  // first maximum wins; a NaN propagates
                        best[j] = v[j];
                        arg[j] = code;
                    }
            }
        const int64_t o = u * VEC;
        if (VEC == 4) {
            __stcs(reinterpret_cast<float4 *>(y + o), make_float4(best[0], best[1 % VEC], best[2 % VEC], best[3 % VEC]));
            *reinterpret_cast<uchar4 *>(idx + o) = make_uchar4(arg[0], arg[1 % VEC], arg[2 % VEC], arg[3 % VEC]);
        } else {
            y[o] = best[0];
            idx[o] = arg[0];
        }
    }
}

template <int VEC>
__global__ void __launch_bounds__(kThreads) k_maxpool_bwd(const float *__restrict__ gy, const unsigned char *__restrict__ idx,
                                                         float *__restrict__ dx, const PoolParams P, int64_t n_units) {
    const int CV = P.C / VEC;
    for (int64_t u = (int64_t)blockIdx.x * kThreads + threadIdx.x; u < n_units; u += (int64_t)gridDim.x * kThreads) {
        const int cv = (int)(u % CV);
        int64_t r = u / CV;
        const int iw = (int)(r % P.W);
        r /= P.W;
        const int ih = (int)(r % P.H);
        const int64_t b = r / P.H;
        float acc[VEC];
#pragma unroll
        for (int j = 0; j < VEC; ++j) acc[j] = 0.f;
        // windows (oh, ow) with oh*SH <= ih < oh*SH + PH, likewise along the width
        const int oh_hi = min(ih / P.SH, P.OH - 1), ow_hi = min(iw / P.SW, P.OW - 1);
        const int oh_lo = max(0, (ih - P.PH + P.SH) / P.SH), ow_lo = max(0, (iw - P.PW + P.SW) / P.SW);
        for (int oh = oh_lo; oh <= oh_hi; ++oh)
            for (int ow = ow_lo; ow <= ow_hi; ++ow) {
                const int ph = ih - oh * P.SH, pw = iw - ow * P.SW;
                if (ph >= P.PH || pw >= P.PW) continue;
                const unsigned char code = (unsigned char)(ph * P.PW + pw);
                const int64_t o = (((b * P.OH + oh) * P.OW + ow) * CV + cv) * VEC;
                if (VEC == 4) {
                    const uchar4 a = *reinterpret_cast<const uchar4 *>(idx + o);
                    const float4 g = __ldg(reinterpret_cast<const float4 *>(gy + o));
                    if (a.x == code) acc[0] = __fadd_rn(acc[0], g.x);
                    if (a.y == code) acc[1 % VEC] = __fadd_rn(acc[1 % VEC], g.y);
                    if (a.z == code) acc[2 % VEC] = __fadd_rn(acc[2 % VEC], g.z);
                    if (a.w == code) acc[3 % VEC] = __fadd_rn(acc[3 % VEC], g.w);
                } else {
                    if (idx[o] == code) acc[0] = __fadd_rn(acc[0], __ldg(gy + o));
                }
            }
        const int64_t o = u * VEC;
        if (VEC == 4)
            __stcs(reinterpret_cast<float4 *>(dx + o), make_float4(acc[0], acc[1 % VEC], acc[2 % VEC], acc[3 % VEC]));
        else
            dx[o] = acc[0];
    }
}


// Non-overlapping windows (stride == pool size): one thread per output element group scatters its gradient to the
// PH x PW positions of its window (the winner gets gy, the others zero), so every covered input element is written exactly
// once and no search over windows is needed.  Rows / columns beyond the last full window are zeroed by the caller.
template <int VEC>
__global__ void __launch_bounds__(kThreads) k_maxpool_bwd_tiled(const float *__restrict__ gy, const unsigned char *__restrict__ idx,
                                                               float *__restrict__ dx, const PoolParams P, int64_t n_units,
                                                               const FastDiv div_cv, const FastDiv div_ow, const FastDiv div_oh) {
    const int CV = P.C / VEC;
    for (int64_t u = (int64_t)blockIdx.x * kThreads + threadIdx.x; u < n_units; u += (int64_t)gridDim.x * kThreads) {
        const uint32_t r0 = fastdiv((uint32_t)u, div_cv);
        const int cv = (int)((uint32_t)u - r0 * (uint32_t)CV);
        const uint32_t r1 = fastdiv(r0, div_ow);
        const int ow = (int)(r0 - r1 * (uint32_t)P.OW);
        const uint32_t b = fastdiv(r1, div_oh);
        const int oh = (int)(r1 - b * (uint32_t)P.OH);
        const int64_t o = u * VEC;
        float g[VEC];
        unsigned char a[VEC];
        if (VEC == 4) {
            const float4 t = __ldcs(reinterpret_cast<const float4 *>(gy + o));
            const uchar4 c = *reinterpret_cast<const uchar4 *>(idx + o);
            g[0] = t.x; g[1 % VEC] = t.y; g[2 % VEC] = t.z; g[3 % VEC] = t.w;
            a[0] = c.x; a[1 % VEC] = c.y; a[2 % VEC] = c.z; a[3 % VEC] = c.w;
        } else {
            g[0] = __ldcs(gy + o);
            a[0] = idx[o];
        }
        float *dst = dx + (((int64_t)b * P.H + (int64_t)oh * P.PH) * P.W + (int64_t)ow * P.PW) * P.C + cv * VEC;
        for (int ph = 0; ph < P.PH; ++ph)
            for (int pw = 0; pw < P.PW; ++pw) {
                const unsigned char code = (unsigned char)(ph * P.PW + pw);
                float *q = dst + ((int64_t)ph * P.W + pw) * P.C;
                if (VEC == 4)
                    __stcs(reinterpret_cast<float4 *>(q), make_float4(a[0] == code ? g[0] : 0.f, a[1 % VEC] == code ? g[1 % VEC] : 0.f,
                                                                       a[2 % VEC] == code ? g[2 % VEC] : 0.f, a[3 % VEC] == code ? g[3 % VEC] : 0.f));
                else
                    *q = a[0] == code ? g[0] : 0.f;
            }
    }
}

static int pool_check(const PoolParams &p) {
    if (p.B <= 0 || p.H <= 0 || p.W <= 0 || p.C <= 0 || p.PH <= 0 || p.PW <= 0 || p.SH <= 0 || p.SW <= 0) return HGQ_ERR_SIZE;
    if (p.PH * p.PW > 255 || p.PH > p.H || p.PW > p.W) return HGQ_ERR_SIZE;
    if (p.OH != (p.H - p.PH) / p.SH + 1 || p.OW != (p.W - p.PW) / p.SW + 1) return HGQ_ERR_SIZE;
    return HGQ_OK;
}

static unsigned pool_grid(int64_t n_units) {
    int64_t g = (n_units + kThreads - 1) / kThreads;
    const int64_t cap = (int64_t)num_sms() * 32;
    return (unsigned)(g < cap ? g : cap);
}

}  // namespace hgq

using namespace hgq;

extern "C" int hgq_maxpool2d_fwd(const float *x, float *y, unsigned char *argmax, int64_t B, int H, int W, int C, int pool_h,
                                 int pool_w, int stride_h, int stride_w, int OH, int OW, void *stream) {
    if (x == nullptr || y == nullptr || argmax == nullptr) return HGQ_ERR_NULL;
    const PoolParams p{B, H, W, C, OH, OW, pool_h, pool_w, stride_h, stride_w};
    if (int e = pool_check(p)) return e;
    cudaStream_t st = (cudaStream_t)stream;
    const bool vec = (C % 4 == 0) && aligned(x, 16) && aligned(y, 16) && aligned(argmax, 4);
    const int cvn = vec ? C / 4 : C;
    const int64_t n_units = B * OH * OW * cvn;
    if (n_units >= ((int64_t)1 << 31)) return HGQ_ERR_SIZE;
    const FastDiv d_cv = make_fastdiv((uint32_t)cvn), d_ow = make_fastdiv((uint32_t)OW), d_oh = make_fastdiv((uint32_t)OH);
    if (vec)
        k_maxpool_fwd<4><<<pool_grid(n_units), kThreads, 0, st>>>(x, y, argmax, p, n_units, d_cv, d_ow, d_oh);
    else
        k_maxpool_fwd<1><<<pool_grid(n_units), kThreads, 0, st>>>(x, y, argmax, p, n_units, d_cv, d_ow, d_oh);
    return check_launch();
}

extern "C" int hgq_maxpool2d_bwd(const float *gy, const unsigned char *argmax, float *dx, int64_t B, int H, int W, int C,
                                 int pool_h, int pool_w, int stride_h, int stride_w, int OH, int OW, void *stream) {
    if (gy == nullptr || dx == nullptr || argmax == nullptr) return HGQ_ERR_NULL;
    const PoolParams p{B, H, W, C, OH, OW, pool_h, pool_w, stride_h, stride_w};
    if (int e = pool_check(p)) return e;
    cudaStream_t st = (cudaStream_t)stream;
    const bool vec = (C % 4 == 0) && aligned(gy, 16) && aligned(dx, 16) && aligned(argmax, 4);
    if (stride_h == pool_h && stride_w == pool_w && B * OH * OW * (int64_t)C < ((int64_t)1 << 31)) {
        // non-overlapping windows: scatter per window; input rows / columns behind the last full window get no gradient
        if (OH * pool_h != H || OW * pool_w != W) {
            cudaError_t ce = cudaMemsetAsync(dx, 0, (size_t)B * H * W * C * sizeof(float), st);
            if (ce != cudaSuccess) return (int)ce;
        }
        const int cvn = vec ? C / 4 : C;
        const int64_t n_out = B * OH * OW * cvn;
        const FastDiv d_cv = make_fastdiv((uint32_t)cvn), d_ow = make_fastdiv((uint32_t)OW), d_oh = make_fastdiv((uint32_t)OH);
        if (vec)
            k_maxpool_bwd_tiled<4><<<pool_grid(n_out), kThreads, 0, st>>>(gy, argmax, dx, p, n_out, d_cv, d_ow, d_oh);
        else
            k_maxpool_bwd_tiled<1><<<pool_grid(n_out), kThreads, 0, st>>>(gy, argmax, dx, p, n_out, d_cv, d_ow, d_oh);
        return check_launch();
    }
    const int64_t n_units = B * H * W * (vec ? C / 4 : C);
    if (vec)
        k_maxpool_bwd<4><<<pool_grid(n_units), kThreads, 0, st>>>(gy, argmax, dx, p, n_units);
    else
        k_maxpool_bwd<1><<<pool_grid(n_units), kThreads, 0, st>>>(gy, argmax, dx, p, n_units);
    return check_launch();
}
