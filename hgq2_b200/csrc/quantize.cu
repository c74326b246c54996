// K1: elementwise fixed-point quantizer, forward and surrogate-gradient backward.
//
// Stands in for stateless_quantizer(x, k, i, f, training, seed_gen) and
// stateless_quantizer.round(x, f, ...) as called from
// src/hgq/quantizer/internal/fixed_point_quantizer.py:147,288,295,305,405, plus the reductions
// that DefaultBitwidthMapper adds around them (src/hgq/quantizer/internal/base.py:182-186):
// bw_to_x's backward (sum of the bitwidth gradients over the broadcast rows) and
// x_to_bw_absmax.
//
// All kernels are HBM-bound streaming kernels: 128-bit coalesced accesses with streaming cache
// hints, several independent loads in flight per thread, and grids that are a multiple of the
// SM count.  Two parameter layouts:
//   full       k/i/f have one entry per element (the standalone sweep);
//   broadcast  k/i/f have P entries and x is [rows, P]; a thread keeps the parameters of its
//              columns in registers and accumulates the column reductions privately.
#include <cuda_runtime.h>

#include "hgq_common.cuh"
#include "hgq_math.cuh"

namespace hgq {

std::atomic<int64_t> g_launches{0};

// ---- vector access helpers -------------------------------------------------------------------
template <int VEC>
struct Acc;

template <>
struct Acc<4> {
    static __device__ __forceinline__ void ldf(const float *p, int64_t v, float (&o)[4]) {
        const float4 t = __ldcs(reinterpret_cast<const float4 *>(p) + v);
        o[0] = t.x; o[1] = t.y; o[2] = t.z; o[3] = t.w;
    }
    static __device__ __forceinline__ void ldf_cached(const float *p, int64_t v, float (&o)[4]) {
        const float4 t = __ldg(reinterpret_cast<const float4 *>(p) + v);
        o[0] = t.x; o[1] = t.y; o[2] = t.z; o[3] = t.w;
    }
    static __device__ __forceinline__ void ldk(const uint8_t *p, int64_t v, float (&o)[4]) {
        const uchar4 t = __ldcs(reinterpret_cast<const uchar4 *>(p) + v);
        o[0] = (float)t.x; o[1] = (float)t.y; o[2] = (float)t.z; o[3] = (float)t.w;
    }
    static __device__ __forceinline__ void st(float *p, int64_t v, const float (&o)[4]) {
        __stcs(reinterpret_cast<float4 *>(p) + v, make_float4(o[0], o[1], o[2], o[3]));
    }
};

template <>
struct Acc<1> {
    static __device__ __forceinline__ void ldf(const float *p, int64_t v, float (&o)[1]) { o[0] = __ldcs(p + v); }
    static __device__ __forceinline__ void ldf_cached(const float *p, int64_t v, float (&o)[1]) { o[0] = __ldg(p + v); }
    static __device__ __forceinline__ void ldk(const uint8_t *p, int64_t v, float (&o)[1]) { o[0] = (float)__ldcs(p + v); }
    static __device__ __forceinline__ void st(float *p, int64_t v, const float (&o)[1]) { __stcs(p + v, o[0]); }
};

template <int RM, int OM>
__device__ __forceinline__ float fwd_one(float x, float kf, float i, float f, bool zero, float *rounded = nullptr) {
    const Params p = make_params(kf, OM == OM_NONE ? 0.f : i, f);
    return zero ? quantize<RM, OM, false, true>(x, p, rounded) : quantize<RM, OM, false, false>(x, p, rounded);
}

// ---- full layout -----------------------------------------------------------------------------
// One CTA covers kThreads * U consecutive vectors; a thread issues all its loads (U per stream)
// before the first use.
template <int RM, int OM, int VEC, int U>
__global__ void __launch_bounds__(kThreads) k_fwd_full(const float *__restrict__ x, const uint8_t *__restrict__ k,
                                                       const float *__restrict__ i, const float *__restrict__ f,
                                                       float *__restrict__ y, int64_t nvec, bool zero) {
    const int64_t base = (int64_t)blockIdx.x * (kThreads * U) + threadIdx.x;
    float xv[U][VEC], kv[U][VEC], iv[U][VEC], fv[U][VEC];
#pragma unroll
    for (int u = 0; u < U; ++u) {
        const int64_t v = base + (int64_t)u * kThreads;
        if (v < nvec) {
            Acc<VEC>::ldf(x, v, xv[u]);
            Acc<VEC>::ldf(f, v, fv[u]);
            if (OM != OM_NONE) {
                Acc<VEC>::ldf(i, v, iv[u]);
                Acc<VEC>::ldk(k, v, kv[u]);
            }
        }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
        const int64_t v = base + (int64_t)u * kThreads;
        if (v < nvec) {
            float o[VEC];
#pragma unroll
            for (int c = 0; c < VEC; ++c)
                o[c] = fwd_one<RM, OM>(xv[u][c], OM == OM_NONE ? 0.f : kv[u][c], OM == OM_NONE ? 0.f : iv[u][c],
                                       fv[u][c], zero);
            Acc<VEC>::st(y, v, o);
        }
    }
}

template <int RM, int OM, int VEC, int U>
__global__ void __launch_bounds__(kThreads) k_bwd_full(const float *__restrict__ g, const float *__restrict__ x,
                                                       const uint8_t *__restrict__ k, const float *__restrict__ i,
                                                       const float *__restrict__ f, float *__restrict__ dx,
                                                       float *__restrict__ di, float *__restrict__ df, int64_t nvec) {
    const int64_t base = (int64_t)blockIdx.x * (kThreads * U) + threadIdx.x;
    float gv[U][VEC], xv[U][VEC], kv[U][VEC], iv[U][VEC], fv[U][VEC];
#pragma unroll
    for (int u = 0; u < U; ++u) {
        const int64_t v = base + (int64_t)u * kThreads;
        if (v < nvec) {
            Acc<VEC>::ldf(g, v, gv[u]);
            Acc<VEC>::ldf(x, v, xv[u]);
            Acc<VEC>::ldf(f, v, fv[u]);
            if (OM != OM_NONE) {
                Acc<VEC>::ldf(i, v, iv[u]);
                Acc<VEC>::ldk(k, v, kv[u]);
            }
        }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
        const int64_t v = base + (int64_t)u * kThreads;
        if (v < nvec) {
            float odx[VEC], odi[VEC], odf[VEC];
#pragma unroll
            for (int c = 0; c < VEC; ++c) {
                const Params p = make_params(OM == OM_NONE ? 0.f : kv[u][c], OM == OM_NONE ? 0.f : iv[u][c], fv[u][c]);
                quantize_grad<RM, OM>(gv[u][c], xv[u][c], p, odx[c], odi[c], odf[c]);
            }
            Acc<VEC>::st(dx, v, odx);
            Acc<VEC>::st(df, v, odf);
            if (di) Acc<VEC>::st(di, v, odi);
        }
    }
}

// ---- broadcast layout ------------------------------------------------------------------------
template <int RM, int OM, int VEC, int U>
__global__ void __launch_bounds__(kThreads) k_fwd_bcast(const float *__restrict__ x, const uint8_t *__restrict__ k,
                                                        const float *__restrict__ i, const float *__restrict__ f,
                                                        float *__restrict__ y, unsigned *__restrict__ absmax,
                                                        int64_t rows, int64_t V, int TX, int64_t rowsPerBlock,
                                                        bool zero) {
    const int tx = threadIdx.x & (TX - 1);
    const int ty = threadIdx.x / TX;
    const int TY = kThreads / TX;
    const int64_t col = (int64_t)blockIdx.x * TX + tx;
    const bool active = col < V;
    const int64_t r0 = (int64_t)blockIdx.y * rowsPerBlock;
    const int64_t r1 = min(rows, r0 + rowsPerBlock);

    Params p[VEC];
    unsigned amax[VEC];
#pragma unroll
    for (int c = 0; c < VEC; ++c) amax[c] = 0u;
    if (active) {
        float kv[VEC], iv[VEC], fv[VEC];
        Acc<VEC>::ldf_cached(f, col, fv);
        if (OM != OM_NONE) {
            Acc<VEC>::ldf_cached(i, col, iv);
            Acc<VEC>::ldk(k, col, kv);
        }
#pragma unroll
        for (int c = 0; c < VEC; ++c)
            p[c] = make_params(OM == OM_NONE ? 0.f : kv[c], OM == OM_NONE ? 0.f : iv[c], fv[c]);

        for (int64_t r = r0 + ty; r < r1; r += (int64_t)TY * U) {
            float xv[U][VEC];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int64_t rr = r + (int64_t)u * TY;
                if (rr < r1) Acc<VEC>::ldf(x, rr * V + col, xv[u]);
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int64_t rr = r + (int64_t)u * TY;
                if (rr < r1) {
                    float o[VEC];
#pragma unroll
                    for (int c = 0; c < VEC; ++c) {
                        float xq;
                        o[c] = zero ? quantize<RM, OM, false, true>(xv[u][c], p[c], &xq)
                                    : quantize<RM, OM, false, false>(xv[u][c], p[c], &xq);
                        amax[c] = max(amax[c], __float_as_uint(fabsf(xq)));
                    }
                    Acc<VEC>::st(y, rr * V + col, o);
                }
            }
        }
    }
    if (absmax != nullptr) {
        // |v| of non-negative floats orders like the unsigned bit pattern; NaN sorts above +inf.
        __shared__ unsigned red[kThreads * VEC];
#pragma unroll
        for (int c = 0; c < VEC; ++c) red[threadIdx.x * VEC + c] = amax[c];
        __syncthreads();
        if (ty == 0 && active) {
#pragma unroll
            for (int c = 0; c < VEC; ++c) {
                unsigned m = 0u;
                for (int j = 0; j < TY; ++j) m = max(m, red[(j * TX + tx) * VEC + c]);
                atomicMax(absmax + col * VEC + c, m);
            }
        }
    }
}

// Stage 1 of the broadcast backward: dx elementwise, per-CTA column partial sums of di/df written
// to ws[(blockIdx.y) * P + column] (di plane first, df plane after rowBlocks * P floats).
template <int RM, int OM, int VEC, int U>
__global__ void __launch_bounds__(kThreads) k_bwd_bcast(const float *__restrict__ g, const float *__restrict__ x,
                                                        const uint8_t *__restrict__ k, const float *__restrict__ i,
                                                        const float *__restrict__ f, float *__restrict__ dx,
                                                        float *__restrict__ ws, bool want_di, int64_t rows, int64_t V,
                                                        int TX, int64_t rowsPerBlock) {
    const int tx = threadIdx.x & (TX - 1);
    const int ty = threadIdx.x / TX;
    const int TY = kThreads / TX;
    const int64_t col = (int64_t)blockIdx.x * TX + tx;
    const bool active = col < V;
    const int64_t r0 = (int64_t)blockIdx.y * rowsPerBlock;
    const int64_t r1 = min(rows, r0 + rowsPerBlock);

    Params p[VEC];
    float sdi[VEC], sdf[VEC];
#pragma unroll
    for (int c = 0; c < VEC; ++c) sdi[c] = sdf[c] = 0.f;
    if (active) {
        float kv[VEC], iv[VEC], fv[VEC];
        Acc<VEC>::ldf_cached(f, col, fv);
        if (OM != OM_NONE) {
            Acc<VEC>::ldf_cached(i, col, iv);
            Acc<VEC>::ldk(k, col, kv);
        }
#pragma unroll
        for (int c = 0; c < VEC; ++c)
            p[c] = make_params(OM == OM_NONE ? 0.f : kv[c], OM == OM_NONE ? 0.f : iv[c], fv[c]);

        for (int64_t r = r0 + ty; r < r1; r += (int64_t)TY * U) {
            float gv[U][VEC], xv[U][VEC];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int64_t rr = r + (int64_t)u * TY;
                if (rr < r1) {
                    Acc<VEC>::ldf(g, rr * V + col, gv[u]);
                    Acc<VEC>::ldf(x, rr * V + col, xv[u]);
                }
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int64_t rr = r + (int64_t)u * TY;
                if (rr < r1) {
                    float odx[VEC];
#pragma unroll
                    for (int c = 0; c < VEC; ++c) {
                        float a, b;
                        quantize_grad<RM, OM>(gv[u][c], xv[u][c], p[c], odx[c], a, b);
                        sdi[c] = __fadd_rn(sdi[c], a);
                        sdf[c] = __fadd_rn(sdf[c], b);
                    }
                    if (dx) Acc<VEC>::st(dx, rr * V + col, odx);
                }
            }
        }
    }
    __shared__ float red[2][kThreads * VEC];
#pragma unroll
    for (int c = 0; c < VEC; ++c) {
        red[0][threadIdx.x * VEC + c] = sdi[c];
        red[1][threadIdx.x * VEC + c] = sdf[c];
    }
    __syncthreads();
    if (ty == 0 && active) {
        const int64_t P = V * VEC;
        float *wdi = ws + (int64_t)blockIdx.y * P;
        float *wdf = ws + (int64_t)gridDim.y * P + (int64_t)blockIdx.y * P;
#pragma unroll
        for (int c = 0; c < VEC; ++c) {
            float a = 0.f, b = 0.f;
            for (int j = 0; j < TY; ++j) {
                a = __fadd_rn(a, red[0][(j * TX + tx) * VEC + c]);
                b = __fadd_rn(b, red[1][(j * TX + tx) * VEC + c]);
            }
            if (want_di) wdi[col * VEC + c] = a;
            wdf[col * VEC + c] = b;
        }
    }
}

// Stage 2: out[c] = sum over row blocks of ws[rb * P + c], in double, in a fixed order: one warp per column, lane l adds
// the row blocks l, l + 32, ... in sequence, then the 32 lane sums are combined by a fixed shuffle tree.
__global__ void __launch_bounds__(kThreads) k_colsum_stage2(const float *__restrict__ ws, float *__restrict__ di,
                                                            float *__restrict__ df, int64_t P, int rowBlocks) {
    const int lane = threadIdx.x & 31;
    const int64_t c = (int64_t)blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5);
    if (c >= P) return;
    const float *src = blockIdx.y == 0 ? ws : ws + (int64_t)rowBlocks * P;
    float *dst = blockIdx.y == 0 ? di : df;
    if (dst == nullptr) return;
    double acc = 0.0;
    for (int rb = lane; rb < rowBlocks; rb += 32) acc += (double)src[(int64_t)rb * P + c];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) dst[c] = (float)acc;
}

// ---- dispatch --------------------------------------------------------------------------------
constexpr int kUFwd = 2, kUBwd = 2, kUBcast = 4;

template <int RM, int OM>
static int launch_fwd(const float *x, const uint8_t *k, const float *i, const float *f, float *y, float *absmax,
                      int64_t n, int64_t period, bool zero, cudaStream_t st) {
    const bool full = (period == n);
    bool can_vec = aligned(x, 16) && aligned(y, 16) && aligned(f, 16);
    if (OM != OM_NONE) can_vec = can_vec && aligned(i, 16) && aligned(k, 4);
    if (full) {
        const int64_t nvec = can_vec ? n / 4 : 0;
        if (nvec > 0) {
            const int64_t per = (int64_t)kThreads * kUFwd;
            k_fwd_full<RM, OM, 4, kUFwd><<<(unsigned)((nvec + per - 1) / per), kThreads, 0, st>>>(x, k, i, f, y, nvec, zero);
            if (int e = check_launch()) return e;
        }
        const int64_t done = nvec * 4, rem = n - done;
        if (rem > 0) {
            const int64_t per = (int64_t)kThreads * kUFwd;
            k_fwd_full<RM, OM, 1, kUFwd><<<(unsigned)((rem + per - 1) / per), kThreads, 0, st>>>(
                x + done, k ? k + done : k, i ? i + done : i, f + done, y + done, rem, zero);
            if (int e = check_launch()) return e;
        }
        return HGQ_OK;
    }
    const int64_t rows = n / period;
    const BcastGeom ge = bcast_geom(rows, period, can_vec, kUBcast);
    if (absmax) {
        cudaError_t e = cudaMemsetAsync(absmax, 0, sizeof(float) * period, st);
        if (e != cudaSuccess) return (int)e;
    }
    dim3 grid((unsigned)ge.colTiles, (unsigned)ge.rowBlocks);
    if (ge.vec == 4)
        k_fwd_bcast<RM, OM, 4, kUBcast><<<grid, kThreads, 0, st>>>(x, k, i, f, y, (unsigned *)absmax, rows, ge.V, ge.TX,
                                                                 ge.rowsPerBlock, zero);
    else
        k_fwd_bcast<RM, OM, 1, kUBcast><<<grid, kThreads, 0, st>>>(x, k, i, f, y, (unsigned *)absmax, rows, ge.V, ge.TX,
                                                                 ge.rowsPerBlock, zero);
    return check_launch();
}

template <int RM, int OM>
static int launch_bwd(const float *g, const float *x, const uint8_t *k, const float *i, const float *f, float *dx,
                      float *di, float *df, int64_t n, int64_t period, void *ws, size_t ws_bytes, cudaStream_t st) {
    const bool full = (period == n);
    bool can_vec = aligned(x, 16) && aligned(g, 16) && aligned(f, 16) && aligned(dx, 16);
    if (OM != OM_NONE) can_vec = can_vec && aligned(i, 16) && aligned(k, 4);
    if (full) {
        can_vec = can_vec && aligned(df, 16) && aligned(di, 16);
        const int64_t nvec = can_vec ? n / 4 : 0;
        if (nvec > 0) {
            const int64_t per = (int64_t)kThreads * kUBwd;
            k_bwd_full<RM, OM, 4, kUBwd><<<(unsigned)((nvec + per - 1) / per), kThreads, 0, st>>>(g, x, k, i, f, dx, di, df, nvec);
            if (int e = check_launch()) return e;
        }
        const int64_t done = nvec * 4, rem = n - done;
        if (rem > 0) {
            const int64_t per = (int64_t)kThreads * kUBwd;
            k_bwd_full<RM, OM, 1, kUBwd><<<(unsigned)((rem + per - 1) / per), kThreads, 0, st>>>(
                g + done, x + done, k ? k + done : k, i ? i + done : i, f + done, dx + done, di ? di + done : di,
                df + done, rem);
            if (int e = check_launch()) return e;
        }
        return HGQ_OK;
    }
    const int64_t rows = n / period;
    const BcastGeom ge = bcast_geom(rows, period, can_vec, kUBcast);
    const size_t need = (size_t)2 * ge.rowBlocks * period * sizeof(float);
    if (ws == nullptr || ws_bytes < need) return HGQ_ERR_WORKSPACE;
    if (!aligned(ws, 4)) return HGQ_ERR_ALIGN;
    dim3 grid((unsigned)ge.colTiles, (unsigned)ge.rowBlocks);
    const bool want_di = (di != nullptr) && (OM == OM_SAT || OM == OM_SAT_SYM);
    if (ge.vec == 4)
        k_bwd_bcast<RM, OM, 4, kUBcast><<<grid, kThreads, 0, st>>>(g, x, k, i, f, dx, (float *)ws, want_di, rows, ge.V, ge.TX,
                                                                 ge.rowsPerBlock);
    else
        k_bwd_bcast<RM, OM, 1, kUBcast><<<grid, kThreads, 0, st>>>(g, x, k, i, f, dx, (float *)ws, want_di, rows, ge.V, ge.TX,
                                                                 ge.rowsPerBlock);
    if (int e = check_launch()) return e;
    if (di != nullptr && !want_di) {
        cudaError_t e = cudaMemsetAsync(di, 0, sizeof(float) * period, st);
        if (e != cudaSuccess) return (int)e;
    }
    dim3 g2((unsigned)((period + kThreads / 32 - 1) / (kThreads / 32)), 2);
    k_colsum_stage2<<<g2, kThreads, 0, st>>>((const float *)ws, want_di ? di : nullptr, df, period, ge.rowBlocks);
    return check_launch();
}

#define HGQ_DISPATCH_RM(RMV, ...)                                        \
    switch (RMV) {                                                       \
        case RM_TRN: { constexpr int RM = RM_TRN; __VA_ARGS__; } break;         \
        case RM_RND: { constexpr int RM = RM_RND; __VA_ARGS__; } break;         \
        case RM_RND_CONV: { constexpr int RM = RM_RND_CONV; __VA_ARGS__; } break; \
        default: return HGQ_ERR_MODE;                                    \
    }

static int check_common(const void *x, const void *f, int64_t n, int64_t &period, int round_mode, int overflow_mode,
                        unsigned flags) {
    if (n < 0 || period < 0) return HGQ_ERR_SIZE;
    if (period == 0) period = n;
    if (n > 0 && (period > n || n % period != 0)) return HGQ_ERR_SIZE;
    if (round_mode < 0 || round_mode > 2 || overflow_mode < 0 || overflow_mode > 3) return HGQ_ERR_MODE;
    if (flags & ~(HGQ_FLAG_TRAINING | HGQ_FLAG_ZERO_NONPOS)) return HGQ_ERR_MODE;
    if (n > 0 && (x == nullptr || f == nullptr)) return HGQ_ERR_NULL;
    return HGQ_OK;
}

}  // namespace hgq

using namespace hgq;

extern "C" int hgq_quantize_fwd(const float *x, const uint8_t *k, const float *i, const float *f, float *y,
                                float *absmax, int64_t n, int64_t period, int round_mode, int overflow_mode,
                                unsigned flags, void *stream) {
    if (int e = check_common(x, f, n, period, round_mode, overflow_mode, flags)) return e;
    if (n == 0) {
        if (absmax != nullptr && period > 0) {  // the maximum over zero rows of |.|
            const cudaError_t ce = cudaMemsetAsync(absmax, 0, (size_t)period * sizeof(float), (cudaStream_t)stream);
            if (ce != cudaSuccess) return (int)ce;
        }
        return HGQ_OK;
    }
    if (y == nullptr) return HGQ_ERR_NULL;
    // WRAP leaves the value unwrapped while training (the integer bits are tracked instead).
    int om = overflow_mode;
    if (om == OM_WRAP && (flags & HGQ_FLAG_TRAINING)) om = OM_NONE;
    if (om != OM_NONE && (k == nullptr || i == nullptr)) return HGQ_ERR_NULL;
    if (!aligned(x, 4) || !aligned(y, 4) || !aligned(f, 4) || !aligned(i, 4) || !aligned(absmax, 4)) return HGQ_ERR_ALIGN;
    if (absmax != nullptr && period == n) return HGQ_ERR_SIZE;  // absmax is a broadcast-layout reduction
    const bool zero = (flags & HGQ_FLAG_ZERO_NONPOS) != 0;
    if (zero && om == OM_NONE) return HGQ_ERR_MODE;  // the zeroing is an eval-mode step; eval never rounds only
    cudaStream_t st = (cudaStream_t)stream;
    HGQ_DISPATCH_RM(round_mode, {
        switch (om) {
            case OM_NONE: return launch_fwd<RM, OM_NONE>(x, k, i, f, y, absmax, n, period, false, st);
            case OM_WRAP: return launch_fwd<RM, OM_WRAP>(x, k, i, f, y, absmax, n, period, zero, st);
            case OM_SAT: return launch_fwd<RM, OM_SAT>(x, k, i, f, y, absmax, n, period, zero, st);
            default: return launch_fwd<RM, OM_SAT_SYM>(x, k, i, f, y, absmax, n, period, zero, st);
        }
    });
    return HGQ_OK;
}

extern "C" size_t hgq_quantize_bwd_workspace(int64_t n, int64_t period) {
    if (n <= 0 || period <= 0 || period >= n || n % period != 0) return 0;
    const int64_t rows = n / period;
    const BcastGeom a = bcast_geom(rows, period, true, kUBcast);
    const BcastGeom b = bcast_geom(rows, period, false, kUBcast);
    const int rb = a.rowBlocks > b.rowBlocks ? a.rowBlocks : b.rowBlocks;
    return (size_t)2 * rb * period * sizeof(float);
}

extern "C" int hgq_quantize_bwd(const float *g, const float *x, const uint8_t *k, const float *i, const float *f,
                                float *dx, float *di, float *df, int64_t n, int64_t period, int round_mode,
                                int overflow_mode, unsigned flags, void *workspace, size_t workspace_bytes,
                                void *stream) {
    if (int e = check_common(x, f, n, period, round_mode, overflow_mode, flags)) return e;
    if (flags & HGQ_FLAG_ZERO_NONPOS) return HGQ_ERR_MODE;  // the backward exists for training only
    if (n == 0) {
        // an empty batch: the sums over zero rows are zero
        cudaStream_t st0 = (cudaStream_t)stream;
        for (float *out : {df, di}) {
            if (out == nullptr || period <= 0) continue;
            const cudaError_t ce = cudaMemsetAsync(out, 0, (size_t)period * sizeof(float), st0);
            if (ce != cudaSuccess) return (int)ce;
        }
        return HGQ_OK;
    }
    if (g == nullptr || df == nullptr) return HGQ_ERR_NULL;
    if (dx == nullptr && period == n) return HGQ_ERR_NULL;
    int om = overflow_mode;
    if (om == OM_WRAP) om = OM_NONE;  // training-mode WRAP is rounding only
    if (om != OM_NONE && (k == nullptr || i == nullptr)) return HGQ_ERR_NULL;
    if (!aligned(g, 4) || !aligned(x, 4) || !aligned(f, 4) || !aligned(i, 4) || !aligned(dx, 4) || !aligned(di, 4) ||
        !aligned(df, 4))
        return HGQ_ERR_ALIGN;
    cudaStream_t st = (cudaStream_t)stream;
    HGQ_DISPATCH_RM(round_mode, {
        switch (om) {
            case OM_NONE: return launch_bwd<RM, OM_NONE>(g, x, k, i, f, dx, di, df, n, period, workspace, workspace_bytes, st);
            case OM_SAT: return launch_bwd<RM, OM_SAT>(g, x, k, i, f, dx, di, df, n, period, workspace, workspace_bytes, st);
            default: return launch_bwd<RM, OM_SAT_SYM>(g, x, k, i, f, dx, di, df, n, period, workspace, workspace_bytes, st);
        }
    });
    return HGQ_OK;
}

extern "C" int64_t hgq_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

extern "C" int hgq_abi_version(void) { return 1; }

extern "C" const char *hgq_status_string(int status) {
    switch (status) {
        case HGQ_OK: return "ok";
        case HGQ_ERR_NULL: return "a required pointer is NULL";
        case HGQ_ERR_SIZE: return "a size or shape argument is invalid";
        case HGQ_ERR_MODE: return "unknown mode or flag";
        case HGQ_ERR_ALIGN: return "a pointer is misaligned for its element type";
        case HGQ_ERR_WORKSPACE: return "workspace missing or too small";
        case HGQ_ERR_DEVICE: return "the current device is not sm_100";
        case HGQ_ERR_TIMEOUT: return "a bounded device-side wait gave up";
        default: break;
    }
    if (status > 0) return cudaGetErrorString((cudaError_t)status);
    return "unknown status";
}

// ---- backward entry for callers that cannot allocate device memory --------------------------------
//
// Some hosts of this library may not create device allocations of their own: a plugin that runs inside
// a framework whose memory pool already owns the whole GPU (a cudaMalloc from the plugin would fail or
// starve the pool), or a service with a fixed, audited memory budget where every allocation has to be
// accounted for before start-up.  For them the column-sum partials of the broadcast-layout backward
// live in this fixed array instead of in a caller-provided workspace.  Every GPU that loads the library
// holds the array until the process exits.
namespace {

constexpr size_t kNoAllocScratchBytes = HGQ_NOALLOC_SCRATCH_BYTES;
__device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];

constexpr int kNoAllocMaxDevices = 64;
std::atomic<void *> g_noalloc_addr[kNoAllocMaxDevices];  // device address of g_noalloc_scratch, per device (null: not looked up yet)

// In host code `g_noalloc_scratch` is only a handle for the runtime, not an address a kernel can use:
// the device address is looked up once per device, with that device current.
int noalloc_scratch_address(void **out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= kNoAllocMaxDevices) return HGQ_ERR_DEVICE;
    void *p = g_noalloc_addr[dev].load(std::memory_order_acquire);
    if (p == nullptr) {
        e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (e != cudaSuccess) return (int)e;
        if (p == nullptr) return HGQ_ERR_DEVICE;
        g_noalloc_addr[dev].store(p, std::memory_order_release);  // first callers that race here store the same address
    }
    *out = p;
    return HGQ_OK;
}

}  // namespace

extern "C" int hgq_quantize_bwd_noalloc(const float *g, const float *x, const uint8_t *k, const float *i,
                                        const float *f, float *dx, float *di, float *df, int64_t n, int64_t period,
                                        int round_mode, int overflow_mode, unsigned flags, void *stream) {
    if (n < 0 || period < 0) return HGQ_ERR_SIZE;
    const size_t need = hgq_quantize_bwd_workspace(n, period == 0 ? n : period);
    if (need > kNoAllocScratchBytes) return HGQ_ERR_SIZE;  // beyond the built-in scratch: use hgq_quantize_bwd
    void *scratch = nullptr;
    if (need > 0) {
        if (int e = noalloc_scratch_address(&scratch)) return e;
    }
    // Nothing in the scratch has to start at zero: the first kernel writes every partial the second one reads.
    return hgq_quantize_bwd(g, x, k, i, f, dx, di, df, n, period, round_mode, overflow_mode, flags, scratch,
                            need > 0 ? kNoAllocScratchBytes : 0, stream);
}
