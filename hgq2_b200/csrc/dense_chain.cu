// K2m (a stack of small dense layers in one launch): forward and backward of consecutive QDense layers whose widths are at
// most 64, with the activations of a 128-row tile staying in shared memory from layer to layer.
//
// Stands in for QDense.call (src/hgq/layers/core/dense.py:60-68) applied layer after layer with a rounding-only input
// quantizer each (the training-mode WRAP activation quantizer, src/hgq/quantizer/internal/fixed_point_quantizer.py:403-424)
// and for the autograd backward of that stack:
//     forward, layer l:   xq = round(x_l * 2^f) / 2^f,  y_l = act(xq @ Wq_l + bq_l),  x_{l+1} = y_l,  absmax_l = max |xq|
//     backward, layer l:  G = dY_l * (y_l > 0);  dXq = G @ Wq_l^T;  dWq_l = xq^T @ G;  dbq_l = sum_r G;
//                         df_l[k] = sum_r (-ln2 (xq - x_l)) * dXq;  dY_{l-1} = dXq
// Why a kernel of its own: a jet-tagger MLP (16 -> 64 -> 32 -> 32 -> 5 at batch 16384) is one 128-row tile per SM.  On the
// tensor-core kernels every layer is a launch whose single tile walks the whole chain of dependent latencies (weights ->
// copy -> conversion -> product -> read-back -> store): 7 to 8 microseconds forward and 14 to 19 backward per layer for a
// few hundred nanoseconds of arithmetic.  Here the four layers share one launch, the products are fp32 FMAs on the CUDA
// cores (420 MFLOP per step: microseconds), and only the layer outputs the backward needs go to memory.
// Per-block partial sums of dWq / dbq / df are reduced in a fixed order by a second kernel: results do not depend on scheduling.
// HBM traffic: x and every y_l once forward; dY, x, every y_l once backward.
#include <cuda_runtime.h>

#include "../../include/hgq_b200.h"
#include "hgq_common.cuh"
#include "hgq_math.cuh"

namespace hgq {

constexpr int kMcThreads = 256;
constexpr int kMcRows = 128;      // rows of a tile
constexpr int kMcWidth = 64;      // largest layer width
constexpr int kMcLd = 68;         // row stride (floats) of an activation tile in shared memory: 16-byte aligned rows
constexpr int kMcMaxLayers = HGQ_CHAIN_MAX_LAYERS;

struct McLayer {
    const float *qf, *wq, *bq;
    float *y, *absmax, *dwq, *dbq, *df;
    int K, N, relu, rm;
    int part_off;  // offset (floats) of this layer's [dWq | dbq | df] record inside a block's partial record
};

struct McParams {
    const float *x, *gy;
    float *dx, *part;
    int64_t M, tiles;
    int n, part_stride;
    McLayer L[kMcMaxLayers];
};

__device__ __forceinline__ float mc_round(float v, float s, float inv, int rm) {
    const float xs = __fmul_rn(v, s);
    const float q = (rm == RM_RND) ? floorf(__fadd_rn(xs, 0.5f)) : ((rm == RM_TRN) ? floorf(xs) : rintf(xs));
    return __fmul_rn(q, inv);
}

// Output tile of a product with `groups` groups of four output columns: thread t takes column group t % groups and the rows
// slot, slot + slots, ... of the tile (slots = 256 / groups threads per column group, at most 8 rows each for groups <= 16).
struct McMap {
    int groups, slots, cg, slot;
    bool active;
};
__device__ __forceinline__ McMap mc_map(int width, int tid) {
    McMap m;
    m.groups = (width + 3) >> 2;
    m.slots = kMcThreads / m.groups;
    m.cg = tid % m.groups;
    m.slot = tid / m.groups;
    m.active = m.slot < m.slots;
    return m;
}

// ---- forward --------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kMcThreads) k_dense_chain_fwd(const McParams P) {
    extern __shared__ __align__(16) float smem_f[];
    float *buf0 = smem_f;                                   // [128][68] activations entering the current layer
    float *buf1 = buf0 + kMcRows * kMcLd;                   // [128][68] activations leaving it
    float *W = buf1 + kMcRows * kMcLd;                      // [K][Nw] weights, Nw = 4 * groups, zero beyond N
    float *bias = W + kMcWidth * kMcWidth;                  // [64]
    float *sc = bias + kMcWidth;                            // [64] 2^f
    float *isc = sc + kMcWidth;                             // [64] 2^-f
    unsigned *colmax = reinterpret_cast<unsigned *>(isc + kMcWidth);  // [64] bits of the column maxima of |xq|
    const int tid = threadIdx.x;

    for (int64_t tile = blockIdx.x; tile < P.tiles; tile += gridDim.x) {
        const int64_t row0 = tile * kMcRows;
        const int rows_here = (int)((P.M - row0) < kMcRows ? (P.M - row0) : kMcRows);
        float *in = buf0, *out = buf1;
        {   // the tile of the first layer's input
            const int K0 = P.L[0].K;
            for (int e = tid; e < kMcRows * K0; e += kMcThreads) {
                const int r = e / K0, k = e - r * K0;
                in[r * kMcLd + k] = (r < rows_here) ? __ldcs(P.x + (row0 + r) * K0 + k) : 0.f;
            }
        }
        for (int l = 0; l < P.n; ++l) {
            const McLayer &Ly = P.L[l];
            const int K = Ly.K, N = Ly.N;
            const McMap m = mc_map(N, tid);
            const int Nw = m.groups * 4;
            for (int e = tid; e < K * Nw; e += kMcThreads) {
                const int k = e / Nw, n = e - k * Nw;
                W[e] = (n < N) ? __ldg(Ly.wq + k * N + n) : 0.f;
            }
            if (tid < kMcWidth) {
                bias[tid] = (Ly.bq != nullptr && tid < N) ? __ldg(Ly.bq + tid) : 0.f;
                const int fi = (tid < K) ? __float2int_rn(__ldg(Ly.qf + tid)) : 0;
                sc[tid] = pow2i(fi);
                isc[tid] = pow2i(-fi);
                colmax[tid] = 0u;
            }
            __syncthreads();
            // input quantizer in place, column maxima of the rounded values over the rows that exist
            if (kMcThreads % K == 0) {  // a thread stays in one column
                const int k = tid % K;
                const float s = sc[k], inv = isc[k];
                float mx = 0.f;
                for (int r = tid / K; r < kMcRows; r += kMcThreads / K) {
                    const float q = mc_round(in[r * kMcLd + k], s, inv, Ly.rm);
                    in[r * kMcLd + k] = q;
                    if (r < rows_here) mx = fmaxf(mx, fabsf(q));
                }
                if (Ly.absmax != nullptr) atomicMax(colmax + k, __float_as_uint(mx));
            } else {
                for (int e = tid; e < kMcRows * K; e += kMcThreads) {
                    const int r = e / K, k = e - r * K;
                    const float q = mc_round(in[r * kMcLd + k], sc[k], isc[k], Ly.rm);
                    in[r * kMcLd + k] = q;
                    if (Ly.absmax != nullptr && r < rows_here) atomicMax(colmax + k, __float_as_uint(fabsf(q)));
                }
            }
            __syncthreads();
            if (Ly.absmax != nullptr && tid < K) atomicMax(reinterpret_cast<unsigned *>(Ly.absmax) + tid, colmax[tid]);
            // y = act(xq @ W + b): rows slot + j * slots of column group cg
            if (m.active) {
                float acc[8][4];
#pragma unroll
                for (int j = 0; j < 8; ++j)
#pragma unroll
                    for (int c = 0; c < 4; ++c) acc[j][c] = 0.f;
                const float *arow = in + m.slot * kMcLd;
                const int rstep = m.slots * kMcLd;
                for (int k = 0; k < K; ++k) {
                    const float4 w4 = *reinterpret_cast<const float4 *>(W + k * Nw + m.cg * 4);
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        if (m.slot + j * m.slots < kMcRows) {
                            const float a = arow[j * rstep + k];
                            acc[j][0] = __fmaf_rn(a, w4.x, acc[j][0]);
                            acc[j][1] = __fmaf_rn(a, w4.y, acc[j][1]);
                            acc[j][2] = __fmaf_rn(a, w4.z, acc[j][2]);
                            acc[j][3] = __fmaf_rn(a, w4.w, acc[j][3]);
                        }
                    }
                }
                const float lo = Ly.relu ? 0.f : -INFINITY;
                const int n0 = m.cg * 4;
                const bool vec = (N % 4 == 0) && aligned(Ly.y, 16);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int r = m.slot + j * m.slots;
                    if (r < kMcRows) {
                        float4 o;
                        o.x = fmaxf(__fadd_rn(acc[j][0], bias[n0]), lo);
                        o.y = fmaxf(__fadd_rn(acc[j][1], bias[n0 + 1]), lo);
                        o.z = fmaxf(__fadd_rn(acc[j][2], bias[n0 + 2]), lo);
                        o.w = fmaxf(__fadd_rn(acc[j][3], bias[n0 + 3]), lo);
                        *reinterpret_cast<float4 *>(out + r * kMcLd + n0) = o;
                        if (r < rows_here) {
                            float *dst = Ly.y + (row0 + r) * N + n0;
                            if (vec) {
                                *reinterpret_cast<float4 *>(dst) = o;
                            } else {
                                const float ov[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
                                for (int c = 0; c < 4; ++c)
                                    if (n0 + c < N) dst[c] = ov[c];
                            }
                        }
                    }
                }
            }
            __syncthreads();
            float *t = in; in = out; out = t;
        }
    }
}

// ---- backward -------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kMcThreads) k_dense_chain_bwd(const McParams P) {
    extern __shared__ __align__(16) float smem_f[];
    float *G = smem_f;                                      // [128][68] gradient entering the current layer (its output side)
    float *D = G + kMcRows * kMcLd;                         // [128][68] gradient leaving it (dXq)
    float *XQ = D + kMcRows * kMcLd;                        // [128][68] rounded inputs
    float *ER = XQ + kMcRows * kMcLd;                       // [128][68] -ln2 (xq - x)
    float *WT = ER + kMcRows * kMcLd;                       // [N][Kw] transposed weights, Kw = 4 * groups of K
    float *red = WT + kMcWidth * kMcWidth;                  // [256][4] per-thread df partials
    float *sc = red + kMcThreads * 4;                       // [64], [64]
    float *isc = sc + kMcWidth;
    float *acc_s = isc + kMcWidth;                          // per layer [dWq (K x N) | dbq (N) | df (K)] sums over this block's tiles
    const int tid = threadIdx.x;

    for (int e = tid; e < P.part_stride; e += kMcThreads) acc_s[e] = 0.f;
    __syncthreads();

    for (int64_t tile = blockIdx.x; tile < P.tiles; tile += gridDim.x) {
        const int64_t row0 = tile * kMcRows;
        const int rows_here = (int)((P.M - row0) < kMcRows ? (P.M - row0) : kMcRows);
        {
            const int NL = P.L[P.n - 1].N;
            for (int e = tid; e < kMcRows * NL; e += kMcThreads) {
                const int r = e / NL, n = e - r * NL;
                G[r * kMcLd + n] = (r < rows_here) ? __ldcs(P.gy + (row0 + r) * NL + n) : 0.f;
            }
        }
        float *g_in = G, *g_out = D;
        for (int l = P.n - 1; l >= 0; --l) {
            const McLayer &Ly = P.L[l];
            const int K = Ly.K, N = Ly.N;
            const McMap mk = mc_map(K, tid);    // dXq tile: column groups over k
            const McMap mn = mc_map(N, tid);    // dWq tile: column groups over n
            const int Kw = mk.groups * 4, Nw = mn.groups * 4;
            float *a_l = acc_s + Ly.part_off;
            __syncthreads();  // the previous layer's readers of WT / XQ / ER / red are done
            if (tid < kMcWidth) {
                const int fi = (tid < K) ? __float2int_rn(__ldg(Ly.qf + tid)) : 0;
                sc[tid] = pow2i(fi);
                isc[tid] = pow2i(-fi);
            }
            for (int e = tid; e < N * Kw; e += kMcThreads) {  // coalesced over n in memory, transposed into shared memory
                const int k = e / N, n = e - k * N;
                if (k < Kw) WT[n * Kw + k] = (k < K) ? __ldg(Ly.wq + k * N + n) : 0.f;
            }
            if (Ly.relu) {
                for (int e = tid; e < kMcRows * N; e += kMcThreads) {
                    const int r = e / N, n = e - r * N;
                    if (r < rows_here && !(__ldcs(Ly.y + (row0 + r) * N + n) > 0.f)) g_in[r * kMcLd + n] = 0.f;
                }
            }
            // zero the padding columns the float4 reads of the dWq product touch
            if (Nw != N)
                for (int e = tid; e < kMcRows * (Nw - N); e += kMcThreads) {
                    const int r = e / (Nw - N), n = N + (e - r * (Nw - N));
                    g_in[r * kMcLd + n] = 0.f;
                }
            __syncthreads();  // sc / isc
            {
                const float *xl = (l == 0) ? P.x : P.L[l - 1].y;
                for (int e = tid; e < kMcRows * K; e += kMcThreads) {
                    const int r = e / K, k = e - r * K;
                    const float v = (r < rows_here) ? __ldcs(xl + (row0 + r) * K + k) : 0.f;
                    const float q = mc_round(v, sc[k], isc[k], Ly.rm);
                    XQ[r * kMcLd + k] = q;
                    ER[r * kMcLd + k] = __fmul_rn(__fsub_rn(q, v), -kLn2);
                }
            }
            __syncthreads();
            // ---- dXq = G @ W^T, and the df terms of this thread's elements -------------------------------------------------
            float dfp[4] = {0.f, 0.f, 0.f, 0.f};
            if (mk.active) {
                float acc[8][4];
#pragma unroll
                for (int j = 0; j < 8; ++j)
#pragma unroll
                    for (int c = 0; c < 4; ++c) acc[j][c] = 0.f;
                const float *grow = g_in + mk.slot * kMcLd;
                const int rstep = mk.slots * kMcLd;
                for (int n = 0; n < N; ++n) {
                    const float4 w4 = *reinterpret_cast<const float4 *>(WT + n * Kw + mk.cg * 4);
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        if (mk.slot + j * mk.slots < kMcRows) {
                            const float g = grow[j * rstep + n];
                            acc[j][0] = __fmaf_rn(g, w4.x, acc[j][0]);
                            acc[j][1] = __fmaf_rn(g, w4.y, acc[j][1]);
                            acc[j][2] = __fmaf_rn(g, w4.z, acc[j][2]);
                            acc[j][3] = __fmaf_rn(g, w4.w, acc[j][3]);
                        }
                    }
                }
                const int k0 = mk.cg * 4;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int r = mk.slot + j * mk.slots;
                    if (r < kMcRows) {
                        const float4 er = *reinterpret_cast<const float4 *>(ER + r * kMcLd + k0);
                        dfp[0] = __fmaf_rn(er.x, acc[j][0], dfp[0]);
                        dfp[1] = __fmaf_rn(er.y, acc[j][1], dfp[1]);
                        dfp[2] = __fmaf_rn(er.z, acc[j][2], dfp[2]);
                        dfp[3] = __fmaf_rn(er.w, acc[j][3], dfp[3]);
                        *reinterpret_cast<float4 *>(g_out + r * kMcLd + k0) = make_float4(acc[j][0], acc[j][1], acc[j][2], acc[j][3]);
                        if (l == 0 && P.dx != nullptr && r < rows_here) {
#pragma unroll
                            for (int c = 0; c < 4; ++c)
                                if (k0 + c < K) P.dx[(row0 + r) * K + k0 + c] = acc[j][c];
                        }
                    }
                }
            }
            *reinterpret_cast<float4 *>(red + tid * 4) = make_float4(dfp[0], dfp[1], dfp[2], dfp[3]);
            // ---- dWq += xq^T @ G: thread t takes column group t % groups(N) and the inputs slot, slot + slots, ... ------------
            if (mn.active) {
                float acc[4][4];
#pragma unroll
                for (int j = 0; j < 4; ++j)
#pragma unroll
                    for (int c = 0; c < 4; ++c) acc[j][c] = 0.f;
                const int kpt = (K + mn.slots - 1) / mn.slots;  // inputs per thread: at most 4 (64 inputs, 16 slots)
                for (int r = 0; r < kMcRows; ++r) {
                    const float4 g4 = *reinterpret_cast<const float4 *>(g_in + r * kMcLd + mn.cg * 4);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int k = mn.slot + j * mn.slots;
                        if (j < kpt && k < K) {
                            const float xv = XQ[r * kMcLd + k];
                            acc[j][0] = __fmaf_rn(xv, g4.x, acc[j][0]);
                            acc[j][1] = __fmaf_rn(xv, g4.y, acc[j][1]);
                            acc[j][2] = __fmaf_rn(xv, g4.z, acc[j][2]);
                            acc[j][3] = __fmaf_rn(xv, g4.w, acc[j][3]);
                        }
                    }
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int k = mn.slot + j * mn.slots;
                    if (j < kpt && k < K) {
#pragma unroll
                        for (int c = 0; c < 4; ++c) {
                            const int n = mn.cg * 4 + c;
                            if (n < N) a_l[k * N + n] = __fadd_rn(a_l[k * N + n], acc[j][c]);
                        }
                    }
                }
            }
            // dbq += column sums of G (fixed order over the rows)
            if (tid < N) {
                float s = 0.f;
                for (int r = 0; r < kMcRows; ++r) s = __fadd_rn(s, g_in[r * kMcLd + tid]);
                a_l[K * N + tid] = __fadd_rn(a_l[K * N + tid], s);
            }
            __syncthreads();  // red complete
            if (tid < K) {   // df[k]: the partials of the threads that hold column k, in slot order
                const int cg = tid >> 2, c = tid & 3;
                float s = 0.f;
                for (int slot = 0; slot < mk.slots; ++slot) s = __fadd_rn(s, red[(slot * mk.groups + cg) * 4 + c]);
                a_l[K * N + N + tid] = __fadd_rn(a_l[K * N + N + tid], s);
            }
            float *t = g_in; g_in = g_out; g_out = t;
        }
        __syncthreads();
    }
    __syncthreads();
    float *pb = P.part + (int64_t)blockIdx.x * P.part_stride;
    for (int e = tid; e < P.part_stride; e += kMcThreads) pb[e] = acc_s[e];
}

// Sums the blocks' partial records in a fixed order (in double) and scatters element e of the record to the layer output it
// belongs to.  A block owns eight consecutive elements; its 32 groups of eight lanes walk the records 32 apart.
__global__ void __launch_bounds__(kThreads) k_dense_chain_stage2(const McParams P, int nparts) {
    __shared__ double red[kThreads / 32][8];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, sub = lane >> 3, j = lane & 7;
    const int e = blockIdx.x * 8 + j;
    double acc = 0.0;
    if (e < P.part_stride) {
#pragma unroll 4
        for (int p = warp * 4 + sub; p < nparts; p += kThreads / 8) acc += (double)P.part[(int64_t)p * P.part_stride + e];
    }
    acc += __shfl_down_sync(0xffffffffu, acc, 16);
    acc += __shfl_down_sync(0xffffffffu, acc, 8);
    if (sub == 0) red[warp][j] = acc;
    __syncthreads();
    if (threadIdx.x < 8 && e < P.part_stride) {
        double a = 0.0;
#pragma unroll
        for (int w = 0; w < kThreads / 32; ++w) a += red[w][threadIdx.x];
        for (int l = 0; l < P.n; ++l) {
            const McLayer &Ly = P.L[l];
            const int o = e - Ly.part_off, nw = Ly.K * Ly.N;
            if (o < 0 || o >= nw + Ly.N + Ly.K) continue;
            if (o < nw) Ly.dwq[o] = (float)a;
            else if (o < nw + Ly.N) { if (Ly.dbq != nullptr) Ly.dbq[o - nw] = (float)a; }
            else if (Ly.df != nullptr) Ly.df[o - nw - Ly.N] = (float)a;
            break;
        }
    }
}

static size_t mc_fwd_smem() { return (size_t)(2 * kMcRows * kMcLd + kMcWidth * kMcWidth + 4 * kMcWidth) * sizeof(float); }
static size_t mc_bwd_smem(int part_stride) {
    return (size_t)(4 * kMcRows * kMcLd + kMcWidth * kMcWidth + kMcThreads * 4 + 2 * kMcWidth + part_stride) * sizeof(float);
}

static int mc_fill(int n_layers, const hgq_chain_layer *layers, bool backward, McParams &p) {
    if (layers == nullptr) return HGQ_ERR_NULL;
    if (n_layers < 1 || n_layers > kMcMaxLayers) return HGQ_ERR_SIZE;
    int off = 0;
    for (int l = 0; l < n_layers; ++l) {
        const hgq_chain_layer &s = layers[l];
        if (s.K < 1 || s.K > kMcWidth || s.N < 1 || s.N > kMcWidth) return HGQ_ERR_SIZE;
        if (l > 0 && s.K != layers[l - 1].N) return HGQ_ERR_SIZE;
        if (s.round_mode < 0 || s.round_mode > 2) return HGQ_ERR_MODE;
        if (s.qf == nullptr || s.wq == nullptr || s.y == nullptr) return HGQ_ERR_NULL;
        if (backward && s.dwq == nullptr) return HGQ_ERR_NULL;
        McLayer &d = p.L[l];
        d.qf = s.qf; d.wq = s.wq; d.bq = s.bq; d.y = s.y; d.absmax = s.absmax; d.dwq = s.dwq; d.dbq = s.dbq; d.df = s.df;
        d.K = s.K; d.N = s.N; d.relu = s.relu ? 1 : 0; d.rm = s.round_mode; d.part_off = off;
        off += s.K * s.N + s.N + s.K;
    }
    p.n = n_layers;
    p.part_stride = off;
    if (mc_bwd_smem(off) > 226 * 1024) return HGQ_ERR_SIZE;
    return HGQ_OK;
}

static int mc_grid(int64_t tiles) { return (int)(tiles < num_sms() ? tiles : num_sms()); }

}  // namespace hgq

using namespace hgq;

extern "C" int hgq_dense_chain_supported(int n_layers, const hgq_chain_layer *layers) {
    if (layers == nullptr || n_layers < 1 || n_layers > kMcMaxLayers) return 0;
    int off = 0;
    for (int l = 0; l < n_layers; ++l) {
        if (layers[l].K < 1 || layers[l].K > kMcWidth || layers[l].N < 1 || layers[l].N > kMcWidth) return 0;
        if (l > 0 && layers[l].K != layers[l - 1].N) return 0;
        off += layers[l].K * layers[l].N + layers[l].N + layers[l].K;
    }
    return mc_bwd_smem(off) <= 226 * 1024 ? 1 : 0;
}

extern "C" size_t hgq_dense_chain_workspace(int64_t M, int n_layers, const hgq_chain_layer *layers) {
    if (M <= 0 || !hgq_dense_chain_supported(n_layers, layers)) return 0;
    size_t off = 0;
    for (int l = 0; l < n_layers; ++l) off += (size_t)layers[l].K * layers[l].N + layers[l].N + layers[l].K;
    return (size_t)num_sms() * off * sizeof(float);
}

extern "C" int hgq_dense_chain_fwd(const float *x, int64_t M, int n_layers, const hgq_chain_layer *layers, void *stream) {
    if (x == nullptr) return HGQ_ERR_NULL;
    if (M <= 0) return HGQ_ERR_SIZE;
    McParams p;
    if (int e = mc_fill(n_layers, layers, false, p)) return e;
    p.x = x; p.gy = nullptr; p.dx = nullptr; p.part = nullptr; p.M = M; p.tiles = (M + kMcRows - 1) / kMcRows;
    const size_t smem = mc_fwd_smem();
    cudaError_t ce = cudaFuncSetAttribute(k_dense_chain_fwd, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (ce != cudaSuccess) return (int)ce;
    k_dense_chain_fwd<<<mc_grid(p.tiles), kMcThreads, smem, (cudaStream_t)stream>>>(p);
    return check_launch();
}

extern "C" int hgq_dense_chain_bwd(const float *gy, const float *x, float *dx, int64_t M, int n_layers, const hgq_chain_layer *layers,
                                   void *workspace, size_t workspace_bytes, void *stream) {
    if (gy == nullptr || x == nullptr) return HGQ_ERR_NULL;
    if (M <= 0) return HGQ_ERR_SIZE;
    McParams p;
    if (int e = mc_fill(n_layers, layers, true, p)) return e;
    p.x = x; p.gy = gy; p.dx = dx; p.M = M; p.tiles = (M + kMcRows - 1) / kMcRows;
    const int grid = mc_grid(p.tiles);
    if (workspace == nullptr || workspace_bytes < (size_t)grid * p.part_stride * sizeof(float)) return HGQ_ERR_WORKSPACE;
    if (!aligned(workspace, 16)) return HGQ_ERR_ALIGN;
    p.part = (float *)workspace;
    const size_t smem = mc_bwd_smem(p.part_stride);
    cudaError_t ce = cudaFuncSetAttribute(k_dense_chain_bwd, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (ce != cudaSuccess) return (int)ce;
    cudaStream_t st = (cudaStream_t)stream;
    k_dense_chain_bwd<<<grid, kMcThreads, smem, st>>>(p);
    if (int e = check_launch()) return e;
    k_dense_chain_stage2<<<(p.part_stride + 7) / 8, kThreads, 0, st>>>(p, grid);
    return check_launch();
}
