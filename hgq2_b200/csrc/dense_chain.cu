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

constexpr int kMcThreads = 512;
constexpr int kMcRows = 128;      // most rows of a tile (the shared-memory buffers are this tall)
constexpr int kMcWidth = 64;      // largest layer width
constexpr int kMcLd = 68;         // row stride (floats) of an activation tile in shared memory: 16-byte aligned rows
constexpr int kMcMaxLayers = HGQ_CHAIN_MAX_LAYERS;

struct McLayer {
    const float *qf, *wq, *bq;
    float *y, *absmax, *dwq, *dbq, *df;
    int K, N, relu, rm;
    int part_off;  // offset (floats) of this layer's [dWq (K x N) | dbq (N) | df (K)] record inside a block's partial record
    int w_off;     // offset (floats) of this layer's weights inside the shared-memory weight area (forward: [K][Nw], backward: [N][Kw])
};

struct McParams {
    const float *x, *gy;
    float *dx, *part;
    int64_t M, tiles;
    int n, part_stride, w_total;
    int R;  // rows of a tile: as few as spread the batch over every SM (a multiple of 8, at most 128)
    McLayer L[kMcMaxLayers];
};

// 4-byte asynchronous copy global -> shared (zero when `valid` is false): a thread issues all of its copies and waits once,
// so the loads of every layer's weights overlap instead of each loop iteration waiting for its own
__device__ __forceinline__ void mc_cp4(float *dst, const float *src, bool valid) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    const int bytes = valid ? 4 : 0;
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(d), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mc_cp_wait() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// Phase timing of block 0 (stand-alone profiling builds only): time since the previous mark, added to slot i.
#ifdef HGQ_MC_PROF
__device__ unsigned long long g_mc_prof[32];
__device__ __forceinline__ unsigned long long mc_now() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
#define MC_DECL unsigned long long mc_t0 = mc_now()
#define MC_MARK(i)                                           \
    do {                                                     \
        if (blockIdx.x == 0 && threadIdx.x == 0) {           \
            const unsigned long long mc_t = mc_now();        \
            g_mc_prof[i] += mc_t - mc_t0;                    \
            mc_t0 = mc_t;                                    \
        }                                                    \
    } while (0)
#else
#define MC_DECL
#define MC_MARK(i)
#endif

__device__ __forceinline__ float mc_round(float v, float s, float inv, int rm) {
    const float xs = __fmul_rn(v, s);
    const float q = (rm == RM_RND) ? floorf(__fadd_rn(xs, 0.5f)) : ((rm == RM_TRN) ? floorf(xs) : rintf(xs));
    return __fmul_rn(q, inv);
}

// Output tile of a product with `groups` groups of four output columns: thread t takes column group t % groups and the rows
// (or inputs) slot, slot + slots, ... (slots = threads / groups per column group).
struct McMap {
    int groups, slots, cg, slot;
    bool active;
};
__device__ __forceinline__ McMap mc_map(int R, int width, int tid) {
    McMap m;
    m.groups = (width + 3) >> 2;
    // several rows per thread: a 16-byte shared-memory load occupies the load unit for four cycles, so a thread with a single
    // row (one 16-byte and one 4-byte load per four FMAs) would be bound by it.  Four rows for wide outputs; two for narrow
    // ones, where four would leave most warps waiting at the barrier behind a few.
    const int rows_per_thread = m.groups >= 12 ? 4 : 2;
    m.slots = min(kMcThreads / m.groups, (R + rows_per_thread - 1) / rows_per_thread);
    m.cg = tid % m.groups;
    m.slot = tid / m.groups;
    m.active = m.slot < m.slots;
    return m;
}
constexpr int kMcRowsPerThread = 4;  // 128 rows over at least 32 slots (at most 16 column groups)

// f(r, c) for every element of a [128, width] tile.  When the thread count is a multiple of the width a thread stays in one
// column and walks rows a fixed step apart (no division per element: these loops, not the products, were most of the
// instructions of a first version); otherwise elements are dealt out in order.
template <class F>
__device__ __forceinline__ void mc_foreach(int R, int width, int tid, F f) {
    if (kMcThreads % width == 0) {
        const int c = tid % width, step = kMcThreads / width;
#pragma unroll 4
        for (int r = tid / width; r < R; r += step) f(r, c);
    } else {
        for (int e = tid; e < R * width; e += kMcThreads) {
            const int r = e / width;
            f(r, e - r * width);
        }
    }
}

// a tile of a row-major [M, width] matrix into shared memory (rows beyond the matrix read as zero)
__device__ __forceinline__ void mc_load_tile(int R, float *dst, const float *src, int64_t row0, int rows_here, int width, int tid) {
    if ((width & 3) == 0 && aligned(src, 16)) {
        const float4 *s4 = reinterpret_cast<const float4 *>(src + row0 * width);
        const int w4 = width >> 2;
        mc_foreach(R, w4, tid, [&](int r, int c) {
            const float4 v = (r < rows_here) ? __ldcs(s4 + r * w4 + c) : make_float4(0.f, 0.f, 0.f, 0.f);
            *reinterpret_cast<float4 *>(dst + r * kMcLd + c * 4) = v;
        });
    } else {
        const float *s1 = src + row0 * width;
        mc_foreach(R, width, tid, [&](int r, int c) { dst[r * kMcLd + c] = (r < rows_here) ? __ldcs(s1 + r * width + c) : 0.f; });
    }
}

// zero where the layer's output was not positive (the ReLU mask of the gradient)
__device__ __forceinline__ void mc_relu_mask(int R, float *g, const float *y, int64_t row0, int rows_here, int width, int tid) {
    if ((width & 3) == 0 && aligned(y, 16)) {
        const float4 *y4 = reinterpret_cast<const float4 *>(y + row0 * width);
        const int w4 = width >> 2;
        mc_foreach(R, w4, tid, [&](int r, int c) {
            if (r < rows_here) {
                const float4 v = __ldcs(y4 + r * w4 + c);
                float4 *gp = reinterpret_cast<float4 *>(g + r * kMcLd + c * 4);
                float4 t = *gp;
                t.x = v.x > 0.f ? t.x : 0.f; t.y = v.y > 0.f ? t.y : 0.f; t.z = v.z > 0.f ? t.z : 0.f; t.w = v.w > 0.f ? t.w : 0.f;
                *gp = t;
            }
        });
    } else {
        const float *y1 = y + row0 * width;
        mc_foreach(R, width, tid, [&](int r, int c) {
            if (r < rows_here && !(__ldcs(y1 + r * width + c) > 0.f)) g[r * kMcLd + c] = 0.f;
        });
    }
}

// acc[j][0..3] = sum_i A[row_j][i] * B[i][4 cg .. 4 cg + 3] for the JN rows slot, slot + slots, ... of this thread: A is an
// activation tile (row stride kMcLd), B a weight matrix with row stride ldb.  Rows beyond the tile are clamped (computed,
// not stored by the callers), so the loop has no predicate; JN is the number of rows a thread really has (1, 2 or 4).
template <int JN>
__device__ __forceinline__ void mc_rows_product(int R, const float *A, const float *B, int ldb, int depth, const McMap &m, float (&acc)[4][4]) {
    const float *ap[JN];
#pragma unroll
    for (int j = 0; j < JN; ++j) ap[j] = A + min(m.slot + j * m.slots, R - 1) * kMcLd;
    const float *bp = B + m.cg * 4;
#pragma unroll 4
    for (int i = 0; i < depth; ++i) {
        const float4 b4 = *reinterpret_cast<const float4 *>(bp + i * ldb);
#pragma unroll
        for (int j = 0; j < JN; ++j) {
            const float a = ap[j][i];
            acc[j][0] = __fmaf_rn(a, b4.x, acc[j][0]);
            acc[j][1] = __fmaf_rn(a, b4.y, acc[j][1]);
            acc[j][2] = __fmaf_rn(a, b4.z, acc[j][2]);
            acc[j][3] = __fmaf_rn(a, b4.w, acc[j][3]);
        }
    }
}
__device__ __forceinline__ void mc_rows_product_any(int R, const float *A, const float *B, int ldb, int depth, const McMap &m, float (&acc)[4][4]) {
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[j][c] = 0.f;
    const int jn = (R + m.slots - 1) / m.slots;  // 4 unless the tile is shorter than four rows per slot
    if (jn <= 1) mc_rows_product<1>(R, A, B, ldb, depth, m, acc);
    else if (jn == 2) mc_rows_product<2>(R, A, B, ldb, depth, m, acc);
    else mc_rows_product<4>(R, A, B, ldb, depth, m, acc);
}

// ---- forward --------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kMcThreads) k_dense_chain_fwd(const McParams P) {
    extern __shared__ __align__(16) float smem_f[];
    float *buf0 = smem_f;                                   // [128][68] activations entering the current layer
    float *buf1 = buf0 + kMcRows * kMcLd;                   // [128][68] activations leaving it
    float *bias = buf1 + kMcRows * kMcLd;                   // [layers][64]
    float *sc = bias + kMcMaxLayers * kMcWidth;             // [layers][64] 2^f
    float *isc = sc + kMcMaxLayers * kMcWidth;              // [layers][64] 2^-f
    unsigned *colmax = reinterpret_cast<unsigned *>(isc + kMcMaxLayers * kMcWidth);  // [layers][64] bits of max |xq| per column
    float *Wall = reinterpret_cast<float *>(colmax + kMcMaxLayers * kMcWidth);       // every layer's [K][Nw], zero beyond N
    const int tid = threadIdx.x, R = P.R;
    MC_DECL;

    // every layer's weights, bias and scales once per block
    for (int l = 0; l < P.n; ++l) {
        const McLayer &Ly = P.L[l];
        const int K = Ly.K, N = Ly.N, Nw = ((N + 3) >> 2) * 4;
        float *W = Wall + Ly.w_off;
        for (int e = tid; e < K * Nw; e += kMcThreads) {
            const int k = e / Nw, n = e - k * Nw;
            mc_cp4(W + e, Ly.wq + k * N + min(n, N - 1), n < N);
        }
        if (tid < kMcWidth) {
            bias[l * kMcWidth + tid] = (Ly.bq != nullptr && tid < N) ? __ldg(Ly.bq + tid) : 0.f;
            const int fi = (tid < K) ? __float2int_rn(__ldg(Ly.qf + tid)) : 0;
            sc[l * kMcWidth + tid] = pow2i(fi);
            isc[l * kMcWidth + tid] = pow2i(-fi);
            colmax[l * kMcWidth + tid] = 0u;
        }
    }
    mc_cp_wait();
    __syncthreads();
    MC_MARK(0);

    for (int64_t tile = blockIdx.x; tile < P.tiles; tile += gridDim.x) {
        const int64_t row0 = tile * R;
        const int rows_here = (int)((P.M - row0) < R ? (P.M - row0) : R);
        float *in = buf0, *out = buf1;
        {   // the tile of x, rounded by the first layer's input quantizer on its way into shared memory
            const McLayer &L0 = P.L[0];
            const int K0 = L0.K;
            const float *x0 = P.x + row0 * K0;
            const bool track = L0.absmax != nullptr, one_column = (kMcThreads % K0 == 0);  // one_column: see mc_foreach
            float mx = 0.f;
            mc_foreach(R, K0, tid, [&](int r, int k) {
                const float v = (r < rows_here) ? __ldcs(x0 + r * K0 + k) : 0.f;
                const float q = mc_round(v, sc[k], isc[k], L0.rm);
                in[r * kMcLd + k] = q;
                if (track && r < rows_here) {
                    if (one_column) mx = fmaxf(mx, fabsf(q));
                    else atomicMax(colmax + k, __float_as_uint(fabsf(q)));
                }
            });
            if (track && one_column) atomicMax(colmax + tid % K0, __float_as_uint(mx));
        }
        __syncthreads();
        MC_MARK(1);
        for (int l = 0; l < P.n; ++l) {
            const McLayer &Ly = P.L[l];
            const int K = Ly.K, N = Ly.N;
            const McMap m = mc_map(R, N, tid);
            const int Nw = m.groups * 4;
            // y = act(xq @ W + b): rows slot + j * slots of column group cg
            if (m.active && m.slot < R) {
                float acc[kMcRowsPerThread][4];
                mc_rows_product_any(R, in, Wall + Ly.w_off, Nw, K, m, acc);
                MC_MARK(4);
                const float lo = Ly.relu ? 0.f : -INFINITY;
                const int n0 = m.cg * 4;
                const float4 b4 = *reinterpret_cast<const float4 *>(bias + l * kMcWidth + n0);
                const bool vec = (N % 4 == 0) && aligned(Ly.y, 16);
                // the next layer's input quantizer is applied here, on the way into shared memory (the value as computed
                // goes to memory for the backward)
                const bool more = l + 1 < P.n;
                const int ln = more ? l + 1 : l;
                const float4 s4 = *reinterpret_cast<const float4 *>(sc + ln * kMcWidth + n0);
                const float4 i4 = *reinterpret_cast<const float4 *>(isc + ln * kMcWidth + n0);
                const int rm_n = P.L[ln].rm;
                float mx[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int j = 0; j < kMcRowsPerThread; ++j) {
                    const int r = m.slot + j * m.slots;
                    if (r < R) {
                        float4 o;
                        o.x = fmaxf(__fadd_rn(acc[j][0], b4.x), lo);
                        o.y = fmaxf(__fadd_rn(acc[j][1], b4.y), lo);
                        o.z = fmaxf(__fadd_rn(acc[j][2], b4.z), lo);
                        o.w = fmaxf(__fadd_rn(acc[j][3], b4.w), lo);
                        if (more) {
                            float4 q;
                            q.x = mc_round(o.x, s4.x, i4.x, rm_n); q.y = mc_round(o.y, s4.y, i4.y, rm_n);
                            q.z = mc_round(o.z, s4.z, i4.z, rm_n); q.w = mc_round(o.w, s4.w, i4.w, rm_n);
                            *reinterpret_cast<float4 *>(out + r * kMcLd + n0) = q;
                            if (r < rows_here) {
                                mx[0] = fmaxf(mx[0], fabsf(q.x)); mx[1] = fmaxf(mx[1], fabsf(q.y));
                                mx[2] = fmaxf(mx[2], fabsf(q.z)); mx[3] = fmaxf(mx[3], fabsf(q.w));
                            }
                        }
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
                if (more && P.L[ln].absmax != nullptr) {
#pragma unroll
                    for (int c = 0; c < 4; ++c)
                        if (n0 + c < N) atomicMax(colmax + ln * kMcWidth + n0 + c, __float_as_uint(mx[c]));
                }
                MC_MARK(5);
            }
            __syncthreads();
            MC_MARK(3);
            float *t = in; in = out; out = t;
        }
    }
    // the block's column maxima into the callers' statistics
    for (int e = tid; e < P.n * kMcWidth; e += kMcThreads) {
        const int l = e / kMcWidth, k = e - l * kMcWidth;
        if (k < P.L[l].K && P.L[l].absmax != nullptr) atomicMax(reinterpret_cast<unsigned *>(P.L[l].absmax) + k, colmax[e]);
    }
}

// ---- backward -------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kMcThreads) k_dense_chain_bwd(const McParams P) {
    extern __shared__ __align__(16) float smem_f[];
    float *G = smem_f;                                      // [128][68] gradient entering the current layer (its output side)
    float *D = G + kMcRows * kMcLd;                         // [128][68] gradient leaving it (dXq)
    float *XQ = D + kMcRows * kMcLd;                        // [128][68] rounded inputs
    float *XR = XQ + kMcRows * kMcLd;                       // [128][68] inputs as stored
    float *red = XR + kMcRows * kMcLd;                      // [512] partial df sums
    float *red_b = red + kMcThreads;                        // [512] partial bias-gradient sums
    float *scratch = red_b + kMcThreads;                    // [512][16] partial weight-gradient sums of the row splits
    float *sc = scratch + kMcThreads * 16;                   // [layers][64], [layers][64]
    float *isc = sc + kMcMaxLayers * kMcWidth;
    float *acc_s = isc + kMcMaxLayers * kMcWidth;           // per layer [dWq | dbq | df] sums over this block's tiles
    float *WTall = acc_s + ((P.part_stride + 3) & ~3);      // every layer's transposed weights [N][Kw], zero beyond K
    const int tid = threadIdx.x, R = P.R;
    MC_DECL;

    for (int e = tid; e < P.part_stride; e += kMcThreads) acc_s[e] = 0.f;
    for (int l = 0; l < P.n; ++l) {
        const McLayer &Ly = P.L[l];
        const int K = Ly.K, N = Ly.N, Kw = ((K + 3) >> 2) * 4;
        float *WT = WTall + Ly.w_off;
        for (int e = tid; e < Kw * N; e += kMcThreads) {  // coalesced over n in memory, transposed into shared memory
            const int k = e / N, n = e - k * N;
            mc_cp4(WT + n * Kw + k, Ly.wq + min(k, K - 1) * N + n, k < K);
        }
        if (tid < kMcWidth) {
            const int fi = (tid < K) ? __float2int_rn(__ldg(Ly.qf + tid)) : 0;
            sc[l * kMcWidth + tid] = pow2i(fi);
            isc[l * kMcWidth + tid] = pow2i(-fi);
        }
    }
    mc_cp_wait();
    __syncthreads();
    MC_MARK(0);

    for (int64_t tile = blockIdx.x; tile < P.tiles; tile += gridDim.x) {
        const int64_t row0 = tile * R;
        const int rows_here = (int)((P.M - row0) < R ? (P.M - row0) : R);
        mc_load_tile(R, G, P.gy, row0, rows_here, P.L[P.n - 1].N, tid);
        if (P.L[P.n - 1].relu) {  // the mask of the last layer comes from its stored output; the others' from shared memory
            __syncthreads();
            mc_relu_mask(R, G, P.L[P.n - 1].y, row0, rows_here, P.L[P.n - 1].N, tid);
        }
        float *g_in = G, *g_out = D;
        __syncthreads();  // the tile's gradient is in place
        for (int l = P.n - 1; l >= 0; --l) {
            const McLayer &Ly = P.L[l];
            const int K = Ly.K, N = Ly.N;
            const McMap mk = mc_map(R, K, tid);    // dXq tile: column groups over k
            const int n_groups = (N + 3) >> 2;
            const int Kw = mk.groups * 4, Nw = n_groups * 4;
            const float *WT = WTall + Ly.w_off;
            const float *sc_l = sc + l * kMcWidth, *isc_l = isc + l * kMcWidth;
            float *a_l = acc_s + Ly.part_off;
            // (no barrier here: the sums that end a layer touch only the block's records and the scratch areas, which the
            // next layer writes after its own load barrier)
            MC_MARK(1);
            // this layer's inputs as stored and rounded
            {
                const float *xl = ((l == 0) ? P.x : P.L[l - 1].y) + row0 * K;
                if ((K & 3) == 0 && aligned(xl, 16)) {  // 16 bytes per load: the whole tile is in flight at once
                    const int w4 = K >> 2;
                    mc_foreach(R, w4, tid, [&](int r, int c) {
                        const float4 v = (r < rows_here) ? __ldcs(reinterpret_cast<const float4 *>(xl + r * K) + c) : make_float4(0.f, 0.f, 0.f, 0.f);
                        const float4 s4 = *reinterpret_cast<const float4 *>(sc_l + c * 4), i4 = *reinterpret_cast<const float4 *>(isc_l + c * 4);
                        *reinterpret_cast<float4 *>(XR + r * kMcLd + c * 4) = v;
                        *reinterpret_cast<float4 *>(XQ + r * kMcLd + c * 4) =
                            make_float4(mc_round(v.x, s4.x, i4.x, Ly.rm), mc_round(v.y, s4.y, i4.y, Ly.rm), mc_round(v.z, s4.z, i4.z, Ly.rm),
                                        mc_round(v.w, s4.w, i4.w, Ly.rm));
                    });
                } else {
                    mc_foreach(R, K, tid, [&](int r, int k) {
                        const float v = (r < rows_here) ? __ldcs(xl + r * K + k) : 0.f;
                        XR[r * kMcLd + k] = v;
                        XQ[r * kMcLd + k] = mc_round(v, sc_l[k], isc_l[k], Ly.rm);
                    });
                    if (Kw != K)  // the padding columns the 16-byte reads of the dWq product touch
                        for (int e = tid; e < R * (Kw - K); e += kMcThreads) {
                            const int r = e / (Kw - K), k = K + (e - r * (Kw - K));
                            XQ[r * kMcLd + k] = 0.f;
                        }
                }
            }
            if (Nw != N)  // the padding columns the float4 reads of the dWq product touch
                for (int e = tid; e < R * (Nw - N); e += kMcThreads) {
                    const int r = e / (Nw - N), n = N + (e - r * (Nw - N));
                    g_in[r * kMcLd + n] = 0.f;
                }
            __syncthreads();
            MC_MARK(2);
            MC_MARK(3);
            // ---- dXq = G @ W^T ------------------------------------------------------------------------------------------------
            if (mk.active && mk.slot < R) {
                float acc[kMcRowsPerThread][4];
                mc_rows_product_any(R, g_in, WT, Kw, N, mk, acc);
                const int k0 = mk.cg * 4;
#pragma unroll
                for (int j = 0; j < kMcRowsPerThread; ++j) {
                    const int r = mk.slot + j * mk.slots;
                    if (r < R) {
                        *reinterpret_cast<float4 *>(g_out + r * kMcLd + k0) = make_float4(acc[j][0], acc[j][1], acc[j][2], acc[j][3]);
                        if (l == 0 && P.dx != nullptr && r < rows_here) {
#pragma unroll
                            for (int c = 0; c < 4; ++c)
                                if (k0 + c < K) P.dx[(row0 + r) * K + k0 + c] = acc[j][c];
                        }
                    }
                }
            }
            MC_MARK(4);
            // ---- dWq += xq^T @ G ---------------------------------------------------------------------------------------------------
            // A unit is (four inputs, four outputs): its sixteen sums run over the rows, two 16-byte loads per sixteen FMAs.
            // There are far fewer units than threads, so the rows of a unit are split among `splits` threads (partial sums to
            // shared memory, combined below in a fixed order).
            const int units = mk.groups * n_groups;
            const int splits = max(1, min(kMcThreads / units, R >> 3));  // at least eight rows per split
            const int rps = (R + splits - 1) / splits;  // rows per split
            if (tid < units * splits) {
                const int unit = tid % units, sp = tid / units;
                const int kg = unit / n_groups, cg = unit - kg * n_groups;
                const int r0 = sp * rps, r1 = min(R, r0 + rps);
                float a[4][4];
#pragma unroll
                for (int i = 0; i < 4; ++i)
#pragma unroll
                    for (int c = 0; c < 4; ++c) a[i][c] = 0.f;
                const float *xp = XQ + kg * 4, *gq = g_in + cg * 4;
#pragma unroll 4
                for (int r = r0; r < r1; ++r) {
                    const float4 g4 = *reinterpret_cast<const float4 *>(gq + r * kMcLd);
                    const float4 x4 = *reinterpret_cast<const float4 *>(xp + r * kMcLd);
                    const float xv[4] = {x4.x, x4.y, x4.z, x4.w};
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        a[i][0] = __fmaf_rn(xv[i], g4.x, a[i][0]); a[i][1] = __fmaf_rn(xv[i], g4.y, a[i][1]);
                        a[i][2] = __fmaf_rn(xv[i], g4.z, a[i][2]); a[i][3] = __fmaf_rn(xv[i], g4.w, a[i][3]);
                    }
                }
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    *reinterpret_cast<float4 *>(scratch + (tid * 4 + i) * 4) = make_float4(a[i][0], a[i][1], a[i][2], a[i][3]);
            }
            __syncthreads();  // dXq complete
            MC_MARK(5);
            // ---- df[k] += sum_r -ln2 (xq - x) dXq: thread t takes column t % K and the rows t / K, t / K + subsets, ... --------
            const int subsets = kMcThreads / K;
            if (tid < subsets * K) {
                const int k = tid % K;
                float s = 0.f;
                const bool mask_below = l > 0 && P.L[l - 1].relu;
#pragma unroll 4
                for (int r = tid / K; r < R; r += subsets) {
                    const float xv = XR[r * kMcLd + k], d = g_out[r * kMcLd + k];
                    const float er = __fmul_rn(__fsub_rn(XQ[r * kMcLd + k], xv), -kLn2);
                    s = __fmaf_rn(er, d, s);
                    // the layer below wrote xv as its output: its ReLU passes the gradient where that was positive
                    if (mask_below && !(xv > 0.f)) g_out[r * kMcLd + k] = 0.f;
                }
                red[tid] = s;
            }
            // ---- dbq += column sums of G: thread t takes column t % N and the rows t / N, t / N + subsets_b, ... --------------------
            const int subsets_b = kMcThreads / N;
            if (tid < subsets_b * N) {
                const int n = tid % N;
                float s = 0.f;
#pragma unroll 4
                for (int r = tid / N; r < R; r += subsets_b) s = __fadd_rn(s, g_in[r * kMcLd + n]);
                red_b[tid] = s;
            }
            __syncthreads();
            MC_MARK(6);
            if (tid < K) {
                float s = 0.f;
                for (int sub = 0; sub < subsets; ++sub) s = __fadd_rn(s, red[sub * K + tid]);
                a_l[K * N + N + tid] = __fadd_rn(a_l[K * N + N + tid], s);
            }
            if (tid < N) {
                float s = 0.f;
                for (int sub = 0; sub < subsets_b; ++sub) s = __fadd_rn(s, red_b[sub * N + tid]);
                a_l[K * N + tid] = __fadd_rn(a_l[K * N + tid], s);
            }
            for (int e = tid; e < K * N; e += kMcThreads) {  // the row splits of every weight, in order
                const int k = e / N, n = e - k * N;
                const int unit = (k >> 2) * n_groups + (n >> 2), off = (k & 3) * 4 + (n & 3);
                float t = 0.f;
                for (int sp = 0; sp < splits; ++sp) t = __fadd_rn(t, scratch[(sp * units + unit) * 16 + off]);
                a_l[e] = __fadd_rn(a_l[e], t);
            }
            float *t = g_in; g_in = g_out; g_out = t;
        }
        __syncthreads();
    }
    __syncthreads();
    MC_MARK(7);
    float *pb = P.part + (int64_t)blockIdx.x * P.part_stride;
    for (int e = tid; e < P.part_stride; e += kMcThreads) pb[e] = acc_s[e];
    MC_MARK(8);
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

static size_t mc_fwd_smem(int w_total) {
    return (size_t)(2 * kMcRows * kMcLd + 4 * kMcMaxLayers * kMcWidth + w_total) * sizeof(float);
}
static size_t mc_bwd_smem(int part_stride, int w_total) {
    return (size_t)(4 * kMcRows * kMcLd + 18 * kMcThreads + 2 * kMcMaxLayers * kMcWidth + ((part_stride + 3) & ~3) + w_total) * sizeof(float);
}

// widths, record offsets and the shared-memory weight area of a stack; HGQ_OK when both kernels fit
static int mc_plan(int n_layers, const hgq_chain_layer *layers, bool backward, McParams &p) {
    if (layers == nullptr) return HGQ_ERR_NULL;
    if (n_layers < 1 || n_layers > kMcMaxLayers) return HGQ_ERR_SIZE;
    int off = 0, wf = 0, wb = 0;
    for (int l = 0; l < n_layers; ++l) {
        const hgq_chain_layer &s = layers[l];
        if (s.K < 1 || s.K > kMcWidth || s.N < 1 || s.N > kMcWidth) return HGQ_ERR_SIZE;
        if (l > 0 && s.K != layers[l - 1].N) return HGQ_ERR_SIZE;
        McLayer &d = p.L[l];
        d.K = s.K; d.N = s.N; d.part_off = off;
        d.w_off = backward ? wb : wf;
        off += s.K * s.N + s.N + s.K;
        wf += s.K * ((s.N + 3) / 4 * 4);
        wb += s.N * ((s.K + 3) / 4 * 4);
    }
    p.n = n_layers;
    p.part_stride = off;
    p.w_total = backward ? wb : wf;
    if (mc_fwd_smem(wf) > 226 * 1024 || mc_bwd_smem(off, wb) > 226 * 1024) return HGQ_ERR_SIZE;
    return HGQ_OK;
}

static int mc_fill(int n_layers, const hgq_chain_layer *layers, bool backward, McParams &p) {
    if (int e = mc_plan(n_layers, layers, backward, p)) return e;
    for (int l = 0; l < n_layers; ++l) {
        const hgq_chain_layer &s = layers[l];
        if (s.round_mode < 0 || s.round_mode > 2) return HGQ_ERR_MODE;
        if (s.qf == nullptr || s.wq == nullptr || s.y == nullptr) return HGQ_ERR_NULL;
        if (backward && s.dwq == nullptr) return HGQ_ERR_NULL;
        McLayer &d = p.L[l];
        d.qf = s.qf; d.wq = s.wq; d.bq = s.bq; d.y = s.y; d.absmax = s.absmax; d.dwq = s.dwq; d.dbq = s.dbq; d.df = s.df;
        d.relu = s.relu ? 1 : 0; d.rm = s.round_mode;
    }
    return HGQ_OK;
}

static int mc_grid(int64_t tiles) { return (int)(tiles < num_sms() ? tiles : num_sms()); }

// rows per tile: as few as give every SM a tile (a multiple of 8), at most 128
static void mc_tiles(int64_t M, McParams &p) {
    int64_t r = (M + num_sms() - 1) / num_sms();
    r = (r + 7) / 8 * 8;
    p.R = (int)(r < 8 ? 8 : (r > kMcRows ? kMcRows : r));
    p.tiles = (M + p.R - 1) / p.R;
}

}  // namespace hgq

using namespace hgq;

extern "C" int hgq_dense_chain_supported(int n_layers, const hgq_chain_layer *layers) {
    McParams p;
    return mc_plan(n_layers, layers, true, p) == HGQ_OK ? 1 : 0;
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
    p.x = x; p.gy = nullptr; p.dx = nullptr; p.part = nullptr; p.M = M;
    mc_tiles(M, p);
    const size_t smem = mc_fwd_smem(p.w_total);
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
    p.x = x; p.gy = gy; p.dx = dx; p.M = M;
    mc_tiles(M, p);
    const int grid = mc_grid(p.tiles);
    if (workspace == nullptr || workspace_bytes < (size_t)grid * p.part_stride * sizeof(float)) return HGQ_ERR_WORKSPACE;
    if (!aligned(workspace, 16)) return HGQ_ERR_ALIGN;
    p.part = (float *)workspace;
    const size_t smem = mc_bwd_smem(p.part_stride, p.w_total);
    cudaError_t ce = cudaFuncSetAttribute(k_dense_chain_bwd, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (ce != cudaSuccess) return (int)ce;
    cudaStream_t st = (cudaStream_t)stream;
    k_dense_chain_bwd<<<grid, kMcThreads, smem, st>>>(p);
    if (int e = check_launch()) return e;
    k_dense_chain_stage2<<<(p.part_stride + 7) / 8, kThreads, 0, st>>>(p, grid);
    return check_launch();
}
