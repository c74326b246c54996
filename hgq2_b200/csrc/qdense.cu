// K2 (dense / einsum-dense forward): input quantizer -> bf16 tensor-core GEMM -> bias -> activation,
// one pass over the activations.
//
// Stands in for QDense.call (src/hgq/layers/core/dense.py:60-68) and QEinsumDense.call
// (src/hgq/layers/core/einsum_dense.py:72-83) when the contraction runs over the trailing input axis:
//     y = act( iq(x) @ Wq + bq )
// x is [M, K] raw fp32 activations, the input quantizer's parameters are a [rows_period, K] table (row r of
// x uses table row r % rows_period: the bitwidth tensor has the batch axis set to 1), Wq [K, N] and bq [N]
// are the already quantised kernel and bias.  The per-entry max |round(x)| that the WRAP integer-bit
// tracking needs (fixed_point_quantizer.py:405-413) is a side output, so the activations are read once and
// the quantised activations never touch HBM.
//
// Shapes are skinny (K, N <= 256) so the kernel is HBM-bound: 4 (K + N) bytes per row.  A persistent CTA
// keeps the whole quantised weight matrix in shared memory as bf16 and streams 128-row tiles:
//   all threads   load a 128 x 64 fp32 slab with 128-bit loads, quantise it in registers, split every value
//                 exactly into up to three bf16 terms (3 x 8 significant bits = the 24 of fp32) and store
//                 them in the no-swizzle core-matrix layout the tensor core reads;
//   one thread    issues tcgen05.mma (M = 128, N = padded N, K = 16 per instruction, fp32 accumulate in
//                 TMEM) for every pair of non-zero terms, then tcgen05.commit to an mbarrier;
//   all threads   wait (bounded), read the accumulator back with tcgen05.ld, add the bias, apply the
//                 activation and store y.
// A tile whose values all fit 8 significant bits costs one MMA per K step; the extra terms appear only when
// the data need them, and the result is then still exact whenever the reference's fp32 sum is.
// Several CTAs are resident per SM, so one CTA's loads overlap another's MMA and epilogue.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "hgq_common.cuh"
#include "hgq_math.cuh"
#include "tc05.cuh"

namespace hgq {

constexpr int kQdThreads = 256;
constexpr int kQdTileM = 128;
constexpr int kQdKC = 64;                      // K slab held in shared memory at a time
constexpr int kQdATermBytes = kQdTileM * kQdKC * 2;  // 16 KB per bf16 term
constexpr int kQdMaxTable = 8192;              // abs-max table entries (rows_period * K)

enum : int { ACT_NONE = 0, ACT_RELU = 1 };
enum : unsigned { ST_TIMEOUT = 1u };

struct QdParams {
    const float *x;
    const uint8_t *qk;   // input quantizer k / i / f tables [rows_period, K]; qf == nullptr: no input quantizer
    const float *qi;
    const float *qf;
    const float *wq;     // [K, N]
    const float *bq;     // [N] or nullptr
    float *y;            // [M, N]
    unsigned *amax_part; // [gridDim.x, rows_period * K] abs-max partials, or nullptr
    unsigned *status;
    int64_t M;
    int K, N, Kpad, Npad;
    int rows_period;
    int rm, om, act, zero;
    int64_t num_tiles;
};

__device__ __forceinline__ float quantize_rt(float v, float kf, float i, float f, int rm, int om, bool zero, float &rounded) {
    Params p = make_params(kf, i, f);
    if (zero && ((kf != 0.f ? 1 : 0) + p.ii + p.fi <= 0)) {
        rounded = 0.f;
        return 0.f;
    }
    float xq;
    switch (rm) {
        case RM_TRN: xq = round_to_f<RM_TRN>(v, p); break;
        case RM_RND: xq = round_to_f<RM_RND>(v, p); break;
        default: xq = round_to_f<RM_RND_CONV>(v, p); break;
    }
    rounded = xq;
    switch (om) {
        case OM_WRAP: return overflow<OM_WRAP, false>(xq, p);
        case OM_SAT: return overflow<OM_SAT, false>(xq, p);
        case OM_SAT_SYM: return overflow<OM_SAT_SYM, false>(xq, p);
        default: return xq;
    }
}

__global__ void __launch_bounds__(kQdThreads) k_qdense_fwd(const QdParams P) {
    extern __shared__ __align__(128) unsigned char smem[];
    // carve: A terms | B terms | abs-max table | barrier + tmem slot
    unsigned char *A = smem;                                        // 3 x 16 KB
    unsigned char *B = A + 3 * kQdATermBytes;                       // 3 x Kpad*Npad*2
    const int b_term_bytes = P.Kpad * P.Npad * 2;
    unsigned *amax_s = reinterpret_cast<unsigned *>(B + 3 * b_term_bytes);
    const int table = (P.amax_part != nullptr) ? P.rows_period * P.K : 0;
    uint64_t *bar = reinterpret_cast<uint64_t *>(reinterpret_cast<unsigned char *>(amax_s) + ((table * 4 + 15) / 16) * 16);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bar + 1);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int K = P.K, N = P.N, Kpad = P.Kpad, Npad = P.Npad;
    const uint32_t tmem_cols = Npad < 32 ? 32u : (uint32_t)Npad;  // Npad is a power of two >= 16

    // ---- one-time set-up ------------------------------------------------------------------------
    if (tid == 0) {
        tc::mbar_init(bar, 1);
        tc::mbar_init_fence();
    }
    if (warp == 0) tc::tmem_alloc(tmem_slot, tmem_cols);
    for (int e = tid; e < table; e += kQdThreads) amax_s[e] = 0u;
    // weights: fp32 [K, N] -> up to three bf16 terms, K-major core matrices: (n/8, k/8) -> 128-byte block
    int w_lo = 0, w_lo2 = 0;
    for (int e = tid; e < Kpad * Npad; e += kQdThreads) {
        const int n = e % Npad, k = e / Npad;
        const float w = (k < K && n < N) ? __ldg(P.wq + (int64_t)k * N + n) : 0.f;
        __nv_bfloat16 h, l, l2;
        tc::split3(w, h, l, l2);
        const int off = ((n >> 3) * (Kpad >> 3) + (k >> 3)) * 128 + (n & 7) * 16 + (k & 7) * 2;
        *reinterpret_cast<__nv_bfloat16 *>(B + off) = h;
        *reinterpret_cast<__nv_bfloat16 *>(B + b_term_bytes + off) = l;
        *reinterpret_cast<__nv_bfloat16 *>(B + 2 * b_term_bytes + off) = l2;
        w_lo |= (__bfloat16_as_ushort(l) & 0x7fff) != 0;
        w_lo2 |= (__bfloat16_as_ushort(l2) & 0x7fff) != 0;
    }
    const int any_w_lo = __syncthreads_or(w_lo);
    const int any_w_lo2 = __syncthreads_or(w_lo2);
    const int n_w = any_w_lo2 ? 3 : (any_w_lo ? 2 : 1);
    tc::fence_smem_to_async();
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t idesc = tc::make_idesc_bf16(Npad, false, false);
    const uint32_t a_base = tc::smem_u32(A), b_base = tc::smem_u32(B);
    const uint32_t sbo_a = (kQdKC / 8) * 128, sbo_b = (uint32_t)(Kpad >> 3) * 128;
    uint32_t phase = 0;
    bool ok = true;

    const int r8 = lane & 7, q4 = lane >> 3;
    const int n_chunks = (Kpad + kQdKC - 1) / kQdKC;
    const bool vec_ok = (K % 4 == 0) && aligned(P.x, 16) && (P.qf == nullptr || aligned(P.qf, 16));

    for (int64_t tile = blockIdx.x; tile < P.num_tiles && ok; tile += gridDim.x) {
        const int64_t row0 = tile * kQdTileM;
        for (int ch = 0; ch < n_chunks && ok; ++ch) {
            // ---- load + quantise + split one 128 x 64 slab ----------------------------------------
            int a_lo = 0, a_lo2 = 0;
            float xv[4][8];
            bool valid[4];
#pragma unroll
            for (int it = 0; it < 4; ++it) {
                const int c = it * 8 + warp, mg = c >> 1, kg = (c & 1) * 4 + q4;
                const int64_t row = row0 + mg * 8 + r8;
                const int k0 = ch * kQdKC + kg * 8;
                valid[it] = row < P.M && k0 < K;
                if (valid[it] && vec_ok && k0 + 8 <= K) {
                    const float4 v0 = __ldcs(reinterpret_cast<const float4 *>(P.x + row * K + k0));
                    const float4 v1 = __ldcs(reinterpret_cast<const float4 *>(P.x + row * K + k0 + 4));
                    xv[it][0] = v0.x; xv[it][1] = v0.y; xv[it][2] = v0.z; xv[it][3] = v0.w;
                    xv[it][4] = v1.x; xv[it][5] = v1.y; xv[it][6] = v1.z; xv[it][7] = v1.w;
                } else {
#pragma unroll
                    for (int j = 0; j < 8; ++j) xv[it][j] = (valid[it] && k0 + j < K) ? __ldcs(P.x + row * K + k0 + j) : 0.f;
                }
            }
#pragma unroll
            for (int it = 0; it < 4; ++it) {
                const int c = it * 8 + warp, mg = c >> 1, kg = (c & 1) * 4 + q4;
                const int64_t row = row0 + mg * 8 + r8;
                const int k0 = ch * kQdKC + kg * 8;
                uint32_t hi[4], lo[4], lo2[4];
                const int pr = (int)(row % P.rows_period);
#pragma unroll
                for (int j = 0; j < 8; j += 2) {
                    float v[2];
#pragma unroll
                    for (int u = 0; u < 2; ++u) {
                        float val = xv[it][j + u];
                        const int k = k0 + j + u;
                        if (P.qf != nullptr && valid[it] && k < K) {
                            const int pe = pr * K + k;
                            const float f = __ldg(P.qf + pe);
                            const float kf = (P.om == OM_NONE) ? 0.f : (float)__ldg(P.qk + pe);
                            const float ii = (P.om == OM_NONE) ? 0.f : __ldg(P.qi + pe);
                            float rounded;
                            val = quantize_rt(val, kf, ii, f, P.rm, P.om, P.zero != 0, rounded);
                            if (table) atomicMax(amax_s + pe, __float_as_uint(fabsf(rounded)));
                        }
                        v[u] = val;
                    }
                    __nv_bfloat16 h0, l0, m0, h1, l1, m1;
                    tc::split3(v[0], h0, l0, m0);
                    tc::split3(v[1], h1, l1, m1);
                    hi[j >> 1] = tc::pack2(h0, h1);
                    lo[j >> 1] = tc::pack2(l0, l1);
                    lo2[j >> 1] = tc::pack2(m0, m1);
                    a_lo |= (lo[j >> 1] & 0x7fff7fffu) != 0;
                    a_lo2 |= (lo2[j >> 1] & 0x7fff7fffu) != 0;
                }
                const int off = (mg * 8 + kg) * 128 + r8 * 16;
                *reinterpret_cast<uint4 *>(A + off) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
                *reinterpret_cast<uint4 *>(A + kQdATermBytes + off) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
                *reinterpret_cast<uint4 *>(A + 2 * kQdATermBytes + off) = make_uint4(lo2[0], lo2[1], lo2[2], lo2[3]);
            }
            const int any_lo = __syncthreads_or(a_lo);
            const int any_lo2 = __syncthreads_or(a_lo2);
            tc::fence_smem_to_async();
            __syncthreads();
            // ---- tensor-core GEMM on the slab -------------------------------------------------------
            if (tid == 0) {
                tc::fence_after_sync();
                const int n_a = any_lo2 ? 3 : (any_lo ? 2 : 1);
                const int kleft = Kpad - ch * kQdKC;
                const int ksteps = (kleft < kQdKC ? kleft : kQdKC) / 16;
                for (int s = 0; s < ksteps; ++s) {
                    for (int ta = 0; ta < n_a; ++ta) {
                        const uint64_t da = tc::make_smem_desc(a_base + ta * kQdATermBytes + s * 256, 128, sbo_a);
                        for (int tw = 0; tw < n_w; ++tw) {
                            const uint64_t db = tc::make_smem_desc(b_base + tw * b_term_bytes + (ch * (kQdKC / 16) + s) * 256, 128, sbo_b);
                            tc::mma_bf16(tmem_base, da, db, idesc, !(ch == 0 && s == 0 && ta == 0 && tw == 0));
                        }
                    }
                }
                tc::commit(bar);
            }
            // every thread waits: the slab buffers are rewritten next and the epilogue reads TMEM
            const bool waited = tc::mbar_wait(bar, phase);
            phase ^= 1u;
            ok = __syncthreads_and(waited ? 1 : 0) != 0;  // one verdict for the whole CTA: nobody is left behind at a barrier
            if (!ok && tid == 0 && P.status) atomicOr(P.status, ST_TIMEOUT);
        }
        if (!ok) break;
        // ---- epilogue: TMEM -> registers -> bias, activation -> global ------------------------------
        tc::fence_after_sync();
        {
            const int qlane = (warp & 3) * 32, half = warp >> 2;
            const int64_t row = row0 + qlane + lane;
            const int cbeg = half * (Npad / 2), cend = cbeg + Npad / 2;
            for (int c0 = cbeg; c0 < cend; c0 += 8) {
                float v[8];
                tc::tmem_ld8(tmem_base + ((uint32_t)qlane << 16) + (uint32_t)c0, v);
                if (row < P.M && c0 < N) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        float o = v[j];
                        if (P.bq != nullptr && c0 + j < N) o = __fadd_rn(o, __ldg(P.bq + c0 + j));
                        if (P.act == ACT_RELU) o = o > 0.f ? o : 0.f;
                        v[j] = o;
                    }
                    float *dst = P.y + row * N + c0;
                    if ((N % 4 == 0) && c0 + 8 <= N) {
                        __stcs(reinterpret_cast<float4 *>(dst), make_float4(v[0], v[1], v[2], v[3]));
                        __stcs(reinterpret_cast<float4 *>(dst) + 1, make_float4(v[4], v[5], v[6], v[7]));
                    } else {
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            if (c0 + j < N) __stcs(dst + j, v[j]);
                    }
                }
            }
        }
        tc::fence_before_sync();
        __syncthreads();  // all TMEM reads done before the next tile's first MMA overwrites the accumulator
    }

    // ---- tear-down ----------------------------------------------------------------------------------
    __syncthreads();
    if (table) {
        unsigned *dst = P.amax_part + (int64_t)blockIdx.x * table;
        for (int e = tid; e < table; e += kQdThreads) dst[e] = amax_s[e];
    }
    tc::fence_before_sync();
    __syncthreads();
    if (warp == 0) tc::tmem_dealloc(tmem_base, tmem_cols);
}

// max over the per-CTA partial tables (non-negative floats order like their bit patterns)
__global__ void __launch_bounds__(kThreads) k_amax_stage2(const unsigned *__restrict__ part, float *__restrict__ out,
                                                         int table, int nparts) {
    const int e = blockIdx.x * kThreads + threadIdx.x;
    if (e >= table) return;
    unsigned m = 0u;
    for (int p = 0; p < nparts; ++p) m = max(m, part[(int64_t)p * table + e]);
    out[e] = __uint_as_float(m);
}

struct QdGeom {
    int Kpad, Npad, grid;
    size_t smem;
    int64_t tiles;
};

static int qd_geom(int64_t M, int K, int N, int rows_period, bool want_amax, QdGeom &g) {
    if (M <= 0 || K <= 0 || N <= 0 || rows_period <= 0) return HGQ_ERR_SIZE;
    if (K > 256 || N > 128) return HGQ_ERR_SIZE;
    if (want_amax && (int64_t)rows_period * K > kQdMaxTable) return HGQ_ERR_SIZE;
    g.Kpad = (K + 15) / 16 * 16;
    g.Npad = pow2ceil(N < 16 ? 16 : N);
    const size_t table = want_amax ? (size_t)rows_period * K : 0;
    g.smem = 3 * (size_t)kQdATermBytes + 3 * (size_t)g.Kpad * g.Npad * 2 + (table * 4 + 15) / 16 * 16 + 64;
    if (g.smem > 200 * 1024) return HGQ_ERR_SIZE;
    g.tiles = (M + kQdTileM - 1) / kQdTileM;
    int per_sm = (int)((220 * 1024) / (g.smem + 1024));
    if (per_sm > 4) per_sm = 4;
    if (per_sm < 1) per_sm = 1;
    // TMEM: 512 columns per SM
    const int cols = g.Npad < 32 ? 32 : g.Npad;
    if (per_sm * cols > 512) per_sm = 512 / cols;
    int64_t grid = (int64_t)kNumSMs * per_sm;
    if (grid > g.tiles) grid = g.tiles;
    g.grid = (int)grid;
    return HGQ_OK;
}

}  // namespace hgq

using namespace hgq;

extern "C" size_t hgq_qdense_fwd_workspace(int64_t M, int K, int N, int rows_period) {
    QdGeom g;
    if (qd_geom(M, K, N, rows_period, true, g) != HGQ_OK) return 0;
    return (size_t)g.grid * rows_period * K * sizeof(unsigned);
}

extern "C" int hgq_qdense_fwd(const float *x, const uint8_t *qk, const float *qi, const float *qf, int rows_period,
                              int round_mode, int overflow_mode, unsigned flags, const float *wq, const float *bq,
                              int activation, float *y, float *absmax, int64_t M, int K, int N, void *workspace,
                              size_t workspace_bytes, unsigned *status, void *stream) {
    if (x == nullptr || wq == nullptr || y == nullptr) return HGQ_ERR_NULL;
    if (round_mode < 0 || round_mode > 2 || overflow_mode < 0 || overflow_mode > 3) return HGQ_ERR_MODE;
    if (activation != ACT_NONE && activation != ACT_RELU) return HGQ_ERR_MODE;
    if (flags & ~(HGQ_FLAG_TRAINING | HGQ_FLAG_ZERO_NONPOS)) return HGQ_ERR_MODE;
    int om = overflow_mode;
    if (om == OM_WRAP && (flags & HGQ_FLAG_TRAINING)) om = OM_NONE;
    const int zero = (flags & HGQ_FLAG_ZERO_NONPOS) ? 1 : 0;
    if (zero && om == OM_NONE) return HGQ_ERR_MODE;
    if (qf != nullptr && om != OM_NONE && (qk == nullptr || qi == nullptr)) return HGQ_ERR_NULL;
    if (absmax != nullptr && qf == nullptr) return HGQ_ERR_NULL;
    QdGeom g;
    if (int e = qd_geom(M, K, N, rows_period, absmax != nullptr, g)) return e;
    const size_t need = absmax ? (size_t)g.grid * rows_period * K * sizeof(unsigned) : 0;
    if (absmax && (workspace == nullptr || workspace_bytes < need)) return HGQ_ERR_WORKSPACE;
    cudaError_t ce = cudaFuncSetAttribute(k_qdense_fwd, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)g.smem);
    if (ce != cudaSuccess) return (int)ce;
    QdParams p;
    p.x = x; p.qk = qk; p.qi = qi; p.qf = qf; p.wq = wq; p.bq = bq; p.y = y;
    p.amax_part = absmax ? (unsigned *)workspace : nullptr;
    p.status = status;
    p.M = M; p.K = K; p.N = N; p.Kpad = g.Kpad; p.Npad = g.Npad;
    p.rows_period = rows_period; p.rm = round_mode; p.om = om; p.act = activation; p.zero = zero;
    p.num_tiles = g.tiles;
    cudaStream_t st = (cudaStream_t)stream;
    k_qdense_fwd<<<g.grid, kQdThreads, g.smem, st>>>(p);
    if (int e = check_launch()) return e;
    if (absmax) {
        const int table = rows_period * K;
        k_amax_stage2<<<(table + kThreads - 1) / kThreads, kThreads, 0, st>>>((const unsigned *)workspace, absmax, table, g.grid);
        return check_launch();
    }
    return HGQ_OK;
}
