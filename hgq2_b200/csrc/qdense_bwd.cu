// K2b (dense / einsum-dense backward): one pass over dY, y and x produces dX, dWq, dbq and the input quantizer's
// fractional-bit gradient.
//
// Stands in for the autograd backward of QDense.call / QEinsumDense.call (src/hgq/layers/core/dense.py:60-68,
// einsum_dense.py:72-83) with a rounding-only input quantizer (the training-mode WRAP activation quantizer,
// src/hgq/quantizer/internal/fixed_point_quantizer.py:403-424):
//     G   = dY * (y > 0)                      (ReLU mask; G = dY without activation)
//     dXq = G @ Wq^T          dX = dXq        (straight-through rounding)
//     df[p, k]  = sum over rows r = p (mod rows_period) of (-ln2 (xq - x)) * dXq
//     dWq = xq^T @ G          dbq = sum_r G
// Per 128-row tile the CTA converts G and the recomputed xq to bf16 terms in shared memory (two terms each: 16
// significant bits, far inside the 1e-4 gradient tolerance; the weights are split exactly), then one thread issues
//   MMA1  dXq [128 x K]   = G (K-major over n)      x  Wq rows (K-major over n)       accumulator 1 in TMEM
//   MMA2  dWq [K+1 x N]  += xq^T (MN-major, + a row of ones that yields dbq)  x  G (MN-major)   accumulator 2 in TMEM,
// the second accumulating over all tiles of the CTA.  The same G buffer serves as the A operand of MMA1 and as the B
// operand of MMA2: a core matrix "8 rows x 8 columns, 16 bytes per row" is both a K-major and an MN-major core.
// The epilogue reads dXq back, forms the df terms against x (re-read, L2-resident) and writes dX through a swizzled
// staging block as full lines.  Per-CTA partials of dWq / dbq / df go to scratch and are reduced in a fixed order by a
// second kernel, so results do not depend on scheduling.
// HBM-bound: 4 (2N + 2K) bytes per row (dY, y, x in; dX out).
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdlib>

#include "hgq_common.cuh"
#include "hgq_math.cuh"
#include "tc05.cuh"

namespace hgq {

constexpr int kQbThreads = 512;
constexpr int kQbTileM = 128;
constexpr int kQbXTermBytes = 128 * 128 * 2;  // xq^T operand: 128 rows x 128 (padded) columns of bf16

struct QbParams {
    const float *gy, *y, *x, *qf, *wq;
    float *dx;
    float *part;        // per-CTA partials: [(K+1) x N] dWq|dbq, then [rows_period x K] df
    unsigned *status;
    int64_t M, num_tiles, ldx, lddx;  // row strides (floats) of x and dx: >= K, so a column slice of a wider matrix works
    int K, N, Kp, Np, Kt;
    int rows_period, rm, relu, want_df;
    int gy_repeat;     // each row of gy serves gy_repeat consecutive rows (the gradient of a sum over an axis); 1 = one each
    FastDiv gy_div;
};

// two-term bf16 split of a pair: hi = RN(v), lo = RN(v - hi)
__device__ __forceinline__ void split2_pair(float v0, float v1, uint32_t &hi, uint32_t &lo) {
    const __nv_bfloat162 h2 = __floats2bfloat162_rn(v0, v1);
    hi = *reinterpret_cast<const uint32_t *>(&h2);
    const float r0 = __fsub_rn(v0, __uint_as_float(hi << 16));
    const float r1 = __fsub_rn(v1, __uint_as_float(hi & 0xffff0000u));
    const __nv_bfloat162 l2 = __floats2bfloat162_rn(r0, r1);
    lo = *reinterpret_cast<const uint32_t *>(&l2);
}

template <bool CONV>
__device__ __forceinline__ float round_e(float v, uint32_t ebyte, float rbias) {
    const uint32_t sbits = ebyte << 23;  // 2^f
    // scaling by a power of two is exact, so one fused multiply-add gives RN(v * 2^f + bias) bit for bit
    const float q = CONV ? rintf(__fmul_rn(v, __uint_as_float(sbits))) : floorf(__fmaf_rn(v, __uint_as_float(sbits), rbias));
    return __fmul_rn(q, __uint_as_float(0x7F000000u - sbits));
}

template <bool CONV>
__global__ void __launch_bounds__(kQbThreads) k_qdense_bwd(const QbParams P) {
    extern __shared__ __align__(128) unsigned char smem[];
    const int K = P.K, N = P.N, Kp = P.Kp, Np = P.Np;
    const int CGn = Np >> 3, CGk = Kp >> 3;              // 8-column groups of G and of x
    const int g_term_bytes = kQbTileM * Np * 2;
    const int w_term_bytes = Kp * Np * 2;
    // carve: G terms (2) | xq^T terms (2) | W terms (3) | rounding-error stash | exponent table | barrier + tmem slot
    unsigned char *G = smem;
    unsigned char *X = G + 2 * g_term_bytes;
    unsigned char *W = X + 2 * kQbXTermBytes;
    const int Kd = Kp + 4;                                          // stash row stride (floats): 16-byte accesses of 8 rows spread over the banks
    float *dstash = reinterpret_cast<float *>(W + 3 * w_term_bytes);  // [128][Kd]: -ln2 * (round(x) - x), consumed by the epilogue
    const int stash_bytes = (P.want_df && P.qf != nullptr) ? kQbTileM * Kd * 4 : 0;
    const int Ke = P.Kt + 8;
    unsigned char *etab = reinterpret_cast<unsigned char *>(dstash) + stash_bytes;
    const int tab_bytes = (P.qf != nullptr) ? (P.rows_period * Ke + 15) / 16 * 16 : 0;
    uint64_t *bar = reinterpret_cast<uint64_t *>(etab + tab_bytes);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bar + 1);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    uint32_t tmem_cols = 32;
    while ((int)tmem_cols < Kp + 2 * Np) tmem_cols <<= 1;  // dXq | dWq from the hi and the lo term of G

    // ---- set-up -------------------------------------------------------------------------------------------------
    if (tid == 0) {
        tc::mbar_init(bar, 2);  // two issuing threads (one per product) commit to it
        tc::mbar_init_fence();
    }
    if (warp == 0) tc::tmem_alloc(tmem_slot, tmem_cols);
    if (P.qf != nullptr)
        for (int e = tid; e < P.rows_period * P.Kt; e += kQbThreads) {
            const int pr = e / P.Kt, k = e % P.Kt;
            const int fi = (k < K) ? __float2int_rn(__ldg(P.qf + pr * K + k)) : 0;
            etab[pr * Ke + k] = (unsigned char)(max(-126, min(127, fi)) + 127);
        }
    // xq^T operand: zero everywhere (padding rows k >= K stay zero for ever), ones in row k = K when no conversion
    // group covers it (K % 8 == 0); otherwise the conversion loop writes that 1.0 itself
    for (int e = tid; e < 2 * kQbXTermBytes / 16; e += kQbThreads) reinterpret_cast<uint4 *>(X)[e] = make_uint4(0, 0, 0, 0);
    __syncthreads();
    if ((K & 7) == 0)
        for (int r = tid; r < kQbTileM; r += kQbThreads)
            *reinterpret_cast<unsigned short *>(X + ((r >> 3) * 16 + (K >> 3)) * 128 + (r & 7) * 16) = 0x3F80;  // bf16 1.0
    // weights as the B operand of MMA1: rows k (the MMA's N index), contraction n; core (k/8, n/8)
    int w_lo = 0, w_lo2 = 0;
    for (int e = tid; e < Kp * Np; e += kQbThreads) {
        const int n = e % Np, k = e / Np;
        const float w = (k < K && n < N) ? __ldg(P.wq + (int64_t)k * N + n) : 0.f;
        __nv_bfloat16 h, l, l2;
        tc::split3(w, h, l, l2);
        const int off = ((k >> 3) * CGn + (n >> 3)) * 128 + (k & 7) * 16 + (n & 7) * 2;
        *reinterpret_cast<__nv_bfloat16 *>(W + off) = h;
        *reinterpret_cast<__nv_bfloat16 *>(W + w_term_bytes + off) = l;
        *reinterpret_cast<__nv_bfloat16 *>(W + 2 * w_term_bytes + off) = l2;
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
    const uint32_t acc1 = tmem_base, acc2 = tmem_base + (uint32_t)Kp;
    const uint32_t idesc1 = tc::make_idesc_bf16(Kp, false, false);
    const uint32_t idesc2 = tc::make_idesc_bf16(2 * Np, true, true);
    const uint32_t g_base = tc::smem_u32(G), x_base = tc::smem_u32(X), w_base = tc::smem_u32(W);

    const int r8 = lane & 7, q4 = lane >> 3;
    const bool vec_n = (N % 4 == 0) && aligned(P.gy, 16) && (P.y == nullptr || aligned(P.y, 16));
    const bool vec_k = (K % 4 == 0) && aligned(P.x, 16) && (P.ldx % 4 == 0) && (P.lddx % 4 == 0) && (P.dx == nullptr || aligned(P.dx, 16));
    const float rbias = (P.rm == RM_RND) ? 0.5f : 0.f;
    const uint32_t rp = (uint32_t)P.rows_period;  // divides 128 (checked on the host), so a tile starts at table row 0
    uint32_t phase = 0;
    bool ok = true;
    bool first_tile = true;

    // epilogue ownership: thread = (lane quarter q, column part cp): row r = 32 q + lane and the 8-column chunks
    // cp and cp + 4 of the accumulator (Kp <= 64: at most 8 chunks)
    const int qlane = (warp & 3) * 32, cpart = warp >> 2;
    const int nchunk = Kp >> 3;
    float df_r[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) df_r[j] = 0.f;

    // ---- per-thread constants of the dX staging (the same (row, chunk) pairs in every tile) -------------------------------
    // The staging floats are laid over exactly those 128-byte blocks of the xq^T buffers that the next tile's conversion
    // rewrites (row groups x the first Kp/8 column groups of both terms), so the zero padding and the ones row are never
    // disturbed.  A 16-byte chunk index is XOR-swizzled with the row to spread the banks.
    const int C = Kp >> 2;                  // 16-byte chunks per row
    const int swm = ((C & -C) - 1) & 7;     // XOR mask that stays inside the row
    auto st_off = [&](int rr, int c4s) -> int {  // byte offset inside X of the staged chunk (row, swizzled chunk)
        const int L = rr * Kp + (c4s << 2);
        const int b = L >> 5, within = L & 31;
        const int t = b / (16 * CGk), rem = b - t * (16 * CGk);
        const int rg = rem / CGk, kg = rem - rg * CGk;
        return t * kQbXTermBytes + (rg * 16 + kg) * 128 + within * 4;
    };
    int st_w[4];                            // where this thread parks its up to 4 chunks of dXq (row qlane + lane)
#pragma unroll
    for (int ci = 0; ci < 2; ++ci)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int c4 = (cpart + 4 * ci) * 2 + h, r = qlane + lane;
            st_w[ci * 2 + h] = (cpart + 4 * ci < nchunk) ? st_off(r, c4 ^ (r & swm)) : -1;
        }
    const int cv = K >> 2;                  // valid chunks per row of dX (vector path)
    int st_r[4], gl_r[4];                   // copy-out: staged chunk -> float4 index inside the tile's dX block
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int g = tid + kQbThreads * i;
        if (vec_k && g < kQbTileM * cv) {
            const int rr = g / cv, c4 = g - rr * cv;
            st_r[i] = st_off(rr, c4 ^ (rr & swm));
            gl_r[i] = rr * (int)(P.lddx >> 2) + c4;  // chunk index relative to the tile start, rows lddx floats apart
        } else {
            st_r[i] = -1;
            gl_r[i] = 0;
        }
    }

    // ---- slab ownership (the same in every tile) and the register prefetch ----------------------------------------------
    // G: unit u of a thread is combo c = u * 16 + warp -> row group mg = c / CG4g, column groups (c % CG4g) * 4 + q4;
    // x: likewise with CG4k.  The raw values of the first two G units and of both x units of the NEXT tile are fetched
    // into registers right after the MMAs of the current tile are issued, so their latency hides behind the wait and
    // the epilogue.
    const int CG4g = (CGn + 3) >> 2, combos_g = 16 * CG4g;  // <= 64
    const int CG4k = (CGk + 3) >> 2, combos_k = 16 * CG4k;  // <= 32
    float gv[2][8], yv[2][8], xv[2][8];
    auto load_g = [&](int u, int slot, int64_t t_row0) {
        const int c = u * 16 + warp;
        const int mg = c / CG4g, kg = (c - mg * CG4g) * 4 + q4;
        const bool act = c < combos_g && kg < CGn;
        const int64_t row = t_row0 + mg * 8 + r8;
        const int n0 = kg * 8;
        const int64_t grow = (P.gy_repeat > 1) ? (int64_t)fastdiv((uint32_t)row, P.gy_div) : row;  // M < 2^31 when repeating
        if (act && row < P.M && vec_n && n0 + 8 <= N) {
            const float4 a0 = __ldg(reinterpret_cast<const float4 *>(P.gy + grow * N + n0));
            const float4 a1 = __ldg(reinterpret_cast<const float4 *>(P.gy + grow * N + n0 + 4));
            gv[slot][0] = a0.x; gv[slot][1] = a0.y; gv[slot][2] = a0.z; gv[slot][3] = a0.w;
            gv[slot][4] = a1.x; gv[slot][5] = a1.y; gv[slot][6] = a1.z; gv[slot][7] = a1.w;
            if (P.relu) {
                const float4 y0 = __ldcs(reinterpret_cast<const float4 *>(P.y + row * N + n0));
                const float4 y1 = __ldcs(reinterpret_cast<const float4 *>(P.y + row * N + n0 + 4));
                yv[slot][0] = y0.x; yv[slot][1] = y0.y; yv[slot][2] = y0.z; yv[slot][3] = y0.w;
                yv[slot][4] = y1.x; yv[slot][5] = y1.y; yv[slot][6] = y1.z; yv[slot][7] = y1.w;
            }
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const bool in = act && row < P.M && n0 + j < N;
                gv[slot][j] = in ? __ldg(P.gy + grow * N + n0 + j) : 0.f;
                yv[slot][j] = (in && P.relu) ? __ldcs(P.y + row * N + n0 + j) : 1.f;
            }
        }
    };
    auto store_g = [&](int u, int slot) {
        const int c = u * 16 + warp;
        const int mg = c / CG4g, kg = (c - mg * CG4g) * 4 + q4;
        if (!(c < combos_g && kg < CGn)) return;
        if (P.relu) {
#pragma unroll
            for (int j = 0; j < 8; ++j) gv[slot][j] = yv[slot][j] > 0.f ? gv[slot][j] : 0.f;
        }
        uint32_t hi[4], lo[4];
#pragma unroll
        for (int j = 0; j < 8; j += 2) split2_pair(gv[slot][j], gv[slot][j + 1], hi[j >> 1], lo[j >> 1]);
        // core (row group, term, column group): the two terms of a row group are adjacent, so MMA2 takes both as one
        // operand of 2 Np columns with a uniform 128-byte group stride
        const int off = (mg * 2 * CGn + kg) * 128 + r8 * 16;
        *reinterpret_cast<uint4 *>(G + off) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
        *reinterpret_cast<uint4 *>(G + CGn * 128 + off) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
    };
    auto load_x = [&](int u, int64_t t_row0) {
        const int c = u * 16 + warp;
        const int mg = c / CG4k, kg = (c - mg * CG4k) * 4 + q4;
        const bool act = c < combos_k && kg < CGk;
        const int64_t row = t_row0 + mg * 8 + r8;
        const int k0 = kg * 8;
        if (act && row < P.M && vec_k && k0 + 8 <= K) {
            const float4 a0 = __ldcs(reinterpret_cast<const float4 *>(P.x + row * P.ldx + k0));
            const float4 a1 = __ldcs(reinterpret_cast<const float4 *>(P.x + row * P.ldx + k0 + 4));
            xv[u][0] = a0.x; xv[u][1] = a0.y; xv[u][2] = a0.z; xv[u][3] = a0.w;
            xv[u][4] = a1.x; xv[u][5] = a1.y; xv[u][6] = a1.z; xv[u][7] = a1.w;
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) xv[u][j] = (act && row < P.M && k0 + j < K) ? __ldcs(P.x + row * P.ldx + k0 + j) : 0.f;
        }
    };
    if ((int64_t)blockIdx.x < P.num_tiles) {
        load_g(0, 0, (int64_t)blockIdx.x * kQbTileM);
        load_g(1, 1, (int64_t)blockIdx.x * kQbTileM);
        load_x(0, (int64_t)blockIdx.x * kQbTileM);
        load_x(1, (int64_t)blockIdx.x * kQbTileM);
    }

    for (int64_t tile = blockIdx.x; tile < P.num_tiles && ok; tile += gridDim.x) {
        const int64_t row0 = tile * kQbTileM;
        // ---- G = dY (* relu mask), two bf16 terms, core (row/8, n/8) ------------------------------------------------
        store_g(0, 0);
        store_g(1, 1);
        if (combos_g > 32) {  // wide outputs (N > 64): the remaining units are fetched here, not prefetched
            load_g(2, 0, row0);
            load_g(3, 1, row0);
            store_g(2, 0);
            store_g(3, 1);
        }
        // ---- xq = round(x), two bf16 terms, transposed operand: core (row/8, k/8) in a 16-group-wide buffer ----------
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int c = u * 16 + warp;
            const int mg = c / CG4k, kg = (c - mg * CG4k) * 4 + q4;
            if (!(c < combos_k && kg < CGk)) continue;
            const int k0 = kg * 8, rl = mg * 8 + r8;
            if (P.qf != nullptr) {
                const uint32_t pr = (uint32_t)rl % rp;
                const uint2 eb = *reinterpret_cast<const uint2 *>(etab + pr * Ke + k0);
                float d[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const float xq = round_e<CONV>(xv[u][j], ((j < 4 ? eb.x : eb.y) >> ((j & 3) * 8)) & 0xffu, rbias);
                    d[j] = __fmul_rn(__fsub_rn(xq, xv[u][j]), -kLn2);
                    xv[u][j] = xq;
                }
                if (stash_bytes) {
                    *reinterpret_cast<float4 *>(dstash + rl * Kd + k0) = make_float4(d[0], d[1], d[2], d[3]);
                    *reinterpret_cast<float4 *>(dstash + rl * Kd + k0 + 4) = make_float4(d[4], d[5], d[6], d[7]);
                }
            }
            if (k0 + 8 > K) {
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    if (k0 + j >= K) xv[u][j] = (k0 + j == K) ? 1.f : 0.f;  // the row of ones that accumulates dbq
            }
            uint32_t hi[4], lo[4];
#pragma unroll
            for (int j = 0; j < 8; j += 2) split2_pair(xv[u][j], xv[u][j + 1], hi[j >> 1], lo[j >> 1]);
            const int off = (mg * 16 + kg) * 128 + r8 * 16;
            *reinterpret_cast<uint4 *>(X + off) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
            *reinterpret_cast<uint4 *>(X + kQbXTermBytes + off) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
        }
        tc::fence_smem_to_async();
        __syncthreads();
        // ---- tensor cores -------------------------------------------------------------------------------------------
        // The two products are issued by two threads (lane 0 of warps 0 and 1) with descriptors advanced by addition: one
        // thread building every descriptor from scratch is a serial critical path while the CTA waits.
        if (tid == 0) {
            tc::fence_after_sync();
            // MMA1: dXq = G x Wq^T, contraction over n in steps of 16 (start address + 256 bytes = + 16 units per step)
            bool first = true;
            for (int tg = 0; tg < 2; ++tg)
                for (int tw = 0; tw < n_w; ++tw) {
                    uint64_t da = tc::make_smem_desc(g_base + tg * CGn * 128, 128, (uint32_t)CGn * 256);
                    uint64_t db = tc::make_smem_desc(w_base + tw * w_term_bytes, 128, (uint32_t)CGn * 128);
                    for (int s = 0; s < Np / 16; ++s) {
                        tc::mma_bf16(acc1, da, db, idesc1, !first);
                        first = false;
                        da += 16;
                        db += 16;
                    }
                }
            tc::commit(bar);
        } else if (tid == 32) {
            tc::fence_after_sync();
            // MMA2: dWq (+ dbq row) += xq^T x G, contraction over the 128 rows in steps of 16; both operands MN-major:
            // stride between 8-groups along M/N = 128 B (sbo), between 8-groups along the rows = one buffer row (lbo)
            bool first = first_tile;
            // an MMA is bound by reading its 128-row A operand from shared memory whatever N is: both terms of G go through
            // one MMA as 2 Np columns; the two halves of the accumulator are added when the partials are written
            const uint32_t a_step = (2 * 16 * 128) >> 4, b_step = (uint32_t)(4 * CGn * 128) >> 4;
            for (int tx = 0; tx < 2; ++tx) {
                uint64_t da = tc::make_smem_desc(x_base + tx * kQbXTermBytes, 16 * 128, 128);
                uint64_t db = tc::make_smem_desc(g_base, (uint32_t)CGn * 256, 128);
                for (int s = 0; s < kQbTileM / 16; ++s) {
                    tc::mma_bf16(acc2, da, db, idesc2, !first);
                    first = false;
                    da += a_step;
                    db += b_step;
                }
            }
            tc::commit(bar);
        }
        first_tile = false;
        {   // next tile's raw operands start their trip from HBM now
            const int64_t ntile = tile + gridDim.x;
            if (ntile < P.num_tiles) {
                load_g(0, 0, ntile * kQbTileM);
                load_g(1, 1, ntile * kQbTileM);
                load_x(0, ntile * kQbTileM);
                load_x(1, ntile * kQbTileM);
            }
        }
        const bool waited = (warp == 0) ? tc::mbar_wait(bar, phase) : true;
        phase ^= 1u;
        ok = __syncthreads_and(waited ? 1 : 0) != 0;
        if (!ok) {
            if (tid == 0 && P.status) atomicOr(P.status, 1u);
            break;
        }
        // ---- epilogue: dXq -> df terms, dX ----------------------------------------------------------------------------
        tc::fence_after_sync();
        {
            const int r = qlane + lane;
            float v[16];
#pragma unroll
            for (int ci = 0; ci < 2; ++ci) {
                const int chunk = cpart + 4 * ci;  // warp-uniform
                if (chunk < nchunk) tc::tmem_ld8v(acc1 + ((uint32_t)qlane << 16) + (uint32_t)(chunk * 8), v + ci * 8);
            }
            if (stash_bytes) {
#pragma unroll
                for (int ci = 0; ci < 2; ++ci) {
                    const int kb = (cpart + 4 * ci) * 8;
                    if (cpart + 4 * ci < nchunk) {
                        const float4 d0 = *reinterpret_cast<const float4 *>(dstash + r * Kd + kb);
                        const float4 d1 = *reinterpret_cast<const float4 *>(dstash + r * Kd + kb + 4);
                        const float d[8] = {d0.x, d0.y, d0.z, d0.w, d1.x, d1.y, d1.z, d1.w};
#pragma unroll
                        for (int j = 0; j < 8; ++j) df_r[ci * 8 + j] = fmaf(d[j], v[ci * 8 + j], df_r[ci * 8 + j]);
                    }
                }
            }
            if (P.dx != nullptr) {
#pragma unroll
                for (int q = 0; q < 4; ++q)
                    if (st_w[q] >= 0)
                        *reinterpret_cast<float4 *>(X + st_w[q]) = make_float4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
                __syncthreads();
                const int64_t rows_here = (P.M - row0) < kQbTileM ? (P.M - row0) : kQbTileM;
                if (vec_k) {
                    float4 *dst = reinterpret_cast<float4 *>(P.dx + row0 * P.lddx);
                    const int limit = (int)rows_here * (int)(P.lddx >> 2);
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        if (st_r[i] >= 0 && gl_r[i] < limit) __stcs(dst + gl_r[i], *reinterpret_cast<const float4 *>(X + st_r[i]));
                } else {
                    for (int g = tid; g < (int)rows_here * K; g += kQbThreads) {
                        const int rr = g / K, k = g - rr * K;
                        __stcs(P.dx + (row0 + rr) * P.lddx + k,
                               *reinterpret_cast<const float *>(X + st_off(rr, (k >> 2) ^ (rr & swm)) + (k & 3) * 4));
                    }
                }
            }
        }
        tc::fence_before_sync();
        __syncthreads();
    }

    // ---- per-CTA partials: dWq | dbq from accumulator 2, df from the registers ------------------------------------------
    const bool did_work = (int64_t)blockIdx.x < P.num_tiles;
    float *pw = P.part + (int64_t)blockIdx.x * ((int64_t)(K + 1) * N + (int64_t)P.rows_period * K);
    float *pdf = pw + (int64_t)(K + 1) * N;
    if (ok && did_work) {
        tc::fence_after_sync();
        const int r = qlane + lane;  // accumulator lane = k index (lane K holds dbq)
        const int ncol = Np >> 2;    // columns per thread
        for (int c0 = cpart * ncol; c0 < (cpart + 1) * ncol; c0 += 8) {
            float v[8], v2[8];
            tc::tmem_ld8v(acc2 + ((uint32_t)qlane << 16) + (uint32_t)c0, v);
            tc::tmem_ld8v(acc2 + ((uint32_t)qlane << 16) + (uint32_t)(Np + c0), v2);
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = __fadd_rn(v[j], v2[j]);
            if (r <= K)
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    if (c0 + j < N) pw[(int64_t)r * N + c0 + j] = v[j];
        }
    } else {
        for (int e = tid; e < (K + 1) * N; e += kQbThreads) pw[e] = 0.f;
    }
    if (P.want_df && P.qf != nullptr) {
        // rows of the tile that share a table row are summed in a fixed order through shared memory
        __syncthreads();
        float *st = reinterpret_cast<float *>(X);  // [128][Kp]
        const int r = qlane + lane;
#pragma unroll
        for (int ci = 0; ci < 2; ++ci)
            if (cpart + 4 * ci < nchunk)
#pragma unroll
                for (int j = 0; j < 8; ++j) st[r * Kp + (cpart + 4 * ci) * 8 + j] = df_r[ci * 8 + j];
        __syncthreads();
        for (int e = tid; e < P.rows_period * K; e += kQbThreads) {
            const int pr = e / K, k = e - pr * K;
            float a = 0.f;
            for (int rr = pr; rr < kQbTileM; rr += P.rows_period) a = __fadd_rn(a, st[rr * Kp + k]);
            pdf[e] = a;
        }
    }
    tc::fence_before_sync();
    __syncthreads();
    if (warp == 0) tc::tmem_dealloc(tmem_base, tmem_cols);
}

// Sum of the per-CTA partials, in double and in a fixed order: element e of the partial vector [dWq | dbq | df] goes to
// its own output array.  A block owns eight consecutive elements; its 32 groups of eight lanes (four per warp) walk the
// partial records 32 apart, so that a few hundred records cost about ten loads per thread, all in flight together (the
// launch sits on the critical path of a step and is pure latency).
constexpr int kQbS2Elems = 8;
__global__ void __launch_bounds__(kThreads) k_qb_stage2(const float *__restrict__ part, int64_t stride, int nparts,
                                                       float *__restrict__ dw, int64_t nw, float *__restrict__ db, int64_t nb,
                                                       float *__restrict__ df, int64_t nf) {
    __shared__ double red[kThreads / 32][kQbS2Elems];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, sub = lane >> 3, j = lane & 7;
    const int64_t e = (int64_t)blockIdx.x * kQbS2Elems + j;
    const int64_t n = nw + nb + nf;
    double acc = 0.0;
    if (e < n) {
#pragma unroll 4
        for (int p = warp * 4 + sub; p < nparts; p += kThreads / 8) acc += (double)part[(int64_t)p * stride + e];
    }
    acc += __shfl_down_sync(0xffffffffu, acc, 16);
    acc += __shfl_down_sync(0xffffffffu, acc, 8);
    if (sub == 0) red[warp][j] = acc;
    __syncthreads();
    if (threadIdx.x < kQbS2Elems && e < n) {
        double a = 0.0;
#pragma unroll
        for (int w = 0; w < kThreads / 32; ++w) a += red[w][threadIdx.x];
        if (e < nw) dw[e] = (float)a;
        else if (e < nw + nb) { if (db != nullptr) db[e - nw] = (float)a; }
        else if (df != nullptr) df[e - nw - nb] = (float)a;
    }
}

int qdense_bwd_ws_launch(const float *gy, int gy_repeat, const float *y, const float *x, int64_t ldx, const float *qf,
                         int rows_period, int round_mode, const float *wq, float *dx, int64_t lddx, int dx_accumulate, float *part,
                         bool want_df, int64_t M, int K, int N, unsigned *status, cudaStream_t st, int *records);
bool qdense_bwd_ws_covers(int K, int N, int rows_period, bool relu, bool has_q);

// HGQ_QDENSE_BWD_WS=0 in the environment keeps every call on the general kernel (for comparisons).
static bool bwd_ws_enabled() {
    static const bool on = [] {
        const char *v = getenv("HGQ_QDENSE_BWD_WS");
        return !(v != nullptr && v[0] == '0');
    }();
    return on;
}

struct QbGeom {
    int Kp, Np, Kt, grid;
    size_t smem;
    int64_t tiles, part_stride;
};

static int qb_geom(int64_t M, int K, int N, int rows_period, QbGeom &g) {
    if (M <= 0 || K <= 0 || N <= 0 || rows_period <= 0) return HGQ_ERR_SIZE;
    if (K > 64 || N > 128) return HGQ_ERR_SIZE;
    if (kQbTileM % rows_period != 0) return HGQ_ERR_SIZE;
    g.Kp = (K + 15) / 16 * 16;
    g.Np = (N + 15) / 16 * 16;
    g.Kt = (K + 7) / 8 * 8;
    const size_t tab = ((size_t)rows_period * (g.Kt + 8) + 15) / 16 * 16;
    g.smem = 2 * (size_t)kQbTileM * g.Np * 2 + 2 * (size_t)kQbXTermBytes + 3 * (size_t)g.Kp * g.Np * 2 +
             (size_t)kQbTileM * (g.Kp + 4) * 4 + tab + 64;
    if (g.smem > 226 * 1024) return HGQ_ERR_SIZE;
    g.tiles = (M + kQbTileM - 1) / kQbTileM;
    int64_t grid = num_sms();  // 512 threads, > 113 KB shared memory: one CTA per SM
    if (grid > g.tiles) grid = g.tiles;
    g.grid = (int)grid;
    g.part_stride = (int64_t)(K + 1) * N + (int64_t)rows_period * K;
    return HGQ_OK;
}

}  // namespace hgq

using namespace hgq;

extern "C" size_t hgq_qdense_bwd_workspace(int64_t M, int K, int N, int rows_period) {
    QbGeom g;
    if (qb_geom(M, K, N, rows_period, g) != HGQ_OK) return 0;
    return (size_t)2 * num_sms() * g.part_stride * sizeof(float);  // the warp-specialised kernel writes two records per CTA
}

extern "C" int hgq_qdense_bwd(const float *gy, const float *y, const float *x, const float *qf, int rows_period,
                              int round_mode, const float *wq, float *dx, float *dwq, float *dbq, float *df, int64_t M,
                              int K, int N, void *workspace, size_t workspace_bytes, unsigned *status, void *stream) {
    return hgq_qdense_bwd_strided(gy, 1, y, x, K, qf, rows_period, round_mode, wq, dx, K, dwq, dbq, df, M, K, N, workspace,
                                  workspace_bytes, status, stream);
}

extern "C" int hgq_qdense_bwd_strided(const float *gy, int gy_repeat, const float *y, const float *x, int64_t ldx, const float *qf,
                                      int rows_period, int round_mode, const float *wq, float *dx, int64_t lddx, float *dwq,
                                      float *dbq, float *df, int64_t M, int K, int N, void *workspace, size_t workspace_bytes,
                                      unsigned *status, void *stream) {
    return hgq_qdense_bwd_accumulate(gy, gy_repeat, y, x, ldx, qf, rows_period, round_mode, wq, dx, lddx, 0, dwq, dbq, df, M, K, N,
                                     workspace, workspace_bytes, status, stream);
}

extern "C" int hgq_qdense_bwd_accumulate_supported(int K, int N, int rows_period, int relu, int has_quantizer) {
    return (bwd_ws_enabled() && qdense_bwd_ws_covers(K, N, rows_period, relu != 0, has_quantizer != 0)) ? 1 : 0;
}

extern "C" int hgq_qdense_bwd_accumulate(const float *gy, int gy_repeat, const float *y, const float *x, int64_t ldx, const float *qf,
                                         int rows_period, int round_mode, const float *wq, float *dx, int64_t lddx, int dx_accumulate,
                                         float *dwq, float *dbq, float *df, int64_t M, int K, int N, void *workspace,
                                         size_t workspace_bytes, unsigned *status, void *stream) {
    if (gy == nullptr || x == nullptr || wq == nullptr || dwq == nullptr) return HGQ_ERR_NULL;
    if (ldx < K || (dx != nullptr && lddx < K)) return HGQ_ERR_SIZE;
    if (gy_repeat < 1 || (gy_repeat > 1 && M >= ((int64_t)1 << 31))) return HGQ_ERR_SIZE;
    if (round_mode < 0 || round_mode > 2) return HGQ_ERR_MODE;
    if (df != nullptr && qf == nullptr) return HGQ_ERR_NULL;
    QbGeom g;
    if (int e = qb_geom(M, K, N, rows_period, g)) return e;
    const size_t need = (size_t)2 * g.grid * g.part_stride * sizeof(float);
    if (workspace == nullptr || workspace_bytes < need) return HGQ_ERR_WORKSPACE;
    if (!aligned(workspace, 16)) return HGQ_ERR_ALIGN;
    const int64_t nw_ = (int64_t)K * N, nf_ = (int64_t)rows_period * K;
    if (bwd_ws_enabled()) {
        int records = 0;
        const int r = qdense_bwd_ws_launch(gy, gy_repeat, y, x, ldx, qf, rows_period, round_mode, wq, dx, lddx, dx_accumulate,
                                           (float *)workspace, df != nullptr, M, K, N, status, (cudaStream_t)stream, &records);
        if (r < 0) return -r;
        if (r == 1) {
            if (int e = check_launch()) return e;
            k_qb_stage2<<<(unsigned)((g.part_stride + kQbS2Elems - 1) / kQbS2Elems), kThreads, 0, (cudaStream_t)stream>>>(
                (const float *)workspace, g.part_stride, records, dwq, nw_, dbq, N, df, df != nullptr ? nf_ : 0);
            return check_launch();
        }
    }
    if (dx_accumulate && dx != nullptr) return HGQ_ERR_SIZE;  // only the warp-specialised kernel adds into dx
    QbParams p;
    p.gy = gy; p.y = y; p.x = x; p.qf = qf; p.wq = wq; p.dx = dx;
    p.part = (float *)workspace;
    p.status = status;
    p.gy_repeat = gy_repeat; p.gy_div = make_fastdiv((uint32_t)gy_repeat);
    p.M = M; p.num_tiles = g.tiles; p.ldx = ldx; p.lddx = (dx != nullptr) ? lddx : K;
    p.K = K; p.N = N; p.Kp = g.Kp; p.Np = g.Np; p.Kt = g.Kt;
    p.rows_period = rows_period; p.rm = round_mode; p.relu = (y != nullptr) ? 1 : 0; p.want_df = (df != nullptr) ? 1 : 0;
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t ce;
    if (round_mode == RM_RND_CONV) {
        ce = cudaFuncSetAttribute(k_qdense_bwd<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)g.smem);
        if (ce != cudaSuccess) return (int)ce;
        k_qdense_bwd<true><<<g.grid, kQbThreads, g.smem, st>>>(p);
    } else {
        ce = cudaFuncSetAttribute(k_qdense_bwd<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)g.smem);
        if (ce != cudaSuccess) return (int)ce;
        k_qdense_bwd<false><<<g.grid, kQbThreads, g.smem, st>>>(p);
    }
    if (int e = check_launch()) return e;
    const int64_t nw = (int64_t)K * N, nf = (int64_t)rows_period * K;
    k_qb_stage2<<<(unsigned)((g.part_stride + kQbS2Elems - 1) / kQbS2Elems), kThreads, 0, st>>>(p.part, g.part_stride, g.grid, dwq, nw, dbq, N,
                                                                           df, df != nullptr ? nf : 0);
    if (int e = check_launch()) return e;
    return HGQ_OK;
}
