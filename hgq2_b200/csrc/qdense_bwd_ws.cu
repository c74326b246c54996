// K2b, warp-specialised (dense / einsum-dense backward): the contract of k_qdense_bwd in qdense_bwd.cu --
//     G = dY * (y > 0);  dXq = G @ Wq^T;  dX = dXq;  df[p, k] = sum_{r = p mod P} (-ln2 (round(x) - x)) dXq;
//     dWq = round(x)^T @ G;  dbq = sum_r G
// (the autograd backward of QDense.call / QEinsumDense.call, src/hgq/layers/core/dense.py:60-68, einsum_dense.py:72-83,
// with a rounding-only input quantizer, src/hgq/quantizer/internal/fixed_point_quantizer.py:403-424) -- for the shapes that
// carry the training workloads: K, N multiples of 4 that pad to 16 / 32 / 64, rows_period dividing 128.
//
// One persistent CTA per SM, three roles that meet only at mbarriers (no CTA-wide barrier inside the tile loop):
//   8 producer warps  stream dY, y and x of the NEXT tile into thread-private shared-memory slots with cp.async while they
//                     convert the current one: G (masked) and round(x) are split into two bf16 terms each and stored as
//                     tensor-core operands; the column sums of G (dbq) stay in registers across tiles.  A slot is
//                     refilled the moment its contents sit in registers, so one tile of raw data is always in flight.
//   1 issuing warp    MMA1  dXq[128 x K] = G x Wq^T into one of two accumulators in tensor memory;
//                     MMA2  dWq += xq^T x G with BOTH bf16 terms of xq stacked along M (rows 0..63 the high terms, rows
//                     64..127 the low terms) and both terms of G side by side along N: one M = 128 product per 16 rows
//                     instead of two, accumulated over all tiles of the CTA.
//   8 epilogue warps  read dXq back (tcgen05.ld), hand the accumulator back at once, transpose through a warp-private
//                     buffer and, piece by piece in coalesced order, re-read x (an L2 hit: the producers fetched it a few
//                     microseconds earlier), form the fractional-bit gradient terms and write dX.  The df sums live in
//                     registers across tiles (a lane meets the same table rows and columns in every tile).
// Per-CTA partials (two records: the rows of the accumulator that hold the high and the low terms of xq) are reduced in a
// fixed order by k_qb_stage2.  HBM-bound: 4 (2N + 2K) bytes per row.
// Every wait is bounded (polls and wall time); a role that gives up raises an abort word that ends the other roles' loops,
// the status word tells the host, and the CTA still frees its tensor memory.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "hgq_common.cuh"
#include "hgq_math.cuh"
#include "tc05.cuh"

namespace hgq {

constexpr int kBwTileM = 128;
constexpr int kBwProdWarps = 8, kBwProd = kBwProdWarps * 32;
constexpr int kBwEpiWarps = 8;
constexpr int kBwIssueWarp = kBwProdWarps + kBwEpiWarps;
constexpr int kBwThreads = (kBwProdWarps + kBwEpiWarps + 1) * 32;
constexpr int kBwXBytes = 128 * 128 * 2;      // xq^T operand: 128 rows x (64 high-term + 64 low-term) columns of bf16
constexpr int kBwOutWarpBytes = 4096;         // transposition buffer of one epilogue warp: 32 rows x 32 floats
constexpr unsigned kBwTimeout = 1u;

struct BwParams {
    const float *gy, *y, *x, *qf, *wq;
    float *dx;
    float *part;        // two records per CTA: [(K+1) x N] dWq|dbq, then [rows_period x K] df
    unsigned *status;
    int64_t M, num_tiles, ldx, lddx;
    int K, N, Kp, Np, Kt;
    int rows_period, rm, relu, want_df;
    int gy_repeat;
    FastDiv gy_div;
};

__device__ __forceinline__ void bw_arrive(uint64_t *bar) {
    asm volatile(
        "{\n\t"
        ".reg .b64 st;\n\t"
        "mbarrier.arrive.shared::cta.b64 st, [%0];\n\t"
        "}\n" ::"r"(tc::smem_u32(bar))
        : "memory");
}

__device__ __forceinline__ unsigned long long bw_now() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Wait for a phase of an mbarrier; gives up when another role has raised the abort word, after 2 s of wall time or after
// 2^24 polls, whichever comes first.
__device__ __forceinline__ bool bw_wait(uint64_t *bar, uint32_t parity, volatile int *abort_word) {
    if (tc::mbar_wait(bar, parity, 64)) return true;
    const unsigned long long t0 = bw_now();
    for (uint32_t it = 0; it < (1u << 16); ++it) {
        if (tc::mbar_wait(bar, parity, 256)) return true;
        if (*abort_word) return false;
        if (bw_now() - t0 > 2000000000ull) return false;
    }
    return false;
}

__device__ __forceinline__ void bw_split2_pair(float v0, float v1, uint32_t &hi, uint32_t &lo) {
    const __nv_bfloat162 h2 = __floats2bfloat162_rn(v0, v1);
    hi = *reinterpret_cast<const uint32_t *>(&h2);
    const float r0 = __fsub_rn(v0, __uint_as_float(hi << 16));
    const float r1 = __fsub_rn(v1, __uint_as_float(hi & 0xffff0000u));
    const __nv_bfloat162 l2 = __floats2bfloat162_rn(r0, r1);
    lo = *reinterpret_cast<const uint32_t *>(&l2);
}

template <bool CONV>
__device__ __forceinline__ float bw_round_e(float v, uint32_t ebyte, float rbias) {
    const uint32_t sbits = ebyte << 23;  // 2^f
    // scaling by a power of two is exact, so one fused multiply-add gives RN(v * 2^f + bias) bit for bit
    const float q = CONV ? rintf(__fmul_rn(v, __uint_as_float(sbits))) : floorf(__fmaf_rn(v, __uint_as_float(sbits), rbias));
    return __fmul_rn(q, __uint_as_float(0x7F000000u - sbits));
}

__device__ __forceinline__ int bw_swz(int r, int C) { return C == 8 ? (r & 7) : (C == 4 ? ((r >> 1) & 3) : ((r >> 2) & 1)); }

__device__ __forceinline__ void bw_cp16(uint32_t dst, const float *src, bool in) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(in ? 16 : 0) : "memory");
}

template <bool CONV>
__global__ void __launch_bounds__(kBwThreads, 1) k_qdense_bwd_ws(const BwParams P) {
    extern __shared__ __align__(128) unsigned char smem[];
    const int K = P.K, N = P.N, Kp = P.Kp, Np = P.Np;
    const int CGn = Np >> 3, CGk = Kp >> 3;  // 8-column groups of G and of x: 2, 4 or 8 each
    const int ITG = CGn >> 1, ITX = CGk >> 1;  // units (8 rows x 8 columns) a producer thread converts per tile
    const bool has_q = P.qf != nullptr;
    const int g_bytes = 2 * kBwTileM * Np * 2;  // both bf16 terms
    const int w_term_bytes = Kp * Np * 2;
    // carve: G operand | xq^T operand | W terms (3) | raw slots (dY, y, x) | transposition buffers | exponent table |
    // barriers, TMEM slot, abort word
    unsigned char *G = smem;
    unsigned char *X = G + g_bytes;
    unsigned char *W = X + kBwXBytes;
    unsigned char *raw = W + 3 * w_term_bytes;
    const int n_raw_units = ITG * (P.relu ? 2 : 1) + ITX;
    unsigned char *outst = raw + n_raw_units * kBwProd * 32;
    const int Ke = P.Kt + 8;
    unsigned char *etab = outst + kBwEpiWarps * kBwOutWarpBytes;
    const int tab_bytes = has_q ? (P.rows_period * Ke + 15) / 16 * 16 : 0;
    uint64_t *full = reinterpret_cast<uint64_t *>(etab + tab_bytes);
    uint64_t *stage_free = full + 1, *acc_full = full + 2, *acc_empty = full + 4;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(full + 6);
    int *abort_word = reinterpret_cast<int *>(tmem_slot + 1);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    uint32_t tmem_cols = 32;
    while ((int)tmem_cols < 2 * Kp + 2 * Np) tmem_cols <<= 1;  // two dXq accumulators | dWq from both terms of G

    // ---- one-time set-up (all threads) -------------------------------------------------------------------------------
    if (tid == 0) {
        tc::mbar_init(full, kBwProdWarps);
        tc::mbar_init(stage_free, 1);
        for (int a = 0; a < 2; ++a) {
            tc::mbar_init(acc_full + a, 1);
            tc::mbar_init(acc_empty + a, kBwEpiWarps);
        }
        *abort_word = 0;
        tc::mbar_init_fence();
    }
    if (warp == kBwIssueWarp) tc::tmem_alloc(tmem_slot, tmem_cols);
    if (has_q)
        for (int e = tid; e < P.rows_period * P.Kt; e += kBwThreads) {
            const int pr = e / P.Kt, k = e % P.Kt;
            const int fi = (k < K) ? __float2int_rn(__ldg(P.qf + pr * K + k)) : 0;
            etab[pr * Ke + k] = (unsigned char)(max(-126, min(127, fi)) + 127);
        }
    // the xq^T operand: column groups that no conversion unit writes (k >= Kp of either term) stay zero for ever
    for (int e = tid; e < kBwXBytes / 16; e += kBwThreads) reinterpret_cast<uint4 *>(X)[e] = make_uint4(0, 0, 0, 0);
    // weights as the B operand of MMA1: rows k (the product's N index), contraction n; core (k/8, n/8)
    int w_lo = 0, w_lo2 = 0;
    for (int e = tid; e < Kp * Np; e += kBwThreads) {
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
    const uint32_t acc2 = tmem_base + 2u * (uint32_t)Kp;
    const bool did_work = (int64_t)blockIdx.x < P.num_tiles;
    float *rec_hi = P.part + (int64_t)(2 * blockIdx.x) * ((int64_t)(K + 1) * N + (int64_t)P.rows_period * K);
    float *rec_lo = rec_hi + ((int64_t)(K + 1) * N + (int64_t)P.rows_period * K);

    if (warp < kBwProdWarps) {
        // ================================ producers ==================================================================
        // unit u = it * 32 + warp * 4 + q4: row group mg = u / CG, column group kg = u % CG (fixed per thread, because CG
        // divides 32); a quarter-warp (r8 = 0..7) fills one 128-byte core matrix.
        const int r8 = lane & 7, q4 = lane >> 3;
        const int ubase = warp * 4 + q4;
        const int kg_g = ubase % CGn, kg_x = ubase % CGk;
        const float rbias = (P.rm == RM_RND) ? 0.5f : 0.f;
        const uint32_t raw_base = tc::smem_u32(raw);
        // slot s of this thread: raw + (s * 256 + tid) * 32 bytes; slots: [0, ITG) dY, [ITG, 2 ITG) y (if relu), then x
        const int y_slot0 = ITG, x_slot0 = ITG * (P.relu ? 2 : 1);
        auto fetch_g = [&](int it, int64_t tile) {
            const int mg = (it * 32 + ubase) / CGn;
            const int64_t row = tile * kBwTileM + mg * 8 + r8;
            const int n0 = kg_g * 8;
            const bool row_in = tile < P.num_tiles && row < P.M;
            const int64_t grow = (P.gy_repeat > 1) ? (int64_t)fastdiv((uint32_t)(row_in ? row : 0), P.gy_div) : row;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const bool in = row_in && (n0 + 4 * h) < N;  // N % 4 == 0: a 16-byte piece is all inside or all outside
                bw_cp16(raw_base + (uint32_t)(((it * kBwProd + tid) * 2 + h) * 16), in ? P.gy + grow * N + n0 + 4 * h : P.gy, in);
                if (P.relu)
                    bw_cp16(raw_base + (uint32_t)((((y_slot0 + it) * kBwProd + tid) * 2 + h) * 16),
                            in ? P.y + row * N + n0 + 4 * h : P.gy, in);
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
        };
        auto fetch_x = [&](int it, int64_t tile) {
            const int mg = (it * 32 + ubase) / CGk;
            const int64_t row = tile * kBwTileM + mg * 8 + r8;
            const int k0 = kg_x * 8;
            const bool row_in = tile < P.num_tiles && row < P.M;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const bool in = row_in && (k0 + 4 * h) < K;
                bw_cp16(raw_base + (uint32_t)((((x_slot0 + it) * kBwProd + tid) * 2 + h) * 16),
                        in ? P.x + row * P.ldx + k0 + 4 * h : P.x, in);
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
        };
        // one commit group per unit, in unit order; past the last tile the groups are empty, so "all but the newest
        // (units - 1) groups have landed" always means "this unit has landed"
        for (int it = 0; it < ITG; ++it) fetch_g(it, blockIdx.x);
        for (int it = 0; it < ITX; ++it) fetch_x(it, blockIdx.x);
        const int units = ITG + ITX;

        float dbq_r[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) dbq_r[j] = 0.f;
        const uint32_t rp = (uint32_t)P.rows_period;  // divides 128: a tile starts at table row 0
        uint32_t n = 0;
        bool ok = true;
        for (int64_t tile = blockIdx.x; tile < P.num_tiles && ok; tile += gridDim.x, ++n) {
            const int64_t next = tile + gridDim.x;
            // the products of the previous tile must have finished reading the operand stage
            if (n > 0) {
                const bool w = bw_wait(stage_free, (n - 1) & 1u, abort_word);
                if (!__all_sync(0xffffffffu, w)) { ok = false; break; }
            }
            // ---- G = dY (* relu mask): two bf16 terms, core (row group, term, column group) -----------------------------
            for (int it = 0; it < ITG; ++it) {
                // units - 1 newer groups may still be in flight
                if (units == 2) asm volatile("cp.async.wait_group 1;" ::: "memory");
                else if (units == 3) asm volatile("cp.async.wait_group 2;" ::: "memory");
                else if (units == 4) asm volatile("cp.async.wait_group 3;" ::: "memory");
                else if (units == 5) asm volatile("cp.async.wait_group 4;" ::: "memory");
                else if (units == 6) asm volatile("cp.async.wait_group 5;" ::: "memory");
                else asm volatile("cp.async.wait_group 7;" ::: "memory");
                const unsigned char *sg = raw + (size_t)((it * kBwProd + tid) * 32);
                const float4 a0 = *reinterpret_cast<const float4 *>(sg), a1 = *reinterpret_cast<const float4 *>(sg + 16);
                float gv[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
                if (P.relu) {
                    const unsigned char *sy = raw + (size_t)(((y_slot0 + it) * kBwProd + tid) * 32);
                    const float4 y0 = *reinterpret_cast<const float4 *>(sy), y1 = *reinterpret_cast<const float4 *>(sy + 16);
                    const float yv[8] = {y0.x, y0.y, y0.z, y0.w, y1.x, y1.y, y1.z, y1.w};
#pragma unroll
                    for (int j = 0; j < 8; ++j) gv[j] = yv[j] > 0.f ? gv[j] : 0.f;
                }
                fetch_g(it, next);  // the slots just read are free again
#pragma unroll
                for (int j = 0; j < 8; ++j) dbq_r[j] = __fadd_rn(dbq_r[j], gv[j]);
                uint32_t hi[4], lo[4];
#pragma unroll
                for (int j = 0; j < 8; j += 2) bw_split2_pair(gv[j], gv[j + 1], hi[j >> 1], lo[j >> 1]);
                const int mg = (it * 32 + ubase) / CGn;
                const int off = (mg * 2 * CGn + kg_g) * 128 + r8 * 16;
                *reinterpret_cast<uint4 *>(G + off) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
                *reinterpret_cast<uint4 *>(G + CGn * 128 + off) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
            }
            // ---- xq = round(x): two bf16 terms stacked along M of the transposed operand ---------------------------------
            for (int it = 0; it < ITX; ++it) {
                if (units == 2) asm volatile("cp.async.wait_group 1;" ::: "memory");
                else if (units == 3) asm volatile("cp.async.wait_group 2;" ::: "memory");
                else if (units == 4) asm volatile("cp.async.wait_group 3;" ::: "memory");
                else if (units == 5) asm volatile("cp.async.wait_group 4;" ::: "memory");
                else if (units == 6) asm volatile("cp.async.wait_group 5;" ::: "memory");
                else asm volatile("cp.async.wait_group 7;" ::: "memory");
                const unsigned char *sx = raw + (size_t)(((x_slot0 + it) * kBwProd + tid) * 32);
                const float4 a0 = *reinterpret_cast<const float4 *>(sx), a1 = *reinterpret_cast<const float4 *>(sx + 16);
                float xv[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
                fetch_x(it, next);
                const int mg = (it * 32 + ubase) / CGk;
                if (has_q) {
                    const uint32_t pr = (uint32_t)(mg * 8 + r8) % rp;
                    const uint2 eb = *reinterpret_cast<const uint2 *>(etab + pr * Ke + kg_x * 8);
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        xv[j] = bw_round_e<CONV>(xv[j], ((j < 4 ? eb.x : eb.y) >> ((j & 3) * 8)) & 0xffu, rbias);
                }
                uint32_t hi[4], lo[4];
#pragma unroll
                for (int j = 0; j < 8; j += 2) bw_split2_pair(xv[j], xv[j + 1], hi[j >> 1], lo[j >> 1]);
                const int off = (mg * 16 + kg_x) * 128 + r8 * 16;
                *reinterpret_cast<uint4 *>(X + off) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
                *reinterpret_cast<uint4 *>(X + 8 * 128 + off) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
            }
            tc::fence_smem_to_async();
            __syncwarp();
            if (lane == 0) bw_arrive(full);
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        if (!ok) {
            *reinterpret_cast<volatile int *>(abort_word) = 1;
            if (lane == 0 && P.status) atomicOr(P.status, kBwTimeout);
        }
        // ---- dbq of this CTA: threads that share a column group are summed in a fixed order through the raw slots ----------
        asm volatile("bar.sync 1, %0;" ::"n"(kBwProd) : "memory");
        float *red = reinterpret_cast<float *>(raw);  // [256][8]
#pragma unroll
        for (int j = 0; j < 8; ++j) red[tid * 8 + j] = dbq_r[j];
        asm volatile("bar.sync 1, %0;" ::"n"(kBwProd) : "memory");
        for (int nn = tid; nn < N; nn += kBwProd) {
            const int kg = nn >> 3, j = nn & 7;
            float a = 0.f;
            for (int t = 0; t < kBwProd; ++t) {
                const int tub = (t >> 5) * 4 + ((t & 31) >> 3);
                if (tub % CGn == kg) a = __fadd_rn(a, red[t * 8 + j]);
            }
            rec_hi[(int64_t)K * N + nn] = did_work ? a : 0.f;
            rec_lo[(int64_t)K * N + nn] = 0.f;
        }
    } else if (warp == kBwIssueWarp) {
        // ================================ tensor-core issue ==========================================================
        const uint32_t idesc1 = tc::make_idesc_bf16(Kp, false, false);
        const uint32_t idesc2 = tc::make_idesc_bf16(2 * Np, true, true);
        const uint32_t g_base = tc::smem_u32(G), x_base = tc::smem_u32(X), w_base = tc::smem_u32(W);
        uint32_t n = 0;
        bool ok = true;
        for (int64_t tile = blockIdx.x; tile < P.num_tiles && ok; tile += gridDim.x, ++n) {
            const uint32_t a = n & 1u, ause = n >> 1;
            bool w = bw_wait(full, n & 1u, abort_word);
            // the epilogue must have drained this accumulator (tile n - 2) before the first product overwrites it
            if (w && ause > 0) w = bw_wait(acc_empty + a, (ause - 1) & 1u, abort_word);
            if (!__all_sync(0xffffffffu, w)) { ok = false; break; }
            tc::fence_after_sync();
            if (lane == 0) {
                // MMA1: dXq = G x Wq^T, contraction over n in steps of 16 (+ 256 bytes = + 16 descriptor units per step)
                const uint32_t acc1 = tmem_base + a * (uint32_t)Kp;
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
                // MMA2: dWq += xq^T x G, contraction over the 128 rows in steps of 16; both operands MN-major: stride between
                // 8-groups along M / N = 128 bytes, between 8-groups along the rows = one buffer row
                uint64_t da = tc::make_smem_desc(x_base, 16 * 128, 128);
                uint64_t db = tc::make_smem_desc(g_base, (uint32_t)CGn * 256, 128);
                const uint32_t a_step = (2 * 16 * 128) >> 4, b_step = (uint32_t)(4 * CGn * 128) >> 4;
                for (int s = 0; s < kBwTileM / 16; ++s) {
                    tc::mma_bf16(acc2, da, db, idesc2, !(n == 0 && s == 0));
                    da += a_step;
                    db += b_step;
                }
                tc::commit(stage_free);
                tc::commit(acc_full + a);
            }
            __syncwarp();
        }
        if (!ok) {
            *reinterpret_cast<volatile int *>(abort_word) = 1;
            if (lane == 0 && P.status) atomicOr(P.status, kBwTimeout);
        }
    } else {
        // ================================ epilogue ===================================================================
        // Warp e reads TMEM lanes 32 (e & 3) .. + 31 (the rows of the tile it owns) and the column half e >> 2.
        const int e = warp - kBwProdWarps, q = e & 3, part = e >> 2;
        float *ost = reinterpret_cast<float *>(outst + e * kBwOutWarpBytes);  // 32 rows x wc floats
        const int wc = Kp >> 1;          // 8, 16 or 32 columns per warp
        const int cv = wc >> 2;          // float4 chunks per row piece: 2, 4 or 8
        const int rows_it = 32 / cv;     // rows one copy-out iteration covers
        const int c0 = part * wc;
        const int my_rr = lane / cv, my_c4 = lane % cv;  // this lane's piece in iteration i: row my_rr + rows_it * i
        const int my_col = c0 + my_c4 * 4;               // its 4 columns (the same in every iteration and tile)
        const bool col_in = my_col < K;                  // K % 4 == 0
        const float rbias = (P.rm == RM_RND) ? 0.5f : 0.f;
        const bool do_df = P.want_df && has_q;
        float acc_df[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) acc_df[j] = 0.f;
        uint32_t n = 0;
        bool ok = true;
        for (int64_t tile = blockIdx.x; tile < P.num_tiles && ok; tile += gridDim.x, ++n) {
            const uint32_t a = n & 1u, ause = n >> 1;
            const int64_t wrow0 = tile * kBwTileM + q * 32;
            // x pieces of this tile (L2 hits: the producers fetched the lines a moment ago): the first four start their trip
            // before the accumulator is waited for, the rest once the accumulator's registers are free again
            auto load_x = [&](int i) -> float4 {
                const int64_t row = wrow0 + my_rr + rows_it * i;
                if (do_df && i < cv && row < P.M && col_in) return __ldg(reinterpret_cast<const float4 *>(P.x + row * P.ldx + my_col));
                return make_float4(0.f, 0.f, 0.f, 0.f);
            };
            float4 xa[4], xb[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) xa[i] = load_x(i);
            const bool w = bw_wait(acc_full + a, ause & 1u, abort_word);
            if (!__all_sync(0xffffffffu, w)) { ok = false; break; }
            tc::fence_after_sync();
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + a * (uint32_t)Kp + (uint32_t)c0;
            const int swz_w = bw_swz(lane, cv);
            for (int cb = 0; cb < wc; cb += 16) {  // 16 columns at a time keeps the register footprint down
                float v[16];
                if (wc >= 16) tc::tmem_ld16v(taddr + (uint32_t)cb, v);
                else tc::tmem_ld8v(taddr, v);
                if (cb + 16 >= wc) {  // the accumulator is in registers: hand it back to the issuing warp
                    tc::fence_before_sync();
                    __syncwarp();
                    if (lane == 0) bw_arrive(acc_empty + a);
                }
#pragma unroll
                for (int j = 0; j < 16; j += 4)
                    if (cb + j < wc)
                        *reinterpret_cast<float4 *>(ost + lane * wc + ((((cb + j) >> 2) ^ swz_w) << 2)) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) xb[i] = load_x(4 + i);
            __syncwarp();
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                if (i < cv) {
                    const int rr = my_rr + rows_it * i;
                    const int64_t row = wrow0 + rr;
                    const float4 o = *reinterpret_cast<const float4 *>(ost + rr * wc + ((my_c4 ^ bw_swz(rr, cv)) << 2));
                    if (do_df) {
                        const uint32_t pr = (uint32_t)(q * 32 + rr) % (uint32_t)P.rows_period;
                        const uint32_t eb = *reinterpret_cast<const uint32_t *>(etab + pr * Ke + my_col);
                        const float4 xp = (i < 4) ? xa[i & 3] : xb[i & 3];
                        const float xs[4] = {xp.x, xp.y, xp.z, xp.w};
                        const float os[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const float xq = bw_round_e<CONV>(xs[j], (eb >> (j * 8)) & 0xffu, rbias);
                            const float d = __fmul_rn(__fsub_rn(xq, xs[j]), -kLn2);
                            acc_df[i * 4 + j] = fmaf(d, os[j], acc_df[i * 4 + j]);
                        }
                    }
                    if (P.dx != nullptr && row < P.M && col_in)
                        __stcs(reinterpret_cast<float4 *>(P.dx + row * P.lddx + my_col), o);
                }
            }
            __syncwarp();  // the transposition buffer is reused by the next tile
        }
        if (!ok) {
            *reinterpret_cast<volatile int *>(abort_word) = 1;
            if (lane == 0 && P.status) atomicOr(P.status, kBwTimeout);
        }
        // ---- dWq partials: the accumulator of MMA2 is final once the last tile's commit has arrived (waited for above) -----
        // lanes 0..63 hold the sums over the high terms of xq (row k), lanes 64..127 those over the low terms
        if (ok && did_work) {
            tc::fence_after_sync();
            const int m = q * 32 + lane;          // accumulator lane
            const int k = m & 63;
            float *rec = (m < 64) ? rec_hi : rec_lo;
            const int ncol = Np >> 1;             // columns per warp of a lane quarter
            for (int cc = part * ncol; cc < (part + 1) * ncol; cc += 8) {
                float v1[8], v2[8];
                tc::tmem_ld8v(acc2 + ((uint32_t)(q * 32) << 16) + (uint32_t)cc, v1);
                tc::tmem_ld8v(acc2 + ((uint32_t)(q * 32) << 16) + (uint32_t)(Np + cc), v2);
                if (k < K)
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        if (cc + j < N) rec[(int64_t)k * N + cc + j] = __fadd_rn(v1[j], v2[j]);
            }
        } else {
            for (int idx = (warp - kBwProdWarps) * 32 + lane; idx < K * N; idx += kBwEpiWarps * 32) {
                rec_hi[idx] = 0.f;
                rec_lo[idx] = 0.f;
            }
        }
        // ---- df partials: rows of the tile that share a table row are summed in a fixed order through shared memory -------
        if (do_df) {
            // every epilogue warp is past its last tile: the operand buffers are idle (the last products have completed)
            asm volatile("bar.sync 2, %0;" ::"n"(kBwEpiWarps * 32) : "memory");
            float *st = reinterpret_cast<float *>(X);  // [128][Kp] floats <= 32 KB, the size of the xq^T operand
#pragma unroll
            for (int i = 0; i < 8; ++i)
                if (i < cv) {
                    const int rr = q * 32 + my_rr + rows_it * i;
#pragma unroll
                    for (int j = 0; j < 4; ++j) st[rr * Kp + my_col + j] = acc_df[i * 4 + j];
                }
            asm volatile("bar.sync 2, %0;" ::"n"(kBwEpiWarps * 32) : "memory");
            float *pdf_hi = rec_hi + (int64_t)(K + 1) * N, *pdf_lo = rec_lo + (int64_t)(K + 1) * N;
            for (int idx = (warp - kBwProdWarps) * 32 + lane; idx < P.rows_period * K; idx += kBwEpiWarps * 32) {
                const int pr = idx / K, k = idx - pr * K;
                float a = 0.f;
                for (int rr = pr; rr < kBwTileM; rr += P.rows_period) a = __fadd_rn(a, st[rr * Kp + k]);
                pdf_hi[idx] = (ok && did_work) ? a : 0.f;
                pdf_lo[idx] = 0.f;
            }
        }
    }

    // ---- tear-down ----------------------------------------------------------------------------------------------------
    tc::fence_before_sync();
    __syncthreads();
    if (warp == kBwIssueWarp) tc::tmem_dealloc(tmem_base, tmem_cols);
}

static size_t qdense_bwd_ws_smem(int Kp, int Np, int Kt, int rows_period, bool relu, bool has_q) {
    const int ITG = (Np >> 3) >> 1, ITX = (Kp >> 3) >> 1;
    const size_t g_bytes = 2 * (size_t)kBwTileM * Np * 2;
    const size_t raw = (size_t)(ITG * (relu ? 2 : 1) + ITX) * kBwProd * 32;
    const size_t tab = has_q ? ((size_t)rows_period * (Kt + 8) + 15) / 16 * 16 : 0;
    return g_bytes + kBwXBytes + 3 * (size_t)Kp * Np * 2 + raw + (size_t)kBwEpiWarps * kBwOutWarpBytes + tab + 6 * 8 + 32;
}

// Launches the warp-specialised backward when it covers the call: returns 1 with the number of partial records in
// *records, 0 when the call is not covered (the caller takes the general kernel), or a negative CUDA error code.
int qdense_bwd_ws_launch(const float *gy, int gy_repeat, const float *y, const float *x, int64_t ldx, const float *qf,
                         int rows_period, int round_mode, const float *wq, float *dx, int64_t lddx, float *part, bool want_df,
                         int64_t M, int K, int N, unsigned *status, cudaStream_t st, int *records) {
    const int Kp = (K + 15) / 16 * 16, Np = (N + 15) / 16 * 16, Kt = (K + 7) / 8 * 8;
    auto pow2_16_64 = [](int v) { return v == 16 || v == 32 || v == 64; };
    if (!pow2_16_64(Kp) || !pow2_16_64(Np) || K % 4 != 0 || N % 4 != 0) return 0;
    if (kBwTileM % rows_period != 0) return 0;
    if (!aligned(gy, 16) || !aligned(x, 16) || (y != nullptr && !aligned(y, 16)) || (dx != nullptr && !aligned(dx, 16))) return 0;
    if (ldx % 4 != 0 || (dx != nullptr && lddx % 4 != 0)) return 0;
    const size_t smem = qdense_bwd_ws_smem(Kp, Np, Kt, rows_period, y != nullptr, qf != nullptr);
    if (smem > 227 * 1024) return 0;
    BwParams p;
    p.gy = gy; p.y = y; p.x = x; p.qf = qf; p.wq = wq; p.dx = dx; p.part = part; p.status = status;
    p.M = M; p.num_tiles = (M + kBwTileM - 1) / kBwTileM; p.ldx = ldx; p.lddx = (dx != nullptr) ? lddx : K;
    p.K = K; p.N = N; p.Kp = Kp; p.Np = Np; p.Kt = Kt;
    p.rows_period = rows_period; p.rm = round_mode; p.relu = (y != nullptr) ? 1 : 0; p.want_df = want_df ? 1 : 0;
    p.gy_repeat = gy_repeat; p.gy_div = make_fastdiv((uint32_t)gy_repeat);
    const int g = (int)(p.num_tiles < num_sms() ? p.num_tiles : num_sms());
    *records = 2 * g;
    cudaError_t ce;
    if (round_mode == RM_RND_CONV) {
        ce = cudaFuncSetAttribute(k_qdense_bwd_ws<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (ce != cudaSuccess) return -(int)ce;
        k_qdense_bwd_ws<true><<<g, kBwThreads, smem, st>>>(p);
    } else {
        ce = cudaFuncSetAttribute(k_qdense_bwd_ws<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (ce != cudaSuccess) return -(int)ce;
        k_qdense_bwd_ws<false><<<g, kBwThreads, smem, st>>>(p);
    }
    return 1;
}

}  // namespace hgq
