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
// With the template parameter TMA the raw tiles are fetched by the copy engine instead: an extra loader warp issues tiled
// bulk-tensor copies (cp.async.bulk.tensor.2d, 128 rows x 32 floats, 128-byte swizzle; tensor maps over this GPU's dY, y
// and x only) as soon as every producer warp has taken its units out of a buffer, and the producers issue no copies at
// all.  (A dY that repeats rows -- the gradient of a sum -- has no tiled description and keeps the cp.async route.)
// Per-CTA partials (two records: the rows of the accumulator that hold the high and the low terms of xq) are reduced in a
// fixed order by k_qb_stage2.  HBM-bound: 4 (2N + 2K) bytes per row.
// Every wait is bounded (polls and wall time); a role that gives up raises an abort word that ends the other roles' loops,
// the status word tells the host, and the CTA still frees its tensor memory.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdlib>
#include <cstring>

#include "hgq_common.cuh"
#include "hgq_math.cuh"
#include "tc05.cuh"

namespace hgq {

constexpr int kBwTileM = 128;
constexpr int kBwProdWarps = 8, kBwProd = kBwProdWarps * 32;
constexpr int kBwEpiWarps = 8;
constexpr int kBwIssueWarp = kBwProdWarps + kBwEpiWarps;
constexpr int kBwThreads = (kBwProdWarps + kBwEpiWarps + 1) * 32;
constexpr int kBwLoadWarp = kBwIssueWarp + 1;  // bulk-copy loader (TMA variant only)
constexpr int kBwXBytes = 128 * 128 * 2;      // xq^T operand: 128 rows x (64 high-term + 64 low-term) columns of bf16
constexpr int kBwOutWarpBytes = 4096;         // transposition buffer of one epilogue warp: 32 rows x 32 floats
constexpr unsigned kBwTimeout = 1u;

struct BwParams {
    const float *gy, *y, *x, *qf, *wq;
    float *dx;
    int dx_accumulate;  // dx += dXq instead of dx = dXq (several layers that read the same input add their gradients up)
    float *part;        // two records per CTA: [(K+1) x N] dWq|dbq, then [rows_period x K] df
    unsigned *status;
    int64_t M, num_tiles, ldx, lddx;
    int K, N, Kp, Np, Kt;
    int rows_period, rm, relu, want_df;
    int gy_repeat;
    FastDiv gy_div;
    int g_box_rows;     // TMA variant: rows of dY one tile needs (128, or 128 / gy_repeat, at least 1, when dY repeats rows)
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

__device__ __forceinline__ void bw_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile(
        "{\n\t"
        ".reg .b64 st;\n\t"
        "mbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1;\n\t"
        "}\n" ::"r"(tc::smem_u32(bar)), "r"(bytes)
        : "memory");
}

// One tiled 2-D bulk copy global -> shared (this CTA's own shared memory), completion bytes counted on `bar`.
__device__ __forceinline__ void bw_tma_load_2d(uint32_t dst, const CUtensorMap *map, int c0, int c1, uint64_t *bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
                 "l"(map), "r"(c0), "r"(c1), "r"(tc::smem_u32(bar))
                 : "memory");
}

__device__ __forceinline__ int bw_swz(int r, int C) { return C == 8 ? (r & 7) : (C == 4 ? ((r >> 1) & 3) : ((r >> 2) & 1)); }

__device__ __forceinline__ void bw_cp16(uint32_t dst, const float *src, bool in) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(in ? 16 : 0) : "memory");
}

// The kernel is a template on the padded widths (CGN = Np / 8 and CGK = Kp / 8 column groups: 2, 4 or 8 each), on the
// ReLU mask and on the rounding flavour, so that every loop below has a constant trip count and every shared-memory offset
// is an immediate: the kernel is bound by the number of instructions it issues, not by bytes.
template <bool CONV, int CGN, int CGK, bool RELU, bool TMA>
__global__ void __launch_bounds__(kBwThreads + (TMA ? 32 : 0), 1) k_qdense_bwd_ws(const BwParams P, const __grid_constant__ CUtensorMap map_g,
                                                                                 const __grid_constant__ CUtensorMap map_y,
                                                                                 const __grid_constant__ CUtensorMap map_x) {
    constexpr int Np = CGN * 8, Kp = CGK * 8;
    constexpr int ITG = CGN / 2, ITX = CGK / 2;  // units (8 rows x 8 columns) a producer thread converts per tile
    constexpr int UNITS = ITG + ITX;
    constexpr int g_bytes = 2 * kBwTileM * Np * 2;  // both bf16 terms
    constexpr int w_term_bytes = Kp * Np * 2;
    constexpr int n_raw_units = ITG * (RELU ? 2 : 1) + ITX;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char *smem = smem_raw + ((1024u - (tc::smem_u32(smem_raw) & 1023u)) & 1023u);  // the carve starts on a 1 KB boundary
    const int K = P.K, N = P.N;
    const bool has_q = P.qf != nullptr;
    // carve: G operand | xq^T operand | W terms (3) | raw slots (dY, y, x) | transposition buffers | exponent table |
    // barriers, TMEM slot, abort word
    unsigned char *G = smem;
    unsigned char *X = G + g_bytes;
    unsigned char *W = X + kBwXBytes;
    constexpr int raw_off = (g_bytes + kBwXBytes + 3 * w_term_bytes + 1023) / 1024 * 1024;  // bulk copies land on a 1 KB boundary
    unsigned char *raw = smem + raw_off;
    unsigned char *outst = raw + n_raw_units * kBwProd * 32;
    const int Ke = P.Kt + 8;
    unsigned char *etab = outst + kBwEpiWarps * kBwOutWarpBytes;
    const int tab_bytes = has_q ? (P.rows_period * Ke + 15) / 16 * 16 : 0;
    uint64_t *full = reinterpret_cast<uint64_t *>(etab + tab_bytes);
    uint64_t *stage_free = full + 1, *acc_full = full + 2, *acc_empty = full + 4;
    uint64_t *rawg_full = full + 6, *rawg_empty = full + 7, *rawx_full = full + 8, *rawx_empty = full + 9;  // TMA variant
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(full + 10);
    int *abort_word = reinterpret_cast<int *>(tmem_slot + 1);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    constexpr uint32_t tmem_cols = (2 * Kp + 2 * Np) <= 32 ? 32u : (2 * Kp + 2 * Np) <= 64 ? 64u : (2 * Kp + 2 * Np) <= 128 ? 128u : 256u;

    // ---- one-time set-up (all threads) -------------------------------------------------------------------------------
    if (tid == 0) {
        tc::mbar_init(full, kBwProdWarps);
        tc::mbar_init(stage_free, 1);
        for (int a = 0; a < 2; ++a) {
            tc::mbar_init(acc_full + a, 1);
            tc::mbar_init(acc_empty + a, kBwEpiWarps);
        }
        tc::mbar_init(rawg_full, 1);   // the loader's expect_tx arrival (+ the copies' bytes)
        tc::mbar_init(rawx_full, 1);
        tc::mbar_init(rawg_empty, kBwProdWarps);
        tc::mbar_init(rawx_empty, kBwProdWarps);
        *abort_word = 0;
        tc::mbar_init_fence();
    }
    // The loader warp (TMA variant) takes no part in the conversions below: once the barriers exist it has the copy engine
    // fetch the CTA's first tile, so that the copies fly while the other warps convert the weights (on a launch of one
    // tile per CTA -- small batches -- that is a microsecond or more of the launch's length).
    constexpr int kSetupThreads = kBwThreads;  // the last warp is the loader
    constexpr int IBG = (CGN >= 4 ? 128 : 64), IBX = (CGK >= 4 ? 128 : 64);  // bytes per row of a raw box
    auto fetch_g = [&](int64_t tile) {
        const uint32_t raw_u = tc::smem_u32(raw);
        const uint32_t rawy_u = raw_u + 128 * Np * 4;
        const int g_boxes = (N + 31) / 32;  // a column half that lies past N is not fetched
        const int row0 = (int)(tile * kBwTileM);
        const int R = P.g_box_rows;  // 128 unless dY repeats rows
        const int grow0 = (P.gy_repeat > 1) ? (int)(tile * kBwTileM / P.gy_repeat) : row0;
        bw_expect_tx(rawg_full, (uint32_t)(g_boxes * IBG * (R + (RELU ? 128 : 0))));
        for (int b = 0; b < g_boxes; ++b) {
            bw_tma_load_2d(raw_u + b * R * IBG, &map_g, b * 32, grow0, rawg_full);
            if (RELU) bw_tma_load_2d(rawy_u + b * 128 * IBG, &map_y, b * 32, row0, rawg_full);
        }
    };
    auto fetch_x = [&](int64_t tile) {
        const uint32_t rawx_u = tc::smem_u32(raw) + 128 * Np * 4 * (RELU ? 2 : 1);
        const int x_boxes = (K + 31) / 32;
        bw_expect_tx(rawx_full, (uint32_t)(x_boxes * 128 * IBX));
        for (int b = 0; b < x_boxes; ++b) bw_tma_load_2d(rawx_u + b * 128 * IBX, &map_x, b * 32, (int)(tile * kBwTileM), rawx_full);
    };
    const bool is_loader = TMA && warp == kBwLoadWarp;
    if (TMA) {
        __syncthreads();  // the barriers are initialised
        if (is_loader && lane == 0 && (int64_t)blockIdx.x < P.num_tiles) {
            fetch_g(blockIdx.x);
            fetch_x(blockIdx.x);
        }
    }
    if (warp == kBwIssueWarp) tc::tmem_alloc(tmem_slot, tmem_cols);
    if (has_q && !is_loader)
        for (int e = tid; e < P.rows_period * P.Kt; e += kSetupThreads) {
            const int pr = e / P.Kt, k = e % P.Kt;
            const int fi = (k < K) ? __float2int_rn(__ldg(P.qf + pr * K + k)) : 0;
            etab[pr * Ke + k] = (unsigned char)(max(-126, min(127, fi)) + 127);
        }
    // the xq^T operand: column groups that no conversion unit writes (k >= Kp of either term) stay zero for ever
    for (int e = tid; e < kBwXBytes / 16 && !is_loader; e += kSetupThreads) reinterpret_cast<uint4 *>(X)[e] = make_uint4(0, 0, 0, 0);
    // weights as the B operand of MMA1: rows k (the product's N index), contraction n; core (k/8, n/8)
    int w_lo = 0, w_lo2 = 0;
    for (int e = tid; e < Kp * Np && !is_loader; e += kSetupThreads) {
        const int n = e % Np, k = e / Np;
        const float w = (k < K && n < N) ? __ldg(P.wq + (int64_t)k * N + n) : 0.f;
        __nv_bfloat16 h, l, l2;
        tc::split3(w, h, l, l2);
        const int off = ((k >> 3) * CGN + (n >> 3)) * 128 + (k & 7) * 16 + (n & 7) * 2;
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
    const int64_t rec_stride = (int64_t)(K + 1) * N + (int64_t)P.rows_period * K;
    float *rec_hi = P.part + (int64_t)(2 * blockIdx.x) * rec_stride;
    float *rec_lo = rec_hi + rec_stride;
    const int64_t tile_step = (int64_t)gridDim.x * kBwTileM;  // rows between two tiles of this CTA

    if (warp < kBwProdWarps) {
        // ================================ producers ==================================================================
        // unit u = it * 32 + warp * 4 + q4: row group mg = u / CG, column group kg = u % CG (fixed per thread, because CG
        // divides 32); a quarter-warp (r8 = 0..7) fills one 128-byte core matrix.
        const int r8 = lane & 7, q4 = lane >> 3;
        const int ubase = warp * 4 + q4;
        const int kg_g = ubase % CGN, kg_x = ubase % CGK;
        const int mg_g0 = ubase / CGN, mg_x0 = ubase / CGK;  // row group of unit `it`: mg0 + it * (32 / CG)
        const float rbias = (P.rm == RM_RND) ? 0.5f : 0.f;
        // Raw data travel in WARP-private 1 KB slots, filled cooperatively: the four units a warp converts in one iteration
        // are 8 (or 16) consecutive rows x 128 (or 64) contiguous bytes, and one cp.async instruction of the warp copies
        // whole 128-byte (64-byte) row segments -- every 32-byte sector it asks L2 for is used in full.  (With one private
        // slot per thread, a thread's two 16-byte copies sit in two instructions that each touch half of 32 sectors: the
        // L2 request rate, not HBM, then sets the pace.)  A 16-byte piece lands at an XOR-swizzled place in its row so that
        // the quarter-warp that later reads one unit (8 rows, same piece) hits 8 different bank groups.
        // slot s of this warp: raw + (s * 8 + warp) * 1024 bytes; slots: [0, ITG) dY, [ITG, 2 ITG) y (if RELU), then x
        constexpr int y_slot0 = ITG, x_slot0 = ITG * (RELU ? 2 : 1);
        constexpr int SEG_G = CGN >= 4 ? 8 : 4, SEG_X = CGK >= 4 ? 8 : 4;  // 16-byte pieces per row of a slot
        auto swz_of = [](int row_local, int segs) { return segs == 8 ? (row_local & 7) : ((row_local >> 1) & 3); };
        const uint32_t raw_warp = tc::smem_u32(raw) + (uint32_t)warp * 1024u;
        const unsigned char *raw_warp_p = raw + (size_t)warp * 1024;
        // copy geometry of this lane (two pieces per slot: c = lane and c = 32 + lane)
        int g_src[2], g_dst[2], x_src[2], x_dst[2];
        bool g_col[2], x_col[2];
        const int kg0_g = (warp * 4) % CGN, kg0_x = (warp * 4) % CGK;
#pragma unroll
        for (int j2 = 0; j2 < 2; ++j2) {
            const int c = j2 * 32 + lane;
            const int rl_g = c / SEG_G, sg_g = c % SEG_G, rl_x = c / SEG_X, sg_x = c % SEG_X;
            g_src[j2] = rl_g * N + kg0_g * 8 + sg_g * 4;  // floats from the first row of the slot (row stride N)
            g_col[j2] = kg0_g * 8 + sg_g * 4 < N;          // N % 4 == 0: a 16-byte piece is all inside or all outside
            g_dst[j2] = rl_g * SEG_G * 16 + ((sg_g ^ swz_of(rl_g, SEG_G)) * 16);
            x_src[j2] = rl_x;                               // row only: the row stride of x is a runtime value
            x_col[j2] = kg0_x * 8 + sg_x * 4 < K;
            x_dst[j2] = rl_x * SEG_X * 16 + ((sg_x ^ swz_of(rl_x, SEG_X)) * 16);
        }
        const int x_colf = kg0_x * 8 + (lane % SEG_X) * 4;  // c % SEG_X is the same for both pieces (32 % SEG_X == 0)
        // where this thread finds the two 16-byte halves of the unit it converts
        const int rl_gu = CGN >= 4 ? r8 : ((q4 >> 1) * 8 + r8), sg_gu = CGN >= 4 ? q4 * 2 : (q4 & 1) * 2;
        const int rl_xu = CGK >= 4 ? r8 : ((q4 >> 1) * 8 + r8), sg_xu = CGK >= 4 ? q4 * 2 : (q4 & 1) * 2;
        const int g_rd0 = rl_gu * SEG_G * 16 + ((sg_gu ^ swz_of(rl_gu, SEG_G)) * 16);
        const int g_rd1 = rl_gu * SEG_G * 16 + (((sg_gu + 1) ^ swz_of(rl_gu, SEG_G)) * 16);
        const int x_rd0 = rl_xu * SEG_X * 16 + ((sg_xu ^ swz_of(rl_xu, SEG_X)) * 16);
        const int x_rd1 = rl_xu * SEG_X * 16 + (((sg_xu + 1) ^ swz_of(rl_xu, SEG_X)) * 16);
        const bool linear_gy = P.gy_repeat <= 1;
        // first row of the tile being FETCHED (one tile ahead of the one being converted)
        int64_t f_row0 = (int64_t)blockIdx.x * kBwTileM;
        auto fetch_g = [&](int it) {
            const int64_t row_first = f_row0 + ((it * 32 + warp * 4) / CGN) * 8;
            const uint32_t dst = raw_warp + (uint32_t)(it * 8 * 1024), dsty = raw_warp + (uint32_t)((y_slot0 + it) * 8 * 1024);
#pragma unroll
            for (int j2 = 0; j2 < 2; ++j2) {
                const int rl = (j2 * 32 + lane) / SEG_G;
                const int64_t row = row_first + rl;
                const bool in = row < P.M && g_col[j2];
                if (linear_gy) {
                    bw_cp16(dst + (uint32_t)g_dst[j2], in ? P.gy + row_first * N + g_src[j2] : P.gy, in);
                } else {
                    const int64_t grow = (int64_t)fastdiv((uint32_t)(in ? row : 0), P.gy_div);
                    bw_cp16(dst + (uint32_t)g_dst[j2], in ? P.gy + grow * N + (g_src[j2] - rl * N) : P.gy, in);
                }
                if (RELU) bw_cp16(dsty + (uint32_t)g_dst[j2], in ? P.y + row_first * N + g_src[j2] : P.gy, in);
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
        };
        auto fetch_x = [&](int it) {
            const int64_t row_first = f_row0 + ((it * 32 + warp * 4) / CGK) * 8;
            const uint32_t dst = raw_warp + (uint32_t)((x_slot0 + it) * 8 * 1024);
#pragma unroll
            for (int j2 = 0; j2 < 2; ++j2) {
                const int64_t row = row_first + x_src[j2];
                const bool in = row < P.M && x_col[j2];
                bw_cp16(dst + (uint32_t)x_dst[j2], in ? P.x + row * P.ldx + x_colf : P.x, in);
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
        };
        // one commit group per unit, in unit order; past the last tile every row is out of range and the copies fetch
        // nothing, so "all but the newest UNITS - 1 groups have landed" always means "this unit has landed"
        if (!TMA) {
#pragma unroll
            for (int it = 0; it < ITG; ++it) fetch_g(it);
#pragma unroll
            for (int it = 0; it < ITX; ++it) fetch_x(it);
            f_row0 += tile_step;
        }
        // where this thread finds its unit (row group mg, column group kg) in a tile the copy engine wrote: one 128-row copy
        // per 32 columns (column half kg / 4), rows of IB = min(32, columns) * 4 bytes, 16-byte chunks XOR-swizzled with
        // the row (128-byte rows: chunk ^ (row & 7); 64-byte rows: chunk ^ ((row >> 1) & 3)); row & 7 = r8 here
        constexpr int IBG = (CGN >= 4 ? 128 : 64), IBX = (CGK >= 4 ? 128 : 64);
        const int swg = (IBG == 128) ? r8 : ((r8 >> 1) & 3), swx = (IBX == 128) ? r8 : ((r8 >> 1) & 3);
        const int tg_rd0 = (kg_g >> 2) * (128 * IBG) + r8 * IBG + ((((kg_g & 3) * 2) ^ swg) * 16);
        const int tg_rd1 = (kg_g >> 2) * (128 * IBG) + r8 * IBG + ((((kg_g & 3) * 2 + 1) ^ swg) * 16);
        const int tx_rd0 = (kg_x >> 2) * (128 * IBX) + r8 * IBX + ((((kg_x & 3) * 2) ^ swx) * 16);
        const int tx_rd1 = (kg_x >> 2) * (128 * IBX) + r8 * IBX + ((((kg_x & 3) * 2 + 1) ^ swx) * 16);
        constexpr int g_stream_bytes = 128 * Np * 4, x_stream_bytes = 128 * Kp * 4;  // one raw tile of dY (or y) / of x
        const unsigned char *raw_y = raw + g_stream_bytes, *raw_x = raw + g_stream_bytes * (RELU ? 2 : 1);

        float dbq_r[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) dbq_r[j] = 0.f;
        const uint32_t rp = (uint32_t)P.rows_period;  // divides 128: a tile starts at table row 0
        uint32_t n = 0;
        bool ok = true;
        for (int64_t tile = blockIdx.x; tile < P.num_tiles && ok; tile += gridDim.x, ++n) {
            // the products of the previous tile must have finished reading the operand stage
            if (n > 0) {
                const bool w = bw_wait(stage_free, (n - 1) & 1u, abort_word);
                if (!__all_sync(0xffffffffu, w)) { ok = false; break; }
            }
            // ---- G = dY (* relu mask): two bf16 terms, core (row group, term, column group) -----------------------------
#pragma unroll
            for (int it = 0; it < ITG; ++it) {
                float4 a0, a1, y0, y1;
                if (TMA) {
                    if (it == 0) {
                        const bool w = bw_wait(rawg_full, n & 1u, abort_word);
                        if (!__all_sync(0xffffffffu, w)) { ok = false; break; }
                    }
                    const int ro = (mg_g0 + it * (32 / CGN)) * 8 * IBG;
                    if (P.gy_repeat > 1) {
                        // dY repeats rows (gy_repeat is a multiple of 8): the 8 rows of a unit share one stored row, jr of the
                        // g_box_rows rows fetched for this tile; every lane of a quarter-warp reads the same 32 bytes
                        const int jr = ((mg_g0 + it * (32 / CGN)) * 8 / P.gy_repeat) % P.g_box_rows;
                        const int base = (kg_g >> 2) * (P.g_box_rows * IBG) + jr * IBG;
                        // the swizzle is a function of the shared-memory address (the raw tiles start on a 1 KB boundary)
                        const int sw = (IBG == 128) ? ((base >> 7) & 7) : ((base >> 7) & 3);
                        a0 = *reinterpret_cast<const float4 *>(raw + base + ((((kg_g & 3) * 2) ^ sw) * 16));
                        a1 = *reinterpret_cast<const float4 *>(raw + base + ((((kg_g & 3) * 2 + 1) ^ sw) * 16));
                    } else {
                        a0 = *reinterpret_cast<const float4 *>(raw + ro + tg_rd0);
                        a1 = *reinterpret_cast<const float4 *>(raw + ro + tg_rd1);
                    }
                    if (RELU) {
                        y0 = *reinterpret_cast<const float4 *>(raw_y + ro + tg_rd0);
                        y1 = *reinterpret_cast<const float4 *>(raw_y + ro + tg_rd1);
                    }
                    if (it == ITG - 1) {  // every lane holds its last unit of dY / y in registers: the buffers may be refilled
                        __syncwarp();
                        if (lane == 0) bw_arrive(rawg_empty);
                    }
                } else {
                    asm volatile("cp.async.wait_group %0;" ::"n"(UNITS - 1) : "memory");
                    __syncwarp();  // every lane's copies of this slot have landed
                    const unsigned char *sg = raw_warp_p + it * 8 * 1024;
                    a0 = *reinterpret_cast<const float4 *>(sg + g_rd0);
                    a1 = *reinterpret_cast<const float4 *>(sg + g_rd1);
                    if (RELU) {
                        const unsigned char *sy = raw_warp_p + (y_slot0 + it) * 8 * 1024;
                        y0 = *reinterpret_cast<const float4 *>(sy + g_rd0);
                        y1 = *reinterpret_cast<const float4 *>(sy + g_rd1);
                    }
                    __syncwarp();  // every lane has read its part: the slot is free
                    fetch_g(it);   // the next tile's data for this slot start their trip
                }
                float gv[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
                if (RELU) {
                    const float yv[8] = {y0.x, y0.y, y0.z, y0.w, y1.x, y1.y, y1.z, y1.w};
#pragma unroll
                    for (int j = 0; j < 8; ++j) gv[j] = yv[j] > 0.f ? gv[j] : 0.f;
                }
#pragma unroll
                for (int j = 0; j < 8; ++j) dbq_r[j] = __fadd_rn(dbq_r[j], gv[j]);
                uint32_t hi[4], lo[4];
#pragma unroll
                for (int j = 0; j < 8; j += 2) bw_split2_pair(gv[j], gv[j + 1], hi[j >> 1], lo[j >> 1]);
                const int off = ((mg_g0 + it * (32 / CGN)) * 2 * CGN + kg_g) * 128 + r8 * 16;
                *reinterpret_cast<uint4 *>(G + off) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
                *reinterpret_cast<uint4 *>(G + CGN * 128 + off) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
            }
            // ---- xq = round(x): two bf16 terms stacked along M of the transposed operand ---------------------------------
#pragma unroll
            for (int it = 0; it < ITX; ++it) {
                float4 a0, a1;
                if (TMA) {
                    if (it == 0) {
                        const bool w = bw_wait(rawx_full, n & 1u, abort_word);
                        if (!__all_sync(0xffffffffu, w)) { ok = false; break; }
                    }
                    const int ro = (mg_x0 + it * (32 / CGK)) * 8 * IBX;
                    a0 = *reinterpret_cast<const float4 *>(raw_x + ro + tx_rd0);
                    a1 = *reinterpret_cast<const float4 *>(raw_x + ro + tx_rd1);
                    if (it == ITX - 1) {
                        __syncwarp();
                        if (lane == 0) bw_arrive(rawx_empty);
                    }
                } else {
                    asm volatile("cp.async.wait_group %0;" ::"n"(UNITS - 1) : "memory");
                    __syncwarp();
                    const unsigned char *sx = raw_warp_p + (x_slot0 + it) * 8 * 1024;
                    a0 = *reinterpret_cast<const float4 *>(sx + x_rd0);
                    a1 = *reinterpret_cast<const float4 *>(sx + x_rd1);
                    __syncwarp();
                    fetch_x(it);
                }
                float xv[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
                const int mg = mg_x0 + it * (32 / CGK);
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
            if (!ok) break;  // a wait inside the unit loops gave up
            f_row0 += tile_step;
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
                if (tub % CGN == kg) a = __fadd_rn(a, red[t * 8 + j]);
            }
            rec_hi[(int64_t)K * N + nn] = did_work ? a : 0.f;
            rec_lo[(int64_t)K * N + nn] = 0.f;
        }
    } else if (warp == kBwIssueWarp) {
        // ================================ tensor-core issue ==========================================================
        constexpr uint32_t idesc1 = tc::make_idesc_bf16(Kp, false, false);
        constexpr uint32_t idesc2 = tc::make_idesc_bf16(2 * Np, true, true);
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
                        uint64_t da = tc::make_smem_desc(g_base + tg * CGN * 128, 128, (uint32_t)CGN * 256);
                        uint64_t db = tc::make_smem_desc(w_base + tw * w_term_bytes, 128, (uint32_t)CGN * 128);
#pragma unroll
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
                uint64_t db = tc::make_smem_desc(g_base, (uint32_t)CGN * 256, 128);
                constexpr uint32_t a_step = (2 * 16 * 128) >> 4, b_step = (uint32_t)(4 * CGN * 128) >> 4;
#pragma unroll
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
    } else if (TMA && warp == kBwLoadWarp) {
        // ================================ bulk-copy loader (TMA variant) ===========================================
        // Keeps one raw tile in flight per stream: as soon as every producer warp has taken its units of dY / y (of x) out
        // of the buffer, the copy engine fetches the next tile's into it.  The whole warp walks the loop (it stays
        // converged for the tear-down barrier); lane 0 issues.
        // (the first tile's copies were issued during the set-up)
        uint32_t n = 0;
        bool ok = true;
        for (int64_t tile = blockIdx.x; tile < P.num_tiles && ok; tile += gridDim.x, ++n) {
            if (n == 0) continue;
            {
                const bool w = bw_wait(rawg_empty, (n - 1) & 1u, abort_word);
                if (!__all_sync(0xffffffffu, w)) { ok = false; break; }
            }
            if (lane == 0) fetch_g(tile);
            __syncwarp();
            {
                const bool w = bw_wait(rawx_empty, (n - 1) & 1u, abort_word);
                if (!__all_sync(0xffffffffu, w)) { ok = false; break; }
            }
            if (lane == 0) fetch_x(tile);
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
        float *ost = reinterpret_cast<float *>(outst + e * kBwOutWarpBytes);  // 32 rows x WC floats
        constexpr int WC = Kp / 2;        // 8, 16 or 32 columns per warp
        constexpr int CV = WC / 4;        // float4 chunks per row piece: 2, 4 or 8
        constexpr int ROWS_IT = 32 / CV;  // rows one copy-out iteration covers
        const int c0 = part * WC;
        const int my_rr = lane / CV, my_c4 = lane % CV;  // this lane's piece in iteration i: row my_rr + ROWS_IT * i
        const int my_col = c0 + my_c4 * 4;               // its 4 columns (the same in every iteration and tile)
        const bool col_in = my_col < K;                  // K % 4 == 0
        const float rbias = (P.rm == RM_RND) ? 0.5f : 0.f;
        const bool do_df = P.want_df && has_q;
        const bool load_x = do_df && col_in;
        const bool store_dx = P.dx != nullptr && col_in;
        float acc_df[CV * 4];
#pragma unroll
        for (int j = 0; j < CV * 4; ++j) acc_df[j] = 0.f;
        // table bytes of this lane's pieces: row (q * 32 + my_rr + ROWS_IT * i) % rows_period, columns my_col .. + 3 -- the same
        // in every tile (tiles start at multiples of 128, which rows_period divides)
        const unsigned char *etab_my = etab + my_col;
        const uint32_t swz_w = (uint32_t)bw_swz(lane, CV);
        const float *x_my = P.x + ((int64_t)blockIdx.x * kBwTileM + q * 32 + my_rr) * P.ldx + my_col;
        float *dx_my = P.dx + ((int64_t)blockIdx.x * kBwTileM + q * 32 + my_rr) * P.lddx + my_col;
        const int64_t x_it = (int64_t)ROWS_IT * P.ldx, dx_it = (int64_t)ROWS_IT * P.lddx;
        const int64_t x_tile = tile_step * P.ldx, dx_tile = tile_step * P.lddx;
        uint32_t n = 0;
        bool ok = true;
        for (int64_t tile = blockIdx.x; tile < P.num_tiles && ok; tile += gridDim.x, ++n, x_my += x_tile, dx_my += dx_tile) {
            const uint32_t a = n & 1u, ause = n >> 1;
            const int64_t rows_left = P.M - (tile * kBwTileM + q * 32 + my_rr);  // row of piece i is in range iff ROWS_IT * i < rows_left
            // x pieces of this tile (L2 hits: the producers fetched the lines a moment ago): the first half starts its trip
            // before the accumulator is waited for, the rest once the accumulator's registers are free again
            float4 xa[(CV + 1) / 2], xb[(CV + 1) / 2];
#pragma unroll
            for (int i = 0; i < (CV + 1) / 2; ++i)
                xa[i] = (load_x && ROWS_IT * i < rows_left) ? __ldg(reinterpret_cast<const float4 *>(x_my + i * x_it)) : make_float4(0.f, 0.f, 0.f, 0.f);
            const bool w = bw_wait(acc_full + a, ause & 1u, abort_word);
            if (!__all_sync(0xffffffffu, w)) { ok = false; break; }
            tc::fence_after_sync();
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + a * (uint32_t)Kp + (uint32_t)c0;
#pragma unroll
            for (int cb = 0; cb < WC; cb += 16) {  // 16 columns at a time keeps the register footprint down
                float v[16];
                if (WC >= 16) tc::tmem_ld16v(taddr + (uint32_t)cb, v);
                else tc::tmem_ld8v(taddr, v);
                if (cb + 16 >= WC) {  // the accumulator is in registers: hand it back to the issuing warp
                    tc::fence_before_sync();
                    __syncwarp();
                    if (lane == 0) bw_arrive(acc_empty + a);
                }
#pragma unroll
                for (int j = 0; j < 16; j += 4)
                    if (cb + j < WC)
                        *reinterpret_cast<float4 *>(ost + lane * WC + ((((cb + j) >> 2) ^ swz_w) << 2)) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
            }
#pragma unroll
            for (int i = 0; i < CV / 2; ++i) {
                const int ii = (CV + 1) / 2 + i;
                xb[i] = (load_x && ROWS_IT * ii < rows_left) ? __ldg(reinterpret_cast<const float4 *>(x_my + ii * x_it)) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
            __syncwarp();
#pragma unroll
            for (int i = 0; i < CV; ++i) {
                const int rr = my_rr + ROWS_IT * i;
                const float4 o = *reinterpret_cast<const float4 *>(ost + rr * WC + ((my_c4 ^ bw_swz(rr, CV)) << 2));
                if (do_df) {
                    const uint32_t pr = (uint32_t)(q * 32 + rr) % (uint32_t)P.rows_period;
                    const uint32_t eb = *reinterpret_cast<const uint32_t *>(etab_my + pr * Ke);
                    const float4 xp = (i < (CV + 1) / 2) ? xa[i < (CV + 1) / 2 ? i : 0] : xb[i >= (CV + 1) / 2 ? i - (CV + 1) / 2 : 0];
                    const float xs[4] = {xp.x, xp.y, xp.z, xp.w};
                    const float os[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float xq = bw_round_e<CONV>(xs[j], (eb >> (j * 8)) & 0xffu, rbias);
                        const float d = __fmul_rn(__fsub_rn(xq, xs[j]), -kLn2);
                        acc_df[i * 4 + j] = fmaf(d, os[j], acc_df[i * 4 + j]);
                    }
                }
                if (store_dx && ROWS_IT * i < rows_left) {
                    float4 out = o;
                    if (P.dx_accumulate) {
                        const float4 old = __ldcs(reinterpret_cast<const float4 *>(dx_my + i * dx_it));
                        out.x = __fadd_rn(old.x, o.x); out.y = __fadd_rn(old.y, o.y); out.z = __fadd_rn(old.z, o.z); out.w = __fadd_rn(old.w, o.w);
                    }
                    __stcs(reinterpret_cast<float4 *>(dx_my + i * dx_it), out);
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
            constexpr int ncol = Np / 2;          // columns per warp of a lane quarter
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
            for (int i = 0; i < CV; ++i) {
                const int rr = q * 32 + my_rr + ROWS_IT * i;
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
    const size_t operands = (g_bytes + kBwXBytes + 3 * (size_t)Kp * Np * 2 + 1023) / 1024 * 1024;  // the raw tiles start on a 1 KB boundary
    return 1024 + operands + raw + (size_t)kBwEpiWarps * kBwOutWarpBytes + tab + 10 * 8 + 32;  // + room to align the carve itself
}

// cuTensorMapEncodeTiled through the runtime's driver entry point query (the library does not link against libcuda)
typedef CUresult (*BwEncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                    const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static BwEncodeTiledFn bw_encode_tiled_fn() {
    static const BwEncodeTiledFn fn = [] {
        void *ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess) {
            cudaGetLastError();
            return (BwEncodeTiledFn) nullptr;
        }
        return (BwEncodeTiledFn)ptr;
    }();
    return fn;
}

// HGQ_QDENSE_BWD_TMA=0 / 1 in the environment picks how raw tiles are fetched (cooperative cp.async / bulk tensor copies).
static bool bw_tma_enabled() {
    static const bool on = [] {
        const char *v = getenv("HGQ_QDENSE_BWD_TMA");
        return v != nullptr ? v[0] != '0' : true;
    }();
    return on;
}

// A tensor map over a row-major fp32 matrix [rows, cols] with row stride ld floats (this GPU's memory only): boxes of 128
// rows x min(32, padded columns) floats, swizzled over the box's row length (128 or 64 bytes), zeros outside.
static bool bw_make_tmap(CUtensorMap *map, const float *base, int64_t rows, int cols, int64_t ld, int padded_cols,
                         int box_rows = kBwTileM) {
    const BwEncodeTiledFn enc = bw_encode_tiled_fn();
    if (enc == nullptr || base == nullptr) return false;
    const cuuint32_t inner = padded_cols >= 32 ? 32u : 16u;
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld * 4};
    const cuuint32_t box[2] = {inner, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    return enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
               inner == 32 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Launches the warp-specialised backward when it covers the call: returns 1 with the number of partial records in
// *records, 0 when the call is not covered (the caller takes the general kernel), or a negative CUDA error code.
// Shapes the warp-specialised backward covers (pointer alignment aside).
bool qdense_bwd_ws_covers(int K, int N, int rows_period, bool relu, bool has_q) {
    const int Kp = (K + 15) / 16 * 16, Np = (N + 15) / 16 * 16, Kt = (K + 7) / 8 * 8;
    auto pow2_16_64 = [](int v) { return v == 16 || v == 32 || v == 64; };
    if (!pow2_16_64(Kp) || !pow2_16_64(Np) || K % 4 != 0 || N % 4 != 0 || rows_period <= 0 || kBwTileM % rows_period != 0) return false;
    return qdense_bwd_ws_smem(Kp, Np, Kt, rows_period, relu, has_q) <= 227 * 1024;
}

int qdense_bwd_ws_launch(const float *gy, int gy_repeat, const float *y, const float *x, int64_t ldx, const float *qf,
                         int rows_period, int round_mode, const float *wq, float *dx, int64_t lddx, int dx_accumulate, float *part,
                         bool want_df, int64_t M, int K, int N, unsigned *status, cudaStream_t st, int *records) {
    const int Kp = (K + 15) / 16 * 16, Np = (N + 15) / 16 * 16, Kt = (K + 7) / 8 * 8;
    auto pow2_16_64 = [](int v) { return v == 16 || v == 32 || v == 64; };
    if (!pow2_16_64(Kp) || !pow2_16_64(Np) || K % 4 != 0 || N % 4 != 0) return 0;
    if (kBwTileM % rows_period != 0) return 0;
    if (!aligned(gy, 16) || !aligned(x, 16) || (y != nullptr && !aligned(y, 16)) || (dx != nullptr && !aligned(dx, 16))) return 0;
    if (ldx % 4 != 0 || (dx != nullptr && lddx % 4 != 0)) return 0;
    const size_t smem = qdense_bwd_ws_smem(Kp, Np, Kt, rows_period, y != nullptr, qf != nullptr);
    if (smem > 227 * 1024) return 0;
    BwParams p;
    p.gy = gy; p.y = y; p.x = x; p.qf = qf; p.wq = wq; p.dx = dx; p.dx_accumulate = dx_accumulate; p.part = part; p.status = status;
    p.M = M; p.num_tiles = (M + kBwTileM - 1) / kBwTileM; p.ldx = ldx; p.lddx = (dx != nullptr) ? lddx : K;
    p.K = K; p.N = N; p.Kp = Kp; p.Np = Np; p.Kt = Kt;
    p.rows_period = rows_period; p.rm = round_mode; p.relu = (y != nullptr) ? 1 : 0; p.want_df = want_df ? 1 : 0;
    p.gy_repeat = gy_repeat; p.gy_div = make_fastdiv((uint32_t)gy_repeat);
    const int g = (int)(p.num_tiles < num_sms() ? p.num_tiles : num_sms());
    *records = 2 * g;
    const int cgn = Np / 8, cgk = Kp / 8;
    const bool relu = y != nullptr, conv = round_mode == RM_RND_CONV;
    // bulk tensor copies: rows must fit a 32-bit coordinate; a dY that repeats rows (the gradient of a sum over an axis) has a
    // tiled description when a group of 8 rows shares one stored row and a tile covers whole stored rows
    CUtensorMap map_g, map_y, map_x;
    memset(&map_g, 0, sizeof(map_g)); memset(&map_y, 0, sizeof(map_y)); memset(&map_x, 0, sizeof(map_x));
    const bool rep_ok = gy_repeat == 1 || (gy_repeat % 8 == 0 && M % gy_repeat == 0 &&
                                           ((gy_repeat <= kBwTileM && kBwTileM % gy_repeat == 0) || gy_repeat % kBwTileM == 0));
    p.g_box_rows = gy_repeat == 1 ? kBwTileM : (gy_repeat >= kBwTileM ? 1 : kBwTileM / gy_repeat);
    const bool tma = bw_tma_enabled() && rep_ok && M < ((int64_t)1 << 31) &&
                     bw_make_tmap(&map_g, gy, M / gy_repeat, N, N, Np, p.g_box_rows) &&
                     (!relu || bw_make_tmap(&map_y, y, M, N, N, Np)) && bw_make_tmap(&map_x, x, M, K, ldx, Kp);
    cudaError_t ce = cudaSuccess;
    bool launched = false;
#define HGQ_BW_CASE1(CV_, CGN_, CGK_, RELU_, TMA_)                                                                           \
    do {                                                                                                                    \
        ce = cudaFuncSetAttribute(k_qdense_bwd_ws<CV_, CGN_, CGK_, RELU_, TMA_>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                  (int)smem);                                                                               \
        if (ce != cudaSuccess) return -(int)ce;                                                                             \
        k_qdense_bwd_ws<CV_, CGN_, CGK_, RELU_, TMA_><<<g, kBwThreads + (TMA_ ? 32 : 0), smem, st>>>(p, map_g, map_y, map_x); \
        launched = true;                                                                                                    \
    } while (0)
#define HGQ_BW_CASE(CV_, CGN_, CGK_, RELU_)                                                                                  \
    if (!launched && conv == CV_ && cgn == CGN_ && cgk == CGK_ && relu == RELU_) {                                           \
        if (tma) HGQ_BW_CASE1(CV_, CGN_, CGK_, RELU_, true);                                                                 \
        else HGQ_BW_CASE1(CV_, CGN_, CGK_, RELU_, false);                                                                    \
    }
#define HGQ_BW_SHAPES(CV_, RELU_)                                                                                           \
    HGQ_BW_CASE(CV_, 2, 2, RELU_) HGQ_BW_CASE(CV_, 2, 4, RELU_) HGQ_BW_CASE(CV_, 2, 8, RELU_)                               \
    HGQ_BW_CASE(CV_, 4, 2, RELU_) HGQ_BW_CASE(CV_, 4, 4, RELU_) HGQ_BW_CASE(CV_, 4, 8, RELU_)                               \
    HGQ_BW_CASE(CV_, 8, 2, RELU_) HGQ_BW_CASE(CV_, 8, 4, RELU_) HGQ_BW_CASE(CV_, 8, 8, RELU_)
    HGQ_BW_SHAPES(false, false)
    HGQ_BW_SHAPES(false, true)
    HGQ_BW_SHAPES(true, false)
    HGQ_BW_SHAPES(true, true)
#undef HGQ_BW_SHAPES
#undef HGQ_BW_CASE
#undef HGQ_BW_CASE1
    if (!launched) return 0;
    return 1;
}

}  // namespace hgq
