// K2w (dense / einsum-dense forward, warp-specialised): y = act( iq(x) @ Wq + bq ) for the training-mode case in which
// the input quantizer only rounds (WRAP overflow in training), the contract of k_qdense_fwd in qdense.cu.
//
// Stands in for QDense.call (src/hgq/layers/core/dense.py:60-68) and QEinsumDense.call
// (src/hgq/layers/core/einsum_dense.py:72-83); the per-entry max |round(x)| of the WRAP integer-bit tracking
// (fixed_point_quantizer.py:405-413) is a side output.
//
// One persistent CTA per SM with three roles that meet only at mbarriers, never at a CTA-wide barrier:
//   NPW producer warps (8): fetch a 128 x 64 fp32 slab (cp.async into thread-private slots, two slabs ahead), quantise it
//               in registers, split every value exactly into bf16 terms and store them as no-swizzle K-major core
//               matrices into one of two operand stages; arrive on full[stage];
//   EW epilogue warps (8): wait for acc_full[acc], read their 32 rows of the accumulator with tcgen05.ld (up to 32 columns
//               at a time; the two warps of a lane quarter take alternate column pieces), release the accumulator
//               (acc_empty[acc]), add bias, apply the activation, transpose through a warp-private 4 KB buffer and write
//               whole 128-byte row pieces;
//   the last warp waits for full[stage] and for a free accumulator, issues tcgen05.mma (M = 128, N = padded N, K = 16)
//               for every pair of terms, commits to empty[stage] and, after the last slab of a tile, to acc_full[acc].
// With two operand stages and two accumulators in tensor memory the conversion of tile t + 1 overlaps the products of
// tile t and the write-out of tile t - 1.  HBM-bound: 4 (K + N) bytes per row.
// Raw slabs reach shared memory in one of two ways (template parameter TMA): every producer thread copies its own pieces
// with cp.async into thread-private slots, or an extra loader warp has the copy engine fetch the whole 128 x 64 slab as
// two tiled bulk-tensor copies (cp.async.bulk.tensor.2d, 128 rows x 32 floats each, 128-byte swizzle, completion counted
// on an mbarrier), from a tensor map over this GPU's x alone.  Rows past the end of x and columns past K arrive as zeros.
// Every wait is bounded (polls and wall time); a wait that gives up sets an abort word that ends every role's loop, the
// status word tells the host, and the CTA still frees its tensor memory.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdlib>
#include <cstring>

#include "hgq_common.cuh"
#include "hgq_math.cuh"
#include "tc05.cuh"

namespace hgq {

// The kernel is a template on its warp split: NPW producer warps (8 or 16), EW epilogue warps (4 or 8), one issuing warp.
constexpr int kWsTileM = 128;
constexpr int kWsKC = 64;                            // K slab of one operand stage
constexpr int kWsTermBytes = kWsTileM * kWsKC * 2;   // 16 KB per bf16 term
constexpr int kWsStageBytes = 3 * kWsTermBytes;      // hi, lo and (rarely non-zero) third term
constexpr int kWsFetchBytes = kWsTileM * kWsKC * 4;  // raw fp32 slab in flight
constexpr int kWsOutWarpBytes = 4096;                // transposition buffer of one epilogue warp: 32 rows x 32 floats
constexpr unsigned kWsTimeout = 1u;                  // status bit, same meaning as in the other tensor-core kernels

// Abs-max bookkeeping (max over rows of |round(x)| per entry of the quantizer table):
//   REGS1 / REGS2  one K slab and a period that divides 128: a tile starts at table row 0, so the table rows (one when the
//          period divides 64, else two) and the 8 columns of a thread never change; maxima live in registers and are merged
//          through a table in shared memory (atomic max on the bit patterns) when the CTA is done
//   PLAIN  period 64 or 128, several K slabs: rows that share a table entry fall to the same thread, plain
//          read-modify-write of the table in shared memory
//   REGS2X2  as REGS2 for TWO K slabs (K up to 128): a second set of registers holds the maxima of the second slab's
//          columns; the merge table has no row padding so that 64 x 128 entries fit the (single) raw-slab buffer
enum : int { WS_AMAX_NONE = 0, WS_AMAX_REGS1 = 1, WS_AMAX_PLAIN = 2, WS_AMAX_REGS2 = 3, WS_AMAX_REGS2X2 = 4 };

struct WsParams {
    const float *x, *qf, *wq, *bq;
    float *y;
    unsigned *amax_part;  // [gridDim.x, rows_period * K] abs-max partials, or nullptr
    int amax_direct;      // amax_part is the [rows_period * K] result itself: merge by atomic max
    unsigned *status;
    int64_t M, num_tiles;
    int K, N, Kpad, Npad, Kt, rows_period;
    int rm, act;
    int depth;            // raw slabs in flight ahead of the conversion: 1 or 2
    int tma_store;        // the epilogue hands finished 128 x 32 blocks to the copy engine (tiled bulk-tensor stores)
    float *pool_out;      // [M / pool_rows, N]: pool_scale * (sum of y over every group of pool_rows consecutive rows), or nullptr
    int pool_rows;        // 32, 64 or 128 (bulk-store path only)
    float pool_scale;
};

__device__ __forceinline__ void ws_arrive(uint64_t *bar) {
    asm volatile(
        "{\n\t"
        ".reg .b64 st;\n\t"
        "mbarrier.arrive.shared::cta.b64 st, [%0];\n\t"
        "}\n" ::"r"(tc::smem_u32(bar))
        : "memory");
}

__device__ __forceinline__ unsigned long long ws_now() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Wait for a phase of an mbarrier; gives up when another role has raised the abort word, after 2 s of wall time or
// after 2^24 polls, whichever comes first.
__device__ __forceinline__ bool ws_wait(uint64_t *bar, uint32_t parity, volatile int *abort_word) {
    if (tc::mbar_wait(bar, parity, 64)) return true;
    const unsigned long long t0 = ws_now();
    for (uint32_t it = 0; it < (1u << 16); ++it) {
        if (tc::mbar_wait(bar, parity, 256)) return true;
        if (*abort_word) return false;
        if (ws_now() - t0 > 2000000000ull) return false;
    }
    return false;
}

__device__ __forceinline__ void ws_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile(
        "{\n\t"
        ".reg .b64 st;\n\t"
        "mbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1;\n\t"
        "}\n" ::"r"(tc::smem_u32(bar)), "r"(bytes)
        : "memory");
}

// One tiled 2-D bulk copy global -> shared (this CTA's own shared memory), completion bytes counted on `bar`.
__device__ __forceinline__ void ws_tma_load_2d(uint32_t dst, const CUtensorMap *map, int c0, int c1, uint64_t *bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
                 "l"(map), "r"(c0), "r"(c1), "r"(tc::smem_u32(bar))
                 : "memory");
}

// One tiled 2-D bulk copy shared -> global; rows / columns outside the tensor are not written.
__device__ __forceinline__ void ws_tma_store_2d(const CUtensorMap *map, int c0, int c1, uint32_t src) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%1, %2}], [%3];" ::"l"(map), "r"(c0), "r"(c1), "r"(src)
                 : "memory");
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}

// Barrier of `count` threads that also ANDs a predicate over them: every participant learns whether all of them are fine.
__device__ __forceinline__ bool ws_bar_and(int id, int count, bool pred) {
    uint32_t r;
    asm volatile(
        "{\n\t"
        ".reg .pred p, q;\n\t"
        "setp.ne.b32 p, %3, 0;\n\t"
        "bar.red.and.pred q, %1, %2, p;\n\t"
        "selp.u32 %0, 1, 0, q;\n\t"
        "}\n"
        : "=r"(r)
        : "r"(id), "r"(count), "r"(pred ? 1u : 0u)
        : "memory");
    return r != 0;
}

__device__ __forceinline__ int ws_swz(int r, int C) { return C == 8 ? (r & 7) : (C == 4 ? ((r >> 1) & 3) : ((r >> 2) & 1)); }

template <bool RCONV, int AMAX, int NPW, int EW, bool TMA>
__global__ void __launch_bounds__((NPW + EW + 1 + (TMA ? 1 : 0)) * 32, 1) k_qdense_fwd_ws(const WsParams P,
                                                                                       const __grid_constant__ CUtensorMap tmap,
                                                                                       const __grid_constant__ CUtensorMap tmap_y) {
    constexpr int kWsProdWarps = NPW, kWsProd = NPW * 32, kWsEpiWarps = EW, kWsIssueWarp = NPW + EW;
    constexpr int kWsLoadWarp = NPW + EW + 1;  // TMA only
    constexpr int ITS = 32 / NPW;       // 8-row groups a producer thread converts per slab
    constexpr int ROWSTEP = NPW * 4;    // their distance in rows
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char *smem = smem_raw + ((1024u - (tc::smem_u32(smem_raw) & 1023u)) & 1023u);  // the carve starts on a 1 KB boundary
    // carve: operand stages | raw-slab slots | transposition buffers | B terms | bias | exponent table | abs-max table |
    // barriers, TMEM slot, flags
    unsigned char *A = smem;
    unsigned char *fetch = A + 2 * kWsStageBytes;
    unsigned char *outst = fetch + P.depth * kWsFetchBytes;
    unsigned char *B = outst + EW * kWsOutWarpBytes;
    const int b_term_bytes = P.Kpad * P.Npad * 2;
    float *bias_s = reinterpret_cast<float *>(B + 3 * b_term_bytes);
    const int Ke = P.Kt + 8;  // row stride of the exponent table: 8-byte reads of 8 rows hit 8 bank pairs
    const int tab_bytes = (P.rows_period * Ke + 15) / 16 * 16;
    unsigned char *etab = reinterpret_cast<unsigned char *>(bias_s + P.Npad);
    const int Ks = (AMAX == WS_AMAX_REGS2X2) ? P.Kt : P.Kt + 4;  // abs-max table row: 16-byte accesses of 8 rows hit 8 bank groups
    // PLAIN keeps the abs-max table beside the exponent table; the register modes merge through the raw-slab slots, which
    // are idle by then
    constexpr bool amax_regs = (AMAX == WS_AMAX_REGS1 || AMAX == WS_AMAX_REGS2 || AMAX == WS_AMAX_REGS2X2);
    const int amax_elems = (AMAX == WS_AMAX_PLAIN) ? P.rows_period * Ks : 0;
    float *amax_t = amax_regs ? reinterpret_cast<float *>(fetch) : reinterpret_cast<float *>(etab + tab_bytes);
    uint64_t *full = reinterpret_cast<uint64_t *>(etab + tab_bytes + amax_elems * 4);
    uint64_t *empty = full + 2, *acc_full = full + 4, *acc_empty = full + 6;
    uint64_t *raw_full = full + 8, *raw_empty = full + 10;  // TMA only: a raw slab has landed / has been read by every producer
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(full + 12);
    int *dirty3 = reinterpret_cast<int *>(tmem_slot + 1);  // per stage: some tile needed the third term (sticky)
    int *abort_word = dirty3 + 2;
    float *pool_s = reinterpret_cast<float *>(abort_word + 2);  // row-group sums only: [2 column parts][4 warps][32] floats

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int K = P.K, N = P.N, Kpad = P.Kpad, Npad = P.Npad;
    const uint32_t tmem_cols = 2 * Npad < 32 ? 32u : (uint32_t)(2 * Npad);  // two accumulators; Npad is a power of two

    // ---- one-time set-up (all threads) -------------------------------------------------------------------------------
    if (tid == 0) {
        for (int s = 0; s < 2; ++s) {
            tc::mbar_init(full + s, kWsProdWarps);  // one arrival per producer warp
            tc::mbar_init(empty + s, 1);      // tcgen05.commit
            tc::mbar_init(acc_full + s, 1);   // tcgen05.commit
            tc::mbar_init(acc_empty + s, kWsEpiWarps);  // one arrival per epilogue warp
            tc::mbar_init(raw_full + s, 1);             // the loader's expect_tx arrival (+ the copies' bytes)
            tc::mbar_init(raw_empty + s, kWsProdWarps);
            dirty3[s] = 0;
        }
        *abort_word = 0;
        tc::mbar_init_fence();
        if (TMA && (tc::smem_u32(fetch) & 1023u) != 0) {  // the swizzled copies need a 1 KB aligned destination
            *abort_word = 1;
            if (P.status) atomicOr(P.status, kWsTimeout);
        }
    }
    // The loader warp (TMA variant) takes no part in the conversions below: once the barriers exist it has the copy engine
    // fetch the CTA's first `depth` slabs, so that the copies fly while the other warps convert the weights (on a launch of
    // one tile per CTA -- small batches -- that is a microsecond or more of the launch's length).
    constexpr int kSetupThreads = (NPW + EW + 1) * 32;  // the last warp is the loader
    const int n_chunks = (Kpad + kWsKC - 1) / kWsKC;
    auto fetch_slab = [&](int64_t tile, int ch, uint32_t rb) {
        const int c0 = ch * kWsKC;
        const int halves = (K - c0 > 32) ? 2 : 1;  // a column half that lies past K is not fetched at all
        ws_expect_tx(raw_full + rb, (uint32_t)(halves * (kWsFetchBytes / 2)));
        const uint32_t dst = tc::smem_u32(fetch) + rb * kWsFetchBytes;
        for (int hcol = 0; hcol < halves; ++hcol)
            ws_tma_load_2d(dst + hcol * (kWsFetchBytes / 2), &tmap, c0 + hcol * 32, (int)(tile * kWsTileM), raw_full + rb);
    };
    const bool is_loader = TMA && warp == kWsLoadWarp;
    if (TMA) {
        __syncthreads();  // the barriers are initialised, the abort word is set
        if (is_loader && lane == 0 && *reinterpret_cast<volatile int *>(abort_word) == 0) {
            uint32_t n = 0;
            for (int64_t tile = blockIdx.x; tile < P.num_tiles && n < (uint32_t)P.depth; tile += gridDim.x)
                for (int ch = 0; ch < n_chunks && n < (uint32_t)P.depth; ++ch, ++n) fetch_slab(tile, ch, P.depth == 2 ? (n & 1u) : 0u);
        }
    }
    if (warp == kWsIssueWarp) tc::tmem_alloc(tmem_slot, tmem_cols);
    for (int e = tid; e < Npad && !is_loader; e += kSetupThreads) bias_s[e] = (P.bq != nullptr && e < N) ? __ldg(P.bq + e) : 0.f;
    for (int e = tid; e < amax_elems && !is_loader; e += kSetupThreads) amax_t[e] = 0.f;
    for (int e = tid; e < P.rows_period * P.Kt && !is_loader; e += kSetupThreads) {
        const int pr = e / P.Kt, k = e % P.Kt;
        const int fi = (k < K) ? __float2int_rn(__ldg(P.qf + pr * K + k)) : 0;
        etab[pr * Ke + k] = (unsigned char)(max(-126, min(127, fi)) + 127);
    }
    // the third-term buffers hold zeros until a tile needs them
    for (int s = 0; s < 2; ++s)
        for (int e = tid; e < kWsTermBytes / 16 && !is_loader; e += kSetupThreads)
            reinterpret_cast<uint4 *>(A + s * kWsStageBytes + 2 * kWsTermBytes)[e] = make_uint4(0, 0, 0, 0);
    // weights: fp32 [K, N] -> up to three bf16 terms, K-major core matrices: (n/8, k/8) -> 128-byte block
    int w_lo = 0, w_lo2 = 0;
    for (int e = tid; e < Kpad * Npad && !is_loader; e += kSetupThreads) {
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

    if (warp < kWsProdWarps) {
        // ================================ producers ==================================================================
        // slab mapping: lane = (q4, r8); warp w in iteration it handles row group mg = (it * NPW + w) / 2 and the 8-column
        // group kg = (w & 1) * 4 + q4.  A quarter-warp (r8 = 0..7) fills one 128-byte core matrix.
        const int r8 = lane & 7, q4 = lane >> 3;
        const int kg = (warp & 1) * 4 + q4;
        const float rbias = (P.rm == RM_RND) ? 0.5f : 0.f;
        const uint32_t fetch_base = tc::smem_u32(fetch);
        // Requests run `depth` slabs ahead of the conversion; every request closes one cp.async group (an empty one past
        // the last slab), so "all but the newest depth - 1 groups have landed" always means "this slab has landed".
        const int depth = P.depth;
        int64_t pf_tile = blockIdx.x;
        int pf_ch = 0;
        uint32_t pf_n = 0;
        auto request = [&]() {
            if (pf_tile < P.num_tiles) {
                const int k0 = pf_ch * kWsKC + kg * 8;
                const uint32_t buf = fetch_base + (depth == 2 ? (pf_n & 1u) : 0u) * kWsFetchBytes;
#pragma unroll
                for (int it = 0; it < ITS; ++it) {
                    const int64_t row = pf_tile * kWsTileM + it * ROWSTEP + (warp >> 1) * 8 + r8;
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const bool in = row < P.M && (k0 + 4 * h) < K;  // K % 4 == 0: a 16-byte piece is all inside or all outside
                        const float *src = in ? P.x + row * K + k0 + 4 * h : P.x;
                        const uint32_t dst = buf + (uint32_t)(((it * 2 + h) * kWsProd + tid) * 16);
                        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(in ? 16 : 0) : "memory");
                    }
                }
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
            if (++pf_ch == n_chunks) { pf_ch = 0; pf_tile += gridDim.x; }
            ++pf_n;
        };
        if (!TMA)
            for (int d = 0; d < depth; ++d) request();
        // where this thread finds its unit of iteration it in a slab the copy engine wrote: column half kg / 4 (one 16 KB
        // copy each), row it * ROWSTEP + (warp / 2) * 8 + r8 of 128 bytes, 16-byte chunk XOR (row & 7) = r8 (128-byte swizzle)
        const int tma_rd0 = (kg >> 2) * (kWsFetchBytes / 2) + ((warp >> 1) * 8 + r8) * 128 + ((((kg & 3) * 2) ^ r8) * 16);
        const int tma_rd1 = (kg >> 2) * (kWsFetchBytes / 2) + ((warp >> 1) * 8 + r8) * 128 + ((((kg & 3) * 2 + 1) ^ r8) * 16);

        const uint32_t rp = (uint32_t)P.rows_period;
        const bool rp_pow2 = (rp & (rp - 1)) == 0;
        uint32_t base_pr = (uint32_t)(((int64_t)blockIdx.x * kWsTileM) % P.rows_period);
        const uint32_t step_pr = (uint32_t)(((int64_t)gridDim.x * kWsTileM) % P.rows_period);
        float amax_r[2][8], amax_x[2][8];  // amax_x: the second K slab (REGS2X2)
#pragma unroll
        for (int j = 0; j < 8; ++j) amax_r[0][j] = amax_r[1][j] = amax_x[0][j] = amax_x[1][j] = 0.f;

        uint32_t n = 0;  // slabs produced so far
        bool ok = true;
        for (int64_t tile = blockIdx.x; tile < P.num_tiles && ok; tile += gridDim.x, base_pr = (base_pr + step_pr) % rp) {
            for (int ch = 0; ch < n_chunks && ok; ++ch, ++n) {
                const int s = (int)(n & 1u);
                const uint32_t use = n >> 1;
                unsigned char *As = A + s * kWsStageBytes;
                float xv[ITS][8];
                if (TMA) {
                    const uint32_t rb = depth == 2 ? (n & 1u) : 0u, ruse = depth == 2 ? (n >> 1) : n;
                    const bool w = ws_wait(raw_full + rb, ruse & 1u, abort_word);
                    if (!__all_sync(0xffffffffu, w)) { ok = false; break; }
                    const unsigned char *buf = fetch + rb * kWsFetchBytes;
                    const bool col_in = ch * kWsKC + kg * 8 < K;  // a column half the loader did not fetch holds nothing
#pragma unroll
                    for (int it = 0; it < ITS; ++it) {
                        const float4 v0 = *reinterpret_cast<const float4 *>(buf + it * ROWSTEP * 128 + tma_rd0);
                        const float4 v1 = *reinterpret_cast<const float4 *>(buf + it * ROWSTEP * 128 + tma_rd1);
                        xv[it][0] = col_in ? v0.x : 0.f; xv[it][1] = col_in ? v0.y : 0.f; xv[it][2] = col_in ? v0.z : 0.f;
                        xv[it][3] = col_in ? v0.w : 0.f; xv[it][4] = col_in ? v1.x : 0.f; xv[it][5] = col_in ? v1.y : 0.f;
                        xv[it][6] = col_in ? v1.z : 0.f; xv[it][7] = col_in ? v1.w : 0.f;
                    }
                    __syncwarp();  // every lane holds its units in registers: the slab buffer may be refilled
                    if (lane == 0) ws_arrive(raw_empty + rb);
                } else {
                    if (depth == 2) asm volatile("cp.async.wait_group 1;" ::: "memory");
                    else asm volatile("cp.async.wait_group 0;" ::: "memory");
                    const unsigned char *buf = fetch + (depth == 2 ? (n & 1u) : 0u) * kWsFetchBytes;
#pragma unroll
                    for (int it = 0; it < ITS; ++it) {
                        const float4 v0 = *reinterpret_cast<const float4 *>(buf + ((it * 2 + 0) * kWsProd + tid) * 16);
                        const float4 v1 = *reinterpret_cast<const float4 *>(buf + ((it * 2 + 1) * kWsProd + tid) * 16);
                        xv[it][0] = v0.x; xv[it][1] = v0.y; xv[it][2] = v0.z; xv[it][3] = v0.w;
                        xv[it][4] = v1.x; xv[it][5] = v1.y; xv[it][6] = v1.z; xv[it][7] = v1.w;
                    }
                    request();  // the slots just read are free again (their contents sit in registers)
                }
                // the products that read this stage two slabs ago must have completed (they were issued a whole slab ago)
                if (use > 0) {
                    const bool w = ws_wait(empty + s, (use - 1) & 1u, abort_word);
                    if (!__all_sync(0xffffffffu, w)) { ok = false; break; }
                }
                // third term: values with more than 16 significant bits.  Once a stage has carried one, every thread
                // rewrites its part of the stage's third buffer on every slab (zeros where it has none); until then the
                // buffer holds the zeros of the set-up and the issuing warp skips it.
                int d3 = *reinterpret_cast<volatile int *>(dirty3 + s);
                const int k0 = ch * kWsKC + kg * 8;
#pragma unroll
                for (int it = 0; it < ITS; ++it) {
                    const int lrow = it * ROWSTEP + (warp >> 1) * 8 + r8;
                    const bool valid = (tile * kWsTileM + lrow) < P.M && k0 < K;
                    if (valid) {
                        const uint32_t lr = base_pr + (uint32_t)lrow;
                        const int pr = (int)(rp_pow2 ? (lr & (rp - 1)) : (lr % rp));
                        const uint2 eb = *reinterpret_cast<const uint2 *>(etab + pr * Ke + k0);
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            const uint32_t sbits = (((j < 4 ? eb.x : eb.y) >> ((j & 3) * 8)) & 0xffu) << 23;  // 2^f
                            // scaling by a power of two is exact, so one fused multiply-add gives RN(x * 2^f + bias) bit for bit
                            const float q = RCONV ? rintf(__fmul_rn(xv[it][j], __uint_as_float(sbits)))
                                                  : floorf(__fmaf_rn(xv[it][j], __uint_as_float(sbits), rbias));
                            xv[it][j] = __fmul_rn(q, __uint_as_float(0x7F000000u - sbits));  // * 2^-f
                        }
                        if (AMAX == WS_AMAX_REGS2X2) {
                            const int ri = it & 1;
                            if (ch == 0) {
#pragma unroll
                                for (int j = 0; j < 8; ++j) amax_r[ri][j] = fmaxf(amax_r[ri][j], fabsf(xv[it][j]));
                            } else {
#pragma unroll
                                for (int j = 0; j < 8; ++j) amax_x[ri][j] = fmaxf(amax_x[ri][j], fabsf(xv[it][j]));
                            }
                        } else if (AMAX == WS_AMAX_REGS1 || AMAX == WS_AMAX_REGS2) {
                            const int ri = (AMAX == WS_AMAX_REGS2) ? (it & 1) : 0;  // REGS2: the table row alternates with it
#pragma unroll
                            for (int j = 0; j < 8; ++j) amax_r[ri][j] = fmaxf(amax_r[ri][j], fabsf(xv[it][j]));
                        } else if (AMAX == WS_AMAX_PLAIN) {
                            const int te = pr * Ks + k0;
                            float4 m0 = *reinterpret_cast<float4 *>(amax_t + te), m1 = *reinterpret_cast<float4 *>(amax_t + te + 4);
                            m0.x = fmaxf(m0.x, fabsf(xv[it][0])); m0.y = fmaxf(m0.y, fabsf(xv[it][1]));
                            m0.z = fmaxf(m0.z, fabsf(xv[it][2])); m0.w = fmaxf(m0.w, fabsf(xv[it][3]));
                            m1.x = fmaxf(m1.x, fabsf(xv[it][4])); m1.y = fmaxf(m1.y, fabsf(xv[it][5]));
                            m1.z = fmaxf(m1.z, fabsf(xv[it][6])); m1.w = fmaxf(m1.w, fabsf(xv[it][7]));
                            *reinterpret_cast<float4 *>(amax_t + te) = m0;
                            *reinterpret_cast<float4 *>(amax_t + te + 4) = m1;
                        }
                    }
                    // exact bf16 terms: a float whose low 16 bits are zero *is* a bf16 (top 16 bits), the common case
                    uint32_t hi[4], lo[4] = {0u, 0u, 0u, 0u}, t3[4] = {0u, 0u, 0u, 0u};
                    uint32_t lowbits = 0u;
#pragma unroll
                    for (int j = 0; j < 8; ++j) lowbits |= __float_as_uint(xv[it][j]);
                    if ((lowbits & 0xFFFFu) == 0u) {
#pragma unroll
                        for (int j = 0; j < 8; j += 2)
                            hi[j >> 1] = __byte_perm(__float_as_uint(xv[it][j]), __float_as_uint(xv[it][j + 1]), 0x7632);
                    } else {
                        int need3 = 0;
#pragma unroll
                        for (int j = 0; j < 8; j += 2) {
                            __nv_bfloat16 h0, l0, m0, h1, l1, m1;
                            tc::split3(xv[it][j], h0, l0, m0);
                            tc::split3(xv[it][j + 1], h1, l1, m1);
                            hi[j >> 1] = tc::pack2(h0, h1);
                            lo[j >> 1] = tc::pack2(l0, l1);
                            t3[j >> 1] = tc::pack2(m0, m1);
                            need3 |= (t3[j >> 1] & 0x7fff7fffu) != 0;
                        }
                        if (need3 && !d3) { atomicOr(dirty3 + s, 1); d3 = 1; }
                    }
                    const int off = (lrow >> 3) * 1024 + kg * 128 + r8 * 16;
                    *reinterpret_cast<uint4 *>(As + off) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
                    *reinterpret_cast<uint4 *>(As + kWsTermBytes + off) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
                    if (d3) *reinterpret_cast<uint4 *>(As + 2 * kWsTermBytes + off) = make_uint4(t3[0], t3[1], t3[2], t3[3]);
                }
                tc::fence_smem_to_async();
                __syncwarp();
                if (lane == 0) ws_arrive(full + s);
            }
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        if (!ok) {
            *reinterpret_cast<volatile int *>(abort_word) = 1;
            if (lane == 0 && P.status) atomicOr(P.status, kWsTimeout);
        }
        // ---- abs-max partials of this CTA -----------------------------------------------------------------------------
        if (AMAX != WS_AMAX_NONE) {
            if (amax_regs) {
                asm volatile("bar.sync 1, %0;" ::"n"(kWsProd) : "memory");  // every producer is done with the raw-slab slots
                for (int e = tid; e < P.rows_period * Ks; e += kWsProd) amax_t[e] = 0.f;
                asm volatile("bar.sync 1, %0;" ::"n"(kWsProd) : "memory");
#pragma unroll
                for (int ri = 0; ri < ((AMAX == WS_AMAX_REGS2 || AMAX == WS_AMAX_REGS2X2) ? 2 : 1); ++ri) {
                    const int pr = (ri * ROWSTEP + (warp >> 1) * 8 + r8) % P.rows_period;
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        if (kg * 8 + j < K) atomicMax(reinterpret_cast<unsigned *>(amax_t) + pr * Ks + kg * 8 + j, __float_as_uint(amax_r[ri][j]));
                    if (AMAX == WS_AMAX_REGS2X2) {
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            if (kWsKC + kg * 8 + j < K)
                                atomicMax(reinterpret_cast<unsigned *>(amax_t) + pr * Ks + kWsKC + kg * 8 + j, __float_as_uint(amax_x[ri][j]));
                    }
                }
            }
            asm volatile("bar.sync 1, %0;" ::"n"(kWsProd) : "memory");
            const int table = P.rows_period * K;
            if (P.amax_direct) {
                for (int e = tid; e < table; e += kWsProd) {
                    const unsigned v = __float_as_uint(amax_t[(e / K) * Ks + (e % K)]);
                    if (v != 0u) atomicMax(P.amax_part + e, v);
                }
            } else {
                unsigned *dst = P.amax_part + (int64_t)blockIdx.x * table;
                for (int e = tid; e < table; e += kWsProd) dst[e] = __float_as_uint(amax_t[(e / K) * Ks + (e % K)]);
            }
        }
    } else if (warp == kWsIssueWarp) {
        // ================================ tensor-core issue ==========================================================
        // The whole warp walks the loop (so that it stays converged for the barriers of the tear-down); lane 0 issues.
        const uint32_t idesc = tc::make_idesc_bf16(Npad, false, false);
        const uint32_t a_base = tc::smem_u32(A), b_base = tc::smem_u32(B);
        const uint32_t sbo_a = (kWsKC / 8) * 128, sbo_b = (uint32_t)(Kpad >> 3) * 128;
        uint32_t n = 0, ti = 0;
        bool ok = true;
        for (int64_t tile = blockIdx.x; tile < P.num_tiles && ok; tile += gridDim.x, ++ti) {
            const uint32_t a = ti & 1u, ause = ti >> 1;
            for (int ch = 0; ch < n_chunks && ok; ++ch, ++n) {
                const uint32_t s = n & 1u, use = n >> 1;
                bool w = ws_wait(full + s, use & 1u, abort_word);
                // the epilogue must have drained this accumulator (tile ti - 2) before the first product overwrites it
                if (w && ch == 0 && ause > 0) w = ws_wait(acc_empty + a, (ause - 1) & 1u, abort_word);
                if (!__all_sync(0xffffffffu, w)) { ok = false; break; }
                tc::fence_after_sync();
                if (lane == 0) {
                    const int n_a = *reinterpret_cast<volatile int *>(dirty3 + s) ? 3 : 2;
                    const int kleft = Kpad - ch * kWsKC;
                    const int ksteps = (kleft < kWsKC ? kleft : kWsKC) / 16;
                    const uint32_t tacc = tmem_base + a * (uint32_t)Npad;
                    bool first = (ch == 0);
                    for (int ks = 0; ks < ksteps; ++ks) {
                        uint64_t da = tc::make_smem_desc(a_base + s * kWsStageBytes + ks * 256, 128, sbo_a);
                        for (int ta = 0; ta < n_a; ++ta, da += (uint64_t)(kWsTermBytes >> 4)) {
                            uint64_t db = tc::make_smem_desc(b_base + (ch * (kWsKC / 16) + ks) * 256, 128, sbo_b);
                            for (int tw = 0; tw < n_w; ++tw, db += (uint64_t)(b_term_bytes >> 4)) {
                                tc::mma_bf16(tacc, da, db, idesc, !first);
                                first = false;
                            }
                        }
                    }
                    tc::commit(empty + s);
                    if (ch == n_chunks - 1) tc::commit(acc_full + a);
                }
                __syncwarp();
            }
        }
        if (!ok) {
            *reinterpret_cast<volatile int *>(abort_word) = 1;
            if (lane == 0 && P.status) atomicOr(P.status, kWsTimeout);
        }
    } else if (TMA && warp == kWsLoadWarp) {
        // ================================ bulk-copy loader (TMA variant) ===========================================
        // One thread keeps `depth` raw slabs in flight: it waits until every producer warp has taken its units out of a slab
        // buffer, then has the copy engine fetch the next slab into it.  The whole warp walks the loop (it stays converged
        // for the tear-down barrier); lane 0 issues.
        const int depth = P.depth;
        const uint32_t fetch_base = tc::smem_u32(fetch);
        uint32_t n = 0;
        bool ok = *reinterpret_cast<volatile int *>(abort_word) == 0;
        for (int64_t tile = blockIdx.x; tile < P.num_tiles && ok; tile += gridDim.x) {
            for (int ch = 0; ch < n_chunks && ok; ++ch, ++n) {
                const uint32_t rb = depth == 2 ? (n & 1u) : 0u, ruse = depth == 2 ? (n >> 1) : n;
                if (ruse == 0) continue;  // the first `depth` slabs were requested during the set-up
                const bool w = ws_wait(raw_empty + rb, (ruse - 1) & 1u, abort_word);
                if (!__all_sync(0xffffffffu, w)) { ok = false; break; }
                if (lane == 0) fetch_slab(tile, ch, rb);
                __syncwarp();
            }
        }
        if (!ok) {
            *reinterpret_cast<volatile int *>(abort_word) = 1;
            if (lane == 0 && P.status) atomicOr(P.status, kWsTimeout);
        }
    } else {
        // ================================ epilogue ===================================================================
        // Warp e reads TMEM lanes 32 (e & 3) .. + 31 (the rows of the tile it owns); with eight warps the column pieces
        // alternate between the two warps of a lane quarter.  wc columns per tcgen05.ld.
        const int e = warp - kWsProdWarps, q = e & 3, part = e >> 2;
        constexpr int NPARTS = EW / 4;
        float *ost = reinterpret_cast<float *>(outst + e * kWsOutWarpBytes);  // 32 rows x wc floats
        const int wc = (Npad / NPARTS) < 32 ? (Npad / NPARTS) : 32, C = wc >> 2;
        const int swz_w = ws_swz(lane, C);
        const int last_c0 = Npad - wc * (NPARTS - part);  // this warp's last piece
        const float act_lo = (P.act == ACT_RELU) ? 0.f : -INFINITY;
        const bool vec_out = (N % 4 == 0) && aligned(P.y, 16);
        uint32_t ti = 0;
        bool ok = true;
        // With bulk stores (tma_store, wc = 32): the four warps that share `part` fill one 128-row x 32-column block in
        // shared memory (128-byte rows, 16-byte chunks XOR-swizzled with the row) and one of their threads hands it to the
        // copy engine; a block is reused once the previous store has read it.  The four warps meet at a named barrier that
        // also carries each warp's wait outcome, so that all of them leave the loop together if a wait gave up.
        const bool tstore = P.tma_store != 0;
        unsigned char *box = outst + part * 16384;
        const bool leader = (q == 0 && lane == 0);
        const int row_t = q * 32 + lane;
        for (int64_t tile = blockIdx.x; tile < P.num_tiles && ok; tile += gridDim.x, ++ti) {
            const uint32_t a = ti & 1u, ause = ti >> 1;
            bool w = ws_wait(acc_full + a, ause & 1u, abort_word);
            w = __all_sync(0xffffffffu, w);
            if (tstore) {
                if (leader) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");  // the block's last store has read it
                w = ws_bar_and(3 + part, 128, w);
            }
            if (!w) { ok = false; break; }
            tc::fence_after_sync();
            const int64_t wrow0 = tile * kWsTileM + q * 32;  // first row of this warp
            const int rows_w = (int)((P.M - wrow0) < 32 ? ((P.M - wrow0) < 0 ? 0 : (P.M - wrow0)) : 32);
            for (int c0 = part * wc; c0 < Npad; c0 += NPARTS * wc) {
                float v[32];
                const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + a * (uint32_t)Npad + (uint32_t)c0;
                if (wc == 32) tc::tmem_ld32v(taddr, v);
                else if (wc == 16) tc::tmem_ld16v(taddr, v);
                else tc::tmem_ld8v(taddr, v);
                if (c0 == last_c0) {  // the accumulator is in registers: hand it back to the issuing warp
                    tc::fence_before_sync();
                    __syncwarp();
                    if (lane == 0) ws_arrive(acc_empty + a);
                }
                if (tstore) {
                    if (c0 != part * wc) {  // a later piece of the same tile: wait for the store of the previous one
                        if (leader) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                        asm volatile("bar.sync %0, 128;" ::"r"(3 + part) : "memory");
                    }
#pragma unroll
                    for (int j = 0; j < 32; j += 4) {
                        const float4 b = *reinterpret_cast<const float4 *>(bias_s + c0 + j);
                        float4 o;
                        o.x = fmaxf(__fadd_rn(v[j], b.x), act_lo); o.y = fmaxf(__fadd_rn(v[j + 1], b.y), act_lo);
                        o.z = fmaxf(__fadd_rn(v[j + 2], b.z), act_lo); o.w = fmaxf(__fadd_rn(v[j + 3], b.w), act_lo);
                        *reinterpret_cast<float4 *>(box + row_t * 128 + (((j >> 2) ^ (lane & 7)) << 4)) = o;
                    }
                    tc::fence_smem_to_async();
                    asm volatile("bar.sync %0, 128;" ::"r"(3 + part) : "memory");
                    if (leader) ws_tma_store_2d(&tmap_y, c0, (int)(tile * kWsTileM), tc::smem_u32(box));
                    // Sum over groups of pool_rows consecutive rows (the reduction over an axis that follows the layer), from
                    // the finished block while the copy engine reads it.  lane = column; every warp adds its own 32 rows
                    // (four interleaved partial sums, combined as (a0 + a1) + (a2 + a3): a fixed order; one row of the block
                    // per load: 32 lanes read 32 different words of a 128-byte row, whatever the chunk swizzle).  Groups of 64
                    // or 128 rows: the warps of a group leave their sums in shared memory, meet at a named barrier, and the
                    // group's first warp adds them in ascending row order.  Groups never straddle the end of y (M is a
                    // multiple of pool_rows), so a group is written iff its first row exists.
                    if (P.pool_out != nullptr) {
                        float a4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                        for (int rr = 0; rr < 32; ++rr) {
                            const int r = q * 32 + rr;
                            a4[rr & 3] = __fadd_rn(a4[rr & 3], *reinterpret_cast<const float *>(box + r * 128 + ((((lane >> 2) ^ (r & 7)) << 4) | ((lane & 3) << 2))));
                        }
                        float sum = __fadd_rn(__fadd_rn(a4[0], a4[1]), __fadd_rn(a4[2], a4[3]));
                        const int wpg = P.pool_rows >> 5;  // warps per group: 1, 2 or 4
                        if (wpg > 1) {
                            float *slot = pool_s + part * 128;
                            slot[q * 32 + lane] = sum;
                            if (wpg == 2) asm volatile("bar.sync %0, 64;" ::"r"(5 + part * 2 + (q >> 1)) : "memory");
                            else asm volatile("bar.sync %0, 128;" ::"r"(3 + part) : "memory");
                            if ((q & (wpg - 1)) == 0) {
                                sum = slot[q * 32 + lane];
                                for (int k2 = 1; k2 < wpg; ++k2) sum = __fadd_rn(sum, slot[(q + k2) * 32 + lane]);
                            }
                        }
                        const int64_t grow = tile * kWsTileM + q * 32;
                        if ((q & (wpg - 1)) == 0 && grow < P.M && c0 + lane < N)
                            P.pool_out[(grow / P.pool_rows) * N + c0 + lane] = __fmul_rn(sum, P.pool_scale);
                    }
                    continue;
                }
#pragma unroll
                for (int j = 0; j < 32; j += 4) {
                    if (j < wc) {
                        const float4 b = *reinterpret_cast<const float4 *>(bias_s + c0 + j);
                        float4 o;
                        o.x = fmaxf(__fadd_rn(v[j], b.x), act_lo); o.y = fmaxf(__fadd_rn(v[j + 1], b.y), act_lo);
                        o.z = fmaxf(__fadd_rn(v[j + 2], b.z), act_lo); o.w = fmaxf(__fadd_rn(v[j + 3], b.w), act_lo);
                        *reinterpret_cast<float4 *>(ost + lane * wc + (((j >> 2) ^ swz_w) << 2)) = o;
                    }
                }
                __syncwarp();
                const int my_n = (N - c0) < wc ? ((N - c0) < 0 ? 0 : (N - c0)) : wc;  // valid columns of the piece
                float *ydst = P.y + wrow0 * N + c0;
                if (vec_out) {
                    const int cv = my_n >> 2;
                    const int total = rows_w * cv;
                    if (cv == 8) {
                        for (int g = lane; g < total; g += 32) {
                            const int rr = g >> 3, c4 = g & 7;
                            const float4 o = *reinterpret_cast<const float4 *>(ost + rr * wc + ((c4 ^ ws_swz(rr, C)) << 2));
                            __stcs(reinterpret_cast<float4 *>(ydst + (int64_t)rr * N) + c4, o);
                        }
                    } else {
                        for (int g = lane; g < total; g += 32) {
                            const int rr = g / cv, c4 = g - rr * cv;
                            const float4 o = *reinterpret_cast<const float4 *>(ost + rr * wc + ((c4 ^ ws_swz(rr, C)) << 2));
                            __stcs(reinterpret_cast<float4 *>(ydst + (int64_t)rr * N) + c4, o);
                        }
                    }
                } else {
                    const int total = rows_w * my_n;
                    for (int g = lane; g < total; g += 32) {
                        const int rr = g / my_n, c = g - rr * my_n;
                        __stcs(ydst + (int64_t)rr * N + c, ost[rr * wc + ((((c >> 2) ^ ws_swz(rr, C)) << 2) | (c & 3))]);
                    }
                }
                __syncwarp();  // the transposition buffer is reused by the next piece / the next tile
            }
        }
        if (tstore && leader) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");  // every store of this CTA has landed
        if (!ok) {
            *reinterpret_cast<volatile int *>(abort_word) = 1;
            if (lane == 0 && P.status) atomicOr(P.status, kWsTimeout);
        }
    }

    // ---- tear-down ----------------------------------------------------------------------------------------------------
    tc::fence_before_sync();
    __syncthreads();
    if (warp == kWsIssueWarp) tc::tmem_dealloc(tmem_base, tmem_cols);
}

static size_t qdense_ws_smem(int Kpad, int Npad, int Kt, int rows_period, bool amax_table, int depth, int ew) {
    const size_t tab_bytes = ((size_t)rows_period * (Kt + 8) + 15) / 16 * 16;
    return 2 * (size_t)kWsStageBytes + (size_t)depth * kWsFetchBytes + (size_t)ew * kWsOutWarpBytes + 3 * (size_t)Kpad * Npad * 2 +
           (size_t)Npad * 4 + tab_bytes + (amax_table ? (size_t)rows_period * (Kt + 4) * 4 : 0) + 12 * 8 + 32;
}

// cuTensorMapEncodeTiled through the runtime's driver entry point query (the library does not link against libcuda)
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_tiled_fn() {
    static const EncodeTiledFn fn = [] {
        void *ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess) {
            cudaGetLastError();
            return (EncodeTiledFn) nullptr;
        }
        return (EncodeTiledFn)ptr;
    }();
    return fn;
}

// HGQ_QDENSE_TMA=0 / 1 in the environment picks how raw slabs are fetched (thread-private cp.async / bulk tensor copies).
static bool ws_tma_enabled() {
    static const bool on = [] {
        const char *v = getenv("HGQ_QDENSE_TMA");
        return v != nullptr ? v[0] != '0' : true;  // measured faster on every layer shape of the training workloads
    }();
    return on;
}

// HGQ_QDENSE_TMA_STORE=0 / 1: the epilogue writes y through its transposition buffers / through bulk tensor stores.
static bool ws_tma_store_enabled() {
    static const bool on = [] {
        const char *v = getenv("HGQ_QDENSE_TMA_STORE");
        return v != nullptr ? v[0] != '0' : true;  // measured faster on every layer shape of the training workloads
    }();
    return on;
}

// A tensor map over x [M, K] fp32 (this GPU's memory only): boxes of 128 rows x 32 floats, 128-byte swizzle, zeros outside.
static bool ws_make_tmap(CUtensorMap *map, const float *x, int64_t M, int K) {
    const EncodeTiledFn enc = encode_tiled_fn();
    if (enc == nullptr) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)M};
    const cuuint64_t strides[1] = {(cuuint64_t)K * 4};
    const cuuint32_t box[2] = {32, (cuuint32_t)kWsTileM};
    const cuuint32_t estr[2] = {1, 1};
    return enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float *>(x), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Warp split: 8 producer and 8 epilogue warps.  Measured on the particle-layer shape (ms per launch): 8/8 0.53, 16/8 0.63,
// 8/4 0.77, 16/4 0.80 -- more producer warps cost registers and add per-warp overhead, fewer epilogue warps fall behind.
constexpr int kWsNpw = 8, kWsEw = 8;

// Abs-max bookkeeping mode, raw slabs in flight and shared-memory size of a launch; false when the kernel does not cover it.
static bool ws_plan(int Kpad, int Npad, int Kt, int rows_period, bool want_amax, int &amax_mode, int &depth, size_t &smem) {
    if (2 * Npad > 512) return false;
    const bool one_slab = Kpad <= kWsKC;
    const int rowstep = kWsNpw * 4;
    depth = 2;
    amax_mode = WS_AMAX_NONE;
    if (want_amax) {
        const bool plain_ok = (rows_period % rowstep == 0) && (kWsTileM % rows_period == 0);
        if (one_slab && rowstep % rows_period == 0) amax_mode = WS_AMAX_REGS1;
        else if (one_slab && (2 * rowstep) % rows_period == 0 && (size_t)rows_period * (Kt + 4) * 4 <= kWsFetchBytes) amax_mode = WS_AMAX_REGS2;
        else if (Kpad > kWsKC && Kpad <= 2 * kWsKC && (2 * rowstep) % rows_period == 0 && (size_t)rows_period * Kt * 4 <= kWsFetchBytes)
            amax_mode = WS_AMAX_REGS2X2;
        else if (plain_ok) amax_mode = WS_AMAX_PLAIN;
        else return false;
    }
    const bool amax_table = amax_mode == WS_AMAX_PLAIN;
    smem = qdense_ws_smem(Kpad, Npad, Kt, rows_period, amax_table, depth, kWsEw);
    if (smem > 227 * 1024) {
        depth = 1;
        smem = qdense_ws_smem(Kpad, Npad, Kt, rows_period, amax_table, depth, kWsEw);
    }
    return smem + 1024 <= 227 * 1024;  // + room to start the carve on a 1 KB boundary
}

// Whether a forward call with these sizes can also produce the sums over groups of pool_rows consecutive rows (pointer
// alignment aside: x, y 16-byte aligned).
bool qdense_ws_pool_supported(int64_t M, int K, int N, int Kpad, int Npad, int Kt, int rows_period, int pool_rows, bool want_amax) {
    if (K % 4 != 0 || N % 4 != 0 || Npad / (kWsEw / 4) < 32 || M <= 0 || M >= ((int64_t)1 << 31)) return false;
    if ((pool_rows != 32 && pool_rows != 64 && pool_rows != 128) || M % pool_rows != 0) return false;
    if (!ws_tma_store_enabled() || encode_tiled_fn() == nullptr) return false;
    int amax_mode, depth;
    size_t smem;
    return ws_plan(Kpad, Npad, Kt, rows_period, want_amax, amax_mode, depth, smem);
}

// Launches the warp-specialised kernel when it covers the call; returns 1 with the grid size in *grid, 0 when the call is
// not covered (the caller then takes the general kernel), or a negative CUDA error code.
int qdense_ws_launch(const float *x, const float *qf, int rows_period, int round_mode, const float *wq, const float *bq,
                     int activation, float *y, unsigned *amax_part, int amax_direct, float *pool_out, int pool_rows,
                     float pool_scale, int64_t M, int K, int N, int Kpad, int Npad, int Kt, unsigned *status, cudaStream_t st,
                     int *grid) {
    if (qf == nullptr || K % 4 != 0 || !aligned(x, 16) || !aligned(y, 4)) return 0;
    if (pool_out != nullptr && ((pool_rows != 32 && pool_rows != 64 && pool_rows != 128) || M % pool_rows != 0)) return 0;
    constexpr int npw = kWsNpw, ew = kWsEw;
    const bool want_amax = amax_part != nullptr;
    int depth = 2, amax_mode = WS_AMAX_NONE;
    size_t smem = 0;
    if (!ws_plan(Kpad, Npad, Kt, rows_period, want_amax, amax_mode, depth, smem)) return 0;
    WsParams p;
    p.x = x; p.qf = qf; p.wq = wq; p.bq = bq; p.y = y; p.amax_part = amax_part; p.amax_direct = amax_direct; p.status = status;
    p.M = M; p.num_tiles = (M + kWsTileM - 1) / kWsTileM;
    p.K = K; p.N = N; p.Kpad = Kpad; p.Npad = Npad; p.Kt = Kt; p.rows_period = rows_period;
    p.rm = round_mode; p.act = activation; p.depth = depth;
    const int g = (int)(p.num_tiles < num_sms() ? p.num_tiles : num_sms());
    *grid = g;
    CUtensorMap tmap;
    memset(&tmap, 0, sizeof(tmap));
    // the bulk copies want x 16-byte aligned with rows a multiple of 16 bytes (K % 4 == 0, checked above)
    const bool tma = ws_tma_enabled() && M < ((int64_t)1 << 31) && ws_make_tmap(&tmap, x, M, K);
    CUtensorMap tmap_y;
    memset(&tmap_y, 0, sizeof(tmap_y));
    // bulk stores of 128 x 32 blocks: y rows a multiple of 16 bytes, 32 columns per epilogue warp (padded N >= 64)
    const bool tstore = ws_tma_store_enabled() && N % 4 == 0 && aligned(y, 16) && Npad / (ew / 4) >= 32 && M < ((int64_t)1 << 31) &&
                        ws_make_tmap(&tmap_y, y, M, N);
    p.tma_store = tstore ? 1 : 0;
    if (pool_out != nullptr && !tstore) return 0;  // the row-group sums are taken from the blocks of the bulk-store path
    p.pool_out = pool_out; p.pool_rows = pool_rows; p.pool_scale = pool_scale;
    if (pool_out != nullptr) smem += 1024;  // the warps' partial sums
    smem += 1024;  // room to start the carve on a 1 KB boundary whatever the base of dynamic shared memory is
    if (smem > 227 * 1024) return 0;
#define HGQ_WS_LAUNCH1(CV, AM, PW, EWW, TM)                                                                                      \
    do {                                                                                                                        \
        cudaError_t ce = cudaFuncSetAttribute(k_qdense_fwd_ws<CV, AM, PW, EWW, TM>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                              (int)smem);                                                                       \
        if (ce != cudaSuccess) return -(int)ce;                                                                                 \
        k_qdense_fwd_ws<CV, AM, PW, EWW, TM><<<g, (PW + EWW + 1 + (TM ? 1 : 0)) * 32, smem, st>>>(p, tmap, tmap_y);                      \
    } while (0)
#define HGQ_WS_LAUNCH(CV, AM, PW, EWW)                 \
    do {                                               \
        if (tma) HGQ_WS_LAUNCH1(CV, AM, PW, EWW, true); \
        else HGQ_WS_LAUNCH1(CV, AM, PW, EWW, false);    \
    } while (0)
#define HGQ_WS_MODES(CV, PW, EWW)                                                     \
    switch (amax_mode) {                                                              \
        case WS_AMAX_NONE: HGQ_WS_LAUNCH(CV, WS_AMAX_NONE, PW, EWW); break;           \
        case WS_AMAX_REGS1: HGQ_WS_LAUNCH(CV, WS_AMAX_REGS1, PW, EWW); break;         \
        case WS_AMAX_REGS2: HGQ_WS_LAUNCH(CV, WS_AMAX_REGS2, PW, EWW); break;         \
        case WS_AMAX_REGS2X2: HGQ_WS_LAUNCH(CV, WS_AMAX_REGS2X2, PW, EWW); break;     \
        default: HGQ_WS_LAUNCH(CV, WS_AMAX_PLAIN, PW, EWW); break;                    \
    }
    if (round_mode == RM_RND_CONV) { HGQ_WS_MODES(true, npw, ew) } else { HGQ_WS_MODES(false, npw, ew) }
#undef HGQ_WS_MODES
#undef HGQ_WS_LAUNCH
#undef HGQ_WS_LAUNCH1
    return 1;
}

}  // namespace hgq
