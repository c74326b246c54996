// K6w (per-head attention products, warp-specialised): the contract of k_attn_heads in attn.cu --
//   kind 0:  out_HTS[b,h,t,s] = sum_d  x_SHD[b,t,h,d] * y_SHD[b,s,h,d]        scores = Q K^T;   dP = dO V^T
//   kind 1:  out_SHD[b,t,h,d] = sum_s  x_HTS[b,h,t,s] * y_SHD[b,s,h,d]        context = P V;    dQ = dS K
//   kind 2:  out_SHD[b,s,h,d] = sum_t  x_HTS[b,h,t,s] * y_SHD[b,t,h,d]        dV = P^T dO;      dK = dS^T Q
// (the contractions of QMultiHeadAttention._compute_attention, src/hgq/layers/attn/mha.py:434-470, and of their backward)
// -- with the roles of a tile split over the warps of ONE persistent CTA per SM, so that the fetch of tile t + 2, the
// conversion of tile t + 1, the products of tile t and the write-out of tile t - 1 overlap:
//   loader warp      has the copy engine fetch the tile's raw boxes (tiled bulk-tensor copies of 32 columns with the 128-byte
//                    swizzle, from tensor maps over this GPU's x and y; two raw buffers);
//   16 converter warps split the raw fp32 values into two bf16 terms and store them as the no-swizzle core matrices of
//                    attn.cu's layouts into one of two operand stages, a quarter-warp per core matrix;
//   issuing warp     one tcgen05.mma chain per head and pair of terms into one of two accumulator sets in tensor memory;
//   4 epilogue warps read their row of the accumulator of their head and write it out (256-bit stores).
// The general kernel (attn.cu: four CTAs per SM, each doing these phases one after the other) waits on global loads most of
// the time (long-scoreboard stall 18.8 per issue); here the copy engine keeps two tiles in flight per SM.
// A tile is one pair of heads of one sample; both terms of both operands always go through the tensor cores (a zero low
// term costs four short products, far below the time the tile's bytes take).  HBM-bound: 4 (2 L D + L L) bytes per head.
// Every wait is bounded (polls, wall time, abort word); a role that gives up sets the status word and the CTA still
// frees its tensor memory.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdlib>
#include <cstring>

#include "hgq_common.cuh"
#include "tc05.cuh"
#include "tmap.cuh"

namespace hgq {

constexpr int kAwL = 64;
constexpr int kAwConvWarps = 16, kAwConv = kAwConvWarps * 32;
constexpr int kAwEpiWarps = 4;
constexpr int kAwIssueWarp = kAwConvWarps + kAwEpiWarps;  // two issuing warps, one per head of the pair
constexpr int kAwLoadWarp = kAwIssueWarp + 2;
constexpr int kAwThreads = (kAwLoadWarp + 1) * 32;

struct AwParams {
    float *out;
    unsigned *status;
    int64_t num_tiles;
    int H, D;
};

__device__ __forceinline__ void aw_arrive(uint64_t *bar) {
    asm volatile(
        "{\n\t"
        ".reg .b64 st;\n\t"
        "mbarrier.arrive.shared::cta.b64 st, [%0];\n\t"
        "}\n" ::"r"(tc::smem_u32(bar))
        : "memory");
}

__device__ __forceinline__ unsigned long long aw_now() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Wait for a phase of an mbarrier; gives up when another role has raised the abort word, after 2 s of wall time or after
// 2^24 polls, whichever comes first.
__device__ __forceinline__ bool aw_wait(uint64_t *bar, uint32_t parity, volatile int *abort_word) {
    if (tc::mbar_wait(bar, parity, 64)) return true;
    const unsigned long long t0 = aw_now();
    for (uint32_t it = 0; it < (1u << 16); ++it) {
        if (tc::mbar_wait(bar, parity, 256)) return true;
        if (*abort_word) return false;
        if (aw_now() - t0 > 2000000000ull) return false;
    }
    return false;
}

#ifdef HGQ_AW_PROF
// Profiling build (a stand-alone harness defines HGQ_AW_PROF): CTA 0 adds up, per role, the time spent inside each kind of
// wait and in the whole loop; g_aw_prof[role * 4 + k].
__device__ unsigned long long g_aw_prof[16];
#define AW_T0() const unsigned long long _t0 = aw_now()
#define AW_ACC(slot) do { aw_acc[(slot) & 3] += aw_now() - _t0; } while (0)
#define AW_DECL() unsigned long long aw_acc[4] = {0, 0, 0, 0}
#define AW_FLUSH(role) do { if (blockIdx.x == 0 && lane == 0) for (int _k = 0; _k < 4; ++_k) g_aw_prof[(role) * 4 + _k] = aw_acc[_k]; } while (0)
#else
#define AW_T0() do { } while (0)
#define AW_ACC(slot) do { } while (0)
#define AW_DECL() do { } while (0)
#define AW_FLUSH(role) do { } while (0)
#endif

__device__ __forceinline__ void aw_split2(float v0, float v1, uint32_t &hi, uint32_t &lo) {
    const __nv_bfloat162 h2 = __floats2bfloat162_rn(v0, v1);
    hi = *reinterpret_cast<const uint32_t *>(&h2);
    const float r0 = __fsub_rn(v0, __uint_as_float(hi << 16));
    const float r1 = __fsub_rn(v1, __uint_as_float(hi & 0xffff0000u));
    const __nv_bfloat162 l2 = __floats2bfloat162_rn(r0, r1);
    lo = *reinterpret_cast<const uint32_t *>(&l2);
}

// Where the copy engine put the eight floats (row r, float columns fc .. fc + 7, fc a multiple of 8) of a tensor fetched as
// boxes of 32 columns x `box_rows` rows with the 128-byte swizzle: two 16-byte chunks of row r of box fc / 32.
__device__ __forceinline__ void aw_raw_chunks(const unsigned char *base, int box_rows, int r, int fc, const float4 *&p0, const float4 *&p1) {
    const unsigned char *row = base + (fc >> 5) * box_rows * 128 + r * 128;
    const int c0 = (fc & 31) >> 2;  // even
    p0 = reinterpret_cast<const float4 *>(row + ((c0 ^ (r & 7)) << 4));
    p1 = reinterpret_cast<const float4 *>(row + (((c0 + 1) ^ (r & 7)) << 4));
}

// eight floats of a raw box -> one 16-byte row of a core matrix in each of the two term planes
__device__ __forceinline__ int aw_put8(const float4 *p0, const float4 *p1, unsigned char *hi_plane, unsigned char *lo_plane, int off) {
    const float4 a = *p0, b = *p1;
    uint32_t hi[4], lo[4];
    aw_split2(a.x, a.y, hi[0], lo[0]);
    aw_split2(a.z, a.w, hi[1], lo[1]);
    aw_split2(b.x, b.y, hi[2], lo[2]);
    aw_split2(b.z, b.w, hi[3], lo[3]);
    *reinterpret_cast<uint4 *>(hi_plane + off) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
    *reinterpret_cast<uint4 *>(lo_plane + off) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
    return ((lo[0] | lo[1] | lo[2] | lo[3]) & 0x7fff7fffu) != 0;  // some low term is not (+-) zero
}

template <int KIND>
__global__ void __launch_bounds__(kAwThreads, 1) k_attn_heads_ws(const AwParams P, const __grid_constant__ CUtensorMap map_x,
                                                                const __grid_constant__ CUtensorMap map_y) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    // the swizzled boxes need 1 KB aligned destinations whatever the base of dynamic shared memory is
    unsigned char *smem = smem_raw + ((1024u - (tc::smem_u32(smem_raw) & 1023u)) & 1023u);
    constexpr int L = kAwL;
    const int D = P.D, H = P.H, DG = D >> 3;
    const int Ka = (KIND == 0) ? D : L;          // contraction length
    const int Nn = (KIND == 0) ? L : D;          // columns of a product
    const int a_term = 128 * Ka * 2;             // A: 128 rows x Ka, one bf16 term
    const int b_term = Nn * Ka * 2;              // B of one head, one term
    const int oper_bytes = 2 * a_term + 4 * b_term;
    const int rawx_bytes = (KIND == 0) ? L * 2 * D * 4 : 128 * L * 4;
    const int rawy_bytes = L * 2 * D * 4;
    const int raw_bytes = rawx_bytes + rawy_bytes;
    unsigned char *OPER = smem;                    // [2 stages]: A [2 terms], B [2 heads][2 terms]
    unsigned char *RAW = OPER + 2 * oper_bytes;    // [2 buffers]: x box, y box
    uint64_t *raw_full = reinterpret_cast<uint64_t *>(RAW + 2 * raw_bytes);
    uint64_t *raw_empty = raw_full + 2, *op_full = raw_full + 4, *op_empty = raw_full + 6, *acc_full = raw_full + 8,
             *acc_empty = raw_full + 10;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(raw_full + 12);
    int *abort_word = reinterpret_cast<int *>(tmem_slot + 1);
    // per operand stage and issuing warp: bit 0 / 1 = some low term of A / B is non-zero (else its products are skipped)
    int *lo_flags = abort_word + 1;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    uint32_t tmem_cols = 32;
    while ((int)tmem_cols < 4 * Nn) tmem_cols <<= 1;  // two accumulator sets of two heads
    if (tid == 0) {
        for (int s = 0; s < 2; ++s) {
            tc::mbar_init(raw_full + s, 1);               // the loader's expect_tx arrival (+ the copies' bytes)
            tc::mbar_init(raw_empty + s, kAwConvWarps);   // one arrival per converter warp
            tc::mbar_init(op_full + s, kAwConvWarps);
            tc::mbar_init(op_empty + s, 2);               // tcgen05.commit of each issuing warp
            tc::mbar_init(acc_full + s, 2);
            lo_flags[2 * s] = lo_flags[2 * s + 1] = 0;
            tc::mbar_init(acc_empty + s, kAwEpiWarps);    // one arrival per epilogue warp
        }
        *abort_word = 0;
        tc::mbar_init_fence();
    }
    if (warp == kAwIssueWarp) tc::tmem_alloc(tmem_slot, tmem_cols);
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    const int pairs = H >> 1;

    if (warp < kAwConvWarps) {
        // ================================ converters =================================================================
        AW_DECL();
        uint32_t n = 0;
        bool ok = true;
        for (int64_t tile = blockIdx.x; tile < P.num_tiles && ok; tile += gridDim.x, ++n) {
            const uint32_t s = n & 1u, use = n >> 1;
            bool w;
            { AW_T0(); w = aw_wait(raw_full + s, use & 1u, abort_word); AW_ACC(0); }
            { AW_T0(); if (w && use > 0) w = aw_wait(op_empty + s, (use - 1) & 1u, abort_word); AW_ACC(1); }  // the products of tile n - 2 have read the stage
            if (!__all_sync(0xffffffffu, w)) { ok = false; break; }
            AW_T0();
            const unsigned char *RX = RAW + s * raw_bytes, *RY = RX + rawx_bytes;
            unsigned char *A = OPER + s * oper_bytes;
            unsigned char *Bm = A + 2 * a_term;
            const float4 *p0, *p1;
            int lo_a = 0, lo_b = 0;
            // The 8 lanes of a quarter-warp take the 8 rows of ONE core matrix (r8 = u & 7): their 16-byte stores fill 128
            // contiguous bytes, and their reads of the swizzled raw rows hit 8 different chunk positions -- no bank conflicts
            // on either side (with a quarter-warp spread over 8 core matrices every store hit one bank group 8 times, and
            // the stores of a tile alone took 1.3 us of the SM's shared-memory port).
            // A operand: both heads (layouts of attn.cu)
            if (KIND == 0) {
                for (int u = tid; u < 128 * DG; u += kAwConv) {
                    const int r8 = u & 7, v = u >> 3, rg = v / DG, dg = v - rg * DG;
                    const int hh = rg >> 3, t = (rg & 7) * 8 + r8, row = hh * 64 + t;
                    aw_raw_chunks(RX, 64, t, hh * D + dg * 8, p0, p1);
                    lo_a |= aw_put8(p0, p1, A, A + a_term, ((row >> 3) * DG + dg) * 128 + (row & 7) * 16);
                }
            } else if (KIND == 1) {
                for (int u = tid; u < 128 * 8; u += kAwConv) {
                    const int r8 = u & 7, sg = (u >> 3) & 7, row = (u >> 6) * 8 + r8;
                    aw_raw_chunks(RX, 128, row, sg * 8, p0, p1);
                    lo_a |= aw_put8(p0, p1, A, A + a_term, ((row >> 3) * 8 + sg) * 128 + (row & 7) * 16);
                }
            } else {
                for (int u = tid; u < 128 * 8; u += kAwConv) {
                    const int r8 = u & 7, sg = (u >> 3) & 7, rg = u >> 6;
                    const int hh = rg >> 3, t = (rg & 7) * 8 + r8, mg = hh * 8 + sg;
                    aw_raw_chunks(RX, 128, hh * 64 + t, sg * 8, p0, p1);
                    lo_a |= aw_put8(p0, p1, A, A + a_term, ((t >> 3) * 16 + mg) * 128 + (t & 7) * 16);
                }
            }
            // B operands: one per head; rows r (kind 0: the product's columns s; kinds 1, 2: the contraction index)
            for (int u = tid; u < 128 * DG; u += kAwConv) {
                const int r8 = u & 7, v = u >> 3;
                const int dg = v % DG, hh = (v / DG) & 1, r = (v / (2 * DG)) * 8 + r8;
                unsigned char *base = Bm + hh * 2 * b_term;
                aw_raw_chunks(RY, 64, r, hh * D + dg * 8, p0, p1);
                lo_b |= aw_put8(p0, p1, base, base + b_term, ((r >> 3) * DG + dg) * 128 + (r & 7) * 16);
            }
            { AW_T0(); tc::fence_smem_to_async(); AW_ACC(3); }
            const int fl = (__any_sync(0xffffffffu, lo_a) ? 1 : 0) | (__any_sync(0xffffffffu, lo_b) ? 2 : 0);
            if (lane == 0) {
                if (fl) {
                    atomicOr(lo_flags + 2 * s, fl);
                    atomicOr(lo_flags + 2 * s + 1, fl);
                }
                aw_arrive(op_full + s);
                aw_arrive(raw_empty + s);
            }
            AW_ACC(2);
        }
        if (warp == 0) AW_FLUSH(0);
        if (!ok) {
            *reinterpret_cast<volatile int *>(abort_word) = 1;
            if (lane == 0 && P.status) atomicOr(P.status, 1u);
        }
    } else if (warp == kAwIssueWarp || warp == kAwIssueWarp + 1) {
        // ================================ tensor-core issue ==========================================================
        const uint32_t idesc = tc::make_idesc_bf16(Nn, KIND == 2, KIND != 0);
        AW_DECL();
        uint32_t n = 0;
        bool ok = true;
        for (int64_t tile = blockIdx.x; tile < P.num_tiles && ok; tile += gridDim.x, ++n) {
            const uint32_t s = n & 1u, use = n >> 1;
            bool w;
            { AW_T0(); w = aw_wait(op_full + s, use & 1u, abort_word); AW_ACC(4); }
            { AW_T0(); if (w && use > 0) w = aw_wait(acc_empty + s, (use - 1) & 1u, abort_word); AW_ACC(5); }  // the epilogue has read accumulator set s
            if (!__all_sync(0xffffffffu, w)) { ok = false; break; }
            AW_T0();
            // Products with a low term that is zero everywhere are skipped.  Each issuing warp has its own copy of the flags
            // and clears it before its commit: the converters set them again only after op_empty, i.e. after both commits.
            const int fl = *reinterpret_cast<volatile int *>(lo_flags + 2 * s + (warp - kAwIssueWarp));
            const int n_a = (fl & 1) ? 2 : 1, n_b = (fl & 2) ? 2 : 1;
            if (lane == 0) {
                tc::fence_after_sync();
                const uint32_t a_base = tc::smem_u32(OPER + s * oper_bytes), b_base = a_base + 2 * a_term;
                {
                    const int hh = warp - kAwIssueWarp;
                    const uint32_t acc = tmem_base + (uint32_t)(s * 2 * Nn + hh * Nn);
                    const uint32_t bb = b_base + hh * 2 * b_term;
                    bool first = true;
                    for (int ta = 0; ta < n_a; ++ta)
                        for (int tb = 0; tb < n_b; ++tb) {
                            uint64_t da, db;
                            uint32_t a_step, b_step;
                            if (KIND == 0) {         // A, B K-major: cores adjacent along K 128 B apart, row groups DG * 128 apart
                                da = tc::make_smem_desc(a_base + ta * a_term, 128, (uint32_t)DG * 128);
                                db = tc::make_smem_desc(bb + tb * b_term, 128, (uint32_t)DG * 128);
                                a_step = b_step = 256 >> 4;
                            } else if (KIND == 1) {  // A K-major (8 s groups per row group); B MN-major: d groups 128 B apart, r groups DG * 128
                                da = tc::make_smem_desc(a_base + ta * a_term, 128, 8 * 128);
                                db = tc::make_smem_desc(bb + tb * b_term, (uint32_t)DG * 128, 128);
                                a_step = 256 >> 4;
                                b_step = (uint32_t)(2 * DG * 128) >> 4;
                            } else {                 // A MN-major: m groups 128 B apart, t groups 16 * 128 apart
                                da = tc::make_smem_desc(a_base + ta * a_term, 16 * 128, 128);
                                db = tc::make_smem_desc(bb + tb * b_term, (uint32_t)DG * 128, 128);
                                a_step = (2 * 16 * 128) >> 4;
                                b_step = (uint32_t)(2 * DG * 128) >> 4;
                            }
                            for (int ks = 0; ks < Ka / 16; ++ks) {
                                tc::mma_bf16(acc, da, db, idesc, !first);
                                first = false;
                                da += a_step;
                                db += b_step;
                            }
                        }
                }
                lo_flags[2 * s + (warp - kAwIssueWarp)] = 0;
                __threadfence_block();
                tc::commit(op_empty + s);   // the operand stage may be overwritten once these products have completed
                tc::commit(acc_full + s);
            }
            __syncwarp();
            AW_ACC(6);
        }
        AW_FLUSH(1);
        if (!ok) {
            *reinterpret_cast<volatile int *>(abort_word) = 1;
            if (lane == 0 && P.status) atomicOr(P.status, 1u);
        }
    } else if (warp == kAwLoadWarp) {
        // ================================ bulk-copy loader ===========================================================
        // x at (column, row) = (h0 D, b L) of [B L, H D] (kind 0) or (0, (b H + h0) L) of [B H L, L]; y at (h0 D, b L).
        // h0 is even and D a multiple of 16: the column offsets are multiples of 128 bytes.
        AW_DECL();
        uint32_t n = 0;
        bool ok = true;
        for (int64_t tile = blockIdx.x; tile < P.num_tiles && ok; tile += gridDim.x, ++n) {
            const uint32_t s = n & 1u, use = n >> 1;
            if (use > 0) {
                AW_T0();
                const bool w = aw_wait(raw_empty + s, (use - 1) & 1u, abort_word);
                AW_ACC(8);
                if (!__all_sync(0xffffffffu, w)) { ok = false; break; }
            }
            if (lane == 0) {
                const int64_t b = tile / pairs;
                const int h0 = (int)(tile - b * pairs) * 2;
                const uint32_t rx = tc::smem_u32(RAW + s * raw_bytes), ry = rx + rawx_bytes;
                tma::expect_tx(raw_full + s, (uint32_t)raw_bytes);
                const int nb_shd = (2 * D) >> 5;  // boxes of 32 columns that cover the two heads' columns: 1 or 2
                if (KIND == 0) {
                    for (int j = 0; j < nb_shd; ++j) tma::load_2d(rx + j * 64 * 128, &map_x, h0 * D + 32 * j, (int)(b * L), raw_full + s);
                } else {
                    for (int j = 0; j < 2; ++j) tma::load_2d(rx + j * 128 * 128, &map_x, 32 * j, (int)((b * H + h0) * L), raw_full + s);
                }
                for (int j = 0; j < nb_shd; ++j) tma::load_2d(ry + j * 64 * 128, &map_y, h0 * D + 32 * j, (int)(b * L), raw_full + s);
            }
            __syncwarp();
        }
        AW_FLUSH(2);
        if (!ok) {
            *reinterpret_cast<volatile int *>(abort_word) = 1;
            if (lane == 0 && P.status) atomicOr(P.status, 1u);
        }
    } else {
        // ================================ epilogue ===================================================================
        // thread = row r of the pair (head r / 64, position r % 64); its head's accumulator holds the row's Nn columns
        const int e = warp - kAwConvWarps;
        const int r = e * 32 + lane, hh = r >> 6, i = r & 63;
        const int64_t row_shd = (int64_t)H * D;
        AW_DECL();
        uint32_t n = 0;
        bool ok = true;
        for (int64_t tile = blockIdx.x; tile < P.num_tiles && ok; tile += gridDim.x, ++n) {
            const uint32_t s = n & 1u, use = n >> 1;
            bool w;
            { AW_T0(); w = aw_wait(acc_full + s, use & 1u, abort_word); AW_ACC(12); }
            if (!__all_sync(0xffffffffu, w)) { ok = false; break; }
            AW_T0();
            tc::fence_after_sync();
            const int64_t b = tile / pairs;
            const int h0 = (int)(tile - b * pairs) * 2;
            float *dst = (KIND == 0) ? P.out + ((b * H + h0 + hh) * L + i) * L : P.out + (b * L + i) * row_shd + (int64_t)(h0 + hh) * D;
            const uint32_t taddr = tmem_base + ((uint32_t)(e * 32) << 16) + (uint32_t)(s * 2 * Nn + hh * Nn);
            for (int c0 = 0; c0 < Nn; c0 += 16) {
                float v[16];
                tc::tmem_ld16v(taddr + (uint32_t)c0, v);
                if (c0 + 16 >= Nn) {  // the row is in registers: hand the accumulator set back to the issuing warp
                    tc::fence_before_sync();
                    __syncwarp();
                    if (lane == 0) aw_arrive(acc_empty + s);
                }
                float lo8[8], hi8[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) { lo8[j] = v[j]; hi8[j] = v[8 + j]; }
                stcs8(dst + c0, lo8);
                stcs8(dst + c0 + 8, hi8);
            }
            AW_ACC(13);
        }
        if (e == 0) AW_FLUSH(3);
        if (!ok) {
            *reinterpret_cast<volatile int *>(abort_word) = 1;
            if (lane == 0 && P.status) atomicOr(P.status, 1u);
        }
    }

    // ---- tear-down ----------------------------------------------------------------------------------------------------
    tc::fence_before_sync();
    __syncthreads();
    if (warp == kAwIssueWarp) tc::tmem_dealloc(tmem_base, tmem_cols);
}

static size_t aw_smem(int kind, int D) {
    const int Ka = kind == 0 ? D : kAwL, Nn = kind == 0 ? kAwL : D;
    const size_t oper = 2 * (size_t)128 * Ka * 2 + 4 * (size_t)Nn * Ka * 2;
    const size_t raw = (kind == 0 ? (size_t)kAwL * 2 * D * 4 : (size_t)128 * kAwL * 4) + (size_t)kAwL * 2 * D * 4;
    return 2 * oper + 2 * raw + 12 * 8 + 96 + 1024;  // + room to start the carve on a 1 KB boundary
}

// HGQ_ATTN_WS=0 in the environment keeps every product on the general kernel (for comparisons).
static bool aw_enabled() {
    static const bool on = [] {
        const char *v = getenv("HGQ_ATTN_WS");
        return !(v != nullptr && v[0] == '0');
    }();
    return on;
}

static bool aw_all_kinds() {
    static const bool on = [] {
        const char *v = getenv("HGQ_ATTN_WS");
        return v != nullptr && v[0] == '2';
    }();
    return on;
}

// Launches the warp-specialised kernel when it covers the call: returns 1, 0 when not covered (the caller takes the general
// kernel), or a negative CUDA error code.
int attn_ws_launch(int kind, const float *x, const float *y, float *out, int64_t B, int L, int H, int D, unsigned *status,
                   cudaStream_t st) {
    if (!aw_enabled() || L != kAwL) return 0;
    // kind 0 (few input bytes, 32 KB written per tile) is faster on the general kernel with its raw boxes fetched by the
    // copy engine (0.19-0.20 ms against 0.23 ms here on 8192 x 4 heads); HGQ_ATTN_WS=2 sends it here all the same
    if (kind == 0 && !aw_all_kinds()) return 0;
    const int64_t rows_shd = B * L, rows_hts = B * H * L;
    if (rows_hts >= ((int64_t)1 << 31)) return 0;
    const size_t smem = aw_smem(kind, D);
    if (smem > 227 * 1024) return 0;
    CUtensorMap map_x, map_y;
    memset(&map_x, 0, sizeof(map_x));
    memset(&map_y, 0, sizeof(map_y));
    // tensor maps over this GPU's x and y alone, boxes of 32 columns with the 128-byte swizzle: [B L, H D] in boxes of 64
    // rows, [B H L, L] in boxes of 128 rows
    const bool ok = (kind == 0 ? tma::make_map_2d(&map_x, x, rows_shd, (int64_t)H * D, (int64_t)H * D, 32, kAwL, true)
                               : tma::make_map_2d(&map_x, x, rows_hts, L, L, 32, 128, true)) &&
                    tma::make_map_2d(&map_y, y, rows_shd, (int64_t)H * D, (int64_t)H * D, 32, kAwL, true);
    if (!ok) return 0;
    AwParams p;
    p.out = out; p.status = status; p.H = H; p.D = D;
    p.num_tiles = B * (H / 2);
    const int grid = (int)(p.num_tiles < num_sms() ? p.num_tiles : num_sms());
    cudaError_t ce = cudaSuccess;
#define HGQ_AW_LAUNCH(KIND_)                                                                                         \
    do {                                                                                                            \
        ce = cudaFuncSetAttribute(k_attn_heads_ws<KIND_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);  \
        if (ce != cudaSuccess) return -(int)ce;                                                                     \
        k_attn_heads_ws<KIND_><<<grid, kAwThreads, smem, st>>>(p, map_x, map_y);                                    \
    } while (0)
    if (kind == 0) HGQ_AW_LAUNCH(0);
    else if (kind == 1) HGQ_AW_LAUNCH(1);
    else HGQ_AW_LAUNCH(2);
#undef HGQ_AW_LAUNCH
    return 1;
}

}  // namespace hgq
