// K6 (per-head products of multi-head attention on the tensor cores): the two activation-activation contractions of
// QMultiHeadAttention._compute_attention (src/hgq/layers/attn/mha.py:434-470, einsum 'aecd,abcd->acbe' for the scores and
// 'acbe,aecd->abcd' for the context) and the four products of their backward.
//
// Tensors: "SHD" = [B, L, H, D] (projections, context and their gradients: heads interleaved in memory), "HTS" =
// [B, H, L, L] (scores, probabilities and their gradients), L = 64 positions, D = 16 or 32 per head.
//   kind 0:  out_HTS[b,h,t,s] = sum_d  x_SHD[b,t,h,d] * y_SHD[b,s,h,d]        scores = Q K^T;   dP = dO V^T
//   kind 1:  out_SHD[b,t,h,d] = sum_s  x_HTS[b,h,t,s] * y_SHD[b,s,h,d]        context = P V;    dQ = dS K
//   kind 2:  out_SHD[b,s,h,d] = sum_t  x_HTS[b,h,t,s] * y_SHD[b,t,h,d]        dV = P^T dO;      dK = dS^T Q
// A tile is one pair of heads of one sample: the A operand holds the 2 x 64 rows of both heads (the M = 128 of one
// tcgen05.mma), and one product per head multiplies it with that head's B operand into its own accumulator; each
// accumulator is valid in the 64 rows of its head (the other 64 rows are computed against the wrong head and dropped).
// Operands are read strided straight from the [B, L, H, D] / [B, H, L, L] tensors (no transposed copies), split into
// two bf16 terms (exact up to 16 significant bits: the quantised projections and probabilities; gradients are rounded
// at 2^-17 relative) and stored as no-swizzle core matrices: K-major where the contraction index is contiguous in memory,
// MN-major where the row / column index is.  HBM-bound: 4 (2 L D + L L) bytes per head and product.
// Raw operands reach the CTA in one of two ways (template parameter TMA): every thread loads its own 32-byte pieces, or
// (kind 0) the copy engine fetches the tile's two boxes (tiled bulk-tensor copies from tensor maps over this GPU's x and y,
// completion counted on an mbarrier) into a raw buffer that the threads convert from; the copies of tile t + 1 are issued
// as soon as tile t has been converted, so they run under its products and its write-out.  Measured on 8192 x 4 heads:
// kind 0 0.212 -> 0.193 ms; kinds 1 and 2, whose 32 KB raw box leaves room for two or three CTAs per SM instead of four,
// 0.245 -> 0.270 and 0.266 -> 0.265 ms, so they keep the per-thread loads.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdlib>
#include <cstring>

#include "hgq_common.cuh"
#include "tc05.cuh"
#include "tmap.cuh"

namespace hgq {

int attn_ws_launch(int kind, const float *x, const float *y, float *out, int64_t B, int L, int H, int D, unsigned *status,
                   cudaStream_t st);

constexpr int kAtThreads = 256;
constexpr int kAtL = 64;

struct AtParams {
    const float *x, *y;
    float *out;
    unsigned *status;
    int64_t B, num_tiles;
    int H, D;
};

__device__ __forceinline__ void at_split2(float v0, float v1, uint32_t &hi, uint32_t &lo) {
    const __nv_bfloat162 h2 = __floats2bfloat162_rn(v0, v1);
    hi = *reinterpret_cast<const uint32_t *>(&h2);
    const float r0 = __fsub_rn(v0, __uint_as_float(hi << 16));
    const float r1 = __fsub_rn(v1, __uint_as_float(hi & 0xffff0000u));
    const __nv_bfloat162 l2 = __floats2bfloat162_rn(r0, r1);
    lo = *reinterpret_cast<const uint32_t *>(&l2);
}

// eight floats -> one 16-byte row of a core matrix in each of the two term planes
__device__ __forceinline__ int at_cvt8(const float (&v)[8], unsigned char *hi_plane, unsigned char *lo_plane, int off) {
    uint32_t hi[4], lo[4];
    at_split2(v[0], v[1], hi[0], lo[0]);
    at_split2(v[2], v[3], hi[1], lo[1]);
    at_split2(v[4], v[5], hi[2], lo[2]);
    at_split2(v[6], v[7], hi[3], lo[3]);
    *reinterpret_cast<uint4 *>(hi_plane + off) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
    *reinterpret_cast<uint4 *>(lo_plane + off) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
    return ((lo[0] | lo[1] | lo[2] | lo[3]) & 0x7fff7fffu) != 0;
}

// eight consecutive floats from the raw buffer in shared memory (SH, 32-byte aligned) or from global memory
template <bool SH>
__device__ __forceinline__ int at_put8(const float *src, unsigned char *hi_plane, unsigned char *lo_plane, int off) {
    float v[8];
    if (SH) {
        const float4 a = *reinterpret_cast<const float4 *>(src), b = *reinterpret_cast<const float4 *>(src + 4);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    } else {
        ldcs8(src, v);  // one 32-byte sector per thread and instruction; every operand element is read once per product
    }
    return at_cvt8(v, hi_plane, lo_plane, off);
}

// eight floats (row r, float columns fc .. fc + 7) of a [64, 2 D] raw tensor that the copy engine delivered as boxes of 32
// columns x 64 rows with the 128-byte swizzle: 16-byte chunk c of a row sits at chunk position c ^ (r & 7)
__device__ __forceinline__ int at_put8_swz(const unsigned char *raw, int r, int fc, unsigned char *hi_plane, unsigned char *lo_plane, int off) {
    const unsigned char *row = raw + (fc >> 5) * kAtL * 128 + r * 128;
    const int c0 = (fc & 31) >> 2;
    const float4 a = *reinterpret_cast<const float4 *>(row + ((c0 ^ (r & 7)) << 4));
    const float4 b = *reinterpret_cast<const float4 *>(row + (((c0 + 1) ^ (r & 7)) << 4));
    const float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    return at_cvt8(v, hi_plane, lo_plane, off);
}

template <int KIND, bool TMA>
__global__ void __launch_bounds__(kAtThreads) k_attn_heads(const AtParams P, const __grid_constant__ CUtensorMap map_x,
                                                          const __grid_constant__ CUtensorMap map_y) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    // the swizzled raw boxes (TMA) need 1 KB aligned destinations whatever the base of dynamic shared memory is
    unsigned char *smem = TMA ? smem_raw + ((1024u - (tc::smem_u32(smem_raw) & 1023u)) & 1023u) : smem_raw;
    constexpr int L = kAtL;
    const int D = P.D, H = P.H, DG = D >> 3;
    // operand geometry
    const int Ka = (KIND == 0) ? D : L;          // contraction length
    const int Nn = (KIND == 0) ? L : D;          // columns of a product
    const int a_term = 128 * Ka * 2;             // A: 128 rows x Ka
    const int b_term = Nn * Ka * 2;              // B of one head
    unsigned char *A = smem;                     // [2 terms]
    unsigned char *Bm = A + 2 * a_term;          // [2 heads][2 terms]
    // raw boxes (TMA): x and y are [64, 2 D] floats each, fetched as boxes of 32 columns with the 128-byte swizzle (one
    // box for D = 16, two for D = 32); every size is a multiple of 1 KB
    static_assert(!TMA || KIND == 0, "bulk tensor copies are used for kind 0 only");
    const int rawx_bytes = TMA ? L * 2 * D * 4 : 0;
    const int rawy_bytes = TMA ? L * 2 * D * 4 : 0;
    float *RX = reinterpret_cast<float *>(Bm + 4 * b_term);
    float *RY = reinterpret_cast<float *>(Bm + 4 * b_term + rawx_bytes);
    uint64_t *bar = reinterpret_cast<uint64_t *>(Bm + 4 * b_term + rawx_bytes + rawy_bytes);
    uint64_t *full = bar + 1;  // TMA: the raw boxes of the next tile have landed
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bar + 2);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    uint32_t tmem_cols = 32;
    while ((int)tmem_cols < 2 * Nn) tmem_cols <<= 1;
    if (tid == 0) {
        tc::mbar_init(bar, 2);  // one issuing thread per head commits to it
        tc::mbar_init(full, 1); // the expect_tx arrival of the thread that issues the copies (+ their bytes)
        tc::mbar_init_fence();
    }
    if (warp == 0) tc::tmem_alloc(tmem_slot, tmem_cols);
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t a_base = tc::smem_u32(A), b_base = tc::smem_u32(Bm);
    const uint32_t idesc = tc::make_idesc_bf16(Nn, KIND == 2, KIND != 0);
    const int pairs = H >> 1;
    const int64_t LL = (int64_t)L * L, row_shd = (int64_t)H * D;

    // the two boxes of a tile: x and y at (column, row) = (h0 D, b L) of [B L, H D].  h0 is even and D a multiple of 16:
    // the column offsets are multiples of 128 bytes.
    auto fetch = [&](int64_t t) {
        const int64_t tb = t / pairs;
        const int th0 = (int)(t - tb * pairs) * 2;
        tma::expect_tx(full, (uint32_t)(rawx_bytes + rawy_bytes));
        for (int j = 0; j < ((2 * D) >> 5); ++j) {
            tma::load_2d(tc::smem_u32(RX) + j * L * 128, &map_x, th0 * D + 32 * j, (int)(tb * L), full);
            tma::load_2d(tc::smem_u32(RY) + j * L * 128, &map_y, th0 * D + 32 * j, (int)(tb * L), full);
        }
    };
    if (TMA && tid == 0 && (int64_t)blockIdx.x < P.num_tiles) fetch(blockIdx.x);

    uint32_t phase = 0, full_phase = 0;
    bool ok = true;
    bool pending = TMA && (int64_t)blockIdx.x < P.num_tiles;  // copies issued whose arrival nobody has waited for yet
    for (int64_t tile = blockIdx.x; tile < P.num_tiles && ok; tile += gridDim.x) {
        const int64_t b = tile / pairs;
        const int h0 = (int)(tile - b * pairs) * 2;
        // TMA: the tile's rows in the raw buffers (row pitch 2 D floats)
        const float *x_shd = TMA ? RX : P.x + b * L * row_shd + (int64_t)h0 * D;   // kind 0: x[b, 0, h0, 0]
        const float *x_hts = TMA ? RX : P.x + (b * H + h0) * LL;                   // kinds 1, 2: x[b, h0, 0, 0]
        const float *y_shd = TMA ? RY : P.y + b * L * row_shd + (int64_t)h0 * D;
        const int64_t pitch_x = TMA ? 2 * D : row_shd, pitch_y = pitch_x;
        int lo_a = 0, lo_b = 0;
        if (TMA) {
            const bool got = tc::mbar_wait(full, full_phase);
            if (!__syncthreads_and(got ? 1 : 0)) {
                if (tid == 0 && P.status) atomicOr(P.status, 1u);
                ok = false;
                break;
            }
            full_phase ^= 1u;
            pending = false;
        }
        // ---- A operand: both heads ------------------------------------------------------------------------------------------
        if (KIND == 0) {
            // rows (hh, t), contraction d: K-major, core (row group, d group); unit = (t, hh, d group): a row of the pair is
            // 2 D contiguous floats in memory
            for (int u = tid; u < 128 * DG; u += kAtThreads) {
                // the 8 lanes of a quarter-warp take the 8 rows of one core matrix: their 16-byte stores fill 128 contiguous
                // bytes instead of hitting one bank group 8 times (and, with the raw box in shared memory, their reads of the
                // swizzled rows hit 8 different chunk positions)
                const int r8 = u & 7, v = u >> 3, rg = v / DG;
                const int dg = v - rg * DG, hh = rg >> 3, t = (rg & 7) * 8 + r8;
                const int row = hh * 64 + t;
                if (TMA) lo_a |= at_put8_swz(reinterpret_cast<const unsigned char *>(RX), t, hh * D + dg * 8, A, A + a_term, ((row >> 3) * DG + dg) * 128 + (row & 7) * 16);
                else lo_a |= at_put8<false>(x_shd + t * pitch_x + hh * D + dg * 8, A, A + a_term, ((row >> 3) * DG + dg) * 128 + (row & 7) * 16);
            }
        } else if (KIND == 1) {
            // rows (hh, t), contraction s: K-major, core (row group, s group): a row is 64 contiguous floats
            for (int u = tid; u < 128 * 8; u += kAtThreads) {
                const int r8 = u & 7, sg = (u >> 3) & 7, row = (u >> 6) * 8 + r8;  // a quarter-warp = the 8 rows of one core matrix
                lo_a |= at_put8<TMA>(x_hts + (int64_t)row * L + sg * 8, A, A + a_term, ((row >> 3) * 8 + sg) * 128 + (row & 7) * 16);
            }
        } else {
            // rows m = (hh, s), contraction t: MN-major, core (t group, m group) = 8 t x 8 m; a row t of a head is 64 contiguous s
            for (int u = tid; u < 128 * 8; u += kAtThreads) {
                const int r8 = u & 7, sg = (u >> 3) & 7, rg = u >> 6;  // a quarter-warp = the 8 positions t of one core matrix
                const int hh = rg >> 3, t = (rg & 7) * 8 + r8;
                const int mg = hh * 8 + sg;
                lo_a |= at_put8<TMA>(x_hts + hh * LL + (int64_t)t * L + sg * 8, A, A + a_term, ((t >> 3) * 16 + mg) * 128 + (t & 7) * 16);
            }
        }
        // ---- B operands: one per head -----------------------------------------------------------------------------------------
        if (KIND == 0) {
            // rows s (the product's columns), contraction d: K-major, core (s group, d group)
            for (int u = tid; u < 128 * DG; u += kAtThreads) {
                const int r8 = u & 7, v = u >> 3;
                const int dg = v % DG, hh = (v / DG) & 1, s = (v / (2 * DG)) * 8 + r8;
                unsigned char *base = Bm + hh * 2 * b_term;
                if (TMA) lo_b |= at_put8_swz(reinterpret_cast<const unsigned char *>(RY), s, hh * D + dg * 8, base, base + b_term, ((s >> 3) * DG + dg) * 128 + (s & 7) * 16);
                else lo_b |= at_put8<false>(y_shd + s * pitch_y + hh * D + dg * 8, base, base + b_term, ((s >> 3) * DG + dg) * 128 + (s & 7) * 16);
            }
        } else {
            // columns d, contraction r (s or t): MN-major, core (r group, d group) = 8 r x 8 d
            for (int u = tid; u < 128 * DG; u += kAtThreads) {
                const int r8 = u & 7, v = u >> 3;
                const int dg = v % DG, hh = (v / DG) & 1, r = (v / (2 * DG)) * 8 + r8;
                unsigned char *base = Bm + hh * 2 * b_term;
                lo_b |= at_put8<TMA>(y_shd + r * pitch_y + hh * D + dg * 8, base, base + b_term, ((r >> 3) * DG + dg) * 128 + (r & 7) * 16);
            }
        }
        tc::fence_smem_to_async();
        const int n_a = __syncthreads_or(lo_a) ? 2 : 1;
        const int n_b = __syncthreads_or(lo_b) ? 2 : 1;
        // every thread is done with the raw buffers: the next tile's boxes may land while this one is multiplied and written
        if (TMA && tile + gridDim.x < P.num_tiles) {
            if (tid == 0) fetch(tile + gridDim.x);
            pending = true;
        }
        // ---- one issuing thread per head ------------------------------------------------------------------------------------------
        if (lane == 0 && warp < 2) {
            tc::fence_after_sync();
            const int hh = warp;
            const uint32_t acc = tmem_base + (uint32_t)(hh * Nn);
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
                    for (int s = 0; s < Ka / 16; ++s) {
                        tc::mma_bf16(acc, da, db, idesc, !first);
                        first = false;
                        da += a_step;
                        db += b_step;
                    }
                }
            tc::commit(bar);
        }
        const bool waited = (warp == 0) ? tc::mbar_wait(bar, phase) : true;
        phase ^= 1u;
        ok = __syncthreads_and(waited ? 1 : 0) != 0;
        if (!ok) {
            if (tid == 0 && P.status) atomicOr(P.status, 1u);
            break;
        }
        // ---- epilogue: row r of the pair lives in accumulator r / 64 ------------------------------------------------------------
        tc::fence_after_sync();
        {
            const int qlane = (warp & 3) * 32, half = warp >> 2;
            const int r = qlane + lane, hh = r >> 6, i = r & 63;
            const int ncol = Nn >> 1;  // columns per thread
            float *dst = (KIND == 0) ? P.out + ((b * H + h0 + hh) * L + i) * L : P.out + (b * L + i) * row_shd + (int64_t)(h0 + hh) * D;
            for (int c0 = half * ncol; c0 < (half + 1) * ncol; c0 += 8) {
                float v[8];
                tc::tmem_ld8v(tmem_base + ((uint32_t)qlane << 16) + (uint32_t)(hh * Nn + c0), v);
                stcs8(dst + c0, v);
            }
        }
        tc::fence_before_sync();
        __syncthreads();
    }
    // a wait gave up while copies were still on their way: give them (bounded) time to land before the CTA's shared
    // memory is handed to another CTA
    if (TMA && !ok && pending) (void)tc::mbar_wait(full, full_phase);
    tc::fence_before_sync();
    __syncthreads();
    if (warp == 0) tc::tmem_dealloc(tmem_base, tmem_cols);
}

static size_t at_smem(int kind, int D, bool tma) {
    const int Ka = kind == 0 ? D : kAtL, Nn = kind == 0 ? kAtL : D;
    const size_t raw = tma ? 2 * (size_t)kAtL * 2 * D * 4 : 0;  // the raw boxes of x and y (kind 0)
    return 2 * (size_t)128 * Ka * 2 + 4 * (size_t)Nn * Ka * 2 + raw + 64 + (tma ? 1024 : 0);  // + room to align the carve to 1 KB
}

// HGQ_ATTN_TMA=0 in the environment keeps the per-thread loads (for comparisons).
static bool at_tma_enabled() {
    static const bool on = [] {
        const char *v = getenv("HGQ_ATTN_TMA");
        return !(v != nullptr && v[0] == '0');
    }();
    return on;
}

}  // namespace hgq

using namespace hgq;

extern "C" int hgq_attn_heads_supported(int64_t B, int L, int H, int D) {
    return (B > 0 && L == kAtL && H > 0 && H % 2 == 0 && (D == 16 || D == 32)) ? 1 : 0;
}

extern "C" int hgq_attn_heads_matmul(int kind, const float *x, const float *y, float *out, int64_t B, int L, int H, int D,
                                     unsigned *status, void *stream) {
    if (x == nullptr || y == nullptr || out == nullptr) return HGQ_ERR_NULL;
    if (kind < 0 || kind > 2) return HGQ_ERR_MODE;
    if (!hgq_attn_heads_supported(B, L, H, D)) return HGQ_ERR_SIZE;
    if (!aligned(x, 32) || !aligned(y, 32) || !aligned(out, 32)) return HGQ_ERR_ALIGN;  // 256-bit accesses
    {
        const int r = attn_ws_launch(kind, x, y, out, B, L, H, D, status, (cudaStream_t)stream);
        if (r < 0) return -r;
        if (r == 1) return check_launch();
    }
    AtParams p;
    p.x = x; p.y = y; p.out = out; p.status = status;
    p.B = B; p.H = H; p.D = D;
    p.num_tiles = B * (H / 2);
    // kind 0: tensor maps over this GPU's x and y alone, [B L, H D] with boxes [64, 2 D]
    CUtensorMap map_x, map_y;
    memset(&map_x, 0, sizeof(map_x));
    memset(&map_y, 0, sizeof(map_y));
    const int64_t rows_shd = B * L;
    const bool tma = kind == 0 && at_tma_enabled() && rows_shd < ((int64_t)1 << 31) &&
                     tma::make_map_2d(&map_x, x, rows_shd, (int64_t)H * D, (int64_t)H * D, 32, kAtL, true) &&
                     tma::make_map_2d(&map_y, y, rows_shd, (int64_t)H * D, (int64_t)H * D, 32, kAtL, true);
    const size_t smem = at_smem(kind, D, tma);
    int per_sm = (int)((228 * 1024) / (smem + 1024));
    const int cap = 4;  // measured optimum for all three kinds with per-thread loads (3 and 5 resident CTAs are both slower)
    if (per_sm > cap) per_sm = cap;
    if (per_sm < 1) return HGQ_ERR_SIZE;
    int64_t grid = (int64_t)num_sms() * per_sm;
    if (grid > p.num_tiles) grid = p.num_tiles;
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t ce = cudaSuccess;
#define HGQ_AT_LAUNCH(KIND_, TMA_)                                                                                          \
    do {                                                                                                                   \
        ce = cudaFuncSetAttribute(k_attn_heads<KIND_, TMA_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);      \
        if (ce != cudaSuccess) return (int)ce;                                                                             \
        k_attn_heads<KIND_, TMA_><<<(unsigned)grid, kAtThreads, smem, st>>>(p, map_x, map_y);                              \
    } while (0)
    if (kind == 0) { if (tma) HGQ_AT_LAUNCH(0, true); else HGQ_AT_LAUNCH(0, false); }
    else if (kind == 1) HGQ_AT_LAUNCH(1, false);
    else HGQ_AT_LAUNCH(2, false);
#undef HGQ_AT_LAUNCH
    return check_launch();
}
