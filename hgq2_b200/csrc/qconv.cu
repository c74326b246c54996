// K2d (unit-stride 2-D convolution, forward and input gradient): y = act(conv2d(x, wq) + bq), channels-last, as an
// implicit GEMM in which the tensor core reads shifted windows of ONE shared-memory copy of the image.
//
// Stands in for the contraction of QBaseConv.call (src/hgq/layers/conv.py:72-89) on already quantised operands, and,
// run over the output gradient with the flipped, transposed kernel, for its input gradient.
//
// The zero-padded image of the whole batch is viewed as one line of pixels q = (b * Hp + yp) * Wp + xp with
// Hp = OH + (KH-1) dil_h, Wp = OW + (KW-1) dil_w.  Tap (kh, kw) of output position q reads pixel
// q + kh dil_h Wp + kw dil_w: a constant shift.  A CTA stages Pt + halo consecutive pixels once, as bf16 terms laid out
// [term][channel group of 8][pixel] x 16 bytes.  Eight consecutive pixels of one channel group are then exactly one
// 8 x 16-byte core matrix of a K-major operand, so the A operand of "128 output positions x (tap, 8 channels)" is a
// descriptor whose start address is the staged image advanced by 16 * shift bytes -- no patch matrix, no gather, no
// copy per tap.  One MMA contracts two (tap, channel group) octets: the leading-dimension offset of the descriptor is
// the distance between the two octets' windows.  Positions whose window crosses the right or bottom edge are computed
// and dropped (Hp Wp / (OH OW) redundancy).
// Operands are split into two bf16 terms each (exact up to 16 significant bits, the range of quantised activations
// and weights; wider values are rounded at 2^-17 relative); products accumulate in fp32 in tensor memory.
// HBM-bound: 4 (C + N) bytes per output pixel; the image is read once plus the halo of each tile (L2 hits).
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "hgq_common.cuh"
#include "tc05.cuh"

namespace hgq {

int qconv2d_gather_supported(int64_t B, int H, int W, int C, int KH, int KW, int N, int OH, int OW);
int qconv2d_gather_launch(const float *x, int64_t B, int H, int W, int C, const float *wq, const float *bq, int activation,
                          float *y, int KH, int KW, int N, int OH, int OW, int stride_h, int stride_w, int dil_h, int dil_w,
                          int pad_top, int pad_left, unsigned *status, void *stream);

constexpr int kClThreads = 256;

struct ClParams {
    const float *x, *wq, *bq;
    float *y;
    unsigned *status;
    int64_t Q, num_tiles;      // padded positions of the whole batch; tiles of Pt positions
    int H, W, C, N, Np, OH, OW, Hp, Wp, KH, KW, dh, dw, pt, pl;
    int ncg, nsteps, MB, npx;  // channel groups, MMA K-steps, 128-row blocks per tile, staged pixels per tile
    int cgb;                   // bytes from one channel group's pixels to the next (see cl_group_pad)
    int act;
    FastDiv div_img, div_row, div_cg;  // by Hp * Wp, by Wp and by the number of channel groups
};

__device__ __forceinline__ void cl_split2(float v0, float v1, uint32_t &hi, uint32_t &lo) {
    const __nv_bfloat162 h2 = __floats2bfloat162_rn(v0, v1);
    hi = *reinterpret_cast<const uint32_t *>(&h2);
    const float r0 = __fsub_rn(v0, __uint_as_float(hi << 16));
    const float r1 = __fsub_rn(v1, __uint_as_float(hi & 0xffff0000u));
    const __nv_bfloat162 l2 = __floats2bfloat162_rn(r0, r1);
    lo = *reinterpret_cast<const uint32_t *>(&l2);
}

// VEC_C: the channel count is a multiple of four (16-byte pixels, 128-bit loads); the other instantiation reads images
// such as RGB with scalar loads and is kept apart so that the common case stays at 64 registers (four resident CTAs).
template <bool VEC_C>
__global__ void __launch_bounds__(kClThreads, VEC_C ? 4 : 3) k_qconv_s1(const ClParams P) {
    extern __shared__ __align__(128) unsigned char smem[];
    const int Np = P.Np, ncg = P.ncg, nsteps = P.nsteps, MB = P.MB, npx = P.npx;
    const int Pt = MB * 128;
    const int cg_bytes = P.cgb;                    // one channel group of one term: npx pixels of 16 bytes, padded
    const int img_term_bytes = ncg * cg_bytes;
    const int w_step_bytes = Np * 32;              // one K = 16 step of the weights: Np rows x 16 bf16
    const int w_term_bytes = nsteps * w_step_bytes;
    unsigned char *IMG = smem;                                          // [2 terms][ncg] x cg_bytes
    unsigned char *WT = IMG + 2 * img_term_bytes;                       // [2 terms][nsteps][Np/8][2 halves] x 128 B
    int2 *steps = reinterpret_cast<int2 *>(WT + 2 * w_term_bytes);      // per step: A start offset, A leading offset
    float *bias_s = reinterpret_cast<float *>(steps + nsteps);
    uint64_t *bar = reinterpret_cast<uint64_t *>(bias_s + Np);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bar + 1);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    uint32_t tmem_cols = 32;
    while ((int)tmem_cols < MB * Np) tmem_cols <<= 1;

    // ---- set-up -------------------------------------------------------------------------------------------------------
    if (tid == 0) {
        tc::mbar_init(bar, (uint32_t)MB);  // one issuing thread per 128-position block commits to it
        tc::mbar_init_fence();
    }
    if (warp == 0) tc::tmem_alloc(tmem_slot, tmem_cols);
    const int T = P.KH * P.KW, n_oct = ncg * T;
    // octet o = (channel group, tap), taps in (kh, kw) order: the window offsets grow with o
    for (int s = tid; s < nsteps; s += kClThreads) {
        const int o0 = 2 * s, o1 = 2 * s + 1;
        const int cg0 = o0 / T, t0 = o0 - cg0 * T;
        const int off0 = cg0 * cg_bytes + ((t0 / P.KW) * P.dh * P.Wp + (t0 % P.KW) * P.dw) * 16;
        int lbo = 0;  // odd octet count: the second half re-reads the first window against zero weights
        if (o1 < n_oct) {
            const int cg1 = o1 / T, t1 = o1 - cg1 * T;
            lbo = cg1 * cg_bytes + ((t1 / P.KW) * P.dh * P.Wp + (t1 % P.KW) * P.dw) * 16 - off0;
        }
        steps[s] = make_int2(off0, lbo);
    }
    for (int e = tid; e < Np; e += kClThreads) bias_s[e] = (P.bq != nullptr && e < P.N) ? __ldg(P.bq + e) : 0.f;
    // weights -> two bf16 terms; a thread converts the eight channels of (output channel n, octet o): step o/2, half o&1.
    // Eight loads in flight per thread and one 16-byte store per term: the conversion of a 288 x 64 kernel is 9 rounds
    // per CTA, and the eight threads of a quarter-warp fill the eight rows of one core matrix (no bank conflict).
    int w_lo = 0;
    const int np_shift = 31 - __clz(Np);  // Np is a power of two
    for (int e = tid; e < nsteps * 2 * Np; e += kClThreads) {
        const int n = e & (Np - 1), o = e >> np_shift;
        const int cg = o / T, t = o - cg * T;
        float w8[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int c = cg * 8 + j;
            w8[j] = (o < n_oct && c < P.C && n < P.N) ? __ldg(P.wq + ((int64_t)t * P.C + c) * P.N + n) : 0.f;
        }
        uint32_t hi[4], lo[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) cl_split2(w8[2 * j], w8[2 * j + 1], hi[j], lo[j]);
        const int off = (o >> 1) * w_step_bytes + ((n >> 3) * 2 + (o & 1)) * 128 + (n & 7) * 16;
        *reinterpret_cast<uint4 *>(WT + off) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
        *reinterpret_cast<uint4 *>(WT + w_term_bytes + off) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
        w_lo |= ((lo[0] | lo[1] | lo[2] | lo[3]) & 0x7fff7fffu) != 0;
    }
    const int n_w = __syncthreads_or(w_lo) ? 2 : 1;
    tc::fence_smem_to_async();
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t idesc = tc::make_idesc_bf16(Np, false, false);
    const uint32_t img_base = tc::smem_u32(IMG), w_base = tc::smem_u32(WT);
    const int HWp = P.Hp * P.Wp;
    constexpr bool vec_c = VEC_C;
    const bool half_group = (P.C & 7) != 0;  // C % 8 == 4: the last channel group holds four channels
    const float act_lo = (P.act == ACT_RELU) ? 0.f : -INFINITY;
    const bool vec_out = (P.N % 4 == 0) && aligned(P.y, 16);
    const int n_units = npx * ncg;

    uint32_t phase = 0;
    bool ok = true;
    for (int64_t tile = blockIdx.x; tile < P.num_tiles && ok; tile += gridDim.x) {
        const int64_t q0 = tile * Pt;
        // ---- stage the tile's pixels (with halo): fp32 -> two bf16 terms --------------------------------------------------
        int lo_any = 0;
        for (int u0 = tid; u0 < n_units; u0 += 4 * kClThreads) {
            float4 v[4][2];
            int dst[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int u = u0 + i * kClThreads;
                v[i][0] = v[i][1] = make_float4(0.f, 0.f, 0.f, 0.f);
                dst[i] = -1;
                if (u < n_units) {
                    const int p = (int)fastdiv((uint32_t)u, P.div_cg), cg = u - p * ncg;
                    dst[i] = cg * cg_bytes + p * 16;
                    const int64_t q = q0 + p;
                    if (q < P.Q) {
                        const int b = (int)fastdiv((uint32_t)q, P.div_img);   // Q < 2^31 (checked on the host)
                        const int rem = (int)((uint32_t)q - (uint32_t)b * (uint32_t)HWp);
                        const int yp = (int)fastdiv((uint32_t)rem, P.div_row), xp = rem - yp * P.Wp;
                        const int ih = yp - P.pt, iw = xp - P.pl;
                        if ((unsigned)ih < (unsigned)P.H && (unsigned)iw < (unsigned)P.W) {
                            const float *src = P.x + (((int64_t)b * P.H + ih) * P.W + iw) * P.C + cg * 8;
                            if (vec_c) {
                                v[i][0] = __ldg(reinterpret_cast<const float4 *>(src));
                                if (!half_group || cg + 1 < ncg) v[i][1] = __ldg(reinterpret_cast<const float4 *>(src + 4));
                            } else {  // channel count not a multiple of four (an RGB image): pixels are not 16-byte aligned
                                const int nc = min(8, P.C - cg * 8);
                                float t8[8];
#pragma unroll
                                for (int j = 0; j < 8; ++j) t8[j] = (j < nc) ? __ldg(src + j) : 0.f;
                                v[i][0] = make_float4(t8[0], t8[1], t8[2], t8[3]);
                                v[i][1] = make_float4(t8[4], t8[5], t8[6], t8[7]);
                            }
                        }
                    }
                }
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                if (dst[i] < 0) continue;
                uint32_t hi[4], lo[4];
                cl_split2(v[i][0].x, v[i][0].y, hi[0], lo[0]);
                cl_split2(v[i][0].z, v[i][0].w, hi[1], lo[1]);
                cl_split2(v[i][1].x, v[i][1].y, hi[2], lo[2]);
                cl_split2(v[i][1].z, v[i][1].w, hi[3], lo[3]);
                lo_any |= ((lo[0] | lo[1] | lo[2] | lo[3]) & 0x7fff7fffu) != 0;
                *reinterpret_cast<uint4 *>(IMG + dst[i]) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
                *reinterpret_cast<uint4 *>(IMG + img_term_bytes + dst[i]) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
            }
        }
        tc::fence_smem_to_async();
        const int n_x = __syncthreads_or(lo_any) ? 2 : 1;
        // ---- tensor cores: every 128-position block x every K step x the term pairs ------------------------------------------
        // lane 0 of warps 0 .. MB-1 each issue the MMAs of one 128-position block (its own accumulator): a single issuing
        // thread would be the critical path while the whole CTA waits
        if (lane == 0 && warp < MB) {
            tc::fence_after_sync();
            const int mb = warp;
            const uint32_t acc = tmem_base + (uint32_t)(mb * Np);
            bool first = true;
            for (int s = 0; s < nsteps; ++s) {
                const int2 so = steps[s];
                for (int tx = 0; tx < n_x; ++tx) {
                    const uint64_t da = tc::make_smem_desc(img_base + tx * img_term_bytes + so.x + mb * 2048, (uint32_t)so.y, 128);
                    for (int tw = 0; tw < n_w; ++tw) {
                        const uint64_t db = tc::make_smem_desc(w_base + tw * w_term_bytes + s * w_step_bytes, 128, 256);
                        tc::mma_bf16(acc, da, db, idesc, !first);
                        first = false;
                    }
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
        // ---- epilogue: + bias, activation, valid positions out ---------------------------------------------------------------
        tc::fence_after_sync();
        {
            const int qlane = (warp & 3) * 32, half = warp >> 2;
            const int ncol = Np >> 1;  // columns per thread: 8, 16, 32 or 64
            for (int mb = 0; mb < MB; ++mb) {
                const int64_t q = q0 + mb * 128 + qlane + lane;
                float *dst = nullptr;
                if (q < P.Q) {
                    const int b = (int)fastdiv((uint32_t)q, P.div_img);
                    const int rem = (int)((uint32_t)q - (uint32_t)b * (uint32_t)HWp);
                    const int yp = (int)fastdiv((uint32_t)rem, P.div_row), xp = rem - yp * P.Wp;
                    if (yp < P.OH && xp < P.OW) dst = P.y + (((int64_t)b * P.OH + yp) * P.OW + xp) * P.N;
                }
                for (int c0 = half * ncol; c0 < (half + 1) * ncol; c0 += 8) {
                    float v[8];
                    tc::tmem_ld8v(tmem_base + ((uint32_t)qlane << 16) + (uint32_t)(mb * Np + c0), v);
                    if (dst == nullptr) continue;
#pragma unroll
                    for (int j = 0; j < 8; ++j) v[j] = fmaxf(__fadd_rn(v[j], bias_s[c0 + j]), act_lo);
                    if (vec_out && c0 + 8 <= P.N) {
                        __stcs(reinterpret_cast<float4 *>(dst + c0), make_float4(v[0], v[1], v[2], v[3]));
                        __stcs(reinterpret_cast<float4 *>(dst + c0 + 4), make_float4(v[4], v[5], v[6], v[7]));
                    } else {
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            if (c0 + j < P.N) __stcs(dst + c0 + j, v[j]);
                    }
                }
            }
        }
        tc::fence_before_sync();
        __syncthreads();
    }
    tc::fence_before_sync();
    __syncthreads();
    if (warp == 0) tc::tmem_dealloc(tmem_base, tmem_cols);
}

// Padding between the pixel arrays of consecutive channel groups.  The staging threads of a quarter-warp hold consecutive
// (pixel, group) units: 8 / groups pixels of every group.  With group arrays a multiple of 128 bytes apart their 16-byte
// stores would fall on the same banks (2-, 4- or 8-way conflicts); a stride of 128 / groups bytes modulo 128 lets the
// eight stores tile the 32 banks.  Descriptors address windows in 16-byte units, so any multiple of 16 is a legal stride.
int cl_group_pad(int groups) { return groups >= 8 ? 16 : groups >= 4 ? 32 : groups >= 2 ? 64 : 0; }

struct ClGeom {
    int Np, Hp, Wp, ncg, nsteps, MB, npx, cgb, grid;
    size_t smem;
    int64_t Q, tiles;
};

static size_t cl_smem(int MB, int halo, int ncg, int nsteps, int Np, int &npx) {
    npx = (MB * 128 + halo + 7) / 8 * 8;
    return 2 * (size_t)ncg * (npx * 16 + cl_group_pad(ncg)) + 2 * (size_t)nsteps * Np * 32 + (size_t)nsteps * 8 + (size_t)Np * 4 + 64;
}

static int cl_geom(int64_t B, int H, int W, int C, int KH, int KW, int N, int OH, int OW, int dh, int dw, ClGeom &g) {
    if (B <= 0 || H <= 0 || W <= 0 || C <= 0 || KH <= 0 || KW <= 0 || N <= 0 || OH <= 0 || OW <= 0) return HGQ_ERR_SIZE;
    if (N > 128) return HGQ_ERR_SIZE;
    g.Np = 16;
    while (g.Np < N) g.Np <<= 1;
    g.Hp = OH + (KH - 1) * dh;
    g.Wp = OW + (KW - 1) * dw;
    g.Q = B * g.Hp * g.Wp;
    if (g.Q >= ((int64_t)1 << 31) || B * H * W * C >= ((int64_t)1 << 31)) return HGQ_ERR_SIZE;
    g.ncg = (C + 7) / 8;
    g.nsteps = (g.ncg * KH * KW + 1) / 2;
    const int halo = (KH - 1) * dh * g.Wp + (KW - 1) * dw;
    // the largest tile that keeps three CTAs resident (shared memory) and their accumulators within tensor memory
    g.MB = 0;
    for (int mb = 4; mb >= 1; mb >>= 1) {
        if (mb * g.Np > 128 && mb > 1) continue;
        int npx;
        const size_t sm = cl_smem(mb, halo, g.ncg, g.nsteps, g.Np, npx);
        if (sm <= 72 * 1024 || mb == 1) {
            g.MB = mb; g.npx = npx; g.smem = sm;
            g.cgb = npx * 16 + cl_group_pad(g.ncg);
            break;
        }
    }
    if (g.MB == 0 || g.smem > 226 * 1024) return HGQ_ERR_SIZE;
    // window offsets must fit the descriptor's 14-bit (x 16 bytes) leading-dimension field
    if ((size_t)g.ncg * g.cgb >= (1u << 18)) return HGQ_ERR_SIZE;
    g.tiles = (g.Q + g.MB * 128 - 1) / (g.MB * 128);
    int per_sm = (int)((228 * 1024) / (g.smem + 1024));
    if (per_sm > 4) per_sm = 4;
    int tm = 32;
    while (tm < g.MB * g.Np) tm <<= 1;
    if (per_sm * tm > 512) per_sm = 512 / tm;
    if (per_sm < 1) return HGQ_ERR_SIZE;
    int64_t grid = (int64_t)num_sms() * per_sm;
    if (grid > g.tiles) grid = g.tiles;
    g.grid = (int)grid;
    return HGQ_OK;
}

}  // namespace hgq

using namespace hgq;

extern "C" int hgq_qconv2d_supported(int64_t B, int H, int W, int C, int KH, int KW, int N, int OH, int OW) {
    return qconv2d_gather_supported(B, H, W, C, KH, KW, N, OH, OW);
}

extern "C" int hgq_qconv2d_unit_stride_supported(int64_t B, int H, int W, int C, int KH, int KW, int N, int OH, int OW,
                                                 int dil_h, int dil_w) {
    ClGeom g;
    return (dil_h > 0 && dil_w > 0 && cl_geom(B, H, W, C, KH, KW, N, OH, OW, dil_h, dil_w, g) == HGQ_OK) ? 1 : 0;
}

extern "C" int hgq_qconv2d_fwd(const float *x, int64_t B, int H, int W, int C, const float *wq, const float *bq, int activation,
                               float *y, int KH, int KW, int N, int OH, int OW, int stride_h, int stride_w, int dil_h,
                               int dil_w, int pad_top, int pad_left, unsigned *status, void *stream) {
    if (x == nullptr || wq == nullptr || y == nullptr) return HGQ_ERR_NULL;
    if (activation != ACT_NONE && activation != ACT_RELU) return HGQ_ERR_MODE;
    if (stride_h <= 0 || stride_w <= 0 || dil_h <= 0 || dil_w <= 0) return HGQ_ERR_SIZE;
    ClGeom g;
    const bool unit = stride_h == 1 && stride_w == 1 && pad_top >= 0 && pad_left >= 0 &&
                      cl_geom(B, H, W, C, KH, KW, N, OH, OW, dil_h, dil_w, g) == HGQ_OK;
    if (!unit)
        return qconv2d_gather_launch(x, B, H, W, C, wq, bq, activation, y, KH, KW, N, OH, OW, stride_h, stride_w, dil_h, dil_w,
                                     pad_top, pad_left, status, stream);
    if (!aligned(x, (C % 4 == 0) ? 16 : 4) || !aligned(y, 4)) return HGQ_ERR_ALIGN;
    ClParams p;
    p.x = x; p.wq = wq; p.bq = bq; p.y = y; p.status = status;
    p.Q = g.Q; p.num_tiles = g.tiles;
    p.H = H; p.W = W; p.C = C; p.N = N; p.Np = g.Np; p.OH = OH; p.OW = OW; p.Hp = g.Hp; p.Wp = g.Wp;
    p.KH = KH; p.KW = KW; p.dh = dil_h; p.dw = dil_w; p.pt = pad_top; p.pl = pad_left;
    p.ncg = g.ncg; p.nsteps = g.nsteps; p.MB = g.MB; p.npx = g.npx; p.cgb = g.cgb; p.act = activation;
    p.div_img = make_fastdiv((uint32_t)(g.Hp * g.Wp));
    p.div_row = make_fastdiv((uint32_t)g.Wp);
    p.div_cg = make_fastdiv((uint32_t)g.ncg);
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t ce;
    if (C % 4 == 0) {
        ce = cudaFuncSetAttribute(k_qconv_s1<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)g.smem);
        if (ce != cudaSuccess) return (int)ce;
        k_qconv_s1<true><<<g.grid, kClThreads, g.smem, st>>>(p);
    } else {
        ce = cudaFuncSetAttribute(k_qconv_s1<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)g.smem);
        if (ce != cudaSuccess) return (int)ce;
        k_qconv_s1<false><<<g.grid, kClThreads, g.smem, st>>>(p);
    }
    return check_launch();
}
