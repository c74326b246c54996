// K2c (convolution weight gradient): dWq = patches(xq)^T @ G and dbq = sum G over all output pixels, with
// G = dY * (y > 0) written out once for the transposed convolution that yields dX.
//
// Stands in for the kernel/bias part of the autograd backward of QBaseConv.call (src/hgq/layers/conv.py:72-89).
// The patch matrix [B*OH*OW, KH*KW*C] is never materialised: per 128-pixel tile and per block of 128 patch columns
// the CTA gathers the image values straight into the transposed (MN-major) tensor-core operand as two bf16 terms
// (16 significant bits: exact for quantised activations of up to 16 bits), G likewise, and one thread issues
//   acc[kb] [128 k x N] += patches[:, kb]^T x G      (contraction over the tile's 128 pixels)
// with one fp32 accumulator per column block in tensor memory, kept across all tiles of the CTA.  A constant column of
// ones appended to the patch matrix makes row K of the product the bias gradient.  Per-CTA partials go to scratch and
// are summed in a fixed order by a second kernel, so the result does not depend on scheduling.
// Traffic: dY, y in and G out once (12 N bytes per pixel); the image is read through L1/L2 (each pixel serves up to
// KH*KW patches).
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdlib>

#include "hgq_common.cuh"
#include "tc05.cuh"

namespace hgq {

int cl_group_pad(int groups);  // qconv.cu: padding between the pixel arrays of consecutive channel groups

constexpr int kCwThreads = 256;
constexpr int kCwTileM = 128;
constexpr int kCwXTermBytes = 128 * 128 * 2;

struct CwParams {
    const float *x, *gy, *y;
    float *gm;          // masked gradient out (NULL: no activation, G = dY is used as it is)
    float *part;        // per-CTA partials [(K + 1) x N]
    unsigned *status;
    int64_t M, num_tiles;
    int K, N, Np, nkb;
    int H, W, C, OH, OW, KH, KW, sh, sw, dh, dw, pt, pl;
};

__device__ __forceinline__ void cw_split2(float v0, float v1, uint32_t &hi, uint32_t &lo) {
    const __nv_bfloat162 h2 = __floats2bfloat162_rn(v0, v1);
    hi = *reinterpret_cast<const uint32_t *>(&h2);
    const float r0 = __fsub_rn(v0, __uint_as_float(hi << 16));
    const float r1 = __fsub_rn(v1, __uint_as_float(hi & 0xffff0000u));
    const __nv_bfloat162 l2 = __floats2bfloat162_rn(r0, r1);
    lo = *reinterpret_cast<const uint32_t *>(&l2);
}

__global__ void __launch_bounds__(kCwThreads) k_qconv_wgrad(const CwParams P) {
    extern __shared__ __align__(128) unsigned char smem[];
    const int K = P.K, N = P.N, Np = P.Np, nkb = P.nkb;
    const int CGn = Np >> 3;
    const int g_term_bytes = kCwTileM * Np * 2;
    unsigned char *G = smem;
    unsigned char *X = G + 2 * g_term_bytes;
    int *koff4 = reinterpret_cast<int *>(X + 2 * kCwXTermBytes);   // per 4-column piece: image offset, -1 = ones, -2 = zero
    short *tap4 = reinterpret_cast<short *>(koff4 + nkb * 32);     // (dy << 8) | dx, tap displacement from the patch origin
    uint64_t *bar = reinterpret_cast<uint64_t *>(reinterpret_cast<unsigned char *>(tap4) + (nkb * 64 + 15) / 16 * 16);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bar + 1);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    uint32_t tmem_cols = 32;
    while ((int)tmem_cols < nkb * Np) tmem_cols <<= 1;

    if (tid == 0) {
        tc::mbar_init(bar, 1);
        tc::mbar_init_fence();
    }
    if (warp == 0) tc::tmem_alloc(tmem_slot, tmem_cols);
    for (int e = tid; e < nkb * 32; e += kCwThreads) {
        const int k = e << 2;
        if (k < K) {
            const int tap = k / P.C, c = k - tap * P.C, kh = tap / P.KW, kw = tap - kh * P.KW;
            const int dy = kh * P.dh, dx = kw * P.dw;
            koff4[e] = (dy * P.W + dx) * P.C + c;
            tap4[e] = (short)((dy << 8) | dx);
        } else {
            koff4[e] = (k == K) ? -1 : -2;
            tap4[e] = 0;
        }
    }
    for (int e = tid; e < 2 * kCwXTermBytes / 16; e += kCwThreads) reinterpret_cast<uint4 *>(X)[e] = make_uint4(0, 0, 0, 0);
    tc::fence_smem_to_async();
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t idesc = tc::make_idesc_bf16(Np, true, true);
    const uint32_t g_base = tc::smem_u32(G), x_base = tc::smem_u32(X);

    const int r8 = lane & 7, q4 = lane >> 3;
    const bool vec_n = (N % 4 == 0) && aligned(P.gy, 16) && (P.y == nullptr || aligned(P.y, 16)) &&
                       (P.gm == nullptr || aligned(P.gm, 16));
    const bool relu = P.y != nullptr;
    const int CG4g = (CGn + 3) >> 2, combos_g = 16 * CG4g;
    const int64_t ohw = (int64_t)P.OH * P.OW;
    // a single column block: groups that lie wholly in the zero padding stay zero for ever and are never rewritten
    const int live_kg = (nkb == 1) ? ((K >> 2) + 2) >> 1 : 16;  // 8-column groups that hold data or the ones column

    uint32_t phase = 0;
    bool ok = true, issued = false, first_tile = true;

    for (int64_t tile = blockIdx.x; tile < P.num_tiles && ok; tile += gridDim.x) {
        const int64_t row0 = tile * kCwTileM;
        // this thread's two pixel rows of the tile: local rows (h * 8 + warp) * 8 + r8
        int64_t pbase[2];
        int pih[2], piw[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int64_t row = row0 + (h * 8 + warp) * 8 + r8;
            if (row < P.M) {
                const int64_t b = row / ohw;
                const int rem = (int)(row - b * ohw);
                const int oh = rem / P.OW, ow = rem - oh * P.OW;
                pih[h] = oh * P.sh - P.pt;
                piw[h] = ow * P.sw - P.pl;
                pbase[h] = ((b * P.H + pih[h]) * P.W + piw[h]) * P.C;
            } else {
                pih[h] = -(1 << 20);  // every tap falls outside the image: the row gathers zeros
                piw[h] = 0;
                pbase[h] = 0;
            }
        }
        for (int kb = 0; kb < nkb && ok; ++kb) {
            // the previous product still reads both operand buffers
            if (issued) {
                const bool waited = (warp == 0) ? tc::mbar_wait(bar, phase) : true;
                phase ^= 1u;
                ok = __syncthreads_and(waited ? 1 : 0) != 0;
                if (!ok) break;
                issued = false;
            }
            if (kb == 0) {
                // ---- G = dY (* relu mask): out to memory for the dX pass, two bf16 terms to shared memory ----------------
                for (int u = 0; u * 8 < combos_g; ++u) {
                    const int c = u * 8 + warp;
                    const int mg = c / CG4g, kg = (c - mg * CG4g) * 4 + q4;
                    if (!(c < combos_g && kg < CGn)) continue;
                    const int64_t row = row0 + mg * 8 + r8;
                    const int n0 = kg * 8;
                    float g[8];
                    if (row < P.M && vec_n && n0 + 8 <= N) {
                        const float4 a0 = __ldcs(reinterpret_cast<const float4 *>(P.gy + row * N + n0));
                        const float4 a1 = __ldcs(reinterpret_cast<const float4 *>(P.gy + row * N + n0 + 4));
                        g[0] = a0.x; g[1] = a0.y; g[2] = a0.z; g[3] = a0.w; g[4] = a1.x; g[5] = a1.y; g[6] = a1.z; g[7] = a1.w;
                        if (relu) {
                            const float4 y0 = __ldcs(reinterpret_cast<const float4 *>(P.y + row * N + n0));
                            const float4 y1 = __ldcs(reinterpret_cast<const float4 *>(P.y + row * N + n0 + 4));
                            const float yy[8] = {y0.x, y0.y, y0.z, y0.w, y1.x, y1.y, y1.z, y1.w};
#pragma unroll
                            for (int j = 0; j < 8; ++j) g[j] = yy[j] > 0.f ? g[j] : 0.f;
                        }
                        if (P.gm != nullptr) {
                            *reinterpret_cast<float4 *>(P.gm + row * N + n0) = make_float4(g[0], g[1], g[2], g[3]);
                            *reinterpret_cast<float4 *>(P.gm + row * N + n0 + 4) = make_float4(g[4], g[5], g[6], g[7]);
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            const bool in = row < P.M && n0 + j < N;
                            float v = in ? __ldcs(P.gy + row * N + n0 + j) : 0.f;
                            if (in && relu) v = __ldcs(P.y + row * N + n0 + j) > 0.f ? v : 0.f;
                            if (in && P.gm != nullptr) P.gm[row * N + n0 + j] = v;
                            g[j] = v;
                        }
                    }
                    uint32_t hi[4], lo[4];
#pragma unroll
                    for (int j = 0; j < 8; j += 2) cw_split2(g[j], g[j + 1], hi[j >> 1], lo[j >> 1]);
                    const int off = (mg * CGn + kg) * 128 + r8 * 16;
                    *reinterpret_cast<uint4 *>(G + off) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
                    *reinterpret_cast<uint4 *>(G + g_term_bytes + off) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
                }
            }
            // ---- patches of column block kb, transposed operand: core (row/8, k/8) in a 16-group-wide buffer ------------
            int lo_any = 0;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int mg = h * 8 + warp;
                float4 v[8];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int kg = i * 4 + q4;
#pragma unroll
                    for (int hh = 0; hh < 2; ++hh) {
                        const int p4 = kb * 32 + kg * 2 + hh;
                        const int ko = koff4[p4];
                        float4 t = make_float4(ko == -1 ? 1.f : 0.f, 0.f, 0.f, 0.f);
                        if (ko >= 0) {
                            const int tp = tap4[p4];
                            const int ih = pih[h] + (tp >> 8), iw = piw[h] + (tp & 0xff);
                            if ((unsigned)ih < (unsigned)P.H && (unsigned)iw < (unsigned)P.W)
                                t = __ldg(reinterpret_cast<const float4 *>(P.x + pbase[h] + ko));
                        }
                        v[i * 2 + hh] = t;
                    }
                }
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int kg = i * 4 + q4;
                    if (kg >= live_kg) continue;
                    uint32_t hi[4], lo[4];
                    cw_split2(v[i * 2].x, v[i * 2].y, hi[0], lo[0]);
                    cw_split2(v[i * 2].z, v[i * 2].w, hi[1], lo[1]);
                    cw_split2(v[i * 2 + 1].x, v[i * 2 + 1].y, hi[2], lo[2]);
                    cw_split2(v[i * 2 + 1].z, v[i * 2 + 1].w, hi[3], lo[3]);
                    lo_any |= ((lo[0] | lo[1] | lo[2] | lo[3]) & 0x7fff7fffu) != 0;
                    const int off = (mg * 16 + kg) * 128 + r8 * 16;
                    *reinterpret_cast<uint4 *>(X + off) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
                    *reinterpret_cast<uint4 *>(X + kCwXTermBytes + off) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
                }
            }
            tc::fence_smem_to_async();
            const int n_x = __syncthreads_or(lo_any) ? 2 : 1;
            if (tid == 0) {
                tc::fence_after_sync();
                const uint32_t acc = tmem_base + (uint32_t)(kb * Np);
                for (int s = 0; s < kCwTileM / 16; ++s)
                    for (int tx = 0; tx < n_x; ++tx) {
                        const uint64_t da = tc::make_smem_desc(x_base + tx * kCwXTermBytes + s * (2 * 16 * 128), 16 * 128, 128);
                        for (int tg = 0; tg < 2; ++tg) {
                            const uint64_t db =
                                tc::make_smem_desc(g_base + tg * g_term_bytes + s * (2 * CGn * 128), (uint32_t)CGn * 128, 128);
                            tc::mma_bf16(acc, da, db, idesc, !(first_tile && s == 0 && tx == 0 && tg == 0));
                        }
                    }
                tc::commit(bar);
            }
            issued = true;
        }
        first_tile = false;
    }
    if (issued && ok) {
        const bool waited = (warp == 0) ? tc::mbar_wait(bar, phase) : true;
        ok = __syncthreads_and(waited ? 1 : 0) != 0;
    }
    if (!ok && tid == 0 && P.status) atomicOr(P.status, 1u);

    // ---- per-CTA partial: rows k < K are dWq, row K is dbq ------------------------------------------------------------------
    float *pw = P.part + (int64_t)blockIdx.x * ((int64_t)(K + 1) * N);
    if (ok && (int64_t)blockIdx.x < P.num_tiles) {
        tc::fence_after_sync();
        const int qlane = (warp & 3) * 32, half = warp >> 2;
        const int ncol = Np >> 1;
        for (int kb = 0; kb < nkb; ++kb) {
            const int k = kb * 128 + qlane + lane;
            for (int c0 = half * ncol; c0 < (half + 1) * ncol; c0 += 8) {
                float v[8];
                tc::tmem_ld8v(tmem_base + ((uint32_t)qlane << 16) + (uint32_t)(kb * Np + c0), v);
                if (k <= K)
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        if (c0 + j < N) pw[(int64_t)k * N + c0 + j] = v[j];
            }
        }
    } else {
        for (int e = tid; e < (K + 1) * N; e += kCwThreads) pw[e] = 0.f;
    }
    tc::fence_before_sync();
    __syncthreads();
    if (warp == 0) tc::tmem_dealloc(tmem_base, tmem_cols);
}

// Element e of the per-CTA partial records [dWq | dbq] summed over the CTAs into its own output array, in double and in a
// fixed order, so the result does not depend on scheduling.  A block owns eight consecutive elements; its 32 groups of
// eight lanes walk the records 32 apart (about ten loads per thread, all in flight together: the launch is pure latency
// on the critical path of a step).
constexpr int kCwS2Elems = 8;
__global__ void __launch_bounds__(kThreads) k_cw_stage2(const float *__restrict__ part, int64_t stride, float *__restrict__ dw,
                                                       int64_t nw, float *__restrict__ db, int64_t nb, int nparts) {
    __shared__ double red[kThreads / 32][kCwS2Elems];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, sub = lane >> 3, j = lane & 7;
    const int64_t e = (int64_t)blockIdx.x * kCwS2Elems + j;
    const int64_t n = nw + nb;
    double acc = 0.0;
    if (e < n) {
#pragma unroll 4
        for (int p = warp * 4 + sub; p < nparts; p += kThreads / 8) acc += (double)part[(int64_t)p * stride + e];
    }
    acc += __shfl_down_sync(0xffffffffu, acc, 16);
    acc += __shfl_down_sync(0xffffffffu, acc, 8);
    if (sub == 0) red[warp][j] = acc;
    __syncthreads();
    if (threadIdx.x < kCwS2Elems && e < n) {
        double a = 0.0;
#pragma unroll
        for (int w = 0; w < kThreads / 32; ++w) a += red[w][threadIdx.x];
        if (e < nw) dw[e] = (float)a;
        else db[e - nw] = (float)a;
    }
}


// ---- unit-stride variant: shifted windows of one staged image -------------------------------------------------------------
// With the padded images of the batch viewed as one line of pixels q (row pitch Wp, see the forward kernel), the weight
// gradient of tap (kh, kw) is  dW[kh, kw, c, n] = sum_q X[q + kh dil_h Wp + kw dil_w, c] * G[q, n]  with G zero at
// positions that are not outputs.  X and G of Pt consecutive positions are staged once as [term][group of 8
// channels][pixel] x 16 bytes, which is the MN-major core-matrix layout with the pixels as the contraction index.  The
// 128 rows of one A operand are "16 consecutive horizontal shifts x 8 channels": the stride between row groups is one
// pixel (16 dil_w bytes), so a single descriptor yields all KW taps of a kernel row at once (rows of shifts >= KW are
// computed and ignored).  One accumulator per (kh, channel group) in tensor memory, kept across the tiles of the CTA.
struct CsParams {
    const float *x, *gy, *y;
    float *gm, *part;
    unsigned *status;
    int64_t Q, num_tiles;
    int H, W, C, N, Np, OH, OW, Hp, Wp, KH, KW, dh, dw, pt, pl;
    int ncg, ng, Pt, npx, stack;
    int cgb, ggb;  // bytes between the pixel arrays of consecutive channel groups of the image / of G (padded: cl_group_pad)
    FastDiv div_img, div_row, div_cg;  // by Hp * Wp, by Wp and by the number of channel groups
};

// VEC_C: see k_qconv_s1 (scalar image loads live in their own instantiation).  NT threads per CTA: 256 when three CTAs
// fit an SM; when tensor memory or shared memory leave room for fewer, the CTA is made wider instead (512 / 1024 threads),
// so that the staging loops -- latency-bound global loads -- still have 24 to 32 warps per SM behind them (layer 2 of the
// small CNN ran one 8-warp CTA per SM: 12 % of the warp slots, 0.226 ms; see the profile summary).
template <bool VEC_C, int NT>
__global__ void __launch_bounds__(NT) k_qconv_wgrad_s1(const CsParams P) {
    extern __shared__ __align__(128) unsigned char smem[];
    const int Np = P.Np, ncg = P.ncg, ng = P.ng, Pt = P.Pt, npx = P.npx, N = P.N;
    const int cg_bytes = P.cgb, img_term = ncg * cg_bytes;
    const int gg_bytes = P.ggb, g_term = ng * gg_bytes;
    unsigned char *IMG = smem;
    unsigned char *GS = IMG + 2 * img_term;
    float *red = reinterpret_cast<float *>(GS + 2 * g_term);           // [256][8] bias-gradient partials
    uint64_t *bar = reinterpret_cast<uint64_t *>(red + NT * 8);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bar + 1);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int n_acc = P.KH * ncg;
    const int acc_cols = P.stack ? 2 * Np : Np;
    uint32_t tmem_cols = 32;
    while ((int)tmem_cols < n_acc * acc_cols) tmem_cols <<= 1;
    if (tid == 0) {
        tc::mbar_init(bar, (uint32_t)P.KH);  // one issuing thread per kernel row commits to it
        tc::mbar_init_fence();
    }
    if (warp == 0) tc::tmem_alloc(tmem_slot, tmem_cols);
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t idesc = tc::make_idesc_bf16(acc_cols, true, true);
    const uint32_t img_base = tc::smem_u32(IMG), g_base = tc::smem_u32(GS);
    const int HWp = P.Hp * P.Wp;
    constexpr bool vec_c = VEC_C;
    const bool half_group = (P.C & 7) != 0;
    const bool relu = P.y != nullptr;
    const int n_units_x = npx * ncg, n_units_g = Pt * ng;
    const int ng_shift = 31 - __clz(ng);
    const int my_g = tid % ng;  // NT is a multiple of ng: a thread always stages the same 8 output channels
    float db_r[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) db_r[j] = 0.f;

    uint32_t phase = 0;
    bool ok = true, first_tile = true;
    for (int64_t tile = blockIdx.x; tile < P.num_tiles && ok; tile += gridDim.x) {
        const int64_t q0 = tile * Pt;
        int lo_any = 0;
        // ---- image pixels q0 .. q0 + npx ------------------------------------------------------------------------------------
        for (int u0 = tid; u0 < n_units_x; u0 += 4 * NT) {
            float4 v[4][2];
            int dst[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int u = u0 + i * NT;
                v[i][0] = v[i][1] = make_float4(0.f, 0.f, 0.f, 0.f);
                dst[i] = -1;
                if (u < n_units_x) {
                    const int p = (int)fastdiv((uint32_t)u, P.div_cg), cg = u - p * ncg;
                    dst[i] = cg * cg_bytes + p * 16;
                    const int64_t q = q0 + p;
                    if (q < P.Q) {
                        const int b = (int)fastdiv((uint32_t)q, P.div_img);
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
                cw_split2(v[i][0].x, v[i][0].y, hi[0], lo[0]);
                cw_split2(v[i][0].z, v[i][0].w, hi[1], lo[1]);
                cw_split2(v[i][1].x, v[i][1].y, hi[2], lo[2]);
                cw_split2(v[i][1].z, v[i][1].w, hi[3], lo[3]);
                lo_any |= ((lo[0] | lo[1] | lo[2] | lo[3]) & 0x7fff7fffu) != 0;
                *reinterpret_cast<uint4 *>(IMG + dst[i]) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
                *reinterpret_cast<uint4 *>(IMG + img_term + dst[i]) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
            }
        }
        // ---- G = dY (* relu mask) at the output positions, zero elsewhere; masked gradient out -----------------------------------
        for (int u = tid; u < n_units_g; u += NT) {
            const int p = u >> ng_shift;  // ng is a power of two; u % ng == my_g
            const int64_t q = q0 + p;
            float g[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) g[j] = 0.f;
            const int n0 = my_g * 8;
            if (q < P.Q && n0 < N) {
                const int b = (int)fastdiv((uint32_t)q, P.div_img);
                const int rem = (int)((uint32_t)q - (uint32_t)b * (uint32_t)HWp);
                const int yp = (int)fastdiv((uint32_t)rem, P.div_row), xp = rem - yp * P.Wp;
                if (yp < P.OH && xp < P.OW) {
                    const int64_t o = (((int64_t)b * P.OH + yp) * P.OW + xp) * N + n0;
                    const bool second = n0 + 4 < N;  // N % 4 == 0 (checked on the host)
                    const float4 a0 = __ldcs(reinterpret_cast<const float4 *>(P.gy + o));
                    const float4 a1 = second ? __ldcs(reinterpret_cast<const float4 *>(P.gy + o + 4)) : make_float4(0.f, 0.f, 0.f, 0.f);
                    g[0] = a0.x; g[1] = a0.y; g[2] = a0.z; g[3] = a0.w; g[4] = a1.x; g[5] = a1.y; g[6] = a1.z; g[7] = a1.w;
                    if (relu) {
                        const float4 y0 = __ldcs(reinterpret_cast<const float4 *>(P.y + o));
                        const float4 y1 = second ? __ldcs(reinterpret_cast<const float4 *>(P.y + o + 4)) : make_float4(0.f, 0.f, 0.f, 0.f);
                        const float yy[8] = {y0.x, y0.y, y0.z, y0.w, y1.x, y1.y, y1.z, y1.w};
#pragma unroll
                        for (int j = 0; j < 8; ++j) g[j] = yy[j] > 0.f ? g[j] : 0.f;
                        *reinterpret_cast<float4 *>(P.gm + o) = make_float4(g[0], g[1], g[2], g[3]);
                        if (second) *reinterpret_cast<float4 *>(P.gm + o + 4) = make_float4(g[4], g[5], g[6], g[7]);
                    }
#pragma unroll
                    for (int j = 0; j < 8; ++j) db_r[j] = __fadd_rn(db_r[j], g[j]);
                }
            }
            uint32_t hi[4], lo[4];
#pragma unroll
            for (int j = 0; j < 8; j += 2) cw_split2(g[j], g[j + 1], hi[j >> 1], lo[j >> 1]);
            const int off = my_g * gg_bytes + p * 16;
            *reinterpret_cast<uint4 *>(GS + off) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
            *reinterpret_cast<uint4 *>(GS + g_term + off) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
        }
        tc::fence_smem_to_async();
        const int n_x = __syncthreads_or(lo_any) ? 2 : 1;
        // Issue is spread over KH threads (lane 0 of warps 0 .. KH-1, one kernel row each): a single thread building
        // descriptors and issuing every MMA of the tile would be the critical path while the whole CTA waits.
        // An MMA is bound by reading its 128-row A operand (4 KB) from shared memory whatever N is, so both bf16 terms of G
        // go through ONE MMA as 2 Np columns when tensor memory allows (`stack`; the term planes are contiguous, so one
        // uniform group stride covers them); the two halves of the accumulator are added in the final epilogue.
        if (lane == 0 && warp < P.KH) {
            tc::fence_after_sync();
            const int kh = warp;
            const int n_b = P.stack ? 1 : 2;
            const uint64_t db0 = tc::make_smem_desc(g_base, 128, (uint32_t)gg_bytes);
            for (int cg = 0; cg < ncg; ++cg) {
                const uint32_t acc = tmem_base + (uint32_t)((kh * ncg + cg) * acc_cols);
                const uint64_t da0 = tc::make_smem_desc(img_base + cg * cg_bytes + kh * P.dh * P.Wp * 16, 128, (uint32_t)(16 * P.dw));
                bool first = first_tile;
                for (int tx = 0; tx < n_x; ++tx)
                    for (int tg = 0; tg < n_b; ++tg) {
                        // the start-address field counts 16-byte units: + 16 per K step of 16 pixels (256 bytes)
                        uint64_t da = da0 + (uint64_t)((tx * img_term) >> 4);
                        uint64_t db = db0 + (uint64_t)((tg * g_term) >> 4);
#pragma unroll 4
                        for (int ks = 0; ks < Pt / 16; ++ks) {
                            tc::mma_bf16(acc, da, db, idesc, !first);
                            first = false;
                            da += 16;
                            db += 16;
                        }
                    }
            }
            tc::commit(bar);
        }
        first_tile = false;
        const bool waited = (warp == 0) ? tc::mbar_wait(bar, phase) : true;
        phase ^= 1u;
        ok = __syncthreads_and(waited ? 1 : 0) != 0;
    }
    if (!ok && tid == 0 && P.status) atomicOr(P.status, 1u);

    // ---- per-CTA partial: rows (tap, channel) of dWq, then dbq -----------------------------------------------------------------
    const int K = P.KH * P.KW * P.C;
    float *pw = P.part + (int64_t)blockIdx.x * ((int64_t)(K + 1) * N);
    if (ok) {
        tc::fence_after_sync();
        const int qlane = (warp & 3) * 32, half = (warp >> 2) & 1;
        const int ncol = Np >> 1;
        const int m = qlane + lane, kw = m >> 3, c8 = m & 7;  // accumulator row = (horizontal shift, channel in group)
        for (int kh = 0; kh < (warp < 8 ? P.KH : 0); ++kh)  // eight warps read the accumulators out
            for (int cg = 0; cg < ncg; ++cg) {
                const int c = cg * 8 + c8;
                const bool live = kw < P.KW && c < P.C;
                const int64_t krow = (int64_t)((kh * P.KW + kw) * P.C + c) * N;
                for (int c0 = half * ncol; c0 < (half + 1) * ncol; c0 += 8) {
                    float v[8];
                    tc::tmem_ld8v(tmem_base + ((uint32_t)qlane << 16) + (uint32_t)((kh * ncg + cg) * acc_cols + c0), v);
                    if (P.stack) {
                        float v2[8];
                        tc::tmem_ld8v(tmem_base + ((uint32_t)qlane << 16) + (uint32_t)((kh * ncg + cg) * acc_cols + Np + c0), v2);
#pragma unroll
                        for (int j = 0; j < 8; ++j) v[j] = __fadd_rn(v[j], v2[j]);
                    }
                    if (live)
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            if (c0 + j < N) pw[krow + c0 + j] = v[j];
                }
            }
    } else {
        for (int e = tid; e < K * N; e += NT) pw[e] = 0.f;
    }
    // bias gradient: threads with the same channel group are summed in a fixed order
    __syncthreads();
#pragma unroll
    for (int j = 0; j < 8; ++j) red[tid * 8 + j] = db_r[j];
    __syncthreads();
    if (tid < ng * 8) {
        const int g = tid >> 3, j = tid & 7;
        float a = 0.f;
        for (int t = g; t < NT; t += ng) a = __fadd_rn(a, red[t * 8 + j]);
        if (g * 8 + j < N) pw[(int64_t)K * N + g * 8 + j] = a;
    }
    tc::fence_before_sync();
    __syncthreads();
    if (warp == 0) tc::tmem_dealloc(tmem_base, tmem_cols);
}

struct CsGeom {
    int Np, Hp, Wp, ncg, ng, Pt, npx, grid, stack, nt;
    size_t smem;
    int64_t Q, tiles;
};

static int cs_geom(int64_t B, int H, int W, int C, int KH, int KW, int N, int OH, int OW, int dh, int dw, CsGeom &g) {
    if (B <= 0 || H <= 0 || W <= 0 || C <= 0 || KH <= 0 || KW <= 0 || N <= 0 || OH <= 0 || OW <= 0) return HGQ_ERR_SIZE;
    if (N % 4 != 0 || N > 128 || KW > 16) return HGQ_ERR_SIZE;
    g.Np = 16;
    while (g.Np < N) g.Np <<= 1;
    g.ng = g.Np / 8;
    g.ncg = (C + 7) / 8;
    if (KH * g.ncg * g.Np > 512) return HGQ_ERR_SIZE;
    g.Hp = OH + (KH - 1) * dh;
    g.Wp = OW + (KW - 1) * dw;
    g.Q = B * g.Hp * g.Wp;
    if (g.Q >= ((int64_t)1 << 31) || B * H * W * C >= ((int64_t)1 << 31)) return HGQ_ERR_SIZE;
    const int reach = (KH - 1) * dh * g.Wp + 15 * dw;  // furthest pixel an operand row may read beyond its own position
    g.Pt = 0;
    for (int pt = 512; pt >= 128; pt >>= 1) {
        const int npx = (pt + reach + 7) / 8 * 8;
        const size_t sm = 2 * (size_t)g.ncg * (npx * 16 + cl_group_pad(g.ncg)) + 2 * (size_t)g.ng * (pt * 16 + cl_group_pad(g.ng)) +
                          (size_t)kCwThreads * 32 + 64;
        if (sm <= 100 * 1024 || pt == 128) {
            g.Pt = pt; g.npx = npx; g.smem = sm;
            break;
        }
    }
    if (g.smem > 226 * 1024) return HGQ_ERR_SIZE;
    if (16 * dw >= (1 << 18)) return HGQ_ERR_SIZE;
    g.tiles = (g.Q + g.Pt - 1) / g.Pt;
    int per_sm = (int)((228 * 1024) / (g.smem + 1024));
    if (per_sm > 3) per_sm = 3;
    g.stack = (KH * g.ncg * 2 * g.Np <= 512 && 2 * g.Np <= 256) ? 1 : 0;
    int tm = 32;
    while (tm < KH * g.ncg * g.Np * (g.stack ? 2 : 1)) tm <<= 1;
    if (per_sm * tm > 512) per_sm = 512 / tm;
    if (per_sm < 1) return HGQ_ERR_SIZE;
    // fewer than three resident CTAs: wider CTAs (the bias-gradient scratch grows with the thread count)
    g.nt = kCwThreads;
    const int want = per_sm == 1 ? 1024 : (per_sm == 2 ? 512 : kCwThreads);
    if (want > kCwThreads) {
        const size_t sm2 = g.smem + (size_t)(want - kCwThreads) * 32;
        if (sm2 <= 226 * 1024 && (int)((228 * 1024) / (sm2 + 1024)) >= per_sm) {
            g.nt = want;
            g.smem = sm2;
        }
    }
    int64_t grid = (int64_t)num_sms() * per_sm;
    if (grid > g.tiles) grid = g.tiles;
    g.grid = (int)grid;
    return HGQ_OK;
}

struct CwGeom {
    int Np, nkb, grid;
    size_t smem;
    int64_t tiles, M;
};

static int cw_geom(int64_t B, int H, int W, int C, int KH, int KW, int N, int OH, int OW, CwGeom &g) {
    if (B <= 0 || H <= 0 || W <= 0 || C <= 0 || KH <= 0 || KW <= 0 || N <= 0 || OH <= 0 || OW <= 0) return HGQ_ERR_SIZE;
    if (C % 4 != 0 || N > 128) return HGQ_ERR_SIZE;
    if (B * H * W * C >= ((int64_t)1 << 31)) return HGQ_ERR_SIZE;
    const int K = KH * KW * C;
    g.Np = (N + 15) / 16 * 16;
    g.nkb = (K + 1 + 127) / 128;
    if (g.nkb * g.Np > 512) return HGQ_ERR_SIZE;
    g.M = B * OH * OW;
    g.tiles = (g.M + kCwTileM - 1) / kCwTileM;
    g.smem = 2 * (size_t)kCwTileM * g.Np * 2 + 2 * (size_t)kCwXTermBytes + (size_t)g.nkb * 32 * 4 + ((size_t)g.nkb * 64 + 15) / 16 * 16 + 64;
    int per_sm = (int)((228 * 1024) / (g.smem + 1024));
    if (per_sm > 2) per_sm = 2;
    if (per_sm == 2 && g.nkb * g.Np > 256) {  // two resident CTAs could not both hold their accumulators in tensor memory
        g.smem = 120 * 1024;
        per_sm = 1;
    }
    if (per_sm < 1 || g.smem > 226 * 1024) return HGQ_ERR_SIZE;
    int64_t grid = (int64_t)num_sms() * per_sm;
    if (grid > g.tiles) grid = g.tiles;
    g.grid = (int)grid;
    return HGQ_OK;
}

}  // namespace hgq

using namespace hgq;

extern "C" size_t hgq_qconv2d_wgrad_workspace(int64_t B, int H, int W, int C, int KH, int KW, int N, int OH, int OW) {
    CwGeom g;
    CsGeom gs;
    if (cw_geom(B, H, W, C, KH, KW, N, OH, OW, g) != HGQ_OK && cs_geom(B, H, W, C, KH, KW, N, OH, OW, 1, 1, gs) != HGQ_OK) return 0;
    if (C % 4 != 0 && cs_geom(B, H, W, C, KH, KW, N, OH, OW, 1, 1, gs) != HGQ_OK) return 0;  // only the unit-stride kernel takes such images
    return (size_t)3 * num_sms() * ((size_t)KH * KW * C + 1) * N * sizeof(float);
}

extern "C" int hgq_qconv2d_wgrad(const float *x, const float *gy, const float *y, float *gm, float *dwq, float *dbq, int64_t B,
                                 int H, int W, int C, int KH, int KW, int N, int OH, int OW, int stride_h, int stride_w,
                                 int dil_h, int dil_w, int pad_top, int pad_left, void *workspace, size_t workspace_bytes,
                                 unsigned *status, void *stream) {
    if (x == nullptr || gy == nullptr || dwq == nullptr) return HGQ_ERR_NULL;
    if ((y == nullptr) != (gm == nullptr)) return HGQ_ERR_NULL;
    if (stride_h <= 0 || stride_w <= 0 || dil_h <= 0 || dil_w <= 0) return HGQ_ERR_SIZE;
    if (KH * dil_h > 127 || KW * dil_w > 127 || pad_top < 0 || pad_left < 0) return HGQ_ERR_SIZE;
    if (!aligned(x, (C % 4 == 0) ? 16 : 4)) return HGQ_ERR_ALIGN;
    const int K = KH * KW * C;
    const int64_t stride = (int64_t)(K + 1) * N;
    cudaStream_t st = (cudaStream_t)stream;
    CsGeom gs;
    if (stride_h == 1 && stride_w == 1 && aligned(gy, 16) && (y == nullptr || (aligned(y, 16) && aligned(gm, 16))) &&
        cs_geom(B, H, W, C, KH, KW, N, OH, OW, dil_h, dil_w, gs) == HGQ_OK) {
        const size_t need_s = (size_t)gs.grid * stride * sizeof(float);
        if (workspace == nullptr || workspace_bytes < need_s) return HGQ_ERR_WORKSPACE;
        CsParams q;
        q.x = x; q.gy = gy; q.y = y; q.gm = gm; q.part = (float *)workspace; q.status = status;
        q.Q = gs.Q; q.num_tiles = gs.tiles;
        q.H = H; q.W = W; q.C = C; q.N = N; q.Np = gs.Np; q.OH = OH; q.OW = OW; q.Hp = gs.Hp; q.Wp = gs.Wp;
        q.KH = KH; q.KW = KW; q.dh = dil_h; q.dw = dil_w; q.pt = pad_top; q.pl = pad_left;
        q.ncg = gs.ncg; q.ng = gs.ng; q.Pt = gs.Pt; q.npx = gs.npx; q.stack = gs.stack;
        q.cgb = gs.npx * 16 + cl_group_pad(gs.ncg); q.ggb = gs.Pt * 16 + cl_group_pad(gs.ng);
        q.div_img = make_fastdiv((uint32_t)(gs.Hp * gs.Wp));
        q.div_row = make_fastdiv((uint32_t)gs.Wp);
        q.div_cg = make_fastdiv((uint32_t)gs.ncg);
        cudaError_t ce = cudaSuccess;
#define HGQ_CS_LAUNCH(VEC_, NT_)                                                                                             \
    do {                                                                                                                    \
        ce = cudaFuncSetAttribute(k_qconv_wgrad_s1<VEC_, NT_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)gs.smem);  \
        if (ce != cudaSuccess) return (int)ce;                                                                              \
        k_qconv_wgrad_s1<VEC_, NT_><<<gs.grid, NT_, gs.smem, st>>>(q);                                                      \
    } while (0)
        if (C % 4 == 0) {
            if (gs.nt == 1024) HGQ_CS_LAUNCH(true, 1024);
            else if (gs.nt == 512) HGQ_CS_LAUNCH(true, 512);
            else HGQ_CS_LAUNCH(true, 256);
        } else {
            if (gs.nt == 1024) HGQ_CS_LAUNCH(false, 1024);
            else if (gs.nt == 512) HGQ_CS_LAUNCH(false, 512);
            else HGQ_CS_LAUNCH(false, 256);
        }
#undef HGQ_CS_LAUNCH
        if (int e = check_launch()) return e;
        const int64_t nw = (int64_t)K * N;
        const int64_t nb1 = dbq != nullptr ? N : 0;
        k_cw_stage2<<<(unsigned)((nw + nb1 + kCwS2Elems - 1) / kCwS2Elems), kThreads, 0, st>>>(q.part, stride, dwq, nw, dbq, nb1, gs.grid);
        return check_launch();
    }
    CwGeom g;
    if (int e = cw_geom(B, H, W, C, KH, KW, N, OH, OW, g)) return e;
    const size_t need = (size_t)g.grid * stride * sizeof(float);
    if (workspace == nullptr || workspace_bytes < need) return HGQ_ERR_WORKSPACE;
    CwParams p;
    p.x = x; p.gy = gy; p.y = y; p.gm = gm; p.part = (float *)workspace; p.status = status;
    p.M = g.M; p.num_tiles = g.tiles; p.K = K; p.N = N; p.Np = g.Np; p.nkb = g.nkb;
    p.H = H; p.W = W; p.C = C; p.OH = OH; p.OW = OW; p.KH = KH; p.KW = KW;
    p.sh = stride_h; p.sw = stride_w; p.dh = dil_h; p.dw = dil_w; p.pt = pad_top; p.pl = pad_left;
    cudaError_t ce = cudaFuncSetAttribute(k_qconv_wgrad, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)g.smem);
    if (ce != cudaSuccess) return (int)ce;
    k_qconv_wgrad<<<g.grid, kCwThreads, g.smem, st>>>(p);
    if (int e = check_launch()) return e;
    const int64_t nw = (int64_t)K * N;
    const int64_t nb = dbq != nullptr ? N : 0;
    k_cw_stage2<<<(unsigned)((nw + nb + kCwS2Elems - 1) / kCwS2Elems), kThreads, 0, st>>>(p.part, stride, dwq, nw, dbq, nb, g.grid);
    return check_launch();
}
