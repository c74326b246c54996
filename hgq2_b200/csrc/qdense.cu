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
// Shapes are skinny (N <= 128; K as far as the three weight terms, 6 K N bytes, fit shared memory beside the tile buffers:
// 256 inputs at 64 outputs, 1500 at 16) so the kernel is HBM-bound: 4 (K + N) bytes per row.  A persistent CTA
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
#include <stdlib.h>

#include "hgq_common.cuh"
#include "hgq_math.cuh"
#include "tc05.cuh"

namespace hgq {

constexpr int kQdThreads = 256;
constexpr int kQdTileM = 128;
constexpr int kQdKC = 64;                      // K slab held in shared memory at a time
constexpr int kQdATermBytes = kQdTileM * kQdKC * 2;  // 16 KB per bf16 term
constexpr int kQdStageBytes = kQdTileM * kQdKC * 4;  // 32 KB: one raw fp32 slab in flight
constexpr int kQdMaxTable = 8192;              // abs-max table entries (rows_period * K)

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
    int amax_direct;     // amax_part is the [rows_period * K] result itself: merge by atomic max
    unsigned *status;
    int64_t M;
    int K, N, Kpad, Npad;
    int rows_period;
    int rm, om, act, zero;
    int Kt;              // row stride of the packed parameter tables in shared memory (K rounded up to 8)
    int64_t num_tiles;
    // implicit-GEMM convolution: x is a channels-last image [B, H, W, C] (C % 4 == 0), row m = (b, oh, ow), column
    // k = ((kh * KW) + kw) * C + c reads x[b, oh*sh - pt + kh*dh, ow*sw - pl + kw*dw, c]; outside the image reads as zero
    int conv, H, W, C, OH, OW, KH, KW, sh, sw, dh, dw, pt, pl;
};

// Abs-max bookkeeping variants (the statistic is max over rows of |round(x)| per quantizer-table entry):
//   AMAX_NONE   not requested
//   AMAX_REGS   rows_period == 1, one K slab: a thread's 8 columns never change, maxima live in registers
//   AMAX_PLAIN  rows_period in {32, 64, 128}: rows that share a table entry fall to the same thread, plain smem update
//   AMAX_ATOMIC anything else: shared-memory atomics
enum : int { AMAX_NONE = 0, AMAX_REGS = 1, AMAX_PLAIN = 2, AMAX_ATOMIC = 3 };

// FASTQ: the input quantizer only rounds (training-mode WRAP, the default for activations).  Then the per-column
// scale 2^f comes from a one-byte-per-entry exponent table in shared memory (2^-f is derived by flipping the exponent)
// and the element loop is branch-free; everything else goes through the generic per-element routine.
template <bool FASTQ, bool CONV, int AMAX>
__global__ void __launch_bounds__(kQdThreads) k_qdense_fwd(const QdParams P) {
    extern __shared__ __align__(128) unsigned char smem[];
    // carve: A terms (hi, lo) | raw-slab staging | B terms | bias | quantizer tables | abs-max table | barrier + tmem slot
    unsigned char *A = smem;                                        // 2 x 16 KB
    unsigned char *stage = A + 2 * kQdATermBytes;                   // 32 KB, thread-private 16-byte slots
    unsigned char *B = stage + kQdStageBytes;                       // 3 x Kpad*Npad*2
    const int b_term_bytes = P.Kpad * P.Npad * 2;
    float *bias_s = reinterpret_cast<float *>(B + 3 * b_term_bytes);  // Npad floats
    // convolution: per 4-column piece of the K axis its address offset and its tap displacement (dy, dx)
    int *koff4 = reinterpret_cast<int *>(bias_s + P.Npad);
    const int kp4 = P.conv ? (P.Kpad >> 2) : 0;
    short *tap4 = reinterpret_cast<short *>(koff4 + kp4);          // (dy << 8) | (dx & 0xff), both int8
    const int conv_bytes = P.conv ? ((kp4 * 6 + 15) / 16) * 16 : 0;
    // FASTQ: one byte per entry, the biased exponent of 2^f, row stride Kt + 8 (8-byte reads of 8 rows hit 8 bank pairs)
    // generic: f, i as int8 and k as uint8, row stride Kt
    const int Ke = P.Kt + 8;
    const int tab_bytes = (P.qf != nullptr) ? (P.rows_period * Ke + 15) / 16 * 16 : 0;
    unsigned char *etab = reinterpret_cast<unsigned char *>(bias_s + P.Npad) + conv_bytes;
    signed char *ftab = reinterpret_cast<signed char *>(etab);
    signed char *itab = ftab + tab_bytes;
    unsigned char *ktab = reinterpret_cast<unsigned char *>(itab + tab_bytes);
    const int Ks = P.Kt + 4;                                        // abs-max table row: 16-byte accesses of 8 rows hit 8 bank groups
    float *amax_t = reinterpret_cast<float *>(etab + (FASTQ ? 1 : 3) * tab_bytes);
    const int amax_elems = (AMAX != AMAX_NONE) ? P.rows_period * Ks : 0;
    uint64_t *bar = reinterpret_cast<uint64_t *>(amax_t + amax_elems);
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
    for (int e = tid; e < Npad; e += kQdThreads) bias_s[e] = (P.bq != nullptr && e < N) ? __ldg(P.bq + e) : 0.f;
    for (int e = tid; e < amax_elems; e += kQdThreads) amax_t[e] = 0.f;
    for (int e = tid; e < kp4; e += kQdThreads) {
        const int k = e << 2, tap = k / P.C, c = k - tap * P.C, kh = tap / P.KW, kw = tap - kh * P.KW;
        const int dy = kh * P.dh - P.pt, dx = kw * P.dw - P.pl;
        koff4[e] = (dy * P.W + dx) * P.C + c;
        tap4[e] = (short)(((dy & 0xff) << 8) | (dx & 0xff));
    }
    if (P.qf != nullptr) {
        const bool need_ki = (P.om != OM_NONE);
        for (int e = tid; e < P.rows_period * P.Kt; e += kQdThreads) {
            const int pr = e / P.Kt, k = e % P.Kt;
            const bool in = k < K;
            const int fi = in ? __float2int_rn(__ldg(P.qf + pr * K + k)) : 0;
            if (FASTQ) {
                etab[pr * Ke + k] = (unsigned char)(max(-126, min(127, fi)) + 127);
            } else {
                ftab[e] = (signed char)fi;
                itab[e] = (in && need_ki) ? (signed char)__float2int_rn(__ldg(P.qi + pr * K + k)) : (signed char)0;
                ktab[e] = (in && need_ki) ? __ldg(P.qk + pr * K + k) : (unsigned char)0;
            }
        }
    }
    // zero the low-order term buffer once; it is rewritten only while some slab needs it
    for (int e = tid; e < kQdATermBytes / 16; e += kQdThreads) reinterpret_cast<uint4 *>(A + kQdATermBytes)[e] = make_uint4(0, 0, 0, 0);
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
    int lo_dirty = 0;
    float amax_r[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) amax_r[j] = 0.f;

    // slab mapping: lane = (q4, r8); warp w in iteration it handles row group mg = (it*8 + w) / 2 and the four
    // 8-column groups kg = ((it*8 + w) & 1) * 4 + q4.  A quarter-warp (8 lanes, r8 = 0..7) fills one 128-byte core matrix.
    const int r8 = lane & 7, q4 = lane >> 3;
    const int n_chunks = (Kpad + kQdKC - 1) / kQdKC;
    const bool vec_ok = (K % 4 == 0) && aligned(P.x, 16);  // convolution: C % 4 == 0 is checked on the host
    const float rbias = (P.rm == RM_RND) ? 0.5f : 0.f;
    const float act_lo = (P.act == ACT_RELU) ? 0.f : -INFINITY;

    // Software pipeline: while a slab is converted, multiplied and written out, the next slab's raw fp32 data is already
    // on its way from HBM into the staging buffer (cp.async, 16 bytes per request, each thread fetching exactly the
    // pieces it will itself consume, so no barrier guards the staging area).
    const bool use_async = vec_ok;
    // convolution: image offset of the patch origin and the origin's (ih, iw) for the four rows this thread serves in a
    // tile; recomputed when the prefetch moves on to a new tile
    int64_t cv_base[4];
    int cv_ih[4], cv_iw[4];
    auto prefetch = [&](int64_t t_row0, int t_ch) {
        if (P.conv && t_ch == 0) {
#pragma unroll
            for (int it = 0; it < 4; ++it) {
                const int64_t row = t_row0 + (((it * 8 + warp) >> 1) * 8) + r8;
                const int64_t b = row / ((int64_t)P.OH * P.OW);
                const int rem = (int)(row - b * ((int64_t)P.OH * P.OW));
                const int oh = rem / P.OW, ow = rem - oh * P.OW;
                cv_ih[it] = oh * P.sh;
                cv_iw[it] = ow * P.sw;
                cv_base[it] = ((b * P.H + cv_ih[it]) * P.W + cv_iw[it]) * P.C;
            }
        }
#pragma unroll
        for (int it = 0; it < 4; ++it) {
            const int c = it * 8 + warp, mg = c >> 1, kg = (c & 1) * 4 + q4;
            const int64_t row = t_row0 + mg * 8 + r8;
            const int k0 = t_ch * kQdKC + kg * 8;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                bool in = row < P.M && (k0 + 4 * h) < K;  // K % 4 == 0: a 16-byte piece is all inside or all outside
                const float *src = P.x;
                if (P.conv) {
                    if (in) {
                        const int p4 = (k0 + 4 * h) >> 2;
                        const int t = tap4[p4];
                        const int ih = cv_ih[it] + (int)(signed char)(t >> 8), iw = cv_iw[it] + (int)(signed char)(t & 0xff);
                        in = (unsigned)ih < (unsigned)P.H && (unsigned)iw < (unsigned)P.W;
                        if (in) src = P.x + cv_base[it] + koff4[p4];
                    }
                } else if (in) {
                    src = P.x + row * K + k0 + 4 * h;
                }
                const uint32_t dst = tc::smem_u32(stage) + (uint32_t)(((it * 2 + h) * kQdThreads + tid) * 16);
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(in ? 16 : 0) : "memory");
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    if (use_async && (int64_t)blockIdx.x < P.num_tiles) prefetch((int64_t)blockIdx.x * kQdTileM, 0);

    // table row of a slab row: (row0 + local row) mod rows_period, kept in 32-bit arithmetic (a mask when the period is a
    // power of two); the tile's base residue advances by a fixed amount from one tile of this CTA to the next.
    const uint32_t rp = (uint32_t)P.rows_period;
    const bool rp_pow2 = (rp & (rp - 1)) == 0;
    uint32_t base_pr = (uint32_t)(((int64_t)blockIdx.x * kQdTileM) % P.rows_period);
    const uint32_t step_pr = (uint32_t)(((int64_t)gridDim.x * kQdTileM) % P.rows_period);

    for (int64_t tile = blockIdx.x; tile < P.num_tiles && ok; tile += gridDim.x, base_pr = (base_pr + step_pr) % rp) {
        const int64_t row0 = tile * kQdTileM;
        for (int ch = 0; ch < n_chunks && ok; ++ch) {
            // ---- fetch + quantise + split one 128 x 64 slab ---------------------------------------
            int a_lo = 0, a_lo2 = 0;
            float xv[4][8];
            bool valid[4];
            if (use_async) {
                asm volatile("cp.async.wait_group 0;" ::: "memory");
#pragma unroll
                for (int it = 0; it < 4; ++it) {
                    const int c = it * 8 + warp, mg = c >> 1, kg = (c & 1) * 4 + q4;
                    valid[it] = (row0 + mg * 8 + r8) < P.M && (ch * kQdKC + kg * 8) < K;
                    const float4 v0 = *reinterpret_cast<const float4 *>(stage + ((it * 2 + 0) * kQdThreads + tid) * 16);
                    const float4 v1 = *reinterpret_cast<const float4 *>(stage + ((it * 2 + 1) * kQdThreads + tid) * 16);
                    xv[it][0] = v0.x; xv[it][1] = v0.y; xv[it][2] = v0.z; xv[it][3] = v0.w;
                    xv[it][4] = v1.x; xv[it][5] = v1.y; xv[it][6] = v1.z; xv[it][7] = v1.w;
                }
                // the staging slots are free again (their contents sit in registers): start the next slab's fetch
                int nch = ch + 1;
                int64_t ntile = tile;
                if (nch == n_chunks) { nch = 0; ntile = tile + gridDim.x; }
                if (ntile < P.num_tiles) prefetch(ntile * kQdTileM, nch);
            } else {
#pragma unroll
                for (int it = 0; it < 4; ++it) {
                    const int c = it * 8 + warp, mg = c >> 1, kg = (c & 1) * 4 + q4;
                    const int64_t row = row0 + mg * 8 + r8;
                    const int k0 = ch * kQdKC + kg * 8;
                    valid[it] = row < P.M && k0 < K;
#pragma unroll
                    for (int j = 0; j < 8; ++j) xv[it][j] = (valid[it] && k0 + j < K) ? __ldcs(P.x + row * K + k0 + j) : 0.f;
                }
            }
#pragma unroll
            for (int it = 0; it < 4; ++it) {
                const int c = it * 8 + warp, mg = c >> 1, kg = (c & 1) * 4 + q4;
                const int64_t row = row0 + mg * 8 + r8;
                const int k0 = ch * kQdKC + kg * 8;
                if (P.qf != nullptr && valid[it]) {
                    const uint32_t lr = base_pr + (uint32_t)(mg * 8 + r8);
                    const int pr = (int)(rp_pow2 ? (lr & (rp - 1)) : (lr % rp));
                    const int te = pr * Ks + k0;  // abs-max table index (multiple of 4 floats)
                    if (FASTQ) {
                        const uint2 eb = *reinterpret_cast<const uint2 *>(etab + pr * Ke + k0);
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            const uint32_t sbits = (((j < 4 ? eb.x : eb.y) >> ((j & 3) * 8)) & 0xffu) << 23;  // 2^f
                            // scaling by a power of two is exact, so one fused multiply-add gives RN(x * 2^f + bias) bit for bit
                            const float q = CONV ? rintf(__fmul_rn(xv[it][j], __uint_as_float(sbits)))
                                                 : floorf(__fmaf_rn(xv[it][j], __uint_as_float(sbits), rbias));
                            xv[it][j] = __fmul_rn(q, __uint_as_float(0x7F000000u - sbits));  // * 2^-f
                        }
                    } else {
                        const int teb = pr * P.Kt + k0;
                        const uint2 fb = *reinterpret_cast<const uint2 *>(ftab + teb);
                        const uint2 ib = *reinterpret_cast<const uint2 *>(itab + teb);
                        const uint2 kb = *reinterpret_cast<const uint2 *>(ktab + teb);
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            const int sh = (j & 3) * 8;
                            const int fi = (int)(signed char)(((j < 4 ? fb.x : fb.y) >> sh) & 0xff);
                            const int ii = (int)(signed char)(((j < 4 ? ib.x : ib.y) >> sh) & 0xff);
                            const float kf = (float)(((j < 4 ? kb.x : kb.y) >> sh) & 0xff);
                            float rounded;
                            const float o = quantize_rt(xv[it][j], kf, (float)ii, (float)fi, P.rm, P.om, P.zero != 0, rounded);
                            // the statistic is taken on the rounded value, the GEMM consumes the overflow-handled one
                            if (AMAX != AMAX_NONE && k0 + j < K) atomicMax(reinterpret_cast<unsigned *>(amax_t) + te + j, __float_as_uint(fabsf(rounded)));
                            xv[it][j] = o;
                        }
                    }
                    if (FASTQ && AMAX == AMAX_REGS) {
#pragma unroll
                        for (int j = 0; j < 8; ++j) amax_r[j] = fmaxf(amax_r[j], fabsf(xv[it][j]));
                    } else if (FASTQ && AMAX == AMAX_PLAIN) {
                        float4 m0 = *reinterpret_cast<float4 *>(amax_t + te), m1 = *reinterpret_cast<float4 *>(amax_t + te + 4);
                        m0.x = fmaxf(m0.x, fabsf(xv[it][0])); m0.y = fmaxf(m0.y, fabsf(xv[it][1]));
                        m0.z = fmaxf(m0.z, fabsf(xv[it][2])); m0.w = fmaxf(m0.w, fabsf(xv[it][3]));
                        m1.x = fmaxf(m1.x, fabsf(xv[it][4])); m1.y = fmaxf(m1.y, fabsf(xv[it][5]));
                        m1.z = fmaxf(m1.z, fabsf(xv[it][6])); m1.w = fmaxf(m1.w, fabsf(xv[it][7]));
                        *reinterpret_cast<float4 *>(amax_t + te) = m0;
                        *reinterpret_cast<float4 *>(amax_t + te + 4) = m1;
                    } else if (FASTQ && AMAX == AMAX_ATOMIC) {
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            if (k0 + j < K) atomicMax(reinterpret_cast<unsigned *>(amax_t) + te + j, __float_as_uint(fabsf(xv[it][j])));
                    }
                }
                // exact bf16 terms: a float whose low 16 bits are zero *is* a bf16 (top 16 bits), the common case
                uint32_t hi[4], lo[4] = {0u, 0u, 0u, 0u};
                uint32_t lowbits = 0u;
#pragma unroll
                for (int j = 0; j < 8; ++j) lowbits |= __float_as_uint(xv[it][j]);
                int my_lo = 0;
                if ((lowbits & 0xFFFFu) == 0u) {
#pragma unroll
                    for (int j = 0; j < 8; j += 2)
                        hi[j >> 1] = __byte_perm(__float_as_uint(xv[it][j]), __float_as_uint(xv[it][j + 1]), 0x7632);
                } else {
#pragma unroll
                    for (int j = 0; j < 8; j += 2) {
                        __nv_bfloat16 h0, l0, m0, h1, l1, m1;
                        tc::split3(xv[it][j], h0, l0, m0);
                        tc::split3(xv[it][j + 1], h1, l1, m1);
                        hi[j >> 1] = tc::pack2(h0, h1);
                        lo[j >> 1] = tc::pack2(l0, l1);
                        my_lo |= (lo[j >> 1] & 0x7fff7fffu) != 0;
                        a_lo2 |= (tc::pack2(m0, m1) & 0x7fff7fffu) != 0;
                    }
                }
                a_lo |= my_lo;
                const int off = (mg * 8 + kg) * 128 + r8 * 16;
                *reinterpret_cast<uint4 *>(A + off) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
                if (my_lo || lo_dirty) *reinterpret_cast<uint4 *>(A + kQdATermBytes + off) = make_uint4(lo[0], lo[1], lo[2], lo[3]);  // lo_dirty: see below
            }
            const int any_lo = __syncthreads_or(a_lo);
            const int any_lo2 = any_lo ? __syncthreads_or(a_lo2) : 0;
            // the epilogue parks the output block in the operand buffers, so the lo buffer never stays clean across tiles;
            // within a multi-slab tile it stays clean only if this slab left it so
            lo_dirty = any_lo;
            tc::fence_smem_to_async();
            __syncthreads();
            // ---- tensor-core GEMM on the slab -------------------------------------------------------
            const int kleft = Kpad - ch * kQdKC;
            const int ksteps = (kleft < kQdKC ? kleft : kQdKC) / 16;
            if (tid == 0) {
                tc::fence_after_sync();
                const int n_a = any_lo ? 2 : 1;
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
            // one warp polls the mbarrier, the others park at the CTA barrier; the outcome is CTA-wide so that nobody is left
            // behind at a later barrier
            bool waited = (warp == 0) ? tc::mbar_wait(bar, phase) : true;
            phase ^= 1u;
            ok = __syncthreads_and(waited ? 1 : 0) != 0;
            if (ok && any_lo2) {
                // rare: values with more than 16 significant bits.  Their third term goes through the (now idle) lo
                // buffer in a second pass; xv still holds the slab.
#pragma unroll
                for (int it = 0; it < 4; ++it) {
                    const int c = it * 8 + warp, mg = c >> 1, kg = (c & 1) * 4 + q4;
                    uint32_t t3[4];
#pragma unroll
                    for (int j = 0; j < 8; j += 2) {
                        __nv_bfloat16 h0, l0, m0, h1, l1, m1;
                        tc::split3(xv[it][j], h0, l0, m0);
                        tc::split3(xv[it][j + 1], h1, l1, m1);
                        t3[j >> 1] = tc::pack2(m0, m1);
                    }
                    *reinterpret_cast<uint4 *>(A + kQdATermBytes + (mg * 8 + kg) * 128 + r8 * 16) = make_uint4(t3[0], t3[1], t3[2], t3[3]);
                }
                lo_dirty = 1;
                tc::fence_smem_to_async();
                __syncthreads();
                if (tid == 0) {
                    tc::fence_after_sync();
                    for (int s = 0; s < ksteps; ++s) {
                        const uint64_t da = tc::make_smem_desc(a_base + kQdATermBytes + s * 256, 128, sbo_a);
                        for (int tw = 0; tw < n_w; ++tw) {
                            const uint64_t db = tc::make_smem_desc(b_base + tw * b_term_bytes + (ch * (kQdKC / 16) + s) * 256, 128, sbo_b);
                            tc::mma_bf16(tmem_base, da, db, idesc, true);
                        }
                    }
                    tc::commit(bar);
                }
                waited = (warp == 0) ? tc::mbar_wait(bar, phase) : true;
                phase ^= 1u;
                ok = __syncthreads_and(waited ? 1 : 0) != 0;
            }
            if (!ok && tid == 0 && P.status) atomicOr(P.status, ST_TIMEOUT);
        }
        if (!ok) break;
        // ---- epilogue: TMEM -> registers -> bias, activation -> shared memory -> coalesced global stores ----------
        // The accumulator is taken in blocks of W = min(Npad, 64) columns.  Thread (lane quarter q, half h) reads W/2
        // columns of its row in one tcgen05.ld, applies bias and activation and parks them in the (idle) operand
        // buffers with an XOR swizzle on the 16-byte chunk index; then all threads copy the block out so that a warp
        // writes whole contiguous lines.
        tc::fence_after_sync();
        {
            const int W = Npad < 64 ? Npad : 64;       // block width (floats), 16 / 32 / 64
            const int C = W >> 2;                      // 16-byte chunks per staged row
            const int wc = W >> 1;                     // columns per thread: 8 / 16 / 32
            const int qlane = (warp & 3) * 32, half = warp >> 2;
            const int r = qlane + lane;                // row of the tile held by this thread
            float *ost = reinterpret_cast<float *>(A);  // 128 x W floats <= 32 KB
            for (int cb = 0; cb < Npad; cb += W) {
                float v[32];
                const uint32_t taddr = tmem_base + ((uint32_t)qlane << 16) + (uint32_t)(cb + half * wc);
                if (wc == 32) tc::tmem_ld32v(taddr, v);
                else if (wc == 16) tc::tmem_ld16v(taddr, v);
                else tc::tmem_ld8v(taddr, v);
                const int swz = (C == 4) ? ((r >> 1) & 3) : (r & 7);
#pragma unroll
                for (int j = 0; j < 32; j += 4) {
                    if (j < wc) {
                        const int c = half * wc + j;   // column inside the block
                        const float4 b = *reinterpret_cast<const float4 *>(bias_s + cb + c);
                        float4 o;
                        o.x = fmaxf(__fadd_rn(v[j], b.x), act_lo); o.y = fmaxf(__fadd_rn(v[j + 1], b.y), act_lo);
                        o.z = fmaxf(__fadd_rn(v[j + 2], b.z), act_lo); o.w = fmaxf(__fadd_rn(v[j + 3], b.w), act_lo);
                        *reinterpret_cast<float4 *>(ost + r * W + (((c >> 2) ^ swz) << 2)) = o;
                    }
                }
                __syncthreads();
                const int ncols = (N - cb) < W ? (N - cb) : W;  // valid columns of this block
                const int64_t rows_here = (P.M - row0) < kQdTileM ? (P.M - row0) : kQdTileM;
                if ((N & 3) == 0) {
                    const int cv = ncols >> 2;  // valid chunks per row
                    const bool cv_pow2 = (cv & (cv - 1)) == 0;
                    const int cv_shift = 31 - __clz(cv);
                    for (int g = tid; g < (int)rows_here * cv; g += kQdThreads) {
                        const int rr = cv_pow2 ? (g >> cv_shift) : (g / cv);
                        const int c4 = g - rr * cv;
                        const int sw = (C == 4) ? ((rr >> 1) & 3) : (rr & 7);
                        const float4 o = *reinterpret_cast<const float4 *>(ost + rr * W + ((c4 ^ sw) << 2));
                        __stcs(reinterpret_cast<float4 *>(P.y + (row0 + rr) * N + cb) + c4, o);
                    }
                } else {
                    for (int g = tid; g < (int)rows_here * ncols; g += kQdThreads) {
                        const int rr = g / ncols, c = g - rr * ncols;
                        const int sw = (C == 4) ? ((rr >> 1) & 3) : (rr & 7);
                        __stcs(P.y + (row0 + rr) * N + cb + c, ost[rr * W + ((((c >> 2) ^ sw) << 2) | (c & 3))]);
                    }
                }
                __syncthreads();  // the staging block is reused by the next column block / the next slab
            }
        }
        lo_dirty = 1;
        tc::fence_before_sync();
        __syncthreads();  // all TMEM reads done before the next tile's first MMA overwrites the accumulator
    }

    // ---- tear-down ----------------------------------------------------------------------------------
    __syncthreads();
    if (AMAX != AMAX_NONE) {
        if (AMAX == AMAX_REGS) {  // a thread's columns: kg = (warp & 1) * 4 + q4 in every iteration
            const int k0 = ((warp & 1) * 4 + q4) * 8;
#pragma unroll
            for (int j = 0; j < 8; ++j)
                if (k0 + j < K) atomicMax(reinterpret_cast<unsigned *>(amax_t) + k0 + j, __float_as_uint(amax_r[j]));
            __syncthreads();
        }
        const int table = P.rows_period * K;
        if (P.amax_direct) {
            for (int e = tid; e < table; e += kQdThreads) {
                const unsigned v = __float_as_uint(amax_t[(e / K) * Ks + (e % K)]);
                if (v != 0u) atomicMax(P.amax_part + e, v);
            }
        } else {
            unsigned *dst = P.amax_part + (int64_t)blockIdx.x * table;
            for (int e = tid; e < table; e += kQdThreads) dst[e] = __float_as_uint(amax_t[(e / K) * Ks + (e % K)]);
        }
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

int qdense_ws_launch(const float *x, const float *qf, int rows_period, int round_mode, const float *wq, const float *bq,
                     int activation, float *y, unsigned *amax_part, int amax_direct, float *pool_out, int pool_rows,
                     float pool_scale, int64_t M, int K, int N, int Kpad, int Npad, int Kt, unsigned *status, cudaStream_t st,
                     int *grid);

bool qdense_ws_pool_supported(int64_t M, int K, int N, int Kpad, int Npad, int Kt, int rows_period, int pool_rows, bool want_amax);

// HGQ_QDENSE_WS=0 in the environment keeps every call on the general kernel (for comparisons).
static bool ws_enabled() {
    static const bool on = [] {
        const char *v = getenv("HGQ_QDENSE_WS");
        return !(v != nullptr && v[0] == '0');
    }();
    return on;
}

struct QdGeom {
    int Kpad, Npad, Kt, grid;
    size_t smem;
    int64_t tiles;
};

static int qd_geom(int64_t M, int K, int N, int rows_period, bool want_amax, bool fastq, QdGeom &g, int kmax = 4096) {
    if (M <= 0 || K <= 0 || N <= 0 || rows_period <= 0) return HGQ_ERR_SIZE;
    if (K > kmax || N > 128) return HGQ_ERR_SIZE;
    if (want_amax && (int64_t)rows_period * K > kQdMaxTable) return HGQ_ERR_SIZE;
    g.Kpad = (K + 15) / 16 * 16;
    g.Npad = pow2ceil(N < 16 ? 16 : N);
    const size_t table = want_amax ? (size_t)rows_period * K : 0;
    (void)table;
    g.Kt = (K + 7) / 8 * 8;
    if ((size_t)rows_period * (g.Kt + 8) > 16384) return HGQ_ERR_SIZE;
    const size_t tab_bytes = ((size_t)rows_period * (g.Kt + 8) + 15) / 16 * 16;
    // A terms (2), staging, B terms (3), bias, quantizer tables (3 byte planes), abs-max table, barrier + TMEM slot
    g.smem = 2 * (size_t)kQdATermBytes + kQdStageBytes + 3 * (size_t)g.Kpad * g.Npad * 2 + (size_t)g.Npad * 4 +
             (fastq ? 1 : 3) * tab_bytes +
             (want_amax ? (size_t)rows_period * (g.Kt + 4) * 4 : 0) + 64 + (size_t)g.Kpad * 2 + 32;
    if (g.smem > 226 * 1024) return HGQ_ERR_SIZE;
    g.tiles = (M + kQdTileM - 1) / kQdTileM;
    int per_sm = (int)((228 * 1024) / (g.smem + 1024));  // 228 KB of shared memory per SM, 1 KB reserved per resident CTA
    if (per_sm > 4) per_sm = 4;
    if (per_sm < 1) per_sm = 1;
    // TMEM: 512 columns per SM
    const int cols = g.Npad < 32 ? 32 : g.Npad;
    if (per_sm * cols > 512) per_sm = 512 / cols;
    int64_t grid = (int64_t)num_sms() * per_sm;
    if (grid > g.tiles) grid = g.tiles;
    g.grid = (int)grid;
    return HGQ_OK;
}

}  // namespace hgq

using namespace hgq;

extern "C" size_t hgq_qdense_fwd_workspace(int64_t M, int K, int N, int rows_period) {
    QdGeom g;
    if (qd_geom(M, K, N, rows_period, true, false, g) != HGQ_OK) return 0;
    return (size_t)num_sms() * 4 * rows_period * K * sizeof(unsigned);  // room for the largest grid any variant launches
}

extern "C" int hgq_qdense_fwd_pooled_supported(int64_t M, int K, int N, int rows_period, int pool_rows, int want_absmax) {
    QdGeom g;
    if (qd_geom(M, K, N, rows_period, want_absmax != 0, true, g) != HGQ_OK || !ws_enabled()) return 0;
    return qdense_ws_pool_supported(M, K, N, g.Kpad, g.Npad, g.Kt, rows_period, pool_rows, want_absmax != 0) ? 1 : 0;
}

extern "C" int hgq_qdense_fwd(const float *x, const uint8_t *qk, const float *qi, const float *qf, int rows_period,
                              int round_mode, int overflow_mode, unsigned flags, const float *wq, const float *bq,
                              int activation, float *y, float *absmax, int64_t M, int K, int N, void *workspace,
                              size_t workspace_bytes, unsigned *status, void *stream) {
    return hgq_qdense_fwd_pooled(x, qk, qi, qf, rows_period, round_mode, overflow_mode, flags, wq, bq, activation, y, absmax, nullptr,
                                 0, 0.f, M, K, N, workspace, workspace_bytes, status, stream);
}

extern "C" int hgq_qdense_fwd_pooled(const float *x, const uint8_t *qk, const float *qi, const float *qf, int rows_period,
                                     int round_mode, int overflow_mode, unsigned flags, const float *wq, const float *bq,
                                     int activation, float *y, float *absmax, float *pool_out, int pool_rows, float pool_scale,
                                     int64_t M, int K, int N, void *workspace, size_t workspace_bytes, unsigned *status,
                                     void *stream) {
    if (x == nullptr || wq == nullptr || y == nullptr) return HGQ_ERR_NULL;
    if (round_mode < 0 || round_mode > 2 || overflow_mode < 0 || overflow_mode > 3) return HGQ_ERR_MODE;
    if (activation != ACT_NONE && activation != ACT_RELU) return HGQ_ERR_MODE;
    if (flags & ~(HGQ_FLAG_TRAINING | HGQ_FLAG_ZERO_NONPOS | HGQ_FLAG_ABSMAX_ACCUMULATE)) return HGQ_ERR_MODE;
    const bool direct = (flags & HGQ_FLAG_ABSMAX_ACCUMULATE) != 0 && absmax != nullptr;
    int om = overflow_mode;
    if (om == OM_WRAP && (flags & HGQ_FLAG_TRAINING)) om = OM_NONE;
    const int zero = (flags & HGQ_FLAG_ZERO_NONPOS) ? 1 : 0;
    if (zero && om == OM_NONE) return HGQ_ERR_MODE;
    if (qf != nullptr && om != OM_NONE && (qk == nullptr || qi == nullptr)) return HGQ_ERR_NULL;
    if (absmax != nullptr && qf == nullptr) return HGQ_ERR_NULL;
    QdGeom g;
    if (int e = qd_geom(M, K, N, rows_period, absmax != nullptr, (qf != nullptr) && (om == OM_NONE), g)) return e;
    const size_t need = (absmax && !direct) ? (size_t)g.grid * rows_period * K * sizeof(unsigned) : 0;
    if (need && (workspace == nullptr || workspace_bytes < need)) return HGQ_ERR_WORKSPACE;
    QdParams p;
    p.x = x; p.qk = qk; p.qi = qi; p.qf = qf; p.wq = wq; p.bq = bq; p.y = y;
    p.amax_part = absmax ? (direct ? (unsigned *)absmax : (unsigned *)workspace) : nullptr;
    p.amax_direct = direct ? 1 : 0;
    p.status = status;
    p.M = M; p.K = K; p.N = N; p.Kpad = g.Kpad; p.Npad = g.Npad; p.Kt = g.Kt;
    p.rows_period = rows_period; p.rm = round_mode; p.om = om; p.act = activation; p.zero = zero;
    p.num_tiles = g.tiles;
    p.conv = 0;
    cudaStream_t st = (cudaStream_t)stream;
    const bool fastq = (qf != nullptr) && (om == OM_NONE);
    const bool conv = (round_mode == RM_RND_CONV);
    if (fastq && ws_enabled()) {
        // the common training case has a warp-specialised kernel of its own
        int ws_grid = 0;
        const int r = qdense_ws_launch(x, qf, rows_period, round_mode, wq, bq, activation, y, p.amax_part, p.amax_direct, pool_out,
                                       pool_rows, pool_scale, M, K, N, g.Kpad, g.Npad, g.Kt, status, st, &ws_grid);
        if (r < 0) return -r;
        if (r == 1) {
            if (int e = check_launch()) return e;
            if (absmax && !direct) {
                const int table = rows_period * K;
                k_amax_stage2<<<(table + kThreads - 1) / kThreads, kThreads, 0, st>>>((const unsigned *)workspace, absmax, table, ws_grid);
                return check_launch();
            }
            return HGQ_OK;
        }
    }
    if (pool_out != nullptr) return HGQ_ERR_SIZE;  // row-group sums exist in the warp-specialised kernel's bulk-store path only
    int amax_mode = AMAX_NONE;
    if (absmax) {
        if (!fastq) amax_mode = AMAX_ATOMIC;
        else if (rows_period == 1 && g.Kpad <= kQdKC) amax_mode = AMAX_REGS;
        else if (rows_period == 32 || rows_period == 64 || rows_period == 128) amax_mode = AMAX_PLAIN;
        else amax_mode = AMAX_ATOMIC;
    }
#define HGQ_QD_LAUNCH(FQ, CV, AM)                                                                                     \
    do {                                                                                                              \
        cudaError_t ce = cudaFuncSetAttribute(k_qdense_fwd<FQ, CV, AM>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                              (int)g.smem);                                                           \
        if (ce != cudaSuccess) return (int)ce;                                                                        \
        k_qdense_fwd<FQ, CV, AM><<<g.grid, kQdThreads, g.smem, st>>>(p);                                              \
    } while (0)
    if (!fastq) {
        if (amax_mode == AMAX_NONE) HGQ_QD_LAUNCH(false, false, AMAX_NONE);
        else HGQ_QD_LAUNCH(false, false, AMAX_ATOMIC);
    } else if (conv) {
        switch (amax_mode) {
            case AMAX_NONE: HGQ_QD_LAUNCH(true, true, AMAX_NONE); break;
            case AMAX_REGS: HGQ_QD_LAUNCH(true, true, AMAX_REGS); break;
            case AMAX_PLAIN: HGQ_QD_LAUNCH(true, true, AMAX_PLAIN); break;
            default: HGQ_QD_LAUNCH(true, true, AMAX_ATOMIC); break;
        }
    } else {
        switch (amax_mode) {
            case AMAX_NONE: HGQ_QD_LAUNCH(true, false, AMAX_NONE); break;
            case AMAX_REGS: HGQ_QD_LAUNCH(true, false, AMAX_REGS); break;
            case AMAX_PLAIN: HGQ_QD_LAUNCH(true, false, AMAX_PLAIN); break;
            default: HGQ_QD_LAUNCH(true, false, AMAX_ATOMIC); break;
        }
    }
#undef HGQ_QD_LAUNCH
    if (int e = check_launch()) return e;
    if (absmax && !direct) {
        const int table = rows_period * K;
        k_amax_stage2<<<(table + kThreads - 1) / kThreads, kThreads, 0, st>>>((const unsigned *)workspace, absmax, table, g.grid);
        return check_launch();
    }
    return HGQ_OK;
}


namespace hgq {

// Convolution by patch gather on the dense kernel (any stride); the extern "C" entry points that dispatch to it live with
// the unit-stride kernel.
int qconv2d_gather_supported(int64_t B, int H, int W, int C, int KH, int KW, int N, int OH, int OW) {
    if (B <= 0 || H <= 0 || W <= 0 || C <= 0 || KH <= 0 || KW <= 0 || N <= 0 || OH <= 0 || OW <= 0) return 0;
    if (C % 4 != 0) return 0;
    QdGeom g;
    return qd_geom(B * OH * OW, KH * KW * C, N, 1, false, false, g, 640) == HGQ_OK ? 1 : 0;
}

int qconv2d_gather_launch(const float *x, int64_t B, int H, int W, int C, const float *wq, const float *bq, int activation,
                               float *y, int KH, int KW, int N, int OH, int OW, int stride_h, int stride_w, int dil_h,
                               int dil_w, int pad_top, int pad_left, unsigned *status, void *stream) {
    if (x == nullptr || wq == nullptr || y == nullptr) return HGQ_ERR_NULL;
    if (activation != ACT_NONE && activation != ACT_RELU) return HGQ_ERR_MODE;
    if (!qconv2d_gather_supported(B, H, W, C, KH, KW, N, OH, OW)) return HGQ_ERR_SIZE;
    if (stride_h <= 0 || stride_w <= 0 || dil_h <= 0 || dil_w <= 0) return HGQ_ERR_SIZE;
    if (pad_top < -127 || pad_top > 127 || pad_left < -127 || pad_left > 127 || KH * dil_h > 127 || KW * dil_w > 127) return HGQ_ERR_SIZE;
    if (!aligned(x, 16) || !aligned(y, 4)) return HGQ_ERR_ALIGN;
    const int64_t M = B * OH * OW;
    const int K = KH * KW * C;
    QdGeom g;
    if (int e = qd_geom(M, K, N, 1, false, false, g, 640)) return e;
    QdParams p{};
    p.x = x; p.wq = wq; p.bq = bq; p.y = y; p.status = status;
    p.M = M; p.K = K; p.N = N; p.Kpad = g.Kpad; p.Npad = g.Npad; p.Kt = g.Kt;
    p.rows_period = 1; p.rm = RM_RND; p.om = OM_NONE; p.act = activation; p.zero = 0;
    p.num_tiles = g.tiles;
    p.conv = 1; p.H = H; p.W = W; p.C = C; p.OH = OH; p.OW = OW; p.KH = KH; p.KW = KW;
    p.sh = stride_h; p.sw = stride_w; p.dh = dil_h; p.dw = dil_w; p.pt = pad_top; p.pl = pad_left;
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t ce = cudaFuncSetAttribute(k_qdense_fwd<false, false, AMAX_NONE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)g.smem);
    if (ce != cudaSuccess) return (int)ce;
    k_qdense_fwd<false, false, AMAX_NONE><<<g.grid, kQdThreads, g.smem, st>>>(p);
    return check_launch();
}

}  // namespace hgq
