// K4: bit-accurate quantised softmax, forward and backward, one pass each.
//
// Stands in for QSoftmax.call (src/hgq/layers/softmax.py:114-132) in its stable form without mask, together with the
// four table quantizers of its two QUnaryFunctionLUT sub-layers (src/hgq/layers/activation.py:58-61) and the layer's
// own output quantizer (src/hgq/layers/core/base.py:105-110), in training mode:
//     d = max_j(s) - s;  a = Q1(d);  e = exp(-a * scaler);  b = Q2(e);  S = sum_j b;  t = Q3(S);
//     v = 1 / (t + eps);  u = Q4(v);  z = b * u;  y = Q5(z)
// Q1..Q4 have one (k, i, f) each (heterogeneous_axis = ()), Q5 has a [rows_period, L] table (the bitwidth tensor of the
// scores with the batch axis set to 1).  The reference runs this as ~25 eager element-wise passes over the score
// tensor per direction; here a warp owns a row (L = 32 / 64 / 128 scores, 1 / 2 / 4 per lane), keeps it in registers,
// and the score tensor is read once (forward) or twice (backward: s and dL/dy) and written once.
// HBM-bound: 8 B per score forward, 12 B backward.
//
// Side outputs of the forward: the abs-max statistics the WRAP quantizers track (scalars for Q1 and Q3, a table for Q5;
// Q2 and Q4 are table outputs, which the layer forces to SAT).
// The backward recomputes the chain from s and accumulates the surrogate gradients of all five quantizers: scalars are
// summed per thread, then per CTA in a fixed order, then over CTAs by a second kernel; the Q5 table gradient is owned
// by the warp lanes of the CTA that handles that table row for a range of batches.
#include <cuda_runtime.h>

#include <cstdlib>

#include "hgq_common.cuh"
#include "hgq_math.cuh"

namespace hgq {

struct SQuant {            // one stateless quantizer with scalar parameters (device pointers to single elements)
    const uint8_t *k;
    const float *i, *f;
    int rm, om;            // om: OM_NONE (rounding only), OM_SAT, OM_SAT_SYM
};

struct SmParams {
    const float *s;        // [R, L] scores, R = batches * rows_period
    const float *gy;       // backward: dL/dy
    float *y;              // forward output / backward ds
    SQuant q1, q2, q3, q4;
    const uint8_t *k5;     // Q5 tables [rows_period, L]
    const float *i5, *f5;
    int rm5, om5;
    float scaler, eps;
    unsigned *amax1;       // forward: scalar abs-max of round(d) (as bits), or nullptr
    unsigned *amax3;       // forward: scalar abs-max of round(S) (as bits), or nullptr
    unsigned *amax5;       // forward: [rows_period, L] abs-max of round(z), or nullptr
    float *part;           // backward: per-CTA partials: 8 scalars (di1, df1, di2, df2, di3, df3, di4, df4), then per
                           // (split, table row) L floats of df5 and L floats of di5
    int64_t batches;
    int rows_period, L, splits;
};

constexpr int kSmWarps = 8;
constexpr float kNegInf = -3.402823466e38f;

// A quantizer boiled down to launch-uniform constants, so that forward and backward are branch-free:
// rounding-only quantizers get infinite clip bounds, SAT / SAT_SYM differ only in `lo` and in one select.
struct QC {
    float s, inv;      // 2^f, 2^-f
    float lo, hi;      // clip bounds (+-inf when the quantizer only rounds)
    float ci, cf;      // ln2 * 2^i, ln2 * 2^-f
    float kf, rbias;   // keep_negative as float; 0.5 for RND, 0 for TRN
    bool conv, sym;    // round-half-even; symmetric lower bound
    bool clips;        // false: the quantizer only rounds (launch-uniform, so branching on it does not diverge)
};

__device__ __forceinline__ QC make_qc(float kf, float i, float f, int rm, int om) {
    QC c;
    const Params p = make_params(kf, i, f);
    c.s = p.s; c.inv = p.inv; c.kf = kf;
    c.conv = (rm == RM_RND_CONV);
    c.rbias = (rm == RM_RND) ? 0.5f : 0.f;
    c.sym = (om == OM_SAT_SYM);
    c.clips = (om != OM_NONE);
    if (om == OM_NONE) {
        c.lo = -INFINITY; c.hi = INFINITY; c.ci = 0.f; c.cf = 0.f;
    } else {
        c.hi = __fsub_rn(p.p2i, p.inv);
        c.lo = (om == OM_SAT) ? __fmul_rn(-p.p2i, kf) : __fmul_rn(-c.hi, kf);
        c.ci = __fmul_rn(p.p2i, kLn2);
        c.cf = __fmul_rn(p.inv, kLn2);
    }
    return c;
}

__device__ __forceinline__ QC load_q(const SQuant &q) {
    const float f = __ldg(q.f);
    const float kf = (q.om == OM_NONE) ? 0.f : (float)__ldg(q.k);
    const float i = (q.om == OM_NONE) ? 0.f : __ldg(q.i);
    return make_qc(kf, i, f, q.rm, q.om);
}

// Mode knowledge at compile time.  CL: 0 = the quantizer only rounds, 1 = it clips, 2 = decided at run time (launch-uniform
// flag).  RD: 0 = it rounds by floor(x 2^f + bias) (RND: bias 1/2, TRN: bias 0), 1 = round-half-even, 2 = decided at run
// time.
template <int RD>
__device__ __forceinline__ float qc_round(float x, const QC &c) {
    const float xs = __fmul_rn(x, c.s);
    const float q = (RD == 1 || (RD == 2 && c.conv)) ? rintf(xs) : floorf(__fadd_rn(xs, c.rbias));
    return __fmul_rn(q, c.inv);
}
template <int CL, int RD>
__device__ __forceinline__ float qc_fwd(float x, const QC &c, float &rounded) {
    rounded = qc_round<RD>(x, c);
    if (CL == 0) return rounded;
    return clipf(rounded, c.lo, c.hi);  // +-inf bounds when a run-time quantizer only rounds
}
// same arithmetic as quantize_grad<> in hgq_math.cuh, with the mode folded into the constants; xq = qc_round(x, c) is
// passed in by callers that already have it from the forward chain
template <int CL>
__device__ __forceinline__ void qc_bwd_r(float g, float x, float xq, const QC &c, float &dx, float &di, float &df) {
    const float df_r = __fmul_rn(__fmul_rn(__fsub_rn(xq, x), -kLn2), g);
    if (CL == 0 || (CL == 2 && !c.clips)) {  // rounding only: straight-through value gradient, no integer-bit gradient
        dx = g;
        di = 0.f;
        df = df_r;
        return;
    }
    const bool pass = (xq >= c.lo) && (xq <= c.hi);
    const bool to_hi = (xq > c.hi) || (c.hi < c.lo);
    const bool to_lo = (xq < c.lo) && (c.lo < c.hi);
    const float ghi = to_hi ? g : 0.f;
    const float glo = to_lo ? -__fmul_rn(g, c.kf) : 0.f;
    dx = pass ? g : 0.f;
    const float m = __fadd_rn(ghi, glo);
    di = c.sym ? __fmul_rn(m, c.ci) : __fadd_rn(__fmul_rn(ghi, c.ci), __fmul_rn(glo, c.ci));
    df = __fadd_rn(pass ? df_r : 0.f, __fmul_rn(c.sym ? m : ghi, c.cf));
}

// Kernel variants: 0 = every mode decided at run time; 1 .. 4 = the training set-up of the layer: Q1, Q3, Q5 round by
// floor, the two table outputs Q2 and Q4 saturate, Q3 and Q5 (WRAP quantizers) only round; Q1 only rounds (1, 3) or
// saturates (2, 4); the table outputs round by floor (1, 2) or half-even (3, 4: what the layer forces them to).
template <int V> struct Modes {
    static constexpr int C1 = V == 0 ? 2 : ((V == 2 || V == 4) ? 1 : 0);
    static constexpr int C2 = V == 0 ? 2 : 1;
    static constexpr int C3 = V == 0 ? 2 : 0;
    static constexpr int C4 = C2;
    static constexpr int C5 = C3;
    static constexpr int RA = V == 0 ? 2 : 0;                  // rounding of Q1, Q3, Q5
    static constexpr int RT = V == 0 ? 2 : (V >= 3 ? 1 : 0);   // rounding of the table outputs Q2, Q4
};

template <int VE>
__device__ __forceinline__ void load_row(const float *p, int lane, float (&v)[VE]) {
    if (VE == 8) {
        float t[8];
        ldcs8(p + lane * 8, t);
#pragma unroll
        for (int j = 0; j < VE; ++j) v[j] = t[j];
    } else if (VE == 4) {
        const float4 t = __ldcs(reinterpret_cast<const float4 *>(p) + lane);
        v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
    } else if (VE == 2) {
        const float2 t = __ldcs(reinterpret_cast<const float2 *>(p) + lane);
        v[0] = t.x; v[1] = t.y;
    } else {
        v[0] = __ldcs(p + lane);
    }
}

template <int VE>
__device__ __forceinline__ void store_row(float *p, int lane, const float (&v)[VE]) {
    if (VE == 8) {
        float t[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) t[j] = v[j < VE ? j : 0];
        stcs8(p + lane * 8, t);
    } else if (VE == 4) __stcs(reinterpret_cast<float4 *>(p) + lane, make_float4(v[0], v[1], v[2], v[3]));
    else if (VE == 2) __stcs(reinterpret_cast<float2 *>(p) + lane, make_float2(v[0], v[1]));
    else __stcs(p + lane, v[0]);
}

// Reductions over the LPR lanes that share a row (LPR = 32: the warp; 16: each half of it holds a row of its own).
// Fixed butterflies: every lane of the row ends with the same value.
template <int LPR>
__device__ __forceinline__ float row_max(float v) {
#pragma unroll
    for (int o = LPR / 2; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
template <int LPR>
__device__ __forceinline__ float row_sum(float v) {
#pragma unroll
    for (int o = LPR / 2; o > 0; o >>= 1) v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
template <int LPR>
__device__ __forceinline__ int row_sum_int(int v) {
#pragma unroll
    for (int o = LPR / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Forward chain of one row.  Fills b[] (quantised exponentials), returns u and the intermediate scalars.
template <int VE, int LPR, int V>
__device__ __forceinline__ void chain_fwd(const SmParams &P, const QC &q1, const QC &q2, const QC &q3, const QC &q4,
                                          const float (&s)[VE], float (&e)[VE], float (&b)[VE], float &m, float &S,
                                          float &t_rounded, float &v, float &u, float (&ra)[VE], float (&rb)[VE],
                                          float &u_rounded) {
    using Mo = Modes<V>;
    float mx = kNegInf;
#pragma unroll
    for (int j = 0; j < VE; ++j) mx = fmaxf(mx, s[j]);
    m = row_max<LPR>(mx);
    float part = 0.f;
#pragma unroll
    for (int j = 0; j < VE; ++j) {
        const float a = qc_fwd<Mo::C1, Mo::RA>(__fsub_rn(m, s[j]), q1, ra[j]);
        e[j] = expf(__fmul_rn(-a, P.scaler));
        b[j] = qc_fwd<Mo::C2, Mo::RT>(e[j], q2, rb[j]);
        part = __fadd_rn(part, b[j]);
    }
    S = row_sum<LPR>(part);
    const float t = qc_fwd<Mo::C3, Mo::RA>(S, q3, t_rounded);
    v = __fdiv_rn(1.f, __fadd_rn(t, P.eps));
    u = qc_fwd<Mo::C4, Mo::RT>(v, q4, u_rounded);
}

template <int VE>
__device__ __forceinline__ void load_q5(const SmParams &P, int p, int col0, QC (&q5)[VE]) {
#pragma unroll
    for (int j = 0; j < VE; ++j) {
        const int c = p * P.L + col0 + j;
        q5[j] = make_qc((P.om5 == OM_NONE) ? 0.f : (float)__ldg(P.k5 + c), (P.om5 == OM_NONE) ? 0.f : __ldg(P.i5 + c),
                        __ldg(P.f5 + c), P.rm5, P.om5);
    }
}

// grid = (rows_period, splits); CTA (p, sp) handles table row p for the batches sp, sp + splits, ...: row-group g of the CTA
// (8 warps x 32 / LPR rows per warp) takes every (8 * 32 / LPR)-th of those, so the Q5 statistics of table row p are owned
// by this CTA's lanes.  A row-group without a batch left repeats the first group's row of its warp and discards the result.
template <int VE, int LPR, int V>
__global__ void __launch_bounds__(kSmWarps * 32, VE == 8 ? 3 : 1) k_qsoftmax_fwd(const SmParams P) {
    using Mo = Modes<V>;
    constexpr int RPW = 32 / LPR;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int rl = lane % LPR, sub = lane / LPR;
    const int p = blockIdx.x, sp = blockIdx.y, L = P.L;
    const QC q1 = load_q(P.q1), q2 = load_q(P.q2), q3 = load_q(P.q3), q4 = load_q(P.q4);
    QC q5[VE];
    load_q5<VE>(P, p, rl * VE, q5);
    float am5[VE], am3 = 0.f, am1 = 0.f;
#pragma unroll
    for (int j = 0; j < VE; ++j) am5[j] = 0.f;
    const int64_t step = (int64_t)P.splits * kSmWarps * RPW;
    for (int64_t bt0 = (int64_t)sp + (int64_t)(warp * RPW) * P.splits; bt0 < P.batches; bt0 += step) {
        const int64_t mine = bt0 + (int64_t)sub * P.splits;
        const bool valid = mine < P.batches;
        const int64_t row = (valid ? mine : bt0) * P.rows_period + p;
        float s[VE], e[VE], b[VE], y[VE];
        load_row<VE>(P.s + row * L, rl, s);
        float m, S, tr, v, u, ur, ra[VE], rb[VE];
        chain_fwd<VE, LPR, V>(P, q1, q2, q3, q4, s, e, b, m, S, tr, v, u, ra, rb, ur);
        if (valid) {
            am3 = fmaxf(am3, fabsf(tr));
#pragma unroll
            for (int j = 0; j < VE; ++j) {
                float r;
                am1 = fmaxf(am1, fabsf(ra[j]));
                y[j] = qc_fwd<Mo::C5, Mo::RA>(__fmul_rn(b[j], u), q5[j], r);
                am5[j] = fmaxf(am5[j], fabsf(r));
            }
            store_row<VE>(P.y + row * L, rl, y);
        }
    }
    if (P.amax5 != nullptr) {
#pragma unroll
        for (int j = 0; j < VE; ++j) atomicMax(P.amax5 + p * L + rl * VE + j, __float_as_uint(am5[j]));
    }
    if (P.amax3 != nullptr && rl == 0) atomicMax(P.amax3, __float_as_uint(am3));
    if (P.amax1 != nullptr) {
        am1 = row_max<32>(am1);
        if (lane == 0) atomicMax(P.amax1, __float_as_uint(am1));
    }
}

// Resident CTAs: the per-row dependency chains (reductions, exp, divide) need many warps to hide; measured on 134 M
// scores with a warp per row: 1.46 ms at two CTAs per SM, 1.22 at three, 1.16 at four.  With eight scores per lane the
// chain of a lane is long enough by itself: two CTAs without spills (0.69 ms) beat three with spills (0.70).
template <int VE, int LPR, int V>
__global__ void __launch_bounds__(kSmWarps * 32, VE == 8 ? 2 : 4) k_qsoftmax_bwd(const SmParams P) {
    using Mo = Modes<V>;
    constexpr int RPW = 32 / LPR;
    constexpr int LL = VE * LPR;  // = L
    __shared__ float red[kSmWarps][8];
    __shared__ float red5[kSmWarps * RPW][2][LL];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int rl = lane % LPR, sub = lane / LPR;
    const int p = blockIdx.x, sp = blockIdx.y, L = P.L;
    const QC q1 = load_q(P.q1), q2 = load_q(P.q2), q3 = load_q(P.q3), q4 = load_q(P.q4);
    QC q5[VE];
    load_q5<VE>(P, p, rl * VE, q5);
    float acc[8];  // di1, df1, di2, df2, di3, df3, di4, df4 (per thread; the per-row scalars are added by one lane per row)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    float adf5[VE], adi5[VE];
#pragma unroll
    for (int j = 0; j < VE; ++j) adf5[j] = adi5[j] = 0.f;

    const int64_t step = (int64_t)P.splits * kSmWarps * RPW;
    for (int64_t bt0 = (int64_t)sp + (int64_t)(warp * RPW) * P.splits; bt0 < P.batches; bt0 += step) {
        const int64_t mine = bt0 + (int64_t)sub * P.splits;
        const bool valid = mine < P.batches;
        const int64_t row = (valid ? mine : bt0) * P.rows_period + p;
        float s[VE], g[VE], e[VE], b[VE];
        load_row<VE>(P.s + row * L, rl, s);
        load_row<VE>(P.gy + row * L, rl, g);
        if (!valid) {
#pragma unroll
            for (int j = 0; j < VE; ++j) g[j] = 0.f;  // a zero upstream gradient: every contribution below is +-0
        }
        float m, S, tr, v, u, ur, ra[VE], rb[VE];
        chain_fwd<VE, LPR, V>(P, q1, q2, q3, q4, s, e, b, m, S, tr, v, u, ra, rb, ur);
        // y = Q5(b u): gradient to z, Q5's own parameters
        float gb[VE], gu_part = 0.f;
#pragma unroll
        for (int j = 0; j < VE; ++j) {
            float gz, di, df;
            const float z = __fmul_rn(b[j], u);
            qc_bwd_r<Mo::C5>(g[j], z, qc_round<Mo::RA>(z, q5[j]), q5[j], gz, di, df);
            adf5[j] = __fadd_rn(adf5[j], df);
            if (Mo::C5 != 0) adi5[j] = __fadd_rn(adi5[j], di);
            gb[j] = __fmul_rn(gz, u);
            gu_part = fmaf(gz, b[j], gu_part);
        }
        const float gu = row_sum<LPR>(gu_part);
        // u = Q4(v), v = 1 / (t + eps), t = Q3(S): row scalars, identical on every lane of the row
        float gv, di4, df4, gS, di3, df3;
        qc_bwd_r<Mo::C4>(gu, v, ur, q4, gv, di4, df4);
        const float gt = __fmul_rn(-gv, __fmul_rn(v, v));
        qc_bwd_r<Mo::C3>(gt, S, tr, q3, gS, di3, df3);
        if (rl == 0) {
            acc[4] = __fadd_rn(acc[4], di3); acc[5] = __fadd_rn(acc[5], df3);
            acc[6] = __fadd_rn(acc[6], di4); acc[7] = __fadd_rn(acc[7], df4);
        }
        // b = Q2(e), e = exp(-a c), a = Q1(d), d = m - s
        float gd[VE], gm_part = 0.f;
        int ties_part = 0;
#pragma unroll
        for (int j = 0; j < VE; ++j) {
            float ge, di2, df2, di1, df1;
            qc_bwd_r<Mo::C2>(__fadd_rn(gb[j], gS), e[j], rb[j], q2, ge, di2, df2);
            const float ga = __fmul_rn(ge, __fmul_rn(-P.scaler, e[j]));
            qc_bwd_r<Mo::C1>(ga, __fsub_rn(m, s[j]), ra[j], q1, gd[j], di1, df1);
            if (Mo::C1 != 0) acc[0] = __fadd_rn(acc[0], di1);
            acc[1] = __fadd_rn(acc[1], df1);
            acc[2] = __fadd_rn(acc[2], di2); acc[3] = __fadd_rn(acc[3], df2);
            gm_part = __fadd_rn(gm_part, gd[j]);
            ties_part += (s[j] == m) ? 1 : 0;
        }
        const float gm = row_sum<LPR>(gm_part);
        const int ties = row_sum_int<LPR>(ties_part);
        const float share = __fdiv_rn(gm, (float)ties);  // the max spreads its gradient evenly over the tied maxima
        float ds[VE];
#pragma unroll
        for (int j = 0; j < VE; ++j) ds[j] = __fadd_rn(-gd[j], (s[j] == m) ? share : 0.f);
        if (valid) store_row<VE>(P.y + row * L, rl, ds);
    }
    // ---- CTA partials, fixed order --------------------------------------------------------------------------------------
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const float vsum = row_sum<32>(acc[j]);
        if (lane == 0) red[warp][j] = vsum;
    }
#pragma unroll
    for (int j = 0; j < VE; ++j) {
        red5[warp * RPW + sub][0][rl * VE + j] = adf5[j];
        red5[warp * RPW + sub][1][rl * VE + j] = adi5[j];
    }
    __syncthreads();
    const int64_t cta = (int64_t)blockIdx.y * gridDim.x + blockIdx.x;
    float *pc = P.part + cta * (8 + 2 * (int64_t)L);
    if (threadIdx.x < 8) {
        float a8 = 0.f;
        for (int w = 0; w < kSmWarps; ++w) a8 = __fadd_rn(a8, red[w][threadIdx.x]);
        pc[threadIdx.x] = a8;
    }
    for (int c = threadIdx.x; c < 2 * L; c += kSmWarps * 32) {
        const int which = c / L, col = c - which * L;
        float a5 = 0.f;
        for (int w = 0; w < kSmWarps * RPW; ++w) a5 = __fadd_rn(a5, red5[w][which][col]);
        pc[8 + c] = a5;
    }
}

// tables: out[which][p * L + col] = sum over the splits of CTA (p, split); scalars: out8[j] = sum over all CTAs, one warp
// per scalar (lanes stride over the CTAs, then a fixed shuffle tree), done by the last block
__global__ void __launch_bounds__(kThreads) k_qsoftmax_stage2(const float *__restrict__ part, float *__restrict__ out8,
                                                             float *__restrict__ df5, float *__restrict__ di5,
                                                             int rows_period, int L, int splits) {
    const int64_t stride = 8 + 2 * (int64_t)L;
    const int64_t ncta = (int64_t)rows_period * splits;
    if (blockIdx.x == gridDim.x - 1) {
        const int j = threadIdx.x >> 5, lane = threadIdx.x & 31;  // kThreads = 256: warps 0..7 <-> the 8 scalars
        double a = 0.0;
        for (int64_t c = lane; c < ncta; c += 32) a += (double)part[c * stride + j];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
        if (lane == 0) out8[j] = (float)a;
        return;
    }
    const int64_t tbl = (int64_t)rows_period * L;
    const int64_t q = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    if (q < 2 * tbl) {
        const int64_t which = q / tbl, idx = q - which * tbl;
        const int64_t p = idx / L, col = idx - p * L;
        double a = 0.0;
        for (int sp = 0; sp < splits; ++sp) a += (double)part[((int64_t)sp * rows_period + p) * stride + 8 + which * L + col];
        float *dst = which == 0 ? df5 : di5;
        if (dst) dst[idx] = (float)a;
    }
}

static int sm_splits(int64_t batches, int rows_period) {
    int64_t s = ((int64_t)num_sms() * 8 + rows_period - 1) / rows_period;
    const int64_t maxs = (batches + kSmWarps - 1) / kSmWarps;
    if (s > maxs) s = maxs;
    if (s < 1) s = 1;
    if (s > 65535) s = 65535;
    return (int)s;
}

static int sm_check(const SmParams &p, int64_t R) {
    if (R <= 0 || p.rows_period <= 0 || R % p.rows_period != 0) return HGQ_ERR_SIZE;
    if (p.L != 32 && p.L != 64 && p.L != 128) return HGQ_ERR_SIZE;
    if (!p.s || !p.y || !p.f5 || !p.q1.f || !p.q2.f || !p.q3.f || !p.q4.f) return HGQ_ERR_NULL;
    const SQuant *qs[4] = {&p.q1, &p.q2, &p.q3, &p.q4};
    for (const SQuant *q : qs) {
        if (q->rm < 0 || q->rm > 2) return HGQ_ERR_MODE;
        if (q->om != OM_NONE && q->om != OM_SAT && q->om != OM_SAT_SYM) return HGQ_ERR_MODE;
        if (q->om != OM_NONE && (!q->k || !q->i)) return HGQ_ERR_NULL;
    }
    if (p.rm5 < 0 || p.rm5 > 2) return HGQ_ERR_MODE;
    if (p.om5 != OM_NONE && p.om5 != OM_SAT && p.om5 != OM_SAT_SYM) return HGQ_ERR_MODE;
    if (p.om5 != OM_NONE && (!p.k5 || !p.i5)) return HGQ_ERR_NULL;
    if (!aligned(p.s, 16) || !aligned(p.y, 16) || (p.gy && !aligned(p.gy, 16))) return HGQ_ERR_ALIGN;
    return HGQ_OK;
}

// Kernel variant of a launch (see Modes<>): 1 / 2 when the modes are those of the layer in training, else 0.
static int sm_variant(const SmParams &p) {
    static const bool general_only = [] {  // HGQ_QSOFTMAX_GENERAL=1: every launch on the run-time variant (for comparisons)
        const char *v = getenv("HGQ_QSOFTMAX_GENERAL");
        return v != nullptr && v[0] == '1';
    }();
    if (general_only) return 0;
    if (p.q1.rm == RM_RND_CONV || p.q3.rm == RM_RND_CONV || p.rm5 == RM_RND_CONV) return 0;
    if ((p.q2.rm == RM_RND_CONV) != (p.q4.rm == RM_RND_CONV)) return 0;
    if (p.q2.om == OM_NONE || p.q4.om == OM_NONE || p.q3.om != OM_NONE || p.om5 != OM_NONE) return 0;
    return (p.q1.om == OM_NONE ? 1 : 2) + (p.q2.rm == RM_RND_CONV ? 2 : 0);
}

// Lanes per row of 64 scores: 8 (eight scores per lane, four rows per warp) unless HGQ_QSOFTMAX_LANES in the environment says
// 16 or 32 (for comparisons).  Measured on 134 M scores, forward / backward: 32 lanes 0.46 / 1.02 ms, 16 lanes 0.38 / 0.75,
// 8 lanes 0.29 / 0.69: fewer lanes per row mean fewer shuffle steps and less per-row scalar work repeated on every lane.
static int sm_lanes() {
    static const int lanes = [] {
        const char *v = getenv("HGQ_QSOFTMAX_LANES");
        const int n = v != nullptr ? atoi(v) : 8;
        return (n == 16 || n == 32) ? n : 8;
    }();
    return lanes;
}

// the 8-lane organisation moves 32 bytes per lane at a time
static bool sm_aligned32(const SmParams &p) { return aligned(p.s, 32) && aligned(p.y, 32) && (!p.gy || aligned(p.gy, 32)); }

#define HGQ_SM_LAUNCH(KERN, ...)                                                          \
    do {                                                                                  \
        switch (sm_variant(p)) {                                                          \
            case 1: KERN<__VA_ARGS__, 1><<<grid, kSmWarps * 32, 0, st>>>(p); break;       \
            case 2: KERN<__VA_ARGS__, 2><<<grid, kSmWarps * 32, 0, st>>>(p); break;       \
            case 3: KERN<__VA_ARGS__, 3><<<grid, kSmWarps * 32, 0, st>>>(p); break;       \
            case 4: KERN<__VA_ARGS__, 4><<<grid, kSmWarps * 32, 0, st>>>(p); break;       \
            default: KERN<__VA_ARGS__, 0><<<grid, kSmWarps * 32, 0, st>>>(p); break;      \
        }                                                                                 \
    } while (0)
// L = 128: a warp per row, four scores per lane; L = 64: 8 lanes per row (or 16 / 32); L = 32: 16 lanes, two scores per lane
#define HGQ_SM_DISPATCH(KERN)                                                             \
    do {                                                                                  \
        const int lanes = sm_lanes();                                                     \
        if (L == 128) HGQ_SM_LAUNCH(KERN, 4, 32);                                         \
        else if (L == 64 && lanes == 8 && sm_aligned32(p)) HGQ_SM_LAUNCH(KERN, 8, 8);     \
        else if (L == 64 && lanes != 32) HGQ_SM_LAUNCH(KERN, 4, 16);                      \
        else if (L == 64) HGQ_SM_LAUNCH(KERN, 2, 32);                                     \
        else HGQ_SM_LAUNCH(KERN, 2, 16);                                                  \
    } while (0)

}  // namespace hgq

using namespace hgq;

// The C ABI passes the five quantizers as host arrays of five entries each: qk[5], qi[5], qf[5] hold device pointers
// (entries 0..3 point at single elements, entry 4 at the [rows_period, L] tables), qrm[5], qom[5] the modes.
static SmParams sm_make(const float *s, const float *gy, float *y, const uint8_t *const *qk, const float *const *qi,
                        const float *const *qf, const int *qrm, const int *qom, float scaler, float eps, int64_t R, int L,
                        int rows_period) {
    SmParams p{};
    p.s = s; p.gy = gy; p.y = y;
    SQuant *qs[4] = {&p.q1, &p.q2, &p.q3, &p.q4};
    for (int j = 0; j < 4; ++j) {
        qs[j]->k = qk[j]; qs[j]->i = qi[j]; qs[j]->f = qf[j]; qs[j]->rm = qrm[j]; qs[j]->om = qom[j];
    }
    p.k5 = qk[4]; p.i5 = qi[4]; p.f5 = qf[4]; p.rm5 = qrm[4]; p.om5 = qom[4];
    p.scaler = scaler; p.eps = eps;
    p.rows_period = rows_period; p.L = L;
    p.batches = rows_period > 0 ? R / rows_period : 0;
    p.splits = sm_splits(p.batches, rows_period > 0 ? rows_period : 1);
    return p;
}

extern "C" int hgq_qsoftmax_fwd(const float *s, float *y, const uint8_t *const *qk, const float *const *qi,
                                const float *const *qf, const int *qrm, const int *qom, float scaler, float eps,
                                float *absmax_exp_in, float *absmax_inv_in, float *absmax_out, int64_t R, int L,
                                int rows_period, void *stream) {
    if (!qk || !qi || !qf || !qrm || !qom) return HGQ_ERR_NULL;
    SmParams p = sm_make(s, nullptr, y, qk, qi, qf, qrm, qom, scaler, eps, R, L, rows_period);
    if (int e = sm_check(p, R)) return e;
    cudaStream_t st = (cudaStream_t)stream;
    p.amax1 = (unsigned *)absmax_exp_in;
    p.amax3 = (unsigned *)absmax_inv_in;
    p.amax5 = (unsigned *)absmax_out;
    if (absmax_exp_in) {
        cudaError_t e = cudaMemsetAsync(absmax_exp_in, 0, sizeof(float), st);
        if (e != cudaSuccess) return (int)e;
    }
    if (absmax_inv_in) {
        cudaError_t e = cudaMemsetAsync(absmax_inv_in, 0, sizeof(float), st);
        if (e != cudaSuccess) return (int)e;
    }
    if (absmax_out) {
        cudaError_t e = cudaMemsetAsync(absmax_out, 0, sizeof(float) * (size_t)rows_period * L, st);
        if (e != cudaSuccess) return (int)e;
    }
    dim3 grid((unsigned)rows_period, (unsigned)p.splits);
    HGQ_SM_DISPATCH(k_qsoftmax_fwd);
    return check_launch();
}

extern "C" size_t hgq_qsoftmax_bwd_workspace(int64_t R, int L, int rows_period) {
    if (R <= 0 || rows_period <= 0 || R % rows_period != 0) return 0;
    const int splits = sm_splits(R / rows_period, rows_period);
    return (size_t)rows_period * splits * (8 + 2 * (size_t)L) * sizeof(float);
}

extern "C" int hgq_qsoftmax_bwd(const float *gy, const float *s, float *ds, const uint8_t *const *qk,
                                const float *const *qi, const float *const *qf, const int *qrm, const int *qom,
                                float scaler, float eps, float *dscalars8, float *df_out, float *di_out, int64_t R, int L,
                                int rows_period, void *workspace, size_t workspace_bytes, void *stream) {
    if (!qk || !qi || !qf || !qrm || !qom || !gy || !dscalars8) return HGQ_ERR_NULL;
    SmParams p = sm_make(s, gy, ds, qk, qi, qf, qrm, qom, scaler, eps, R, L, rows_period);
    if (int e = sm_check(p, R)) return e;
    const size_t need = hgq_qsoftmax_bwd_workspace(R, L, rows_period);
    if (workspace == nullptr || workspace_bytes < need) return HGQ_ERR_WORKSPACE;
    p.part = (float *)workspace;
    cudaStream_t st = (cudaStream_t)stream;
    dim3 grid((unsigned)rows_period, (unsigned)p.splits);
    HGQ_SM_DISPATCH(k_qsoftmax_bwd);
    if (int e = check_launch()) return e;
    const int64_t n2 = 2 * (int64_t)rows_period * L;
    k_qsoftmax_stage2<<<(unsigned)((n2 + kThreads - 1) / kThreads) + 1, kThreads, 0, st>>>(p.part, dscalars8, df_out, di_out, rows_period,
                                                                                   L, p.splits);
    return check_launch();
}
