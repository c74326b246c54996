// Per-element fixed-point quantizer arithmetic shared by every kernel in this library.
//
// The arithmetic restates, operation by operation in fp32, the stateless fixed-point quantizer
// of the `quantizers` package (>=1.2.2) that HGQ2 calls at
// src/hgq/quantizer/internal/fixed_point_quantizer.py:58,147,288,405.  Every step is a single
// IEEE-754 fp32 operation written with an explicit round-to-nearest intrinsic so that the
// compiler cannot contract a multiply and an add into an FMA: results are bit-identical to the
// same sequence evaluated on a CPU.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace hgq {

enum : int { RM_TRN = 0, RM_RND = 1, RM_RND_CONV = 2 };
enum : int { OM_NONE = 0, OM_WRAP = 1, OM_SAT = 2, OM_SAT_SYM = 3 };

constexpr float kLn2 = 0.693147180559945309417f;  // rounds to 0x3f317218, same as float(np.log(2))

// 2^n for an integer n, exact. n is clamped to the normal range of fp32.
__device__ __forceinline__ float pow2i(int n) {
    n = max(-126, min(127, n));
    return __int_as_float((n + 127) << 23);
}

template <int RM>
__device__ __forceinline__ float round_scaled(float xs) {
    if (RM == RM_RND) return floorf(__fadd_rn(xs, 0.5f));
    if (RM == RM_TRN) return floorf(xs);
    return rintf(xs);  // RND_CONV: ties to even
}

// clip(v, lo, hi) with the semantics of min(max(v, lo), hi) that propagates NaN in v and yields
// hi when lo > hi.
__device__ __forceinline__ float clipf(float v, float lo, float hi) {
    v = (v < lo) ? lo : v;
    v = (v > hi) ? hi : v;
    return v;
}

struct Params {
    float s;     // 2^f
    float inv;   // 2^-f
    float p2i;   // 2^i
    float kf;    // k as float (0 or 1)
    int ii, fi;  // integer i, f
};

__device__ __forceinline__ Params make_params(float kf, float i, float f) {
    Params p;
    p.fi = __float2int_rn(f);
    p.ii = __float2int_rn(i);
    p.s = pow2i(p.fi);
    p.inv = pow2i(-p.fi);
    p.p2i = pow2i(p.ii);
    p.kf = kf;
    return p;
}

// Rounded value xq = rnd(x * 2^f) / 2^f  (division by a power of two == multiplication by its
// exact reciprocal).
template <int RM>
__device__ __forceinline__ float round_to_f(float x, const Params &p) {
    return __fmul_rn(round_scaled<RM>(__fmul_rn(x, p.s)), p.inv);
}

// Overflow handling applied to an already rounded value.
template <int OM, bool TRAINING>
__device__ __forceinline__ float overflow(float xq, const Params &p) {
    if (OM == OM_NONE) return xq;
    if (OM == OM_WRAP) {
        if (TRAINING) return xq;
        // ((xq + bias) mod 2^(i+k)) - bias with bias = k 2^(i+k-1); python-style mod computed as
        // t - m floor(t / m), exact because m is a power of two.
        const int bk = p.ii + (p.kf != 0.f ? 1 : 0);
        const float m = pow2i(bk);
        const float minv = pow2i(-bk);
        const float bias = __fmul_rn(p.kf, pow2i(bk - 1));
        const float t = __fadd_rn(xq, bias);
        float r = __fsub_rn(t, __fmul_rn(m, floorf(__fmul_rn(t, minv))));
        if (r == 0.f) r = copysignf(0.f, t);  // a zero remainder keeps the sign of the dividend
        return __fsub_rn(r, bias);
    }
    const float hi = __fsub_rn(p.p2i, p.inv);
    const float lo = (OM == OM_SAT) ? __fmul_rn(-p.p2i, p.kf) : __fmul_rn(-hi, p.kf);
    return clipf(xq, lo, hi);
}

template <int RM, int OM, bool TRAINING, bool ZERO>
__device__ __forceinline__ float quantize(float x, const Params &p, float *rounded = nullptr) {
    const float xq = round_to_f<RM>(x, p);
    if (rounded) *rounded = xq;
    float y = overflow<OM, TRAINING>(xq, p);
    if (ZERO) {
        const int kk = (p.kf != 0.f) ? 1 : 0;
        if (kk + p.ii + p.fi <= 0) y = 0.f;
    }
    return y;
}

// Surrogate gradients of quantize<RM, OM, training=true>.
//   rounding:   dx = g,  df = (-ln2 * (xq - x)) * g
//   SAT/SAT_SYM: the clip routes g to the bound that was hit (hi = 2^i - 2^-f, lo = -k 2^i or
//   -k hi) and d(2^i)/di = ln2 2^i, d(2^-f)/df = -ln2 2^-f.  When lo > hi every element counts
//   as clipped at the top (the clamp-backward convention of torch autograd).
template <int RM, int OM>
__device__ __forceinline__ void quantize_grad(float g, float x, const Params &p, float &dx,
                                              float &di, float &df) {
    const float xq = round_to_f<RM>(x, p);
    const float delta = __fsub_rn(xq, x);
    const float df_r = __fmul_rn(__fmul_rn(delta, -kLn2), g);
    if (OM == OM_NONE || OM == OM_WRAP) {
        dx = g;
        di = 0.f;
        df = df_r;
        return;
    }
    const float hi = __fsub_rn(p.p2i, p.inv);
    const float lo = (OM == OM_SAT) ? __fmul_rn(-p.p2i, p.kf) : __fmul_rn(-hi, p.kf);
    const bool pass = (xq >= lo) && (xq <= hi);
    const bool to_hi = (xq > hi) || (hi < lo);
    const bool to_lo = (xq < lo) && (lo < hi);
    const float ci = __fmul_rn(p.p2i, kLn2);
    const float cf = __fmul_rn(p.inv, kLn2);
    const float ghi = to_hi ? g : 0.f;
    const float glo = to_lo ? -__fmul_rn(g, p.kf) : 0.f;
    dx = pass ? g : 0.f;
    if (OM == OM_SAT) {
        di = __fadd_rn(__fmul_rn(ghi, ci), __fmul_rn(glo, ci));
        df = __fadd_rn(pass ? df_r : 0.f, __fmul_rn(ghi, cf));
    } else {
        const float m = __fadd_rn(ghi, glo);
        di = __fmul_rn(m, ci);
        df = __fadd_rn(pass ? df_r : 0.f, __fmul_rn(m, cf));
    }
}

// ---- runtime-mode variants (mode is uniform across a launch; used where a kernel applies several quantizers) ----------
__device__ __forceinline__ float quantize_rt(float v, float kf, float i, float f, int rm, int om, bool zero, float &rounded) {
    Params p = make_params(kf, i, f);
    if (zero && ((kf != 0.f ? 1 : 0) + p.ii + p.fi <= 0)) {
        rounded = 0.f;
        return 0.f;
    }
    float xq;
    switch (rm) {
        case RM_TRN: xq = round_to_f<RM_TRN>(v, p); break;
        case RM_RND: xq = round_to_f<RM_RND>(v, p); break;
        default: xq = round_to_f<RM_RND_CONV>(v, p); break;
    }
    rounded = xq;
    switch (om) {
        case OM_WRAP: return overflow<OM_WRAP, false>(xq, p);
        case OM_SAT: return overflow<OM_SAT, false>(xq, p);
        case OM_SAT_SYM: return overflow<OM_SAT_SYM, false>(xq, p);
        default: return xq;
    }
}

// surrogate gradients of the training-mode quantizer with runtime modes (om: NONE / SAT / SAT_SYM; WRAP counts as NONE)
__device__ __forceinline__ void quantize_grad_rt(float g, float x, float kf, float i, float f, int rm, int om, float &dx,
                                                 float &di, float &df) {
    const Params p = make_params(kf, i, f);
#define HGQ_QG(RMV)                                                                                      \
    switch (om) {                                                                                        \
        case OM_SAT: quantize_grad<RMV, OM_SAT>(g, x, p, dx, di, df); break;                             \
        case OM_SAT_SYM: quantize_grad<RMV, OM_SAT_SYM>(g, x, p, dx, di, df); break;                     \
        default: quantize_grad<RMV, OM_NONE>(g, x, p, dx, di, df); break;                                \
    }
    switch (rm) {
        case RM_TRN: HGQ_QG(RM_TRN) break;
        case RM_RND: HGQ_QG(RM_RND) break;
        default: HGQ_QG(RM_RND_CONV) break;
    }
#undef HGQ_QG
}

}  // namespace hgq
