"""torch.autograd bridges between the layer classes and the CUDA kernels."""

from __future__ import annotations

import torch

from .. import kernels, routes
from ..backend import bookkeeping

_ones: dict = {}


def _one(device) -> torch.Tensor:
    t = _ones.get(device)
    if t is None:
        t = torch.ones((), dtype=torch.float32, device=device)
        _ones[device] = t
    return t


class EbopsDenseFn(torch.autograd.Function):
    """ebops = scale * (sum(bw_in @ bw_w) + mean(bw_bias) * out_size); gradient to the three bitwidth tensors."""

    @staticmethod
    def forward(ctx, bw_in, bw_w, bw_bias, out_size, scale):
        _, e_f, _, d_in, d_w, d_b = kernels.ebops_dense(bw_in, bw_w, bw_bias, out_size, scale, _one(bw_in.device))
        ctx.save_for_backward(d_in, d_w, d_b)
        return e_f

    @staticmethod
    def backward(ctx, g):
        d_in, d_w, d_b = ctx.saved_tensors
        return g * d_in, g * d_w, (g * d_b if d_b is not None else None), None, None


class EbopsConv2dFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, bw_in, bw_w, bw_bias, out_hw, strides, dilation, pad_tl, out_size, scale_main, scale_bias):
        _, e_f, _, d_in, d_w, d_b = kernels.ebops_conv2d(bw_in, bw_w, bw_bias, out_hw, strides, dilation, pad_tl, out_size,
                                                         scale_main, scale_bias, _one(bw_in.device))
        ctx.save_for_backward(d_in, d_w, d_b)
        return e_f

    @staticmethod
    def backward(ctx, g):
        d_in, d_w, d_b = ctx.saved_tensors
        return g * d_in, g * d_w, (g * d_b if d_b is not None else None), None, None, None, None, None, None, None


class QDenseFusedFn(torch.autograd.Function):
    """y = act(iq(x) @ wq + bq) through the fused tensor-core kernel; also returns the abs-max of the rounded input.

    ``k``, ``i``, ``f`` are the input quantizer's tables already shaped [rows_period, K] (``i``/``k`` None for
    rounding-only).  Backward: dY (masked by the activation) -> dWq, dbq, dXq with library GEMMs, then the
    quantizer's surrogate backward kernel turns dXq into dx and the column-summed bitwidth gradients.
    """

    @staticmethod
    def forward(ctx, x, wq, bq, k, i, f, rows_period, round_mode, overflow_mode, training, zero, activation, want_absmax,
                out_shape=None):
        y, amax = kernels.qdense_fwd(x, k, i, f, rows_period, round_mode, overflow_mode, training, zero, wq, bq, activation,
                                     want_absmax)
        if out_shape is not None:
            # the layer's output shape is given here, not by a view outside: the incoming gradient then arrives as autograd
            # made it (e.g. the stride-0 expansion of a sum's gradient), not reshaped into a dense copy
            y = y.view(out_shape)
        ctx.save_for_backward(x, wq, k, i, f, y if activation == 'relu' else None)
        ctx.meta = (rows_period, round_mode, overflow_mode, training, zero, activation, bq is not None)
        if amax is None:
            amax = torch.empty(0, device=x.device)
        ctx.mark_non_differentiable(amax)
        return y, amax

    @staticmethod
    def backward(ctx, gy, _gamax):
        x, wq, k, i, f, y = ctx.saved_tensors
        rows_period, rm, om, training, zero, activation, has_bias = ctx.meta
        K, N = wq.shape
        gy_repeat = 1
        if (gy.dim() == 3 and gy.stride(1) == 0 and gy.stride(2) == 1 and gy.stride(0) == N and gy.size(1) > 1
                and x.numel() // K < (1 << 31)):
            gy_repeat, gy = gy.size(1), gy[:, 0, :]  # gradient of a sum over axis 1: one stored row per sample
        else:
            gy = gy.contiguous()
        need_x, need_w, need_b, _, need_i, need_f = ctx.needs_input_grad[:6]
        round_only = f is not None and (om == 'NONE' or (om == 'WRAP' and training)) and not zero
        if fused_bwd_enabled and need_w and (f is None or round_only) and kernels.qdense_bwd_supported(x.numel() // K, K, N, rows_period):
            dx, dwq, dbq, df = kernels.qdense_bwd(gy, y if activation == 'relu' else None, x, f, rows_period, rm, wq,
                                                  want_dx=need_x, want_db=has_bias and need_b, want_df=bool(need_f),
                                                  gy_repeat=gy_repeat)
            if dx is not None:
                dx = dx.view(x.shape)
            if df is not None:
                df = df.view(f.shape)
            di = torch.zeros_like(i) if (need_i and i is not None) else None
            return dx, dwq, dbq, None, di, df, None, None, None, None, None, None, None, None
        if fused_bwd_enabled and need_w and kernels.qdense_bwd_supported(x.numel() // K, K, N, 1):
            # an input quantizer that clips (SAT / SAT_SYM, or WRAP outside training): the quantised activations are formed by
            # the quantizer kernel, the three products run on the fused backward kernel as for a layer without input
            # quantizer, and the quantizer's surrogate backward turns dXq into dx and the bitwidth gradients
            x2 = x.reshape(-1, K)
            xq = kernels.quantize_fwd(x2, k, i, f, rm, om, training=training, zero_nonpos=zero)
            want_dxq = bool(need_x or need_f or need_i)
            dxq, dwq, dbq, _ = kernels.qdense_bwd(gy, y if activation == 'relu' else None, xq, None, 1, rm, wq, want_dx=want_dxq,
                                                  want_db=has_bias and need_b, want_df=False, gy_repeat=gy_repeat)
            dx = di = df = None
            if want_dxq:
                om_b = 'NONE' if (om == 'WRAP' and training) else om
                dx, di, df = kernels.quantize_bwd(dxq, x2, k, i, f, rm, om_b, want_dx=need_x,
                                                  want_di=bool(need_i) and om_b in ('SAT', 'SAT_SYM'))
                if need_i and di is None and i is not None:
                    di = torch.zeros_like(i)
                if dx is not None:
                    dx = dx.view(x.shape)
            return dx, dwq, dbq, None, di, df, None, None, None, None, None, None, None, None
        routes.fallback('cuBLAS backward of a dense layer', f'M={x.numel() // K} K={K} N={N} period={rows_period} {rm}/{om}')
        if gy_repeat > 1:
            gy = gy.unsqueeze(1).expand(-1, gy_repeat, -1)
        if activation == 'relu':
            gy = gy * (y > 0).view(gy.shape)
        g2 = gy.reshape(-1, N)
        x2 = x.reshape(-1, K)
        dbq = g2.sum(0) if (has_bias and need_b) else None
        dwq = None
        if need_w:
            xq = x2 if f is None else kernels.quantize_fwd(x2, k, i, f, rm, om, training=training, zero_nonpos=zero)
            dwq = xq.t() @ g2
        dx = di = df = None
        if need_x or need_f or need_i:
            dxq = g2 @ wq.t()
            if f is None:
                dx = dxq
            else:
                om_b = 'NONE' if (om == 'WRAP' and training) else om
                dx, di, df = kernels.quantize_bwd(dxq, x2, k, i, f, rm, om_b, want_dx=need_x,
                                                  want_di=bool(need_i) and om_b in ('SAT', 'SAT_SYM'))
                if need_i and di is None and i is not None:
                    di = torch.zeros_like(i)
            if dx is not None:
                dx = dx.view(x.shape)
        return dx, dwq, dbq, None, di, df, None, None, None, None, None, None, None, None


# ---- dispatch of a dense-like layer onto the fused kernel ------------------------------------------------------
fused_enabled = True  # module switch (tests compare the fused and the unfused formulation)
fused_bwd_enabled = True


def _amax_to_shape(t: torch.Tensor, shape) -> torch.Tensor:
    """Reduce ``t`` (already broadcast-compatible with ``shape``) to ``shape`` by max over the expanded axes."""
    dims = [d for d, (a, b) in enumerate(zip(t.shape, shape)) if b == 1 and a != 1]
    return torch.amax(t, dim=dims, keepdim=True) if dims else t


def fused_dense_call(layer, inputs, n_contract: int, qkernel, qbias, training, apply_iq: bool = True):
    """act(iq(x) @ qkernel + qbias) through the fused kernel, or None if this call has to take the unfused route.

    ``inputs`` is [batch, free..., contracted...] with ``n_contract`` trailing contracted axes; ``qkernel`` is the
    quantised kernel viewed as [K, N]; ``qbias`` the quantised bias as [N] or None.  ``apply_iq=False``: the caller has
    already quantised ``inputs`` (layers that need the quantised activations themselves, e.g. for batch moments).
    """
    if not fused_enabled or not inputs.is_cuda or inputs.dtype != torch.float32 or inputs.dim() < 2:
        return None
    act_spec = getattr(layer, '_activation_spec', None)
    act_fused = act_spec if act_spec in (None, 'relu') else None
    shape = tuple(inputs.shape)
    K = 1
    for d in shape[len(shape) - n_contract:]:
        K *= d
    N = qkernel.shape[-1]
    M = inputs.numel() // K
    k = i = f = None
    rows_period, rm, om, tr, zero, track, bw_shape, table_shape = 1, 'RND', 'NONE', True, False, None, None, None
    if layer.enable_iq and apply_iq:
        q = layer.iq
        if q.scaler is not None or q.affine is not None or (q.qnoise_factor is not None and training):
            return None
        iq = q.quantizer
        if getattr(iq, '__dummy__', False):
            return None  # nothing to quantise: the plain fp32 library product is the reference behaviour
        if True:
            plan = iq.fusion_plan(training)
            if plan is None:
                return None
            bw_shape = tuple(plan['f'].shape)
            if len(bw_shape) != len(shape):
                return None
            free = bw_shape[1:len(shape) - n_contract]
            if all(d == 1 for d in free):
                table_shape = (1,) * (len(shape) - n_contract) + shape[len(shape) - n_contract:]
            else:
                table_shape = (1,) + shape[1:]
                for d in shape[1:len(shape) - n_contract]:
                    rows_period *= d
            expand = lambda t: None if t is None else t.expand(table_shape).reshape(rows_period, K)  # noqa: E731
            k, i, f = expand(plan['k']), expand(plan['i']), expand(plan['f'])
            if k is not None:
                k = k.contiguous()
            rm, om, tr, zero, track = plan['round_mode'], plan['overflow_mode'], plan['training'], plan['zero'], plan['track']
    if not kernels.qdense_supported(M, K, N, rows_period):
        return None
    want_amax = track is not None
    y, amax = QDenseFusedFn.apply(inputs, qkernel, qbias, k, i, f, rows_period, rm, om, tr, zero, act_fused, want_amax,
                                  shape[:len(shape) - n_contract] + (N,))
    if want_amax:
        with bookkeeping(amax):
            track(_amax_to_shape(amax.view(table_shape), bw_shape), inputs)
    if act_spec is not None and act_fused is None:
        y = layer.activation(y)
    return y


class QConv2dFusedFn(torch.autograd.Function):
    """act(conv2d(xq, wq) + bq), channels-last, on the implicit-GEMM tensor-core kernels (stride-1 input gradient).

    ``xq`` is the already quantised image [B, H, W, C] and ``wq`` the quantised kernel [KH, KW, C, N].  ``cp`` channels of
    zero padding are appended first when the kernels at hand need 16-byte pixels (0 when they read the image as it is).
    Backward: one pass forms G = gy * (y > 0), the
    kernel and bias gradients; the input gradient is the same forward kernel run over G with the flipped, transposed
    kernel.
    """

    @staticmethod
    def forward(ctx, xq, wq, bq, activation, strides, dilation, pad_tl, out_hw, cp=0):
        KH, KW, C, N = wq.shape
        if cp:
            xq = torch.nn.functional.pad(xq, (0, cp))
            wq = torch.nn.functional.pad(wq, (0, 0, 0, cp))
        xq = xq.contiguous()
        y = kernels.qconv2d_fwd(xq, wq.reshape(-1, N), bq, activation, KH, KW, out_hw, strides, dilation, pad_tl)
        ctx.save_for_backward(xq, wq, y if activation == 'relu' else None)
        ctx.geom = (KH, KW, C, N, cp, strides, dilation, pad_tl, bq is not None)
        return y

    @staticmethod
    def backward(ctx, gy):
        xq, wq, y = ctx.saved_tensors
        KH, KW, C, N, cp, strides, dilation, pad_tl, has_bias = ctx.geom
        need_x, need_w, need_b = ctx.needs_input_grad[:3]
        g, dwq, dbq = kernels.qconv2d_wgrad(xq, gy, y, KH, KW, strides, dilation, pad_tl, has_bias and need_b)
        dwq = dwq.view(KH, KW, C + cp, N)
        if cp:
            dwq = dwq[:, :, :C, :]
        dx = None
        if need_x:
            B, H, W, Cp = xq.shape
            wt = wq.flip(0, 1).permute(0, 1, 3, 2).reshape(KH * KW * N, Cp)
            dx = kernels.qconv2d_fwd(g, wt, None, None, KH, KW, (H, W), (1, 1), dilation,
                                     ((KH - 1) * dilation[0] - pad_tl[0], (KW - 1) * dilation[1] - pad_tl[1]))
            if cp:
                dx = dx[..., :C]
        return dx, (dwq if need_w else None), dbq, None, None, None, None, None, None


def conv_padding_channels(B, H, W, C, KH, KW, N, OH, OW, dil):
    """How many zero channels must be appended to the image so that the unit-stride implicit-GEMM kernels (forward, input
    gradient, weight gradient) cover the convolution: 0 when they read it as it is, None when they do not cover it."""
    if N % 4 != 0 or KH * KW * N > 640:
        return None

    def covered(c):
        if c > 128:
            return False
        if c % 4 == 0:
            return (kernels.qconv2d_supported(B, H, W, c, KH, KW, N, OH, OW) and kernels.qconv2d_supported(B, OH, OW, N, KH, KW, c, H, W)
                    and kernels.qconv2d_wgrad_supported(B, H, W, c, KH, KW, N, OH, OW))
        # unaligned pixels (an RGB image): only the unit-stride kernels read them in place
        return (kernels.qconv2d_unit_stride_supported(B, H, W, c, KH, KW, N, OH, OW, dil)
                and kernels.qconv2d_unit_stride_supported(B, OH, OW, N, KH, KW, c, H, W, dil)
                and kernels.qconv2d_wgrad_supported(B, H, W, c, KH, KW, N, OH, OW))

    cp = 0 if covered(C) else (-C) % 4
    if cp and not covered(C + cp):
        return None
    return cp


def fused_conv2d_call(layer, xq, qkernel, qbias):
    """The fused convolution of a QConv2D layer on its quantised operands, or None when the shape is not covered."""
    if not fused_enabled or not xq.is_cuda or xq.dtype != torch.float32 or xq.dim() != 4:
        return None
    act_spec = getattr(layer, '_activation_spec', None)
    if act_spec not in (None, 'relu'):
        return None
    n_filters = qkernel.shape[-1]
    if n_filters % 4 != 0:
        # the kernels write output pixels as 16-byte pieces: filters of zeros make up the count and are cut off afterwards
        extra = (-n_filters) % 4
        qkernel = torch.nn.functional.pad(qkernel, (0, extra))
        qbias = None if qbias is None else torch.nn.functional.pad(qbias, (0, extra))
        y = _fused_conv2d(layer, xq, qkernel, qbias, act_spec)
        return None if y is None else y[..., :n_filters]
    return _fused_conv2d(layer, xq, qkernel, qbias, act_spec)


def _fused_conv2d(layer, xq, qkernel, qbias, act_spec):
    if tuple(layer.strides) != (1, 1):
        return strided_conv2d_call(layer, xq, qkernel, qbias, act_spec)
    B, H, W, C = xq.shape
    KH, KW, _, N = qkernel.shape
    (pt, _), (pl, _) = layer._pads(H, W)
    _, OH, OW, _ = layer.compute_output_shape(tuple(xq.shape))
    dil = tuple(layer.dilation_rate)
    cp = conv_padding_channels(B, H, W, C, KH, KW, N, OH, OW, dil)
    if cp is None:
        return None
    return QConv2dFusedFn.apply(xq, qkernel, qbias, act_spec, tuple(layer.strides), dil, (pt, pl), (OH, OW), cp)


def space_to_depth_operands(x, kernel, pad_tl, strides, out_hw):
    """The operands of the unit-stride 'valid' convolution that equals conv(x, kernel) with the given strides and top / left
    zero padding on its first out_hw outputs: x [B, H, W, C] -> [B, OH + KH' - 1, OW + KW' - 1, sh sw C] and kernel
    [KH, KW, C, N] -> [KH', KW', sh sw C, N] with KH' = ceil(KH / sh), KW' = ceil(KW / sw) (see strided_conv2d_call).  Plain
    tensor algebra: differentiable, and the same on any device."""
    (pt, pl), (sh, sw), (OH, OW) = pad_tl, strides, out_hw
    B, H, W, C = x.shape
    KH, KW, _, N = kernel.shape
    KHs, KWs = -(-KH // sh), -(-KW // sw)
    Hs, Ws = OH + KHs - 1, OW + KWs - 1          # blocks the outputs reach
    Cs = sh * sw * C
    # image: pad (or crop rows / columns no output reads) to Hs sh x Ws sw, then blocks -> channels
    x = torch.nn.functional.pad(x, (0, 0, pl, Ws * sw - W - pl, pt, Hs * sh - H - pt))
    x = x.reshape(B, Hs, sh, Ws, sw, C).permute(0, 1, 3, 2, 4, 5).reshape(B, Hs, Ws, Cs)
    w = torch.nn.functional.pad(kernel, (0, 0, 0, 0, 0, KWs * sw - KW, 0, KHs * sh - KH))
    w = w.reshape(KHs, sh, KWs, sw, C, N).permute(0, 2, 1, 3, 4, 5).reshape(KHs, KWs, Cs, N)
    return x, w


def strided_conv2d_call(layer, xq, qkernel, qbias, act_spec):
    """A strided convolution as a unit-stride one (space to depth), so that forward, input gradient and weight gradient all run
    on the unit-stride implicit-GEMM kernels: the zero-padded image is regrouped into blocks of sh x sw pixels whose pixels
    become channels, x'[b, i, j, (a, e, c)] = x[b, i sh + a, j sw + e, c], and the kernel likewise,
    w'[p, q, (a, e, c), n] = w[p sh + a, q sw + e, c, n] (zero where p sh + a >= KH or q sw + e >= KW); then
    y[b, oy, ox] = sum_{p, q} x'[b, oy + p, ox + q] . w'[p, q].  The regrouping is a copy made by torch (autograd maps the
    gradients back through it); the contraction is QConv2dFusedFn.  None when the regrouped shape is not covered."""
    sh, sw = (int(v) for v in layer.strides)
    if tuple(layer.dilation_rate) != (1, 1):
        return None
    B, H, W, C = xq.shape
    KH, KW, _, N = qkernel.shape
    (pt, _), (pl, _) = layer._pads(H, W)
    _, OH, OW, _ = layer.compute_output_shape(tuple(xq.shape))
    KHs, KWs = -(-KH // sh), -(-KW // sw)
    cp = conv_padding_channels(B, OH + KHs - 1, OW + KWs - 1, sh * sw * C, KHs, KWs, N, OH, OW, (1, 1))
    if cp is None:
        return None
    x, w = space_to_depth_operands(xq, qkernel, (pt, pl), (sh, sw), (OH, OW))
    return QConv2dFusedFn.apply(x, w, qbias, act_spec, (1, 1), (1, 1), (0, 0), (OH, OW), cp)


class AttnScoresFn(torch.autograd.Function):
    """scores[b, h, t, s] = sum_d q[b, t, h, d] k[b, s, h, d] on the per-head tensor-core kernel, with its backward."""

    @staticmethod
    def forward(ctx, key, query):
        B, L, H, D = query.shape
        ctx.save_for_backward(key, query)
        return kernels.attn_heads_matmul(0, query, key, B, L, H, D)

    @staticmethod
    def backward(ctx, gs):
        key, query = ctx.saved_tensors
        B, L, H, D = query.shape
        gs = gs.contiguous()
        dq = kernels.attn_heads_matmul(1, gs, key, B, L, H, D) if ctx.needs_input_grad[1] else None     # dS K
        dk = kernels.attn_heads_matmul(2, gs, query, B, L, H, D) if ctx.needs_input_grad[0] else None   # dS^T Q
        return dk, dq


class AttnContextFn(torch.autograd.Function):
    """out[b, t, h, d] = sum_s p[b, h, t, s] v[b, s, h, d] on the per-head tensor-core kernel, with its backward."""

    @staticmethod
    def forward(ctx, probs, value):
        B, L, H, D = value.shape
        ctx.save_for_backward(probs, value)
        return kernels.attn_heads_matmul(1, probs, value, B, L, H, D)

    @staticmethod
    def backward(ctx, go):
        probs, value = ctx.saved_tensors
        B, L, H, D = value.shape
        go = go.contiguous()
        dp = kernels.attn_heads_matmul(0, go, value, B, L, H, D) if ctx.needs_input_grad[0] else None   # dO V^T
        dv = kernels.attn_heads_matmul(2, probs, go, B, L, H, D) if ctx.needs_input_grad[1] else None   # P^T dO
        return dp, dv


def attn_products_supported(query, key, value) -> bool:
    """Self-attention shapes the per-head kernels cover: equal [B, 64, H, D] projections, D = 16 or 32, H even."""
    if not fused_enabled or not query.is_cuda or query.dtype != torch.float32 or query.dim() != 4:
        return False
    if tuple(query.shape) != tuple(key.shape) or tuple(query.shape) != tuple(value.shape):
        return False
    B, L, H, D = query.shape
    return kernels.attn_heads_supported(B, L, H, D)


class QSoftmaxFusedFn(torch.autograd.Function):
    """Training-mode QSoftmax through the fused kernels.  ``params`` is a flat tuple of 15 tensors: (k, i, f) of the exp
    table's input and output quantizers, of the inverse table's input and output quantizers (one element each) and of the
    layer's output quantizer ([rows_period * L] tables); ``i`` / ``k`` are None for a rounding-only quantizer."""

    @staticmethod
    def forward(ctx, s, modes, scaler, eps, rows_period, want_amax3, want_amax5, want_amax1, *params):
        quants = [(params[3 * j], params[3 * j + 1], params[3 * j + 2], modes[j][0], modes[j][1]) for j in range(5)]
        quants = [(None if k is None else (k if k.dtype == torch.uint8 else k.to(torch.uint8)), i, f, rm, om)
                  for k, i, f, rm, om in quants]
        y, a3, a5, a1 = kernels.qsoftmax_fwd(s, quants, scaler, eps, rows_period, want_amax3, want_amax5, want_amax1)
        ctx.save_for_backward(s, *[t for q in quants for t in q[:3]])
        ctx.meta = (modes, scaler, eps, rows_period, [None if t is None else tuple(t.shape) for t in params])
        empty = torch.empty(0, device=s.device)
        a1 = empty if a1 is None else a1
        a3 = empty if a3 is None else a3
        a5 = empty if a5 is None else a5
        ctx.mark_non_differentiable(a3, a5, a1)
        return y, a3, a5, a1

    @staticmethod
    def backward(ctx, gy, _g3, _g5, _g1):
        s, *flat = ctx.saved_tensors
        modes, scaler, eps, rows_period, shapes = ctx.meta
        quants = [(flat[3 * j], flat[3 * j + 1], flat[3 * j + 2], modes[j][0], modes[j][1]) for j in range(5)]
        want_di5 = modes[4][1] in ('SAT', 'SAT_SYM')
        ds, sc, df5, di5 = kernels.qsoftmax_bwd(gy, s, quants, scaler, eps, rows_period, want_di5)
        grads = []
        for j in range(5):
            k, i, f = flat[3 * j], flat[3 * j + 1], flat[3 * j + 2]
            if j < 4:
                gi = sc[2 * j].reshape(shapes[3 * j + 1]) if i is not None else None
                gf = sc[2 * j + 1].reshape(shapes[3 * j + 2])
            else:
                gi = None if i is None else (di5.view(shapes[13]) if di5 is not None else torch.zeros(shapes[13], device=s.device))
                gf = df5.view(shapes[14])
            grads += [None, gi, gf]
        return (ds, None, None, None, None, None, None, None, *grads)
