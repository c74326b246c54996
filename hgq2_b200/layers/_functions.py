"""torch.autograd bridges between the layer classes and the CUDA kernels."""

from __future__ import annotations

import torch

from .. import kernels

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
    def forward(ctx, x, wq, bq, k, i, f, rows_period, round_mode, overflow_mode, training, zero, activation, want_absmax):
        y, amax = kernels.qdense_fwd(x, k, i, f, rows_period, round_mode, overflow_mode, training, zero, wq, bq, activation,
                                     want_absmax)
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
        gy = gy.contiguous()
        need_x, need_w, need_b, _, need_i, need_f = ctx.needs_input_grad[:6]
        round_only = f is not None and (om == 'NONE' or (om == 'WRAP' and training)) and not zero
        if fused_bwd_enabled and need_w and (f is None or round_only) and kernels.qdense_bwd_supported(x.numel() // K, K, N, rows_period):
            dx, dwq, dbq, df = kernels.qdense_bwd(gy, y if activation == 'relu' else None, x, f, rows_period, rm, wq,
                                                  want_dx=need_x, want_db=has_bias and need_b, want_df=bool(need_f))
            if dx is not None:
                dx = dx.view(x.shape)
            if df is not None:
                df = df.view(f.shape)
            di = torch.zeros_like(i) if (need_i and i is not None) else None
            return dx, dwq, dbq, None, di, df, None, None, None, None, None, None, None
        if activation == 'relu':
            gy = gy * (y > 0)
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
        return dx, dwq, dbq, None, di, df, None, None, None, None, None, None, None


# ---- dispatch of a dense-like layer onto the fused kernel ------------------------------------------------------
fused_enabled = True  # module switch (tests compare the fused and the unfused formulation)
fused_bwd_enabled = True


def _amax_to_shape(t: torch.Tensor, shape) -> torch.Tensor:
    """Reduce ``t`` (already broadcast-compatible with ``shape``) to ``shape`` by max over the expanded axes."""
    dims = [d for d, (a, b) in enumerate(zip(t.shape, shape)) if b == 1 and a != 1]
    return torch.amax(t, dim=dims, keepdim=True) if dims else t


def fused_dense_call(layer, inputs, n_contract: int, qkernel, qbias, training):
    """act(iq(x) @ qkernel + qbias) through the fused kernel, or None if this call has to take the unfused route.

    ``inputs`` is [batch, free..., contracted...] with ``n_contract`` trailing contracted axes; ``qkernel`` is the
    quantised kernel viewed as [K, N]; ``qbias`` the quantised bias as [N] or None.
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
    if layer.enable_iq:
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
    y, amax = QDenseFusedFn.apply(inputs, qkernel, qbias, k, i, f, rows_period, rm, om, tr, zero, act_fused, want_amax)
    y = y.view(shape[:len(shape) - n_contract] + (N,))
    if want_amax:
        track(_amax_to_shape(amax.view(table_shape), bw_shape), inputs)
    if act_spec is not None and act_fused is None:
        y = layer.activation(y)
    return y
