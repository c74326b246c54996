"""CUDA-backed stateless fixed-point quantizer with the interface of ``quantizers.get_fixed_quantizer``.

This is the narrowest seam of the reference: ``FixedPointQuantizerBase.build`` installs
``get_fixed_quantizer(round_mode, overflow_mode)`` (src/hgq/quantizer/internal/fixed_point_quantizer.py:58)
and every quantizer call goes through ``q(x, k, i, f, training, seed_gen)`` (:147) or
``q.round(x, f, stochastic, seed_gen)`` (:288,295,305,405).  The object returned here has the same
attributes and call signatures; forward and backward are single launches of the K1 kernels.  Bitwidth
tensors are *not* broadcast to ``x.shape`` first: a parameter tensor whose leading axes are 1 is read in
place (the "broadcast layout"), and its gradient comes back already summed over those axes.
"""

from __future__ import annotations

import torch

from .. import kernels

_DETERMINISTIC = ('TRN', 'RND', 'RND_CONV')


def trailing_period(x_shape, p_shape) -> bool:
    """True if p_shape is x_shape with some leading axes set to 1 (so p repeats with period p.numel())."""
    ps = (1,) * (len(x_shape) - len(p_shape)) + tuple(p_shape)
    if len(ps) != len(x_shape):
        return False
    lead = 0
    while lead < len(ps) and ps[lead] == 1:
        lead += 1
    return tuple(ps[lead:]) == tuple(x_shape[lead:])


def _layout(x: torch.Tensor, k, i, f):
    """Flat parameter tensors the kernels can read in place, or materialised broadcasts when the bitwidth shape
    has a size-1 axis after a heterogeneous one.  k, i, f share one shape (one bitwidth mapper)."""
    shapes = {tuple(p.shape) for p in (k, i, f) if p is not None}
    if len(shapes) != 1:
        raise ValueError(f'k, i, f must share one shape, got {shapes}')
    (pshape,) = shapes
    if trailing_period(tuple(x.shape), pshape):
        return [None if p is None else p.contiguous() for p in (k, i, f)], False
    return [None if p is None else p.expand(x.shape).contiguous() for p in (k, i, f)], True


class _QuantizeFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, k, i, f, round_mode, overflow_mode, training, zero_nonpos):
        x = x.contiguous()
        k8 = None if k is None else (k if k.dtype == torch.uint8 else k.to(torch.uint8))
        (kk, ii, ff), mat = _layout(x, k8, i, f)
        ctx.save_for_backward(x, kk, ii, ff)
        ctx.meta = (round_mode, overflow_mode, mat, tuple(f.shape))
        return kernels.quantize_fwd(x, kk, ii, ff, round_mode, overflow_mode, training=training, zero_nonpos=zero_nonpos)

    @staticmethod
    def backward(ctx, g):
        x, kk, ii, ff = ctx.saved_tensors
        rm, om, mat, pshape = ctx.meta
        need_x, _, need_i, need_f = ctx.needs_input_grad[:4]
        want_di = bool(need_i) and om in ('SAT', 'SAT_SYM')
        dx, di, df = kernels.quantize_bwd(g.contiguous(), x, kk, ii, ff, rm, om, want_dx=need_x, want_di=want_di)

        def shaped(t):
            if t is None:
                return None
            return t.view(x.shape).sum_to_size(pshape) if mat else t.view(pshape)

        gi = None
        if need_i:
            gi = shaped(di) if want_di else torch.zeros(pshape, device=x.device)
        return (dx if need_x else None), None, gi, (shaped(df) if need_f else None), None, None, None, None


class _RoundAbsmaxFn(torch.autograd.Function):
    """round(x, f) with the per-column max |round(x, f)| as a second, non-differentiable output."""

    @staticmethod
    def forward(ctx, x, f, round_mode):
        x = x.contiguous()
        ff = f.contiguous()
        ctx.save_for_backward(x, ff)
        ctx.meta = (round_mode, tuple(f.shape))
        if ff.numel() == x.numel():  # nothing to reduce over
            y = kernels.quantize_fwd(x, None, None, ff, round_mode, 'NONE', training=True)
            amax = y.abs()
        else:
            y, amax = kernels.quantize_fwd(x, None, None, ff, round_mode, 'NONE', training=True, want_absmax=True)
        ctx.mark_non_differentiable(amax)
        return y, amax

    @staticmethod
    def backward(ctx, g, _g_amax):
        x, ff = ctx.saved_tensors
        rm, pshape = ctx.meta
        need_x, need_f = ctx.needs_input_grad[:2]
        dx, _, df = kernels.quantize_bwd(g.contiguous(), x, None, None, ff, rm, 'NONE', want_dx=need_x, want_di=False)
        return (dx if need_x else None), (df.view(pshape) if need_f else None), None


def round_with_absmax(x, f, round_mode: str):
    return _RoundAbsmaxFn.apply(x, f, round_mode)


class FixedQuantizer:
    """``q(x, k, i, f, training, seed_gen)`` and ``q.round(x, f, stochastic, seed_gen)`` on CUDA tensors."""

    def __init__(self, round_mode: str, overflow_mode: str):
        self.round_mode = round_mode.upper()
        self.overflow_mode = overflow_mode.upper()
        if self.round_mode.startswith('S_'):
            raise NotImplementedError('stochastic rounding modes are outside the accelerated path')
        if self.round_mode not in _DETERMINISTIC:
            raise ValueError(f'unknown round mode {round_mode}')
        if self.overflow_mode not in ('WRAP', 'SAT', 'SAT_SYM'):
            raise ValueError(f'unknown overflow mode {overflow_mode}')
        self.stochastic = False

    def __call__(self, x, k, i, f, training=False, seed_gen=None, zero_nonpos: bool = False):
        return _QuantizeFn.apply(x, k, i, f, self.round_mode, self.overflow_mode, bool(training), zero_nonpos)

    def round(self, x, f, stochastic=False, seed_gen=None):
        if stochastic:
            raise NotImplementedError('stochastic rounding modes are outside the accelerated path')
        return _QuantizeFn.apply(x, None, None, f, self.round_mode, 'NONE', True, False)


def get_fixed_quantizer(round_mode: str = 'TRN', overflow_mode: str = 'WRAP') -> FixedQuantizer:
    return FixedQuantizer(round_mode, overflow_mode)


class _RoundConv(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        return torch.round(x)

    @staticmethod
    def backward(ctx, g):
        return g


def round_conv(x: torch.Tensor) -> torch.Tensor:
    """Round-half-even with a straight-through gradient (src/hgq/quantizer/internal/base.py:19-28)."""
    return _RoundConv.apply(x)
