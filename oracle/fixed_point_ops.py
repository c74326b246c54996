"""CPU oracle for the stateless fixed-point quantizer.  TEST INFRASTRUCTURE, not product code.

Only tests/, __graft_entry__.smoke() and the cpu_baseline / reference legs of bench.py may
import this module; nothing under hgq2_b200/ does.

What it restates
----------------
HGQ2 obtains its quantizer arithmetic from the third-party package ``quantizers``
(``quantizers>=1.2.2`` in HGQ2's pyproject.toml:26; floor-pinned, no lock file, not vendored in
the HGQ2 tree):

    from quantizers.fixed_point._fixed_point_ops import _get_fixed_quantizer, round_conv
        -- src/hgq/quantizer/internal/fixed_point_quantizer.py:9-10
    self.stateless_quantizer = get_fixed_quantizer(round_mode, overflow_mode)     -- :58
    self.stateless_quantizer(inputs, k, i, f, training is True, self.seed_gen)   -- :147
    self.stateless_quantizer.round(inputs, f, stochastic, self.seed_gen)         -- :288,295,305,405

This file restates that package's published algorithm as a sequence of single fp32 PyTorch CPU
operations (the reference executes the same kind of sequence eagerly through Keras' torch
backend), with the surrogate gradients written out in closed form:

    round(x, f):        s = 2**f;  xq = rnd(x * s) / s
                        TRN floor, RND floor(. + 0.5), RND_CONV round-half-even
                        dx = g;  df = (-ln2 * (xq - x)) * g
    WRAP (eval):        ((xq + bias) mod 2**(i+k)) - bias,  bias = k * 2**(i+k-1)
    WRAP (training):    xq  (the integer bits are tracked by the stateful layer instead)
    SAT:                clip(xq, -k * 2**i, 2**i - 2**-f)
    SAT_SYM:            clip(xq, -k * (2**i - 2**-f), 2**i - 2**-f)
                        clip backward as torch.clamp(min=tensor, max=tensor): g goes to x inside
                        [lo, hi], to hi above it, to lo below it; d(2**i)/di = ln2 2**i,
                        d(2**-f)/df = -ln2 2**-f.

PARITY UNPINNED: the HGQ2 tree holds no golden vector, known-answer test or fixture for this
boundary (its tests compare against external hardware emulators, tests/base.py:207-275, and
assert only that gradients are non-zero, tests/base.py:302-336), and ``quantizers`` itself
cannot be installed here.  The forward semantics are anchored on the in-tree facts instead: the
range/step properties (fixed_point_quantizer.py:107-120), the eval zeroing (:148-149), the
integer (k, i, f) contract of the export plugins (_alkaid_keras_plugin/_base.py:19-27) and the
ap_fixed meaning of the mode names; tests/test_oracle.py checks them.  Gradient values are this
file's statement of the package's surrogate and are not pinned by anything in the HGQ2 tree.
"""

from __future__ import annotations

import numpy as np
import torch

LN2 = float(np.float32(np.log(2.0)))

ROUND_MODES = ('TRN', 'RND', 'RND_CONV')
OVERFLOW_MODES = ('WRAP', 'SAT', 'SAT_SYM')


def _f32(t) -> torch.Tensor:
    return torch.as_tensor(t, dtype=torch.float32)


def _rnd(xs: torch.Tensor, round_mode: str) -> torch.Tensor:
    if round_mode == 'TRN':
        return torch.floor(xs)
    if round_mode == 'RND':
        return torch.floor(xs + 0.5)
    if round_mode == 'RND_CONV':
        return torch.round(xs)  # ties to even
    raise ValueError(f'unsupported round mode {round_mode}')


def round_fwd(x, f, round_mode: str) -> torch.Tensor:
    x, f = _f32(x), _f32(f)
    s = 2.0**f
    return _rnd(x * s, round_mode) / s


def bounds(k, i, f, overflow_mode: str):
    k, i, f = _f32(k), _f32(i), _f32(f)
    hi = 2.0**i - 2.0**-f
    lo = -(2.0**i) * k if overflow_mode == 'SAT' else -hi * k
    return lo, hi


def quantize_fwd(x, k, i, f, round_mode: str, overflow_mode: str, training: bool = False) -> torch.Tensor:
    """stateless_quantizer(x, k, i, f, training, None) for the deterministic round modes."""
    x, k, i, f = _f32(x), _f32(k), _f32(i), _f32(f)
    xq = round_fwd(x, f, round_mode)
    if overflow_mode == 'WRAP':
        if training:
            return xq
        bk = i + k
        bias = k * 2.0 ** (bk - 1)
        return torch.remainder(xq + bias, 2.0**bk) - bias
    if overflow_mode in ('SAT', 'SAT_SYM'):
        lo, hi = bounds(k, i, f, overflow_mode)
        return torch.clamp(xq, min=lo, max=hi)
    raise ValueError(f'unsupported overflow mode {overflow_mode}')


def quantize_bwd(g, x, k, i, f, round_mode: str, overflow_mode: str):
    """Element-wise (dx, di, df) of the training-mode quantizer; all inputs already broadcast."""
    g, x, k, i, f = _f32(g), _f32(x), _f32(k), _f32(i), _f32(f)
    xq = round_fwd(x, f, round_mode)
    delta = xq - x
    df_r = (delta * (-LN2)) * g
    if overflow_mode in ('WRAP', 'NONE'):
        return g.clone(), torch.zeros_like(g), df_r
    lo, hi = bounds(k, i, f, overflow_mode)
    zero = torch.zeros_like(g)
    inside = (xq >= lo) & (xq <= hi)
    to_hi = (xq > hi) | (hi < lo)
    to_lo = (xq < lo) & (lo < hi)
    ci = (2.0**i) * LN2
    cf = (2.0**-f) * LN2
    ghi = torch.where(to_hi, g, zero)
    glo = torch.where(to_lo, -(g * k), zero)
    dx = torch.where(inside, g, zero)
    df_in = torch.where(inside, df_r, zero)
    if overflow_mode == 'SAT':
        di = ghi * ci + glo * ci
        df = df_in + ghi * cf
    else:
        m = ghi + glo
        di = m * ci
        df = df_in + m * cf
    return dx, di, df


class _Quant(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, k, i, f, round_mode, overflow_mode, training):
        ctx.save_for_backward(x, k, i, f)
        ctx.modes = (round_mode, overflow_mode)
        return quantize_fwd(x, k, i, f, round_mode, overflow_mode, training)

    @staticmethod
    def backward(ctx, g):
        x, k, i, f = ctx.saved_tensors
        rm, om = ctx.modes
        shape = torch.broadcast_shapes(x.shape, k.shape, i.shape, f.shape)
        dx, di, df = quantize_bwd(g, x.expand(shape), k.expand(shape), i.expand(shape), f.expand(shape), rm, om)
        return _sum_to(dx, x.shape), None, _sum_to(di, i.shape), _sum_to(df, f.shape), None, None, None


def _sum_to(t: torch.Tensor, shape) -> torch.Tensor:
    return t.sum_to_size(shape) if tuple(t.shape) != tuple(shape) else t


class FixedQuantizer:
    """Object with the interface HGQ2 expects from ``get_fixed_quantizer(round_mode, overflow_mode)``."""

    def __init__(self, round_mode: str, overflow_mode: str):
        self.round_mode = round_mode.upper()
        self.overflow_mode = overflow_mode.upper()
        if self.round_mode not in ROUND_MODES:
            raise ValueError(f'unsupported round mode {round_mode} (stochastic modes are out of scope)')
        if self.overflow_mode not in OVERFLOW_MODES:
            raise ValueError(f'unsupported overflow mode {overflow_mode}')
        self.stochastic = False

    def __call__(self, x, k, i, f, training=False, seed_gen=None):
        return _Quant.apply(_f32(x), _f32(k), _f32(i), _f32(f), self.round_mode, self.overflow_mode, bool(training))

    def round(self, x, f, stochastic=False, seed_gen=None):
        assert not stochastic
        z = torch.zeros((), dtype=torch.float32)
        return _Quant.apply(_f32(x), z, z, _f32(f), self.round_mode, 'WRAP', True)


def get_fixed_quantizer(round_mode: str = 'TRN', overflow_mode: str = 'WRAP') -> FixedQuantizer:
    return FixedQuantizer(round_mode, overflow_mode)


class _RoundConvSTE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        return torch.round(x)

    @staticmethod
    def backward(ctx, g):
        return g


def round_conv(x: torch.Tensor) -> torch.Tensor:
    """round-half-even with a straight-through gradient (src/hgq/quantizer/internal/base.py:19-28)."""
    return _RoundConvSTE.apply(x)


# ---- a literal autograd composition, used only to cross-check the closed-form backward ---------
def quantize_autograd(x, k, i, f, round_mode: str, overflow_mode: str):
    """Forward built from differentiable torch ops with a straight-through rnd(); training mode."""
    s = 2.0**f
    xs = x * s
    q = xs + (_rnd(xs, round_mode) - xs).detach()
    xq = q / s
    if overflow_mode == 'WRAP':
        return xq
    hi = 2.0**i - 2.0**-f
    lo = -(2.0**i) * k if overflow_mode == 'SAT' else -hi * k
    return torch.clamp(xq, min=lo, max=hi)
