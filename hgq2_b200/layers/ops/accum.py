"""Quantised accumulation over axes: ``QSum`` and ``QMeanPow2`` (interface of src/hgq/layers/ops/accum.py:10-81).

Both quantise their input and add it up over ``axes``; the result is multiplied by a power of two (1 for a sum unless
given, the power of two nearest to 1 / count for the mean), which costs no arithmetic in fixed point.
"""

from __future__ import annotations

from collections.abc import Sequence
from math import log2, prod

import torch

from ...quantizer.config import QuantizerConfig
from ..core.base import QLayerBaseSingleInput


def _as_axes(axes) -> tuple:
    return tuple(axes) if isinstance(axes, Sequence) else (axes,)


def _positive(axes, rank: int) -> tuple:
    return tuple(sorted(a % rank for a in axes))


class QSum(QLayerBaseSingleInput):
    def __init__(self, iq_conf: QuantizerConfig | None = None, axes: int | Sequence[int] = -1, scale: float = 1.0,
                 keepdims: bool = False, **kwargs):
        if kwargs.get('axis') is not None:
            raise AssertionError(f'Use "axes" instead of "axis" in {type(self).__name__}.')
        super().__init__(iq_conf=iq_conf, **kwargs)
        if not log2(scale).is_integer():
            raise AssertionError('Scale must be a power of 2.')
        self.axes = _as_axes(axes)
        self._scale, self._keepdims = scale, keepdims

    scale = property(lambda self: self._scale)
    keepdims = property(lambda self: self._keepdims)

    def build(self, input_shape):
        super().build(input_shape)
        self.axes = _positive(self.axes, len(input_shape))

    def compute_output_shape(self, input_shape):
        reduced = set(_positive(self.axes, len(input_shape)))
        if self._keepdims:
            return tuple(1 if a in reduced else d for a, d in enumerate(input_shape))
        return tuple(d for a, d in enumerate(input_shape) if a not in reduced)

    def call(self, inputs, training=None):
        x = self.iq(inputs, training=training) if self.enable_iq else inputs
        return torch.sum(x, dim=self.axes, keepdim=self._keepdims) * self._scale

    def _compute_ebops(self, shape):
        # an adder tree over the axes: every input bit is added once, except the narrowest operand of each sum, times the
        # reference's 0.65 cost factor for accumulators (accum.py:39-43)
        bits = self.iq.bits_(tuple(shape))
        return (bits.sum() - torch.amin(bits, dim=self.axes).sum()) * 0.65

    def get_config(self):
        config = super().get_config()
        config.update(axes=self.axes, scale=self._scale, keepdims=self._keepdims)
        return config


class QMeanPow2(QSum):
    """Mean whose divisor is rounded to the nearest power of two, fixed when the layer is built."""

    def __init__(self, iq_conf: QuantizerConfig | None = None, axes: int | Sequence[int] = -1, keepdims: bool = False, **kwargs):
        super().__init__(iq_conf=iq_conf, axes=axes, keepdims=keepdims, **kwargs)

    def build(self, input_shape):
        super().build(input_shape)
        count = prod(int(input_shape[a]) for a in self.axes)
        self._scale = 2.0 ** round(log2(1.0 / count))

    def get_config(self):
        config = super().get_config()
        del config['scale']
        return config
