"""QSum / QMeanPow2: quantised accumulation over axes (mirror of src/hgq/layers/ops/accum.py:10-81)."""

from __future__ import annotations

from collections.abc import Sequence
from math import log2, prod

import torch

from ...quantizer.config import QuantizerConfig
from ..core.base import QLayerBaseSingleInput


class QSum(QLayerBaseSingleInput):
    """sum(iq(x), axes) * scale, scale a power of two (accum.py:10-60)."""

    def __init__(self, iq_conf: QuantizerConfig | None = None, axes: int | Sequence[int] = -1, scale: float = 1.0,
                 keepdims: bool = False, **kwargs):
        super().__init__(iq_conf=iq_conf, **kwargs)
        assert kwargs.get('axis', None) is None, f'Use "axes" instead of "axis" in {self.__class__.__name__} ({self.name}).'
        self.axes = tuple(axes) if isinstance(axes, Sequence) else (axes,)
        assert log2(scale).is_integer(), 'Scale must be a power of 2.'
        self._scale = scale
        self._keepdims = keepdims

    def build(self, input_shape):
        super().build(input_shape)
        self.axes = tuple(sorted(i if i >= 0 else i + len(input_shape) for i in self.axes))

    @property
    def scale(self):
        return self._scale

    @property
    def keepdims(self):
        return self._keepdims

    def compute_output_shape(self, input_shape):
        shape = list(input_shape)
        axes = sorted(i if i >= 0 else i + len(shape) for i in self.axes)
        for a in reversed(axes):
            if self.keepdims:
                shape[a] = 1
            else:
                del shape[a]
        return tuple(shape)

    def _compute_ebops(self, shape):
        bits = self.iq.bits_(tuple(shape))
        ebops = torch.sum(bits) - torch.sum(torch.amin(bits, dim=self.axes))
        return ebops * 0.65  # the reference's accumulator cost model (accum.py:42)

    def call(self, inputs, training=None):
        if self.enable_iq:
            inputs = self.iq(inputs, training=training)
        return torch.sum(inputs, dim=self.axes, keepdim=self.keepdims) * self.scale

    def get_config(self):
        config = super().get_config()
        config.update({'axes': self.axes, 'scale': self.scale, 'keepdims': self.keepdims})
        return config


class QMeanPow2(QSum):
    """Mean with the divisor rounded to the nearest power of two (accum.py:63-81)."""

    def __init__(self, iq_conf: QuantizerConfig | None = None, axes: int | Sequence[int] = -1, keepdims: bool = False, **kwargs):
        super().__init__(iq_conf=iq_conf, axes=axes, keepdims=keepdims, **kwargs)

    def build(self, input_shape):
        super().build(input_shape)
        scale = 1.0 / prod([input_shape[i] for i in self.axes])
        self._scale = 2.0 ** round(log2(scale))

    def get_config(self):
        config = super().get_config()
        config.pop('scale')
        return config
