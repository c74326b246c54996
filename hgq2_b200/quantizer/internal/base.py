"""Quantizer base classes and the bitwidth mapper (mirror of src/hgq/quantizer/internal/base.py)."""

from __future__ import annotations

from collections.abc import Sequence

import numpy as np
import torch

from ...backend import Layer, epsilon, numbers  # noqa: F401
from ..fixed_point_ops import round_conv  # noqa: F401


def _large_number(dtype):
    return 3e4 if str(dtype) == 'float16' else 1e9


class BitwidthMapperBase:
    """Maps a bitwidth tensor onto the tensor it quantizes (and statistics of that tensor back)."""

    def bw_to_x(self, bw, x_shape):
        raise NotImplementedError

    def x_to_bw_absmax(self, x):
        raise NotImplementedError

    def x_to_bw_sign(self, x):
        raise NotImplementedError

    def inference_weight_shape(self, input_shape) -> tuple[int, ...]:
        raise NotImplementedError

    def get_config(self):
        raise NotImplementedError

    @classmethod
    def from_config(cls, config):
        return cls(**config)


def check_axis(axis: Sequence[int], ndim: int):
    axis = [a if a >= 0 else a + ndim for a in axis]
    assert all(0 <= a < ndim for a in axis), f'Invalid axis {axis} for shape {ndim}.'
    return axis


class DefaultBitwidthMapper(BitwidthMapperBase):
    """Bitwidth tensor = input shape with the homogeneous axes set to 1 (base.py:148-196 of the reference)."""

    def __init__(self, heterogeneous_axis: Sequence[int] | None = None, homogeneous_axis: Sequence[int] | None = None, **kwargs):
        _shape_inferenced = kwargs.pop('_shape_inferenced', False)
        if not _shape_inferenced:
            assert (heterogeneous_axis is None) ^ (homogeneous_axis is None), (
                'Only one of quantize_dims and skip_dims can be specified.'
            )
        self.heterogeneous_axis = heterogeneous_axis
        self.homogeneous_axis = homogeneous_axis
        self._shape_inferenced = _shape_inferenced

    def inference_weight_shape(self, input_shape):
        N = len(input_shape)
        axis = np.arange(N)
        if self.heterogeneous_axis is not None:
            self.heterogeneous_axis = tuple(check_axis(self.heterogeneous_axis, N))
            self.homogeneous_axis = tuple(int(a) for a in np.setdiff1d(axis, self.heterogeneous_axis))
        elif self.homogeneous_axis is not None:
            self.homogeneous_axis = tuple(check_axis(self.homogeneous_axis, N))
            self.heterogeneous_axis = tuple(int(a) for a in np.setdiff1d(axis, self.homogeneous_axis))
        weight_shape = [1] * N
        for i in self.heterogeneous_axis:
            assert input_shape[i] is not None, (
                f'Unable to heterogeneously quantize axis {i} with unknown shape. Input shape: {input_shape}.'
            )
            weight_shape[i] = int(input_shape[i])
        self._shape_inferenced = True
        return tuple(weight_shape)

    def bw_to_x(self, bw, x_shape):
        return torch.broadcast_to(bw, tuple(x_shape))

    def x_to_bw_absmax(self, x):
        ax = tuple(self.homogeneous_axis)
        return torch.amax(torch.abs(x), dim=ax, keepdim=True) if ax else torch.abs(x)

    def x_to_bw_sign(self, x):
        ax = tuple(self.homogeneous_axis)
        neg = x < 0
        return torch.amax(neg, dim=ax, keepdim=True) if ax else neg

    def get_config(self):
        return dict(
            heterogeneous_axis=self.heterogeneous_axis,
            homogeneous_axis=self.homogeneous_axis,
            _shape_inferenced=self._shape_inferenced,
        )


class TrainableQuantizerBase(Layer):
    """Abstract base class for all quantizers."""

    __dummy__ = False

    def __init__(self, **kwargs):
        homogeneous_axis = kwargs.pop('homogeneous_axis', ())
        heterogeneous_axis = kwargs.pop('heterogeneous_axis', None)
        bw_mapper = kwargs.pop('bw_mapper', None) or DefaultBitwidthMapper(heterogeneous_axis, homogeneous_axis)
        self._seed = kwargs.pop('seed', 0)
        super().__init__(**kwargs)
        self.bw_mapper = bw_mapper
        self.supports_masking = True

    def call(self, inputs, training=None):
        raise NotImplementedError

    def compute_output_shape(self, input_shape):
        return input_shape

    @property
    def bits(self):
        raise NotImplementedError

    @property
    def fbits(self):
        raise NotImplementedError

    @property
    def min(self):
        raise NotImplementedError

    @property
    def max(self):
        raise NotImplementedError

    @property
    def epsilon(self):
        raise NotImplementedError


class DummyQuantizer(TrainableQuantizerBase):
    __dummy__ = True

    def call(self, inputs, training=None):
        return inputs

    @property
    def bits(self):
        return torch.zeros((), dtype=torch.float32)

    @property
    def fbits(self):
        return torch.zeros((), dtype=torch.float32)

    @property
    def min(self):
        return -_large_number(self.dtype)

    @property
    def max(self):
        return _large_number(self.dtype)

    @property
    def epsilon(self):
        return epsilon()

    def __repr__(self):
        return f'{self.__class__.__name__}(name={self.name}, built={self.built})'
