"""Quantised pooling layers, channels_last (mirror of src/hgq/layers/pooling.py): input quantizer + the plain pooling op,
EBOPs = sum of the input bits * parallelization_factor / n_parallel."""

from __future__ import annotations

from math import prod

import torch
import torch.nn.functional as F

from ..backend import MaxPooling2D
from ..quantizer.config import QuantizerConfig
from .core.base import QLayerBaseSingleInput


def _pair(v):
    return (int(v), int(v)) if isinstance(v, int) else tuple(int(a) for a in v)


class QBasePooling(QLayerBaseSingleInput):
    """pooling.py:23-47."""

    def __init__(self, *args, parallelization_factor=-1, data_format=None, **kwargs):
        if data_format not in (None, 'channels_last'):
            raise NotImplementedError('only channels_last is supported')
        self.parallelization_factor = parallelization_factor
        self.data_format = 'channels_last'
        super().__init__(*args, **kwargs)

    def _pool(self, inputs):
        raise NotImplementedError

    def _compute_ebops(self, shape):
        bw_inp = self.iq.bits_(tuple(shape))
        return torch.sum(bw_inp) * self.parallelization_factor / self.n_parallel

    def call(self, inputs, training=None):
        if self.enable_iq:
            inputs = self.iq(inputs, training=training)
        return self._pool(inputs)

    def build(self, input_shape):
        super().build(input_shape)
        out = self.compute_output_shape(input_shape)
        self.n_parallel = prod(int(d) for d in out[1:-1])
        if self.parallelization_factor <= 0:
            self.parallelization_factor = self.n_parallel


class _Windowed2D(QBasePooling):
    def __init__(self, pool_size, strides=None, padding='valid', data_format=None, name=None,
                 iq_conf: QuantizerConfig | None = None, oq_conf: QuantizerConfig | None = None, **kwargs):
        if padding != 'valid':
            raise NotImplementedError("only padding='valid' is supported")
        self.pool_size = _pair(pool_size)
        self.strides = self.pool_size if strides is None else _pair(strides)
        self.padding = padding
        super().__init__(data_format=data_format, name=name, iq_conf=iq_conf, oq_conf=oq_conf, **kwargs)

    def compute_output_shape(self, input_shape):
        b, h, w, c = input_shape
        return (b, (h - self.pool_size[0]) // self.strides[0] + 1, (w - self.pool_size[1]) // self.strides[1] + 1, c)


class QMaxPooling2D(_Windowed2D):
    """pooling.py:146-167; the pooling itself runs on the library's max-pooling kernels."""

    def _pool(self, inputs):
        return MaxPooling2D.call(self, inputs)


class QAveragePooling2D(_Windowed2D):
    """pooling.py:74-95."""

    def _pool(self, inputs):
        y = F.avg_pool2d(inputs.permute(0, 3, 1, 2), self.pool_size, self.strides)
        return y.permute(0, 2, 3, 1)


class _Windowed1D(QBasePooling):
    """[batch, steps, channels] inputs: the 2-D pooling of an image of one row."""

    def __init__(self, pool_size, strides=None, padding='valid', data_format=None, name=None,
                 iq_conf: QuantizerConfig | None = None, oq_conf: QuantizerConfig | None = None, **kwargs):
        if padding != 'valid':
            raise NotImplementedError("only padding='valid' is supported")
        one = lambda v: int(v[0]) if isinstance(v, (tuple, list)) else int(v)  # noqa: E731
        self.pool_size = (1, one(pool_size))
        self.strides = self.pool_size if strides is None else (1, one(strides))
        self.padding = padding
        super().__init__(data_format=data_format, name=name, iq_conf=iq_conf, oq_conf=oq_conf, **kwargs)

    def compute_output_shape(self, input_shape):
        b, w, c = input_shape
        return (b, (w - self.pool_size[1]) // self.strides[1] + 1, c)


class QMaxPooling1D(_Windowed1D):
    """pooling.py:122-143, on the max-pooling kernels of the 2-D layer."""

    def _pool(self, inputs):
        return MaxPooling2D.call(self, inputs.unsqueeze(1)).squeeze(1)


class QAveragePooling1D(_Windowed1D):
    """pooling.py:50-71."""

    def _pool(self, inputs):
        return F.avg_pool1d(inputs.permute(0, 2, 1), self.pool_size[1], self.strides[1]).permute(0, 2, 1)


class _Global(QBasePooling):
    def __init__(self, data_format=None, keepdims=False, iq_conf: QuantizerConfig | None = None,
                 oq_conf: QuantizerConfig | None = None, **kwargs):
        self.keepdims = keepdims
        super().__init__(data_format=data_format, iq_conf=iq_conf, oq_conf=oq_conf, **kwargs)

    def compute_output_shape(self, input_shape):
        shape = tuple(input_shape)
        mid = (1,) * (len(shape) - 2) if self.keepdims else ()
        return (shape[0],) + mid + (shape[-1],)


class QGlobalAveragePooling1D(_Global):
    def _pool(self, inputs):
        return inputs.mean(dim=1, keepdim=self.keepdims)


class QGlobalAveragePooling2D(_Global):
    def _pool(self, inputs):
        return inputs.mean(dim=(1, 2), keepdim=self.keepdims)


class QGlobalMaxPooling1D(_Global):
    def _pool(self, inputs):
        return inputs.amax(dim=1, keepdim=self.keepdims)


class QGlobalMaxPooling2D(_Global):
    def _pool(self, inputs):
        return inputs.amax(dim=(1, 2), keepdim=self.keepdims)
