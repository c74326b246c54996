"""QConv2D / QConv1D: act(conv(iq(x), kq(W)) + bq(b)) with EBOPs (mirror of src/hgq/layers/conv.py, ranks 2 and 1,
channels_last)."""

from __future__ import annotations

from math import ceil, prod

import torch
import torch.nn.functional as F

from .. import routes
from ..backend import activation_name, get_activation, get_initializer, take_prepared
from ..quantizer import Quantizer
from ..quantizer.config import QuantizerConfig
from ._functions import EbopsConv2dFn, fused_conv2d_call
from .core.base import QLayerBaseSingleInput


def _pair(v):
    return (int(v), int(v)) if isinstance(v, int) else tuple(int(a) for a in v)


def same_padding(size: int, kernel: int, stride: int, dilation: int) -> tuple[int, int]:
    """(before, after) zero padding of TensorFlow/Keras 'same' convolution along one axis."""
    out = ceil(size / stride)
    total = max((out - 1) * stride + (kernel - 1) * dilation + 1 - size, 0)
    return total // 2, total - total // 2


class _Conv2dFullPrecision(torch.autograd.Function):
    """torch's conv2d with the cuDNN flags of the forward call (fp32 operands, no TF32) applied to its backward too:
    autograd runs the backward outside the ``with`` block of the forward, so the flags are set again around it."""

    @staticmethod
    def forward(ctx, x, w, strides, dilation):
        ctx.save_for_backward(x, w)
        ctx.geom = (strides, dilation)
        return F.conv2d(x, w, stride=strides, dilation=dilation)

    @staticmethod
    def backward(ctx, gy):
        x, w = ctx.saved_tensors
        strides, dilation = ctx.geom
        with torch.backends.cudnn.flags(enabled=True, benchmark=True, deterministic=False, allow_tf32=False):
            gx = torch.nn.grad.conv2d_input(x.shape, w, gy, stride=strides, dilation=dilation) if ctx.needs_input_grad[0] else None
            gw = torch.nn.grad.conv2d_weight(x, w.shape, gy, stride=strides, dilation=dilation) if ctx.needs_input_grad[1] else None
        return gx, gw, None, None


class QConv2D(QLayerBaseSingleInput):
    rank = 2

    def __init__(self, filters, kernel_size, strides=(1, 1), padding='valid', data_format=None, dilation_rate=(1, 1),
                 groups=1, activation=None, use_bias=True, kernel_initializer='glorot_uniform', bias_initializer='zeros',
                 kernel_regularizer=None, bias_regularizer=None, activity_regularizer=None, kernel_constraint=None,
                 bias_constraint=None, kq_conf: None | QuantizerConfig = None, iq_conf: None | QuantizerConfig = None,
                 bq_conf: None | QuantizerConfig = None, parallelization_factor=-1, **kwargs):
        super().__init__(iq_conf=iq_conf, **kwargs)
        if data_format not in (None, 'channels_last'):
            raise NotImplementedError('only channels_last is supported')
        if groups != 1:
            raise NotImplementedError('grouped convolutions are not supported')
        if padding not in ('valid', 'same'):
            raise NotImplementedError(f'padding {padding!r} is not supported')
        self.data_format = 'channels_last'
        self.filters = int(filters)
        self.kernel_size = _pair(kernel_size)
        self.strides = _pair(strides)
        self.dilation_rate = _pair(dilation_rate)
        self.padding = padding
        self.use_bias = use_bias
        self._activation_spec = activation
        self.activation = get_activation(activation)
        self.kernel_initializer = get_initializer(kernel_initializer)
        self.bias_initializer = get_initializer(bias_initializer)
        self.kernel_regularizer, self.bias_regularizer = kernel_regularizer, bias_regularizer
        self.kernel_constraint, self.bias_constraint = kernel_constraint, bias_constraint
        kq_conf = kq_conf or QuantizerConfig('default', 'weight')
        self._kq = Quantizer(kq_conf, name=f'{self.name}_kq')
        bq_conf = bq_conf or QuantizerConfig('default', 'bias')
        self._bq = Quantizer(bq_conf, name=f'{self.name}_bq') if use_bias else None
        self.parallelization_factor = parallelization_factor
        self.bias = None

    @property
    def kq(self):
        return self._kq

    @property
    def bq(self):
        return self._bq

    @property
    def kernel(self):
        return self._kernel.value

    def _pads(self, h, w):
        if self.padding == 'valid':
            return (0, 0), (0, 0)
        return (same_padding(h, self.kernel_size[0], self.strides[0], self.dilation_rate[0]),
                same_padding(w, self.kernel_size[1], self.strides[1], self.dilation_rate[1]))

    def compute_output_shape(self, input_shape):
        b, h, w, _ = input_shape
        (pt, pb), (pl, pr) = self._pads(h, w)
        oh = (h + pt + pb - (self.kernel_size[0] - 1) * self.dilation_rate[0] - 1) // self.strides[0] + 1
        ow = (w + pl + pr - (self.kernel_size[1] - 1) * self.dilation_rate[1] - 1) // self.strides[1] + 1
        return (b, oh, ow, self.filters)

    def build(self, input_shape):
        # kernel and bias before the base classes' beta / ebops: the reference's variable order
        c = int(input_shape[-1])
        self._kernel = self.add_weight(name='kernel', shape=self._kernel_shape(c),
                                       initializer=self.kernel_initializer, regularizer=self.kernel_regularizer,
                                       constraint=self.kernel_constraint)
        if self.use_bias:
            self._bias = self.add_weight(name='bias', shape=(self.filters,), initializer=self.bias_initializer,
                                         regularizer=self.bias_regularizer, constraint=self.bias_constraint)
            self.bias = self._bias.value
        super().build(input_shape)
        self.kq.build(tuple(self._kernel.shape))
        self.kq.built = True
        if self.use_bias:
            self.bq.build(tuple(self._bias.shape))
            self.bq.built = True
        self._built_hw = self._image_hw(input_shape)
        out = self.compute_output_shape(input_shape)
        self.n_parallel = prod(int(d) for d in out[1:-1])
        if self.parallelization_factor <= 0:
            self.parallelization_factor = self.n_parallel

    def _kernel_shape(self, channels):
        return self.kernel_size + (channels, self.filters)

    def _image_hw(self, input_shape):
        return (int(input_shape[1]), int(input_shape[2]))

    def convolution_op(self, inputs, kernel):
        """channels_last 2-D convolution through the library (shapes the implicit-GEMM kernels do not cover)."""
        (pt, pb), (pl, pr) = self._pads(inputs.shape[1], inputs.shape[2])
        x = inputs.permute(0, 3, 1, 2)
        if pt or pb or pl or pr:
            x = F.pad(x, (pl, pr, pt, pb))
        # NHWC data viewed as NCHW is exactly torch's channels_last layout; giving the (tiny) kernel the same layout lets
        # cuDNN run its NHWC kernels end to end, so no transposition of the activations happens on either side
        w = kernel.permute(3, 2, 0, 1).contiguous(memory_format=torch.channels_last)
        # The library convolution must multiply fp32 operands at full precision in forward *and* backward (the reference's
        # tests pin matmul precision to 'highest'; cuDNN's TF32 default would round operands to 10 mantissa bits), and is
        # left to time its algorithms per shape (its heuristic picks FFT-based kernels with layout transposes for these
        # small 3x3 cases).  Both settings are scoped to this call: the process-wide cuDNN flags are the host's.
        with torch.backends.cudnn.flags(enabled=True, benchmark=True, deterministic=False, allow_tf32=False):
            y = _Conv2dFullPrecision.apply(x, w, self.strides, self.dilation_rate)
        return y.permute(0, 2, 3, 1)

    def prepare_params(self):
        """The parameter-only part of a call: (quantised kernel, quantised bias)."""
        return self.qkernel, (self.qbias if self.use_bias else None)

    def call(self, inputs, training=None):
        if self.enable_iq:
            inputs = self.iq(inputs, training=training)
        qkernel, qbias = take_prepared(self) or self.prepare_params()
        return self._contract(inputs, qkernel, qbias)

    def _contract(self, inputs, qkernel, qbias):
        """act(conv(inputs, qkernel) + qbias) on quantised operands: [B, H, W, C] image, [KH, KW, C, N] kernel."""
        fused = fused_conv2d_call(self, inputs, qkernel, qbias)
        if fused is not None:
            return fused
        routes.fallback('cudnn.conv2d', f'{type(self).__name__} {self.name}')
        outputs = self.convolution_op(inputs, qkernel)
        if self.use_bias:
            outputs = outputs + qbias.reshape(1, 1, 1, self.filters)
        if self.activation is not None:
            return self.activation(outputs)
        return outputs

    def _compute_ebops(self, shape):
        shape = tuple(shape)
        _, h, w, _ = shape
        bw_inp = self.iq.bits_(shape)[0]
        bw_ker = self.kq.bits_(tuple(self._kernel.shape))
        bw_bias = self.bq.bits_(tuple(self._bias.shape)) if self.bq is not None else None
        (pt, _), (pl, _) = self._pads(h, w)
        out = self.compute_output_shape(shape)
        size = float(prod(shape[:-1]) * self.filters)
        return EbopsConv2dFn.apply(bw_inp, bw_ker, bw_bias, (out[1], out[2]), self.strides, self.dilation_rate, (pt, pl),
                                   size, self.parallelization_factor / self.n_parallel, 1.0)

    def get_config(self):
        config = super().get_config()
        config.update({
            'filters': self.filters, 'kernel_size': self.kernel_size, 'strides': self.strides, 'padding': self.padding,
            'dilation_rate': self.dilation_rate, 'activation': activation_name(self._activation_spec),
            'use_bias': self.use_bias, 'kq_conf': self.kq.config,
            'bq_conf': self.bq.config if self.bq is not None else None,
            'parallelization_factor': self.parallelization_factor,
        })
        return config

    @property
    def qkernel(self):
        return self.kq(self._kernel.value)

    @property
    def qbias(self):
        if self.bias is None:
            return None
        return self.bq(self._bias.value)


class QConv1D(QConv2D):
    """act(conv1d(iq(x), kq(W)) + bq(b)) on [batch, steps, channels] inputs (QConv1D of src/hgq/layers/conv.py:127-174; the
    call and the EBOPs are QBaseConv's, conv.py:72-102): QConv2D's kernels on an image of one row.  The kernel variable has the
    reference's shape [kernel_size, channels, filters].  padding: 'valid', 'same' or 'causal' (kernel_size - 1 dilated steps of
    zeros in front, none behind, as keras' Conv1D)."""

    rank = 1

    def __init__(self, filters, kernel_size, strides=1, padding='valid', data_format=None, dilation_rate=1, **kwargs):
        def one(v):
            return int(v[0]) if isinstance(v, (tuple, list)) else int(v)

        causal = padding == 'causal'
        super().__init__(filters, (1, one(kernel_size)), strides=(1, one(strides)), padding='valid' if causal else padding,
                         data_format=data_format, dilation_rate=(1, one(dilation_rate)), **kwargs)
        if causal:
            self.padding = 'causal'

    def _pads(self, h, w):
        if self.padding == 'causal':
            return (0, 0), ((self.kernel_size[1] - 1) * self.dilation_rate[1], 0)
        return super()._pads(h, w)

    def _kernel_shape(self, channels):
        return (self.kernel_size[1], channels, self.filters)

    def _image_hw(self, input_shape):
        return (1, int(input_shape[1]))

    def compute_output_shape(self, input_shape):
        if len(input_shape) == 4:  # the one-row image the 2-D kernels see
            return super().compute_output_shape(input_shape)
        b, w, c = input_shape
        out = super().compute_output_shape((b, 1, w, c))
        return (out[0], out[2], out[3])

    def call(self, inputs, training=None):
        if self.enable_iq:
            inputs = self.iq(inputs, training=training)
        qkernel, qbias = take_prepared(self) or self.prepare_params()
        return self._contract(inputs.unsqueeze(1), qkernel.unsqueeze(0), qbias).squeeze(1)

    def _compute_ebops(self, shape):
        shape = tuple(shape)
        _, w, _ = shape
        bw_inp = self.iq.bits_(shape)[0].unsqueeze(0)
        bw_ker = self.kq.bits_(tuple(self._kernel.shape)).unsqueeze(0)
        bw_bias = self.bq.bits_(tuple(self._bias.shape)) if self.bq is not None else None
        (pt, _), (pl, _) = self._pads(1, w)
        out = self.compute_output_shape(shape)
        size = float(prod(shape[:-1]) * self.filters)
        return EbopsConv2dFn.apply(bw_inp, bw_ker, bw_bias, (1, out[1]), self.strides, self.dilation_rate, (pt, pl),
                                   size, self.parallelization_factor / self.n_parallel, 1.0)

    def get_config(self):
        config = super().get_config()
        config.update({'kernel_size': (self.kernel_size[1],), 'strides': (self.strides[1],),
                       'dilation_rate': (self.dilation_rate[1],)})
        return config
