"""QDense: act(iq(x) @ kq(W) + bq(b)) with EBOPs (mirror of src/hgq/layers/core/dense.py:13-102)."""

from __future__ import annotations

from math import prod

import torch

from ... import routes
from ...backend import activation_name, get_activation, get_initializer, moments, take_prepared
from ...quantizer import Quantizer
from ...quantizer.config import QuantizerConfig
from .._functions import EbopsDenseFn, fused_dense_call
from .base import QLayerBaseSingleInput


class QDense(QLayerBaseSingleInput):
    def __init__(self, units, activation=None, use_bias=True, kernel_initializer='glorot_uniform',
                 bias_initializer='zeros', kernel_regularizer=None, bias_regularizer=None, activity_regularizer=None,
                 kernel_constraint=None, bias_constraint=None, kq_conf: None | QuantizerConfig = None,
                 iq_conf: None | QuantizerConfig = None, bq_conf: None | QuantizerConfig = None,
                 parallelization_factor=-1, **kwargs):
        super().__init__(iq_conf=iq_conf, **kwargs)
        self.units = int(units)
        self._activation_spec = activation
        self.activation = get_activation(activation)
        self.use_bias = use_bias
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

    def build(self, input_shape):
        # kernel and bias first, then the base classes' beta / ebops: the variable order of the reference, whose Keras base
        # layer builds before QLayerBase adds its own (src/hgq/layers/core/base.py:186-203)
        in_dim = int(input_shape[-1])
        self._kernel = self.add_weight(name='kernel', shape=(in_dim, self.units), initializer=self.kernel_initializer,
                                       regularizer=self.kernel_regularizer, constraint=self.kernel_constraint)
        if self.use_bias:
            self._bias = self.add_weight(name='bias', shape=(self.units,), initializer=self.bias_initializer,
                                         regularizer=self.bias_regularizer, constraint=self.bias_constraint)
            self.bias = self._bias.value
        super().build(input_shape)
        self.n_parallel = prod(int(d) for d in input_shape[1:-1])
        if self.parallelization_factor < 0:
            self.parallelization_factor = self.n_parallel
        self.kq.build(tuple(self._kernel.shape))
        self.kq.built = True
        if self.bias is not None:
            self.bq.build(tuple(self._bias.shape))
            self.bq.built = True

    def compute_output_shape(self, input_shape):
        return tuple(input_shape[:-1]) + (self.units,)

    def prepare_params(self):
        """The parameter-only part of a call: (quantised kernel, quantised bias)."""
        return self.qkernel, (self.qbias if self.bias is not None else None)

    def call(self, inputs, training=None):
        qkernel, qbias = take_prepared(self) or self.prepare_params()
        y = fused_dense_call(self, inputs, 1, qkernel, qbias, training)
        if y is not None:
            return y
        routes.fallback('torch.matmul', f'QDense {self.name}')
        if self.enable_iq:
            inputs = self.iq(inputs, training=training)
        x = torch.matmul(inputs, qkernel)
        if qbias is not None:
            x = x + qbias
        if self.activation is not None:
            x = self.activation(x)
        return x

    def _compute_ebops(self, shape):
        shape = tuple(shape)
        K = shape[-1]
        bw_inp = self.iq.bits_(shape).reshape(-1, K)
        bw_ker = self.kq.bits_(tuple(self._kernel.shape))
        bw_bias = self.bq.bits_(tuple(self._bias.shape)) if self.bq is not None else None
        out_size = prod(shape[:-1]) * self.units
        return EbopsDenseFn.apply(bw_inp, bw_ker, bw_bias, float(out_size), self.parallelization_factor / self.n_parallel)

    def get_config(self):
        config = super().get_config()
        config.update({
            'units': self.units, 'activation': activation_name(self._activation_spec), 'use_bias': self.use_bias,
            'kq_conf': self.kq.config, 'bq_conf': self.bq.config if self.bq is not None else None,
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


class QBatchNormDense(QDense):
    """Batch normalisation of the (quantised) input folded into the dense kernel before it is quantised
    (mirror of src/hgq/layers/core/dense.py:105-254):

        mean, var = moments(iq(x));  scaler = bn_gamma / sqrt(var + epsilon)
        y = act( iq(x) @ kq(scaler[:, None] * W) + bq(b - mean @ W) )

    Training uses the batch moments and updates the moving averages; otherwise the moving averages are used.
    """

    def __init__(self, units, activation=None, use_bias=True, *, scale=True, momentum=0.99, epsilon=1e-3,
                 bn_gamma_initializer='ones', moving_mean_initializer='zeros', moving_variance_initializer='ones',
                 bn_gamma_regularizer=None, bn_gamma_constraint=None, synchronized=False, **dense_kwargs):
        # every other argument (initializers, regularizers, constraints, kq_conf / iq_conf / bq_conf, ...) is QDense's
        if not use_bias:
            raise AssertionError('BatchNormDense must have `use_bias=True`')
        super().__init__(units, activation=activation, use_bias=True, **dense_kwargs)
        self.scale, self.synchronized = scale, synchronized
        self.momentum, self.epsilon = float(momentum), epsilon
        self.bn_gamma_initializer = get_initializer(bn_gamma_initializer)
        self.moving_mean_initializer = get_initializer(moving_mean_initializer)
        self.moving_variance_initializer = get_initializer(moving_variance_initializer)
        self.bn_gamma_regularizer, self.bn_gamma_constraint = bn_gamma_regularizer, bn_gamma_constraint

    def build(self, input_shape):
        super().build(input_shape)
        shape = (int(input_shape[-1]),)
        self.reduction_axis = tuple(range(len(input_shape) - 1))
        if self.scale:
            self._bn_gamma = self.add_weight(shape=shape, name='bn_gamma', initializer=self.bn_gamma_initializer,
                                             regularizer=self.bn_gamma_regularizer, constraint=self.bn_gamma_constraint)
        self.moving_mean = self.add_weight(shape=shape, name='moving_mean', initializer=self.moving_mean_initializer,
                                           trainable=False)
        self.moving_variance = self.add_weight(shape=shape, name='moving_variance',
                                               initializer=self.moving_variance_initializer, trainable=False)

    prepare_params = None  # kernel and bias depend on the batch statistics: nothing to queue ahead

    @property
    def bn_gamma(self):
        return self._bn_gamma.value

    def get_fused_qkernel_and_qbias(self, mean, var):
        bn_gamma = self._bn_gamma.value if self.scale else 1
        scaler = bn_gamma / torch.sqrt(var + self.epsilon)
        kernel = self._kernel.value
        fused_qkernel = self.kq(scaler[:, None] * kernel)
        offset = -torch.matmul(mean, kernel)
        fused_qbias = self.bq(self._bias.value + offset)
        return fused_qkernel, fused_qbias

    def call(self, inputs, training=None):
        if self.enable_iq:
            inputs = self.iq(inputs, training=training)
        if training and self.trainable:
            mean, var = moments(inputs, self.reduction_axis, synchronized=self.synchronized)
            self.moving_mean.assign(self.moving_mean.value * self.momentum + mean.detach() * (1.0 - self.momentum))
            self.moving_variance.assign(self.moving_variance.value * self.momentum + var.detach() * (1.0 - self.momentum))
        else:
            var, mean = self.moving_variance.value, self.moving_mean.value
        qkernel, qbias = self.get_fused_qkernel_and_qbias(mean, var)
        y = fused_dense_call(self, inputs, 1, qkernel, qbias, training, apply_iq=False)
        if y is not None:
            return y
        routes.fallback('torch.matmul', f'QBatchNormDense {self.name}')
        x = torch.matmul(inputs, qkernel) + qbias
        if self.activation is not None:
            x = self.activation(x)
        return x

    def get_config(self):
        config = super().get_config()
        config.update({
            'scale': self.scale, 'momentum': self.momentum, 'epsilon': self.epsilon,
            'bn_gamma_initializer': self.bn_gamma_initializer, 'moving_mean_initializer': self.moving_mean_initializer,
            'moving_variance_initializer': self.moving_variance_initializer,
            'bn_gamma_regularizer': self.bn_gamma_regularizer, 'bn_gamma_constraint': self.bn_gamma_constraint,
            'synchronized': self.synchronized,
        })
        return config

    @property
    def qkernel(self):
        return self.get_fused_qkernel_and_qbias(self.moving_mean.value, self.moving_variance.value)[0]

    @property
    def qbias(self):
        return self.get_fused_qkernel_and_qbias(self.moving_mean.value, self.moving_variance.value)[1]
