"""QBatchNormalization: batch normalisation as a quantised per-channel scale and offset
(mirror of src/hgq/layers/batch_normalization.py:11-210)."""

from __future__ import annotations

from math import prod

import torch

from ..backend import get_initializer, moments
from ..quantizer import Quantizer
from ..quantizer.config import QuantizerConfig
from .core.base import QLayerBaseSingleInput


class QBatchNormalization(QLayerBaseSingleInput):
    """y = iq(x) * kq(scale) + bq(offset), scale = bn_gamma / sqrt(var + epsilon), offset = bn_beta - mean * scale, with the
    batch moments of iq(x) in training (moving averages updated) and the moving moments otherwise.  Without ``center``
    the reference uses 1 in place of bn_beta (batch_normalization.py:118-121,146-149); so does this class."""

    def __init__(self, axis=-1, momentum=0.99, epsilon=1e-3, center=True, scale=True, beta_initializer='zeros',
                 gamma_initializer='ones', moving_mean_initializer='zeros', moving_variance_initializer='ones',
                 beta_regularizer=None, gamma_regularizer=None, beta_constraint=None, gamma_constraint=None,
                 synchronized=False, kq_conf: None | QuantizerConfig = None, iq_conf: None | QuantizerConfig = None,
                 bq_conf: None | QuantizerConfig = None, **kwargs):
        super().__init__(iq_conf=iq_conf, **kwargs)
        self.axis = int(axis)
        self.momentum, self.epsilon = float(momentum), float(epsilon)
        self.center, self.scale, self.synchronized = center, scale, synchronized
        self.beta_initializer = get_initializer(beta_initializer)
        self.gamma_initializer = get_initializer(gamma_initializer)
        self.moving_mean_initializer = get_initializer(moving_mean_initializer)
        self.moving_variance_initializer = get_initializer(moving_variance_initializer)
        self.beta_regularizer, self.gamma_regularizer = beta_regularizer, gamma_regularizer
        self.beta_constraint, self.gamma_constraint = beta_constraint, gamma_constraint
        kq_conf = kq_conf or QuantizerConfig('default', 'weight')
        self._kq = Quantizer(kq_conf, name=f'{self.name}_kq')
        bq_conf = bq_conf or QuantizerConfig('default', 'bias')
        self._bq = Quantizer(bq_conf, name=f'{self.name}_bq')

    @property
    def kq(self):
        return self._kq

    @property
    def bq(self):
        return self._bq

    def build(self, input_shape):
        # the normalisation variables first, then the base classes' beta / ebops: the reference's variable order
        if self.axis < 0:
            self.axis += len(input_shape)
        dim = (int(input_shape[self.axis]),)
        self._bn_gamma = self.add_weight(shape=dim, name='bn_gamma', initializer=self.gamma_initializer,
                                         regularizer=self.gamma_regularizer, constraint=self.gamma_constraint) if self.scale else None
        self._bn_beta = self.add_weight(shape=dim, name='bn_beta', initializer=self.beta_initializer,
                                        regularizer=self.beta_regularizer, constraint=self.beta_constraint) if self.center else None
        self.moving_mean = self.add_weight(shape=dim, name='moving_mean', initializer=self.moving_mean_initializer, trainable=False)
        self.moving_variance = self.add_weight(shape=dim, name='moving_variance', initializer=self.moving_variance_initializer,
                                               trainable=False)
        self._reduction_axes = tuple(a for a in range(len(input_shape)) if a != self.axis)
        super().build(input_shape)
        self.bq.build(dim)
        self.bq.built = True
        self.kq.build(dim)
        self.kq.built = True
        shape = [1] * len(input_shape)
        shape[self.axis] = dim[0]
        self._shape = tuple(shape)

    @property
    def bn_gamma(self):
        return self._bn_gamma.value if self._bn_gamma is not None else None

    @property
    def bn_beta(self):
        return self._bn_beta.value if self._bn_beta is not None else None

    def _affine(self, mean, variance):
        bn_gamma = self._bn_gamma.value if self.scale else 1
        bn_beta = self._bn_beta.value if self.center else 1
        scale = bn_gamma / torch.sqrt(variance + self.epsilon)
        return scale, bn_beta - mean * scale

    @property
    def qscaler_and_qoffset(self):
        scale, offset = self._affine(self.moving_mean.value, self.moving_variance.value)
        return self.kq(scale, training=False), self.bq(offset, training=False)

    def compute_output_shape(self, input_shape):
        return tuple(input_shape)

    def call(self, inputs, training=None):
        if self.enable_iq:
            inputs = self.iq(inputs, training=training)
        if training:
            mean, variance = moments(inputs, self._reduction_axes, synchronized=self.synchronized)
            self.moving_mean.assign(self.moving_mean.value * self.momentum + mean.detach() * (1.0 - self.momentum))
            self.moving_variance.assign(self.moving_variance.value * self.momentum + variance.detach() * (1.0 - self.momentum))
            scale, offset = self._affine(mean, variance)
        else:
            scale, offset = self._affine(self.moving_mean.value, self.moving_variance.value)
        qscale = self.kq(scale, training=training).reshape(self._shape)
        qoffset = self.bq(offset, training=training).reshape(self._shape)
        return inputs * qscale + qoffset

    def _compute_ebops(self, shape):
        shape = tuple(shape)
        bw_inp = self.iq.bits_(shape)
        dim = tuple(self.moving_mean.shape)
        bw_ker = self.kq.bits_(dim).reshape(self._shape)
        bw_bias = self.bq.bits_(dim).reshape(self._shape)
        return torch.sum(bw_inp * bw_ker) + torch.mean(bw_bias) * float(prod(shape))

    def get_config(self):
        config = super().get_config()
        config.update({
            'axis': self.axis, 'momentum': self.momentum, 'epsilon': self.epsilon, 'center': self.center, 'scale': self.scale,
            'synchronized': self.synchronized, 'kq_conf': self.kq.config, 'bq_conf': self.bq.config,
        })
        return config
