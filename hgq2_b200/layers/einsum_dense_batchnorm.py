"""QEinsumDenseBatchnorm: an einsum-dense layer whose batch normalisation is folded into kernel and bias before they are
quantised (mirror of src/hgq/layers/einsum_dense_batchnorm.py:11-300)."""

from __future__ import annotations

import torch

from ..backend import epsilon as keras_epsilon
from ..backend import get_initializer, moments
from ..quantizer.config import QuantizerConfig
from .core.einsum_dense import QEinsumDense, analyze_einsum


class QEinsumDenseBatchnorm(QEinsumDense):
    """Training: x = einsum(eq, iq(inputs), W) gives the batch moments over every output axis that is not normalised;
    scaler = gamma / sqrt(var + eps); y = act(einsum(eq, iq(inputs), kq(W * scaler)) + bq(b - mean * scaler)).
    Otherwise the moving moments are used.  ``eps`` is the backend's fuzz factor (1e-7), as in the reference
    (einsum_dense_batchnorm.py:172), not the ``epsilon`` argument."""

    def __init__(self, equation, output_shape, activation=None, bias_axes=None, *, normalize_axes: str | None = None,
                 momentum=0.99, epsilon=1e-3, center=True, scale=True, beta_initializer='zeros', gamma_initializer='ones',
                 moving_mean_initializer='zeros', moving_variance_initializer='ones', beta_regularizer=None,
                 gamma_regularizer=None, beta_constraint=None, gamma_constraint=None, synchronized=False, **einsum_kwargs):
        # every other argument (initializers, regularizers, constraints, kq_conf / iq_conf / bq_conf, ...) is QEinsumDense's
        super().__init__(equation, output_shape, activation=activation, bias_axes=bias_axes, **einsum_kwargs)
        self.synchronized, self.center, self.scale = synchronized, center, scale
        self.momentum, self.epsilon = float(momentum), float(epsilon)
        self.gamma_initializer = get_initializer(gamma_initializer)
        self.moving_mean_initializer = get_initializer(moving_mean_initializer)
        self.moving_variance_initializer = get_initializer(moving_variance_initializer)
        self.gamma_regularizer, self.gamma_constraint = gamma_regularizer, gamma_constraint
        self.normalize_axes = normalize_axes or bias_axes
        if self.normalize_axes is None:
            raise AssertionError('Either normalize_axes or bias_axes must be provided.')
        self._check_normalize_axes()

    prepare_params = None  # kernel and bias depend on the batch statistics: nothing to queue ahead

    def _check_normalize_axes(self):
        kernel_axes, output_axes = self.equation.split(',')[1].split('->')
        for c in self.normalize_axes:
            if c not in kernel_axes:
                raise ValueError(f'Axis {c} not found in kernel axes {kernel_axes}')
            if c not in output_axes:
                raise ValueError(f'Axis {c} not found in output axes {output_axes}')
            if self.bias_axes and c not in self.bias_axes:
                raise ValueError(f'Axis {c} not found in bias axes {self.bias_axes}')

    def _compute_fused_einsum_specs(self, input_shape):
        kernel_axes, output_axes = self.equation.split(',')[1].split('->')
        _, cast_shape, output_shape = analyze_einsum(self.equation, self.normalize_axes, tuple(input_shape), self.partial_output_shape)
        normalize_axes = ''.join(c for c in kernel_axes if c in self.normalize_axes)
        self._reduction_axes = tuple(i for i, c in enumerate(output_axes) if c not in normalize_axes)
        norm_shape = tuple(int(output_shape[i]) for i, c in enumerate(output_axes) if c in normalize_axes)
        self._norm_offset_cast_shape = cast_shape
        self.fused_kernel_equation = f'{kernel_axes},{normalize_axes}->{kernel_axes}'
        return norm_shape

    def build(self, input_shape):
        super().build(input_shape)
        norm_shape = self._compute_fused_einsum_specs(input_shape)
        if self.scale:
            self._bn_gamma = self.add_weight(shape=norm_shape, name='gamma', initializer=self.gamma_initializer,
                                             regularizer=self.gamma_regularizer, constraint=self.gamma_constraint)
        assert self.bias is not None
        self._bias.trainable = self.center
        self.moving_mean = self.add_weight(shape=norm_shape, name='moving_mean', initializer=self.moving_mean_initializer,
                                           trainable=False)
        self.moving_variance = self.add_weight(shape=norm_shape, name='moving_variance',
                                               initializer=self.moving_variance_initializer, trainable=False)

    @property
    def bn_gamma(self):
        return self._bn_gamma.value

    def get_fused_qkernel_and_qbias(self, training, mean, var):
        bn_gamma = self._bn_gamma.value if self.scale else 1
        scaler = bn_gamma / torch.sqrt(var + keras_epsilon())
        fused_kernel = torch.einsum(self.fused_kernel_equation, self._kernel.value, scaler)
        fused_qkernel = self.kq(fused_kernel, training=training)
        offset = (-mean * scaler).reshape(self._norm_offset_cast_shape)
        fused_qbias = self.bq(self._bias.value + offset, training=training)
        return fused_qkernel, fused_qbias

    @property
    def qkernel(self):
        return self.get_fused_qkernel_and_qbias(False, self.moving_mean.value, self.moving_variance.value)[0]

    @property
    def qbias(self):
        return self.get_fused_qkernel_and_qbias(False, self.moving_mean.value, self.moving_variance.value)[1]

    def call(self, inputs, training=None):
        if self.enable_iq:
            inputs = self.iq(inputs, training=training)
        if training and self.trainable:
            x = torch.einsum(self.equation, inputs, self._kernel.value)
            mean, var = moments(x, self._reduction_axes, synchronized=self.synchronized)
            self.moving_mean.assign(self.moving_mean.value * self.momentum + mean.detach() * (1.0 - self.momentum))
            self.moving_variance.assign(self.moving_variance.value * self.momentum + var.detach() * (1.0 - self.momentum))
        else:
            var, mean = self.moving_variance.value, self.moving_mean.value
        qkernel, qbias = self.get_fused_qkernel_and_qbias(training, mean, var)
        return self._contract(inputs, qkernel, qbias, training, apply_iq=False)

    def get_config(self):
        config = super().get_config()
        config.update({
            'normalize_axes': self.normalize_axes, 'momentum': self.momentum, 'epsilon': self.epsilon, 'center': self.center,
            'scale': self.scale, 'gamma_initializer': self.gamma_initializer,
            'moving_mean_initializer': self.moving_mean_initializer,
            'moving_variance_initializer': self.moving_variance_initializer, 'gamma_regularizer': self.gamma_regularizer,
            'gamma_constraint': self.gamma_constraint, 'synchronized': self.synchronized,
        })
        return config
