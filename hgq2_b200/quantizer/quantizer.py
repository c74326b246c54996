"""``Quantizer``: the layer every quantised layer holds for its inputs, weights, biases and outputs.

It owns an internal quantizer chosen by a ``QuantizerConfig`` and adds the optional pre-scaling, the training-time noise
blend and the output affine map around it (interface of src/hgq/quantizer/quantizer.py:20-104).
"""

from __future__ import annotations

from ..backend import Layer
from .config import QuantizerConfig, all_quantizer_keys


def _config_from_arguments(args, kwargs):
    """``Quantizer(config)``, ``Quantizer(config=config)`` or ``Quantizer(q_type, place, **overrides)`` -> (config, rest)."""
    if len(args) == 1 and isinstance(args[0], QuantizerConfig):
        return args[0], kwargs
    given = kwargs.pop('config', None)
    if isinstance(given, QuantizerConfig):
        return given, kwargs
    assert given is None, f'config must be a QuantizerConfig object, got {given}'
    overrides = {}
    for key in [k for k in kwargs if k in all_quantizer_keys]:
        overrides[key] = kwargs.pop(key)
    return QuantizerConfig(*args, **overrides), kwargs


def _spread(attribute: str):
    """Method that broadcasts the internal quantizer's bitwidth-shaped ``attribute`` to a data shape."""

    def method(self, shape):
        inner = self.quantizer
        return inner.bw_mapper.bw_to_x(getattr(inner, attribute), shape)

    method.__name__ = attribute + '_'
    return method


class Quantizer(Layer):
    def __init__(self, *args, **kwargs):
        self.config, kwargs = _config_from_arguments(args, kwargs)
        super().__init__(**kwargs)
        self.supports_masking = True
        self.scaler, self.affine, self.qnoise_factor = self.config.scaler, self.config.affine, self.config.qnoise_factor
        self.quantizer = self.config.get_quantizer()

    def get_quantizer_config_kwargs(self, *args, **kwargs):
        return _config_from_arguments(args, kwargs)

    def build(self, input_shape):
        inner = self.quantizer
        inner.build(input_shape)
        inner.built = True
        super().build(input_shape)

    def call(self, inputs, training=None):
        x = inputs if self.scaler is None else inputs / self.scaler
        y = self.quantizer.call(x, training=training)
        if self.scaler is not None:
            y = y * self.scaler
        if training and self.qnoise_factor is not None:
            y = x + self.qnoise_factor * (y - x)
        if self.affine is not None:
            gain, offset = self.affine
            y = y * gain + offset
        return y

    # bitwidth-shaped properties of the internal quantizer, and the same broadcast to a data shape
    bits = property(lambda self: self.quantizer.bits)
    fbits = property(lambda self: self.quantizer.fbits)
    q_type = property(lambda self: self.config.q_type)
    bits_ = _spread('bits')
    fbits_ = _spread('fbits')
    min_ = _spread('min')
    max_ = _spread('max')
    epsilon_ = _spread('epsilon')

    def get_config(self):
        config = super().get_config()
        config['config'] = self.config
        return config

    def __repr__(self):
        return f'{type(self).__name__}(q_type={self.q_type}, name={self.name}, built={self.built})'
