"""The generic ``Quantizer`` layer: scaler / noise blend / affine around an internal quantizer.

Mirror of src/hgq/quantizer/quantizer.py:20-104.
"""

from __future__ import annotations

from ..backend import Layer
from .config import QuantizerConfig, all_quantizer_keys


class Quantizer(Layer):
    """Wraps an internal quantizer behind one interface.  ``Quantizer(config)`` or
    ``Quantizer(q_type='default', place='datalane', **config_overrides)``."""

    def __init__(self, *args, **kwargs):
        self.config, kwargs = self.get_quantizer_config_kwargs(*args, **kwargs)
        super().__init__(**kwargs)
        self.supports_masking = True
        self.qnoise_factor = self.config.qnoise_factor
        self.scaler = self.config.scaler
        self.affine = self.config.affine
        self.quantizer = self.config.get_quantizer()

    def build(self, input_shape):
        self.quantizer.build(input_shape)
        self.quantizer.built = True
        super().build(input_shape)

    def get_quantizer_config_kwargs(self, *args, **kwargs):
        if len(args) == 1 and isinstance(args[0], QuantizerConfig):
            return args[0], kwargs
        config = kwargs.pop('config', None)
        if isinstance(config, QuantizerConfig):
            return config, kwargs
        assert config is None, f'config must be a QuantizerConfig object, got {config}'
        own = {k: kwargs.pop(k) for k in list(kwargs) if k in all_quantizer_keys}
        return QuantizerConfig(*args, **own), kwargs

    def call(self, inputs, training=None):
        if self.scaler is not None:
            inputs = inputs / self.scaler
        outputs = self.quantizer.call(inputs, training=training)
        if self.scaler is not None:
            outputs = outputs * self.scaler
        if self.qnoise_factor is not None and training:
            outputs = inputs + self.qnoise_factor * (outputs - inputs)
        if self.affine is not None:
            outputs = outputs * self.affine[0] + self.affine[1]
        return outputs

    def get_config(self):
        config = super().get_config()
        config['config'] = self.config
        return config

    @property
    def bits(self):
        return self.quantizer.bits

    @property
    def fbits(self):
        return self.quantizer.fbits

    @property
    def q_type(self):
        return self.config.q_type

    def __repr__(self):
        return f'{self.__class__.__name__}(q_type={self.config.q_type}, name={self.name}, built={self.built})'

    def bits_(self, shape):
        return self.quantizer.bw_mapper.bw_to_x(self.bits, shape)

    def fbits_(self, shape):
        return self.quantizer.bw_mapper.bw_to_x(self.fbits, shape)

    def min_(self, shape):
        return self.quantizer.bw_mapper.bw_to_x(self.quantizer.min, shape)

    def max_(self, shape):
        return self.quantizer.bw_mapper.bw_to_x(self.quantizer.max, shape)

    def epsilon_(self, shape):
        return self.quantizer.bw_mapper.bw_to_x(self.quantizer.epsilon, shape)
