"""Base classes of the quantised layers and the metaclass that adds EBOPs and the output quantizer.

Mirror of src/hgq/layers/core/base.py.  ``QLayerMeta`` replaces ``call`` of every concrete layer class
once (on first instantiation, reference :57-116): after the layer's own ``call`` it computes the
layer's EBOPs at batch size 1, stores them in the uint32 ``ebops`` variable, adds ``ebops * beta`` to
the losses, and applies the output quantizer if one is enabled.
"""

from __future__ import annotations

import inspect
from abc import ABCMeta
from collections.abc import Iterable, Sequence
from functools import wraps

import torch

from ...backend import Constant, Initializer, Layer, bookkeeping
from ...config.layer import global_config
from ...quantizer import Quantizer, QuantizerConfig


class QLayerMeta(ABCMeta):
    _wrapped_cls: set = set()

    def __call__(cls, *args, **kwargs):
        if cls in QLayerMeta._wrapped_cls:
            return super().__call__(*args, **kwargs)
        QLayerMeta._wrapped_cls.add(cls)
        original_call = cls.call
        if original_call is not Layer.call and cls._compute_ebops is not QLayerBase._compute_ebops:
            signature = inspect.signature(original_call)
            has_training = 'training' in signature.parameters
            has_var_keyword = any(v.kind == inspect.Parameter.VAR_KEYWORD for v in signature.parameters.values())
            new_signature = signature
            if not has_training and not has_var_keyword:
                params = dict(signature.parameters)
                params['training'] = inspect.Parameter('training', inspect.Parameter.KEYWORD_ONLY, default=None)
                new_signature = signature.replace(parameters=list(params.values()))

            # An inherited call that a parent class already wrapped is not wrapped again: the reference wraps it a second
            # time when the parent was instantiated first (QMeanPow2 after QSum), which adds the EBOPs loss term twice
            # depending on instantiation order; here the accounting happens once whatever the order.
            if not getattr(cls, '__no_wrap_call__', False) and not getattr(original_call, '__ebops_wrapped__', False):

                @wraps(original_call)
                def call(self, *args, **kwargs):
                    training = kwargs.get('training', None) if has_training else kwargs.pop('training', None)
                    r = original_call(self, *args, **kwargs)
                    if (training or training == 'tracing') and self.enable_ebops:  # noqa: E712
                        tensors = args[0] if isinstance(args[0], (tuple, list)) else args
                        with bookkeeping():
                            self._account_ebops(*((1,) + tuple(t.shape[1:]) for t in tensors))
                    if not self.enable_oq or self.__output_quantizer_handled__:
                        return r
                    assert not isinstance(r, (tuple, list)), (
                        f'Layer {self.name}({type(self)}) returns multiple outputs, which must be handled in subclasses.'
                    )
                    return self.oq(r, training=training)

                call.__signature__ = new_signature
                call.__ebops_wrapped__ = True
                cls.call = call
        return super().__call__(*args, **kwargs)


class QLayerBase(Layer, metaclass=QLayerMeta):
    """Owns the optional input/output quantizers and the ``beta`` / ``ebops`` variables of a quantised layer."""

    __output_quantizer_handled__ = False

    def __init__(self, enable_ebops: bool | None = None, beta0=None, enable_oq: bool | None = None,
                 enable_iq: bool | None = None, oq_conf: QuantizerConfig | None = None, ebops_factor: float = 1.0,
                 **kwargs):
        super().__init__(**kwargs)
        beta0 = beta0 if beta0 is not None else global_config['beta0']
        beta0 = Constant(float(beta0)) if not isinstance(beta0, Initializer) else beta0
        self._enable_iq = enable_iq if enable_iq is not None else global_config['enable_iq']
        self._enable_oq = enable_oq if enable_oq is not None else global_config['enable_oq']
        if enable_ebops is None:
            enable_ebops = global_config['enable_ebops'] and self.enable_iq
        self._enable_ebops = enable_ebops
        self._beta0 = beta0
        self.ebops_factor = ebops_factor
        self._beta = None
        self._ebops = None
        if self.enable_oq:
            oq_conf = oq_conf or QuantizerConfig('default', 'datalane')
            self._oq = Quantizer(oq_conf, name=f'{self.name}_oq')

    @property
    def enable_iq(self):
        return self._enable_iq

    @property
    def enable_oq(self):
        return self._enable_oq

    @property
    def oq(self):
        if not self.enable_oq:
            raise AttributeError(f'oq has been disabled for {self.name}.')
        return self._oq

    @property
    def beta(self):
        if self._beta is None:
            return torch.zeros((), dtype=torch.float32)
        return self._beta.value.detach()

    @property
    def ebops(self):
        if self._ebops is None:
            return torch.zeros((), dtype=torch.uint32)
        return self._ebops.value.detach()

    @property
    def enable_ebops(self):
        return self._enable_ebops

    def build(self, *args, **kwargs):
        super().build(*args, **kwargs)
        if self.enable_ebops:
            self._beta = self.add_weight(name='beta', shape=(), initializer=self._beta0, trainable=False)
            self._ebops = self.add_weight(name='ebops', shape=(), initializer=Constant(0.0), trainable=False, dtype='uint32')
        else:
            self._beta = None
            self._ebops = None
        if not self.enable_oq or self.oq.built:
            return
        self.try_build_output_quantizer(*args, **kwargs)

    def try_build_output_quantizer(self, input_shape=None, *args, **kwargs):
        try:
            output_shape = self.compute_output_shape(input_shape)
        except Exception:
            return
        self.oq.build(output_shape)
        self.oq.built = True

    def get_config(self):
        config = super().get_config()
        config.update(
            {
                'enable_ebops': self.enable_ebops,
                'ebops_factor': self.ebops_factor,
                'beta0': self._beta0,
                'enable_oq': self.enable_oq,
                'enable_iq': self.enable_iq,
                'oq_conf': self.oq.config if self.enable_oq else None,
            }
        )
        return config

    def _compute_ebops(self, *args, **kwargs):
        raise NotImplementedError('This method is abstract and should be implemented in subclasses.')

    def _account_ebops(self, *shapes):
        """What the call wrapper does after a training forward: EBOPs at batch 1 -> uint32 variable and loss term."""
        ebops = self._compute_ebops(*shapes) * self.ebops_factor
        self._ebops.assign(ebops.detach().to(torch.uint32))
        self.add_loss(ebops * self.beta)


class QLayerBaseSingleInput(QLayerBase):
    def __init__(self, iq_conf: QuantizerConfig | None = None, **kwargs):
        super().__init__(**kwargs)
        if self.enable_iq:
            iq_conf = iq_conf or QuantizerConfig('default', 'datalane')
            self._iq = Quantizer(iq_conf, name=f'{self.name}_iq')

    @property
    def iq(self):
        if not self.enable_iq:
            raise AttributeError(f'iq has been disabled for {self.name}.')
        return self._iq

    def build(self, input_shape):
        super().build(input_shape)
        if self.enable_iq and not self._iq.built:
            self.iq.build(input_shape)
            self.iq.built = True

    def get_config(self):
        config = super().get_config()
        config['iq_conf'] = self.iq.config if self.enable_iq else None
        return config


class MultipleQuantizers(Layer):
    def __init__(self, configs: Sequence[QuantizerConfig], **kwargs):
        super().__init__(**kwargs)
        self.quantizers = torch.nn.ModuleList(Quantizer(config) for config in configs)

    def call(self, x, **kwargs):
        assert len(self) == len(x), f'{self.name} ({self.__class__.__name__}) expects {len(self)} inputs, got {len(x)}.'
        return tuple(f(x_, **kwargs) for f, x_ in zip(self, x))

    def build(self, shapes):
        for q, shape in zip(self.quantizers, shapes):
            q.build(shape)
            q.built = True
        self.built = True

    def __bool__(self):
        return len(self.quantizers) > 0

    def __len__(self):
        return len(self.quantizers)

    def __getitem__(self, item):
        return self.quantizers[item]

    def __iter__(self):
        return iter(self.quantizers)


class QLayerBaseMultiInputs(QLayerBase):
    def __init__(self, iq_confs: Sequence[QuantizerConfig] | QuantizerConfig | None = None, **kwargs):
        super().__init__(**kwargs)
        if self.enable_iq:
            self._iq_confs = iq_confs if iq_confs is not None else QuantizerConfig('default', 'datalane')

    @property
    def iq(self):
        if not self.enable_iq:
            raise AttributeError(f'iq has been disabled for {self.name}.')
        if not self.built:
            raise AttributeError(f'iqs is not available before build for {self.name}.')
        return self._iq

    @property
    def iq_confs(self):
        assert self.enable_iq, f'iq_confs has been disabled for {self.name}.'
        return self._iq_confs

    def build(self, input_shape):
        super().build(input_shape)
        if not self.enable_iq:
            return
        n_input = len(input_shape)
        for shape in input_shape:
            assert isinstance(shape, Iterable), f'each element of input_shape must be iterable, got {shape}'
        if isinstance(self.iq_confs, QuantizerConfig):
            self._iq_confs = [self.iq_confs] * n_input
        assert len(self.iq_confs) == n_input, (
            f'number of iq_confs must match number of inputs, got {len(self._iq_confs)} != {n_input}'
        )
        self._iq = MultipleQuantizers(self._iq_confs)
        self._iq.build(input_shape)
