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


def _with_ebops_and_oq(layer_call):
    """``layer_call`` followed by what every quantised layer does after its own computation: account the EBOPs of the call
    (training and calibration only) and quantise the output if the layer has an output quantizer it does not apply
    itself.  ``training`` is accepted even if ``layer_call`` does not take it."""
    signature = inspect.signature(layer_call)
    parameters = signature.parameters
    takes_training = 'training' in parameters
    takes_kwargs = any(p.kind is inspect.Parameter.VAR_KEYWORD for p in parameters.values())

    @wraps(layer_call)
    def call(self, *args, **kwargs):
        training = kwargs.get('training') if takes_training else kwargs.pop('training', None)
        result = layer_call(self, *args, **kwargs)
        if self.enable_ebops and (training or training == 'tracing'):  # noqa: E712 -- may be a flag object
            inputs = args[0] if isinstance(args[0], (tuple, list)) else args
            with bookkeeping():
                self._account_ebops(*[(1,) + tuple(t.shape[1:]) for t in inputs])
        if self.enable_oq and not self.__output_quantizer_handled__:
            if isinstance(result, (tuple, list)):
                raise AssertionError(f'Layer {self.name}({type(self)}) returns multiple outputs, which must be handled in subclasses.')
            result = self.oq(result, training=training)
        return result

    if not takes_training and not takes_kwargs:
        extra = inspect.Parameter('training', inspect.Parameter.KEYWORD_ONLY, default=None)
        call.__signature__ = signature.replace(parameters=[*parameters.values(), extra])
    call.__ebops_wrapped__ = True
    return call


class QLayerMeta(ABCMeta):
    """On the first instantiation of a concrete layer class, swaps its ``call`` for the wrapped one (the reference does the
    same at src/hgq/layers/core/base.py:57-116).  A ``call`` inherited from a parent that is already wrapped is left alone:
    the reference wraps it a second time when the parent class was instantiated first (QMeanPow2 after QSum), which adds
    the EBOPs loss term twice depending on instantiation order; here the accounting happens once whatever the order."""

    _wrapped_cls: set = set()

    def __call__(cls, *args, **kwargs):
        if cls not in QLayerMeta._wrapped_cls:
            QLayerMeta._wrapped_cls.add(cls)
            own = cls.call
            concrete = own is not Layer.call and cls._compute_ebops is not QLayerBase._compute_ebops
            if concrete and not getattr(cls, '__no_wrap_call__', False) and not getattr(own, '__ebops_wrapped__', False):
                cls.call = _with_ebops_and_oq(own)
        return super().__call__(*args, **kwargs)


def _choose(value, key):
    """An explicit constructor argument wins over the layer-scope default."""
    return global_config[key] if value is None else value


def _default_datalane(conf):
    return conf if conf is not None else QuantizerConfig('default', 'datalane')


class QLayerBase(Layer, metaclass=QLayerMeta):
    """What every quantised layer has besides its own computation (interface of src/hgq/layers/core/base.py:119-262):
    the switches ``enable_iq`` / ``enable_oq`` / ``enable_ebops`` resolved against the layer scope, an optional output
    quantizer ``oq``, and, when EBOPs are accounted, the scalar variables ``beta`` (loss weight, fp32) and ``ebops`` (last
    estimate, uint32)."""

    __output_quantizer_handled__ = False

    def __init__(self, enable_ebops: bool | None = None, beta0=None, enable_oq: bool | None = None,
                 enable_iq: bool | None = None, oq_conf: QuantizerConfig | None = None, ebops_factor: float = 1.0,
                 **kwargs):
        super().__init__(**kwargs)
        self._enable_iq = _choose(enable_iq, 'enable_iq')
        self._enable_oq = _choose(enable_oq, 'enable_oq')
        # without an input quantizer there are no input bitwidths to cost
        self._enable_ebops = (global_config['enable_ebops'] and self._enable_iq) if enable_ebops is None else enable_ebops
        beta0 = _choose(beta0, 'beta0')
        self._beta0 = beta0 if isinstance(beta0, Initializer) else Constant(float(beta0))
        self.ebops_factor = ebops_factor
        self._beta = self._ebops = None
        if self._enable_oq:
            self._oq = Quantizer(_default_datalane(oq_conf), name=f'{self.name}_oq')

    enable_iq = property(lambda self: self._enable_iq)
    enable_oq = property(lambda self: self._enable_oq)
    enable_ebops = property(lambda self: self._enable_ebops)

    @property
    def oq(self):
        if self._enable_oq:
            return self._oq
        raise AttributeError(f'oq has been disabled for {self.name}.')

    def _scalar(self, variable, dtype):
        return torch.zeros((), dtype=dtype) if variable is None else variable.value.detach()

    beta = property(lambda self: self._scalar(self._beta, torch.float32))
    ebops = property(lambda self: self._scalar(self._ebops, torch.uint32))

    def build(self, *args, **kwargs):
        super().build(*args, **kwargs)
        self._beta = self._ebops = None
        if self._enable_ebops:
            self._beta = self.add_weight(name='beta', shape=(), initializer=self._beta0, trainable=False)
            self._ebops = self.add_weight(name='ebops', shape=(), initializer=Constant(0.0), trainable=False, dtype='uint32')
        if self._enable_oq and not self._oq.built:
            self.try_build_output_quantizer(*args, **kwargs)

    def try_build_output_quantizer(self, input_shape=None, *args, **kwargs):
        """Builds ``oq`` on the layer's output shape when that can be told from the input shape alone."""
        try:
            output_shape = self.compute_output_shape(input_shape)
        except Exception:
            return
        self._oq.build(output_shape)
        self._oq.built = True

    def get_config(self):
        config = super().get_config()
        config.update(enable_ebops=self._enable_ebops, ebops_factor=self.ebops_factor, beta0=self._beta0,
                      enable_oq=self._enable_oq, enable_iq=self._enable_iq,
                      oq_conf=self._oq.config if self._enable_oq else None)
        return config

    def _compute_ebops(self, *args, **kwargs):
        raise NotImplementedError('This method is abstract and should be implemented in subclasses.')

    def _account_ebops(self, *shapes):
        """EBOPs of one call at batch size 1: stored (truncated to uint32) in ``ebops`` and added, times ``beta``, to the
        losses of the pass."""
        ebops = self._compute_ebops(*shapes) * self.ebops_factor
        self._ebops.assign(ebops.detach().to(torch.uint32))
        self.add_loss(ebops * self.beta)


class QLayerBaseSingleInput(QLayerBase):
    """A quantised layer with one input and one input quantizer ``iq``."""

    def __init__(self, iq_conf: QuantizerConfig | None = None, **kwargs):
        super().__init__(**kwargs)
        if self._enable_iq:
            self._iq = Quantizer(_default_datalane(iq_conf), name=f'{self.name}_iq')

    @property
    def iq(self):
        if self._enable_iq:
            return self._iq
        raise AttributeError(f'iq has been disabled for {self.name}.')

    def build(self, input_shape):
        super().build(input_shape)
        if self._enable_iq and not self._iq.built:
            self._iq.build(input_shape)
            self._iq.built = True

    def get_config(self):
        config = super().get_config()
        config['iq_conf'] = self._iq.config if self._enable_iq else None
        return config


class MultipleQuantizers(Layer):
    """One ``Quantizer`` per input of a multi-input layer; calling it quantises a sequence element by element."""

    def __init__(self, configs: Sequence[QuantizerConfig], **kwargs):
        super().__init__(**kwargs)
        self.quantizers = torch.nn.ModuleList([Quantizer(c) for c in configs])

    def build(self, shapes):
        for quantizer, shape in zip(self.quantizers, shapes):
            quantizer.build(shape)
            quantizer.built = True
        self.built = True

    def call(self, x, **kwargs):
        if len(x) != len(self.quantizers):
            raise AssertionError(f'{self.name} ({type(self).__name__}) expects {len(self.quantizers)} inputs, got {len(x)}.')
        return tuple(q(t, **kwargs) for q, t in zip(self.quantizers, x))

    def __len__(self):
        return len(self.quantizers)

    def __bool__(self):
        return len(self) > 0

    def __iter__(self):
        return iter(self.quantizers)

    def __getitem__(self, item):
        return self.quantizers[item]


class QLayerBaseMultiInputs(QLayerBase):
    """A quantised layer with several inputs: ``iq`` is a ``MultipleQuantizers`` built once the number of inputs is known;
    ``iq_confs`` may be one config for all inputs or one per input."""

    def __init__(self, iq_confs: Sequence[QuantizerConfig] | QuantizerConfig | None = None, **kwargs):
        super().__init__(**kwargs)
        if self._enable_iq:
            self._iq_confs = _default_datalane(iq_confs)

    @property
    def iq(self):
        if not self._enable_iq:
            raise AttributeError(f'iq has been disabled for {self.name}.')
        if not self.built:
            raise AttributeError(f'iqs is not available before build for {self.name}.')
        return self._iq

    @property
    def iq_confs(self):
        assert self._enable_iq, f'iq_confs has been disabled for {self.name}.'
        return self._iq_confs

    def build(self, input_shape):
        super().build(input_shape)
        if not self._enable_iq:
            return
        shapes = list(input_shape)
        for shape in shapes:
            if not isinstance(shape, Iterable):
                raise AssertionError(f'each element of input_shape must be iterable, got {shape}')
        confs = self._iq_confs
        if isinstance(confs, QuantizerConfig):
            confs = [confs] * len(shapes)
        if len(confs) != len(shapes):
            raise AssertionError(f'number of iq_confs must match number of inputs, got {len(confs)} != {len(shapes)}')
        self._iq_confs = confs
        self._iq = MultipleQuantizers(confs)
        self._iq.build(shapes)

    def get_config(self):
        config = super().get_config()
        config['iq_confs'] = self._iq_confs if self._enable_iq else None
        return config
