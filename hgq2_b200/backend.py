"""The small slice of the Keras-3 layer protocol that the HGQ2 hot path relies on, on plain PyTorch.

HGQ2's quantizers and layers are ``keras.layers.Layer`` subclasses; under the Keras torch backend
such a layer *is* a ``torch.nn.Module`` whose variables wrap ``torch.nn.Parameter``s.  Keras is
not a dependency of this package, so the few protocol pieces the path touches are provided here
with Keras' names and meaning:

    Layer.add_weight(name, shape, initializer, trainable, dtype, constraint, regularizer)
    Layer.build(input_shape) / built, Layer.__call__(*args, training=None, **kw) with the
    call-context propagation of ``training`` to nested layers, Layer.add_loss / losses,
    Variable.assign / numpy / value / constraint / regularizer, trainable_variables, ...

A model built from these layers trains with any torch optimizer; ``hgq2_b200.train`` has the step
that also applies constraints and regularizers the way Keras' trainer does.
"""

from __future__ import annotations

import math
import threading
from collections.abc import Callable, Sequence

import numpy as np
import torch
from torch import nn

_DTYPES = {
    'float32': torch.float32, 'uint8': torch.uint8, 'int32': torch.int32, 'uint32': torch.uint32, 'bool': torch.bool,
    'float64': torch.float64,
}


def epsilon() -> float:
    """Keras' fuzz factor (keras.config.epsilon() default)."""
    return 1e-7


_default_device: torch.device | None = None


def set_default_device(device) -> None:
    global _default_device
    _default_device = torch.device(device) if device is not None else None


def default_device() -> torch.device:
    if _default_device is not None:
        return _default_device
    if torch.cuda.is_available():
        return torch.device('cuda', torch.cuda.current_device())
    return torch.device('cpu')


# ---- initializers ------------------------------------------------------------------------------
class Initializer:
    def __call__(self, shape, dtype=torch.float32, device=None) -> torch.Tensor:
        raise NotImplementedError

    def clone(self):
        import copy

        return copy.copy(self)


class Constant(Initializer):
    def __init__(self, value=0.0):
        self.value = value

    def __call__(self, shape, dtype=torch.float32, device=None):
        # built on the host and copied over: a variable's initial value costs no kernel launch on the device
        return torch.full(tuple(shape), float(self.value), dtype=torch.float32).to(dtype).to(device)

    def get_config(self):
        return {'value': self.value}


class Zeros(Constant):
    def __init__(self):
        super().__init__(0.0)


class Ones(Constant):
    def __init__(self):
        super().__init__(1.0)


def _fans(shape):
    shape = tuple(shape)
    if len(shape) < 1:
        return 1, 1
    if len(shape) == 1:
        return shape[0], shape[0]
    if len(shape) == 2:
        return shape[0], shape[1]
    receptive = int(np.prod(shape[:-2]))
    return shape[-2] * receptive, shape[-1] * receptive


class GlorotUniform(Initializer):
    """U(-l, l), l = sqrt(6 / (fan_in + fan_out)); drawn with numpy so CPU and GPU models agree."""

    def __init__(self, seed=None):
        self.seed = seed

    def __call__(self, shape, dtype=torch.float32, device=None):
        fan_in, fan_out = _fans(shape)
        limit = math.sqrt(6.0 / max(1.0, fan_in + fan_out))
        rng = np.random.default_rng(self.seed)
        w = rng.uniform(-limit, limit, size=tuple(shape)).astype(np.float32)
        return torch.from_numpy(w).to(device=device, dtype=dtype)


class RandomNormal(Initializer):
    def __init__(self, mean=0.0, stddev=0.05, seed=None):
        self.mean, self.stddev, self.seed = mean, stddev, seed

    def __call__(self, shape, dtype=torch.float32, device=None):
        rng = np.random.default_rng(self.seed)
        w = (rng.standard_normal(tuple(shape)) * self.stddev + self.mean).astype(np.float32)
        return torch.from_numpy(w).to(device=device, dtype=dtype)


def get_initializer(spec) -> Initializer:
    if isinstance(spec, Initializer):
        return spec
    if spec is None or spec == 'zeros':
        return Zeros()
    if spec == 'ones':
        return Ones()
    if spec == 'glorot_uniform':
        return GlorotUniform()
    if isinstance(spec, (int, float)):
        return Constant(spec)
    raise ValueError(f'unknown initializer {spec!r}')


# ---- variables ---------------------------------------------------------------------------------
class Variable:
    """A named tensor owned by a layer.  Trainable float variables wrap an ``nn.Parameter``."""

    def __init__(self, value: torch.Tensor, name: str, trainable: bool, dtype: str, constraint=None, regularizer=None):
        self.name = name
        self.path = name
        self.dtype = dtype
        self.constraint = constraint
        self.regularizer = regularizer
        self._trainable = bool(trainable) and value.is_floating_point()
        self._p = nn.Parameter(value, requires_grad=self._trainable)

    @property
    def trainable(self) -> bool:
        return self._trainable

    @trainable.setter
    def trainable(self, v: bool):
        self._trainable = bool(v) and self._p.is_floating_point()
        self._p.requires_grad_(self._trainable)

    @property
    def value(self) -> nn.Parameter:
        return self._p

    @property
    def shape(self):
        return tuple(self._p.shape)

    def assign(self, value) -> None:
        with torch.no_grad():
            v = torch.as_tensor(value, device=self._p.device)
            self._p.copy_(v.to(self._p.dtype).reshape(self._p.shape) if v.numel() == self._p.numel() else v.to(self._p.dtype).expand(self._p.shape))

    def numpy(self) -> np.ndarray:
        return self._p.detach().cpu().numpy()

    def __repr__(self):
        return f'<Variable {self.path} shape={self.shape} dtype={self.dtype} trainable={self.trainable}>'


# ---- bookkeeping stream ------------------------------------------------------------------------
# The integer-bit tracking of the WRAP quantizers and the EBOPs terms are long chains of tiny kernels on bitwidth-shaped
# tensors.  They depend on a layer's abs-max statistics but nothing downstream in the forward pass depends on them (until
# the losses are summed), so they run on a second stream, forked from and later joined to the stream that carries the
# activations: in the captured step graph this becomes a parallel branch, and autograd replays the backward of those
# nodes on the same second stream.
overlap_bookkeeping = True
_side_streams: dict = {}
# gradients of parameters first touched on the second stream are accumulated there on purpose
if hasattr(torch.autograd.graph, 'set_warn_on_accumulate_grad_stream_mismatch'):
    torch.autograd.graph.set_warn_on_accumulate_grad_stream_mismatch(False)


class bookkeeping:
    """``with bookkeeping(t1, t2, ...):`` -- run the body on the device's bookkeeping stream, ordered after everything
    queued so far on the current stream.  The tensors named are inputs of the body that were allocated on the current
    stream; they are marked as in use by the second stream so that their memory is not handed out again early."""

    def __init__(self, *tensors):
        self.tensors = tensors
        self._ctx = None

    def __enter__(self):
        if not overlap_bookkeeping or not torch.cuda.is_available():
            return self
        dev = torch.cuda.current_device()
        main = torch.cuda.current_stream()
        side = _side_streams.get(dev)
        if side is None:
            side = _side_streams[dev] = torch.cuda.Stream(device=dev)
        if main == side:  # nested region
            return self
        side.wait_stream(main)
        for t in self.tensors:
            if t is not None and t.is_cuda:
                t.record_stream(side)
        self._ctx = torch.cuda.stream(side)
        self._ctx.__enter__()
        return self

    def __exit__(self, *exc):
        if self._ctx is not None:
            self._ctx.__exit__(*exc)
        return False


def queue_params(layers) -> None:
    """Queue the parameter-only part of the coming calls of ``layers`` (their quantised kernels and biases) on the second
    stream, where it runs beside the first layers' activation kernels; each layer picks its result up with
    ``take_prepared``."""
    if not overlap_bookkeeping or not torch.cuda.is_available():
        return
    for layer in layers:
        prep = getattr(layer, 'prepare_params', None)
        if prep is not None and layer.built:
            with bookkeeping():
                layer._prepared = prep()
                layer._prepared_event = torch.cuda.Event()
                layer._prepared_event.record()


def take_prepared(layer):
    """The (quantised kernel, quantised bias) a ``Sequential`` queued ahead for this call of ``layer``, or None.  The current
    stream is made to wait for them."""
    p = getattr(layer, '_prepared', None)
    if p is None:
        return None
    layer._prepared = None
    main = torch.cuda.current_stream()
    main.wait_event(layer._prepared_event)
    for t in p:
        if t is not None:
            t.record_stream(main)
    return p


def current_pass() -> int:
    """Number of the top-level layer call in progress (0 outside any call)."""
    return _ctx.pass_id if _ctx.depth > 0 else 0


def join_bookkeeping() -> None:
    """Make the current stream wait for the bookkeeping stream (before its results -- loss terms -- are consumed)."""
    if not torch.cuda.is_available():
        return
    side = _side_streams.get(torch.cuda.current_device())
    if side is not None and torch.cuda.current_stream() != side:
        torch.cuda.current_stream().wait_stream(side)


# ---- call context ------------------------------------------------------------------------------
class _CallContext(threading.local):
    def __init__(self):
        self.depth = 0
        self.training = None
        self.root = None
        self.pass_id = 0  # number of the current top-level call: per-pass memos (rounded bitwidths) are keyed on it


_ctx = _CallContext()


class Layer(nn.Module):
    _name_counters: dict[str, int] = {}

    def __init__(self, name: str | None = None, trainable: bool = True, dtype: str = 'float32', **kwargs):
        super().__init__()
        if kwargs:
            raise TypeError(f'unexpected arguments for {type(self).__name__}: {sorted(kwargs)}')
        if name is None:
            base = _snake(type(self).__name__)
            n = Layer._name_counters.get(base, 0)
            Layer._name_counters[base] = n + 1
            name = base if n == 0 else f'{base}_{n}'
        self.name = name
        self._trainable = trainable
        self._dtype = dtype
        self.built = False
        self._variables: list[Variable] = []
        self._losses: list[torch.Tensor] = []
        self.supports_masking = False

    # -- keras-style attributes
    @property
    def dtype(self) -> str:
        return self._dtype

    @property
    def trainable(self) -> bool:
        return self._trainable

    @trainable.setter
    def trainable(self, v: bool):
        self._trainable = v

    def add_weight(self, shape=(), initializer=None, dtype=None, trainable=True, name=None, constraint=None,
                   regularizer=None, autocast=True, **_ignored) -> Variable:
        dtype = dtype or 'float32'
        init = get_initializer(initializer)
        value = init(tuple(shape), dtype=_DTYPES[dtype], device=default_device())
        v = Variable(value, name or f'variable_{len(self._variables)}', trainable and self._trainable, dtype, constraint,
                     regularizer)
        v.path = f'{self.name}/{v.name}'
        self._variables.append(v)
        self.register_parameter(f'_v{len(self._variables) - 1}_{v.name}', v.value)
        return v

    def build(self, *args, **kwargs):
        self.built = True

    def compute_output_shape(self, input_shape):
        return input_shape

    def add_loss(self, loss) -> None:
        (_ctx.root if _ctx.root is not None else self)._losses.append(loss)

    @property
    def losses(self) -> list[torch.Tensor]:
        """Losses added during the last top-level call, plus the weight regularisers of every sublayer."""
        out = list(self._losses)
        for layer in self._flatten_layers():
            for v in layer._variables:
                if v.regularizer is not None and v.trainable:
                    out.append(v.regularizer(v.value))
        return out

    def _flatten_layers(self, include_self: bool = True, recursive: bool = True):
        seen = []
        if include_self:
            seen.append(self)
        for m in (self.modules() if recursive else self.children()):
            if m is not self and isinstance(m, Layer):
                seen.append(m)
        return seen

    @property
    def variables(self) -> list[Variable]:
        return [v for layer in self._flatten_layers() for v in layer._variables]

    @property
    def trainable_variables(self) -> list[Variable]:
        return [v for v in self.variables if v.trainable]

    @property
    def non_trainable_variables(self) -> list[Variable]:
        return [v for v in self.variables if not v.trainable]

    def _maybe_build(self, args):
        if self.built:
            return
        shapes = [_shape_of(a) for a in args]
        self.build(*shapes) if len(shapes) != 1 else self.build(shapes[0])
        self.built = True

    def __call__(self, *args, **kwargs):
        top = _ctx.depth == 0
        explicit = kwargs.get('training', None)
        prev_training = _ctx.training
        if explicit is not None:
            _ctx.training = explicit
        training = _ctx.training
        if top:
            _ctx.root = self
            _ctx.pass_id += 1
            self._losses = []
        if _accepts_training(self):
            kwargs['training'] = training
        else:
            kwargs.pop('training', None)
        _ctx.depth += 1
        try:
            self._maybe_build(args)
            return self.call(*args, **kwargs)
        finally:
            _ctx.depth -= 1
            if _ctx.depth == 0:
                join_bookkeeping()  # state, EBOPs and loss terms written on the second stream are visible to the caller
            _ctx.training = prev_training
            if top:
                _ctx.root = None

    def call(self, *args, **kwargs):
        raise NotImplementedError

    def forward(self, *args, **kwargs):  # nn.Module protocol
        return self.__call__(*args, **kwargs)

    def get_config(self):
        return {'name': self.name, 'trainable': self.trainable, 'dtype': self.dtype}


class Lambda(Layer):
    """Wraps a tensor function as a layer (keras.layers.Lambda)."""

    def __init__(self, function, **kwargs):
        super().__init__(**kwargs)
        self.function = function

    def call(self, inputs):
        return self.function(inputs)


class Flatten(Layer):
    def call(self, inputs):
        return inputs.reshape(inputs.shape[0], -1)


class MaxPooling2D(Layer):
    """channels_last 2-D max pooling, 'valid' padding."""

    def __init__(self, pool_size=(2, 2), strides=None, **kwargs):
        super().__init__(**kwargs)
        self.pool_size = (pool_size, pool_size) if isinstance(pool_size, int) else tuple(pool_size)
        self.strides = self.pool_size if strides is None else ((strides, strides) if isinstance(strides, int) else tuple(strides))

    def call(self, inputs):
        if inputs.is_cuda and inputs.dtype == torch.float32 and self.pool_size[0] * self.pool_size[1] <= 255:
            return _MaxPool2dFn.apply(inputs, self.pool_size, self.strides)
        y = torch.nn.functional.max_pool2d(inputs.permute(0, 3, 1, 2), self.pool_size, self.strides)  # channels_last in, channels_last out
        return y.permute(0, 2, 3, 1)


class _MaxPool2dFn(torch.autograd.Function):
    """Max pooling on the library's own kernels: one byte of arg-max per output element instead of an int64 index."""

    @staticmethod
    def forward(ctx, x, pool, strides):
        from . import kernels

        y, arg = kernels.maxpool2d_fwd(x, pool, strides)
        ctx.save_for_backward(arg)
        ctx.geom = (tuple(x.shape), pool, strides)
        return y

    @staticmethod
    def backward(ctx, gy):
        from . import kernels

        (arg,) = ctx.saved_tensors
        shape, pool, strides = ctx.geom
        return kernels.maxpool2d_bwd(gy, arg, shape, pool, strides), None, None


class Sequential(Layer):
    """A linear stack of layers (keras.Sequential)."""

    def __init__(self, layers=(), **kwargs):
        super().__init__(**kwargs)
        self.layers = nn.ModuleList(layer if isinstance(layer, Layer) else Lambda(layer) for layer in layers)

    def build(self, input_shape):
        self.built = True

    def call(self, inputs, training=None):
        if training and torch.is_tensor(inputs) and inputs.is_cuda:
            queue_params(self.layers)
        x = inputs
        for layer in self.layers:
            x = layer(x, training=training)
        return x


_training_arg_cache: dict = {}


def _accepts_training(layer: Layer) -> bool:
    fn = type(layer).call  # keyed on the function: QLayerMeta swaps a class's call once
    r = _training_arg_cache.get(fn)
    if r is None:
        import inspect

        sig = inspect.signature(fn)
        r = 'training' in sig.parameters or any(p.kind == p.VAR_KEYWORD for p in sig.parameters.values())
        _training_arg_cache[fn] = r
    return r


def _shape_of(a):
    if isinstance(a, (tuple, list)):
        return [_shape_of(x) for x in a]
    return tuple(a.shape)


def _snake(name: str) -> str:
    out = []
    for i, ch in enumerate(name):
        if ch.isupper() and i and (not name[i - 1].isupper() or (i + 1 < len(name) and name[i + 1].islower())):
            out.append('_')
        out.append(ch.lower())
    return ''.join(out)


# The process group the batch statistics of ``moments(..., synchronized=True)`` are averaged over: the group of the active
# ``train.DataParallel`` (set while its context is entered), else the default group.
moments_group = None


def moments(x: torch.Tensor, axes, keepdims: bool = False, synchronized: bool = False):
    """Mean and variance over ``axes`` the way keras.ops.moments computes them on the torch backend
    (Var = E[x^2] - E[x]^2).  ``synchronized``: average both statistics over the ranks of the active data-parallel group
    (``moments_group``; the default process group when none is active; equal shard sizes), differentiably -- the torch
    backend of Keras refuses this flag; data-parallel training here supports it."""
    axes = tuple(axes) if not isinstance(axes, int) else (axes,)
    mean = torch.mean(x, dim=axes, keepdim=True)
    mean_sq = torch.mean(torch.square(x), dim=axes, keepdim=True)
    if synchronized:
        import torch.distributed as dist

        if dist.is_available() and dist.is_initialized() and dist.get_world_size(moments_group) > 1:
            import torch.distributed.nn.functional as dfn

            stats = dfn.all_reduce(torch.cat([mean.reshape(-1), mean_sq.reshape(-1)]), group=moments_group)
            stats = stats / dist.get_world_size(moments_group)
            mean, mean_sq = stats[:mean.numel()].view_as(mean), stats[mean.numel():].view_as(mean_sq)
    variance = mean_sq - torch.square(mean)
    if not keepdims:
        mean = mean.squeeze(axes) if axes else mean
        variance = variance.squeeze(axes) if axes else variance
    return mean, variance


# ---- activations -------------------------------------------------------------------------------
def get_activation(spec) -> Callable | None:
    if spec is None or spec == 'linear':
        return None
    if callable(spec):
        return spec
    if spec == 'relu':
        return torch.relu
    if spec == 'softmax':
        return lambda x: torch.softmax(x, dim=-1)
    if spec == 'tanh':
        return torch.tanh
    if spec == 'sigmoid':
        return torch.sigmoid
    raise ValueError(f'unknown activation {spec!r}')


def activation_name(spec) -> str | None:
    if spec is None or spec == 'linear':
        return None
    return spec if isinstance(spec, str) else getattr(spec, '__name__', 'custom')


numbers = (int, float, np.integer, np.floating)

__all__ = ['Layer', 'Sequential', 'Lambda', 'Flatten', 'MaxPooling2D', 'Variable', 'Initializer', 'Constant', 'Zeros', 'Ones', 'GlorotUniform', 'RandomNormal',
           'get_initializer', 'get_activation', 'activation_name', 'epsilon', 'numbers', 'default_device',
           'set_default_device', 'Sequence']
