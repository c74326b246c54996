"""Stateful fixed-point quantizers, KBI and KIF parametrisations.

Mirror of src/hgq/quantizer/internal/fixed_point_quantizer.py: same constructor arguments,
variable names (``k`` uint8; ``b``/``i`` or ``i``/``f`` fp32; scalar ``i_decay_speed`` for WRAP),
properties and ``call(inputs, training)`` branches.  The element-wise work runs in the K1 CUDA
kernels through ``get_fixed_quantizer``; what stays in PyTorch is arithmetic on the bitwidth-shaped
tensors themselves (a few hundred elements).
"""

from __future__ import annotations

import weakref

import numpy as np
import torch

from ...backend import Constant, Initializer, bookkeeping, current_pass, epsilon
from ...constraints import Constraint, MinMax
from ...regularizers import Regularizer
from .. import fixed_point_ops
from ..fixed_point_ops import get_fixed_quantizer, round_conv
from .base import DefaultBitwidthMapper, TrainableQuantizerBase, numbers


# Set by hgq2_b200.train.DataParallel: a function applied to the abs-max statistics of *activations* before they
# update the integer bits (a MAX all-reduce over the data-parallel ranks).  None = single process.
absmax_sync_hook = None


def _sync_absmax(absmax, inputs):
    if absmax_sync_hook is not None and not isinstance(inputs, torch.nn.Parameter):
        return absmax_sync_hook(absmax.contiguous())
    return absmax


def _fused_track_kif(absmax, f_var, i_var, decay_var) -> bool:
    """i <- max(i - decay, minimal_i_given_xf(absmax, round(f))) in one kernel launch; False if the tensors do not qualify."""
    from ... import kernels

    am = absmax.reshape(i_var.value.shape)
    if not (am.is_cuda and kernels.track_supported(am.contiguous(), f_var.value, i_var.value)):
        return False
    kernels.track_kif(am.contiguous(), f_var.value.detach(), i_var.value.detach(), decay_var.value)
    return True


def _fused_track_kbi(absmax, b_var, i_var, decay_var, symmetric) -> bool:
    from ... import kernels

    c = i_var.constraint
    if c is None:
        lo, hi = float('-inf'), float('inf')
    elif isinstance(c, MinMax):
        lo, hi = c.min_value, c.max_value
    else:
        return False
    am = absmax.reshape(i_var.value.shape)
    if not (am.is_cuda and kernels.track_supported(am.contiguous(), b_var.value, i_var.value)):
        return False
    kernels.track_kbi(am.contiguous(), b_var.value.detach(), i_var.value.detach(), decay_var.value, symmetric, lo, hi)
    return True


def minimal_i_given_xb(x, b, symmetric=False):
    """Fewest integer bits that hold |x| with b total bits (reference :16-22)."""
    eps = epsilon()
    if symmetric:
        return torch.ceil(torch.log2((x + eps) / (1 - 2.0**-b + eps)))
    i_pos = torch.ceil(torch.log2((x + eps) / (1 - 2.0**-b + eps)))
    i_neg = torch.ceil(torch.log2(-x - eps))
    return torch.where(b > 0, torch.where(x >= 0, i_pos, i_neg), torch.full_like(i_pos, 32.0))


def minimal_i_given_xf(x, f, symmetric=False):
    """Fewest integer bits that hold |x| with f fractional bits (reference :25-31)."""
    eps = epsilon()
    if symmetric:
        return torch.ceil(torch.log2(torch.abs(x) + 2.0**-f))
    i_pos = torch.ceil(torch.log2(x + 2.0**-f))
    i_neg = torch.ceil(torch.log2(-x - eps))
    return torch.where(x >= 0, i_pos, i_neg)


class FixedPointQuantizerBase(TrainableQuantizerBase):
    """Abstract base class for all fixed-point quantizers."""

    def __init__(self, **kwargs):
        super().__init__(**kwargs)
        self._seed_gen = None
        self._is_weight = False

    @property
    def round_mode(self) -> str:
        return self._round_mode

    @property
    def overflow_mode(self) -> str:
        return self._overflow_mode

    @property
    def seed_gen(self):
        return self._seed_gen

    def build(self, input_shape):
        super().build(input_shape)
        self.stateless_quantizer = get_fixed_quantizer(self.round_mode, self.overflow_mode)
        if self.overflow_mode == 'WRAP':
            init = self._i_decay_speed0
            self._i_decay_speed = self.add_weight(name='i_decay_speed', shape=(), initializer=init, trainable=False)
        self._symmetric = self.overflow_mode.endswith('SYM')

    @property
    def symmetric(self):
        return self._symmetric

    def _rounded(self, var):
        """round_conv(variable), computed once per forward pass and variable state: the properties b / i / f / bits are
        read several times in one pass (quantizer call, fused-kernel plan, EBOPs), each read otherwise costing a launch
        forward and a gradient sum backward."""
        p = var.value
        tag = (current_pass(), p._version, torch.is_grad_enabled(), p.requires_grad)
        memo = self.__dict__.setdefault('_round_memo', {})
        hit = memo.get(var.name)
        if tag[0] != 0 and hit is not None and hit[0] == tag:
            r = hit[1]()
            if r is not None:
                return r
        r = round_conv(p)
        # a weak reference: the result lives as long as the pass's autograd graph uses it and no longer (a strong one would
        # keep the variable's gradient accumulator alive across steps, pinned to the stream of the step that made it)
        memo[var.name] = (tag, weakref.ref(r))
        return r

    def _state_written(self, var) -> None:
        """A kernel wrote the variable in place (no version bump): drop its memo."""
        self.__dict__.get('_round_memo', {}).pop(var.name, None)

    @property
    def i_decay_speed(self):
        return self._i_decay_speed.value.detach()

    @property
    def kif(self):
        raise NotImplementedError

    @property
    def bits(self):
        planned = self.__dict__.get('_engine_bits')
        if planned is not None:  # a step engine holds this quantizer's bit counts as a table of its own (hgq2_b200.engine)
            return planned
        if self.overflow_mode != 'SAT':
            return self.b
        return self.b + self.k

    @property
    def fbits(self):
        b = self.b
        if self.overflow_mode == 'WRAP':
            return b + self.k * (b > 0).to(b.dtype)
        return b + self.k

    @property
    def min(self):
        if self.symmetric:
            return -self.k * (2.0**self.i - 2.0**-self.f)
        return -self.k * (2.0**self.i)

    @property
    def max(self):
        return 2.0**self.i - 2.0**-self.f

    @property
    def epsilon(self):
        return 2.0**-self.f

    def get_any_k(self, inputs):
        return self.bw_mapper.x_to_bw_sign(inputs)

    def __repr__(self) -> str:
        if not self.built:
            return f'{self.__class__.__name__}({self.round_mode}, {self.overflow_mode}, name={self.name}, built=False)'
        k, i, f = (t.detach().cpu().numpy() for t in (self.k, self.i, self.f))
        return (
            f'{self.__class__.__name__}(k={np.mean(k):.2f}±{np.std(k):.2f}, i={np.mean(i):.2f}±{np.std(i):.2f}, '
            f'f={np.mean(f):.2f}±{np.std(f):.2f}, {self.round_mode}, {self.overflow_mode}, name={self.name})'
        )

    # -- helpers on top of the CUDA seam ---------------------------------------------------------
    def _round_and_absmax(self, inputs, f):
        """round(inputs, f) plus x_to_bw_absmax of the result, fused in one kernel when the mapper is the default one."""
        if isinstance(self.bw_mapper, DefaultBitwidthMapper) and fixed_point_ops.trailing_period(inputs.shape, f.shape):
            r, amax = fixed_point_ops.round_with_absmax(inputs, f, self.round_mode)
            return r, amax.view(f.shape)
        r = self.stateless_quantizer.round(inputs, f, False, self.seed_gen)
        return r, self.bw_mapper.x_to_bw_absmax(r.detach())

    def call(self, inputs, training=None):
        k, i, f = self.kif
        zero = not training  # eval: where(k + i + f > 0, ret, 0), fused into the kernel
        return self.stateless_quantizer(inputs, self._k.value, i, f, training is True, self.seed_gen, zero_nonpos=zero)

    # -- inline application by a consumer kernel ---------------------------------------------------
    def fusion_plan(self, training):
        """How a consuming kernel applies this quantizer to its input inline, mirroring the branches of ``call``.

        Returns None when the call cannot be inlined (calibration mode, or a state update that must see the whole
        tensor before any element is quantised); otherwise a dict with the stateless quantizer's modes and flags,
        the bitwidth-shaped ``k``, ``i``, ``f`` tensors (differentiable), and ``track``: a function the caller
        invokes with the abs-max of the rounded input to update the integer bits, or None.
        """
        if training == 'tracing':  # noqa: E712
            return None
        plan = dict(round_mode=self.round_mode, k=self._k.value, track=None)
        if self.overflow_mode == 'WRAP' and self.trainable:
            if training:
                return self._wrap_training_plan(plan)
            if self._is_weight and (self._kif_like or self.round_mode == 'RND'):
                plan.update(overflow_mode='NONE', training=True, zero=False, i=None, f=self.f)
                return plan
        k, i, f = self.kif
        plan.update(overflow_mode=self.overflow_mode, training=training is True, zero=not training, i=i, f=f)
        return plan

    _kif_like = False

    def _wrap_training_plan(self, plan):
        return None


class FixedPointQuantizerKBI(FixedPointQuantizerBase):
    """Fixed-point quantizer parameterised by keep_negative, total bits and integer bits."""

    def __init__(
        self,
        k0: numbers | bool | Initializer,
        b0: numbers | Initializer,
        i0: numbers | Initializer,
        round_mode: str,
        overflow_mode: str,
        bc: Constraint | None = MinMax(0, 12),
        ic: Constraint | None = None,
        br: Regularizer | None = None,
        ir: Regularizer | None = None,
        i_decay_speed: numbers = float('inf'),
        is_weight: bool = False,
        **kwargs,
    ):
        super().__init__(**kwargs)
        if not isinstance(k0, Initializer) and not isinstance(b0, Initializer) and not isinstance(i0, Initializer):
            k0 = int(k0)
            assert k0 == 0 or k0 == 1, f'Invalid k0 value {k0}: must be 0 or 1.'
            assert b0 >= 0, f'Invalid b0 value {b0}: must be non-negative.'
        self._k0 = k0 if isinstance(k0, Initializer) else Constant(float(k0))
        self._b0 = b0 if isinstance(b0, Initializer) else Constant(float(b0))
        self._i0 = i0 if isinstance(i0, Initializer) else Constant(float(i0))
        self._i_decay_speed0 = i_decay_speed if isinstance(i_decay_speed, Initializer) else Constant(float(i_decay_speed))
        self._round_mode = round_mode.upper()
        self._overflow_mode = overflow_mode.upper()
        self.b_constraint = bc
        self.i_constraint = ic
        self.b_regularizer = br
        self.i_regularizer = ir
        self._is_weight = is_weight
        self.validate_config()

    def build(self, input_shape):
        bw_shape = self.bw_mapper.inference_weight_shape(input_shape)
        self._k = self.add_weight(name='k', shape=bw_shape, initializer=self._k0, trainable=False, dtype='uint8')
        self._b = self.add_weight(
            name='b', shape=bw_shape, initializer=self._b0, trainable=True, constraint=self.b_constraint,
            regularizer=self.b_regularizer,
        )
        i_trainable = self.overflow_mode != 'WRAP'
        self._i = self.add_weight(
            name='i', shape=bw_shape, initializer=self._i0, trainable=i_trainable, constraint=self.i_constraint,
            regularizer=self.i_regularizer,
        )
        super().build(input_shape)

    @property
    def k(self):
        return self._k.value.to(torch.float32)

    @property
    def b(self):
        return self._rounded(self._b)

    @property
    def i(self):
        return self._rounded(self._i)

    @property
    def f(self):
        return self.b - self.i

    @property
    def kif(self):
        k, b, i = self.k, self.b, self.i
        return k, i, b - i

    def get_minimal_i(self, inputs):
        xr = self.bw_mapper.x_to_bw_absmax(inputs)
        return minimal_i_given_xb(xr, self.b.detach(), self.symmetric)

    def validate_config(self):
        assert self.b_constraint is None or isinstance(self.b_constraint, Constraint)
        assert self.i_constraint is None or isinstance(self.i_constraint, Constraint)
        assert self.b_regularizer is None or isinstance(self.b_regularizer, Regularizer)
        assert self.i_regularizer is None or isinstance(self.i_regularizer, Regularizer)

    def call(self, inputs, training=None):
        if self.overflow_mode == 'WRAP' and self.trainable:
            if training or training == 'tracing':  # noqa: E712 -- training may be a wrapper object
                xr = _sync_absmax(self.bw_mapper.x_to_bw_absmax(inputs.detach()), inputs)
                if training and _fused_track_kbi(xr, self._b, self._i, self._i_decay_speed, self.symmetric):
                    self._state_written(self._i)
                    return self.stateless_quantizer.round(inputs, self.f, False, self.seed_gen)
                new_i = minimal_i_given_xb(xr, self.b.detach(), self.symmetric)
                if training:
                    new_i = torch.maximum(self._i.value.detach() - self.i_decay_speed, new_i)
                    if self._i.constraint is not None:
                        new_i = self._i.constraint(new_i)
                    self._i.assign(new_i)
                    return self.stateless_quantizer.round(inputs, self.f, False, self.seed_gen)
                new_i = torch.maximum(self.i.detach(), new_i)
                if self._i.constraint is not None:
                    new_i = self._i.constraint(new_i)
                f = self.b.detach() - new_i
                rinputs = self.stateless_quantizer.round(inputs, f, False, self.seed_gen)
                new_k = self.get_any_k(rinputs.detach()) & (self.b.detach() > 0)
                self._k.assign((self._k.value.bool() | new_k).to(torch.uint8))
                self._i.assign(new_i)
                return rinputs
            if self._is_weight and self.stateless_quantizer.round_mode == 'RND':
                return self.stateless_quantizer.round(inputs, self.f, False, self.seed_gen)
        return super().call(inputs, training is True)


class FixedPointQuantizerKIF(FixedPointQuantizerBase):
    """Fixed-point quantizer parameterised by keep_negative, integer bits and fractional bits."""

    def __init__(
        self,
        k0: numbers | bool,
        i0: numbers,
        f0: numbers,
        round_mode: str,
        overflow_mode: str,
        ic: Constraint | None = None,
        fc: Constraint | None = None,
        ir: Regularizer | None = None,
        fr: Regularizer | None = None,
        i_decay_speed: numbers = float('inf'),
        is_weight: bool = False,
        **kwargs,
    ):
        super().__init__(**kwargs)
        if not isinstance(k0, Initializer) and not isinstance(i0, Initializer) and not isinstance(f0, Initializer):
            k0 = int(k0)
            assert k0 == 0 or k0 == 1, f'Invalid k0 value {k0}: must be 0 or 1.'
            assert i0 + f0 >= 0, f'Invalid i0+f0 value {i0 + f0}: must be non-negative.'
        self._k0 = k0 if isinstance(k0, Initializer) else Constant(float(k0))
        self._i0 = i0 if isinstance(i0, Initializer) else Constant(float(i0))
        self._f0 = f0 if isinstance(f0, Initializer) else Constant(float(f0))
        self._i_decay_speed0 = i_decay_speed if isinstance(i_decay_speed, Initializer) else Constant(float(i_decay_speed))
        self._round_mode = round_mode.upper()
        self._overflow_mode = overflow_mode.upper()
        self.i_constraint = ic
        self.f_constraint = fc
        self.i_regularizer = ir
        self.f_regularizer = fr
        self._is_weight = is_weight
        self.validate_config()

    def build(self, input_shape):
        bw_shape = self.bw_mapper.inference_weight_shape(input_shape)
        self._k = self.add_weight(name='k', shape=bw_shape, initializer=self._k0, trainable=False, dtype='uint8')
        i_trainable = self.overflow_mode != 'WRAP'
        self._i = self.add_weight(
            name='i', shape=bw_shape, initializer=self._i0, trainable=i_trainable, constraint=self.i_constraint,
            regularizer=self.i_regularizer,
        )
        self._f = self.add_weight(
            name='f', shape=bw_shape, initializer=self._f0, trainable=True, constraint=self.f_constraint,
            regularizer=self.f_regularizer,
        )
        super().build(input_shape)

    def call(self, inputs, training=None):
        if self.overflow_mode == 'WRAP' and self.trainable:
            f = self.f
            if training or training == 'tracing':  # noqa: E712
                rinputs, absmax = self._round_and_absmax(inputs, f)
                if training:
                    with bookkeeping(absmax):  # nothing downstream in this forward pass reads the updated integer bits
                        am = _sync_absmax(absmax, inputs)
                        if _fused_track_kif(am, self._f, self._i, self._i_decay_speed):
                            self._state_written(self._i)
                        else:
                            _new_i = minimal_i_given_xf(am, f.detach(), self.symmetric)
                            new_i = torch.maximum(self._i.value.detach() - self.i_decay_speed, _new_i)
                            self._i.assign(new_i)
                    return rinputs
                # tracing
                _new_i = minimal_i_given_xf(_sync_absmax(absmax, inputs), f.detach(), self.symmetric)
                if self._i.constraint is not None:
                    _new_i = self._i.constraint(_new_i)
                new_i = torch.maximum(self.i.detach(), _new_i)
                new_k = self.get_any_k(rinputs.detach())
                self._k.assign((self._k.value.bool() | new_k).to(torch.uint8))
                self._i.assign(new_i)
                return rinputs
            if self._is_weight:
                return self.stateless_quantizer.round(inputs, f, False, self.seed_gen)
        return super().call(inputs, training is True)

    _kif_like = True

    def _wrap_training_plan(self, plan):
        f = self.f

        def track(absmax, inputs=None):
            am = _sync_absmax(absmax.view(f.shape), inputs)
            if _fused_track_kif(am, self._f, self._i, self._i_decay_speed):
                self._state_written(self._i)
                return
            _new_i = minimal_i_given_xf(am, f.detach(), self.symmetric)
            self._i.assign(torch.maximum(self._i.value.detach() - self.i_decay_speed, _new_i))

        plan.update(overflow_mode='NONE', training=True, zero=False, i=None, f=f, track=track)
        return plan

    @property
    def k(self):
        return self._k.value.to(torch.float32)

    @property
    def b(self):
        return torch.relu(self.i + self.f)

    @property
    def i(self):
        return self._rounded(self._i)

    @property
    def f(self):
        return self._rounded(self._f)

    @property
    def kif(self):
        return self.k, self.i, self.f

    def get_minimal_i(self, inputs):
        xr = self.bw_mapper.x_to_bw_absmax(inputs)
        return minimal_i_given_xf(xr, self.f.detach(), self.symmetric)

    def validate_config(self):
        assert self.f_constraint is None or isinstance(self.f_constraint, Constraint)
        assert self.i_constraint is None or isinstance(self.i_constraint, Constraint)
        assert self.f_regularizer is None or isinstance(self.f_regularizer, Regularizer)
        assert self.i_regularizer is None or isinstance(self.i_regularizer, Regularizer)
