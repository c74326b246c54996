"""QSoftmax: bit-accurate softmax through two quantised lookup "tables" (mirror of src/hgq/layers/softmax.py).

stable form:  d = max(x) - x;  e = exp_table(d) = oq(exp(-scaler * iq(d)));  s = sum(e);  y = e * inv_table(s)
with inv_table(s) = oq(1 / (iq(s) + eps)).  The table output quantizers are forced to SAT + RND_CONV with k = 0
(reference :65-75).
"""

from __future__ import annotations

from collections.abc import Sequence
from math import prod

import torch

from .. import routes
from ..backend import bookkeeping, epsilon
from ..config.layer import global_config
from ..quantizer import QuantizerConfig
from . import _functions
from .activation import QUnaryFunctionLUT
from .core.base import QLayerBaseSingleInput


class QSoftmax(QLayerBaseSingleInput):
    def __init__(self, axis: int | Sequence[int] | None = None, iq_conf: None | QuantizerConfig = None, stable=True,
                 enable_iq: None | bool = False, exp_iq_conf: None | QuantizerConfig = None,
                 exp_oq_conf: None | QuantizerConfig = None, inv_iq_conf: None | QuantizerConfig = None,
                 inv_oq_conf: None | QuantizerConfig = None, allow_heterogeneous_table: bool = False,
                 input_scaler: float = 1.0, parallelization_factor: int = -1, enable_ebops: None | bool = None, **kwargs):
        axes = kwargs.pop('axes', None)
        assert axis is None or axes is None, 'Use only one of `axis` or `axes`.'
        self.axes = axes or (tuple(axis) if isinstance(axis, Sequence) else (axis,) if axis is not None else (-1,))
        if enable_ebops is None:
            enable_ebops = global_config['enable_ebops']
        super().__init__(iq_conf=iq_conf, enable_iq=enable_iq, enable_ebops=enable_ebops, **kwargs)
        self.stable = stable
        self.parallelization_factor = parallelization_factor
        self._allow_heterogeneous_table = allow_heterogeneous_table
        self.input_scaler = input_scaler

        def _inv(x):
            return 1.0 / (x + epsilon())

        def _exp(x):
            return torch.exp(-x * self.input_scaler) if self.stable else torch.exp(x * self.input_scaler)

        inv_iq_conf = inv_iq_conf or QuantizerConfig('default', 'datalane')
        exp_iq_conf = exp_iq_conf or QuantizerConfig('default', 'datalane')
        exp_oq_conf = exp_oq_conf or QuantizerConfig('default', 'table')
        inv_oq_conf = inv_oq_conf or QuantizerConfig('default', 'table')
        if not self._allow_heterogeneous_table:
            for conf in (inv_iq_conf, exp_iq_conf):
                conf.config['heterogeneous_axis'] = ()
                conf.config['homogeneous_axis'] = None
        for conf in (inv_oq_conf, exp_oq_conf):
            if 'k0' in conf.config:
                conf.config['k0'] = 0
            conf.config['overflow_mode'] = 'SAT'
            conf.config['round_mode'] = 'RND_CONV'
        self.inv_table = QUnaryFunctionLUT(_inv, inv_iq_conf, inv_oq_conf, enable_iq=True, enable_oq=True,
                                           allow_heterogeneous_table=allow_heterogeneous_table, name=f'{self.name}_inv_table',
                                           enable_ebops=self.enable_ebops, beta0=self._beta0.clone())
        self.exp_table = QUnaryFunctionLUT(_exp, exp_iq_conf, exp_oq_conf, enable_iq=self.stable, enable_oq=True,
                                           allow_heterogeneous_table=allow_heterogeneous_table, allow_heterogeneous_input=True,
                                           name=f'{self.name}_exp_table', enable_ebops=self.enable_ebops and stable,
                                           beta0=self._beta0.clone())
        self.supports_masking = True

    def build(self, input_shape):
        self.exp_table.build(input_shape)
        self.exp_table.built = True
        self.axes = tuple(sorted(i if i >= 0 else i + len(input_shape) for i in self.axes))
        inv_shape = list(input_shape)
        for i in self.axes:
            inv_shape[i] = 1
        self.inv_table.build(tuple(inv_shape))
        self.inv_table.built = True
        super().build(input_shape)

    def _fused_call(self, inputs, training):
        """The whole chain (both tables, their quantizers and the output quantizer) in one kernel per direction, or None
        when this call does not fit it: training forward only, stable form, softmax over the trailing axis, table
        quantizers with one (k, i, f) each, every quantizer in a mode the kernel applies inline."""
        from .. import kernels

        if not (_functions.fused_enabled and training is True and self.stable and not self.enable_iq and self.enable_oq):
            return None
        if not inputs.is_cuda or inputs.dim() < 2 or self.axes != (inputs.dim() - 1,):
            return None
        L = inputs.shape[-1]
        if not kernels.qsoftmax_supported(L):
            return None
        qs = (self.exp_table.iq, self.exp_table.oq, self.inv_table.iq, self.inv_table.oq, self.oq)
        plans = []
        for j, q in enumerate(qs):
            if q.scaler is not None or q.affine is not None or q.qnoise_factor is not None:
                return None
            iq = q.quantizer
            if getattr(iq, '__dummy__', False):
                return None
            plan = iq.fusion_plan(training)
            if plan is None or plan['zero'] or plan['overflow_mode'] not in ('NONE', 'SAT', 'SAT_SYM'):
                return None
            if j < 4 and plan['f'].numel() != 1:
                return None
            plans.append(plan)
        p5 = plans[4]
        full = (1,) + tuple(inputs.shape[1:])
        if len(p5['f'].shape) != len(full):
            return None
        rows_period = 1
        for d in full[1:-1]:
            rows_period *= d
        if inputs.numel() % (rows_period * L) != 0:
            return None
        params = []
        for j, plan in enumerate(plans):
            for key in ('k', 'i', 'f'):
                t = plan[key]
                if t is not None and j == 4:
                    t = t.expand(full).reshape(rows_period * L)
                params.append(t)
        modes = tuple((plan['round_mode'], plan['overflow_mode']) for plan in plans)
        if plans[1]['track'] is not None or plans[3]['track'] is not None:
            return None  # a table output that tracks its integer bits (the layer forces them to SAT, so this is a custom setup)
        y, a3, a5, a1 = _functions.QSoftmaxFusedFn.apply(inputs, modes, float(self.input_scaler), float(epsilon()), rows_period,
                                                         plans[2]['track'] is not None, p5['track'] is not None,
                                                         plans[0]['track'] is not None, *params)
        with bookkeeping(a1, a3, a5):
            if plans[0]['track'] is not None:  # the exp table's input quantizer in WRAP mode (the layer's default)
                plans[0]['track'](a1.view(plans[0]['f'].shape), None)
            if plans[2]['track'] is not None:
                plans[2]['track'](a3.view(plans[2]['f'].shape), None)
            if p5['track'] is not None:
                p5['track'](_functions._amax_to_shape(a5.view(full), tuple(p5['f'].shape)), None)
            # the sub-layers' own bookkeeping that their wrapped call would have done
            inv_shape = tuple(1 if ax in self.axes else d for ax, d in enumerate(full))
            if self.exp_table.enable_ebops:
                self.exp_table._account_ebops(full)
            if self.inv_table.enable_ebops:
                self.inv_table._account_ebops(inv_shape)
        return y

    def call(self, inputs, training=None, mask=None):
        self.__output_quantizer_handled__ = False
        if mask is None:
            y = self._fused_call(inputs, training)
            if y is not None:
                self.__output_quantizer_handled__ = True  # the kernel applied self.oq; the call wrapper must not repeat it
                return y
        if training is True and inputs.is_cuda:
            routes.fallback('softmax chain in torch', f'QSoftmax {self.name}')
        if self.enable_iq:
            inputs = self.iq(inputs, training=training)
        if self.stable:
            if mask is not None:
                mask = mask.to(inputs.dtype)
                inputs = mask * inputs - (1 - mask) * 1e9
            inputs = torch.amax(inputs, dim=self.axes, keepdim=True) - inputs
        exp_inp = self.exp_table(inputs, training=training)
        if mask is not None:
            exp_inp = mask.to(inputs.dtype) * exp_inp
        sums = torch.sum(exp_inp, dim=self.axes, keepdim=True)
        divisor = self.inv_table(sums, training=training)
        return exp_inp * divisor

    def _compute_ebops(self, shape):
        shape = tuple(shape)
        accum_shape = tuple(1 if i in self.axes else s for i, s in enumerate(shape))
        max_instance = prod(accum_shape)
        n_instance = self.parallelization_factor if self.parallelization_factor > 0 else max_instance
        factor = n_instance / max_instance
        inp_bits = self.iq.bits_(shape) if self.enable_iq else 0
        exp_bits = self.exp_table.oq.bits_(shape)
        inv_bits = self.inv_table.oq.bits_(accum_shape)
        if self.stable:
            substract_ebops = torch.sum(inp_bits) if self.enable_iq else torch.sum(self.exp_table.iq.bits_(shape))
        else:
            substract_ebops = 0
        accum_ebops = torch.sum(exp_bits) - torch.sum(torch.amin(exp_bits, dim=self.axes))
        mult_ebops = torch.sum(exp_bits * inv_bits)
        ebops = substract_ebops + accum_ebops + mult_ebops
        if not self.stable:
            ebops = ebops + torch.sum((2.0**inp_bits) * exp_bits) * 1e-4
        return ebops * factor

    def compute_output_shape(self, input_shape):
        return input_shape

    @property
    def ebops(self):
        own = self._ebops.value.detach().to(torch.int64) if self._ebops is not None else 0
        total = own + self.exp_table.ebops.to(torch.int64) + self.inv_table.ebops.to(torch.int64)
        return round(float(total))
