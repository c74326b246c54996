"""QEinsumDense: act(einsum(eq, iq(x), kq(W)) + bq(b)) with EBOPs (mirror of src/hgq/layers/core/einsum_dense.py)."""

from __future__ import annotations

from math import prod

import torch

from ... import routes
from ...backend import activation_name, get_activation, get_initializer, take_prepared
from ...quantizer import Quantizer
from ...quantizer.config import QuantizerConfig
from .._functions import EbopsDenseFn, fused_dense_call
from .base import QLayerBaseSingleInput


def _einsum_free0_size(equation: str, input_shape) -> int:
    """Product of the non-batch input axes that are looped over rather than contracted (reference :10-20)."""
    _inp, _ker_out = equation.split(',', 1)
    _ker, _out = _ker_out.split('->', 1)
    elided_size = len(input_shape) - len(_inp) + 3
    _inp = _inp.replace('...', '?' * elided_size)
    n_parallel = 1
    for ax, dim in zip(_inp[1:], input_shape[1:]):
        if ax not in _ker and (ax in _out or ax == '?'):
            assert dim is not None, f'Cannot determine input loop size for einsum eq: {equation} with input shape {input_shape}'
            n_parallel *= int(dim)
    return n_parallel


def analyze_einsum(equation: str, bias_axes, input_shape, output_shape):
    """Kernel shape, bias shape and full output shape of an ellipsis-free 'ab,bc->ac'-style equation, following the
    conventions of Keras' EinsumDense (output_shape excludes the batch axis; the bias spans the output axes from its
    first axis to the last, with 1 for axes it does not name)."""
    if '...' in equation:
        raise NotImplementedError('einsum equations with an ellipsis are not supported')
    inp, rest = equation.split(',', 1)
    ker, out = rest.split('->', 1)
    output_shape = (output_shape,) if isinstance(output_shape, int) else tuple(output_shape)
    full_out = (input_shape[0],) + output_shape
    assert len(full_out) == len(out), f'output_shape {output_shape} does not match "{out}"'
    in_dims = {c: input_shape[j] for j, c in enumerate(inp)}
    out_dims = {c: full_out[j] for j, c in enumerate(out)}
    kernel_shape = []
    for c in ker:
        if c in in_dims:
            kernel_shape.append(int(in_dims[c]))
        elif c in out_dims:
            kernel_shape.append(int(out_dims[c]))
        else:
            raise ValueError(f'kernel axis {c} of "{equation}" is in neither input nor output')
    bias_shape = None
    if bias_axes is not None:
        for c in bias_axes:
            if c not in out:
                raise ValueError(f'bias axis {c} is not in the output spec "{out}"')
        first = min(out.find(c) for c in bias_axes)
        bias_shape = tuple(int(out_dims[c]) if c in bias_axes else 1 for c in out[first:])
    return tuple(kernel_shape), bias_shape, full_out


class QEinsumDense(QLayerBaseSingleInput):
    def __init__(self, equation, output_shape, activation=None, bias_axes=None, kernel_initializer='glorot_uniform',
                 bias_initializer='zeros', kernel_regularizer=None, bias_regularizer=None, kernel_constraint=None,
                 bias_constraint=None, kq_conf: None | QuantizerConfig = None, iq_conf: None | QuantizerConfig = None,
                 bq_conf: None | QuantizerConfig = None, parallelization_factor: int = -1, **kwargs):
        super().__init__(iq_conf=iq_conf, **kwargs)
        self.equation = equation.replace(' ', '')
        self.partial_output_shape = (output_shape,) if isinstance(output_shape, int) else tuple(output_shape)
        self.bias_axes = bias_axes
        self._activation_spec = activation
        self.activation = get_activation(activation)
        self.kernel_initializer = get_initializer(kernel_initializer)
        self.bias_initializer = get_initializer(bias_initializer)
        self.kernel_regularizer, self.bias_regularizer = kernel_regularizer, bias_regularizer
        self.kernel_constraint, self.bias_constraint = kernel_constraint, bias_constraint
        kq_conf = kq_conf or QuantizerConfig('default', 'weight')
        self._kq = Quantizer(kq_conf, name=f'{self.name}_kq')
        bq_conf = bq_conf or QuantizerConfig('default', 'bias')
        self._bq = None if bias_axes is None else Quantizer(bq_conf, name=f'{self.name}_bq')
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
        # kernel and bias before the base classes' beta / ebops: the reference's variable order
        kshape, bshape, full_out = analyze_einsum(self.equation, self.bias_axes, tuple(input_shape), self.partial_output_shape)
        self.full_output_shape = full_out
        self._kernel = self.add_weight(name='kernel', shape=kshape, initializer=self.kernel_initializer,
                                       regularizer=self.kernel_regularizer, constraint=self.kernel_constraint)
        if bshape is not None:
            self._bias = self.add_weight(name='bias', shape=bshape, initializer=self.bias_initializer,
                                         regularizer=self.bias_regularizer, constraint=self.bias_constraint)
            self.bias = self._bias.value
        super().build(input_shape)
        self.n_parallel = _einsum_free0_size(self.equation, input_shape)
        if self.parallelization_factor < 0:
            self.parallelization_factor = self.n_parallel
        self.kq.build(tuple(self._kernel.shape))
        self.kq.built = True
        if self.bias is not None:
            self.bq.build(tuple(self._bias.shape))
            self.bq.built = True
        self.ebops_equation = self.equation.split('->')[0] + '->'
        self._matmul_form = self._analyze_matmul_form()

    def _analyze_matmul_form(self):
        """(number of trailing contracted input axes, K, N) if the equation is '<free><con>,<con><kfree>-><free><kfree>'
        -- a plain [M, K] x [K, N] product after reshaping -- and the bias is a function of the kernel's free axes only."""
        inp, rest = self.equation.split(',', 1)
        ker, out = rest.split('->', 1)
        con = [c for c in ker if c in inp]
        n_con = len(con)
        if n_con == 0 or len(set(inp)) != len(inp) or len(set(ker)) != len(ker):
            return None
        kfree = ker[n_con:]
        if inp[-n_con:] != ''.join(con) or ker[:n_con] != ''.join(con) or any(c in inp for c in kfree):
            return None
        if out != inp[:-n_con] + kfree:
            return None
        kshape = tuple(self._kernel.shape)
        K = 1
        for d in kshape[:n_con]:
            K *= d
        N = 1
        for d in kshape[n_con:]:
            N *= d
        if self.bias is not None:
            spec = out[len(out) - len(self._bias.shape):]
            if any(c not in kfree for c, d in zip(spec, self._bias.shape) if d != 1) or len(spec) > len(kfree):
                return None
        return n_con, K, N, kshape[n_con:]

    def compute_output_shape(self, input_shape):
        return (input_shape[0],) + tuple(self.full_output_shape[1:])

    def prepare_params(self):
        """The parameter-only part of a call: (quantised kernel, quantised bias)."""
        return self.kq(self._kernel.value), (self.bq(self._bias.value) if self.bias is not None else None)

    def call(self, inputs, training=None):
        qkernel, qbias = take_prepared(self) or self.prepare_params()
        return self._contract(inputs, qkernel, qbias, training, apply_iq=True)

    def _contract(self, inputs, qkernel, qbias, training, apply_iq: bool):
        """act(einsum(eq, iq(x), qkernel) + qbias): the fused tensor-core kernel when the equation is a plain matrix
        product, the library einsum otherwise.  ``apply_iq=False``: ``inputs`` are already quantised."""
        if self._matmul_form is not None:
            n_con, K, N, kfree_shape = self._matmul_form
            qb = None
            if qbias is not None:
                qb = qbias.reshape((1,) * (len(kfree_shape) - qbias.dim()) + tuple(qbias.shape)).expand(kfree_shape).reshape(N)
            y = fused_dense_call(self, inputs, n_con, qkernel.reshape(K, N), qb, training, apply_iq=apply_iq)
            if y is not None:
                return y.reshape((inputs.shape[0],) + tuple(self.full_output_shape[1:]))
        routes.fallback('torch.einsum', f'QEinsumDense {self.name} "{self.equation}"')
        if self.enable_iq and apply_iq:
            inputs = self.iq(inputs, training=training)
        x = torch.einsum(self.equation, inputs, qkernel)
        if qbias is not None:
            x = x + qbias
        if self.activation is not None:
            x = self.activation(x)
        return x

    def _compute_ebops(self, shape):
        # einsum('inp,ker->') sums in[...] * ker[...] over every index; with the shared indices moved to the back of the
        # input and the front of the kernel it is the same [P, K] x [K, N] bit product a dense layer has.
        inp, ker = self.ebops_equation[:-2].split(',')
        bw_inp = self.iq.bits_(tuple(shape))
        bw_ker = self.kq.bits_(tuple(self._kernel.shape))
        shared = [c for c in ker if c in inp]
        in_perm = [inp.index(c) for c in inp if c not in shared] + [inp.index(c) for c in shared]
        ker_perm = [ker.index(c) for c in shared] + [ker.index(c) for c in ker if c not in shared]
        K = prod(int(bw_ker.shape[ker.index(c)]) for c in shared)
        a = bw_inp.permute(in_perm).reshape(-1, K)
        b = bw_ker.permute(ker_perm).reshape(K, -1)
        bw_bias = self.bq.bits_(tuple(self._bias.shape)).reshape(-1) if self.bq is not None else None
        size = float(prod(int(d) for d in self.full_output_shape[1:]))
        return EbopsDenseFn.apply(a, b, bw_bias, size, self.parallelization_factor / self.n_parallel)

    def get_config(self):
        config = super().get_config()
        config.update({
            'equation': self.equation, 'output_shape': self.partial_output_shape, 'bias_axes': self.bias_axes,
            'activation': activation_name(self._activation_spec), 'kq_conf': self.kq.config,
            'bq_conf': self.bq.config if self.bq is not None else None,
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
