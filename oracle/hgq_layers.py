"""CPU oracle for the stateful quantizers and quantised layers.  TEST INFRASTRUCTURE, not product code.

Only tests/, __graft_entry__.smoke() and bench.py's cpu_baseline / reference legs may import this.

Plain-PyTorch fp32 CPU restatement of the reference's Python, one class per reference class, each
method citing the lines it follows.  It keeps the reference's formulation on purpose -- bitwidths
broadcast to the activation shape, abs-max as a separate reduction, EBOPs as an fp32
matmul/einsum/conv of bitwidth tensors, torch autograd for everything -- so that it checks the fused
CUDA path against the reference's own op sequence, and so that timing it is timing what the
reference does on a CPU.

PARITY UNPINNED for gradient values and for forward edge cases: see oracle/fixed_point_ops.py.
"""

from __future__ import annotations

from math import prod

import torch
import torch.nn.functional as F

from . import fixed_point_ops as O

EPS = 1e-7  # keras.config.epsilon()


def _leaf(t, requires_grad):
    t = torch.as_tensor(t).detach().clone().float()
    return t.requires_grad_(bool(requires_grad))


def minimal_i_given_xb(x, b, symmetric=False):
    """src/hgq/quantizer/internal/fixed_point_quantizer.py:16-22"""
    if symmetric:
        return torch.ceil(torch.log2((x + EPS) / (1 - 2.0**-b + EPS)))
    i_pos = torch.ceil(torch.log2((x + EPS) / (1 - 2.0**-b + EPS)))
    i_neg = torch.ceil(torch.log2(-x - EPS))
    return torch.where(b > 0, torch.where(x >= 0, i_pos, i_neg), torch.full_like(i_pos, 32.0))


def minimal_i_given_xf(x, f, symmetric=False):
    """src/hgq/quantizer/internal/fixed_point_quantizer.py:25-31"""
    if symmetric:
        return torch.ceil(torch.log2(torch.abs(x) + 2.0**-f))
    i_pos = torch.ceil(torch.log2(x + 2.0**-f))
    i_neg = torch.ceil(torch.log2(-x - EPS))
    return torch.where(x >= 0, i_pos, i_neg)


class OracleFixedQuantizer:
    """FixedPointQuantizerKBI / KIF (fixed_point_quantizer.py:153-459) with state held in leaf tensors."""

    def __init__(self, kind, k, i, bf, round_mode, overflow_mode, homogeneous_axis, i_decay_speed=float('inf'),
                 is_weight=False, trainable=True, i_constraint=None, scaler=None, affine=None, qnoise_factor=None):
        assert kind in ('kbi', 'kif')
        self.kind = kind
        self.round_mode, self.overflow_mode = round_mode.upper(), overflow_mode.upper()
        self.homogeneous_axis = tuple(homogeneous_axis)
        self.is_weight, self.trainable = is_weight, trainable
        self.i_constraint = i_constraint
        self.scaler, self.affine, self.qnoise_factor = scaler, affine, qnoise_factor
        self._k = torch.as_tensor(k).detach().clone().to(torch.uint8)
        i_trainable = trainable and self.overflow_mode != 'WRAP'
        self._i = _leaf(i, i_trainable)
        if kind == 'kbi':
            self._b = _leaf(bf, trainable)
        else:
            self._f = _leaf(bf, trainable)
        self.i_decay_speed = torch.tensor(float(i_decay_speed))
        self.q = O.get_fixed_quantizer(self.round_mode, self.overflow_mode)
        self.symmetric = self.overflow_mode.endswith('SYM')

    # -- properties (:244-265, :431-449)
    @property
    def k(self):
        return self._k.float()

    @property
    def i(self):
        return O.round_conv(self._i)

    @property
    def b(self):
        return O.round_conv(self._b) if self.kind == 'kbi' else torch.relu(self.i + self.f)

    @property
    def f(self):
        return self.b - self.i if self.kind == 'kbi' else O.round_conv(self._f)

    @property
    def kif(self):
        return self.k, self.i, self.f

    @property
    def bits(self):  # :92-97
        return self.b if self.overflow_mode != 'SAT' else self.b + self.k

    def trainable_leaves(self):
        out = {}
        for name in ('_b', '_i', '_f'):
            t = getattr(self, name, None)
            if t is not None and t.requires_grad:
                out[name[1:]] = t
        return out

    # -- bitwidth mapper (base.py:182-189)
    def _absmax(self, x):
        ax = self.homogeneous_axis
        return torch.amax(torch.abs(x), dim=ax, keepdim=True) if ax else torch.abs(x)

    def _anyneg(self, x):
        ax = self.homogeneous_axis
        return torch.amax(x < 0, dim=ax, keepdim=True) if ax else (x < 0)

    def bits_(self, shape):  # quantizer.py:86-88
        return torch.broadcast_to(self.bits, tuple(shape))

    # -- calls
    def _base_call(self, x, training):  # :142-150
        k, i, f = self.kif
        k, i, f = (torch.broadcast_to(t, x.shape) for t in (k, i, f))
        ret = self.q(x, k, i, f, training is True, None)
        if not training:
            ret = torch.where(k + i + f > 0, ret, torch.zeros_like(ret))
        return ret

    def _internal_call(self, x, training):
        wrap = self.overflow_mode == 'WRAP' and self.trainable
        if self.kind == 'kbi':  # :277-307
            if wrap:
                if training or training == 'tracing':
                    new_i = minimal_i_given_xb(self._absmax(x.detach()), self.b.detach(), self.symmetric)
                    if training:
                        new_i = torch.maximum(self._i.detach() - self.i_decay_speed, new_i)
                        if self.i_constraint is not None:
                            new_i = self.i_constraint(new_i)
                        self._i.data.copy_(new_i)
                        return self.q.round(x, torch.broadcast_to(self.f, x.shape), False, None)
                    new_i = torch.maximum(self.i.detach(), new_i)
                    if self.i_constraint is not None:
                        new_i = self.i_constraint(new_i)
                    f = torch.broadcast_to(self.b.detach() - new_i, x.shape)
                    r = self.q.round(x, f, False, None)
                    new_k = self._anyneg(r.detach()) & (self.b.detach() > 0)
                    self._k = (self._k.bool() | new_k).to(torch.uint8)
                    self._i.data.copy_(new_i)
                    return r
                if self.is_weight and self.round_mode == 'RND':
                    return self.q.round(x, torch.broadcast_to(self.f, x.shape), False, None)
            return self._base_call(x, training is True)
        # kif :401-429
        if wrap:
            f = torch.broadcast_to(self.f, x.shape)
            r = self.q.round(x, f, False, None)
            if training or training == 'tracing':
                _new_i = minimal_i_given_xf(self._absmax(r.detach()), self.f.detach(), self.symmetric)
                if training:
                    new_i = torch.maximum(self._i.detach() - self.i_decay_speed, _new_i)
                    self._i.data.copy_(new_i)
                else:
                    if self.i_constraint is not None:
                        _new_i = self.i_constraint(_new_i)
                    new_i = torch.maximum(self.i.detach(), _new_i)
                    self._k = (self._k.bool() | self._anyneg(r.detach())).to(torch.uint8)
                    self._i.data.copy_(new_i)
                return r
            if self.is_weight:
                return r
        return self._base_call(x, training is True)

    def __call__(self, x, training=None):  # Quantizer.call, quantizer.py:49-60
        inputs = x / self.scaler if self.scaler is not None else x
        out = self._internal_call(inputs, training)
        if self.scaler is not None:
            out = out * self.scaler
        if self.qnoise_factor is not None and training:
            out = inputs + self.qnoise_factor * (out - inputs)
        if self.affine is not None:
            out = out * self.affine[0] + self.affine[1]
        return out


class OracleQLayer:
    """The EBOPs / output-quantizer wrapper of QLayerMeta (layers/core/base.py:88-110)."""

    def __init__(self, iq, kq, bq, oq, beta, ebops_factor, enable_ebops, activation):
        self.iq, self.kq, self.bq, self.oq = iq, kq, bq, oq
        self.beta = torch.tensor(float(beta))
        self.ebops_factor = ebops_factor
        self.enable_ebops = enable_ebops
        self.activation = activation
        self.ebops = torch.zeros((), dtype=torch.uint32)
        self.losses: list[torch.Tensor] = []

    def quantizers(self):
        return {n: q for n, q in (('iq', self.iq), ('kq', self.kq), ('bq', self.bq), ('oq', self.oq)) if q is not None}

    def __call__(self, x, training=None):
        self.losses = []
        r = self.call(x, training)
        if (training or training == 'tracing') and self.enable_ebops:
            shape = (1,) + tuple(x.shape[1:])
            ebops = self._compute_ebops(shape) * self.ebops_factor
            self.ebops = ebops.detach().to(torch.uint32)
            self.ebops_f = ebops.detach()
            self.losses.append(ebops * self.beta)
        if self.oq is not None:
            r = self.oq(r, training)
        return r

    def _act(self, x):
        if self.activation is None:
            return x
        if self.activation == 'relu':
            return torch.relu(x)
        raise NotImplementedError(self.activation)


class OracleQDense(OracleQLayer):
    """QDense (layers/core/dense.py:60-80)."""

    def __init__(self, kernel, bias, n_parallel, parallelization_factor, **kw):
        super().__init__(**kw)
        self.kernel = _leaf(kernel, True)
        self.bias = _leaf(bias, True) if bias is not None else None
        self.n_parallel, self.pf = n_parallel, parallelization_factor

    def call(self, x, training):
        if self.iq is not None:
            x = self.iq(x, training)
        y = torch.matmul(x, self.kq(self.kernel, training))
        if self.bias is not None:
            y = y + self.bq(self.bias, training)
        return self._act(y)

    def _compute_ebops(self, shape):
        bw_inp = self.iq.bits_(shape)
        bw_ker = self.kq.bits_(self.kernel.shape)
        ebops = torch.sum(torch.matmul(bw_inp, bw_ker))
        if self.bq is not None:
            bw_bias = self.bq.bits_(self.bias.shape)
            size = float(prod(shape[:-1]) * self.kernel.shape[-1])
            ebops = ebops + torch.mean(bw_bias) * size
        return ebops * self.pf / self.n_parallel


class OracleQEinsumDense(OracleQLayer):
    """QEinsumDense (layers/core/einsum_dense.py:72-93)."""

    def __init__(self, equation, kernel, bias, full_output_shape, n_parallel, parallelization_factor, **kw):
        super().__init__(**kw)
        self.equation = equation
        self.kernel = _leaf(kernel, True)
        self.bias = _leaf(bias, True) if bias is not None else None
        self.full_output_shape = full_output_shape
        self.n_parallel, self.pf = n_parallel, parallelization_factor

    def call(self, x, training):
        qk = self.kq(self.kernel, training)
        if self.iq is not None:
            x = self.iq(x, training)
        y = torch.einsum(self.equation, x, qk)
        if self.bias is not None:
            y = y + self.bq(self.bias, training)
        return self._act(y)

    def _compute_ebops(self, shape):
        bw_inp = self.iq.bits_(shape)
        bw_ker = self.kq.bits_(self.kernel.shape)
        ebops = torch.einsum(self.equation.split('->')[0] + '->', bw_inp, bw_ker)
        if self.bq is not None:
            bw_bias = self.bq.bits_(self.bias.shape)
            size = float(prod(self.full_output_shape[1:]))
            ebops = ebops + torch.mean(bw_bias) * size
        return ebops * self.pf / self.n_parallel


class OracleQConv2D(OracleQLayer):
    """QConv2D (layers/conv.py:72-102), channels_last."""

    def __init__(self, kernel, bias, strides, dilation, pads, n_parallel, parallelization_factor, **kw):
        super().__init__(**kw)
        self.kernel = _leaf(kernel, True)
        self.bias = _leaf(bias, True) if bias is not None else None
        self.strides, self.dilation, self.pads = strides, dilation, pads
        self.n_parallel, self.pf = n_parallel, parallelization_factor

    def conv(self, x, w):
        (pt, pb), (pl, pr) = self.pads
        x = x.permute(0, 3, 1, 2)
        if pt or pb or pl or pr:
            x = F.pad(x, (pl, pr, pt, pb))
        return F.conv2d(x, w.permute(3, 2, 0, 1).contiguous(), stride=self.strides, dilation=self.dilation).permute(0, 2, 3, 1)

    def call(self, x, training):
        if self.iq is not None:
            x = self.iq(x, training)
        y = self.conv(x, self.kq(self.kernel, training))
        if self.bias is not None:
            y = y + self.bq(self.bias, training).reshape(1, 1, 1, -1)
        return self._act(y)

    def _compute_ebops(self, shape):
        bw_inp = self.iq.bits_(shape)
        bw_ker = self.kq.bits_(self.kernel.shape)
        ebops = torch.sum(self.conv(bw_inp, bw_ker))
        ebops = ebops * (self.pf / self.n_parallel)
        if self.bq is not None:
            size = float(prod(shape[:-1]) * self.kernel.shape[-1])
            bw_bias = self.bq.bits_(self.bias.shape)
            ebops = ebops + torch.mean(bw_bias) * size
        return ebops


class OracleQConv1D(OracleQConv2D):
    """QConv1D (layers/conv.py:127-174; call and EBOPs of QBaseConv, conv.py:72-102), channels_last: [B, W, C] inputs,
    [KW, C, N] kernel.  `pads` = (left, right); 'causal' is (dilation (KW - 1), 0)."""

    def conv(self, x, w):
        pl, pr = self.pads
        x = x.permute(0, 2, 1)
        if pl or pr:
            x = F.pad(x, (pl, pr))
        return F.conv1d(x, w.permute(2, 1, 0).contiguous(), stride=self.strides, dilation=self.dilation).permute(0, 2, 1)

    def call(self, x, training):
        if self.iq is not None:
            x = self.iq(x, training)
        y = self.conv(x, self.kq(self.kernel, training))
        if self.bias is not None:
            y = y + self.bq(self.bias, training).reshape(1, 1, -1)
        return self._act(y)


# ---- building an oracle twin of a product object (reads variables by their reference names) ----
def _np(v):
    return v.value.detach().cpu()


def mirror_quantizer(q):
    """Oracle twin of a hgq2_b200 ``Quantizer`` (or None)."""
    if q is None:
        return None
    iq = q.quantizer
    if getattr(iq, '__dummy__', False):
        raise NotImplementedError('dummy quantizer')
    cfg = q.config
    kind = cfg.q_type
    bf = _np(iq._b) if kind == 'kbi' else _np(iq._f)
    decay = float(_np(iq._i_decay_speed)) if iq.overflow_mode == 'WRAP' else float('inf')
    return OracleFixedQuantizer(
        kind, _np(iq._k), _np(iq._i), bf, iq.round_mode, iq.overflow_mode, iq.bw_mapper.homogeneous_axis, decay,
        iq._is_weight, iq.trainable, iq.i_constraint, q.scaler, q.affine, q.qnoise_factor,
    )


def mirror_layer(layer):
    """Oracle twin of a built hgq2_b200 QDense / QEinsumDense / QConv2D / QConv1D."""
    name = type(layer).__name__
    common = dict(
        iq=mirror_quantizer(layer.iq) if layer.enable_iq else None, kq=mirror_quantizer(layer.kq),
        bq=mirror_quantizer(layer.bq), oq=mirror_quantizer(layer.oq) if layer.enable_oq else None,
        beta=float(layer.beta) if layer.enable_ebops else 0.0, ebops_factor=layer.ebops_factor,
        enable_ebops=layer.enable_ebops, activation=layer.get_config()['activation'],
    )
    kernel = _np(layer._kernel)
    bias = _np(layer._bias) if layer.bias is not None else None
    if name == 'QDense':
        return OracleQDense(kernel, bias, layer.n_parallel, layer.parallelization_factor, **common)
    if name == 'QEinsumDense':
        return OracleQEinsumDense(layer.equation, kernel, bias, layer.full_output_shape, layer.n_parallel,
                                  layer.parallelization_factor, **common)
    if name == 'QConv2D':
        h, w = layer._built_hw
        return OracleQConv2D(kernel, bias, layer.strides, layer.dilation_rate, layer._pads(h, w), layer.n_parallel,
                             layer.parallelization_factor, **common)
    if name == 'QConv1D':
        _, w = layer._built_hw
        return OracleQConv1D(kernel, bias, layer.strides[1], layer.dilation_rate[1], layer._pads(1, w)[1], layer.n_parallel,
                             layer.parallelization_factor, **common)
    raise NotImplementedError(name)


# ---- config 5: lookup-table activations, softmax, multi-head attention ---------------------------------------
class OracleQUnaryLUT(OracleQLayer):
    """QUnaryFunctionLUT (layers/activation.py:58-67)."""

    def __init__(self, fn, **kw):
        super().__init__(kq=None, bq=None, activation=None, **kw)
        self.fn = fn

    def call(self, x, training):
        if self.iq is not None:
            x = self.iq(x, training)
        return self.fn(x)

    def _compute_ebops(self, shape):
        return torch.sum((2.0 ** self.iq.bits_(shape)) * self.oq.bits_(shape)) * 1e-4


class OracleQSoftmax(OracleQLayer):
    """QSoftmax (layers/softmax.py:114-161), stable form, no mask."""

    def __init__(self, axes, exp_table, inv_table, stable, pf, **kw):
        super().__init__(kq=None, bq=None, activation=None, **kw)
        self.axes, self.exp_table, self.inv_table, self.stable, self.pf = tuple(axes), exp_table, inv_table, stable, pf

    def call(self, x, training):
        if self.iq is not None:
            x = self.iq(x, training)
        if self.stable:
            x = torch.amax(x, dim=self.axes, keepdim=True) - x
        e = self.exp_table(x, training)
        s = torch.sum(e, dim=self.axes, keepdim=True)
        d = self.inv_table(s, training)
        self.sub_losses = self.exp_table.losses + self.inv_table.losses
        return e * d

    def __call__(self, x, training=None):
        r = super().__call__(x, training)
        self.losses = self.losses + self.sub_losses
        return r

    def _compute_ebops(self, shape):
        accum_shape = tuple(1 if i in self.axes else s for i, s in enumerate(shape))
        max_instance = prod(accum_shape)
        factor = (self.pf if self.pf > 0 else max_instance) / max_instance
        inp_bits = self.iq.bits_(shape) if self.iq is not None else 0
        exp_bits = self.exp_table.oq.bits_(shape)
        inv_bits = self.inv_table.oq.bits_(accum_shape)
        if self.stable:
            sub = torch.sum(inp_bits) if self.iq is not None else torch.sum(self.exp_table.iq.bits_(shape))
        else:
            sub = 0
        accum = torch.sum(exp_bits) - torch.sum(torch.amin(exp_bits, dim=self.axes))
        mult = torch.sum(exp_bits * inv_bits)
        ebops = sub + accum + mult
        if not self.stable:
            ebops = ebops + torch.sum((2.0**inp_bits) * exp_bits) * 1e-4
        return ebops * factor

    def total_ebops(self):
        return int(self.ebops.to(torch.int64) + self.exp_table.ebops.to(torch.int64) + self.inv_table.ebops.to(torch.int64))


class OracleQMHA(OracleQLayer):
    """QMultiHeadAttention (layers/attn/mha.py:386-537) for [B, T, D] inputs, no masks, no dropout."""

    def __init__(self, q, k, v, o, softmax, pf, **kw):
        super().__init__(iq=None, kq=None, bq=None, activation=None, **kw)
        self.q, self.k, self.v, self.o, self.softmax, self.pf = q, k, v, o, softmax, pf

    def __call__(self, x, training=None):
        self.losses = []
        query = self.q(x, training)
        key = self.k(x, training)
        value = self.v(x, training)
        scores = torch.einsum('aecd,abcd->acbe', key, query)
        scores = self.softmax(scores, training)
        out = torch.einsum('acbe,aecd->abcd', scores, value)
        out = self.o(out, training)
        if self.oq is not None:
            out = self.oq(out, training)
        for sub in (self.q, self.k, self.v, self.softmax, self.o):
            self.losses += sub.losses
        if training and self.enable_ebops:
            T, S = x.shape[1], x.shape[1]
            N = self.q.full_output_shape[2]
            bw_q = self.q.oq.bits_((1,) + tuple(self.q.full_output_shape[1:]))
            bw_k = self.k.oq.bits_((1,) + tuple(self.k.full_output_shape[1:]))
            bw_v = self.v.oq.bits_((1,) + tuple(self.v.full_output_shape[1:]))
            bw_a = self.softmax.oq.bits_((1, N, T, S))
            ebops = torch.einsum('aecd,abcd->', bw_q, bw_k) + torch.einsum('acbe,aecd->', bw_a, bw_v)
            if self.pf > 0:
                ebops = ebops * self.pf
            ebops = ebops * self.ebops_factor
            self.ebops = ebops.detach().to(torch.uint32)
            self.losses.append(ebops * self.beta)
        return out

    def total_ebops(self):
        return int(sum(int(p.ebops.to(torch.int64)) for p in (self.q, self.k, self.v, self.o)) + int(self.ebops.to(torch.int64))
                   + self.softmax.total_ebops())

    def qlayers(self):
        return [self.q, self.k, self.v, self.o, self.softmax, self.softmax.exp_table, self.softmax.inv_table]


def _common_kw(layer):
    return dict(
        iq=mirror_quantizer(layer.iq) if layer.enable_iq else None, oq=mirror_quantizer(layer.oq) if layer.enable_oq else None,
        beta=float(layer.beta) if layer.enable_ebops else 0.0, ebops_factor=layer.ebops_factor, enable_ebops=layer.enable_ebops,
    )


def mirror_lut(layer):
    return OracleQUnaryLUT(layer.activation, **_common_kw(layer))


def mirror_softmax(layer):
    return OracleQSoftmax(layer.axes, mirror_lut(layer.exp_table), mirror_lut(layer.inv_table), layer.stable,
                          layer.parallelization_factor, **_common_kw(layer))


def mirror_mha(layer):
    kw = dict(oq=mirror_quantizer(layer.oq) if layer.enable_oq else None, beta=float(layer.beta) if layer.enable_ebops else 0.0,
              ebops_factor=layer.ebops_factor, enable_ebops=layer.enable_ebops)
    q, k, v = mirror_layer(layer._query_dense), mirror_layer(layer._key_dense), mirror_layer(layer._value_dense)
    # fuse='qkv' / 'kv' share ONE input quantizer object between the projections (mha.py:201-206): its state then
    # advances once per projection call, so the twin must share it too
    if layer._query_dense.enable_iq and layer._query_dense._iq is layer._value_dense._iq:
        q.iq = v.iq
    if layer._key_dense.enable_iq and layer._key_dense._iq is layer._value_dense._iq:
        k.iq = v.iq
    return OracleQMHA(q, k, v, mirror_layer(layer._output_dense), mirror_softmax(layer._softmax), layer.parallelization_factor,
                      **kw)


# ---- accumulation, merge and pooling layers (layers/ops/accum.py, layers/ops/merge.py, layers/pooling.py) --------------
class OracleQSum(OracleQLayer):
    """QSum / QMeanPow2 (layers/ops/accum.py:10-81): sum(iq(x), axes) * scale; EBOPs 0.65 (sum bits - sum min bits)."""

    def __init__(self, axes, scale, keepdims, **kw):
        super().__init__(kq=None, bq=None, activation=None, **kw)
        self.axes, self.scale, self.keepdims = tuple(axes), scale, keepdims

    def call(self, x, training):
        if self.iq is not None:
            x = self.iq(x, training)
        return torch.sum(x, dim=self.axes, keepdim=self.keepdims) * self.scale

    def _compute_ebops(self, shape):
        bits = self.iq.bits_(shape)
        return (torch.sum(bits) - torch.sum(torch.amin(bits, dim=self.axes))) * 0.65


class OracleQPool(OracleQLayer):
    """QBasePooling (layers/pooling.py:23-47): pool(iq(x)); EBOPs sum(bits) * parallelization_factor / n_parallel."""

    def __init__(self, fn, n_parallel, parallelization_factor, **kw):
        super().__init__(kq=None, bq=None, activation=None, **kw)
        self.fn, self.n_parallel, self.pf = fn, n_parallel, parallelization_factor

    def call(self, x, training):
        if self.iq is not None:
            x = self.iq(x, training)
        return self.fn(x)

    def _compute_ebops(self, shape):
        return torch.sum(self.iq.bits_(shape)) * self.pf / self.n_parallel


class OracleQMerge(OracleQLayer):
    """QMerge and its subclasses (layers/ops/merge.py): one quantizer per input, then an element-wise merge."""

    def __init__(self, kind, iqs, scale=1.0, **kw):
        super().__init__(iq=None, kq=None, bq=None, activation=None, **kw)
        self.kind, self.iqs, self.scale = kind, iqs, scale

    def quantizers(self):
        d = {f'iq{n}': q for n, q in enumerate(self.iqs or [])}
        if self.oq is not None:
            d['oq'] = self.oq
        return d

    def __call__(self, xs, training=None):
        self.losses = []
        if self.iqs is not None:
            xs = [q(x, training) for q, x in zip(self.iqs, xs)]
        out = xs[0]
        for t in xs[1:]:
            out = {'add': torch.add, 'sub': torch.sub, 'mul': torch.mul, 'max': torch.maximum, 'min': torch.minimum}[self.kind](out, t)
        out = out * self.scale if self.scale != 1.0 else out
        if (training or training == 'tracing') and self.enable_ebops:
            bitss = [q.bits_((1,) + tuple(x.shape[1:])) for q, x in zip(self.iqs, xs)]
            if self.kind == 'sub':
                e = torch.sum(torch.maximum(bitss[0], bitss[1]))
            elif self.kind == 'mul':
                p = bitss[0]
                for b in bitss[1:]:
                    p = p * b
                e = torch.sum(p)
            else:
                least = bitss[0]
                for b in bitss[1:]:
                    least = torch.minimum(least, b)
                e = torch.sum(sum(bitss)) - torch.sum(least)
                e = e * (0.65 if self.kind == 'add' else 1.0)
            e = e * self.ebops_factor
            self.ebops = e.detach().to(torch.uint32)
            self.ebops_f = e.detach()
            self.losses.append(e * self.beta)
        if self.oq is not None:
            out = self.oq(out, training)
        return out


def mirror_op_layer(layer):
    """Oracle twin of a built hgq2_b200 accumulation / pooling / merge layer."""
    import torch.nn.functional as F

    name = type(layer).__name__
    common = dict(
        oq=mirror_quantizer(layer.oq) if layer.enable_oq else None, beta=float(layer.beta) if layer.enable_ebops else 0.0,
        ebops_factor=layer.ebops_factor, enable_ebops=layer.enable_ebops,
    )
    if name in ('QSum', 'QMeanPow2'):
        return OracleQSum(layer.axes, layer.scale, layer.keepdims, iq=mirror_quantizer(layer.iq) if layer.enable_iq else None, **common)
    merges = {'QAdd': 'add', 'QAveragePow2': 'add', 'QSubtract': 'sub', 'QMultiply': 'mul', 'QMaximum': 'max', 'QMinimum': 'min'}
    if name in merges:
        iqs = [mirror_quantizer(q) for q in layer.iq] if layer.enable_iq else None
        return OracleQMerge(merges[name], iqs, scale=getattr(layer, '_scale', 1.0), **common)
    pools = {
        'QMaxPooling2D': lambda l: (lambda t: F.max_pool2d(t.permute(0, 3, 1, 2), l.pool_size, l.strides).permute(0, 2, 3, 1)),
        'QAveragePooling2D': lambda l: (lambda t: F.avg_pool2d(t.permute(0, 3, 1, 2), l.pool_size, l.strides).permute(0, 2, 3, 1)),
        'QMaxPooling1D': lambda l: (lambda t: F.max_pool1d(t.permute(0, 2, 1), l.pool_size[1], l.strides[1]).permute(0, 2, 1)),
        'QAveragePooling1D': lambda l: (lambda t: F.avg_pool1d(t.permute(0, 2, 1), l.pool_size[1], l.strides[1]).permute(0, 2, 1)),
        'QGlobalAveragePooling1D': lambda l: (lambda t: t.mean(dim=1, keepdim=l.keepdims)),
        'QGlobalAveragePooling2D': lambda l: (lambda t: t.mean(dim=(1, 2), keepdim=l.keepdims)),
        'QGlobalMaxPooling1D': lambda l: (lambda t: t.amax(dim=1, keepdim=l.keepdims)),
        'QGlobalMaxPooling2D': lambda l: (lambda t: t.amax(dim=(1, 2), keepdim=l.keepdims)),
    }
    if name in pools:
        return OracleQPool(pools[name](layer), layer.n_parallel, layer.parallelization_factor,
                           iq=mirror_quantizer(layer.iq) if layer.enable_iq else None, **common)
    raise NotImplementedError(name)


# ---- batch-normalisation layers -----------------------------------------------------------------------------------------
def _moments(x, axes):
    """keras.ops.moments on the torch backend: Var = E[x^2] - E[x]^2, statistics squeezed."""
    axes = tuple(axes)
    mean = torch.mean(x, dim=axes, keepdim=True)
    var = torch.mean(torch.square(x), dim=axes, keepdim=True) - torch.square(mean)
    return mean.squeeze(axes), var.squeeze(axes)


class OracleQBatchNormDense(OracleQDense):
    """QBatchNormDense (layers/core/dense.py:105-254)."""

    def __init__(self, bn_gamma, moving_mean, moving_variance, momentum, epsilon, trainable=True, **kw):
        super().__init__(**kw)
        self.bn_gamma = _leaf(bn_gamma, True) if bn_gamma is not None else None
        self.moving_mean, self.moving_variance = moving_mean.detach().clone(), moving_variance.detach().clone()
        self.momentum, self.epsilon, self.trainable = momentum, epsilon, trainable

    def call(self, x, training):
        if self.iq is not None:
            x = self.iq(x, training)
        if training and self.trainable:  # :206-214
            mean, var = _moments(x, range(x.dim() - 1))
            self.moving_mean = self.moving_mean * self.momentum + mean.detach() * (1.0 - self.momentum)
            self.moving_variance = self.moving_variance * self.momentum + var.detach() * (1.0 - self.momentum)
        else:
            mean, var = self.moving_mean, self.moving_variance
        gamma = self.bn_gamma if self.bn_gamma is not None else 1
        scaler = gamma / torch.sqrt(var + self.epsilon)  # :186-198
        qk = self.kq(scaler[:, None] * self.kernel, training)
        qb = self.bq(self.bias + (-torch.matmul(mean, self.kernel)), training)
        return self._act(torch.matmul(x, qk) + qb)


class OracleQEinsumDenseBatchnorm(OracleQEinsumDense):
    """QEinsumDenseBatchnorm (layers/einsum_dense_batchnorm.py:96-228)."""

    def __init__(self, fused_kernel_equation, reduction_axes, cast_shape, bn_gamma, moving_mean, moving_variance, momentum,
                 trainable=True, **kw):
        super().__init__(**kw)
        self.fused_kernel_equation, self.reduction_axes, self.cast_shape = fused_kernel_equation, reduction_axes, cast_shape
        self.bn_gamma = _leaf(bn_gamma, True) if bn_gamma is not None else None
        self.moving_mean, self.moving_variance = moving_mean.detach().clone(), moving_variance.detach().clone()
        self.momentum, self.trainable = momentum, trainable

    def call(self, x, training):
        if self.iq is not None:
            x = self.iq(x, training)
        if training and self.trainable:  # :203-219
            y0 = torch.einsum(self.equation, x, self.kernel)
            mean, var = _moments(y0, self.reduction_axes)
            self.moving_mean = self.moving_mean * self.momentum + mean.detach() * (1.0 - self.momentum)
            self.moving_variance = self.moving_variance * self.momentum + var.detach() * (1.0 - self.momentum)
        else:
            mean, var = self.moving_mean, self.moving_variance
        gamma = self.bn_gamma if self.bn_gamma is not None else 1
        scaler = gamma / torch.sqrt(var + 1e-7)  # the backend fuzz factor, :172
        qk = self.kq(torch.einsum(self.fused_kernel_equation, self.kernel, scaler), training)
        qb = self.bq(self.bias + (-mean * scaler).reshape(self.cast_shape), training)
        return self._act(torch.einsum(self.equation, x, qk) + qb)


class OracleQBatchNorm(OracleQLayer):
    """QBatchNormalization (layers/batch_normalization.py:123-207)."""

    def __init__(self, axis, bn_gamma, bn_beta, moving_mean, moving_variance, momentum, epsilon, **kw):
        super().__init__(activation=None, **kw)
        self.axis = axis
        self.bn_gamma = _leaf(bn_gamma, True) if bn_gamma is not None else None
        self.bn_beta = _leaf(bn_beta, True) if bn_beta is not None else None
        self.moving_mean, self.moving_variance = moving_mean.detach().clone(), moving_variance.detach().clone()
        self.momentum, self.epsilon = momentum, epsilon

    def call(self, x, training):
        if self.iq is not None:
            x = self.iq(x, training)
        if training:
            mean, var = _moments(x, [a for a in range(x.dim()) if a != self.axis])
            self.moving_mean = self.moving_mean * self.momentum + mean.detach() * (1.0 - self.momentum)
            self.moving_variance = self.moving_variance * self.momentum + var.detach() * (1.0 - self.momentum)
        else:
            mean, var = self.moving_mean, self.moving_variance
        gamma = self.bn_gamma if self.bn_gamma is not None else 1
        beta = self.bn_beta if self.bn_beta is not None else 1
        scale = gamma / torch.sqrt(var + self.epsilon)
        offset = beta - mean * scale
        shape = [1] * x.dim()
        shape[self.axis] = x.shape[self.axis]
        return x * self.kq(scale, training).reshape(shape) + self.bq(offset, training).reshape(shape)

    def _compute_ebops(self, shape):
        bshape = [1] * len(shape)
        bshape[self.axis] = shape[self.axis]
        n = (shape[self.axis],)
        bw_inp = self.iq.bits_(shape)
        return torch.sum(bw_inp * self.kq.bits_(n).reshape(bshape)) + torch.mean(self.bq.bits_(n).reshape(bshape)) * float(prod(shape))


def mirror_bn_layer(layer):
    """Oracle twin of a built hgq2_b200 QBatchNormDense / QEinsumDenseBatchnorm / QBatchNormalization."""
    name = type(layer).__name__
    common = dict(
        iq=mirror_quantizer(layer.iq) if layer.enable_iq else None, kq=mirror_quantizer(layer.kq), bq=mirror_quantizer(layer.bq),
        oq=mirror_quantizer(layer.oq) if layer.enable_oq else None, beta=float(layer.beta) if layer.enable_ebops else 0.0,
        ebops_factor=layer.ebops_factor, enable_ebops=layer.enable_ebops,
    )
    mm, mv = _np(layer.moving_mean), _np(layer.moving_variance)
    if name == 'QBatchNormalization':
        return OracleQBatchNorm(layer.axis, _np(layer._bn_gamma) if layer.scale else None, _np(layer._bn_beta) if layer.center else None,
                                mm, mv, layer.momentum, layer.epsilon, **common)
    common['activation'] = layer.get_config()['activation']
    gamma = _np(layer._bn_gamma) if layer.scale else None
    if name == 'QBatchNormDense':
        return OracleQBatchNormDense(gamma, mm, mv, layer.momentum, layer.epsilon, kernel=_np(layer._kernel), bias=_np(layer._bias),
                                     n_parallel=layer.n_parallel, parallelization_factor=layer.parallelization_factor, **common)
    if name == 'QEinsumDenseBatchnorm':
        return OracleQEinsumDenseBatchnorm(layer.fused_kernel_equation, layer._reduction_axes, layer._norm_offset_cast_shape, gamma,
                                           mm, mv, layer.momentum, equation=layer.equation, kernel=_np(layer._kernel),
                                           bias=_np(layer._bias), full_output_shape=layer.full_output_shape,
                                           n_parallel=layer.n_parallel, parallelization_factor=layer.parallelization_factor, **common)
    raise NotImplementedError(name)
