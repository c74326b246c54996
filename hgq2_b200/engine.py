"""Static execution plan of a QAT step: forward and backward of a ``Sequential`` of quantised layers as a fixed list of
kernel launches, with no autograd graph and no per-tensor bitwidth arithmetic.

What the layer classes do call by call through torch (``round_conv`` of every bitwidth variable, ``f = b - i``,
``bits = relu(i + f)``, one quantizer call per kernel and per bias, one tracking update per WRAP quantizer, the autograd
backward of all of that) is the bulk of a step's launches for the models this package targets -- several hundred
element-wise launches on tensors of a few hundred elements.  The engine replaces it by five batched launches over
descriptor tables (``csrc/params.cu``), and drives the layer kernels itself:

    tables_forward -> weights_forward -> layer forward kernels -> loss
        (second stream, after the forward:  one MAX all-reduce of all abs-max statistics -> tables_track_bits -> EBOPs)
    -> layer backward kernels -> weights_backward -> tables_backward

Every quantizer of the model owns a *slot*: derived tables I = round(i), F = round(f) (or round(b) - round(i)),
BITS, and the gradients dI / dF / dBITS w.r.t. them, all views into flat buffers.  Layer kernels read the tables in place
and write their bitwidth gradients straight into the slot; EBOPs kernels read BITS and write dBITS; the last kernel turns
(dI, dF, dBITS) into the gradients of the raw variables inside the flat gradient bucket that the optimizer and the
gradient all-reduce work on.  Quantizer state (``i`` of WRAP quantizers, the layers' ``ebops`` variables) is updated in
the layers' own variables, so the model object stays what the reference's would be after the same step.

The engine covers the layer types and quantizer configurations of the benchmark workloads (see ``_make_node``); a model
it does not cover raises ``Unsupported`` at construction and the trainer keeps the autograd path.  Results are those of
the autograd path: the same kernels run on the same operands.
"""

from __future__ import annotations

import ctypes
import os
import math

import numpy as np
import torch

from . import _lib, kernels, routes
from .backend import Flatten, Lambda, MaxPooling2D, Sequential
from .constraints import MinMax
from .layers._functions import conv_padding_channels
from .layers.attn.mha import QMultiHeadAttention
from .layers.conv import QConv2D
from .layers.core.dense import QDense
from .layers.core.einsum_dense import QEinsumDense
from .quantizer.internal.base import DefaultBitwidthMapper
from .quantizer.internal.fixed_point_quantizer import FixedPointQuantizerKBI, FixedPointQuantizerKIF

_OM = _lib.OVERFLOW_MODES
_RM = _lib.ROUND_MODES


class Unsupported(Exception):
    """The model (or this call's shapes) is outside what the engine covers; the autograd path handles it."""


def _require(cond, why):
    if not cond:
        raise Unsupported(why)


class Slot:
    """One quantizer's place in the flat table buffers."""

    def __init__(self, wrapper, index, role):
        _require(wrapper.scaler is None and wrapper.affine is None and wrapper.qnoise_factor is None,
                 f'{wrapper.name}: scaler / affine / qnoise_factor')
        q = wrapper.quantizer
        _require(isinstance(q, (FixedPointQuantizerKBI, FixedPointQuantizerKIF)), f'{wrapper.name}: {type(q).__name__}')
        _require(isinstance(q.bw_mapper, DefaultBitwidthMapper), f'{wrapper.name}: custom bitwidth mapper')
        _require(q.trainable, f'{wrapper.name}: frozen quantizer')
        self.wrapper, self.q, self.index, self.role = wrapper, q, index, role
        self.kbi = isinstance(q, FixedPointQuantizerKBI)
        self.shape = tuple(q._k.shape)
        self.n = int(q._k.value.numel())
        self.wrap = q.overflow_mode == 'WRAP'
        self.tracked_act = False     # integer bits follow an abs-max statistic of activations (set by the consumer)
        self.tracked_weight = False  # integer bits follow the weight itself (set by Engine._add_weight)
        self.absmax = None
        self.I = self.F = self.BITS = self.dI = self.dF = self.dBITS = None

    # how a kernel applies this quantizer to activations in training: rounding only for WRAP, the full quantizer otherwise
    @property
    def act_mode(self):
        return 'NONE' if self.wrap else self.q.overflow_mode


class _Node:
    def check(self, batch):
        """Raise ``Unsupported`` if a batch of this size falls outside the kernels this node launches (called before the
        first step touches any state)."""

    def post_allocate(self, eng):
        """Called once the flat buffers exist."""

    def forward(self, x):
        raise NotImplementedError

    def backward(self, g, need_dx=True):
        raise NotImplementedError

    def ebops(self, eng, dense_items):
        """Queue this node's EBOPs kernels (second stream, after the tables hold the tracked bits); dense layers append
        their term to ``dense_items`` instead, and the engine launches those together."""

    def autograd_ebops(self):
        """EBOPs terms computed through torch on the BITS leaves (layers without a direct kernel); returns loss terms."""
        return []


class _Reshape(_Node):
    def __init__(self, fn):
        self.fn = fn

    def forward(self, x):
        self.in_shape = x.shape
        return self.fn(x)

    def backward(self, g, need_dx=True):
        return g.reshape(self.in_shape)


class _Reduce(_Node):
    """sum or mean over axis 1 (what the benchmark models pool with): the gradient is the stride-0 expansion of the
    incoming one, which the dense backward kernel reads in place."""

    def __init__(self, mean):
        self.mean = mean
        self.ready = None  # the result, when the layer before produced it in its own kernel (see _Dense.pool)

    def forward(self, x):
        self.in_shape = x.shape
        if self.ready is not None:
            out, self.ready = self.ready, None
            return out
        return x.mean(dim=1) if self.mean else x.sum(dim=1)

    def backward(self, g, need_dx=True):
        if self.mean:
            g = g * (1.0 / self.in_shape[1])
        return g.unsqueeze(1).expand(self.in_shape)


class _Autograd(_Node):
    """Any other tensor function: differentiated locally by torch."""

    def __init__(self, fn):
        self.fn = fn

    def forward(self, x):
        self.xin = x.detach().requires_grad_()
        with torch.enable_grad():
            self.y = self.fn(self.xin)
        return self.y.detach()

    def backward(self, g, need_dx=True):
        (gx,) = torch.autograd.grad(self.y, self.xin, g)
        self.xin = self.y = None
        return gx


def _lambda_node(layer, in_shape):
    """A Lambda that is a plain sum / mean over axis 1 gets the native node; anything else is differentiated by torch."""
    if len(in_shape) >= 3:
        probe = torch.from_numpy(np.random.default_rng(0).standard_normal((2,) + tuple(in_shape[1:])).astype(np.float32))
        try:
            out = layer.function(probe)
            if out.shape == probe.sum(dim=1).shape:
                if torch.allclose(out, probe.sum(dim=1), rtol=1e-6, atol=1e-6):
                    return _Reduce(False)
                if torch.allclose(out, probe.mean(dim=1), rtol=1e-6, atol=1e-6):
                    return _Reduce(True)
        except Exception:
            pass
    return _Autograd(layer.function)


class _MaxPool(_Node):
    def __init__(self, layer):
        self.pool, self.strides = layer.pool_size, layer.strides
        _require(self.pool[0] * self.pool[1] <= 255, 'pooling window over 255 positions')

    def forward(self, x):
        y, self.arg = kernels.maxpool2d_fwd(x, self.pool, self.strides)
        self.in_shape = tuple(x.shape)
        return y

    def backward(self, g, need_dx=True):
        return kernels.maxpool2d_bwd(g.contiguous(), self.arg, self.in_shape, self.pool, self.strides)


class _Dense(_Node):
    """QDense / QEinsumDense whose equation is a plain matrix product over the trailing input axes."""

    def __init__(self, eng, layer, in_shape):
        self.layer = layer
        _require(layer._activation_spec in (None, 'relu'), f'{layer.name}: activation {layer._activation_spec}')
        _require(layer.enable_iq, f'{layer.name}: no input quantizer')
        if isinstance(layer, QEinsumDense):
            _require(layer._matmul_form is not None, f'{layer.name}: equation {layer.equation} is not a matrix product')
            n_con, K, N, _ = layer._matmul_form
        else:
            n_con, K, N = 1, int(in_shape[-1]), layer.units
        self.n_con, self.K, self.N = n_con, K, N
        self.relu = layer._activation_spec == 'relu'
        self.out_tail = tuple(layer.compute_output_shape((1,) + tuple(in_shape[1:]))[1:])
        self.P = int(np.prod(in_shape[1:len(in_shape) - n_con])) if len(in_shape) - n_con > 1 else 1
        self.iq = eng.slot(layer.iq, 'act')
        _require(not self.iq.kbi and self.iq.wrap, f'{layer.name}: input quantizer must be (k, i, f) in WRAP mode')
        _require(self.iq.n == self.P * K, f'{layer.name}: input bitwidth table {self.iq.shape} is not per activation')
        self.iq.tracked_act = True
        self.kq = eng.slot(layer.kq, 'weight')
        self.wq, self.dwq = eng.add_weight(layer._kernel, self.kq)
        self.bq = self.bias_q = self.dbq = None
        if layer.bias is not None:
            _require(layer._bias.value.numel() == N, f'{layer.name}: bias does not span the output features')
            self.bq = eng.slot(layer.bq, 'weight')
            self.bias_q, self.dbq = eng.add_weight(layer._bias, self.bq)
        self.oq = None
        if layer.enable_oq and not layer.__output_quantizer_handled__:
            self.oq = eng.slot(layer.oq, 'act')
            _require(not self.oq.kbi and self.oq.wrap, f'{layer.name}: output quantizer must be (k, i, f) in WRAP mode')
            _require(self.oq.n == int(np.prod(self.out_tail)), f'{layer.name}: output bitwidth table is not per activation')
            self.oq.tracked_act = True
        self.eb_index = eng.new_ebops_term() if layer.enable_ebops else None
        self.pool = None        # the _Reduce node that follows, when it sums this layer's output over its P rows per sample
        self._pool_ok = {}      # batch -> whether the forward kernel can produce that sum itself

    def check(self, batch):
        K, N, P = self.K, self.N, self.P
        M = batch * P
        if not (kernels.qdense_supported(M, K, N, P) and kernels.qdense_bwd_supported(M, K, N, P)):
            raise Unsupported(f'{self.layer.name}: M={M} K={K} N={N} period={P} outside the fused kernels')
        self._pool_ok[batch] = self.pool is not None and kernels.qdense_pooled_supported(M, K, N, P, P)

    def post_allocate(self, eng):
        self.wq, self.dwq = self.wq.t, self.dwq.t
        if self.bias_q is not None:
            self.bias_q, self.dbq = self.bias_q.t, self.dbq.t

    def forward(self, x):
        K, N, P = self.K, self.N, self.P
        x = x.contiguous()
        rm = self.iq.q.round_mode
        if self._pool_ok.get(x.shape[0], False):
            # the reduction over the P rows of a sample that follows the layer, taken from the finished blocks on chip
            y, _, pooled = kernels.qdense_fwd(x, None, None, self.iq.F.view(P, K), P, rm, 'NONE', True, False, self.wq.view(K, N),
                                              self.bias_q, 'relu' if self.relu else None, True, absmax_out=self.iq.absmax,
                                              absmax_accumulate=True, pool_rows=P, pool_scale=(1.0 / P) if self.pool.mean else 1.0)
            self.pool.ready = pooled
        else:
            y, _ = kernels.qdense_fwd(x, None, None, self.iq.F.view(P, K), P, rm, 'NONE', True, False, self.wq.view(K, N),
                                      self.bias_q, 'relu' if self.relu else None, True, absmax_out=self.iq.absmax,
                                      absmax_accumulate=True)  # the step zeroed the statistics of every quantizer at its start
        self.x, self.y = x, (y if (self.relu or self.oq is not None) else None)
        out_shape = (x.shape[0],) + self.out_tail
        if self.oq is not None:
            y = kernels.quantize_fwd(y, None, None, self.oq.F.view(-1), self.oq.q.round_mode, 'NONE', training=True,
                                     want_absmax=True, absmax_out=self.oq.absmax)[0]
        return y.view(out_shape)

    def backward(self, g, need_dx=True, dx_into=None):
        """``dx_into``: a tensor of the input's shape that the input gradient is added to (see ``accumulates``)."""
        K, N, P = self.K, self.N, self.P
        M = self.x.numel() // K
        if self.oq is not None:
            # a rounding-only quantizer passes the gradient through unchanged: only its df is computed, nothing is copied
            g = g.contiguous().view(M, N)
            kernels.quantize_bwd(g, self.y, None, None, self.oq.F.view(-1), self.oq.q.round_mode, 'NONE', want_dx=False,
                                 want_di=False, out_df=self.oq.dF.view(-1))
        gy_repeat = 1
        if (g.dim() == 3 and g.stride(1) == 0 and g.stride(2) == 1 and g.stride(0) == N and g.size(1) > 1 and M < (1 << 31)):
            gy_repeat, g = g.size(1), g[:, 0, :]  # the gradient of a sum over axis 1: one stored row per sample
        else:
            g = g.contiguous()
        dx, _, _, _ = kernels.qdense_bwd(g, self.y if self.relu else None, self.x, self.iq.F.view(-1), P, self.iq.q.round_mode,
                                         self.wq.view(K, N), want_dx=need_dx, want_db=self.dbq is not None, want_df=True,
                                         gy_repeat=gy_repeat, out_dwq=self.dwq.view(K, N), out_dbq=self.dbq,
                                         out_df=self.iq.dF.view(-1), dx_into=dx_into if need_dx else None)
        x_shape = self.x.shape
        self.x = self.y = None
        return dx.view(x_shape) if dx is not None else None

    def accumulates(self) -> bool:
        """Whether this layer's backward kernel can add its input gradient to an existing tensor."""
        return kernels.qdense_bwd_accumulates(self.K, self.N, self.P, self.relu)

    def ebops(self, eng, dense_items):
        if self.eb_index is None:
            return
        layer = self.layer
        out_size = float(self.P * self.N) if not isinstance(layer, QEinsumDense) else float(np.prod(layer.full_output_shape[1:]))
        scale = layer.parallelization_factor / layer.n_parallel * layer.ebops_factor
        dense_items.append((self.iq.BITS.view(self.P, self.K), self.kq.BITS.view(self.K, self.N),
                            None if self.bq is None else self.bq.BITS.view(-1), out_size, scale, layer._beta.value,
                            (layer._ebops.value, eng.eb_loss[self.eb_index], self.iq.dBITS.view(self.P, self.K),
                             self.kq.dBITS.view(self.K, self.N), None if self.bq is None else self.bq.dBITS.view(-1))))


class _DenseChain(_Node):
    """Consecutive QDense layers with one row per sample, at most 64 inputs and outputs each and no output quantizer, run as
    ONE forward and ONE backward launch for batches of at most one 128-row tile per SM (hgq_dense_chain_fwd / _bwd: the
    activations of a tile stay in shared memory from layer to layer).  On the tensor-core kernels every layer of such a batch
    is a launch that walks its whole chain of dependent latencies for a single tile.  Larger batches keep the per-layer
    tensor-core kernels, which are bound by memory there and faster than fp32 FMAs."""

    def __init__(self, nodes):
        self.nodes = nodes
        self._use = {}
        self._keep = None

    @staticmethod
    def chainable(node) -> bool:
        return (isinstance(node, _Dense) and node.P == 1 and node.n_con == 1 and len(node.out_tail) == 1 and node.oq is None
                and node.pool is None and node.K <= 64 and node.N <= 64)

    def check(self, batch):
        for n in self.nodes:
            n.check(batch)
        sms = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
        self._use[batch] = (os.environ.get('HGQ_DENSE_CHAIN', '1') != '0' and batch <= 128 * sms
                            and kernels.dense_chain_supported([self.nodes[0].K] + [n.N for n in self.nodes]))

    def post_allocate(self, eng):
        for n in self.nodes:
            n.post_allocate(eng)

    def forward(self, x):
        if not self._use.get(x.shape[0], False):
            for n in self.nodes:
                x = n.forward(x)
            return x
        x = x.contiguous()
        M = x.shape[0]
        specs = []
        for n in self.nodes:
            specs.append(dict(K=n.K, N=n.N, relu=n.relu, round_mode=n.iq.q.round_mode, qf=n.iq.F.view(-1), wq=n.wq.view(n.K, n.N),
                              bq=n.bias_q, y=torch.empty((M, n.N), dtype=torch.float32, device=x.device), absmax=n.iq.absmax,
                              dwq=n.dwq.view(n.K, n.N), dbq=n.dbq, df=n.iq.dF.view(-1)))
        layers = kernels.dense_chain_layers(specs)
        kernels.dense_chain_fwd(x, layers, len(specs))
        self._keep = (x, layers, specs)  # the descriptor array holds raw addresses: the tensors stay alive until the backward
        return specs[-1]['y']

    def backward(self, g, need_dx=True):
        if self._keep is None:
            for j in range(len(self.nodes) - 1, -1, -1):
                g = self.nodes[j].backward(g, need_dx=need_dx or j > 0)
            return g
        x, layers, specs = self._keep
        self._keep = None
        g = g.contiguous()
        dx = torch.empty_like(x) if need_dx else None
        kernels.dense_chain_bwd(g, x, dx, layers, len(specs))
        return dx

    def ebops(self, eng, dense_items):
        for n in self.nodes:
            n.ebops(eng, dense_items)


class _Conv(_Node):
    """QConv2D / QConv1D on the implicit-GEMM kernels (unit stride), its input quantizer as a rounding pass of its own.  A
    1-D layer is an image of one row: [B, W, C] activations are [B, 1, W, C] in memory as they stand."""

    def __init__(self, eng, layer, in_shape):
        self.layer = layer
        _require(layer._activation_spec in (None, 'relu'), f'{layer.name}: activation {layer._activation_spec}')
        _require(layer.enable_iq and not (layer.enable_oq and not layer.__output_quantizer_handled__), f'{layer.name}: iq / oq set-up')
        _require(tuple(layer.strides) == (1, 1), f'{layer.name}: strided convolution')
        self.relu = layer._activation_spec == 'relu'
        self.one_d = layer.rank == 1
        if self.one_d:
            (_, W, C), H = in_shape, 1
            (KW, _, N), KH = layer._kernel.shape, 1
            self.out = (1, 1) + tuple(layer.compute_output_shape((1, W, C))[1:])
        else:
            _, H, W, C = in_shape
            KH, KW, _, N = layer._kernel.shape
            self.out = layer.compute_output_shape((1, H, W, C))
        self.geom = (H, W, C, KH, KW, N)
        (pt, _), (pl, _) = layer._pads(H, W)
        self.pad_tl, self.dil = (pt, pl), tuple(layer.dilation_rate)
        self.iq = eng.slot(layer.iq, 'act')
        _require(not self.iq.kbi and self.iq.wrap, f'{layer.name}: input quantizer must be (k, i, f) in WRAP mode')
        _require(self.iq.n == H * W * C, f'{layer.name}: input bitwidth table is not per activation')
        self.iq.tracked_act = True
        self.kq = eng.slot(layer.kq, 'weight')
        self.wq, self.dwq = eng.add_weight(layer._kernel, self.kq)
        self.bq = self.bias_q = self.dbq = None
        if layer.use_bias:
            self.bq = eng.slot(layer.bq, 'weight')
            self.bias_q, self.dbq = eng.add_weight(layer._bias, self.bq)
        self.eb_index = eng.new_ebops_term() if layer.enable_ebops else None

    def check(self, batch):
        H, W, C, KH, KW, N = self.geom
        _, OH, OW, _ = self.out
        cp = conv_padding_channels(batch, H, W, C, KH, KW, N, OH, OW, self.dil)
        _require(cp == 0, f'{self.layer.name}: shape outside the implicit-GEMM kernels' if cp is None else
                 f'{self.layer.name}: needs channel padding')

    def post_allocate(self, eng):
        self.wq, self.dwq = self.wq.t, self.dwq.t
        if self.bias_q is not None:
            self.bias_q, self.dbq = self.bias_q.t, self.dbq.t

    def forward(self, x):
        H, W, C, KH, KW, N = self.geom
        x = x.contiguous().view(-1, H, W, C)
        _, OH, OW, _ = self.out
        xq = kernels.quantize_fwd(x, None, None, self.iq.F.view(-1), self.iq.q.round_mode, 'NONE', training=True,
                                  want_absmax=True, absmax_out=self.iq.absmax)[0]
        y = kernels.qconv2d_fwd(xq, self.wq.view(KH * KW * C, N), self.bias_q, 'relu' if self.relu else None, KH, KW, (OH, OW),
                                (1, 1), self.dil, self.pad_tl)
        self.x, self.xq, self.y = x, xq, (y if self.relu else None)
        return y.view(-1, OW, N) if self.one_d else y

    def backward(self, g, need_dx=True):
        H, W, C, KH, KW, N = self.geom
        _, OH, OW, _ = self.out
        gm, _, _ = kernels.qconv2d_wgrad(self.xq, g.contiguous().view(-1, OH, OW, N), self.y, KH, KW, (1, 1), self.dil, self.pad_tl, self.dbq is not None,
                                         out_dwq=self.dwq.view(KH * KW * C, N), out_dbq=self.dbq)
        # the input gradient is the same convolution kernel over the masked gradient with the flipped, transposed kernel
        wt = self.wq.view(KH, KW, C, N).flip(0, 1).permute(0, 1, 3, 2).reshape(KH * KW * N, C)
        dxq = kernels.qconv2d_fwd(gm, wt, None, None, KH, KW, (H, W), (1, 1), self.dil,
                                  ((KH - 1) * self.dil[0] - self.pad_tl[0], (KW - 1) * self.dil[1] - self.pad_tl[1]))
        # the rounding-only input quantizer passes dxq through unchanged: only its df is computed
        kernels.quantize_bwd(dxq, self.x, None, None, self.iq.F.view(-1), self.iq.q.round_mode, 'NONE', want_dx=False,
                             want_di=False, out_df=self.iq.dF.view(-1))
        self.x = self.xq = self.y = None
        if not need_dx:
            return None
        return dxq.view(-1, W, C) if self.one_d else dxq

    def ebops(self, eng, dense_items):
        if self.eb_index is None:
            return
        H, W, C, KH, KW, N = self.geom
        layer = self.layer
        _, OH, OW, _ = self.out
        size = float(H * W * N)
        scale = layer.parallelization_factor / layer.n_parallel * layer.ebops_factor
        kernels.ebops_conv2d(self.iq.BITS.view(H, W, C), self.kq.BITS.view(KH, KW, C, N),
                             None if self.bq is None else self.bq.BITS.view(-1), (OH, OW), (1, 1), self.dil, self.pad_tl, size,
                             scale, layer.ebops_factor, layer._beta.value,
                             out=(layer._ebops.value, eng.eb_loss[self.eb_index], self.iq.dBITS.view(H, W, C),
                                  self.kq.dBITS.view(KH, KW, C, N), None if self.bq is None else self.bq.dBITS.view(-1)))


class _Softmax(_Node):
    """QSoftmax in its fused form (stable, trailing axis, scalar table quantizers)."""

    def __init__(self, eng, layer, in_shape):
        self.layer = layer
        _require(layer.stable and not layer.enable_iq and layer.enable_oq, f'{layer.name}: softmax set-up')
        self.L = int(in_shape[-1])
        _require(kernels.qsoftmax_supported(self.L) and tuple(layer.axes) == (len(in_shape) - 1,), f'{layer.name}: softmax axis / length')
        self.rows_period = int(np.prod(in_shape[1:-1]))
        wrappers = (layer.exp_table.iq, layer.exp_table.oq, layer.inv_table.iq, layer.inv_table.oq, layer.oq)
        self.slots = [eng.slot(w, 'act') for w in wrappers]
        for j, s in enumerate(self.slots):
            _require(s.q.overflow_mode in ('WRAP', 'SAT', 'SAT_SYM'), f'{layer.name}: overflow mode')
            if j < 4:
                _require(s.n == 1, f'{layer.name}: heterogeneous table quantizer')
            else:
                _require(s.n == self.rows_period * self.L, f'{layer.name}: output bitwidth table is not per activation')
            if s.wrap:
                _require(j in (0, 2, 4) and not s.kbi, f'{layer.name}: WRAP quantizer on a table output')
                s.tracked_act = True
        self.full = (1,) + tuple(in_shape[1:])

    def post_allocate(self, eng):
        # the four scalar slots were created back to back: their dI (and dF) entries sit 4 floats apart in one plane
        s0 = self.slots[0]
        assert [s.index for s in self.slots[:4]] == list(range(s0.index, s0.index + 4))
        stride = (self.slots[1].dI.data_ptr() - s0.dI.data_ptr()) // 4
        self.dI4 = torch.as_strided(s0.dI, (4,), (stride,))
        self.dF4 = torch.as_strided(s0.dF, (4,), (stride,))

    def _quants(self):
        out = []
        for s in self.slots:
            full = not s.wrap
            out.append((s.q._k.value.view(-1) if full else None, s.I.view(-1) if full else None, s.F.view(-1), s.q.round_mode,
                        s.act_mode))
        return out

    def forward(self, x):
        from .backend import epsilon

        s1, _, s3, _, s5 = self.slots
        self.s = x.contiguous()
        y, _, _, _ = kernels.qsoftmax_fwd(self.s, self._quants(), float(self.layer.input_scaler), float(epsilon()), self.rows_period,
                                          s3.tracked_act, s5.tracked_act, s1.tracked_act,
                                          out_amax=(s1.absmax, s3.absmax, s5.absmax))
        return y

    def backward(self, g, need_dx=True):
        from .backend import epsilon

        s5 = self.slots[4]
        want_di5 = s5.act_mode in ('SAT', 'SAT_SYM')
        ds, sc, df5, di5 = kernels.qsoftmax_bwd(g.contiguous(), self.s, self._quants(), float(self.layer.input_scaler), float(epsilon()),
                                                self.rows_period, want_di5)
        sc = sc.view(4, 2)  # (di, df) of the four scalar quantizers; di is zero for a rounding-only one
        self.dI4.copy_(sc[:, 0])
        self.dF4.copy_(sc[:, 1])
        s5.dF.view(-1).copy_(df5)
        if di5 is not None:
            s5.dI.view(-1).copy_(di5)
        self.s = None
        return ds


class _Attention(_Node):
    """QMultiHeadAttention for self-attention on [batch, 64, features]: four projections, the per-head tensor-core products
    and the fused softmax."""

    def __init__(self, eng, layer, in_shape):
        self.layer = layer
        _require(layer._fuse == 'none', f'{layer.name}: fused projections share one quantizer')
        _require(layer._inverse_sqrt_key_dim == 1.0, f'{layer.name}: score scale outside the exp table')
        self.q = _Dense(eng, layer._query_dense, in_shape)
        self.k = _Dense(eng, layer._key_dense, in_shape)
        self.v = _Dense(eng, layer._value_dense, in_shape)
        T, H, D = layer._query_dense.full_output_shape[1:]
        _require(layer._key_dim == layer._value_dim, f'{layer.name}: value_dim differs from key_dim')
        self.geom = (int(T), int(H), int(D))
        self.softmax = _Softmax(eng, layer._softmax, (None, H, T, T))
        self.o = _Dense(eng, layer._output_dense, (None, T, H, D))
        self.oq = None
        if layer.enable_oq:
            self.oq = eng.slot(layer.oq, 'act')
            _require(not self.oq.kbi and self.oq.wrap, f'{layer.name}: output quantizer must be (k, i, f) in WRAP mode')
            self.oq.tracked_act = True
        self.has_ebops = layer.enable_ebops
        self.in_shape = in_shape

    def check(self, batch):
        T, H, D = self.geom
        if not kernels.attn_heads_supported(batch, T, H, D):
            raise Unsupported(f'{self.layer.name}: attention shape B={batch} L={T} H={H} D={D}')
        for d in (self.q, self.k, self.v, self.o):
            d.check(batch)

    def post_allocate(self, eng):
        for d in (self.q, self.k, self.v, self.o, self.softmax):
            d.post_allocate(eng)

    def forward(self, x):
        T, H, D = self.geom
        B = x.shape[0]
        q, k, v = self.q.forward(x), self.k.forward(x), self.v.forward(x)
        s = kernels.attn_heads_matmul(0, q, k, B, T, H, D)
        p = self.softmax.forward(s)
        o = kernels.attn_heads_matmul(1, p, v, B, T, H, D)
        self.saved = (q, k, v, p)
        y = self.o.forward(o)
        if self.oq is not None:
            self.y_pre = y
            y = kernels.quantize_fwd(y, None, None, self.oq.F.view(-1), self.oq.q.round_mode, 'NONE', training=True,
                                     want_absmax=True, absmax_out=self.oq.absmax)[0]
        return y

    def backward(self, g, need_dx=True):
        T, H, D = self.geom
        q, k, v, p = self.saved
        B = q.shape[0]
        if self.oq is not None:
            g = g.contiguous()
            kernels.quantize_bwd(g, self.y_pre, None, None, self.oq.F.view(-1), self.oq.q.round_mode, 'NONE', want_dx=False,
                                 want_di=False, out_df=self.oq.dF.view(-1))
            self.y_pre = None
        go = self.o.backward(g).contiguous()
        dp = kernels.attn_heads_matmul(0, go, v, B, T, H, D)
        dv = kernels.attn_heads_matmul(2, p, go, B, T, H, D)
        ds = self.softmax.backward(dp)
        dq = kernels.attn_heads_matmul(1, ds, k, B, T, H, D)
        dk = kernels.attn_heads_matmul(2, ds, q, B, T, H, D)
        self.saved = None
        # the three projections read the same input: the key and value backward kernels add their input gradients to the
        # query's in place (where the kernel covers the shape; two separate additions otherwise)
        dx = self.q.backward(dq, need_dx)
        dxk = self.k.backward(dk, need_dx, dx_into=dx if (need_dx and self.k.accumulates()) else None)
        dxv = self.v.backward(dv, need_dx, dx_into=dx if (need_dx and self.v.accumulates()) else None)
        if not need_dx:
            return None
        if dxk.data_ptr() != dx.data_ptr():
            dx.add_(dxk)
        if dxv.data_ptr() != dx.data_ptr():
            dx.add_(dxv)
        return dx

    def ebops(self, eng, dense_items):
        for d in (self.q, self.k, self.v, self.o):
            d.ebops(eng, dense_items)

    def autograd_ebops(self):
        """The terms without a kernel of their own (the two activation-activation products, the softmax and its two
        tables), through the layers' own formulas on the BITS leaves."""
        layer = self.layer
        if not self.has_ebops:
            return []
        terms = []
        T = self.geom[0]
        sm = layer._softmax
        full = (1, self.geom[1], T, T)
        inv_shape = (1, self.geom[1], T, 1)
        for sub, shape in ((sm.exp_table, full), (sm.inv_table, inv_shape), (sm, full)):
            if sub.enable_ebops:
                e = sub._compute_ebops(shape) * sub.ebops_factor
                sub._ebops.assign(e.detach().to(torch.uint32))
                terms.append(e * sub.beta)
        e = layer._compute_ebops((1,) + tuple(self.in_shape[1:])) * layer.ebops_factor
        layer._ebops.assign(e.detach().to(torch.uint32))
        terms.append(e * layer.beta)
        return terms


class Engine:
    def __init__(self, model, state):
        _require(isinstance(model, Sequential), 'not a Sequential model')
        _require(state.params.is_cuda, 'parameters are not on a CUDA device')
        _require(hasattr(model, 'input_shape'), 'the model does not state its input shape')
        self.model, self.state = model, state
        self.dev = state.params.device
        self.slots: list[Slot] = []
        self._slot_of: dict[int, Slot] = {}
        self._weights = []  # (variable, slot, offset into the qweights buffer)
        self._wfloats = 0
        self._n_eb = 0
        shape = (None,) + tuple(model.input_shape)
        self.nodes: list[_Node] = []
        for layer in model.layers:
            node, shape = self._make_node(layer, shape)
            self.nodes.append(node)
        _require(self.slots, 'no quantised layer')
        # a dense layer followed by a sum / mean over its row axis hands the reduction to its own forward kernel
        for a, b in zip(self.nodes, self.nodes[1:]):
            if isinstance(a, _Dense) and isinstance(b, _Reduce) and a.oq is None and len(a.out_tail) == 2 and a.out_tail[0] == a.P:
                a.pool = b
        # runs of small dense layers become one node (one forward and one backward launch for the whole run)
        merged: list[_Node] = []
        for node in self.nodes:
            if _DenseChain.chainable(node) and merged and isinstance(merged[-1], (_Dense, _DenseChain)) and \
                    _DenseChain.chainable(merged[-1].nodes[-1] if isinstance(merged[-1], _DenseChain) else merged[-1]):
                last = merged.pop()
                merged.append(_DenseChain((last.nodes if isinstance(last, _DenseChain) else [last]) + [node]))
            else:
                merged.append(node)
        self.nodes = merged
        self._allocate()
        for node in self.nodes:
            node.post_allocate(self)
        self._side = torch.cuda.Stream(device=self.dev)
        self.dp = None
        self._checked_batches = set()

    def check(self, batch: int) -> None:
        """Raises ``Unsupported`` if a batch of this size is outside the kernels of some node."""
        if batch in self._checked_batches:
            return
        for node in self.nodes:
            node.check(batch)
        self._checked_batches.add(batch)

    # -- construction --------------------------------------------------------------------------------------------------
    def _make_node(self, layer, in_shape):
        if isinstance(layer, QMultiHeadAttention):
            _require(len(in_shape) == 3, 'attention input rank')
            return _Attention(self, layer, in_shape), in_shape
        if isinstance(layer, (QDense, QEinsumDense)) and type(layer) in (QDense, QEinsumDense):
            return _Dense(self, layer, in_shape), layer.compute_output_shape(in_shape)
        if isinstance(layer, QConv2D):
            return _Conv(self, layer, in_shape), layer.compute_output_shape(in_shape)
        if isinstance(layer, MaxPooling2D):
            _, h, w, c = in_shape
            oh, ow = (h - layer.pool_size[0]) // layer.strides[0] + 1, (w - layer.pool_size[1]) // layer.strides[1] + 1
            return _MaxPool(layer), (None, oh, ow, c)
        if isinstance(layer, Flatten):
            return _Reshape(lambda x: x.reshape(x.shape[0], -1)), (None, int(np.prod(in_shape[1:])))
        if isinstance(layer, Lambda):
            node = _lambda_node(layer, in_shape)
            out = layer.function(torch.zeros((2,) + tuple(in_shape[1:])))
            return node, (None,) + tuple(out.shape[1:])
        raise Unsupported(f'layer type {type(layer).__name__}')

    def slot(self, wrapper, role) -> Slot:
        q = wrapper.quantizer
        _require(id(q) not in self._slot_of, f'{wrapper.name}: one quantizer used in two places')
        s = Slot(wrapper, len(self.slots), role)
        self.slots.append(s)
        self._slot_of[id(q)] = s
        return s

    def add_weight(self, variable, slot):
        n = int(variable.value.numel())
        _require(slot.n == n, f'{variable.path}: bitwidth table is not per weight')
        if slot.wrap:
            slot.tracked_weight = True
        off = self._wfloats
        self._wfloats += (n + 3) // 4 * 4
        self._weights.append((variable, slot, off, n))
        # views are made in _allocate; hand out lazy handles now
        h_q, h_d = _Lazy(), _Lazy()
        self._weights[-1] += (h_q, h_d)
        return h_q, h_d

    def new_ebops_term(self) -> int:
        self._n_eb += 1
        return self._n_eb - 1

    def _allocate(self):
        dev = self.dev
        total = sum((s.n + 3) // 4 * 4 for s in self.slots)
        self.tables = torch.zeros(3 * total, dtype=torch.float32, device=dev)
        n_abs = sum((s.n + 3) // 4 * 4 for s in self.slots if s.tracked_act)
        # table gradients and abs-max statistics share one buffer: one memset at the start of a step clears both
        self._cleared = torch.zeros(3 * total + max(n_abs, 1), dtype=torch.float32, device=dev)
        self.tgrads = self._cleared[:3 * total]
        self.absmax = self._cleared[3 * total:]
        self.qweights = torch.zeros(max(self._wfloats, 1), dtype=torch.float32, device=dev)
        self.dqweights = torch.zeros(max(self._wfloats, 1), dtype=torch.float32, device=dev)
        self.eb_loss = torch.zeros(max(self._n_eb, 1), dtype=torch.float32, device=dev)
        off = a_off = 0
        for s in self.slots:
            pad = (s.n + 3) // 4 * 4
            for j, name in enumerate(('I', 'F', 'BITS')):
                setattr(s, name, self.tables[off + j * total:off + j * total + s.n].view(s.shape))
                setattr(s, 'd' + name, self.tgrads[off + j * total:off + j * total + s.n].view(s.shape))
            off += pad
            if s.tracked_act:
                s.absmax = self.absmax[a_off:a_off + s.n]
                a_off += pad
        for variable, slot, woff, n, h_q, h_d in self._weights:
            h_q.bind(self.qweights[woff:woff + n])
            h_d.bind(self.dqweights[woff:woff + n])
        # every trainable variable of the model must get its gradient from the engine's two backward kernels
        covered = set()
        slot_descs = (_lib.SlotDesc * len(self.slots))()
        for s, d in zip(self.slots, slot_descs):
            q = s.q
            a_var = q._b if s.kbi else q._f
            d.a_raw, d.i_raw, d.k = a_var.value.data_ptr(), q._i.value.data_ptr(), q._k.value.data_ptr()
            d.I, d.F, d.BITS = s.I.data_ptr(), s.F.data_ptr(), s.BITS.data_ptr()
            d.dI, d.dF, d.dBITS = s.dI.data_ptr(), s.dF.data_ptr(), s.dBITS.data_ptr()
            d.g_a = a_var.value.grad.data_ptr() if a_var.trainable else None
            d.g_i = q._i.value.grad.data_ptr() if q._i.trainable else None
            covered.update(id(v) for v in (a_var, q._i) if v.trainable)
            d.absmax = s.absmax.data_ptr() if s.tracked_act else None
            d.decay = q._i_decay_speed.value.data_ptr() if s.wrap else None
            d.n, d.kind = s.n, (1 if s.kbi else 0)
            d.om, d.rm = _OM[q.overflow_mode], _RM[q.round_mode]
            d.symmetric, d.tracked_weight = int(q.symmetric), int(s.tracked_weight)
            lo, hi = -math.inf, math.inf
            c = q._i.constraint
            if c is not None:
                _require(isinstance(c, MinMax), f'{s.wrapper.name}: constraint {type(c).__name__} on i')
                lo, hi = c.min_value, c.max_value
            d.i_lo, d.i_hi = lo, hi
            if s.tracked_act:
                _require(not s.kbi, f'{s.wrapper.name}: (k, b, i) activation quantizer in WRAP mode')
            if s.role == 'act' and not s.tracked_act:
                _require(not s.wrap, f'{s.wrapper.name}: WRAP activation quantizer without a tracked statistic')
        weight_descs = (_lib.WeightDesc * max(len(self._weights), 1))()
        for (variable, slot, woff, n, h_q, h_d), d in zip(self._weights, weight_descs):
            d.w_raw, d.wq, d.dwq = variable.value.data_ptr(), h_q.t.data_ptr(), h_d.t.data_ptr()
            d.g_w = variable.value.grad.data_ptr() if variable.trainable else None
            covered.add(id(variable))
            d.n, d.slot = n, slot.index
            d.mode = 2 if slot.tracked_weight else 0
        missing = [v.path for v in self.state.variables if id(v) not in covered]
        _require(not missing, f'variables outside the engine: {missing[:4]}')
        self._slot_descs = self._upload(slot_descs)
        self._weight_descs = self._upload(weight_descs)
        self._max_slot = max(s.n for s in self.slots)
        self._max_weight = max((w[3] for w in self._weights), default=0)
        # BITS leaves for the EBOPs terms that go through torch: gradients accumulate into dBITS in place
        for s in self.slots:
            s.BITS.requires_grad_()
            s.BITS.grad = s.dBITS

    def _upload(self, array):
        raw = np.frombuffer(ctypes.string_at(ctypes.addressof(array), ctypes.sizeof(array)), dtype=np.uint8).copy()
        return torch.from_numpy(raw).to(self.dev)

    # -- one step ------------------------------------------------------------------------------------------------------
    def forward_backward(self, x, y, loss_fn):
        """Forward, loss, backward of one batch; gradients of every trainable variable land in the flat bucket.  Returns
        (task loss, total loss) like ``Trainer.forward_backward``."""
        from .train import sparse_categorical_crossentropy

        self.check(int(x.shape[0]))
        main = torch.cuda.current_stream(self.dev)
        side = self._side
        n_slots, n_weights = len(self.slots), len(self._weights)
        with torch.no_grad():
            self._cleared.zero_()
            kernels.tables_forward(self._slot_descs, n_slots, self._max_slot)
            kernels.weights_forward(self._weight_descs, n_weights, self._max_weight, self._slot_descs)
            h = x
            for node in self.nodes:
                h = node.forward(h)
            # second stream: statistics -> integer bits -> BITS -> EBOPs (nothing in the backward pass reads them)
            side.wait_stream(main)
            with torch.cuda.stream(side):
                if self.dp is not None and self.dp.world > 1 and self.absmax.numel() > 1:
                    self.dp.absmax_sync(self.absmax)
                kernels.tables_track_bits(self._slot_descs, n_slots, self._max_slot)
                dense_items = []
                for node in self.nodes:
                    node.ebops(self, dense_items)
                if dense_items:  # every dense layer's term in one launch
                    kernels.ebops_dense_batch(dense_items)
                eb_total = self.eb_loss.sum() if self._n_eb else None
                with torch.enable_grad():
                    self._install_bits(True)
                    try:
                        terms = [t for node in self.nodes for t in node.autograd_ebops()]
                        if terms:
                            extra = terms[0]
                            for t in terms[1:]:
                                extra = extra + t
                            extra.backward()
                            eb_total = extra.detach() if eb_total is None else eb_total + extra.detach()
                    finally:
                        self._install_bits(False)
            # loss and backward on the main stream
            if loss_fn is sparse_categorical_crossentropy and h.dim() == 2 and h.shape[1] <= 64 and y.dtype == torch.int64:
                task, g = kernels.softmax_xent(h, y)
            else:
                logits = h.detach().requires_grad_()
                with torch.enable_grad():
                    task = loss_fn(logits, y)
                    (g,) = torch.autograd.grad(task, logits)
                task = task.detach()
            for j in range(len(self.nodes) - 1, -1, -1):
                g = self.nodes[j].backward(g, need_dx=j > 0)
            main.wait_stream(side)
            kernels.weights_backward(self._weight_descs, n_weights, self._max_weight, self._slot_descs)
            kernels.tables_backward(self._slot_descs, n_slots, self._max_slot)
            total = task if eb_total is None else task + eb_total
            return task, total + self.state.regularization_loss()

    def _install_bits(self, on: bool):
        for s in self.slots:
            if on:
                s.q.__dict__['_engine_bits'] = s.BITS
            else:
                s.q.__dict__.pop('_engine_bits', None)


class _Lazy:
    """A view into a buffer that is allocated after the nodes are built; behaves like the tensor once bound."""

    t = None

    def bind(self, t):
        self.t = t

    def view(self, *shape):
        return self.t.view(*shape)

    def data_ptr(self):
        return self.t.data_ptr()
