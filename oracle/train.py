"""CPU oracle of the QAT step (forward, loss, backward, Adam, constraints).  TEST INFRASTRUCTURE.

Restates what Keras' torch trainer does with an HGQ2 model (external to the HGQ2 tree; HGQ2 contributes the
layers' ``add_loss(ebops * beta)`` terms, layers/core/base.py:104, the MonoL1 regularisers attached at
fixed_point_quantizer.py:225-241,382-397 and the constraints applied after the optimizer update):

    y = model(x, training=True); loss = task(y, labels) + sum(model.losses)   # losses: EBOPs terms + regularisers
    grads = d loss / d trainable;  Keras Adam update;  variable.assign(constraint(variable))
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

from . import hgq_layers as OL


class OracleSequential:
    def __init__(self, layers):
        self.layers = layers

    def __call__(self, x, training=None):
        self.losses = []
        for layer in self.layers:
            if isinstance(layer, OL.OracleQLayer):
                x = layer(x, training)
                self.losses += layer.losses
            else:
                x = layer(x)
        return x

    def qlayers(self):
        return [l for l in self.layers if isinstance(l, OL.OracleQLayer)]


def mirror_model(model):
    """Oracle twin of a built hgq2_b200 Sequential, plus the list of (oracle leaf, product Variable) pairs."""
    out = []
    for layer in model.layers:
        name = type(layer).__name__
        if name in ('QDense', 'QEinsumDense', 'QConv2D', 'QConv1D'):
            out.append(OL.mirror_layer(layer))
        elif name == 'QMultiHeadAttention':
            out.append(OL.mirror_mha(layer))
        elif name == 'Lambda':
            out.append(layer.function)
        elif name == 'Flatten':
            out.append(lambda t: t.reshape(t.shape[0], -1))
        elif name == 'MaxPooling2D':
            ps, st = layer.pool_size, layer.strides
            out.append(lambda t, ps=ps, st=st: F.max_pool2d(t.permute(0, 3, 1, 2), ps, st).permute(0, 2, 3, 1))
        else:
            raise NotImplementedError(name)
    twin = OracleSequential(out)
    pairs = []

    def quantizer_pairs(pl_q, ol_q):
        iq = pl_q.quantizer
        for vname, leaf in ol_q.trainable_leaves().items():
            pairs.append((leaf, getattr(iq, '_' + vname), None, None))

    for pl, ol in zip(model.layers, out):
        if not isinstance(ol, OL.OracleQLayer):
            continue
        if isinstance(ol, OL.OracleQMHA):
            for pd, od in ((pl._query_dense, ol.q), (pl._key_dense, ol.k), (pl._value_dense, ol.v), (pl._output_dense, ol.o)):
                pairs.append((od.kernel, pd._kernel, None, None))
                if od.bias is not None:
                    pairs.append((od.bias, pd._bias, None, None))
                for qname, oq in od.quantizers().items():
                    if qname == 'iq' and any(oq is q2 for q2 in ()):
                        continue
                    quantizer_pairs(getattr(pd, qname), oq)
            sm, osm = pl._softmax, ol.softmax
            quantizer_pairs(sm.oq, osm.oq)
            for tp, to in ((sm.exp_table, osm.exp_table), (sm.inv_table, osm.inv_table)):
                quantizer_pairs(tp.iq, to.iq)
                quantizer_pairs(tp.oq, to.oq)
            if ol.oq is not None:
                quantizer_pairs(pl.oq, ol.oq)
            continue
        pairs.append((ol.kernel, pl._kernel, None, None))
        if ol.bias is not None:
            pairs.append((ol.bias, pl._bias, None, None))
        for qname, oq in ol.quantizers().items():
            pq = getattr(pl, qname).quantizer
            for vname, leaf in oq.trainable_leaves().items():
                pairs.append((leaf, getattr(pq, '_' + vname), None, None))
    return twin, pairs


class OracleAdam:
    """Keras Adam + per-variable regulariser (as a loss term) + constraint, on (leaf, product Variable) pairs."""

    def __init__(self, pairs, lr=1e-3, b1=0.9, b2=0.999, eps=1e-7):
        self.pairs = pairs
        self.lr, self.b1, self.b2, self.eps = lr, b1, b2, eps
        self.m = [torch.zeros_like(p[0]) for p in pairs]
        self.v = [torch.zeros_like(p[0]) for p in pairs]
        self.t = 0

    def regularization_loss(self):
        total = torch.zeros(())
        for leaf, var, _, _ in self.pairs:
            if var.regularizer is not None:
                total = total + var.regularizer.l1 * torch.sum(leaf)
        return total

    def step(self):
        self.t += 1
        alpha = self.lr * (1 - self.b2**self.t) ** 0.5 / (1 - self.b1**self.t)
        with torch.no_grad():
            for j, (leaf, var, _, _) in enumerate(self.pairs):
                g = leaf.grad
                self.m[j] = self.b1 * self.m[j] + (1 - self.b1) * g
                self.v[j] = self.b2 * self.v[j] + (1 - self.b2) * g * g
                leaf -= alpha * self.m[j] / (torch.sqrt(self.v[j]) + self.eps)
                c = var.constraint
                if c is not None:
                    leaf.copy_(c(leaf))
                leaf.grad = None


def train_step(twin: OracleSequential, opt: OracleAdam, x, y, loss_fn):
    pred = twin(x, training=True)
    task = loss_fn(pred, y)
    total = task + sum(twin.losses) + opt.regularization_loss()
    total.backward()
    opt.step()
    return total.detach()


class TracingFlag:
    """Compares equal to 'tracing' and is falsy (utils/minmax_trace.py:25-33)."""

    def __eq__(self, other):
        return other == 'tracing'

    def __hash__(self):
        return hash('tracing')

    def __bool__(self):
        return False


def _all_quantizers(obj, seen=None):
    """Every OracleFixedQuantizer reachable from an oracle layer (attributes, nested oracle layers, lists/tuples)."""
    seen = set() if seen is None else seen
    if id(obj) in seen:
        return
    seen.add(id(obj))
    if isinstance(obj, OL.OracleFixedQuantizer):
        yield obj
        return
    if isinstance(obj, (list, tuple)):
        for v in obj:
            yield from _all_quantizers(v, seen)
    elif isinstance(obj, (OL.OracleQLayer, OracleSequential)):
        for v in vars(obj).values():
            yield from _all_quantizers(v, seen)


def trace_minmax(twin: OracleSequential, x: torch.Tensor, reset=True, batch_size=1024):
    """utils/minmax_trace.py:35-99 on the oracle twin: reset i (-1e9) and k (0) of the trainable WRAP quantizers, run
    the data in batches with training == 'tracing', return (total EBOPs, outputs)."""
    if reset:
        for q in _all_quantizers(twin):
            if q.overflow_mode == 'WRAP' and q.trainable:
                q._i.data.fill_(-1e9)
                q._k = torch.zeros_like(q._k)
    outs = []
    with torch.no_grad():
        for s in range(0, len(x), batch_size):
            outs.append(twin(x[s:s + batch_size], training=TracingFlag()))
    total = 0
    for l in twin.qlayers():
        if l.enable_ebops:
            total += l.total_ebops() if hasattr(l, 'total_ebops') else int(l.ebops.item())
    return total, torch.cat(outs)
