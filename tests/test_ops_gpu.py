"""Accumulation, merge and pooling layers against the CPU oracle: outputs, exact EBOPs, gradients, quantizer state."""

import numpy as np
import pytest
import torch

from oracle import hgq_layers as OL

pytestmark = pytest.mark.gpu


def rel_close(a, b, rtol, what):
    a = a.detach().cpu().double().numpy()
    b = b.detach().cpu().double().numpy()
    scale = max(np.abs(b).max(), 1e-30)
    err = np.abs(a - b).max() / scale
    assert err <= rtol, f'{what}: {err:.3e} > {rtol}'


def scopes(q_type, overflow_mode):
    from hgq2_b200.config import LayerConfigScope, QuantizerConfigScope

    return (QuantizerConfigScope(place='datalane', default_q_type=q_type, overflow_mode=overflow_mode, round_mode='RND'),
            LayerConfigScope(beta0=1e-3, enable_ebops=True))


def grid(rng, shape):
    return (np.round(np.clip(rng.standard_normal(shape), -5, 5) * 256) / 256).astype(np.float32)


def perturb(q, rng):
    """Integer perturbation of the trainable bitwidths (tests/base.py:161-182 of the reference)."""
    iq = q.quantizer
    for name in ('_f', '_b', '_i'):
        v = getattr(iq, name, None)
        if v is not None and v.trainable:
            v.assign(v.value.detach() + torch.from_numpy(rng.integers(-2, 3, tuple(v.shape)).astype(np.float32)).to(v.value.device))


def check_quantizers(pairs):
    for pq, tq in pairs:
        q = pq.quantizer
        assert torch.equal(q._i.value.detach().cpu(), tq._i.detach())
        assert torch.equal(q._k.value.cpu(), tq._k)
        for vname, leaf in tq.trainable_leaves().items():
            g = getattr(q, '_' + vname).value.grad
            assert g is not None, vname
            rel_close(g, leaf.grad, 1e-4, f'd{vname}')


SINGLE = [
    ('QSum', dict(axes=1), (60, 9, 6)),
    ('QSum', dict(axes=(1, 2), scale=0.25, keepdims=True), (40, 5, 4, 6)),
    ('QMeanPow2', dict(axes=1), (50, 16, 7)),
    ('QMaxPooling2D', dict(pool_size=2), (30, 9, 8, 8)),
    ('QAveragePooling2D', dict(pool_size=2), (30, 8, 8, 5)),
    ('QMaxPooling1D', dict(pool_size=2), (30, 9, 8)),
    ('QMaxPooling1D', dict(pool_size=3, strides=2), (30, 11, 5)),
    ('QAveragePooling1D', dict(pool_size=2), (30, 8, 5)),
    ('QGlobalAveragePooling1D', dict(), (40, 8, 6)),
    ('QGlobalAveragePooling2D', dict(keepdims=True), (30, 4, 4, 6)),
    ('QGlobalMaxPooling1D', dict(), (40, 8, 6)),
    ('QGlobalMaxPooling2D', dict(), (30, 4, 4, 6)),
]


@pytest.mark.parametrize('q_type,overflow_mode', [('kif', 'WRAP'), ('kbi', 'SAT')])
@pytest.mark.parametrize('cls,kwargs,shape', SINGLE)
def test_single_input_op_layers(cls, kwargs, shape, q_type, overflow_mode):
    from hgq2_b200 import layers as L

    rng = np.random.default_rng(13)
    a, l = scopes(q_type, overflow_mode)
    with a, l:
        layer = getattr(L, cls)(**kwargs)
    x_np = grid(rng, shape)
    x = torch.from_numpy(x_np).cuda()
    layer(x[:2], training=False)
    perturb(layer.iq, rng)
    twin = OL.mirror_op_layer(layer)
    xg, xc = x.clone().requires_grad_(), torch.from_numpy(x_np).requires_grad_()
    y, yc = layer(xg, training=True), twin(xc, training=True)
    assert tuple(y.shape) == tuple(yc.shape) == tuple(layer.compute_output_shape(shape))
    rel_close(y, yc, 1e-5, 'output')
    assert int(layer.ebops.item()) == int(twin.ebops.item()) and int(twin.ebops.item()) > 0
    w = torch.from_numpy(rng.standard_normal(tuple(yc.shape)).astype(np.float32))
    ((y * w.cuda()).sum() + sum(layer.losses)).backward()
    ((yc * w).sum() + sum(twin.losses)).backward()
    rel_close(xg.grad, xc.grad, 1e-4, 'dx')
    check_quantizers([(layer.iq, twin.iq)])
    rel_close(layer(x, training=False), twin(torch.from_numpy(x_np), training=False), 1e-5, 'eval output')


@pytest.mark.parametrize('q_type,overflow_mode', [('kif', 'WRAP'), ('kbi', 'SAT')])
@pytest.mark.parametrize('cls,n_in', [('QAdd', 3), ('QAveragePow2', 4), ('QSubtract', 2), ('QMultiply', 2), ('QMaximum', 3),
                                      ('QMinimum', 2)])
def test_merge_layers(cls, n_in, q_type, overflow_mode):
    from hgq2_b200 import layers as L

    rng = np.random.default_rng(17)
    a, l = scopes(q_type, overflow_mode)
    with a, l:
        layer = getattr(L, cls)()
    xs_np = [grid(rng, (50, 6, 5)) for _ in range(n_in)]
    xs = [torch.from_numpy(v).cuda() for v in xs_np]
    layer([t[:2] for t in xs], training=False)
    for q in layer.iq:
        perturb(q, rng)
    twin = OL.mirror_op_layer(layer)
    xg = [t.clone().requires_grad_() for t in xs]
    xc = [torch.from_numpy(v).requires_grad_() for v in xs_np]
    y, yc = layer(xg, training=True), twin(xc, training=True)
    rel_close(y, yc, 1e-5, 'output')
    assert int(layer.ebops.item()) == int(twin.ebops.item()) and int(twin.ebops.item()) > 0
    w = torch.from_numpy(rng.standard_normal(tuple(yc.shape)).astype(np.float32))
    ((y * w.cuda()).sum() + sum(layer.losses)).backward()
    ((yc * w).sum() + sum(twin.losses)).backward()
    for g, gc in zip(xg, xc):
        rel_close(g.grad, gc.grad, 1e-4, 'dx')
    check_quantizers(list(zip(layer.iq, twin.iqs)))
