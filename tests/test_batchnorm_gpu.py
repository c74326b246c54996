"""Batch-normalisation layers (QBatchNormDense, QEinsumDenseBatchnorm, QBatchNormalization) against the CPU oracle, and
the behavioural check of the reference's tests/test_batchnorm.py (dummy quantizers => plain batch normalisation)."""

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


def make_scopes(q_type, overflow_mode, beta0=1e-3):
    from hgq2_b200.config import LayerConfigScope, QuantizerConfigScope

    scope_w = QuantizerConfigScope(default_q_type=q_type, place=('weight', 'bias'), k0=1, i0=3, f0=4, heterogeneous_axis=None,
                                   homogeneous_axis=(), overflow_mode=overflow_mode, round_mode='RND')
    scope_a = QuantizerConfigScope(default_q_type='kif', place='datalane', heterogeneous_axis=None, homogeneous_axis=(0,),
                                   overflow_mode=overflow_mode, round_mode='RND')
    return scope_w, scope_a, LayerConfigScope(beta0=beta0, enable_ebops=True)


def grid_input(rng, shape):
    return (np.round(np.clip(rng.standard_normal(shape), -5, 5) * 256) / 256).astype(np.float32)


def randomise(layer, rng):
    """Non-trivial statistics and affine parameters, assigned from numpy on both sides."""
    dev = layer.moving_mean.value.device
    n = tuple(layer.moving_mean.shape)
    layer.moving_mean.assign(torch.from_numpy(rng.standard_normal(n).astype(np.float32)).to(dev))
    layer.moving_variance.assign(torch.from_numpy(rng.uniform(0.5, 4.0, n).astype(np.float32)).to(dev))
    for name in ('_bn_gamma', '_bn_beta'):
        v = getattr(layer, name, None)
        if v is not None:
            v.assign(torch.from_numpy(rng.uniform(0.5, 1.5, tuple(v.shape)).astype(np.float32)).to(dev))
    if getattr(layer, '_bias', None) is not None:
        layer._bias.assign(torch.from_numpy(rng.standard_normal(tuple(layer._bias.shape)).astype(np.float32)).to(dev))


def run_pair(layer, x_np, rng):
    x = torch.from_numpy(x_np).cuda()
    layer(x[:4], training=False)
    randomise(layer, rng)
    twin = OL.mirror_bn_layer(layer)
    for step in range(2):  # two steps: the second one sees the updated moving statistics and integer bits
        xg, xc = x.clone().requires_grad_(), torch.from_numpy(x_np).requires_grad_()
        y, yc = layer(xg, training=True), twin(xc, training=True)
        rel_close(y, yc, 1e-5, f'output, step {step}')
        assert int(layer.ebops.item()) == int(twin.ebops.item()) and int(twin.ebops.item()) > 0
        w = torch.from_numpy(rng.standard_normal(tuple(yc.shape)).astype(np.float32))
        for v in layer.trainable_variables:
            v.value.grad = None
        ((y * w.cuda()).sum() / x.shape[0] + sum(layer.losses)).backward()
        ((yc * w).sum() / x.shape[0] + sum(twin.losses)).backward()
        rel_close(xg.grad, xc.grad, 1e-4, 'dx')
        rel_close(layer.moving_mean.value, twin.moving_mean, 1e-5, 'moving_mean')
        rel_close(layer.moving_variance.value, twin.moving_variance, 1e-5, 'moving_variance')
        for pname, leaf in (('_kernel', getattr(twin, 'kernel', None)), ('_bias', getattr(twin, 'bias', None)),
                            ('_bn_gamma', twin.bn_gamma), ('_bn_beta', getattr(twin, 'bn_beta', None))):
            if leaf is not None and leaf.requires_grad:
                rel_close(getattr(layer, pname).value.grad, leaf.grad, 1e-4, f'd{pname}')
                leaf.grad = None
        for qname, tq in twin.quantizers().items():
            pq = getattr(layer, qname).quantizer
            assert torch.equal(pq._i.value.detach().cpu(), tq._i.detach()), qname
            for vname, lf in tq.trainable_leaves().items():
                rel_close(getattr(pq, '_' + vname).value.grad, lf.grad, 1e-4, f'd {qname}.{vname}')
                lf.grad = None
    rel_close(layer(x, training=False), twin(torch.from_numpy(x_np), training=False), 1e-5, 'eval output')


@pytest.mark.parametrize('q_type,overflow_mode', [('kbi', 'WRAP'), ('kif', 'SAT')])
def test_qbatchnorm_dense(q_type, overflow_mode):
    from hgq2_b200.layers import QBatchNormDense

    rng = np.random.default_rng(21)
    w, a, l = make_scopes(q_type, overflow_mode)
    with w, a, l:
        layer = QBatchNormDense(8, activation='relu')
    run_pair(layer, grid_input(rng, (300, 12)), rng)


@pytest.mark.parametrize('q_type,overflow_mode', [('kbi', 'WRAP'), ('kif', 'SAT')])
@pytest.mark.parametrize('equation,in_shape,out_shape,bias_axes', [
    ('bpc,cd->bpd', (9, 6), (9, 8), 'd'),
    ('Bij,ijk->Bik', (3, 4), (3, 6), 'ik'),
])
def test_qeinsum_dense_batchnorm(equation, in_shape, out_shape, bias_axes, q_type, overflow_mode):
    from hgq2_b200.layers import QEinsumDenseBatchnorm

    rng = np.random.default_rng(22)
    w, a, l = make_scopes(q_type, overflow_mode)
    with w, a, l:
        layer = QEinsumDenseBatchnorm(equation, out_shape, bias_axes=bias_axes, activation='relu')
    run_pair(layer, grid_input(rng, (200,) + in_shape), rng)


@pytest.mark.parametrize('q_type,overflow_mode', [('kbi', 'WRAP'), ('kif', 'SAT')])
@pytest.mark.parametrize('center,scale', [(True, True), (False, True)])
def test_qbatch_normalization(center, scale, q_type, overflow_mode):
    from hgq2_b200.layers import QBatchNormalization

    rng = np.random.default_rng(23)
    w, a, l = make_scopes(q_type, overflow_mode)
    with w, a, l:
        layer = QBatchNormalization(axis=2, center=center, scale=scale)
    run_pair(layer, grid_input(rng, (128, 6, 8)), rng)


def test_dummy_quantizers_give_plain_batch_normalisation():
    # tests/test_batchnorm.py:43-58 of the reference: momentum 0, dummy quantizers
    from hgq2_b200.config import LayerConfigScope, QuantizerConfigScope
    from hgq2_b200.layers import QBatchNormalization

    rng = np.random.default_rng(3)
    with QuantizerConfigScope(default_q_type='dummy'), LayerConfigScope(enable_ebops=False):
        bn = QBatchNormalization(axis=2, momentum=0.0)
    x = torch.from_numpy(grid_input(rng, (64, 6, 8))).cuda()
    y = bn(x, training=True)
    y_eval = bn(x, training=False)
    mean = x.mean(dim=(0, 1), keepdim=True)
    var = (x * x).mean(dim=(0, 1), keepdim=True) - mean * mean
    ref = (x - mean) / torch.sqrt(var + bn.epsilon)
    assert float((y.detach() - ref).abs().max()) <= 1e-5
    assert float((y_eval - ref).abs().max()) <= 1e-5
