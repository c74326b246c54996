"""Layer-level parity on the GPU: hgq2_b200 layers (CUDA kernels) against the CPU oracle twin.

Follows the conventions of the reference's own layer tests (tests/base.py of HGQ2): inputs on a 2^-8
grid clipped to +-5, per-element bitwidths perturbed by assignment, {kif,kbi} x {WRAP,SAT} x {TRN,RND},
per-element and per-tensor activation bitwidths, beta0 chosen so the EBOPs term shows in the gradients.
Quantized tensors, integer bit counts and EBOPs must match exactly; outputs / loss within rel 1e-5 and
gradients within rel 1e-4 (the tolerances the path is specified to).
"""

import numpy as np
import pytest
import torch

from oracle import hgq_layers as OL

pytestmark = pytest.mark.gpu


def make_scopes(q_type, overflow_mode, round_mode, parallel_io, beta0=1e-3):
    from hgq2_b200.config import LayerConfigScope, QuantizerConfigScope

    het, hom = (None, (0,)) if parallel_io else ((), None)
    scope_w = QuantizerConfigScope(default_q_type=q_type, place=('weight', 'bias'), k0=1, i0=2, f0=2,
                                   heterogeneous_axis=None, homogeneous_axis=(), overflow_mode=overflow_mode,
                                   round_mode='RND' if q_type == 'kbi' else round_mode)
    scope_a = QuantizerConfigScope(default_q_type='kif', place=('datalane', 'table'), heterogeneous_axis=het,
                                   homogeneous_axis=hom, overflow_mode=overflow_mode, round_mode=round_mode)
    scope_l = LayerConfigScope(beta0=beta0, enable_ebops=True)
    return scope_w, scope_a, scope_l


def perturb(layer, rng, parallel_io):
    """Random per-element bitwidths, assigned like tests/base.py:161-182 of the reference does."""
    from hgq2_b200.quantizer.internal import FixedPointQuantizerKBI, FixedPointQuantizerKIF

    for q in layer._flatten_layers():
        if isinstance(q, FixedPointQuantizerKBI):
            b = rng.integers(0, 6, q._b.shape)
            if np.all(b == 0):
                b.ravel()[0] = 1
            q._b.assign(torch.from_numpy(b.astype(np.float32)))
        elif isinstance(q, FixedPointQuantizerKIF) and parallel_io:
            f = rng.integers(2, 6, q._f.shape)
            q._f.assign(torch.from_numpy(f.astype(np.float32)))
    if layer.bias is not None:
        layer._bias.assign(torch.from_numpy(rng.standard_normal(layer._bias.shape).astype(np.float32)))


def grid_input(rng, shape):
    return (np.round(np.clip(rng.standard_normal(shape), -5, 5) * 256) / 256).astype(np.float32)


def rel_close(a, b, rtol, what, scale=None):
    a = a.detach().cpu().double().numpy()
    b = b.detach().cpu().double().numpy()
    scale = max(np.abs(b).max(), 1e-30) if scale is None else scale
    err = np.abs(a - b).max() / scale
    assert err <= rtol, f'{what}: max error {err:.3e} relative to max |ref| {scale:.3e} exceeds {rtol}'


def run_pair(layer, x_np, rng, check_eval=True):
    """One training forward + backward on both sides; returns nothing, asserts parity."""
    x = torch.from_numpy(x_np).cuda()
    layer(x[:2], training=False) if not layer.built else None  # build
    twin = OL.mirror_layer(layer)
    xg = x.clone().requires_grad_()
    xc = torch.from_numpy(x_np).requires_grad_()
    y = layer(xg, training=True)
    yc = twin(xc, training=True)
    rel_close(y, yc, 1e-5, 'output')
    w = torch.from_numpy(rng.standard_normal(tuple(yc.shape)).astype(np.float32))
    loss = (y * w.cuda()).sum() / x.shape[0] + sum(layer.losses)
    lossc = (yc * w).sum() / x.shape[0] + sum(twin.losses)
    # the bitwidth regularisers (MonoL1: l1 * sum of the variable) are part of the product layer's losses
    for qname, tq in twin.quantizers().items():
        pq = getattr(layer, qname).quantizer
        for vname, leaf in tq.trainable_leaves().items():
            reg = getattr(pq, '_' + vname).regularizer
            if reg is not None:
                lossc = lossc + reg.l1 * leaf.sum()
    # the loss is a sum of signed terms that largely cancel: its fp32 summation error is relative to sum |terms|
    rel_close(loss, lossc, 1e-5, 'loss', scale=float((yc.detach() * w).abs().sum() / x.shape[0] + abs(float(lossc.detach()))))
    # EBOPs: exact integer
    assert int(layer.ebops.item()) == int(twin.ebops.item()), (int(layer.ebops.item()), int(twin.ebops.item()))
    loss.backward()
    lossc.backward()
    rel_close(xg.grad, xc.grad, 1e-4, 'dx')
    rel_close(layer._kernel.value.grad, twin.kernel.grad, 1e-4, 'dkernel')
    if layer.bias is not None:
        rel_close(layer._bias.value.grad, twin.bias.grad, 1e-4, 'dbias')
    for qname, tq in twin.quantizers().items():
        pq = getattr(layer, qname).quantizer
        # state after the call (WRAP integer-bit tracking) and integer bit counts
        assert torch.equal(pq._i.value.detach().cpu(), tq._i.detach()), f'{qname}._i after training call'
        assert torch.equal(pq._k.value.cpu(), tq._k), f'{qname}._k'
        assert torch.equal(pq.bits.detach().cpu(), tq.bits.detach()), f'{qname}.bits'
        for vname, leaf in tq.trainable_leaves().items():
            g = getattr(pq, '_' + vname).value.grad
            assert g is not None, f'{qname}.{vname} has no gradient'
            rel_close(g, leaf.grad, 1e-4, f'd {qname}.{vname}')
    if check_eval:
        ye = layer(x, training=False)
        yec = twin(torch.from_numpy(x_np), training=False)
        rel_close(ye, yec, 1e-5, 'eval output')


MODES = [(q, o, r) for q in ('kif', 'kbi') for o in ('WRAP', 'SAT') for r in ('TRN', 'RND')]


@pytest.mark.parametrize('parallel_io', [True, False])
@pytest.mark.parametrize('q_type,overflow_mode,round_mode', MODES)
def test_qdense(q_type, overflow_mode, round_mode, parallel_io):
    from hgq2_b200.layers import QDense

    rng = np.random.default_rng(42)
    sw, sa, sl = make_scopes(q_type, overflow_mode, round_mode, parallel_io)
    with sw, sa, sl:
        layer = QDense(7, activation='relu', name=f'd_{q_type}_{overflow_mode}_{round_mode}_{parallel_io}')
    x = grid_input(rng, (500, 12))
    layer(torch.from_numpy(x[:2]).cuda(), training=False)
    perturb(layer, rng, parallel_io)
    from hgq2_b200 import routes

    routes.reset()
    run_pair(layer, x, rng)
    assert not routes.fallbacks(), routes.fallbacks()  # saturating input quantizers included: no library GEMM in the backward


@pytest.mark.parametrize('q_type,overflow_mode,round_mode', [('kbi', 'WRAP', 'RND'), ('kif', 'SAT', 'TRN')])
@pytest.mark.parametrize('equation,in_shape,out_shape,bias_axes', [
    ('bpc,cd->bpd', (9, 6), (9, 5), 'd'),
    ('abc,cde->abde', (8, 6), (8, 2, 3), 'de'),
    ('abcd,cde->abe', (8, 2, 3), (8, 5), 'e'),
    ('ab,bc->ac', (6,), (4,), None),
])
def test_qeinsum_dense(q_type, overflow_mode, round_mode, equation, in_shape, out_shape, bias_axes):
    from hgq2_b200.layers import QEinsumDense

    rng = np.random.default_rng(7)
    sw, sa, sl = make_scopes(q_type, overflow_mode, round_mode, True)
    with sw, sa, sl:
        layer = QEinsumDense(equation, out_shape, bias_axes=bias_axes, activation='relu')
    x = grid_input(rng, (200,) + in_shape)
    layer(torch.from_numpy(x[:2]).cuda(), training=False)
    perturb(layer, rng, True)
    run_pair(layer, x, rng)


@pytest.mark.parametrize('q_type,overflow_mode,round_mode', [('kbi', 'WRAP', 'RND'), ('kif', 'SAT', 'TRN'), ('kbi', 'SAT', 'RND')])
@pytest.mark.parametrize('padding,strides', [('valid', 1), ('same', 1), ('valid', 2), ('same', 2)])
@pytest.mark.parametrize('filters', [5, 8])  # 5: filters of zeros make up a multiple of four
def test_qconv2d(q_type, overflow_mode, round_mode, padding, strides, filters):
    from hgq2_b200.layers import QConv2D

    rng = np.random.default_rng(9)
    sw, sa, sl = make_scopes(q_type, overflow_mode, round_mode, True)
    with sw, sa, sl:
        layer = QConv2D(filters, 3, strides=strides, padding=padding, activation='relu' if filters == 5 else None)
    x = grid_input(rng, (40, 9, 8, 3))
    layer(torch.from_numpy(x[:2]).cuda(), training=False)
    perturb(layer, rng, True)
    run_pair(layer, x, rng)


def test_qconv2d_takes_the_fused_route():
    from hgq2_b200 import _lib
    from hgq2_b200.layers import QConv2D

    rng = np.random.default_rng(3)
    sw, sa, sl = make_scopes('kif', 'WRAP', 'RND', True)
    with sw, sa, sl:
        layer = QConv2D(16, 3, activation='relu')
    x = grid_input(rng, (64, 12, 12, 4))
    layer(torch.from_numpy(x[:2]).cuda(), training=False)
    perturb(layer, rng, True)
    before = _lib.lib().hgq_launch_count()
    run_pair(layer, x, rng)
    # forward + weight gradient (2 launches + reductions) + input gradient: the library convolution is not on this path
    assert _lib.lib().hgq_launch_count() - before >= 6


def test_dummy_quantizer_equals_plain_layer():
    # with q_type 'dummy' a quantised layer computes exactly what the plain layer computes
    # (tests/test_dense.py:31-46 of the reference)
    from hgq2_b200.config import LayerConfigScope, QuantizerConfigScope
    from hgq2_b200.layers import QDense

    rng = np.random.default_rng(1)
    with QuantizerConfigScope(default_q_type='dummy'), LayerConfigScope(enable_ebops=False):
        layer = QDense(6)
    x = torch.from_numpy(grid_input(rng, (50, 10))).cuda()
    y = layer(x, training=True)
    ref = x @ layer.kernel + layer.bias
    assert torch.equal(y, ref)


def test_scopes_restore_defaults():
    from hgq2_b200.config import LayerConfigScope, QuantizerConfigScope, global_config
    from hgq2_b200.quantizer.config import default_configs, default_q_type

    before = {k: dict(v) for k, v in default_configs.items()}
    q_before = dict(default_q_type)
    g_before = dict(global_config)
    with QuantizerConfigScope(default_q_type='kif', place='weight', overflow_mode='SAT', f0=3, i0=1), LayerConfigScope(beta0=1.0):
        assert default_q_type['weight'] == 'kif'
        assert default_configs[('kif', 'weight')]['f0'] == 3 and default_configs[('kbi', 'weight')]['b0'] == 4
        assert global_config['beta0'] == 1.0
    assert {k: dict(v) for k, v in default_configs.items()} == before
    assert dict(default_q_type) == q_before and dict(global_config) == g_before


@pytest.mark.parametrize('q_type,overflow_mode,round_mode', [('kbi', 'WRAP', 'RND'), ('kif', 'SAT', 'TRN'), ('kif', 'WRAP', 'RND')])
@pytest.mark.parametrize('padding', ['valid', 'same', 'causal'])
@pytest.mark.parametrize('conv_params', [
    # the parameter sets of the reference's own QConv1D test (tests/test_conv.py:17-23) on wider inputs, plus a dilated kernel
    {'kernel_size': 1, 'strides': 2, 'parallelization_factor': -1},
    {'kernel_size': 3, 'strides': 1, 'parallelization_factor': -1},
    {'kernel_size': 2, 'strides': 2, 'parallelization_factor': 1},
    {'kernel_size': 3, 'strides': 1, 'dilation_rate': 2},
])
@pytest.mark.parametrize('filters', [4, 16])
def test_qconv1d(q_type, overflow_mode, round_mode, padding, conv_params, filters):
    from hgq2_b200.layers import QConv1D

    rng = np.random.default_rng(11)
    sw, sa, sl = make_scopes(q_type, overflow_mode, round_mode, True)
    with sw, sa, sl:
        layer = QConv1D(filters, padding=padding, activation='relu' if filters == 16 else None, **conv_params)
    x = grid_input(rng, (48, 14, 4))
    layer(torch.from_numpy(x[:2]).cuda(), training=False)
    assert tuple(layer._kernel.shape) == (conv_params['kernel_size'], 4, filters)  # the reference's variable shape
    perturb(layer, rng, True)
    run_pair(layer, x, rng)


def test_qconv1d_takes_the_fused_route():
    from hgq2_b200 import _lib
    from hgq2_b200.layers import QConv1D

    rng = np.random.default_rng(4)
    sw, sa, sl = make_scopes('kif', 'WRAP', 'RND', True)
    with sw, sa, sl:
        layer = QConv1D(16, 5, padding='causal', activation='relu')
    x = grid_input(rng, (256, 50, 8))
    layer(torch.from_numpy(x[:2]).cuda(), training=False)
    perturb(layer, rng, True)
    from hgq2_b200 import routes

    routes.reset()
    before = _lib.lib().hgq_launch_count()
    run_pair(layer, x, rng)
    assert _lib.lib().hgq_launch_count() - before >= 6
    assert not routes.fallbacks(), routes.fallbacks()


@pytest.mark.parametrize('q_type,overflow_mode,round_mode', [('kbi', 'WRAP', 'RND'), ('kif', 'SAT', 'TRN')])
@pytest.mark.parametrize('padding', ['valid', 'same'])
@pytest.mark.parametrize('conv_params', [
    # the parameter sets of the reference's own QConv2D test (tests/test_conv.py:66-73) on its 6 x 6 x 2 inputs and on larger ones
    {'kernel_size': (1, 1), 'strides': (3, 5), 'parallelization_factor': -1},
    {'kernel_size': (3, 3), 'strides': (1, 1), 'parallelization_factor': -1},
    {'kernel_size': (3, 2), 'strides': (1, 3), 'parallelization_factor': 1},
    {'kernel_size': (2, 3), 'strides': (4, 2), 'parallelization_factor': 1},
])
@pytest.mark.parametrize('in_shape,filters', [((6, 6, 2), 4), ((17, 19, 4), 4), ((6, 6, 2), 1), ((9, 10, 3), 5)])
def test_qconv2d_strided_takes_the_fused_route(q_type, overflow_mode, round_mode, padding, conv_params, in_shape, filters):
    """Strided convolutions run on the unit-stride tensor-core kernels after a space-to-depth regrouping: no library
    convolution, and the same parity bounds as everything else."""
    from hgq2_b200 import routes
    from hgq2_b200.layers import QConv2D

    rng = np.random.default_rng(13)
    sw, sa, sl = make_scopes(q_type, overflow_mode, round_mode, True)
    with sw, sa, sl:
        layer = QConv2D(filters, padding=padding, activation='relu', **conv_params)
    x = grid_input(rng, (32,) + in_shape)
    layer(torch.from_numpy(x[:2]).cuda(), training=False)
    perturb(layer, rng, True)
    routes.reset()
    run_pair(layer, x, rng)
    assert not routes.fallbacks(), routes.fallbacks()


@pytest.mark.parametrize('features,units', [(784, 10), (1152, 16), (320, 64)])
def test_wide_qdense_takes_the_fused_route(features, units):
    """A classifier head behind a Flatten (hundreds of inputs, few outputs): forward in one launch with the whole kernel in shared
    memory, backward as one launch per block of 64 inputs; no library matmul."""
    from hgq2_b200 import routes
    from hgq2_b200.layers import QDense

    rng = np.random.default_rng(21)
    sw, sa, sl = make_scopes('kif', 'WRAP', 'RND', True)
    with sw, sa, sl:
        layer = QDense(units, activation='relu')
    x = grid_input(rng, (256, features))
    layer(torch.from_numpy(x[:2]).cuda(), training=False)
    perturb(layer, rng, True)
    routes.reset()
    run_pair(layer, x, rng)
    assert not routes.fallbacks(), routes.fallbacks()
