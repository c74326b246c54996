"""A stack of small dense layers in one launch (hgq_dense_chain_fwd / _bwd) against the oracle's op sequence evaluated in
float64: every layer's output and abs-max statistic, the input gradient, and every layer's dWq, dbq and df."""

import numpy as np
import pytest
import torch

from oracle import fixed_point_ops as O

pytestmark = pytest.mark.gpu


def _stack(rng, widths, relus, rms, M, bias=True):
    x = torch.from_numpy((rng.standard_normal((M, widths[0])) * 2).astype(np.float32))
    layers = []
    for l, (K, N) in enumerate(zip(widths[:-1], widths[1:])):
        layers.append(dict(
            K=K, N=N, relu=relus[l], round_mode=rms[l],
            qf=torch.from_numpy(rng.integers(1, 7, K).astype(np.float32)),
            wq=torch.from_numpy(np.round(rng.uniform(-1.5, 1.5, (K, N)) * 32) / 32).float(),
            bq=(torch.from_numpy(np.round(rng.uniform(-1, 1, N) * 16) / 16).float() if bias else None),
        ))
    return x, layers


def _reference_backward(inputs, outputs, layers, gy):
    """float64 backward of the stack from the oracle's definitions.  ``inputs[l]`` / ``outputs[l]`` are the fp32 activations
    entering / leaving layer l as the forward wrote them, so that a rounding decision at a grid boundary and the sign of an
    output at zero are taken on the same values on both sides."""
    g = gy.double()
    grads = []
    for L, x_l, y_l in zip(reversed(layers), reversed(inputs), reversed(outputs)):
        f = L['qf'].view(1, -1).expand(x_l.shape[0], -1)
        xq = O.round_fwd(x_l, f, L['round_mode']).double()
        if L['relu']:
            g = g * (y_l > 0)
        dxq = g @ L['wq'].double().t()
        grads.append(dict(dwq=xq.t() @ g, dbq=g.sum(0), df=((xq - x_l.double()) * (-O.LN2) * dxq).sum(0)))
        g = dxq
    return list(reversed(grads)), g


def _rel(a, b):
    b = b.double()
    return float((a.cpu().double() - b).abs().max() / max(float(b.abs().max()), 1e-30))


@pytest.mark.parametrize('widths,relus,M', [
    ((16, 64, 32, 32, 5), (True, True, True, False), 16384),   # the jet-tagger MLP at its benchmark batch
    ((16, 64, 32, 32, 5), (True, True, True, False), 128 * 3 + 17),
    ((27, 20, 5), (False, True), 1000),                         # widths that are no multiple of four
    ((64, 64), (True,), 129),
    ((3, 7, 64, 1), (True, False, True), 50),
    ((8, 8, 8, 8, 8, 8, 8, 8, 8), (True,) * 8, 300),            # eight layers
    ((16, 64, 32, 5), (True, True, False), 128 * 300 + 5),      # more tiles than SMs: a block walks several, ragged last tile
])
@pytest.mark.parametrize('rm', ['RND', 'TRN', 'RND_CONV'])
def test_dense_chain_forward_and_backward(widths, relus, M, rm):
    from hgq2_b200 import kernels as K

    rng = np.random.default_rng(len(widths) * 1000 + M)
    n = len(widths) - 1
    x, layers = _stack(rng, widths, relus, [rm] * n, M)
    assert K.dense_chain_supported(widths)
    dev = torch.device('cuda')
    xd = x.to(dev)
    specs = []
    for L in layers:
        s = {k: (v.to(dev) if torch.is_tensor(v) else v) for k, v in L.items()}
        s['y'] = torch.empty(M, L['N'], device=dev)
        s['absmax'] = torch.zeros(L['K'], device=dev)
        s['dwq'] = torch.full((L['K'], L['N']), float('nan'), device=dev)
        s['dbq'] = torch.full((L['N'],), float('nan'), device=dev)
        s['df'] = torch.full((L['K'],), float('nan'), device=dev)
        specs.append(s)
    arr = K.dense_chain_layers(specs)
    K.dense_chain_fwd(xd, arr, n)
    gy = torch.from_numpy(rng.standard_normal((M, widths[-1])).astype(np.float32))
    dx = torch.full((M, widths[0]), float('nan'), device=dev)
    K.dense_chain_bwd(gy.to(dev), xd, dx, arr, n)
    torch.cuda.synchronize()
    # forward: every layer on the fp32 activations the previous one wrote
    h = x
    inputs, outputs = [], []
    for l, s in enumerate(specs):
        f = layers[l]['qf'].view(1, -1).expand(M, -1)
        xq = O.round_fwd(h, f, rm)
        y_here = (xq.double() @ layers[l]['wq'].double() + layers[l]['bq'].double())
        if layers[l]['relu']:
            y_here = y_here.clamp_min(0)
        assert _rel(s['y'], y_here) <= 1e-6, (l, 'y', _rel(s['y'], y_here))
        assert torch.equal(s['absmax'].cpu(), xq.abs().amax(0)), (l, 'absmax')
        inputs.append(h)
        h = s['y'].cpu()
        outputs.append(h)
    grads, dx_ref = _reference_backward(inputs, outputs, layers, gy)
    assert _rel(dx, dx_ref) <= 1e-4, ('dx', _rel(dx, dx_ref))
    for l, (s, g) in enumerate(zip(specs, grads)):
        for name in ('dwq', 'dbq', 'df'):
            assert _rel(s[name], g[name]) <= 1e-4, (l, name, _rel(s[name], g[name]))


def test_dense_chain_is_repeatable_and_accumulates_statistics():
    from hgq2_b200 import kernels as K

    rng = np.random.default_rng(5)
    widths, M = (16, 64, 32, 5), 4000
    x, layers = _stack(rng, widths, (True, True, False), ['RND'] * 3, M)
    dev = torch.device('cuda')
    outs = []
    for _ in range(2):
        specs = []
        for L in layers:
            s = {k: (v.to(dev) if torch.is_tensor(v) else v) for k, v in L.items()}
            s.update(y=torch.empty(M, L['N'], device=dev), absmax=torch.full((L['K'],), 0.5, device=dev),
                     dwq=torch.empty(L['K'], L['N'], device=dev), dbq=torch.empty(L['N'], device=dev), df=torch.empty(L['K'], device=dev))
            specs.append(s)
        arr = K.dense_chain_layers(specs)
        K.dense_chain_fwd(x.to(dev), arr, 3)
        gy = torch.from_numpy(np.random.default_rng(6).standard_normal((M, 5)).astype(np.float32)).to(dev)
        K.dense_chain_bwd(gy, x.to(dev), None, arr, 3)
        outs.append(specs)
    for a, b in zip(*outs):
        for name in ('y', 'absmax', 'dwq', 'dbq', 'df'):
            assert torch.equal(a[name], b[name]), name
        assert float(a['absmax'].min()) >= 0.5  # merged into what was there


def test_dense_chain_limits():
    from hgq2_b200 import kernels as K

    assert K.dense_chain_supported((16, 64, 32, 32, 5))
    assert not K.dense_chain_supported((16, 65))
    assert not K.dense_chain_supported((128, 16))
    assert not K.dense_chain_supported((8,) * 10)  # nine layers
