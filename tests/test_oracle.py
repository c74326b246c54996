"""CPU checks that pin the oracle itself (no GPU, no CUDA library)."""

import json

import numpy as np
import pytest
import torch

from oracle import fixed_point_ops as O

MODES = [(rm, om) for rm in O.ROUND_MODES for om in O.OVERFLOW_MODES]


def test_pow2_is_exact_on_this_host():
    # the oracle writes 2.0**f like the reference does; it is only a valid checker if that is exact
    f = torch.arange(-100, 101, dtype=torch.float32)
    assert torch.equal(2.0**f, torch.ldexp(torch.ones_like(f), f.int()))


def test_known_answers(golden_dir):
    rows = json.loads((golden_dir / 'quantizer_kat.json').read_text())
    for row in rows:
        k, i, f = (torch.tensor(float(v)) for v in row['kif'])
        for rm, expect in row['expect'].items():
            for om, e in zip(O.OVERFLOW_MODES, expect):
                y = O.quantize_fwd(torch.tensor(row['x']), k, i, f, rm, om, training=False)
                assert float(y) == e, (row, rm, om, float(y))


@pytest.mark.parametrize('rm,om', MODES)
def test_range_and_grid(rm, om):
    # eval-mode outputs lie on the 2^-f grid inside [min, max] of the reference's range properties
    # (src/hgq/quantizer/internal/fixed_point_quantizer.py:107-120)
    rng = np.random.default_rng(0)
    n = 20000
    x = torch.from_numpy((rng.standard_normal(n) * 8).astype(np.float32))
    k = torch.from_numpy(rng.integers(0, 2, n).astype(np.float32))
    i = torch.from_numpy(rng.integers(-1, 5, n).astype(np.float32))
    f = torch.from_numpy(rng.integers(1, 8, n).astype(np.float32))
    y = O.quantize_fwd(x, k, i, f, rm, om, training=False)
    hi = 2.0**i - 2.0**-f
    lo = -k * (hi if om == 'SAT_SYM' else 2.0**i)
    if om == 'SAT_SYM':
        # WRAP/SAT use the asymmetric two's-complement range
        pass
    lo_eff = lo if om != 'WRAP' else -k * 2.0**i
    assert bool(((y >= lo_eff) & (y <= hi)).all())
    assert torch.equal(y * 2.0**f, torch.round(y * 2.0**f))
    # in-range inputs are only rounded
    inside = (x >= lo_eff + 1) & (x <= hi - 1)
    assert torch.equal(y[inside], O.round_fwd(x, f, rm)[inside])


@pytest.mark.parametrize('rm,om', MODES)
def test_golden_reproducible(rm, om, quantizer_golden):
    z, _ = quantizer_golden  # made by the real `quantizers` package when that file exists: then this test pins the oracle
    t = {n: torch.from_numpy(z[n].astype(np.float32)) for n in ('x', 'k', 'i', 'f', 'g')}
    for training in (False, True):
        y = O.quantize_fwd(t['x'], t['k'], t['i'], t['f'], rm, om, training).numpy()
        ref = z[f"y_{'train' if training else 'eval'}_{rm}_{om}"]
        assert np.array_equal(y.view(np.int32), ref.view(np.int32))
    dx, di, df = O.quantize_bwd(t['g'], t['x'], t['k'], t['i'], t['f'], rm, om)
    for name, v in (('dx', dx), ('di', di), ('df', df)):
        assert np.array_equal(v.numpy().view(np.int32), z[f'{name}_{rm}_{om}'].view(np.int32))


@pytest.mark.parametrize('rm,om', MODES)
def test_closed_form_backward_matches_autograd(rm, om):
    # the closed-form surrogate equals torch autograd through the forward op sequence with a
    # straight-through rnd(); float64 keeps the comparison free of cancellation noise
    rng = np.random.default_rng(3)
    n = 5000
    x = torch.from_numpy(rng.standard_normal(n) * 4).double().requires_grad_()
    k = torch.from_numpy(rng.integers(0, 2, n).astype(np.float64))
    i = torch.from_numpy(rng.integers(-2, 7, n).astype(np.float64)).requires_grad_()
    f = torch.from_numpy(rng.integers(0, 9, n).astype(np.float64)).requires_grad_()
    g = torch.from_numpy(rng.standard_normal(n))
    y = O.quantize_autograd(x, k, i, f, rm, om)
    y.backward(g)
    dx, di, df = O.quantize_bwd(g.float(), x.detach().float().double().float(), k.float(), i.detach().float(), f.detach().float(), rm, om)
    # the closed form ran on fp32-rounded x; redo autograd on the same values for a fair check
    x32 = x.detach().float().double().requires_grad_()
    i2, f2 = i.detach().clone().requires_grad_(), f.detach().clone().requires_grad_()
    O.quantize_autograd(x32, k, i2, f2, rm, om).backward(g.float().double())
    np.testing.assert_allclose(dx.numpy(), x32.grad.numpy(), rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(df.numpy(), f2.grad.numpy(), rtol=1e-4, atol=1e-5)
    if om != 'WRAP':
        np.testing.assert_allclose(di.numpy(), i2.grad.numpy(), rtol=1e-5, atol=1e-6)


def test_quantizer_object_interface():
    q = O.get_fixed_quantizer('rnd', 'sat')
    assert q.round_mode == 'RND' and q.overflow_mode == 'SAT' and q.stochastic is False
    x = torch.tensor([0.3, 9.0, -9.0], requires_grad=True)
    i = torch.tensor(2.0, requires_grad=True)
    f = torch.tensor(2.0, requires_grad=True)
    y = q(x, torch.tensor(1.0), i, f, True, None)
    assert y.tolist() == [0.25, 3.75, -4.0]
    y.sum().backward()
    assert x.grad.tolist() == [1.0, 0.0, 0.0]
    assert i.grad.shape == () and f.grad.shape == ()
    r = q.round(torch.tensor([0.3, 9.0]), torch.tensor(1.0))
    assert r.tolist() == [0.5, 9.0]
    with pytest.raises(ValueError):
        O.get_fixed_quantizer('S_RND', 'WRAP')
