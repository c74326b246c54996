"""Parity of the K1 CUDA kernels (through the C ABI) with the CPU oracle and the golden fixtures."""

import numpy as np
import pytest
import torch

from oracle import fixed_point_ops as O

pytestmark = pytest.mark.gpu

MODES = [(rm, om) for rm in O.ROUND_MODES for om in O.OVERFLOW_MODES]


def bits(t):
    # canonical bit pattern: -0.0 is folded onto +0.0.  The sign of a zero produced by a clip is
    # not defined by the reference (torch.clamp returns the bound or the value depending on the
    # operand order of the SIMD max instruction it happens to be compiled to); every other value,
    # NaN payloads included, must match bit for bit.
    a = t.detach().cpu().numpy().astype(np.float32, copy=True).ravel()
    a[a == 0] = 0.0
    return a.view(np.int32)


def assert_bit_equal(a, b, what=''):
    a, b = bits(a), bits(b)
    if not np.array_equal(a, b):
        bad = np.flatnonzero(a != b)
        raise AssertionError(f'{what}: {bad.size} of {a.size} differ, first at {bad[:5]}: '
                             f'{a.view(np.float32).ravel()[bad[:5]]} vs {b.view(np.float32).ravel()[bad[:5]]}')


def dev(*arrs):
    return [torch.from_numpy(np.ascontiguousarray(a)).cuda() for a in arrs]


@pytest.fixture(scope='module')
def K():
    from hgq2_b200 import kernels

    return kernels


@pytest.mark.parametrize('rm,om', MODES)
def test_golden_forward_backward(K, rm, om, quantizer_golden):
    z, _ = quantizer_golden  # the reference-made file when present, else the oracle-made one
    x, k, i, f, g = dev(z['x'], z['k'], z['i'], z['f'], z['g'])
    assert_bit_equal(K.quantize_fwd(x, k, i, f, rm, om, training=False), torch.from_numpy(z[f'y_eval_{rm}_{om}']), 'eval')
    assert_bit_equal(K.quantize_fwd(x, k, i, f, rm, om, training=True), torch.from_numpy(z[f'y_train_{rm}_{om}']), 'train')
    dx, di, df = K.quantize_bwd(g, x, k, i, f, rm, om)
    assert_bit_equal(dx, torch.from_numpy(z[f'dx_{rm}_{om}']), 'dx')
    assert_bit_equal(di, torch.from_numpy(z[f'di_{rm}_{om}']), 'di')
    assert_bit_equal(df, torch.from_numpy(z[f'df_{rm}_{om}']), 'df')


@pytest.mark.parametrize('n', [0, 1, 3, 4, 5, 255, 1024, 2049, 100003])
@pytest.mark.parametrize('offset', [0, 1])
def test_ragged_sizes_and_misaligned_views(K, n, offset):
    # sizes that are not multiples of the vector width and pointers that are not 16-byte aligned
    rng = np.random.default_rng(n + 7 * offset)
    m = n + offset
    x = (rng.standard_normal(m) * 4).astype(np.float32)
    k = rng.integers(0, 2, m).astype(np.uint8)
    i = rng.integers(-2, 7, m).astype(np.float32)
    f = rng.integers(0, 9, m).astype(np.float32)
    g = rng.standard_normal(m).astype(np.float32)
    dx_, dk, di_, df_, dg = (t[offset:] for t in dev(x, k, i, f, g))
    cx, ck, ci, cf, cg = (torch.from_numpy(a[offset:]) for a in (x, k, i, f, g))
    for rm, om in (('RND', 'SAT'), ('TRN', 'WRAP'), ('RND_CONV', 'SAT_SYM')):
        y = K.quantize_fwd(dx_, dk, di_, df_, rm, om)
        assert_bit_equal(y, O.quantize_fwd(cx, ck.float(), ci, cf, rm, om), f'fwd {rm} {om}')
        if n:
            a, b, c = K.quantize_bwd(dg, dx_, dk, di_, df_, rm, om)
            ea, eb, ec = O.quantize_bwd(cg, cx, ck.float(), ci, cf, rm, om)
            assert_bit_equal(a, ea, 'dx'); assert_bit_equal(b, eb, 'di'); assert_bit_equal(c, ec, 'df')


@pytest.mark.parametrize('rm,om', MODES)
def test_exhaustive_small_parameters(K, rm, om):
    # every (k, i, f) in a small box against a dense grid of x, including range edges and ties
    ks, is_, fs = np.meshgrid([0, 1], np.arange(-3, 5), np.arange(-2, 7), indexing='ij')
    xs = np.concatenate([np.arange(-40, 40, 0.0625), [1e-20, -1e-20, 1e6, -1e6]]).astype(np.float32)
    P = ks.size
    x = np.repeat(xs[:, None], P, 1)
    k = np.broadcast_to(ks.ravel().astype(np.uint8), x.shape)
    i = np.broadcast_to(is_.ravel().astype(np.float32), x.shape)
    f = np.broadcast_to(fs.ravel().astype(np.float32), x.shape)
    dxv, dk, di_, df_ = dev(x, k, i, f)
    for training in (False, True):
        y = K.quantize_fwd(dxv, dk, di_, df_, rm, om, training=training)
        e = O.quantize_fwd(torch.from_numpy(x), torch.from_numpy(k.astype(np.float32)), torch.from_numpy(i.copy()),
                           torch.from_numpy(f.copy()), rm, om, training)
        assert_bit_equal(y, e, f'training={training}')


@pytest.mark.parametrize('shape,pshape', [((64, 16), (1, 16)), ((33, 7), (1, 7)), ((5, 3, 20), (1, 3, 20)),
                                          ((1000, 64), (1, 64)), ((17, 3600), (1, 3600)), ((4096, 1), (1, 1)),
                                          ((3, 5, 8), (1, 1, 8)), ((9, 1028), (1, 1028))])
@pytest.mark.parametrize('rm,om', [('RND', 'WRAP'), ('RND', 'SAT'), ('TRN', 'SAT_SYM')])
def test_broadcast_layout(K, shape, pshape, rm, om):
    rng = np.random.default_rng(11)
    x = (rng.standard_normal(shape) * 4).astype(np.float32)
    g = rng.standard_normal(shape).astype(np.float32)
    k = rng.integers(0, 2, pshape).astype(np.uint8)
    i = rng.integers(-1, 4, pshape).astype(np.float32)
    f = rng.integers(0, 7, pshape).astype(np.float32)
    dxv, dg, dk, di_, df_ = dev(x, g, k, i, f)
    cx, cg, ck, ci, cf = (torch.from_numpy(a.astype(np.float32)) for a in (x, g, k, i, f))
    for training in (False, True):
        y, amax = K.quantize_fwd(dxv, dk, di_, df_, rm, om, training=training, want_absmax=True)
        assert_bit_equal(y, O.quantize_fwd(cx, ck, ci, cf, rm, om, training), 'y')
        r = O.round_fwd(cx, cf, rm).abs().reshape(-1, int(np.prod(pshape))).amax(0)
        assert_bit_equal(amax, r, 'absmax')
    a, b, c = K.quantize_bwd(dg, dxv, dk, di_, df_, rm, om)
    shp = torch.broadcast_shapes(cx.shape, ci.shape)
    ea, eb, ec = O.quantize_bwd(cg, cx, ck.expand(shp), ci.expand(shp), cf.expand(shp), rm, om)
    assert_bit_equal(a, ea, 'dx')
    P = int(np.prod(pshape))
    # column sums: order of summation differs, so compare against a float64 sum with a tolerance
    eb64 = eb.double().reshape(-1, P).sum(0).numpy()
    ec64 = ec.double().reshape(-1, P).sum(0).numpy()
    scale_b = eb.abs().double().reshape(-1, P).sum(0).numpy() + 1e-30
    scale_c = ec.abs().double().reshape(-1, P).sum(0).numpy() + 1e-30
    assert np.all(np.abs(b.cpu().numpy().ravel() - eb64) <= 1e-5 * scale_b)
    assert np.all(np.abs(c.cpu().numpy().ravel() - ec64) <= 1e-5 * scale_c)


def test_broadcast_backward_is_deterministic(K):
    rng = np.random.default_rng(5)
    x, g = dev((rng.standard_normal((20000, 64)) * 4).astype(np.float32), rng.standard_normal((20000, 64)).astype(np.float32))
    k, i, f = dev(np.ones((1, 64), np.uint8), np.full((1, 64), 2, np.float32), np.full((1, 64), 3, np.float32))
    r1 = K.quantize_bwd(g, x, k, i, f, 'RND', 'SAT')
    r2 = K.quantize_bwd(g, x, k, i, f, 'RND', 'SAT')
    for a, b in zip(r1, r2):
        assert_bit_equal(a, b)


def test_eval_zeroing_flag(K):
    # y = 0 where k + i + f <= 0 (src/hgq/quantizer/internal/fixed_point_quantizer.py:148-149)
    x, = dev(np.linspace(-3, 3, 64, dtype=np.float32))
    k, = dev(np.zeros(64, np.uint8))
    i, = dev(np.full(64, -2, np.float32))
    f, = dev(np.where(np.arange(64) % 2 == 0, 2, 5).astype(np.float32))
    y = K.quantize_fwd(x, k, i, f, 'RND', 'SAT', zero_nonpos=True)
    e = O.quantize_fwd(x.cpu(), k.cpu().float(), i.cpu(), f.cpu(), 'RND', 'SAT')
    e = torch.where(k.cpu().float() + i.cpu() + f.cpu() > 0, e, torch.zeros_like(e))
    assert_bit_equal(y, e)
    assert (y[::2] == 0).all()


def test_round_only_needs_no_k_i(K):
    x, f = dev(np.linspace(-3, 3, 1000, dtype=np.float32), np.full(1000, 3, np.float32))
    y = K.quantize_fwd(x, None, None, f, 'RND', 'NONE')
    assert_bit_equal(y, O.round_fwd(x.cpu(), f.cpu(), 'RND'))


def test_size_independent_properties_at_scale(K):
    # idempotence and range membership on 2^24 elements (too many for the oracle in a unit test)
    n = 1 << 24
    gen = torch.Generator(device='cuda').manual_seed(0)
    x = torch.randn(n, device='cuda', generator=gen) * 4
    k = torch.randint(0, 2, (n,), device='cuda', generator=gen, dtype=torch.uint8)
    i = torch.randint(-2, 7, (n,), device='cuda', generator=gen).float()
    f = torch.randint(0, 9, (n,), device='cuda', generator=gen).float()
    for rm, om in MODES:
        y = K.quantize_fwd(x, k, i, f, rm, om)
        y2 = K.quantize_fwd(y, k, i, f, rm, om)
        nd = (i + f) >= 0  # with i + f < 0 the range is narrower than one step and nothing is representable
        assert torch.equal(y[nd], y2[nd]), (rm, om)
        hi = torch.exp2(i) - torch.exp2(-f)
        lo = -k.float() * (hi if om == 'SAT_SYM' else torch.exp2(i))
        ok = (y <= hi) & (y >= lo) | (hi < lo) | ~nd
        assert bool(ok.all()), (rm, om)


def test_fused_integer_bit_tracking_matches_the_elementwise_formulation():
    # one-launch tracking kernels against minimal_i_given_xf / minimal_i_given_xb + max(i - decay, .), bit for bit
    from hgq2_b200 import kernels
    from hgq2_b200.quantizer.internal.fixed_point_quantizer import minimal_i_given_xb, minimal_i_given_xf

    rng = np.random.default_rng(8)
    n = 5000
    absmax = torch.from_numpy(np.abs(rng.standard_normal(n) * 10 ** rng.uniform(-4, 3, n)).astype(np.float32)).cuda()
    absmax[::97] = 0.0
    absmax[1::97] = 2.0 ** torch.from_numpy(rng.integers(-6, 7, absmax[1::97].numel()).astype(np.float32)).cuda()  # exact powers of two
    raw = torch.from_numpy((rng.integers(-3, 10, n) + rng.uniform(-0.4, 0.4, n)).astype(np.float32)).cuda()
    i0 = torch.from_numpy(rng.uniform(-4, 8, n).astype(np.float32)).cuda()
    decay = torch.tensor(0.01, device='cuda')
    # kif
    want = torch.maximum(i0 - decay, minimal_i_given_xf(absmax, torch.round(raw)))
    got = i0.clone()
    kernels.track_kif(absmax, raw, got, decay)
    assert torch.equal(got, want)
    # kbi, plain and symmetric, with and without a clamp
    for sym in (False, True):
        for lo, hi in ((float('-inf'), float('inf')), (-2.0, 5.0)):
            want = torch.clamp(torch.maximum(i0 - decay, minimal_i_given_xb(absmax, torch.round(raw), sym)), lo, hi)
            got = i0.clone()
            kernels.track_kbi(absmax, raw, got, decay, sym, lo, hi)
            assert torch.equal(torch.nan_to_num(got, nan=-777.0), torch.nan_to_num(want, nan=-777.0)), (sym, lo, hi)


def test_empty_inputs_are_no_ops():
    # zero elements (an empty batch): nothing is launched, empty results come back, reductions are zero
    from hgq2_b200 import kernels

    dev = 'cuda'
    f = torch.full((1, 7), 3.0, device=dev)
    k = torch.ones((1, 7), dtype=torch.uint8, device=dev)
    i = torch.full((1, 7), 2.0, device=dev)
    x = torch.empty((0, 7), device=dev)
    y, amax = kernels.quantize_fwd(x, k, i, f, 'RND', 'SAT', training=True, want_absmax=True)
    assert tuple(y.shape) == (0, 7) and float(amax.abs().sum()) == 0.0
    dx, di, df = kernels.quantize_bwd(x.clone(), x, k, i, f, 'RND', 'SAT')
    assert tuple(dx.shape) == (0, 7) and float(di.abs().sum()) == 0.0 and float(df.abs().sum()) == 0.0
    e = torch.empty(0, device=dev)
    ye = kernels.quantize_fwd(e, torch.empty(0, dtype=torch.uint8, device=dev), e, e, 'TRN', 'WRAP')
    assert ye.numel() == 0
