"""The fused quantise -> tensor-core GEMM -> bias/activation kernel against the oracle's op sequence."""

import numpy as np
import pytest
import torch

from oracle import fixed_point_ops as O

pytestmark = pytest.mark.gpu


def _ref(x, k, i, f, rm, om, training, w, b, act, rows_period):
    M, K = x.shape
    rep = M // rows_period + 1
    kk, ii, ff = (t.repeat(rep, 1)[:M] for t in (k.float(), i, f))
    xq = O.quantize_fwd(x, kk, ii, ff, rm, om, training)
    y = (xq.double() @ w.double())
    if b is not None:
        y = y + b.double()
    if act == 'relu':
        y = torch.relu(y)
    amax = torch.zeros(rows_period, K)
    r = O.round_fwd(x, ff, rm).abs()
    for p in range(rows_period):
        amax[p] = r[p::rows_period].amax(0)
    return y, amax


@pytest.mark.parametrize('M,K,N,rows_period', [
    (1000, 16, 64, 1), (128 * 37 + 5, 64, 64, 64), (4096, 64, 32, 1), (513, 32, 5, 1), (300, 27, 16, 1),
    (2048, 128, 64, 64), (640, 64, 128, 8), (129, 64, 10, 3), (7, 16, 64, 1), (50000, 64, 64, 1), (3000, 144, 32, 1),
    (300, 1152, 12, 1), (500, 784, 32, 1),  # a classifier head behind a Flatten
])
@pytest.mark.parametrize('rm,om,training', [('RND', 'WRAP', True), ('TRN', 'SAT', True), ('RND', 'WRAP', False)])
def test_fused_dense_forward(M, K, N, rows_period, rm, om, training):
    from hgq2_b200 import kernels

    rng = np.random.default_rng(M + K + N)
    x = torch.from_numpy((rng.standard_normal((M, K)) * 3).astype(np.float32))
    k = torch.from_numpy(rng.integers(0, 2, (rows_period, K)).astype(np.uint8))
    i = torch.from_numpy(rng.integers(0, 4, (rows_period, K)).astype(np.float32))
    f = torch.from_numpy(rng.integers(1, 7, (rows_period, K)).astype(np.float32))
    w = torch.from_numpy(np.round(rng.uniform(-2, 2, (K, N)) * 64) / 64).float()   # 8-bit weights
    b = torch.from_numpy(np.round(rng.standard_normal(N) * 16) / 16).float()
    for act in (None, 'relu'):
        y, amax = kernels.qdense_fwd(x.cuda(), k.cuda(), i.cuda(), f.cuda(), rows_period, rm, om, training, False, w.cuda(),
                                     b.cuda(), act, True)
        kernels.check_status(y.device)
        yr, ar = _ref(x, k, i, f, rm, om, training, w, b, act, rows_period)
        err = (y.cpu().double() - yr).abs().max() / max(float(yr.abs().max()), 1e-30)
        assert err <= 2e-7, f'act={act}: relative error {err:.3e}'
        assert torch.equal(amax.cpu().view(rows_period, K), ar), 'absmax'


@pytest.mark.parametrize('M,K,N,pool_rows,rows_period', [
    (64 * 301, 16, 64, 64, 64),    # the particle layers: 64 particles per sample; the last tile holds one sample
    (64 * 300, 64, 64, 64, 64),
    (32 * 77, 32, 64, 32, 32),     # a group per epilogue warp
    (128 * 9, 64, 128, 128, 1),    # a group per tile, two column pieces per epilogue warp
    (64 * 10, 64, 36, 64, 64),     # padded output columns
])
def test_fused_dense_forward_with_row_group_sums(M, K, N, pool_rows, rows_period):
    """hgq_qdense_fwd_pooled: the sums over groups of consecutive rows come out of the forward kernel and equal the sums
    of the y it writes (exactly for quantised operands: every partial sum is exact in fp32), scaled as asked."""
    import os

    from hgq2_b200 import kernels

    # the sums are taken from the blocks of the warp-specialised kernel's bulk-store path: with that path switched off in
    # the environment (the child-process runs below) the query must say no, and callers keep their separate reduction
    on = os.environ.get('HGQ_QDENSE_WS', '1') != '0' and os.environ.get('HGQ_QDENSE_TMA_STORE', '1') != '0'
    assert kernels.qdense_pooled_supported(M, K, N, rows_period, pool_rows) == on
    assert not kernels.qdense_pooled_supported(M + 4, K, N, rows_period, pool_rows)  # groups must tile the rows
    if not on:
        return
    rng = np.random.default_rng(M + N)
    x = torch.from_numpy((rng.standard_normal((M, K)) * 3).astype(np.float32)).cuda()
    f = torch.from_numpy(rng.integers(1, 7, (rows_period, K)).astype(np.float32)).cuda()
    w = torch.from_numpy(np.round(rng.uniform(-2, 2, (K, N)) * 64) / 64).float().cuda()
    b = torch.from_numpy(np.round(rng.standard_normal(N) * 16) / 16).float().cuda()
    for act, scale in ((None, 1.0), ('relu', 1.0 / pool_rows)):
        y0, a0 = kernels.qdense_fwd(x, None, None, f, rows_period, 'RND', 'WRAP', True, False, w, b, act, True)
        y, a, pooled = kernels.qdense_fwd(x, None, None, f, rows_period, 'RND', 'WRAP', True, False, w, b, act, True,
                                          pool_rows=pool_rows, pool_scale=scale)
        kernels.check_status(y.device)
        assert torch.equal(y, y0) and torch.equal(a, a0)
        want = y.view(M // pool_rows, pool_rows, N).double().sum(dim=1) * scale
        assert pooled.shape == (M // pool_rows, N)
        assert torch.equal(pooled.double(), want), float((pooled.double() - want).abs().max())


def test_fused_dense_is_exact_for_wide_values():
    # operands that need two and three bf16 terms: 14-bit activations, 12- and 20-bit weights
    from hgq2_b200 import kernels

    rng = np.random.default_rng(0)
    M, K, N = 1024, 64, 64
    x = torch.from_numpy((rng.standard_normal((M, K)) * 20).astype(np.float32))
    f = torch.full((1, K), 8.0)
    for wbits in (6, 12, 20):
        w = torch.from_numpy(np.round(rng.uniform(-1, 1, (K, N)) * 2**wbits) / 2**wbits).float()
        y, _ = kernels.qdense_fwd(x.cuda(), None, None, f.cuda(), 1, 'RND', 'WRAP', True, False, w.cuda(), None, None, False)
        kernels.check_status(y.device)
        xq = O.round_fwd(x, f.expand(M, K), 'RND')
        yr = xq.double() @ w.double()
        err = (y.cpu().double() - yr).abs().max() / float(yr.abs().max())
        # 14-bit x wbits-bit products summed over 64 terms need more than fp32's 24 bits once wbits > 4: the sum is
        # then rounded (by the reference too); the split operands themselves stay exact
        assert err <= (2e-7 if wbits <= 6 else 1e-6), (wbits, float(err))


def test_fused_dense_activations_beyond_two_terms():
    # quantised activations with more than 16 significant bits appear only in some tiles, late in a CTA's sequence of
    # tiles and in single elements: the third bf16 term must be picked up exactly where it is needed.  Every sum here
    # is exact in fp32 (one wide value per row, weights are powers of two), so the comparison is bit for bit.
    from hgq2_b200 import kernels

    rng = np.random.default_rng(5)
    M, K, N = 128 * 400 + 17, 64, 32
    x = torch.from_numpy(np.round(rng.standard_normal((M, K)) * 4).astype(np.float32))  # integers: few bits
    wide = torch.from_numpy((rng.standard_normal(M) * 20).astype(np.float32))
    col = torch.from_numpy(rng.integers(0, K, M))
    rows = torch.cat([torch.arange(128 * 200, 128 * 260), torch.tensor([128 * 300 + 5, M - 3])])
    x[rows] = 0.0
    x[rows, col[rows]] = wide[rows]
    f = torch.full((1, K), 20.0)
    w = torch.from_numpy(rng.choice([-1.0, 1.0], (K, N)) * 2.0 ** -rng.integers(0, 7, (K, N))).float()
    y, amax = kernels.qdense_fwd(x.cuda(), None, None, f.cuda(), 1, 'RND', 'WRAP', True, False, w.cuda(), None, None, True)
    kernels.check_status(y.device)
    xq = O.round_fwd(x, f.expand(M, K), 'RND')
    assert int((xq[rows].view(torch.int32) & 0xff).ne(0).sum()) > 1000  # the wide rows do need a third term
    yr = (xq.double() @ w.double()).float()
    assert torch.equal(y.cpu(), yr)
    assert torch.equal(amax.cpu().view(1, K), xq.abs().amax(0, keepdim=True))


def test_fused_dense_no_input_quantizer_and_limits():
    from hgq2_b200 import _lib, kernels

    rng = np.random.default_rng(1)
    x = torch.from_numpy(rng.standard_normal((300, 48)).astype(np.float32))
    w = torch.from_numpy(rng.standard_normal((48, 24)).astype(np.float32))
    y, _ = kernels.qdense_fwd(x.cuda(), None, None, None, 1, 'RND', 'WRAP', True, False, w.cuda(), None, None, False)
    kernels.check_status(y.device)
    yr = x.double() @ w.double()
    assert float((y.cpu().double() - yr).abs().max() / yr.abs().max()) <= 1e-6  # full-width operands: fp32 rounding of the sum
    # limits: at most 128 outputs; inputs as far as the weight terms fit shared memory beside the tile buffers
    assert kernels.qdense_supported(100, 300, 64, 1) and kernels.qdense_supported(100, 1152, 16, 1)
    assert not kernels.qdense_supported(100, 600, 64, 1)
    assert not kernels.qdense_supported(100, 64, 200, 1)
    L = _lib.lib()
    assert L.hgq_qdense_fwd(1, None, None, None, 1, 1, 1, 0, 1, None, 0, 1, None, 100, 600, 64, None, 0, None, None) == -2


@pytest.mark.parametrize('M,K,N,rows_period', [
    (1000, 16, 64, 1), (128 * 21 + 5, 64, 64, 64), (4096, 64, 32, 1), (513, 32, 5, 1), (300, 24, 16, 8), (640, 64, 128, 32),
    (129, 27, 10, 1), (7, 16, 64, 1), (60000, 64, 64, 64), (2000, 48, 40, 2), (3000, 128, 64, 64), (700, 96, 32, 1),
    (128 * 50 + 9, 64, 128, 64),  # 128 outputs
    (300, 1152, 12, 1), (500, 784, 32, 1),  # a classifier head behind a Flatten: 18 / 13 blocks of 64 inputs
])
@pytest.mark.parametrize('rm,relu,quant', [('RND', True, True), ('TRN', False, True), ('RND_CONV', True, True), ('RND', True, False)])
def test_fused_dense_backward(M, K, N, rows_period, rm, relu, quant):
    from hgq2_b200 import kernels

    rng = np.random.default_rng(M + 3 * K + N)
    x = torch.from_numpy((rng.standard_normal((M, K)) * 3).astype(np.float32))
    f = torch.from_numpy(rng.integers(1, 7, (rows_period, K)).astype(np.float32))
    w = torch.from_numpy(np.round(rng.uniform(-2, 2, (K, N)) * 64) / 64).float()
    gy = torch.from_numpy(rng.standard_normal((M, N)).astype(np.float32))
    y = torch.from_numpy(rng.standard_normal((M, N)).astype(np.float32)).clamp_min(0)
    dx, dwq, dbq, df = kernels.qdense_bwd(gy.cuda(), y.cuda() if relu else None, x.cuda(), f.cuda() if quant else None, rows_period,
                                          rm, w.cuda(), True, True, quant)
    kernels.check_status(dx.device)
    # reference in float64 from the oracle's definitions
    g = (gy * (y > 0)) if relu else gy
    rep = M // rows_period + 1
    ff = f.repeat(rep, 1)[:M]
    xq = O.round_fwd(x, ff, rm) if quant else x
    dxr = g.double() @ w.double().t()
    dwr = xq.double().t() @ g.double()
    dbr = g.double().sum(0)

    def rel(a, b):
        return float((a.cpu().double() - b).abs().max() / max(float(b.abs().max()), 1e-30))

    assert rel(dx, dxr) <= 2e-5, ('dx', rel(dx, dxr))
    assert rel(dwq, dwr) <= 5e-5, ('dwq', rel(dwq, dwr))
    assert rel(dbq, dbr) <= 5e-5, ('dbq', rel(dbq, dbr))
    if quant:
        t = ((xq - x).double() * (-O.LN2)) * dxr
        dfr = torch.stack([t[p::rows_period].sum(0) for p in range(rows_period)])
        assert rel(df.view(rows_period, K), dfr) <= 5e-5, ('df', rel(df.view(rows_period, K), dfr))


def test_fused_dense_backward_is_deterministic():
    from hgq2_b200 import kernels

    rng = np.random.default_rng(0)
    M, K, N = 50000, 64, 64
    x = torch.from_numpy((rng.standard_normal((M, K)) * 3).astype(np.float32)).cuda()
    f = torch.full((64, K), 5.0).cuda()
    w = torch.from_numpy(np.round(rng.uniform(-2, 2, (K, N)) * 64) / 64).float().cuda()
    gy = torch.from_numpy(rng.standard_normal((M, N)).astype(np.float32)).cuda()
    a = kernels.qdense_bwd(gy, None, x, f, 64, 'RND', w, True, True, True)
    b = kernels.qdense_bwd(gy, None, x, f, 64, 'RND', w, True, True, True)
    for u, v in zip(a, b):
        assert torch.equal(u, v)


def test_fused_dense_backward_with_repeated_gradient_rows():
    # the gradient of a sum over an axis: one stored row of dY per group of 64 rows, read in place
    from hgq2_b200 import kernels

    rng = np.random.default_rng(5)
    B, P, K, N = 37, 64, 64, 64
    M = B * P
    x = torch.from_numpy((rng.standard_normal((M, K)) * 3).astype(np.float32)).cuda()
    f = torch.from_numpy(rng.integers(1, 7, (P, K)).astype(np.float32)).cuda()
    w = torch.from_numpy(np.round(rng.uniform(-2, 2, (K, N)) * 64) / 64).float().cuda()
    g = torch.from_numpy(rng.standard_normal((B, N)).astype(np.float32)).cuda()
    y = torch.from_numpy(rng.standard_normal((M, N)).astype(np.float32)).cuda()
    full = g.unsqueeze(1).expand(B, P, N).reshape(M, N).contiguous()
    ref = kernels.qdense_bwd(full, y, x, f, P, 'RND', w, True, True, True)
    got = kernels.qdense_bwd(g, y, x, f, P, 'RND', w, True, True, True, gy_repeat=P)
    kernels.check_status(x.device)
    for a, b in zip(got, ref):
        assert torch.equal(a, b)


def test_general_forward_kernel_on_the_same_cases():
    # HGQ_QDENSE_WS=0 (read once per process) keeps every forward call on the general kernel: the forward cases above are
    # run again in a child process so that both kernels stay covered by the same references
    import os
    import subprocess
    import sys

    env = dict(os.environ, HGQ_QDENSE_WS='0')
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, '-m', 'pytest', os.path.join(root, 'tests', 'test_qdense_gpu.py'), '-q', '-x', '-m', 'gpu',
                        '-k', 'test_fused_dense_forward or beyond_two_terms or wide_values', '-p', 'no:cacheprovider'],
                       cwd=root, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]


@pytest.mark.parametrize('M,K,N,rows_period,relu,want_dx', [
    (128 * 300 + 77, 32, 64, 128, True, True), (5000, 64, 16, 4, False, True), (128 * 150, 16, 32, 16, True, False),
    (9, 64, 64, 1, True, True), (128 * 149 + 1, 20, 28, 2, True, True),
])
def test_warp_specialised_backward_shapes(M, K, N, rows_period, relu, want_dx):
    """Shapes inside the warp-specialised backward kernel's cover (K, N multiples of 4 padding to 16 / 32 / 64): several
    tiles per CTA, a ragged last tile, padded columns, no input gradient wanted."""
    from hgq2_b200 import kernels

    rng = np.random.default_rng(M + K + N)
    x = torch.from_numpy((rng.standard_normal((M, K)) * 3).astype(np.float32))
    f = torch.from_numpy(rng.integers(1, 7, (rows_period, K)).astype(np.float32))
    w = torch.from_numpy(np.round(rng.uniform(-2, 2, (K, N)) * 64) / 64).float()
    gy = torch.from_numpy(rng.standard_normal((M, N)).astype(np.float32))
    y = torch.from_numpy(rng.standard_normal((M, N)).astype(np.float32)).clamp_min(0)
    dx, dwq, dbq, df = kernels.qdense_bwd(gy.cuda(), y.cuda() if relu else None, x.cuda(), f.cuda(), rows_period, 'RND', w.cuda(),
                                          want_dx, True, True)
    kernels.check_status(dwq.device)
    g = (gy * (y > 0)) if relu else gy
    ff = f.repeat(M // rows_period + 1, 1)[:M]
    xq = O.round_fwd(x, ff, 'RND')
    dxr = g.double() @ w.double().t()

    def rel(a, b):
        return float((a.cpu().double() - b).abs().max() / max(float(b.abs().max()), 1e-30))

    assert (dx is None) == (not want_dx)
    if want_dx:
        assert rel(dx, dxr) <= 2e-5
    assert rel(dwq, xq.double().t() @ g.double()) <= 5e-5
    assert rel(dbq, g.double().sum(0)) <= 5e-5
    t = ((xq - x).double() * (-O.LN2)) * dxr
    dfr = torch.stack([t[p::rows_period].sum(0) for p in range(rows_period)])
    assert rel(df.view(rows_period, K), dfr) <= 5e-5


@pytest.mark.parametrize('M,K,N,rows_period,relu', [(128 * 40 + 17, 64, 64, 64, False), (4096, 16, 64, 1, True), (777, 32, 16, 4, True)])
def test_backward_adds_its_input_gradient_in_place(M, K, N, rows_period, relu):
    """hgq_qdense_bwd_accumulate: dx += the layer's input gradient (what layers that share an input need), every other
    output as without the flag."""
    import os

    from hgq2_b200 import kernels

    on = os.environ.get('HGQ_QDENSE_BWD_WS', '1') != '0'
    assert kernels.qdense_bwd_accumulates(K, N, rows_period, relu) == on
    assert not kernels.qdense_bwd_accumulates(K, 10, rows_period, relu)  # widths the warp-specialised kernel does not cover
    if not on:
        return
    gen = torch.Generator(device='cuda').manual_seed(M)
    x = torch.randn(M, K, device='cuda', generator=gen) * 2
    f = torch.randint(2, 7, (rows_period, K), device='cuda', generator=gen).float()
    w = torch.randint(-64, 64, (K, N), device='cuda', generator=gen).float() / 32
    y = torch.randn(M, N, device='cuda', generator=gen) if relu else None
    gy = torch.randn(M, N, device='cuda', generator=gen)
    dx, dw, db, df = (t.clone() for t in kernels.qdense_bwd(gy, y, x, f.view(-1), rows_period, 'RND', w, True, True, True))
    base = torch.randn(M, K, device='cuda', generator=gen)
    acc = base.clone()
    dx2, dw2, db2, df2 = kernels.qdense_bwd(gy, y, x, f.view(-1), rows_period, 'RND', w, True, True, True, dx_into=acc)
    kernels.check_status(x.device)
    assert dx2.data_ptr() == acc.data_ptr()
    assert torch.equal(acc, base + dx)
    assert torch.equal(dw2, dw) and torch.equal(db2, db) and torch.equal(df2, df)


def test_general_backward_kernel_on_the_same_cases():
    # HGQ_QDENSE_BWD_WS=0 (read once per process) keeps every backward call on the general kernel: the backward cases
    # above run again in a child process so that both kernels stay covered by the same references
    import os
    import subprocess
    import sys

    env = dict(os.environ, HGQ_QDENSE_BWD_WS='0')
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, '-m', 'pytest', os.path.join(root, 'tests', 'test_qdense_gpu.py'), '-q', '-x', '-m', 'gpu',
                        '-k', 'backward and not general', '-p', 'no:cacheprovider'],
                       cwd=root, env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]


def test_cp_async_variants_on_the_same_cases():
    # HGQ_QDENSE_TMA=0 / HGQ_QDENSE_BWD_TMA=0 / HGQ_QDENSE_TMA_STORE=0 (read once per process) keep the warp-specialised kernels
    # on their cp.async fetch and their transposition-buffer stores instead of the bulk tensor copies: forward and backward cases run again in a child process, so that both ways
    # of fetching stay covered by the same references
    import os
    import subprocess
    import sys

    env = dict(os.environ, HGQ_QDENSE_TMA='0', HGQ_QDENSE_BWD_TMA='0', HGQ_QDENSE_TMA_STORE='0')
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, '-m', 'pytest', os.path.join(root, 'tests', 'test_qdense_gpu.py'), '-q', '-x', '-m', 'gpu',
                        '-k', 'not general and not cp_async', '-p', 'no:cacheprovider'],
                       cwd=root, env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
