"""Properties that need no oracle, checked at the benchmark's FULL sizes (where the CPU oracle would take minutes): the
quantizer sweep's 2^28 elements, the particle layer's 4.19 M rows, the transformer's 134 M attention scores and its other
per-head products at batch 8192, the three convolution layers of the small CNN at batch 4096.

* idempotence and range membership of the quantizer; its backward passes the gradient or zero;
* shard invariance: a contiguous shard of the input gives the same bits as the same slice of the full result (what the
  multi-GPU sweep and the data-parallel step rely on), and reductions over the batch are the reductions of the shards;
* exact homogeneity under scaling by powers of two (weights and bias x 2 => outputs x 2; upstream gradient x 2 => every
  gradient x 2), which holds bit for bit in binary floating point when nothing over- or underflows;
* sampled outputs against the definition evaluated in float64 on the GPU (exact equality where the operands lie on grids
  coarse enough for fp32 sums to be exact).
"""

import pytest
import torch

pytestmark = pytest.mark.gpu

MODES = [(rm, om) for rm in ('RND', 'TRN') for om in ('WRAP', 'SAT', 'SAT_SYM')]


@pytest.fixture(scope='module')
def sweep_inputs():
    n = 1 << 28
    gen = torch.Generator(device='cuda').manual_seed(0)
    x = torch.randn(n, device='cuda', generator=gen) * 4
    k = torch.randint(0, 2, (n,), device='cuda', generator=gen, dtype=torch.uint8)
    i = torch.randint(-2, 7, (n,), device='cuda', generator=gen).float()
    f = torch.randint(0, 9, (n,), device='cuda', generator=gen).float()
    g = torch.randn(n, device='cuda', generator=gen)
    yield x, k, i, f, g
    del x, k, i, f, g
    torch.cuda.empty_cache()


@pytest.mark.parametrize('rm,om', MODES)
def test_quantizer_sweep_at_2_to_the_28(sweep_inputs, rm, om):
    from hgq2_b200 import kernels as K

    x, k, i, f, g = sweep_inputs
    n = x.numel()
    y = K.quantize_fwd(x, k, i, f, rm, om)
    # idempotence (where i + f >= 0: otherwise the range is narrower than one step) and range membership
    y2 = K.quantize_fwd(y, k, i, f, rm, om)
    nd = (i + f) >= 0
    assert torch.equal(torch.where(nd, y, y2), y2), 'idempotence'
    del y2
    hi = torch.exp2(i) - torch.exp2(-f)
    lo = -k.float() * (hi if om == 'SAT_SYM' else torch.exp2(i))
    assert bool(((y <= hi) & (y >= lo) | (hi < lo) | ~nd).all()), 'range'
    del hi, lo, nd
    # shard invariance: the second quarter alone
    a, b = n // 4, n // 2
    ys = K.quantize_fwd(x[a:b], k[a:b], i[a:b], f[a:b], rm, om)
    assert torch.equal(ys, y[a:b]), 'shard'
    del ys, y
    # backward: dx is g or 0 (or -g k for the wrapped lower edge of SAT_SYM's surrogate is not produced: straight-through),
    # and every gradient doubles exactly with the upstream gradient
    dx, di, df = K.quantize_bwd(g, x, k, i, f, rm, om)
    assert bool(((dx == g) | (dx == 0)).all()), 'dx is g or 0'
    g2 = g * 2
    dx2, di2, df2 = K.quantize_bwd(g2, x, k, i, f, rm, om)
    assert torch.equal(dx2, dx * 2) and torch.equal(df2, df * 2), 'homogeneity'
    if di is not None:
        assert torch.equal(di2, di * 2)


def test_particle_layer_at_4_million_rows():
    from hgq2_b200 import kernels as K

    M, Kd, N, rp = 65536 * 64, 64, 64, 64
    gen = torch.Generator(device='cuda').manual_seed(1)
    x = torch.randn(M, Kd, device='cuda', generator=gen) * 2
    f = torch.randint(2, 8, (rp, Kd), device='cuda', generator=gen).float()
    w = torch.randint(-128, 128, (Kd, N), device='cuda', generator=gen).float() / 64
    b = torch.randint(-16, 16, (N,), device='cuda', generator=gen).float() / 8
    y, amax, pooled = K.qdense_fwd(x, None, None, f, rp, 'RND', 'WRAP', True, False, w, b, 'relu', True, pool_rows=64)
    K.check_status(x.device)
    # weights and bias x 2 => outputs x 2, bit for bit; the statistic does not depend on them
    y2, amax2 = K.qdense_fwd(x, None, None, f, rp, 'RND', 'WRAP', True, False, w * 2, b * 2, 'relu', True)
    assert torch.equal(y2, y * 2) and torch.equal(amax2, amax)
    del y2
    # the sums over the 64 particles of a sample equal the sums of the y written
    assert torch.equal(pooled.double(), y.view(M // 64, 64, N).double().sum(dim=1))
    # shard invariance (the second half of the samples) and the statistic as the maximum over the shards
    h = M // 2
    ya, aa = K.qdense_fwd(x[:h], None, None, f, rp, 'RND', 'WRAP', True, False, w, b, 'relu', True)
    yb, ab = K.qdense_fwd(x[h:], None, None, f, rp, 'RND', 'WRAP', True, False, w, b, 'relu', True)
    assert torch.equal(ya, y[:h]) and torch.equal(yb, y[h:])
    assert torch.equal(torch.maximum(aa, ab), amax)
    del ya, yb
    # backward: shard invariance of dX; dWq, dbq, df of the whole batch = sums over the shards; exact doubling with dY
    gy = torch.randn(M, N, device='cuda', generator=gen)
    dx, dw, db, df = K.qdense_bwd(gy, y, x, f.view(-1), rp, 'RND', w, want_dx=True, want_db=True, want_df=True)
    dx, dw, db, df = dx.clone(), dw.clone(), db.clone(), df.clone()
    K.check_status(x.device)
    dxa, dwa, dba, dfa = (t.clone() for t in K.qdense_bwd(gy[:h], y[:h], x[:h], f.view(-1), rp, 'RND', w, True, True, True))
    dxb, dwb, dbb, dfb = (t.clone() for t in K.qdense_bwd(gy[h:], y[h:], x[h:], f.view(-1), rp, 'RND', w, True, True, True))
    assert torch.equal(dxa, dx[:h]) and torch.equal(dxb, dx[h:])
    for whole, parts, name in ((dw, dwa + dwb, 'dWq'), (db, dba + dbb, 'dbq'), (df, dfa + dfb, 'df')):
        err = float((whole - parts).abs().max() / whole.abs().max())
        assert err <= 2e-5, (name, err)  # bf16-term products summed in a different grouping
    del dxa, dxb
    dx2, dw2, db2, df2 = K.qdense_bwd(gy * 2, y, x, f.view(-1), rp, 'RND', w, want_dx=True, want_db=True, want_df=True)
    assert torch.equal(dx2, dx * 2) and torch.equal(dw2, dw * 2) and torch.equal(db2, db * 2) and torch.equal(df2, df * 2)


def test_attention_scores_at_134_million():
    from hgq2_b200 import kernels as K

    B, H, L, D, rp = 8192, 4, 64, 16, 256
    gen = torch.Generator(device='cuda').manual_seed(2)
    q = torch.randint(-512, 512, (B, L, H, D), device='cuda', generator=gen).float() / 64
    k = torch.randint(-512, 512, (B, L, H, D), device='cuda', generator=gen).float() / 64
    s = K.attn_heads_matmul(0, q, k, B, L, H, D)
    K.check_status(q.device)
    # a shard of the batch gives the same scores; scaling one operand by 2 doubles them
    assert torch.equal(K.attn_heads_matmul(0, q[B // 2:], k[B // 2:], B // 2, L, H, D), s[B // 2:])
    assert torch.equal(K.attn_heads_matmul(0, q * 2, k, B, L, H, D), s * 2)
    one = lambda v, dt=torch.float32: torch.full((1,), v, dtype=dt, device='cuda')
    k0 = one(0, torch.uint8)
    f5 = torch.randint(4, 10, (rp * L,), device='cuda', generator=gen).float()
    quants = [(k0, one(4.0), one(6.0), 'RND', 'SAT'), (k0, one(1.0), one(9.0), 'RND', 'SAT'), (None, None, one(3.0), 'RND', 'NONE'),
              (k0, one(1.0), one(9.0), 'RND', 'SAT'), (None, None, f5, 'RND', 'NONE')]
    s = s.view(B, rp, L)
    p, a3, a5, a1 = K.qsoftmax_fwd(s, quants, 0.25, 1e-7, rp, True, True, True)
    # probabilities: non-negative, at most 1 + one step of the coarsest output grid, invariant under a shift of a row
    assert float(p.min()) >= 0.0 and float(p.max()) <= 1.0 + 2.0 ** -4
    p_shift, *_ = K.qsoftmax_fwd(s + 8.0, quants, 0.25, 1e-7, rp, False, False, False)
    assert torch.equal(p_shift, p)  # the scores lie on a 2^-12 grid, so s + 8 is exact and max - s is unchanged
    del p_shift
    h = B // 2
    pa, a3a, a5a, a1a = K.qsoftmax_fwd(s[:h], quants, 0.25, 1e-7, rp, True, True, True)
    pb, a3b, a5b, a1b = K.qsoftmax_fwd(s[h:], quants, 0.25, 1e-7, rp, True, True, True)
    assert torch.equal(pa, p[:h]) and torch.equal(pb, p[h:])
    for whole, x1, x2 in ((a3, a3a, a3b), (a5, a5a, a5b), (a1, a1a, a1b)):
        assert torch.equal(torch.maximum(x1, x2), whole)
    del pa, pb
    g = torch.randn(B, rp, L, device='cuda', generator=gen)
    ds, sc, df5, _ = K.qsoftmax_bwd(g, s, quants, 0.25, 1e-7, rp, False)
    ds, sc, df5 = ds.clone(), sc.clone(), df5.clone()
    # rows of ds sum to ~0 where no quantizer clipped would be too strong a statement; shard invariance and doubling hold exactly
    dsa = K.qsoftmax_bwd(g[:h], s[:h], quants, 0.25, 1e-7, rp, False)[0]
    assert torch.equal(dsa, ds[:h])
    del dsa
    ds2, sc2, df52, _ = K.qsoftmax_bwd(g * 2, s, quants, 0.25, 1e-7, rp, False)
    assert torch.equal(ds2, ds * 2) and torch.equal(sc2, sc * 2) and torch.equal(df52, df5 * 2)


@pytest.mark.parametrize('H,C,N', [(32, 4, 16), (15, 16, 32), (6, 32, 64)])
def test_convolution_layers_at_batch_4096(H, C, N):
    """The three layers of the small CNN at the benchmark batch: forward, input gradient and weight gradient.
    Operands on coarse binary grids make every product and sum exact in fp32, so sampled outputs must EQUAL a float64
    evaluation of the definition, and shards / sums of shards must equal the whole bit for bit."""
    from hgq2_b200 import kernels as K

    B, OH = 4096, H - 2
    gen = torch.Generator(device='cuda').manual_seed(H)
    x = torch.randint(0, 32, (B, H, H, C), device='cuda', generator=gen).float() / 32          # 5-bit activations
    w = torch.randint(-64, 64, (3, 3, C, N), device='cuda', generator=gen).float() / 64        # 7-bit weights
    b = torch.randint(-8, 8, (N,), device='cuda', generator=gen).float() / 8
    y = K.qconv2d_fwd(x, w.reshape(-1, N), b, 'relu', 3, 3, (OH, OH), (1, 1), (1, 1), (0, 0))
    K.check_status(x.device)
    assert y.shape == (B, OH, OH, N)
    # sampled output pixels against the definition in float64
    n_s = 4096
    bi = torch.randint(0, B, (n_s,), device='cuda', generator=gen)
    oy = torch.randint(0, OH, (n_s,), device='cuda', generator=gen)
    ox = torch.randint(0, OH, (n_s,), device='cuda', generator=gen)
    dy, dx_ = torch.meshgrid(torch.arange(3, device='cuda'), torch.arange(3, device='cuda'), indexing='ij')
    patches = x[bi[:, None, None], oy[:, None, None] + dy, ox[:, None, None] + dx_]             # [n_s, 3, 3, C]
    ref = torch.einsum('sklc,klcn->sn', patches.double(), w.double()) + b.double()
    assert torch.equal(y[bi, oy, ox].double(), ref.clamp_min(0))
    # shard invariance
    h = B // 2
    assert torch.equal(K.qconv2d_fwd(x[h:].contiguous(), w.reshape(-1, N), b, 'relu', 3, 3, (OH, OH), (1, 1), (1, 1), (0, 0)), y[h:])
    # backward on an upstream gradient with 6 significant bits: masked gradient, weight / bias / input gradients
    gy = torch.randint(-32, 32, (B, OH, OH, N), device='cuda', generator=gen).float() / 32
    gm, dw, db = K.qconv2d_wgrad(x, gy, y, 3, 3, (1, 1), (1, 1), (0, 0), True)
    gm, dw, db = gm.clone(), dw.clone(), db.clone()
    K.check_status(x.device)
    assert torch.equal(gm, gy * (y > 0))
    assert torch.equal(db, gm.double().sum(dim=(0, 1, 2)).float())  # exact partial sums, one rounding to fp32 at the end
    _, dwa, dba = (t.clone() for t in K.qconv2d_wgrad(x[:h].contiguous(), gy[:h].contiguous(), y[:h].contiguous(), 3, 3, (1, 1),
                                                      (1, 1), (0, 0), True))
    _, dwb, dbb = K.qconv2d_wgrad(x[h:].contiguous(), gy[h:].contiguous(), y[h:].contiguous(), 3, 3, (1, 1), (1, 1), (0, 0), True)
    # sums of up to 3.7 M exact products exceed 24 bits: the whole and the sum of the shards agree to fp32 rounding
    err = float((dw - (dwa + dwb)).abs().max() / dw.abs().max())
    assert err <= 2e-6, err
    # one tap of the weight gradient against the definition in float64 (tap (1, 2))
    ref_tap = torch.einsum('bijc,bijn->cn', x[:, 1:1 + OH, 2:2 + OH].double(), gm.double())
    err = float((dw.view(3, 3, C, N)[1, 2].double() - ref_tap).abs().max() / ref_tap.abs().max())
    assert err <= 2e-6, err
    wt = w.flip(0, 1).permute(0, 1, 3, 2).reshape(9 * N, C).contiguous()
    dxg = K.qconv2d_fwd(gm, wt, None, None, 3, 3, (H, H), (1, 1), (1, 1), (2, 2))
    K.check_status(x.device)
    iy = torch.randint(0, H, (n_s,), device='cuda', generator=gen)
    ix = torch.randint(0, H, (n_s,), device='cuda', generator=gen)
    gp = torch.nn.functional.pad(gm, (0, 0, 2, 2, 2, 2))                                         # zeros around the gradient
    gpatch = gp[bi[:, None, None], iy[:, None, None] + 2 - dy, ix[:, None, None] + 2 - dx_]      # g[y - kh, x - kw]
    refx = torch.einsum('skln,klcn->sc', gpatch.double(), w.double())
    assert torch.equal(dxg[bi, iy, ix].double(), refx)
    assert torch.equal(K.qconv2d_fwd(gm[h:].contiguous(), wt, None, None, 3, 3, (H, H), (1, 1), (1, 1), (2, 2)), dxg[h:])


def test_attention_products_at_batch_8192():
    """context = P V, dQ = dS K and dV = P^T dO at the transformer's full batch: sampled heads against float64, shards and
    exact doubling."""
    from hgq2_b200 import kernels as K

    B, H, L, D = 8192, 4, 64, 16
    gen = torch.Generator(device='cuda').manual_seed(3)
    v = torch.randint(-512, 512, (B, L, H, D), device='cuda', generator=gen).float() / 64       # 10-bit projections
    p = torch.randint(0, 256, (B, H, L, L), device='cuda', generator=gen).float() / 256         # 8-bit probabilities
    g = torch.randn(B, H, L, L, device='cuda', generator=gen)
    sb = torch.randint(0, B, (64,), device='cuda', generator=gen)
    h = B // 2
    ctx = K.attn_heads_matmul(1, p, v, B, L, H, D)                                               # [B, L, H, D]
    K.check_status(v.device)
    ref = torch.einsum('bhts,bshd->bthd', p[sb].double(), v[sb].double())
    assert torch.equal(ctx[sb].double(), ref)  # 8-bit x 10-bit products, 64 terms: exact in fp32
    assert torch.equal(K.attn_heads_matmul(1, p[h:], v[h:], h, L, H, D), ctx[h:])
    assert torch.equal(K.attn_heads_matmul(1, p, v * 2, B, L, H, D), ctx * 2)
    dq = K.attn_heads_matmul(1, g, v, B, L, H, D)                                                # fp32 left operand
    ref = torch.einsum('bhts,bshd->bthd', g[sb].double(), v[sb].double())
    err = float((dq[sb].double() - ref).abs().max() / ref.abs().max())
    assert err <= 2e-5, err  # two bf16 terms of the gradient: 16 significant bits
    assert torch.equal(K.attn_heads_matmul(1, g[h:], v[h:], h, L, H, D), dq[h:])
    assert torch.equal(K.attn_heads_matmul(1, g * 2, v, B, L, H, D), dq * 2)
    dv = K.attn_heads_matmul(2, g, v, B, L, H, D)                                                # G^T V: [B, L, H, D]
    K.check_status(v.device)
    ref = torch.einsum('bhts,bthd->bshd', g[sb].double(), v[sb].double())
    err = float((dv[sb].double() - ref).abs().max() / ref.abs().max())
    assert err <= 2e-5, err
    assert torch.equal(K.attn_heads_matmul(2, g[h:], v[h:], h, L, H, D), dv[h:])
    assert torch.equal(K.attn_heads_matmul(2, g * 2, v, B, L, H, D), dv * 2)
