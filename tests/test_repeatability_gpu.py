"""Launch-to-launch repeatability: the same inputs give the same bits on every launch (all reductions are done in fixed
orders; abs-max statistics are order-independent), for the tensor-core kernels and the fused softmax."""

import pytest
import torch

pytestmark = pytest.mark.gpu

REPEATS = 25


def _same(fn):
    first = [t.clone() for t in fn()]
    for _ in range(REPEATS):
        for a, b in zip(first, fn()):
            assert torch.equal(a, b)


def test_dense_forward_and_backward_repeat_bit_for_bit():
    from hgq2_b200 import kernels as K

    gen = torch.Generator(device='cuda').manual_seed(0)
    M, Kd, N, rp = 128 * 700 + 64, 64, 64, 64
    x = torch.randn(M, Kd, device='cuda', generator=gen) * 2
    f = torch.randint(2, 8, (rp, Kd), device='cuda', generator=gen).float()
    w = torch.randint(-128, 128, (Kd, N), device='cuda', generator=gen).float() / 64
    b = torch.randint(-16, 16, (N,), device='cuda', generator=gen).float() / 8
    gy = torch.randn(M, N, device='cuda', generator=gen)
    y, _, _ = K.qdense_fwd(x, None, None, f, rp, 'RND', 'WRAP', True, False, w, b, 'relu', True, pool_rows=64)
    y = y.clone()
    _same(lambda: K.qdense_fwd(x, None, None, f, rp, 'RND', 'WRAP', True, False, w, b, 'relu', True, pool_rows=64))
    _same(lambda: K.qdense_bwd(gy, y, x, f.view(-1), rp, 'RND', w, want_dx=True, want_db=True, want_df=True))
    K.check_status(x.device)


def test_attention_products_and_softmax_repeat_bit_for_bit():
    from hgq2_b200 import kernels as K

    gen = torch.Generator(device='cuda').manual_seed(1)
    B, L, H, D, rp = 512, 64, 4, 16, 256
    q = torch.randint(-512, 512, (B, L, H, D), device='cuda', generator=gen).float() / 64
    k = torch.randint(-512, 512, (B, L, H, D), device='cuda', generator=gen).float() / 64
    g = torch.randn(B, H, L, L, device='cuda', generator=gen)
    go = torch.randn(B, L, H, D, device='cuda', generator=gen)
    for kind, a, b in ((0, q, k), (0, go, k), (1, g, k), (2, g, q), (2, g, go)):
        _same(lambda: (K.attn_heads_matmul(kind, a, b, B, L, H, D),))
    one = lambda v, dt=torch.float32: torch.full((1,), v, dtype=dt, device='cuda')
    k0 = one(0, torch.uint8)
    quants = [(k0, one(4.0), one(6.0), 'RND', 'SAT'), (k0, one(1.0), one(9.0), 'RND', 'SAT'), (None, None, one(3.0), 'RND', 'NONE'),
              (k0, one(1.0), one(9.0), 'RND', 'SAT'), (None, None, torch.full((rp * L,), 8.0, device='cuda'), 'RND', 'NONE')]
    s = torch.round(torch.randn(B, rp, L, device='cuda', generator=gen) * 3 * 64) / 64
    gs = torch.randn(B, rp, L, device='cuda', generator=gen)
    _same(lambda: K.qsoftmax_fwd(s, quants, 0.25, 1e-7, rp, True, True, True))
    _same(lambda: K.qsoftmax_bwd(gs, s, quants, 0.25, 1e-7, rp, False)[:3])
    K.check_status(s.device)
