"""EBOPs of several dense layers in one launch (hgq_ebops_dense_batch) against the per-layer kernel and the definition."""

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_batched_dense_ebops_equal_the_per_layer_kernel():
    from hgq2_b200 import kernels as K

    rng = np.random.default_rng(0)
    dev = torch.device('cuda')
    shapes = [(1, 16, 64), (1, 64, 32), (64, 16, 64), (1, 300, 7), (3, 5, 5)] * 4  # 20 layers: two launches of at most 16
    items, singles, defs = [], [], []
    for j, (P, Kd, N) in enumerate(shapes):
        bw_in = torch.from_numpy(rng.integers(0, 9, (P, Kd)).astype(np.float32)).to(dev)
        bw_w = torch.from_numpy(rng.integers(0, 7, (Kd, N)).astype(np.float32)).to(dev)
        bw_b = torch.from_numpy(rng.integers(0, 7, (N,)).astype(np.float32)).to(dev) if j % 3 else None
        beta = torch.tensor(1e-3 * (j + 1), device=dev)
        out_size, scale = float(P * N), 0.5 + j
        out = (torch.zeros((), dtype=torch.uint32, device=dev), torch.zeros((), device=dev), torch.zeros_like(bw_in),
               torch.zeros_like(bw_w), None if bw_b is None else torch.zeros_like(bw_b))
        items.append((bw_in, bw_w, bw_b, out_size, scale, beta, out))
        singles.append(K.ebops_dense(bw_in, bw_w, bw_b, out_size, scale, beta))
        e = scale * (float((bw_in.double().sum(0) * bw_w.double().sum(1)).sum()) + (float(bw_b.double().mean()) * out_size if bw_b is not None else 0.0))
        defs.append(e)
    K.ebops_dense_batch(items)
    torch.cuda.synchronize()
    for (e_u, e_f, loss, d_in, d_w, d_b), item, e in zip(singles, items, defs):
        b_u, b_loss, b_in, b_w, b_b = item[6]
        assert int(b_u.item()) == int(e_u.item()) == int(e)
        assert torch.equal(b_loss, loss) and torch.equal(b_in, d_in) and torch.equal(b_w, d_w)
        if b_b is not None:
            assert torch.equal(b_b, d_b)


def test_batched_dense_ebops_argument_errors():
    from hgq2_b200 import _lib

    L = _lib.lib()
    arr = (_lib.EbopsDenseDesc * 1)()
    assert L.hgq_ebops_dense_batch(None, 1, None) == -1
    assert L.hgq_ebops_dense_batch(arr, 0, None) == -2 and L.hgq_ebops_dense_batch(arr, 17, None) == -2
    assert L.hgq_ebops_dense_batch(arr, 1, None) == -2  # P = K = N = 0
