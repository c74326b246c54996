"""The entry point for callers that cannot allocate device memory, hgq_quantize_bwd_noalloc.

Such callers (a plugin living inside a framework whose pool owns the GPU, a service with a fixed memory
budget) cannot hand the broadcast-layout backward a workspace, so the library keeps the scratch in a fixed
device array.  The test calls the entry through the C ABI twice in a row, with different shapes so that the
second call runs over the first call's leftovers, and requires exactly the outputs of the workspace-taking
entry (same kernels, fixed reduction order: the results are bit-identical).  It also checks the size limit.
This file sorts last on purpose: a run that stops at the first failure has then run every other test.
"""

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

MODES = {'TRN': 0, 'RND': 1}
OVF = {'WRAP': 1, 'SAT': 2, 'SAT_SYM': 3}


def _case(rows, period, seed):
    rng = np.random.default_rng(seed)
    x = torch.from_numpy((rng.standard_normal((rows, period)) * 4).astype(np.float32)).cuda()
    g = torch.from_numpy(rng.standard_normal((rows, period)).astype(np.float32)).cuda()
    k = torch.from_numpy(rng.integers(0, 2, period).astype(np.uint8)).cuda()
    i = torch.from_numpy(rng.integers(-1, 4, period).astype(np.float32)).cuda()
    f = torch.from_numpy(rng.integers(0, 7, period).astype(np.float32)).cuda()
    return g, x, k, i, f


def _run(entry, g, x, k, i, f, rm, om, ws=None):
    from hgq2_b200 import _lib

    L = _lib.lib()
    n, period = x.numel(), f.numel()
    dx = torch.full_like(x, float('nan'))
    di = torch.full((period,), float('nan'), device=x.device)
    df = torch.full((period,), float('nan'), device=x.device)
    st = _lib.stream_handle()
    if entry == 'noalloc':
        rc = L.hgq_quantize_bwd_noalloc(g.data_ptr(), x.data_ptr(), k.data_ptr(), i.data_ptr(), f.data_ptr(), dx.data_ptr(),
                                        di.data_ptr(), df.data_ptr(), n, period, rm, om, 0, st)
    else:
        rc = L.hgq_quantize_bwd(g.data_ptr(), x.data_ptr(), k.data_ptr(), i.data_ptr(), f.data_ptr(), dx.data_ptr(),
                                di.data_ptr(), df.data_ptr(), n, period, rm, om, 0, ws.data_ptr(), ws.numel(), st)
    assert rc == 0, _lib.lib().hgq_status_string(rc)
    torch.cuda.synchronize()
    return dx, di, df


def test_noalloc_matches_workspace_entry_on_two_calls_in_a_row():
    from hgq2_b200 import _lib

    L = _lib.lib()
    # second shape is smaller and differently tiled than the first: stale partials of call 1 lie beyond and between
    # the words call 2 writes
    shapes = [(4099, 96), (777, 20)]
    combos = [(MODES['RND'], OVF['SAT']), (MODES['TRN'], OVF['SAT_SYM'])]
    for (rows, period), (rm, om), seed in zip(shapes, combos, (1, 2)):
        g, x, k, i, f = _case(rows, period, seed)
        need = L.hgq_quantize_bwd_workspace(x.numel(), period)
        assert 0 < need <= (8 << 20)
        ws = torch.empty(need, dtype=torch.uint8, device='cuda')
        ref = _run('workspace', g, x, k, i, f, rm, om, ws)
        got = _run('noalloc', g, x, k, i, f, rm, om)
        for name, a, b in zip(('dx', 'di', 'df'), got, ref):
            assert not torch.isnan(a).any(), name
            assert torch.equal(a, b), f'{name} differs from hgq_quantize_bwd for shape {(rows, period)}'


def test_noalloc_full_layout_and_limit():
    from hgq2_b200 import _lib

    L = _lib.lib()
    # full layout: no scratch involved, any size goes through
    g, x, k, i, f = _case(1, 5000, 3)
    ref = _run('workspace', g, x, k, i, f, 1, 2, torch.empty(16, dtype=torch.uint8, device='cuda'))
    got = _run('noalloc', g, x, k, i, f, 1, 2)
    for a, b in zip(got, ref):
        assert torch.equal(a, b)
    # a shape whose partials exceed the built-in scratch is refused before anything is launched
    rows, period = 4096, 1 << 16
    assert L.hgq_quantize_bwd_workspace(rows * period, period) > (8 << 20)
    before = L.hgq_launch_count()
    rc = L.hgq_quantize_bwd_noalloc(1, 1, 1, 1, 1, 1, 1, 1, rows * period, period, 1, 2, 0, None)
    assert rc == -2 and L.hgq_launch_count() == before
