"""Host-side logic of the data-parallel QAT step on CPU ranks (gloo, world_size 2): batch sharding, the flat
gradient bucket and its averaging, and the MAX exchange of abs-max statistics.  No kernel runs here; the model
is a plain torch module standing in for the quantised layers."""

import os
import socket
import sys
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


def _free_port():
    with socket.socket() as s:
        s.bind(('127.0.0.1', 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out):
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port))
    dist.init_process_group('gloo', rank=rank, world_size=world)
    try:
        from hgq2_b200.backend import Layer, set_default_device
        from hgq2_b200.constraints import MinMax
        from hgq2_b200.quantizer.internal import fixed_point_quantizer as fpq
        from hgq2_b200.regularizers import MonoL1
        from hgq2_b200.train import DataParallel, FlatState, shard_batch

        set_default_device('cpu')

        class Toy(Layer):
            def build(self, shape):
                self.w = self.add_weight(name='w', shape=(shape[-1], 3), initializer=0.5)
                self.b = self.add_weight(name='b', shape=(5,), initializer=2.0, constraint=MinMax(0, 4), regularizer=MonoL1(1e-3))

            def call(self, x):
                return x @ self.w.value + self.b.value[:3]

        torch.manual_seed(0)
        X = torch.randn(8, 4)
        model = Toy()
        model(X[:1])
        state = FlatState(model)
        dp = DataParallel()
        assert dp.world == world and dp.rank == rank
        # bucket layout: every variable is a 16-byte aligned view, constraints / regularisers tabulated per element
        assert state.offsets == [0, 12] and state.n == 20
        assert model.w.value.data_ptr() == state.params.data_ptr()
        assert state.lo[12:17].tolist() == [0.0] * 5 and state.hi[12:17].tolist() == [4.0] * 5
        assert state.l1[12:17].tolist() == pytest.approx([1e-3] * 5) and float(state.l1[:12].abs().sum()) == 0.0
        # sharded forward/backward, then the averaged bucket equals the full-batch gradient
        sl = shard_batch(X.shape[0], rank, world)
        state.zero_grad()
        model(X[sl]).pow(2).mean().backward()
        state.check_views()
        dp.sync_gradients(state.grads)
        ref_model = Toy()
        ref_model(X[:1])
        ref_model(X).pow(2).mean().backward()
        assert torch.allclose(model.w.value.grad, ref_model.w.value.grad, atol=1e-6)
        assert torch.allclose(model.b.value.grad, ref_model.b.value.grad, atol=1e-6)
        # abs-max statistics: the hook is installed only inside the context and takes the max over ranks
        assert fpq.absmax_sync_hook is None
        stat = X[sl].abs().amax(0, keepdim=True)
        with dp:
            assert fpq.absmax_sync_hook is not None
            synced = fpq._sync_absmax(stat.clone(), X[sl])
            same = fpq._sync_absmax(stat.clone(), torch.nn.Parameter(X[sl]))  # parameters are identical on all ranks
        assert fpq.absmax_sync_hook is None
        assert torch.equal(synced, X.abs().amax(0, keepdim=True))
        assert torch.equal(same, stat)
        # synchronised batch moments: each rank's shard yields the moments of the whole batch, gradients included
        from hgq2_b200.backend import moments

        xs = X[sl].clone().requires_grad_()
        m, v = moments(xs, (0,), synchronized=True)
        (m.sum() + (v * torch.arange(1.0, 5.0)).sum()).backward()
        xf = X.clone().requires_grad_()
        mf, vf = moments(xf, (0,))
        (mf.sum() + (vf * torch.arange(1.0, 5.0)).sum()).backward()
        assert torch.allclose(m, mf, atol=1e-6) and torch.allclose(v, vf, atol=1e-6)
        # the full-batch loss is counted once per rank here, hence the factor world on the shard's gradient
        assert torch.allclose(xs.grad, xf.grad[sl] * world, atol=1e-6)
        out.put((rank, 'ok'))
    except Exception as e:  # surface the failure in the parent
        import traceback

        out.put((rank, traceback.format_exc()))
        raise e
    finally:
        dist.destroy_process_group()


def test_data_parallel_plumbing_world2():
    ctx = mp.get_context('spawn')
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    results = [out.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    for rank, msg in results:
        assert msg == 'ok', f'rank {rank}:\n{msg}'


def test_shard_batch():
    from hgq2_b200.train import shard_batch

    assert [shard_batch(16, r, 4) for r in range(4)] == [slice(0, 4), slice(4, 8), slice(8, 12), slice(12, 16)]
    with pytest.raises(ValueError):
        shard_batch(10, 0, 4)
