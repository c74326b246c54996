"""Data-parallel QAT on two GPUs (NCCL): two ranks on half batches must end up with the parameters, quantizer state and
EBOPs of one rank on the whole batch."""

import os
import socket
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent

WORKER = r'''
import os, sys
import numpy as np, torch, torch.distributed as dist, torch.nn.functional as F
sys.path.insert(0, os.environ['HGQ_ROOT'])
from hgq2_b200 import workloads
from hgq2_b200.train import DataParallel, Trainer, shard_batch

rank, world = int(os.environ['RANK']), int(os.environ['WORLD_SIZE'])
torch.cuda.set_device(int(os.environ['LOCAL_RANK']))
dist.init_process_group('nccl', device_id=torch.device('cuda', int(os.environ['LOCAL_RANK'])))

def run(builder, X, Y, dp):
    model = workloads.build(builder())
    tr = Trainer(model, F.cross_entropy, dp=dp)
    n = X.shape[0]
    sl = shard_batch(n, rank, world) if dp is not None else slice(None)
    want_peers = dp is not None and os.environ.get('HGQ_PEER_EXCHANGE', '1') != '0'
    assert (tr.peers is not None) == want_peers, (tr.peers, want_peers)  # gradient exchange inside the optimizer kernel, or NCCL
    losses = [float(tr.step(X[sl], Y[sl])) for _ in range(3)]
    tr.capture(X[sl], Y[sl], warmup=1)  # then the same step as a CUDA graph: one more eager step, two replays
    losses += [float(tr.step(X[sl], Y[sl])) for _ in range(2)]
    tr.check_status(wait=True)
    state = [(v.path, v.value.detach().clone()) for v in model.non_trainable_variables]
    return losses, tr.state.params.clone(), state, [int(l.ebops.item()) for l in model.layers if hasattr(l, '_ebops')]

# the small MLP ([1, F] abs-max tables) and the particle-set tagger ([1, 64, C] tables, a gradient that arrives as the
# expansion of a sum over the particles)
CASES = (('jet_tagger_mlp', workloads.jet_tagger_mlp, (4096, 16)), ('particle_tagger', workloads.particle_tagger, (512, 64, 16)))
for name, builder, shape in CASES:
    X = torch.from_numpy(np.random.default_rng(1).standard_normal(shape).astype(np.float32)).cuda()
    Y = torch.from_numpy(np.random.default_rng(2).integers(0, 5, shape[0])).cuda()
    l_dp, p_dp, s_dp, e_dp = run(builder, X, Y, DataParallel())
    l_1, p_1, s_1, e_1 = run(builder, X, Y, None)
    assert e_dp == e_1, (name, e_dp, e_1)
    scale = float(p_1.abs().max())
    assert float((p_dp - p_1).abs().max()) <= 2e-3 * 3, (name, float((p_dp - p_1).abs().max()))
    frac_bad = float(((p_dp - p_1).abs() > 1e-5 * scale + 1e-7).float().mean())
    assert frac_bad <= 5e-3, (name, frac_bad)
    for (path, a), (_, b) in zip(s_dp, s_1):  # quantizer state (tracked integer bits, keep-negative flags) and EBOPs: identical
        assert torch.equal(a, b), (name, path)
    # every rank holds the same parameters
    q = p_dp.clone(); dist.all_reduce(q, op=dist.ReduceOp.MAX); assert torch.equal(q, p_dp), name
    if rank == 0:
        print('DP_OK', name, 'world', world, 'losses dp', [round(v, 6) for v in l_dp], 'single', [round(v, 6) for v in l_1],
              'ebops', e_dp, 'max |dparam|', float((p_dp - p_1).abs().max()), flush=True)
dist.destroy_process_group()
'''


@pytest.mark.parametrize('peer_exchange', ['1', '0'])
def test_two_rank_data_parallel_matches_single_rank(tmp_path, peer_exchange):
    """peer_exchange '1': the gradient sum over peer memory inside the optimizer kernel (the default on one node);
    '0': NCCL all-reduce followed by the optimizer kernel."""
    if torch.cuda.device_count() < 2:
        pytest.skip('needs 2 GPUs')
    script = tmp_path / 'dp_worker.py'
    script.write_text(WORKER)
    with socket.socket() as s:
        s.bind(('127.0.0.1', 0))
        port = s.getsockname()[1]
    env = dict(os.environ, HGQ_ROOT=str(ROOT), NCCL_NVLS_ENABLE='0', HGQ_PEER_EXCHANGE=peer_exchange)
    r = subprocess.run([sys.executable, '-m', 'torch.distributed.run', '--nnodes=1', '--nproc-per-node=2', '--master-addr', '127.0.0.1',
                        '--master-port', str(port), str(script)], capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0 and r.stdout.count('DP_OK') == 2, r.stdout[-2000:] + r.stderr[-4000:]
    print(r.stdout)
