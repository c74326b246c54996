"""Calibration (trace_minmax) of the benchmark models against the CPU oracle: quantizer state after the pass is
identical, EBOPs are identical integers, outputs agree."""

import numpy as np
import pytest
import torch

from oracle import train as OT

pytestmark = pytest.mark.gpu


def quantizer_state(model):
    out = []
    for m in model.modules():
        if hasattr(m, '_i_decay_speed'):
            out.append((m._i.value.detach().cpu().clone(), m._k.value.cpu().clone()))
    return out


@pytest.mark.parametrize('name,shape,draw', [
    ('jet_tagger_mlp', (700, 16), 'normal'),
    ('particle_tagger', (150, 64, 16), 'normal'),
    ('small_cnn', (70, 32, 32, 3), 'uniform'),
])
def test_trace_minmax_matches_oracle(name, shape, draw):
    from hgq2_b200 import workloads
    from hgq2_b200.utils import trace_minmax

    rng = np.random.default_rng(5)
    x = (rng.standard_normal(shape) * 1.5 if draw == 'normal' else rng.random(shape) * 2 - 0.5).astype(np.float32)
    model = workloads.build(getattr(workloads, name)())
    twin, _ = OT.mirror_model(model)
    total = trace_minmax(model, x, batch_size=64)
    ototal, oy = OT.trace_minmax(twin, torch.from_numpy(x), batch_size=64)
    assert total == ototal and total > 0
    got = quantizer_state(model)
    want = [(q._i.detach(), q._k) for q in OT._all_quantizers(twin) if q.overflow_mode == 'WRAP' and q.trainable]
    assert len(want) > 0 and len(got) == len(want)
    # module traversal order differs between the two sides: compare as multisets of (shape, integer bits, sign bits)
    key = lambda t: (tuple(t[0].shape), t[0].flatten().tolist(), t[1].flatten().tolist())  # noqa: E731
    assert sorted(map(key, got)) == sorted(map(key, want))
    # continuing without reset only widens
    y = trace_minmax(model, x, reset=False, batch_size=64, return_results=True)
    assert y.shape[0] == shape[0]
    err = np.abs(y - oy.numpy()).max() / max(np.abs(oy.numpy()).max(), 1e-30)
    assert err <= 1e-5, err
    assert trace_minmax(model, x, reset=False, batch_size=64) == total


def test_training_flag_wrapper_semantics():
    from hgq2_b200.utils import TrainingFlagWrapper

    t = TrainingFlagWrapper('tracing')
    assert t == 'tracing' and not t and not (t == True)  # noqa: E712
    assert bool(TrainingFlagWrapper(True))
