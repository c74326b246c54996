import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

os.environ.setdefault('MKL_NUM_THREADS', '1')
os.environ.setdefault('OPENBLAS_NUM_THREADS', '1')


def pytest_configure(config):
    config.addinivalue_line('markers', 'gpu: needs a CUDA device (run on a B200 with -m gpu)')


def pytest_collection_modifyitems(config, items):
    try:
        import torch

        has_gpu = torch.cuda.is_available()
    except Exception:
        has_gpu = False
    if has_gpu:
        return
    skip = pytest.mark.skip(reason='no CUDA device')
    for item in items:
        if 'gpu' in item.keywords:
            item.add_marker(skip)


@pytest.fixture(autouse=True)
def reproducible_initializers(monkeypatch):
    """Initializers built without a seed draw from consecutive fixed seeds (restarted for every test) instead of from OS
    entropy, so that a test sees the same weights in every run and in every test order."""
    import copy
    import itertools

    from hgq2_b200 import backend

    seeds = itertools.count(20240)
    for cls in (backend.GlorotUniform, backend.RandomNormal):
        original = cls.__call__

        def call(self, *args, _original=original, **kwargs):
            if self.seed is None:
                self = copy.copy(self)
                self.seed = next(seeds)
            return _original(self, *args, **kwargs)

        monkeypatch.setattr(cls, '__call__', call)


@pytest.fixture(scope='session')
def golden_dir():
    return ROOT / 'tests' / 'golden'


@pytest.fixture(scope='session')
def quantizer_golden(golden_dir):
    """The stateless quantizer's golden arrays: the file made by the real ``quantizers`` package
    (tests/golden/make_reference_golden.py) when someone has produced it, else the oracle-made one.  Returns
    (arrays, pinned): ``pinned`` says whether the arrays come from the reference itself."""
    import numpy as np

    ref = golden_dir / 'quantizer_golden_reference.npz'
    if ref.exists():
        return np.load(ref), True
    return np.load(golden_dir / 'quantizer_golden.npz'), False
