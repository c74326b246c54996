"""Calibration pass: with a calibration dataset, find the integer bits the WRAP-mode quantizers of a model need.

Mirror of ``src/hgq/utils/minmax_trace.py:13-99``: the integer bits (and the sign bit) of every trainable WRAP
quantizer are reset, the dataset is run through the model with ``training`` set to an object that compares equal to
``'tracing'`` and is falsy, which makes each quantizer widen ``i`` / set ``k`` to cover what it sees
(``fixed_point_quantizer.py:289-300,414-422``), and the layers' EBOPs are recomputed with the new bitwidths.
"""

from __future__ import annotations

from collections.abc import Sequence

import numpy as np
import torch

from ..backend import Layer


class TrainingFlagWrapper:
    """``== 'tracing'`` is True while ``bool()`` is False (minmax_trace.py:25-33)."""

    def __init__(self, value):
        self.value = value

    def __eq__(self, other):
        return self.value == other

    def __hash__(self):
        return hash(self.value)

    def __bool__(self):
        return self.value is True


def _reset_minmax(layer: Layer) -> None:
    """minmax_trace.py:13-22: i <- -1e9 and k <- 0 for every trainable quantizer that tracks its range (WRAP)."""
    for sub in layer.modules():
        if hasattr(sub, '_i_decay_speed') and getattr(sub, 'trainable', True):
            sub._i.assign(torch.full_like(sub._i.value, -1e9))
            sub._k.assign(torch.zeros_like(sub._k.value))


def _batches(data, batch_size: int):
    if isinstance(data, (tuple, list)) and not torch.is_tensor(data):
        n = len(data[0])
        for s in range(0, n, batch_size):
            yield tuple(d[s:s + batch_size] for d in data)
    else:
        for s in range(0, len(data), batch_size):
            yield data[s:s + batch_size]


def _to_device(x, device):
    if isinstance(x, tuple):
        return tuple(_to_device(v, device) for v in x)
    t = x if torch.is_tensor(x) else torch.from_numpy(np.ascontiguousarray(x))
    return t.to(device)


def trace_minmax(model: Layer, data, reset: bool = True, batch_size: int = 1024, verbose: int | bool = 0,
                 return_results: bool = False, device=None):
    """Returns the model's total EBOPs after calibration, or the model outputs on ``data`` if ``return_results``.

    ``data``: an array / tensor (or a sequence of them for a multi-input model) whose first axis is the sample axis.
    """
    if device is None:
        p = next(iter(model.parameters()), None)
        device = p.device if p is not None else torch.device('cpu')
    if reset:
        _reset_minmax(model)
    results = []
    flag = TrainingFlagWrapper('tracing')
    with torch.no_grad():
        for batch in _batches(data, batch_size):
            xb = _to_device(batch, device)
            r = model(*xb, training=flag) if isinstance(xb, tuple) else model(xb, training=flag)
            if return_results:
                results.append(tuple(t.cpu().numpy() for t in r) if isinstance(r, (tuple, list)) else r.cpu().numpy())
    record: dict[str, int] = {}
    layers: Sequence = getattr(model, 'layers', None) or [m for m in model.modules() if m is not model]
    for layer in layers:
        if getattr(layer, 'enable_ebops', False):
            record[layer.name] = int(layer.ebops)
    if verbose and record:
        width = max(max(map(len, record.keys())), 5)
        for k, v in record.items():
            print(f'{k:{width}}: {v}')
        print(f'Total: {sum(record.values())}')
    if return_results:
        if results and isinstance(results[0], tuple):
            return tuple(np.concatenate([r[i] for r in results]) for i in range(len(results[0])))
        return np.concatenate(results)
    return int(sum(record.values()))
