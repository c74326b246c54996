"""Saving and loading the variables of a model under Keras-style paths.

Keras' weight files address every variable by the path of attribute names that leads from the model to the layer owning
it, followed by ``vars/<index in creation order>`` (keras/src/saving/saving_lib.py); a ``layers`` list contributes
``layers/<layer name>``.  The classes of this package keep the reference's attribute names (``_iq``, ``_kq``, ``_bq``,
``_oq``, ``quantizer`` -- src/hgq/layers/core/base.py:132-231, src/hgq/quantizer/quantizer.py:20-47), so the same walk
yields the same paths, e.g. ``layers/q_dense/_kq/quantizer/vars/1``.  The container here is a NumPy ``.npz`` archive (no
HDF5 library is assumed); the path scheme has not been checked against a Keras-written file.
"""

from __future__ import annotations

import numpy as np
import torch

from ..backend import Layer


def _children(layer: Layer):
    """(attribute name, sub-layer) pairs in attribute-name order; members of a layer list are named by their ``name``."""
    out = []
    for attr, child in sorted(layer._modules.items()):
        if isinstance(child, Layer):
            out.append((attr, child))
        elif isinstance(child, (torch.nn.ModuleList, torch.nn.ModuleDict)):
            items = child.items() if isinstance(child, torch.nn.ModuleDict) else ((getattr(m, 'name', str(j)), m) for j, m in enumerate(child))
            for name, m in items:
                if isinstance(m, Layer):
                    out.append((f'{attr}/{name}', m))
    return out


def state_tree(model: Layer, prefix: str = '') -> dict[str, 'Layer']:
    """path -> layer for ``model`` and every layer below it (a shared layer is listed once, under its first path)."""
    tree, seen = {}, set()

    def walk(layer, path):
        if id(layer) in seen:
            return
        seen.add(id(layer))
        tree[path] = layer
        for attr, child in _children(layer):
            walk(child, f'{path}/{attr}' if path else attr)

    walk(model, prefix)
    return tree


def save_own_variables(layer: Layer, store: dict, path: str = '') -> None:
    """The Keras protocol: the layer's own variables, in creation order, under the keys '0', '1', ..."""
    for j, v in enumerate(layer._variables):
        key = f'{path}/vars/{j}' if path else f'vars/{j}'
        store[key] = v.value.detach().cpu().numpy()


def load_own_variables(layer: Layer, store, path: str = '') -> None:
    for j, v in enumerate(layer._variables):
        key = f'{path}/vars/{j}' if path else f'vars/{j}'
        if key not in store:
            raise KeyError(f'{key} (variable {v.path}) is missing from the weight store')
        a = np.asarray(store[key])
        if tuple(a.shape) != tuple(v.shape):
            raise ValueError(f'{key}: stored shape {tuple(a.shape)} does not match {v.path} {tuple(v.shape)}')
        v.assign(torch.from_numpy(a.copy()).to(v.value.device))


def save_weights(model: Layer, filepath: str) -> None:
    """Write every variable of a built model to ``filepath`` (.npz)."""
    store: dict = {}
    for path, layer in state_tree(model).items():
        save_own_variables(layer, store, path)
    np.savez(filepath, **store)


def load_weights(model: Layer, filepath: str) -> None:
    """Assign the variables of a built model from a file written by ``save_weights``."""
    with np.load(filepath) as store:
        for path, layer in state_tree(model).items():
            load_own_variables(layer, store, path)
