"""Weight files: Keras-style variable paths and a save / load round trip (host logic only, no kernel runs)."""

import numpy as np
import torch


def build_model():
    from hgq2_b200.backend import Sequential, set_default_device
    from hgq2_b200.config import LayerConfigScope, QuantizerConfigScope
    from hgq2_b200.layers import QDense

    set_default_device('cpu')
    with QuantizerConfigScope(place='datalane', default_q_type='kif', overflow_mode='WRAP'), LayerConfigScope(beta0=1e-5):
        layers = [QDense(8, activation='relu', name='q_dense'), QDense(3, name='q_dense_1')]
    model = Sequential(layers, name='sequential')
    shape = (None, 6)
    for layer in layers:
        layer.build(shape)
        layer.built = True
        shape = layer.compute_output_shape(shape)
    return model


def test_paths_follow_the_attribute_walk():
    from hgq2_b200.utils import state_tree

    tree = state_tree(build_model())
    assert 'layers/q_dense' in tree and 'layers/q_dense_1' in tree
    for attr in ('_iq', '_kq', '_bq'):
        assert f'layers/q_dense/{attr}/quantizer' in tree
    names = [v.name for v in tree['layers/q_dense/_kq/quantizer']._variables]
    assert names[:3] == ['k', 'b', 'i']  # creation order of the kbi weight quantizer's variables
    assert [v.name for v in tree['layers/q_dense']._variables] == ['kernel', 'bias', 'beta', 'ebops']


def test_save_load_round_trip(tmp_path):
    from hgq2_b200.utils import load_weights, save_weights

    a, b = build_model(), build_model()
    rng = np.random.default_rng(0)
    for v in a.variables:
        if v.value.is_floating_point():
            v.assign(torch.from_numpy(rng.standard_normal(tuple(v.shape)).astype(np.float32)))
    path = str(tmp_path / 'weights.npz')
    save_weights(a, path)
    assert any(not torch.equal(va.value, vb.value) for va, vb in zip(a.variables, b.variables))
    load_weights(b, path)
    assert len(a.variables) == len(b.variables) > 10
    for va, vb in zip(a.variables, b.variables):
        assert va.path.split('/')[-1] == vb.path.split('/')[-1] and torch.equal(va.value, vb.value)
