"""QSoftmax and QMultiHeadAttention (CUDA kernels for every quantizer and projection) against their CPU oracle twins."""

import numpy as np
import pytest
import torch

from oracle import hgq_layers as OL

pytestmark = pytest.mark.gpu


def close(a, b, rtol, what):
    a = a.detach().cpu().double().numpy()
    b = b.detach().cpu().double().numpy()
    scale = max(np.abs(b).max(), 1e-30)
    err = np.abs(a - b).max() / scale
    assert err <= rtol, f'{what}: error {err:.3e} relative to max |ref| {scale:.3e} exceeds {rtol}'


def compare_quantizer_grads(pairs):
    """pairs: (product Quantizer, oracle quantizer, label)."""
    for pq, oq, label in pairs:
        iq = pq.quantizer
        assert torch.equal(iq._i.value.detach().cpu(), oq._i.detach()), f'{label}._i'
        assert torch.equal(iq.bits.detach().cpu(), oq.bits.detach()), f'{label}.bits'
        for vname, leaf in oq.trainable_leaves().items():
            g = getattr(iq, '_' + vname).value.grad
            assert g is not None, f'{label}.{vname} got no gradient'
            close(g, leaf.grad, 1e-4, f'd {label}.{vname}')


def scopes(beta0=1e-3):
    from hgq2_b200.config import LayerConfigScope, QuantizerConfigScope

    a = QuantizerConfigScope(place='datalane', default_q_type='kif', overflow_mode='WRAP', round_mode='RND', i0=4, f0=8)
    t = QuantizerConfigScope(place='table', b0=10, i0=1)
    return a, t, LayerConfigScope(beta0=beta0, enable_ebops=True)


def test_qsoftmax_matches_oracle():
    from hgq2_b200.layers import QSoftmax
    from hgq2_b200.quantizer import QuantizerConfig

    rng = np.random.default_rng(0)
    a, t, l = scopes()
    with a, t, l:
        layer = QSoftmax(axis=-1, enable_oq=True, exp_iq_conf=QuantizerConfig(place='datalane', overflow_mode='SAT', i0=4, f0=6),
                         input_scaler=0.25)
    x_np = (np.round(rng.standard_normal((64, 4, 16, 16)) * 3 * 64) / 64).astype(np.float32)
    x = torch.from_numpy(x_np).cuda().requires_grad_()
    layer(x.detach()[:2], training=False)
    twin = OL.mirror_softmax(layer)
    xc = torch.from_numpy(x_np).requires_grad_()
    y, yc = layer(x, training=True), twin(xc, training=True)
    close(y, yc, 1e-5, 'softmax output')
    assert layer.ebops == twin.total_ebops()
    w = torch.from_numpy(rng.standard_normal(tuple(yc.shape)).astype(np.float32))
    ((y * w.cuda()).sum() + sum(layer.losses)).backward()
    ((yc * w).sum() + sum(twin.losses)).backward()
    close(x.grad, xc.grad, 1e-4, 'dx')
    compare_quantizer_grads([(layer.oq, twin.oq, 'oq'), (layer.exp_table.iq, twin.exp_table.iq, 'exp.iq'),
                             (layer.exp_table.oq, twin.exp_table.oq, 'exp.oq'), (layer.inv_table.iq, twin.inv_table.iq, 'inv.iq'),
                             (layer.inv_table.oq, twin.inv_table.oq, 'inv.oq')])
    close(layer(x.detach(), training=False), twin(torch.from_numpy(x_np), training=False), 1e-5, 'eval output')


@pytest.mark.parametrize('fuse', ['none', 'qkv'])
def test_qmha_matches_oracle(fuse):
    from hgq2_b200.layers import QMultiHeadAttention
    from hgq2_b200.workloads import randomize_weight_bits

    rng = np.random.default_rng(1)
    a, t, l = scopes()
    with a, t, l:
        layer = QMultiHeadAttention(2, 8, fuse=fuse, name=f'mha_{fuse}')
    x_np = (np.round(rng.standard_normal((48, 12, 16)) * 64) / 64).astype(np.float32)
    x = torch.from_numpy(x_np).cuda().requires_grad_()
    layer(x.detach()[:2], training=False)
    randomize_weight_bits(layer, 3, 7)
    twin = OL.mirror_mha(layer)
    xc = torch.from_numpy(x_np).requires_grad_()
    y, yc = layer(x, training=True), twin(xc, training=True)
    close(y, yc, 1e-5, 'attention output')
    assert int(layer.ebops) == twin.total_ebops(), (int(layer.ebops), twin.total_ebops())
    w = torch.from_numpy(rng.standard_normal(tuple(yc.shape)).astype(np.float32))
    ((y * w.cuda()).sum() / 48 + sum(layer.losses)).backward()
    ((yc * w).sum() / 48 + sum(twin.losses)).backward()
    close(x.grad, xc.grad, 1e-4, 'dx')
    for pl, ol, name in ((layer._query_dense, twin.q, 'q'), (layer._key_dense, twin.k, 'k'), (layer._value_dense, twin.v, 'v'),
                         (layer._output_dense, twin.o, 'o')):
        close(pl._kernel.value.grad, ol.kernel.grad, 1e-4, f'd {name}.kernel')
        pairs = [(pl.kq, ol.kq, f'{name}.kq')]
        if pl.enable_oq:
            pairs.append((pl.oq, ol.oq, f'{name}.oq'))
        if pl.enable_iq and not (fuse == 'qkv' and name in ('q', 'k')):
            pairs.append((pl.iq, ol.iq, f'{name}.iq'))
        compare_quantizer_grads(pairs)
    close(layer(x.detach(), training=False), twin(torch.from_numpy(x_np), training=False), 1e-5, 'eval output')


@pytest.mark.parametrize('B,H,D', [(3, 4, 16), (5, 2, 32), (130, 4, 16)])
def test_per_head_attention_products(B, H, D):
    # the three product kinds of the per-head tensor-core kernel against float64 einsums
    from hgq2_b200 import kernels

    L = 64
    rng = np.random.default_rng(B + H + D)
    q = torch.from_numpy((np.round(rng.standard_normal((B, L, H, D)) * 64) / 64).astype(np.float32))
    k = torch.from_numpy((np.round(rng.standard_normal((B, L, H, D)) * 64) / 64).astype(np.float32))
    p = torch.from_numpy(rng.standard_normal((B, H, L, L)).astype(np.float32))
    assert kernels.attn_heads_supported(B, L, H, D)
    s = kernels.attn_heads_matmul(0, q.cuda(), k.cuda(), B, L, H, D)
    kernels.check_status(s.device)
    ref = torch.einsum('bthd,bshd->bhts', q.double(), k.double())
    assert float((s.cpu().double() - ref).abs().max()) <= 1e-6 * float(ref.abs().max())
    o = kernels.attn_heads_matmul(1, p.cuda(), k.cuda(), B, L, H, D)
    ref = torch.einsum('bhts,bshd->bthd', p.double(), k.double())
    assert float((o.cpu().double() - ref).abs().max()) <= 3e-5 * float(ref.abs().max())
    g = kernels.attn_heads_matmul(2, p.cuda(), q.cuda(), B, L, H, D)
    kernels.check_status(g.device)
    ref = torch.einsum('bhts,bthd->bshd', p.double(), q.double())
    assert float((g.cpu().double() - ref).abs().max()) <= 3e-5 * float(ref.abs().max())


@pytest.mark.parametrize('switches', [
    # the general per-head kernel with per-thread loads, a whole warp per softmax row, softmax modes decided at run time
    dict(HGQ_ATTN_WS='0', HGQ_ATTN_TMA='0', HGQ_QSOFTMAX_LANES='32', HGQ_QSOFTMAX_GENERAL='1'),
    # the general per-head kernel with Q K^T's raw boxes from the copy engine (the default for that product) for all products
    dict(HGQ_ATTN_WS='0'),
    # the warp-specialised per-head kernel for Q K^T too (by default it takes the other two kinds of product)
    dict(HGQ_ATTN_WS='2'),
])
def test_other_kernel_organisations_on_the_same_cases(switches):
    # the switches are read once per process: the cases of this file and the attention / softmax cases at the benchmark
    # shape run again in a child process, so that every organisation stays covered by the same references
    import os
    import subprocess
    import sys

    env = dict(os.environ, **switches)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, '-m', 'pytest', os.path.join(root, 'tests', 'test_attention_gpu.py'),
                        os.path.join(root, 'tests', 'test_benchmark_shapes_gpu.py'), '-q', '-x', '-m', 'gpu',
                        '-k', '(softmax or qmha or per_head) and not other_kernel_organisations', '-p', 'no:cacheprovider'],
                       cwd=root, env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
