"""Parity on the code paths the benchmark workloads actually take: the shapes of the transformer workload (sequence 64,
model width 64, four heads of width 16) reach the per-head tensor-core attention products, the fused softmax chain with a
[256, 64] output-quantizer table and the column-blocked dense backward of the 128 -> 64 layer -- kernels that smaller test
shapes never launch.  Every case also asserts, from the per-entry-point call counters, that those kernels ran and that no
layer fell back to a library routine (the cases run in strict mode, where a fallback raises)."""

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


def scopes(beta0=1e-3):
    from hgq2_b200.config import LayerConfigScope, QuantizerConfigScope

    w = QuantizerConfigScope(place='weight', default_q_type='kbi', overflow_mode='SAT_SYM', round_mode='RND', b0=8, i0=2)
    a = QuantizerConfigScope(place='datalane', default_q_type='kif', overflow_mode='WRAP', round_mode='RND', i0=4, f0=8)
    t = QuantizerConfigScope(place='table', b0=10, i0=1)
    return w, a, t, LayerConfigScope(beta0=beta0, enable_ebops=True)


def compare_quantizer(pq, oq, label, gtol=1e-4):
    iq = pq.quantizer
    assert torch.equal(iq._i.value.detach().cpu(), oq._i.detach()), f'{label}._i'
    assert torch.equal(iq.bits.detach().cpu(), oq.bits.detach()), f'{label}.bits'
    for vname, leaf in oq.trainable_leaves().items():
        g = getattr(iq, '_' + vname).value.grad
        assert g is not None, f'{label}.{vname} got no gradient'
        close(g, leaf.grad, gtol if leaf.numel() > 4 else 2e-3, f'd {label}.{vname}')


@pytest.mark.parametrize('exp_iq_mode', ['SAT', 'WRAP'])
def test_qsoftmax_rows_of_64_with_a_256_row_table(exp_iq_mode):
    """Scores [B, 4, 64, 64]: L = 64, output-quantizer table [256, 64].  With exp_iq_mode 'WRAP' the exp table's input
    quantizer tracks its integer bits from the kernel's abs-max side output (the layer's default configuration)."""
    from hgq2_b200 import routes
    from hgq2_b200.layers import QSoftmax
    from hgq2_b200.quantizer import QuantizerConfig

    rng = np.random.default_rng(0)
    w, a, t, l = scopes()
    with w, a, t, l:
        layer = QSoftmax(axis=-1, enable_oq=True, input_scaler=0.25, name=f'sm64_{exp_iq_mode}',
                         exp_iq_conf=QuantizerConfig(place='datalane', overflow_mode=exp_iq_mode, k0=0, i0=4, f0=6),
                         inv_iq_conf=QuantizerConfig(place='datalane', k0=0, i0=7, f0=3))
    x_np = (np.round(rng.standard_normal((12, 4, 64, 64)) * 3 * 64) / 64).astype(np.float32)
    x = torch.from_numpy(x_np).cuda().requires_grad_()
    layer(x.detach()[:2], training=False)
    twin = OL.mirror_softmax(layer)
    xc = torch.from_numpy(x_np).requires_grad_()
    routes.reset()
    for step in range(2):  # two calls: the tracked integer bits of the first feed the EBOPs of the second
        x.grad = None
        xc.grad = None
        for q in layer._flatten_layers():
            for v in q._variables:
                v.value.grad = None
        for leaf in [t_ for q in (twin.oq, twin.exp_table.iq, twin.exp_table.oq, twin.inv_table.iq, twin.inv_table.oq)
                     for t_ in q.trainable_leaves().values()]:
            leaf.grad = None
        with routes.strict_mode():
            y = layer(x, training=True)
        yc = twin(xc, training=True)
        close(y, yc, 1e-5, f'softmax output, call {step}')
        assert layer.ebops == twin.total_ebops(), f'EBOPs, call {step}'
        wgt = torch.from_numpy(rng.standard_normal(tuple(yc.shape)).astype(np.float32))
        ((y * wgt.cuda()).sum() + sum(layer.losses)).backward()
        ((yc * wgt).sum() + sum(twin.losses)).backward()
        close(x.grad, xc.grad, 1e-4, f'dx, call {step}')
        for pq, oq, name in ((layer.oq, twin.oq, 'oq'), (layer.exp_table.iq, twin.exp_table.iq, 'exp.iq'),
                             (layer.exp_table.oq, twin.exp_table.oq, 'exp.oq'), (layer.inv_table.iq, twin.inv_table.iq, 'inv.iq'),
                             (layer.inv_table.oq, twin.inv_table.oq, 'inv.oq')):
            compare_quantizer(pq, oq, f'{name}, call {step}')
    assert routes.counts['hgq_qsoftmax_fwd'] == 2 and routes.counts['hgq_qsoftmax_bwd'] == 2, dict(routes.counts)
    assert not routes.fallbacks()


@pytest.mark.parametrize('B,T,L,table_round,exp_iq_mode', [
    (13, 64, 64, 'RND', 'SAT'),        # half a warp per row; the last row-group of a CTA has no batch left
    (13, 64, 64, 'RND', 'WRAP'),       # ... with a rounding-only table index
    (13, 64, 64, 'RND_CONV', 'SAT'),   # round-half-even tables: the kernel variant with every mode decided at run time
    (21, 8, 32, 'RND', 'SAT'),         # rows of 32: half a warp per row, two scores per lane
    (7, 4, 128, 'RND', 'WRAP'),        # rows of 128: a warp per row, four scores per lane
    (7, 4, 128, 'TRN', 'SAT'),
])
def test_qsoftmax_kernel_variants(B, T, L, table_round, exp_iq_mode):
    """Every organisation of the fused softmax kernels (lanes per row, scores per lane, modes known at compile time or
    not) against the oracle: outputs, EBOPs, input gradient, every quantizer's gradients and tracked state."""
    from hgq2_b200 import routes
    from hgq2_b200.config import QuantizerConfigScope
    from hgq2_b200.layers import QSoftmax
    from hgq2_b200.quantizer import QuantizerConfig

    rng = np.random.default_rng(L + B)
    w, a, t, l = scopes()
    t2 = QuantizerConfigScope(place='table', b0=10, i0=1, round_mode=table_round)
    with w, a, t, t2, l:
        layer = QSoftmax(axis=-1, enable_oq=True, input_scaler=0.25, name=f'smv_{B}_{L}_{table_round}_{exp_iq_mode}',
                         exp_iq_conf=QuantizerConfig(place='datalane', overflow_mode=exp_iq_mode, k0=0, i0=4, f0=6),
                         inv_iq_conf=QuantizerConfig(place='datalane', k0=0, i0=7, f0=3))
    x_np = (np.round(rng.standard_normal((B, 4, T, L)) * 3 * 64) / 64).astype(np.float32)
    x = torch.from_numpy(x_np).cuda().requires_grad_()
    layer(x.detach()[:2], training=False)
    twin = OL.mirror_softmax(layer)
    xc = torch.from_numpy(x_np).requires_grad_()
    routes.reset()
    with routes.strict_mode():
        y = layer(x, training=True)
    yc = twin(xc, training=True)
    close(y, yc, 1e-5, 'softmax output')
    assert layer.ebops == twin.total_ebops()
    wgt = torch.from_numpy(rng.standard_normal(tuple(yc.shape)).astype(np.float32))
    ((y * wgt.cuda()).sum() + sum(layer.losses)).backward()
    ((yc * wgt).sum() + sum(twin.losses)).backward()
    close(x.grad, xc.grad, 1e-4, 'dx')
    for pq, oq, name in ((layer.oq, twin.oq, 'oq'), (layer.exp_table.iq, twin.exp_table.iq, 'exp.iq'),
                         (layer.exp_table.oq, twin.exp_table.oq, 'exp.oq'), (layer.inv_table.iq, twin.inv_table.iq, 'inv.iq'),
                         (layer.inv_table.oq, twin.inv_table.oq, 'inv.oq')):
        compare_quantizer(pq, oq, name)
    assert routes.counts['hgq_qsoftmax_fwd'] == 1 and routes.counts['hgq_qsoftmax_bwd'] == 1, dict(routes.counts)


def test_qsoftmax_rows_of_64_from_a_16_byte_aligned_buffer():
    """Scores that start on a 16-byte but not a 32-byte boundary take the 16-lanes-per-row organisation (the 8-lane one
    moves 32 bytes per lane): same outputs and statistics bit for bit, gradients within the summation-order noise."""
    from hgq2_b200 import kernels

    dev = torch.device('cuda', 0)
    gen = torch.Generator(device=dev).manual_seed(3)
    B, rp, L = 13, 256, 64
    n = B * rp * L
    s = torch.round(torch.randn(n, device=dev, generator=gen) * 3 * 64) / 64
    gy = torch.randn(n, device=dev, generator=gen)
    hold = torch.empty(n + 8, device=dev)
    s_off = hold[4:4 + n]
    s_off.copy_(s)
    assert s.data_ptr() % 32 == 0 and s_off.data_ptr() % 32 == 16
    one = lambda v, dt=torch.float32: torch.full((1,), v, dtype=dt, device=dev)
    k0 = one(0, torch.uint8)
    f5 = torch.randint(4, 10, (rp * L,), device=dev, generator=gen).float()
    quants = [(k0, one(4.0), one(6.0), 'RND', 'SAT'), (k0, one(1.0), one(9.0), 'RND', 'SAT'), (None, None, one(3.0), 'RND', 'NONE'),
              (k0, one(1.0), one(9.0), 'RND', 'SAT'), (None, None, f5, 'RND', 'NONE')]
    outs = []
    for src in (s, s_off):
        x = src.view(B, rp, L)
        y, a3, a5, a1 = kernels.qsoftmax_fwd(x, quants, 0.25, 1e-7, rp, True, True, True)
        ds, sc, df5, _ = kernels.qsoftmax_bwd(gy.view(B, rp, L), x, quants, 0.25, 1e-7, rp, False)
        outs.append((y, a3, a5, a1, ds, sc, df5))
    for j, name in enumerate(('y', 'amax3', 'amax5', 'amax1')):
        assert torch.equal(outs[0][j], outs[1][j]), name
    for j, name in ((4, 'ds'), (5, 'scalars'), (6, 'df5')):
        close(outs[1][j], outs[0][j], 1e-5, name)


def test_qsoftmax_compile_time_variants_agree():
    """The kernel variants with the modes known at compile time against one another: a table index quantizer that saturates
    at a range nothing reaches (variants 2 / 4) must give the bits of one that only rounds (variants 1 / 3), for table
    outputs that round by floor and half-even."""
    from hgq2_b200 import kernels

    dev = torch.device('cuda', 0)
    gen = torch.Generator(device=dev).manual_seed(5)
    B, rp, L = 9, 256, 64
    s = (torch.round(torch.randn(B, rp, L, device=dev, generator=gen) * 3 * 64) / 64)
    gy = torch.randn(B, rp, L, device=dev, generator=gen)
    one = lambda v, dt=torch.float32: torch.full((1,), v, dtype=dt, device=dev)
    k0 = one(0, torch.uint8)
    f5 = torch.randint(4, 10, (rp * L,), device=dev, generator=gen).float()
    for table_round in ('RND', 'RND_CONV'):
        outs = []
        for q1 in ((None, None, one(6.0), 'RND', 'NONE'), (k0, one(20.0), one(6.0), 'RND', 'SAT')):
            quants = [q1, (k0, one(1.0), one(9.0), table_round, 'SAT'), (None, None, one(3.0), 'RND', 'NONE'),
                      (k0, one(1.0), one(9.0), table_round, 'SAT'), (None, None, f5, 'RND', 'NONE')]
            y, a3, a5, a1 = kernels.qsoftmax_fwd(s, quants, 0.25, 1e-7, rp, True, True, True)
            ds, sc, df5, _ = kernels.qsoftmax_bwd(gy, s, quants, 0.25, 1e-7, rp, False)
            outs.append((y.clone(), a3.clone(), a5.clone(), a1.clone(), ds.clone(), sc.clone(), df5.clone()))
        for j, name in enumerate(('y', 'amax3', 'amax5', 'amax1', 'ds', 'scalars', 'df5')):
            assert torch.equal(outs[0][j], outs[1][j]), (table_round, name)


def test_qmha_at_the_benchmark_shape():
    """QMultiHeadAttention(4 heads, key_dim 16) on [B, 64, 64]: projections on the fused dense kernels, Q K^T and P V (and
    the four products of their backward) on the per-head tensor-core kernel, the scores through the fused softmax."""
    from hgq2_b200 import kernels, routes
    from hgq2_b200.layers import QMultiHeadAttention
    from hgq2_b200.quantizer import QuantizerConfig
    from hgq2_b200.workloads import randomize_weight_bits

    rng = np.random.default_rng(1)
    w, a, t, l = scopes()
    with w, a, t, l:
        layer = QMultiHeadAttention(
            4, 16, name='mha_bench_shape',
            softmax_exp_iq_conf=QuantizerConfig(place='datalane', overflow_mode='SAT', k0=0, i0=4, f0=6),
            softmax_inv_iq_conf=QuantizerConfig(place='datalane', k0=0, i0=7, f0=3))
    B = 12
    x_np = (np.round(rng.standard_normal((B, 64, 64)) * 64) / 64).astype(np.float32)
    x = torch.from_numpy(x_np).cuda().requires_grad_()
    layer(x.detach()[:2], training=False)
    randomize_weight_bits(layer, 4, 8)
    twin = OL.mirror_mha(layer)
    xc = torch.from_numpy(x_np).requires_grad_()
    routes.reset()
    with routes.strict_mode():
        y = layer(x, training=True)
    yc = twin(xc, training=True)
    close(y, yc, 1e-5, 'attention output')
    assert int(layer.ebops) == twin.total_ebops(), (int(layer.ebops), twin.total_ebops())
    wgt = torch.from_numpy(rng.standard_normal(tuple(yc.shape)).astype(np.float32))
    with routes.strict_mode():
        ((y * wgt.cuda()).sum() / B + sum(layer.losses)).backward()
    ((yc * wgt).sum() / B + sum(twin.losses)).backward()
    kernels.check_status(x.device)
    close(x.grad, xc.grad, 1e-4, 'dx')
    for pl, ol, name in ((layer._query_dense, twin.q, 'q'), (layer._key_dense, twin.k, 'k'), (layer._value_dense, twin.v, 'v'),
                         (layer._output_dense, twin.o, 'o')):
        close(pl._kernel.value.grad, ol.kernel.grad, 1e-4, f'd {name}.kernel')
        compare_quantizer(pl.kq, ol.kq, f'{name}.kq')
        if pl.enable_oq:
            compare_quantizer(pl.oq, ol.oq, f'{name}.oq')
        compare_quantizer(pl.iq, ol.iq, f'{name}.iq')
    sm, smt = layer._softmax, twin.softmax
    for pq, oq, name in ((sm.oq, smt.oq, 'softmax.oq'), (sm.exp_table.iq, smt.exp_table.iq, 'exp.iq'),
                         (sm.exp_table.oq, smt.exp_table.oq, 'exp.oq'), (sm.inv_table.iq, smt.inv_table.iq, 'inv.iq'),
                         (sm.inv_table.oq, smt.inv_table.oq, 'inv.oq')):
        compare_quantizer(pq, oq, name)
    # 2 forward products + 4 backward products on the per-head kernel, the softmax chain fused, no library contraction
    assert routes.counts['hgq_attn_heads_matmul'] == 6, dict(routes.counts)
    assert routes.counts['hgq_qsoftmax_fwd'] == 1 and routes.counts['hgq_qsoftmax_bwd'] == 1
    assert routes.counts['hgq_qdense_fwd'] == 4
    assert not routes.fallbacks(), routes.fallbacks()


def test_qdense_128_to_64_takes_the_column_blocked_backward():
    """QDense 128 -> 64 on [B, 64, 128] with a per-activation [64, 128] table: the backward runs as two launches of the
    strided kernel (one per block of 64 input columns), with the gradient of a mean over the sequence read in place."""
    from hgq2_b200 import kernels, routes
    from hgq2_b200.layers import QDense
    from hgq2_b200.workloads import randomize_weight_bits

    rng = np.random.default_rng(2)
    w, a, t, l = scopes()
    with w, a, t, l:
        layer = QDense(64, name='ffn_out_bench_shape')
    B = 24
    x_np = (np.round(np.clip(rng.standard_normal((B, 64, 128)), -5, 5) * 256) / 256).astype(np.float32)
    x = torch.from_numpy(x_np).cuda().requires_grad_()
    layer(x.detach()[:2], training=False)
    randomize_weight_bits(layer, 4, 8)
    twin = OL.mirror_layer(layer)
    xc = torch.from_numpy(x_np).requires_grad_()
    routes.reset()
    with routes.strict_mode():
        y = layer(x, training=True)
        yc = twin(xc, training=True)
        close(y, yc, 1e-5, 'output')
        assert int(layer.ebops.item()) == int(twin.ebops.item())
        wgt = torch.from_numpy(rng.standard_normal((B, 64)).astype(np.float32))
        ((y.mean(dim=1) * wgt.cuda()).sum() + sum(layer.losses)).backward()
    ((yc.mean(dim=1) * wgt).sum() + sum(twin.losses)).backward()
    kernels.check_status(x.device)
    close(x.grad, xc.grad, 1e-4, 'dx')
    close(layer._kernel.value.grad, twin.kernel.grad, 1e-4, 'dkernel')
    close(layer._bias.value.grad, twin.bias.grad, 1e-4, 'dbias')
    for qname, tq in twin.quantizers().items():
        compare_quantizer(getattr(layer, qname), tq, qname)
    assert routes.counts['hgq_qdense_bwd_strided'] == 2, dict(routes.counts)
    assert not routes.fallbacks(), routes.fallbacks()


def test_transformer_block_steps_at_the_benchmark_shape():
    """Two full QAT steps of the transformer workload at its real sequence length, width and head count (small batch)
    against the oracle, in strict mode."""
    from hgq2_b200 import routes, workloads
    from tests.test_train_gpu import run_steps

    rng = np.random.default_rng(1)
    x = rng.standard_normal((16, 64, 64)).astype(np.float32)
    y = np.random.default_rng(2).integers(0, 5, 16)
    for engine in (True, False):  # the static step plan and the autograd path launch the same kernels here
        routes.reset()
        with routes.strict_mode():
            run_steps(workloads.transformer_block, x, y, steps=2, engine=engine)
        # two training steps: 2 forward + 4 backward products each on the per-head kernel (+ 2 of the build-time forward)
        assert routes.counts['hgq_attn_heads_matmul'] == 12 + 2, dict(routes.counts)
        assert routes.counts['hgq_qsoftmax_bwd'] == 2
        assert routes.counts['hgq_qdense_bwd_strided'] >= 2 * 8
        assert not routes.fallbacks(), routes.fallbacks()


@pytest.mark.parametrize('name,shape,classes,draw', [
    ('jet_tagger_mlp', (256, 16), 5, 'normal'),
    ('particle_tagger', (24, 64, 16), 5, 'normal'),
    ('small_cnn', (16, 32, 32, 3), 10, 'uniform'),
    ('transformer_block', (8, 64, 64), 5, 'normal'),
])
def test_every_benchmark_model_steps_without_a_library_fallback(name, shape, classes, draw):
    """A captured-graph QAT step of each benchmark model, at the layer shapes the benchmark uses, runs in strict mode:
    no layer leaves the package's kernels for torch.matmul / cuBLAS / cuDNN / torch.einsum."""
    from hgq2_b200 import routes, workloads
    from hgq2_b200.train import Trainer, sparse_categorical_crossentropy

    rng = np.random.default_rng(1)
    x_np = (rng.standard_normal(shape) if draw == 'normal' else rng.random(shape)).astype(np.float32)
    y_np = np.random.default_rng(2).integers(0, classes, shape[0])
    model = workloads.build(getattr(workloads, name)())
    tr = Trainer(model, sparse_categorical_crossentropy)
    assert tr.engine is not None, tr.engine_refusal  # the static step plan covers every benchmark model
    x, y = torch.from_numpy(x_np).cuda(), torch.from_numpy(y_np).cuda()
    routes.reset()
    with routes.strict_mode():
        tr.capture(x, y, warmup=2, double_buffer=True)
        loss = float(tr.step(x, y))
        loss2 = float(tr.step_prefetched(tr.prefetch(torch.from_numpy(x_np).pin_memory(), torch.from_numpy(y_np).pin_memory())))
    tr.check_status(wait=True)
    assert tr.engine is not None, tr.engine_refusal
    assert np.isfinite(loss) and np.isfinite(loss2)
    assert not routes.fallbacks(), routes.fallbacks()
    at_launches = routes.counts  # every launch of this package's own kernels is counted; none may be a library contraction
    assert at_launches['hgq_tables_forward'] >= 1 and at_launches['hgq_tables_backward'] >= 1


def test_static_step_plan_equals_the_autograd_path():
    """Three steps of the small MLP through the static plan and through the layers' autograd path: same losses, same
    parameters, same quantizer state and EBOPs (both run the same kernels on the same operands; only the order of a few
    fp32 additions differs)."""
    from hgq2_b200 import workloads
    from hgq2_b200.train import Trainer, sparse_categorical_crossentropy

    rng = np.random.default_rng(3)
    xs = [torch.from_numpy(rng.standard_normal((1024, 16)).astype(np.float32)).cuda() for _ in range(3)]
    ys = [torch.from_numpy(rng.integers(0, 5, 1024)).cuda() for _ in range(3)]
    out = []
    for engine in (True, False):
        model = workloads.build(workloads.jet_tagger_mlp())
        tr = Trainer(model, sparse_categorical_crossentropy, engine=engine)
        losses = [float(tr.step(x, y)) for x, y in zip(xs, ys)]
        state = [v.value.detach().clone() for v in model.non_trainable_variables]
        out.append((losses, tr.state.params.clone(), state))
    (l_e, p_e, s_e), (l_a, p_a, s_a) = out
    assert np.allclose(l_e, l_a, rtol=1e-6), (l_e, l_a)
    assert float((p_e - p_a).abs().max()) <= 1e-5, float((p_e - p_a).abs().max())
    for a, b in zip(s_e, s_a):
        assert torch.equal(a, b)


def test_strict_mode_refuses_a_fallback():
    from hgq2_b200 import routes
    from hgq2_b200.config import LayerConfigScope, QuantizerConfigScope
    from hgq2_b200.layers import QDense

    with QuantizerConfigScope(place='datalane', default_q_type='kif', overflow_mode='WRAP'), LayerConfigScope(enable_ebops=True):
        layer = QDense(300, name='too_wide_for_the_fused_kernel')  # N > 256: outside the tensor-core kernel's limits
    x = torch.randn(64, 16, device='cuda')
    layer(x, training=False)
    with routes.strict_mode():
        with pytest.raises(routes.FallbackError):
            layer(x, training=True)
    y = layer(x, training=True)  # outside strict mode the library product runs and is counted
    assert y.shape == (64, 300) and routes.fallbacks().get('torch.matmul', 0) >= 1


def test_trainer_reports_a_kernel_that_gave_up():
    """A tensor-core kernel whose bounded wait runs out leaves a mark in the device status word; the trainer reads the
    word back behind every step and raises at the next one.  The mark is set from the host here."""
    from hgq2_b200 import _lib, kernels, workloads
    from hgq2_b200.train import Trainer, sparse_categorical_crossentropy

    model = workloads.build(workloads.jet_tagger_mlp())
    tr = Trainer(model, sparse_categorical_crossentropy)
    x = torch.randn(256, 16, device='cuda')
    y = torch.randint(0, 5, (256,), device='cuda')
    tr.capture(x, y, warmup=2)
    tr.step(x, y)
    tr.check_status(wait=True)  # clean so far
    kernels.status_word(x.device).fill_(1)  # what a kernel does when it gives up
    tr.step(x, y)  # this step's read-back carries the mark
    torch.cuda.synchronize()
    with pytest.raises(_lib.HGQError) as err:
        tr.step(x, y)
    assert err.value.status == -7
    tr.step(x, y)  # the word was cleared when it was reported
    tr.check_status(wait=True)


def test_quantizer_wrapper_scaler_affine_noise_on_a_layer():
    """Quantizer(scaler, affine, qnoise_factor) as the input quantizer of a dense layer (the unfused route)."""
    from hgq2_b200.config import LayerConfigScope, QuantizerConfigScope
    from hgq2_b200.layers import QDense
    from hgq2_b200.quantizer import QuantizerConfig
    from tests.test_layers_gpu import grid_input, perturb, run_pair

    rng = np.random.default_rng(7)
    with QuantizerConfigScope(place=('weight', 'bias'), default_q_type='kbi', overflow_mode='SAT_SYM'), \
            QuantizerConfigScope(place='datalane', default_q_type='kif', overflow_mode='SAT', round_mode='RND'), \
            LayerConfigScope(beta0=1e-3, enable_ebops=True):
        layer = QDense(9, activation='relu', name='d_scaled_iq',
                       iq_conf=QuantizerConfig('kif', 'datalane', scaler=0.5, affine=(2.0, 0.125), qnoise_factor=0.75,
                                               overflow_mode='SAT', i0=3, f0=4))
    x = grid_input(rng, (300, 12))
    layer(torch.from_numpy(x[:2]).cuda(), training=False)
    perturb(layer, rng, True)
    run_pair(layer, x, rng)
