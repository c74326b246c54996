"""Full QAT steps (forward, backward, fused Adam, constraints) of the benchmark models against the CPU oracle."""

import numpy as np
import pytest
import torch
import torch.nn.functional as F

from oracle import train as OT

pytestmark = pytest.mark.gpu


def close(a, b, rtol, what):
    a = a.detach().cpu().double().numpy()
    b = b.detach().cpu().double().numpy()
    scale = max(np.abs(b).max(), 1e-30)
    err = np.abs(a - b).max() / scale
    assert err <= rtol, f'{what}: error {err:.3e} (relative to max |ref| = {scale:.3e}) exceeds {rtol}'


def ce(pred, y):
    return F.cross_entropy(pred, y)


def run_steps(builder, x_np, y_np, steps=3, beta0=1e-5, lr=1e-3, engine=True):
    from hgq2_b200 import workloads
    from hgq2_b200.train import Trainer

    model = workloads.build(builder(beta0=beta0))
    twin, pairs = OT.mirror_model(model)
    oopt = OT.OracleAdam(pairs, lr=lr)
    tr = Trainer(model, ce, learning_rate=lr, engine=engine)  # engine=True: the static step plan must cover the model
    x, y = torch.from_numpy(x_np).cuda(), torch.from_numpy(y_np).cuda()
    xc, yc = torch.from_numpy(x_np), torch.from_numpy(y_np)
    for s in range(steps):
        # forward + backward on both sides: loss, EBOPs and every gradient before the optimizer touches them
        _, loss = tr.forward_backward(x, y)
        tr.state.check_views()
        pred = twin(xc, training=True)
        oloss = ce(pred, yc) + sum(twin.losses) + oopt.regularization_loss()
        oloss.backward()
        close(loss, oloss, 1e-5, f'loss at step {s}')
        for pl, ol in zip([l for l in model.layers if hasattr(l, '_ebops')], twin.qlayers()):
            want = ol.total_ebops() if hasattr(ol, 'total_ebops') else int(ol.ebops.item())
            assert int(pl.ebops) == want, f'EBOPs of {pl.name} at step {s}'
        for leaf, var, _, _ in pairs:
            g = var.value.grad
            if var.regularizer is not None:  # the product adds the regulariser's constant gradient inside the optimizer
                g = g + var.regularizer.l1
            # a per-tensor (scalar) bitwidth gradient is a sum of millions of signed terms that largely cancel; its error
            # is set by the summation order relative to sum |terms|, not to the (tiny) result, hence the looser bound
            close(g, leaf.grad, 1e-4 if leaf.numel() > 4 else 2e-3, f'gradient of {var.path} at step {s}')
        tr.opt.step()
        oopt.step()
        # Adam normalises each element's step to ~lr whatever the gradient's size, so an element whose gradient is
        # at the noise floor may move differently; all others must agree closely
        for leaf, var, _, _ in pairs:
            d = (var.value.detach().cpu() - leaf.detach()).abs()
            scale = float(leaf.detach().abs().max()) + 1e-30
            assert float(d.max()) <= 2.0 * lr * (s + 1), f'{var.path} after step {s}: {float(d.max())}'
            n_bad = int((d > 1e-5 * scale + 1e-7).sum())
            # small tensors (a 64-element bias that starts at zero): a handful of noise-floor gradients is a larger share
            allowed = max(2, int((5e-3 if d.numel() > 1024 else 5e-2) * d.numel()))
            assert n_bad <= allowed, f'{var.path} after step {s}: {n_bad} of {d.numel()} elements moved differently'
    return model, twin


@pytest.mark.parametrize('engine', [True, False])
def test_jet_tagger_mlp_steps(engine):
    from hgq2_b200 import workloads

    rng = np.random.default_rng(1)
    x = rng.standard_normal((2048, 16)).astype(np.float32)
    y = np.random.default_rng(2).integers(0, 5, 2048)
    run_steps(workloads.jet_tagger_mlp, x, y, steps=3, beta0=1e-5, engine=engine)


@pytest.mark.parametrize('engine', [True, False])
def test_particle_tagger_steps(engine):
    from hgq2_b200 import workloads

    rng = np.random.default_rng(1)
    x = rng.standard_normal((96, 64, 16)).astype(np.float32)
    y = np.random.default_rng(2).integers(0, 5, 96)
    run_steps(workloads.particle_tagger, x, y, steps=2, engine=engine)


@pytest.mark.parametrize('engine', [True, False])
def test_small_cnn_steps(engine):
    from hgq2_b200 import workloads

    rng = np.random.default_rng(1)
    x = rng.uniform(0, 1, (48, 32, 32, 3)).astype(np.float32)
    y = np.random.default_rng(2).integers(0, 10, 48)
    run_steps(workloads.small_cnn, x, y, steps=2, engine=engine)


def _conv1d_net(beta0=1e-5):
    """Two causal / valid QConv1D layers (the second dilated) on [B, 24, 8] sequences, Flatten (160 features), QDense -> 5."""
    from hgq2_b200 import workloads as W
    from hgq2_b200.backend import Flatten, Sequential
    from hgq2_b200.layers import QConv1D, QDense

    w, a, l = W._scopes(3, 6, beta0)
    with w, a, l:
        layers = W._seeded([
            QConv1D(16, 5, padding='causal', activation='relu'),
            QConv1D(8, 3, dilation_rate=2, activation='relu'),
            Flatten(), QDense(5),
        ])
    model = Sequential(layers, name='conv1d_net')
    model.input_shape = (24, 8)
    model.weight_bits = (3, 8)
    return model


@pytest.mark.parametrize('engine', [True, False])
def test_conv1d_net_steps(engine):
    """QConv1D layers in a full QAT step: the static step plan runs them on the 2-D implicit-GEMM kernels as images of one
    row (engine=True: the plan must cover the model, no library convolution)."""
    from hgq2_b200 import routes

    rng = np.random.default_rng(5)
    x = rng.standard_normal((64, 24, 8)).astype(np.float32)
    y = np.random.default_rng(6).integers(0, 5, 64)
    routes.reset()
    run_steps(_conv1d_net, x, y, steps=2, engine=engine)
    assert not routes.fallbacks(), routes.fallbacks()


def test_transformer_block_steps():
    # sequence 16: outside the per-head attention kernel, so this model takes the autograd path (torch.einsum products)
    from hgq2_b200 import workloads

    rng = np.random.default_rng(1)
    x = rng.standard_normal((32, 16, 32)).astype(np.float32)
    y = np.random.default_rng(2).integers(0, 5, 32)
    run_steps(lambda beta0: workloads.transformer_block(seq=16, d_model=32, heads=2, beta0=beta0), x, y, steps=2, engine=None)


def _attention_behind_a_dense_layer(beta0=1e-5):
    """QDense 64 -> 64, then QMultiHeadAttention(4 heads, key_dim 16) on [B, 64, 64], mean over the sequence, QDense -> 5:
    the attention layer is not the first one, so its three input projections must hand an input gradient back."""
    from hgq2_b200 import workloads as W
    from hgq2_b200.backend import Lambda, Sequential
    from hgq2_b200.config import QuantizerConfigScope
    from hgq2_b200.layers import QDense, QMultiHeadAttention
    from hgq2_b200.quantizer import QuantizerConfig

    w, a, l = W._scopes(4, 8, beta0)
    t = QuantizerConfigScope(place='table', b0=10, i0=1)
    with w, a, t, l:
        layers = W._seeded([
            QDense(64, activation='relu'),
            QMultiHeadAttention(4, 16,
                                softmax_exp_iq_conf=QuantizerConfig(place='datalane', overflow_mode='SAT', k0=0, i0=4, f0=6),
                                softmax_inv_iq_conf=QuantizerConfig(place='datalane', k0=0, i0=7, f0=3)),
            Lambda(lambda x: x.mean(dim=1), name='mean_sequence'),
            QDense(5),
        ])
    model = Sequential(layers, name='attention_behind_dense')
    model.input_shape = (64, 64)
    model.weight_bits = (4, 8)
    return model


def test_attention_layer_that_is_not_the_first_layer():
    """The key and value projections' backward kernels add their input gradients to the query projection's in place
    (hgq_qdense_bwd_accumulate); loss, EBOPs, gradients and updates against the oracle as for the other models."""
    from hgq2_b200 import routes

    rng = np.random.default_rng(1)
    x = rng.standard_normal((8, 64, 64)).astype(np.float32)
    y = np.random.default_rng(2).integers(0, 5, 8)
    routes.reset()
    with routes.strict_mode():
        run_steps(_attention_behind_a_dense_layer, x, y, steps=2, engine=True)
    assert routes.counts['hgq_qdense_bwd_accumulate'] == 2 * 2, dict(routes.counts)


def test_adam_kernel_matches_keras_rule():
    from hgq2_b200 import _lib

    n = 1003
    g = torch.Generator().manual_seed(0)
    w0, gr = torch.randn(n, generator=g), torch.randn(n, generator=g)
    lo, hi = torch.full((n,), -0.5), torch.full((n,), 0.7)
    l1 = torch.full((n,), 1e-3)
    w, m, v = w0.clone().cuda(), torch.zeros(n).cuda(), torch.zeros(n).cuda()
    gd, lod, hid, l1d = gr.cuda(), lo.cuda(), hi.cuda(), l1.cuda()  # keep the device copies alive across the calls
    step = torch.zeros((), dtype=torch.int64).cuda()
    wr, mr, vr = w0.clone().double(), torch.zeros(n).double(), torch.zeros(n).double()
    for t in range(1, 4):
        st = _lib.lib().hgq_adam_step(w.data_ptr(), gd.data_ptr(), m.data_ptr(), v.data_ptr(), lod.data_ptr(),
                                      hid.data_ptr(), l1d.data_ptr(), n, 1e-3, 0.9, 0.999, 1e-7, 0.5,
                                      step.data_ptr(), _lib.stream_handle())
        assert st == 0
        ge = gr.double() * 0.5 + l1.double()
        mr = 0.9 * mr + 0.1 * ge
        vr = 0.999 * vr + 0.001 * ge * ge
        alpha = 1e-3 * (1 - 0.999**t) ** 0.5 / (1 - 0.9**t)
        wr = torch.clamp(wr - alpha * mr / (vr.sqrt() + 1e-7), -0.5, 0.7)
        torch.cuda.synchronize()
        np.testing.assert_allclose(w.cpu().numpy(), wr.numpy(), rtol=2e-5, atol=1e-7)
    assert int(step.item()) == 3


def test_graph_captured_step_equals_eager_steps():
    from hgq2_b200 import workloads
    from hgq2_b200.train import Trainer

    rng = np.random.default_rng(1)
    xs = [torch.from_numpy(rng.standard_normal((512, 16)).astype(np.float32)).cuda() for _ in range(3)]
    ys = [torch.from_numpy(rng.integers(0, 5, 512)).cuda() for _ in range(3)]
    results = []
    for graphed in (False, True):
        model = workloads.build(workloads.jet_tagger_mlp())
        tr = Trainer(model, ce)
        if graphed:
            snap = tr.state.params.clone()
            m, v, t = tr.opt.m.clone(), tr.opt.v.clone(), tr.opt.step_count.clone()
            qstate = [(var, var.value.detach().clone()) for var in model.non_trainable_variables]
            tr.capture(xs[0], ys[0], warmup=2)
            # undo the warm-up and capture-time updates so both runs start from the same state
            tr.state.params.copy_(snap); tr.opt.m.copy_(m); tr.opt.v.copy_(v); tr.opt.step_count.copy_(t)
            for var, val in qstate:
                var.value.data.copy_(val)
        losses = [float(tr.step(x, y)) for x, y in zip(xs, ys)]
        results.append((losses, tr.state.params.clone(), [int(l.ebops.item()) for l in model.layers]))
    (l0, p0, e0), (l1, p1, e1) = results
    assert l0 == l1, (l0, l1)
    assert torch.equal(p0, p1)
    assert e0 == e1


@pytest.mark.parametrize('B,C', [(1, 5), (777, 5), (65536, 10), (300, 64)])
def test_fused_softmax_cross_entropy(B, C):
    from hgq2_b200.train import sparse_categorical_crossentropy

    rng = np.random.default_rng(B + C)
    z = torch.from_numpy((rng.standard_normal((B, C)) * 3).astype(np.float32))
    y = torch.from_numpy(rng.integers(0, C, B))
    zc = z.clone().double().requires_grad_()
    ref = F.cross_entropy(zc, y)
    (ref * 1.7).backward()
    zg = z.cuda().requires_grad_()
    loss = sparse_categorical_crossentropy(zg, y.cuda())
    (loss * 1.7).backward()
    assert abs(float(loss) - float(ref)) <= 1e-6 * max(abs(float(ref)), 1.0)
    err = float((zg.grad.cpu().double() - zc.grad).abs().max() / zc.grad.abs().max())
    assert err <= 1e-5, err


def test_steps_with_the_fused_loss_match_the_oracle():
    from hgq2_b200 import workloads
    from hgq2_b200.train import Trainer, sparse_categorical_crossentropy

    rng = np.random.default_rng(1)
    x_np = rng.standard_normal((2048, 16)).astype(np.float32)
    y_np = np.random.default_rng(2).integers(0, 5, 2048)
    model = workloads.build(workloads.jet_tagger_mlp())
    twin, pairs = OT.mirror_model(model)
    oopt = OT.OracleAdam(pairs, lr=1e-3)
    tr = Trainer(model, sparse_categorical_crossentropy)
    _, loss = tr.forward_backward(torch.from_numpy(x_np).cuda(), torch.from_numpy(y_np).cuda())
    oloss = ce(twin(torch.from_numpy(x_np), training=True), torch.from_numpy(y_np)) + sum(twin.losses) + oopt.regularization_loss()
    oloss.backward()
    close(loss, oloss, 1e-5, 'loss')
    for leaf, var, _, _ in pairs:
        g = var.value.grad
        if var.regularizer is not None:
            g = g + var.regularizer.l1
        close(g, leaf.grad, 1e-4 if leaf.numel() > 4 else 2e-3, f'gradient of {var.path}')
