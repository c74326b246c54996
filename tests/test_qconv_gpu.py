"""The implicit-GEMM convolution kernels against torch's fp32 convolution on quantised operands."""

import numpy as np
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def grid(rng, shape, bits=6):
    return (np.round(rng.standard_normal(shape) * 2**bits) / 2**bits).astype(np.float32)


def ref_conv(x, w, b, stride, dil, pads, relu):
    (pt, pb), (pl, pr) = pads
    xx = F.pad(x.permute(0, 3, 1, 2).double(), (pl, pr, pt, pb))
    y = F.conv2d(xx, w.permute(3, 2, 0, 1).double(), stride=stride, dilation=dil).permute(0, 2, 3, 1)
    if b is not None:
        y = y + b.double()
    return torch.relu(y) if relu else y


@pytest.mark.parametrize('B,H,W,C,KH,KW,N,stride,pads', [
    (9, 32, 32, 4, 3, 3, 16, (1, 1), ((0, 0), (0, 0))),
    (5, 15, 15, 16, 3, 3, 32, (1, 1), ((0, 0), (0, 0))),
    (7, 6, 6, 32, 3, 3, 64, (1, 1), ((0, 0), (0, 0))),
    (4, 9, 8, 8, 3, 3, 5, (1, 1), ((1, 1), (1, 1))),
    (3, 11, 10, 4, 3, 2, 12, (2, 2), ((0, 1), (0, 0))),
    (2, 7, 7, 64, 3, 3, 32, (1, 1), ((2, 2), (2, 2))),
])
def test_implicit_gemm_conv_forward(B, H, W, C, KH, KW, N, stride, pads):
    from hgq2_b200 import kernels

    rng = np.random.default_rng(B + H + C + N)
    x = torch.from_numpy(grid(rng, (B, H, W, C)))
    w = torch.from_numpy(grid(rng, (KH, KW, C, N), 5))
    b = torch.from_numpy(grid(rng, (N,), 4))
    (pt, pb), (pl, pr) = pads
    OH = (H + pt + pb - KH) // stride[0] + 1
    OW = (W + pl + pr - KW) // stride[1] + 1
    assert kernels.qconv2d_supported(B, H, W, C, KH, KW, N, OH, OW)
    for relu in (False, True):
        y = kernels.qconv2d_fwd(x.cuda(), w.reshape(-1, N).cuda(), b.cuda(), 'relu' if relu else None, KH, KW, (OH, OW), stride,
                                (1, 1), (pt, pl))
        kernels.check_status(y.device)
        yr = ref_conv(x, w, b, stride, (1, 1), pads, relu)
        assert tuple(y.shape) == tuple(yr.shape)
        err = float((y.cpu().double() - yr).abs().max() / max(float(yr.abs().max()), 1e-30))
        assert err <= 2e-7, err


@pytest.mark.parametrize('B,H,W,C,KH,KW,N,stride,pads,relu', [
    (9, 32, 32, 4, 3, 3, 16, (1, 1), ((0, 0), (0, 0)), True),
    (5, 15, 15, 16, 3, 3, 32, (1, 1), ((0, 0), (0, 0)), True),
    (37, 6, 6, 32, 3, 3, 64, (1, 1), ((0, 0), (0, 0)), True),
    (4, 9, 8, 8, 3, 3, 5, (1, 1), ((1, 1), (1, 1)), False),
    (3, 11, 10, 4, 3, 2, 12, (2, 2), ((0, 1), (0, 0)), True),
    (2, 7, 7, 64, 3, 3, 32, (1, 1), ((2, 2), (2, 2)), False),
    (600, 12, 12, 8, 3, 3, 16, (1, 1), ((0, 0), (0, 0)), True),
])
def test_implicit_gemm_conv_weight_gradient(B, H, W, C, KH, KW, N, stride, pads, relu):
    from hgq2_b200 import kernels

    rng = np.random.default_rng(B + H + C + N)
    x = torch.from_numpy(grid(rng, (B, H, W, C)))
    w = torch.from_numpy(grid(rng, (KH, KW, C, N), 5)).requires_grad_(True)
    b = torch.from_numpy(grid(rng, (N,), 4)).requires_grad_(True)
    (pt, pb), (pl, pr) = pads
    y = ref_conv(x, w, b, stride, (1, 1), pads, relu)
    gy = torch.from_numpy(rng.standard_normal(tuple(y.shape)).astype(np.float32))
    (y * gy.double()).sum().backward()
    assert kernels.qconv2d_wgrad_supported(B, H, W, C, KH, KW, N, y.shape[1], y.shape[2])
    gm, dw, db = kernels.qconv2d_wgrad(x.cuda(), gy.cuda(), y.detach().float().cuda() if relu else None, KH, KW, stride, (1, 1),
                                       (pt, pl), True)
    kernels.check_status(gm.device)
    g_ref = gy * (y.detach() > 0) if relu else gy
    assert torch.equal(gm.cpu(), g_ref.float())
    for got, ref in ((dw.cpu().reshape(KH, KW, C, N), w.grad), (db.cpu(), b.grad)):
        err = float((got.double() - ref.double()).abs().max() / max(float(ref.abs().max()), 1e-30))
        assert err <= 3e-5, err


@pytest.mark.parametrize('B,H,W,C,KH,KW,N,pads', [
    (9, 32, 32, 4, 3, 3, 16, ((0, 0), (0, 0))),
    (5, 15, 15, 16, 3, 3, 32, ((0, 0), (0, 0))),
    (7, 6, 6, 32, 3, 3, 64, ((0, 0), (0, 0))),
    (4, 9, 8, 8, 3, 3, 8, ((1, 1), (1, 1))),
])
def test_input_gradient_as_flipped_convolution(B, H, W, C, KH, KW, N, pads):
    from hgq2_b200 import kernels

    rng = np.random.default_rng(B + H + C + N)
    x = torch.from_numpy(grid(rng, (B, H, W, C))).requires_grad_(True)
    w = torch.from_numpy(grid(rng, (KH, KW, C, N), 5))
    (pt, pb), (pl, pr) = pads
    y = ref_conv(x, w, None, (1, 1), (1, 1), pads, False)
    gy = torch.from_numpy(rng.standard_normal(tuple(y.shape)).astype(np.float32))
    (y * gy.double()).sum().backward()
    wt = w.flip(0, 1).permute(0, 1, 3, 2).reshape(KH * KW * N, C).contiguous()
    dx = kernels.qconv2d_fwd(gy.cuda(), wt.cuda(), None, None, KH, KW, (H, W), (1, 1), (1, 1), (KH - 1 - pt, KW - 1 - pl))
    kernels.check_status(dx.device)
    err = float((dx.cpu().double() - x.grad.double()).abs().max() / float(x.grad.abs().max()))
    assert err <= 5e-6, err


@pytest.mark.parametrize('shape,pool,strides', [
    ((5, 30, 30, 16), (2, 2), (2, 2)),
    ((3, 13, 13, 32), (2, 2), (2, 2)),
    ((4, 9, 11, 6), (3, 2), (2, 1)),
    ((2, 8, 8, 3), (3, 3), (1, 1)),
])
def test_max_pooling_matches_torch_including_ties(shape, pool, strides):
    from hgq2_b200 import kernels

    rng = np.random.default_rng(11)
    # a coarse grid after ReLU: many exact ties inside a window, so the arg-max rule is exercised
    x = torch.from_numpy(np.maximum(np.round(rng.standard_normal(shape) * 2) / 2, 0).astype(np.float32))
    xr = x.clone().requires_grad_()
    yr = F.max_pool2d(xr.permute(0, 3, 1, 2), pool, strides).permute(0, 2, 3, 1)
    gy = torch.from_numpy(rng.standard_normal(tuple(yr.shape)).astype(np.float32))
    (yr * gy).sum().backward()
    y, arg = kernels.maxpool2d_fwd(x.cuda(), pool, strides)
    assert torch.equal(y.cpu(), yr.detach())
    dx = kernels.maxpool2d_bwd(gy.cuda(), arg, shape, pool, strides)
    assert float((dx.cpu() - xr.grad).abs().max()) <= 1e-6 * float(gy.abs().max()) * pool[0] * pool[1]


def test_rgb_image_is_read_in_place():
    # C = 3: pixels are 12 bytes apart; the unit-stride kernels read them with scalar loads instead of a padded copy
    from hgq2_b200 import kernels

    rng = np.random.default_rng(3)
    B, H, W, C, N = 6, 32, 32, 3, 16
    x = torch.from_numpy(grid(rng, (B, H, W, C)))
    w = torch.from_numpy(grid(rng, (3, 3, C, N), 5)).requires_grad_(True)
    b = torch.from_numpy(grid(rng, (N,), 4)).requires_grad_(True)
    xr = x.clone().requires_grad_()
    y = ref_conv(xr, w, b, (1, 1), (1, 1), ((0, 0), (0, 0)), True)
    gy = torch.from_numpy(rng.standard_normal(tuple(y.shape)).astype(np.float32))
    (y * gy.double()).sum().backward()
    assert kernels.qconv2d_unit_stride_supported(B, H, W, C, 3, 3, N, 30, 30)
    yk = kernels.qconv2d_fwd(x.cuda(), w.detach().reshape(-1, N).cuda(), b.detach().cuda(), 'relu', 3, 3, (30, 30), (1, 1), (1, 1), (0, 0))
    assert float((yk.cpu().double() - y.detach()).abs().max()) <= 2e-7 * float(y.abs().max())
    gm, dw, db = kernels.qconv2d_wgrad(x.cuda(), gy.cuda(), yk, 3, 3, (1, 1), (1, 1), (0, 0), True)
    assert float((dw.cpu().reshape(3, 3, C, N).double() - w.grad).abs().max()) <= 3e-5 * float(w.grad.abs().max())
    assert float((db.cpu().double() - b.grad).abs().max()) <= 3e-5 * float(b.grad.abs().max())
    wt = w.detach().flip(0, 1).permute(0, 1, 3, 2).reshape(9 * N, C).contiguous()
    dx = kernels.qconv2d_fwd(gm, wt.cuda(), None, None, 3, 3, (H, W), (1, 1), (1, 1), (2, 2))
    kernels.check_status(dx.device)
    assert float((dx.cpu().double() - xr.grad).abs().max()) <= 5e-6 * float(xr.grad.abs().max())
