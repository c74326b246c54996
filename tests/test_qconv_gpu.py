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
