"""Host-side logic of the convolution layers, on the CPU: the space-to-depth regrouping that turns a strided convolution into a
unit-stride one, and the output shapes / paddings of QConv1D against torch's own convolutions."""

import pytest
import torch
import torch.nn.functional as F


@pytest.mark.parametrize('H,W,C,N,KH,KW,sh,sw,pads', [
    (9, 8, 3, 8, 3, 3, 2, 2, ((0, 0), (0, 0))),
    (9, 8, 3, 8, 3, 3, 2, 2, ((1, 1), (0, 1))),        # 'same' at stride 2
    (6, 6, 2, 4, 1, 1, 3, 5, ((0, 0), (0, 0))),        # the parameter sets of the reference's own test (tests/test_conv.py:66-73)
    (6, 6, 2, 4, 3, 2, 1, 3, ((1, 1), (0, 0))),
    (6, 6, 2, 4, 2, 3, 4, 2, ((0, 0), (0, 1))),
    (17, 19, 4, 4, 2, 3, 4, 2, ((0, 0), (0, 0))),
    (1, 14, 4, 16, 1, 3, 1, 2, ((0, 0), (2, 0))),      # a 1-D layer with causal padding at stride 2
])
def test_space_to_depth_operands_give_the_strided_convolution(H, W, C, N, KH, KW, sh, sw, pads):
    from hgq2_b200.layers._functions import space_to_depth_operands

    gen = torch.Generator().manual_seed(H * 100 + W)
    x = torch.randint(-8, 8, (3, H, W, C), generator=gen).float() / 8       # small integers: every sum is exact in fp32
    w = torch.randint(-8, 8, (KH, KW, C, N), generator=gen).float() / 8
    (pt, pb), (pl, pr) = pads
    ref = F.conv2d(F.pad(x.permute(0, 3, 1, 2), (pl, pr, pt, pb)), w.permute(3, 2, 0, 1).contiguous(), stride=(sh, sw)).permute(0, 2, 3, 1)
    OH, OW = ref.shape[1:3]
    xs, ws = space_to_depth_operands(x, w, (pt, pl), (sh, sw), (OH, OW))
    assert xs.shape == (3, OH + ws.shape[0] - 1, OW + ws.shape[1] - 1, sh * sw * C) and ws.shape[2:] == (sh * sw * C, N)
    y = F.conv2d(xs.permute(0, 3, 1, 2), ws.permute(3, 2, 0, 1).contiguous()).permute(0, 2, 3, 1)
    assert torch.equal(y, ref)
    # the regrouping is differentiable: gradients flow back to the image and the kernel as through the strided convolution
    x1, w1 = x.clone().requires_grad_(), w.clone().requires_grad_()
    x2, w2 = x.clone().requires_grad_(), w.clone().requires_grad_()
    g = torch.randint(-4, 4, ref.shape, generator=gen).float()
    (F.conv2d(F.pad(x1.permute(0, 3, 1, 2), (pl, pr, pt, pb)), w1.permute(3, 2, 0, 1), stride=(sh, sw)).permute(0, 2, 3, 1) * g).sum().backward()
    a, b = space_to_depth_operands(x2, w2, (pt, pl), (sh, sw), (OH, OW))
    (F.conv2d(a.permute(0, 3, 1, 2), b.permute(3, 2, 0, 1)).permute(0, 2, 3, 1) * g).sum().backward()
    assert torch.equal(x1.grad, x2.grad) and torch.equal(w1.grad, w2.grad)


@pytest.mark.parametrize('padding', ['valid', 'same', 'causal'])
@pytest.mark.parametrize('kernel_size,strides,dilation', [(1, 2, 1), (3, 1, 1), (2, 2, 1), (3, 1, 2), (5, 3, 1)])
@pytest.mark.parametrize('steps', [6, 14, 15])
def test_qconv1d_shapes_and_paddings(padding, kernel_size, strides, dilation, steps):
    """compute_output_shape and the paddings of QConv1D follow keras' Conv1D rules ('same': ceil(steps / stride) outputs with the
    surplus padding behind; 'causal': (kernel_size - 1) dilation zeros in front)."""
    from hgq2_b200.layers import QConv1D

    layer = QConv1D(4, kernel_size, strides=strides, padding=padding, dilation_rate=dilation)
    (pt, pb), (pl, pr) = layer._pads(1, steps)
    assert (pt, pb) == (0, 0)
    out = layer.compute_output_shape((2, steps, 3))
    x = torch.zeros(2, 3, steps + pl + pr)
    ref_len = F.conv1d(x, torch.zeros(4, 3, kernel_size), stride=strides, dilation=dilation).shape[-1]
    assert out == (2, ref_len, 4)
    span = (kernel_size - 1) * dilation
    if padding == 'valid':
        assert (pl, pr) == (0, 0)
    elif padding == 'causal':
        assert (pl, pr) == (span, 0) and ref_len == (steps - 1) // strides + 1
    else:
        assert ref_len == -(-steps // strides) and pl <= pr <= pl + 1
