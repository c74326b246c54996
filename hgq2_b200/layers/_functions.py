"""torch.autograd bridges between the layer classes and the CUDA kernels."""

from __future__ import annotations

import torch

from .. import kernels

_ones: dict = {}


def _one(device) -> torch.Tensor:
    t = _ones.get(device)
    if t is None:
        t = torch.ones((), dtype=torch.float32, device=device)
        _ones[device] = t
    return t


class EbopsDenseFn(torch.autograd.Function):
    """ebops = scale * (sum(bw_in @ bw_w) + mean(bw_bias) * out_size); gradient to the three bitwidth tensors."""

    @staticmethod
    def forward(ctx, bw_in, bw_w, bw_bias, out_size, scale):
        _, e_f, _, d_in, d_w, d_b = kernels.ebops_dense(bw_in, bw_w, bw_bias, out_size, scale, _one(bw_in.device))
        ctx.save_for_backward(d_in, d_w, d_b)
        return e_f

    @staticmethod
    def backward(ctx, g):
        d_in, d_w, d_b = ctx.saved_tensors
        return g * d_in, g * d_w, (g * d_b if d_b is not None else None), None, None


class EbopsConv2dFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, bw_in, bw_w, bw_bias, out_hw, strides, dilation, pad_tl, out_size, scale_main, scale_bias):
        _, e_f, _, d_in, d_w, d_b = kernels.ebops_conv2d(bw_in, bw_w, bw_bias, out_hw, strides, dilation, pad_tl, out_size,
                                                         scale_main, scale_bias, _one(bw_in.device))
        ctx.save_for_backward(d_in, d_w, d_b)
        return e_f

    @staticmethod
    def backward(ctx, g):
        d_in, d_w, d_b = ctx.saved_tensors
        return g * d_in, g * d_w, (g * d_b if d_b is not None else None), None, None, None, None, None, None, None
