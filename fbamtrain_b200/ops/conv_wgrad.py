"""Convolution weight gradient ``dW[o, r, s, c] = Σ_{n,oh,ow} dY[n,oh,ow,o] · X[n, oh·stride + r·dil − pad, …, c]``."""
from __future__ import annotations

import torch


def conv2d_wgrad(x, dy, w_shape, stride, padding, dilation):
    # Interim: library kernel.  The tcgen05 split-K wgrad replaces this.
    o, _, _, c = w_shape
    dw = torch.nn.grad.conv2d_weight(x.permute(0, 3, 1, 2), (o, c, 3, 3), dy.permute(0, 3, 1, 2), stride, padding,
                                     dilation)
    return dw.permute(0, 2, 3, 1).contiguous()
