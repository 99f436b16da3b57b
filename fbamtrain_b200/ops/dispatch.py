"""Backend selection for the functional ops (see the package docstring)."""
from __future__ import annotations

from typing import Optional

import torch

from . import reference as ref

import os

_BACKEND = "auto"  # "auto": native kernels for CUDA tensors, PyTorch on CPU; "torch": PyTorch everywhere

# Per-family preference from the environment, as the reference's FBAMTRAIN_PREFER_{GEMM,CONV2D,MHA}_BACKEND
# (reference: ``src/passes/matmul_pass.cpp:35-62``, ``conv2d_pass.cpp:140-172``, ``mha_attention_pass.cpp:290-313``).
# Values: "native" (the sm_100a kernels of this package; the default) or "torch" (the vendor-library path).
_FAMILIES = ("gemm", "conv2d", "mha")
_prefer = {}
_last = {}


def _read_preferences() -> None:
    _prefer.clear()
    for fam in _FAMILIES:
        raw = os.environ.get(f"FBAMTRAIN_PREFER_{fam.upper()}_BACKEND", "native").strip().lower()
        if raw not in ("native", "torch"):
            raise ValueError(f"FBAMTRAIN_PREFER_{fam.upper()}_BACKEND must be 'native' or 'torch', got '{raw}'")
        _prefer[fam] = raw


_read_preferences()


def last_backend(family: str) -> str:
    """Which implementation the most recent call of an op family used: "native", "torch" or "" (not called yet).
    Tests assert on it the way the reference's tests assert that the expected backend was chosen."""
    return _last.get(family, "")


def set_backend(name: str) -> None:
    global _BACKEND
    if name not in ("auto", "torch"):
        raise ValueError("backend must be 'auto' or 'torch'")
    _BACKEND = name


def get_backend() -> str:
    return _BACKEND


_warned_dtypes = set()


def _native(t: torch.Tensor, dtype: Optional[torch.dtype] = None, family: Optional[str] = None) -> bool:
    """The hand-written kernels compute in bf16 or fp16 (fp32 accumulate; one library per element type).  CUDA
    tensors of another activation dtype (fp32 debugging runs) take the PyTorch definitions, i.e. the vendor
    libraries."""
    use = _native_inner(t, dtype, family)
    if family is not None:
        _last[family] = "native" if use else "torch"
    return use


def _native_inner(t: torch.Tensor, dtype: Optional[torch.dtype], family: Optional[str]) -> bool:
    if not (t.is_cuda and _BACKEND == "auto"):
        return False
    if family is not None and _prefer.get(family, "native") == "torch":
        return False
    dtype = dtype or t.dtype
    if dtype in (torch.bfloat16, torch.float16):
        return True
    if dtype not in _warned_dtypes:
        _warned_dtypes.add(dtype)
        from ..utils.logging import LOG
        LOG("WARN", f"ops: {dtype} activations on a GPU run on the PyTorch / vendor-library path; the sm_100a kernels "
                    "of this package compute in bf16 or fp16")
    return False


def cell_embed(cells, cp_embed, pos_embed, colour_embed, out_dtype):
    if _native(cells, out_dtype):
        from .native_ops import cell_embed as f
        return f(cells, cp_embed, pos_embed, colour_embed, out_dtype)
    return ref.cell_embed(cells, cp_embed, pos_embed, colour_embed, out_dtype)


def conv2d_nhwc(x, w_ohwi, stride: int, padding: int, dilation: int):
    # the implicit-GEMM kernels tile the input channels in blocks of 64; other channel counts take the library
    if x.shape[3] % 64 == 0 and _native(x, family="conv2d"):
        from .native_ops import conv2d_nhwc as f
        return f(x, w_ohwi, stride, padding, dilation)
    return ref.conv2d_nhwc(x, w_ohwi, stride, padding, dilation)


def rms_norm(x, weight, eps: float):
    if _native(x):
        from .native_ops import rms_norm as f
        return f(x, weight, eps)
    return ref.rms_norm(x, weight, eps)


def layer_norm(x, weight, bias, eps: float):
    if _native(x):
        from .native_ops import layer_norm as f
        return f(x, weight, bias, eps)
    return ref.layer_norm(x, weight, bias, eps)


def gelu(x):
    if _native(x):
        from .native_ops import gelu as f
        return f(x)
    return ref.gelu(x)


def geglu(x):
    if _native(x):
        from .native_ops import geglu as f
        return f(x)
    return ref.geglu(x)


def avg_pool2x2_nhwc(x):
    if _native(x):
        from .native_ops import avg_pool2x2_nhwc as f
        return f(x)
    return ref.avg_pool2x2_nhwc(x)


def global_avg_pool_nhwc(x):
    """``(N, H, W, C)`` → ``(N, C)`` mean over the spatial positions (fp32 accumulate)."""
    if _native(x):
        from .native_ops import global_avg_pool_nhwc as f
        return f(x)
    return x.float().mean(dim=(1, 2)).to(x.dtype)


def conv_gelu_stack_pool(x, weights, stride: int, paddings, dilations):
    """``[conv3x3 (no bias) → GELU] x n → mean over positions``: ``(N, H, W, C)`` → ``(N, C_last)``."""
    if _native(x, family="conv2d") and all(w.shape[3] % 64 == 0 for w in weights):
        from .native_ops import conv_gelu_stack_pool as f
        return f(x, weights, stride, paddings, dilations)
    for w, pad, dil in zip(weights, paddings, dilations):
        x = gelu(conv2d_nhwc(x, w, stride, pad, dil))
    return global_avg_pool_nhwc(x)


def embconv_enabled() -> bool:
    """``FBAMTRAIN_EMBCONV=0`` keeps the cell embedding and the first convolution as separate kernels."""
    return os.environ.get("FBAMTRAIN_EMBCONV", "1") != "0"


def cell_conv_gelu_stack_pool(cells, cp_embed, pos_embed, colour_embed, rows: int, cols: int, out_dtype, weights,
                              stride: int, paddings, dilations):
    """``cells (N, rows·cols, 3)`` → cell embedding → ``[conv3x3 (no bias) → GELU] x n`` → mean over positions
    ``(N, C_last)``.  On the native path the embedding and the first convolution are fused into table look-ups
    (``ops/embconv.py``) when the shapes allow; otherwise this is the composition of the separate ops."""
    if (_native(cells, out_dtype, family="conv2d") and embconv_enabled() and
            all(w.shape[3] % 64 == 0 for w in weights)):
        from . import embconv
        if embconv.supported(cells, cp_embed, weights[0]):
            from .native_ops import cell_conv_gelu_stack_pool as f
            return f(cells, cp_embed, pos_embed, colour_embed, rows, cols, weights, stride, paddings, dilations)
    x = cell_embed(cells, cp_embed, pos_embed, colour_embed, out_dtype).view(cells.shape[0], rows, cols, -1)
    return conv_gelu_stack_pool(x, weights, stride, paddings, dilations)


def linear(x, weight, bias: Optional[torch.Tensor] = None, act: str = "none",
           residual: Optional[torch.Tensor] = None):
    """``act(x·Wᵀ + b) [+ residual]``; on the native path the residual rides in the GEMM epilogue."""
    if _native(x, family="gemm"):
        from .native_ops import linear as f
        return f(x, weight, bias, act, residual)
    y = ref.linear(x, weight, bias, act)
    return y if residual is None else y + residual.reshape(y.shape)


def attention(q, k, v, causal: bool):
    if _native(q, family="mha"):
        from .native_ops import attention as f
        return f(q, k, v, causal)
    if q.is_cuda:  # PyTorch baseline on GPU: library flash attention
        import torch.nn.functional as F
        o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=causal)
        return o.transpose(1, 2).contiguous()
    return ref.attention(q, k, v, causal)


def attention_qkv(qkv, causal: bool):
    """Attention on a fused projection output ``(B, T, 3, H, D)`` (q, k, v along dimension 2) → ``(B, T, H, D)``."""
    if _native(qkv, family="mha"):
        from .mha import flash_attention_qkv
        return flash_attention_qkv(qkv, causal)
    return attention(qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2], causal)


def lstm_sequence(x, w_ih, w_hh, b_ih, b_hh, h0, c0, compute_dtype):
    if _native(x, compute_dtype) and x.dtype == compute_dtype:
        from .native_ops import lstm_sequence as f
        return f(x, w_ih, w_hh, b_ih, b_hh, h0, c0, compute_dtype)
    if x.is_cuda and h0.dim() == 1:
        # PyTorch baseline on GPU: the library (cuDNN) LSTM instead of a Python loop over time steps
        b = x.shape[1]
        params = [w_ih.to(compute_dtype), w_hh.to(compute_dtype), b_ih.to(compute_dtype), b_hh.to(compute_dtype)]
        hx = (h0.to(compute_dtype).expand(1, b, -1).contiguous(), c0.to(compute_dtype).expand(1, b, -1).contiguous())
        y, h_n, c_n = torch._VF.lstm(x.to(compute_dtype), hx, params, True, 1, 0.0, True, False, False)
        return y, h_n[0], c_n[0].float()
    return ref.lstm_sequence(x, w_ih, w_hh, b_ih, b_hh, h0, c0, compute_dtype)


def lm_head_ce(x, w_head, targets, vocab: int, scale: float):
    if _native(x):
        from .native_ops import lm_head_ce as f
        return f(x, w_head, targets, vocab, scale)
    return ref.lm_head_ce(x, w_head, targets, vocab, scale)
