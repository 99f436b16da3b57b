"""Functional op layer.

Every op has two implementations with the same signature: the plain-PyTorch definition in
:mod:`.reference` (numerics oracle; the CPU path) and a hand-written sm_100a kernel reached through
:mod:`.native`.  CUDA tensors take the native path; when the compiled library is missing on a
machine with a GPU the call raises instead of silently falling back.  ``set_backend("torch")``
forces the PyTorch definitions on GPU as well — that is how the cuBLAS/cuDNN/SDPA baseline runs.
"""
from __future__ import annotations

from . import reference
from .dispatch import (attention, attention_qkv, avg_pool2x2_nhwc, cell_conv_gelu_stack_pool, cell_embed, conv2d_nhwc, conv_gelu_stack_pool, geglu, gelu, get_backend,
                       layer_norm, linear, lm_head_ce, lstm_sequence, rms_norm, set_backend, global_avg_pool_nhwc)

__all__ = ["reference", "attention", "attention_qkv", "avg_pool2x2_nhwc", "cell_embed", "conv2d_nhwc", "geglu", "gelu",
           "get_backend", "layer_norm", "linear", "lm_head_ce", "lstm_sequence", "rms_norm", "set_backend",
           "global_avg_pool_nhwc", "conv_gelu_stack_pool", "cell_conv_gelu_stack_pool"]
