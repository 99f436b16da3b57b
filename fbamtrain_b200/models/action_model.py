"""Action model: streaming LSTM → causal attention blocks → linear head → cross-entropy.

The reference's action model is a one-layer LSTM and a bias-free head whose loss is
``Σ CE / (T · total_batch)`` with targets ``token_id mod vocab`` and the head width padded to a
multiple of 8 (reference: ``src/main_action_model.cpp:15-18, 117-203``, ``src/main.cpp:2231-2236,
2428``).  With ``action_blocks > 0`` causal MHA / GELU-MLP / RMSNorm blocks (and a final RMSNorm)
sit between the LSTM and the head.
"""
from __future__ import annotations


import torch
from torch import nn

from .. import ops
from ..config import FbamModelConfiguration
from .blocks import AttentionBlock, RmsNorm
from .init_utils import SeedSequence, fill_uniform_fan_
from .streaming_lstm import StreamingLstm


def padded_vocab(vocab: int) -> int:
    return (vocab + 7) // 8 * 8


class ActionModel(nn.Module):
    def __init__(self, cfg: FbamModelConfiguration, vocab: int, dtype: torch.dtype, seeds: SeedSequence):
        super().__init__()
        self.cfg, self.vocab = cfg, vocab
        h = cfg.hidden
        self.lstm = StreamingLstm(cfg.n_embed, h, cfg.lstm_layers, dtype, seeds,
                                  cfg.streaming_chunk_size, cfg.recompute_interval)
        self.block = nn.ModuleList(
            [AttentionBlock(h, cfg.heads_action, cfg.mlp_dim if cfg.action_mlp_dim else 4 * h, cfg.bias, True,
                            cfg.rms_norm_eps, dtype, seeds) for _ in range(cfg.action_blocks)])
        self.ln_f = RmsNorm(h, cfg.rms_norm_eps, dtype) if cfg.action_blocks > 0 else None
        self.head_weight = nn.Parameter(torch.empty(padded_vocab(vocab), h, dtype=dtype))
        fill_uniform_fan_(self.head_weight.data, h, seeds)
        # The reference's model (one LSTM layer straight into the head) can be streamed chunk by chunk with the
        # head / loss computed per chunk; ``host_offload`` additionally keeps the stored dY chunks in pinned memory.
        self.streaming = cfg.action_blocks == 0 and cfg.lstm_layers == 1
        self.host_offload = False

    def features(self, frame_embeddings: torch.Tensor, state=None):
        """``(B, T, E)`` → hidden states ``(B, T, H)`` and the LSTM's final state."""
        y, st = self.lstm(frame_embeddings.transpose(0, 1).contiguous(), state)
        x = y.transpose(0, 1).contiguous()
        for blk in self.block:
            x = blk(x)
        if self.ln_f is not None:
            x = self.ln_f(x)
        return x, st

    def logits(self, hidden: torch.Tensor) -> torch.Tensor:
        return ops.linear(hidden.reshape(-1, hidden.shape[-1]), self.head_weight, None)[:, : self.vocab]

    def forward(self, frame_embeddings: torch.Tensor, targets: torch.Tensor, loss_scale: float, state=None):
        """Returns ``loss_scale · Σ CE`` over all ``B·T`` positions."""
        if (self.streaming and state is None and frame_embeddings.is_cuda and ops.get_backend() == "auto"
                and frame_embeddings.dtype in (torch.bfloat16, torch.float16)):
            from ..ops.lstm import persistent_ok
            layer = self.lstm.layers[0]
            b, t, e = frame_embeddings.shape
            if persistent_ok(b, layer.hidden) and e % 8 == 0:
                from ..ops.streaming import streaming_lstm_head_ce
                return streaming_lstm_head_ce(frame_embeddings.transpose(0, 1).contiguous(), layer.weights_ih,
                                              layer.weights_hh, layer.bias_ih, layer.bias_hh, layer.h0, layer.c0,
                                              self.head_weight, targets.t().contiguous(), self.vocab, loss_scale,
                                              max(1, self.lstm.chunk_size), self.host_offload)
        x, _ = self.features(frame_embeddings, state)
        return ops.lm_head_ce(x.reshape(-1, x.shape[-1]), self.head_weight, targets.reshape(-1), self.vocab, loss_scale)
