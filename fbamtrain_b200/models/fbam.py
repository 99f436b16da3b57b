"""The full frame-based action model and its checkpoint naming.

``FbamModel.forward(cells, targets, loss_scale)`` runs the frame head over every frame of the
batch, feeds the ``(B, T, n_embed)`` sequence to the action model and returns the scaled summed
cross-entropy.  ``checkpoint_name_map`` gives, for every parameter, its name and storage layout in
the reference's checkpoint files (reference: ``src/framehead_model.cpp:733-778``,
``tensorlib/include/attention.h:137-159``, ``tensorlib/include/streaming_lstm.h:254-264``,
``toyimpl/src/main.py:599-655``): linear / attention / LSTM / head matrices are stored
``(in, out)``, conv weights ``(O, H, W, I)``, the six colour vectors as separate ``(E,)`` tensors.
"""
from __future__ import annotations

from typing import Optional

from typing import Callable, Dict, List, Tuple

import torch
from torch import nn

from ..config import FbamModelConfiguration
from .action_model import ActionModel
from .frame_head import FrameHead
from .init_utils import SeedSequence

_DT = {"fp16": torch.float16, "bf16": torch.bfloat16, "fp32": torch.float32}


def model_dtype(cfg: FbamModelConfiguration) -> torch.dtype:
    return _DT[cfg.dtype]


class FbamModel(nn.Module):
    def __init__(self, cfg: FbamModelConfiguration, vocab: int):
        super().__init__()
        self.cfg = cfg
        self.vocab = cfg.action_vocab or vocab
        dtype = model_dtype(cfg)
        seeds = SeedSequence(cfg.model_init_seed)
        self.frame_head = FrameHead(cfg, dtype, seeds)
        self.action_model = ActionModel(cfg, self.vocab, dtype, seeds)
        self.frame_chunk = 0  # frames per frame-head call; 0 = all at once

    def frame_head_chunk(self, flat_cells: torch.Tensor, recompute: Optional[bool] = None) -> torch.Tensor:
        """The frame head on ``(frames, P, 3)`` cells.  With ``frame_head_recompute`` nothing but the cells and
        the embeddings is kept for the backward, which runs the frame head on the chunk again — the memory of the
        frame head is then one chunk's activations whatever the sequence length (the reference replays and
        recomputes frame by frame: ``src/main.cpp:3354-3483``).  The second forward does not count as useful FLOPs."""
        if recompute is None:
            recompute = self.cfg.frame_head_recompute
        if recompute and torch.is_grad_enabled():
            import contextlib
            from torch.utils.checkpoint import checkpoint
            from ..utils import flops
            return checkpoint(self.frame_head, flat_cells, use_reentrant=False,
                              context_fn=lambda: (contextlib.nullcontext(), flops.not_useful()))
        return self.frame_head(flat_cells)

    def frame_embeddings(self, cells: torch.Tensor) -> torch.Tensor:
        """``cells`` int32 ``(B, T, P, 3)`` → ``(B, T, n_embed)``."""
        b, t, p, _ = cells.shape
        flat = cells.reshape(b * t, p, 3)
        if self.frame_chunk and flat.shape[0] > self.frame_chunk:
            parts = [self.frame_head_chunk(flat[i:i + self.frame_chunk])
                     for i in range(0, flat.shape[0], self.frame_chunk)]
            emb = torch.cat(parts, 0)
        else:
            emb = self.frame_head_chunk(flat)
        return emb.view(b, t, -1)

    def forward(self, cells: torch.Tensor, targets: torch.Tensor, loss_scale: float) -> torch.Tensor:
        return self.action_model(self.frame_embeddings(cells), targets, loss_scale)


# ---------------------------------------------------------------------------------------------
# checkpoint names / layouts
# ---------------------------------------------------------------------------------------------
_COLOUR_NAMES = ("fg_r_embed", "fg_g_embed", "fg_b_embed", "bg_r_embed", "bg_g_embed", "bg_b_embed")


def _t(x: torch.Tensor) -> torch.Tensor:
    return x.t().contiguous()


def _ident(x: torch.Tensor) -> torch.Tensor:
    return x


# Each entry: internal parameter name -> list of (checkpoint name, to_ckpt(tensor), from_ckpt(tensor, internal)->None)
Entry = Tuple[str, Callable[[torch.Tensor], torch.Tensor], Callable[[torch.Tensor], torch.Tensor]]


def checkpoint_name_map(model: FbamModel) -> Dict[str, List[Entry]]:
    """Internal name → [(checkpoint name, internal→stored transform, stored→internal transform)].
    The colour matrix is the only parameter that maps to several stored tensors (one per row)."""
    out: Dict[str, List[Entry]] = {}
    for name, p in model.named_parameters():
        parts = name.split(".")
        scope, rest = parts[0], parts[1:]
        transform_to, transform_from = _ident, _ident
        if scope == "frame_head":
            if rest[0] == "embed":
                if rest[1] == "colour":
                    out[name] = [(f"frame_head.{cn}", (lambda x, i=i: x[i].contiguous()), _ident)
                                 for i, cn in enumerate(_COLOUR_NAMES)]
                    continue
                ck = {"codepoint_embedding": "frame_head.codepoint_embedding",
                      "position_embedding": "frame_head.position_embedding.weight"}[rest[1]]
            elif rest[0] == "downsample_block":
                leaf = {"ln": "ln.weight", "conv_weight": "conv.weight"}[rest[2]]
                ck = f"frame_head.downsample_block.{rest[1]}.{leaf}"
            elif rest[0] == "block":
                ck, transform_to, transform_from = _block_entry("frame_head", rest)
            else:  # proj
                ck = "frame_head.proj." + rest[1]
                if rest[1] == "weight":
                    transform_to = transform_from = _t
        else:
            if rest[0] == "lstm":
                layer, leaf = int(rest[2]), rest[3]
                prefix = "action_model.lstm" if layer == 0 else f"action_model.lstm.{layer}"
                ck = f"{prefix}.{leaf}"
                if leaf in ("weights_ih", "weights_hh"):
                    transform_to = transform_from = _t
            elif rest[0] == "block":
                ck, transform_to, transform_from = _block_entry("action_model", rest)
            elif rest[0] == "ln_f":
                ck = "action_model.ln_f.weight"
            else:
                ck = "action_model.head.weight"
                transform_to = transform_from = _t
        out[name] = [(ck, transform_to, transform_from)]
    return out


def _block_entry(scope: str, rest):
    idx, sub = rest[1], rest[2:]
    base = f"{scope}.block.{idx}."
    if sub[0] in ("ln1", "ln2"):
        return base + f"{sub[0]}.weight", _ident, _ident
    if sub[0] == "attn":
        which = {"qkv": "qkv", "proj": "proj"}[sub[1]]
        if sub[2] == "weight":
            return base + f"attn.w_{which}", _t, _t
        return base + f"attn.b_{which}", _ident, _ident
    # mlp
    if sub[2] == "weight":
        return base + f"mlp.{sub[1]}.weight", _t, _t
    return base + f"mlp.{sub[1]}.bias", _ident, _ident
