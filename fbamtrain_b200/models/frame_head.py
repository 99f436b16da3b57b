"""Frame head: cell embedding → downsample convolutions → (optional) attention blocks → one vector per frame.

Reference structure (``src/framehead_model.cpp:126-175, 339-398, 601-731``): per downsample block
``RMSNorm → conv3x3 (no bias; "dilated": padding = dilation, "geglu": 2C outputs, padding 1) →
GELU (or value·GELU(gate)) → avg_pool2d 2x2``; then ``n_layer`` non-causal attention blocks over the
remaining cells; then mean over cells or the last cell.  Additions, selected by configuration keys
whose defaults reproduce the above: a stride-2 convolution instead of conv+pool, no RMSNorm in front
of the convolutions, per-block channel counts, and a linear projection of the pooled vector.
"""
from __future__ import annotations


import torch
from torch import nn

from .. import ops
from ..config import FbamModelConfiguration
from .blocks import AttentionBlock, Linear, RmsNorm
from .init_utils import SeedSequence, fill_normal_, fill_uniform_fan_


class CellEmbed(nn.Module):
    """Code-point table, position table and six colour-channel vectors, all fp32
    (reference: ``src/framehead_model.cpp:548-554, 733-745``)."""

    def __init__(self, cfg: FbamModelConfiguration, dtype: torch.dtype, seeds: SeedSequence):
        super().__init__()
        e, p = cfg.embed_dim, cfg.frame_rows * cfg.frame_cols
        self.out_dtype = dtype
        self.codepoint_embedding = nn.Parameter(torch.empty(cfg.max_code_point, e, dtype=torch.float32))
        fill_normal_(self.codepoint_embedding.data, seeds)
        self.colour = nn.Parameter(torch.empty(6, e, dtype=torch.float32))  # fg r,g,b then bg r,g,b
        for i in range(6):
            fill_normal_(self.colour.data[i], seeds)
        self.position_embedding = nn.Parameter(torch.empty(p, e, dtype=torch.float32))
        fill_normal_(self.position_embedding.data, seeds)

    def forward(self, cells: torch.Tensor) -> torch.Tensor:
        return ops.cell_embed(cells, self.codepoint_embedding, self.position_embedding, self.colour, self.out_dtype)


class DownsampleBlock(nn.Module):
    def __init__(self, cfg: FbamModelConfiguration, c_in: int, c_out: int, dtype: torch.dtype, seeds: SeedSequence):
        super().__init__()
        self.mode, self.stride = cfg.downsample_conv_mode, cfg.downsample_conv_stride
        self.dilation = cfg.downsample_conv_dilation if self.mode == "dilated" else 1
        self.padding = self.dilation
        self.ln = RmsNorm(c_in, cfg.rms_norm_eps, dtype) if cfg.downsample_norm else None
        conv_out = 2 * c_out if self.mode == "geglu" else c_out
        self.conv_weight = nn.Parameter(torch.empty(conv_out, 3, 3, c_in, dtype=dtype))  # OHWI
        fill_uniform_fan_(self.conv_weight.data, 9 * c_in, seeds)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.ln is not None:
            x = self.ln(x)
        x = ops.conv2d_nhwc(x, self.conv_weight, self.stride, self.padding, self.dilation)
        x = ops.geglu(x) if self.mode == "geglu" else ops.gelu(x)
        if self.stride == 1:
            x = ops.avg_pool2x2_nhwc(x)
        return x


class FrameHead(nn.Module):
    def __init__(self, cfg: FbamModelConfiguration, dtype: torch.dtype, seeds: SeedSequence):
        super().__init__()
        self.cfg = cfg
        self.embed = CellEmbed(cfg, dtype, seeds)
        self.downsample_block = nn.ModuleList(
            [DownsampleBlock(cfg, ci, co, dtype, seeds) for ci, co in cfg.block_channels()])
        feat = cfg.frame_feature_dim
        self.block = nn.ModuleList(
            [AttentionBlock(feat, cfg.n_head, 4 * feat, cfg.bias, False, cfg.rms_norm_eps, dtype, seeds)
             for _ in range(cfg.n_layer)])
        self.proj = Linear(feat, cfg.n_embed, cfg.bias, dtype, seeds) if cfg.frame_proj else None
        if not cfg.frame_proj and feat != cfg.n_embed:
            raise ValueError("frame feature width differs from n_embed: enable 'frame_proj'")

    def forward(self, cells: torch.Tensor) -> torch.Tensor:
        """``cells`` int32 ``(N, rows*cols, 3)`` → ``(N, n_embed)``."""
        cfg = self.cfg
        n = cells.shape[0]
        fusable = (len(self.block) == 0 and cfg.frame_head_reduction_strategy == "mean" and
                   len(self.downsample_block) > 0 and
                   all(b.ln is None and b.mode == "dilated" and b.stride == 2 for b in self.downsample_block))
        if fusable:   # cells → (embedding + first conv as table look-ups) → conv → GELU chain → pooled frame vector
            blocks, emb = self.downsample_block, self.embed
            v = ops.cell_conv_gelu_stack_pool(cells, emb.codepoint_embedding, emb.position_embedding, emb.colour,
                                              cfg.frame_rows, cfg.frame_cols, emb.out_dtype,
                                              [b.conv_weight for b in blocks], 2, [b.padding for b in blocks],
                                              [b.dilation for b in blocks])
            return self.proj(v) if self.proj is not None else v
        x = self.embed(cells).view(n, cfg.frame_rows, cfg.frame_cols, cfg.embed_dim)
        for blk in self.downsample_block:
            x = blk(x)
        if len(self.block) == 0 and cfg.frame_head_reduction_strategy == "mean":
            v = ops.global_avg_pool_nhwc(x)
        else:
            tok = x.reshape(n, -1, x.shape[-1])
            for blk in self.block:
                tok = blk(tok)
            if cfg.frame_head_reduction_strategy == "mean":
                v = tok.float().mean(dim=1).to(tok.dtype)
            else:
                v = tok[:, -1, :]
        if self.proj is not None:
            v = self.proj(v)
        return v
