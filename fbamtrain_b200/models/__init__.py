"""Model family: cell-embedding + convolutional frame head, streaming LSTM + causal-attention action model."""
from .frame_head import CellEmbed, DownsampleBlock, FrameHead
from .blocks import AttentionBlock, Embedding, Mean, MlpBlock, RmsNorm, LayerNorm, Linear, FullMhaAttention
from .streaming_lstm import StreamingLstm
from .action_model import ActionModel
from .fbam import FbamModel, model_dtype, checkpoint_name_map

__all__ = ["Embedding", "Mean", "CellEmbed", "DownsampleBlock", "FrameHead", "AttentionBlock", "MlpBlock", "RmsNorm", "LayerNorm",
           "Linear", "FullMhaAttention", "StreamingLstm", "ActionModel", "FbamModel", "model_dtype",
           "checkpoint_name_map"]
