"""Parts that layers are put together from: norms, position encodings, mixers, feed-forwards, blocks."""
from .base import (Block, CacheSpec, FeedForward, LayerSlot, Mixer, Norm, Part, PositionEncoding, StateSpec,
                   StepContext, StreamOp, make_part, part_kinds, register_part)
from .linear import GroupedLinear, Linear
from .norm import DynamicTanh, L2Norm, LayerNorm, RMSNorm
from .position import (NoPositionEncoding, RotaryEncoding, leading_rotary_inv_freq, partial_rotary_inv_freq,
                       rotary_inv_freq, yarn_inv_freq)
from .attention import PagedAttention, distance_bias_table, distance_bucket
from .latent import LatentAttention
from .mlstm import MLSTMMixer, fused_mlstm_columns
from .feedforward import DenseMLP, DenseSwiGLU, MoESigmoidTop1, MoESigmoidTopK, MoESigmoidTopKGated
from .block import ParallelBlock, PreNormBlock
from .stream import ReinjectInput
from .hyper import GroupRMSNorm, HyperBlock, PairEmbedding
from .wkv import WKVMixer
from .mamba import BranchPair, SelectiveScanMixer, StateSpaceDualityMixer, ssd_projection_order

__all__ = ["Block", "CacheSpec", "FeedForward", "LayerSlot", "Mixer", "Norm", "Part", "PositionEncoding",
           "StateSpec", "StepContext", "make_part", "part_kinds", "register_part", "GroupedLinear", "Linear",
           "L2Norm", "RMSNorm", "NoPositionEncoding", "RotaryEncoding", "rotary_inv_freq", "PagedAttention",
           "DenseSwiGLU", "MoESigmoidTop1", "PreNormBlock", "StreamOp", "partial_rotary_inv_freq", "MLSTMMixer",
           "fused_mlstm_columns", "DenseMLP", "MoESigmoidTopK", "ParallelBlock", "ReinjectInput", "GroupRMSNorm",
           "HyperBlock", "PairEmbedding", "WKVMixer", "BranchPair", "SelectiveScanMixer", "leading_rotary_inv_freq", "DynamicTanh", "LatentAttention", "MoESigmoidTopKGated", "StateSpaceDualityMixer",
           "ssd_projection_order", "distance_bias_table", "distance_bucket", "LayerNorm", "yarn_inv_freq"]
