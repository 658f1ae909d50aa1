from .attention import CausalSelfAttention
from .base import Block, FeedForward, Mixer, Norm, Part, PositionEncoding
from .block import OutputNormBlock, ParallelBlock, PreNormBlock, SandwichBlock
from .conv_attention import TalkingConvAttention
from .embedding import LinearReadout, StreamVectors, TiedReadout, TokenEmbedding
from .feed_forward import DenseFeedForward, GatedFeedForward, PolyNormFeedForward
from .latent_attention import LatentAttention
from .lightning import LightningAttention, Retention
from .matrix_memory import MatrixMemory
from .norm import LayerNorm, RmsNorm
from .routed import RoutedFeedForward
from .selective_scan import SelectiveScan
from .side_by_side import SideBySideMixers
from .sigmoid_attention import SigmoidAttention
from .token_shift import TokenShift
from .position import HalfSplitRotary, InterleavedRotary, LearnedPositions, NoPositions

__all__ = ["CausalSelfAttention", "Block", "FeedForward", "Mixer", "Norm", "Part", "PositionEncoding", "PreNormBlock",
           "LinearReadout", "StreamVectors", "TiedReadout", "TokenEmbedding", "DenseFeedForward", "GatedFeedForward", "LatentAttention",
           "LightningAttention", "MatrixMemory", "ParallelBlock", "RoutedFeedForward", "SideBySideMixers",
           "LayerNorm", "RmsNorm", "InterleavedRotary", "LearnedPositions", "NoPositions", "SandwichBlock",
           "TalkingConvAttention", "PolyNormFeedForward", "Retention", "SelectiveScan", "HalfSplitRotary", "OutputNormBlock",
           "SigmoidAttention", "TokenShift"]
