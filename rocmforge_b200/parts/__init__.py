from .base import (Part, Norm, PositionEncoding, Mixer, FeedForward, Block, Registry,
                   NORMS, POSITIONS, MIXERS, FEED_FORWARDS, BLOCKS)
from .linear import Linear
from .norm import RMSNorm
from .rope import NeoxRope
from .attention import GQAAttention
from .mlp import GatedMLP
from .block import PreNormBlock
from .embedding import TokenEmbedding, OutputHead
from .base import NormedMean
from .block import SandwichBlock
from .mlp import SquaredReluMLP
from .experts import RoutedExperts
from .retention import Retention
from .parallel import ParallelMixer
from .offsets import PassOffsets
from .gla import GatedLinearAttention
from .embedding import LearnedPositions
from .norm import DynamicTanh
from .rope import YarnRope
from .block import ScaledPreNormBlock
from .mlp import SummedFeedForward
from .mlstm import MatrixMemory
from .mamba2 import StateSpaceDuality
from .latent import LatentAttention
from .delta import GatedDeltaRule
