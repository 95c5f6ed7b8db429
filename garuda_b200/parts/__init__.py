"""Parts a decoder is put together from. Importing the package registers the
built-in ones."""
from .base import (Part, Norm, PositionEncoding, Mixer, FeedForward, ResidualBranch, Connection, TensorSpec, PagedKV,
                   PagedLatent, FixedState, LayerCache, PartSpec, build_part, register_mixer,
                   register_feed_forward, register_norm, register_position_encoding,
                   register_block, register_branch, register_connection, register_gate,
                   SublayerGate)
from .norm import RMSNorm, LayerNorm
from .rotary import Rotary, NoPositions, RotaryParams
from .attention import PagedAttention, CappedSinkAttention, NormedKeyAttention, ConvolvedAttention
from .mingru import MinGRU
from .delta_rule import ChannelDeltaRule, HeadDeltaRule, GeneralDeltaRule
from .mlp import SwiGLU, GatedFeedForward, PlainFeedForward
from .latent_attention import LatentAttention
from .experts import RoutedExperts
from .token_side import TokenSide
from .block import BlockSpec, PreNormBlock, SublayerNormBlock, PostNormBlock, LinearSigmoidGate, BranchOutputs
from .parallel import ParallelMixers
from .hyper import StreamMixing, StreamPreNormBlock
