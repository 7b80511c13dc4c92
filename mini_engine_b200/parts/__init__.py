from .base import (AddedToResidual, PendingNorm, Upcoming, DiskSource, FeedForward, KVCacheNeed, Mixer, Norm, ParamDecl, Part,
                   PositionEncoding, StateNeed)
from .registry import (PartSpec, build_block, build_part, register_block, register_feed_forward, register_mixer,
                       register_norm, register_position_encoding, registered)
from .norm import RMSNorm
from .rope import RotaryEmbedding
from .linear import Linear
from .attention import GQAAttention
from .mlp import SwiGLU
from .embed import LMHead, TokenEmbedding
from .block import Block, BlockSpec, PreNormBlock, SharedRef
from .model import DecoderModel, LayerCall, ModelPlan
