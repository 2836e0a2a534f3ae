from .base import (AttentionLike, Block, CacheArray, CacheNeed, Delta, Embedding, FeedForward, Head, Mixer, Norm, Part,
                   PositionEncoding, StateNeed, make_block, make_embedding, make_feed_forward, make_head, make_mixer,
                   make_norm, make_position, register_block, register_embedding, register_feed_forward,
                   register_head, register_mixer, register_norm, register_position)
from . import (attention, blocks, dense, embedding, gated_attention, head, latent_attention, layernorm,  # noqa: F401
               matrix_memory, positions, retention, rmsnorm, rotary_attention, routed, state_space, token_input)  # (importing them registers the built-in kinds)
from .attention import PagedAttention
from .blocks import ParallelBlock, PreNormBlock, SandwichBlock, ScaledPreNormBlock
from .dense import DenseFeedForward, GatedFeedForward, NoFeedForward
from .gated_attention import GatedAttention
from .latent_attention import LatentAttention
from .matrix_memory import MatrixMemoryMixer
from .retention import RetentionMixer
from .rmsnorm import RMSNorm
from .rotary_attention import RotaryAttention
from .rotation import blended_frequencies, rotary_frequencies
from .token_input import TokenGatedInput
from .routed import RoutedFeedForward
from .state_space import StateSpaceMixer
from .embedding import TokenTable
from .head import LinearHead
from .layernorm import LayerNorm, NoNorm
from .positions import LearnedPositions, NoPositions
