from .base import (Block, CacheTensor, CompositeNeed, FeedForward, KVNeed, Mixer, Norm, PagedNeed, Part, PositionEncoding, StateNeed,
                   build_block, build_part, register_part)
from .norm import DeltaSum, LayerNorm, PendingUpdate, RMSNorm, ScalarRMSNorm
from .rope import NoPositionEncoding, RotaryEncoding
from .attention import GQAttention
from .mlp import ActivationMLP, SwiGLU
from .routed_experts import RoutedExperts
from .block import DepthStack, ParallelBlock, PostNormBlock, PreNormBlock
from .gated_recurrence import GatedLinearRecurrence
from .linear_attention import DecayLinearAttention
from .pooled_attention import PooledWindowAttention
from .parallel import ParallelMixer
from .state_space import SelectiveStateSpace
from .latent_attention import LatentAttention
from .masked_attention import MaskedAttention
from .streams import StreamBlock, StreamConnection

__all__ = ["Block", "CacheTensor", "CompositeNeed", "FeedForward", "KVNeed", "Mixer", "Norm", "PagedNeed", "Part", "PositionEncoding",
           "StateNeed",
           "build_block", "build_part", "register_part", "RMSNorm", "NoPositionEncoding", "RotaryEncoding",
           "GQAttention", "SwiGLU", "PreNormBlock", "LayerNorm", "PendingUpdate", "DecayLinearAttention",
           "PooledWindowAttention", "ParallelMixer", "StreamBlock", "StreamConnection", "DeltaSum", "ActivationMLP",
           "RoutedExperts", "ParallelBlock", "SelectiveStateSpace", "LatentAttention", "MaskedAttention",
           "ScalarRMSNorm", "DepthStack", "PostNormBlock", "GatedLinearRecurrence"]
