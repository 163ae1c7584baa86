"""Parts of a model: norm, position encoding, mixer, feed-forward, block; and the model built of them."""
from .base import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITIONS, ResidualStream, Runtime, StepContext, part_class,
                   register)
from .program import HostIO, Program, ProgramRunner
from .norm import RMSNorm
from .rope import RotaryTables
from .attention import Attention
from .feed_forward import SwiGLU
from .block import PreNormBlock
from .layernorm import LayerNorm
from .glu import GLU
from .linear_attention import LinearAttention
from .conv_attention import ConvAttention
from .postnorm_block import PostNormBlock
from .latent_attention import LatentAttention
from .selective_scan import SelectiveScan
from .routed_experts import RoutedExperts
from .sandwich_block import SandwichBlock
from .reinject import Reinject
from .mlp import MLP
from .parallel_mixer import ParallelMixer
from .step_vector import StepVector
from .delta_rule import DeltaRule
from .model import Model, cache_needs, model_manifest, state_needs

__all__ = ["BLOCKS", "FEED_FORWARDS", "MIXERS", "NORMS", "POSITIONS", "ResidualStream", "Runtime", "StepContext", "Program",
           "ProgramRunner", "HostIO", "part_class", "register", "RMSNorm", "RotaryTables", "Attention", "SwiGLU",
           "PreNormBlock", "LayerNorm", "GLU", "LinearAttention", "ConvAttention", "PostNormBlock", "LatentAttention",
           "SelectiveScan", "RoutedExperts", "SandwichBlock", "Reinject", "MLP", "ParallelMixer", "StepVector", "DeltaRule", "Model", "cache_needs", "model_manifest",
           "state_needs"]
