from .base import (Block, CompositeRequest, FeedForward, KeyValueRequest, LayerSpec, Mixer, ModelPlan, Norm,
                   Part, PartSpec, PositionEncoding, ScheduleEntry, StateRequest)
from .linear import LinearWeight
from .norm import LayerNorm, RMSNorm, StreamCast
from .rope import DistancePenalty, RotaryEmbedding
from .attention import Attention
from .mlp import GatedMLP, PlainMLP
from .recurrent import (GatedDeltaRule, GatedLinearRecurrence, GeneralizedDeltaRule, MatrixMemory, Retention,
                        StateSpaceDuality)
from .latent import LatentAttention
from .parallel import ParallelMixer
from .moe import MixtureOfExperts
from .block import (PostNormBlock, PostNormMixerBlock, PreNormBlock, PreNormMixerBlock, SandwichNormBlock,
                    SandwichNormMixerBlock, ScaledPreNormBlock, ScaledPreNormMixerBlock)

__all__ = ["Block", "CompositeRequest", "FeedForward", "KeyValueRequest", "LayerSpec", "Mixer", "ModelPlan", "Norm",
           "Part", "PartSpec", "PositionEncoding", "ScheduleEntry", "StateRequest", "LinearWeight",
           "RMSNorm", "RotaryEmbedding", "DistancePenalty", "Attention", "GatedMLP", "Retention", "GatedDeltaRule",
           "GatedLinearRecurrence", "LatentAttention",
           "ParallelMixer", "MixtureOfExperts", "PreNormBlock", "PreNormMixerBlock", "SandwichNormBlock",
           "SandwichNormMixerBlock", "LayerNorm", "StreamCast", "PlainMLP", "StateSpaceDuality", "MatrixMemory",
           "PostNormBlock", "PostNormMixerBlock", "GeneralizedDeltaRule", "ScaledPreNormBlock", "ScaledPreNormMixerBlock"]
