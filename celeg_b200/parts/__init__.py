"""Parts a model is put together from, and their registries."""
from .registry import CATEGORIES, part_factory, register_part, registered
from .options import KernelOptions
from .runtime import Runtime, StepContext
from . import norms, positions, mixers, recurrent, latent, feed_forward, arrangement, ends, stream_parts  # register the built-in kinds
from .mixers import AttentionMixer, PagedBinding, PreparedAttentionMixer, ShortConvMixer, StateBinding
from .norms import DynamicTanh, LayerNorm, RmsNorm
from .recurrent import GatedDeltaMixer, MlstmMixer
from .positions import SplitHalfRope
from .feed_forward import SwiGluFeedForward
from .arrangement import PreNormResidual
from .ends import EmbeddingInput, NormHeadOutput

__all__ = ["CATEGORIES", "part_factory", "register_part", "registered", "KernelOptions", "Runtime", "StepContext",
           "AttentionMixer", "PreparedAttentionMixer", "PagedBinding", "ShortConvMixer", "StateBinding", "RmsNorm", "LayerNorm", "DynamicTanh", "MlstmMixer", "GatedDeltaMixer", "SplitHalfRope",
           "SwiGluFeedForward", "PreNormResidual", "EmbeddingInput", "NormHeadOutput"]
