"""The parts a model is put together from, and their registries.  Importing this package registers
the built-in parts."""
from . import (attention, block, decay_attention, depth, entry, lanes, latent_attention, mamba2, mlp, moe, norm, parallel,  # noqa: F401
               rglru, rope)                                                                                               # (registration)
from .cache_need import CompositeNeed, FixedStateNeed, FixedStateView, PagedKVNeed, PagedKVView, PagedLatentNeed
from .context import BuildContext
from .linear import Linear
from .registry import (register_block, register_combiner, register_entry, register_feed_forward, register_mixer, register_norm,
                       register_position)
from .spec import (AttentionSpec, DecayAttentionSpec, DenseActSpec, DepthAverageSpec, EntrySpec, InputMixSpec,
                   LatentAttentionSpec, LayerSpec, Mamba2Spec, ModelSpec, NormSpec, ParallelMixersSpec, PositionSpec, RoutedExpertsSpec, Stage, SwiGLUSpec, TensorRole)

__all__ = ["CompositeNeed", "DecayAttentionSpec", "EntrySpec", "InputMixSpec", "ParallelMixersSpec", "register_entry", "FixedStateNeed", "FixedStateView", "PagedKVNeed", "PagedKVView", "PagedLatentNeed", "BuildContext", "Linear",
           "register_combiner", "DenseActSpec", "DepthAverageSpec", "LatentAttentionSpec", "Mamba2Spec",
           "register_block", "register_feed_forward", "register_mixer", "register_norm",
           "register_position", "AttentionSpec", "LayerSpec", "ModelSpec", "NormSpec", "PositionSpec",
           "RoutedExpertsSpec", "Stage", "SwiGLUSpec", "TensorRole"]
