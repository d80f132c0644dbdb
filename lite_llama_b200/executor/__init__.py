"""Host-side mirror of the reference's executor surface (lite_llama/executor/*): the per-step
attention metadata, the KV pool + bump allocator, and the ModelRunner that drives the B200 kernels."""

from .attention_metadata import AttentionMetadata
from .kv_cache_manager import KVCacheManager
from .model_config import (BlockAttentionSpec, DecayAttentionSpec, DenseMlpSpec, LatentAttentionSpec, LayeredConfig,
                           LayerSpec, Mamba2Spec, MinGruSpec, ModelConfig, MoeMlpSpec, PRESETS, RgLruSpec, SideBySideSpec,
                           SinkAttentionSpec)
from .model_runner import ModelRunner, RequestState
from .ragged_batch import RaggedBatch
from .state_manager import RecurrentStateManager

__all__ = ["AttentionMetadata", "KVCacheManager", "ModelConfig", "PRESETS", "ModelRunner", "RequestState", "RaggedBatch",
           "RecurrentStateManager", "LayeredConfig", "LayerSpec", "Mamba2Spec", "SinkAttentionSpec", "DenseMlpSpec",
           "LatentAttentionSpec", "MoeMlpSpec", "MinGruSpec", "RgLruSpec", "BlockAttentionSpec", "DecayAttentionSpec",
           "SideBySideSpec"]
