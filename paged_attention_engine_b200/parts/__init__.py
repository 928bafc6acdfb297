from .base import (
    BLOCKS, CONNECTIONS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITION_ENCODINGS,
    REGISTRIES, Block, CacheNeed, EntryCache, Part, Registry, Runtime, StateNeed, TensorSpec,
    layer_part_specs, with_sub_parts,
)
from . import (attention, blocks, connections, delta_rule, feed_forward, gated_attention, heads, latent_attention, matrix_memory, norms,
               rotary, scored_attention)  # noqa: F401  (registration)

__all__ = [
    "BLOCKS", "CONNECTIONS", "EMBEDDINGS", "FEED_FORWARDS", "HEADS", "MIXERS", "NORMS", "POSITION_ENCODINGS",
    "REGISTRIES", "Block", "CacheNeed", "EntryCache", "Part", "Registry", "Runtime", "StateNeed", "TensorSpec",
    "layer_part_specs", "with_sub_parts",
]
