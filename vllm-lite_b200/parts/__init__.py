"""Model parts: descriptions (`spec`), registries (`registry`) and the standard
implementations, which register themselves when this package is imported."""
from . import spec, registry                      # noqa: F401
from . import norm, rope, attention, mlp, block, embedding, head   # noqa: F401  (registration)
from .model import CausalLM, cache_needs, declare_model  # noqa: F401
from .registry import BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITIONS  # noqa: F401
