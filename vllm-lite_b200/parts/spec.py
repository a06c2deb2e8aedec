"""Descriptions of model parts as plain data.

A model is a `ModelPlan`: an embedding, a list of layer descriptions, the order
in which layers run, a final norm and an output head (each of them a part).  Every description is a
frozen dataclass whose `kind` names the implementation in the part registries
(`parts.registry`); sizes and constants are fields, never code.  Layers may
differ from one another, and `order` may name a layer twice or let a layer read
the cache that an earlier call wrote.

Descriptions hold no tensors and import nothing from the GPU side, so the
configuration, the weight loader, the random-weights writer and the CPU tests
can all work from them.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Tuple


@dataclass(frozen=True)
class TensorDecl:
    """One tensor that a part binds by name.

    `init` names the distribution of the random-weights mode: "linear"
    (N(0, std)), "norm" (1 + N(0, norm_std)).  `store` is the dtype the tensor
    has in a written folder and the least precision it is kept in:
    "model" (the model dtype, bfloat16 on disk) or "float32".
    """
    shape: Tuple[int, ...]
    init: str = "linear"
    store: str = "model"


@dataclass(frozen=True)
class NormSpec:
    size: int
    eps: float
    kind: str = "rms_norm"


@dataclass(frozen=True)
class RotarySpec:
    """Rotate-half rotary position encoding of the first `rotary_dim` features
    of each head; inv_freq[i] = theta^(-2i / rotary_dim)."""
    head_dim: int
    theta: float
    rotary_dim: Optional[int] = None
    kind: str = "rotary"

    @property
    def dim(self) -> int:
        return self.head_dim if self.rotary_dim is None else self.rotary_dim


@dataclass(frozen=True)
class AttentionSpec:
    """Grouped-query attention over a paged key/value cache.

    `window`: None reads every earlier key; w reads the last w keys (the
    query's own position included).  `qk_norm`: norm over head_dim applied to
    every q and k head before the position encoding.  `scale` defaults to
    head_dim ** -0.5.
    """
    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    qk_norm: Optional[NormSpec] = None
    position: Optional[RotarySpec] = None
    window: Optional[int] = None
    scale: Optional[float] = None
    bias: bool = False              # q/k/v projections with a bias vector each (the output projection has none)
    kind: str = "gqa_attention"


@dataclass(frozen=True)
class EmbeddingSpec:
    """Token ids to rows of the residual stream: x[t] = table[id[t]], no scaling."""
    vocab_size: int
    hidden_size: int
    kind: str = "token_embedding"


@dataclass(frozen=True)
class HeadSpec:
    """The output head: logits = h W^T in float32, no bias.  `tied`: W is the embedding's table
    (the head then declares no tensor of its own)."""
    vocab_size: int
    hidden_size: int
    tied: bool = False
    kind: str = "linear_head"


@dataclass(frozen=True)
class SwiGLUSpec:
    hidden_size: int
    intermediate_size: int
    kind: str = "swiglu"


@dataclass(frozen=True)
class BlockSpec:
    """Pre-norm residual block: x += mixer(norm1(x)); x += ffn(norm2(x))."""
    mixer: object
    ffn: object
    norm1: NormSpec
    norm2: NormSpec
    kind: str = "pre_norm"
    # tensor-name prefixes of the four parts inside a layer (norm1, mixer, norm2, feed-forward)
    names: Tuple[str, str, str, str] = ("input_layernorm.", "self_attn.", "post_attention_layernorm.", "mlp.")


@dataclass(frozen=True)
class LayerCall:
    """One entry of the running order.

    `layer` indexes `ModelPlan.layers` (the weights).  `cache_of`, when set, is
    the index of an EARLIER entry of the order whose cache this call reads
    instead of writing one of its own.
    """
    layer: int
    cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelPlan:
    architecture: str
    vocab_size: int
    hidden_size: int
    layers: Tuple[BlockSpec, ...]
    order: Tuple[LayerCall, ...]
    final_norm: NormSpec
    tie_word_embeddings: bool
    max_position_embeddings: int
    layer_prefix: str = "model.layers.{}."
    embed_prefix: str = "model.embed_tokens."
    final_norm_prefix: str = "model.norm."
    head_prefix: str = "lm_head."
    init_std: float = 0.02
    norm_init_std: float = 0.1
    extra: dict = field(default_factory=dict, compare=False, hash=False)
    # The two ends of the model are parts like the layers' (registries EMBEDDINGS and HEADS).  Left None
    # they are the plain ones, described by vocab_size, hidden_size and tie_word_embeddings.
    embedding: Optional[object] = None
    head: Optional[object] = None

    @property
    def embedding_spec(self):
        return self.embedding if self.embedding is not None else EmbeddingSpec(self.vocab_size, self.hidden_size)

    @property
    def head_spec(self):
        return self.head if self.head is not None else HeadSpec(self.vocab_size, self.hidden_size,
                                                                tied=self.tie_word_embeddings)

    def validate(self) -> "ModelPlan":
        for i, call in enumerate(self.order):
            if not 0 <= call.layer < len(self.layers):
                raise ValueError(f"order[{i}] names layer {call.layer}, the plan has {len(self.layers)}")
            if call.cache_of is not None:
                if not 0 <= call.cache_of < i:
                    raise ValueError(f"order[{i}].cache_of={call.cache_of} must name an earlier entry")
                if self.order[call.cache_of].cache_of is not None:
                    raise ValueError(f"order[{i}].cache_of={call.cache_of} names an entry that owns no cache")
        return self
