"""Pre-norm residual block: x += mixer(norm1(x)); x += ffn(norm2(x))
(crates/model/src/components/decoder_block/mod.rs:66-85 of the reference).

The residual stream is float32.  A sub-layer's output is not added at once: it is
left pending and the next norm's kernel adds it while it reads the stream."""
from __future__ import annotations

from .base import prefixed, sub_weights
from .registry import BLOCKS, FEED_FORWARDS, MIXERS, NORMS
from .spec import BlockSpec

# tensor-name prefixes of the block's four parts
NORM1, MIXER, NORM2, FFN = "input_layernorm.", "self_attn.", "post_attention_layernorm.", "mlp."


@BLOCKS.register("pre_norm")
class PreNormBlock:
    @staticmethod
    def declare(spec: BlockSpec) -> dict:
        d = {}
        d.update(prefixed(NORMS.get(spec.norm1.kind).declare(spec.norm1), NORM1))
        d.update(prefixed(MIXERS.get(spec.mixer.kind).declare(spec.mixer), MIXER))
        d.update(prefixed(NORMS.get(spec.norm2.kind).declare(spec.norm2), NORM2))
        d.update(prefixed(FEED_FORWARDS.get(spec.ffn.kind).declare(spec.ffn), FFN))
        return d

    @staticmethod
    def cache_need(spec: BlockSpec):
        return MIXERS.get(spec.mixer.kind).cache_need(spec.mixer)

    def __init__(self, spec: BlockSpec, weights: dict, ctx):
        self.spec = spec
        self.norm1 = NORMS.get(spec.norm1.kind)(spec.norm1, sub_weights(weights, NORM1), ctx)
        self.mixer = MIXERS.get(spec.mixer.kind)(spec.mixer, sub_weights(weights, MIXER), ctx)
        self.norm2 = NORMS.get(spec.norm2.kind)(spec.norm2, sub_weights(weights, NORM2), ctx)
        self.ffn = FEED_FORWARDS.get(spec.ffn.kind)(spec.ffn, sub_weights(weights, FFN), ctx)
        self.graph_safe = bool(getattr(self.mixer, "graph_safe", False) and getattr(self.ffn, "graph_safe", False))

    def __call__(self, residual, step, cache):
        h = self.norm1(residual.x, residual.pending, step, tag="norm1")
        a = self.mixer(h, step, cache)
        h = self.norm2(residual.x, a, step, tag="norm2")
        residual.pending = self.ffn(h, step)
