"""Pre-norm residual block: x += mixer(norm1(x)); x += ffn(norm2(x))
(crates/model/src/components/decoder_block/mod.rs:66-85 of the reference).

The residual stream is float32.  A sub-layer's output is not added at once: it is
left pending and the next norm's kernel adds it while it reads the stream.  In a
step of few rows the norms' kernels are saved altogether where the neighbouring
parts can: the part before a norm adds its result into the stream itself and
leaves the norm's output in factored form (`ScaledRows`), which the part after
the norm takes as it is."""
from __future__ import annotations

from .base import StreamSink, prefixed, sub_weights
from .registry import BLOCKS, FEED_FORWARDS, MIXERS, NORMS
from .spec import BlockSpec

@BLOCKS.register("pre_norm")
class PreNormBlock:
    @staticmethod
    def declare(spec: BlockSpec) -> dict:
        norm1, mixer, norm2, ffn = spec.names
        d = {}
        d.update(prefixed(NORMS.get(spec.norm1.kind).declare(spec.norm1), norm1))
        d.update(prefixed(MIXERS.get(spec.mixer.kind).declare(spec.mixer), mixer))
        d.update(prefixed(NORMS.get(spec.norm2.kind).declare(spec.norm2), norm2))
        d.update(prefixed(FEED_FORWARDS.get(spec.ffn.kind).declare(spec.ffn), ffn))
        return d

    @staticmethod
    def cache_need(spec: BlockSpec):
        return MIXERS.get(spec.mixer.kind).cache_need(spec.mixer)

    def __init__(self, spec: BlockSpec, weights: dict, ctx):
        self.spec = spec
        norm1, mixer, norm2, ffn = spec.names
        self.norm1 = NORMS.get(spec.norm1.kind)(spec.norm1, sub_weights(weights, norm1), ctx)
        self.mixer = MIXERS.get(spec.mixer.kind)(spec.mixer, sub_weights(weights, mixer), ctx)
        self.norm2 = NORMS.get(spec.norm2.kind)(spec.norm2, sub_weights(weights, norm2), ctx)
        self.ffn = FEED_FORWARDS.get(spec.ffn.kind)(spec.ffn, sub_weights(weights, ffn), ctx)
        self.graph_safe = bool(getattr(self.mixer, "graph_safe", False) and getattr(self.ffn, "graph_safe", False))

    chains_norms = True        # __call__ takes `next_norm`

    def input_norm_for_fusion(self, M):
        """The first norm, if the block before may compute it for M rows in factored form."""
        ok = getattr(self.norm1, "factorable", False) and _factors(self.mixer, M)
        return self.norm1 if ok else None

    def __call__(self, residual, step, cache, next_norm=None):
        """next_norm: the norm that will read the stream after this block, when its reader can take
        the factored form (`input_norm_for_fusion` of the next block)."""
        M = step.num_tokens
        if residual.normed is not None and residual.normed_for is self.norm1:
            h = residual.normed                                   # left by the block before
        else:
            h = self.norm1(residual.x, residual.pending, step, tag="norm1")
        residual.pending = residual.normed = residual.normed_for = None
        if _factors(self.mixer, M) and getattr(self.norm2, "factorable", False) and _factors(self.ffn, M):
            h = self.mixer(h, step, cache, sink=_sink(residual, self.norm2))
        else:
            a = self.mixer(h, step, cache)
            h = self.norm2(residual.x, a, step, tag="norm2")
        if next_norm is not None and _factors(self.ffn, M):
            residual.normed = self.ffn(h, step, sink=_sink(residual, next_norm))
            residual.normed_for = next_norm
        else:
            residual.pending = self.ffn(h, step)


def _factors(part, M) -> bool:
    f = getattr(part, "factors_norms", None)
    return bool(f and f(M))


def _sink(residual, norm) -> StreamSink:
    return StreamSink(residual.x, norm.weight, norm.spec.eps, norm.spec.size)
