"""The Qwen3 dense decoder as a plan of parts: every layer is a pre-norm block of
GQA attention (per-head RMS norm of q and k, rotary positions over the whole
head, no window) and a SwiGLU feed-forward
(crates/model/src/components/attention/rope_gqa.rs and
crates/model/src/qwen3/block/construct.rs:219-302 of the reference)."""
from __future__ import annotations

from ..parts.spec import AttentionSpec, BlockSpec, LayerCall, ModelPlan, NormSpec, RotarySpec, SwiGLUSpec
from .qwen3 import ARCHITECTURE, Qwen3Config
from .registry import register_architecture


def qwen3_plan(cfg: Qwen3Config) -> ModelPlan:
    norm = NormSpec(cfg.hidden_size, cfg.rms_norm_eps)
    attention = AttentionSpec(
        hidden_size=cfg.hidden_size, num_heads=cfg.num_attention_heads, num_kv_heads=cfg.num_key_value_heads,
        head_dim=cfg.head_dim, qk_norm=NormSpec(cfg.head_dim, cfg.head_norm_eps),
        position=RotarySpec(cfg.head_dim, cfg.rope_theta), window=None)
    block = BlockSpec(mixer=attention, ffn=SwiGLUSpec(cfg.hidden_size, cfg.intermediate_size), norm1=norm, norm2=norm)
    n = cfg.num_hidden_layers
    return ModelPlan(architecture=ARCHITECTURE, vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size,
                     layers=tuple(block for _ in range(n)), order=tuple(LayerCall(i) for i in range(n)),
                     final_norm=norm, tie_word_embeddings=cfg.tie_word_embeddings,
                     max_position_embeddings=cfg.max_position_embeddings)


register_architecture(ARCHITECTURE, Qwen3Config, qwen3_plan, model_types=("qwen3", "qwen_3"), replace=True)
