"""Each part alone against the plain implementation, a running order that names a
layer twice and shares a cache, and a toy mixer with state of its own that is
registered, built and stepped from this file without a change to the framework."""
from dataclasses import dataclass

import pytest
import torch

import helpers as H
import plain_qwen3 as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def make_step(runner_like_workspace, T):
    from vllm_lite_b200.parts.base import StepBatch, Workspace
    z = torch.zeros(1, dtype=torch.int32, device=DEV)
    return StepBatch(tokens=z, positions=z, req_index=z, cu_seqlens=z, state_slots=z, logit_rows=z, groups=[],
                     entries=[], err=torch.zeros(1, dtype=torch.int32, device=DEV), workspace=Workspace(DEV),
                     num_tokens=T, num_entries=1)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_and_feed_forward_alone(dtype):
    from vllm_lite_b200.parts import FEED_FORWARDS, NORMS
    from vllm_lite_b200.parts.base import BuildContext
    from vllm_lite_b200.parts.spec import NormSpec, SwiGLUSpec
    ctx = BuildContext(torch.device(DEV), dtype)
    T, Hd, I = 11, 72, 200
    tol = dict(atol=1e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=3e-2, rtol=3e-2)
    step = make_step(None, T)
    w = 1 + 0.1 * torch.randn(Hd)
    norm = NORMS.get("rms_norm")(NormSpec(Hd, 1e-4), {"weight": w.to(dtype)}, ctx)
    x = torch.randn(T, Hd, device=DEV)
    h = norm(x, None, step)
    assert h.dtype == dtype
    assert torch.allclose(h.float().cpu(), P.rms_norm(x.cpu(), w.to(dtype).float(), 1e-4), **tol)
    spec = SwiGLUSpec(Hd, I)
    decl = FEED_FORWARDS.get("swiglu").declare(spec)
    assert decl["down_proj.weight"].shape == (Hd, I)
    weights = {k: (torch.randn(d.shape) * 0.1).to(dtype).to(DEV) for k, d in decl.items()}
    ffn = FEED_FORWARDS.get("swiglu")(spec, weights, ctx)
    out = ffn(h, step)
    ref = P.swiglu(h.float().cpu(), {"mlp." + k: v.float().cpu() for k, v in weights.items()}, "")
    assert torch.allclose(out.float().cpu(), ref, **tol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window", [None, 9])
def test_attention_and_block_alone(dtype, window):
    """The attention mixer (with its norm and rotary parts) and a whole pre-norm block, built from
    descriptions of their own at sizes of no model, stepped over pages as a prompt portion, a
    continuation and single tokens, against the plain functions on the whole sequence."""
    from vllm_lite_b200.cache import PagedKV
    from vllm_lite_b200.parts import BLOCKS, MIXERS
    from vllm_lite_b200.parts.base import BuildContext, CallCache, GroupView, Residual
    from vllm_lite_b200.parts.spec import AttentionSpec, BlockSpec, NormSpec, RotarySpec, SwiGLUSpec
    torch.manual_seed(5)
    hidden, nq, nkv, hd, inter, page, theta, eps = 56, 6, 3, 48, 72, 4, 5000.0, 1e-4
    att = AttentionSpec(hidden, nq, nkv, hd, qk_norm=NormSpec(hd, 2e-5), position=RotarySpec(hd, theta), window=window)
    spec = BlockSpec(mixer=att, ffn=SwiGLUSpec(hidden, inter), norm1=NormSpec(hidden, eps), norm2=NormSpec(hidden, eps))
    assert MIXERS.get("gqa_attention").cache_need(att) == PagedKV(nkv, hd, window)
    decl = BLOCKS.get("pre_norm").declare(spec)
    assert decl["self_attn.q_proj.weight"].shape == (nq * hd, hidden) and decl["self_attn.k_norm.weight"].shape == (hd,)
    w = {k: ((1 + 0.1 * torch.randn(d.shape)) if d.init == "norm" else torch.randn(d.shape) * 0.08).to(dtype)
         for k, d in decl.items()}
    ctx = BuildContext(torch.device(DEV), dtype)
    block = BLOCKS.get("pre_norm")(spec, {k: v.to(DEV) for k, v in w.items()}, ctx)
    n = 23
    x0 = torch.randn(n, hidden)
    # plain: the block on the whole sequence
    wf = {"L." + k: v.float() for k, v in w.items()}
    cfg = dict(num_attention_heads=nq, num_key_value_heads=nkv, head_dim=hd, rms_norm_eps=eps, rope_theta=theta)
    h = P.rms_norm(x0, wf["L.input_layernorm.weight"], eps)
    q = P.rope(P.head_norm(P.linear(h, wf["L.self_attn.q_proj.weight"]).view(n, nq, hd), wf["L.self_attn.q_norm.weight"], 2e-5), range(n), theta)
    k = P.rope(P.head_norm(P.linear(h, wf["L.self_attn.k_proj.weight"]).view(n, nkv, hd), wf["L.self_attn.k_norm.weight"], 2e-5), range(n), theta)
    v = P.linear(h, wf["L.self_attn.v_proj.weight"]).view(n, nkv, hd)
    a_ref = P.linear(P.causal_attention(q, k, v, window=window).reshape(n, nq * hd), wf["L.self_attn.o_proj.weight"])
    x1 = x0 + a_ref
    ref = x1 + P.swiglu(P.rms_norm(x1, wf["L.post_attention_layernorm.weight"], eps), wf, "L.")
    # engine parts: portions of 9, 2, then single tokens, pages in shuffled order
    pages = 8
    kc = torch.zeros(pages, nkv, page, hd, device=DEV, dtype=dtype)
    vc = torch.zeros_like(kc)
    table = torch.tensor([[5, 2, 7, 0, 3, 6]], dtype=torch.int32, device=DEV)
    cache = CallCache(group=0, k=kc, v=vc, writes=True)
    outs, attn_outs, start = [], [], 0
    for count in [9, 2] + [1] * 12:
        pos = torch.arange(start, start + count, dtype=torch.int32, device=DEV)
        slots = (table[0, (pos // page).long()] * page + pos % page).to(torch.int32)
        step = make_step(None, count)
        step.positions, step.req_index = pos, torch.zeros(count, dtype=torch.int32, device=DEV)
        step.groups = [GroupView(page, table, slots, max_context=start + count)]
        step.max_query_len = count
        step.query_tiles = torch.tensor([[0, 0, count, start]], dtype=torch.int32, device=DEV)
        res = Residual(x0[start:start + count].to(DEV).contiguous())
        hh = block.norm1(res.x, None, step, tag="n1")
        attn_outs.append(block.mixer(hh, step, cache).float().cpu())
        res2 = Residual(x0[start:start + count].to(DEV).contiguous())
        block(res2, step, cache)                                   # the whole block (writes the same cache rows again)
        outs.append((res2.x + res2.pending.float()).cpu())
        start += count
    tol = dict(atol=2e-5, rtol=1e-4) if dtype == torch.float32 else dict(atol=4e-2, rtol=4e-2)
    assert torch.allclose(torch.cat(attn_outs), a_ref, **tol)
    assert torch.allclose(torch.cat(outs), ref, **tol)


def plain_with_order(cfg, w, ids, order, share):
    """The plain model with a running order: layer indices, and for each call whether it
    reuses the keys/values of an earlier call (then only its queries are its own)."""
    cfg = P.normalise_config(cfg)
    n = len(ids)
    pos = list(range(n))
    x = P.embedding(ids, w["model.embed_tokens.weight"])
    kv = {}
    nq, nkv, d, eps = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"], cfg["rms_norm_eps"]
    for call, (layer, src) in enumerate(zip(order, share)):
        pre = f"model.layers.{layer}."
        h = P.rms_norm(x, w[pre + "input_layernorm.weight"], eps)
        q = P.linear(h, w[pre + "self_attn.q_proj.weight"]).view(n, nq, d)
        q = P.rope(P.head_norm(q, w[pre + "self_attn.q_norm.weight"], eps), pos, cfg["rope_theta"])
        if src is None:
            k = P.linear(h, w[pre + "self_attn.k_proj.weight"]).view(n, nkv, d)
            k = P.rope(P.head_norm(k, w[pre + "self_attn.k_norm.weight"], eps), pos, cfg["rope_theta"])
            v = P.linear(h, w[pre + "self_attn.v_proj.weight"]).view(n, nkv, d)
            kv[call] = (k, v)
        else:
            k, v = kv[src]
        o = P.causal_attention(q, k, v)
        x = x + P.linear(o.reshape(n, nq * d), w[pre + "self_attn.o_proj.weight"])
        x = x + P.swiglu(P.rms_norm(x, w[pre + "post_attention_layernorm.weight"], eps), w, pre)
    return P.linear(P.rms_norm(x, w["model.norm.weight"], eps), w["model.embed_tokens.weight"])


def test_order_may_repeat_a_layer_and_share_a_cache():
    from vllm_lite_b200.config import plan_from_config_json
    from vllm_lite_b200.engine import ModelRunner, StepEntry, load_model_dir
    from vllm_lite_b200.parts.spec import LayerCall, ModelPlan
    _, base, weights = load_model_dir(H.model_dir("A"), "float32", DEV)
    order = (LayerCall(0), LayerCall(1), LayerCall(1), LayerCall(0, cache_of=0))
    plan = ModelPlan(**{**base.__dict__, "order": order})
    runner = ModelRunner(plan, weights, dtype=torch.float32, device=DEV, page_size=16, num_pages=8, max_requests=2)
    assert len(runner.layout.paged_members[0]) == 3                     # three calls own a cache, one borrows
    toks = H.tokens_for("A", 40, 5)
    cfg, w = H.plain_model("A")
    ref = plain_with_order(cfg, w, toks, [0, 1, 1, 0], [None, None, None, 0])
    got = torch.cat([runner.step([StepEntry("r", toks[:23], list(range(23)))]).cpu(),   # a step's logits live
                     runner.step([StepEntry("r", toks[23:25], [0, 1])]).cpu(),          # until the next step
                     runner.step([StepEntry("r", toks[25:], list(range(15)))]).cpu()])
    runner.check_device_errors()
    assert float((got - ref).abs().max()) <= H.TOL["float32"] * float(ref.abs().max())
    assert not torch.allclose(ref, P.forward(cfg, w, toks), atol=1e-3)   # the order matters


def plain_with_windows(cfg, w, ids, windows):
    """The plain model with a window per layer (None: every earlier key)."""
    cfg = P.normalise_config(cfg)
    n = len(ids)
    pos = list(range(n))
    nq, nkv, d, eps = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"], cfg["rms_norm_eps"]
    x = P.embedding(ids, w["model.embed_tokens.weight"])
    for layer, window in enumerate(windows):
        pre = f"model.layers.{layer}."
        h = P.rms_norm(x, w[pre + "input_layernorm.weight"], eps)
        q = P.rope(P.head_norm(P.linear(h, w[pre + "self_attn.q_proj.weight"]).view(n, nq, d), w[pre + "self_attn.q_norm.weight"], eps), pos, cfg["rope_theta"])
        k = P.rope(P.head_norm(P.linear(h, w[pre + "self_attn.k_proj.weight"]).view(n, nkv, d), w[pre + "self_attn.k_norm.weight"], eps), pos, cfg["rope_theta"])
        v = P.linear(h, w[pre + "self_attn.v_proj.weight"]).view(n, nkv, d)
        x = x + P.linear(P.causal_attention(q, k, v, window=window).reshape(n, nq * d), w[pre + "self_attn.o_proj.weight"])
        x = x + P.swiglu(P.rms_norm(x, w[pre + "post_attention_layernorm.weight"], eps), w, pre)
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings") else w["lm_head.weight"]
    return P.linear(P.rms_norm(x, w["model.norm.weight"], eps), head)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_layers_with_a_window_get_pages_of_their_own_and_give_them_back(dtype):
    """A toy architecture over the tiny B weights: layers 0 and 2 read every key, layer 1 the last 20.
    The windowed layer's group has a pool so small that it only works if pages behind the window
    return; logits still match the plain implementation at every position."""
    import dataclasses
    from vllm_lite_b200.config import Qwen3Config, plan_from_config_json, register_architecture, unregister_architecture
    from vllm_lite_b200.engine import ModelRunner, load_model_dir
    from vllm_lite_b200.parts.spec import ModelPlan
    window = 20

    def plan(cfg):
        base = plan_from_config_json({**H.TINY_B, "architectures": ["Qwen3ForCausalLM"]})[1]
        layers = list(base.layers)
        layers[1] = dataclasses.replace(layers[1], mixer=dataclasses.replace(layers[1].mixer, window=window))
        return ModelPlan(**{**base.__dict__, "architecture": "ToyWindowLM", "layers": tuple(layers)})

    register_architecture("ToyWindowLM", Qwen3Config, plan)
    try:
        import json, shutil
        d = H.tmp_root() / "toy_window"
        shutil.copytree(H.model_dir("B"), d, dirs_exist_ok=True)
        (d / "config.json").write_text(json.dumps({**H.TINY_B, "architectures": ["ToyWindowLM"]}))
        _, p, weights = load_model_dir(d, dtype, DEV)
        page = 8
        # 150 tokens need 19 pages in the full group; the windowed group gets 7: (20 + 17 + 8) / 8 rounded up
        runner = ModelRunner(p, weights, dtype=torch.bfloat16 if dtype == "bfloat16" else torch.float32, device=DEV,
                             page_size=page, num_pages=[19, 7], max_requests=2)
        assert [g.window for g in runner.layout.paged_groups] == [None, window]
        assert runner.layout.paged_members == [[0, 2], [1]]
        toks = H.tokens_for("B", 150, 77)
        schedule, pos = [], 0
        for n in [17, 2, 9, 1, 1, 16, 3] + [1] * 40 + [11, 2] + [1] * 100:
            n = min(n, 150 - pos)
            if n <= 0:
                break
            schedule.append(([("r", toks[pos:pos + n], list(range(n)))], []))
            pos += n
        assert pos == 150
        rows = H.run_schedule(runner, schedule)
        cfg, w = H.plain_model("B")
        ref = plain_with_windows(cfg, w, toks, [None, window, None])
        assert not torch.allclose(ref, H.plain_logits("B", toks), atol=1e-3)          # the window matters
        for (rid, i), row in rows.items():
            err = float((row - ref[i]).abs().max()) / float(ref[i].abs().max())
            assert err <= H.TOL[dtype], (i, err)
        held = [sum(pg >= 0 for pg in t) for t in runner.cache.requests["r"].block_tables]
        assert held[0] == 19 and held[1] <= 4
        runner.release("r")
        assert runner.cache.free_pages() == [19, 7]
    finally:
        unregister_architecture("ToyWindowLM")


# ---- a toy mixer with state of its own, defined here ---------------------------------
@dataclass(frozen=True)
class DecaySpec:
    hidden_size: int
    decay: float
    kind: str = "toy_decay"


class DecayMixer:
    """s_t = decay * s_{t-1} + h_t;  out_t = s_t W^T.  The state s is one vector per request."""

    @staticmethod
    def declare(spec):
        from vllm_lite_b200.parts.spec import TensorDecl
        return {"mix.weight": TensorDecl((spec.hidden_size, spec.hidden_size))}

    @staticmethod
    def cache_need(spec):
        from vllm_lite_b200.cache import FixedState
        return FixedState((spec.hidden_size,))

    def __init__(self, spec, weights, ctx):
        self.spec, self.w, self.dtype = spec, weights["mix.weight"].float(), ctx.dtype

    def __call__(self, h, step, cache):
        out = torch.empty_like(h)
        t = 0
        for entry in step.entries:                        # portions of a request arrive in order
            s = cache.state[entry.state_slot]
            for i in range(t, t + entry.count):
                s = self.spec.decay * s + h[i].float()
                out[i] = (s @ self.w.T).to(self.dtype)
            cache.state[entry.state_slot] = s
            t += entry.count
        return out


def plain_decay_model(cfg, w, ids, decay):
    """Layer 0: decay mixer + feed-forward; layer 1: the attention block of the plain model."""
    cfg = P.normalise_config(cfg)
    x = P.embedding(ids, w["model.embed_tokens.weight"])
    pre = "model.layers.0."
    h = P.rms_norm(x, w[pre + "input_layernorm.weight"], cfg["rms_norm_eps"])
    s, outs = torch.zeros(cfg["hidden_size"]), []
    for t in range(len(ids)):
        s = decay * s + h[t]
        outs.append(s @ w[pre + "self_attn.mix.weight"].T)
    x = x + torch.stack(outs)
    x = x + P.swiglu(P.rms_norm(x, w[pre + "post_attention_layernorm.weight"], cfg["rms_norm_eps"]), w, pre)
    x = P.decoder_block(x, list(range(len(ids))), w, 1, cfg)
    return P.linear(P.rms_norm(x, w["model.norm.weight"], cfg["rms_norm_eps"]), w["model.embed_tokens.weight"])


def test_toy_mixer_with_state_registers_builds_and_steps():
    from vllm_lite_b200.config import Qwen3Config, plan_from_config_json, register_architecture, unregister_architecture
    from vllm_lite_b200.engine import ModelRunner, StepEntry, load_model_dir
    from vllm_lite_b200.parts import MIXERS, declare_model
    from vllm_lite_b200.parts.spec import BlockSpec, ModelPlan
    from vllm_lite_b200.weights import random_tensors, write_safetensors
    import json

    def plan(cfg):
        base = plan_from_config_json({**H.TINY_A, "architectures": ["Qwen3ForCausalLM"]})[1]
        toy = BlockSpec(mixer=DecaySpec(cfg.hidden_size, 0.75), ffn=base.layers[0].ffn,
                        norm1=base.layers[0].norm1, norm2=base.layers[0].norm2)
        return ModelPlan(**{**base.__dict__, "architecture": "ToyDecayLM", "layers": (toy, base.layers[1])})

    MIXERS.register("toy_decay", DecayMixer)
    register_architecture("ToyDecayLM", Qwen3Config, plan)
    try:
        cfg_json = {**H.TINY_A, "architectures": ["ToyDecayLM"]}
        d = H.tmp_root() / "toy_decay"
        d.mkdir(exist_ok=True)
        (d / "config.json").write_text(json.dumps(cfg_json))
        _, p = plan_from_config_json(cfg_json)
        decl = declare_model(p)
        assert "model.layers.0.self_attn.mix.weight" in decl and "model.layers.0.self_attn.q_proj.weight" not in decl
        write_safetensors(d / "model.safetensors", random_tensors(decl, 3, std=0.05))
        _, p, weights = load_model_dir(d, "float32", DEV)
        runner = ModelRunner(p, weights, dtype=torch.float32, device=DEV, page_size=16, num_pages=8, max_requests=3)
        assert len(runner.layout.state_groups) == 1 and len(runner.layout.paged_groups) == 1
        a, b = H.tokens_for("A", 30, 1), H.tokens_for("A", 19, 2)
        cfg, w = P.read_model_dir(d)
        ref_a, ref_b = plain_decay_model(cfg, w, a, 0.75), plain_decay_model(cfg, w, b, 0.75)
        rows = H.run_schedule(runner, [
            ([("a", a[:11], list(range(11)))], []),
            ([("a", a[11:13], [0, 1]), ("b", b[:19], list(range(19)))], ["b"]),
            ([("a", a[13:], list(range(17)))], ["a"]),
            ([("b2", b, list(range(19)))], ["b2"]),          # b's slot is used again and starts from zero
        ])
        for (rid, pos), row in rows.items():
            ref = ref_a if rid == "a" else ref_b
            assert float((row - ref[pos]).abs().max()) <= 5e-5 * float(ref.abs().max()), (rid, pos)
    finally:
        MIXERS.unregister("toy_decay")
        unregister_architecture("ToyDecayLM")


# ---- a toy position encoding and a toy routed feed-forward, defined here -----------------------
@dataclass(frozen=True)
class LearnedPositionSpec:
    head_dim: int
    max_positions: int
    kind: str = "toy_learned_position"


class LearnedPosition:
    """q_head += table[pos], k_head += table[pos]; not known to the fused kernel, so it acts by itself."""

    @staticmethod
    def declare(spec):
        from vllm_lite_b200.parts.spec import TensorDecl
        return {"table": TensorDecl((spec.max_positions, spec.head_dim))}

    def __init__(self, spec, weights, ctx):
        self.spec, self.table = spec, weights["table"]

    def fused_rotary(self):
        return None

    def apply(self, qkv, positions, num_heads, num_kv_heads, head_dim, step):
        T = qkv.shape[0]
        qk = qkv[:, :(num_heads + num_kv_heads) * head_dim].view(T, num_heads + num_kv_heads, head_dim)
        add = self.table[positions.long().clamp(min=0)].to(qkv.dtype)
        qk += add[:, None, :]


@dataclass(frozen=True)
class RoutedSpec:
    hidden_size: int
    intermediate_size: int
    num_experts: int
    kind: str = "toy_routed"


class RoutedFeedForward:
    """Top-1 routing: e = argmax(softmax(h R^T)); y = p_e * W2[e] relu(W1[e] h).  Router in float32."""

    @staticmethod
    def declare(spec):
        from vllm_lite_b200.parts.spec import TensorDecl
        d = {"router.weight": TensorDecl((spec.num_experts, spec.hidden_size))}
        for e in range(spec.num_experts):
            d[f"experts.{e}.w1.weight"] = TensorDecl((spec.intermediate_size, spec.hidden_size))
            d[f"experts.{e}.w2.weight"] = TensorDecl((spec.hidden_size, spec.intermediate_size))
        return d

    def __init__(self, spec, weights, ctx):
        self.spec, self.w, self.dtype = spec, {k: v.float() for k, v in weights.items()}, ctx.dtype

    def __call__(self, h, step):
        return routed_reference(h.float(), self.w, self.spec.num_experts, "").to(self.dtype)


def routed_reference(h, w, num_experts, prefix):
    probs = torch.softmax(h @ w[prefix + "router.weight"].T, dim=-1)
    p, e = probs.max(dim=-1)
    out = torch.zeros_like(h)
    for k in range(num_experts):
        rows = (e == k).nonzero().flatten()
        if rows.numel():
            hid = torch.relu(h[rows] @ w[prefix + f"experts.{k}.w1.weight"].T)
            out[rows] = p[rows, None] * (hid @ w[prefix + f"experts.{k}.w2.weight"].T)
    return out


def plain_toy_mix(cfg, w, ids, rotary_dim, num_experts):
    """Layer 0: attention with learned positions (no rotation) and the routed feed-forward;
    layer 1: attention rotating only the first `rotary_dim` features of each head, SwiGLU."""
    cfg = P.normalise_config(cfg)
    n = len(ids)
    pos = list(range(n))
    nq, nkv, d, eps = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"], cfg["rms_norm_eps"]
    x = P.embedding(ids, w["model.embed_tokens.weight"])
    for layer in range(2):
        pre = f"model.layers.{layer}."
        h = P.rms_norm(x, w[pre + "input_layernorm.weight"], eps)
        q = P.linear(h, w[pre + "self_attn.q_proj.weight"]).view(n, nq, d)
        k = P.linear(h, w[pre + "self_attn.k_proj.weight"]).view(n, nkv, d)
        v = P.linear(h, w[pre + "self_attn.v_proj.weight"]).view(n, nkv, d)
        if layer == 0:
            table = w[pre + "self_attn.rotary.table"][:n]
            q, k = q + table[:, None, :], k + table[:, None, :]
        q, k = P.head_norm(q, w[pre + "self_attn.q_norm.weight"], eps), P.head_norm(k, w[pre + "self_attn.k_norm.weight"], eps)
        if layer == 1:
            q = torch.cat([P.rope(q[..., :rotary_dim], pos, cfg["rope_theta"]), q[..., rotary_dim:]], dim=-1)
            k = torch.cat([P.rope(k[..., :rotary_dim], pos, cfg["rope_theta"]), k[..., rotary_dim:]], dim=-1)
        x = x + P.linear(P.causal_attention(q, k, v).reshape(n, nq * d), w[pre + "self_attn.o_proj.weight"])
        h = P.rms_norm(x, w[pre + "post_attention_layernorm.weight"], eps)
        x = x + (routed_reference(h, w, num_experts, pre + "mlp.") if layer == 0 else P.swiglu(h, w, pre))
    return P.linear(P.rms_norm(x, w["model.norm.weight"], eps), w["model.embed_tokens.weight"])


def test_toy_position_encoding_and_routed_feed_forward_register_and_step():
    import dataclasses, json
    from vllm_lite_b200.config import Qwen3Config, plan_from_config_json, register_architecture, unregister_architecture
    from vllm_lite_b200.engine import ModelRunner, load_model_dir
    from vllm_lite_b200.parts import FEED_FORWARDS, POSITIONS, declare_model
    from vllm_lite_b200.parts.spec import ModelPlan, RotarySpec
    from vllm_lite_b200.weights import random_tensors, write_safetensors
    experts, rotary_dim = 3, 8

    def plan(cfg):
        base = plan_from_config_json({**H.TINY_A, "architectures": ["Qwen3ForCausalLM"]})[1]
        l0, l1 = base.layers
        l0 = dataclasses.replace(l0, mixer=dataclasses.replace(l0.mixer, position=LearnedPositionSpec(cfg.head_dim, 64)),
                                 ffn=RoutedSpec(cfg.hidden_size, 40, experts))
        l1 = dataclasses.replace(l1, mixer=dataclasses.replace(
            l1.mixer, position=RotarySpec(cfg.head_dim, cfg.rope_theta, rotary_dim=rotary_dim)))
        return ModelPlan(**{**base.__dict__, "architecture": "ToyMixLM", "layers": (l0, l1)})

    POSITIONS.register("toy_learned_position", LearnedPosition)
    FEED_FORWARDS.register("toy_routed", RoutedFeedForward)
    register_architecture("ToyMixLM", Qwen3Config, plan)
    try:
        cfg_json = {**H.TINY_A, "architectures": ["ToyMixLM"]}
        d = H.tmp_root() / "toy_mix"
        d.mkdir(exist_ok=True)
        (d / "config.json").write_text(json.dumps(cfg_json))
        _, p = plan_from_config_json(cfg_json)
        decl = declare_model(p)
        assert "model.layers.0.self_attn.rotary.table" in decl and "model.layers.0.mlp.experts.2.w2.weight" in decl
        assert "model.layers.0.mlp.gate_proj.weight" not in decl and "model.layers.1.mlp.gate_proj.weight" in decl
        write_safetensors(d / "model.safetensors", random_tensors(decl, 9, std=0.08))
        _, p, weights = load_model_dir(d, "float32", DEV)
        runner = ModelRunner(p, weights, dtype=torch.float32, device=DEV, page_size=16, num_pages=8, max_requests=3)
        assert not runner.decode_graphs                      # the toy feed-forward did not declare itself graph safe
        a, b = H.tokens_for("A", 41, 3), H.tokens_for("A", 14, 4)
        cfg, w = P.read_model_dir(d)
        ref = {"a": plain_toy_mix(cfg, w, a, rotary_dim, experts), "b": plain_toy_mix(cfg, w, b, rotary_dim, experts)}
        rows = H.run_schedule(runner, [
            ([("a", a[:19], list(range(19)))], []),
            ([("a", a[19:21], [0, 1]), ("b", b, list(range(14)))], ["b"]),
            ([("a", a[21:22], [0])], []),
            ([("a", a[22:], list(range(19)))], ["a"]),
        ])
        for (rid, pos), row in rows.items():
            assert float((row - ref[rid][pos]).abs().max()) <= 5e-5 * float(ref[rid].abs().max()), (rid, pos)
    finally:
        POSITIONS.unregister("toy_learned_position")
        FEED_FORWARDS.unregister("toy_routed")
        unregister_architecture("ToyMixLM")


# ---- toy ends of the model and a toy head norm, defined here ---------------------------------------
@dataclass(frozen=True)
class ScaledEmbeddingSpec:
    vocab_size: int
    hidden_size: int
    scale: float
    kind: str = "toy_scaled_embedding"


class ScaledEmbedding:
    """x[t] = scale * table[id[t]]: the gather is the framework's kernel, the scaling this part's own."""
    graph_safe = True

    @staticmethod
    def declare(spec):
        from vllm_lite_b200.parts.spec import TensorDecl
        return {"weight": TensorDecl((spec.vocab_size, spec.hidden_size))}

    def __init__(self, spec, weights, ctx):
        self.spec, self.table = spec, weights["weight"]

    def tied_weight(self):
        return self.table

    def __call__(self, step, x):
        from vllm_lite_b200.csrc import ops
        ops.embed(step.tokens, self.table, x, step.err)
        return x.mul_(self.spec.scale)


@dataclass(frozen=True)
class CappedHeadSpec:
    vocab_size: int
    hidden_size: int
    cap: float
    kind: str = "toy_capped_head"


class CappedHead:
    """logits = cap * tanh(h W^T / cap) with a matrix of its own."""
    graph_safe = True

    @staticmethod
    def declare(spec):
        from vllm_lite_b200.parts.spec import TensorDecl
        return {"weight": TensorDecl((spec.vocab_size, spec.hidden_size))}

    def __init__(self, spec, weights, ctx, embedding=None):
        from vllm_lite_b200.parts.linear import Linear
        self.spec, self.proj = spec, Linear(weights["weight"])

    def __call__(self, h, step):
        y = self.proj(h, step, "logits", out_dtype=torch.float32)
        return y.div_(self.spec.cap).tanh_().mul_(self.spec.cap)


class CenteredHeadNorm:
    """A head norm that is not an RMS norm: (x - mean) / sqrt(var + eps) * w over head_dim.  It offers
    no fused_rms(), so the attention mixer lets it edit the heads itself."""

    @staticmethod
    def declare(spec):
        from vllm_lite_b200.parts.spec import TensorDecl
        return {"weight": TensorDecl((spec.size,), init="norm")}

    def __init__(self, spec, weights, ctx):
        self.spec, self.weight = spec, weights["weight"].float()

    def apply_heads(self, qkv, first_head, num_heads, head_dim, step):
        T = qkv.shape[0]
        v = qkv[:, first_head * head_dim:(first_head + num_heads) * head_dim].view(T, num_heads, head_dim)
        v.copy_(centered_norm(v.float(), self.weight, self.spec.eps).to(qkv.dtype))


def centered_norm(x, w, eps):
    c = x - x.mean(dim=-1, keepdim=True)
    return c / torch.sqrt((c * c).mean(dim=-1, keepdim=True) + eps) * w


def plain_toy_ends(cfg, w, ids, scale, cap):
    """Scaled embedding; layer 0 with q/k/v biases and the centred head norm, layer 1 as in the plain
    model; capped head with a matrix of its own although the configuration ties the embeddings."""
    cfg = P.normalise_config(cfg)
    n, pos = len(ids), list(range(len(ids)))
    nq, nkv, d, eps = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"], cfg["rms_norm_eps"]
    x = scale * P.embedding(ids, w["model.embed_tokens.weight"])
    pre = "model.layers.0.self_attn."
    h = P.rms_norm(x, w["model.layers.0.input_layernorm.weight"], eps)
    q = (P.linear(h, w[pre + "q_proj.weight"]) + w[pre + "q_proj.bias"]).view(n, nq, d)
    k = (P.linear(h, w[pre + "k_proj.weight"]) + w[pre + "k_proj.bias"]).view(n, nkv, d)
    v = (P.linear(h, w[pre + "v_proj.weight"]) + w[pre + "v_proj.bias"]).view(n, nkv, d)
    q = P.rope(centered_norm(q, w[pre + "q_norm.weight"], eps), pos, cfg["rope_theta"])
    k = P.rope(centered_norm(k, w[pre + "k_norm.weight"], eps), pos, cfg["rope_theta"])
    x = x + P.linear(P.causal_attention(q, k, v).reshape(n, nq * d), w[pre + "o_proj.weight"])
    x = x + P.swiglu(P.rms_norm(x, w["model.layers.0.post_attention_layernorm.weight"], eps), w, "model.layers.0.")
    x = P.decoder_block(x, pos, w, 1, cfg)
    y = P.linear(P.rms_norm(x, w["model.norm.weight"], eps), w["lm_head.weight"])
    return cap * torch.tanh(y / cap)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_embedding_head_head_norm_and_biases_register_and_step(dtype):
    """The two ends of the model are parts like the others: a scaled embedding and a capped head defined
    here replace the plain ones; a head norm of another kind than RMS is dispatched to, not run as RMS;
    and projections may carry a bias.  Nothing of the framework is edited."""
    import dataclasses, json
    from vllm_lite_b200.config import Qwen3Config, plan_from_config_json, register_architecture, unregister_architecture
    from vllm_lite_b200.engine import ModelRunner, load_model_dir
    from vllm_lite_b200.parts import EMBEDDINGS, HEADS, NORMS, declare_model
    from vllm_lite_b200.parts.spec import ModelPlan, NormSpec
    from vllm_lite_b200.weights import random_tensors, write_safetensors
    scale, cap = 3.5, 0.4

    def plan(cfg):
        base = plan_from_config_json({**H.TINY_A, "architectures": ["Qwen3ForCausalLM"]})[1]
        l0, l1 = base.layers
        mixer = dataclasses.replace(l0.mixer, bias=True, qk_norm=NormSpec(cfg.head_dim, cfg.rms_norm_eps, kind="toy_centered"))
        return ModelPlan(**{**base.__dict__, "architecture": "ToyEndsLM", "layers": (dataclasses.replace(l0, mixer=mixer), l1),
                            "embedding": ScaledEmbeddingSpec(cfg.vocab_size, cfg.hidden_size, scale),
                            "head": CappedHeadSpec(cfg.vocab_size, cfg.hidden_size, cap)})

    EMBEDDINGS.register("toy_scaled_embedding", ScaledEmbedding)
    HEADS.register("toy_capped_head", CappedHead)
    NORMS.register("toy_centered", CenteredHeadNorm)
    register_architecture("ToyEndsLM", Qwen3Config, plan)
    try:
        cfg_json = {**H.TINY_A, "architectures": ["ToyEndsLM"]}
        d = H.tmp_root() / f"toy_ends_{dtype}"
        d.mkdir(exist_ok=True)
        (d / "config.json").write_text(json.dumps(cfg_json))
        _, p = plan_from_config_json(cfg_json)
        decl = declare_model(p)
        assert "lm_head.weight" in decl and "model.layers.0.self_attn.k_proj.bias" in decl
        assert "model.layers.1.self_attn.k_proj.bias" not in decl
        store = torch.float32 if dtype == "float32" else torch.bfloat16
        write_safetensors(d / "model.safetensors", random_tensors(decl, 4, std=0.06, dtype=store))
        _, p, weights = load_model_dir(d, dtype, DEV)
        runner = ModelRunner(p, weights, dtype=store, device=DEV, page_size=16, num_pages=8, max_requests=3)
        a, b = H.tokens_for("A", 37, 5), H.tokens_for("A", 12, 6)
        cfg, w = P.read_model_dir(d)
        ref = {"a": plain_toy_ends(cfg, w, a, scale, cap), "b": plain_toy_ends(cfg, w, b, scale, cap)}
        assert not torch.allclose(ref["a"], P.forward(cfg, w, a), atol=1e-2)
        rows = H.run_schedule(runner, [
            ([("a", a[:17], list(range(17)))], []),
            ([("a", a[17:19], [0, 1]), ("b", b, list(range(12)))], ["b"]),
            ([("a", a[19:20], [0])], []),
            ([("a", a[20:21], [0])], []),
            ([("a", a[21:], list(range(16)))], ["a"]),
        ])
        tol = 5e-5 if dtype == "float32" else H.TOL["bfloat16"]
        for (rid, pos), row in rows.items():
            assert float((row - ref[rid][pos]).abs().max()) <= tol * float(ref[rid].abs().max()), (rid, pos)
    finally:
        EMBEDDINGS.unregister("toy_scaled_embedding")
        HEADS.unregister("toy_capped_head")
        NORMS.unregister("toy_centered")
        unregister_architecture("ToyEndsLM")


def test_a_head_norm_that_offers_neither_form_is_refused_when_the_model_is_built():
    from vllm_lite_b200.parts import MIXERS, NORMS
    from vllm_lite_b200.parts.base import BuildContext
    from vllm_lite_b200.parts.spec import AttentionSpec, NormSpec, RotarySpec

    class Useless:
        declare = staticmethod(lambda spec: {})
        def __init__(self, spec, weights, ctx):
            pass

    NORMS.register("toy_useless", Useless)
    try:
        spec = AttentionSpec(32, 2, 1, 16, qk_norm=NormSpec(16, 1e-6, kind="toy_useless"), position=RotarySpec(16, 1e4))
        cls = MIXERS.get("gqa_attention")
        w = {k: torch.zeros(d.shape, device=DEV, dtype=torch.bfloat16) for k, d in cls.declare(spec).items()}
        with pytest.raises(TypeError, match="head norm"):
            cls(spec, w, BuildContext(torch.device(DEV), torch.bfloat16))
        with pytest.raises(ValueError, match="head_dim"):
            cls(AttentionSpec(32, 2, 1, 24), {}, BuildContext(torch.device(DEV), torch.bfloat16))
    finally:
        NORMS.unregister("toy_useless")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("tied", [False, True])
def test_embedding_and_output_head_alone(dtype, tied):
    """The two ends of a model as parts of their own, at sizes of no model: the gather into the float32
    stream (an id outside the table is flagged, never read, and its row is zero) and the float32 logits of chosen
    rows, with a matrix of the head's own or the embedding's table."""
    from vllm_lite_b200.parts import EMBEDDINGS, HEADS
    from vllm_lite_b200.parts.base import BuildContext
    from vllm_lite_b200.parts.spec import EmbeddingSpec, HeadSpec
    torch.manual_seed(3)
    V, Hd, T = 211, 88, 9
    ctx = BuildContext(torch.device(DEV), dtype)
    es, hs = EmbeddingSpec(V, Hd), HeadSpec(V, Hd, tied=tied)
    assert EMBEDDINGS.get(es.kind).declare(es)["weight"].shape == (V, Hd)
    assert ("weight" in HEADS.get(hs.kind).declare(hs)) == (not tied)
    table = (torch.randn(V, Hd) * 0.3).to(dtype)
    own = (torch.randn(V, Hd) * 0.3).to(dtype)
    emb = EMBEDDINGS.get(es.kind)(es, {"weight": table.to(DEV)}, ctx)
    head = HEADS.get(hs.kind)(hs, {} if tied else {"weight": own.to(DEV)}, ctx, embedding=emb)
    step = make_step(None, T)
    ids = torch.tensor([0, 5, V - 1, 17, 17, 3, 99, 210, 1], dtype=torch.int32)
    step.tokens = ids.to(DEV)
    x = torch.full((T, Hd), 7.0, device=DEV)
    emb(step, x)
    assert torch.equal(x.cpu(), table.float()[ids.long()])
    assert int(step.err.item()) == 0
    step.tokens = torch.tensor([2, V, 4] + [0] * (T - 3), dtype=torch.int32, device=DEV)      # V lies outside the table
    y = torch.full((T, Hd), 7.0, device=DEV)
    emb(step, y)
    assert int(step.err.item()) & 1 and bool((y[1] == 0.0).all()) and torch.equal(y[0].cpu(), table.float()[2])
    h = (torch.randn(4, Hd, device=DEV) * 0.5).to(dtype)
    logits = head(h, step)
    assert logits.dtype == torch.float32 and logits.shape == (4, V)
    ref = h.float().cpu() @ (table if tied else own).float().T
    tol = dict(atol=1e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)
    assert torch.allclose(logits.cpu(), ref, **tol)
    with pytest.raises(ValueError, match="tied"):
        HEADS.get(hs.kind)(HeadSpec(V, Hd, tied=True), {}, ctx, embedding=None)
