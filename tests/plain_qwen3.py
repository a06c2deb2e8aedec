"""Plain, slow implementation of the Qwen3 dense decoder, whole sequences, no cache.

It is the oracle of the tests.  It shares no code with the product path: it
reads config.json and model.safetensors itself, works on the CPU in float32 (or
float64), and has one function for each part.  Each function is written from
the formulas of pplmx/vllm-lite (paths are relative to that project) and cites
the file and lines it was written from.

The reference project is a Rust workspace; no Rust toolchain and no copy of its
tensor library are available where these tests run, so the reference's own model
code can be neither imported nor compiled here.  This file therefore rests on
the formulas, not on outputs of the reference.  One deliberate reading is
recorded where the reference wires a mean-subtracting layer norm object into its
Qwen3 blocks (crates/model/src/components/decoder_block/mod.rs:23-24): the
architecture's key is `rms_norm_eps` and the formula taken here is the RMS one
of crates/model/src/components/norm/rms_norm.rs:26-49 at every norm site.
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np
import torch


# --------------------------------------------------------------------------
# reading a model folder (independent of the product's loader)
# --------------------------------------------------------------------------

_ST_DTYPES = {"F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16,
              "I32": torch.int32, "I64": torch.int64}


def read_safetensors(path) -> dict:
    """Tensor name -> torch tensor, widened to float32 like the reference's
    loader does (crates/model/src/loader/io.rs:82-140)."""
    raw = Path(path).read_bytes()
    (hlen,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + hlen])
    base = 8 + hlen
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        lo, hi = meta["data_offsets"]
        dt = _ST_DTYPES[meta["dtype"]]
        t = torch.frombuffer(bytearray(raw[base + lo:base + hi]), dtype=dt).reshape(meta["shape"])
        out[name] = t.float() if dt.is_floating_point else t
    return out


def read_model_dir(model_dir):
    cfg = json.loads((Path(model_dir) / "config.json").read_text())
    weights = read_safetensors(Path(model_dir) / "model.safetensors")
    return cfg, weights


# --------------------------------------------------------------------------
# parts
# --------------------------------------------------------------------------

def embedding(ids, table):
    """x_t = E[id_t], no scaling.  crates/model/src/causal_lm/mod.rs:28-46."""
    return table[torch.as_tensor(ids, dtype=torch.long)]


def rms_norm(x, weight, eps):
    """x / sqrt(mean(x^2) + eps) * w over the last axis.
    crates/model/src/components/norm/rms_norm.rs:26-49."""
    variance = (x * x).mean(dim=-1, keepdim=True)
    return x / torch.sqrt(variance + eps) * weight


def linear(x, weight):
    """y = x W^T, weight stored [out, in], no bias when built from weights.
    crates/model/src/components/attention/gqa/norm.rs:21-26,
    crates/model/src/components/attention/gqa/mod.rs:120-123."""
    return x @ weight.T


def rope_inv_freq(head_dim, theta):
    """inv_freq[i] = theta^(-2i/d), i < d/2, in float32.
    crates/model/src/components/positional/rope.rs:498-503."""
    half = head_dim // 2
    th = np.float32(theta)
    return torch.tensor([float(np.power(th, np.float32(-2.0) * np.float32(i) / np.float32(head_dim)))
                         for i in range(half)], dtype=torch.float32)


def rope(x, positions, theta):
    """Rotate-half pairing (x_i, x_{i+d/2}) of [tokens, heads, d]; the angle is
    (f32)pos * inv_freq[i]; x1' = x1 cos - x2 sin, x2' = x2 cos + x1 sin.
    crates/model/src/components/positional/rope.rs:507-558."""
    d = x.shape[-1]
    half = d // 2
    inv = rope_inv_freq(d, theta)
    pos = torch.as_tensor(positions, dtype=torch.float32)
    angle = (pos[:, None] * inv[None, :])            # float32 product, as the reference
    cos = torch.cos(angle.double()).to(x.dtype)[:, None, :]
    sin = torch.sin(angle.double()).to(x.dtype)[:, None, :]
    x1, x2 = x[..., :half], x[..., half:]
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1)


def head_norm(x, weight, eps):
    """Per (token, head) norm over head_dim with one weight vector shared by all
    heads, applied to q and k before the rotation; v is not normed.
    crates/model/src/components/attention/rope_gqa.rs:214-248."""
    return rms_norm(x, weight, eps)


def causal_attention(q, k, v, window=None):
    """q [P,nq,d], k,v [P,nkv,d].  Query head j reads KV head j // (nq/nkv)
    (crates/model/src/components/attention/util.rs:55-87); scores q.k, mask
    (key position <= query position) added first, then * 1/sqrt(d), softmax
    with the maximum subtracted, then the weighted sum of v
    (crates/model/src/components/attention/util.rs:150-176).  `window`, when
    given, keeps only the last `window` keys of each query; the reference
    parses sliding_window and drops it for this architecture
    (crates/model/src/config/hyperparams.rs:153)."""
    P, nq, d = q.shape
    nkv = k.shape[1]
    g = nq // nkv
    out = torch.empty_like(q)
    row = torch.arange(P)[:, None]
    col = torch.arange(P)[None, :]
    keep = col <= row
    if window is not None:
        keep = keep & (col > row - window)
    for j in range(nq):
        kvh = j // g
        s = q[:, j] @ k[:, kvh].T
        s = torch.where(keep, s, torch.full_like(s, float("-inf"))) * (d ** -0.5)
        s = s - s.max(dim=-1, keepdim=True).values
        p = torch.exp(s)
        p = p / p.sum(dim=-1, keepdim=True)
        out[:, j] = p @ v[:, kvh]
    return out


def attention_block(h, positions, w, prefix, cfg):
    """project -> head norm -> rotation -> attention -> output projection.
    crates/model/src/components/attention/rope_gqa.rs:261-305,
    crates/model/src/components/attention/paged_gqa.rs:170-181."""
    P = h.shape[0]
    nq, nkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    eps = cfg["rms_norm_eps"]
    q = linear(h, w[prefix + "self_attn.q_proj.weight"]).view(P, nq, d)
    k = linear(h, w[prefix + "self_attn.k_proj.weight"]).view(P, nkv, d)
    v = linear(h, w[prefix + "self_attn.v_proj.weight"]).view(P, nkv, d)
    q = head_norm(q, w[prefix + "self_attn.q_norm.weight"], eps)
    k = head_norm(k, w[prefix + "self_attn.k_norm.weight"], eps)
    q = rope(q, positions, cfg["rope_theta"])
    k = rope(k, positions, cfg["rope_theta"])
    o = causal_attention(q, k, v)
    return linear(o.reshape(P, nq * d), w[prefix + "self_attn.o_proj.weight"])


def swiglu(h, w, prefix):
    """down(silu(gate(h)) * up(h)), silu(z) = z / (1 + exp(-z)), no biases.
    crates/model/src/components/mlp/swiglu.rs:18-31."""
    g = linear(h, w[prefix + "mlp.gate_proj.weight"])
    u = linear(h, w[prefix + "mlp.up_proj.weight"])
    return linear(g / (1.0 + torch.exp(-g)) * u, w[prefix + "mlp.down_proj.weight"])


def decoder_block(x, positions, w, layer, cfg):
    """norm -> attention -> + residual -> norm -> feed-forward -> + residual.
    crates/model/src/components/decoder_block/mod.rs:66-85."""
    prefix = f"model.layers.{layer}."
    eps = cfg["rms_norm_eps"]
    h = rms_norm(x, w[prefix + "input_layernorm.weight"], eps)
    x = x + attention_block(h, positions, w, prefix, cfg)
    h = rms_norm(x, w[prefix + "post_attention_layernorm.weight"], eps)
    return x + swiglu(h, w, prefix)


def normalise_config(cfg):
    cfg = dict(cfg)
    cfg.setdefault("num_key_value_heads", cfg["num_attention_heads"])
    cfg.setdefault("head_dim", cfg["hidden_size"] // cfg["num_attention_heads"])
    cfg.setdefault("rope_theta", 10000.0)
    cfg.setdefault("tie_word_embeddings", False)
    return cfg


def forward(cfg, w, ids, dtype=torch.float32):
    """Logits [P, V] of one whole sequence at positions 0..P-1:
    embed -> layers -> final norm -> lm head (tied: the embedding table).
    crates/model/src/causal_lm/mod.rs:180-221,
    crates/model/src/causal_lm/weights.rs:19-36."""
    cfg = normalise_config(cfg)
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in w.items()}
    positions = list(range(len(ids)))
    x = embedding(ids, w["model.embed_tokens.weight"])
    for layer in range(cfg["num_hidden_layers"]):
        x = decoder_block(x, positions, w, layer, cfg)
    h = rms_norm(x, w["model.norm.weight"], cfg["rms_norm_eps"])
    head = w["model.embed_tokens.weight"] if cfg["tie_word_embeddings"] else w["lm_head.weight"]
    return linear(h, head)


# --------------------------------------------------------------------------
# sampling (crates/core/src/sampling.rs)
# --------------------------------------------------------------------------

def argmax(logits):
    """Ties go to the lowest index.  crates/traits/src/sampling.rs:439-453."""
    best, arg = -math.inf, 0
    for i, v in enumerate(logits):
        if v > best:
            best, arg = v, i
    return arg


def apply_repeat_penalty(logits, seen, penalty):
    """Once per distinct seen id: l >= 0 ? l / p : l * p.
    crates/core/src/sampling.rs:670-688."""
    out = list(logits)
    for t in set(seen):
        if t < len(out):
            out[t] = out[t] / penalty if out[t] >= 0 else out[t] * penalty
    return out


def apply_presence_penalty(logits, seen, penalty):
    """l -= penalty once per distinct seen id.  crates/core/src/sampling.rs:716-730."""
    out = list(logits)
    for t in set(seen):
        if t < len(out):
            out[t] -= penalty
    return out


def apply_logit_bias(logits, bias):
    """l[id] += b, ids beyond the vocabulary ignored.  crates/core/src/sampling.rs:760-775."""
    out = list(logits)
    for t, b in bias.items():
        if 0 <= int(t) < len(out):
            out[int(t)] += b
    return out


def top_k_mask(logits, k):
    """The k-th largest value is the threshold; l < threshold becomes -inf, ties
    at the threshold are kept.  crates/core/src/sampling.rs:525-539."""
    k = min(k, len(logits))
    thr = sorted(logits, reverse=True)[k - 1]
    return [v if v >= thr else -math.inf for v in logits]


def temperature_probs(logits, temperature):
    """softmax(l / T) with the maximum subtracted, in index order.
    crates/core/src/sampling.rs:192-245."""
    s = np.asarray(logits, dtype=np.float64) / temperature
    s = np.where(np.isnan(s), -np.inf, s)
    e = np.exp(s - s.max())
    return e / e.sum()


def temperature_sample(logits, temperature, u):
    """Inverse CDF in index order: the first i with u <= cumsum_i, else the last
    index.  crates/core/src/sampling.rs:237-245."""
    if temperature <= 0:
        return argmax(logits)
    c = np.cumsum(temperature_probs(logits, temperature))
    idx = int(np.searchsorted(c, u, side="left"))
    return min(idx, len(logits) - 1)


def top_p_keep(logits, top_p):
    """Indices kept by the nucleus: sorted by probability descending, the
    shortest prefix whose cumulative probability exceeds top_p (the crossing
    token included).  crates/core/src/sampling.rs:247-308."""
    p = temperature_probs(logits, 1.0)
    order = sorted(range(len(p)), key=lambda i: (-p[i], i))
    total, keep = 0.0, []
    for i in order:
        keep.append(i)
        total += p[i]
        if total > top_p:
            break
    return keep
