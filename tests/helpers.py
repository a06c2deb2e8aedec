"""Shared by the tests: the two tiny configurations, model folders in temporary
places, the plain implementation's logits, and replay of a schedule of steps."""
from __future__ import annotations

import functools
import json
import tempfile
from pathlib import Path

import numpy as np
import torch

import plain_qwen3 as plain

# Two tiny configurations that differ in every size and option.
TINY_A = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_size=64, num_hidden_layers=2,
              num_attention_heads=4, num_key_value_heads=2, head_dim=16, intermediate_size=128, vocab_size=256,
              rope_theta=10000.0, rms_norm_eps=1e-6, tie_word_embeddings=True, max_position_embeddings=256)
TINY_B = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_size=96, num_hidden_layers=3,
              num_attention_heads=8, num_key_value_heads=2, head_dim=32, intermediate_size=160, vocab_size=333,
              rope_theta=1000000.0, rms_norm_eps=1e-5, tie_word_embeddings=False, max_position_embeddings=512)
# head size 64: the size class of the tcgen05 / TMA attention kernels (used for long portions and, with
# pages of 64 positions, for decoding); the other sizes are again no powers of two
TINY_C = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_size=72, num_hidden_layers=2,
              num_attention_heads=6, num_key_value_heads=2, head_dim=64, intermediate_size=104, vocab_size=301,
              rope_theta=50000.0, rms_norm_eps=3e-6, tie_word_embeddings=False, max_position_embeddings=640)
# a long context: decoding crosses the bounds (1,024, 2,048) that the decode graphs are recorded for
TINY_L = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_size=80, num_hidden_layers=2,
              num_attention_heads=5, num_key_value_heads=1, head_dim=32, intermediate_size=112, vocab_size=199,
              rope_theta=200000.0, rms_norm_eps=2e-6, tie_word_embeddings=True, max_position_embeddings=4096)
TINY = {"L": dict(config=TINY_L, seed=4, std=0.05, page_size=16),
        "A": dict(config=TINY_A, seed=0, std=0.02, page_size=16),
        "B": dict(config=TINY_B, seed=1, std=0.05, page_size=8),
        "C": dict(config=TINY_C, seed=2, std=0.04, page_size=16)}

# max |engine - plain| allowed, as a fraction of max |plain| over the compared rows.  The run's summary
# prints the worst error of every comparison (conftest.py); the worst ever seen were 1.4e-2 in bfloat16
# and 7.5e-6 in float32 (both at real layer widths, sums over 12,288 products), so the bfloat16 bound
# stands at twice that; float32 at tiny sizes stays below 1.3e-6.
TOL = {"float32": 2e-5, "bfloat16": 2.8e-2}

_tmp_root = None


def tmp_root() -> Path:
    global _tmp_root
    if _tmp_root is None:
        _tmp_root = tempfile.TemporaryDirectory(prefix="vl_b200_tests_")
    return Path(_tmp_root.name)


def _store(dtype) -> str:
    """The precision a case's folder is written in: a float32 engine is given weights with all their
    bits (a path that dropped low bits of a weight would show), a bfloat16 engine bfloat16 ones."""
    return "float32" if str(dtype).endswith("float32") else "bfloat16"


@functools.lru_cache(maxsize=None)
def _model_dir(which: str, store: str) -> Path:
    from vllm_lite_b200.weights import write_model_dir
    spec = TINY[which]
    d = tmp_root() / f"tiny_{which}_{store}"
    write_model_dir(d, spec["config"], spec["seed"], std=spec["std"],
                    dtype=torch.float32 if store == "float32" else torch.bfloat16)
    return d


def model_dir(which: str, dtype="bfloat16") -> Path:
    return _model_dir(which, _store(dtype))


@functools.lru_cache(maxsize=None)
def _plain_model(which: str, store: str):
    return plain.read_model_dir(_model_dir(which, store))


def plain_model(which: str, dtype="bfloat16"):
    return _plain_model(which, _store(dtype))


def tokens_for(which: str, length: int, seed: int):
    rng = np.random.default_rng(1000 + seed)
    return [int(t) for t in rng.integers(0, TINY[which]["config"]["vocab_size"], size=length)]


_plain_cache = {}


def plain_logits(which: str, tokens, dtype="bfloat16") -> torch.Tensor:
    key = (which, _store(dtype), tuple(tokens))
    if key not in _plain_cache:
        cfg, w = plain_model(which, dtype)
        _plain_cache[key] = plain.forward(cfg, w, list(tokens))
    return _plain_cache[key]


def make_runner(which: str, dtype: str, num_pages: int, page_size=None, max_requests=8, native_host=True, **kw):
    from vllm_lite_b200.engine import ModelRunner, load_model_dir
    _, plan, weights = load_model_dir(model_dir(which, dtype), dtype, "cuda:0")
    return ModelRunner(plan, weights, dtype=torch.bfloat16 if dtype == "bfloat16" else torch.float32,
                       device="cuda:0", page_size=page_size or TINY[which]["page_size"], num_pages=num_pages,
                       max_requests=max_requests, native_host=native_host, **kw)


def run_schedule(runner, schedule):
    """schedule: list of steps; a step is (entries, end) with entries = [(id, tokens, want)].
    Returns {(id, position): logits row (CPU float32)}."""
    from vllm_lite_b200.engine import StepEntry
    fed, rows = {}, {}
    for entries, end in schedule:
        out = runner.step([StepEntry(i, t, w) for i, t, w in entries])
        runner.check_device_errors()
        out = out.float().cpu()
        r = 0
        for i, t, w in entries:
            base = fed.get(i, 0)
            for place in w:
                rows[(i, base + place)] = out[r].clone()
                r += 1
            fed[i] = base + len(t)
        assert r == out.shape[0]
        for i in end:
            runner.release(i)
            fed.pop(i, None)
        runner.cache.check_invariants()
    return rows


WORST = {}        # (what, configuration, dtype) -> the largest error any comparison saw; printed when the run ends


def assert_rows_match(rows, which, requests, dtype, what=""):
    """rows: {(id, position): row}; requests: {id: tokens}."""
    assert rows, "nothing was compared"
    worst = 0.0
    for (rid, pos), row in rows.items():
        ref = plain_logits(which, requests[rid], dtype)[pos]
        scale = float(ref.abs().max())
        err = float((row - ref).abs().max()) / max(scale, 1e-12)
        worst = max(worst, err)
        assert err <= TOL[dtype], (f"{what} {which}/{dtype}: request {rid} position {pos}: "
                                   f"max|diff|/max|ref| = {err:.3e} > {TOL[dtype]:.1e}")
    key = (what, which, dtype)
    WORST[key] = max(WORST.get(key, 0.0), worst)
    return worst
