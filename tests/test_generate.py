"""Generation through the Python entry point and the command line."""
import math
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import helpers as H
import plain_qwen3 as P

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def plain_greedy(which, prompt, n):
    toks = list(prompt)
    for _ in range(n):
        toks.append(P.argmax(H.plain_logits(which, toks)[-1].tolist()))
    return toks[len(prompt):]


def engine(which, dtype="float32", **kw):
    from vllm_lite_b200 import LLMEngine
    kw.setdefault("kv_blocks", 64)
    return LLMEngine(str(H.model_dir(which)), dtype=dtype, block_size=H.TINY[which]["page_size"], **kw)


@pytest.mark.parametrize("which,lengths", [("A", [5, 17, 33]), ("B", [1, 9, 40, 64, 100])])
def test_greedy_generation_matches_the_plain_implementation(which, lengths):
    prompts = [H.tokens_for(which, n, 50 + i) for i, n in enumerate(lengths)]
    eng = engine(which, max_num_batched_tokens=48, prefill_chunk_size=13)
    outs = eng.generate(prompts, max_tokens=16)
    for p, o in zip(prompts, outs):
        assert o == plain_greedy(which, p, 16)
    st = eng.stats()
    assert st["free_pages"] == [64] and st["finished"] == len(prompts)


def test_greedy_generation_bfloat16_follows_the_plain_logits():
    """bfloat16 may pick another token where two logits are close; every chosen token must be
    within bfloat16 tolerance of the plain maximum given the tokens chosen so far."""
    which = "B"
    prompts = [H.tokens_for(which, n, 60 + i) for i, n in enumerate([9, 40])]
    outs = engine(which, "bfloat16").generate(prompts, max_tokens=12)
    for p, o in zip(prompts, outs):
        toks = list(p)
        for t in o:
            row = H.plain_logits(which, toks)[-1]
            assert float(row.max() - row[t]) <= H.TOL["bfloat16"] * float(row.abs().max()) * 2
            toks.append(t)


def test_preemption_by_recompute_gives_the_same_tokens():
    which = "B"
    prompts = [H.tokens_for(which, n, 70 + i) for i, n in enumerate([30, 28, 25])]
    want = [plain_greedy(which, p, 20) for p in prompts]
    eng = engine(which, kv_blocks=15, max_model_len=64)            # 120 slots for 3 x ~50 tokens: someone must yield
    outs = eng.generate(prompts, max_tokens=20)
    assert eng.stats()["preemptions"] >= 1
    assert outs == want and eng.stats()["free_pages"] == [15]


def test_temperature_sampling_with_a_seed():
    from vllm_lite_b200 import SamplingParams
    from vllm_lite_b200.sampling import seeded_uniform
    which = "B"
    prompt = H.tokens_for(which, 9, 80)
    params = SamplingParams(temperature=0.8, seed=1234)
    a = engine(which).generate([prompt], max_tokens=10, sampling_params=params)[0]
    b = engine(which).generate([prompt, prompt[:5]], max_tokens=10, sampling_params=params)[0]
    assert a == b                                                   # same seed, same prompt, whatever the batch
    c = engine(which).generate([prompt], max_tokens=10, sampling_params=SamplingParams(temperature=0.8, seed=99))[0]
    assert a != c
    toks = list(prompt)
    for step, t in enumerate(a):                                    # each draw is the inverse CDF at u(seed, step)
        u = seeded_uniform(1234, step)
        cdf = np.cumsum(P.temperature_probs(H.plain_logits(which, toks)[-1].tolist(), 0.8))
        lo = cdf[t - 1] if t else 0.0
        assert lo - 1e-4 <= u <= cdf[t] + 1e-4
        toks.append(t)


def test_stop_sequence_and_step_outputs():
    from vllm_lite_b200 import SamplingParams
    which = "B"
    prompt = H.tokens_for(which, 17, 90)
    free = plain_greedy(which, prompt, 8)
    stop = free[2:4]
    expect = next(free[:n] for n in range(2, 9) if free[:n][-2:] == stop)     # the first suffix match ends it
    eng = engine(which)
    sid = eng.add_request(prompt, 8, SamplingParams(stop_token_sequences=[stop]))
    outs = []
    while eng.has_unfinished():
        outs += eng.step()
    assert [o.token for o in outs] == expect and outs[-1].finished and outs[-1].finish_reason == "stop"
    assert all(o.seq_id == sid for o in outs)
    with pytest.raises(ValueError):
        eng.add_request([999999], 4)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_steps_launched_ahead_change_nothing_but_the_timing(dtype):
    """With lookahead the engine launches the next decode step before it has read this step's
    tokens.  Tokens, finish reasons and the books are those of the engine that waits: greedy and
    seeded temperature requests, one that ends on a stop sequence, one that arrives later, one
    that is cancelled while a step launched ahead holds it."""
    from vllm_lite_b200 import SamplingParams
    which = "B"
    prompts = [H.tokens_for(which, n, 200 + i) for i, n in enumerate([12, 30, 7, 21])]
    stop = plain_greedy(which, prompts[2], 6)[3:5]

    def run(lookahead):
        eng = engine(which, dtype=dtype, lookahead=lookahead, max_num_batched_tokens=64, prefill_chunk_size=16)
        ids = [eng.add_request(prompts[0], 14),
               eng.add_request(prompts[1], 9, SamplingParams(temperature=0.7, seed=5)),
               eng.add_request(prompts[2], 12, SamplingParams(stop_token_sequences=[stop]))]
        got, ahead, steps = {}, 0, 0
        while eng.has_unfinished():
            for o in eng.step():
                got.setdefault(o.seq_id, []).append((o.token, o.finished, o.finish_reason))
            ahead += eng._ahead is not None
            steps += 1
            if steps == 5:
                ids.append(eng.add_request(prompts[3], 30))
            if len(ids) == 4 and len(got.get(ids[3], [])) == 6 and ids[3] in eng.sequences and eng.sequences[ids[3]].status == "running":
                eng.cancel_request(ids[3])
        eng.runner.check_device_errors()
        eng.runner.cache.check_invariants()
        assert eng.stats()["free_pages"] == [64] and eng.stats()["running"] == 0
        return [got[i] for i in ids], ahead

    waited, n0 = run(False)
    ahead, n1 = run(True)
    assert n0 == 0 and n1 > 5                      # steps were in fact launched ahead
    assert waited[0][-1][1:] == (True, "length") and waited[2][-1][1:] == (True, "stop")
    assert ahead[0][-1][1:] == (True, "length") and ahead[2][-1][1:] == (True, "stop")
    assert [len(r) for r in ahead[:2]] == [len(r) for r in waited[:2]] == [14, 9] and len(ahead[3]) == len(waited[3]) == 6
    if dtype == "float32":
        # float32 results do not depend on what shares a step, so the tokens are the same to the last one
        # (in bfloat16 a request that joins or leaves a step one step later moves roundings, and a
        # near tie may fall the other way)
        assert ahead[:3] == waited[:3] and ahead[3][:6] == waited[3][:6]


def test_long_steps_are_launched_without_dependent_launch():
    """Steps of few tokens overlap each kernel's start with the end of the one before (programmatic
    dependent launch); steps of many tokens are launched the plain way.  The switch follows the step."""
    from vllm_lite_b200.csrc import build, ops
    from vllm_lite_b200.engine import StepEntry
    from vllm_lite_b200.engine.runner import PDL_MAX_TOKENS
    which = "B"
    runner = engine(which, dtype="bfloat16").runner
    long = H.tokens_for(which, PDL_MAX_TOKENS + 6, 300)
    def told():                                     # what every loaded library was last told
        return {int(build.load(lib, dict([("FA_HD", int(var[5:]))]) if var else None).vl_get_pdl())
                for lib, var in ops._pdl_libs}
    whole = runner.step([StepEntry("a", long, [len(long) - 1])]).clone()
    assert ops._pdl is False and told() == {0}
    runner.step([StepEntry("a", [5], [0])])
    assert ops._pdl is True and told() == {1}
    runner.step([StepEntry("b", long[:10], [])])
    assert ops._pdl is True and told() == {1}
    cut = runner.step([StepEntry("b", long[10:], [len(long) - 11])])      # 60 tokens, with the attribute
    runner.check_device_errors()
    tol = H.TOL["bfloat16"] * float(whole.abs().max())
    assert float((whole - cut).abs().max()) <= tol


def test_command_line(tmp_path):
    which = "A"
    prompt = H.tokens_for(which, 12, 95)
    cmd = [sys.executable, "-m", "vllm_lite_b200", "--model", str(H.model_dir(which)), "--dtype", "float32",
           "--kv-blocks", "32", "--max-tokens", "6", "--prompt-ids", ",".join(map(str, prompt)), "--log-level", "warn"]
    proc = subprocess.run(cmd, capture_output=True, text=True, cwd=ROOT, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [int(t) for t in proc.stdout.strip().split(",")] == plain_greedy(which, prompt, 6)
    bad = subprocess.run([sys.executable, "-m", "vllm_lite_b200", "--prompt-ids", "1,2"], capture_output=True, text=True,
                         cwd=ROOT, env={k: v for k, v in __import__("os").environ.items() if k != "VLLM_MODEL"})
    assert bad.returncode == 2 and "--model" in bad.stderr


def test_stats_report_step_counts_and_times_by_kind():
    which = "B"
    eng = engine(which, dtype="bfloat16", max_num_batched_tokens=32, prefill_chunk_size=16)
    eng.generate([H.tokens_for(which, 40, 400), H.tokens_for(which, 9, 401)], max_tokens=40)
    times = eng.stats()["step_times"]
    assert set(times) == {"prompt", "mixed", "decode"}
    assert times["prompt"]["steps"] >= 1 and times["decode"]["steps"] >= 30
    assert times["prompt"]["steps"] + times["mixed"]["steps"] + times["decode"]["steps"] >= 40
    d = times["decode"]
    assert d["host_ms_p50"] is not None and 0 < d["host_ms_p50"] <= d["host_ms_p90"]
    torch.cuda.synchronize()
    sampled = sum(t["device_samples"] for t in eng.stats()["step_times"].values())
    assert sampled >= 2                                     # every 16th step is timed on the device
    assert all(t["device_ms_p50"] is None or t["device_ms_p50"] > 0 for t in eng.stats()["step_times"].values())
