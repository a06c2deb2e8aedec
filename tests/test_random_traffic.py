"""Random schedules and random traffic: what no hand-written case thought of.

`test_random_cuts` feeds the step function schedules drawn at random (up to four live requests, portions
of 1 to 200 tokens beside single tokens, requests left out of steps, wanted places anywhere, just enough
pages) and compares every wanted row with the plain implementation.  `test_random_requests` drives
`LLMEngine` with requests that arrive over time under random limits (token budget, portion size, batch
size, pools small enough to force pre-emption, steps launched ahead or not) and compares the greedy
tokens with the plain implementation's."""
import random

import pytest

import helpers as H
import plain_qwen3 as P

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("seed", range(12))
def test_random_cuts(seed):
    rng = random.Random(seed)
    which = ["A", "B", "C"][seed % 3]
    dtype = rng.choice(["float32", "bfloat16"])
    page = rng.choice([8, 16, 64]) if which == "C" else H.TINY[which]["page_size"]
    lens = {f"r{i}": rng.randint(1, 300 if which == "C" else 110) for i in range(rng.randint(2, 6))}
    reqs = {k: H.tokens_for(which, n, seed * 10 + i) for i, (k, n) in enumerate(lens.items())}
    fed = {k: 0 for k in reqs}
    live, pending, schedule, wanted = [], list(reqs), [], 0
    while pending or live:
        while pending and len(live) < 4 and (not live or rng.random() < 0.6):
            live.append(pending.pop(0))
        entries, end = [], []
        for k in list(live):
            if rng.random() < 0.25 and len(live) > 1:
                continue                                # this request sits the step out
            left = lens[k] - fed[k]
            mode = rng.random()
            n = 1 if mode < 0.4 else min(left, rng.randint(2, 20) if mode < 0.8 else rng.randint(2, 200))
            n = max(1, min(n, left))
            want = sorted(rng.sample(range(n), rng.randint(1 if n == left else 0, min(n, 3))))
            wanted += len(want)
            entries.append((k, reqs[k][fed[k]:fed[k] + n], want))
            fed[k] += n
            if fed[k] == lens[k]:
                end.append(k)
                live.remove(k)
        if entries:
            schedule.append((entries, end))
    pages = sum(-(-n // page) for n in lens.values())
    runner = H.make_runner(which, dtype, num_pages=pages, page_size=page)
    rows = H.run_schedule(runner, schedule)
    assert len(rows) == wanted > 0
    H.assert_rows_match(rows, which, reqs, dtype, f"random cuts, seed {seed}")
    assert runner.cache.free_pages() == [pages]


def plain_greedy(which, prompt, n):
    toks = list(prompt)
    for _ in range(n):
        toks.append(P.argmax(H.plain_logits(which, toks)[-1].tolist()))
    return toks[len(prompt):]


@pytest.mark.parametrize("seed", range(10))
def test_random_requests(seed):
    from vllm_lite_b200 import LLMEngine
    rng = random.Random(1000 + seed)
    which = ["A", "B", "C"][seed % 3]
    page = H.TINY[which]["page_size"]
    nreq = rng.randint(2, 7)
    prompts = [H.tokens_for(which, rng.randint(1, 60), seed * 20 + i) for i in range(nreq)]
    limits = [rng.randint(1, 24) for _ in range(nreq)]
    blocks = max(rng.choice([12, 20, 64]), 1 + max(-(-(len(p) + m) // page) for p, m in zip(prompts, limits)))
    eng = LLMEngine(str(H.model_dir(which)), dtype="float32", block_size=page, kv_blocks=blocks,
                    max_batch_size=rng.choice([2, 4, 8]), max_num_batched_tokens=rng.choice([16, 48, 256]),
                    prefill_chunk_size=rng.choice([5, 16, 64]), max_model_len=128, lookahead=seed % 4 != 3)
    arrivals = sorted(rng.randint(0, 15) for _ in range(nreq))
    ids, got, step, added = {}, {}, 0, 0
    while added < nreq or eng.has_unfinished():
        while added < nreq and arrivals[added] <= step:
            ids[eng.add_request(prompts[added], limits[added])] = added
            added += 1
        for o in eng.step():
            got.setdefault(ids[o.seq_id], []).append(o.token)
        step += 1
        assert step < 3000
    eng.runner.check_device_errors()
    eng.runner.cache.check_invariants()
    assert eng.stats()["free_pages"] == [blocks]
    for i in range(nreq):
        assert got.get(i) == plain_greedy(which, prompts[i], limits[i]), i
