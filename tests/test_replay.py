"""The engine against the plain implementation under every way of cutting the work:
each request alone and whole; most of it in one step and the last 32 tokens one by
one; portions of changing size down to two tokens; and up to four live requests
mixed, portions of some beside decoded tokens of others, with so few pages that
they are used again.  In float32 and in bfloat16, on the tiny configurations."""
import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import helpers as H

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
CASES = [(w, d) for w in ("A", "B", "C") for d in ("float32", "bfloat16")]
LENGTHS = {"A": [5, 17, 33, 70], "B": [1, 9, 40, 64, 100], "C": [3, 64, 65, 128]}


def pages_for(which, tokens):
    ps = H.TINY[which]["page_size"]
    return -(-tokens // ps)


@pytest.mark.parametrize("which,dtype", CASES)
def test_whole(which, dtype):
    runner = H.make_runner(which, dtype, num_pages=pages_for(which, 128))
    for n, length in enumerate(LENGTHS[which]):
        toks = H.tokens_for(which, length, n)
        rows = H.run_schedule(runner, [([("r", toks, list(range(length)))], ["r"])])
        H.assert_rows_match(rows, which, {"r": toks}, dtype, "whole")
    assert runner.cache.free_pages() == [pages_for(which, 128)]


@pytest.mark.parametrize("which,dtype", CASES)
def test_last_32_decoded(which, dtype):
    length = 100
    toks = H.tokens_for(which, length, 7)
    runner = H.make_runner(which, dtype, num_pages=pages_for(which, 128))
    head = length - 32
    schedule = [([("r", toks[:head], [head - 1])], [])]
    schedule += [([("r", [toks[p]], [0])], []) for p in range(head, length)]
    rows = H.run_schedule(runner, schedule)
    assert len(rows) == 33
    H.assert_rows_match(rows, which, {"r": toks}, dtype, "decode")


@pytest.mark.parametrize("which,dtype", CASES)
def test_first_tokens(which, dtype):
    """The very first positions of a sequence, fed one by one from an empty cache."""
    toks = H.tokens_for(which, 6, 3)
    runner = H.make_runner(which, dtype, num_pages=4)
    rows = H.run_schedule(runner, [([("r", [t], [0])], []) for t in toks])
    H.assert_rows_match(rows, which, {"r": toks}, dtype, "first tokens")


@pytest.mark.parametrize("which,dtype", CASES)
def test_changing_portions(which, dtype):
    length = 120
    toks = H.tokens_for(which, length, 11)
    runner = H.make_runner(which, dtype, num_pages=pages_for(which, 128))
    sizes = [7, 2, 13, 3, 2, 16, 5, 2, 31, 8, 2, 17, 2, 2, 3]
    schedule, p, k = [], 0, 0
    while p < length:
        n = min(sizes[k % len(sizes)], length - p)
        k += 1
        schedule.append(([("r", toks[p:p + n], list(range(n)))], []))
        p += n
    rows = H.run_schedule(runner, schedule)
    assert len(rows) == length
    H.assert_rows_match(rows, which, {"r": toks}, dtype, "portions")


def mixed_schedule(which):
    """Six requests, at most four live, portions beside decoded tokens; a pool that forces reuse."""
    lens = {"a": 50, "b": 37, "c": 64, "d": 21, "e": 45, "f": 30}
    reqs = {k: H.tokens_for(which, n, 20 + i) for i, (k, n) in enumerate(lens.items())}
    fed = {k: 0 for k in reqs}
    def take(k, n, want="all"):
        t = reqs[k][fed[k]:fed[k] + n]
        fed[k] += len(t)
        w = list(range(len(t))) if want == "all" else ([len(t) - 1] if want == "last" else [])
        return (k, t, w)
    S = []
    S.append(([take("a", 20), take("b", 30)], []))                                  # two prompt portions
    S.append(([take("a", 30, "last"), take("c", 9), take("b", 1)], []))            # a ends its prompt, c starts
    S.append(([take("c", 2), take("d", 21), take("b", 1)], ["a"]))                 # four live; a's pages return
    S.append(([take("c", 23, "none"), take("e", 13), take("b", 1)], ["d"]))        # e takes pages a held
    S.append(([take("c", 1), take("e", 1), take("f", 2), take("b", 4)], ["b"]))    # decoded tokens beside portions
    S.append(([take("c", 1), take("e", 7), take("f", 11)], []))
    S.append(([take("c", 28), take("e", 24), take("f", 17)], ["c", "e", "f"]))
    for k in lens:
        assert fed[k] == lens[k], (k, fed[k])
    return reqs, S


@pytest.mark.parametrize("which,dtype", CASES)
def test_mixed_with_page_reuse(which, dtype):
    reqs, schedule = mixed_schedule(which)
    # live tokens peak at 37 + 50 + 11 (a, b, c) etc.; give just enough pages that reuse is forced
    ps = H.TINY[which]["page_size"]
    live_peak, live = 0, {}
    for entries, end in schedule:
        for k, t, _ in entries:
            live[k] = live.get(k, 0) + len(t)
        live_peak = max(live_peak, sum(-(-n // ps) for n in live.values()))
        for k in end:
            live.pop(k)
    total_pages = sum(-(-len(t) // ps) for t in reqs.values())
    assert live_peak < total_pages
    runner = H.make_runner(which, dtype, num_pages=live_peak)
    rows = H.run_schedule(runner, schedule)
    H.assert_rows_match(rows, which, reqs, dtype, "mixed")
    assert runner.cache.free_pages() == [live_peak]


@pytest.mark.parametrize("page_size", [16, 64])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_portions_and_head_size_64(dtype, page_size, monkeypatch):
    """A configuration with 64-wide heads and prompts of several hundred tokens: in bfloat16 the
    portions of more than 64 tokens run on the tcgen05 attention kernel and, with pages of 64
    positions, decoding on the persistent TMA kernel (which the engine picks for steps that read many
    keys: the bound is lowered here so that this small model's steps take it).  Whole prompt; two long
    portions and 32 tokens one by one; and steps that hold a long portion of one request beside decoded
    tokens of two others."""
    from vllm_lite_b200.csrc import ops
    monkeypatch.setattr(ops, "STREAM_DECODE_MIN_KEYS", 0)
    which = "C"
    toks = H.tokens_for(which, 332, 41)
    pages = -(-400 // page_size) + 2
    runner = H.make_runner(which, dtype, num_pages=pages, page_size=page_size)
    rows = H.run_schedule(runner, [([("r", toks, [0, 63, 64, 127, 128, 200, 331])], ["r"])])
    H.assert_rows_match(rows, which, {"r": toks}, dtype, "whole, long")
    schedule = [([("r", toks[:130], [129])], []), ([("r", toks[130:300], [0, 100, 169])], [])]
    schedule += [([("r", [toks[p]], [0])], []) for p in range(300, 332)]
    rows = H.run_schedule(runner, schedule + [([("r", [5], [])], ["r"])])
    assert len(rows) == 36
    H.assert_rows_match(rows, which, {"r": toks + [5]}, dtype, "long portions, then decode")
    reqs = {"a": H.tokens_for(which, 90, 42), "b": H.tokens_for(which, 150, 43), "c": H.tokens_for(which, 260, 44)}
    need = sum(-(-len(t) // page_size) for t in reqs.values())
    runner = H.make_runner(which, dtype, num_pages=need, page_size=page_size)
    S = [([("a", reqs["a"][:80], [79]), ("b", reqs["b"][:140], [139])], []),
         ([("a", reqs["a"][80:81], [0]), ("b", reqs["b"][140:141], [0]), ("c", reqs["c"][:129], [0, 128])], []),
         ([("a", reqs["a"][81:82], [0]), ("c", reqs["c"][129:259], [129]), ("b", reqs["b"][141:142], [0])], []),
         ([("c", reqs["c"][259:], [0]), ("a", reqs["a"][82:], [7]), ("b", reqs["b"][142:], [7])], ["a", "b", "c"])]
    rows = H.run_schedule(runner, S)
    H.assert_rows_match(rows, which, reqs, dtype, "long portions beside decoded tokens")
    assert runner.cache.free_pages() == [need]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_python_and_native_host_paths_agree(dtype):
    """The batch laid out by the Python reference code and by the C++ core gives the same logits, bit for bit."""
    reqs, schedule = mixed_schedule("B")
    a = H.run_schedule(H.make_runner("B", dtype, num_pages=40, native_host=True), schedule)
    b = H.run_schedule(H.make_runner("B", dtype, num_pages=40, native_host=False), schedule)
    assert a.keys() == b.keys()
    for k in a:
        assert torch.equal(a[k], b[k]), k


@pytest.mark.parametrize("which", ["A", "B", "C"])
def test_cuts_agree_bitwise_in_float32(which):
    """The float32 kernels add in an order that depends on positions alone, so a
    position's logits are bit-for-bit the same however the tokens were cut."""
    toks = H.tokens_for(which, 60, 5)
    runner = H.make_runner(which, "float32", num_pages=pages_for(which, 192))
    whole = H.run_schedule(runner, [([("w", toks, list(range(60)))], ["w"])])
    other = H.tokens_for(which, 23, 6)
    cut = H.run_schedule(runner, [
        ([("o", other[:20], [])], []),
        ([("x", toks[:17], list(range(17))), ("o", other[20:21], [0])], []),
        ([("o", other[21:22], [0]), ("x", toks[17:19], [0, 1])], []),
        ([("x", toks[19:60], list(range(41)))], ["x", "o"])])
    for p in range(60):
        assert torch.equal(whole[("w", p)], cut[("x", p)]), f"position {p} differs between cuts"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(dtype):
    which = "B"
    length = 260
    toks = H.tokens_for(which, length, 31)
    runner = H.make_runner(which, dtype, num_pages=pages_for(which, 264))
    schedule = [([("r", toks[:4], [3])], [])] + [([("r", [toks[p]], [0])], []) for p in range(4, length)]
    rows = H.run_schedule(runner, schedule)
    H.assert_rows_match(rows, which, {"r": toks}, dtype, "long decode")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(dtype, tmp_path):
    """bin/trace_run as a user calls it: steps on stdin, <step>.f32 files out."""
    which = "A"
    toks = H.tokens_for(which, 40, 41)
    other = H.tokens_for(which, 12, 42)
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": toks[:25], "want": [0, 24]}], "end": []},
        {"step": 1, "entries": [{"id": "b", "tokens": other, "want": []}], "end": []},
        {"step": 2, "entries": [{"id": "a", "tokens": toks[25:27], "want": [0, 1]},
                                {"id": "b", "tokens": [3], "want": []}], "end": ["b"]},
        {"step": 3, "entries": [{"id": "a", "tokens": toks[27:], "want": [12]}], "end": ["a"]},
    ]
    env = dict(os.environ)
    proc = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(H.model_dir(which, dtype)),
                           "--dtype", dtype, "--out", str(tmp_path), "--max-tokens", "128"],
                          input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True,
                          env=env, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(4)]
    assert not (tmp_path / "1.f32").exists()
    V = H.TINY[which]["config"]["vocab_size"]
    ref = H.plain_logits(which, toks, dtype)
    got = {0: [0, 24], 2: [25, 26], 3: [39]}
    for step, positions in got.items():
        arr = np.fromfile(tmp_path / f"{step}.f32", dtype="<f4").reshape(-1, V)
        assert arr.shape[0] == len(positions)
        for row, pos in zip(arr, positions):
            err = float(np.abs(row - ref[pos].numpy()).max()) / float(ref[pos].abs().max())
            assert err <= H.TOL[dtype], (step, pos, err)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_real_layer_sizes_against_the_plain_implementation(dtype):
    """Two layers of Qwen3-8B width (hidden 4096, 32/8 heads of 128, intermediate 12288) with a small
    vocabulary, against the plain implementation on the CPU: a prompt of 2,100 tokens whole (in bfloat16 the
    paired tcgen05 products with and without the fused activation and the tcgen05 attention at head size
    128), the same prompt cut 1,300 + 800 (the library's products beside the fused tcgen05 one), then 30
    tokens one by one (the weight-streaming products with the norms folded in, through the graph).  The
    float32 engine holds weights with all their bits."""
    import plain_qwen3 as P
    from vllm_lite_b200.engine import ModelRunner, StepEntry, random_model
    cfg = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_size=4096, num_hidden_layers=2,
               num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=12288, vocab_size=2048,
               rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=4096)
    toks = [int(t) for t in np.random.default_rng(5).integers(0, 2048, size=2130)]
    store = torch.float32 if dtype == "float32" else torch.bfloat16
    # the tensors a folder written with this seed would hold (tests/test_weights.py checks that they are)
    _, plan, weights = random_model(cfg, seed=3, dtype=dtype, device="cuda:0", store_dtype=store)
    ref = P.forward(cfg, {k: v.float().cpu() for k, v in weights.items()}, toks)
    runner = ModelRunner(plan, weights, dtype=store, device="cuda:0", page_size=16, num_pages=290, max_requests=2)
    del weights
    whole_places = [0, 63, 64, 700, 1023, 1299, 1300, 2047, 2099]
    whole = runner.step([StepEntry("r", toks[:2100], whole_places)]).float().cpu()
    first = runner.step([StepEntry("s", toks[:1300], [0, 63, 64, 700, 1023, 1299])]).float().cpu()
    second = runner.step([StepEntry("s", toks[1300:2100], [0, 747, 799])]).float().cpu()
    runner.release("s")
    cut = torch.cat([first, second])
    if dtype == "float32":                              # the same prompt cut in two gives the same bits
        assert torch.equal(cut, whole)
    decoded = [runner.step([StepEntry("r", [toks[p]], [0])]).float().cpu() for p in range(2100, 2130)]
    runner.check_device_errors()
    assert runner.graph_replays >= 28
    got = torch.cat([whole, cut] + decoded)
    want = ref[whole_places + whole_places + list(range(2100, 2130))]
    err = (got - want).abs().amax(dim=1) / want.abs().amax(dim=1)
    key = ("real layer sizes", "8B x 2 layers", dtype)
    H.WORST[key] = max(H.WORST.get(key, 0.0), float(err.max()))
    assert float(err.max()) <= H.TOL[dtype], err
    del runner
    torch.cuda.empty_cache()


@pytest.mark.parametrize("live", [12, 33, 70])
@pytest.mark.parametrize("which,dtype", [(w, d) for w in ("B", "C") for d in ("float32", "bfloat16")])
def test_many_requests_decode_in_one_step(which, dtype, live):
    """Decode steps of more than 8 requests: the batch is padded to 16, 64 or 128 places and replayed
    from a graph, the bfloat16 products of 16 rows run in the weight-streaming kernel with its second row
    tile, those of 64 and 128 rows in the library, and the decode attention picks other chunk sizes.  The requests' prompts are of unequal length and arrive several to a step,
    on pages that earlier requests held; then every request decodes, all in one step, six times."""
    ps = H.TINY[which]["page_size"]
    lens = [3 + (7 * i) % 41 for i in range(live)]
    decoded = 6
    reqs = {i: H.tokens_for(which, lens[i] + decoded, 500 + i) for i in range(live)}
    need = sum(-(-(n + decoded) // ps) for n in lens)
    runner = H.make_runner(which, dtype, num_pages=need, max_requests=live)
    # earlier requests take every page once and give it back, so that the pages are used again
    fill, taken = [], 0
    while taken + 5 <= need:
        fill.append((f"x{len(fill)}", H.tokens_for(which, 5 * ps, 900 + len(fill)), []))
        taken += 5
    schedule = [(fill[k:k + 4], [f[0] for f in fill[k:k + 4]]) for k in range(0, len(fill), 4)]
    # prompts, seven to a step
    fed = {}
    for k in range(0, live, 7):
        entries = [(i, reqs[i][:lens[i]], [lens[i] - 1]) for i in range(k, min(k + 7, live))]
        schedule.append((entries, []))
    for i in range(live):
        fed[i] = lens[i]
    for _ in range(decoded):
        schedule.append(([(i, [reqs[i][fed[i]]], [0]) for i in range(live)], []))
        for i in range(live):
            fed[i] += 1
    schedule[-1] = (schedule[-1][0], list(range(live)))
    before = runner.graph_replays
    rows = H.run_schedule(runner, schedule)
    assert len(rows) == live * (decoded + 1)
    assert runner.graph_replays - before >= decoded - 1          # the decode steps ran from the graph of their bucket
    assert any(k[0] == (16 if live == 12 else 64 if live == 33 else 128) for k in runner._graphs)
    H.assert_rows_match(rows, which, reqs, dtype, f"{live} requests decoding")
    assert runner.cache.free_pages() == [need]


@pytest.mark.parametrize("ahead", [False, True])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decoding_across_the_context_bounds_of_the_graphs(dtype, ahead):
    """Decode graphs are recorded for a bound on the context (1,024, 2,048, ... up to the longest the
    runner takes).  A request decodes across 1,024 and across 2,048 beside a short one: the step picks
    the graph of the next bound when a request passes one, and a step launched ahead (its tokens still on
    the device) is refused while no graph for the new bound exists, and taken afterwards."""
    from vllm_lite_b200.engine import StepEntry
    which = "L"
    toks = H.tokens_for(which, 2075, 61)
    short = H.tokens_for(which, 70, 62)
    runner = H.make_runner(which, dtype, num_pages=-(-2075 // 16) + 6, max_requests=4, max_context=4096)
    rows, refused, taken = {}, 0, 0

    def keep(out, places):
        out = out.float().cpu()
        for r, (rid, pos) in enumerate(places):
            rows[(rid, pos)] = out[r].clone()

    def decode(lo, hi, s_at):
        """tokens lo..hi-1 of the long request one by one, the short request's beside them"""
        nonlocal refused, taken
        for k, p in enumerate(range(lo, hi)):
            ids, places = ["r", "s"], [("r", p), ("s", s_at + k)]
            feed = [toks[p], short[s_at + k]]
            out = None
            if ahead and k > 0:
                src = torch.tensor(feed, dtype=torch.int32, device="cuda:0")
                out = runner.step_ahead(ids, src, p + 1)
                refused += out is None
                taken += out is not None
            if out is None:
                out = runner.step([StepEntry(i, [t], [0]) for i, t in zip(ids, feed)])
            keep(out, places)
            runner.check_device_errors()
        return s_at + (hi - lo)

    keep(runner.step([StepEntry("r", toks[:1015], [1014]), StepEntry("s", short[:5], [4])]), [("r", 1014), ("s", 4)])
    s_at = decode(1015, 1040, 5)                       # passes 1,024
    keep(runner.step([StepEntry("r", toks[1040:2040], [999])]), [("r", 2039)])
    s_at = decode(2040, 2075, s_at)                    # passes 2,048
    bounds = sorted(k[1] for k in runner._graphs if k[0] == 2)
    assert bounds == [1024, 2048, 4096], bounds
    if ahead:
        assert refused == 2 and taken == 25 + 35 - 2 - 2      # refused once at each bound passed
    H.assert_rows_match(rows, which, {"r": toks, "s": short}, dtype, "across context bounds" + (", ahead" if ahead else ""))
    # a step launched ahead with too small a bound changes nothing
    before = runner.cached_tokens("r")
    assert runner.step_ahead(["r", "s"], torch.zeros(2, dtype=torch.int32, device="cuda:0"), before) is None
    assert runner.cached_tokens("r") == before
    runner.cache.check_invariants()


def test_decode_steps_fold_the_head_work_into_the_attention(monkeypatch):
    """bfloat16, few chunks per token: a decode step launches no kernel for the head norm, the rotation and the cache
    write (the decode attention does them on the way), a prompt portion does; the logits agree with the plain
    implementation either way, and with the fold switched off the same steps give the same bits."""
    from vllm_lite_b200.csrc import ops
    from vllm_lite_b200.parts import attention_dispatch
    which, dtype = "B", "bfloat16"
    toks = H.tokens_for(which, 60, 77)
    schedule = [([("r", toks[:40], [39])], [])] + [([("r", [toks[p]], [0])], []) for p in range(40, 60)]
    schedule[-1] = (schedule[-1][0], ["r"])
    calls = []
    real = ops.qk_norm_rope_write
    monkeypatch.setattr(ops, "qk_norm_rope_write", lambda qkv, *a, **k: (calls.append(qkv.shape[0]), real(qkv, *a, **k))[1])
    runner = H.make_runner(which, dtype, num_pages=12)
    rows = H.run_schedule(runner, schedule)
    layers = H.TINY[which]["config"]["num_hidden_layers"]
    assert calls == [40] * layers, calls                         # the prompt portion only (decode steps: none, eager or in a graph)
    H.assert_rows_match(rows, which, {"r": toks}, dtype, "head work folded into the decode attention")
    monkeypatch.setattr(attention_dispatch, "FOLD_MAX_CHUNKS", 0)
    del calls[:]
    plain_way = H.run_schedule(H.make_runner(which, dtype, num_pages=12), schedule)
    assert len(calls) > layers                                   # now every step that is not replayed from a graph calls it
    for key, row in rows.items():
        assert torch.equal(row, plain_way[key]), key
