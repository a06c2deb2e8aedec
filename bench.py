"""Decode and prefill throughput of the engine at Qwen3-8B layer sizes on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--context 4096] [--layers 36]
    python bench.py --size 14b --context 8192 --continuous 32      (continuous batching, a line of its own)

Prints ONE JSON line.  `value` is decoded tokens per second of K decode steps at the
given batch, timed on the device with CUDA events (weights, 16 GB, are far larger than
L2, so every step reads them from HBM).  `e2e` is the same metric through the Python
entry point (`LLMEngine.step`): host token ids in through pinned memory, sampled ids
back to the host, every step.  `prefill` is one 2,048-token prompt, `points` are decode
at batch 1 and 64 and `prefill_default`, the same prompt through `LLMEngine` with the scheduler's default
limits (tokens per second to the first token, wall clock); `roofline` relates the decode step to the bytes
it must read.
Weights are random (seeded), prompts are seeded uniform token ids.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

QWEN3_8B = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_size=4096, num_hidden_layers=36,
                num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=12288,
                vocab_size=151936, rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False,
                max_position_embeddings=40960)
# the other dense sizes of the architecture (layers, hidden, heads, intermediate); kv heads 8, head_dim 128
SIZES = {"8b": (36, 4096, 32, 12288), "14b": (40, 5120, 40, 17408), "32b": (64, 5120, 64, 25600)}
METRIC = "decode tok/s at batch 8 (Qwen3-8B, bf16)"
PREFILL_TOKENS = 2048


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.is_file():
        d = json.loads(p.read_text())
        return dict(hbm_gbs=d["hbm_gbs"], bf16_tflops=d["bf16_tflops"],
                    bf16_tflops_sustained=d.get("bf16_tflops_sustained", d["bf16_tflops"]), source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.samples, self.proc, self.thread = [], None, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return self
        def pump():
            for line in self.proc.stdout:
                self.samples.append((time.time(), line.strip()))
        self.thread = threading.Thread(target=pump, daemon=True)
        self.thread.start()
        return self

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self, t0, t1):
        rows = [l.split(", ") for t, l in self.samples if t0 <= t <= t1] or [l.split(", ") for _, l in self.samples]
        rows = [r for r in rows if len(r) == 6 and r[0].isdigit()]
        if not rows:
            return None
        mhz = sorted(int(r[0]) for r in rows)
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[2 + i].strip().lower() == "active" for r in rows)]
        return {"sm_mhz": mhz[len(mhz) // 2], "sm_max_mhz": int(rows[0][1]), "reasons": reasons, "samples": len(rows)}


def model_bytes_and_flops(cfg, layers):
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nq, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    per_layer = (nq + 2 * nkv) * hd * H + H * nq * hd + 3 * H * I          # matrix elements of one layer
    norms = layers * (2 * H + 2 * hd) + H
    weight_bytes = 2 * (layers * per_layer + V * H) + 4 * norms            # bf16 matrices, every one read once
    kv_bytes_per_token = layers * 2 * nkv * hd * 2
    T = PREFILL_TOKENS
    prefill_flops = 2 * T * layers * per_layer + layers * 4 * nq * hd * (T * (T + 1) // 2) + 2 * V * H
    return weight_bytes, kv_bytes_per_token, prefill_flops


def reference_arm():
    print(json.dumps({"impl": "reference", "unavailable":
                      "pplmx/vllm-lite is a Rust workspace (no setup.py or pyproject.toml; pip reports 'not "
                      "installable') and no cargo/rustc toolchain or crate registry exists offline"}))
    return 0


def decode_run(runner, sampler, batch, context, warmup, steps, fill, vocab, tag):
    """W + K decode steps of `batch` requests that end at `context` tokens each.
    Returns (ms per step, kernel launches per step, mean context over the timed steps)."""
    import torch
    from vllm_lite_b200.csrc import ops
    from vllm_lite_b200.engine import StepEntry
    from vllm_lite_b200.sampling import SamplingParams
    start_len = context - (warmup + steps)
    ids = [f"{tag}{i}" for i in range(batch)]
    gen = torch.Generator().manual_seed(1234)
    for rid in ids:
        if fill == "prefill":                           # the cache holds what a real prompt leaves
            prompt = torch.randint(0, vocab, (start_len,), generator=gen).tolist()
            for lo in range(0, start_len, PREFILL_TOKENS):
                runner.step([StepEntry(rid, prompt[lo:lo + PREFILL_TOKENS], [])])
        else:                                           # pages are taken; their contents are random numbers
            runner.cache.admit(rid)
            runner.cache.append(rid, start_len)
    greedy = [SamplingParams()] * batch
    def one(step):
        entries = [StepEntry(rid, [(7 * i + 13 * step) % vocab], [0]) for i, rid in enumerate(ids)]
        logits = runner.step(entries)
        sampler.sample(logits, greedy, [()] * batch)
    for s in range(warmup):
        one(s)
    torch.cuda.synchronize()
    n0 = ops.launch_count
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for s in range(steps):
        one(warmup + s)
    t1.record()
    torch.cuda.synchronize()
    ms = t0.elapsed_time(t1) / steps
    launches = (ops.launch_count - n0) / steps
    runner.check_device_errors()
    for rid in ids:
        runner.release(rid)
    return ms, launches, start_len + warmup + (steps - 1) / 2 + 1


def prefill_run(runner, vocab, repeats=3):
    import torch
    from vllm_lite_b200.engine import StepEntry
    gen = torch.Generator().manual_seed(99)
    times = []
    for r in range(repeats + 1):
        prompt = torch.randint(0, vocab, (PREFILL_TOKENS,), generator=gen).tolist()
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        runner.step([StepEntry("prefill", prompt, [PREFILL_TOKENS - 1])])
        t1.record()
        torch.cuda.synchronize()
        runner.release("prefill")
        if r:                                            # the first run warms up
            times.append(t0.elapsed_time(t1))
    times.sort()
    return times[len(times) // 2]


def prefill_default_run(engine, vocab, repeats=3):
    """What a user gets for one 2,048-token prompt: through LLMEngine with the scheduler's default limits
    (4,096 tokens a step, portions of 512 beside decoding requests), host ids in, the first token out.
    Returns tokens per second (median of `repeats` after one warm-up run)."""
    import torch
    cfg = engine.scheduler.config
    saved = (cfg.max_num_batched_tokens, cfg.prefill_chunk_size)
    cfg.max_num_batched_tokens, cfg.prefill_chunk_size = 4096, 512
    gen = torch.Generator().manual_seed(77)
    times = []
    try:
        for r in range(repeats + 1):
            prompt = torch.randint(0, vocab, (PREFILL_TOKENS,), generator=gen).tolist()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            engine.add_request(prompt, max_tokens=1)
            out = []
            while engine.has_unfinished():
                out += engine.step()
            dt = time.perf_counter() - t0
            assert len(out) == 1 and out[0].finished
            if r:
                times.append(dt)
    finally:
        cfg.max_num_batched_tokens, cfg.prefill_chunk_size = saved
    times.sort()
    return PREFILL_TOKENS / times[len(times) // 2]


def e2e_run(engine, batch, context, warmup, steps, vocab):
    """The same decode steps through LLMEngine.step: host ids in, sampled ids out, every step."""
    import torch
    gen = torch.Generator().manual_seed(4321)
    # A request decodes while the prompts of the later ones are computed (a prompt takes `fill` steps): the
    # earlier a request comes, the shorter its prompt, so that all of them end the timed steps just below
    # `context` (and none crosses the context bound its decode graph was recorded for in mid-measurement).
    fill = -(-context // PREFILL_TOKENS) + 1
    for i in range(batch):
        prompt_len = max(16, context - (warmup + steps) - (batch - 1 - i) * fill - 4)
        engine.add_request(torch.randint(0, vocab, (prompt_len,), generator=gen).tolist(),
                           max_tokens=engine.scheduler.config.max_model_len - prompt_len)
        while any(s.remaining > 1 for s in engine.scheduler.running) or engine.scheduler.waiting:
            engine.step()
    for _ in range(warmup):
        engine.step()
    torch.cuda.synchronize()
    h2d0, t0 = engine.runner.uploaded_bytes, time.perf_counter()
    produced = 0
    for _ in range(steps):
        produced += len(engine.step())
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    h2d = (engine.runner.uploaded_bytes - h2d0) / steps
    for seq in list(engine.scheduler.running):
        engine.cancel_request(seq.seq_id)
    assert produced == batch * steps, (produced, batch, steps)
    if os.environ.get("VLLM_LITE_B200_BENCH_STEP_TIMES"):
        print("step times of the end-to-end run:", json.dumps(engine.stats()["step_times"]["decode"]), file=sys.stderr)
    return produced / dt, h2d, 4 * batch


def continuous_run(engine, requests, vocab, prompt_range, out_len):
    """Continuous batching through LLMEngine: all requests arrive at once with prompts of seeded
    uniform length, each generates `out_len` tokens.  Wall clock around the whole run, host token
    ids in and out.  Returns the figures of the JSON line."""
    import random
    import torch
    rng = random.Random(0)
    gen = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, vocab, (rng.randint(*prompt_range),), generator=gen).tolist() for _ in range(requests)]
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for p in prompts:
        engine.add_request(p, out_len)
    kinds = {"prompt": [0, 0.0], "mixed": [0, 0.0], "decode": [0, 0.0]}
    produced = 0
    before = dict(engine.scheduler.stats)
    while engine.has_unfinished():
        s0 = time.perf_counter()
        produced += len(engine.step())
        now = dict(engine.scheduler.stats)
        pre, dec = now["prefill_tokens"] - before["prefill_tokens"], now["decode_tokens"] - before["decode_tokens"]
        kind = "mixed" if pre and dec else "prompt" if pre else "decode"
        kinds[kind][0] += 1
        kinds[kind][1] += time.perf_counter() - s0
        before = now
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    engine.runner.check_device_errors()
    prompt_tokens = sum(len(p) for p in prompts)
    return {"value": round(produced / dt, 1), "unit": "generated tokens/s", "requests": requests,
            "prompt_tokens": prompt_tokens, "generated_tokens": produced, "seconds": round(dt, 3),
            "all_tokens_per_s": round((prompt_tokens + produced) / dt, 1),
            "steps": {k: v[0] for k, v in kinds.items()},
            "ms_per_step": {k: round(v[1] / v[0] * 1e3, 3) if v[0] else None for k, v in kinds.items()},
            "preemptions": engine.scheduler.stats["preemptions"],
            # host time of LLMEngine.step() and device time of every 16th step, by kind (median, 90th percentile)
            "step_times": engine.stats()["step_times"]}


def check_fp32(cfg, layers, tokens=1024):
    """The whole model in true float32 at full depth: a prompt run whole, the same prompt cut into
    portions of changing size beside another request's tokens, and its last tokens one by one must give
    the same bits at every compared position (the float32 kernels add in an order that depends on
    positions alone).  Prints one JSON line; exit code 0 only when every row is equal."""
    import torch
    from vllm_lite_b200.engine import ModelRunner, StepEntry, random_model
    vocab = cfg["vocab_size"]
    _, plan, weights = random_model(cfg, seed=0, dtype="float32", device="cuda:0", store_dtype=torch.float32)
    runner = ModelRunner(plan, weights, dtype=torch.float32, device="cuda:0", page_size=16,
                         num_pages=3 * (tokens // 16 + 2), max_requests=4, own_weights=True)
    del weights
    gen = torch.Generator().manual_seed(7)
    toks = torch.randint(0, vocab, (tokens,), generator=gen).tolist()
    other = torch.randint(0, vocab, (64,), generator=gen).tolist()
    places = sorted({0, 1, 15, 16, 17, tokens // 3, tokens // 2} | set(range(tokens - 9, tokens)))
    t0 = time.time()
    whole = runner.step([StepEntry("w", toks, places)]).clone()
    runner.release("w")
    rows, fed, k, o = {}, 0, 0, 0
    sizes = [299, 2, 17, 128, 1, 64, 3]
    while fed < tokens - 8:
        n = min(sizes[k % len(sizes)], tokens - 8 - fed)
        k += 1
        want = [p - fed for p in places if fed <= p < fed + n]
        entries = [StepEntry("c", toks[fed:fed + n], want)]
        if o < len(other):                              # another request's tokens share the step
            m = 1 if k % 2 else 5
            entries.insert(k % 2, StepEntry("o", other[o:o + m], []))
            o += m
        out = runner.step(entries)
        for r, w in enumerate(want):
            rows[fed + w] = out[r].clone()
        fed += n
    for p in range(tokens - 8, tokens):                 # the last tokens one by one (the decode path)
        rows[p] = runner.step([StepEntry("c", [toks[p]], [0])])[0].clone()
    runner.check_device_errors()
    torch.cuda.synchronize()
    unequal = [p for i, p in enumerate(places) if not torch.equal(rows[p], whole[i])]
    worst = max(float((rows[p] - whole[i]).abs().max()) for i, p in enumerate(places))
    print(json.dumps({"check": "float32, whole prompt against portions of changing size and single tokens",
                      "model": f"{layers} layers, hidden {cfg['hidden_size']}, vocabulary {vocab}", "tokens": tokens,
                      "rows_compared": len(places), "rows_equal_bit_for_bit": len(places) - len(unequal),
                      "max_abs_difference": worst, "seconds": round(time.time() - t0, 1)}))
    return 0 if not unequal else 1


def read_ceiling(cfg, batch, context):
    """What ONE launch that must read a given number of bytes can reach, at the sizes of a decode step's
    kernels: a kernel that only reads (csrc/memprobe.cu) beside the engine's own kernel for each of them.
    Every launch reads memory that L2 does not hold (8 copies of the operands in turn), launches follow one
    another inside a CUDA graph with programmatic dependent launch on, as in a decode step.  One JSON line."""
    import torch
    from vllm_lite_b200.csrc import ops
    dev = "cuda:0"
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nq, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    M, L = batch, 8
    ops.set_pdl(True)
    err = torch.zeros(1, dtype=torch.int32, device=dev)

    def in_graph(fn):                                   # microseconds per launch, L launches a replay
        fn(); torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            fn()
        for _ in range(3):
            g.replay()
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(10):
            g.replay()
        t1.record(); torch.cuda.synchronize()
        return t0.elapsed_time(t1) / 10 / L * 1e3

    def weights(n, k):
        return [torch.randn(n, k, device=dev, dtype=torch.bfloat16) for _ in range(L)]

    nw = torch.ones(H, device=dev)
    x = torch.randn(M, H, device=dev)
    part = torch.zeros(ops.NORM_PARTIALS, 16, device=dev)
    rows = torch.empty(M, H, device=dev, dtype=torch.bfloat16)
    out = {}

    def product(name, n, k, **kw):
        ws = weights(n, k)
        a = torch.randn(M, k, device=dev, dtype=torch.bfloat16)
        width = n // 2 if kw.get("swiglu") else n
        c = torch.empty(M, width, device=dev, dtype=kw.pop("out_dtype", torch.bfloat16))
        sink = kw.pop("sink", False)
        gu = torch.empty(M, n, device=dev, dtype=torch.bfloat16) if M > ops.SMALL_M else None
        def ours():
            for w in ws:
                if M > ops.SMALL_M:                   # more rows than the weight-streaming product takes: the library
                    if kw.get("swiglu"):
                        torch.mm(a, w.t(), out=gu)
                    else:
                        torch.mm(a, w.t(), out=c)
                elif sink:
                    ops.gemm_bf16_small_m(a, w, rows, err, sink=(x, nw, part))
                else:
                    ops.gemm_bf16_small_m(a, w, c, err, **kw)
        nbytes = n * k * 2
        def plain():
            for w in ws:
                ops.read_only(w, nbytes)
        out[name] = {"MB": round(nbytes / 1e6, 1), "engine_us": round(in_graph(ours), 1), "read_only_us": round(in_graph(plain), 1)}
        del ws

    product("qkv", (nq + 2 * nkv) * hd, H, scaled=(part, 1, 1e-6, H))
    product("o", H, nq * hd, sink=True)
    product("gate_up", 2 * I, H, swiglu=True, scaled=(part, 1, 1e-6, H))
    product("down", H, I, sink=True)
    if M <= ops.SMALL_M:
        product("head", V, H, out_dtype=torch.float32)
    # decode attention: `batch` requests of `context` keys, pages of 16 in a row
    page, nblk = 16, context // 16 + 1
    caches = [(torch.randn(batch * nblk, nkv, page, hd, device=dev, dtype=torch.bfloat16),
               torch.randn(batch * nblk, nkv, page, hd, device=dev, dtype=torch.bfloat16)) for _ in range(L)]
    table = torch.arange(batch * nblk, device=dev, dtype=torch.int32).view(batch, nblk)
    qkv = torch.randn(batch, (nq + 2 * nkv) * hd, device=dev, dtype=torch.bfloat16)
    o = torch.empty(batch, nq * hd, device=dev, dtype=torch.bfloat16)
    req = torch.arange(batch, dtype=torch.int32, device=dev)
    pos = torch.full((batch,), context - 1, dtype=torch.int32, device=dev)
    chunk = ops.decode_chunk_for(batch, nkv, context, head_dim=hd)
    S, na, nm = ops.decode_attention_scratch(batch, nq, hd, context, chunk)
    pa, pm = torch.empty(na, device=dev), torch.empty(nm, device=dev)
    arr = torch.zeros(ops.flash_decode_arrivals(batch, nq, nkv), dtype=torch.int32, device=dev)
    def attention():
        for kc, vc in caches:
            ops.flash_decode(qkv, o, kc, vc, table, req, pos, nq, nkv, hd, hd ** -0.5, 0, context, pa, pm, err,
                             chunk=chunk, arrivals=arr)
    kv_bytes = batch * context * nkv * hd * 2 * 2
    def attention_plain():
        for kc, vc in caches:
            ops.read_only(kc, kv_bytes // 2 // 16 * 16)
            ops.read_only(vc, kv_bytes // 2 // 16 * 16)
    out["attention"] = {"MB": round(kv_bytes / 1e6, 1), "engine_us": round(in_graph(attention), 1),
                        "read_only_us": round(in_graph(attention_plain), 1), "read_only_launches": 2}
    assert int(err.item()) == 0
    pk = peaks()
    for v in out.values():
        v["at_copy_peak_us"] = round(v["MB"] * 1e6 / (pk["hbm_gbs"] * 1e9) * 1e6, 1)
    print(json.dumps({"read_ceiling": out, "batch": batch, "context": context, "copy_peak_gbs": pk["hbm_gbs"],
                      "how": "microseconds a launch, 8 launches over memory L2 does not hold, in a CUDA graph, dependent launches on"}))
    return 0


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--size", default="8b", choices=sorted(SIZES), help="layer sizes of Qwen3-8B (default), 14B or 32B")
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the size has (both numbers are reported)")
    ap.add_argument("--block-size", type=int, default=64, help="positions per page of the cache")
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 / 64 points and the prefill")
    ap.add_argument("--only-prefill", action="store_true", help="time the 2,048-token prefill alone (for profiling)")
    ap.add_argument("--no-e2e", action="store_true", help="skip the run through the Python entry point (for profiling)")
    ap.add_argument("--kv-fill", default="prefill", choices=["prefill", "random"],
                    help="what the cache holds before decoding: what real prompts leave, or random numbers (for profiling)")
    ap.add_argument("--continuous", type=int, default=0, metavar="REQUESTS",
                    help="instead of the decode steps: continuous batching of this many requests through LLMEngine, prompts "
                         "uniform in [256, context/2], 512 generated tokens each (steps and warmup are not used)")
    ap.add_argument("--kv-blocks", default=None, metavar="N|auto",
                    help="pages of the cache: a count, or 'auto' = sized from the memory left after the weights (the "
                         "default for --size 32b); default otherwise: what the largest batch needs at --context")
    ap.add_argument("--read-ceiling", action="store_true",
                    help="instead of timing steps: every kernel of a decode step alone beside a kernel that only reads as many bytes")
    ap.add_argument("--check-fp32", action="store_true",
                    help="instead of timing: the model in true float32, whole prompt against cut prompt, bit for bit")
    args = ap.parse_args(argv)
    if args.impl == "reference":
        return reference_arm()
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not built")
        return 2
    warmup = max(args.warmup, 3)

    import torch
    from vllm_lite_b200.csrc import ops
    from vllm_lite_b200.engine import LLMEngine, random_model
    full_layers, hidden, heads, inter = SIZES[args.size]
    if args.layers is None:
        args.layers = full_layers
    cfg = dict(QWEN3_8B, num_hidden_layers=args.layers, hidden_size=hidden, num_attention_heads=heads,
               intermediate_size=inter)
    vocab = cfg["vocab_size"]
    if args.check_fp32:
        return check_fp32(cfg, args.layers)
    if args.read_ceiling:
        return read_ceiling(cfg, args.batch, args.context)
    _, plan, weights = random_model(cfg, seed=0, dtype="bfloat16", device="cuda:0")
    if args.continuous:
        R, out_len, prompt_range = args.continuous, 512, (256, args.context // 2)
        pages = R * (-(-(prompt_range[1] + out_len) // args.block_size) + 1) + 64
        engine = LLMEngine(plan=plan, weights=weights, dtype="bfloat16", kv_blocks=pages, block_size=args.block_size, max_batch_size=R,
                           max_num_batched_tokens=4096, prefill_chunk_size=512, max_model_len=args.context)
        del weights
        continuous_run(engine, min(R, 4), vocab, (256, 512), 16)          # warm-up: builds, graphs of the small buckets
        clocks = ClockSampler().start()
        w0 = time.time()
        out = continuous_run(engine, R, vocab, prompt_range, out_len)
        clocks.stop()
        out = {"metric": f"continuous batching, generated tok/s (Qwen3-{args.size.upper()}, bf16)", **out, "n_gpus": 1,
               "dtype": "bf16", "data": "synthetic (random weights N(0,0.02), uniform token ids)",
               "config": {"model": f"Qwen3-{args.size.upper()} layer sizes", "layers": args.layers, "layers_full": full_layers,
                          "context": args.context, "prompt_lengths": f"uniform in [{prompt_range[0]}, {prompt_range[1]}]",
                          "generated_each": out_len, "block_size": args.block_size, "max_num_batched_tokens": 4096,
                          "prefill_chunk_size": 512, "timing": "wall clock around the whole run, host ids in and out"},
               "clocks": clocks.summary(w0, time.time())}
        print(json.dumps(out))
        return 0
    big = args.batch if args.no_points else max(args.batch, 64)
    # In the end-to-end run the requests' prompts are computed one after the other while the earlier requests
    # already decode: every request needs room for the tokens it generates meanwhile.
    slack = 64 + args.batch * (args.context // PREFILL_TOKENS + 2)
    pages = big * (-(-(args.context + slack) // args.block_size) + 1) + PREFILL_TOKENS // args.block_size + 64
    if args.kv_blocks == "auto" or (args.kv_blocks is None and args.size == "32b"):
        pages = None                                      # the engine sizes the cache from what the weights leave
    elif args.kv_blocks is not None:
        pages = int(args.kv_blocks)
    engine = LLMEngine(plan=plan, weights=weights, dtype="bfloat16", kv_blocks=pages, block_size=args.block_size, max_batch_size=big,
                       max_num_batched_tokens=PREFILL_TOKENS, prefill_chunk_size=PREFILL_TOKENS,
                       max_model_len=args.context + slack)
    del weights
    runner, sampler = engine.runner, engine.sampler
    for t in runner.storage.paged:                        # pages that no prompt wrote hold random numbers
        t.normal_()
    weight_bytes, kv_per_token, prefill_flops = model_bytes_and_flops(cfg, args.layers)
    pk = peaks()

    if args.only_prefill:
        pms = prefill_run(runner, vocab, repeats=max(1, min(args.steps, 5)))
        print(json.dumps({"prefill": {"value": round(PREFILL_TOKENS / pms * 1000.0, 1), "tokens": PREFILL_TOKENS,
                                      "ms": round(pms, 3), "layers": args.layers,
                                      "frac": round(prefill_flops / (pms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)}}))
        return 0
    clocks = ClockSampler().start()
    w0 = time.time()
    ms, launches, mean_ctx = decode_run(runner, sampler, args.batch, args.context, warmup, args.steps, args.kv_fill, vocab, "d")
    w1 = time.time()
    e2e_tps, h2d, d2h = (0.0, 0, 0) if args.no_e2e else e2e_run(engine, args.batch, args.context, warmup, args.steps, vocab)
    clocks.stop()
    value = args.batch * 1000.0 / ms
    step_bytes = weight_bytes + args.batch * mean_ctx * kv_per_token
    achieved = step_bytes / (ms * 1e-3) / 1e9
    out = {
        "metric": METRIC.replace("8B", args.size.upper()).replace("batch 8", f"batch {args.batch}"), "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": warmup, "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic (random weights N(0,0.02), uniform token ids)",
        "config": {"model": f"Qwen3-{args.size.upper()} layer sizes", "layers": args.layers, "layers_full": full_layers,
                   "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
                   "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"], "vocab": vocab,
                   "global_batch": args.batch, "seq_len": args.context, "block_size": args.block_size, "parallelism": "single GPU",
                   "kv_fill": "real prefill" if args.kv_fill == "prefill" else "random numbers", "l2": f"inputs (weights {weight_bytes / 1e9:.0f} GB) larger than L2, no flush",
                   "peaks": pk["source"], "kv_pages": sum(p.size for p in runner.cache.pools)},
        "clocks": clocks.summary(w0, w1),
        "e2e": None if args.no_e2e else {"value": round(e2e_tps, 1), "unit": "tokens/s", "h2d_bytes_per_step": int(h2d),
                                         "d2h_bytes_per_step": d2h},
        "gpu_launches": int(round(launches * args.steps)),
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
    }
    if not args.no_points:
        pms = prefill_run(runner, vocab)
        # frac: of the burst peak of the library product (one launch timed alone); the step itself is a
        # long run of products under the power cap, for which the sustained figure is the fair one
        out["prefill"] = {"value": round(PREFILL_TOKENS / pms * 1000.0, 1), "tokens": PREFILL_TOKENS, "ms": round(pms, 3),
                          "frac": round(prefill_flops / (pms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4),
                          "frac_of_sustained": round(prefill_flops / (pms * 1e-3) / (pk["bf16_tflops_sustained"] * 1e12), 4)}
        ms1, _, _ = decode_run(runner, sampler, 1, args.context, warmup, args.steps, "prefill", vocab, "s")
        ms64, _, _ = decode_run(runner, sampler, 64, args.context, warmup, args.steps, args.kv_fill, vocab, "l")
        out["points"] = {"decode_b1": round(1000.0 / ms1, 1), "decode_b64": round(64 * 1000.0 / ms64, 1),
                         "prefill_default": round(prefill_default_run(engine, vocab), 1)}
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
