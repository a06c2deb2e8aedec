"""Command line of the engine.

    python -m vllm_lite_b200 --model DIR --prompt-ids 1,2,3 --max-tokens 16
    python -m vllm_lite_b200 init --config config.json --out DIR --seed 0

Flags that the reference's server has keep its names, defaults and environment
variables (crates/server/src/cli/args.rs:144-186): `--model/-m` is required
(VLLM_MODEL) and is a local folder that is never downloaded, `--kv-blocks` (VLLM_KV_BLOCKS; the
reference's default is 1024, here the cache is sized from the GPU's free memory when the flag
is absent, under `--gpu-memory-fraction`), `--max-batch-size` (256, VLLM_MAX_BATCH_SIZE), `--max-model-len`
(VLLM_MAX_MODEL_LEN), `--tensor-parallel-size` (1) and `--kv-quantization`
(false), which are accepted only at those values because the engine runs on one
GPU with an unquantized cache, and `--log-level`.  The server's network and
speculative-decoding flags have no counterpart.  Prompts are token ids (the engine
has no tokenizer): a comma-separated list, or a file with one prompt per line.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
from pathlib import Path


def _env(name, default=None):
    v = os.environ.get(name)
    return default if v in (None, "") else v


def _bounded(lo, hi, what):
    def parse(s):
        v = int(s)
        if not lo <= v <= hi:
            raise argparse.ArgumentTypeError(f"{what} must lie in [{lo}, {hi}], got {v}")
        return v
    return parse


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="vllm-lite_b200", description="Qwen3 dense inference engine for one B200")
    sub = ap.add_subparsers(dest="command")
    init = sub.add_parser("init", help="write a model folder with random weights")
    init.add_argument("--config", required=True, help="config.json of the architecture")
    init.add_argument("--out", required=True, help="folder to write (config.json, model.safetensors)")
    init.add_argument("--seed", type=int, default=0)
    init.add_argument("--std", type=float, default=None, help="standard deviation of the matrices (default 0.02)")

    ap.add_argument("--model", "-m", default=_env("VLLM_MODEL"), help="model folder (config.json + safetensors)")
    ap.add_argument("--kv-blocks", type=_bounded(1, 1 << 24, "--kv-blocks"),
                    default=(int(_env("VLLM_KV_BLOCKS")) if _env("VLLM_KV_BLOCKS") else None),
                    help="pages of the cache; without it the cache is sized from the GPU's free memory")
    ap.add_argument("--gpu-memory-fraction", type=float, default=0.9,
                    help="share of the memory free after loading that cache and activations may take (no --kv-blocks)")
    ap.add_argument("--max-batch-size", type=_bounded(1, 4096, "--max-batch-size"),
                    default=int(_env("VLLM_MAX_BATCH_SIZE", 256)))
    ap.add_argument("--max-model-len", type=_bounded(1, 4_000_000, "--max-model-len"),
                    default=(int(_env("VLLM_MAX_MODEL_LEN")) if _env("VLLM_MAX_MODEL_LEN") else None))
    ap.add_argument("--tensor-parallel-size", "-t", type=int, default=int(_env("VLLM_TENSOR_PARALLEL_SIZE", 1)))
    ap.add_argument("--kv-quantization", action="store_true",
                    default=_env("VLLM_KV_QUANTIZATION", "false").lower() in ("1", "true"))
    ap.add_argument("--log-level", default=_env("VLLM_LOG_LEVEL", "info"))
    ap.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    ap.add_argument("--block-size", type=_bounded(1, 256, "--block-size"), default=64,
                    help="positions per page of the cache (the reference's constant is 16; 64 suits the TMA copies)")
    ap.add_argument("--max-num-batched-tokens", type=int, default=4096)
    ap.add_argument("--prefill-chunk-size", type=int, default=512)
    ap.add_argument("--prompt-ids", action="append", default=[],
                    help="comma-separated token ids, or a file with one such line per prompt; may repeat")
    ap.add_argument("--max-tokens", type=int, default=16)
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--top-k", type=int, default=0)
    ap.add_argument("--top-p", type=float, default=1.0)
    ap.add_argument("--repeat-penalty", type=float, default=1.0)
    ap.add_argument("--presence-penalty", type=float, default=0.0)
    ap.add_argument("--seed", type=int, default=None)
    return ap


def read_prompts(specs):
    prompts = []
    for spec in specs:
        lines = Path(spec).read_text().splitlines() if os.path.isfile(spec) else [spec]
        for line in lines:
            line = line.strip()
            if line:
                prompts.append([int(t) for t in line.replace(",", " ").split()])
    return prompts


def main(argv=None) -> int:
    ap = build_parser()
    args = ap.parse_args(argv)
    if args.command == "init":
        from .weights import write_model_dir
        cfg = json.loads(Path(args.config).read_text())
        d = write_model_dir(args.out, cfg, args.seed, std=args.std)
        print(f"wrote {d}")
        return 0
    if not args.model:
        ap.error("the following arguments are required: --model/-m (or VLLM_MODEL)")
    if not os.path.isdir(args.model):
        ap.error(f"--model {args.model!r} is not a folder; models are never downloaded")
    if args.tensor_parallel_size != 1:
        ap.error("--tensor-parallel-size: this engine runs on one GPU")
    if args.kv_quantization:
        ap.error("--kv-quantization: the cache is not quantized in this engine")
    prompts = read_prompts(args.prompt_ids)
    if not prompts:
        ap.error("give at least one prompt with --prompt-ids")
    from .engine import LLMEngine
    from .sampling import SamplingParams
    verbose = args.log_level.lower() in ("debug", "info", "trace")
    t0 = time.time()
    engine = LLMEngine(args.model, dtype=args.dtype, kv_blocks=args.kv_blocks, block_size=args.block_size,
                       max_batch_size=args.max_batch_size, max_num_batched_tokens=args.max_num_batched_tokens,
                       prefill_chunk_size=args.prefill_chunk_size, max_model_len=args.max_model_len,
                       gpu_memory_fraction=args.gpu_memory_fraction)
    if verbose:
        print(f"[vllm-lite_b200] model loaded in {time.time() - t0:.1f} s", file=sys.stderr)
    params = SamplingParams(temperature=args.temperature, top_k=args.top_k, top_p=args.top_p,
                            repeat_penalty=args.repeat_penalty, presence_penalty=args.presence_penalty,
                            seed=args.seed)
    t0 = time.time()
    outs = engine.generate(prompts, max_tokens=args.max_tokens, sampling_params=params)
    dt = time.time() - t0
    for o in outs:
        print(",".join(str(t) for t in o))
    if verbose:
        n = sum(len(o) for o in outs)
        print(f"[vllm-lite_b200] {n} tokens in {dt:.2f} s ({n / max(dt, 1e-9):.1f} tok/s); {engine.stats()}",
              file=sys.stderr)
    return 0


if __name__ == "__main__":
    sys.exit(main())
