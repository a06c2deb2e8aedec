"""The command line's decisions that need no GPU: flags and environment variables with the reference's
names, refusals, prompt files, and the random-weights folder."""
import json

import pytest

import helpers as H
import plain_qwen3 as P
from vllm_lite_b200 import cli


def test_flags_carry_the_reference_names_defaults_and_environment(monkeypatch):
    for name in ("VLLM_MODEL", "VLLM_KV_BLOCKS", "VLLM_MAX_BATCH_SIZE", "VLLM_MAX_MODEL_LEN"):
        monkeypatch.delenv(name, raising=False)
    args = cli.build_parser().parse_args(["-m", "/x"])
    # no --kv-blocks: the cache is sized from the GPU (the reference's default of 1,024 pages is not kept)
    assert (args.model, args.kv_blocks, args.max_batch_size, args.max_model_len) == ("/x", None, 256, None)
    assert args.gpu_memory_fraction == 0.9
    assert (args.tensor_parallel_size, args.kv_quantization, args.temperature, args.max_tokens) == (1, False, 0.0, 16)
    monkeypatch.setenv("VLLM_MODEL", "/from/env")
    monkeypatch.setenv("VLLM_KV_BLOCKS", "77")
    monkeypatch.setenv("VLLM_MAX_BATCH_SIZE", "5")
    args = cli.build_parser().parse_args([])
    assert (args.model, args.kv_blocks, args.max_batch_size) == ("/from/env", 77, 5)
    args = cli.build_parser().parse_args(["--model", "/flag", "--kv-blocks", "9"])     # a flag wins over the environment
    assert (args.model, args.kv_blocks) == ("/flag", 9)


@pytest.mark.parametrize("argv,needle", [
    (["--prompt-ids", "1,2"], "--model"),
    (["--model", "/no/such/folder", "--prompt-ids", "1"], "never downloaded"),
    (["--model", ".", "--tensor-parallel-size", "2", "--prompt-ids", "1"], "one GPU"),
    (["--model", ".", "--kv-quantization", "--prompt-ids", "1"], "not quantized"),
    (["--model", "."], "at least one prompt"),
    (["--model", ".", "--kv-blocks", "0", "--prompt-ids", "1"], "--kv-blocks"),
])
def test_refusals_come_before_anything_touches_a_gpu(argv, needle, monkeypatch, capsys):
    monkeypatch.delenv("VLLM_MODEL", raising=False)
    with pytest.raises(SystemExit) as e:
        cli.main(argv)
    assert e.value.code == 2
    assert needle in capsys.readouterr().err


def test_prompts_from_lists_and_files(tmp_path):
    f = tmp_path / "prompts.txt"
    f.write_text("1, 2,3\n\n7 8\n")
    assert cli.read_prompts(["4,5", str(f)]) == [[4, 5], [1, 2, 3], [7, 8]]


def test_init_writes_a_folder_that_the_seed_determines(tmp_path):
    cfg = tmp_path / "config.json"
    cfg.write_text(json.dumps(H.TINY_B))
    a, b, c = tmp_path / "a", tmp_path / "b", tmp_path / "c"
    assert cli.main(["init", "--config", str(cfg), "--out", str(a), "--seed", "3", "--std", "0.05"]) == 0
    assert cli.main(["init", "--config", str(cfg), "--out", str(b), "--seed", "3", "--std", "0.05"]) == 0
    assert cli.main(["init", "--config", str(cfg), "--out", str(c), "--seed", "4", "--std", "0.05"]) == 0
    assert (a / "model.safetensors").read_bytes() == (b / "model.safetensors").read_bytes()
    assert (a / "model.safetensors").read_bytes() != (c / "model.safetensors").read_bytes()
    cj, w = P.read_model_dir(a)                                   # the plain reader takes what was written
    assert cj["hidden_size"] == H.TINY_B["hidden_size"] and "lm_head.weight" in w
    assert P.forward(cj, w, [1, 2, 3]).shape == (3, H.TINY_B["vocab_size"])


def test_trace_run_without_a_gpu_says_so_and_exits(tmp_path):
    """No CPU path: the replay program refuses loudly where there is no CUDA device."""
    import subprocess
    import sys
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present: the replay tests cover the program")
    root = H.Path(__file__).resolve().parent.parent
    proc = subprocess.run([sys.executable, str(root / "bin" / "trace_run"), "--model", str(H.model_dir("A")),
                           "--dtype", "float32", "--out", str(tmp_path / "out"), "--max-tokens", "64"],
                          input="", capture_output=True, text=True, timeout=300)
    assert proc.returncode == 3 and "no CUDA device" in proc.stderr


def test_the_engine_has_no_cpu_path():
    from vllm_lite_b200.engine import ModelRunner, StepError
    with pytest.raises(StepError, match="CUDA device only"):
        ModelRunner(None, {}, device="cpu")
