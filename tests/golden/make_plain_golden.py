"""Writes tests/golden/plain_tiny.json: logits of the plain implementation on the tiny configurations.

    python tests/golden/make_plain_golden.py

The reference project cannot be compiled where these tests run (a Rust workspace, no toolchain),
so these numbers are NOT outputs of the reference: they pin the plain implementation and the seeded
random weights, so that an edit to either shows as a failing test instead of moving the oracle
silently.  Per configuration: the token ids, the first eight logits of the first and of the last
position, and the sum and the sum of squares of all logits, computed in float64 by
`plain_qwen3.forward`.
"""
import json
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))
sys.path.insert(0, str(HERE.parent.parent))


def summary(which: str, length: int = 12) -> dict:
    import torch
    import helpers as H
    import plain_qwen3 as P
    cfg, w = H.plain_model(which)
    toks = H.tokens_for(which, length, 7)
    logits = P.forward(cfg, w, toks, dtype=torch.float64)
    return {"tokens": toks, "first": logits[0, :8].tolist(), "last": logits[-1, :8].tolist(),
            "sum": float(logits.sum()), "sum_squares": float((logits * logits).sum())}


if __name__ == "__main__":
    out = {which: summary(which) for which in ("A", "B", "C")}
    (HERE / "plain_tiny.json").write_text(json.dumps(out, indent=1) + "\n")
    print(f"wrote {HERE / 'plain_tiny.json'}")
