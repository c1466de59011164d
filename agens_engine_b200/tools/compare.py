"""Quality gates on saved outputs: KL / top-1 agreement of two logits files, equality of two token lists.

Reference: ``tools/compare_logits.py`` and ``tools/compare_tokens.py`` (used by its ``m1-kv --cmp-logits`` and
token-equality gates).  Logits files are ``torch.save``d tensors ``[rows, vocab]`` (or ``[vocab]``); token files are
JSON lists or JSON objects with a ``tokens`` key.
"""
from __future__ import annotations

import json
import sys

import torch


def compare_logits(a_path: str, b_path: str) -> dict:
    return logits_report(torch.load(a_path), torch.load(b_path))


def logits_report(a: torch.Tensor, b: torch.Tensor) -> dict:
    """Mean / max KL(a || b) of the softmax rows, top-1 agreement and the largest absolute difference."""
    a, b = a.detach().double().cpu(), b.detach().double().cpu()
    a, b = a.reshape(-1, a.shape[-1]), b.reshape(-1, b.shape[-1])
    if a.shape != b.shape:
        raise ValueError(f"shapes differ: {tuple(a.shape)} vs {tuple(b.shape)}")
    p, q = torch.log_softmax(a, -1), torch.log_softmax(b, -1)
    kl = (p.exp() * (p - q)).sum(-1)
    return {"rows": a.shape[0], "mean_kl": float(kl.mean()), "max_kl": float(kl.max()),
            "top1_agreement": float((a.argmax(-1) == b.argmax(-1)).double().mean()), "max_abs_diff": float((a - b).abs().max())}


def _tokens(path: str):
    d = json.load(open(path))
    return d["tokens"] if isinstance(d, dict) else d


def compare_tokens(a_path: str, b_path: str) -> dict:
    a, b = _tokens(a_path), _tokens(b_path)
    n = min(len(a), len(b))
    first = next((i for i in range(n) if a[i] != b[i]), None)
    return {"equal": a == b, "len_a": len(a), "len_b": len(b), "first_difference": first,
            "agreement": sum(int(x == y) for x, y in zip(a, b)) / max(n, 1)}


def main(argv=None) -> int:
    argv = sys.argv[1:] if argv is None else argv
    if len(argv) != 3 or argv[0] not in ("logits", "tokens"):
        print("usage: python -m agens_engine_b200.tools.compare logits|tokens A B")
        return 2
    rep = compare_logits(argv[1], argv[2]) if argv[0] == "logits" else compare_tokens(argv[1], argv[2])
    print(json.dumps(rep))
    return 0 if (rep.get("equal", True) and rep.get("top1_agreement", 1.0) >= 0.98) else 1


if __name__ == "__main__":
    sys.exit(main())
