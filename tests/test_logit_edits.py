"""Penalties and logit bias of the serving loop (`Engine._edit_logits`): the incremental device-side counts give the
same rows as the direct restatement of the rule, step after step (reference: crates/agens-server/src/sampling.rs)."""
import torch

from agens_engine_b200.serve.engine import Engine, Request


def _direct(row, prompt, out, s):
    row = row.clone()
    rep = float(s.get("repetition_penalty", 1))
    if rep != 1:
        for t in set(prompt) | set(out):
            row[t] = row[t] / rep if row[t] > 0 else row[t] * rep
    pres, freq = float(s.get("presence_penalty", 0)), float(s.get("frequency_penalty", 0))
    for t in set(out):
        row[t] -= pres + freq * float(out.count(t))
    for k, v in (s.get("logit_bias") or {}).items():
        row[int(k)] += float(v)
    return row


def test_incremental_penalties_match_the_direct_rule():
    g = torch.Generator().manual_seed(0)
    V = 300
    samplings = [{"repetition_penalty": 1.3}, {"presence_penalty": 0.7, "frequency_penalty": 0.25},
                 {"repetition_penalty": 0.8, "presence_penalty": -0.5, "logit_bias": {"7": 3.0, "299": -2.0}}, {"temperature": 0.7}]
    reqs = [Request(rid=i, prompt=torch.randint(0, V, (20,), generator=g).tolist(), sampling=s) for i, s in enumerate(samplings)]
    for step in range(6):
        logits = torch.randn(len(reqs), V, generator=g)
        want = torch.stack([_direct(logits[i], r.prompt, r.out, r.sampling) if r.needs_logit_edits() else logits[i] for i, r in enumerate(reqs)])
        Engine._edit_logits(None, logits, reqs)
        assert torch.allclose(logits, want, rtol=0, atol=1e-6), step
        for r in reqs:                                  # one to three new tokens per step, with repeats
            r.out += torch.randint(0, 12, (1 + step % 3,), generator=g).tolist()
    assert reqs[3].pen_state is None and reqs[0].pen_state["n"] == len(reqs[0].out) - (1 + 5 % 3)
