"""Serving benchmark through the engine loop: C concurrent requests with random prompts, seeded sampling, continuous
batching on one GPU (or this rank's shard under torchrun).  Reports aggregate output tokens/s, p50 time to first token
and ms per scheduler step -- the shape of the reference's server-mode numbers (README.md:292, 16 / 32 / 48 concurrent
requests at temperature and top-p sampling).

    python -m agens_engine_b200.bench_engine --concurrency 16 --prompt 1024 --new-tokens 128
"""
from __future__ import annotations

import argparse
import json
import time

import torch


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="dense-32b")
    ap.add_argument("--concurrency", type=int, default=16)
    ap.add_argument("--prompt", type=int, default=1024)
    ap.add_argument("--new-tokens", type=int, default=128)
    ap.add_argument("--temperature", type=float, default=0.7)
    ap.add_argument("--top-p", type=float, default=0.9)
    ap.add_argument("--prefill-chunk", type=int, default=2048)
    ap.add_argument("--row-graphs", type=int, default=1)
    args = ap.parse_args(argv)

    from .cli import _named_config
    from .models.dense import DenseModel
    from .serve.engine import Engine

    cfg = _named_config(args.model)
    C = args.concurrency
    m = DenseModel.random_init(cfg, "cuda:0", seed=0, max_seqs=C, max_ctx=args.prompt + args.new_tokens + 32,
                               prefill_chunk=args.prefill_chunk)
    m.row_graphs = bool(args.row_graphs)
    first_at, done_at, count = {}, {}, {}
    t0 = [0.0]

    def emit(rid, toks, finished, err):
        now = time.perf_counter()
        if toks and rid not in first_at:
            first_at[rid] = now - t0[0]
        count[rid] = count.get(rid, 0) + len(toks)
        if finished:
            done_at[rid] = now - t0[0]
        return False

    eng = Engine(m, emit, max_batch=min(C, 32))
    g = torch.Generator().manual_seed(7)
    prompts = [torch.randint(0, cfg.vocab, (args.prompt,), generator=g).tolist() for _ in range(C)]
    samp = lambda i: {"max_new_tokens": args.new_tokens, "temperature": args.temperature, "top_p": args.top_p, "seed": 100 + i,
                      "ignore_eos": True}
    # warm-up: one short request end to end (lazy allocations, graph captures of the common shapes)
    eng.submit(prompts[0][:64], {"max_new_tokens": 4})
    eng.run_until_idle()
    first_at.clear(); done_at.clear(); count.clear()
    steps0 = eng.stats.steps
    torch.cuda.synchronize()
    t0[0] = time.perf_counter()
    rids = [eng.submit(p, samp(i)) for i, p in enumerate(prompts)]
    eng.run_until_idle()
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0[0]
    total = sum(count[r] for r in rids)
    ttft = sorted(first_at[r] for r in rids)
    decode_start = max(first_at[r] for r in rids)               # all prompts prefilled: pure batched decode afterwards
    tail_tokens = total - C
    status = int(m.status.item()) | int(m.ws.status.item())
    print(json.dumps({
        "metric": "engine_aggregate_tok_s", "model": cfg.name, "concurrency": C, "prompt": args.prompt, "new_tokens": args.new_tokens,
        "sampling": {"temperature": args.temperature, "top_p": args.top_p, "seeded": True},
        "wall_s": round(wall, 3), "output_tokens": total, "aggregate_tok_s": round(total / wall, 1),
        "decode_phase_tok_s": round(tail_tokens / max(wall - decode_start, 1e-9), 1),
        "ttft_p50_s": round(ttft[len(ttft) // 2], 3), "ttft_max_s": round(ttft[-1], 3),
        "scheduler_steps": eng.stats.steps - steps0, "peak_batch": eng.stats.peak_batch, "row_graphs": bool(args.row_graphs),
        "device_status": status, "timing": "wall clock around submit .. idle, device synchronised on both sides"}))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
