#!/usr/bin/env python
"""Headline benchmark: greedy decode throughput of the 32B mixed-bit dense GQA decoder (BASELINE config 2/3).

    python bench.py --gpus N --steps K --warmup W            # N = 1: TP1; N > 1: launched by torchrun, TP N

Random-init weights of the named architecture are quantised on the device (2/3/4 bits per linear from a seeded
assignment, group 128), a synthetic 2048-token prompt is prefilled (untimed), then W warm-up and exactly K timed
decode steps run as CUDA-graph replays.  One step streams every weight of the model (>= 12 GB, far larger than the
126 MB L2), so no explicit L2 flush is needed between steps.  Timing: CUDA events on the launching stream, a barrier
and a device synchronise on both sides, max over ranks.  `e2e` repeats the measurement through the public step API
with the token fed from pinned host memory and read back to the host every step.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

METRIC = "decode_tok_s_32b_mixedbit"
BASELINE_TOK_S = 315.0   # reference README.md:290 (2 x cc 9.0 GPUs, tp2, MTP speculation, its own hybrid 32B model)


def reference_arm(args):
    """The reference's own kernel library (built unmodified by baseline/build_reference.py) on the same linear shapes;
    nothing of this package runs on that path."""
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "baseline"))
    try:
        import reference_arm as R
    except Exception as e:          # the driver expects one JSON line and exit code 0 whatever happens here
        print(json.dumps({"impl": "reference", "unavailable": f"baseline/reference_arm.py could not be imported: {e}"}))
        return 0
    try:
        return R.run(args)
    except Exception as e:
        print(json.dumps({"impl": "reference", "unavailable": f"reference arm failed: {type(e).__name__}: {e}"[:300]}))
        return 0


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs (read-only query)."""

    def __init__(self, index: int):
        self.index, self.rows, self.stop_evt, self.proc = index, [], threading.Event(), None

    def start(self):
        q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.th = threading.Thread(target=self._read, daemon=True)
        self.th.start()

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        sm = sorted(int(float(r[0])) for r in self.rows if r and r[0].replace(".", "").isdigit())
        mx = [int(float(r[1])) for r in self.rows if len(r) > 1 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) > 3 + i and r[3 + i].lower().startswith("active") for r in self.rows)]
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": reasons,
                "samples": len(sm)}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=0, help="debug only: fewer layers (the result is then not the named config)")
    ap.add_argument("--prompt", type=int, default=2048)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--prefill-chunk", type=int, default=2048)
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)

    import torch
    import torch.distributed as dist
    from agens_engine_b200.models import config as C

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = f"cuda:{local}"
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device(dev))
    warmup = max(args.warmup, 3)

    cfg = C.dense_32b(seed=0)
    if args.layers:
        cfg = C.scaled(cfg, args.layers)
    if world > 1:
        from agens_engine_b200.parallel.tp_model import TpDenseModel
        model = TpDenseModel.random_init(cfg, dev, seed=0, rank=rank, world=world, max_seqs=args.batch,
                                         max_ctx=args.prompt + warmup + 2 * args.steps + 64, prefill_chunk=args.prefill_chunk)
    else:
        from agens_engine_b200.models.dense import DenseModel
        model = DenseModel.random_init(cfg, dev, seed=0, max_seqs=args.batch,
                                       max_ctx=args.prompt + warmup + 2 * args.steps + 64, prefill_chunk=args.prefill_chunk)
    g = torch.Generator().manual_seed(1234)
    firsts = []
    pre0, pre1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    pre0.record()
    for s in range(args.batch):
        prompt = torch.randint(0, cfg.vocab, (args.prompt,), generator=g)
        model.new_seq(s)
        first, _ = model.prefill(s, prompt)
        firsts.append(first)
    pre1.record()
    torch.cuda.synchronize()
    prefill_ms = pre0.elapsed_time(pre1)        # untimed for the headline; reported as time to first token of the prompt
    seqs = list(range(args.batch))
    total_steps = warmup + 2 * args.steps
    model.decode_setup(seqs, firsts, total_steps)
    graph = model.decode_graph()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(warmup):
        graph.replay()
    # ---- device-timed region: exactly K steps ----
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        graph.replay()
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    clocks = sampler.stop() if rank == 0 else None

    # ---- end to end through the step API: pinned H2D of the token, D2H of the result, every step ----
    tok_in = torch.empty(args.batch, dtype=torch.int32).pin_memory()
    tok_out = torch.empty(args.batch, dtype=torch.int32).pin_memory()
    tok_in.copy_(model.last_ids[:args.batch].cpu())
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        model.step_host(tok_in, tok_out)
        tok_in.copy_(tok_out)
    barrier()
    e2e_s = time.perf_counter() - t0

    status = int(model.status.item()) | int(model.ws.status.item())
    if world > 1:
        t = torch.tensor([ms, e2e_s * 1e3, float(status)], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_ms, status = float(t[0]), float(t[1]), int(t[2])
    else:
        e2e_ms = e2e_s * 1e3
    if rank == 0:
        toks = args.steps * args.batch
        value = toks / (ms / 1e3)
        out = {
            "metric": METRIC, "value": round(value, 2), "unit": "tok/s", "n_gpus": world, "steps": args.steps,
            "warmup": warmup, "ms_per_step": round(ms / args.steps, 4), "higher_is_better": True, "scaling": "strong",
            "vs_baseline": round(value / BASELINE_TOK_S, 3), "dtype": "bf16", "data": "synthetic",
            "config": {"model": cfg.name + " (64 layers, d 5120, 64q/8kv x 128, ffn 25600, vocab 151936; weights 2/3/4-bit "
                                "seeded per linear, group 128, fp16 scale+zero; bf16 activations and paged KV)",
                       "global_batch": args.batch, "seq_len": args.prompt, "parallelism": f"tp{world}",
                       "decode": "greedy, CUDA graph per step",
                       "l2": "inputs larger than L2 (every step streams all weights, %.1f GB per GPU)" % (model.weight_bytes() / 1e9)},
            "e2e": {"value": round(toks / (e2e_ms / 1e3), 2), "unit": "tok/s", "h2d_bytes_per_step": 4 * args.batch,
                    "d2h_bytes_per_step": 4 * args.batch},
            "gpu_launches": model.launches_per_step(args.batch) * args.steps,
            "prefill": {"tokens": args.prompt * args.batch, "ms": round(prefill_ms, 1),
                        "tok_s": round(args.prompt * args.batch / (prefill_ms / 1e3), 1), "note": "first call includes one-time set-up"},
            "clocks": clocks, "device_status": status, "impl": "ours",
        }
        if args.layers:
            out["invalid"] = "debug run with fewer layers than the named config"
        print(json.dumps(out))
    if world > 1:
        torch.cuda.synchronize()
        model.close()
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
