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
    import threading
    rank0 = int(os.environ.get("RANK", "0")) == 0

    def give_up(why):
        # one JSON line from rank 0, exit code 0 on every rank, no teardown (a blocked collective must not hold the job)
        if rank0:
            print(json.dumps({"impl": "reference", "unavailable": why[:300]}))
        sys.stdout.flush()
        os._exit(0)

    limit = float(os.environ.get("B200E_REF_ARM_LIMIT_S", "900"))
    timer = threading.Timer(limit, give_up, args=(f"reference arm did not finish within {limit:.0f} s",))
    timer.daemon = True
    timer.start()
    try:
        rc = R.run(args)
        timer.cancel()
        return rc
    except Exception as e:
        timer.cancel()
        give_up(f"reference arm failed: {type(e).__name__}: {e}")


def _open(args, max_seqs, max_ctx, prefill_chunk):
    """Model of this rank (TP when launched by torchrun) with random-init weights of the named architecture."""
    import torch
    import torch.distributed as dist
    from agens_engine_b200.models import config as C
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = f"cuda:{local}"
    if world > 1 and not dist.is_initialized():
        dist.init_process_group("nccl", device_id=torch.device(dev))
    cfg = C.dense_32b(seed=0)
    if args.layers:
        cfg = C.scaled(cfg, args.layers)
    kw = dict(max_seqs=max_seqs, max_ctx=max_ctx, prefill_chunk=prefill_chunk)
    if world > 1:
        from agens_engine_b200.parallel.tp_model import TpDenseModel
        m = TpDenseModel.random_init(cfg, dev, seed=0, rank=rank, world=world, **kw)
    else:
        from agens_engine_b200.models.dense import DenseModel
        m = DenseModel.random_init(cfg, dev, seed=0, **kw)
    return m, cfg, rank, world, dev


def other_modes(args):
    """Secondary measurements named by the benchmark configs: time to first token at long context, and aggregate
    throughput of the serving loop (sampled requests; with the companion drafter in `spec` mode).  Device work is
    bracketed by synchronisation on both sides; multi-GPU numbers are the maximum over ranks."""
    import torch
    import torch.distributed as dist
    if args.mode == "ttft":
        chunk = max(args.prefill_chunk, 2048)
        m, cfg, rank, world, dev = _open(args, 1, args.ctx + 64, chunk)
        g = torch.Generator().manual_seed(99)
        # a short warm-up prompt first (lazy module loads, attribute calls), on its own sequence slot
        m.new_seq(0)
        m.prefill(0, torch.randint(0, cfg.vocab, (min(4096, args.ctx),), generator=g))
        m.free_seq(0)
        times = []
        for rep in range(max(1, args.steps if args.steps < 8 else 1)):
            prompt = torch.randint(0, cfg.vocab, (args.ctx,), generator=g)
            m.new_seq(0)
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            first, _ = m.prefill(0, prompt)
            e1.record()
            torch.cuda.synchronize()
            t = torch.tensor([e0.elapsed_time(e1)], device=dev)
            if world > 1:
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
            times.append(float(t[0]) / 1e3)
            m.free_seq(0)
        times.sort()
        if rank == 0:
            p50 = times[len(times) // 2]
            print(json.dumps({"metric": "ttft_p50_s", "value": round(p50, 3), "unit": "s", "higher_is_better": False, "n_gpus": world,
                              "ctx": args.ctx, "prefill_chunk": chunk, "prefill_tok_s": round(args.ctx / p50, 1), "repeats": len(times),
                              "dtype": "bf16", "data": "synthetic", "device_status": m.device_status(),
                              "config": {"model": cfg.name, "parallelism": f"tp{world}", "kv": "all resident (no host tier)"},
                              "timing": "CUDA events around prefill() of the whole prompt incl. the first token's lm_head; max over ranks"}))
        if world > 1:
            m.close(); dist.barrier(); dist.destroy_process_group()
        return 0
    # ---- serve / spec: the engine loop -------------------------------------------------------------------------------
    from agens_engine_b200.serve.engine import Engine
    C_, P, N = args.concurrency, args.prompt, args.new_tokens
    spec = args.mode == "spec"
    depth = args.draft_depth if spec else 0
    m, cfg, rank, world, dev = _open(args, C_, P + N + 64, max(args.prefill_chunk, 2048))
    ctrl = None
    model = m
    if world > 1:
        from agens_engine_b200.parallel import driver as D
        ctrl = D.control_group()
        if rank > 0:
            D.follow(m, ctrl)
            torch.cuda.synchronize(); m.close(); dist.barrier(); dist.destroy_process_group()
            return 0
        model = D.TpDriver(m, ctrl)
    sources = None
    if spec:
        from agens_engine_b200.models import config as MC
        from agens_engine_b200.models.dense import DenseModel
        from agens_engine_b200.spec import CopyLookupSource, ModelSource
        drafter = DenseModel.random_init(MC.drafter_0p6b(), dev, seed=1, max_seqs=C_, max_ctx=P + N + 64, prefill_chunk=2048,
                                         bf16_linears=os.environ.get("B200E_DRAFTER_BF16", "1") == "1")   # the reference's drafter is bf16
        drafter.row_graphs = True
        sources = lambda: [CopyLookupSource(), ModelSource(drafter, depth)]
    first_at, count, t0 = {}, {}, [0.0]

    def emit(rid, toks, finished, err):
        if toks and rid not in first_at:
            first_at[rid] = time.perf_counter() - t0[0]
        count[rid] = count.get(rid, 0) + len(toks)
        return False
    eng = Engine(model, emit, sources_factory=sources, max_drafts=depth, max_batch=C_)
    g = torch.Generator().manual_seed(7)
    prompts = [torch.randint(0, cfg.vocab, (P,), generator=g).tolist() for _ in range(C_)]

    def samp(i):
        s = {"max_new_tokens": N, "seed": 100 + i, "ignore_eos": True}
        if spec:
            if i % 2:
                s.update(temperature=0.8)
            else:
                s.update(temperature=0.0)
        else:
            s.update(temperature=0.7, top_p=0.9)
        return s
    eng.submit(prompts[0][:64], {"max_new_tokens": 4})
    eng.run_until_idle()
    first_at.clear(); count.clear()
    steps0 = eng.stats.steps
    torch.cuda.synchronize()
    t0[0] = time.perf_counter()
    rids = [eng.submit(p, samp(i)) for i, p in enumerate(prompts)]
    eng.run_until_idle()
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0[0]
    total = sum(count.get(r, 0) for r in rids)
    ttft = sorted(first_at.get(r, wall) for r in rids)
    decode_start = ttft[-1]
    out = {"metric": "serve_aggregate_tok_s" if not spec else "spec_aggregate_tok_s", "value": round(total / wall, 1), "unit": "tok/s",
           "higher_is_better": True, "n_gpus": world, "dtype": "bf16", "data": "synthetic",
           "decode_phase_tok_s": round((total - C_) / max(wall - decode_start, 1e-9), 1),
           "ttft_p50_s": round(ttft[len(ttft) // 2], 3), "wall_s": round(wall, 2), "output_tokens": total,
           "scheduler_steps": eng.stats.steps - steps0, "device_status": m.device_status(),
           "config": {"model": cfg.name, "parallelism": f"tp{world}", "concurrency": C_, "prompt": P, "new_tokens": N,
                      "sampling": "half greedy, half temperature 0.8, seeded" if spec else "temperature 0.7, top-p 0.9, seeded"},
           "timing": "wall clock around submit .. idle on the scheduling rank, device synchronised on both sides"}
    if spec:
        st = eng.spec.stats
        out["draft_depth"] = depth
        out["accepted_per_step"] = round(st.accepted / max(st.steps, 1), 3)
        out["spec_steps"] = st.steps
    print(json.dumps(out))
    if world > 1:
        model.shutdown()
        torch.cuda.synchronize(); m.close(); dist.barrier(); dist.destroy_process_group()
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
    ap.add_argument("--mode", default="decode", choices=["decode", "ttft", "serve", "spec"],
                    help="decode: the headline metric (default).  ttft: time to first token of one --ctx token prompt.  "
                         "serve: C concurrent sampled requests through the engine loop (benchmark config 3).  "
                         "spec: the same loop with the 0.6B drafter, half greedy / half sampled (benchmark config 5)")
    ap.add_argument("--ctx", type=int, default=131072, help="ttft mode: prompt length")
    ap.add_argument("--concurrency", type=int, default=16)
    ap.add_argument("--new-tokens", type=int, default=1024)
    ap.add_argument("--draft-depth", type=int, default=4)
    ap.add_argument("--step-kernel", type=int, default=-1, help="1 / 0: force the persistent step kernel on / off (default: B200E_STEP)")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    if args.step_kernel >= 0:
        os.environ["B200E_STEP"] = str(args.step_kernel)
    if args.mode != "decode":
        return other_modes(args)

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
