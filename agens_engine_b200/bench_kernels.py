"""Device-timed micro-benchmarks of the hot kernels with achieved-vs-roofline fractions.

Counterpart of the reference's ``kernels/bench/bench_gemv.cu`` / ``bench_w4h.cu`` / ``bench_read.cu``.  Every number
is taken with CUDA events on the launching stream after warm-up; the L2 is flushed between timed launches by writing
a buffer larger than L2 (256 MiB).  Roofline denominators come from ``MEASURED_PEAKS.json`` when present.

    python -m agens_engine_b200.bench_kernels gemv [--m 1] [--small]
    python -m agens_engine_b200.bench_kernels attn
    python -m agens_engine_b200.bench_kernels gemm
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

from . import _lib
from .ops import linear as L


def peaks() -> dict:
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "src": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "src": "fallback"}


class L2Flusher:
    def __init__(self, dev):
        self.buf = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def __call__(self):
        self.buf.fill_(1)


def time_cuda(fn, iters=20, warmup=5, flush=None):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        if flush:
            flush()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1) * 1e3)
    ts.sort()
    return ts[len(ts) // 2], ts[0]


def graph_time_us(launch_all, n_launch: int, iters: int = 10, warmup: int = 3):
    """Capture ``launch_all`` (which issues ``n_launch`` kernels on the current stream) into one CUDA graph and
    return the median device time per launch.  Launch gaps disappear, as in a captured decode step; the caller makes
    the launches touch more bytes than L2 holds so that every launch streams from HBM."""
    st = torch.cuda.Stream()
    with torch.cuda.stream(st):
        launch_all()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=st):
            launch_all()
        for _ in range(warmup):
            g.replay()
        torch.cuda.synchronize()
        ts = []
        for _ in range(iters):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            g.replay()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1) * 1e3 / n_launch)
    ts.sort()
    return ts[len(ts) // 2], ts[0]


def bench_gemv(args):
    dev = "cuda:0"
    pk = peaks()
    ws = L.GemvWorkspace(dev, floats=16 << 20)
    ws.mm_min_rows = 33                      # times the GEMV family itself; above 8 rows its activation staging only fits small k slices
    shapes = [("qkv", 10240, 5120), ("o", 5120, 8192), ("gate_up", 51200, 5120), ("down", 5120, 25600),
              ("lm_head", 151936, 5120)]
    if args.small:
        shapes = [("gate_up", 51200, 5120)]
    rows = []
    for name, n, k in shapes:
        for bits in ([4] if name == "lm_head" else [2, 3, 4]):
            for _ in (0,):
                ks_list = sorted({1, L.choose_ks(n, k), L.choose_ks(n, k, 1280), L.choose_ks(n, k, 5120)})
                for ks in ks_list:
                    lin = L.WqLinear.random(n, k, bits, 128, dev, seed=1, ks=ks)
                    nbytes = lin.nbytes()
                    ncopy = max(2, min(24, (512 << 20) // nbytes + 1))   # rotate over > 512 MiB of weights: L2 stays cold
                    lins = [lin] + [L.WqLinear(n, k, bits, 128, lin.wq.clone(), ks, lin.rb)
                                    for _ in range(ncopy - 1)]
                    x = torch.randn(args.m, k, device=dev).to(torch.bfloat16)
                    out = torch.empty(args.m, n, dtype=torch.bfloat16, device=dev)

                    def launch_all():
                        for ln in lins:
                            L.gemv(ln, x, ws, out=out)

                    med, best = graph_time_us(launch_all, len(lins))
                    gbs = nbytes / med / 1e3
                    rows.append(dict(name=name, n=n, k=k, bits=bits, ks=ks, m=args.m, us=round(med, 2),
                                     best_us=round(best, 2), gbs=round(gbs, 1), frac=round(gbs / pk["hbm_gbs"], 3),
                                     copies=ncopy))
                    print(json.dumps(rows[-1]), flush=True)
                    del lins
    print(json.dumps({"peaks": pk, "timing": "CUDA graph of back-to-back launches over rotating weight copies "
                      "(> 512 MiB, larger than L2); median per launch"}))


def profile_gemv(args):
    """A handful of plain launches of one configuration, for a profiler capture of a small case."""
    dev = "cuda:0"
    ws = L.GemvWorkspace(dev, floats=16 << 20)
    n, k = 51200, 5120
    lins = [L.WqLinear.random(n, k, args.bits, 128, dev, seed=i, ks=args.ks or L.choose_ks(n, k)) for i in range(3)]
    x = torch.randn(args.m, k, device=dev).to(torch.bfloat16)
    out = torch.empty(args.m, n, dtype=torch.bfloat16, device=dev)
    for _ in range(2):
        for ln in lins:
            L.gemv(ln, x, ws, out=out)
    torch.cuda.synchronize()
    print("profile_gemv done")


def bench_gemm(args):
    """tcgen05 GEMM vs the library GEMM (torch.matmul -> cuBLAS) on the prefill shapes of the 32B model."""
    from .ops import gemm as G
    dev = "cuda:0"
    pk = peaks()
    flush = L2Flusher(dev)
    shapes = [("qkv", 10240, 5120), ("o", 5120, 8192), ("gate_up", 51200, 5120), ("down", 5120, 25600)]
    for M in ([2048] if args.small else [512, 2048, 8192]):
        for name, n, k in shapes:
            a = torch.randn(M, k, device=dev).to(torch.bfloat16)
            b = (torch.randn(n, k, device=dev) * 0.02).to(torch.bfloat16)
            out = torch.empty(M, n, dtype=torch.bfloat16, device=dev)
            ours, _ = time_cuda(lambda: G.gemm_bf16(a, b, out=out), iters=10, warmup=3, flush=flush)
            lib, _ = time_cuda(lambda: torch.matmul(a, b.t(), out=out), iters=10, warmup=3, flush=flush)
            fl = 2.0 * M * n * k
            print(json.dumps(dict(name=name, M=M, n=n, k=k, ours_us=round(ours, 1), cublas_us=round(lib, 1),
                                  ours_tflops=round(fl / ours / 1e6, 1), cublas_tflops=round(fl / lib / 1e6, 1),
                                  frac_of_measured_peak=round(fl / ours / 1e6 / pk["bf16_tflops"], 3))), flush=True)
    print(json.dumps({"peaks": pk, "timing": "CUDA events, median of 10, L2 flushed between launches"}))


def bench_bf16(args):
    """bf16 GEMV (linears kept in bf16) on the shapes of the 0.6B drafter and of the 32B model, ``--m`` rows: launches
    back to back in a CUDA graph over rotating weight copies larger than L2, device time per launch and the fraction of
    the measured copy bandwidth the weight stream reaches."""
    dev = "cuda:0"
    pk = peaks()
    ws = L.GemvWorkspace(dev, floats=1 << 16)
    shapes = [("drafter qkv", 4096, 1024), ("drafter gate_up", 6144, 1024), ("drafter down", 1024, 3072), ("32b qkv", 10240, 5120),
              ("32b o", 5120, 8192), ("32b gate_up", 51200, 5120), ("32b down", 5120, 25600)]
    for name, n, k in shapes[:4] if args.small else shapes:
        w = (torch.randn(n, k, device=dev) * 0.02).to(torch.bfloat16)
        ncopy = max(4, min(64, (512 << 20) // (n * k * 2) + 1))
        lins = [L.Bf16Linear(n, k, w.clone()) for _ in range(ncopy)]
        x = torch.randn(args.m, k, device=dev).to(torch.bfloat16)
        out = torch.empty(args.m, n, dtype=torch.bfloat16, device=dev)

        def launch_all():
            for ln in lins:
                L.gemv(ln, x, ws, out=out)
        us, best = graph_time_us(launch_all, ncopy)
        gbs = n * k * 2 / us / 1e3
        print(json.dumps(dict(name=name, n=n, k=k, m=args.m, us=round(us, 2), best_us=round(best, 2), weight_gbs=round(gbs, 1),
                              frac_of_measured_copy=round(gbs / pk["hbm_gbs"], 3))), flush=True)
    print(json.dumps({"peaks": pk, "timing": "CUDA graph of back-to-back launches over rotating weight copies (> L2), median of 10"}))


def trace_gemv(args):
    """Phase stamps of the GEMV on the 32B shapes (m rows), captured inside a CUDA graph of back-to-back launches over
    rotating weight copies: where the time of one launch goes (start skew, prefetch issue, dependency wait, activation
    staging, first weights, k loop of the first item, hand-off + epilogue)."""
    import numpy as np
    dev = "cuda:0"
    ws = L.GemvWorkspace(dev, floats=16 << 20)
    tr = torch.zeros(600 * 8 * 8, dtype=torch.int64, device=dev)
    L.TRACE_BUFFER = tr
    shapes = [(10240, 5120), (5120, 8192), (51200, 5120), (5120, 25600)]
    for n, k in shapes[:1] if args.small else shapes:
        lin = L.WqLinear.random(n, k, args.bits, 128, dev, seed=1)
        ncopy = max(4, min(16, (512 << 20) // lin.nbytes() + 1))
        lins = [L.WqLinear(n, k, args.bits, 128, lin.wq.clone(), lin.ks, lin.rb) for _ in range(ncopy)]
        x = torch.randn(args.m, k, device=dev).to(torch.bfloat16)
        out = torch.empty(args.m, n, dtype=torch.bfloat16, device=dev)

        def launch_all():
            for ln in lins:
                L.gemv(ln, x, ws, out=out)

        med, _ = graph_time_us(launch_all, len(lins))
        t = tr.cpu().numpy().reshape(-1, 8)
        t = t[t[:, 0] > 0]
        base = t[:, 0].min()
        q = lambda a: [round(float(np.percentile(a, p)) / 1e3, 2) for p in (0, 50, 100)]
        print(json.dumps(dict(n=n, k=k, bits=args.bits, m=args.m, ks=lin.ks, rb=lin.rb, us_per_launch=round(med, 2), warps=len(t),
                              start_skew=q(t[:, 0] - base), prefetch_issue=q(t[:, 1] - t[:, 0]), dependency_wait=q(t[:, 2] - t[:, 1]),
                              activation_staging=q(t[:, 3] - t[:, 2]), first_weights=q(t[:, 4] - t[:, 3]),
                              k_loop_first_item=q(t[:, 5] - t[:, 3]), handoff_epilogue=q(t[:, 6] - t[:, 5]),
                              end=q(t[:, 6] - base), unit="us [min, median, max] over warps of the last launch")), flush=True)
    L.TRACE_BUFFER = None


def bench_mm(args):
    """Mixed-bit tcgen05 GEMM (in-kernel dequantisation) on the 32B shapes for m rows, CUDA-graph timing over rotating
    weight copies larger than L2."""
    dev = "cuda:0"
    pk = peaks()
    ws = L.GemvWorkspace(dev, floats=16 << 20)
    lib = _lib.cuda_lib()
    shapes = [("qkv", 10240, 5120), ("o", 5120, 8192), ("gate_up", 51200, 5120), ("down", 5120, 25600), ("lm_head", 151936, 5120)]
    for name, n, k in shapes[2:3] if args.small else shapes:
        for bits in ([4] if name == "lm_head" else [2, 3, 4]):
            lin = L.WqLinear.random(n, k, bits, 128, dev, seed=1)
            nb = lin.nbytes()
            ncopy = max(3, min(12, (512 << 20) // nb + 1))
            lins = [lin] + [L.WqLinear(n, k, bits, 128, lin.wq.clone(), lin.ks, lin.rb) for _ in range(ncopy - 1)]
            x = torch.randn(args.m, k, device=dev).to(torch.bfloat16)
            out = torch.empty(args.m, n, dtype=torch.bfloat16, device=dev)

            def launch_all():
                for ln in lins:
                    L.mm(ln, x, ws, out=out)

            med, best = graph_time_us(launch_all, len(lins))
            print(json.dumps(dict(name=name, n=n, k=k, bits=bits, m=args.m, ks=lib.b2_wq_mm_ks(n, k), us=round(med, 1),
                                  gbs=round(nb / med / 1e3, 0), frac_hbm=round(nb / med / 1e3 / pk["hbm_gbs"], 3),
                                  tflops=round(2.0 * args.m * n * k / med / 1e6, 1))), flush=True)
    print(json.dumps({"peaks": pk, "timing": "CUDA graph of back-to-back launches (activation prologue + GEMM) over rotating weight "
                      "copies (> 512 MiB); median per launch"}))


def profile_mm(args):
    """Three plain launches of the gate/up shape for a profiler capture of a small case."""
    dev = "cuda:0"
    ws = L.GemvWorkspace(dev, floats=16 << 20)
    n, k = 51200, 5120
    lins = [L.WqLinear.random(n, k, args.bits, 128, dev, seed=i) for i in range(3)]
    x = torch.randn(args.m, k, device=dev).to(torch.bfloat16)
    out = torch.empty(args.m, n, dtype=torch.bfloat16, device=dev)
    for ln in lins:
        L.mm(ln, x, ws, out=out)
    torch.cuda.synchronize()
    print("profile_mm done", int(ws.status.item()))


def _attn_case(ctx: int, rows: int, dev, hq=64, hkv=8, hd=128):
    from .ops import attention as A
    n_pages = (ctx + rows + 15) // 16 + 1
    pool = torch.randn(n_pages, 2, hkv, 16, hd, device=dev).to(torch.bfloat16)
    bt = torch.arange(n_pages, dtype=torch.int32, device=dev)[None, :]
    q = torch.randn(rows, hq * hd, device=dev).to(torch.bfloat16)
    g0, gc, pos, seqv = A.prefill_groups(rows, ctx, 0, dev)
    return A, pool, bt, q, g0, gc, pos, seqv


def bench_attn(args):
    """Paged attention of the 32B shape (64 q / 8 kv heads x 128): one decode row, an 8-row verify block and a 256-row
    prefill chunk (per-warp and CTA-shared K/V ring) at several context lengths; CUDA events, L2 flushed."""
    dev = "cuda:0"
    pk = peaks()
    flush = L2Flusher(dev)
    for ctx in ([2560] if args.small else [2560, 8192, 32768]):
        for rows, split, shared in ((1, 64, False), (8, 64, False), (256, 256, False), (256, 256, True)):
            A, pool, bt, q, g0, gc, pos, seqv = _attn_case(ctx, rows, dev)
            splits = (ctx + rows + split - 1) // split
            po = torch.empty(rows, 64, splits, 128, dtype=torch.float32, device=dev)
            pm = torch.empty(rows, 64, splits, 2, dtype=torch.float32, device=dev)
            out = torch.empty(rows, 64 * 128, dtype=torch.bfloat16, device=dev)
            fn = lambda: A.attn_decode(q, pool, bt, g0, gc, pos, seqv, 64, 8, 128, split, splits, part_o=po, part_ml=pm, out=out,
                                       shared_kv=shared)
            med, _ = time_cuda(fn, iters=10, warmup=3, flush=flush)
            kv_bytes = 2 * 8 * 128 * 2 * (ctx + rows)
            print(json.dumps(dict(ctx=ctx, rows=rows, split_keys=split, shared_kv=shared, us=round(med, 1),
                                  kv_gbs=round(kv_bytes / med / 1e3, 1), frac_hbm_single_read=round(kv_bytes / med / 1e3 / pk["hbm_gbs"], 3),
                                  tflops=round(4.0 * rows * 64 * 128 * (ctx + rows / 2) / med / 1e6, 1))), flush=True)
    # prefill chunks on the tcgen05 kernel against the split-KV kernel (CTA-shared ring), same inputs
    for ctx, rows in ([(2560, 2048)] if args.small else [(0, 2048), (8192, 2048), (32768, 2048), (131072 - 2048, 2048), (8192, 256)]):
        A, pool, bt, q, g0, gc, pos, seqv = _attn_case(ctx, rows, dev)
        out = torch.empty(rows, 64 * 128, dtype=torch.bfloat16, device=dev)
        st = torch.zeros(1, dtype=torch.int32, device=dev)
        fl = 4.0 * rows * 64 * 128 * (ctx + rows / 2)
        med, _ = time_cuda(lambda: A.attn_prefill_tc(q, pool, bt, 0, ctx, 64, 8, status=st, out=out), iters=5, warmup=3, flush=flush)
        rec = dict(kernel="attn_prefill_tc", ctx=ctx, rows=rows, us=round(med, 1), tflops=round(fl / med / 1e6, 1),
                   frac_bf16_peak=round(fl / med / 1e6 / pk["bf16_tflops"], 3), status=int(st.item()))
        if ctx <= 32768:
            med2, _ = time_cuda(lambda: A.attn_prefill(q, pool, bt, 0, ctx, 64, 8, 128, split_keys=256 if ctx < 16384 else 1024,
                                                       tensor_core=False), iters=3, warmup=1, flush=flush)
            rec.update(split_kv_us=round(med2, 1), split_kv_tflops=round(fl / med2 / 1e6, 1))
        print(json.dumps(rec), flush=True)
    print(json.dumps({"peaks": pk, "timing": "CUDA events, median of 10, L2 flushed; split kernel + merge kernel"}))


def profile_attn(args):
    """A few plain launches for a profiler capture: by default a 256-row prefill chunk at an 8K context (CTA-shared
    ring); ``--rows 1 --ctx 32768`` is one decode row over 134 MB of K/V (64-key splits, per-warp ring)."""
    dev = "cuda:0"
    rows, ctx = args.rows, args.ctx
    split = 256 if rows >= 8 else 64
    A, pool, bt, q, g0, gc, pos, seqv = _attn_case(ctx, rows, dev)
    for _ in range(3):
        A.attn_decode(q, pool, bt, g0, gc, pos, seqv, 64, 8, 128, split, (ctx + rows + split - 1) // split, shared_kv=rows >= 8)
    torch.cuda.synchronize()
    print("profile_attn done")


def profile_attn_tc(args):
    """A few plain launches of the tcgen05 prefill attention for a profiler capture: a ``--rows``-token chunk (default
    256 -> use 2048) of the 32B head layout at a ``--ctx``-token context (K/V of 8K tokens: 268 MB per layer pool)."""
    dev = "cuda:0"
    rows, ctx = args.rows, args.ctx
    A, pool, bt, q, g0, gc, pos, seqv = _attn_case(ctx, rows, dev)
    out = torch.empty(rows, 64 * 128, dtype=torch.bfloat16, device=dev)
    st = torch.zeros(1, dtype=torch.int32, device=dev)
    for _ in range(3):
        A.attn_prefill_tc(q, pool, bt, 0, ctx, 64, 8, status=st, out=out)
    torch.cuda.synchronize()
    print("profile_attn_tc done, status", int(st.item()))


def profile_misc(args):
    """Plain launches of the small kernels of a step on 32B shapes, for a profiler capture: RoPE + paged KV store of a
    2048-row chunk, RMSNorm of 2048 x 5120, the sampler on 32 rows of a 151936-entry vocabulary, and two blocks of the
    vision tower (full width) on a 448 x 448 image."""
    from .models.vision import VisionConfig, VisionTower
    from .ops import basic as B
    from .serve import vision as V
    import numpy as np
    dev = "cuda:0"
    hq, hkv, hd, n = 64, 8, 128, 2048
    qkv = torch.randn(n, (hq + 2 * hkv) * hd, device=dev).to(torch.bfloat16)
    inv_freq = (1.0 / (1e6 ** (torch.arange(0, hd, 2, dtype=torch.float32) / hd))).to(dev)
    pos = torch.arange(n, dtype=torch.int32, device=dev)
    seq = torch.zeros(n, dtype=torch.int32, device=dev)
    n_pages = n // 16 + 1
    bt = torch.arange(n_pages, dtype=torch.int32, device=dev)[None, :].contiguous()
    pool = torch.zeros(n_pages, 2, hkv, 16, hd, dtype=torch.bfloat16, device=dev)
    q_out = torch.empty(n, hq * hd, dtype=torch.bfloat16, device=dev)
    x = torch.randn(n, 5120, device=dev).to(torch.bfloat16)
    w = torch.ones(5120, dtype=torch.bfloat16, device=dev)
    logits = torch.randn(32, 151936, device=dev)
    temp = torch.full((32,), 0.7, device=dev); top_p = torch.full((32,), 0.9, device=dev)
    top_k = torch.full((32,), 50, dtype=torch.int32, device=dev)
    seed = torch.arange(32, dtype=torch.int64, device=dev); position = torch.arange(32, dtype=torch.int32, device=dev)
    tower = VisionTower.random_init(VisionConfig(depth=2, out_dim=5120), dev, seed=0)
    img = np.random.default_rng(0).integers(0, 256, size=(448, 448, 3), dtype=np.uint8)
    patches, grid = V.preprocess(img)
    for _ in range(2):
        B.rope_kvstore(qkv, hq, hkv, hd, inv_freq, pos, seq, bt, pool, q_out)
        B.rmsnorm(x, w, 1e-6)
        B.sample_rows(logits, temp, top_k, top_p, None, seed, position)
        tower.encode(torch.from_numpy(patches), grid)
    torch.cuda.synchronize()
    print("profile_misc done")


def profile_gemm(args):
    """Three plain launches of the bf16 tcgen05 GEMM (gate/up shape, 2048 rows) for a profiler capture."""
    from .ops import gemm as G
    dev = "cuda:0"
    a = torch.randn(2048, 5120, device=dev).to(torch.bfloat16)
    b = (torch.randn(51200, 5120, device=dev) * 0.02).to(torch.bfloat16)
    out = torch.empty(2048, 51200, dtype=torch.bfloat16, device=dev)
    for _ in range(3):
        G.gemm_bf16(a, b, out=out)
    torch.cuda.synchronize()
    print("profile_gemm done")


def profile_step(args):
    """Small case for an ncu capture of the persistent decode-step kernel: a 4-layer cut of the 32B model (0.95 GB of
    weights per step, far more than L2), ``--m`` conversations at a ``--ctx``-token context, a few decode steps."""
    from .models import config as C
    from .models.dense import DenseModel
    cfg = C.scaled(C.dense_32b(seed=0), args.layers or 4)
    B = max(1, args.m)
    m = DenseModel.random_init(cfg, "cuda:0", seed=0, max_seqs=B, max_ctx=args.ctx + 64, prefill_chunk=512)
    m.enable_step("on")
    firsts = []
    for s in range(B):
        m.new_seq(s)
        firsts.append(m.prefill(s, torch.randint(0, cfg.vocab, (args.ctx,), generator=torch.Generator().manual_seed(1 + s)))[0])
    seqs = list(range(B))
    m.decode_setup(seqs, firsts, 8)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    m._decode_body(seqs)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(4):
        m._decode_body(seqs)
    e1.record()
    torch.cuda.synchronize()
    print(json.dumps({"what": "profile_step", "layers": cfg.n_layers, "ctx": args.ctx, "rows": B, "us_per_step": e0.elapsed_time(e1) * 250.0,
                      "weight_bytes": m.weight_bytes(), "status": int(m.status.item())}))


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["gemv", "bf16", "attn", "gemm", "profile_gemv", "trace_gemv", "mm", "profile_mm", "profile_attn", "profile_attn_tc", "profile_gemm", "profile_misc", "profile_step"])
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--bits", type=int, default=4)
    ap.add_argument("--ks", type=int, default=0)
    ap.add_argument("--m", type=int, default=1)
    ap.add_argument("--small", action="store_true")
    ap.add_argument("--rows", type=int, default=256)
    ap.add_argument("--ctx", type=int, default=8192)
    args = ap.parse_args(argv)
    if args.what == "gemv":
        bench_gemv(args)
    elif args.what == "bf16":
        bench_bf16(args)
    elif args.what == "profile_gemv":
        profile_gemv(args)
    elif args.what == "gemm":
        bench_gemm(args)
    elif args.what == "trace_gemv":
        trace_gemv(args)
    elif args.what == "mm":
        bench_mm(args)
    elif args.what == "profile_mm":
        profile_mm(args)
    elif args.what == "attn":
        bench_attn(args)
    elif args.what == "profile_attn":
        profile_attn(args)
    elif args.what == "profile_attn_tc":
        profile_attn_tc(args)
    elif args.what == "profile_gemm":
        profile_gemm(args)
    elif args.what == "profile_misc":
        profile_misc(args)
    elif args.what == "profile_step":
        profile_step(args)
    else:
        raise SystemExit(f"{args.what}: not available yet")


if __name__ == "__main__":
    main()
