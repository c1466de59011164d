#!/usr/bin/env python
"""Reference arm of bench.py: the UNMODIFIED kernel library of the reference (``kernels/`` built by its own CMake
project into ``baseline/_ref/libagens_kernels_py.so``, see ``baseline/build_reference.py``) driven through its stock C
ABI (``kernels/include/agens_kernels.h``) on the per-rank linear shapes of the 32B dense decoder.

What is timed is one decode step of the linear path: embedding, per layer RMSNorm -> q/k/v GEMV (one multi-segment
launch) -> o_proj GEMV -> residual add + RMSNorm -> gate/up GEMV -> SiLU*up -> down GEMV -> residual add + RMSNorm, then
the lm_head GEMV and the argmax, captured in a CUDA graph as the reference's runtime does.  Weights are random values
in the reference's own symmetric group-128 container at the same seeded 2/3/4-bit assignment per linear.  Attention,
RoPE / KV store and sampling are NOT run (the reference's attention is built for head_dim 256 and its own hybrid
model); at more than one GPU the two all-reduces per layer run on NCCL inside the same graph, because the
reference's own CUDA-IPC all-reduce waits on peers without a bound and is not run on this pool.  The number is an
upper bound on what the reference could reach for this model: the ratio against it is conservative.

Nothing of ``agens_engine_b200`` is imported here.
"""
from __future__ import annotations

import ctypes as C
import json
import os
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
LIB = HERE / "_ref" / "libagens_kernels_py.so"
LINEARS = ("qkv", "o", "gate_up", "down")


def seeded_bits(seed: int = 0):
    """The 2/3/4-bit assignment of the named benchmark config: one draw per linear, layer-major, from a seeded torch
    CPU generator (the rule the engine under test uses, restated here so that this file imports none of it)."""
    import torch
    names = [f"{l}.{lin}" for l in range(64) for lin in LINEARS]
    gen = torch.Generator().manual_seed(seed)
    idx = torch.randint(0, 3, (len(names),), generator=gen).tolist()
    return {nm: (2, 3, 4)[i] for nm, i in zip(names, idx)}


def unavailable(why: str):
    print(json.dumps({"impl": "reference", "unavailable": why}))
    return 0


def run(args) -> int:
    if not LIB.exists():
        return unavailable("baseline/_ref/libagens_kernels_py.so is missing: run `python baseline/build_reference.py REFERENCE_DIR` "
                           "(CMake + nvcc build of the reference's kernels for sm_100)")
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device(f"cuda:{local}")
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    lib = C.CDLL(str(LIB))
    vp, i32 = C.c_void_p, C.c_int
    lib.ak_wq_kt_weight_bytes.restype = C.c_size_t
    lib.ak_wq_kt_weight_bytes.argtypes = [i32, i32, i32]
    lib.ak_w4_kt_scale_bytes.restype = C.c_size_t
    lib.ak_w4_kt_scale_bytes.argtypes = [i32, i32, i32]
    lib.ak_wq_repack_kt.argtypes = [i32, vp, vp, vp, vp, i32, i32, i32, vp]
    lib.ak_wq_gemv_kt_multi.argtypes = [i32, vp, i32, i32, C.POINTER(vp), C.POINTER(vp), C.POINTER(vp), C.POINTER(i32),
                                        C.POINTER(i32), i32, i32, i32, vp]
    lib.ak_rmsnorm.argtypes = [vp, vp, vp, i32, i32, i32, i32, C.c_float, i32, vp]
    lib.ak_add_rmsnorm.argtypes = [vp, vp, vp, vp, vp, i32, i32, C.c_float, i32, vp]
    lib.ak_silu_mul.argtypes = [vp, vp, i32, i32, vp]
    lib.ak_argmax.argtypes = [vp, i32, i32, i32, vp, vp]
    lib.ak_embed.argtypes = [vp, vp, vp, i32, i32, vp]
    lib.ak_set_device.argtypes = [i32]
    lib.ak_set_device(local)

    L, d, hq, hkv, hd, ffn, vocab, group = 64, 5120, 64, 8, 128, 25600, 151936, 128
    if args.layers:
        L = args.layers
    bits = seeded_bits(0)
    hq_l, hkv_l, ffn_l = hq // world, hkv // world, ffn // world
    vshard = (vocab + world - 1) // world
    vshard = (vshard + 15) // 16 * 16
    st = torch.cuda.current_stream().cuda_stream
    gen = torch.Generator(device=dev).manual_seed(1234 + rank)
    keep = []

    def check(code, what):
        if code != 0:
            raise RuntimeError(f"{what}: CUDA error {code}")

    def make(n, k, b):
        """Random weights of width b in the int4 container -> the reference's KT layout of that width."""
        words = torch.randint(-2 ** 31, 2 ** 31 - 1, (n, k // 8), dtype=torch.int32, device=dev, generator=gen)
        if b == 3:
            words = (words & 0x77777777) + 0x44444444
        elif b == 2:
            words = (words & 0x33333333) + 0x66666666
        scales = (torch.rand(n, k // group, device=dev, generator=gen) * 0.01 + 0.002).to(torch.bfloat16)
        wt = torch.empty(lib.ak_wq_kt_weight_bytes(b, n, k), dtype=torch.uint8, device=dev)
        stt = torch.empty(lib.ak_w4_kt_scale_bytes(n, k, group), dtype=torch.uint8, device=dev)
        check(lib.ak_wq_repack_kt(b, words.data_ptr(), scales.data_ptr(), wt.data_ptr(), stt.data_ptr(), n, k, group, st),
              "ak_wq_repack_kt")
        keep.append((wt, stt))
        return wt, stt

    def seg(ws, ns, ys):
        m = len(ws)
        return ((vp * m)(*[w[0].data_ptr() for w in ws]), (vp * m)(*[w[1].data_ptr() for w in ws]),
                (vp * m)(*[y.data_ptr() for y in ys]), (i32 * m)(*ns), m)

    bf = lambda *s: torch.zeros(*s, dtype=torch.bfloat16, device=dev)
    h, xn, o_out, d_out = bf(d), bf(d), bf(d), bf(d)
    qb, kb, vb = bf(hq_l * hd), bf(hkv_l * hd), bf(hkv_l * hd)
    gu, act = bf(2 * ffn_l), bf(ffn_l)
    logits = bf(vshard)
    out_id = torch.zeros(1, dtype=torch.int32, device=dev)
    ids = torch.randint(0, vocab, (1,), dtype=torch.int32, device=dev, generator=gen)
    embed = (torch.randn(vocab, d, device=dev, generator=gen) * 0.02).to(torch.bfloat16)
    ln = (1.0 + 0.05 * torch.randn(2 * L + 1, d, device=dev, generator=gen)).to(torch.bfloat16)
    layers = []
    wbytes = 0
    for l in range(L):
        bq, bo, bg, bd = (bits[f"{l}.{lin}"] for lin in LINEARS)
        wq, wk, wv = make(hq_l * hd, d, bq), make(hkv_l * hd, d, bq), make(hkv_l * hd, d, bq)
        wo = make(d, hq_l * hd, bo)
        wg, wu = make(ffn_l, d, bg), make(ffn_l, d, bg)
        wd = make(d, ffn_l, bd)
        layers.append((bq, seg([wq, wk, wv], [hq_l * hd, hkv_l * hd, hkv_l * hd], [qb, kb, vb]),
                       bo, seg([wo], [d], [o_out]),
                       bg, seg([wg, wu], [ffn_l, ffn_l], [gu[:ffn_l], gu[ffn_l:]]),
                       bd, seg([wd], [d], [d_out])))
    wlm = make(vshard, d, 4)
    lm = seg([wlm], [vshard], [logits])
    wbytes = sum(w.numel() + s.numel() for w, s in keep)
    torch.cuda.synchronize()
    eps = 1e-6

    def gemv(b, x, sg, k):
        wt, stt, ys, ns, m = sg
        check(lib.ak_wq_gemv_kt_multi(b, x.data_ptr(), 1, m, wt, stt, ys, ns, None, k, group, 0, st), "ak_wq_gemv_kt_multi")

    use_ar = [world > 1]

    def all_reduce(t):
        # The reference sums row-parallel partial rows with its own CUDA-IPC push kernels (kernels/src/tp_ar.cu), whose
        # device-side waits have no bound: they are not run on this pool.  NCCL stands in (library code, captured in
        # the same graph), so that the arm at N > 1 does the cross-GPU work a tensor-parallel step needs.
        if use_ar[0]:
            dist.all_reduce(t)

    def step():
        check(lib.ak_embed(ids.data_ptr(), embed.data_ptr(), h.data_ptr(), 1, d, st), "ak_embed")
        check(lib.ak_rmsnorm(h.data_ptr(), ln[0].data_ptr(), xn.data_ptr(), 1, d, d, d, eps, 0, st), "ak_rmsnorm")
        for l, (bq, sq, bo, so, bg, sg_, bd, sd) in enumerate(layers):
            gemv(bq, xn, sq, d)
            gemv(bo, qb, so, hq_l * hd)                      # attention omitted: o_proj reads the q rows
            all_reduce(o_out)
            check(lib.ak_add_rmsnorm(o_out.data_ptr(), h.data_ptr(), h.data_ptr(), ln[2 * l + 1].data_ptr(), xn.data_ptr(),
                                     1, d, eps, 0, st), "ak_add_rmsnorm")
            gemv(bg, xn, sg_, d)
            check(lib.ak_silu_mul(gu.data_ptr(), act.data_ptr(), 1, ffn_l, st), "ak_silu_mul")
            gemv(bd, act, sd, ffn_l)
            all_reduce(d_out)
            check(lib.ak_add_rmsnorm(d_out.data_ptr(), h.data_ptr(), h.data_ptr(), ln[2 * l + 2].data_ptr(), xn.data_ptr(),
                                     1, d, eps, 0, st), "ak_add_rmsnorm")
        gemv(4, xn, lm, d)
        check(lib.ak_argmax(logits.data_ptr(), 1, vshard, vshard, out_id.data_ptr(), st), "ak_argmax")

    # warm-up outside capture (lazy attribute calls), then one graph per step as the reference's runtime does
    stream = torch.cuda.Stream(device=dev)
    mode = "cuda graph"
    with torch.cuda.stream(stream):
        st = stream.cuda_stream
        step()
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        try:
            with torch.cuda.graph(graph, stream=stream):
                st = torch.cuda.current_stream().cuda_stream
                step()
        except Exception as e:          # capture refused (a call that cannot be captured)
            graph = None
            torch.cuda.synchronize()
            if use_ar[0]:
                # the all-reduce could not be captured: keep the graph (the reference's launch mode) and drop the all-reduce
                use_ar[0] = False
                try:
                    graph = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(graph, stream=stream):
                        st = torch.cuda.current_stream().cuda_stream
                        step()
                    mode = f"cuda graph WITHOUT all-reduce (capture with NCCL failed: {type(e).__name__})"
                except Exception as e2:
                    graph = None
                    mode = f"eager launches (graph capture failed: {type(e2).__name__})"
                    torch.cuda.synchronize()
            else:
                mode = f"eager launches (graph capture failed: {type(e).__name__})"
        st = stream.cuda_stream
        run_step = graph.replay if graph is not None else step

        def barrier():
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()

        warm = max(args.warmup, 3)
        for _ in range(warm):
            run_step()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(args.steps):
            run_step()
        e1.record(stream)
        barrier()
        ms = e0.elapsed_time(e1)
        # end to end: token id from pinned host memory every step, result read back every step
        import time
        tin = torch.zeros(1, dtype=torch.int32).pin_memory()
        tout = torch.zeros(1, dtype=torch.int32).pin_memory()
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            ids.copy_(tin, non_blocking=True)
            run_step()
            tout.copy_(out_id, non_blocking=True)
            stream.synchronize()
            tin.copy_(tout % vocab)
        barrier()
        e2e_ms = (time.perf_counter() - t0) * 1e3
    if world > 1:
        t = torch.tensor([ms, e2e_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_ms = float(t[0]), float(t[1])
    if rank == 0:
        value = args.steps / (ms / 1e3)
        print(json.dumps({
            "impl": "reference", "metric": "decode_tok_s_32b_mixedbit", "value": round(value, 2), "unit": "tok/s",
            "n_gpus": world, "steps": args.steps, "warmup": warm, "ms_per_step": round(ms / args.steps, 4),
            "higher_is_better": True, "scaling": "strong", "dtype": "bf16", "data": "synthetic", "same_config": False,
            "reference_class": "kernels only: the reference's unmodified GEMV / norm / SiLU / argmax kernels built for "
                               "sm_100 from its CMake project, per-rank linear shapes of the 32B dense decoder x "
                               f"{L} layers + lm_head, {mode}; attention, RoPE / KV store and sampling omitted (its "
                               "attention is fixed at head_dim 256); at N > 1 the two all-reduces per layer run on NCCL inside the same graph "
                               "(the reference's own IPC all-reduce spins without bound and is not run here); an upper "
                               "bound on the reference, so the ratio is conservative",
            "config": {"model": "dense-32b linear path (64 layers, d 5120, 64q/8kv x 128, ffn 25600, vocab 151936; 2/3/4-bit "
                                "seeded per linear, symmetric group 128)", "global_batch": 1, "parallelism": f"tp{world}",
                       "weight_gb_per_gpu": round(wbytes / 1e9, 2)},
            "e2e": {"value": round(args.steps / (e2e_ms / 1e3), 2), "unit": "tok/s", "h2d_bytes_per_step": 4,
                    "d2h_bytes_per_step": 4},
        }))
    if world > 1:
        # No teardown of the process group: with NCCL collectives captured in a CUDA graph its destructor has been seen
        # to wait on the watchdog for minutes.  The result is out; every rank leaves at once.
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)
    return 0
