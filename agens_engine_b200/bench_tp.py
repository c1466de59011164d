"""Multi-rank kernel benchmarks (one process per GPU, launched with torch.distributed.run).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29531 \\
        -m agens_engine_b200.bench_tp fused_prefill --rows 2048

``fused_prefill``: the row-parallel linears of a prefill chunk of the 32B model under tensor parallelism (o_proj
5120 x 8192 / N, down_proj 5120 x 25600 / N, bf16 weights as after dequantisation), three routes to the summed chunk on
every rank: (a) fused: tcgen05 GEMM with the reduce-scatter in its epilogue + one combine-and-gather kernel,
(b) unfused: GEMM, then push reduce-scatter and all-gather over the finished product, (c) library baseline: GEMM + NCCL
all-reduce.  Device time with CUDA events (median of 10 after 3 warm-ups, max over ranks), an L2 flush before each.
The roofline of a route is the slower of the GEMM at the measured bf16 peak and the bytes a rank must receive over
NVLink at the measured 770 GB/s peer bandwidth.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["fused_prefill"])
    ap.add_argument("--rows", type=int, default=2048)
    args = ap.parse_args(argv)
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0)))
    torch.cuda.set_device(dev)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    dist.init_process_group("nccl", device_id=dev)
    from .bench_kernels import peaks
    from .ops import gemm as G
    from .parallel.comm import PushComm
    from .parallel.symm import SymmetricInbox
    pk = peaks()
    T, N = args.rows, 5120
    rows_per = (T + world - 1) // world
    big = SymmetricInbox(rank, world, (rows_per * N + 3) // 4 * 4, 6, dev, timeout_s=2.0)
    small = SymmetricInbox(rank, world, 1 << 20, 3, dev, timeout_s=2.0)
    pf, pu = PushComm(big), PushComm(small)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    g = torch.Generator(device=dev).manual_seed(rank)

    def timed(fn):
        ts = []
        for it in range(13):
            flush.fill_(it & 255)
            dist.barrier(); torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(); fn(); e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1) * 1e3)
        ts = sorted(ts[3:])
        t = torch.tensor([ts[len(ts) // 2]], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    for name, k_full in (("o_proj", 8192), ("down_proj", 25600)):
        K = k_full // world
        x = torch.randn(T, K, device=dev, generator=g).to(torch.bfloat16)
        w = (torch.randn(N, K, device=dev, generator=g) * 0.02).to(torch.bfloat16)

        def fused():
            return pf.gemm_reduce_gather(x, w)

        def unfused():
            y = G.gemm_bf16(x, w).float().reshape(-1)
            per = small.slot_stride
            out = torch.empty_like(y)
            step = world * per
            for o in range(0, y.numel(), step):
                m = min(step, y.numel() - o)
                shard = ((m + world - 1) // world + 3) // 4 * 4
                buf = torch.zeros(world * shard, dtype=torch.float32, device=dev)
                buf[:m] = y[o:o + m]
                out[o:o + m] = pu.all_gather(pu.reduce_scatter(buf.view(world, shard))).reshape(-1)[:m]
            return out.view(T, N).to(torch.bfloat16)

        def nccl():
            y = G.gemm_bf16(x, w, out_f32=True)
            dist.all_reduce(y)
            return y.to(torch.bfloat16)

        def gemm_only():
            return G.gemm_bf16(x, w)

        a, b = fused().float(), nccl().float()
        err = (a - b).abs().max().item() / max(b.abs().max().item(), 1e-9)
        t_f, t_u, t_n, t_g = timed(fused), timed(unfused), timed(nccl), timed(gemm_only)
        flops = 2.0 * T * N * K
        link_bytes = 2.0 * (world - 1) / world * T * N * 4          # received per rank: reduce-scatter partials + gathered rows, fp32
        roof_us = max(flops / (pk["bf16_tflops"] * 1e6), link_bytes / 770e3)
        if rank == 0:
            print(json.dumps(dict(linear=name, ranks=world, rows=T, n=N, k_per_rank=K, fused_us=round(t_f, 1), unfused_push_us=round(t_u, 1),
                                  gemm_nccl_us=round(t_n, 1), gemm_alone_us=round(t_g, 1), roofline_us=round(roof_us, 1),
                                  fused_over_roofline=round(t_f / roof_us, 2), rel_err_vs_nccl=float(f"{err:.2e}"))), flush=True)
    torch.cuda.synchronize()
    big.check_status("bench"); small.check_status("bench")
    dist.barrier()
    big.close(); small.close()
    if rank == 0:
        print(json.dumps({"peaks": pk, "nvlink_gbs": 770, "timing": "CUDA events, median of 10, max over ranks, L2 flushed"}))
    dist.barrier()
    os._exit(0)


if __name__ == "__main__":
    main()
