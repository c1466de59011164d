#!/usr/bin/env python
"""Per-kernel timing of the reference's own GEMV kernels (unmodified library, stock C ABI) on the 32B dense shapes, for
the per-kernel table next to this engine's kernels: same method as ``agens_engine_b200/bench_kernels.py`` (a CUDA
graph of back-to-back launches over rotating weight copies larger than L2, median per launch).

    python baseline/reference_kernels.py --m 1 [--m 8 --m 16]

Nothing of ``agens_engine_b200`` is imported.  Weights: random values in the reference's symmetric group-128 container
repacked by its own ``ak_wq_repack_kt``; with AGENS_W4H=1 in the environment its 4-bit linears use its W4H layout.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import sys
from pathlib import Path

LIB = Path(__file__).resolve().parent / "_ref" / "libagens_kernels_py.so"


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--m", type=int, action="append")
    ap.add_argument("--small", action="store_true")
    args = ap.parse_args()
    if not LIB.exists():
        print(json.dumps({"unavailable": "baseline/_ref/libagens_kernels_py.so is missing (python baseline/build_reference.py)"}))
        return 0
    import torch
    dev = torch.device("cuda:0")
    lib = C.CDLL(str(LIB))
    vp, i32 = C.c_void_p, C.c_int
    lib.ak_wq_kt_weight_bytes.restype = C.c_size_t
    lib.ak_wq_kt_weight_bytes.argtypes = [i32, i32, i32]
    lib.ak_w4_kt_scale_bytes.restype = C.c_size_t
    lib.ak_w4_kt_scale_bytes.argtypes = [i32, i32, i32]
    lib.ak_wq_repack_kt.argtypes = [i32, vp, vp, vp, vp, i32, i32, i32, vp]
    lib.ak_wq_gemv_kt_multi.argtypes = [i32, vp, i32, i32, C.POINTER(vp), C.POINTER(vp), C.POINTER(vp), C.POINTER(i32),
                                        C.POINTER(i32), i32, i32, i32, vp]
    gen = torch.Generator(device=dev).manual_seed(5)
    shapes = [("qkv", 10240, 5120), ("o", 5120, 8192), ("gate_up", 51200, 5120), ("down", 5120, 25600), ("lm_head", 151936, 5120)]
    if args.small:
        shapes = shapes[2:3]
    group = 128
    for m in (args.m or [1]):
        for name, n, k in shapes:
            for bits in ([4] if name == "lm_head" else [2, 3, 4]):
                words = torch.randint(-2 ** 31, 2 ** 31 - 1, (n, k // 8), dtype=torch.int32, device=dev, generator=gen)
                if bits == 3:
                    words = (words & 0x77777777) + 0x44444444
                elif bits == 2:
                    words = (words & 0x33333333) + 0x66666666
                scales = (torch.rand(n, k // group, device=dev, generator=gen) * 0.01 + 0.002).to(torch.bfloat16)
                wb, sb = lib.ak_wq_kt_weight_bytes(bits, n, k), lib.ak_w4_kt_scale_bytes(n, k, group)
                ncopy = max(2, min(24, (512 << 20) // (wb + sb) + 1))
                copies = []
                st0 = torch.cuda.current_stream().cuda_stream
                for _ in range(ncopy):
                    wt = torch.empty(wb, dtype=torch.uint8, device=dev)
                    stt = torch.empty(sb, dtype=torch.uint8, device=dev)
                    rc = lib.ak_wq_repack_kt(bits, words.data_ptr(), scales.data_ptr(), wt.data_ptr(), stt.data_ptr(), n, k, group, st0)
                    if rc:
                        raise RuntimeError(f"ak_wq_repack_kt: {rc}")
                    copies.append((wt, stt))
                del words
                x = torch.randn(m, k, device=dev, generator=gen).to(torch.bfloat16)
                y = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
                nn = (i32 * 1)(n)
                arrs = [((vp * 1)(wt.data_ptr()), (vp * 1)(stt.data_ptr()), (vp * 1)(y.data_ptr())) for wt, stt in copies]
                stream = torch.cuda.Stream()

                def launch_all(st):
                    for wa, sa, ya in arrs:
                        rc = lib.ak_wq_gemv_kt_multi(bits, x.data_ptr(), m, 1, wa, sa, ya, nn, None, k, group, 0, st)
                        if rc:
                            raise RuntimeError(f"ak_wq_gemv_kt_multi: {rc}")
                with torch.cuda.stream(stream):
                    launch_all(stream.cuda_stream)
                    stream.synchronize()
                    g = torch.cuda.CUDAGraph()
                    try:
                        with torch.cuda.graph(g, stream=stream):
                            launch_all(torch.cuda.current_stream().cuda_stream)
                        run = g.replay
                        how = "graph"
                    except Exception:
                        torch.cuda.synchronize()
                        run = lambda: launch_all(stream.cuda_stream)
                        how = "eager"
                    for _ in range(3):
                        run()
                    ts = []
                    for _ in range(10):
                        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                        e0.record(stream)
                        run()
                        e1.record(stream)
                        stream.synchronize()
                        ts.append(e0.elapsed_time(e1) * 1e3 / ncopy)
                ts.sort()
                med = ts[len(ts) // 2]
                print(json.dumps(dict(impl="reference", name=name, n=n, k=k, bits=bits, m=m, us=round(med, 2),
                                      gbs=round((wb + sb) / med / 1e3, 1), copies=ncopy, launch=how)), flush=True)
                del copies, arrs
    return 0


if __name__ == "__main__":
    sys.exit(main())
