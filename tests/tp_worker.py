"""Worker of the multi-GPU tests (launched by tests/test_tp_gpu.py through torch.distributed.run, one rank per GPU)."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from agens_engine_b200 import _lib  # noqa: E402
from agens_engine_b200.models import config as C  # noqa: E402
from agens_engine_b200.models import oracle as O  # noqa: E402
from agens_engine_b200.models.dense import DenseModel  # noqa: E402
from agens_engine_b200.parallel.comm import NcclComm, PushComm  # noqa: E402
from agens_engine_b200.parallel.symm import SymmetricInbox  # noqa: E402
from agens_engine_b200.parallel.tp_model import TpDenseModel  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = f"cuda:{local}"
    dist.init_process_group("nccl", device_id=torch.device(dev))
    what = sys.argv[1]
    if what == "collectives":
        inbox = SymmetricInbox(rank, world, 1 << 16, 3, dev, timeout_s=1.0)
        pc, nc = PushComm(inbox), NcclComm()
        torch.manual_seed(rank)
        for it in range(7):                       # more calls than slots: exercises the re-arm rotation
            x = torch.randn(4096 * (1 + it % 3), device=dev)
            a, b = pc.all_reduce(x), nc.all_reduce(x)
            assert torch.allclose(a, b, rtol=1e-6, atol=1e-6), (it, (a - b).abs().max())
            ga = [torch.empty_like(a) for _ in range(world)]
            dist.all_gather(ga, a)
            assert all(torch.equal(ga[0], g) for g in ga)       # rank-ordered sums: identical bits on every rank
            xb = x.to(torch.bfloat16)
            assert torch.allclose(pc.all_reduce(xb, out_dtype=torch.float32), nc.all_reduce(xb, out_dtype=torch.float32), atol=1e-5)
        x = torch.randn(1024, device=dev)
        assert torch.equal(pc.all_gather(x), nc.all_gather(x))
        y = torch.randn(world, 2048, device=dev)
        assert torch.allclose(pc.reduce_scatter(y), nc.reduce_scatter(y), rtol=1e-6, atol=1e-6)
        pc.barrier()
        torch.cuda.synchronize()
        inbox.check_status()
        # GEMM with the reduce-scatter fused into its epilogue (partial tiles stored straight into the owners' inboxes):
        # every rank's rows equal the sum over ranks of the plain products; several calls rotate the slots; row counts
        # that do not divide by the rank count or the tile height
        big = SymmetricInbox(rank, world, 512 * 384, 3, dev, timeout_s=2.0)
        pg = PushComm(big)
        g = torch.Generator(device=dev).manual_seed(100 + rank)
        for T, N, K_ in ((300, 384, 256), (517, 256, 320), (1000, 384, 128), (64 * world, 128, 64)):
            xa = torch.randn(T, K_, device=dev, generator=g).to(torch.bfloat16)
            wb = (torch.randn(N, K_, device=dev, generator=g) * 0.1).to(torch.bfloat16)
            shard, rows_per = pg.gemm_reduce_scatter(xa, wb)
            full = pg.all_gather(shard).view(world * rows_per, N)[:T]
            want = xa.float() @ wb.float().t()
            dist.all_reduce(want)
            assert torch.allclose(full, want, rtol=2e-3, atol=2e-3 * want.abs().max().item()), (T, N, K_, (full - want).abs().max().item())
            fa = [torch.empty_like(full) for _ in range(world)]
            dist.all_gather(fa, full.contiguous())
            assert all(torch.equal(fa[0], f) for f in fa)       # rank-ordered sums: identical bits on every rank
        torch.cuda.synchronize()
        big.check_status("gemm_reduce_scatter")
        big.close()
        # the same linear in two launches: GEMM with the push epilogue, then one combine + gather kernel (bf16 result);
        # seven calls go around the three slot pairs more than twice
        six = SymmetricInbox(rank, world, 512 * 384, 6, dev, timeout_s=2.0)
        ps = PushComm(six)
        for it, (T, N, K_) in enumerate(((300, 384, 256), (517, 256, 320), (1000, 384, 128), (64 * world, 128, 64), (33, 64, 64),
                                         (999, 384, 256), (512, 384, 64))):
            xa = torch.randn(T, K_, device=dev, generator=g).to(torch.bfloat16)
            wb = (torch.randn(N, K_, device=dev, generator=g) * 0.1).to(torch.bfloat16)
            got = ps.gemm_reduce_gather(xa, wb)
            want = xa.float() @ wb.float().t()
            dist.all_reduce(want)
            assert got.shape == (T, N) and (got.float() - want).abs().max().item() <= 0.01 * want.abs().max().item() + 1e-3, (it, T, N, K_)
            fa = [torch.empty_like(got) for _ in range(world)]
            dist.all_gather(fa, got)
            assert all(torch.equal(fa[0], f) for f in fa)
        torch.cuda.synchronize()
        six.check_status("gemm_reduce_gather")
        six.close()
        # a lost message: the last rank drops its push; every rank's bounded wait runs out and reports, nothing hangs
        inbox.timeout_ns = int(0.2e9)
        out = pc.all_reduce(torch.ones(64, device=dev), skip_push=(rank == world - 1))
        torch.cuda.synchronize()
        assert int(inbox.status.item()) == _lib.B2_ERR_TIMEOUT
        try:
            inbox.check_status("all_reduce")
            raise AssertionError("expected a timeout error")
        except _lib.B2Error as e:
            assert e.code == _lib.B2_ERR_TIMEOUT
        # recovery: re-arm, agree on the host, carry on
        dist.barrier()
        inbox.rearm_all()
        torch.cuda.synchronize()
        dist.barrier()
        pc2 = PushComm(inbox)
        inbox.timeout_ns = int(1e9)
        z = pc2.all_reduce(torch.full((64,), float(rank + 1), device=dev))
        torch.cuda.synchronize()
        assert torch.equal(z, torch.full((64,), float(world * (world + 1) // 2), device=dev))
        inbox.check_status()
        inbox.close()
    elif what == "model":
        cfg = C.oracle_tiny()
        if cfg.n_kv_heads % world:
            cfg.n_kv_heads = world * max(1, cfg.n_kv_heads // world)
        ow = O.random_weights(cfg, seed=0)
        torch.manual_seed(0)
        prompt = torch.randint(0, cfg.vocab, (48,))
        m = TpDenseModel.from_oracle(ow, dev, rank, world, max_seqs=1, max_ctx=256)
        m.new_seq(0)
        toks = m.generate_greedy(0, prompt, 16)
        m.inbox.check_status("tp decode")
        print(f"rank {rank}: fused decode done", flush=True)
        ref = None
        if rank == 0:
            r = DenseModel.from_oracle(ow, dev, max_seqs=1, max_ctx=256)
            r.new_seq(0)
            ref = r.generate_greedy(0, prompt, 16)
            agree = sum(int(a == b) for a, b in zip(toks.tolist(), ref.tolist()))
            assert agree >= 14, (toks.tolist(), ref.tolist())
        allt = [None] * world
        dist.all_gather_object(allt, toks.tolist())
        assert all(t == allt[0] for t in allt)          # every rank produced the same tokens
        # teacher-forced logits gate (the reference's TP check: next-token agreement with one GPU and mean KL,
        # README.md:267-272): the same 16 continuation tokens through both models, row by row
        from agens_engine_b200.tools.compare import logits_report
        forced = toks.tolist()
        m.truncate(0, len(prompt))
        rows_tp = torch.stack([m.forward_rows([t], [0], want_logits=True)[1][0] for t in forced])
        all_rows = [None] * world
        dist.all_gather_object(all_rows, rows_tp.cpu())
        assert all(torch.equal(x, all_rows[0]) for x in all_rows)      # replicated logits: bitwise equal on every rank
        if rank == 0:
            r.truncate(0, len(prompt))
            rows_1 = torch.stack([r.forward_rows([t], [0], want_logits=True)[1][0] for t in forced])
            rep = logits_report(rows_1, rows_tp)
            assert rep["top1_agreement"] >= 0.9 and rep["mean_kl"] < 2e-2, rep
            print(f"rank 0: logits gate {rep}", flush=True)
        # the same shards loaded from a checkpoint directory give the same tokens
        import tempfile
        from agens_engine_b200.utils import checkpoint as K
        box = [tempfile.mkdtemp() if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        if rank == 0:
            K.save_oracle(box[0], ow, shards=2)
        dist.barrier()
        c = K.load_model(box[0], dev, rank=rank, world=world, max_seqs=1, max_ctx=256)
        c.new_seq(0)
        assert c.generate_greedy(0, prompt, 16).tolist() == toks.tolist()
        torch.cuda.synchronize()
        dist.barrier()
        c.close()
        # a long prefill chunk takes the fused GEMM + reduce-scatter for its row-parallel linears: the logits after it
        # agree with the unfused route (push reduce-scatter of the finished product) and are the same bits on every rank
        long_prompt = torch.randint(0, cfg.vocab, (700,))
        lg = {}
        for fused in (True, False):
            f = TpDenseModel.from_oracle(ow, dev, rank, world, max_seqs=1, max_ctx=1024, prefill_chunk=512)
            f.fused_prefill = fused
            f.prefill_mm = False                   # the dequantise + bf16 GEMM route for every chunk size
            f.new_seq(0)
            _, lg[fused] = f.prefill(0, long_prompt, want_logits=True)
            assert (f._fused_comm is not None) == fused
            f.inbox.check_status("tp prefill")
            torch.cuda.synchronize(); dist.barrier()
            f.close()
        err = (lg[True] - lg[False]).abs().max().item()
        assert err <= 0.02 * lg[False].abs().max().item(), err
        both = [None] * world
        dist.all_gather_object(both, lg[True].cpu())
        assert all(torch.equal(x, both[0]) for x in both)
        # fused path vs the NCCL baseline path: same tokens
        b = TpDenseModel.from_oracle(ow, dev, rank, world, max_seqs=1, max_ctx=256, use_nccl_decode=True)
        b.new_seq(0)
        print(f"rank {rank}: baseline model built", flush=True)
        tb = b.generate_greedy(0, prompt, 16)
        print(f"rank {rank}: baseline decode done", flush=True)
        agree = sum(int(x == y) for x, y in zip(toks.tolist(), tb.tolist()))
        assert agree >= 14, (toks.tolist(), tb.tolist())
        torch.cuda.synchronize()
        print(f"rank {rank}: closing", flush=True)
        m._graphs.clear(); b._graphs.clear()
        m.close(); b.close()
        print(f"rank {rank}: closed", flush=True)
    elif what == "step":
        # the persistent step kernel under tensor parallelism: row-parallel partials cross NVLink inside the kernel and
        # every rank adds all ranks' fragments in rank order; ranks agree bit for bit and match one GPU within tolerance
        bits = {"0.qkv": 4, "0.o": 3, "0.gate_up": 2, "0.down": 4, "1.qkv": 2, "1.o": 4, "1.gate_up": 3, "1.down": 2}
        cfg = C.ModelConfig("step-tp", 2, 512, 8, 4, 128, 1024, 2048, rope_theta=1e6, group=128, bits=bits, lm_head_bits=4)
        ow = O.random_weights(cfg, seed=3)
        torch.manual_seed(0)
        prompt = torch.randint(0, cfg.vocab, (48,))
        cont = torch.randint(0, cfg.vocab, (4,)).tolist()
        m = TpDenseModel.from_oracle(ow, dev, rank, world, max_seqs=2, max_ctx=256)
        assert m.enable_step() and m.step.world == world
        m.new_seq(0)
        m.prefill(0, prompt)
        rows = []
        for t in cont:
            _, lg = m.forward_rows([t], [0], want_logits=True)
            rows.append(lg[0])
        # the same four tokens as one verify block of a second sequence: bit-identical rows
        m.new_seq(1)
        m.prefill(1, prompt)
        _, blk = m.forward_rows(cont, [1] * 4, want_logits=True)
        for i in range(4):
            assert torch.equal(blk[i], rows[i]), i
        lg = torch.stack(rows)
        assert m.device_status() == 0
        assert m.step.launches >= 5
        allr = [torch.empty_like(lg) for _ in range(world)]
        dist.all_gather(allr, lg)
        assert all(torch.equal(allr[0], x) for x in allr)          # rank-ordered sums: identical bits on every rank
        if rank == 0:
            r = DenseModel.from_oracle(ow, dev, max_seqs=1, max_ctx=256)
            r.new_seq(0)
            r.prefill(0, prompt)
            ref = torch.stack([r.forward_rows([t], [0], want_logits=True)[1][0] for t in cont])
            err = (lg - ref).abs().max().item()
            assert err < 0.02 * ref.abs().max().item(), err
        # greedy decode through the graph-replayed step: every rank produces the same tokens
        m.truncate(0, 48)
        first = int(lg[0].argmax())
        m.decode_setup([0], [first], 8)
        toks = m.decode_steps(8)[:, 0].tolist()
        allt = [None] * world
        dist.all_gather_object(allt, toks)
        assert all(t == allt[0] for t in allt), allt
        assert m.device_status() == 0
        # a rank that does not signal: every rank's bounded barrier wait runs out, the status word says so, nothing
        # hangs; after a host-side agreement the counters are reset and the next step is fine again
        m.step.timeout_ns = int(0.3e9)
        m.step.skip_push = rank == world - 1
        m.forward_rows([cont[0]], [0])
        torch.cuda.synchronize()
        assert m.device_status() == _lib.B2_ERR_TIMEOUT
        m.step.skip_push = False
        dist.barrier()
        m.recover()
        torch.cuda.synchronize()
        dist.barrier()
        m.new_seq(0)
        m.prefill(0, prompt)
        _, again = m.forward_rows([cont[0]], [0], want_logits=True)
        assert m.device_status() == 0
        assert torch.equal(again[0], rows[0])
        torch.cuda.synchronize()
        dist.barrier()
        m._graphs.clear()
        m.close()
    elif what == "engine":
        # rank 0 schedules, the others follow; batched requests equal their solo runs, greedy and sampled
        from agens_engine_b200.parallel import driver as D
        from agens_engine_b200.serve.engine import Engine
        cfg = C.oracle_tiny()
        ow = O.random_weights(cfg, seed=0)
        m = TpDenseModel.from_oracle(ow, dev, rank, world, max_seqs=4, max_ctx=256, prefill_chunk=128)
        ctrl = D.control_group()
        if rank == 0:
            drv = D.TpDriver(m, ctrl)
            torch.manual_seed(5)
            prompts = [torch.randint(0, cfg.vocab, (n,)).tolist() for n in (20, 150, 33)]
            samp = {"max_new_tokens": 12, "temperature": 0.8, "top_k": 30, "seed": 17}

            def serve(reqs):
                got = {}
                eng = Engine(drv, lambda rid, t, f, e: got.setdefault(rid, []).extend(t) or False)
                rids = [eng.submit(p, s) for p, s in reqs]
                eng.run_until_idle(5000)
                assert eng.idle()
                return [got[r] for r in rids]

            reqs = [(p, {"max_new_tokens": 12}) for p in prompts] + [(prompts[0], samp)]
            together = serve(reqs)
            alone = [serve([r])[0] for r in reqs]
            assert together == alone, (together, alone)
            # more than eight rows per step: the tensor-core GEMM + push all-reduce path, pinned for every step
            def serve16(reqs):
                got = {}
                eng = Engine(drv, lambda rid, t, f, e: got.setdefault(rid, []).extend(t) or False, max_batch=4, max_drafts=3)
                rids = [eng.submit(p, s) for p, s in reqs]
                eng.run_until_idle(5000)
                return [got[r] for r in rids]
            t16 = serve16(reqs)
            a16 = [serve16([r])[0] for r in reqs]
            assert t16 == a16 and all(len(t) == 12 for t in t16), (t16, a16)
            # a companion drafter beside the leader (a plain single-GPU model on rank 0): same tokens, drafts accepted
            from agens_engine_b200.spec import CopyLookupSource, ModelSource
            drafter = DenseModel.from_oracle(ow, dev, max_seqs=4, max_ctx=256)
            got = {}
            eng = Engine(drv, lambda rid, t, f, e: got.setdefault(rid, []).extend(t) or False, max_batch=4, max_drafts=3,
                         sources_factory=lambda: [CopyLookupSource(), ModelSource(drafter, 3)])
            rids = [eng.submit(p, s) for p, s in reqs]
            eng.run_until_idle(5000)
            assert [got[r] for r in rids] == t16, ([got[r] for r in rids], t16)
            assert eng.spec.stats.accepted > 0
            # an MTP head beside the leader: unsharded, with its own full lm_head, fed with the leader's replicated hidden
            # rows (prompt positions included); same tokens again
            from agens_engine_b200.models.mtp import MtpHead
            from agens_engine_b200.spec import MtpSource
            head = MtpHead.random_init_for(m)
            assert head.own_lm_head and head.lm_head.n >= cfg.vocab and head.cfg.n_heads == cfg.n_heads
            src = MtpSource(head, depth=2)
            got = {}
            eng = Engine(drv, lambda rid, t, f, e: got.setdefault(rid, []).extend(t) or False, max_batch=4, max_drafts=3,
                         sources_factory=lambda: [src])
            rids = [eng.submit(p, s) for p, s in reqs]
            eng.run_until_idle(5000)
            assert [got[r] for r in rids] == t16, ([got[r] for r in rids], t16)
            assert eng.spec.stats.by_source.get("mtp", [0, 0])[0] > 0 and head.free_pages() == head.n_pages
            drv.set_linear_path(None)
            assert all(len(t) == 12 for t in together) and together[3] != together[0]
            blob = None
            drv.new_seq(0); drv.prefill(0, torch.tensor(prompts[0], dtype=torch.int32))
            blob = drv.park(0); drv.unpark(1, blob); drv.free_seq(1)
            drv.shutdown()
        else:
            D.follow(m, ctrl)
        torch.cuda.synchronize()
        m.inbox.check_status("tp engine")
        dist.barrier()
        m.close()
    dist.barrier()
    dist.destroy_process_group()
    print(f"rank {rank}: {what} ok")


if __name__ == "__main__":
    main()
