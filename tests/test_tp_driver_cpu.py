"""Leader / follower protocol of the tensor-parallel driver on CPU ranks (gloo): forwarded calls are replayed, a call
that fails the same way on every rank does not stop the follower, and a follower that leaves between steps makes the
leader raise instead of blocking (reference: crates/agens-cli/src/tp.rs:190-298, crates/agens-cuda/src/lib.rs:310-322)."""
import multiprocessing as mp
import os
import time

import pytest


class FakeModel:
    """Records calls; `reserve` fails deterministically past 100 tokens, as a KV pool would on every rank alike."""

    def __init__(self):
        self.calls = []

    def new_seq(self, s):
        self.calls.append(("new_seq", s))

    def reserve(self, s, n):
        self.calls.append(("reserve", s, n))
        if n > 100:
            raise RuntimeError("KV pool exhausted")

    def forward_rows(self, ids, seqs, want_logits=False):
        self.calls.append(("forward_rows", tuple(ids), tuple(seqs)))
        return None, None

    def park(self, s):
        self.calls.append(("park", s))
        return {"len": 3}

    def unpark(self, s, blob):
        self.calls.append(("unpark", s, blob["len"]))

    def enable_host_tier(self, window_tokens, batch_pages=256):
        self.calls.append(("enable_host_tier", window_tokens))

    def prefill(self, seq, ids, want_logits=False, image_rows=None, rope_pos3=None, **kw):
        # what a rank needs of an image prompt: the ids, the encoder rows and the position table, bit for bit
        self.calls.append(("prefill", seq, tuple(ids.tolist()), str(image_rows.dtype), tuple(image_rows.shape),
                           float(image_rows.float().sum()), int(rope_pos3.sum())))
        return 0, None


def _rank(rank, world, port, mode, q):
    os.environ.update({"MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port), "RANK": str(rank), "WORLD_SIZE": str(world)})
    import torch.distributed as dist
    from agens_engine_b200.parallel import driver as D
    dist.init_process_group("gloo", rank=rank, world_size=world)
    ctrl = D.control_group(timeout_s=4.0)
    m = FakeModel()
    if rank == 0:
        drv = D.TpDriver(m, ctrl)
        drv.new_seq(0)
        try:
            drv.reserve(0, 1000)
            q.put(("leader", "no error"))
        except RuntimeError as e:
            q.put(("leader", "caught " + str(e)))
        drv.forward_rows([1, 2], [0, 0])
        blob = drv.park(0)
        drv.unpark(1, blob)
        drv.enable_host_tier(4096)
        if mode == "normal":
            import torch
            g = torch.Generator().manual_seed(1)
            rows = torch.randn(300, 64, generator=g).to(torch.bfloat16)           # large tensors travel as raw bytes
            pos3 = torch.arange(3 * 40, dtype=torch.int32).reshape(3, 40)
            drv.prefill(0, torch.arange(40, dtype=torch.int32), image_rows=rows, rope_pos3=pos3)
            q.put(("leader-prefill", m.calls[-1]))
        if mode == "death":
            time.sleep(1.5)                       # the follower has left by now
            t0 = time.time()
            try:
                for _ in range(3):
                    drv.forward_rows([3], [0])
                q.put(("leader", "not noticed"))
            except D.FollowerLost as e:
                q.put(("leader", "lost after %.1fs" % (time.time() - t0)))
        else:
            drv.shutdown()
            q.put(("leader", "done"))
    else:
        if mode == "death":
            # take exactly the six commands of the first part, then leave between steps without saying goodbye
            n = 0
            box = [None]
            while n < 6:
                dist.broadcast_object_list(box, src=0, group=ctrl)
                n += 1
            q.put(("follower", "left"))
            q.close(); q.join_thread()            # flush the message, then vanish without a goodbye
            os._exit(0)
        n = D.follow(m, ctrl, log=lambda s: q.put(("log", s)))
        q.put(("follower", n, m.calls))
    if mode != "death":
        dist.destroy_process_group()


def _run(mode):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29650 + (os.getpid() + (7 if mode == "death" else 0)) % 300
    ps = [ctx.Process(target=_rank, args=(r, 2, port, mode, q)) for r in range(2)]
    for p in ps:
        p.start()
    out = []
    deadline = time.time() + 90
    want = 3 if mode == "death" else 5
    while len(out) < want and time.time() < deadline:
        try:
            out.append(q.get(timeout=1.0))
        except Exception:
            if all(not p.is_alive() for p in ps):
                break
    for p in ps:
        p.join(timeout=20)
        if p.is_alive():
            p.terminate()
    return out


@pytest.mark.timeout(150)
def test_forwarded_calls_and_deterministic_errors():
    out = _run("normal")
    leader = [o for o in out if o[0] == "leader"]
    assert ("leader", "caught KV pool exhausted") in leader and ("leader", "done") in leader
    fol = [o for o in out if o[0] == "follower"][0]
    assert fol[1] == 7                                              # every command was taken, the failing one included
    names = [c[0] for c in fol[2]]
    assert names == ["new_seq", "reserve", "forward_rows", "park", "unpark", "enable_host_tier", "prefill"]
    lead = [o for o in out if o[0] == "leader-prefill"][0][1]
    assert fol[2][-1] == lead and lead[3] == "torch.bfloat16" and lead[4] == (300, 64)   # image rows reach the follower intact
    assert any("KV pool exhausted" in o[1] for o in out if o[0] == "log")


@pytest.mark.timeout(150)
def test_leader_raises_when_a_follower_leaves_between_steps():
    out = _run("death")
    assert ("follower", "left") in out
    leader = [o[1] for o in out if o[0] == "leader" and o[1] != "caught KV pool exhausted"]
    assert leader and leader[0].startswith("lost after"), out
