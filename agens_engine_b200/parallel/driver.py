"""Rank 0 drives, the other ranks follow: every state-changing model call made on rank 0 is first announced to the
followers, which then make the same call, so that the scheduler (one thread on rank 0) can treat a tensor-parallel
model like a local one.

Reference: the leader/follower command interpreter of ``crates/agens-cli/src/tp.rs:190-298`` (re-exec per GPU, file
rendezvous).  Here ranks are ``torch.distributed`` processes; commands travel as pickled tuples over a gloo (CPU) group,
so that no GPU stream ever blocks on the host protocol; the data path stays in the fused kernels.
"""
from __future__ import annotations

import datetime
import os
import subprocess
import sys
from typing import List, Optional, Sequence

import torch
import torch.distributed as dist

_FORWARDED = ("new_seq", "free_seq", "reserve", "truncate", "fork", "forward_rows", "prefill",
              "decode_setup", "decode_steps", "set_linear_path", "recover", "save_session", "load_session",
              "enable_host_tier", "enable_step")


class FollowerLost(RuntimeError):
    """A follower rank is gone (its process ended, or it did not take a command within the control group's time-out).
    The leader cannot go on: the deployment ends with exit code 3, as the reference's leader does when a follower's
    pipe closes (crates/agens-cuda/src/lib.rs:310-322)."""
    fatal = True          # the serving loop stops instead of recovering


class TpDriver:
    """Wraps the rank-0 shard of a tensor-parallel model; attribute reads go to the shard, forwarded calls are
    broadcast first.  ``park``/``unpark`` keep every rank's KV shard on that rank's host (handles are integers)."""

    def __init__(self, model, ctrl_group, children: Optional[Sequence[subprocess.Popen]] = None):
        object.__setattr__(self, "_m", model)
        object.__setattr__(self, "_g", ctrl_group)
        object.__setattr__(self, "_parked", {})
        object.__setattr__(self, "_next", 0)
        object.__setattr__(self, "_children", list(children or ()))

    def _tell(self, cmd):
        """Announces a call to the followers.  A follower whose process has ended is noticed before the broadcast; one
        that stopped answering makes the broadcast run into the control group's time-out: both raise FollowerLost."""
        for c in self._children:
            if c.poll() is not None:
                raise FollowerLost(f"follower process {c.pid} ended with code {c.returncode}")
        try:
            _send(self._g, cmd)
        except FollowerLost:
            raise
        except Exception as e:          # gloo reports a closed connection or a time-out as a RuntimeError
            raise FollowerLost(f"control group: {e}") from e

    def __getattr__(self, name):
        attr = getattr(self._m, name)
        if name in _FORWARDED and callable(attr):
            def call(*a, **kw):
                self._tell((name, _plain(a), _plain(kw)))
                return attr(*a, **kw)
            return call
        return attr

    def __setattr__(self, name, value):
        setattr(self._m, name, value)

    def park(self, seq: int):
        h = self._next
        object.__setattr__(self, "_next", h + 1)
        self._tell(("park", (seq, h), {}))
        self._parked[h] = self._m.park(seq)
        return {"len": self._parked[h]["len"], "handle": h}

    def unpark(self, seq: int, blob):
        self._tell(("unpark", (seq, blob["handle"]), {}))
        self._m.unpark(seq, self._parked.pop(blob["handle"]))

    def shutdown(self):
        try:
            self._tell(("stop", (), {}))
        except FollowerLost:
            pass


def _plain(x):
    """Tensors travel device free: small ones as lists, larger ones (encoder rows of an image, position tables) as their
    raw bytes, which pickle and broadcast at memory speed."""
    if isinstance(x, torch.Tensor):
        t = x.detach().cpu().contiguous()
        if t.numel() <= 1024:
            return ("__tensor__", t.dtype, t.tolist())
        return ("__tensor_bytes__", t.dtype, tuple(t.shape), t.view(torch.uint8).numpy().tobytes())
    if isinstance(x, (list, tuple)):
        return type(x)(_plain(v) for v in x)
    if isinstance(x, dict):
        return {k: _plain(v) for k, v in x.items()}
    return x


def _revive(x):
    if isinstance(x, tuple) and len(x) == 3 and x[0] == "__tensor__":
        return torch.tensor(x[2], dtype=x[1])
    if isinstance(x, tuple) and len(x) == 4 and x[0] == "__tensor_bytes__":
        return torch.frombuffer(bytearray(x[3]), dtype=torch.uint8).view(x[1]).reshape(x[2])
    if isinstance(x, (list, tuple)):
        return type(x)(_revive(v) for v in x)
    if isinstance(x, dict):
        return {k: _revive(v) for k, v in x.items()}
    return x


def _send(group, cmd):
    dist.broadcast_object_list([cmd], src=0, group=group)


def follow(model, ctrl_group, log=None) -> int:
    """Follower loop: executes the leader's calls until it says stop.  Returns the number of calls made.

    The page pools and sequence tables are identical on every rank, so a call that fails with a RuntimeError on the
    leader (KV pool exhausted, context too long, a fork that finds no page) fails the same way here, before any kernel
    is launched: the leader's scheduler catches it and carries on (evicts, re-queues), and so does the follower.  Any
    other exception is a real fault of this rank: it is re-raised, the process ends, and the leader notices."""
    parked = {}
    n = 0
    while True:
        box = [None]
        dist.broadcast_object_list(box, src=0, group=ctrl_group)
        name, a, kw = box[0]
        if name == "stop":
            return n
        a, kw = _revive(a), _revive(kw)
        try:
            if name == "park":
                parked[a[1]] = model.park(a[0])
            elif name == "unpark":
                model.unpark(a[0], parked.pop(a[1]))
            else:
                getattr(model, name)(*a, **kw)
        except RuntimeError as e:
            if log is not None:
                log(f"follower: {name} raised {e} (the leader sees the same and recovers)")
        n += 1


def control_group(timeout_s: Optional[float] = None):
    """A gloo group over all ranks for host-side commands (the default group stays NCCL).  Its time-out bounds how long
    the leader waits for a follower that stopped answering (B200E_TP_TIMEOUT_S, default 120 s; the reference's
    rendezvous time-outs: crates/agens-cli/src/tp.rs:59-72)."""
    t = timeout_s if timeout_s is not None else float(os.environ.get("B200E_TP_TIMEOUT_S", "120"))
    return dist.new_group(backend="gloo", timeout=datetime.timedelta(seconds=t))


def launch(argv: Sequence[str], world: int, log_dir: str = ".", port: Optional[int] = None) -> List[subprocess.Popen]:
    """Starts ranks 1 .. world-1 of this program (same argv) and returns their handles; the caller becomes rank 0 by
    setting the same environment for itself (``rank_env(0, ...)``).  Logs go to ``tp_rank<r>.log``."""
    port = port or 29400 + os.getpid() % 500
    procs = []
    for r in range(1, world):
        env = dict(os.environ, **rank_env(r, world, port))
        log = open(os.path.join(log_dir, f"tp_rank{r}.log"), "w")
        procs.append(subprocess.Popen([sys.executable] + list(argv), env=env, stdout=log, stderr=subprocess.STDOUT))
    os.environ.update(rank_env(0, world, port))
    return procs


def rank_env(rank: int, world: int, port: int) -> dict:
    return {"RANK": str(rank), "LOCAL_RANK": str(rank), "WORLD_SIZE": str(world), "MASTER_ADDR": "127.0.0.1",
            "MASTER_PORT": str(port), "B200E_TP_CHILD": "1" if rank else "0"}
