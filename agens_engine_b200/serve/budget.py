"""Hard per-GPU memory budget: plan at load, size the KV pool from the plan, refuse what does not fit.

Reference behaviour (``crates/agens-cli/src/m1.rs:492-541`` ballast cap, ``:905-974`` plan at load and automatic
GPU-vs-host tier decision, ``plan.rs:182-241``, ``tp.rs:77-90`` minimum over ranks): the budget is a promise about the
device memory one engine process takes on a GPU.  The reference keeps the promise by allocating ballast (everything above
the budget) so that later allocations fail early; on a shared GPU that is not acceptable, so here the promise is kept
on the host:

* :class:`BudgetLedger` books every device allocation of the deployment (weights, KV pool, scratch, peer regions)
  against the budget and raises :class:`BudgetExceeded` before the allocation is made;
* the PyTorch caching allocator of the process is capped at the same number of bytes
  (``torch.cuda.set_per_process_memory_fraction``), so an allocation that was not booked cannot pass the budget either;
* :func:`plan_deployment` runs the planner (``csrc/sched/planner.cpp``) on the architecture and the budget and turns
  its answer into constructor arguments of the model: pages of the KV pool, the context that fits, whether the host
  tier is on and how many pages stay resident.  Under tensor parallelism every rank plans and the minimum is taken.
"""
from __future__ import annotations

import dataclasses
from typing import Callable, Dict, List, Optional

GiB = 1024 ** 3


class BudgetExceeded(RuntimeError):
    pass


class BudgetLedger:
    """Books allocations against a byte budget.  ``budget_bytes <= 0`` means unlimited (everything is still booked,
    so that the report shows where the memory went)."""

    def __init__(self, budget_bytes: int = 0):
        self.budget = int(budget_bytes)
        self.items: Dict[str, int] = {}

    @property
    def used(self) -> int:
        return sum(self.items.values())

    def free(self) -> int:
        return (self.budget - self.used) if self.budget > 0 else 1 << 62

    def book(self, name: str, nbytes: int) -> int:
        nbytes = int(nbytes)
        if self.budget > 0 and self.used + nbytes > self.budget:
            raise BudgetExceeded(f"{name}: {nbytes / GiB:.3f} GiB does not fit: {self.used / GiB:.3f} of {self.budget / GiB:.3f} GiB "
                                 f"are taken ({', '.join(f'{k} {v / GiB:.2f}' for k, v in self.items.items())})")
        self.items[name] = self.items.get(name, 0) + nbytes
        return nbytes

    def release(self, name: str, nbytes: Optional[int] = None):
        cur = self.items.get(name, 0)
        left = 0 if nbytes is None else max(0, cur - int(nbytes))
        if left:
            self.items[name] = left
        else:
            self.items.pop(name, None)

    def alloc(self, name: str, nbytes: int, allocate: Callable[[], object]):
        """Books ``nbytes`` and then calls ``allocate``; the booking is undone when the allocation fails."""
        self.book(name, nbytes)
        try:
            return allocate()
        except Exception:
            self.release(name, nbytes)
            raise

    def report(self) -> List[str]:
        lines = [f"budget: {k}: {v / GiB:.3f} GiB" for k, v in self.items.items()]
        cap = f" of {self.budget / GiB:.2f} GiB" if self.budget > 0 else " (no cap)"
        return lines + [f"budget: total {self.used / GiB:.3f} GiB{cap}"]


@dataclasses.dataclass
class Deployment:
    """What the planner decided for one rank."""
    budget_bytes: int
    n_pages: int               # pages of the GPU KV pool
    max_ctx: int               # context per conversation that the pool (plus the host tier) can hold
    host_tier: bool
    resident_window_tokens: int
    host_pages: int
    fits: bool
    lines: List[str]
    plan: dict


def plan_deployment(cfg, budget_gib: float, wctx: int, max_batch: int, sessions: int, prefill_chunk: int, tp: int = 1,
                    gpu_free_gib: Optional[float] = None, host_avail_gib: float = -1.0, allow_host_tier: bool = True,
                    weights_bytes: Optional[int] = None, dual_layout: bool = False, split_keys: int = 64) -> Deployment:
    """Runs the planner for one rank of a ``tp``-way deployment of the architecture ``cfg`` (the full model's config).
    ``weights_bytes``: measured bytes when the weights are already on the device, else the architecture's estimate
    plus 0.6 GiB of CUDA context; ``dual_layout`` doubles the quantised linears (the step kernel's second layout)."""
    from . import host as H
    if weights_bytes is None:
        lin = cfg.weight_bytes(tp) - cfg.vocab * cfg.d_model * 2
        weights_bytes = cfg.weight_bytes(tp) + (lin if dual_layout else 0) + int(0.6 * GiB)
    p = H.plan(budget_gib=float(budget_gib), gpu_free_gib=float(gpu_free_gib if gpu_free_gib is not None else 170.0),
               weights_bytes=int(weights_bytes), kv_bytes_per_token=int(cfg.kv_bytes_per_token(tp)), page_size=cfg.page_size,
               max_batch=int(max_batch), sessions=int(sessions), prefill_chunk=int(prefill_chunk), d_model=cfg.d_model, ffn=cfg.ffn,
               q_dim=cfg.q_dim, kv_dim=cfg.kv_dim, vocab=cfg.vocab, n_heads=cfg.n_heads, head_dim=cfg.head_dim, tp=int(tp),
               wctx=int(wctx), host_avail_gib=float(host_avail_gib), allow_host_tier=bool(allow_host_tier),
               split_keys=int(split_keys))
    if "error" in p:
        raise ValueError(p["error"])
    ps = cfg.page_size
    want_pages = (wctx + ps - 1) // ps
    # the pool never needs more than every slot at full context; what the plan grants beyond that stays free
    n_pages = int(min(p["pool_pages"], want_pages * max(1, max_batch)))
    max_ctx = int(min(p["context"], wctx))
    host = p["tier"] == "host"
    window = int(p["resident_window_pages"]) * ps
    return Deployment(budget_bytes=int(p["budget_bytes"]), n_pages=n_pages, max_ctx=max_ctx, host_tier=host,
                      resident_window_tokens=window, host_pages=int(p["host_pages"]), fits=bool(p["fits"]), lines=list(p["lines"]),
                      plan=p)


def agree_min(dep: Deployment, all_reduce_min: Callable[[List[int]], List[int]]) -> Deployment:
    """Every rank ends up with the smallest pool and context any rank planned (reference: tp.rs:77-90 agree_min).
    ``all_reduce_min`` maps a list of ints to the element-wise minimum over the ranks."""
    n_pages, max_ctx, window, fits = all_reduce_min([dep.n_pages, dep.max_ctx, dep.resident_window_tokens, int(dep.fits)])
    host = bool(all_reduce_min([0 if dep.host_tier else 1])[0] == 0)       # the tier is on when any rank needs it
    return dataclasses.replace(dep, n_pages=int(n_pages), max_ctx=int(max_ctx), resident_window_tokens=int(window),
                               fits=bool(fits), host_tier=host)


def cap_process(budget_bytes: int, device) -> Optional[float]:
    """Caps the PyTorch caching allocator of this process at ``budget_bytes`` on ``device`` (no ballast: memory above
    the cap simply cannot be obtained through the allocator).  Returns the fraction that was set."""
    import torch
    if budget_bytes <= 0 or not torch.cuda.is_available():
        return None
    total = torch.cuda.get_device_properties(device).total_memory
    frac = min(1.0, budget_bytes / total)
    torch.cuda.set_per_process_memory_fraction(frac, device)
    return frac
