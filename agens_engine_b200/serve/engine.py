"""Continuous-batching engine loop: admits requests against the KV pool, interleaves prefill chunks with batched decode
(or speculative verify) steps, samples on the device, applies reasoning budget / think guard, and streams tokens to
whoever submitted the request.

Plays the role of the reference's continuous loop (``crates/agens-cli/src/serve.rs:1028-1700`` ``run_loop``): admission by the
banker's check (``kv_safe``), shortest-remaining-prefill first with a fairness turn (``pick_prefill``), eviction of the
cheapest victim when the pool runs dry (``pick_victim``; the victim is re-queued and recomputed), one rule for sampling
so that speculation does not change tokens.  The loop itself is a thread of this process; the model calls go to the
GPU through the engine's kernels.
"""
from __future__ import annotations

import dataclasses
import queue
import threading
import time
from typing import Callable, Dict, List, Optional, Sequence

import torch

from ..models.dense import DenseModel, M_ROWS
from ..ops import basic
from ..spec import DraftSource, SamplingState, SpecDecoder
from . import host

WAITING, PREFILL, DECODE, DONE = range(4)


@dataclasses.dataclass
class Request:
    rid: int
    prompt: List[int]
    sampling: dict
    session: str = ""
    state: int = WAITING
    slot: int = -1
    done_prompt: int = 0                  # prompt tokens already prefilled
    out: List[int] = dataclasses.field(default_factory=list)
    t_submit: float = 0.0
    t_last: float = 0.0
    chunk_index: int = 0
    budget: Optional[host.ReasoningBudget] = None
    guard: Optional[host.ThinkGuard] = None
    evictions: int = 0
    parked: Optional[dict] = None         # KV rows in pinned host memory while preempted
    parked_hist: Optional[List[int]] = None
    images: Optional[List[str]] = None    # data: URLs of the request's image parts, in prompt order
    mm: Optional[dict] = None             # serve.vision.VisionFrontEnd.prepare(): encoder rows, positions
    mtp_sinks: Optional[list] = None      # per-chunk feeders of the MTP heads while the prompt prefills
    pen_state: Optional[dict] = None      # device-side token counts of a request with penalties (_edit_logits)

    @property
    def max_new(self) -> int:
        return int(self.sampling.get("max_new_tokens", 256))

    def state_of_sampling(self) -> SamplingState:
        s = self.sampling
        t = float(s.get("temperature", 0.0))
        k = int(s.get("top_k", 0) or 0)
        if k == 1:
            t = 0.0
        return SamplingState(temperature=t, top_k=max(k, 0), top_p=float(s.get("top_p", 1.0)), min_p=float(s.get("min_p", 0.0)),
                             seed=int(s.get("seed", self.rid * 0x9E3779B97F4A7C15 + 1)) & 0x7FFFFFFFFFFFFFFF)

    def needs_logit_edits(self) -> bool:
        s = self.sampling
        return bool(s.get("logit_bias")) or float(s.get("presence_penalty", 0)) != 0 or float(s.get("frequency_penalty", 0)) != 0 \
            or float(s.get("repetition_penalty", 1)) != 1


@dataclasses.dataclass
class EngineStats:
    steps: int = 0
    prefill_chunks: int = 0
    tokens_out: int = 0
    tokens_prefilled: int = 0
    tokens_reused: int = 0
    evictions: int = 0
    rejected: int = 0
    peak_batch: int = 0
    images_encoded: int = 0
    device_errors: int = 0
    # step timing (host clock around a scheduler iteration that did work, device included: every step ends with a
    # read of its tokens), as the reference's per-step statistics (crates/agens-cli/src/serve.rs:149-166)
    last_step_ms: float = 0.0
    decode_ms_sum: float = 0.0
    prefill_ms_sum: float = 0.0
    rows_sum: int = 0

    def prometheus(self, model=None) -> str:
        g = [("b200e_scheduler_steps_total", self.steps), ("b200e_prefill_chunks_total", self.prefill_chunks),
             ("b200e_tokens_prefilled_total", self.tokens_prefilled), ("b200e_tokens_reused_total", self.tokens_reused),
             ("b200e_evictions_total", self.evictions), ("b200e_rejected_total", self.rejected),
             ("b200e_device_errors_total", self.device_errors), ("b200e_peak_batch", self.peak_batch),
             ("b200e_last_step_ms", round(self.last_step_ms, 3)),
             ("b200e_decode_step_ms_avg", round(self.decode_ms_sum / max(self.steps, 1), 3)),
             ("b200e_prefill_chunk_ms_avg", round(self.prefill_ms_sum / max(self.prefill_chunks, 1), 3)),
             ("b200e_rows_per_step_avg", round(self.rows_sum / max(self.steps, 1), 2))]
        if model is not None:
            g.append(("b200e_kv_pages_free", model.free_pages()))
        return "".join(f"{k} {v}\n" for k, v in g)


class Engine:
    """``emit(rid, tokens, finished, error)`` is called from the engine thread with every batch of new tokens; it
    returns True when the receiver is gone (the request is dropped)."""

    def __init__(self, model: DenseModel, emit: Callable[[int, List[int], bool, Optional[str]], bool],
                 sources_factory: Optional[Callable[[], Sequence[DraftSource]]] = None, max_drafts: int = 0,
                 max_batch: Optional[int] = None, think_tokens: Optional[tuple] = None, reserve_ahead: int = 16,
                 keep_sequences: bool = False, prefix_chunk: int = 64, prefix_budget_bytes: int = 1 << 40,
                 invariant: bool = True, vision=None):
        self.m, self.emit = model, emit
        self.vision = vision                           # serve.vision.VisionFrontEnd, or None: requests with images fail
        self.max_batch = min(max_batch or model.max_seqs, model.max_seqs, M_ROWS // 2)
        self.max_rows = min(M_ROWS, getattr(model, "max_rows", M_ROWS))
        self.max_drafts = max_drafts
        if invariant:
            # batch-invariant serving (the reference's server mode): every step uses the same linear kernel whatever the
            # number of rows, so a request's tokens do not depend on what else is running
            rows_cap = self.max_batch * (1 + max_drafts)
            can_step = getattr(model, "step_mode", "off") != "off" and getattr(model, "_step_possible", lambda: False)()
            step_rows = 16 if can_step else 0
            model.set_linear_path(None if rows_cap <= max(8, step_rows) else 1)
            if rows_cap <= step_rows:
                # up to sixteen rows per step: ONE kernel family for every step is the persistent step kernel (on the
                # 32B model 2.7 times the per-op path at eight rows, 1.4 times at sixteen, 0.8 times at one row); beyond
                # eight rows every step uses the work split of the large steps, so that a row's bits do not depend on
                # how many rows share its step
                model.enable_step("on", uniform=rows_cap > 8)
        self.spec = SpecDecoder(model, list(sources_factory()) if sources_factory else [], max_drafts=max_drafts)
        self.think = think_tokens                      # (start id, end id) for budget / guard
        self.reserve_ahead = reserve_ahead
        self.inbox: "queue.Queue[Request]" = queue.Queue()
        self.waiting: List[Request] = []
        self.active: Dict[int, Request] = {}           # slot -> request
        self.free_slots = list(range(model.max_seqs - 1, -1, -1))
        self.stats = EngineStats()
        self.on_stats: Optional[Callable[[EngineStats], None]] = None      # called every few steps (metrics export)
        import os as _os
        w = _os.environ.get("B200E_PROFILE_STEPS", "")
        self._prof = tuple(int(x) for x in w.split(":")) if w.count(":") == 1 and all(x.isdigit() for x in w.split(":")) else None
        self._prof_on = False
        self._stop = threading.Event()
        self.fatal: Optional[BaseException] = None      # set when the loop had to stop for good
        self._thread: Optional[threading.Thread] = None
        self._rid = 0
        self._lock = threading.Lock()
        # Finished sequences stay resident (or parked on the host) so that the next turn of a conversation, or another
        # request with the same prompt prefix, skips the prefill of what is already in the KV cache.
        self.keep_sequences = keep_sequences
        self.kept: Dict[int, dict] = {}                # handle -> {slot | parked, tokens, session, t_last}
        self.by_session: Dict[str, int] = {}
        self._next_handle = 1
        self._prefix_budget = prefix_budget_bytes
        self.prefix = host.PrefixCache(prefix_budget_bytes, prefix_chunk) if keep_sequences else None
        self.prefix_chunk = prefix_chunk

    # ------------------------------------------------------------------------------------------------ submission
    def submit(self, prompt: Sequence[int], sampling: Optional[dict] = None, rid: Optional[int] = None, session: str = "",
               images: Optional[Sequence[str]] = None) -> int:
        """``images``: one ``data:`` URL per image placeholder of the prompt (one placeholder token each, expanded here)."""
        with self._lock:
            if rid is None:
                self._rid += 1
                rid = self._rid
        r = Request(rid, list(prompt), dict(sampling or {}), session, t_submit=time.monotonic(),
                    images=list(images) if images else None)
        self.inbox.put(r)
        return rid

    def start(self):
        self._thread = threading.Thread(target=self.run, name="engine", daemon=True)
        self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread:
            self._thread.join(timeout=30)

    def run(self):
        if self.m.dev.type == "cuda":
            torch.cuda.set_device(self.m.dev)
        while not self._stop.is_set():
            try:
                if not self.step():
                    try:
                        self._intake(self.inbox.get(timeout=0.02))
                    except queue.Empty:
                        pass
            except Exception as e:      # a failed step must not take the engine thread (and every open request) with it
                if getattr(e, "fatal", False):          # e.g. a tensor-parallel follower is gone: nothing to recover to
                    self.fatal = e
                    for r in list(self.active.values()) + list(self.waiting):
                        self.emit(r.rid, [], True, f"engine stopped: {e}")
                    self.active.clear(); self.waiting.clear()
                    return
                self._fail_all(f"engine step failed: {type(e).__name__}: {e}")

    def _intake(self, r: Request):
        """Every request enters through here, whichever wait delivered it: images are decoded and encoded first."""
        if r.images and not self._prepare_images(r):
            return
        self.waiting.append(r)

    def _fail_all(self, why: str):
        """Ends every running request with an error and puts the model back into a usable state (device status words
        cleared, sequences dropped, collective inboxes re-armed; under tensor parallelism the followers do the same)."""
        for r in list(self.active.values()):
            try:
                self.emit(r.rid, [], True, why)
            except Exception:
                pass
            r.state = DONE
        self.active.clear()
        self.spec.hist.clear(); self.spec.samp.clear()
        for src in self.spec.sources:
            reset = getattr(src, "reset", None)
            if reset:
                reset()
        self.kept.clear(); self.by_session.clear()
        if self.prefix is not None:
            self.prefix = host.PrefixCache(self._prefix_budget, self.prefix_chunk)
        try:
            self.m.recover()
        except Exception:
            pass
        self.free_slots = list(range(self.m.max_seqs - 1, -1, -1))
        self.stats.device_errors += 1

    def _check_device(self) -> bool:
        """Reads the device status words once per step (one small copy); a bounded wait that ran out or a bounds check
        that fired means this step's tokens cannot be trusted: nothing of it is delivered."""
        st = self.m.device_status()
        if st == 0:
            return True
        from .._lib import STATUS_NAMES
        self._fail_all(f"device reported: {STATUS_NAMES.get(st, st)}")
        return False

    def idle(self) -> bool:
        return not self.waiting and not self.active and self.inbox.empty()

    def run_until_idle(self, max_steps: int = 1 << 30):
        n = 0
        while not self.idle() and n < max_steps:
            self.step(); n += 1

    # ------------------------------------------------------------------------------------------------ one iteration
    def step(self) -> bool:
        """One scheduler iteration; returns False when there was nothing to do."""
        while True:
            try:
                r = self.inbox.get_nowait()
            except queue.Empty:
                break
            self._intake(r)
        self._admit()
        did = False
        self._profile_window()
        pre = [r for r in self.active.values() if r.state == PREFILL]
        if pre:
            t0 = time.perf_counter()
            torch.cuda.nvtx.range_push("prefill chunk")
            try:
                self._prefill_one(pre)
            finally:
                torch.cuda.nvtx.range_pop()
            self.stats.last_step_ms = (time.perf_counter() - t0) * 1e3
            self.stats.prefill_ms_sum += self.stats.last_step_ms
            did = True
        dec = [r for r in self.active.values() if r.state == DECODE]
        if dec:
            t0 = time.perf_counter()
            torch.cuda.nvtx.range_push(f"decode step ({len(dec)} sequences)")
            steps0 = self.stats.steps
            try:
                self._decode(dec)
            finally:
                torch.cuda.nvtx.range_pop()
            self.stats.last_step_ms = (time.perf_counter() - t0) * 1e3
            if self.stats.steps > steps0:
                self.stats.decode_ms_sum += self.stats.last_step_ms
                self.stats.rows_sum += len(dec)
            did = True
        if did and self.on_stats is not None and (self.stats.steps + self.stats.prefill_chunks) % 16 == 0:
            self.on_stats(self.stats)
        return did

    def _profile_window(self):
        """B200E_PROFILE_STEPS=a:b opens a profiler capture range at scheduler step a and closes it at step b, so that a
        profiler started with capture-range control records exactly those steps (reference: the profiler window of
        kernels/m1/m1_model.cu:3872-3873)."""
        if self._prof is None:
            return
        a, b = self._prof
        n = self.stats.steps
        if not self._prof_on and a <= n < b:
            torch.cuda.synchronize(self.m.dev)
            torch.cuda.cudart().cudaProfilerStart()
            self._prof_on = True
        elif self._prof_on and n >= b:
            torch.cuda.synchronize(self.m.dev)
            torch.cuda.cudart().cudaProfilerStop()
            self._prof_on, self._prof = False, None

    def _prepare_images(self, r: Request) -> bool:
        """Decodes and encodes the request's images on this (the engine's) thread and expands the prompt."""
        try:
            if self.vision is None:
                raise ValueError("this model does not accept images")
            r.mm = self.vision.prepare(r.prompt, r.images)
        except Exception as e:                            # untrusted bytes: whatever goes wrong ends this request only
            self.stats.rejected += 1
            self.emit(r.rid, [], True, f"image input: {e}")
            return False
        r.prompt = list(r.mm["ids"])
        self.stats.images_encoded += len(r.images)
        return True

    # ---- admission -----------------------------------------------------------------------------------------------
    def _pages(self, n_tokens: int) -> int:
        ps = self.m.cfg.page_size
        return (n_tokens + ps - 1) // ps

    def _demand(self, r: Request) -> tuple:
        """(pages it may still take, pages it holds) for the banker's check."""
        total = self._pages(min(len(r.prompt) + r.max_new + self.max_drafts + 1, self.m.max_ctx))
        if r.slot < 0 and r.parked is not None:          # needs its parked rows back at once
            return total, 0
        held = len(self.m.seq_pages.get(r.slot, ())) if r.slot >= 0 else 0
        return max(total - held, 0), held

    def _admit(self):
        keep: List[Request] = []
        for r in self.waiting:
            if len(r.prompt) + 1 > self.m.max_ctx or not r.prompt:
                self.stats.rejected += 1
                self.emit(r.rid, [], True, "prompt does not fit the context window" if r.prompt else "empty prompt")
                continue
            if len(self.active) >= self.max_batch or (not self.free_slots and not self._drop_kept(exclude_session=r.session)):
                keep.append(r); continue
            items = [self._demand(a) for a in self.active.values()] + [self._demand(r)]
            while self.kept and (not host.kv_safe(self.m.free_pages(), items) or self._pages(len(r.prompt) + 1) > self.m.free_pages()):
                if not self._drop_kept(exclude_session=r.session):
                    break
            if self.active and not host.kv_safe(self.m.free_pages(), items):
                keep.append(r); continue
            if not self.active and self._pages(len(r.prompt) + len(r.out) + 1) > self.m.free_pages():
                self.stats.rejected += 1
                self.emit(r.rid, [], True, "prompt does not fit the KV pool")
                continue
            if r.parked is not None and self._pages(int(r.parked["len"]) + 1 + self.max_drafts) > self.m.free_pages():
                keep.append(r); continue
            r.slot = self.free_slots.pop()
            self.spec.samp[r.slot] = r.state_of_sampling()
            if r.parked is not None:                     # preempted earlier: bring its KV rows back and go on decoding
                try:
                    self.m.unpark(r.slot, r.parked)
                except RuntimeError as e:                     # no room after all: give the slot back and wait in line
                    if getattr(e, "fatal", False):         # nothing to recover to (a follower is gone): the run loop ends
                        raise
                    if r.slot in self.m.seq_pages:
                        self.m.free_seq(r.slot)
                    self.spec.samp.pop(r.slot, None)
                    self.free_slots.append(r.slot)
                    r.slot = -1
                    keep.append(r); continue
                self.spec.hist[r.slot] = r.parked_hist
                for s in self.spec.sources:
                    s.begin(r.slot, r.parked_hist)
                r.parked = r.parked_hist = None
                r.state = DECODE
                self.active[r.slot] = r
                continue
            r.state, r.done_prompt, r.chunk_index = PREFILL, 0, 0
            if r.mm is not None or not self._reuse_kept(r):      # image rows are not in the token-keyed prefix cache
                self.m.new_seq(r.slot)
            if self.think and r.sampling.get("reasoning_budget") is not None:
                r.budget = host.ReasoningBudget(int(r.sampling["reasoning_budget"]), float(r.sampling.get("reasoning_soft", 0.0)),
                                                r.prompt, self.think[0], self.think[1])
            if self.think and r.sampling.get("think_guard"):
                g = r.sampling["think_guard"]
                r.guard = host.ThinkGuard(int(g.get("n", 64)), int(g.get("k", 4)), int(g.get("w", 2048)), r.prompt, self.think[0],
                                          self.think[1])
            self.active[r.slot] = r
            self.stats.peak_batch = max(self.stats.peak_batch, len(self.active))
        self.waiting = keep

    # ---- kept sequences: conversations and prompt-prefix reuse ------------------------------------------------------
    def _keep(self, r: Request):
        """The finished request's sequence stays in its slot, findable by session id and by token prefix."""
        n = self.m.seq_len_host[r.slot]
        toks = (r.prompt + r.out)[:n]
        h = self._next_handle
        self._next_handle += 1
        if r.session and r.session in self.by_session:
            self._forget(self.by_session[r.session])
        self.kept[h] = {"slot": r.slot, "parked": None, "tokens": toks, "session": r.session, "t_last": time.monotonic()}
        if r.session:
            self.by_session[r.session] = h
        # one entry per chunk boundary (the cache matches whole chunks); the bytes are booked on the longest one
        # (one pass over the tokens: hashing every prefix from its start cost 18 s for a 128K-token conversation)
        _, evicted = self.prefix.insert_chain(toks, h, self.m.cfg.kv_bytes_per_token() * n)
        for e in evicted:
            if e != h:
                self._forget(e)

    def _forget(self, h: int):
        k = self.kept.pop(h, None)
        if k is None:
            return
        if k["session"] and self.by_session.get(k["session"]) == h:
            self.by_session.pop(k["session"])
        if k["slot"] is not None:
            self.m.free_seq(k["slot"])
            self.free_slots.append(k["slot"])

    def _drop_kept(self, exclude_session: str = "") -> bool:
        """Gives up the least recently used kept sequence: one that belongs to a conversation is parked on the host
        (its slot and pages are freed, the next turn brings it back), an anonymous one is dropped.  Snapshots go before
        conversations, as in the reference's eviction order (serve.rs:616-639)."""
        cands = [(0 if not k["session"] else 1, h, time.monotonic() - k["t_last"], 0) for h, k in self.kept.items()
                 if k["slot"] is not None and not (exclude_session and k["session"] == exclude_session)]
        if not cands:
            return False
        i = host.pick_victim(cands, hold_s=0.0, allow_protected=True)
        if i < 0:
            return False
        h = cands[i][1]
        k = self.kept[h]
        if k["session"]:
            k["parked"] = self.m.park(k["slot"])
            self.free_slots.append(k["slot"])
            k["slot"] = None
        else:
            self._forget(h)
        return True

    def _reuse_kept(self, r: Request) -> bool:
        """Starts ``r`` from a kept sequence when one shares a long enough token prefix: the conversation's own
        sequence is taken over, any other match is forked (full pages shared, copy-on-write by construction: the
        child is cut at a page boundary).  Returns True when the slot now holds a sequence."""
        if not self.keep_sequences:
            return False
        page = self.m.cfg.page_size
        limit = len(r.prompt) - 1                                     # the last prompt token must be fed to get logits
        h = self.by_session.get(r.session) if r.session else None
        if h is not None:
            k = self.kept[h]
            n = 0
            for a, b in zip(k["tokens"], r.prompt[:limit]):
                if a != b:
                    break
                n += 1
            n = n // page * page
            if n >= page:
                self.kept.pop(h); self.by_session.pop(r.session)
                if k["slot"] is None:
                    try:
                        self.m.unpark(r.slot, k["parked"])
                    except RuntimeError as e:                               # pool exhausted: start this turn from scratch
                        if getattr(e, "fatal", False):         # nothing to recover to (a follower is gone): the run loop ends
                            raise
                        if r.slot in self.m.seq_pages:
                            self.m.free_seq(r.slot)
                        return False
                else:                                                  # the request moves into the kept sequence's slot
                    self.spec.samp.pop(r.slot, None)
                    self.free_slots.append(r.slot)
                    r.slot = k["slot"]
                    self.spec.samp[r.slot] = r.state_of_sampling()
                self.m.truncate(r.slot, n)
                r.done_prompt = n
                self.stats.tokens_reused += n
                return True
        n, h = self.prefix.lookup(r.prompt[:limit])
        k = self.kept.get(h) if n >= self.prefix_chunk else None
        if k is None or k["slot"] is None:
            return False
        n = min(n, len(k["tokens"])) // page * page
        try:
            self.m.fork(k["slot"], r.slot)
        except RuntimeError as e:
            if getattr(e, "fatal", False):         # nothing to recover to (a follower is gone): the run loop ends
                raise
            return False
        self.m.truncate(r.slot, n)
        k["t_last"] = time.monotonic()
        r.done_prompt = n
        self.stats.tokens_reused += n
        return True

    # ---- eviction ------------------------------------------------------------------------------------------------
    def _evict_for(self, needy: Request) -> bool:
        """Preempts the most recently submitted other sequence and re-queues it at the head of the line (a decoding
        victim's KV rows wait in pinned host memory and come back bit for bit; a prefilling victim starts over).  False
        if nobody can go."""
        if self._drop_kept():
            return True
        others = [r for r in self.active.values() if r is not needy]
        if not others:
            return False
        v = max(others, key=lambda r: (r.t_submit, r.rid))      # last admitted goes first: the least work is lost
        v.parked = self.m.park(v.slot) if v.state == DECODE else None      # bit-exact resume; a prefilling victim restarts
        v.parked_hist = self.spec.hist.get(v.slot)
        self._release(v, keep_kv=v.parked is not None)
        v.state, v.slot = WAITING, -1
        if v.parked is None:
            v.done_prompt = 0
            v.mtp_sinks = None
        v.evictions += 1
        self.stats.evictions += 1
        self.waiting.insert(0, v)
        return True

    def _release(self, r: Request, keep_kv: bool = False):
        if r.state == DECODE:
            for s in self.spec.sources:
                s.end(r.slot)
        self.spec.hist.pop(r.slot, None)
        self.spec.samp.pop(r.slot, None)
        if not keep_kv:                                  # park() has already given the slot's pages back
            self.m.free_seq(r.slot)
        self.active.pop(r.slot)
        self.free_slots.append(r.slot)

    def _with_room(self, r: Request, fn):
        """Runs ``fn`` and, when the KV pool is exhausted, evicts a victim and retries."""
        while True:
            try:
                return fn()
            except RuntimeError as e:
                if "KV pool exhausted" not in str(e) or not self._evict_for(r):
                    raise

    # ---- prefill -------------------------------------------------------------------------------------------------
    def _prefill_one(self, pre: List[Request]):
        now = time.monotonic()
        i = host.pick_prefill([len(r.prompt) - r.done_prompt for r in pre], [now - r.t_submit for r in pre],
                              self.stats.prefill_chunks)
        r = pre[i if 0 <= i < len(pre) else 0]
        n = min(self.m.prefill_chunk, len(r.prompt) - r.done_prompt)
        if r.mm is not None:
            n = len(r.prompt)                             # the model chunks a prompt with images itself
        chunk = torch.tensor(r.prompt[r.done_prompt:r.done_prompt + n], dtype=torch.int32)
        final = r.done_prompt + n == len(r.prompt)
        sampled = self.spec.samp[r.slot].temperature > 0 or r.needs_logit_edits()
        kw = {}
        if r.mm is not None:
            kw = dict(image_rows=r.mm["rows"], image_pad_id=r.mm["pad_id"], rope_pos3=r.mm["pos3"], pair_axis=r.mm["pair_axis"],
                      rope_next=r.mm["rope_next"])
        # MTP heads get context entries for the prompt positions from the hidden rows of every chunk (single-GPU
        # models; the sink is made at the request's first chunk and covers the positions a prefix cache did not supply)
        mtp = self.spec._mtp if self.spec.mtp_prompt and hasattr(self.m, "hidden_sink") and r.mm is None else []
        if mtp and len(r.prompt) - r.done_prompt > 1 and r.mtp_sinks is None:
            r.mtp_sinks = [s.prefill_sink(r.slot, r.prompt, start=r.done_prompt) for s in mtp]
        sinks = r.mtp_sinks
        if sinks:
            self.m.hidden_sink = lambda pos0, hid: [f(pos0, hid) for f in sinks]
        try:
            res = self._with_room(r, lambda: self.m.prefill(r.slot, chunk, want_logits=final and sampled, **kw))
        except RuntimeError as e:
            if getattr(e, "fatal", False):         # nothing to recover to (a follower is gone): the run loop ends
                raise
            r.mtp_sinks = None
            self._finish(r, error=str(e)); return
        finally:
            if sinks:
                self.m.hidden_sink = None
        if final and not self._check_device():
            return
        r.done_prompt += n
        r.chunk_index += 1
        self.stats.prefill_chunks += 1
        self.stats.tokens_prefilled += n
        if not final:
            return
        tok, logits = res
        if sampled:
            logits = logits[None, :]
            self._edit_logits(logits, [r])
            tok = int(self.spec._sample(logits, [r.slot], [len(r.prompt)])[0])
        self.spec.hist[r.slot] = list(r.prompt) + [tok]
        for s in self.spec.sources:
            s.begin(r.slot, self.spec.hist[r.slot])
        r.mtp_sinks = None
        r.state = DECODE
        self._deliver(r, [tok])

    # ---- decode --------------------------------------------------------------------------------------------------
    def _edit_logits(self, logits: torch.Tensor, rows: List[Request]):
        """Penalties and logit bias, applied in place on the device rows (reference: sampler.rs penalties).  Every
        request with penalties keeps its token counts on the device (how often each id was generated, which ids occur in
        prompt or output); a step uploads only the tokens generated since the last one and edits the row with whole-row
        vector operations."""
        for i, r in enumerate(rows):
            if not r.needs_logit_edits():
                continue
            s = r.sampling
            rep = float(s.get("repetition_penalty", 1))
            pres, freq = float(s.get("presence_penalty", 0)), float(s.get("frequency_penalty", 0))
            row = logits[i]
            if rep != 1 or pres != 0 or freq != 0:
                st = r.pen_state
                if st is None or st["cnt"].device != row.device or st["cnt"].numel() != row.numel():
                    st = r.pen_state = {"cnt": torch.zeros(row.numel(), dtype=torch.int32, device=row.device), "n": 0, "seen": None}
                    if rep != 1:
                        st["seen"] = torch.zeros(row.numel(), dtype=torch.bool, device=row.device)
                        if r.prompt:
                            st["seen"][torch.tensor(r.prompt, dtype=torch.long, device=row.device).clamp_(0, row.numel() - 1)] = True
                new = r.out[st["n"]:]
                if new:
                    t = torch.tensor(new, dtype=torch.long, device=row.device).clamp_(0, row.numel() - 1)
                    st["cnt"].index_add_(0, t, torch.ones_like(t, dtype=torch.int32))
                    if st["seen"] is not None:
                        st["seen"][t] = True
                    st["n"] = len(r.out)
                if rep != 1:
                    row.copy_(torch.where(st["seen"], torch.where(row > 0, row / rep, row * rep), row))
                if pres != 0 or freq != 0:
                    cnt = st["cnt"]
                    row.sub_(torch.where(cnt > 0, pres + freq * cnt.float(), torch.zeros_like(row)))
            for k, v in (s.get("logit_bias") or {}).items():
                if 0 <= int(k) < logits.shape[1]:
                    logits[i, int(k)] += float(v)

    def _decode(self, dec: List[Request]):
        dec = dec[:self.max_batch]
        plain = [r for r in dec if r.needs_logit_edits() or r.budget is not None]
        if plain:
            self._decode_plain(plain)
        fast = [r for r in dec if r not in plain and r.state == DECODE]
        if not fast:
            return
        # verify rows of all sequences must fit one launch
        per = max(1, min(1 + self.max_drafts, self.max_rows // len(fast)))
        self.spec.max_drafts = per - 1
        slots = [r.slot for r in fast]
        try:
            res = self._with_room(fast[0], lambda: self.spec.step([s for s in slots if s in self.active and self.active[s].state == DECODE]))
        except RuntimeError as e:
            if getattr(e, "fatal", False):         # nothing to recover to (a follower is gone): the run loop ends
                raise
            for r in fast:
                self._finish(r, error=str(e))
            return
        if not self._check_device():
            return
        self.stats.steps += 1
        for r in fast:
            if r.slot in res and self.active.get(r.slot) is r and r.state == DECODE:
                self._deliver(r, res[r.slot])

    def _decode_plain(self, rows: List[Request]):
        """One token per sequence with logit edits / forced tokens (no speculation: the edits depend on every token)."""
        m = self.m
        live: List[Request] = []

        def run():
            # an eviction between two attempts may have parked one of the rows: ask only for those still decoding
            live[:] = [r for r in rows if self.active.get(r.slot) is r and r.state == DECODE]
            if not live:
                return None, None
            return m.forward_rows([self.spec.hist[r.slot][-1] for r in live], [r.slot for r in live], want_logits=True)

        try:
            _, logits = self._with_room(rows[0], run)
        except RuntimeError as e:
            if getattr(e, "fatal", False):         # nothing to recover to (a follower is gone): the run loop ends
                raise
            for r in rows:
                if self.active.get(r.slot) is r:
                    self._finish(r, error=str(e))
            return
        rows = list(live)
        if not rows or not self._check_device():
            return
        slots = [r.slot for r in rows]
        pos = [m.seq_len_host[s] for s in slots]
        self._edit_logits(logits, rows)
        forced: Dict[int, int] = {}
        for i, r in enumerate(rows):
            if r.budget is not None:
                act = r.budget.act(len(r.out))
                if act[0] == "force":
                    forced[i] = act[1]
                elif act[0] == "bias":
                    logits[i, act[1]] += act[2]
        toks = self.spec._sample(logits, slots, pos).cpu().tolist()
        self.stats.steps += 1
        for i, r in enumerate(rows):
            t = forced.get(i, toks[i])
            self.spec.hist[r.slot].append(t)
            self._deliver(r, [t])

    # ---- delivery ------------------------------------------------------------------------------------------------
    def _deliver(self, r: Request, toks: List[int]):
        """Hands the step's tokens of ``r`` to the receiver, cutting at a stop token or the length limit.  The sequence
        history already ends with ``toks``."""
        stops = set(r.sampling.get("stop_token_ids") or ())
        min_new = int(r.sampling.get("min_new_tokens", 0))
        out: List[int] = []
        finished = False
        for j, t in enumerate(toks):
            if r.guard is not None:
                t2 = r.guard.filter(t)
                if t2 != t:                                  # the guard closed a runaway think block: continue from its token
                    self._rewrite_tail(r, len(toks), j, t2)
                    out.append(t2); r.out.append(t2)
                    break
            if r.budget is not None:
                r.budget.accept(len(r.out), t)
            out.append(t); r.out.append(t)
            if (t in stops and len(r.out) >= min_new) or len(r.out) >= r.max_new:
                finished = True
                break
        if self.m.seq_len_host.get(r.slot, 0) + 1 >= self.m.max_ctx:
            finished = True
        r.t_last = time.monotonic()
        self.stats.tokens_out += len(out)
        gone = self.emit(r.rid, out, finished, None)
        if finished and not gone and self.keep_sequences and r.mm is None and r.slot in self.active and r.state == DECODE:
            for src in self.spec.sources:
                src.end(r.slot)
            self.spec.hist.pop(r.slot, None); self.spec.samp.pop(r.slot, None)
            self.active.pop(r.slot)
            self._keep(r)
            r.state = DONE
        elif finished or gone:
            self._finish(r, silent=True)

    def _rewrite_tail(self, r: Request, n_step: int, keep: int, tok: int):
        """Of the ``n_step`` tokens this step appended to the history only the first ``keep`` stay, followed by ``tok``;
        the KV rows of the dropped tokens are rolled back (every kept row was part of the verify block)."""
        h = self.spec.hist[r.slot]
        del h[len(h) - n_step + keep:]
        for s in self.spec.sources:
            s.rewind(r.slot, len(h))
        h.append(tok)
        self.m.truncate(r.slot, len(h) - 1)

    def _finish(self, r: Request, error: Optional[str] = None, silent: bool = False):
        if not silent:
            self.emit(r.rid, [], True, error)
        if r.slot in self.active:
            self._release(r)
        r.state = DONE


# ---------------------------------------------------------------------------------------------------------------------
def attach_to_server(engine: Engine, server, context_length: Optional[int] = None):
    """Makes ``engine`` the backend of an OpenAI front end (:class:`agens_engine_b200.serve.server.Server`).  The
    server passes the request's image URLs inside the sampling object (key ``images``)."""
    engine.emit = lambda rid, toks, fin, err: server.push(rid, toks, fin, err)
    engine.on_stats = lambda st: server.set_metrics(st.prometheus(engine.m))

    def generate(rid, prompt, sampling, session):
        images = sampling.pop("images", None) if isinstance(sampling, dict) else None
        engine.submit(prompt, sampling, rid=rid, session=session, images=images)

    server.use_engine(generate, context_length or engine.m.max_ctx, supports_images=engine.vision is not None)
