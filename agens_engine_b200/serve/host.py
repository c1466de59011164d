"""Python bindings of the host-only C++ runtime (``libagens_b200_host.so``): sampler, reasoning budget, think guard,
page allocator, KV admission policy, copy-lookup drafter, prefix cache, memory planner and profiles.  The reference
implements these in Rust (``crates/agens-cli/src/{sampler,lookup,prefix,plan,profile,serve}.rs``)."""
from __future__ import annotations

import array
import ctypes as C
import json
from typing import Dict, List, Optional, Sequence, Tuple

from .. import _lib

_sig_done = False


def lib() -> C.CDLL:
    global _sig_done
    h = _lib.host_lib()
    if not _sig_done:
        vp, i, ll, d, f = C.c_void_p, C.c_int, C.c_longlong, C.c_double, C.c_float
        ip, lp, llp, dp, fp = C.POINTER(C.c_int), C.POINTER(C.c_long), C.POINTER(C.c_longlong), C.POINTER(C.c_double), C.POINTER(C.c_float)
        sig = {
            "b2h_sampler_new": ([C.c_char_p, C.c_ulonglong], vp), "b2h_sampler_free": ([vp], None),
            "b2h_sampler_sample": ([vp, fp, i, ip, fp, i], i), "b2h_sampler_accept": ([vp, i], None),
            "b2h_sampler_needs_logits": ([vp, i], i), "b2h_sampler_uniform": ([vp], d),
            "b2h_budget_new": ([i, d, ip, i, i, i], vp), "b2h_budget_free": ([vp], None),
            "b2h_budget_accept": ([vp, ll, i], None), "b2h_budget_act": ([vp, ll, ip, fp], i),
            "b2h_guard_new": ([i, i, i, ip, i, i, i], vp), "b2h_guard_free": ([vp], None),
            "b2h_guard_filter": ([vp, i, i], i), "b2h_guard_fired": ([vp], ll),
            "b2h_pages_new": ([i, i], vp), "b2h_pages_free": ([vp], None), "b2h_pages_free_count": ([vp], i),
            "b2h_pages_new_seq": ([vp], i), "b2h_pages_reserve": ([vp, i, i], i), "b2h_pages_set_len": ([vp, i, i], None),
            "b2h_pages_len": ([vp, i], i), "b2h_pages_truncate": ([vp, i, i], i), "b2h_pages_fork": ([vp, i, ip, ip], i),
            "b2h_pages_free_seq": ([vp, i], i), "b2h_pages_exclusive": ([vp, i], i), "b2h_pages_refcount": ([vp, i], i),
            "b2h_pages_list": ([vp, i, ip, i], i), "b2h_pages_evict_page": ([vp, i, i], i),
            "b2h_kv_safe": ([C.c_long, lp, lp, i], i),
            "b2h_pick_victim": ([ip, llp, dp, ip, i, d, i], i),
            "b2h_pick_prefill": ([lp, dp, i, C.c_long, i, i], i),
            "b2h_lookup_new": ([], vp), "b2h_lookup_free": ([vp], None), "b2h_lookup_extend": ([vp, ip, i], None),
            "b2h_lookup_truncate": ([vp, i], None), "b2h_lookup_propose": ([vp, ip, ip, i], i),
            "b2h_lookup_record": ([vp, i], None), "b2h_lookup_mean": ([vp, i], d),
            "b2h_prefix_new": ([ll, i], vp), "b2h_prefix_free": ([vp], None),
            "b2h_prefix_lookup": ([vp, ip, i, C.c_ulonglong, llp], i),
            "b2h_prefix_insert": ([vp, ip, i, C.c_ulonglong, ll, ll, llp, i], i),
            "b2h_prefix_insert_chain": ([vp, ip, i, C.c_ulonglong, ll, ll, llp, i], i),
            "b2h_prefix_ref": ([vp, ll, i], None), "b2h_prefix_used": ([vp], ll), "b2h_prefix_evict_lru": ([vp], ll),
            "b2h_plan": ([C.c_char_p], vp), "b2h_profile": ([C.c_char_p, i], vp), "b2h_free_str": ([vp], None),
            "b2h_host_mem_available": ([], ll),
        }
        for name, (args, res) in sig.items():
            fn = getattr(h, name)
            fn.argtypes, fn.restype = args, res
        _sig_done = True
    return h


def _ints(xs: Sequence[int]):
    """A C int array of ``xs`` (through array.array: several times faster than unpacking into the ctypes constructor,
    which matters for prompts of a hundred thousand tokens)."""
    if len(xs) < 64:
        return (C.c_int * len(xs))(*xs)
    try:
        a = array.array("i", xs)
    except (TypeError, OverflowError):                      # elements that are not plain ints: the general constructor
        return (C.c_int * len(xs))(*xs)
    return (C.c_int * len(a)).from_buffer(a)


def _take_json(p) -> dict:
    s = C.cast(p, C.c_char_p).value.decode()
    lib().b2h_free_str(p)
    return json.loads(s)


class Sampler:
    def __init__(self, params: dict, request_id: int = 0):
        self._h = lib().b2h_sampler_new(json.dumps(params).encode(), request_id)
        if not self._h:
            raise ValueError("bad sampling parameters")

    def __del__(self):
        if getattr(self, "_h", None):
            try:
                lib().b2h_sampler_free(self._h)
            except TypeError:                               # interpreter shutdown: the module globals are gone
                pass

    def sample(self, logits, extra: Sequence[Tuple[int, float]] = ()) -> int:
        import numpy as np
        x = np.ascontiguousarray(logits, dtype=np.float32)
        ids = _ints([e[0] for e in extra])
        dl = (C.c_float * len(extra))(*[e[1] for e in extra])
        return lib().b2h_sampler_sample(self._h, x.ctypes.data_as(C.POINTER(C.c_float)), x.size, ids, dl, len(extra))

    def accept(self, tok: int):
        lib().b2h_sampler_accept(self._h, tok)

    def needs_logits(self, vocab_valid: int) -> bool:
        return bool(lib().b2h_sampler_needs_logits(self._h, vocab_valid))

    def uniform(self) -> float:
        return lib().b2h_sampler_uniform(self._h)


class ReasoningBudget:
    def __init__(self, n: int, soft: float, prompt: Sequence[int], start: int, end: int):
        self._h = lib().b2h_budget_new(n, soft, _ints(prompt), len(prompt), start, end)

    def __del__(self):
        if getattr(self, "_h", None):
            try:
                lib().b2h_budget_free(self._h)
            except TypeError:                               # interpreter shutdown: the module globals are gone
                pass

    def accept(self, out_index: int, tok: int):
        lib().b2h_budget_accept(self._h, out_index, tok)

    def act(self, produced: int):
        """Returns ("none",) | ("force", tok) | ("bias", tok, delta)."""
        tok, delta = C.c_int(), C.c_float()
        r = lib().b2h_budget_act(self._h, produced, C.byref(tok), C.byref(delta))
        return ("none",) if r == 0 else (("force", tok.value) if r == 1 else ("bias", tok.value, delta.value))


class ThinkGuard:
    def __init__(self, n: int, k: int, w: int, prompt: Sequence[int], start: int, end: int):
        self._h = lib().b2h_guard_new(n, k, w, _ints(prompt), len(prompt), start, end)

    def __del__(self):
        if getattr(self, "_h", None):
            try:
                lib().b2h_guard_free(self._h)
            except TypeError:                               # interpreter shutdown: the module globals are gone
                pass

    def filter(self, tok: int, pending: bool = True) -> int:
        return lib().b2h_guard_filter(self._h, tok, 1 if pending else 0)

    @property
    def fired(self) -> Optional[int]:
        v = lib().b2h_guard_fired(self._h)
        return None if v < 0 else v


class PageAllocator:
    def __init__(self, n_pages: int, page_size: int = 16):
        self._h = lib().b2h_pages_new(n_pages, page_size)

    def __del__(self):
        if getattr(self, "_h", None):
            try:
                lib().b2h_pages_free(self._h)
            except TypeError:                               # interpreter shutdown: the module globals are gone
                pass

    free_pages = property(lambda self: lib().b2h_pages_free_count(self._h))

    def new_seq(self) -> int:
        return lib().b2h_pages_new_seq(self._h)

    def reserve(self, s: int, n_tokens: int) -> int:
        return lib().b2h_pages_reserve(self._h, s, n_tokens)

    def set_len(self, s: int, n: int):
        lib().b2h_pages_set_len(self._h, s, n)

    def seq_len(self, s: int) -> int:
        return lib().b2h_pages_len(self._h, s)

    def truncate(self, s: int, n: int) -> int:
        return lib().b2h_pages_truncate(self._h, s, n)

    def fork(self, s: int):
        src, dst = C.c_int(), C.c_int()
        c = lib().b2h_pages_fork(self._h, s, C.byref(src), C.byref(dst))
        return c, src.value, dst.value

    def free_seq(self, s: int) -> int:
        return lib().b2h_pages_free_seq(self._h, s)

    def evict_page(self, s: int, index: int) -> int:
        """The page at ``index`` moved to the host tier: frees its GPU page and marks the position -2."""
        return lib().b2h_pages_evict_page(self._h, s, index)

    def exclusive(self, s: int) -> int:
        return lib().b2h_pages_exclusive(self._h, s)

    def refcount(self, page: int) -> int:
        return lib().b2h_pages_refcount(self._h, page)

    def pages(self, s: int) -> List[int]:
        buf = (C.c_int * 65536)()
        n = lib().b2h_pages_list(self._h, s, buf, 65536)
        return list(buf[:max(n, 0)])


def kv_safe(avail: int, items: Sequence[Tuple[int, int]]) -> bool:
    need = (C.c_long * len(items))(*[i[0] for i in items])
    hold = (C.c_long * len(items))(*[i[1] for i in items])
    return bool(lib().b2h_kv_safe(avail, need, hold, len(items)))


def pick_victim(cands: Sequence[Tuple[int, int, float, int]], hold_s: float = 10.0, allow_protected: bool = False) -> int:
    n = len(cands)
    return lib().b2h_pick_victim(_ints([c[0] for c in cands]), (C.c_longlong * n)(*[c[1] for c in cands]),
                                 (C.c_double * n)(*[c[2] for c in cands]), _ints([c[3] for c in cands]), n, hold_s,
                                 1 if allow_protected else 0)


def pick_prefill(remaining: Sequence[int], age_s: Sequence[float], chunk_index: int, fair: int = 4, srpt: bool = True) -> int:
    n = len(remaining)
    return lib().b2h_pick_prefill((C.c_long * n)(*remaining), (C.c_double * n)(*age_s), n, chunk_index, fair, 1 if srpt else 0)


class CopyLookup:
    def __init__(self):
        self._h = lib().b2h_lookup_new()

    def __del__(self):
        if getattr(self, "_h", None):
            try:
                lib().b2h_lookup_free(self._h)
            except TypeError:                               # interpreter shutdown: the module globals are gone
                pass

    def extend(self, toks: Sequence[int]):
        lib().b2h_lookup_extend(self._h, _ints(toks), len(toks))

    def truncate(self, n: int):
        lib().b2h_lookup_truncate(self._h, n)

    def propose(self, copy_only: bool = False):
        out, m = (C.c_int * 8)(), C.c_int()
        n = lib().b2h_lookup_propose(self._h, out, C.byref(m), 1 if copy_only else 0)
        return list(out[:n]), m.value

    def record(self, accepted: int):
        lib().b2h_lookup_record(self._h, accepted)

    def mean(self, bucket: int) -> float:
        return lib().b2h_lookup_mean(self._h, bucket)


class PrefixCache:
    def __init__(self, budget_bytes: int, chunk: int):
        self._h = lib().b2h_prefix_new(budget_bytes, chunk)

    def __del__(self):
        if getattr(self, "_h", None):
            try:
                lib().b2h_prefix_free(self._h)
            except TypeError:                               # interpreter shutdown: the module globals are gone
                pass

    def lookup(self, toks: Sequence[int], salt: int = 0):
        h = C.c_longlong(-1)
        n = lib().b2h_prefix_lookup(self._h, _ints(toks), len(toks), salt, C.byref(h))
        return n, h.value

    def insert(self, toks: Sequence[int], handle: int, nbytes: int, salt: int = 0):
        ev = (C.c_longlong * 64)()
        n = lib().b2h_prefix_insert(self._h, _ints(toks), len(toks), salt, handle, nbytes, ev, 64)
        return n, list(ev[:max(n, 0)])

    def insert_chain(self, toks: Sequence[int], handle: int, nbytes: int, salt: int = 0):
        """One entry per chunk boundary of ``toks`` in one pass (the bytes are booked on the longest); returns
        ``(count, evicted handles)`` like :meth:`insert`."""
        ev = (C.c_longlong * 256)()
        n = lib().b2h_prefix_insert_chain(self._h, _ints(toks), len(toks), salt, handle, nbytes, ev, 256)
        return n, list(ev[:max(n, 0)])

    def ref(self, handle: int, delta: int):
        lib().b2h_prefix_ref(self._h, handle, delta)

    used = property(lambda self: lib().b2h_prefix_used(self._h))

    def evict_lru(self) -> int:
        return lib().b2h_prefix_evict_lru(self._h)


def plan(**kw) -> dict:
    return _take_json(lib().b2h_plan(json.dumps(kw).encode()))


def profile(name: str, tp: int = 1) -> dict:
    return _take_json(lib().b2h_profile(name.encode(), tp))
