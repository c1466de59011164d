"""Speculative decoding: draft sources, verify blocks and acceptance.

A step of a sequence builds a verify block ``[t, d_1 .. d_n]`` (``t`` = the last emitted token, ``d_j`` drafts),
runs it through the target as one group of rows, lets the target name its own token after every row (argmax, or the
positional sample of ``ops.basic.sample_rows``) and accepts draft ``d_{j+1}`` iff it equals the target's token after
row ``j``.  The emitted tokens are therefore exactly what plain decoding would have produced, greedy or sampled
(the sampler's draw depends only on seed, position and logits).  Rejected rows are rolled back by truncating the
sequence; their KV entries are overwritten by the next block.

Draft sources, in the reference's cascade order (``crates/agens-cli/src/spec.rs:44-130``, ``lookup.rs``): copy-lookup over the
sequence's own tokens, the MTP head, the companion drafter model.  Acceptance: ``kernels/m1/m1_model.cu:476-579``.
"""
from __future__ import annotations

import dataclasses
from typing import Dict, List, Optional, Sequence

import torch

from ..models.dense import DenseModel
from ..models.mtp import MtpHead
from ..ops import basic

MAX_BLOCK = 8          # rows of one verify group (bonus + 7 drafts)


class DraftSource:
    """Interface of a draft source for one sequence slot."""
    name = "none"

    def begin(self, seq: int, prompt: Sequence[int]):
        pass

    def propose(self, seq: int, history: Sequence[int], max_n: int) -> List[int]:
        """Drafts continuing ``history`` (whose last element is the next input token)."""
        return []

    def propose_many(self, seqs: Sequence[int], histories: Dict[int, Sequence[int]], max_n: int) -> Dict[int, List[int]]:
        """Drafts for several sequences of one step.  Sources that run a model override this to batch the sequences
        into shared forward passes (the reference drafts a batch per call as well: kernels/m1/m1_mtp.cu ``propose_b``)."""
        return {s: self.propose(s, histories[s], max_n) for s in seqs}

    def feedback(self, seq: int, n_proposed: int, n_accepted: int):
        pass

    def rewind(self, seq: int, n_hist: int):
        """Only the first ``n_hist`` tokens of the history this source has seen are still valid."""

    def end(self, seq: int):
        pass


class CopyLookupSource(DraftSource):
    """Drafts by copying what followed the longest earlier occurrence of the current suffix (host side, C++)."""
    name = "copy"

    def __init__(self):
        from ..serve import host
        self._host = host
        self.tables: Dict[int, object] = {}
        self.fed: Dict[int, int] = {}

    def begin(self, seq, prompt):
        self.tables[seq] = self._host.CopyLookup()
        self.fed[seq] = 0

    def propose(self, seq, history, max_n):
        t = self.tables[seq]
        if self.fed[seq] > len(history):
            t.truncate(len(history)); self.fed[seq] = len(history)
        if self.fed[seq] < len(history):
            t.extend(list(history[self.fed[seq]:])); self.fed[seq] = len(history)
        drafts, _ = t.propose()
        return drafts[:max_n]

    def feedback(self, seq, n_proposed, n_accepted):
        if n_proposed:
            self.tables[seq].record(n_accepted)

    def rewind(self, seq, n_hist):
        if self.fed.get(seq, 0) > n_hist:
            self.tables[seq].truncate(n_hist); self.fed[seq] = n_hist

    def end(self, seq):
        self.tables.pop(seq, None); self.fed.pop(seq, None)


class ModelSource(DraftSource):
    """A small model of the same vocabulary drafting greedily with its own paged KV."""
    name = "drafter"

    def __init__(self, drafter: DenseModel, depth: int = 4):
        self.m, self.depth = drafter, depth

    def begin(self, seq, prompt):
        self.m.new_seq(seq)
        if len(prompt) > 1:
            self.m.prefill(seq, torch.tensor(list(prompt[:-1]), dtype=torch.int32))

    def propose(self, seq, history, max_n):
        m = self.m
        have = m.seq_len_host[seq]
        if have > len(history) - 1:                     # rows fed for drafts that were then rejected
            m.truncate(seq, len(history) - 1); have = len(history) - 1
        missing = list(history[have:])                  # always ends with the next input token
        out = None
        for c in range(0, len(missing), MAX_BLOCK):
            rows = missing[c:c + MAX_BLOCK]
            out, _ = m.forward_rows(rows, [seq] * len(rows))
        drafts = [int(out[-1])]
        while len(drafts) < min(max_n, self.depth):
            out, _ = m.forward_rows([drafts[-1]], [seq])
            drafts.append(int(out[0]))
        return drafts

    def propose_many(self, seqs, histories, max_n):
        """One forward pass per draft position for all sequences together: first the rows every sequence still misses
        (its last emitted tokens, at most eight per pass), then one row per sequence and position.  A step of sixteen
        sequences at depth three is three passes instead of forty-eight."""
        m = self.m
        seqs = list(seqs)
        depth = min(max_n, self.depth)
        if depth <= 0 or not seqs:
            return {s: [] for s in seqs}
        missing = {}
        for s in seqs:
            h = histories[s]
            have = m.seq_len_host[s]
            if have > len(h) - 1:
                m.truncate(s, len(h) - 1); have = len(h) - 1
            missing[s] = list(h[have:])
        last: Dict[int, int] = {}
        todo = seqs
        while todo:
            ids, rows, ends, nxt = [], [], {}, []
            for s in todo:
                take = missing[s][:MAX_BLOCK]
                if len(ids) + len(take) > m.max_rows:
                    nxt.append(s); continue
                ids += take; rows += [s] * len(take)
                missing[s] = missing[s][len(take):]
                ends[s] = len(ids) - 1
                if missing[s]:
                    nxt.append(s)
            out, _ = m.forward_rows(ids, rows)
            oh = out.tolist()
            for s, e in ends.items():
                last[s] = oh[e]
            todo = nxt
        drafts = {s: [last[s]] for s in seqs}
        for _ in range(depth - 1):
            for c in range(0, len(seqs), m.max_rows):
                part = seqs[c:c + m.max_rows]
                out, _ = m.forward_rows([drafts[s][-1] for s in part], part)
                for s, tok in zip(part, out.tolist()):
                    drafts[s].append(tok)
        return drafts

    def rewind(self, seq, n_hist):
        if self.m.seq_len_host[seq] > n_hist:
            self.m.truncate(seq, n_hist)

    def end(self, seq):
        self.m.free_seq(seq)


class MtpSource(DraftSource):
    """Drafts from the target's hidden state through the MTP layer.  Needs the verify step's hidden rows, which the
    decoder hands over through :meth:`absorb`."""
    name = "mtp"

    def __init__(self, head: MtpHead, depth: int = 2):
        self.h, self.depth = head, depth
        self.pending: Dict[int, tuple] = {}
        self.first: Dict[int, int] = {}                 # history index of the token paired with MTP entry 0
        self._fed: Dict[int, torch.Tensor] = {}         # last prompt position's hidden row, kept until the first token is known

    def begin(self, seq, prompt):
        """``prompt`` = the prompt followed by the first generated token.  When the target's prefill handed over its
        hidden rows (:meth:`prefill_sink`), the prompt positions already have their entries and only the last prompt
        position, whose following token is the first generated one, is fed here."""
        if seq in self._fed:
            last_h = self._fed.pop(seq)
            self.absorb(seq, [prompt[-1]], last_h)
            return
        self._fresh(seq)
        self.first[seq] = len(prompt)

    def _fresh(self, seq: int):
        if seq in self.h.seq_pages:                     # a prefill that was given up left its entries behind
            self.h.free_seq(seq)
        self.pending.pop(seq, None); self._fed.pop(seq, None)
        self.h.new_seq(seq)

    def prefill_sink(self, seq: int, prompt: Sequence[int], start: int = 0):
        """Callable for ``DenseModel.hidden_sink`` during the prefill of ``prompt[start:]`` on ``seq``: every chunk's
        hidden rows become context entries of the head (an entry pairs the state at a prompt position with the prompt
        token after it), so that the first draft already attends to the prompt (reference: kernels/m1/m1_mtp.cu:11,
        :768).  ``start`` > 0: the positions before it came from a prefix cache and have no entries."""
        self._fresh(seq)
        self.first[seq] = start + 1
        P = len(prompt)
        toks = torch.tensor(list(prompt), dtype=torch.int32, device=self.h.dev)

        def sink(pos0: int, hidden: torch.Tensor):
            T = hidden.shape[0]
            n = min(pos0 + T, P - 1) - pos0            # the last prompt position waits for the first generated token
            if n > 0:
                self.h.prefill_pairs(seq, toks[pos0 + 1:pos0 + 1 + n], hidden[:n])
            if pos0 + T == P:
                self._fed[seq] = hidden[T - 1:T].clone()
        return sink

    def rewind(self, seq, n_hist):
        keep = max(n_hist - self.first[seq], 0)         # entry e pairs the hidden state with history token first + e
        if self.h.seq_len_host[seq] > keep:
            self.h.truncate(seq, keep)
            self.pending.pop(seq, None)

    def absorb(self, seq: int, tokens_after: Sequence[int], hidden: torch.Tensor):
        """``hidden[i]`` is the target's state at a committed position and ``tokens_after[i]`` the token that follows
        it.  Feeds the pairs to the MTP layer; the last row's output is the first draft."""
        n = len(tokens_after)
        out = None
        for c in range(0, n, MAX_BLOCK):
            e = min(n, c + MAX_BLOCK)
            out = self.h.forward_mtp(list(tokens_after[c:e]), hidden[c:e], [seq] * (e - c))
        self.pending[seq] = (int(out[-1]), self.h.h_a[e - c - 1:e - c].clone(), self.h.seq_len_host[seq])

    def propose(self, seq, history, max_n):
        if seq not in self.pending:
            return []
        first, hid, base = self.pending.pop(seq)
        drafts = [first]
        while len(drafts) < min(max_n, self.depth):
            out = self.h.forward_mtp([drafts[-1]], hid, [seq])
            hid = self.h.h_a[:1].clone()
            drafts.append(int(out[0]))
        self.h.truncate(seq, base)                      # recurrent rows are provisional
        return drafts

    def absorb_many(self, items):
        """:meth:`absorb` for several sequences of one verify step in shared passes through the head: ``items`` is a
        list of (sequence, tokens after, hidden rows)."""
        cap = self.h.cat.shape[0]
        batch: list = []

        def flush():
            ids = [t for _, toks, _ in batch for t in toks]
            rows = [q for q, toks, _ in batch for _ in toks]
            hid = torch.cat([h[:len(toks)] for _, toks, h in batch])
            oh = self.h.forward_mtp(ids, hid, rows).tolist()
            r = 0
            for q, toks, _ in batch:
                r += len(toks)
                self.pending[q] = (oh[r - 1], self.h.h_a[r - 1:r].clone(), self.h.seq_len_host[q])

        n = 0
        for it in items:
            k = len(it[1])
            if k > MAX_BLOCK:
                self.absorb(*it); continue
            if n + k > cap:
                flush(); batch = []; n = 0
            batch.append(it); n += k
        if batch:
            flush()

    def propose_many(self, seqs, histories, max_n):
        res: Dict[int, List[int]] = {s: [] for s in seqs}
        live = [s for s in seqs if s in self.pending]
        if not live:
            return res
        pend = {s: self.pending.pop(s) for s in live}
        hid = {s: pend[s][1] for s in live}
        for s in live:
            res[s] = [pend[s][0]]
        cap = self.h.cat.shape[0]
        for _ in range(min(max_n, self.depth) - 1):          # deeper drafts: one row per sequence and pass
            for c in range(0, len(live), cap):
                part = live[c:c + cap]
                oh = self.h.forward_mtp([res[s][-1] for s in part], torch.cat([hid[s] for s in part]), part).tolist()
                for i, s in enumerate(part):
                    res[s].append(oh[i]); hid[s] = self.h.h_a[i:i + 1].clone()
        for s in live:
            self.h.truncate(s, pend[s][2])                  # recurrent rows are provisional
        return res

    def end(self, seq):
        self.h.free_seq(seq); self.pending.pop(seq, None); self.first.pop(seq, None); self._fed.pop(seq, None)


@dataclasses.dataclass
class SamplingState:
    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 1.0
    min_p: float = 0.0
    seed: int = 0


@dataclasses.dataclass
class SpecStats:
    steps: int = 0
    proposed: int = 0
    accepted: int = 0
    emitted: int = 0
    by_source: Dict[str, List[int]] = dataclasses.field(default_factory=dict)

    def tokens_per_step(self) -> float:
        return self.emitted / max(self.steps, 1)


class SpecDecoder:
    """Drives target + draft sources for a set of sequences."""

    def __init__(self, target: DenseModel, sources: Sequence[DraftSource], max_drafts: int = 4):
        assert 0 <= max_drafts <= MAX_BLOCK - 1
        self.t, self.sources, self.max_drafts = target, list(sources), max_drafts
        self.hist: Dict[int, List[int]] = {}
        self.samp: Dict[int, SamplingState] = {}
        self.stats = SpecStats()
        self._mtp = [s for s in self.sources if isinstance(s, MtpSource)]
        self.mtp_prompt = True      # MTP heads get context entries for the prompt positions (off: entries start at the first generated token)

    # -------------------------------------------------------------------------------------------- sequences
    def begin(self, seq: int, prompt: Sequence[int], sampling: Optional[SamplingState] = None) -> int:
        """Prefills ``prompt`` and returns the first generated token."""
        t = self.t
        t.new_seq(seq)
        self.samp[seq] = sampling or SamplingState()
        sampled = self.samp[seq].temperature > 0
        if self._mtp and self.mtp_prompt and len(prompt) > 1:
            sinks = [mtp.prefill_sink(seq, prompt) for mtp in self._mtp]
            t.hidden_sink = lambda pos0, hid: [f(pos0, hid) for f in sinks]
        try:
            first, logits = t.prefill(seq, torch.tensor(list(prompt), dtype=torch.int32), want_logits=sampled)
        finally:
            t.hidden_sink = None
        if sampled:
            first = int(self._sample(logits[None, :], [seq], [len(prompt)])[0])
        self.hist[seq] = list(prompt) + [first]
        for s in self.sources:
            s.begin(seq, self.hist[seq])
        return first

    def end(self, seq: int):
        for s in self.sources:
            s.end(seq)
        self.t.free_seq(seq)
        self.hist.pop(seq); self.samp.pop(seq)

    # -------------------------------------------------------------------------------------------- one step
    def _sample(self, logits: torch.Tensor, seqs: List[int], positions: List[int]) -> torch.Tensor:
        dev = logits.device
        st = [self.samp[s] for s in seqs]
        # one upload per step: float parameters as their bit patterns, integer parameters, the seeds as two halves
        f = torch.tensor([[x.temperature for x in st], [x.top_p for x in st], [x.min_p for x in st]], dtype=torch.float32)
        seeds = [x.seed & 0x7FFFFFFFFFFFFFFF for x in st]
        i = torch.tensor([[x.top_k for x in st], list(positions), [v & 0x7FFFFFFF for v in seeds], [(v >> 31) & 0x7FFFFFFF for v in seeds],
                          [v >> 62 for v in seeds]], dtype=torch.int32)
        p = torch.cat([f.view(torch.int32), i]).to(dev)
        fl = p[:3].view(torch.float32)
        seed = p[5].long() | (p[6].long() << 31) | (p[7].long() << 62)
        return basic.sample_rows(logits, fl[0], p[3], fl[1], fl[2], seed, p[4], n_valid=self.t.vocab_valid_full())

    def step(self, seqs: Sequence[int], forced_drafts: Optional[Dict[int, List[int]]] = None) -> Dict[int, List[int]]:
        """One verify step for every sequence of ``seqs``; returns the tokens each of them emitted (at least one).
        ``forced_drafts`` overrides the draft sources (tests: corrupted drafts)."""
        t = self.t
        ids, rows_seq, row0, cnt, positions = [], [], [], [], []
        used: Dict[int, tuple] = {}
        # drafts: the sources are asked in their order; each one drafts for all sequences still without drafts at once
        drafts_of: Dict[int, List[int]] = {}
        src_of: Dict[int, DraftSource] = {}
        if forced_drafts is not None:
            for s in seqs:
                if s in forced_drafts:
                    drafts_of[s] = list(forced_drafts[s])[:self.max_drafts]
        waiting = [s for s in seqs if s not in drafts_of]
        if self.max_drafts:
            for src in self.sources:
                if not waiting:
                    break
                got = src.propose_many(waiting, self.hist, self.max_drafts)
                for s in waiting:
                    if got.get(s):
                        drafts_of[s] = list(got[s]); src_of[s] = src
                waiting = [s for s in waiting if s not in drafts_of]
        for s in seqs:
            h = self.hist[s]
            drafts = drafts_of.get(s, [])
            src_used = src_of.get(s)
            room = t.max_ctx - t.seq_len_host[s] - 1
            drafts = drafts[:max(room, 0)]
            used[s] = (src_used, len(drafts))
            row0.append(len(ids)); cnt.append(1 + len(drafts))
            base = t.seq_len_host[s]
            positions += [base + 1 + j for j in range(1 + len(drafts))]
            ids += [h[-1]] + drafts
            rows_seq += [s] * (1 + len(drafts))
        sampled = any(self.samp[s].temperature > 0 for s in seqs)
        base_len = {s: t.seq_len_host[s] for s in seqs}
        out, logits = t.forward_rows(ids, rows_seq, want_logits=sampled)
        target = self._sample(logits, rows_seq, positions) if sampled else out
        dev = t.dev
        ti = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
        n_emit, emitted = basic.spec_accept(ti(ids), target, ti(row0), ti(cnt), MAX_BLOCK)
        both = torch.cat([n_emit.view(-1, 1), emitted], dim=1).cpu().tolist()          # one read-back per step
        n_emit_h, emitted_h = [r[0] for r in both], [r[1:] for r in both]
        result: Dict[int, List[int]] = {}
        absorb = []
        for b, s in enumerate(seqs):
            k = n_emit_h[b]
            toks = emitted_h[b][:k]
            result[s] = toks
            t.truncate(s, base_len[s] + k)
            self.hist[s].extend(toks)
            src, n_prop = used[s]
            self.stats.steps += 1; self.stats.proposed += n_prop; self.stats.accepted += k - 1; self.stats.emitted += k
            if src is not None:
                src.feedback(s, n_prop, k - 1)
                st = self.stats.by_source.setdefault(src.name, [0, 0]); st[0] += n_prop; st[1] += k - 1
            # committed positions of this block: rows 0 .. k-1; the token after row j is toks[j]
            absorb.append((s, toks, t.h_a[row0[b]:row0[b] + k]))
        for mtp in self._mtp:
            mtp.absorb_many(absorb)
        return result

    def generate(self, seq: int, prompt: Sequence[int], n_new: int, sampling: Optional[SamplingState] = None,
                 eos: Optional[int] = None) -> List[int]:
        out = [self.begin(seq, prompt, sampling)]
        while len(out) < n_new and (eos is None or out[-1] != eos):
            out += self.step([seq])[seq]
        self.end(seq)
        return out[:n_new]
