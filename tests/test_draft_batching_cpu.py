"""Batched drafting (``spec/decoder.py::ModelSource.propose_many``) on the CPU with a stand-in drafter: the drafts equal
those of drafting every sequence on its own, the drafter sees every missing token exactly once, and a step of many
sequences takes one forward pass per draft position (plus the passes that catch up on long gaps)."""
import random

import torch

from agens_engine_b200.spec.decoder import MAX_BLOCK, ModelSource


class FakeDrafter:
    """Greedy stand-in: the token after a sequence is a fixed function of everything fed to it so far."""

    def __init__(self, max_rows=32):
        self.max_rows = max_rows
        self.fed, self.seq_len_host, self.calls = {}, {}, 0

    def new_seq(self, s):
        self.fed[s], self.seq_len_host[s] = [], 0

    def free_seq(self, s):
        self.fed.pop(s); self.seq_len_host.pop(s)

    def truncate(self, s, n):
        del self.fed[s][n:]
        self.seq_len_host[s] = n

    def prefill(self, s, ids):
        self.fed[s] += ids.tolist()
        self.seq_len_host[s] = len(self.fed[s])

    def forward_rows(self, ids, seqs, want_logits=False):
        assert 1 <= len(ids) <= self.max_rows
        self.calls += 1
        out = []
        for i, (t, s) in enumerate(zip(ids, seqs)):
            assert i == 0 or seqs[i - 1] == s or s not in seqs[:i], "rows of one sequence must be adjacent"
            self.fed[s].append(int(t))
            self.seq_len_host[s] = len(self.fed[s])
            out.append((sum((j + 1) * v for j, v in enumerate(self.fed[s])) * 31 + 7) % 1000)
        return torch.tensor(out), None


def _histories(rnd, n):
    return {s: [rnd.randrange(1000) for _ in range(rnd.randint(3, 40))] for s in range(n)}


def test_batched_drafts_equal_single_sequence_drafts():
    rnd = random.Random(0)
    for n_seq, depth, rows in ((1, 3, 32), (5, 4, 32), (16, 3, 32), (40, 2, 32), (7, 1, 8)):
        hist = _histories(rnd, n_seq)
        one, many = FakeDrafter(rows), FakeDrafter(rows)
        a, b = ModelSource(one, depth), ModelSource(many, depth)
        for s, h in hist.items():
            k = rnd.randint(1, len(h))                        # how much of the history the drafter has seen (begin feeds all but one)
            a.begin(s, h[:k]); b.begin(s, h[:k])
        want = {s: a.propose(s, hist[s], 4) for s in hist}
        many.calls = 0
        got = b.propose_many(list(hist), hist, 4)
        assert got == want
        assert all(many.fed[s] == one.fed[s] for s in hist)     # the same rows reached both drafters
        assert many.calls <= one.calls and (n_seq == 1 or many.calls < one.calls)
        # a second step after two tokens were accepted and the rest rejected: the drafter is rewound and catches up
        for s in hist:
            hist[s] = hist[s] + want[s][:2]
        want2 = {s: a.propose(s, hist[s], 4) for s in hist}
        assert b.propose_many(list(hist), hist, 4) == want2


def test_sixteen_sequences_at_depth_three_take_three_passes():
    rnd = random.Random(1)
    hist = _histories(rnd, 16)
    d = FakeDrafter(32)
    src = ModelSource(d, 3)
    for s, h in hist.items():
        src.begin(s, h)                                        # the drafter has seen all but the last token
    d.calls = 0
    out = src.propose_many(list(hist), hist, 3)
    assert d.calls == 3 and all(len(v) == 3 for v in out.values())
    # one sequence is far behind (a copy-lookup source served it for a while): its gap is filled eight rows per pass
    hist[0] = hist[0] + [rnd.randrange(1000) for _ in range(20)]
    for s in hist:
        if s:
            hist[s] = hist[s] + out[s][:1]
    d.calls = 0
    out = src.propose_many(list(hist), hist, 3)
    assert d.calls == 3 + 2 and d.seq_len_host[0] == len(hist[0]) + 2
