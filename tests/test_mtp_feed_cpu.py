"""The bookkeeping that feeds an MTP head with the prompt (``spec/decoder.py::MtpSource.prefill_sink`` / ``begin`` /
``rewind``), on the CPU with a stand-in head that records what it is given: every prompt position i < P - 1 is paired
with prompt token i + 1, the last prompt position with the first generated token, whatever the chunking and wherever a
prefix cache let the prefill start (reference: kernels/m1/m1_mtp.cu:11, :768 ``materialize``)."""
import torch

from agens_engine_b200.spec.decoder import MtpSource


class FakeHead:
    """Records (hidden value, token) pairs per sequence; the hidden row of position p is filled with the value p."""

    def __init__(self):
        self.dev = torch.device("cpu")
        self.seq_pages, self.seq_len_host, self.pairs = {}, {}, {}
        self.cat = torch.zeros(32, 8)
        self.h_a = torch.zeros(32, 4)

    def new_seq(self, s):
        self.seq_pages[s], self.seq_len_host[s], self.pairs[s] = [], 0, []

    def free_seq(self, s):
        self.seq_pages.pop(s); self.seq_len_host.pop(s); self.pairs.pop(s)

    def truncate(self, s, n):
        self.seq_len_host[s] = n
        del self.pairs[s][n:]

    def prefill_pairs(self, s, toks, hidden):
        for t, h in zip(toks.tolist(), hidden):
            self.pairs[s].append((int(h[0]), t))
        self.seq_len_host[s] += len(toks)

    def forward_mtp(self, ids, hidden, seqs):
        for t, h, s in zip(ids, hidden, seqs):
            self.pairs[s].append((int(h[0]), t))
            self.seq_len_host[s] += 1
        return torch.tensor([1000 + t for t in ids])


def _hidden(lo, hi):
    return torch.arange(lo, hi, dtype=torch.float32)[:, None].expand(-1, 4).contiguous()


def test_prompt_positions_pair_with_the_next_token():
    for cuts in ([0, 10], [0, 4, 8, 10], [0, 9, 10], [0, 1, 2, 10]):
        head = FakeHead()
        src = MtpSource(head, depth=2)
        prompt = [50 + i for i in range(10)]
        sink = src.prefill_sink(3, prompt)
        for c0, c1 in zip(cuts[:-1], cuts[1:]):
            sink(c0, _hidden(c0, c1))
        assert head.pairs[3] == [(i, prompt[i + 1]) for i in range(9)], cuts      # positions 0..8 with tokens 1..9
        src.begin(3, prompt + [777])                                              # the first generated token arrives
        assert head.pairs[3][-1] == (9, 777) and head.seq_len_host[3] == 10 and src.first[3] == 1
        assert src.pending[3][0] == 1777                                          # the head's output for that row: first draft
        # rewind to a history of 6 tokens keeps the entries of positions 0..4
        src.rewind(3, 6)
        assert head.seq_len_host[3] == 5 and 3 not in src.pending


def test_prefix_cache_start_and_abandoned_prefill():
    head = FakeHead()
    src = MtpSource(head, depth=2)
    prompt = list(range(100, 112))
    sink = src.prefill_sink(0, prompt, start=5)           # positions 0..4 came from a prefix cache: no entries for them
    sink(5, _hidden(5, 9))
    sink(9, _hidden(9, 12))
    assert head.pairs[0] == [(i, prompt[i + 1]) for i in range(5, 11)] and src.first[0] == 6
    src.begin(0, prompt + [9])
    assert head.pairs[0][-1] == (11, 9)
    src.rewind(0, 9)                                      # history of 9 tokens: entries for positions 5..7
    assert head.seq_len_host[0] == 3
    # a prefill that was given up leaves entries behind; the slot's next use starts clean
    sink = src.prefill_sink(0, [1, 2, 3, 4])
    sink(0, _hidden(0, 2))
    sink2 = src.prefill_sink(0, [7, 8, 9])
    assert head.pairs[0] == [] and 0 not in src._fed
    sink2(0, _hidden(0, 3))
    src.begin(0, [7, 8, 9, 5])
    assert head.pairs[0] == [(0, 8), (1, 9), (2, 5)]
    # without a sink (a resumed conversation) the entries start at the next generated token
    src.end(0)
    src.begin(0, [1, 2, 3, 4, 5])
    assert src.first[0] == 5 and head.seq_len_host[0] == 0
