"""Launchers of the small fused ops (``csrc/kernels/sm100/ops_misc.cu``)."""
from __future__ import annotations

from typing import Optional

import torch

from .. import _lib
from .._lib import check, current_stream, ptr


def _status(dev) -> torch.Tensor:
    return torch.zeros(1, dtype=torch.int32, device=dev)


def embed(ids: torch.Tensor, table: torch.Tensor, ss: Optional[torch.Tensor] = None,
          sub_rows: Optional[torch.Tensor] = None, sub_index: Optional[torch.Tensor] = None,
          status: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    lib = _lib.cuda_lib()
    n, d = ids.numel(), table.shape[1]
    h = torch.empty(n, d, dtype=torch.bfloat16, device=table.device) if out is None else out
    status = _status(table.device) if status is None else status
    with torch.cuda.device(table.device):
        check(lib.b2_embed(ptr(ids), n, ptr(table), d, table.shape[0], ptr(sub_rows), ptr(sub_index), ptr(h), h.stride(0), ptr(ss),
                           ptr(status), current_stream()), "b2_embed")
    return h


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float, resid: Optional[torch.Tensor] = None):
    """``y = rmsnorm(x [+ resid]) * w``; with ``resid`` also returns the bf16 sum."""
    lib = _lib.cuda_lib()
    n, d = x.shape
    y = torch.empty_like(x)
    xo = torch.empty_like(x) if resid is not None else None
    with torch.cuda.device(x.device):
        check(lib.b2_rmsnorm(ptr(x), x.stride(0), ptr(resid), resid.stride(0) if resid is not None else 0, ptr(xo),
                             xo.stride(0) if xo is not None else 0, ptr(w), eps, n, d, ptr(y), y.stride(0),
                             current_stream()), "b2_rmsnorm")
    return (y, xo) if resid is not None else y


def sumsq(h: torch.Tensor, ss: torch.Tensor):
    lib = _lib.cuda_lib()
    with torch.cuda.device(h.device):
        check(lib.b2_sumsq(ptr(h), h.stride(0), h.shape[0], h.shape[1], ptr(ss), current_stream()), "b2_sumsq")


def rope_inv_freq(head_dim: int, theta: float, device) -> torch.Tensor:
    """fp32 ``theta ** (-2i / head_dim)`` for ``i < head_dim / 2``, repeated so that index ``i`` and ``i + 1`` of a
    lane's pair read consecutive entries (entry ``i`` belongs to rotary pair ``(i, i + head_dim/2)``)."""
    i = torch.arange(0, head_dim // 2, dtype=torch.float64)
    return (theta ** (-2.0 * i / head_dim)).to(torch.float32).to(device)


def rope_kvstore(qkv: torch.Tensor, hq: int, hkv: int, hd: int, inv_freq: torch.Tensor, tok_pos: torch.Tensor,
                 tok_seq: torch.Tensor, block_table: torch.Tensor, kv_pool: torch.Tensor, q_out: torch.Tensor,
                 rope_pos: Optional[torch.Tensor] = None, status: Optional[torch.Tensor] = None):
    lib = _lib.cuda_lib()
    n = qkv.shape[0]
    status = _status(qkv.device) if status is None else status
    page_size = kv_pool.shape[3]
    with torch.cuda.device(qkv.device):
        check(lib.b2_rope_kvstore(ptr(qkv), qkv.stride(0), n, hq, hkv, hd, ptr(inv_freq), ptr(tok_pos), ptr(rope_pos),
                                  ptr(tok_seq), ptr(block_table), block_table.stride(0), ptr(kv_pool), page_size,
                                  kv_pool.shape[0], ptr(q_out), q_out.stride(0), ptr(status), current_stream()),
              "b2_rope_kvstore")
    return status


def mrope_pair_axis(head_dim: int, sections, interleaved: bool = True, device="cpu") -> torch.Tensor:
    """uint8 [head_dim / 2]: which of the (time, height, width) positions drives each rotary frequency pair.
    ``sections`` = pairs per axis; interleaved: t, h, w, t, h, w, ... while an axis still has pairs left (the layout of
    the reference's text model, rope.cu:62-108), else three contiguous blocks."""
    half = head_dim // 2
    assert sum(sections) == half
    out = []
    if interleaved:
        left = list(sections)
        a = 0
        while len(out) < half:
            if left[a] > 0:
                out.append(a); left[a] -= 1
            a = (a + 1) % 3
    else:
        for a, n in enumerate(sections):
            out += [a] * n
    return torch.tensor(out, dtype=torch.uint8, device=device)


def rope_kvstore_m(qkv: torch.Tensor, hq: int, hkv: int, hd: int, inv_freq: torch.Tensor, tok_pos: torch.Tensor,
                   rope_pos3: torch.Tensor, pair_axis: torch.Tensor, tok_seq: torch.Tensor, block_table: torch.Tensor,
                   kv_pool: torch.Tensor, q_out: torch.Tensor, status: Optional[torch.Tensor] = None):
    """RoPE + KV store with multi-axis positions ``rope_pos3`` int32 [3, n] (time, height, width)."""
    lib = _lib.cuda_lib()
    n = qkv.shape[0]
    status = _status(qkv.device) if status is None else status
    assert rope_pos3.shape == (3, n) and rope_pos3.is_contiguous() and pair_axis.numel() == hd // 2
    with torch.cuda.device(qkv.device):
        check(lib.b2_rope_kvstore_m(ptr(qkv), qkv.stride(0), n, hq, hkv, hd, ptr(inv_freq), ptr(tok_pos), ptr(rope_pos3),
                                    ptr(pair_axis), ptr(tok_seq), ptr(block_table), block_table.stride(0), ptr(kv_pool),
                                    kv_pool.shape[3], kv_pool.shape[0], ptr(q_out), q_out.stride(0), ptr(status),
                                    current_stream()), "b2_rope_kvstore_m")
    return status


def swiglu_interleaved(gu: torch.Tensor) -> torch.Tensor:
    lib = _lib.cuda_lib()
    n, f2 = gu.shape
    act = torch.empty(n, f2 // 2, dtype=torch.bfloat16, device=gu.device)
    with torch.cuda.device(gu.device):
        check(lib.b2_swiglu_interleaved(ptr(gu), gu.stride(0), n, f2 // 2, ptr(act), act.stride(0), current_stream()),
              "b2_swiglu_interleaved")
    return act


def argmax_final(val: torch.Tensor, idx: torch.Tensor, parts: int, n_tok: int, ld: int) -> torch.Tensor:
    lib = _lib.cuda_lib()
    out = torch.empty(n_tok, dtype=torch.int32, device=val.device)
    with torch.cuda.device(val.device):
        check(lib.b2_argmax_final(ptr(val), ptr(idx), parts, ld, n_tok, ptr(out), 0, current_stream()), "b2_argmax_final")
    return out


def argmax_rows(logits: torch.Tensor, n_valid: Optional[int] = None) -> torch.Tensor:
    lib = _lib.cuda_lib()
    out = torch.empty(logits.shape[0], dtype=torch.int32, device=logits.device)
    with torch.cuda.device(logits.device):
        check(lib.b2_argmax_rows(ptr(logits), logits.stride(0), logits.shape[0], n_valid or logits.shape[1], ptr(out),
                                 current_stream()), "b2_argmax_rows")
    return out


def sample_rows(logits: torch.Tensor, temperature: torch.Tensor, top_k: Optional[torch.Tensor], top_p: Optional[torch.Tensor],
                min_p: Optional[torch.Tensor], seed: torch.Tensor, position: torch.Tensor, n_valid: Optional[int] = None,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One token per row of fp32 ``logits``: the inverse CDF of the filtered distribution at the Philox uniform of
    ``(seed[row], position[row])``.  ``temperature`` fp32, ``top_k`` int32, ``top_p``/``min_p`` fp32, ``seed`` int64
    (bit pattern of a uint64), ``position`` int32; a row with ``temperature <= 0`` is greedy."""
    lib = _lib.cuda_lib()
    rows = logits.shape[0]
    assert logits.dtype == torch.float32 and logits.stride(1) == 1
    out = torch.empty(rows, dtype=torch.int32, device=logits.device) if out is None else out
    a = _lib.SampleArgs(ptr(logits), logits.stride(0), n_valid or logits.shape[1], ptr(temperature), ptr(top_k), ptr(top_p),
                        ptr(min_p), ptr(seed), ptr(position), ptr(out))
    with torch.cuda.device(logits.device):
        check(lib.b2_sample_rows(a, rows, current_stream()), "b2_sample_rows")
    return out


def spec_accept(ids: torch.Tensor, target: torch.Tensor, row0: torch.Tensor, cnt: torch.Tensor, max_block: int):
    """Longest-prefix acceptance of verify blocks; returns ``(n_emitted [blocks], emitted [blocks, max_block])``.
    Block b covers rows ``row0[b] .. row0[b] + cnt[b] - 1`` (the bonus token, then the drafts); ``target[r]`` is the
    model's own token after row r; draft j + 1 is accepted iff it equals ``target[j]``.  Host tensors take the same rule
    in plain Python (scheduler tests with a stand-in model)."""
    nb = row0.numel()
    if ids.device.type == "cpu":
        n_emit = torch.empty(nb, dtype=torch.int32)
        emitted = torch.zeros(nb, max_block, dtype=torch.int32)
        il, tl = ids.tolist(), target.tolist()
        for b_, (r0, c) in enumerate(zip(row0.tolist(), cnt.tolist())):
            acc = 0
            while acc + 1 < c and il[r0 + acc + 1] == tl[r0 + acc]:
                acc += 1
            for j in range(acc):
                emitted[b_, j] = il[r0 + j + 1]
            emitted[b_, acc] = tl[r0 + acc]
            n_emit[b_] = acc + 1
        return n_emit, emitted
    lib = _lib.cuda_lib()
    n_emit = torch.empty(nb, dtype=torch.int32, device=ids.device)
    emitted = torch.zeros(nb, max_block, dtype=torch.int32, device=ids.device)
    with torch.cuda.device(ids.device):
        check(lib.b2_spec_accept(ptr(ids), ptr(target), ptr(row0), ptr(cnt), nb, ptr(n_emit), ptr(emitted), max_block,
                                 current_stream()), "b2_spec_accept")
    return n_emit, emitted
