"""Launchers of the hybrid-family kernels (``csrc/kernels/sm100/hybrid_kda.cu``, ``hybrid_misc.cu``): KDA linear
attention pieces, mHC stream boundary, Engram gather, INT8 GEMV / KV helpers and the BCSA far branch."""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from .. import _lib
from .._lib import check, current_stream, ptr

_done = False


def _lib_h():
    global _done
    lib = _lib.cuda_lib()
    if not _done:
        vp, i, l, f = C.c_void_p, C.c_int, C.c_long, C.c_float
        sig = {
            "b2_conv_update": [vp, l, vp, vp, vp, vp, l, i, i, i, i, vp, i, vp],
            "b2_kda_recurrent": [vp, vp, vp, l, l, vp, vp, vp, vp, l, i, i, i, i, i, vp, i, vp],
            "b2_gated_rmsnorm": [vp, l, vp, l, vp, f, vp, l, i, i, vp],
            "b2_mhc_mix": [vp, vp, vp, vp, vp, i, i, i, vp],
            "b2_mhc_combine": [vp, vp, vp, vp, i, i, vp],
            "b2_engram": [vp, i, vp, l, i, i, vp, i, vp],
            "b2_i8_gemv": [vp, vp, vp, l, vp, l, i, i, i, vp],
            "b2_kv_quant_int8": [vp, vp, vp, i, i, vp],
            "b2_kv_dequant_int8": [vp, vp, vp, l, i, vp],
            "b2_block_mean": [vp, vp, l, i, i, vp],
            "b2_bcsa_score": [vp, vp, vp, f, vp, i, i, i, vp],
            "b2_topk_blocks": [vp, i, i, vp, vp, vp],
            "b2_bcsa_gather": [vp, vp, vp, vp, i, i, i, i, i, vp, vp, vp],
            "b2_bcsa_far_attend": [vp, vp, vp, vp, i, i, i, i, f, vp, vp, vp, vp],
        }
        for name, args in sig.items():
            fn = getattr(lib, name)
            fn.argtypes, fn.restype = args, i
        _done = True
    return lib


def _bf(*shape, dev):
    return torch.empty(*shape, dtype=torch.bfloat16, device=dev)


def conv_update(x, state, w, bias=None, n_commit: Optional[int] = None, n_commit_dev=None, silu=True, want_out=True):
    """Causal depthwise conv (width 4) over the T rows of ``x`` [T, dim]; ``state`` [dim, 3] fp32 is advanced by
    ``n_commit`` tokens (default T; -1 leaves it untouched)."""
    T, dim = x.shape
    out = _bf(T, dim, dev=x.device) if want_out else None
    nc = T if n_commit is None else n_commit
    with torch.cuda.device(x.device):
        check(_lib_h().b2_conv_update(ptr(x), x.stride(0), ptr(state), ptr(w), ptr(bias), ptr(out), dim, T, dim, 4, nc,
                                      ptr(n_commit_dev), int(silu), current_stream()), "b2_conv_update")
    return out


def kda_recurrent(q, k, v, g, beta, state, n_commit: Optional[int] = None, n_commit_dev=None, l2norm=True, want_out=True):
    """q, k: bf16 [T, H, 128]; v: bf16 [T, H, V]; g: fp32 [T, H, 128] log decay; beta: fp32 [T, H]; state: fp32
    [H, 128, V] advanced by ``n_commit`` tokens (default T; -1 leaves it untouched).  Returns bf16 [T, H, V]."""
    T, H, K = q.shape
    V = v.shape[2]
    out = _bf(T, H, V, dev=q.device) if want_out else None
    nc = T if n_commit is None else n_commit
    with torch.cuda.device(q.device):
        check(_lib_h().b2_kda_recurrent(ptr(q), ptr(k), ptr(v), H * K, H * V, ptr(g), ptr(beta), ptr(state), ptr(out), H * V, T, H, K,
                                        V, nc, ptr(n_commit_dev), int(l2norm), current_stream()), "b2_kda_recurrent")
    return out


def gated_rmsnorm(o, gate, w, eps=1e-6):
    rows, d = o.shape
    out = torch.empty_like(o)
    with torch.cuda.device(o.device):
        check(_lib_h().b2_gated_rmsnorm(ptr(o), o.stride(0), ptr(gate), gate.stride(0), ptr(w), eps, ptr(out), out.stride(0), rows, d,
                                        current_stream()), "b2_gated_rmsnorm")
    return out


def mhc_mix(H, dyn, statics, iters=10):
    """H: bf16 [T, 4, d]; dyn: fp32 [T, 24]; statics: fp32 [24].  Returns (x bf16 [T, d], coef fp32 [T, 24])."""
    T, _, d = H.shape
    x = _bf(T, d, dev=H.device)
    coef = torch.empty(T, 24, dtype=torch.float32, device=H.device)
    with torch.cuda.device(H.device):
        check(_lib_h().b2_mhc_mix(ptr(H), ptr(dyn), ptr(statics), ptr(coef), ptr(x), T, d, iters, current_stream()), "b2_mhc_mix")
    return x, coef


def mhc_combine(H, y, coef):
    T, _, d = H.shape
    out = torch.empty_like(H)
    with torch.cuda.device(H.device):
        check(_lib_h().b2_mhc_combine(ptr(H), ptr(y), ptr(coef), ptr(out), T, d, current_stream()), "b2_mhc_combine")
    return out


def engram(hist, tables):
    """hist: int32 [T, >= n_orders + 1] (column j = token j steps back, -1 before the start); tables: bf16
    [n_orders, rows, dim] on the device or in mapped pinned host memory.  Returns bf16 [T, n_orders, dim]."""
    T = hist.shape[0]
    n_orders, rows, dim = tables.shape
    out = _bf(T, n_orders, dim, dev=hist.device)
    with torch.cuda.device(hist.device):
        check(_lib_h().b2_engram(ptr(hist), hist.stride(0), ptr(tables), rows, dim, n_orders, ptr(out), T, current_stream()), "b2_engram")
    return out


def engram_rows(hist_row, n_orders: int, rows: int):
    """Host restatement of the hash (tests, table builders)."""
    out = []
    M = (1 << 61) - 1
    for o in range(n_orders):
        h = 0x9E3779B97F4A7C15 & M
        for j in range(o + 1, -1, -1):
            h = (h * 1000003 + (int(hist_row[j]) + 1) * 0x100000001B3) & M
        out.append(h % rows)
    return out


def i8_gemv(W, scale, x):
    n, k = W.shape
    m = x.shape[0]
    y = torch.empty(m, n, dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        check(_lib_h().b2_i8_gemv(ptr(W), ptr(scale), ptr(x), x.stride(0), ptr(y), n, n, k, m, current_stream()), "b2_i8_gemv")
    return y


def kv_quant_int8(x):
    rows, d = x.shape
    q = torch.empty(rows, d, dtype=torch.int8, device=x.device)
    s = torch.empty(rows, dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        check(_lib_h().b2_kv_quant_int8(ptr(x), ptr(q), ptr(s), rows, d, current_stream()), "b2_kv_quant_int8")
    return q, s


def kv_dequant_int8(q, s):
    rows, d = q.shape
    x = _bf(rows, d, dev=q.device)
    with torch.cuda.device(q.device):
        check(_lib_h().b2_kv_dequant_int8(ptr(q), ptr(s), ptr(x), rows, d, current_stream()), "b2_kv_dequant_int8")
    return x


def block_mean(x, blk=4):
    rows, d = x.shape
    out = _bf(rows // blk, d, dev=x.device)
    with torch.cuda.device(x.device):
        check(_lib_h().b2_block_mean(ptr(x), ptr(out), rows // blk, blk, d, current_stream()), "b2_block_mean")
    return out


def bcsa_score(qi, w, kb, scale):
    nb, di = kb.shape
    score = torch.empty(nb, dtype=torch.float32, device=kb.device)
    with torch.cuda.device(kb.device):
        check(_lib_h().b2_bcsa_score(ptr(qi), ptr(w), ptr(kb), scale, ptr(score), nb, qi.shape[0], di, current_stream()), "b2_bcsa_score")
    return score


def topk_blocks(score, k):
    n = score.numel()
    sel = torch.empty(min(n, k), dtype=torch.int32, device=score.device)
    n_sel = torch.zeros(1, dtype=torch.int32, device=score.device)
    with torch.cuda.device(score.device):
        check(_lib_h().b2_topk_blocks(ptr(score), n, k, ptr(sel), ptr(n_sel), current_stream()), "b2_topk_blocks")
    return sel, n_sel


def bcsa_gather(kv_pool, bt_row, sel, n_sel, blk=4):
    _, _, hkv, page, hd = kv_pool.shape
    ms = sel.numel()
    kf, vf = _bf(ms * blk, hkv, hd, dev=kv_pool.device), _bf(ms * blk, hkv, hd, dev=kv_pool.device)
    with torch.cuda.device(kv_pool.device):
        check(_lib_h().b2_bcsa_gather(ptr(kv_pool), ptr(bt_row), ptr(sel), ptr(n_sel), ms, blk, hkv, hd, page, ptr(kf), ptr(vf),
                                      current_stream()), "b2_bcsa_gather")
    return kf, vf


def bcsa_far_attend(q, kf, vf, n_sel, scale, o_loc=None, lse_loc=None, blk=4):
    hq, hd = q.shape
    hkv = kf.shape[1]
    out = _bf(hq, hd, dev=q.device)
    with torch.cuda.device(q.device):
        check(_lib_h().b2_bcsa_far_attend(ptr(q), ptr(kf), ptr(vf), ptr(n_sel), blk, hq, hkv, hd, scale, ptr(o_loc), ptr(lse_loc),
                                          ptr(out), current_stream()), "b2_bcsa_far_attend")
    return out
