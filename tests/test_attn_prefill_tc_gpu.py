"""The tcgen05 prefill attention (``attn_prefill_tc.cu``) against plain fp32 PyTorch causal attention over the same
paged KV cache, and against the split-KV kernel that serves small chunks."""
import math

import pytest
import torch

from agens_engine_b200.ops import attention as A

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _paged(k, v, hkv, perm_seed=0):
    """k, v: [L, hkv, 128] bf16 -> (pool [pages, 2, hkv, 16, 128], block table row) with shuffled page numbers."""
    L = k.shape[0]
    n_pg = (L + 15) // 16
    g = torch.Generator().manual_seed(perm_seed)
    pages = torch.randperm(n_pg + 3, generator=g)[:n_pg]
    pool = torch.zeros(n_pg + 3, 2, hkv, 16, 128, dtype=torch.bfloat16)
    for i in range(n_pg):
        n = min(16, L - 16 * i)
        pool[pages[i], 0, :, :n] = k[16 * i:16 * i + n].transpose(0, 1)
        pool[pages[i], 1, :, :n] = v[16 * i:16 * i + n].transpose(0, 1)
    bt = torch.full((2, n_pg + 2), -1, dtype=torch.int32)
    bt[1, :n_pg] = pages.to(torch.int32)
    return pool, bt


def _ref(q, k, v, pos0, hq, hkv):
    """q [T, hq, 128], k / v [L, hkv, 128] fp32 -> [T, hq, 128]; row t sees keys 0 .. pos0 + t."""
    T = q.shape[0]
    gq = hq // hkv
    kk = k.repeat_interleave(gq, dim=1)           # [L, hq, 128]
    vv = v.repeat_interleave(gq, dim=1)
    s = torch.einsum("thd,lhd->htl", q, kk) / math.sqrt(128.0)
    keys = torch.arange(k.shape[0])[None, None, :]
    lim = (pos0 + torch.arange(T))[None, :, None]
    s = s.masked_fill(keys > lim, float("-inf"))
    p = torch.softmax(s, dim=-1)
    return torch.einsum("htl,lhd->thd", p, vv)


@pytest.mark.parametrize("hq,hkv", [(16, 2), (8, 8), (8, 2)])
@pytest.mark.parametrize("T,pos0", [(64, 0), (200, 0), (96, 333), (37, 1000)])
def test_matches_fp32_reference(hq, hkv, T, pos0):
    torch.manual_seed(hq * 1000 + T + pos0)
    L = pos0 + T
    q = torch.randn(T, hq, 128).to(torch.bfloat16)
    k = torch.randn(L, hkv, 128).to(torch.bfloat16)
    v = torch.randn(L, hkv, 128).to(torch.bfloat16)
    pool, bt = _paged(k, v, hkv, perm_seed=T)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = A.attn_prefill_tc(q.reshape(T, hq * 128).contiguous().to(DEV), pool.to(DEV), bt.to(DEV), 1, pos0, hq, hkv, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    ref = _ref(q.float(), k.float(), v.float(), pos0, hq, hkv)
    err = (out.float().cpu().reshape(T, hq, 128) - ref).abs().max().item()
    assert err < 0.03, err
    # and the split-KV kernel agrees within bf16 rounding of the probabilities
    old = A.attn_prefill(q.reshape(T, hq * 128).contiguous().to(DEV), pool.to(DEV), bt.to(DEV), 1, pos0, hq, hkv, 128,
                         tensor_core=False)
    assert (old.float() - out.float()).abs().max().item() < 0.03


def test_long_context_and_determinism():
    torch.manual_seed(5)
    hq, hkv, T, pos0 = 16, 2, 256, 4096
    L = pos0 + T
    q = torch.randn(T, hq, 128).to(torch.bfloat16)
    k = torch.randn(L, hkv, 128).to(torch.bfloat16)
    v = torch.randn(L, hkv, 128).to(torch.bfloat16)
    pool, bt = _paged(k, v, hkv)
    qd, pd, bd = q.reshape(T, hq * 128).contiguous().to(DEV), pool.to(DEV), bt.to(DEV)
    a = A.attn_prefill_tc(qd, pd, bd, 1, pos0, hq, hkv)
    b = A.attn_prefill_tc(qd, pd, bd, 1, pos0, hq, hkv)
    torch.cuda.synchronize()
    assert torch.equal(a, b)
    ref = _ref(q.float(), k.float(), v.float(), pos0, hq, hkv)
    assert (a.float().cpu().reshape(T, hq, 128) - ref).abs().max().item() < 0.03
