"""GPU gates of the paged decode / verify attention and the fused ops around it, against plain fp32 PyTorch."""
import math

import pytest
import torch

from agens_engine_b200.ops import attention as A
from agens_engine_b200.ops import basic

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _ref_attn(q, k, v, pos, hq, hkv, hd):
    """q [hq, hd], k/v [L, hkv, hd] fp32; keys 0..pos."""
    gq = hq // hkv
    out = torch.empty(hq, hd)
    for h in range(hq):
        kk = k[: pos + 1, h // gq]
        s = (kk @ q[h]) / math.sqrt(hd)
        p = torch.softmax(s, dim=0)
        out[h] = p @ v[: pos + 1, h // gq]
    return out


@pytest.mark.parametrize("hq,hkv,hd", [(16, 2, 128), (4, 2, 64), (8, 8, 128)])
@pytest.mark.parametrize("split", [32, 64])
def test_decode_and_verify_attention(hq, hkv, hd, split):
    torch.manual_seed(0)
    n_seq, n_pages = 3, 64
    lens = [37, 130, 5]           # kv length BEFORE the new tokens
    new = [1, 4, 8]               # query tokens per sequence (decode, verify x4, verify x8)
    pool = torch.zeros(n_pages, 2, hkv, 16, hd, dtype=torch.bfloat16)
    bt = torch.full((n_seq, 16), -1, dtype=torch.int32)
    perm = torch.randperm(n_pages).tolist()
    ks, vs = [], []
    for s in range(n_seq):
        total = lens[s] + new[s]
        k = torch.randn(total, hkv, hd).to(torch.bfloat16)
        v = torch.randn(total, hkv, hd).to(torch.bfloat16)
        ks.append(k.float()); vs.append(v.float())
        for p in range((total + 15) // 16):
            page = perm.pop()
            bt[s, p] = page
            nrow = min(16, total - p * 16)
            pool[page, 0, :, :nrow] = k[p * 16: p * 16 + nrow].permute(1, 0, 2)
            pool[page, 1, :, :nrow] = v[p * 16: p * 16 + nrow].permute(1, 0, 2)
    tok_pos, tok_seq, g0, gc = [], [], [], []
    for s in range(n_seq):
        g0.append(len(tok_pos)); gc.append(new[s])
        for j in range(new[s]):
            tok_pos.append(lens[s] + j); tok_seq.append(s)
    n_tok = len(tok_pos)
    q = torch.randn(n_tok, hq * hd).to(torch.bfloat16)
    max_splits = (max(l + n for l, n in zip(lens, new)) + split - 1) // split
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    out = A.attn_decode(q.to(DEV), pool.to(DEV), bt.to(DEV), i32(g0), i32(gc), i32(tok_pos), i32(tok_seq), hq, hkv, hd,
                        split, max_splits)
    torch.cuda.synchronize()
    for t in range(n_tok):
        ref = _ref_attn(q[t].float().reshape(hq, hd), ks[tok_seq[t]], vs[tok_seq[t]], tok_pos[t], hq, hkv, hd)
        err = (out[t].float().cpu().reshape(hq, hd) - ref).abs().max().item()
        assert err < 0.02, (t, err)
    # verify rows are bit-identical to the same rows computed as single decode steps
    for t in range(n_tok):
        o1 = A.attn_decode(q[t:t + 1].to(DEV), pool.to(DEV), bt.to(DEV), i32([0]), i32([1]), i32([tok_pos[t]]),
                           i32([tok_seq[t]]), hq, hkv, hd, split, max_splits)
        assert torch.equal(o1[0], out[t]), t


def test_rope_kvstore_matches_torch():
    torch.manual_seed(1)
    hq, hkv, hd, n_tok = 8, 2, 128, 5
    theta = 1e6
    qkv = torch.randn(n_tok, (hq + 2 * hkv) * hd).to(torch.bfloat16)
    pos = torch.tensor([0, 1, 17, 300, 70000], dtype=torch.int32)
    seq = torch.tensor([0, 0, 0, 1, 2], dtype=torch.int32)
    bt = torch.full((3, 70000 // 16 + 2), -1, dtype=torch.int32)
    bt[0, 0], bt[0, 1], bt[1, 300 // 16], bt[2, 70000 // 16] = 3, 1, 2, 0
    pool = torch.zeros(4, 2, hkv, 16, hd, dtype=torch.bfloat16, device=DEV)
    q_out = torch.empty(n_tok, hq * hd, dtype=torch.bfloat16, device=DEV)
    inv = basic.rope_inv_freq(hd, theta, DEV)
    st = basic.rope_kvstore(qkv.to(DEV), hq, hkv, hd, inv, pos.to(DEV), seq.to(DEV), bt.to(DEV), pool, q_out)
    assert st.item() == 0

    def rope(x, p):   # x [heads, hd] fp32
        ang = p * inv.cpu().float()
        c, s = torch.cos(ang), torch.sin(ang)
        a, b = x[:, : hd // 2], x[:, hd // 2:]
        return torch.cat([a * c - b * s, b * c + a * s], -1)

    for t in range(n_tok):
        row = qkv[t].float().reshape(hq + 2 * hkv, hd)
        qr = rope(row[:hq], float(pos[t]))
        assert (q_out[t].float().cpu().reshape(hq, hd) - qr).abs().max() < 0.03
        kr = rope(row[hq:hq + hkv], float(pos[t]))
        page = bt[seq[t], pos[t] // 16].item()
        got_k = pool[page, 0, :, pos[t] % 16].float().cpu()
        got_v = pool[page, 1, :, pos[t] % 16].float().cpu()
        assert (got_k - kr).abs().max() < 0.03
        assert torch.equal(got_v, row[hq + hkv:])


def test_rmsnorm_embed_swiglu():
    torch.manual_seed(2)
    d, n = 1024, 6
    x = torch.randn(n, d).to(torch.bfloat16).to(DEV)
    r = torch.randn(n, d).to(torch.bfloat16).to(DEV)
    w = (1 + 0.1 * torch.randn(d)).to(torch.bfloat16).to(DEV)
    y = basic.rmsnorm(x, w, 1e-6)
    xf = x.float()
    ref = xf * torch.rsqrt((xf ** 2).mean(-1, keepdim=True) + 1e-6) * w.float()
    assert (y.float() - ref).abs().max() < 0.03
    y2, xo = basic.rmsnorm(x, w, 1e-6, resid=r)
    s = (x.float() + r.float()).to(torch.bfloat16)
    assert torch.equal(xo, s)
    sf = s.float()
    assert (y2.float() - sf * torch.rsqrt((sf ** 2).mean(-1, keepdim=True) + 1e-6) * w.float()).abs().max() < 0.03
    table = torch.randn(100, d).to(torch.bfloat16).to(DEV)
    ids = torch.tensor([3, 99, 0], dtype=torch.int32, device=DEV)
    ss = torch.zeros(64, device=DEV)
    h = basic.embed(ids, table, ss)
    assert torch.equal(h, table[ids.long()])
    assert torch.allclose(ss[:3], (h.float() ** 2).sum(-1), rtol=1e-5)
    gu = torch.randn(n, 512).to(torch.bfloat16).to(DEV)
    act = basic.swiglu_interleaved(gu)
    g = gu.reshape(n, 32, 2, 8)[:, :, 0].reshape(n, 256).float()
    u = gu.reshape(n, 32, 2, 8)[:, :, 1].reshape(n, 256).float()
    assert (act.float() - torch.nn.functional.silu(g) * u).abs().max() < 0.03


def test_multi_axis_rope_matches_reference():
    """Frequency pair i rotates by the position of its axis (time / height / width); text rows equal plain RoPE."""
    from agens_engine_b200.ops import basic
    torch.manual_seed(5)
    dev = "cuda:0"
    n, hq, hkv, hd = 9, 4, 2, 64
    qkv = torch.randn(n, (hq + 2 * hkv) * hd, device=dev).to(torch.bfloat16)
    inv = basic.rope_inv_freq(hd, 1e6, dev)
    axis = basic.mrope_pair_axis(hd, [11, 11, 10], True, dev)
    assert axis[:7].tolist() == [0, 1, 2, 0, 1, 2, 0] and int((axis == 2).sum()) == 10
    pos3 = torch.randint(0, 50, (3, n), dtype=torch.int32, device=dev)
    pos3[:, :3] = pos3[0, :3]                                   # text rows: same value on every axis
    tok_pos = torch.arange(n, dtype=torch.int32, device=dev)
    seq = torch.zeros(n, dtype=torch.int32, device=dev)
    bt = torch.arange(4, dtype=torch.int32, device=dev)[None, :]
    pool = torch.zeros(4, 2, hkv, 16, hd, dtype=torch.bfloat16, device=dev)
    q = torch.empty(n, hq * hd, dtype=torch.bfloat16, device=dev)
    basic.rope_kvstore_m(qkv.clone(), hq, hkv, hd, inv, tok_pos, pos3.contiguous(), axis, seq, bt, pool, q)
    half = hd // 2
    pp = pos3[axis.long()].T.float()                             # [n, half]: position per pair
    ang = pp * inv[None, :]
    x = qkv[:, :hq * hd].float().view(n, hq, hd)
    ref = torch.cat([x[..., :half] * torch.cos(ang)[:, None] - x[..., half:] * torch.sin(ang)[:, None],
                     x[..., half:] * torch.cos(ang)[:, None] + x[..., :half] * torch.sin(ang)[:, None]], -1)
    assert (q.float().view(n, hq, hd) - ref).abs().max() < 0.02
    q1 = torch.empty_like(q)
    pool1 = torch.zeros_like(pool)
    basic.rope_kvstore(qkv.clone(), hq, hkv, hd, inv, tok_pos, seq, bt, pool1, q1, rope_pos=pos3[0].contiguous())
    assert torch.equal(q1[:3], q[:3]) and torch.equal(pool1[0, 0, :, :3], pool[0, 0, :, :3])


@pytest.mark.parametrize("hq,hkv,hd", [(16, 2, 128), (4, 2, 64)])
def test_shared_kv_ring_is_bit_identical(hq, hkv, hd):
    """The CTA-shared K/V ring (prefill, verify blocks) gives exactly the rows of the per-warp kernel."""
    from agens_engine_b200.ops import attention as A
    torch.manual_seed(6)
    dev = "cuda:0"
    T, pos0, n_pages = 77, 130, 32
    pool = torch.randn(n_pages, 2, hkv, 16, hd, device=dev).to(torch.bfloat16)
    bt = torch.randperm(n_pages, device=dev).to(torch.int32)[None, :]
    q = torch.randn(T, hq * hd, device=dev).to(torch.bfloat16)
    g0, gc, pos, seqv = A.prefill_groups(T, pos0, 0, dev)
    splits = (pos0 + T + 63) // 64
    st = torch.zeros(1, dtype=torch.int32, device=dev)
    a = A.attn_decode(q, pool, bt, g0, gc, pos, seqv, hq, hkv, hd, 64, splits, status=st, shared_kv=False)
    b = A.attn_decode(q, pool, bt, g0, gc, pos, seqv, hq, hkv, hd, 64, splits, status=st, shared_kv=True)
    torch.cuda.synchronize()
    assert int(st.item()) == 0 and torch.equal(a, b)
