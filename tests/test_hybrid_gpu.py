"""Hybrid-family kernels against plain PyTorch fp32 restatements of the same math (reference kernels:
kernels/src/kda_decode.cu, mhc.cu, engram.cu, i8_gemv.cu, kv_tier.cu, far_decode.cu)."""
import math

import pytest
import torch

from agens_engine_b200.ops import hybrid as Hy

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def bf(x):
    return x.to(torch.bfloat16)


def test_conv_update_and_commit():
    torch.manual_seed(0)
    T, dim = 8, 768
    x = bf(torch.randn(T, dim, device=DEV))
    w = bf(torch.randn(dim, 4, device=DEV) * 0.5)
    st0 = torch.randn(dim, 3, device=DEV)
    hist = torch.cat([st0.T, x.float()], 0)                                   # [3 + T, dim]
    ref = torch.stack([(hist[t:t + 4] * w.float().T).sum(0) for t in range(T)])
    ref = ref * torch.sigmoid(ref)
    st = st0.clone()
    out = Hy.conv_update(x, st, w, n_commit=-1)
    assert torch.equal(st, st0)
    assert (out.float() - ref).abs().max() < 0.03
    # commit 5 accepted tokens (count from the device), then single steps equal the block
    n = torch.tensor([5], dtype=torch.int32, device=DEV)
    Hy.conv_update(x, st, w, n_commit=0, n_commit_dev=n, want_out=False)
    assert torch.equal(st, hist[5:8].T.contiguous())
    st2 = st0.clone()
    singles = torch.cat([Hy.conv_update(x[t:t + 1], st2, w) for t in range(T)])
    assert torch.equal(singles, out)


def kda_ref(q, k, v, g, beta, S):
    T, H, K = q.shape
    outs = []
    S = S.clone().double()
    for t in range(T):
        qt, kt = q[t].double(), k[t].double()
        qt = qt / torch.sqrt((qt * qt).sum(-1, keepdim=True) + 1e-6) / math.sqrt(K)
        kt = kt / torch.sqrt((kt * kt).sum(-1, keepdim=True) + 1e-6)
        S = S * torch.exp(g[t].double())[:, :, None]
        pred = torch.einsum("hk,hkv->hv", kt, S)
        d = beta[t].double()[:, None] * (v[t].double() - pred)
        S = S + kt[:, :, None] * d[:, None, :]
        outs.append(torch.einsum("hk,hkv->hv", qt, S))
    return torch.stack(outs), S


def test_kda_recurrence_decode_verify_commit():
    torch.manual_seed(1)
    T, H, K, V = 8, 4, 128, 128
    q, k = bf(torch.randn(T, H, K, device=DEV)), bf(torch.randn(T, H, K, device=DEV))
    v = bf(torch.randn(T, H, V, device=DEV))
    g = -torch.rand(T, H, K, device=DEV) * 0.2
    beta = torch.sigmoid(torch.randn(T, H, device=DEV))
    S0 = torch.randn(H, K, V, device=DEV) * 0.1
    ref_o, ref_S = kda_ref(q, k, v, g, beta, S0)
    S = S0.clone()
    out = Hy.kda_recurrent(q, k, v, g, beta, S, n_commit=-1)                    # verify: state untouched
    assert torch.equal(S, S0)
    assert (out.double() - ref_o).abs().max() < 0.02 * ref_o.abs().max() + 0.01
    Hy.kda_recurrent(q, k, v, g, beta, S, n_commit=0, n_commit_dev=torch.tensor([3], dtype=torch.int32, device=DEV), want_out=False)
    _, ref_S3 = kda_ref(q[:3], k[:3], v[:3], g[:3], beta[:3], S0)
    assert (S.double() - ref_S3).abs().max() < 1e-3
    S2 = S0.clone()
    singles = torch.cat([Hy.kda_recurrent(q[t:t + 1], k[t:t + 1], v[t:t + 1], g[t:t + 1], beta[t:t + 1], S2) for t in range(T)])
    assert torch.equal(singles, out)                                            # verify rows == decode steps, bit for bit
    assert (S2.double() - ref_S).abs().max() < 1e-3
    # long sequential prefill
    T2 = 300
    q2, k2, v2 = bf(torch.randn(T2, H, K, device=DEV)), bf(torch.randn(T2, H, K, device=DEV)), bf(torch.randn(T2, H, V, device=DEV))
    g2, b2 = -torch.rand(T2, H, K, device=DEV) * 0.1, torch.sigmoid(torch.randn(T2, H, device=DEV))
    S3 = torch.zeros(H, K, V, device=DEV)
    o2 = Hy.kda_recurrent(q2, k2, v2, g2, b2, S3)
    r2, rS = kda_ref(q2, k2, v2, g2, b2, torch.zeros(H, K, V, device=DEV))
    assert (o2.double() - r2).abs().max() < 0.02 * r2.abs().max() + 0.01 and (S3.double() - rS).abs().max() < 2e-3


def test_gated_rmsnorm_and_mhc():
    torch.manual_seed(2)
    rows, d = 37, 128
    o, gate, w = bf(torch.randn(rows, d, device=DEV)), bf(torch.randn(rows, d, device=DEV)), bf(1 + 0.1 * torch.randn(d, device=DEV))
    ref = o.float() * torch.rsqrt((o.float() ** 2).mean(-1, keepdim=True) + 1e-6) * w.float() * torch.sigmoid(gate.float())
    assert (Hy.gated_rmsnorm(o, gate, w).float() - ref).abs().max() < 0.03
    T, d = 5, 1024
    H = bf(torch.randn(T, 4, d, device=DEV))
    dyn, stat = torch.randn(T, 24, device=DEV), torch.randn(24, device=DEV) * 0.3
    x, coef = Hy.mhc_mix(H, dyn, stat)
    z = (dyn + stat).double()
    pre, post, res = torch.sigmoid(z[:, :4]), 2 * torch.sigmoid(z[:, 4:8]), torch.exp(z[:, 8:]).view(T, 4, 4)
    for _ in range(10):
        res = res / res.sum(2, keepdim=True)
        res = res / res.sum(1, keepdim=True)
    assert (coef[:, :4].double() - pre).abs().max() < 1e-5 and (coef[:, 8:].double().view(T, 4, 4) - res).abs().max() < 1e-5
    assert (res.sum(1) - 1).abs().max() < 1e-6                                   # doubly stochastic after the column pass
    xr = torch.einsum("ta,tad->td", pre, H.double())
    assert (x.double() - xr).abs().max() < 0.03
    y = bf(torch.randn(T, d, device=DEV))
    Hn = Hy.mhc_combine(H, y, coef)
    Hr = torch.einsum("tab,tbd->tad", res, H.double()) + post[:, :, None] * y.double()[:, None, :]
    assert (Hn.double() - Hr).abs().max() < 0.05


def test_engram_i8_kvint8_blockmean():
    torch.manual_seed(3)
    T, n_orders, rows, dim = 6, 2, 4096, 512
    tables = bf(torch.randn(n_orders, rows, dim, device=DEV))
    hist = torch.randint(0, 50000, (T, 4), dtype=torch.int32, device=DEV)
    hist[0, 1:] = -1
    hist[1, 2:] = -1
    out = Hy.engram(hist, tables)
    hh = hist.cpu().tolist()
    for t in range(T):
        idx = Hy.engram_rows(hh[t], n_orders, rows)
        for o in range(n_orders):
            ok = all(v >= 0 for v in hh[t][:o + 2])
            exp = tables[o, idx[o]] if ok else torch.zeros(dim, device=DEV, dtype=torch.bfloat16)
            assert torch.equal(out[t, o], exp), (t, o)
    # the table may also live in mapped pinned host memory
    host_tab = tables.cpu().pin_memory()
    n, k, m = 1000, 1024, 3
    W = torch.randint(-127, 128, (n, k), dtype=torch.int8, device=DEV)
    sc = torch.rand(n, device=DEV) * 0.01
    x = bf(torch.randn(m, k, device=DEV))
    ref = (x.float() @ W.float().T) * sc
    assert (Hy.i8_gemv(W, sc, x) - ref).abs().max() < 1e-2 * ref.abs().max()
    kv = bf(torch.randn(64, 128, device=DEV))
    q8, s8 = Hy.kv_quant_int8(kv)
    assert torch.allclose(s8, kv.float().abs().amax(1) / 127, rtol=1e-6)
    back = Hy.kv_dequant_int8(q8, s8)
    assert (back.float() - kv.float()).abs().max() <= s8.max() * 0.51 + 0.02
    bm = Hy.block_mean(kv, 4)
    assert (bm.float() - kv.float().view(16, 4, 128).mean(1)).abs().max() < 0.02


def test_bcsa_far_branch():
    torch.manual_seed(4)
    nb, idxh, di = 3000, 4, 128
    qi, kb = bf(torch.randn(idxh, di, device=DEV)), bf(torch.randn(nb, di, device=DEV))
    w = torch.rand(idxh, device=DEV)
    score = Hy.bcsa_score(qi, w, kb, 0.1)
    ref = (torch.relu(qi.float() @ kb.float().T) * w[:, None]).sum(0) * 0.1
    assert (score - ref).abs().max() < 1e-3 * ref.abs().max() + 1e-4
    score[100:140] = score[7]                                                   # ties: lowest indices win
    sel, n_sel = Hy.topk_blocks(score, 512)
    order = sorted(range(nb), key=lambda i: (-float(score[i]), i))[:512]
    assert int(n_sel) == 512 and sel.cpu().tolist() == sorted(order)
    sel_all, n_all = Hy.topk_blocks(score[:100].contiguous(), 512)
    assert int(n_all) == 100 and sel_all.tolist() == list(range(100))
    # gather + far attention + merge with a local branch == attention over the union of rows
    hq, hkv, hd, page, blk = 8, 2, 128, 16, 4
    n_pages = 64
    pool = bf(torch.randn(n_pages, 2, hkv, page, hd, device=DEV))
    bt = torch.randperm(n_pages, device=DEV).to(torch.int32)
    nblk = n_pages * page // blk
    sc2 = torch.randn(nblk, device=DEV)
    sel2, ns2 = Hy.topk_blocks(sc2, 32)
    kf, vf = Hy.bcsa_gather(pool, bt, sel2, ns2, blk)
    rows = torch.cat([torch.arange(b * blk, (b + 1) * blk) for b in sel2.cpu().tolist()])
    pg, inn = bt.cpu()[rows // page].long(), rows % page
    assert torch.equal(kf, pool[pg.to(DEV), 0][:, :, :, :].permute(0, 1, 2, 3)[torch.arange(len(rows)), :, inn.to(DEV)])
    q = bf(torch.randn(hq, hd, device=DEV))
    kl, vl = bf(torch.randn(50, hkv, hd, device=DEV)), bf(torch.randn(50, hkv, hd, device=DEV))
    scale = 1 / math.sqrt(hd)

    def attn(kk, vv):
        kk, vv = kk.float().repeat_interleave(hq // hkv, 1), vv.float().repeat_interleave(hq // hkv, 1)
        s = torch.einsum("hd,nhd->hn", q.float(), kk) * scale
        return torch.einsum("hn,nhd->hd", torch.softmax(s, -1), vv), torch.logsumexp(s, -1)

    o_loc, lse_loc = attn(kl, vl)
    out = Hy.bcsa_far_attend(q, kf, vf, ns2, scale, o_loc.contiguous(), lse_loc.contiguous(), blk)
    ref, _ = attn(torch.cat([kl, kf]), torch.cat([vl, vf]))
    assert (out.float() - ref).abs().max() < 0.03
