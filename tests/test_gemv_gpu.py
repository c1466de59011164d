"""GPU gates of the mixed-bit GEMV (model: the reference's kernels/bench/test_w4.cu and test_wq.cu: GEMV vs a
high-precision reference, batched == single bitwise, repack round trip)."""
import pytest
import torch

from agens_engine_b200 import _lib
from agens_engine_b200.ops import linear as L
from agens_engine_b200.utils import quant

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _mk(n, k, bits, group, seed=0, ks=None):
    torch.manual_seed(seed)
    w = torch.randn(n, k) * 0.02
    ql = quant.quantize(w, bits, group)
    return ql, L.WqLinear.from_quant(ql, DEV, ks=ks)


def _ref(ql, x):
    return x.float().cpu().double() @ ql.dequant().double().t()


@pytest.mark.parametrize("bits", [2, 3, 4])
@pytest.mark.parametrize("group", [64, 128])
@pytest.mark.parametrize("ks", [1, 2, 8])
def test_gemv_matches_fp64(bits, group, ks):
    n, k = 160, 1024
    ql, lin = _mk(n, k, bits, group, ks=ks)
    ws = L.GemvWorkspace(DEV)
    ws.mm_min_rows = 33          # these tests exercise the GEMV at every row count
    for m in (1, 3, 8, 13, 32):
        x = (torch.randn(m, k) * 1.5).to(torch.bfloat16).to(DEV)
        y = L.gemv(lin, x, ws, epi=_lib.EPI_F32)
        ref = _ref(ql, x)
        err = (y.cpu().double() - ref).abs().max().item()
        assert err < 2e-3 * ref.abs().max().item() + 1e-4, (bits, group, m, err)


@pytest.mark.parametrize("bits", [2, 3, 4])
def test_dequant_kernel_matches_cpu(bits):
    ql, lin = _mk(64, 512, bits, 128, seed=3)
    d = lin.dequant().float().cpu()
    assert torch.equal(d, ql.dequant().to(torch.bfloat16).float())
    assert torch.equal(lin.dequant_cpu(), ql.dequant())


@pytest.mark.parametrize("bits", [2, 3, 4])
@pytest.mark.parametrize("sym", [False, True])
def test_device_repack_matches_cpu_pack(bits, sym):
    torch.manual_seed(5)
    n, k, group = 64, 512, 64
    w = torch.randn(n, k) * 0.02
    ql = quant.quantize(w, bits, group, symmetric=sym, scale_dtype=torch.bfloat16 if sym else torch.float16)
    packed = quant.pack_stream(ql.codes, bits)
    lin = L.WqLinear.from_checkpoint(packed, ql.scale.to(torch.bfloat16) if sym else ql.scale,
                                     None if sym else ql.zero, n, k, bits, group, DEV)
    assert torch.equal(lin.wq.cpu(), quant.pack_fm(ql).reshape(-1))


def test_rows_do_not_depend_on_batch():
    """Batch invariance: a token's output bits are the same at m = 1, inside m = 8 and inside m = 16."""
    for bits in (2, 3, 4):
        ql, lin = _mk(128, 2048, bits, 128, seed=bits, ks=2)
        ws = L.GemvWorkspace(DEV)
        ws.mm_min_rows = 33          # these tests exercise the GEMV at every row count
        x = torch.randn(16, 2048).to(torch.bfloat16).to(DEV)
        y16 = L.gemv(lin, x, ws, epi=_lib.EPI_F32)
        y8 = L.gemv(lin, x[:8].contiguous(), ws, epi=_lib.EPI_F32)
        y1 = L.gemv(lin, x[5:6].contiguous(), ws, epi=_lib.EPI_F32)
        assert torch.equal(y16[:8], y8)
        assert torch.equal(y16[5:6], y1)
        lin4 = L.WqLinear(lin.n, lin.k, lin.bits, lin.group, lin.wq, lin.ks, rb=4)
        assert torch.equal(L.gemv(lin4, x[:8].contiguous(), ws, epi=_lib.EPI_F32), y8)
        x32 = torch.cat([x, x], 0)
        y32 = L.gemv(lin, x32, ws, epi=_lib.EPI_F32)
        assert torch.equal(y32[:16], y16) and torch.equal(y32[16:], y16)


def test_gemv_is_deterministic():
    ql, lin = _mk(256, 4096, 3, 128, seed=9, ks=4)
    ws = L.GemvWorkspace(DEV)
    ws.mm_min_rows = 33          # these tests exercise the GEMV at every row count
    x = torch.randn(4, 4096).to(torch.bfloat16).to(DEV)
    y0 = L.gemv(lin, x, ws, epi=_lib.EPI_F32)
    for _ in range(20):
        assert torch.equal(L.gemv(lin, x, ws, epi=_lib.EPI_F32), y0)


def test_norm_prologue_and_residual_epilogue():
    torch.manual_seed(11)
    d, n = 1024, 256
    ql, lin = _mk(n, d, 4, 128, seed=1)
    qlo, lino = _mk(d, n, 4, 128, seed=2, ks=1)
    ws = L.GemvWorkspace(DEV)
    ws.mm_min_rows = 33          # these tests exercise the GEMV at every row count
    m = 3
    h = torch.randn(m, d).to(torch.bfloat16).to(DEV)
    nw = (1 + 0.1 * torch.randn(d)).to(torch.bfloat16).to(DEV)
    ss = torch.zeros(4, L.SS_LD, dtype=torch.float32, device=DEV)
    hf = h.float()
    # partial sums of squares over 4 column slices
    for p in range(4):
        ss[p, :m] = (hf[:, p * 256:(p + 1) * 256] ** 2).sum(-1)
    y = L.gemv(lin, h, ws, pro=_lib.PRO_NORM, ss_in=ss, ss_parts=4, norm_w=nw, eps=1e-6, epi=_lib.EPI_F32)
    xn = (hf * torch.rsqrt((hf ** 2).mean(-1, keepdim=True) + 1e-6) * nw.float()).to(torch.bfloat16)
    ref = _ref(ql, xn)
    assert (y.cpu().double() - ref).abs().max().item() < 3e-3 * ref.abs().max().item() + 1e-4
    # residual epilogue: y = bf16(acc + resid), ss_out = per panel sums of squares of y
    x2 = torch.randn(m, n).to(torch.bfloat16).to(DEV)
    resid = torch.randn(m, d).to(torch.bfloat16).to(DEV)
    ss_out = torch.zeros(lino.n_panels(), L.SS_LD, dtype=torch.float32, device=DEV)
    out = L.gemv(lino, x2, ws, epi=_lib.EPI_RESID, resid=resid, ss_out=ss_out)
    ref2 = (_ref(qlo, x2) + resid.float().cpu().double())
    assert (out.float().cpu().double() - ref2).abs().max().item() < 0.02 * ref2.abs().max().item()
    tot = ss_out[:, :m].sum(0).cpu()
    assert torch.allclose(tot, (out.float() ** 2).sum(-1).cpu(), rtol=1e-4)


def test_swiglu_epilogue():
    torch.manual_seed(12)
    f, d, m = 256, 512, 5
    gate = torch.randn(f, d) * 0.05
    up = torch.randn(f, d) * 0.05
    ql = quant.quantize(quant.interleave_gate_up(gate, up), 4, 128)
    lin = L.WqLinear.from_quant(ql, DEV, ks=2)
    x = torch.randn(m, d).to(torch.bfloat16).to(DEV)
    act = L.gemv(lin, x, L.GemvWorkspace(DEV), epi=_lib.EPI_SWIGLU)
    wd = ql.dequant().reshape(f // 8, 16, d)
    g = (x.float().cpu() @ wd[:, :8].reshape(f, d).t()).to(torch.bfloat16).float()
    u = (x.float().cpu() @ wd[:, 8:].reshape(f, d).t()).to(torch.bfloat16).float()
    ref = (torch.nn.functional.silu(g) * u)
    assert (act.float().cpu() - ref).abs().max().item() < 0.02 * ref.abs().max().item() + 1e-3


def test_argmax_epilogue():
    from agens_engine_b200.ops import basic
    torch.manual_seed(13)
    n, d, m = 1000 * 16, 512, 4
    ql, lin = _mk(n, d, 4, 128, seed=4, ks=2)
    x = torch.randn(m, d).to(torch.bfloat16).to(DEV)
    val = torch.empty(lin.n_panels(), L.SS_LD, dtype=torch.float32, device=DEV)
    idx = torch.empty(lin.n_panels(), L.SS_LD, dtype=torch.int32, device=DEV)
    logits = torch.empty(m, n, dtype=torch.float32, device=DEV)
    L.gemv(lin, x, L.GemvWorkspace(DEV), epi=_lib.EPI_ARGMAX, amax_val=val, amax_idx=idx, n_valid=n - 100, yf=logits)
    ids = basic.argmax_final(val, idx, lin.n_panels(), m, L.SS_LD)
    assert torch.equal(ids.long().cpu(), logits[:, : n - 100].argmax(-1).cpu())
    assert torch.equal(basic.argmax_rows(logits, n - 100).long().cpu(), logits[:, : n - 100].argmax(-1).cpu())


def test_random_init_on_device_is_a_valid_quantisation():
    lin = L.WqLinear.random(64, 512, 3, 128, DEV, seed=42)
    w = lin.dequant_cpu()
    assert abs(w.std().item() - 0.02) < 0.004 and abs(w.mean().item()) < 0.002
    assert torch.equal(lin.dequant().float().cpu(), w.to(torch.bfloat16).float())
