"""Mixed-bit tensor-core GEMM (tcgen05, in-kernel dequantisation) against the fp32 dequantised reference, for every
bit width and group size, split-k and single-slice shapes, all epilogues, and run-to-run determinism."""
import pytest
import torch

from agens_engine_b200 import _lib
from agens_engine_b200.ops import linear as L
from agens_engine_b200.utils import quant

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _lin(n, k, bits, group, seed=0):
    torch.manual_seed(seed)
    w = torch.randn(n, k) * 0.05
    ql = quant.quantize(w, bits, group)
    return L.WqLinear.from_quant(ql, DEV), ql.dequant().to(DEV)


@pytest.mark.parametrize("bits,group", [(4, 128), (3, 128), (2, 128), (4, 64), (3, 64), (2, 64)])
@pytest.mark.parametrize("n,k,m", [(1280, 1024, 16), (256, 5120, 9), (4096 + 32, 512, 40), (640, 2048, 256)])
def test_mm_matches_dequant_reference(bits, group, n, k, m):
    lin, wd = _lin(n, k, bits, group)
    ws = L.GemvWorkspace(DEV)
    torch.manual_seed(1)
    x = torch.randn(m, k, device=DEV).to(torch.bfloat16)
    y = L.mm(lin, x, ws, epi=_lib.EPI_F32)
    ref = x.float() @ wd.T
    torch.cuda.synchronize()
    assert int(ws.status.item()) == 0
    err = (y - ref).abs().max().item()
    assert err < 2e-3 * ref.abs().max().item() + 2e-3, err
    y2 = L.mm(lin, x, ws, epi=_lib.EPI_F32)
    assert torch.equal(y, y2)
    # a row does not depend on how many rows travel with it
    y3 = L.mm(lin, x[: max(1, m // 2)].contiguous(), ws, epi=_lib.EPI_F32)
    assert torch.equal(y3, y[: max(1, m // 2)])


def test_mm_epilogues_match_gemv_semantics():
    n, k, m = 2048, 1024, 24
    lin, wd = _lin(n, k, 4, 128, seed=3)
    ws = L.GemvWorkspace(DEV)
    torch.manual_seed(2)
    h = torch.randn(m, k, device=DEV).to(torch.bfloat16)
    normw = (1 + 0.1 * torch.randn(k, device=DEV)).to(torch.bfloat16)
    ss = torch.zeros(4, L.SS_LD, device=DEV)
    ss[0, :m] = (h.float() ** 2).sum(1)
    xn = (h.float() * torch.rsqrt((h.float() ** 2).mean(1, keepdim=True) + 1e-6) * normw.float()).to(torch.bfloat16)
    # norm prologue + store
    y = L.mm(lin, h, ws, pro=_lib.PRO_NORM, ss_in=ss, ss_parts=1, norm_w=normw, eps=1e-6)
    ref = xn.float() @ wd.T
    assert (y.float() - ref).abs().max() < 0.02 * ref.abs().max() + 0.02
    # residual + statistics
    resid = torch.randn(m, n, device=DEV).to(torch.bfloat16)
    ss_out = torch.zeros(n // 32, L.SS_LD, device=DEV)
    y = L.mm(lin, xn, ws, epi=_lib.EPI_RESID, resid=resid, ss_out=ss_out)
    assert (y.float() - (ref + resid.float())).abs().max() < 0.03 * ref.abs().max() + 0.03
    assert torch.allclose(ss_out[:, :m].sum(0), (y.float() ** 2).sum(1), rtol=1e-3)
    # SwiGLU over interleaved gate / up rows (8 + 8 per 16-row block)
    act = L.mm(lin, xn, ws, epi=_lib.EPI_SWIGLU)
    r = ref.to(torch.bfloat16).float().view(m, n // 16, 2, 8)
    exp = (torch.nn.functional.silu(r[:, :, 0]) * r[:, :, 1]).reshape(m, n // 2)
    assert (act.float() - exp).abs().max() < 0.03 * exp.abs().max() + 0.02
    # argmax partials (+ logits)
    av = torch.empty(n // 32, L.SS_LD, device=DEV)
    ai = torch.empty(n // 32, L.SS_LD, dtype=torch.int32, device=DEV)
    lg = torch.empty(m, n, device=DEV)
    L.mm(lin, xn, ws, epi=_lib.EPI_ARGMAX, amax_val=av, amax_idx=ai, n_valid=n - 40, yf=lg)
    best = av[:, :m].max(0)
    idx = ai[best.indices, torch.arange(m, device=DEV)]
    assert torch.equal(idx.long(), lg[:, : n - 40].argmax(1))
    torch.cuda.synchronize()
    assert int(ws.status.item()) == 0
