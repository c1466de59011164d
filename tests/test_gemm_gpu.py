"""tcgen05 GEMM vs plain fp32 PyTorch (tile edges in M, N and K; residual epilogue; fp32 output)."""
import pytest
import torch

from agens_engine_b200.ops import gemm as G

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (128, 256, 512), (200, 512, 520), (17, 264, 128), (1024, 1280, 1024),
                                   (300, 5120, 2048)])
def test_gemm_matches_fp32(M, N, K):
    torch.manual_seed(M + N + K)
    a = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    b = (torch.randn(N, K, device=DEV) * 0.05).to(torch.bfloat16)
    st = torch.zeros(1, dtype=torch.int32, device=DEV)
    d = G.gemm_bf16(a, b, status=st)
    ref = a.float() @ b.float().t()
    assert st.item() == 0
    assert (d.float() - ref).abs().max().item() < 0.02 * ref.abs().max().item() + 1e-3
    d32 = G.gemm_bf16(a, b, out_f32=True, status=st)
    assert (d32 - ref).abs().max().item() < 2e-3 * ref.abs().max().item() + 1e-4


def test_gemm_residual_and_strides():
    torch.manual_seed(3)
    M, N, K = 192, 768, 256
    abig = torch.randn(M, K + 64, device=DEV).to(torch.bfloat16)
    a = abig[:, :K]
    b = (torch.randn(N, K, device=DEV) * 0.05).to(torch.bfloat16)
    r = torch.randn(M, N, device=DEV).to(torch.bfloat16)
    d = G.gemm_bf16(a, b, resid=r)
    ref = a.float() @ b.float().t() + r.float()
    assert (d.float() - ref).abs().max().item() < 0.02 * ref.abs().max().item()


def test_gemm_deterministic():
    torch.manual_seed(4)
    a = torch.randn(256, 1024, device=DEV).to(torch.bfloat16)
    b = torch.randn(512, 1024, device=DEV).to(torch.bfloat16)
    d0 = G.gemm_bf16(a, b)
    for _ in range(5):
        assert torch.equal(G.gemm_bf16(a, b), d0)
