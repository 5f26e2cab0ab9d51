"""Out-of-bounds check of the kernels' stores with guard bands: ragged shapes (tiles that hang over the edge of the
output) must leave the canaries around every output untouched."""
import pytest
import torch

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


@pytest.mark.parametrize("M,N,K", [(200, 264, 72), (1000, 1288, 520), (136, 72, 64), (1024, 2048, 2048)])
@pytest.mark.parametrize("layout", ["nt", "nn", "tn"])
def test_gemm_stores_stay_inside_the_output(M, N, K, layout):
    from rtp_b200.ops import gemm as G, _lib
    from rtp_b200.utils.guard import guarded_empty, check_guards
    torch.manual_seed(0)
    a_mn, b_mn = layout == "tn", layout in ("nn", "tn")
    a = torch.randn((K, M) if a_mn else (M, K), device="cuda", dtype=BF)
    b = torch.randn((K, N) if b_mn else (N, K), device="cuda", dtype=BF)
    bias = torch.randn(N, device="cuda", dtype=BF)
    out = guarded_empty((M, N), BF, name=f"gemm {layout} {M}x{N}x{K}")
    G.gemm(a, b, a_mn=a_mn, b_mn=b_mn, out=out, bias=bias, act=1)
    torch.cuda.synchronize()
    _lib.check_status()
    check_guards()
    A = a.float().t() if a_mn else a.float()
    B = b.float().t() if b_mn else b.float()
    ref = torch.relu(A @ B.t() + bias.float())
    assert (out.float() - ref).abs().max().item() <= 2e-2 * ref.abs().max().item()


def test_memory_bound_kernels_stay_inside_their_outputs():
    from rtp_b200.ops import kernels as K
    from rtp_b200.utils.guard import guarded_empty, check_guards
    torch.manual_seed(0)
    M, D = 37, 2048
    x = torch.randn(M, D, device="cuda", dtype=BF)
    sub = torch.randn(M, D, device="cuda", dtype=BF)
    g = torch.ones(D, device="cuda", dtype=BF)
    b = torch.zeros(D, device="cuda", dtype=BF)
    y = guarded_empty((M, D), BF, name="norm y")
    h = guarded_empty((M, D), BF, name="norm h")
    mean = guarded_empty((M,), torch.float32, name="mean")
    rstd = guarded_empty((M,), torch.float32, name="rstd")
    K.norm_fwd(x, sub, g, b, out=y, h_out=h, mean_out=mean, rstd_out=rstd)
    cs = guarded_empty((D,), torch.float32, name="colsum")
    K.colsum(x, cs)
    S, B, H = 32, 3, 5
    qkv = torch.randn(S * B, 3 * H * 64, device="cuda", dtype=BF)
    o = guarded_empty((S * B, H * 64), BF, name="attention out")
    K.attn_small_fwd(qkv, S, B, H, out=o)
    dq = guarded_empty((S * B, 3 * H * 64), BF, name="attention dqkv")
    K.attn_small_bwd(qkv, torch.randn(S * B, H * 64, device="cuda", dtype=BF), S, B, H, out=dq)
    torch.cuda.synchronize()
    check_guards()
    assert torch.isfinite(o.float()).all() and torch.isfinite(dq.float()).all()
