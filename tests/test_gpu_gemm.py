"""tcgen05 GEMM kernel vs a plain PyTorch fp32 reference, for every operand layout the linear layers use
(forward x·Wᵀ, input gradient dy·W, weight gradient dyᵀ·x) and every epilogue option."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(a, b, a_mn, b_mn):
    A = a.float().t() if a_mn else a.float()
    B = b.float().t() if b_mn else b.float()
    return A @ B.t()


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
@pytest.mark.parametrize("shape", [(128, 128, 64, 128), (128, 256, 64, 256), (256, 512, 512, 0),
                                   (992, 1280, 2048, 0), (200, 264, 72, 128)])
def test_gemm_layouts(a_mn, b_mn, shape):
    from rtp_b200.ops import gemm as G, _lib
    M, N, K, bn = shape
    torch.manual_seed(0)
    a = torch.randn((K, M) if a_mn else (M, K), device="cuda", dtype=torch.bfloat16)
    b = torch.randn((K, N) if b_mn else (N, K), device="cuda", dtype=torch.bfloat16)
    out = G.gemm(a, b, a_mn=a_mn, b_mn=b_mn, bn=bn)
    torch.cuda.synchronize()
    _lib.check_status()
    r = _ref(a, b, a_mn, b_mn)
    assert (out.float() - r).abs().max().item() <= 1e-2 * r.abs().max().item()


def test_gemm_epilogues():
    from rtp_b200.ops import gemm as G, _lib
    torch.manual_seed(0)
    M, N, K = 512, 768, 256
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    bias = torch.randn(N, device="cuda", dtype=torch.bfloat16)
    c = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
    mask = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
    base = a.float() @ b.float().t()
    out = G.gemm(a, b, bias=bias, act=G.ACT_RELU, c=c, mask=mask, mask_scale=2.0)
    r = torch.relu(base + c.float() + bias.float()) * (mask.float() > 0) * 2.0
    assert (out.float() - r).abs().max().item() <= 1e-2 * r.abs().max().item()
    out = G.gemm(a, b, act=G.ACT_GELU, out_dtype=torch.float32)
    assert (out - torch.nn.functional.gelu(base)).abs().max().item() < 1e-3
    out = G.gemm(a, b, drop_p=0.25, seed=123, offset=7)
    out2 = G.gemm(a, b, drop_p=0.25, seed=123, offset=7)
    assert torch.equal(out, out2)                      # same (seed, offset) -> same mask
    keep = (out != 0)
    assert abs(keep.float().mean().item() - 0.75) < 0.01
    assert ((out.float() - base / 0.75).abs() * keep).max().item() <= 1e-2 * base.abs().max().item() / 0.75
    step = torch.ones(1, dtype=torch.int64, device="cuda")
    # a device-side step counter changes the mask without changing launch arguments
    import ctypes  # noqa: F401
    _lib.check_status()
