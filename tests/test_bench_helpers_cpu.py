"""CPU checks of the host-side helpers around the kernels: roofline arithmetic of bench.py, convolution geometry,
the eligibility rule of the fused convolution and the prefetch chain of the fused trainer."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def test_roofline_fraction_of_readme_config():
    import bench
    cfg = bench.CONFIGS["readme"]
    r1 = bench.roofline(cfg, 1, 5.0)
    assert r1["nvlink_ms_at_770GBs"] == 0.0
    assert abs(r1["bound_ms"] - (r1["gemm_ms_at_peak"] + r1["optimizer_ms_at_copy_bw"])) < 1e-9
    assert 0.0 < r1["achieved_frac"] < 1.0
    r8 = bench.roofline(cfg, 8, 10.0)
    # a rank moves 3 x (N-1)/N of the rotated weights in bf16 per step
    params = cfg["nlayers"] * (4 * cfg["ninp"] ** 2 + 2 * cfg["ninp"] * cfg["nhid"]) + cfg["vocab"] * cfg["ninp"]
    assert abs(r8["nvlink_ms_at_770GBs"] - 3 * 2 * params * 7 / 8 / 770e9 * 1e3) < 1e-6
    assert r8["optimizer_ms_at_copy_bw"] < r1["optimizer_ms_at_copy_bw"]


def test_conv_geometry_matches_torch():
    from rtp_b200.ops.kernels import conv_out_size
    for (H, W, k, s, p, d) in [(28, 28, 3, 1, 0, 1), (14, 15, 5, 2, 2, 1), (32, 20, 3, 2, 1, 2)]:
        y = torch.nn.functional.conv2d(torch.zeros(1, 1, H, W), torch.zeros(1, 1, k, k), stride=s, padding=p, dilation=d)
        assert conv_out_size(H, W, k, s, p, d) == (y.shape[2], y.shape[3])


def test_fused_conv_eligibility():
    from rtp_b200.module.conv import ColumnParallelConv2d
    from rtp_b200.parallel.engine import fused_conv_ok
    x = torch.zeros(2, 32, 8, 8)
    ok = ColumnParallelConv2d(32, 64, 3, world_size=1, rank=0)
    first = ColumnParallelConv2d(1, 32, 3, world_size=1, rank=0)       # patch length 9: not a legal TMA row pitch
    grouped = ColumnParallelConv2d(32, 64, 3, groups=2, world_size=1, rank=0)
    assert fused_conv_ok(ok, x)
    assert not fused_conv_ok(first, torch.zeros(2, 1, 8, 8))
    assert not fused_conv_ok(grouped, x)
    # on CPU the module keeps evaluating through the functional engine
    y = ok(x)
    assert y.shape == (2, 64, 6, 6)


def test_guard_bands_catch_an_overrun():
    import pytest
    from rtp_b200.utils.guard import check_guards, guarded_empty
    t = guarded_empty((5, 7), torch.float32, device="cpu", band=8, name="fine")
    t.zero_()
    check_guards()
    t = guarded_empty((5, 7), torch.float32, device="cpu", band=8, name="overrun")
    torch.as_strided(t, (1,), (1,), storage_offset=t.storage_offset() + 35).fill_(3.0)   # one element past the end
    with pytest.raises(AssertionError, match="AFTER tensor 'overrun'"):
        check_guards()
