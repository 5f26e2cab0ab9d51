"""Single-kernel cases for timing and profiling (used by the ncu summaries under profiles/).

    python -m rtp_b200.bench.kernel_case gemm --m 8192 --n 4096 --k 4096 --layout nt --iters 5
    python -m rtp_b200.bench.kernel_case norm_fwd --m 65536 --d 2048
    python -m rtp_b200.bench.kernel_case adam --n 200000000

Every case allocates inputs larger than the 126 MB L2 (or cycles through several copies), runs 2 warm-up launches and
``--iters`` timed launches (CUDA events) and prints achieved TFLOP/s or GB/s next to the measured peaks of
MEASURED_PEAKS.json when that file is present."""
import argparse
import json
import os

import torch


def _peaks():
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    try:
        with open(p) as f:
            d = json.load(f)
        return d.get("hbm_gbs", 6650.0), d.get("bf16_tflops", 1590.0), "measured"
    except Exception:
        return 6650.0, 1590.0, "fallback"


def _time(fn, iters, warm=3):
    for i in range(warm):
        fn(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(iters):
        fn(warm + i)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("case", choices=["gemm", "norm_fwd", "norm_bwd", "ce", "adam", "attn_fwd", "attn_bwd", "colsum",
                                     "embed", "gate", "rope", "im2col", "flash_fwd", "flash_bwd"])
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--full", action="store_true", help="flash cases: full instead of causal attention")
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--d", type=int, default=2048)
    ap.add_argument("--layout", default="nt", choices=["nt", "nn", "tn"])
    ap.add_argument("--bn", type=int, default=0)
    ap.add_argument("--bias", action="store_true")
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--copies", type=int, default=4, help="operand copies cycled through so that inputs are cold")
    ap.add_argument("--seq", type=int, default=32)
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--heads", type=int, default=32)
    a = ap.parse_args(argv)
    from ..ops import gemm as G, kernels as K, _lib
    dev, bf = "cuda", torch.bfloat16
    hbm, tf, src = _peaks()
    torch.manual_seed(0)
    if a.case == "gemm":
        M, N, Kd = a.m, a.n, a.k
        a_mn = a.layout == "tn"
        b_mn = a.layout in ("nn", "tn")
        As = [torch.randn((Kd, M) if a_mn else (M, Kd), device=dev, dtype=bf) for _ in range(a.copies)]
        Bs = [torch.randn((Kd, N) if b_mn else (N, Kd), device=dev, dtype=bf) for _ in range(a.copies)]
        out = torch.empty(M, N, device=dev, dtype=bf)
        bias = torch.randn(N, device=dev, dtype=bf) if a.bias else None
        ms = _time(lambda i: G.gemm(As[i % a.copies], Bs[i % a.copies], a_mn=a_mn, b_mn=b_mn, out=out, bn=a.bn,
                                    bias=bias), a.iters)
        _lib.check_status()
        t = 2.0 * M * N * Kd / ms / 1e9
        print(json.dumps({"case": "gemm", "layout": a.layout, "M": M, "N": N, "K": Kd, "us": ms * 1e3, "tflops": t,
                          "frac_of_cublas_peak": t / tf, "peaks": src}))
        return
    if a.case in ("norm_fwd", "norm_bwd"):
        M, D = a.m * 8, a.d
        x = torch.randn(M, D, device=dev, dtype=bf)
        sub = torch.randn(M, D, device=dev, dtype=bf)
        g = torch.ones(D, device=dev, dtype=bf)
        b = torch.zeros(D, device=dev, dtype=bf)
        if a.case == "norm_fwd":
            ms = _time(lambda i: K.norm_fwd(x, sub, g, b, drop_p=0.1, seed=1, offset=i), a.iters)
            nbytes = 4 * M * D * 2
        else:
            y, h, mean, rstd = K.norm_fwd(x, sub, g, b)
            ms = _time(lambda i: K.norm_bwd(x, h, g, mean, rstd, drop_p=0.1, seed=1, offset=i), a.iters)
            nbytes = 4 * M * D * 2
        print(json.dumps({"case": a.case, "M": M, "D": D, "us": ms * 1e3, "GBs": nbytes / ms / 1e6,
                          "frac_of_copy_peak": nbytes / ms / 1e6 / hbm, "peaks": src}))
        return
    if a.case == "ce":
        M, V = a.m, 10240
        lg = [torch.randn(M, V, device=dev, dtype=bf) for _ in range(2)]
        t = torch.randint(0, V, (M,), device=dev)
        ms = _time(lambda i: K.cross_entropy_(lg[i % 2], t), a.iters)
        nbytes = M * V * 2 * 4        # three reads + one write of the row
        print(json.dumps({"case": "ce", "M": M, "V": V, "us": ms * 1e3, "GBs": nbytes / ms / 1e6,
                          "frac_of_copy_peak": nbytes / ms / 1e6 / hbm, "peaks": src}))
        return
    if a.case == "adam":
        n = a.n * 1024 * 16 if a.n < 1 << 20 else a.n
        p = torch.randn(n, device=dev).to(bf)
        g = torch.randn(n, device=dev).to(bf)
        m1, m2 = torch.zeros_like(p), torch.zeros_like(p)
        plan = K.AdamPlan([(p, g, m1, m2, 1.0)], dev)
        step = torch.ones(1, dtype=torch.int64, device=dev)
        ms = _time(lambda i: plan.step(step, 1e-3, 0.9, 0.999, 1e-8, clip_value=0.05), a.iters)
        nbytes = n * 2 * 7
        print(json.dumps({"case": "adam", "n": n, "us": ms * 1e3, "GBs": nbytes / ms / 1e6,
                          "frac_of_copy_peak": nbytes / ms / 1e6 / hbm, "peaks": src}))
        return
    if a.case in ("flash_fwd", "flash_bwd"):
        # flash attention on a packed projection [B * S, 3 * H * hd]; FLOPs: 4 S^2 hd per (batch, head) forward (half of it
        # with a causal mask), 2.5 x that in backward (five products; the kernels recompute S and dP: seven)
        from ..ops.flash import flash_attention_packed
        S, B, H, hd = a.seq, a.batch, a.heads, a.head_dim
        causal = not a.full
        qkvs = [(torch.randn(B * S, 3 * H * hd, device=dev, dtype=bf) * 0.5).requires_grad_(True) for _ in range(a.copies)]
        flops = 4.0 * S * S * hd * B * H * (0.5 if causal else 1.0)
        if a.case == "flash_fwd":
            with torch.no_grad():
                ms = _time(lambda i: flash_attention_packed(qkvs[i % a.copies], B, S, H, causal=causal), a.iters)
        else:
            outs = [flash_attention_packed(q, B, S, H, causal=causal) for q in qkvs]
            do = torch.randn_like(outs[0])
            ms = _time(lambda i: torch.autograd.grad(outs[i % a.copies], qkvs[i % a.copies], do, retain_graph=True), a.iters)
            flops *= 2.5
        _lib.check_status()
        t = flops / ms / 1e9
        print(json.dumps({"case": a.case, "S": S, "B": B, "H": H, "head_dim": hd, "causal": causal, "us": ms * 1e3,
                          "tflops": t, "frac_of_cublas_peak": t / tf, "peaks": src}))
        return
    if a.case in ("attn_fwd", "attn_bwd"):
        S, B, H = a.seq, a.batch, a.heads
        qkv = torch.randn(S * B, 3 * H * 64, device=dev, dtype=bf)
        do = torch.randn(S * B, H * 64, device=dev, dtype=bf)
        if a.case == "attn_fwd":
            ms = _time(lambda i: K.attn_small_fwd(qkv, S, B, H, drop_p=0.1, seed=1, offset=i), a.iters)
        else:
            ms = _time(lambda i: K.attn_small_bwd(qkv, do, S, B, H, drop_p=0.1, seed=1, offset=i), a.iters)
        print(json.dumps({"case": a.case, "S": S, "B": B, "H": H, "us": ms * 1e3}))
        return
    if a.case == "colsum":
        x = torch.randn(a.m * 8, a.d, device=dev, dtype=bf)
        ms = _time(lambda i: K.colsum(x), a.iters)
        nbytes = x.numel() * 2
        print(json.dumps({"case": "colsum", "us": ms * 1e3, "GBs": nbytes / ms / 1e6,
                          "frac_of_copy_peak": nbytes / ms / 1e6 / hbm, "peaks": src}))
        return
    if a.case == "gate":
        S, E = a.m * 8, 64
        logits = torch.randn(S, E, device=dev)
        noise = torch.randn(S, E, device=dev)
        ms = _time(lambda i: K.top2_gate(logits, 2 * S // E, noise), a.iters)
        nbytes = S * E * 4 * 3
        print(json.dumps({"case": "gate", "S": S, "E": E, "us": ms * 1e3, "GBs": nbytes / ms / 1e6,
                          "frac_of_copy_peak": nbytes / ms / 1e6 / hbm, "peaks": src}))
        return
    if a.case == "rope":
        B, S, H, hd = 16, a.m // 2, 16, 128
        x = torch.randn(B, S, H, hd, device=dev, dtype=bf)
        fr = torch.outer(torch.arange(S, device=dev, dtype=torch.float32),
                         1.0 / (10000.0 ** (torch.arange(0, hd, 2, device=dev, dtype=torch.float32) / hd)))
        cos, sin = fr.cos(), fr.sin()
        ms = _time(lambda i: K.rope(x, cos, sin), a.iters)
        nbytes = x.numel() * 2 * 2
        print(json.dumps({"case": "rope", "shape": [B, S, H, hd], "us": ms * 1e3, "GBs": nbytes / ms / 1e6,
                          "frac_of_copy_peak": nbytes / ms / 1e6 / hbm, "peaks": src}))
        return
    if a.case == "im2col":
        B, Cc, H, W = 256, 64, 56, 56
        x = torch.randn(B, Cc, H, W, device=dev, dtype=bf)
        ms = _time(lambda i: K.im2col(x, 3, 1, 1, 1), a.iters)
        nbytes = x.numel() * 2 * 10          # one read of x, nine-fold patch matrix written
        print(json.dumps({"case": "im2col", "shape": [B, Cc, H, W], "us": ms * 1e3, "GBs": nbytes / ms / 1e6,
                          "frac_of_copy_peak": nbytes / ms / 1e6 / hbm, "peaks": src}))
        return
    if a.case == "embed":
        V, D, T = 50304, a.d, a.m * 8
        table = torch.randn(V, D, device=dev, dtype=bf)
        ids = torch.randint(0, V, (T,), device=dev)
        out = torch.empty(T, D, device=dev, dtype=bf)
        ms = _time(lambda i: K.embed_fwd(table, ids, out, 0, D=D, scale=2.0), a.iters)
        nbytes = T * D * 2 * 2
        print(json.dumps({"case": "embed", "us": ms * 1e3, "GBs": nbytes / ms / 1e6,
                          "frac_of_copy_peak": nbytes / ms / 1e6 / hbm, "peaks": src}))


if __name__ == "__main__":
    main()
