#!/usr/bin/env python
"""Per-kernel micro-benchmarks with roofline fractions.

    python bench_kernels.py                       # every case, JSON lines
    python bench_kernels.py --case gemm_nt --small   # one case on a small problem (what ncu captures use)

Each case is timed with CUDA events after warm-up, inputs are larger than the 126 MB L2 unless
`--small`, and the achieved rate is reported against the measured peaks in MEASURED_PEAKS.json
(copy bandwidth for memory-bound kernels, cuBLAS bf16 throughput for the GEMMs; "of fallback"
when that file is absent).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d["hbm_gbs"], d["bf16_tflops"], "of measured"
    return 6650.0, 1590.0, "of fallback"


def timeit(fn, iters=10, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(iters):
        fn()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) / iters


def bf(*shape, scale=1.0):
    return (torch.randn(*shape, device="cuda") * scale).to(torch.bfloat16)


def case_gemm_nt(small):
    from moe_b200.ops import gemm as G

    M, N, K = (4096, 4096, 1024) if small else (16384, 4096, 1024)
    a, b = bf(M, K), bf(N, K)
    ms = timeit(lambda: G.gemm_nt(a, b))
    ref = timeit(lambda: a @ b.T)
    return dict(shape=[M, N, K], ms=ms, flops=2.0 * M * N * K, cublas_ms=ref)


def case_gemm_tn(small):
    from moe_b200.ops import gemm as G

    Kc, M, N = (8192, 2048, 1024) if small else (16384, 19000 // 8 * 8, 1024)
    a, b = bf(Kc, M), bf(Kc, N)
    out = torch.zeros(M, N, device="cuda")
    ms = timeit(lambda: G.gemm_tn(a, b, out, beta=1))
    return dict(shape=[M, N, Kc], ms=ms, flops=2.0 * M * N * Kc)


def case_lce(small):
    from moe_b200 import ops

    T, H, V = (2048, 1024, 32768) if small else (16384, 1024, 151936)
    h = bf(T, H).requires_grad_()
    w = (torch.randn(V, H, device="cuda") * 0.02).requires_grad_()
    lab = torch.randint(0, V, (T,), device="cuda")

    def run():
        ops.linear_cross_entropy(h, w, lab).backward()
        h.grad = None
        w.grad = None

    ms = timeit(run, iters=5)
    return dict(shape=[T, H, V], ms=ms, flops=6.0 * T * H * V, bytes=3.0 * T * V * 2)


def case_moe(small):
    from moe_b200 import ops

    T, H, I, E, K = (4096, 1024, 768, 16, 4) if small else (16384, 1024, 768, 16, 4)
    x = bf(T, H).requires_grad_()
    gu = (torch.randn(E, 2 * I, H, device="cuda") * 0.02).requires_grad_()
    dn = (torch.randn(E, H, I, device="cuda") * 0.02).requires_grad_()
    idx = torch.stack([torch.randperm(E, device="cuda")[:K] for _ in range(64)]).repeat(T // 64, 1).int()
    w = torch.rand(T, K, device="cuda").requires_grad_()
    g = bf(T, H)

    def run():
        ops.moe_experts(x, idx, w, gu, dn).backward(g)
        x.grad = gu.grad = dn.grad = w.grad = None

    ms = timeit(run, iters=5)
    return dict(shape=[T, H, I, E, K], ms=ms, flops=18.0 * T * K * H * I)


def case_rmsnorm(small):
    from moe_b200.ops import functional as F

    T, H = (16384, 1024) if small else (131072, 1024)
    x, r = bf(T, H), bf(T, H)
    w = torch.ones(H, device="cuda")
    ms = timeit(lambda: F.add_rmsnorm(x, r, w, 1e-6))
    return dict(shape=[T, H], ms=ms, bytes=4.0 * T * H * 2)


def case_adamw(small):
    from moe_b200.ops import _ext

    e = _ext.load()
    n = (1 << 24) if small else (1 << 28)
    p, g, m, v = (torch.randn(n, device="cuda") for _ in range(4))
    v.abs_()
    p16 = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    hyper = torch.tensor([1e-3, 0.1, 0.05], device="cuda")
    coef = torch.ones(2, device="cuda")
    ms = timeit(lambda: e.adamw(p, g, m, v, p16, hyper, 0.9, 0.95, 1e-8, 0.1, coef))
    return dict(shape=[n], ms=ms, bytes=n * (16.0 + 14.0))


def case_qknorm_rope(small):
    from moe_b200.ops import functional as F

    B, S, nh, nkv, hd = (2, 2048, 16, 8, 128) if small else (8, 2048, 16, 8, 128)
    qkv = bf(B, S, (nh + 2 * nkv) * hd)
    qw, kw = torch.ones(hd, device="cuda"), torch.ones(hd, device="cuda")
    ms = timeit(lambda: F.qk_norm_rope(qkv, qw, kw, B, S, nh, nkv, hd, 1e6, 1e-6))
    return dict(shape=[B, S, nh, nkv, hd], ms=ms, bytes=2.0 * qkv.numel() * 2)


def case_gemm_qkv_rope(small):
    """QKV projection with QK-norm + RoPE in the epilogue, against the plain GEMM followed by the stand-alone kernel."""
    from moe_b200.ops import functional as F
    from moe_b200.ops import gemm as G

    B, S, nh, nkv, hd, H = (2, 2048, 16, 8, 128, 1024) if small else (8, 2048, 16, 8, 128, 1024)
    T, N = B * S, (nh + 2 * nkv) * hd
    x, w = bf(T, H), bf(N, H, scale=0.05)
    qw, kw = torch.ones(hd, device="cuda"), torch.ones(hd, device="cuda")
    cs = F.rope_table(S, hd, 1e6, x.device)
    ms = timeit(lambda: G.gemm_nt_qkrope(x, w, cs, qw, kw, S, nh, nkv, 1e-6))

    def separate():
        qkv = G.gemm_nt(x, w)
        F.qk_norm_rope(qkv.view(B, S, N), qw, kw, B, S, nh, nkv, hd, 1e6, 1e-6)

    ref = timeit(separate)
    return dict(shape=[T, N, H], ms=ms, flops=2.0 * T * N * H, separate_ms=ref)


def case_qknorm_rope_fwd_bwd(small):
    from moe_b200.ops import functional as F

    B, S, nh, nkv, hd = (2, 2048, 16, 8, 128) if small else (8, 2048, 16, 8, 128)
    qkv = bf(B, S, (nh + 2 * nkv) * hd).requires_grad_()
    qw = torch.ones(hd, device="cuda", requires_grad=True)
    kw = torch.ones(hd, device="cuda", requires_grad=True)
    gq, gk, gv = bf(B, S, nh, hd), bf(B, S, nkv, hd), bf(B, S, nkv, hd)

    def run():
        q, k, v = F.qk_norm_rope(qkv, qw, kw, B, S, nh, nkv, hd, 1e6, 1e-6)
        torch.autograd.backward((q, k, v), (gq.view_as(q), gk.view_as(k), gv.view_as(v)))
        qkv.grad = qw.grad = kw.grad = None

    ms = timeit(run)
    # forward reads qkv and writes q, k, v; backward reads the three gradients and the q / k inputs, writes d(qkv)
    return dict(shape=[B, S, nh, nkv, hd], ms=ms, bytes=(2.0 + 2.75) * qkv.numel() * 2)


def case_flash_attn_fwd(small, hd=128):
    import math

    from moe_b200.ops import _ext
    from moe_b200.ops import gemm as G

    e = _ext.load()
    B, S, nh, nkv = (2, 2048, 16, 8) if small else (8, 2048, 16, 8)
    q, k, v = bf(B, S, nh, hd), bf(B, S, nkv, hd), bf(B, S, nkv, hd)
    o, lse = torch.empty_like(q), torch.empty(B, nh, S, device="cuda")
    st = G.status_word(q.device)
    ms = timeit(lambda: e.flash_fwd(q, k, v, o, lse, 1 / math.sqrt(hd), st))
    ref = timeit(lambda: torch.nn.functional.scaled_dot_product_attention(
        q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True, enable_gqa=True))
    return dict(shape=[B, S, nh, nkv, hd], ms=ms, flops=2.0 * B * nh * S * S * hd, sdpa_ms=ref)


def case_flash_attn_fwd_hd64(small):
    return case_flash_attn_fwd(small, hd=64)


def case_flash_attn_bwd(small, hd=128):
    import math

    from moe_b200.ops import _ext
    from moe_b200.ops import gemm as G

    e = _ext.load()
    B, S, nh, nkv = (2, 2048, 16, 8) if small else (8, 2048, 16, 8)
    q, k, v, do = bf(B, S, nh, hd), bf(B, S, nkv, hd), bf(B, S, nkv, hd), bf(B, S, nh, hd)
    o, lse = torch.empty_like(q), torch.empty(B, nh, S, device="cuda")
    st = G.status_word(q.device)
    sc = 1 / math.sqrt(hd)
    e.flash_fwd(q, k, v, o, lse, sc, st)
    dq, dk, dv, delta = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v), torch.empty_like(lse)
    ms = timeit(lambda: e.flash_bwd(q, k, v, o, do, lse, delta, dq, dk, dv, sc, st))
    z = torch.zeros((), dtype=torch.int64, device="cuda")
    lse_nat = (lse * math.log(2)).unsqueeze(-1)
    ref = timeit(lambda: torch.ops.aten._scaled_dot_product_cudnn_attention_backward(
        do.transpose(1, 2), q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), o.transpose(1, 2), lse_nat, z, z,
        None, None, None, S, S, 0.0, True, scale=sc))
    return dict(shape=[B, S, nh, nkv, hd], ms=ms, flops=5.0 * B * nh * S * S * hd, cudnn_ms=ref)


def case_flash_attn_bwd_hd64(small):
    return case_flash_attn_bwd(small, hd=64)


def case_allreduce_emulated(small):
    """Eight ranks emulated on one GPU (flags pre-set): measures the kernel's local memory path only."""
    from moe_b200.ops import _ext
    from moe_b200.ops import gemm as G

    e = _ext.load()
    world, n = 8, (1 << 22) if small else (1 << 26)
    bufs = [torch.randn(n, device="cuda") for _ in range(world)]
    flags = [torch.full((16,), 1 << 30, dtype=torch.int32, device="cuda") for _ in range(world)]
    norms = [torch.zeros(8, device="cuda") for _ in range(world)]
    si, sf = torch.zeros(2, dtype=torch.int32, device="cuda"), torch.zeros(150, device="cuda")
    ep = torch.ones(1, dtype=torch.int32, device="cuda")
    st = G.status_word(torch.device("cuda"))
    args = ([b.data_ptr() for b in bufs], [f.data_ptr() for f in flags], [x.data_ptr() for x in norms], 0)
    ms = timeit(lambda: e.allreduce(*args, 0, world, 0, n, 1.0 / world, ep, 0, True, True, False, 128, si, sf, st, 0))
    return dict(shape=[world, n], ms=ms, bytes=2.0 * n * 4)  # one slice read from 8 buffers + written to 8


CASES = {k[5:]: v for k, v in globals().items() if k.startswith("case_")}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", default="all", choices=["all", *CASES])
    ap.add_argument("--small", action="store_true")
    args = ap.parse_args()
    hbm, tf, tag = peaks()
    for name, fn in CASES.items():
        if args.case not in ("all", name):
            continue
        r = fn(args.small)
        out = {"case": name, **r}
        if "flops" in r:
            out["tflops"] = r["flops"] / r["ms"] / 1e9
            out["frac_of_gemm_peak"] = out["tflops"] / tf
        if "bytes" in r:
            out["gbs"] = r["bytes"] / r["ms"] / 1e6
            out["frac_of_hbm_peak"] = out["gbs"] / hbm
        out["peaks"] = tag
        print(json.dumps(out), flush=True)
    from moe_b200.ops import gemm as G

    G.check_status()


if __name__ == "__main__":
    main()
