"""Kernel micro-benchmarks: CUDA-event timing after warm-up, L2 flushed between timed launches,
achieved TFLOP/s or GB/s and the fraction of the measured peak (MEASURED_PEAKS.json when present).

    python -m incin_b200.benchmarks.kernels --op gemm            # GPT-2 / Llama GEMM shapes vs cuBLAS
    python -m incin_b200.benchmarks.kernels --op gemm --one 4096 4096 4096 --iters 3   # small case for ncu
    python -m incin_b200.benchmarks.kernels --op attention
    python -m incin_b200.benchmarks.kernels --op bandwidth       # norm / xent / adamw
"""
from __future__ import annotations

import argparse
import json
import os

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def peaks() -> dict:
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return json.load(f)
    except Exception:
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "fallback": True}


_flush = None


def flush_l2() -> None:
    global _flush
    if _flush is None:
        _flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    _flush.zero_()  # writes 256 MB, twice the 126 MB L2


def _graph_ms(body, reps: int) -> float:
    """Device milliseconds of `reps` back-to-back executions of body(), replayed from a CUDA graph so
    that no host latency (Python, ctypes, tensor-map encoding) sits between the launches."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    g = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(g, stream=side):
            for _ in range(reps):
                body()
    torch.cuda.current_stream().wait_stream(side)
    g.replay()
    torch.cuda.synchronize()
    best = None
    for _ in range(3):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        g.replay()
        b.record()
        torch.cuda.synchronize()
        t = a.elapsed_time(b)
        best = t if best is None else min(best, t)
    return best


def timeit(fn, iters: int = 10, warmup: int = 3) -> float:
    """Device milliseconds of one call with a cold L2: ([flush L2; fn] x iters) minus ([flush L2] x iters),
    both replayed from CUDA graphs and timed with CUDA events."""
    flush_l2()
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    both = _graph_ms(lambda: (flush_l2(), fn()), iters)
    only_flush = _graph_ms(flush_l2, iters)
    return max(both - only_flush, 1e-6) / iters


def bench_gemm(args) -> list:
    from incin_b200.ops import gemm as G
    pk = peaks()
    shapes = [  # (name, M, N, K, kind)
        ("gpt2 qkv fwd", 8192, 2304, 768, "nt"), ("gpt2 proj fwd", 8192, 768, 768, "nt"),
        ("gpt2 fc fwd", 8192, 3072, 768, "nt"), ("gpt2 out fwd", 8192, 768, 3072, "nt"),
        ("gpt2 lm head", 8192, 50304, 768, "nt"), ("gpt2 fc dgrad", 8192, 768, 3072, "nn"),
        ("gpt2 out dgrad", 8192, 3072, 768, "nn"), ("gpt2 lm dgrad", 8192, 768, 50304, "nn"),
        ("gpt2 fc wgrad", 3072, 768, 8192, "tn"), ("gpt2 proj wgrad", 768, 768, 8192, "tn"),
        ("gpt2 lm wgrad", 50304, 768, 8192, "tn"), ("square 4096", 4096, 4096, 4096, "nt"),
        ("square 8192", 8192, 8192, 8192, "nt"), ("llama ffn", 4096, 11264, 2048, "nt"),
    ]
    if args.one:
        shapes = [("custom", args.one[0], args.one[1], args.one[2], args.kind)]
    if getattr(args, "shapes", None):
        shapes = [sh for sh in shapes if sh[0] in args.shapes]
    rows = []
    for name, M, N, K, kind in shapes:
        if kind == "nt":
            a = torch.randn(M, K, device="cuda").bfloat16()
            b = torch.randn(N, K, device="cuda").bfloat16()
            out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
            ours = lambda: G.gemm(a, b, out, M=M, N=N, K=K, lda=K, ldb=K, ldc=N, tile_n=args.tile_n)
            lib = lambda: torch.matmul(a, b.t(), out=out)
        elif kind == "nn":
            a = torch.randn(M, K, device="cuda").bfloat16()
            b = torch.randn(K, N, device="cuda").bfloat16()
            out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
            ours = lambda: G.gemm(a, b, out, M=M, N=N, K=K, lda=K, ldb=N, ldc=N, b_mn=True, tile_n=args.tile_n)
            lib = lambda: torch.matmul(a, b, out=out)
        else:
            a = torch.randn(K, M, device="cuda").bfloat16()
            b = torch.randn(K, N, device="cuda").bfloat16()
            out = torch.zeros(M, N, dtype=torch.float32, device="cuda")
            sp = G.auto_splits(M, N, K)
            ours = lambda: G.gemm(a, b, out, M=M, N=N, K=K, lda=M, ldb=N, ldc=N, a_mn=True, b_mn=True,
                                  accumulate=True, splits=sp, tile_n=args.tile_n)
            outb = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
            lib = lambda: torch.matmul(a.t(), b, out=outb)
        t_ours = timeit(ours, args.iters)
        t_lib = None if args.no_lib else timeit(lib, args.iters)
        fl = 2.0 * M * N * K
        rows.append({"shape": name, "M": M, "N": N, "K": K, "kind": kind, "ms": round(t_ours, 4),
                     "tflops": round(fl / t_ours / 1e9, 1),
                     "frac_of_measured_burst": round(fl / t_ours / 1e9 / pk["bf16_tflops"], 3),
                     "cublas_ms": None if t_lib is None else round(t_lib, 4),
                     "cublas_tflops": None if t_lib is None else round(fl / t_lib / 1e9, 1)})
        print(json.dumps(rows[-1]), flush=True)
    G.check_status()
    return rows


def bench_bandwidth(args) -> None:
    from incin_b200.ops import kernels as K
    pk = peaks()
    rows, C = 8192, 768
    x = torch.randn(rows, C, device="cuda").bfloat16()
    g = torch.ones(C, device="cuda").bfloat16()
    b = torch.zeros(C, device="cuda").bfloat16()
    big_rows, big_c = 65536, 4096
    xb = torch.randn(big_rows, big_c, device="cuda").bfloat16()
    gb = torch.ones(big_c, device="cuda").bfloat16()
    res = []

    def rec(name, ms, bytes_):
        r = {"kernel": name, "ms": round(ms, 4), "GBs": round(bytes_ / ms / 1e6, 1),
             "frac_of_measured_copy": round(bytes_ / ms / 1e6 / pk["hbm_gbs"], 3)}
        res.append(r)
        print(json.dumps(r), flush=True)

    rec("layernorm_fwd 8192x768", timeit(lambda: K.layernorm_fwd(x, g, b, 1e-5)), 2 * x.numel() * 2)
    ys, means, rstds = K.layernorm_fwd(x, g, b, 1e-5)
    dgs, dbs = torch.zeros(C, device="cuda"), torch.zeros(C, device="cuda")
    rec("layernorm_bwd 8192x768 (+residual gradient)",
        timeit(lambda: K.layernorm_bwd(ys, x, g, means, rstds, ys, dgs, dbs)), 4 * x.numel() * 2)
    dcs = torch.zeros(C, device="cuda")
    rec("layernorm_bwd 8192x768 (+residual gradient, + column sums of dx)",
        timeit(lambda: K.layernorm_bwd(ys, x, g, means, rstds, ys, dgs, dbs, dcs)), 4 * x.numel() * 2)
    # what a plain device copy of the same bytes reaches at this size (launch ramp and tail included)
    x2, x4 = torch.empty_like(x), torch.empty(2, *x.shape, dtype=x.dtype, device="cuda")
    x4s = torch.empty_like(x4)
    rec("copy 8192x768 (torch copy_, bytes of layernorm_fwd)", timeit(lambda: x2.copy_(x)), 2 * x.numel() * 2)
    rec("copy 2x8192x768 (torch copy_, bytes of layernorm_bwd)", timeit(lambda: x4s.copy_(x4)), 4 * x.numel() * 2)
    rec("layernorm_fwd 65536x4096", timeit(lambda: K.layernorm_fwd(xb, gb, None, 1e-5)), 2 * xb.numel() * 2)
    y, mean, rstd = K.layernorm_fwd(xb, gb, None, 1e-5)
    dg = torch.zeros(big_c, device="cuda")
    rec("layernorm_bwd 65536x4096", timeit(lambda: K.layernorm_bwd(y, xb, gb, mean, rstd, None, dg, None)),
        5 * xb.numel() * 2)
    V, ld = 50257, 50304
    logits = torch.randn(8192, ld, device="cuda").bfloat16()
    tgt = torch.randint(0, V, (8192,), device="cuda")
    rec("xent_fwd 8192x50304", timeit(lambda: K.xent_fwd(logits, tgt, V)), logits.numel() * 2)
    loss, lse = K.xent_fwd(logits, tgt, V)
    one = torch.ones(1, device="cuda")
    rec("xent_bwd 8192x50304", timeit(lambda: K.xent_bwd_(logits, tgt, lse, one, 1.0, V)), 2 * logits.numel() * 2)
    rec("xent_fused 8192x50304 (loss + gradient in place)", timeit(lambda: K.xent_fused_(logits, tgt, 1.0 / 8192, V)),
        2 * logits.numel() * 2)
    n = 124 * 1000 * 1000
    w, m, v, gr = (torch.zeros(n, device="cuda") for _ in range(4))
    sh = torch.zeros(n, dtype=torch.bfloat16, device="cuda")
    hyper = torch.tensor([1e-3, 0.9, 0.999, 1e-8, 0.01, 1, 1, 0], device="cuda")
    rec("adamw_flat 124M", timeit(lambda: K.adamw_flat(w, m, v, gr, sh, n, hyper)), n * (4 * 7 + 2))
    rec("fill_f32 124M", timeit(lambda: K.fill_f32_(gr, 0.0)), n * 4)


def attention_error_vs_cpu(qkv: torch.Tensor, do: torch.Tensor, H: int, D: int, b: int, h: int) -> dict:
    """Max abs error of the product path's output and gradients for one (batch, head) slice against an fp32 CPU
    reference of the same math (scores, causal mask, softmax, weighted sum; gradients by CPU autograd): the oracle
    the reference's CPU backend defines (crates/incin-backends/src/cpu/ops/shape_ops.rs:1245-1269)."""
    import math
    from incin_b200.ops import functional as F
    B, T, _ = qkv.shape
    x = qkv.detach().clone().requires_grad_()
    out = F.causal_attention(x, H, D)
    out.backward(do)
    xs = qkv.detach().view(B, T, 3 * H, D)
    q, k, v = (xs[b, :, i * H + h].float().cpu().requires_grad_() for i in range(3))
    s = (q @ k.t()) * (1.0 / math.sqrt(D))
    s = s.masked_fill(~torch.ones(T, T, dtype=torch.bool).tril(), float("-inf"))
    ref = torch.softmax(s, dim=-1) @ v
    ref.backward(do.view(B, T, H, D)[b, :, h].float().cpu())
    g = x.grad.view(B, T, 3 * H, D)
    got = {"out": out.detach().view(B, T, H, D)[b, :, h], "dq": g[b, :, h], "dk": g[b, :, H + h], "dv": g[b, :, 2 * H + h]}
    want = {"out": ref.detach(), "dq": q.grad, "dk": k.grad, "dv": v.grad}
    res = {}
    for name in got:
        a, r = got[name].float().cpu(), want[name]
        res[f"max_abs_err_{name}"] = round(float((a - r).abs().max()), 5)
        res[f"ref_max_{name}"] = round(float(r.abs().max()), 4)
    return res


def bench_attention(args) -> list:
    from incin_b200.ops import functional as F
    pk = peaks()
    out_rows = []

    def emit(row):
        out_rows.append(row)
        print(json.dumps(row), flush=True)

    for (B, H, T, D) in [(8, 12, 1024, 64), (8, 32, 4096, 128)] if not args.one else [tuple(args.one) + (args.head_dim,)]:
        # Q, K, V and dO ~ N(0, 1) from seed 0, softmax scale 1 / sqrt(head_dim)
        gen = torch.Generator(device="cuda").manual_seed(0)
        qkv = torch.randn(B, T, 3 * H * D, device="cuda", generator=gen).bfloat16().requires_grad_()
        do = torch.randn(B, T, H * D, device="cuda", generator=gen).bfloat16()
        for impl in args.impls.split(","):
            F.set_attention_impl(impl)
            if impl == "composed" and B * H * T * T * 2 > 12e9:
                continue
            fwd = lambda: F.causal_attention(qkv, H, D)
            t_f = timeit(fwd, args.iters)

            def fb():
                o = F.causal_attention(qkv, H, D)
                o.backward(do)
            t_fb = timeit(fb, args.iters)
            fl_f = 4.0 * B * H * T * T * D / 2
            emit({"B": B, "H": H, "T": T, "D": D, "impl": impl, "fwd_ms": round(t_f, 4),
                  "fwd_tflops": round(fl_f / t_f / 1e9, 1), "fwd_bwd_ms": round(t_fb, 4),
                  "fwd_bwd_tflops": round(3.5 * fl_f / t_fb / 1e9, 1),
                  "frac_of_measured_burst": round(3.5 * fl_f / t_fb / 1e9 / pk["bf16_tflops"], 3)})
            if impl in ("auto", "flash") and not args.no_check:
                err = attention_error_vs_cpu(qkv, do, H, D, B - 1, H - 1)
                emit({"B": B, "H": H, "T": T, "D": D, "impl": impl, "slice": [B - 1, H - 1], "vs": "fp32 CPU reference", **err})
        # library reference (baseline, not product): torch SDPA
        q, k, v = (torch.randn(B, H, T, D, device="cuda").bfloat16().requires_grad_() for _ in range(3))
        dob = torch.randn(B, H, T, D, device="cuda").bfloat16()

        def sd():
            torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True).backward(dob)
        if not args.no_lib:
            t = timeit(sd, args.iters)
            fl_f = 4.0 * B * H * T * T * D / 2
            emit({"B": B, "H": H, "T": T, "D": D, "impl": "torch-sdpa", "fwd_bwd_ms": round(t, 4),
                  "fwd_bwd_tflops": round(3.5 * fl_f / t / 1e9, 1)})
    return out_rows


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", default="gemm", choices=["gemm", "bandwidth", "attention"])
    ap.add_argument("--one", type=int, nargs=3, default=None, help="M N K (gemm) or B H T (attention)")
    ap.add_argument("--kind", default="nt", choices=["nt", "nn", "tn"])
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--impls", default="auto,composed")
    ap.add_argument("--tile-n", type=int, default=0)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--no-lib", action="store_true", help="skip the cuBLAS / SDPA comparison")
    ap.add_argument("--no-check", action="store_true", help="attention: skip the error check against the fp32 CPU reference")
    args = ap.parse_args()
    {"gemm": bench_gemm, "bandwidth": bench_bandwidth, "attention": bench_attention}[args.op](args)


if __name__ == "__main__":
    main()
