"""Single-kernel micro-benchmarks with roofline fractions: ``python -m research_b200.kernels.microbench <op> ...``.

Each case runs one native kernel on inputs larger than L2, times it with CUDA events after warm-up, and prints
one JSON line with the achieved TFLOP/s or GB/s and the fraction of the measured peak (``MEASURED_PEAKS.json`` at
the repository root when present, else 6.65 TB/s and 1.59 PFLOP/s).  The same command lines are what the ncu
summaries under ``profiles/`` were captured with (``--iters`` small so that a capture ends by itself).
"""

from __future__ import annotations

import argparse
import json
from pathlib import Path

import torch

from research_b200.ops import native

ROOT = Path(__file__).resolve().parent.parent.parent


def peaks() -> dict:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        raw = json.loads(path.read_text())
        return {"hbm_gbs": raw["hbm_gbs"], "bf16_tflops": raw["bf16_tflops"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def timed(fn, warmup: int, iters: int) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / iters


def bf(shape, scale=1.0):
    return (torch.randn(shape, device="cuda") * scale).to(torch.bfloat16)


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("op", choices=["gemm", "attn_fwd", "attn_bwd", "rmsnorm", "rmsnorm_bwd", "dion2", "swiglu", "ce", "adamw", "decode", "moe", "router"])
    ap.add_argument("--experts", type=int, default=64)
    ap.add_argument("--top-k", type=int, default=8)
    ap.add_argument("--m", type=int, default=16384)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--layout", default="nt", choices=["nt", "nn", "tn"])
    ap.add_argument("--batch", type=int, default=2)
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--rows", type=int, default=32768)
    ap.add_argument("--hidden", type=int, default=2048)
    ap.add_argument("--vocab", type=int, default=50304)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--iters", type=int, default=10)
    args = ap.parse_args()
    pk = peaks()
    out: dict = {"op": args.op, "peaks": pk}
    if args.op == "gemm":
        M, N, K = args.m, args.n, args.k
        if args.layout == "nt":
            a, b = bf((M, K)), bf((N, K))
            fn = lambda: native.gemm(a, b, out=c)
        elif args.layout == "nn":
            a, b = bf((M, K)), bf((K, N))
            fn = lambda: native.gemm(a, b, trans_b=False, out=c)
        else:
            a, b = bf((K, M)), bf((K, N))
            fn = lambda: native.gemm(a, b, trans_a=True, trans_b=False, out=c)
        c = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        ms = timed(fn, args.warmup, args.iters)
        tf = 2.0 * M * N * K / ms / 1e9
        out.update(shape=[M, N, K], layout=args.layout, ms=ms, tflops=tf, frac_of_peak=tf / pk["bf16_tflops"])
    elif args.op in ("attn_fwd", "attn_bwd"):
        B, S, H, Hkv, D = args.batch, args.seq, args.heads, args.kv_heads, args.head_dim
        q, k, v = bf((B, S, H, D)), bf((B, S, Hkv, D)), bf((B, S, Hkv, D))
        d_o = bf((B, S, H, D))
        o, lse = native.attn_fwd(q, k, v, causal=True)
        if args.op == "attn_fwd":
            ms = timed(lambda: native.attn_fwd(q, k, v, causal=True), args.warmup, args.iters)
            flops = 4.0 * B * H * S * S * D / 2
        else:
            ms = timed(lambda: native.attn_bwd(q, k, v, o, d_o, lse, causal=True), args.warmup, args.iters)
            flops = 10.0 * B * H * S * S * D / 2
        tf = flops / ms / 1e9
        out.update(shape=[B, S, H, Hkv, D], causal=True, ms=ms, tflops=tf, frac_of_peak=tf / pk["bf16_tflops"])
    elif args.op == "rmsnorm":
        x, w = bf((args.rows, args.hidden)), torch.ones(args.hidden, device="cuda")
        ms = timed(lambda: native.rmsnorm_fwd(x, w, 1e-6), args.warmup, args.iters)
        gbs = 2 * x.numel() * 2 / ms / 1e6
        out.update(shape=[args.rows, args.hidden], ms=ms, gbs=gbs, frac_of_peak=gbs / pk["hbm_gbs"])
    elif args.op == "rmsnorm_bwd":
        x, dy, w = bf((args.rows, args.hidden)), bf((args.rows, args.hidden)), torch.ones(args.hidden, device="cuda")
        rstd = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-6)
        dw = torch.zeros(args.hidden, device="cuda")
        ms = timed(lambda: native.rmsnorm_bwd(x, w, rstd, dy, dw), args.warmup, args.iters)
        gbs = 3 * x.numel() * 2 / ms / 1e6                       # x and dy read, dx written
        out.update(shape=[args.rows, args.hidden], ms=ms, gbs=gbs, frac_of_peak=gbs / pk["hbm_gbs"])
    elif args.op == "dion2":
        # one Dion2 update of a stack of expert matrices without the orthogonaliser: accumulate + select + gather,
        # then apply; algorithmic bytes: m, g read and m written (12 B), w read and written + bf16 copy (10 B)
        n, rows, cols = args.experts // 8 or 1, args.hidden, args.k
        g, m, w = (torch.randn(n, rows, cols, device="cuda") for _ in range(3))
        sh = torch.empty(n, rows, cols, device="cuda", dtype=torch.bfloat16)
        res = {}
        for axis in (0, 1):
            k = (rows if axis == 0 else cols) // 4
            o = bf((n, k, cols) if axis == 0 else (n, rows, k))
            state = {}

            def first():
                state["sel"] = native.dion2_select_stack(g, m, None, n, rows, cols, rows * cols, axis, k, 1e-8)

            def second():
                native.dion2_apply(w, m, o, state["sel"][2], sh, n, rows, cols, k, rows * cols, axis, 0.999, 1e-3, 0.95)

            ms1 = timed(first, args.warmup, args.iters)
            ms2 = timed(second, args.warmup, args.iters)
            b1, b2 = 12 * g.numel() + 4.5 * g.numel() / 4, 10 * g.numel() + 10 * g.numel() / 4
            res[f"axis{axis}"] = {"select_ms": ms1, "select_frac": b1 / ms1 / 1e6 / pk["hbm_gbs"],
                                  "apply_ms": ms2, "apply_frac": b2 / ms2 / 1e6 / pk["hbm_gbs"]}
        out.update(shape=[n, rows, cols], **res)
    elif args.op == "swiglu":
        gu = bf((args.rows, 2 * args.hidden))
        ms = timed(lambda: native.swiglu_fwd(gu), args.warmup, args.iters)
        gbs = 3 * args.rows * args.hidden * 2 / ms / 1e6
        out.update(shape=[args.rows, args.hidden], ms=ms, gbs=gbs, frac_of_peak=gbs / pk["hbm_gbs"])
    elif args.op == "ce":
        rows = min(args.rows, 4096)
        logits = bf((rows, args.vocab), 2.0)
        tgt = torch.randint(0, args.vocab, (rows,), device="cuda", dtype=torch.int32)
        mask = torch.ones(rows, device="cuda", dtype=torch.uint8)
        ms = timed(lambda: native.ce_fwd_bwd(logits, tgt, mask, 1.0 / rows, 0.0), args.warmup, args.iters)
        gbs = 2 * logits.numel() * 2 / ms / 1e6
        out.update(shape=[rows, args.vocab], ms=ms, gbs=gbs, frac_of_peak=gbs / pk["hbm_gbs"],
                   note="algorithmic bytes = one read + one write of the logits")
    elif args.op == "adamw":
        n = args.rows * args.hidden
        p, m, v = (torch.zeros(n, device="cuda") for _ in range(3))
        g = torch.randn(n, device="cuda")
        sh = torch.empty(n, device="cuda", dtype=torch.bfloat16)
        ms = timed(lambda: native.adamw(p, m, v, g, sh, None, 1e-3, 0.9, 0.999, 1e-8, 0.0, 1), args.warmup, args.iters)
        gbs = n * (4 * 4 + 3 * 4 + 2) / ms / 1e6
        out.update(elements=n, ms=ms, gbs=gbs, frac_of_peak=gbs / pk["hbm_gbs"])
    elif args.op == "decode":
        from research_b200.ops.decode import decode_attention

        B, S, H, Hkv, D = args.batch, args.seq, args.heads, args.kv_heads, args.head_dim
        q = bf((B, H, D))
        kc, vc = bf((B, S, Hkv, D)), bf((B, S, Hkv, D))
        lens = torch.full((B,), S, device="cuda", dtype=torch.int32)
        ms = timed(lambda: decode_attention(q, kc, vc, lens, None), args.warmup, args.iters)
        from research_b200.ops.decode import decode_attention_paged

        kp = kc.view(B, S // 128, 128, Hkv, D).permute(0, 1, 3, 2, 4).contiguous()
        vp = vc.view(B, S // 128, 128, Hkv, D).permute(0, 1, 3, 2, 4).contiguous()
        nbytes = 2 * kc.numel() * 2
        for name in ("stream", "registers"):
            ms_paged = timed(lambda: decode_attention_paged(q, kp, vp, lens, None, kernel=name), args.warmup,
                             args.iters)
            out[f"paged_head_major_{name}"] = {"ms": ms_paged, "gbs": nbytes / ms_paged / 1e6,
                                               "frac_of_peak": nbytes / ms_paged / 1e6 / pk["hbm_gbs"]}
        gbs = 2 * kc.numel() * 2 / ms / 1e6
        out.update(shape=[B, S, H, Hkv, D], ms=ms, gbs=gbs, frac_of_peak=gbs / pk["hbm_gbs"])
    elif args.op == "moe":
        from research_b200.ops.grouped import RoutingPlan, _combine_rows, _gather_rows

        T, k, E, H = args.rows, args.top_k, args.experts, args.hidden
        ids = torch.topk(torch.randn(T, E, device="cuda"), k, dim=-1).indices.to(torch.int32)
        x = bf((T, H))
        w = torch.rand(T * k, device="cuda")
        capacity = int(1.25 * T * k / E)
        ms_plan = timed(lambda: RoutingPlan(ids, E, capacity), args.warmup, args.iters)
        plan = RoutingPlan(ids, E, capacity)
        ms_gather = timed(lambda: _gather_rows(x, None, plan), args.warmup, args.iters)
        pad = _gather_rows(x, None, plan)
        ms_combine = timed(lambda: _combine_rows(pad, w, plan), args.warmup, args.iters)
        kept = int((plan.dest >= 0).sum())
        row_bytes = H * 2
        gather_gbs = (kept * 2 * row_bytes) / ms_gather / 1e6          # read a token row, write a padded row
        combine_gbs = (kept * row_bytes + T * row_bytes) / ms_combine / 1e6
        out.update(shape=[T, k, E, H], kept_rows=kept, rows_pad=plan.rows_pad, ms_plan=ms_plan, ms_gather=ms_gather,
                   ms_combine=ms_combine, gather_gbs=gather_gbs, combine_gbs=combine_gbs,
                   gather_frac_of_peak=gather_gbs / pk["hbm_gbs"], combine_frac_of_peak=combine_gbs / pk["hbm_gbs"])
    elif args.op == "router":
        from research_b200.ops.router import load_statistics, load_statistics_reference, route, route_reference

        T, k, E = args.rows, args.top_k, args.experts
        logits = bf((T, E), 1.5).requires_grad_(True)
        bias = torch.zeros(E, device="cuda")
        gw = torch.randn(T, k, device="cuda")

        def fwd_bwd(fn):
            def run():
                logits.grad = None
                _, w, s = fn(logits, bias, k, "sigmoid", 1.0)
                (w * gw).sum().backward()
            return run

        ms_native = timed(fwd_bwd(route), args.warmup, args.iters)
        ms_torch = timed(fwd_bwd(route_reference), args.warmup, args.iters)
        with torch.no_grad():
            ids, w, _ = route(logits, bias, k, "sigmoid", 1.0)
            ms_fwd = timed(lambda: route(logits, bias, k, "sigmoid", 1.0), args.warmup, args.iters)
            ms_stats = timed(lambda: load_statistics(ids, w, E), args.warmup, args.iters)
            ms_stats_torch = timed(lambda: load_statistics_reference(ids, w, E), args.warmup, args.iters)
        out.update(shape=[T, E, k], ms_route_fwd_bwd=ms_native, ms_route_fwd_bwd_torch=ms_torch, ms_route_fwd=ms_fwd,
                   fwd_gbs=(T * E * 2 + T * E * 4 + T * k * 8) / ms_fwd / 1e6, ms_stats=ms_stats,
                   ms_stats_torch=ms_stats_torch,
                   note="fwd_bwd includes the multiply, sum and autograd glue around the kernels in both variants")
    native.check_status()
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
