"""Multi-GPU micro-benchmarks of the kernels that move data between ranks, with roofline fractions.

Run one process per GPU, e.g.
``python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29611 \
-m research_b200.kernels.comm_microbench tp_gemm --batch 2 --seq 8192 --hidden 4096 --cols 3072``.

Cases: ``tp_gemm`` (all-gather -> GEMM and GEMM -> reduce-scatter in one kernel each, against NCCL + GEMM),
``collectives`` (gradient reduce-scatter and weight all-gather: peer loads, ``multimem`` through the switch, NCCL),
``ring_attn`` (context-parallel attention with the K/V exchange inside the kernels against all-gather + attention +
reduce-scatter).

Times are CUDA events on the launching stream after warm-up, maximum over ranks.  The roofline time of a fused
kernel is the slower of its FLOPs at the measured GEMM peak and the bytes that must cross NVLink at the measured
peer-copy bandwidth (770 GB/s per direction); peaks come from ``MEASURED_PEAKS.json`` when present.
"""

from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from research_b200.kernels.microbench import peaks, timed
from research_b200.ops import native
from research_b200.parallel.tensor_fused import TensorParallelFusion

NVLINK_GBS = 770.0


def _max_over_ranks(ms: float) -> float:
    t = torch.tensor([ms], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def bench_collectives(args, rank: int, world: int) -> dict:
    """Reduce-scatter of an fp32 gradient region and all-gather of a bf16 weight region of ``--mib`` MiB per rank."""

    from research_b200.parallel.symmetric import SymmetricArena

    n = args.mib * (1 << 20) // 4 // world * world                    # fp32 elements of the whole region
    per = n // world
    arena = SymmetricArena(dist.group.WORLD, n * 4 + n * 2 + 8192, multicast=True)
    grads, g_off = arena.carve(n, torch.float32)
    weights, w_off = arena.carve(n, torch.bfloat16)
    grads.normal_()
    plain = torch.randn(n, device="cuda")
    out = torch.empty(per, device="cuda")
    w_plain = torch.zeros(n, dtype=torch.bfloat16, device="cuda")
    cases = {
        "reduce_scatter_peer": lambda: arena.reduce_scatter(g_off + 4 * rank * per, per, nvls=False),
        "reduce_scatter_nccl": lambda: dist.reduce_scatter_tensor(out, plain),
        "all_gather_peer": lambda: arena.all_gather(w_off, per * 2, nvls=False),
        "all_gather_nccl": lambda: dist.all_gather_into_tensor(w_plain, w_plain[rank * per:(rank + 1) * per].clone()),
    }
    if arena.mc_ptr:
        cases["reduce_scatter_nvls"] = lambda: arena.reduce_scatter(g_off + 4 * rank * per, per, nvls=True)
        cases["all_gather_nvls"] = lambda: arena.all_gather(w_off, per * 2, nvls=True)
    rows = {}
    for name, fn in cases.items():
        dist.barrier()
        rows[name] = _max_over_ranks(timed(fn, args.warmup, args.iters))
    native.check_status()
    remote = (world - 1) / world
    rs_bytes, ag_bytes = n * 4 * remote, n * 2 * remote              # per rank, in one direction
    out_row = {"case": "collectives", "world": world, "multicast_bound": bool(arena.mc_ptr),
               "region_mib_fp32": n * 4 / 2 ** 20, "ms": {k: round(v, 4) for k, v in rows.items()},
               "reduce_scatter_nvlink_roofline_ms": round(rs_bytes / (NVLINK_GBS * 1e6), 4),
               "all_gather_nvlink_roofline_ms": round(ag_bytes / (NVLINK_GBS * 1e6), 4), "nvlink_gbs": NVLINK_GBS}
    torch.cuda.synchronize()
    dist.barrier()
    arena.close()
    return out_row


def bench_ring_attention(args, rank: int, world: int) -> dict:
    """Forward + backward of context-parallel attention on ``world`` ranks (zig-zag split, causal)."""

    import os
    from types import SimpleNamespace

    from research_b200.parallel import context, ring_attention as ring
    from research_b200.steps.train import context_positions

    B, hq, hkv, D = args.batch, args.heads, args.kv_heads, 128
    s_local = args.seq // world
    ex = SimpleNamespace(cp_size=world, cp_rank=rank, cp_group=dist.group.WORLD)
    cols = torch.as_tensor(context_positions(args.seq, world, rank), device="cuda")
    glob = cols.tolist()
    breaks = [0] + [i for i in range(1, len(glob)) if glob[i] != glob[i - 1] + 1] + [len(glob)]
    chunks = tuple((glob[a], b - a) for a, b in zip(breaks[:-1], breaks[1:]))
    positions = cols.to(torch.int32).repeat(B)
    qkv = (torch.randn(B * s_local, (hq + 2 * hkv) * D, device="cuda") * 0.5).bfloat16().requires_grad_(True)
    go = (torch.randn(B, s_local, hq * D, device="cuda") * 0.5).bfloat16()

    def run():
        qkv.grad = None
        out = context.context_parallel_attention(ex, qkv, None, None, positions, B=B, S=s_local, hq=hq, hkv=hkv, D=D,
                                                 eps=1e-6, theta=10000.0, rope=True, lo=None, chunks=chunks)
        out.backward(go)

    rows = {}
    for mode in ("ring", "gather"):
        os.environ["RESEARCH_B200_RING"] = "1" if mode == "ring" else "0"
        dist.barrier()
        rows[mode] = _max_over_ranks(timed(run, args.warmup, args.iters))
    native.check_status()
    ws = next((w for w in ring._WORKSPACES.values() if w is not None), None)
    pk = peaks()
    # causal attention over the whole sequence, forward 4 and backward 10 units of B * H * S^2 * D / 2, split evenly
    flops = 14.0 * B * hq * args.seq * args.seq * D / 2 / world
    nvlink = 0 if ws is None else 2 * ws.bytes_over_nvlink + ws.bytes_over_nvlink   # K/V twice, dK/dV once
    roof = max(flops / (pk["bf16_tflops"] * 1e9), nvlink / (NVLINK_GBS * 1e6))
    return {"case": "ring_attn", "world": world, "shape": {"B": B, "seq": args.seq, "hq": hq, "hkv": hkv, "D": D},
            "ms_fwd_bwd": {k: round(v, 4) for k, v in rows.items()},
            "speedup_vs_allgather": round(rows["gather"] / rows["ring"], 3),
            "nvlink_bytes_per_rank": int(nvlink), "kv_bytes_lower_bound": int((world - 1) / world * 2 * B * args.seq
                                                                              * hkv * D * 2),
            "roofline_ms": round(roof, 4), "fraction_of_roofline": round(roof / rows["ring"], 3), "peaks": pk}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("case", nargs="?", default="tp_gemm", choices=["tp_gemm", "collectives", "ring_attn"])
    ap.add_argument("--mib", type=int, default=1024, help="collectives: MiB of fp32 gradients in the reduced region")
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--batch", type=int, default=2)
    ap.add_argument("--seq", type=int, default=8192)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--cols", type=int, default=3072, help="output columns of the column-parallel weight shard")
    ap.add_argument("--inner", type=int, default=7168, help="contraction size of the row-parallel weight shard")
    ap.add_argument("--transfer-ctas", type=int, default=16)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    args = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    if args.case != "tp_gemm":
        row = bench_collectives(args, rank, world) if args.case == "collectives" else \
            bench_ring_attention(args, rank, world)
        if rank == 0:
            print(json.dumps(row))
        dist.barrier()
        dist.destroy_process_group()
        return 0
    B, S, H = args.batch, args.seq, args.hidden
    s_local = S // world
    M, m_local = B * S, B * s_local
    pk = peaks()
    ws = TensorParallelFusion(dist.group.WORLD, max_shard_elems=m_local * H, max_out_elems=m_local * H,
                              transfer_ctas=args.transfer_ctas)
    x = (torch.randn(m_local, H, device="cuda") * 0.5).bfloat16()
    w_col = (torch.randn(args.cols, H, device="cuda") * 0.02).bfloat16()
    h = (torch.randn(M, args.inner, device="cuda") * 0.5).bfloat16()
    w_row = (torch.randn(H, args.inner, device="cuda") * 0.02).bfloat16()
    x_full = torch.empty(M, H, dtype=torch.bfloat16, device="cuda")
    y_shard = torch.empty(m_local, H, dtype=torch.bfloat16, device="cuda")

    def nccl_gather_gemm():
        dist.all_gather_into_tensor(x_full, x)
        native.gemm(x_full, w_col)

    def nccl_gemm_scatter():
        dist.reduce_scatter_tensor(y_shard, native.gemm(h, w_row))

    rows = {}
    for name, fn in (("nccl_allgather_then_gemm", nccl_gather_gemm),
                     ("fused_allgather_gemm", lambda: ws.gather_gemm(x, w_col, b_mn=False, chunk_rows=m_local)),
                     ("gemm_only_column", lambda: native.gemm(x_full, w_col)),
                     ("nccl_gemm_then_reducescatter", nccl_gemm_scatter),
                     ("fused_gemm_reducescatter", lambda: ws.gemm_scatter(h, w_row, b_mn=False, chunk_rows=m_local)),
                     ("gemm_only_row", lambda: native.gemm(h, w_row))):
        dist.barrier()
        rows[name] = _max_over_ranks(timed(fn, args.warmup, args.iters))
    native.check_status()
    remote = (world - 1) / world
    col_flops, row_flops = 2.0 * M * H * args.cols, 2.0 * M * args.inner * H
    col_roof = max(col_flops / (pk["bf16_tflops"] * 1e9), M * H * 2 * remote / (NVLINK_GBS * 1e6))
    row_roof = max(row_flops / (pk["bf16_tflops"] * 1e9), M * H * 2 * remote / (NVLINK_GBS * 1e6))
    if rank == 0:
        print(json.dumps({
            "world": world, "transfer_ctas": args.transfer_ctas, "shape": {"M": M, "hidden": H, "cols": args.cols, "inner": args.inner},
            "ms": {k: round(v, 4) for k, v in rows.items()},
            "allgather_gemm": {"roofline_ms": round(col_roof, 4),
                               "fraction_of_roofline": round(col_roof / rows["fused_allgather_gemm"], 3),
                               "speedup_vs_nccl": round(rows["nccl_allgather_then_gemm"] / rows["fused_allgather_gemm"], 3)},
            "gemm_reducescatter": {"roofline_ms": round(row_roof, 4),
                                   "fraction_of_roofline": round(row_roof / rows["fused_gemm_reducescatter"], 3),
                                   "speedup_vs_nccl": round(rows["nccl_gemm_then_reducescatter"] / rows["fused_gemm_reducescatter"], 3)},
            "peaks": pk, "nvlink_gbs": NVLINK_GBS,
        }))
    dist.barrier()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
