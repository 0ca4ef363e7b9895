"""Fused tensor-parallel GEMMs against their NCCL + GEMM formulation, with roofline fractions.

Run one process per GPU, e.g.
``python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29611 \
-m research_b200.parallel.bench_tensor_fused --batch 2 --seq 8192 --hidden 4096 --cols 3072``.

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


def main() -> int:
    ap = argparse.ArgumentParser()
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
