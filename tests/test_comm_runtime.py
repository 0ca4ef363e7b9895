"""Descriptor broker (CPU, two processes) and symmetric-arena collectives (GPU ranks as child processes)."""

import os
import subprocess
import sys
import tempfile
from pathlib import Path

import pytest
import torch

from tests.helpers import run_gloo

ROOT = Path(__file__).resolve().parent.parent


def _broker_worker(rank: int, world: int, tmp: str) -> None:
    import torch.distributed as dist

    from research_b200.parallel.symmetric import exchange_descriptors

    path = os.path.join(tmp, f"payload-{rank}.txt")
    with open(path, "w") as f:
        f.write(f"hello from rank {rank}")
    fd = os.open(path, os.O_RDONLY)
    fds = exchange_descriptors(dist.group.WORLD, fd, tag="test")
    assert len(fds) == world
    for r, got in enumerate(fds):
        # a passed descriptor shares its file offset with every process that holds it: read at an explicit position
        assert os.pread(got, 64, 0).decode() == f"hello from rank {r}"
        if r != rank:
            os.close(got)
    os.close(fd)


def test_descriptor_broker_passes_open_files_between_ranks(tmp_path):
    run_gloo(3, _broker_worker, str(tmp_path))


def test_descriptor_fetch_gives_up_without_a_server(tmp_path):
    from research_b200.native import hostlib

    host = hostlib.load()
    assert host is not None
    rc = host.b200h_fd_fetch(str(tmp_path / "nobody.sock").encode(), 200)
    assert rc < 0  # -ETIMEDOUT / -ENOENT path: bounded, no hang


_GPU_SCRIPT = r"""
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, sys.argv[1])
from research_b200.ops import native
from research_b200.parallel.symmetric import SymmetricArena
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
want_mc = sys.argv[2] == "nvls"
torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
n = 1 << 20
arena = SymmetricArena(dist.group.WORLD, world * n * 4 + world * n * 2 + 4096, multicast=want_mc)
if want_mc:
    assert arena.mc_ptr != 0, "the arena was not bound to a multicast object"
grads, g_off = arena.carve(world * n, torch.float32)
weights, w_off = arena.carve(world * n, torch.bfloat16)
modes = [False, True] if want_mc else [False]          # plain peer loads, then multimem through the switch
for it in range(3):
  for nvls in modes:
    torch.manual_seed(100 * it + rank)
    grads.copy_(torch.randn(world * n, device="cuda"))
    ref = grads.clone()
    dist.all_reduce(ref)
    ref = ref[rank * n:(rank + 1) * n] * 0.5
    sumsq = torch.zeros(1, device="cuda")
    arena.reduce_scatter(g_off + 4 * rank * n, n, scale=0.5, sumsq=sumsq, nvls=nvls)
    native.check_status()
    got = grads[rank * n:(rank + 1) * n]
    assert torch.allclose(got, ref, atol=1e-5, rtol=1e-5), (nvls, (got - ref).abs().max().item())
    assert abs(sumsq.item() - ref.double().pow(2).sum().item()) <= 1e-3 * ref.double().pow(2).sum().item()
    weights.zero_()
    weights[rank * n:(rank + 1) * n] = (rank + 1 + it)
    arena.all_gather(w_off, n * 2, nvls=nvls)
    native.check_status()
    want = torch.arange(1, world + 1, device="cuda").repeat_interleave(n).to(torch.bfloat16) + it
    assert torch.equal(weights, want), nvls
# slices of different sizes per rank (rank 0 owns nothing), a capped grid, a side stream: the shape of the
# bucketed reduction that overlaps the backward pass
side = torch.cuda.Stream()
for nvls in modes:
    torch.manual_seed(7 + rank)
    grads.copy_(torch.randn(world * n, device="cuda"))
    ref = grads.clone()
    dist.all_reduce(ref)
    sizes = [4096 * r for r in range(world)]
    starts = [sum(sizes[:r]) for r in range(world)]
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        arena.reduce_scatter(g_off + 4 * starts[rank], sizes[rank], nvls=nvls, max_ctas=16, channel=6)
    torch.cuda.current_stream().wait_stream(side)
    native.check_status()
    a, b = starts[rank], starts[rank] + sizes[rank]
    assert torch.allclose(grads[a:b], ref[a:b], atol=1e-5, rtol=1e-5), nvls
arena.check_canaries()                      # nothing wrote past the end of a buffer, here or from a peer
torch.cuda.synchronize()
dist.barrier()
arena.close()
dist.destroy_process_group()
print("RANK_OK", rank)
"""


@pytest.mark.gpu
@pytest.mark.parametrize("transport", ["peer", "nvls"])
def test_symmetric_arena_collectives_on_all_visible_gpus(tmp_path, transport):
    """``peer``: plain loads from the peers' arenas.  ``nvls``: the arena is bound to an NVLink multicast object
    and the same collectives also run as ``multimem.ld_reduce`` / ``multimem.st``.  Every rank runs to the end and
    closes the arena (unbinding it) before it exits."""

    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    script = tmp_path / "arena_ranks.py"
    script.write_text(_GPU_SCRIPT)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    port = "29731" if transport == "peer" else "29732"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", port, str(script), str(ROOT), transport]
    proc = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    assert proc.stdout.count("RANK_OK") == world


_TP_SCRIPT = r"""
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, sys.argv[1])
from research_b200.ops import native
from research_b200.parallel.tensor_fused import TensorParallelFusion, column_linear, row_linear
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
B, S, H, I = 2, 512 * world, 512, 1024          # I = this rank's slice of the intermediate size
s_local = S // world
fusion = TensorParallelFusion(dist.group.WORLD, max_shard_elems=B * s_local * max(H, I), max_out_elems=B * s_local * max(H, I))

def gather_seq(t):   # [B, S/tp, C] -> [B, S, C]
    out = [torch.empty_like(t) for _ in range(world)]
    dist.all_gather(out, t.contiguous())
    return torch.cat(out, dim=1)

def scatter_sum_seq(t):   # [B, S, C] partial -> [B, S/tp, C] summed
    full = t.float().clone()
    dist.all_reduce(full)
    return full[:, rank * s_local:(rank + 1) * s_local]

for it in range(3):
    torch.manual_seed(1000 * it + rank)
    x = (torch.randn(B, s_local, H, device="cuda") * 0.5).bfloat16()
    w1 = (torch.randn(I, H, device="cuda") * 0.05).bfloat16()
    w2 = (torch.randn(H, I, device="cuda") * 0.05).bfloat16()
    # raw kernels, both operand layouts
    y, x_full = fusion.gather_gemm(x.reshape(B * s_local, H), w1, b_mn=False, chunk_rows=s_local)
    native.check_status()
    xg = gather_seq(x).reshape(B * S, H)
    assert torch.equal(x_full, xg), "gathered operand differs"
    ref = xg.float() @ w1.float().t()
    assert torch.allclose(y.float(), ref, atol=3e-2, rtol=3e-2), (y.float() - ref).abs().max().item()
    y_t, _ = fusion.gather_gemm(x.reshape(B * s_local, H), w1.t().contiguous(), b_mn=True, chunk_rows=s_local)
    assert torch.allclose(y_t.float(), ref, atol=3e-2, rtol=3e-2)
    h = (torch.randn(B, S, I, device="cuda") * 0.5).bfloat16()
    z = fusion.gemm_scatter(h.reshape(B * S, I), w2, b_mn=False, chunk_rows=s_local)
    native.check_status()
    zref = scatter_sum_seq((h.float() @ w2.float().t())).reshape(B * s_local, H)
    assert torch.allclose(z.float(), zref, atol=6e-2, rtol=3e-2), (z.float() - zref).abs().max().item()
    # autograd chain: column-parallel then row-parallel, against the collective formulation in fp32
    p1 = torch.nn.Parameter(w1.clone()); p2 = torch.nn.Parameter(w2.clone())
    p1.main_grad = torch.zeros(I, H, device="cuda"); p2.main_grad = torch.zeros(H, I, device="cuda")
    xr = x.clone().requires_grad_(True)
    out = row_linear(torch.nn.functional.silu(column_linear(xr, p1, fusion)), p2, fusion)
    g = (torch.randn_like(out.float()) * 0.1).bfloat16()
    out.backward(g)
    native.check_status()
    xf = x.float().clone().requires_grad_(True)
    w1f = w1.float().clone().requires_grad_(True); w2f = w2.float().clone().requires_grad_(True)
    class _G(torch.autograd.Function):
        @staticmethod
        def forward(ctx, t): return gather_seq(t)
        @staticmethod
        def backward(ctx, d): return scatter_sum_seq(d)
    class _S(torch.autograd.Function):
        @staticmethod
        def forward(ctx, t): return scatter_sum_seq(t)
        @staticmethod
        def backward(ctx, d): return gather_seq(d.contiguous())
    ref_out = _S.apply(torch.nn.functional.silu(_G.apply(xf) @ w1f.t()) @ w2f.t())
    ref_out.backward(g.float())
    assert torch.allclose(out.float(), ref_out, atol=6e-2, rtol=5e-2), (out.float() - ref_out).abs().max().item()
    assert torch.allclose(xr.grad.float(), xf.grad, atol=3e-2, rtol=5e-2), (xr.grad.float() - xf.grad).abs().max().item()
    for mg, rg in ((p1.main_grad, w1f.grad), (p2.main_grad, w2f.grad)):
        assert (mg - rg).abs().max().item() <= 0.03 * rg.abs().max().item() + 1e-3
fusion.arena.check_canaries()               # the TMA reduce-adds of the peers stayed inside the output buffer
torch.cuda.synchronize()
dist.barrier()
dist.destroy_process_group()
print("RANK_OK", rank)
"""


@pytest.mark.gpu
def test_fused_tensor_parallel_gemms_match_collective_formulation(tmp_path):
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    script = tmp_path / "tp_ranks.py"
    script.write_text(_TP_SCRIPT)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", "29733", str(script), str(ROOT)]
    proc = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    assert proc.stdout.count("RANK_OK") == world


_EP_SCRIPT = r"""
import os, sys, torch, torch.distributed as dist
from types import SimpleNamespace
sys.path.insert(0, sys.argv[1])
from research_b200.ops import functional as Fn
from research_b200.ops import native
from research_b200.ops.grouped import _GroupedLinearFn
from research_b200.parallel import expert_fused as ef
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
E, k, T = 4 * world, 2, 1536
ex = SimpleNamespace(ep_size=world, ep_rank=rank, ep_group=dist.group.WORLD, ep_dispatcher="all_to_all",
                     extras={"moe_layer_count": 1})
for it, (H, N) in enumerate([(256, 256), (2176, 128), (4096, 64)]):     # 512-byte rows, 17 chunks of 256 bytes, 2 of 4 KB
    torch.manual_seed(100 * it + rank)
    El = E // world
    x = (torch.randn(T, H, device="cuda") * 0.5).bfloat16()
    ids = torch.topk(torch.randn(T, E, device="cuda"), k, dim=-1).indices.to(torch.int32)
    if it == 1:
        ids[:, 0] = 0                                # a hot expert: the capacity drops assignments, others stay empty
        ids[:, 1] = 1 + (ids[:, 1] % 2)
    capacity = int(1.25 * T * k / E)
    w_a = torch.nn.Parameter((torch.randn(El, N, H, device="cuda") * 0.05).bfloat16())
    w_b = torch.nn.Parameter(w_a.detach().clone())
    w_a.main_grad = torch.zeros(El, N, H, device="cuda"); w_b.main_grad = torch.zeros(El, N, H, device="cuda")
    plan = ef.ExpertParallelPlan(ids, E, capacity, ex, H, layer_slot=0)
    ws = plan.ws
    assert ws is not None and ws.xbox is not None and ws.inbox_for(0)[2]
    rows = plan.rows_per_rank
    live = (plan.owner.tile_group >= 0).repeat_interleave(128)                # rows of tiles that hold an expert
    g = (torch.randn(rows, N, device="cuda") * 0.1).bfloat16()
    # push + barrier + grouped GEMM
    xa = x.clone().requires_grad_(True)
    rows_a = ef._EpDispatchFn.apply(xa, plan, ws)
    kept_a = rows_a.detach().clone()
    ya = _GroupedLinearFn.apply(rows_a, w_a, plan.owner, None, ws.outbox[:rows])
    (ya.float() * g.float())[live].sum().backward()
    native.check_status()
    ya = ya.detach().clone()
    # one kernel: the owner pulls the rows and multiplies tiles as they land
    ws.inbox_for(0)[0].fill_(7.0)                                             # nothing of the first pass may survive
    dist.barrier()
    xb = x.clone().requires_grad_(True)
    yb = ef._EpDispatchLinearFn.apply(xb, w_b, plan, ws)
    (yb.float() * g.float())[live].sum().backward()
    native.check_status()
    kept_b = ws.inbox_for(0)[0][:rows]
    assert torch.equal(kept_a[live], kept_b[live]), "dispatched rows differ"
    assert torch.allclose(ya[live].float(), yb[live].float(), atol=1e-2, rtol=1e-2), (ya[live].float() - yb[live].float()).abs().max().item()
    ref = torch.zeros(rows, N, device="cuda")
    tg = plan.owner.tile_group.repeat_interleave(128)
    for e in range(El):
        sel = tg == e
        ref[sel] = kept_a[sel].float() @ w_a[e].float().t()
    assert torch.allclose(yb[live].float(), ref[live], atol=3e-2, rtol=3e-2), (yb[live].float() - ref[live]).abs().max().item()
    assert torch.allclose(xa.grad.float(), xb.grad.float(), atol=1e-2, rtol=1e-2)
    assert (w_a.main_grad - w_b.main_grad).abs().max().item() <= 1e-2 * w_a.main_grad.abs().max().item() + 1e-4
    ws.arena.check_canaries()
    dist.barrier()
torch.cuda.synchronize()
dist.barrier()
dist.destroy_process_group()
print("RANK_OK", rank)
"""


@pytest.mark.gpu
def test_fused_expert_dispatch_gemm_matches_push_then_grouped_gemm(tmp_path):
    """Dispatched rows (bit for bit), expert outputs, input gradients and weight gradients of the kernel that pulls
    rows and multiplies tiles as they land, against the push + barrier + grouped GEMM sequence and an fp32 product."""

    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    script = tmp_path / "ep_ranks.py"
    script.write_text(_EP_SCRIPT)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", RESEARCH_B200_PEER_WAIT_MS="3000")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", "29735", str(script), str(ROOT)]
    proc = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    assert proc.stdout.count("RANK_OK") == world


_TRAIN_SCRIPT = r"""
import json, os, sys, numpy as np, torch, torch.distributed as dist
sys.path.insert(0, sys.argv[1])
from research_b200.config import run_spec_from_mapping
from research_b200.contracts import Batch
from research_b200.ops import native
from research_b200.parallel.mesh import init_distributed
from research_b200.runtime.trainer import Trainer
axes, sizes, flags = json.loads(sys.argv[2]), json.loads(sys.argv[3]), json.loads(sys.argv[4])
init_distributed()
rank = dist.get_rank()
raw = {
    "run": {"id": "fused-parity"},
    "model": {"name": "decoder", "variant": "t", "vocab_size": 1024, "hidden_size": 256, "intermediate_size": 512,
              "num_layers": 2, "num_heads": 4, "n_kv_heads": 2, "max_seq_len": 512, "init": "normal_0.02"},
    "optimizer": {"name": flags.get("optimizer", "adamw"), "grad_clip_norm": 1.0, "schedule": {"peak_lr": 1e-3},
                  "muon_tp_mode": flags.get("muon_tp_mode", "duplicated")},
    "data": {"train_manifest": "unused.json"},
    "training": {"seq_len": 512, "global_batch_size": 4, "target_tokens": 4 * 512 * 8, "precision": "bf16"},
    "mesh": {"axis_names": axes, "axis_sizes": sizes},
    "parallelism": flags.get("parallelism", {}),
}
raw["model"].update(flags.get("model", {}))
trainer = Trainer(run_spec_from_mapping(raw), build_data=False)
rng = np.random.default_rng(0)
losses = []
for step in range(4):
    ids = rng.integers(0, 1024, size=(4, 513)).astype(np.int32)
    batch = Batch(input_ids=ids[:, :-1], target_ids=ids[:, 1:], loss_mask=np.ones((4, 512), dtype=bool))
    m = trainer.train_on([batch])
    losses.append(float(m.loss))
native.check_status()
# the whole logical parameter tree after four steps (a collective gather: every rank takes part)
from research_b200.runtime.state_io import collect_state_tensors
state = collect_state_tensors(trainer)
if rank == 0:
    print("LOSSES", json.dumps(losses))
    np.savez(sys.argv[5], **{k: v for k, v in state.items() if k.startswith("model.")})
dist.barrier()
trainer.close()
dist.destroy_process_group()
"""


def _run_training(tmp_path, world, axes, sizes, flags, peer, port, extra_env=None):
    """Returns ``(losses of four steps, logical parameters after them)`` of a ``world``-rank run."""

    import json

    import numpy as np

    script = tmp_path / "train_ranks.py"
    script.write_text(_TRAIN_SCRIPT)
    out = tmp_path / f"params_{port}.npz"
    # RESEARCH_B200_DEBUG=1: after every step the trainer checks the guard words behind all peer-memory buffers
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", RESEARCH_B200_PEER_COLLECTIVES="1" if peer else "0",
               RESEARCH_B200_DEBUG="1", **(extra_env or {}))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), str(script), str(ROOT), json.dumps(axes),
           json.dumps(sizes), json.dumps(flags), str(out)]
    proc = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    line = [l for l in proc.stdout.splitlines() if l.startswith("LOSSES")][-1]
    with np.load(out) as data:
        params = {k: data[k] for k in data.files}
    return json.loads(line.split(" ", 1)[1]), params


@pytest.mark.gpu
@pytest.mark.parametrize("name,axes,sizes,flags", [
    ("tp2", ["tp"], [2], {"parallelism": {"mode": "ddp", "tensor_parallel": True}}),
    ("fsdp2_muon", ["fsdp"], [2], {"parallelism": {"mode": "fsdp"}, "optimizer": "muon"}),
    # the opt-in form: every layer's gradients are reduced on a side stream while earlier layers are in backward
    ("fsdp2_muon_overlapped_reduce", ["fsdp"], [2], {"parallelism": {"mode": "fsdp"}, "optimizer": "muon",
                                                     "env": {"RESEARCH_B200_OVERLAP_REDUCE": "1"}}),
    ("moe_fsdp2_ep2", ["fsdp"], [2], {
        "parallelism": {"mode": "fsdp", "expert_parallel": True},
        "model": {"name": "trinity", "num_layers": 2, "trinity": {
            "initial_dense_layers": 0, "local_window": 512, "local_layers_per_global": 1, "norm_policy": "afmoe_dual",
            "moe": {"num_experts": 8, "top_k": 2, "expert_intermediate_size": 256, "num_shared_experts": 1,
                    "capacity_factor": 1.5}}}}),
    # a dedicated ep axis: tokens are replicated over it, every rank dispatches its slice of them
    ("moe_ep2_dedicated", ["ep"], [2], {
        "parallelism": {"mode": "ddp", "expert_parallel": True},
        "model": {"name": "trinity", "num_layers": 2, "trinity": {
            "initial_dense_layers": 0, "local_window": 512, "local_layers_per_global": 1, "norm_policy": "afmoe_dual",
            "moe": {"num_experts": 8, "top_k": 2, "expert_intermediate_size": 256, "num_shared_experts": 1,
                    "capacity_factor": 2.0}}}}),
    # Newton-Schulz on tensor-parallel shards: packed Gram reductions through the symmetric arena against NCCL
    ("tp2_muon_distributed", ["tp"], [2], {"parallelism": {"mode": "ddp", "tensor_parallel": True},
                                           "optimizer": "muon", "muon_tp_mode": "distributed"}),
    # context parallelism: K/V exchange inside the attention kernels against all-gather + reduce-scatter
    ("cp2_ring", ["cp"], [2], {"parallelism": {"mode": "ddp", "context_parallel": True},
                               "model": {"attention_doc_mask": False}}),
    # lm_head split over the vocabulary: max / sum-exp / target-logit reductions over the tensor-parallel group
    ("tp2_vocab_parallel_head", ["tp"], [2], {"parallelism": {"mode": "ddp", "tensor_parallel": True,
                                                              "vocab_parallel_head": True}}),
    # weights sharded at rest: every layer's weights are fetched from their owners' arenas before the layer runs
    ("fsdp2_muon_sharded_params", ["fsdp"], [2], {"parallelism": {"mode": "fsdp", "fsdp_resident": False},
                                                  "optimizer": "muon"}),
    # the same FSDP run with the arena bound to an NVLink multicast object (multimem reduce-scatter / all-gather)
    ("fsdp2_muon_nvls", ["fsdp"], [2], {"parallelism": {"mode": "fsdp"}, "optimizer": "muon",
                                        "env": {"RESEARCH_B200_NVLS": "1"}}),
])
def test_training_with_peer_memory_kernels_matches_nccl_path(tmp_path, name, axes, sizes, flags):
    """Four optimizer steps through the peer-memory kernels and through NCCL: the losses agree and so does every
    logical parameter afterwards (a gradient that is wrong but small would move the parameters apart)."""

    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least two GPUs")
    extra = flags.get("env")
    fused, p_fused = _run_training(tmp_path, 2, axes, sizes, flags, True, 29741, extra)
    plain, p_plain = _run_training(tmp_path, 2, axes, sizes, flags, False, 29743)
    assert len(fused) == len(plain) == 4
    for a, b in zip(fused, plain):
        assert abs(a - b) <= 2e-2 * max(1.0, abs(b)), (name, fused, plain)
    assert fused[-1] < fused[0]
    assert set(p_fused) == set(p_plain) and p_fused
    import numpy as np

    for key, want in p_plain.items():
        got = p_fused[key]
        # Four steps at lr 1e-3 move a weight by up to 4e-3.  Adam-style updates turn a rounding-level difference of
        # a tiny gradient into a full-size step for that one element, so single elements may differ by a step or
        # two; a wrong gradient moves whole tensors, which the mean difference catches.
        diff = np.abs(got.astype(np.float64) - want.astype(np.float64))
        # routed models: a token whose k-th and (k+1)-th router scores are a rounding apart may go to another expert
        # on one of the two paths from the second step on, which moves more elements by a step than rounding alone
        # (the router's own small weight matrix takes the brunt of such flips)
        mean_limit = (1.5e-3 if "router" in key else 6e-4) if name.startswith("moe") else 2e-4
        assert diff.mean() <= mean_limit, (name, key, "mean", float(diff.mean()))
        assert diff.max() <= 8e-3, (name, key, "max", float(diff.max()))


@pytest.mark.gpu
def test_bounded_peer_wait_times_out_with_a_status_code():
    """A barrier whose peer never announces itself gives up after its limit and reports a status code; the
    context stays usable (nothing traps, nothing hangs)."""

    import ctypes
    import time

    from research_b200.errors import KernelError
    from research_b200.ops import native
    from research_b200.parallel.symmetric import _comm_lib

    lib = _comm_lib()
    nbytes = lib.b200c_flag_block_bytes()
    blocks = torch.zeros(2, nbytes, dtype=torch.uint8, device="cuda")      # flag blocks of "rank 0" and "rank 1"
    flags = (ctypes.c_void_p * 2)(blocks[0].data_ptr(), blocks[1].data_ptr())
    native.check_status()
    native.set_peer_wait_limit_ms(1500)                                     # training default: 30 s
    t0 = time.perf_counter()
    try:
        rc = lib.b200c_barrier(flags, 2, 0, 7, native.status_word().data_ptr(), native._stream())
        assert rc == 0
        with pytest.raises(KernelError, match="status code 21"):            # ERR_PEER_READY
            native.check_status()
    finally:
        native.set_peer_wait_limit_ms(native.peer_wait_limit_ms())
    waited = time.perf_counter() - t0
    assert 1.0 < waited < 10.0, waited
    # the announcement this rank made is in the peer's block, and the device still works
    ready = blocks[1].view(torch.int32)[:8]
    assert int(ready[0]) == 7
    x = torch.ones(1024, device="cuda")
    assert float(x.sum()) == 1024.0
    native.check_status()
