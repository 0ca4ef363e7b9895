"""Headline benchmark: training throughput (tokens/s, MFU) of the dense ~1.3B decoder on N GPUs of one node.

Config (weak scaling, per-GPU work fixed): 24 layers, d_model 2048, 16 query / 8 KV heads (head_dim 128), SwiGLU
5632, RMSNorm, RoPE, QK-norm, vocab 50304, normal(0, 0.02) init; bf16 compute with fp32 masters; seq_len 4096
with document-boundary attention masks from geometric(mean 1500) document lengths and uniform random token ids;
8 sequences per GPU (global batch 64 at 8 GPUs), grad-accum 1; mesh fsdp=N; Muon on 2-D weights (distributed
over the fsdp axis), AdamW on embeddings, lm_head and norms.

Prints ONE JSON line on rank 0.  ``value`` is device-timed (CUDA events on the compute stream, max over ranks)
over K optimizer steps whose host batches were prepared beforehand; ``e2e`` times K more steps through the public
``Trainer.train_step()`` call with the wall clock between barriers + synchronizes, including the data pipeline,
the pinned host->device copy of every step's tokens and the device->host read of the step's loss.

``--impl reference`` runs the unmodified reference from ``baseline/_ref`` when it can be imported there.
``--impl library`` runs the same model, data, optimizer and mesh of THIS package on stock PyTorch operators only
(cuBLAS matmuls, ``scaled_dot_product_attention``, plain tensor ops in the optimizer, NCCL collectives; none of this
package's kernels): the stand-in for an "NCCL + cuBLAS build" on the same box.  The native line carries that
comparison measured in the same process under ``vs_library`` (``--no-library`` skips it), and at one GPU a
``decode`` record (batch 32, prompt 2048, 256 new tokens, temperature 1.0, top-k 50; ``--no-decode`` skips it).
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

REPO = Path(__file__).resolve().parent

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))


def reference_arm(args) -> int:
    ref = ROOT / "baseline" / "_ref"
    reason = None
    if not (ref / "jaxtitan").is_dir():
        reason = "baseline/_ref/jaxtitan is missing (offline pip install of the reference did not run)"
    else:
        sys.path.insert(0, str(ref))
        try:
            import jax  # noqa: F401
            import jaxtitan.runtime.training  # noqa: F401
        except Exception as exc:  # jax / flax / optax / orbax / grain are not installable offline
            reason = f"reference imports fail in this image: {type(exc).__name__}: {exc}"
    if reason is None:
        reason = "reference importable but its JAX runtime path is not wired for this benchmark"
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": reason}))
    return 0


class ClockSampler:
    """Samples SM clocks / throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.rows: list[list[str]] = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        def pump():
            for line in self.proc.stdout:
                self.rows.append([c.strip() for c in line.split(",")])
        self.thread = threading.Thread(target=pump, daemon=True)
        self.thread.start()

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for r in self.rows:
            if len(r) < 9:
                continue
            try:
                sm.append(float(r[1])); mx.append(float(r[2]))
            except ValueError:
                continue
            for name, val in zip(names, r[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def dense_1p3b_spec(n_gpus: int, manifest: Path, steps_total: int, per_gpu_batch: int, seq_len: int, optimizer: str):
    from research_b200.config import run_spec_from_mapping

    gb = per_gpu_batch * n_gpus
    raw = {
        "run": {"id": "bench-dense-1p3b", "seed": 0, "output_dir": "/tmp/research_b200_bench"},
        "model": {"name": "decoder", "variant": "dense-1p3b", "vocab_size": 50304, "hidden_size": 2048,
                  "intermediate_size": 5632, "num_layers": 24, "num_heads": 16, "n_kv_heads": 8,
                  "max_seq_len": seq_len, "rope_theta": 10000.0, "init": "normal_0.02", "attention_doc_mask": True,
                  "compute_dtype": "bfloat16", "param_dtype": "float32", "remat": "none"},
        "optimizer": {"name": optimizer, "weight_decay": 0.0, "grad_clip_norm": 1.0,
                      "schedule": {"name": "constant", "peak_lr": 3e-4, "warmup_steps": 10}},
        "data": {"train_manifest": str(manifest), "order": "document_buffer", "shuffle_seed": 0,
                 "document_buffer_size": 128, "document_refill_size": 128},
        "training": {"seq_len": seq_len, "global_batch_size": gb, "target_tokens": gb * seq_len * steps_total,
                     "precision": "bf16", "gradient_accumulation_steps": 1},
        "mesh": {"axis_names": ["fsdp"], "axis_sizes": [n_gpus]},
        "parallelism": {"mode": "fsdp"},
    }
    return run_spec_from_mapping(raw)


WORKLOADS = {
    # name: (config file, description, mesh builder)
    "dense_8b": ("dense_8b_fsdp4_tp2_adamw.toml", "dense-8B decoder (32L, d4096, 32q/8kv heads, ffn 14336, vocab 128256)"),
    "moe_7b": ("moe_7b_ep8_dion.toml", "MoE ~7B total (16L, d2048, 64 experts ffn 1024, top-8, 1 shared expert)"),
    "long_context": ("dense_1p3b_cp4_fsdp2_32k.toml", "dense-1.3B decoder, context parallel, seq 32768"),
}


def workload_spec(name: str, n_gpus: int, manifest: Path, steps_total: int, per_gpu_batch: int, seq_len: int | None,
                  optimizer: str | None, context_attention: str = "gather"):
    """The other named workloads, from their TOML files, re-meshed for ``n_gpus`` GPUs of one box."""

    import tomllib

    from research_b200.config import run_spec_from_mapping

    raw = tomllib.loads((REPO / "configs" / WORKLOADS[name][0]).read_text())
    if seq_len:
        raw["training"]["seq_len"] = seq_len
        raw["model"]["max_seq_len"] = seq_len
    seq_len = raw["training"]["seq_len"]
    if optimizer:
        raw["optimizer"]["name"] = optimizer
    if name == "dense_8b":
        tp = 2 if n_gpus >= 2 else 1
        axes, sizes, replicas = ["fsdp", "tensor"], [n_gpus // tp, tp], n_gpus // tp
        raw["parallelism"]["tensor_parallel"] = tp > 1
        parallelism = f"fsdp{n_gpus // tp}xtp{tp}"
    elif name == "long_context":
        cp = min(4, n_gpus)
        axes, sizes, replicas = ["fsdp", "context"], [n_gpus // cp, cp], n_gpus // cp
        raw["parallelism"]["context_parallel"] = cp > 1
        raw["parallelism"]["context_attention"] = context_attention
        parallelism = f"fsdp{n_gpus // cp}xcp{cp}" + ("(ulysses)" if context_attention == "ulysses" and cp > 1 else "")
    else:
        axes, sizes, replicas = ["fsdp"], [n_gpus], n_gpus
        raw["parallelism"]["expert_parallel"] = n_gpus > 1
        parallelism = f"fsdp{n_gpus}+ep{n_gpus}"
    gb = per_gpu_batch * replicas
    raw["mesh"] = {"axis_names": axes, "axis_sizes": sizes}
    raw["data"]["train_manifest"] = str(manifest)
    raw["run"]["output_dir"] = "/tmp/research_b200_bench"
    raw["training"].update(global_batch_size=gb, target_tokens=gb * seq_len * steps_total,
                           gradient_accumulation_steps=1)
    raw["optimizer"]["schedule"] = {"name": "constant", "peak_lr": 3e-4, "warmup_steps": 10}
    raw.pop("evals", None)
    return run_spec_from_mapping(raw), gb, parallelism


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", default="dense_1p3b", choices=["dense_1p3b", *WORKLOADS],
                    help="dense_1p3b is the headline config; the others are the remaining named workloads")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="native", choices=["native", "reference", "library"])
    ap.add_argument("--no-library", action="store_true", help="native arm: skip the in-process library comparison")
    ap.add_argument("--no-decode", action="store_true", help="native arm: skip the generation record (1 GPU only)")
    ap.add_argument("--kernel-table", default=None, metavar="FILE",
                    help="after the timed regions, run one more step under the torch profiler and write rank 0's "
                         "kernel-time table to FILE")
    ap.add_argument("--per-gpu-batch", type=int, default=8)
    ap.add_argument("--seq-len", type=int, default=None)
    ap.add_argument("--optimizer", default=None, choices=["muon", "adamw", "dion"])
    ap.add_argument("--context-attention", default="gather", choices=["gather", "ulysses"],
                    help="long_context only: K/V all-gather (default) or head <-> sequence all-to-all")
    args = ap.parse_args()
    headline = args.workload == "dense_1p3b"
    if headline:
        args.seq_len = args.seq_len or 4096
        args.optimizer = args.optimizer or "muon"
    if args.impl == "reference":
        return reference_arm(args)
    if args.impl == "library":
        os.environ["RESEARCH_B200_LIBRARY"] = "1"
        os.environ["RESEARCH_B200_PEER_COLLECTIVES"] = "0"

    import gc

    import numpy as np
    import torch
    import torch.distributed as dist

    from research_b200.data.synthetic import generate_synthetic_dataset
    from research_b200.ops import native
    from research_b200.parallel.mesh import init_distributed
    from research_b200.runtime.flops import estimate_flops_per_token, estimate_flops_per_token_exact
    from research_b200.runtime.trainer import Trainer

    rank, world = init_distributed()
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}; launch with torch.distributed.run for N>1")
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    K, W = args.steps, max(args.warmup, 3)
    steps_total = W + 2 * K + 2
    data_dir = Path(tempfile.gettempdir()) / f"research_b200_bench_data_{args.workload}_{world}_{args.seq_len}_{steps_total}"
    manifest = data_dir / "manifest.json"
    if headline:
        spec = dense_1p3b_spec(world, manifest, steps_total, args.per_gpu_batch, args.seq_len, args.optimizer)
        gb, parallelism = args.per_gpu_batch * world, f"fsdp{world}"
        model_desc = "dense-1.3B decoder (24L, d2048, 16q/8kv heads, ffn 5632, vocab 50304)"
    else:
        spec, gb, parallelism = workload_spec(args.workload, world, manifest, steps_total, args.per_gpu_batch,
                                              args.seq_len, args.optimizer, args.context_attention)
        model_desc = WORKLOADS[args.workload][1]
    args.seq_len = spec.training.seq_len
    args.optimizer = spec.optimizer.name
    tokens_needed = gb * (args.seq_len + 1) * steps_total
    if rank == 0 and not manifest.exists():
        mean_len = 3000 if args.workload == "dense_8b" else (6000 if args.workload == "long_context" else 1500)
        docs = int(tokens_needed / (mean_len * 0.93) * 1.25) + 256
        vocab = spec.model.vocab_size
        generate_synthetic_dataset(data_dir, seed=0, num_documents=docs, mean_length=mean_len, min_length=16,
                                   max_length=4 * args.seq_len, vocab_size=vocab, eos_id=vocab - 1, val_fraction=0.02,
                                   overwrite=True)
    if world > 1:
        dist.barrier()
    tokens_per_step = gb * args.seq_len

    def sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def measure(label: str) -> dict:
        """Build a trainer, warm up, then the device-timed region and the end-to-end region of one arm."""

        trainer = Trainer(spec)
        for _ in range(W):
            trainer.train_step()
        native.check_status()
        # ---- device-timed region: batches prepared on the host beforehand --------------------------
        prepared = [trainer.next_accumulated_batch() for _ in range(K)]
        sampler = ClockSampler(local_rank)
        sync()
        sampler.start()
        launches0 = native.LAUNCHES
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        last = None
        for batches in prepared:
            last = trainer.train_on(batches)
        end.record()
        sync()
        launches = native.LAUNCHES - launches0
        dev_ms = start.elapsed_time(end)
        # ---- end-to-end region through the public API -----------------------------------------------
        h2d0, d2h0 = trainer.train_step_fn.h2d_bytes[0], trainer.train_step_fn.d2h_bytes[0]
        sync()
        t0 = time.perf_counter()
        for _ in range(K):
            last = trainer.train_step()
        sync()
        e2e_s = time.perf_counter() - t0
        clocks = sampler.stop()
        native.check_status()
        h2d = (trainer.train_step_fn.h2d_bytes[0] - h2d0) / K
        d2h = (trainer.train_step_fn.d2h_bytes[0] - d2h0) / K
        times = torch.tensor([dev_ms, e2e_s * 1e3], dtype=torch.float64, device="cuda")
        if world > 1:
            dist.all_reduce(times, op=dist.ReduceOp.MAX)
        dev_ms, e2e_ms = times.tolist()
        if args.kernel_table and label == "native":
            # one more step under the torch profiler (outside every timed region): kernel time by name, rank 0
            from torch.profiler import ProfilerActivity, profile

            with profile(activities=[ProfilerActivity.CUDA]) as prof:
                trainer.train_step()
                torch.cuda.synchronize()
            if rank == 0:
                Path(args.kernel_table).write_text(
                    prof.key_averages().table(sort_by="cuda_time_total", row_limit=80, max_name_column_width=100))
            sync()
        out = {"label": label, "dev_ms": dev_ms, "e2e_ms": e2e_ms, "h2d": h2d, "d2h": d2h, "launches": launches,
               "clocks": clocks, "loss": None if last is None else round(last.loss, 4),
               "peak_mem_gb": round(torch.cuda.max_memory_allocated() / 2 ** 30, 2)}
        trainer.close()
        del trainer, prepared
        gc.collect()
        torch.cuda.empty_cache()
        torch.cuda.reset_peak_memory_stats()
        return out

    from research_b200.ops import functional as Fn

    arm = measure(args.impl)
    library = None
    if args.impl == "native" and not args.no_library:
        # the same spec on stock PyTorch operators and NCCL, in this process, right after the native arm
        Fn.set_library_mode(True)
        os.environ["RESEARCH_B200_PEER_COLLECTIVES"] = "0"
        try:
            library = measure("library")
        except Exception as exc:  # noqa: BLE001 - the comparison must never take the headline down with it
            library = {"error": f"{type(exc).__name__}: {exc}"[:300]}
        finally:
            Fn.set_library_mode(False)
            os.environ.pop("RESEARCH_B200_PEER_COLLECTIVES", None)
    decode = None
    if args.impl == "native" and world == 1 and headline and not args.no_decode:
        from research_b200.runtime.inference_bench import run_inference_bench

        try:
            rec = run_inference_bench(spec, batch=32, prompt=2048, new_tokens=256, temperature=1.0, top_k=50,
                                      warmup=1, repeats=3)
            decode = {k: (round(v, 3) if isinstance(v, float) else v) for k, v in rec.items()
                      if k in ("metric", "value", "unit", "decode_ms_per_step", "prefill_ms", "prefill_tokens_per_sec",
                               "ttft_ms", "batch", "prompt_tokens", "new_tokens", "temperature", "top_k", "cuda_graph")}
            decode["timing"] = "wall clock between synchronizes, median of 3 runs after 1 warm-up run"
        except Exception as exc:  # noqa: BLE001
            decode = {"error": f"{type(exc).__name__}: {exc}"[:300]}
    dev_ms, e2e_ms, h2d, d2h, launches, clocks = (arm["dev_ms"], arm["e2e_ms"], arm["h2d"], arm["d2h"],
                                                  arm["launches"], arm["clocks"])
    value = tokens_per_step * K / (dev_ms * 1e-3)
    e2e_value = tokens_per_step * K / (e2e_ms * 1e-3)
    fpt = estimate_flops_per_token(spec.model, args.seq_len)
    fpt_exact = estimate_flops_per_token_exact(spec.model, args.seq_len)
    peak = 2.25e15 * world
    if rank == 0:
        out = {
            "metric": "train_tokens_per_sec", "value": round(value, 1), "unit": "tokens/s", "n_gpus": world,
            "steps": K, "warmup": W, "ms_per_step": round(dev_ms / K, 3), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "impl": args.impl,
            "config": {"model": model_desc, "workload": args.workload,
                       "global_batch": gb, "seq_len": args.seq_len, "parallelism": parallelism,
                       "optimizer": args.optimizer, "grad_accum": 1,
                       "doc_masks": "geometric document lengths" if spec.model.attention_doc_mask else "none",
                       "timing": "CUDA events, max over ranks; inputs larger than L2 (activations of all tokens of a "
                                 "step per GPU)"},
            "mfu": round(100.0 * fpt * value / peak, 2), "mfu_exact": round(100.0 * fpt_exact * value / peak, 2),
            "flops_per_token": fpt, "peak_flops_per_gpu": 2.25e15,
            "e2e": {"value": round(e2e_value, 1), "unit": "tokens/s", "ms_per_step": round(e2e_ms / K, 3),
                    "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h)},
            "gpu_launches": int(launches), "clocks": clocks,
            "final_loss": arm["loss"], "peak_mem_gb": arm["peak_mem_gb"],
            "baseline_note": "the reference publishes no B200 number and no number for this config; nearest published: "
                             "dense 1.666B FSDP2xTP2 Muon 8,136 tok/s on 4xH100",
        }
        if library is not None:
            if "error" in library:
                out["vs_library"] = library
            else:
                lib_value = tokens_per_step * K / (library["dev_ms"] * 1e-3)
                lib_e2e = tokens_per_step * K / (library["e2e_ms"] * 1e-3)
                out["vs_library"] = {
                    "what": "same spec on stock PyTorch operators (cuBLAS, scaled_dot_product_attention, tensor-op "
                            "optimizer) and NCCL, same process, same timing; not the reference",
                    "value": round(lib_value, 1), "ms_per_step": round(library["dev_ms"] / K, 3),
                    "ratio": round(value / lib_value, 3), "e2e_value": round(lib_e2e, 1),
                    "e2e_ratio": round(e2e_value / lib_e2e, 3), "gpu_launches": int(library["launches"]),
                    "clocks": library["clocks"], "final_loss": library["loss"], "peak_mem_gb": library["peak_mem_gb"]}
        if decode is not None:
            out["decode"] = decode
        print(json.dumps(out))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
