"""Generation benchmark: prefill latency, time to first token and decode tokens/s.

Methodology follows the reference's inference bench (src/research/utils/inference_bench.py:31-125: timed prefill,
first token, then a fixed number of decode steps) with the batch, prompt length and sampler as parameters, so both
its defaults (batch 1, prompt min(512, S/2), 128 new tokens, greedy) and a serving-like load (batch 32, prompt 2048,
256 new tokens, temperature 1.0, top-k 50) can be run.  Weights are random-init; prompts are uniform random ids.

``python -m research_b200.runtime.inference_bench --config CONFIG.toml --batch 32 --prompt 2048 --new 256 --top-k 50``
"""

from __future__ import annotations

import argparse
import json
import time

import torch

from research_b200.config import load_config
from research_b200.infer import generation


def run_inference_bench(spec, *, batch: int, prompt: int, new_tokens: int, temperature: float, top_k: int | None,
                        warmup: int = 1, repeats: int = 3, seed: int = 0, device: str | None = None,
                        use_graph: bool = True) -> dict:
    import dataclasses
    import os

    from research_b200.config.specs import MeshSpec, ParallelismSpec
    from research_b200.runtime.trainer import Trainer

    if int(os.environ.get("WORLD_SIZE", "1")) == 1:
        # generation runs on one replica: drop the training mesh of the config
        spec = dataclasses.replace(spec, mesh=MeshSpec(), parallelism=ParallelismSpec())
    trainer = Trainer(spec, build_data=False, device=device)
    model = trainer.result.model
    model.eval()
    dev = next(model.parameters()).device
    g = torch.Generator(device="cpu").manual_seed(seed)
    prompts = torch.randint(0, spec.model.vocab_size, (batch, prompt), generator=g, dtype=torch.int32).to(dev)
    cuda = dev.type == "cuda"

    def sync():
        if cuda:
            torch.cuda.synchronize()

    def one_run():
        with torch.no_grad():
            cache = generation.init_kv_cache(model, batch, prompt + new_tokens)
            gen = torch.Generator(device=dev).manual_seed(seed)
            pos = torch.arange(prompt, device=dev, dtype=torch.int32).expand(batch, prompt).contiguous()
            sync()
            t0 = time.perf_counter()
            logits = model.run_with_cache(prompts, pos, cache, last_only=True)[:, -1]
            cache.advance(pos)
            sync()
            t_prefill = time.perf_counter() - t0
            tok, _ = generation.sample_next_token(logits, temperature=temperature, top_k=top_k, top_p=None,
                                                  generator=gen)
            sync()
            t_first = time.perf_counter() - t0
            t1 = time.perf_counter()
            step = None
            if use_graph and cuda:
                step = generation.GraphedDecodeStep(model, cache, tok, prompt)  # capture is outside the timed loop
                sync()
                t1 = time.perf_counter()
            for t in range(new_tokens - 1):
                if step is not None:
                    logits = step(tok, prompt + t)
                else:
                    p1 = torch.full((batch, 1), prompt + t, device=dev, dtype=torch.int32)
                    logits = model.run_with_cache(tok[:, None].to(torch.int32), p1, cache, last_only=True)[:, -1]
                    cache.advance(p1)
                tok, _ = generation.sample_next_token(logits, temperature=temperature, top_k=top_k, top_p=None,
                                                      generator=gen)
            sync()
            t_decode = time.perf_counter() - t1
        return t_prefill, t_first, t_decode

    for _ in range(warmup):
        one_run()
    runs = [one_run() for _ in range(repeats)]
    all_prefill = [1e3 * r[0] for r in runs]
    runs.sort(key=lambda r: r[2])
    _, t_first, t_decode = runs[len(runs) // 2]
    t_prefill = sorted(all_prefill)[len(all_prefill) // 2] * 1e-3        # each figure is the median of its own runs
    steps = max(new_tokens - 1, 1)
    return {
        "metric": "decode_tokens_per_sec",
        "value": batch * steps / t_decode,
        "unit": "tokens/s",
        "decode_ms_per_step": 1e3 * t_decode / steps,
        "prefill_ms": 1e3 * t_prefill,
        "prefill_ms_all_runs": all_prefill,
        "prefill_tokens_per_sec": batch * prompt / t_prefill,
        "ttft_ms": 1e3 * t_first,
        "batch": batch, "prompt_tokens": prompt, "new_tokens": new_tokens, "temperature": temperature, "top_k": top_k,
        "cuda_graph": bool(use_graph and cuda), "model": spec.model.name, "device": str(dev), "dtype": str(next(model.parameters()).dtype),
        "data": "synthetic (random-init weights, uniform random prompt ids)",
    }


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--config", required=True)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--prompt", type=int, default=None)
    ap.add_argument("--new", type=int, default=128)
    ap.add_argument("--temperature", type=float, default=1.0)
    ap.add_argument("--top-k", type=int, default=1)
    ap.add_argument("--repeats", type=int, default=3)
    ap.add_argument("--device", default=None)
    ap.add_argument("--no-graph", action="store_true", help="launch every decode kernel separately")
    args = ap.parse_args(argv)
    spec = load_config(args.config)
    prompt = args.prompt if args.prompt is not None else min(512, spec.model.max_seq_len // 2)
    out = run_inference_bench(spec, batch=args.batch, prompt=prompt, new_tokens=args.new, temperature=args.temperature,
                              top_k=args.top_k, repeats=args.repeats, device=args.device, use_graph=not args.no_graph)
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
