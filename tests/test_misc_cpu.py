"""Small host-side pieces: the library attention path against the oracle, FLOP estimates, the kernel build cache,
the benchmark's reference arm, the named configs."""

import json
import subprocess
import sys
from pathlib import Path

import pytest
import torch

from research_b200.ops import functional as Fn

ROOT = Path(__file__).resolve().parent.parent


@pytest.mark.parametrize("docs", [False, True])
@pytest.mark.parametrize("hq,hkv", [(4, 4), (4, 2)])
def test_library_attention_matches_the_oracle(docs, hq, hkv):
    """The comparison arm's attention (``scaled_dot_product_attention``, grouped-query form, causal flag or a mask
    built from per-row bounds) is the same function as the package's fp32 oracle."""

    torch.manual_seed(0)
    B, S, D = 2, 48, 16
    q, k, v = torch.randn(B, S, hq, D), torch.randn(B, S, hkv, D), torch.randn(B, S, hkv, D)
    lo = None
    if docs:
        lo = torch.zeros(B, S, dtype=torch.int32)
        lo[0, 20:] = 20
        lo[1, 7:] = 7
        lo[1, 30:] = 30
    want = Fn.attention_reference(q, k, v, causal=True, lo=lo, scale=D ** -0.5)
    got = Fn.attention_library(q, k, v, causal=True, lo=lo, scale=D ** -0.5)
    assert torch.allclose(got, want, atol=1e-5, rtol=1e-5)


def test_library_mode_switch_forces_the_plain_implementations():
    assert Fn.native_enabled() and not Fn.library_mode()
    Fn.set_library_mode(True)
    try:
        assert Fn.library_mode() and not Fn.native_enabled()
        assert not Fn.use_native(torch.zeros(2))
    finally:
        Fn.set_library_mode(False)
    assert Fn.native_enabled()


def test_flop_estimates_follow_the_reference_formula():
    from research_b200.config import run_spec_from_mapping
    from research_b200.runtime.flops import estimate_flops_per_token, estimate_flops_per_token_exact
    from tests.helpers import tiny_raw_config

    spec = run_spec_from_mapping(tiny_raw_config(Path("m.json"))).model
    S = 32
    H, I, L, V, heads, kv, D = 64, 128, 2, 256, 4, 2, 16
    matmul = L * (H * heads * D + 2 * H * kv * D + heads * D * H + 3 * H * I) + H * V
    assert estimate_flops_per_token(spec, S) == 6 * matmul + 12 * L * heads * D * S
    exact = estimate_flops_per_token_exact(spec, S)
    assert 0 < exact <= estimate_flops_per_token(spec, S)            # causal attention counts half of the scores


def test_kernel_build_cache_is_keyed_by_the_sources():
    from research_b200.kernels import build

    first = build.build_all()
    again = build.build_all()
    assert again.digest == first.digest and not again.rebuilt
    manifest = json.loads(build.MANIFEST.read_text())
    assert manifest["digest"] == first.digest and manifest["arch"] == "sm_100a"
    assert "-gencode" in manifest["nvcc_flags"] and "arch=compute_100a,code=sm_100a" in manifest["nvcc_flags"]
    assert {"gemm.cu", "attention_fwd.cu", "attention_bwd.cu", "comm_runtime.cu", "comm_gemm.cu"} <= set(manifest["sources"])
    assert build.ensure_current() is not None


def test_benchmark_reference_arm_says_why_it_is_unavailable():
    proc = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference"], capture_output=True,
                          text=True, timeout=120)
    assert proc.returncode == 0, proc.stderr[-2000:]
    line = json.loads(proc.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and isinstance(line["unavailable"], str) and line["unavailable"]


@pytest.mark.parametrize("name", sorted(p.name for p in (ROOT / "configs").glob("*.toml")))
def test_named_configs_load_and_describe_their_mesh(name):
    from research_b200.config import load_config

    spec = load_config(ROOT / "configs" / name)
    assert spec.mesh.device_count >= 1 and spec.training.seq_len <= spec.model.max_seq_len
    assert spec.training.target_tokens >= spec.training.global_batch_size * spec.training.seq_len


def test_dion_optimizer_leaves_are_named_by_selection_axis(tmp_path):
    from research_b200.config import run_spec_from_mapping
    from research_b200.runtime.state_io import optimizer_leaf_names
    from research_b200.runtime.trainer import Trainer
    from tests.helpers import tiny_dataset, tiny_raw_config

    manifest = tiny_dataset(tmp_path)
    raw = tiny_raw_config(manifest, optimizer="muon")
    raw["optimizer"]["name"] = "dion"
    trainer = Trainer(run_spec_from_mapping(raw), device="cpu")
    names = optimizer_leaf_names(trainer)
    momentum = {k[1]: v for k, v in names.items() if k[0] == "momentum"}
    assert momentum and all(".inner_state.momentum." in v for v in momentum.values())
    # clip is chain element 0; the Dion2 groups come before the AdamW fallback, which is last
    adamw_index = int(names[("mu", "embed.embedding")].split(".")[1])
    assert all(int(v.split(".")[1]) < adamw_index for v in momentum.values())
    assert min(int(v.split(".")[1]) for v in momentum.values()) == 1
