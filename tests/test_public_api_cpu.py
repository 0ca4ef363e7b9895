"""The package-level names: every one resolves, aliases point at the right object, importing a package stays lazy."""

import importlib
import subprocess
import sys

import pytest

PACKAGES = ["config", "data", "infer", "kernels", "mesh", "models", "optim", "parallel", "services", "specs", "steps"]


@pytest.mark.parametrize("package", PACKAGES)
def test_every_public_name_resolves(package):
    module = importlib.import_module(f"research_b200.{package}")
    assert module.__all__ == sorted(set(module.__all__)) or package in ("config", "specs")
    for name in module.__all__:
        assert getattr(module, name) is not None, name
    assert set(module.__all__) <= set(dir(module))
    with pytest.raises(AttributeError):
        getattr(module, "no_such_name")


def test_names_a_user_of_the_reference_imports():
    from research_b200.config import load_config, run_spec_from_resolved_mapping  # noqa: F401
    from research_b200.data import (HFStreamingTextPipeline, PreparedTokenGrainPipeline, build_prepared_token_pipeline,  # noqa: F401
                                    inspect_dataset_manifest, prepare_dataset, validate_dataset_manifest)
    from research_b200.infer import KVCache, PagedKVCache, decode_one, generate_tokens, prefill, restore_inference_checkpoint  # noqa: F401
    from research_b200.kernels import compile_kernel_plan, format_kernel_plan, kernel_plan, kernel_registry  # noqa: F401
    from research_b200.mesh import MeshContext, build_mesh_context, require_single_process_runtime, validate_runtime_mesh_spec  # noqa: F401
    from research_b200.models import ModelBuildResult, ParamMeta, ParamMetadata, build_model, count_parameters, dtype_from_name  # noqa: F401
    from research_b200.optim import build_lr_schedule, build_optimizer, optimizer_policy_summary, zeropower_via_newton_schulz  # noqa: F401
    from research_b200.services import LocalArtifactWriter, LocalCheckpointService, LocalOrbaxCheckpointService, initialize_run  # noqa: F401
    from research_b200.specs import DatasetManifest, MeshSpec, ModelSpec, RunSpec, ShardInfo  # noqa: F401
    from research_b200.steps import MoeBalanceState, causal_lm_loss, make_eval_step, make_train_step  # noqa: F401

    assert KVCache is PagedKVCache and ParamMetadata is ParamMeta and LocalOrbaxCheckpointService is LocalCheckpointService


def test_small_api_functions():
    import torch

    from research_b200.config.specs import MeshSpec
    from research_b200.errors import ContractError
    from research_b200.mesh import validate_runtime_mesh_spec
    from research_b200.models import count_parameters, dtype_from_name

    assert dtype_from_name("bfloat16") is torch.bfloat16 and dtype_from_name("float32") is torch.float32
    with pytest.raises(ContractError, match="unsupported dtype name"):
        dtype_from_name("float8")
    validate_runtime_mesh_spec(MeshSpec())
    with pytest.raises(ContractError, match="need 2 devices but the job has 1 ranks"):
        validate_runtime_mesh_spec(MeshSpec(axis_names=("data",), axis_sizes=(2,)))
    with pytest.raises(ContractError, match="unsupported mesh axis"):
        validate_runtime_mesh_spec(MeshSpec(axis_names=("stage",), axis_sizes=(1,)))

    class Meta:
        def __init__(self, shape):
            self.shape = shape

    assert count_parameters([Meta((2, 3)), Meta((4,)), Meta((2, 2, 2))]) == 18


def test_prefill_and_decode_one_match_generation():
    from pathlib import Path

    import torch

    from research_b200.config import run_spec_from_mapping
    from research_b200.infer import decode_one, generate_tokens, init_kv_cache, prefill
    from research_b200.models import apply_model, build_model
    from tests.helpers import tiny_raw_config

    spec = run_spec_from_mapping(tiny_raw_config(Path("m.json")))
    model = build_model(spec.model, seed=0).model.eval()
    prompt = torch.tensor([[5, 9, 2, 7], [1, 1, 3, 8]])
    want = generate_tokens(model, prompt, max_new_tokens=4, top_k=1, page_size=4).generated_ids
    cache = init_kv_cache(model, 2, 8, page_size=4)
    logits = prefill(model, prompt, cache)
    got = []
    for step in range(4):
        token = logits.argmax(-1)
        got.append(token.tolist())
        if step < 3:
            logits = decode_one(model, token, 4 + step, cache)
    assert [list(col) for col in zip(*got)] == want and cache.lengths.tolist() == [7, 7]
    with torch.no_grad():
        full = apply_model(model, prompt.to(torch.int32)).logits
    assert torch.allclose(prefill(model, prompt, init_kv_cache(model, 2, 8, page_size=4)), full[:, -1], atol=2e-4)


def test_importing_the_packages_does_not_import_their_heavy_submodules():
    code = ("import sys; import research_b200.optim, research_b200.models, research_b200.infer, research_b200.steps, "
            "research_b200.services, research_b200.kernels, research_b200.parallel, research_b200.mesh; "
            "heavy = [m for m in ('research_b200.optim.optimizer', 'research_b200.models.transformer', "
            "'research_b200.infer.generation', 'research_b200.steps.train', 'research_b200.parallel.sharding', 'torch') "
            "if m in sys.modules]; print(heavy)")
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=120)
    assert out.returncode == 0 and out.stdout.strip() == "[]", out.stdout + out.stderr


def test_packaging_metadata_names_the_package_and_the_command():
    import tomllib
    from pathlib import Path

    import research_b200

    meta = tomllib.loads((Path(__file__).resolve().parent.parent / "pyproject.toml").read_text())
    assert meta["project"]["name"] == "research_b200" and meta["project"]["scripts"] == {"jaxtitan": "research_b200.cli:main"}
    assert meta["tool"]["setuptools"]["dynamic"]["version"] == {"attr": "research_b200.__version__"}
    assert isinstance(research_b200.__version__, str) and research_b200.__version__
    data = meta["tool"]["setuptools"]["package-data"]["research_b200"]
    assert "ops/csrc/*.cu" in data and "native/*.cpp" in data           # the sources the in-tree build compiles
    from research_b200.cli import main

    assert callable(main)


def test_the_package_imports_nothing_from_outside_itself():
    """Product code never reaches into tests, benchmarks or scratch folders (the reference keeps the same boundary
    between its package and its legacy tree: tests/jaxtitan/test_import_boundary.py)."""

    import re
    from pathlib import Path

    root = Path(__file__).resolve().parent.parent / "research_b200"
    pattern = re.compile(r"^\s*(?:from|import)\s+(tests|bench|_work|__graft_entry__|baseline)\b", re.M)
    offenders = [p.relative_to(root).as_posix() for p in root.rglob("*.py") if pattern.search(p.read_text())]
    assert offenders == []
