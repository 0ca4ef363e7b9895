"""Kernel build cache and kernel plan, with the compiler replaced by a recorder and the tree by a temporary copy."""

import json
from pathlib import Path

import pytest
import torch

from research_b200.config import run_spec_from_mapping
from research_b200.errors import ContractError
from research_b200.kernels import build, registry
from tests.helpers import tiny_raw_config


@pytest.fixture
def fake_tree(tmp_path, monkeypatch):
    """Two kernel sources, a header and a host source in a scratch tree; every build command is recorded and its
    output file is created empty."""

    csrc, native, lib = tmp_path / "csrc", tmp_path / "native", tmp_path / "_lib"
    for d in (csrc, native):
        d.mkdir()
    (csrc / "alpha.cu").write_text("// alpha")
    (csrc / "beta.cu").write_text("// beta")
    (csrc / "common.cuh").write_text("// header")
    (native / "host.cpp").write_text("// host")
    monkeypatch.setattr(build, "CSRC_DIR", csrc)
    monkeypatch.setattr(build, "NATIVE_DIR", native)
    monkeypatch.setattr(build, "LIB_DIR", lib)
    monkeypatch.setattr(build, "KERNEL_LIB", lib / "libb200ops.so")
    monkeypatch.setattr(build, "HOST_LIB", lib / "libb200host.so")
    monkeypatch.setattr(build, "MANIFEST", lib / "build_manifest.json")
    monkeypatch.setattr(build, "nvcc_path", lambda: "/fake/nvcc")
    commands = []

    def record(cmd):
        commands.append(list(cmd))
        Path(cmd[cmd.index("-o") + 1]).write_text("")

    monkeypatch.setattr(build, "_run", record)
    return types_namespace(csrc=csrc, native=native, lib=lib, commands=commands)


def types_namespace(**kw):
    import types

    return types.SimpleNamespace(**kw)


def test_build_compiles_every_source_for_sm_100a_and_links_once(fake_tree):
    result = build.build_all()
    assert result.rebuilt and result.sources == ("alpha.cu", "beta.cu") and len(result.digest) == 64
    compiles = [c for c in fake_tree.commands if "-c" in c]
    links = [c for c in fake_tree.commands if "-shared" in c]
    assert sorted(Path(c[c.index("-c") + 1]).name for c in compiles) == ["alpha.cu", "beta.cu"]
    for c in compiles:
        assert c[0] == "/fake/nvcc" and c[1:3] == ["-gencode", "arch=compute_100a,code=sm_100a"]
        assert "-lineinfo" in c and "-O3" in c and c[c.index("-I") + 1] == str(fake_tree.csrc)
    assert len(links) == 2                                                  # the kernel library and the host library
    kernel_link = next(c for c in links if c[0] == "/fake/nvcc")
    assert kernel_link[kernel_link.index("-o") + 1].endswith("libb200ops.so")
    assert sorted(Path(o).name for o in kernel_link if o.endswith(".o")) == ["alpha.o", "beta.o"]
    host_link = next(c for c in links if c[0] != "/fake/nvcc")
    assert "-pthread" in host_link and host_link[-1].endswith("host.cpp")
    manifest = json.loads(build.MANIFEST.read_text())
    assert manifest == {"digest": result.digest, "arch": "sm_100a", "nvcc_flags": list(build.ARCH_FLAGS + build.NVCC_FLAGS),
                        "sources": ["alpha.cu", "beta.cu"], "host_sources": ["host.cpp"]}


def test_unchanged_tree_is_not_rebuilt_and_any_input_change_is(fake_tree):
    first = build.build_all()
    fake_tree.commands.clear()
    again = build.build_all()
    assert not again.rebuilt and again.digest == first.digest and fake_tree.commands == []
    for path, text in ((fake_tree.csrc / "alpha.cu", "// alpha v2"), (fake_tree.csrc / "common.cuh", "// header v2"),
                       (fake_tree.native / "host.cpp", "// host v2")):
        path.write_text(text)
        fake_tree.commands.clear()
        changed = build.build_all()
        assert changed.rebuilt and changed.digest != first.digest and fake_tree.commands, path.name
        first = changed
    (fake_tree.csrc / "gamma.cu").write_text("// gamma")
    assert build.build_all().sources == ("alpha.cu", "beta.cu", "gamma.cu")
    fake_tree.commands.clear()
    forced = build.build_all(force=True)
    assert forced.rebuilt and len([c for c in fake_tree.commands if "-c" in c]) == 3


def test_missing_library_or_broken_manifest_triggers_a_build(fake_tree):
    build.build_all()
    build.KERNEL_LIB.unlink()
    assert build.build_all().rebuilt
    build.MANIFEST.write_text("{not json")
    assert build.build_all().rebuilt
    build.HOST_LIB.unlink()
    assert build.build_all().rebuilt


def test_ptxas_report_flag_and_failing_compiler(fake_tree, monkeypatch):
    build.build_all(force=True, ptxas_info=True)
    assert all(c[1:3] == ["-Xptxas", "-v"] for c in fake_tree.commands if "-c" in c)

    def fail(cmd):
        raise ContractError(f"build command failed: {' '.join(cmd)}")

    monkeypatch.setattr(build, "_run", fail)
    with pytest.raises(ContractError, match="build command failed: /fake/nvcc"):
        build.build_all(force=True)


def test_without_a_compiler_an_existing_library_is_used_and_a_missing_one_is_an_error(fake_tree, monkeypatch, capsys):
    build.build_all()
    (fake_tree.csrc / "alpha.cu").write_text("// changed")                 # stale library, no compiler to refresh it

    def no_nvcc():
        raise ContractError("nvcc not found; the sm_100a kernel library cannot be built")

    monkeypatch.setattr(build, "nvcc_path", no_nvcc)
    assert build.ensure_current() is None
    assert "using the existing kernel library" in capsys.readouterr().err
    build.KERNEL_LIB.unlink()
    with pytest.raises(ContractError, match="nvcc not found"):
        build.ensure_current()


def test_real_run_helper_reports_the_command_and_its_output():
    with pytest.raises(ContractError, match="build command failed: false"):
        build._run(["false"])
    build._run(["true"])


def test_kernel_plan_selects_native_ops_only_for_bf16_on_cuda():
    spec = run_spec_from_mapping(tiny_raw_config(Path("m.json")))
    cpu = registry.kernel_plan(spec, device=torch.device("cpu"))
    assert cpu["active"] is False and cpu["active_count"] == 0 and cpu["arch"] == "sm_100a"
    assert all(op["fallback"] == "pytorch" and op["fallback_reason"] == "no CUDA device" for op in cpu["ops"])
    assert cpu["fallback_count"] + cpu["unavailable_count"] == len(cpu["ops"])
    fp32_on_gpu = registry.kernel_plan(spec, device=torch.device("cuda"))
    assert fp32_on_gpu["active"] is False
    assert {op["fallback_reason"] for op in fp32_on_gpu["ops"]} == {"fp32 compute uses the PyTorch path"}
    raw = tiny_raw_config(Path("m.json"))
    raw["model"]["compute_dtype"] = "bfloat16"
    raw["training"]["precision"] = "bf16"
    bf16 = run_spec_from_mapping(raw)
    gpu = registry.kernel_plan(bf16, device=torch.device("cuda"))
    built = [op for op in gpu["ops"] if op["built"]]
    assert gpu["active"] is True and gpu["active_count"] == len(built) and all(op["selected"] for op in built)
    assert all(op["fallback_reason"] == "symbol not built" for op in gpu["ops"] if not op["built"])
    names = {op["op"] for op in gpu["ops"]}
    assert {"gemm", "rmsnorm"} <= names and len(names) == len(gpu["ops"])


def test_strict_kernels_refuse_a_fallback_except_for_optional_ops():
    raw = tiny_raw_config(Path("m.json"))
    raw["kernels"] = {"strict": True}
    strict = run_spec_from_mapping(raw)
    plan = registry.kernel_plan(strict, device=torch.device("cpu"))
    with pytest.raises(ContractError, match="kernels.strict=true but these ops would not run natively"):
        registry.require_kernel_plan_supported(plan, strict)
    relaxed = run_spec_from_mapping(tiny_raw_config(Path("m.json")))
    registry.require_kernel_plan_supported(plan, relaxed)
    only_optional = dict(plan, ops=[dict(op, selected=op["op"] not in registry.OPTIONAL_OPS) for op in plan["ops"]])
    registry.require_kernel_plan_supported(only_optional, strict)


def test_registry_rows_name_a_source_and_an_exported_symbol():
    rows = registry.kernel_registry()
    sources = {p.name for p in build.kernel_sources()}
    assert rows and all(r["source"] in sources for r in rows)
    assert all(r["symbol"].startswith(("b200_", "b200c_")) for r in rows)
    assert len({r["op"] for r in rows}) == len(rows)


def test_roofline_denominators_come_from_the_measured_file_or_the_stated_fallback(tmp_path, monkeypatch):
    from research_b200.kernels import microbench

    (tmp_path / "MEASURED_PEAKS.json").write_text(json.dumps({"hbm_gbs": 6500.0, "bf16_tflops": 1600.0, "chip": "B200"}))
    monkeypatch.setattr(microbench, "ROOT", tmp_path)
    assert microbench.peaks() == {"hbm_gbs": 6500.0, "bf16_tflops": 1600.0, "source": "measured"}
    (tmp_path / "MEASURED_PEAKS.json").unlink()
    assert microbench.peaks() == {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}
