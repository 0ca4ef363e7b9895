"""The ``jaxtitan`` command line, driven in process: grammar, text and JSON forms, exit codes."""

import json

import pytest

from research_b200.cli import build_parser, main
from tests.helpers import tiny_dataset, tiny_raw_config, write_toml


@pytest.fixture(scope="module")
def dataset(tmp_path_factory):
    return tiny_dataset(tmp_path_factory.mktemp("cli"))


def _config(tmp_path, dataset, **kw):
    kw.setdefault("output_dir", (tmp_path / "runs").as_posix())
    run_id = kw.get("run_id", "tiny")
    return write_toml(tiny_raw_config(dataset, **kw), tmp_path / f"{run_id}.toml")


def _run(capsys, *argv):
    code = main(list(argv))
    out = capsys.readouterr()
    return code, out.out, out.err


def test_no_command_prints_help_and_version_exits(capsys):
    code, out, _ = _run(capsys)
    assert code == 0 and "usage: jaxtitan" in out and "{config,data,kernels,profile,run,eval,sample}" in out
    with pytest.raises(SystemExit) as exc:
        main(["--version"])
    assert exc.value.code == 0 and "jaxtitan" in capsys.readouterr().out


@pytest.mark.parametrize("argv", [
    ["config"], ["config", "check"], ["data", "check", "m.json"], ["run"], ["run", "train"],
    ["eval", "checkpoint", "runs/x"], ["sample", "checkpoint", "runs/x", "--checkpoint", "latest"],
    ["sample", "checkpoint", "runs/x", "--checkpoint", "latest", "--prompt-ids", "1", "--max-new-tokens", "x"],
    ["kernels", "bench", "softmax", "c.toml"], ["profile", "bench", "attention"], ["nope"],
])
def test_grammar_errors_exit_with_the_parser_code(argv, capsys):
    with pytest.raises(SystemExit) as exc:
        main(argv)
    assert exc.value.code == 2 and "usage:" in capsys.readouterr().err


def test_parser_defaults():
    p = build_parser()
    a = p.parse_args(["sample", "checkpoint", "r", "--checkpoint", "best", "--prompt-ids", "1,2", "--max-new-tokens", "8"])
    assert (a.temperature, a.top_k, a.json, a.max_new_tokens) == (1.0, None, False, 8)
    b = p.parse_args(["profile", "bench", "muon"])
    assert (b.warmup, b.iters, b.artifact_dir, b.trace) == (3, 10, None, False)
    c = p.parse_args(["profile", "analyze", "root"])
    assert c.warmup_steps == 2
    d = p.parse_args(["kernels", "bench", "gemm", "c.toml"])
    assert (d.rows, d.warmup, d.iters) == ("1,4,17,64,256", 5, 20)
    e = p.parse_args(["run", "train", "c.toml"])
    assert e.resume is False and e.overwrite is False
    f = p.parse_args(["data", "synth", "out"])
    assert (f.seed, f.documents, f.vocab_size, f.eos_id, f.val_fraction) == (0, 2000, 50257, 50256, 0.05)


def test_config_check_text_json_and_errors(tmp_path, dataset, capsys):
    cfg = _config(tmp_path, dataset)
    code, out, _ = _run(capsys, "config", "check", str(cfg))
    assert code == 0 and out.strip() == f"ok: {cfg} (run tiny)"
    code, out, _ = _run(capsys, "config", "check", str(cfg), "--json")
    resolved = json.loads(out)
    assert code == 0 and resolved["run_id"] == "tiny" and resolved["model"]["hidden_size"] == 64
    code, out, err = _run(capsys, "config", "check", str(tmp_path / "missing.toml"))
    assert code == 2 and out == "" and err.startswith("error: failed to read config")
    bad = tmp_path / "bad.toml"
    bad.write_text("[run\nid = 3")
    code, _, err = _run(capsys, "config", "check", str(bad))
    assert code == 2 and err.startswith("error: failed to parse config")
    raw = tiny_raw_config(dataset)
    raw["model"]["num_heads"] = 5
    code, _, err = _run(capsys, "config", "check", str(write_toml(raw, tmp_path / "heads.toml")))
    assert code == 2 and err.startswith("error: ") and "num_heads" in err


def test_data_commands(tmp_path, dataset, capsys):
    code, out, _ = _run(capsys, "data", "check", str(dataset), "--tokenizer", "synthetic-uniform", "--verify-checksums")
    assert code == 0 and out.startswith(f"ok: {dataset} (") and "1 shards" in out
    code, out, _ = _run(capsys, "data", "check", str(dataset), "--tokenizer", "synthetic-uniform", "--json")
    assert code == 0 and json.loads(out)["tokenizer_id"] == "synthetic-uniform"
    code, _, err = _run(capsys, "data", "check", str(dataset), "--tokenizer", "gpt2")
    assert code == 2 and "does not match config tokenizer" in err
    code, out, _ = _run(capsys, "data", "inspect", str(dataset), "--seq-len", "32")
    assert code == 0 and "records: seq_len=32" in out and "training config:" in out and "[data]" in out
    code, out, _ = _run(capsys, "data", "inspect", str(dataset), "--json")
    assert code == 0 and json.loads(out)["tokens"]["total"] > 0
    code, _, err = _run(capsys, "data", "inspect", str(dataset), "--seq-len", "0")
    assert code == 2 and "--seq-len must be positive" in err
    out_dir = tmp_path / "synth"
    code, out, _ = _run(capsys, "data", "synth", str(out_dir), "--documents", "20", "--mean-length", "40",
                        "--min-length", "8", "--max-length", "80", "--vocab-size", "64", "--eos-id", "63", "--json")
    assert code == 0 and json.loads(out)["manifest_path"] == (out_dir / "manifest.json").as_posix()
    code, _, err = _run(capsys, "data", "synth", str(out_dir), "--documents", "20", "--vocab-size", "64", "--eos-id", "63")
    assert code == 2 and "already exists" in err
    (tmp_path / "corpus.txt").write_text("\n".join(f"line {i} of the corpus" for i in range(50)))
    prep = tmp_path / "prep.toml"
    prep.write_text('[source]\ntype = "text"\npaths = ["corpus.txt"]\n[tokenizer]\nname = "byte-level"\n'
                    f'[output]\npath = "{(tmp_path / "prepared").as_posix()}"\nmax_tokens = 500\nval_fraction = 0.1\n'
                    '[tokenization]\nworkers = 1\n')
    code, out, _ = _run(capsys, "data", "prepare", str(prep))
    assert code == 0 and out.startswith("prepared 500 tokens at ")
    code, _, err = _run(capsys, "data", "prepare", str(prep))
    assert code == 2 and "rerun with --overwrite" in err
    code, out, _ = _run(capsys, "data", "prepare", str(prep), "--overwrite", "--json")
    assert code == 0 and json.loads(out)["num_tokens"] == 500


def test_kernels_list_and_check(tmp_path, dataset, capsys):
    code, out, _ = _run(capsys, "kernels", "list")
    assert code == 0 and "gemm" in out and "built=" in out
    code, out, _ = _run(capsys, "kernels", "list", "--json")
    kernels = json.loads(out)["kernels"]
    assert {"op", "symbol", "engine", "built"} <= set(kernels[0]) and any("attention" in k["op"] for k in kernels)
    cfg = _config(tmp_path, dataset)
    code, out, _ = _run(capsys, "kernels", "check", str(cfg))
    assert code == 0 and out.startswith("kernel plan: active=False") and "fallback=pytorch" in out
    code, out, _ = _run(capsys, "kernels", "check", str(cfg), "--json")
    plan = json.loads(out)
    assert plan["arch"] == "sm_100a" and plan["active_count"] == 0 and len(plan["ops"]) == len(kernels)
    code, _, err = _run(capsys, "kernels", "compile", str(cfg), "--arch", "SM90")
    assert code == 2 and "targets SM100" in err


def test_run_lifecycle_in_process(tmp_path, dataset, capsys, monkeypatch):
    monkeypatch.setattr("sys.stdin.isatty", lambda: False)
    cfg = _config(tmp_path, dataset, run_id="life", steps=2, checkpoint_every=2, evals=True)
    run_dir = tmp_path / "runs" / "life"
    code, out, _ = _run(capsys, "run", "preflight", str(cfg))
    assert code == 0 and out.startswith("preflight: ok") and "eval: name=validation" in out and not run_dir.exists()
    code, out, _ = _run(capsys, "run", "init", str(cfg))
    assert code == 0 and out.strip() == f"initialized run life at {run_dir}" and (run_dir / "manifest.json").is_file()
    code, _, err = _run(capsys, "run", "init", str(cfg))
    assert code == 2 and "already exists" in err
    code, _, err = _run(capsys, "run", "preflight", str(cfg))
    assert code == 2 and "run directory already exists" in err
    code, _, err = _run(capsys, "run", "train", str(cfg))
    assert code == 2 and "rerun with --overwrite" in err
    code, out, _ = _run(capsys, "run", "train", str(cfg), "--overwrite")
    assert code == 0
    for piece in ("JAX TITAN TRAINING", "run: life", "resume: false", "  model   | decoder/tiny", "  mesh    | cpu | devices 1",
                  "step: 1      | loss:", "eval step 2: loss=", "checkpoint step 2: ", "/checkpoints/000002 reason=cadence", "completed: step=2"):
        assert piece in out, piece
    code, out, _ = _run(capsys, "run", "inspect", str(run_dir))
    assert code == 0 and "status: completed" in out and "final: step=2" in out
    code, out, _ = _run(capsys, "eval", "checkpoint", str(run_dir), "--checkpoint", "best")
    assert code == 0 and out.startswith("evaluated checkpoint step=2 path=checkpoints/")
    code, out, _ = _run(capsys, "sample", "checkpoint", str(run_dir), "--checkpoint", "latest", "--prompt-ids", "1,2",
                        "--max-new-tokens", "3", "--top-k", "1")
    assert code == 0 and out.startswith("sampled checkpoint step=2") and "generated=3 top_k=1" in out
    code, _, err = _run(capsys, "eval", "checkpoint", str(run_dir), "--checkpoint", "7")
    assert code == 2 and "no checkpoint matches '7'" in err
    code, _, err = _run(capsys, "eval", "checkpoint", str(run_dir), "--checkpoint", "newest")
    assert code == 2 and "must be 'best', 'latest', or a step" in err
    code, _, err = _run(capsys, "run", "inspect", str(tmp_path / "runs" / "ghost"))
    assert code == 2 and "run directory does not exist" in err
    # resume to a later target
    text = cfg.read_text().replace(f"target_tokens = {32 * 4 * 2}", f"target_tokens = {32 * 4 * 3}")
    cfg.write_text(text)
    code, out, _ = _run(capsys, "run", "train", str(cfg), "--resume")
    assert code == 0 and "resume: true" in out and "resumed: checkpoint_step=2 step=2" in out and "completed: step=3" in out
    code, out, _ = _run(capsys, "profile", "analyze", str(tmp_path / "runs"), "--warmup-steps", "0")
    assert code == 0 and out.startswith("profile analysis: runs=1 source=runs") and "life" in out
    code, out, _ = _run(capsys, "profile", "analyze", str(tmp_path / "runs"), "--warmup-steps", "0", "--json")
    assert code == 0 and json.loads(out)["runs"][0]["run_id"] == "life"
    code, _, err = _run(capsys, "profile", "analyze", str(tmp_path / "nothing"))
    assert code == 2 and "not a directory" in err
