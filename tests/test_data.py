"""Prepared-token manifests and the deterministic pipelines."""

import json
import struct
from pathlib import Path

import numpy as np
import pytest

from research_b200.data import (build_prepared_token_pipeline, generate_synthetic_dataset, read_token_range,
                                validate_dataset_manifest)
from research_b200.errors import ContractError
from tests.helpers import tiny_dataset


def naive_document_buffer(tokens, offsets, split, seq_len, batch_size, seed, buffer_size, refill_size, batches):
    """Straight restatement of the reference packer (src/jaxtitan/data/pipeline.py:528-704) on Python lists."""

    start, end = split
    spans = {}
    for d in range(len(offsets) - 1):
        a, b = max(int(offsets[d]), start), min(int(offsets[d + 1]), end)
        if b > a:
            spans[d] = (a, b)
    ids = list(spans)
    rng = np.random.default_rng(seed)
    order = [int(v) for v in rng.permutation(np.asarray(ids, dtype=np.int64)).tolist()]
    cursor, queue, active = 0, [], []

    def fill():
        nonlocal cursor, queue
        while len(active) < min(buffer_size, len(ids)):
            if not queue:
                if cursor >= len(order):
                    return
                stop = min(cursor + refill_size, len(order))
                queue = order[cursor:stop]
                cursor = stop
            d = queue.pop(0)
            active.append({"doc_id": d, "cursor": spans[d][0], "end": spans[d][1]})

    fill()
    out = []
    for _ in range(batches):
        rows = []
        for _ in range(batch_size):
            vals, docs = [], []
            while len(vals) < seq_len + 1:
                fill()
                i = int(rng.integers(0, len(active)))
                a = active[i]
                take = min(seq_len + 1 - len(vals), a["end"] - a["cursor"])
                vals.extend(int(v) for v in tokens[a["cursor"]:a["cursor"] + take])
                docs.extend([a["doc_id"]] * take)
                a["cursor"] += take
                if a["cursor"] >= a["end"]:
                    del active[i]
            rows.append((vals, docs))
        out.append(rows)
    return out


def test_document_buffer_matches_reference_algorithm(tmp_path):
    manifest_path = tiny_dataset(tmp_path)
    manifest = validate_dataset_manifest(manifest_path, verify_checksums=True)
    tokens = read_token_range(manifest, 0, manifest.num_tokens)
    offsets = np.fromfile(manifest.data_dir / "document_offsets.u64", dtype="<u8")
    pipe = build_prepared_token_pipeline(manifest_path, tokenizer_id=None, split="train", seq_len=24, batch_size=3,
                                         order="document_buffer", shuffle_seed=11, document_buffer_size=5,
                                         document_refill_size=3)
    want = naive_document_buffer(tokens, offsets, (manifest.train.start, manifest.train.end), 24, 3, 11, 5, 3, 6)
    state = pipe.initial_state()
    for rows in want:
        pb = pipe.next_batch(state)
        state = pb.state
        for r, (vals, docs) in enumerate(rows):
            assert pb.batch.input_ids[r].tolist() == vals[:-1]
            assert pb.batch.target_ids[r].tolist() == vals[1:]
            assert pb.batch.loss_mask[r].tolist() == [docs[i] == docs[i + 1] for i in range(24)]
            assert pb.batch.token_doc_ids[r].tolist() == docs[:-1]


@pytest.mark.parametrize("order", ["sequential", "shuffle", "document_buffer"])
def test_state_roundtrip_gives_the_same_next_batch(tmp_path, order):
    manifest_path = tiny_dataset(tmp_path)
    kw = dict(tokenizer_id="synthetic-uniform", split="train", seq_len=16, batch_size=4, order=order)
    if order != "sequential":
        kw["shuffle_seed"] = 3
    if order == "document_buffer":
        kw.update(document_buffer_size=8, document_refill_size=4)
    pipe = build_prepared_token_pipeline(manifest_path, **kw)
    s = pipe.initial_state()
    s = pipe.next_batch(s).state
    again = pipe.state_from_json(json.loads(json.dumps(pipe.state_to_json(s))))
    a, b = pipe.next_batch(s), pipe.next_batch(again)
    assert np.array_equal(a.batch.input_ids, b.batch.input_ids)
    assert a.state == b.state
    other = build_prepared_token_pipeline(manifest_path, **{**kw, "seq_len": 8})
    with pytest.raises(ContractError, match="data pipeline state seq_len mismatch"):
        other.state_from_json(pipe.state_to_json(s))


def test_sequential_windows_and_exhaustion(tmp_path):
    manifest_path = tiny_dataset(tmp_path, documents=40)
    manifest = validate_dataset_manifest(manifest_path)
    pipe = build_prepared_token_pipeline(manifest_path, tokenizer_id=None, split="val", seq_len=16, batch_size=2)
    s = pipe.initial_state()
    pb = pipe.next_batch(s)
    start = manifest.val.start
    want = read_token_range(manifest, start, start + 17)
    assert pb.batch.input_ids[0].tolist() == want[:-1].tolist()
    assert pb.provenance.row_start_offsets == (start, start + 16)
    with pytest.raises(StopIteration):
        for _ in range(10_000):
            s = pipe.next_batch(s).state


def _corrupt(path: Path, fn):
    raw = json.loads(path.read_text())
    fn(raw)
    path.write_text(json.dumps(raw))


@pytest.mark.parametrize("fn,message", [
    (lambda r: r.update(kind="tokens"), "kind must be training_tokens"),
    (lambda r: r.update(dtype="uint16"), "dtype must be uint32"),
    (lambda r: r["shards"][0].update(start=1), "shards must be contiguous"),
    (lambda r: r["shards"][0].update(path="/abs.bin"), "path must be relative"),
    (lambda r: r["shards"][0].update(path="../x.bin"), "must stay inside the manifest directory"),
    (lambda r: r["splits"]["val"].update(start=0, tokens=r["splits"]["val"]["end"]), "train/val splits overlap"),
    (lambda r: r.update(num_tokens=5), "does not match shard total"),
    (lambda r: r["documents"].update(count=3), "does not match documents.count"),
    (lambda r: r["files"].pop("document_offsets"), "documents metadata requires files.document_offsets"),
])
def test_manifest_corruptions_are_rejected(tmp_path, fn, message):
    manifest_path = tiny_dataset(tmp_path, documents=30)
    _corrupt(manifest_path, fn)
    with pytest.raises(ContractError, match=message):
        validate_dataset_manifest(manifest_path)


def test_checksum_and_tokenizer_mismatch(tmp_path):
    manifest_path = tiny_dataset(tmp_path, documents=30)
    with pytest.raises(ContractError, match="does not match config tokenizer"):
        validate_dataset_manifest(manifest_path, tokenizer_id="gpt2")
    shard = manifest_path.parent / "tokens-00000.bin"
    data = bytearray(shard.read_bytes())
    data[0:4] = struct.pack("<I", 7)
    shard.write_bytes(bytes(data))
    validate_dataset_manifest(manifest_path)
    with pytest.raises(ContractError, match="checksum mismatch"):
        validate_dataset_manifest(manifest_path, verify_checksums=True)


def test_prepare_text_source_with_byte_tokenizer(tmp_path):
    from research_b200.data.prepare import prepare_dataset

    (tmp_path / "corpus.txt").write_text("\n".join(f"document number {i} says hello" for i in range(200)))
    cfg = tmp_path / "prep.toml"
    cfg.write_text('[source]\ntype = "text"\npaths = ["corpus.txt"]\n[tokenizer]\nname = "byte-level"\n'
                   '[output]\npath = "%s"\nmax_tokens = 4000\nval_fraction = 0.1\nshard_tokens = 1500\n'
                   '[tokenization]\nworkers = 1\n' % (tmp_path / "out").as_posix())
    summary = prepare_dataset(cfg)
    assert summary["num_tokens"] == 4000 and summary["shard_count"] == 3 and summary["document_aware"]
    manifest = validate_dataset_manifest(tmp_path / "out" / "manifest.json", tokenizer_id="byte-level",
                                         verify_checksums=True)
    assert manifest.train.end == manifest.val.start
    with pytest.raises(ContractError, match="already exists"):
        prepare_dataset(cfg)


def test_native_window_gather_matches_numpy(tmp_path):
    from research_b200.native import hostlib

    if hostlib.load() is None:
        pytest.skip("host library not built")
    manifest_path = generate_synthetic_dataset(tmp_path / "multi", seed=1, num_documents=50, mean_length=100,
                                               min_length=8, max_length=300, vocab_size=300, eos_id=299,
                                               shard_tokens=1000)
    manifest = validate_dataset_manifest(manifest_path)
    shards = [np.fromfile(manifest.data_dir / s.path, dtype="<u4") for s in manifest.shards]
    bounds = [s.start for s in manifest.shards] + [manifest.num_tokens]
    starts = np.asarray([0, 990, 1500, 2995], dtype=np.int64)
    inp = np.zeros((4, 32), dtype=np.int32)
    tgt = np.zeros((4, 32), dtype=np.int32)
    assert hostlib.gather_windows(shards, bounds, starts, 33, inp, tgt)
    for r, s in enumerate(starts):
        want = read_token_range(manifest, int(s), int(s) + 33).astype(np.int32)
        assert np.array_equal(inp[r], want[:-1]) and np.array_equal(tgt[r], want[1:])


@pytest.mark.parametrize("order", ["sequential", "shuffle", "document_buffer"])
def test_local_rows_keep_the_order_and_read_only_their_tokens(tmp_path, order):
    """A rank of a data-parallel job materialises only its rows: those rows, the pipeline state after every batch
    and the batch's unmasked-token count are the same as when every row is read."""

    manifest = tiny_dataset(tmp_path, documents=400)
    kw = dict(tokenizer_id=None, split="train", seq_len=32, batch_size=8, order=order,
              shuffle_seed=None if order == "sequential" else 3,
              document_buffer_size=8 if order == "document_buffer" else None,
              document_refill_size=8 if order == "document_buffer" else None)
    full = build_prepared_token_pipeline(manifest, **kw)
    part = build_prepared_token_pipeline(manifest, **kw)
    part.set_local_rows(range(2, 4))
    reads = []
    original = part.reader.read
    part.reader.read = lambda a, b: (reads.append(b - a), original(a, b))[1]
    s_full, s_part = full.initial_state(), part.initial_state()
    for _ in range(5):
        a, b = full.next_batch(s_full), part.next_batch(s_part)
        s_full, s_part = a.state, b.state
        assert full.state_to_json(s_full) == part.state_to_json(s_part)
        assert a.provenance == b.provenance
        for name in ("input_ids", "target_ids", "loss_mask"):
            assert np.array_equal(getattr(a.batch, name)[2:4], getattr(b.batch, name)[2:4]), name
        assert not b.batch.input_ids[:2].any() and not b.batch.input_ids[4:].any()
        assert b.batch.mask_count == float(np.asarray(a.batch.loss_mask).sum())
        assert a.batch.mask_count is None
        if a.batch.token_doc_ids is not None:
            assert np.array_equal(a.batch.token_doc_ids[2:4], b.batch.token_doc_ids[2:4])
    assert sum(reads) == 5 * 2 * 33                       # two rows of seq_len + 1 tokens per batch, nothing else
    with pytest.raises(ContractError, match="not inside a batch"):
        part.set_local_rows(range(6, 10))


def test_prepare_records_its_source_and_settings_and_expands_patterns(tmp_path):
    import json

    from research_b200.data.inspect import data_config_snippet, format_inspection, inspect_dataset, record_count
    from research_b200.data.prepare import prepare_dataset, resolve_source_files

    (tmp_path / "part-b.jsonl").write_text("\n".join(json.dumps({"body": f"second file row {i}"}) for i in range(60)))
    (tmp_path / "part-a.jsonl").write_text("\n".join(json.dumps({"body": f"first file row {i}", "n": i})
                                                     for i in range(60)) + "\n" + json.dumps({"n": 1}) + "\n")
    cfg = tmp_path / "prep.toml"
    cfg.write_text('[source]\ntype = "jsonl"\npaths = ["part-*.jsonl"]\ntext_column = "body"\n'
                   '[tokenizer]\nname = "byte-level"\n'
                   '[output]\npath = "%s"\nmax_tokens = 100000\nval_fraction = 0.1\nshard_tokens = 1000\n'
                   '[tokenization]\nworkers = 1\nbatch_docs = 16\n' % (tmp_path / "out").as_posix())
    files = resolve_source_files(["part-*.jsonl"], tmp_path)
    assert [f.name for f in files] == ["part-a.jsonl", "part-b.jsonl"]          # sorted expansion
    with pytest.raises(ContractError, match="did not match any files"):
        resolve_source_files(["nothing-*.jsonl"], tmp_path)
    with pytest.raises(ContractError, match="does not exist"):
        resolve_source_files(["missing.jsonl"], tmp_path)
    with pytest.raises(ContractError, match="must be a file, got directory"):
        resolve_source_files([str(tmp_path)], tmp_path)
    prepare_dataset(cfg)
    raw = json.loads((tmp_path / "out" / "manifest.json").read_text())
    assert raw["source"] == {"type": "jsonl", "paths": ["part-*.jsonl"], "text_column": "body",
                             "resolved_file_count": 2,
                             "resolved_total_bytes": sum(f.stat().st_size for f in files)}
    assert raw["num_docs"] == raw["documents"]["count"] == 120 and raw["source_docs_seen"] == 120
    assert raw["tokenizer"]["eot_token"] == 256 and raw["tokenizer"]["append_eot"] is True
    assert raw["val_fraction"] == 0.1 and raw["max_tokens"] == 100000 and raw["shard_tokens"] == 1000
    assert raw["tokenization"] == {"workers": 1, "batch_docs": 16, "queue_batches": 8}
    assert raw["train_tokens"] + raw["val_tokens"] == raw["num_tokens"] and raw["elapsed_sec"] >= 0
    assert raw["created_at"].endswith("Z") and raw["tokens_per_sec"] > 0
    first = np.fromfile(tmp_path / "out" / "tokens-00000.bin", dtype="<u4")
    assert bytes(first[:16].astype(np.uint8)).decode() == "first file row 0"      # part-a comes first
    # inspection of that dataset
    report = inspect_dataset(tmp_path / "out" / "manifest.json", tokenizer_id="byte-level", verify_checksums=True,
                             seq_len=64)
    assert report["tokens"] == {"total": raw["num_tokens"], "train": raw["train_tokens"], "val": raw["val_tokens"]}
    assert report["source"]["resolved_file_count"] == 2 and report["tokenizer"]["name"] == "byte-level"
    assert report["documents"]["count"] == 120 and report["documents"]["offsets_path"] == "document_offsets.u64"
    assert report["documents"]["lengths"]["min"] == len("first file row 0") + 1
    assert report["shards"]["count"] == len(raw["shards"]) and report["shards"]["checksums_present"]
    assert report["shards"]["bytes"] == 4 * raw["num_tokens"] and len(report["shards"]["files"]) == report["shards"]["count"]
    assert report["records"] == {"seq_len": 64, "train": (raw["train_tokens"] - 1) // 64,
                                 "val": (raw["val_tokens"] - 1) // 64,
                                 "train_document_buffer_rows": raw["train_tokens"] // 65}
    assert record_count(1, 8) == 0 and record_count(9, 8) == 1 and record_count(17, 8) == 2
    text = format_inspection(report)
    for head in ("source: type=jsonl files=2", "tokenizer: byte-level append_eot=True eot=256", "tokens: total=",
                 "documents: count=120", "shards: count=", "document lengths: min=", "records: seq_len=64",
                 "training config:", 'order = "document_buffer"'):
        assert head in text, head
    assert inspect_dataset(tmp_path / "out" / "manifest.json")["records"] is None
    with pytest.raises(ContractError, match="--seq-len must be positive"):
        inspect_dataset(tmp_path / "out" / "manifest.json", seq_len=0)
    with pytest.raises(ContractError, match="does not match config tokenizer"):
        inspect_dataset(tmp_path / "out" / "manifest.json", tokenizer_id="gpt2")
    # the pasted block is a loadable [data] section
    import tomllib

    block = tomllib.loads(data_config_snippet(validate_dataset_manifest(tmp_path / "out" / "manifest.json")))["data"]
    assert block["order"] == "document_buffer" and block["tokenizer_id"] == "byte-level" and block["mode"] == "prepared"
