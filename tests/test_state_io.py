"""Train state <-> checkpoint leaves: leaf names, the 64-bit token counter, saving under one layout and restoring
under another, replacing a step directory."""

import json

import numpy as np
import pytest
import torch

from research_b200.config import run_spec_from_mapping
from research_b200.runtime.state_io import (collect_state_tensors, iter_state_tensors, load_state_tensors,
                                            optimizer_leaf_names)
from research_b200.runtime.trainer import Trainer
from research_b200.services.checkpoints import LocalCheckpointService
from tests.helpers import run_gloo, tiny_dataset, tiny_raw_config


def _trainer(tmp_path, **kw):
    manifest = tmp_path / "ds" / "manifest.json"
    if not manifest.exists():
        manifest = tiny_dataset(tmp_path)
    return Trainer(run_spec_from_mapping(tiny_raw_config(manifest, **kw)), device="cpu")


def test_optimizer_leaves_follow_the_optax_chain_tree(tmp_path):
    """clip -> index 0 (no arrays); Muon with decay -> 1; AdamW fallback -> 2, whose own chain keeps mu / nu under
    element 0 (reference chain: src/jaxtitan/optim/build.py:176-202, 560-656)."""

    trainer = _trainer(tmp_path, optimizer="muon")
    names = optimizer_leaf_names(trainer)
    assert names[("momentum", "layers.0.attn.q.kernel")] == "opt_state.1.inner_state.momentum.layers.0.attn.q.kernel"
    assert names[("mu", "embed.embedding")] == "opt_state.2.inner_state.0.mu.embed.embedding"
    assert names[("nu", "norm.scale")] == "opt_state.2.inner_state.0.nu.norm.scale"
    trainer = _trainer(tmp_path, optimizer="adamw", clip=None)
    names = optimizer_leaf_names(trainer)
    assert names[("mu", "layers.0.attn.q.kernel")] == "opt_state.0.inner_state.0.mu.layers.0.attn.q.kernel"
    leaves = collect_state_tensors(trainer)
    assert set(names.values()) <= set(leaves)


def test_token_counter_beyond_32_bits_round_trips(tmp_path):
    trainer = _trainer(tmp_path)
    trainer.train_step()
    trainer.tokens_seen = (3 << 32) + 12345             # about 13e9 tokens: the uint32 leaf alone would wrap
    leaves = collect_state_tensors(trainer)
    assert leaves["tokens_seen"].dtype == np.uint32 and int(leaves["tokens_seen"]) == 12345
    assert int(leaves["tokens_seen_hi"]) == 3
    other = _trainer(tmp_path)
    load_state_tensors(other, leaves)
    assert other.tokens_seen == (3 << 32) + 12345 and other.step == 1
    for name, value in collect_state_tensors(other).items():
        assert np.array_equal(value, leaves[name]), name
    # a checkpoint written before the high word existed still loads
    del leaves["tokens_seen_hi"]
    load_state_tensors(other, leaves)
    assert other.tokens_seen == 12345


def test_legacy_optimizer_leaf_names_still_load(tmp_path):
    trainer = _trainer(tmp_path, optimizer="muon")
    trainer.train_step()
    leaves = collect_state_tensors(trainer)
    legacy = {}
    for name, value in leaves.items():
        if ".inner_state.momentum." in name:
            name = "opt_state.matrix.momentum." + name.split(".inner_state.momentum.", 1)[1]
        elif ".inner_state.0.mu." in name:
            name = "opt_state.adamw.mu." + name.split(".inner_state.0.mu.", 1)[1]
        elif ".inner_state.0.nu." in name:
            name = "opt_state.adamw.nu." + name.split(".inner_state.0.nu.", 1)[1]
        legacy[name] = value
    other = _trainer(tmp_path, optimizer="muon")
    load_state_tensors(other, legacy)
    for name, value in collect_state_tensors(other).items():
        assert np.array_equal(value, leaves[name]), name


def _save_sharded(rank, world, raw, out_dir):
    trainer = Trainer(run_spec_from_mapping(raw), device="cpu")
    for _ in range(2):
        trainer.train_step()
    svc = LocalCheckpointService(out_dir, is_writer=rank == 0)
    pairs = list(iter_state_tensors(trainer, writer_only=True))
    if rank != 0:
        assert all(value is None for _, value in pairs)          # only the writer assembles arrays
    svc.save(trainer.step, iter_state_tensors(trainer, writer_only=True), {"a": 1}, {"dataset": {"a": 1}}, {"m": 1})
    return {k: torch.from_numpy(np.array(v)) for k, v in collect_state_tensors(trainer).items()}


@pytest.mark.parametrize("optimizer,mesh,parallelism", [
    ("adamw", {"fsdp": 2}, {"mode": "zero2"}),
    ("muon", {"fsdp": 2}, {"mode": "fsdp"}),
    ("muon", {"fsdp": 2}, {"mode": "fsdp", "fsdp_resident": False}),       # weights sharded at rest
])
def test_sharded_save_assembles_on_the_writer_and_restores_on_one_process(tmp_path, optimizer, mesh, parallelism):
    manifest = tiny_dataset(tmp_path)
    raw = tiny_raw_config(manifest, optimizer=optimizer, mesh=mesh, parallelism=parallelism, steps=4)
    results = run_gloo(2, _save_sharded, raw, str(tmp_path / "run"))
    restored = LocalCheckpointService(tmp_path / "run").restore_latest()
    assert restored.step == 2
    for name, want in results[0].items():
        assert np.array_equal(restored.tensors[name].reshape(-1), want.numpy().reshape(-1)), name
    # the same leaves load into an unsharded trainer and come back bit for bit
    single = Trainer(run_spec_from_mapping(tiny_raw_config(manifest, optimizer=optimizer, steps=4)), device="cpu")
    load_state_tensors(single, restored.tensors)
    for name, value in collect_state_tensors(single).items():
        assert np.array_equal(value.reshape(-1), restored.tensors[name].reshape(-1)), name


def test_saving_a_step_twice_replaces_it_only_when_the_new_copy_is_complete(tmp_path):
    svc = LocalCheckpointService(tmp_path)
    svc.save(3, {"x": np.arange(4, dtype=np.float32)}, {"a": 1}, {"dataset": {"a": 1}}, {"v": 1})

    def failing():
        yield "x", np.arange(4, dtype=np.float32) + 1
        raise RuntimeError("producer died")

    with pytest.raises(RuntimeError):
        svc.save(3, failing(), {"a": 1}, {"dataset": {"a": 1}}, {"v": 2})
    kept = svc.restore(3)
    assert kept.metadata == {"v": 1} and np.array_equal(kept.tensors["x"], np.arange(4, dtype=np.float32))
    svc.save(3, {"x": np.arange(4, dtype=np.float32) + 2}, {"a": 1}, {"dataset": {"a": 1}}, {"v": 3})
    assert svc.restore(3).metadata == {"v": 3}
    leftovers = [p.name for p in (tmp_path / "checkpoints").iterdir() if p.name != "000003"]
    assert leftovers == [], leftovers
    assert json.loads((tmp_path / "checkpoints" / "000003" / "_CHECKPOINT_METADATA").read_text())["writer"]


def _reload_sharded(rank, world, raw, ckpt_dir):
    """Restore into a job whose weights are sharded at rest and take one more step."""

    trainer = Trainer(run_spec_from_mapping(raw), device="cpu")
    restored = LocalCheckpointService(ckpt_dir, is_writer=False).restore_latest()
    load_state_tensors(trainer, restored.tensors)
    state = {k: torch.from_numpy(np.array(v)) for k, v in collect_state_tensors(trainer).items()}
    trainer.data_state = trainer.data.state_from_json(restored.dataset_state) if restored.dataset_state.get("backend") \
        else trainer.data_state
    loss = trainer.train_step().loss_sum
    return {"state": state, "loss": loss, "memory": trainer.store.memory_report()}


def test_restore_into_weights_sharded_at_rest(tmp_path):
    manifest = tiny_dataset(tmp_path)
    resident = tiny_raw_config(manifest, optimizer="muon", mesh={"fsdp": 2}, parallelism={"mode": "fsdp"}, steps=4)
    saved = run_gloo(2, _save_sharded, resident, str(tmp_path / "run"))
    sharded = tiny_raw_config(manifest, optimizer="muon", mesh={"fsdp": 2},
                              parallelism={"mode": "fsdp", "fsdp_resident": False}, steps=4)
    a = run_gloo(2, _reload_sharded, sharded, str(tmp_path / "run"))
    b = run_gloo(2, _reload_sharded, resident, str(tmp_path / "run"))
    for name, want in saved[0].items():
        assert np.array_equal(a[0]["state"][name].numpy().reshape(-1), want.numpy().reshape(-1)), name
    assert a[0]["loss"] == pytest.approx(b[0]["loss"], rel=1e-5)           # the step after the restore agrees
    assert a[0]["memory"]["mode"] == "sharded" and b[0]["memory"]["mode"] == "resident"
    assert a[0]["memory"]["compute_bytes"] < b[0]["memory"]["compute_bytes"]


def _write_zarr(leaf, arr, *, chunks, compressor=None, sep=".", order="C", skip=(), fill=0):
    """A zarr-v2 array written by hand, the way another writer of the format would lay it out."""

    import gzip
    import itertools
    import json as _json
    import zlib

    leaf.mkdir(parents=True)
    (leaf / ".zarray").write_text(_json.dumps({
        "zarr_format": 2, "shape": list(arr.shape), "chunks": list(chunks), "dtype": arr.dtype.str, "order": order,
        "compressor": compressor, "filters": None, "fill_value": fill, "dimension_separator": sep}))
    for index in itertools.product(*[range(-(-n // c)) for n, c in zip(arr.shape, chunks)]):
        if index in skip:
            continue
        block = np.full(chunks, fill, dtype=arr.dtype)
        lo = [i * c for i, c in zip(index, chunks)]
        hi = [min(a + c, n) for a, c, n in zip(lo, chunks, arr.shape)]
        block[tuple(slice(0, b - a) for a, b in zip(lo, hi))] = arr[tuple(slice(a, b) for a, b in zip(lo, hi))]
        raw = block.tobytes(order=order)
        kind = None if compressor is None else compressor["id"]
        if kind == "zstd":
            import pyarrow as pa

            raw = pa.Codec("zstd").compress(raw).to_pybytes()
        elif kind == "gzip":
            raw = gzip.compress(raw)
        elif kind == "zlib":
            raw = zlib.compress(raw)
        path = leaf / sep.join(str(i) for i in index)
        path.parent.mkdir(parents=True, exist_ok=True)
        path.write_bytes(raw)


@pytest.mark.parametrize("compressor", [None, {"id": "zstd", "level": 1}, {"id": "gzip", "level": 5}, {"id": "zlib", "level": 1}])
@pytest.mark.parametrize("sep, order", [(".", "C"), ("/", "C"), (".", "F")])
def test_leaves_written_by_other_zarr_writers_are_read(tmp_path, compressor, sep, order):
    from research_b200.services.checkpoints import read_array

    rng = np.random.default_rng(0)
    arr = rng.standard_normal((10, 7)).astype(np.float32)
    _write_zarr(tmp_path / "leaf", arr, chunks=(4, 3), compressor=compressor, sep=sep, order=order)
    got = read_array(tmp_path / "leaf")
    assert got.dtype == np.float32 and np.array_equal(got, arr)             # edge chunks are cut back to the shape
    ints = np.arange(24, dtype=np.int32).reshape(2, 3, 4)
    _write_zarr(tmp_path / "ints", ints, chunks=(1, 3, 2), compressor=compressor, sep=sep, order=order)
    assert np.array_equal(read_array(tmp_path / "ints"), ints)


def test_absent_chunks_hold_the_fill_value_and_bad_leaves_are_refused(tmp_path):
    from research_b200.errors import ContractError
    from research_b200.services.checkpoints import read_array, write_array

    arr = np.arange(16, dtype=np.float32).reshape(4, 4)
    _write_zarr(tmp_path / "sparse", arr, chunks=(2, 2), skip={(1, 1)}, fill=-1.0)
    want = arr.copy()
    want[2:, 2:] = -1.0
    assert np.array_equal(read_array(tmp_path / "sparse"), want)
    write_array(tmp_path / "own", arr)                                       # the form this service writes
    assert np.array_equal(read_array(tmp_path / "own"), arr)
    write_array(tmp_path / "scalar", np.asarray(7, dtype=np.int32))
    assert read_array(tmp_path / "scalar").shape == () and int(read_array(tmp_path / "scalar")) == 7
    _write_zarr(tmp_path / "blosc", arr, chunks=(2, 2))
    meta = json.loads((tmp_path / "blosc" / ".zarray").read_text())
    (tmp_path / "blosc" / ".zarray").write_text(json.dumps({**meta, "compressor": {"id": "blosc", "cname": "lz4"}}))
    with pytest.raises(ContractError, match="unsupported compressor"):
        read_array(tmp_path / "blosc")
    (tmp_path / "blosc" / ".zarray").write_text(json.dumps({**meta, "filters": [{"id": "delta"}]}))
    with pytest.raises(ContractError, match="uses filters"):
        read_array(tmp_path / "blosc")
    (tmp_path / "blosc" / ".zarray").write_text(json.dumps({**meta, "zarr_format": 3}))
    with pytest.raises(ContractError, match="zarr_format 3"):
        read_array(tmp_path / "blosc")
    _write_zarr(tmp_path / "torn", arr, chunks=(2, 2), compressor={"id": "zstd"})
    (tmp_path / "torn" / "0.0").write_bytes(b"not a zstd frame")
    with pytest.raises(ContractError, match="does not decompress"):
        read_array(tmp_path / "torn")
    (tmp_path / "own" / "0.0").write_bytes(b"short")
    with pytest.raises(ContractError, match="missing or has the wrong size"):
        read_array(tmp_path / "own")
