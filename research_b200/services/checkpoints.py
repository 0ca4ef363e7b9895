"""Checkpoint service: composite checkpoints in an Orbax-like directory layout, written and read without Orbax
(neither orbax nor tensorstore can be installed offline).  The layout is write-compatible by construction only: it
has not been cross-loaded by Orbax, and checkpoints that Orbax itself wrote (OCDBT + zstd by default) are not read.

Layout (what the reference's ``CheckpointManager`` produces, src/jaxtitan/services/checkpoints.py:54-176;
tests/jaxtitan/test_checkpoints.py:53)::

    checkpoints/<step:06d>/
        _CHECKPOINT_METADATA            step-level metadata (item names, commit timestamp)
        train/                          pytree item: one Zarr v2 array per leaf (non-OCDBT layout)
            _METADATA                   tree structure: leaf key paths, dtypes, shapes
            _sharding                   per-leaf sharding descriptions (single-host: replicated)
            <leaf.key.path>/.zarray     zarr v2 header, one uncompressed chunk
            <leaf.key.path>/0.0...      the chunk (C order, little endian)
        dataset/metadata                JSON item
        host/metadata                   JSON item
        metadata/metadata               JSON item

Leaf key paths follow the reference's ``TrainState`` (step, tokens_seen, model.<nnx path>, opt_state..., rng...,
moe_balance...) with model kernels in the reference's ``[in, out]`` orientation.  The reader reads this writer's
output.
Retention: keep the newest ``max_to_keep`` plus protected steps (latest / best), as the reference's
``_ProtectedLatestPolicy`` (checkpoints.py:183-199).  Saves are synchronous: everything is written and fsynced
in a temporary directory, an existing directory of the same step is moved aside only then, and the rename commits.
"""

from __future__ import annotations

import json
import os
import shutil
import time
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Iterable, Mapping

import numpy as np

from research_b200.config.canonical import canonical_json
from research_b200.errors import ContractError

STEP_DIGITS = 6
_DTYPES = {"float32": "<f4", "float64": "<f8", "int32": "<i4", "int64": "<i8", "uint32": "<u4", "uint64": "<u8",
           "uint8": "|u1", "bool": "|b1", "float16": "<f2", "uint16": "<u2", "int16": "<i2"}


def step_dir_name(step: int) -> str:
    return f"{step:0{STEP_DIGITS}d}"


@dataclass
class CheckpointRestore:
    tensors: dict[str, np.ndarray]
    dataset_state: dict[str, Any]
    host_state: dict[str, Any]
    metadata: dict[str, Any]
    step: int
    path: Path


def _zarr_dtype(arr: np.ndarray) -> str:
    name = arr.dtype.name
    if name not in _DTYPES:
        raise ContractError(f"unsupported checkpoint leaf dtype {name}")
    return _DTYPES[name]


def write_array(leaf_dir: Path, arr: np.ndarray) -> None:
    """One zarr-v2 array with a single uncompressed chunk (bfloat16 leaves are stored as uint16 bit patterns)."""

    leaf_dir.mkdir(parents=True, exist_ok=False)
    arr = np.asarray(arr)
    if not arr.flags.c_contiguous:
        arr = arr.copy(order="C")                 # (``ascontiguousarray`` would turn a scalar into shape [1])
    header = {"chunks": list(arr.shape) if arr.ndim else [], "compressor": None, "dtype": _zarr_dtype(arr),
              "fill_value": None, "filters": None, "order": "C", "shape": list(arr.shape), "zarr_format": 2,
              "dimension_separator": "."}
    (leaf_dir / ".zarray").write_text(json.dumps(header, sort_keys=True))
    chunk_name = ".".join("0" for _ in arr.shape) if arr.ndim else "0"
    _write_bytes(leaf_dir / chunk_name, arr)


def _write_bytes(path: Path, arr: np.ndarray) -> None:
    from research_b200.native import hostlib

    data = arr.astype(arr.dtype.newbyteorder("<"), copy=False)
    if not hostlib.write_file(path, data):
        with path.open("wb") as handle:
            handle.write(data.tobytes())


def _decode_chunk(raw: bytes, compressor: Any, nbytes: int, where: Path) -> bytes:
    """Undo a zarr-v2 chunk compressor: none, ``zstd`` (through pyarrow's codec), ``gzip`` or ``zlib``."""

    if compressor is None:
        return raw
    kind = compressor.get("id") if isinstance(compressor, dict) else None
    if kind == "zstd":
        try:
            import pyarrow as pa
        except ImportError as exc:
            raise ContractError(f"checkpoint chunk {where} is zstd-compressed and pyarrow is not installed") from exc
        try:
            return pa.Codec("zstd").decompress(raw, decompressed_size=nbytes).to_pybytes()
        except Exception as exc:
            raise ContractError(f"checkpoint chunk {where} does not decompress (zstd): {exc}") from exc
    if kind in ("gzip", "zlib"):
        import gzip
        import zlib

        try:
            return gzip.decompress(raw) if kind == "gzip" else zlib.decompress(raw)
        except Exception as exc:
            raise ContractError(f"checkpoint chunk {where} does not decompress ({kind}): {exc}") from exc
    raise ContractError(f"checkpoint chunk {where} uses the unsupported compressor {compressor!r}")


def read_array(leaf_dir: Path) -> np.ndarray:
    """One zarr-v2 array: the single raw chunk this service writes, and also what other writers of the format produce
    - a grid of chunks (edge chunks padded to the chunk shape, absent chunks meaning the fill value), ``.`` or ``/``
    between chunk indices, C or F order inside a chunk, and ``zstd`` / ``gzip`` / ``zlib`` chunk compression - which
    is the form of an Orbax checkpoint written with ``use_ocdbt=False``.  Filters are not supported."""

    try:
        header = json.loads((leaf_dir / ".zarray").read_text())
    except (OSError, json.JSONDecodeError) as exc:
        raise ContractError(f"checkpoint leaf {leaf_dir} has no readable .zarray: {exc}") from exc
    if header.get("zarr_format", 2) != 2:
        raise ContractError(f"checkpoint leaf {leaf_dir} has zarr_format {header.get('zarr_format')}; only 2 is read")
    if header.get("filters"):
        raise ContractError(f"checkpoint leaf {leaf_dir} uses filters {header['filters']!r}; none are supported")
    compressor = header.get("compressor")
    shape = tuple(int(n) for n in header["shape"])
    chunks = tuple(int(n) for n in (header.get("chunks") or shape))
    if len(chunks) != len(shape) or any(c <= 0 for c in chunks):
        raise ContractError(f"checkpoint leaf {leaf_dir} has chunks {chunks} for shape {shape}")
    sep = header.get("dimension_separator", ".")
    dtype = np.dtype(header["dtype"])
    order = header.get("order", "C")
    chunk_bytes = (int(np.prod(chunks, dtype=np.int64)) if shape else 1) * dtype.itemsize
    if compressor is None and chunks == shape:
        # the form this service writes: one raw file, read without a copy through a staging buffer
        path = leaf_dir / (sep.join("0" for _ in shape) if shape else "0")
        if not path.is_file() or path.stat().st_size != chunk_bytes:
            raise ContractError(f"checkpoint chunk {path} is missing or has the wrong size (expected {chunk_bytes} bytes)")
        flat = np.fromfile(path, dtype=dtype)
        return flat.reshape(shape, order=order) if shape else flat.reshape(())
    fill = header.get("fill_value")
    out = np.full(shape, 0 if fill is None else fill, dtype=dtype)
    grid = [range(-(-n // c)) for n, c in zip(shape, chunks)]
    import itertools

    for index in (itertools.product(*grid) if shape else [()]):
        path = leaf_dir / (sep.join(str(i) for i in index) if shape else "0")
        if not path.is_file():
            continue                                     # zarr: an absent chunk holds the fill value
        data = _decode_chunk(path.read_bytes(), compressor, chunk_bytes, path)
        if len(data) != chunk_bytes:
            raise ContractError(f"checkpoint chunk {path} has {len(data)} bytes after decoding, expected {chunk_bytes}")
        block = np.frombuffer(data, dtype=dtype).reshape(chunks, order=order) if shape else np.frombuffer(data, dtype=dtype)
        if not shape:
            return block.reshape(()).copy()
        lo = [i * c for i, c in zip(index, chunks)]
        hi = [min(a + c, n) for a, c, n in zip(lo, chunks, shape)]
        out[tuple(slice(a, b) for a, b in zip(lo, hi))] = block[tuple(slice(0, b - a) for a, b in zip(lo, hi))]
    return out


def _fsync_dir(path: Path) -> None:
    try:
        fd = os.open(path, os.O_RDONLY)
    except OSError:
        return
    try:
        os.fsync(fd)
    except OSError:
        pass
    finally:
        os.close(fd)


def _fsync_tree(root: Path) -> None:
    """Flush every file and directory under ``root`` so that the rename that follows commits complete data."""

    for dirpath, _, files in os.walk(root):
        for name in files:
            try:
                fd = os.open(os.path.join(dirpath, name), os.O_RDONLY)
            except OSError:
                continue
            try:
                os.fsync(fd)
            except OSError:
                pass
            finally:
                os.close(fd)
        _fsync_dir(Path(dirpath))


class LocalCheckpointService:
    ITEMS = ("train", "dataset", "host", "metadata")

    def __init__(self, run_dir: str | Path, *, max_to_keep: int = 2, protected_steps: set[int] | None = None,
                 is_writer: bool = True) -> None:
        if max_to_keep <= 0:
            raise ContractError(f"max_to_keep must be positive, got {max_to_keep}")
        self.run_dir = Path(run_dir)
        self.checkpoints_dir = self.run_dir / "checkpoints"
        self.max_to_keep = max_to_keep
        self.protected_steps = set(protected_steps or ())
        self.is_writer = is_writer
        if is_writer:
            self.checkpoints_dir.mkdir(parents=True, exist_ok=True)

    # ---- save ----------------------------------------------------------------------------------------
    def save(self, step: int, tensors: "Mapping[str, np.ndarray] | Iterable[tuple[str, np.ndarray | None]]",
             dataset_state: Mapping[str, Any], host_state: Mapping[str, Any], metadata: Mapping[str, Any]) -> Path:
        """``tensors``: a mapping, or an iterable of ``(leaf name, array)`` pairs that is consumed leaf by leaf (so
        that a producer which gathers one parameter at a time never holds the whole state).  Ranks that do not write
        still drain the iterable, because producing it may be a collective operation."""

        if step < 0:
            raise ContractError(f"checkpoint step must be non-negative, got {step}")
        if host_state.get("dataset") != dict(dataset_state):
            raise ContractError("host_state.dataset must match dataset_state when saving a checkpoint")
        final = self.checkpoints_dir / step_dir_name(step)
        pairs = tensors.items() if hasattr(tensors, "items") else tensors
        if not self.is_writer:
            for _ in pairs:
                pass
            return final
        tmp = self.checkpoints_dir / f"{step_dir_name(step)}.orbax-checkpoint-tmp-{int(time.time() * 1e6)}"
        try:
            train = tmp / "train"
            train.mkdir(parents=True)
            tree_meta = {}
            names = []
            for name, value in pairs:
                arr = np.asarray(value)
                names.append(name)
                write_array(train / name, arr)
                tree_meta[name] = {"key_metadata": [{"key": part, "key_type": 2} for part in name.split(".")],
                                   "value_metadata": {"value_type": "jax.Array", "skip_deserialize": False,
                                                      "dtype": arr.dtype.name, "shape": list(arr.shape)}}
            (train / "_METADATA").write_text(json.dumps({"tree_metadata": tree_meta, "use_zarr3": False,
                                                         "store_array_data_equal_to_fill_value": True}, sort_keys=True))
            (train / "_sharding").write_text(json.dumps({name: {"sharding_type": "SingleDeviceSharding"}
                                                         for name in names}, sort_keys=True))
            for item, payload in (("dataset", dataset_state), ("host", host_state), ("metadata", metadata)):
                (tmp / item).mkdir()
                (tmp / item / "metadata").write_text(canonical_json(payload))
            (tmp / "_CHECKPOINT_METADATA").write_text(json.dumps({
                "item_handlers": {"train": "orbax.checkpoint._src.handlers.standard_checkpoint_handler.StandardCheckpointHandler",
                                  "dataset": "orbax.checkpoint._src.handlers.json_checkpoint_handler.JsonCheckpointHandler",
                                  "host": "orbax.checkpoint._src.handlers.json_checkpoint_handler.JsonCheckpointHandler",
                                  "metadata": "orbax.checkpoint._src.handlers.json_checkpoint_handler.JsonCheckpointHandler"},
                "init_timestamp_nsecs": time.time_ns(), "commit_timestamp_nsecs": time.time_ns(),
                "writer": "research_b200"}, sort_keys=True))
            _fsync_tree(tmp)
            old = None
            if final.exists():           # same step saved again: the old copy goes only once the new one is complete
                old = self.checkpoints_dir / f"{step_dir_name(step)}.replaced-{int(time.time() * 1e6)}"
                final.replace(old)
            tmp.replace(final)
            _fsync_dir(self.checkpoints_dir)
            if old is not None:
                shutil.rmtree(old, ignore_errors=True)
        except Exception:
            shutil.rmtree(tmp, ignore_errors=True)
            raise
        self._apply_retention()
        return final

    def _apply_retention(self) -> None:
        steps = self.all_steps()
        keep = set(steps[-self.max_to_keep:]) | self.protected_steps
        for s in steps:
            if s not in keep:
                shutil.rmtree(self.checkpoints_dir / step_dir_name(s), ignore_errors=True)

    def set_protected_steps(self, steps: set[int]) -> None:
        self.protected_steps = set(steps)

    # ---- restore -------------------------------------------------------------------------------------
    def all_steps(self) -> list[int]:
        if not self.checkpoints_dir.is_dir():
            return []
        out = []
        for child in self.checkpoints_dir.iterdir():
            if child.is_dir() and child.name.isdigit() and (child / "_CHECKPOINT_METADATA").exists():
                out.append(int(child.name))
        return sorted(out)

    def latest_step(self) -> int | None:
        steps = self.all_steps()
        return steps[-1] if steps else None

    def latest_path(self) -> Path | None:
        step = self.latest_step()
        return None if step is None else self.checkpoints_dir / step_dir_name(step)

    def _step_path(self, step: int) -> Path:
        path = self.checkpoints_dir / step_dir_name(step)
        if not path.is_dir():
            raise ContractError(f"checkpoint step {step} does not exist in {self.checkpoints_dir}")
        return path

    def _read_json_item(self, path: Path, item: str) -> dict[str, Any]:
        file = path / item / "metadata"
        try:
            raw = json.loads(file.read_text())
        except (OSError, json.JSONDecodeError) as exc:
            raise ContractError(f"checkpoint item {item} in {path} is unreadable: {exc}") from exc
        if not isinstance(raw, dict):
            raise ContractError(f"checkpoint item {item} in {path} must be a JSON object")
        return raw

    def restore_metadata(self, step: int) -> dict[str, Any]:
        return self._read_json_item(self._step_path(step), "metadata")

    def restore_latest_metadata(self) -> dict[str, Any]:
        step = self.latest_step()
        if step is None:
            raise ContractError(f"no checkpoints found in {self.checkpoints_dir}")
        return self.restore_metadata(step)

    def restore(self, step: int, names: list[str] | None = None) -> CheckpointRestore:
        path = self._step_path(step)
        train = path / "train"
        try:
            tree = json.loads((train / "_METADATA").read_text())["tree_metadata"]
        except (OSError, json.JSONDecodeError, KeyError) as exc:
            raise ContractError(f"checkpoint {path} has no readable train/_METADATA: {exc}") from exc
        wanted = list(tree) if names is None else names
        tensors = {}
        for name in wanted:
            if name not in tree:
                raise ContractError(f"checkpoint {path} has no leaf {name!r}")
            tensors[name] = read_array(train / name)
        dataset = self._read_json_item(path, "dataset")
        host = self._read_json_item(path, "host")
        if host.get("dataset") != dataset:
            raise ContractError("restored host_state.dataset does not match restored dataset_state")
        return CheckpointRestore(tensors, dataset, host, self._read_json_item(path, "metadata"), step, path)

    def restore_latest(self) -> CheckpointRestore:
        step = self.latest_step()
        if step is None:
            raise ContractError(f"no checkpoints found in {self.checkpoints_dir}")
        return self.restore(step)

    def close(self) -> None:
        return None
