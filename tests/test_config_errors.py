"""Every cross-section rule and a sample of the per-field rules of the run contract, one case per message.

The messages are part of the public contract (the reference checks each of them:
tests/jaxtitan/test_config.py:230-1533); a valid tiny config is mutated and the loader must refuse it with the
reference's wording."""

import copy
from pathlib import Path

import pytest

from research_b200.config import run_spec_from_mapping
from research_b200.errors import JaxtitanError
from tests.helpers import tiny_raw_config

MOE = dict(num_experts=4, top_k=2, expert_intermediate_size=32, num_shared_experts=1, balance=dict(name="smebu"))


def _base(kind="decoder", **kw):
    return tiny_raw_config(Path("m.json"), kind=kind, **kw)


def _set(raw, dotted, value):
    node = raw
    *parents, leaf = dotted.split(".")
    for key in parents:
        node = node.setdefault(key, {})
    if value is _DELETE:
        node.pop(leaf, None)
    else:
        node[leaf] = value
    return raw


_DELETE = object()


def _mesh(raw, **axes):
    raw["mesh"] = dict(axis_names=list(axes), axis_sizes=list(axes.values()))
    return raw


CASES = [
    # ---- cross-section rules (config/validate.py) --------------------------------------------------------------
    ("max_seq_len", lambda r: _set(r, "model.max_seq_len", 16), r"model.max_seq_len \(16\) must be >= training.seq_len \(32\)"),
    ("target_tokens", lambda r: _set(r, "training.target_tokens", 10), "must cover at least one effective optimizer batch"),
    ("clip_twice", lambda r: _set(r, "training.grad_clip_norm", 1.0), "set grad_clip_norm in either"),
    ("batch_vs_data", lambda r: _mesh(_set(r, "training.global_batch_size", 3), data=2),
     r"training.global_batch_size \(3\) must be divisible by the data axis size \(2\)"),
    ("cp_axis_without_flag", lambda r: _mesh(r, cp=2), "mesh cp axis size greater than 1 requires parallelism.context_parallel=true"),
    ("cp_flag_without_axis", lambda r: _set(r, "parallelism", {"context_parallel": True}),
     "parallelism.context_parallel=true requires a mesh cp axis"),
    ("cp_seq_len", lambda r: _set(_set(_mesh(r, cp=3), "parallelism", {"context_parallel": True}), "training.seq_len", 32),
     r"training.seq_len \(32\) must be divisible by cp axis size \(3\)"),
    ("ulysses_heads", lambda r: _set(_mesh(r, cp=4), "parallelism", {"context_parallel": True, "context_attention": "ulysses"}),
     r"model.n_kv_heads \(2\) must be divisible by tp x cp \(4\)"),
    ("tp_axis_without_flag", lambda r: _mesh(r, tp=2), "mesh tp axis size greater than 1 requires parallelism.tensor_parallel=true"),
    ("tp_flag_without_axis", lambda r: _set(r, "parallelism", {"tensor_parallel": True}),
     "parallelism.tensor_parallel=true requires a mesh tp axis"),
    ("tp_hidden", lambda r: _set(_set(_mesh(r, tp=3), "parallelism", {"tensor_parallel": True}), "training.seq_len", 33),
     r"model.hidden_size \(64\) must be divisible by tp axis size \(3\)"),
    ("tp_vocab", lambda r: _set(_set(_mesh(r, tp=2), "parallelism", {"tensor_parallel": True}), "model.vocab_size", 255),
     r"model.vocab_size \(255\) must be divisible by tp axis size \(2\)"),
    ("tp_seq_len", lambda r: _set(_set(_set(_mesh(r, tp=2), "parallelism", {"tensor_parallel": True}), "training.seq_len", 31),
                                   "training.target_tokens", 31 * 4 * 4),
     r"training.seq_len \(31\) must be divisible by tp axis size \(2\)"),
    ("ddp_with_fsdp_axis", lambda r: _mesh(r, fsdp=2), "parallelism.mode='ddp' requires mesh fsdp axis size to be 1"),
    ("zero2_without_axis", lambda r: _set(r, "parallelism", {"mode": "zero2"}), "parallelism.mode='zero2' requires a mesh fsdp axis"),
    ("fsdp_without_axis", lambda r: _set(r, "parallelism", {"mode": "fsdp"}), "parallelism.mode='fsdp' requires a mesh fsdp axis"),
    ("ep_axis_without_flag", lambda r: _mesh(r, ep=2), "mesh ep axis size greater than 1 requires parallelism.expert_parallel=true"),
    ("ep_needs_moe", lambda r: _set(_mesh(r, ep=2), "parallelism", {"expert_parallel": True}),
     "parallelism.expert_parallel=true requires a Trinity MoE model"),
    ("ep_flag_without_axis", lambda r: _set(r, "parallelism", {"expert_parallel": True}),
     "requires a mesh ep axis or parallelism.mode='fsdp'"),
    ("ep_axis_requires_flag", lambda r: _set(r, "parallelism", {"expert_parallel_axis": "ep"}),
     "parallelism.expert_parallel_axis requires parallelism.expert_parallel=true"),
    ("ep_axis_fsdp_needs_mode", lambda r: _set(_mesh(r, ep=2), "parallelism", {"expert_parallel": True, "expert_parallel_axis": "fsdp"}),
     "parallelism.expert_parallel_axis='fsdp' requires parallelism.mode='fsdp'"),
    ("resident_needs_fsdp", lambda r: _set(r, "parallelism", {"fsdp_resident": False}),
     "parallelism.fsdp_resident=false requires parallelism.mode='fsdp'"),
    ("vocab_parallel_needs_tp", lambda r: _set(r, "parallelism", {"vocab_parallel_head": True}),
     "parallelism.vocab_parallel_head=true requires parallelism.tensor_parallel=true"),
    ("profiling_unreachable", lambda r: _set(r, "profiling", {"enabled": True, "trace_start_step": 50}),
     "profiling.trace_start_step must be reachable by training.target_tokens; trace_start_step=50 estimated_steps=4"),
    # ---- per-section rules (config/specs.py) ----------------------------------------------------------------------
    ("mode_name", lambda r: _set(r, "parallelism", {"mode": "pipeline"}), "parallelism.mode"),
    ("context_attention", lambda r: _set(r, "parallelism", {"context_attention": "ring3"}), "parallelism.context_attention"),
    ("optimizer_name", lambda r: _set(r, "optimizer.name", "sgd"), "optimizer.name"),
    ("muon_tp_mode", lambda r: _set(r, "optimizer.muon_tp_mode", "distributed"),
     "optimizer.muon_tp_mode is only supported when optimizer.name is 'muon'"),
    ("remat", lambda r: _set(r, "model.remat", "half"), "model.remat"),
    ("order", lambda r: _set(r, "data.order", "random"), "data.order must be 'sequential', 'shuffle', or 'document_buffer'"),
    ("shuffle_needs_seed", lambda r: _set(_set(r, "data.order", "shuffle"), "data.shuffle_seed", _DELETE),
     "data.shuffle_seed is required when data.order='shuffle'"),
    ("streaming_with_manifest", lambda r: _set(_set(r, "data.mode", "hf_streaming"), "data.tokenizer_id", "gpt2"),
     "data.train_manifest must be omitted when data.mode='hf_streaming'"),
    ("prepared_without_manifest", lambda r: _set(r, "data.train_manifest", _DELETE), "data.train_manifest is required"),
    ("profiling_steps", lambda r: _set(r, "profiling", {"enabled": True, "trace_steps": 0}), "profiling.trace_steps must be positive, got 0"),
    ("mesh_duplicate_axis", lambda r: _set(r, "mesh", {"axis_names": ["data", "data"], "axis_sizes": [1, 1]}),
     "mesh axis names must be unique"),
    ("mesh_zero_size", lambda r: _set(r, "mesh", {"axis_names": ["data"], "axis_sizes": [0]}), "mesh axis sizes must be positive"),
    ("mesh_length_mismatch", lambda r: _set(r, "mesh", {"axis_names": ["data", "fsdp"], "axis_sizes": [1]}),
     "mesh.axis_names and mesh.axis_sizes must have the same length"),
]

MOE_CASES = [
    ("ep_experts", lambda r: _set(_mesh(r, ep=3), "parallelism", {"expert_parallel": True}),
     r"model.trinity.moe.num_experts \(4\) must be divisible by ep axis size \(3\)"),
    ("efsdp_muon", lambda r: _set(_set(_mesh(r, fsdp=1, ep=2, expert_fsdp=2), "parallelism", {"mode": "fsdp", "expert_parallel": True}),
                                  "optimizer.name", "muon"),
     "optimizer.name='muon' is not supported with expert_fsdp axis size greater than 1"),
    ("efsdp_intermediate", lambda r: _set(_mesh(r, fsdp=1, ep=2, expert_fsdp=3), "parallelism", {"mode": "fsdp", "expert_parallel": True}),
     r"model.trinity.moe.expert_intermediate_size \(32\) must be divisible by expert_fsdp axis size \(3\)"),
    ("top_k", lambda r: _set(r, "model.trinity.moe.top_k", 9), "top_k"),
    ("local_layers", lambda r: _set(r, "model.trinity.local_layers_per_global", -1), "model.trinity.local_layers_per_global"),
    ("route_scale", lambda r: _set(r, "model.trinity.moe.route_scale", 0.0), "model.trinity.moe.route_scale must be positive"),
    ("router_kind", lambda r: _set(r, "model.trinity.moe.router", "tanh"), "model.trinity.moe.router"),
]


@pytest.mark.parametrize("name,mutate,message", CASES, ids=[c[0] for c in CASES])
def test_invalid_dense_config_is_refused_with_the_contract_message(name, mutate, message):
    raw = mutate(copy.deepcopy(_base()))
    with pytest.raises(JaxtitanError, match=message):
        run_spec_from_mapping(raw)


@pytest.mark.parametrize("name,mutate,message", MOE_CASES, ids=[c[0] for c in MOE_CASES])
def test_invalid_moe_config_is_refused_with_the_contract_message(name, mutate, message):
    raw = mutate(copy.deepcopy(_base(kind="trinity")))
    with pytest.raises(JaxtitanError, match=message):
        run_spec_from_mapping(raw)


def test_the_unmutated_configs_load():
    assert run_spec_from_mapping(_base()).model.name == "decoder"
    assert run_spec_from_mapping(_base(kind="trinity")).model.trinity.moe.num_experts == 4
