"""Environment and runtime switches, checked on the host: what each one turns on or off."""

import subprocess
import sys
from pathlib import Path
from types import SimpleNamespace

import pytest
import torch

from research_b200.ops import functional as Fn
from research_b200.ops import native

ROOT = Path(__file__).resolve().parent.parent


def _probe(env: dict, code: str) -> str:
    import os

    proc = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=120, cwd=ROOT,
                          env={**os.environ, **env})
    assert proc.returncode == 0, proc.stderr[-2000:]
    return proc.stdout.strip().splitlines()[-1]


def test_deterministic_switch_is_read_from_the_environment_and_settable():
    code = "from research_b200.ops import native; print(native.deterministic())"
    assert _probe({"RESEARCH_B200_DETERMINISTIC": "1"}, code) == "True"
    assert _probe({"RESEARCH_B200_DETERMINISTIC": "0"}, code) == "False"
    assert not native.deterministic()
    native.set_deterministic(True)
    try:
        assert native.deterministic() and Fn._ordered_sums_only()
    finally:
        native.set_deterministic(False)
    assert not Fn._ordered_sums_only()


def test_deterministic_mode_turns_the_arrival_ordered_kernels_off():
    """The fused tensor-parallel GEMMs, the in-kernel K/V exchange and the fused expert dispatch all add partial
    results in arrival order: the switch routes around them (the NCCL formulations have a fixed order)."""

    from research_b200.parallel import expert_fused, ring_attention

    q = torch.zeros(1, 256, 2, 64, dtype=torch.bfloat16)
    ex = SimpleNamespace(cp_size=2)
    native.set_deterministic(True)
    try:
        assert not expert_fused.fused_gemm_requested()
        assert not ring_attention.ring_available(ex, q, 256, 2, 64, [(0, 128), (384, 128)])
    finally:
        native.set_deterministic(False)
    assert expert_fused.fused_gemm_requested()


@pytest.mark.parametrize("value,expect", [("0", "False"), ("1", "True")])
def test_fused_expert_dispatch_switch(value, expect):
    code = "from research_b200.parallel import expert_fused as e; print(e.fused_gemm_requested())"
    assert _probe({"RESEARCH_B200_MOE_FUSED": value}, code) == expect


def test_peer_wait_limit_is_clamped_and_lands_in_the_status_words():
    code = "from research_b200.ops import native; print(native.peer_wait_limit_ms())"
    assert _probe({"RESEARCH_B200_PEER_WAIT_MS": "1234"}, code) == "1234"
    assert _probe({"RESEARCH_B200_PEER_WAIT_MS": "0"}, code) == "1"            # never "no limit"
    assert native.peer_wait_limit_ms() >= 1


def test_nvls_is_opt_in():
    code = "from research_b200.parallel.symmetric import nvls_requested; print(nvls_requested())"
    assert _probe({"RESEARCH_B200_NVLS": "1"}, code) == "True"
    assert _probe({"RESEARCH_B200_NVLS": ""}, code) == "False"


def test_dion2_kernel_size_rules():
    assert native.dion2_supported(8, 2048, 1408, 2048 * 1408, 0)
    assert native.dion2_supported(8, 2048, 1408, 2 * 2048 * 1408, 1)           # row ranges of a fused entry
    assert not native.dion2_supported(1, 64, 66, 64 * 66, 0)                   # rows are not 16-byte multiples
    assert not native.dion2_supported(1, 64, 16384, 64 * 16384, 1)             # more slices than the rank kernel holds
    assert not native.dion2_supported(0, 64, 64, 4096, 0)


def test_wave_splits_fills_whole_waves_and_respects_the_slice_floor():
    # 16 x 8 output tiles on 148 SMs: 128 tiles leave 20 SMs idle, a second K slice would need two waves for 256
    assert native.wave_splits(2048, 2048, 32768) in (1, 2, 3, 4, 5, 6, 7, 8)
    assert native.wave_splits(128, 256, 1024) == 1                               # slices of at least 1024 rows
    for m, n, k in [(2048, 2048, 32768), (4096, 2048, 32768), (2048, 8192, 16384)]:
        s = native.wave_splits(m, n, k)
        assert (k // 64) % s == 0 and k // s >= 1024
