"""The kernels' status word is checked on every training step, without any debug switch."""

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _smoke_trainer():
    from research_b200.config import run_spec_from_mapping
    from research_b200.runtime.trainer import Trainer

    raw = {
        "run": {"id": "status"},
        "model": {"name": "decoder", "variant": "smoke", "vocab_size": 1024, "hidden_size": 256,
                  "intermediate_size": 512, "num_layers": 2, "num_heads": 2, "n_kv_heads": 1, "max_seq_len": 256,
                  "rope_theta": 10000.0, "init": "normal_0.02"},
        "optimizer": {"name": "adamw", "schedule": {"peak_lr": 1e-3}},
        "data": {"train_manifest": "unused.json"},
        "training": {"seq_len": 256, "global_batch_size": 2, "target_tokens": 2 * 256 * 8, "precision": "bf16"},
    }
    return Trainer(run_spec_from_mapping(raw), build_data=False)


def _batch():
    from research_b200.contracts import Batch

    ids = np.random.default_rng(0).integers(0, 1024, size=(2, 257)).astype(np.int32)
    return Batch(input_ids=ids[:, :-1], target_ids=ids[:, 1:], loss_mask=np.ones((2, 256), dtype=bool),
                 token_doc_ids=None)


def test_train_step_raises_when_a_bounded_wait_gave_up(monkeypatch):
    """A kernel whose bounded wait ran out writes a code to the status word and skips its work; the step that
    follows must fail loudly on the host instead of training on partial data."""

    from research_b200.errors import KernelError
    from research_b200.ops import native

    monkeypatch.delenv("RESEARCH_B200_DEBUG", raising=False)
    trainer = _smoke_trainer()
    assert not trainer.debug_checks
    trainer.train_on([_batch()])                                  # a clean step passes
    native.status_word()[0:1].fill_(21)                            # what a timed-out peer wait leaves behind
    with pytest.raises(KernelError, match="status code 21"):
        trainer.train_on([_batch()])
    assert int(native.status_word()[0].item()) == 0                # cleared, so the next check starts clean
    assert int(native.status_word()[2].item()) == native.peer_wait_limit_ms()   # the configured limit survives
    trainer.train_on([_batch()])
