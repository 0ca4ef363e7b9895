"""One optimizer step on hand-made batches: loss normalisation, masking, z-loss, accumulation, clipping, learning
rate timing - each against the same quantity computed directly from the model's logits."""

import math

import numpy as np
import pytest
import torch

from research_b200.config import run_spec_from_mapping
from research_b200.contracts import Batch
from research_b200.runtime.trainer import Trainer
from tests.helpers import tiny_dataset, tiny_raw_config


@pytest.fixture(scope="module")
def manifest(tmp_path_factory):
    return tiny_dataset(tmp_path_factory.mktemp("step"))


def _trainer(manifest, **kw):
    z = kw.pop("z_loss_weight", None)
    schedule = kw.pop("schedule", None)
    raw = tiny_raw_config(manifest, **kw)
    if z is not None:
        raw["training"]["loss"] = {"z_loss_weight": z}
    if schedule is not None:
        raw["optimizer"]["schedule"] = schedule
    return Trainer(run_spec_from_mapping(raw), device="cpu")


def _batch(rows, seq=32, seed=0, mask=None):
    rng = np.random.default_rng(seed)
    tokens = rng.integers(0, 256, size=(rows, seq + 1), dtype=np.int64).astype(np.int32)
    m = np.ones((rows, seq), dtype=np.bool_) if mask is None else mask
    return Batch(input_ids=tokens[:, :-1].copy(), target_ids=tokens[:, 1:].copy(), loss_mask=m)


def _params(trainer):
    return {e.name: e.param.detach().clone() for e in trainer.store.entries}


def _direct(trainer, batch):
    """Masked CE sum, mask count and sum of logsumexp^2 straight from the logits."""

    model = trainer.result.model
    with torch.no_grad():
        logits = model(torch.from_numpy(batch.input_ids)).logits.double()
    lse = torch.logsumexp(logits, -1)
    target = logits.gather(-1, torch.from_numpy(batch.target_ids).long().unsqueeze(-1)).squeeze(-1)
    mask = torch.from_numpy(batch.loss_mask).double()
    return float(((lse - target) * mask).sum()), float(mask.sum()), float((lse.pow(2) * mask).sum())


def test_loss_is_the_masked_sum_over_the_masked_count(manifest):
    trainer = _trainer(manifest)
    mask = np.ones((4, 32), dtype=np.bool_)
    mask[0, :10] = False
    mask[3] = False
    batch = _batch(4, mask=mask)
    want_sum, want_count, _ = _direct(trainer, batch)
    metrics = trainer.train_on([batch])
    assert metrics.token_count == want_count == 4 * 32 - 10 - 32
    assert metrics.loss_sum == pytest.approx(want_sum, rel=1e-5) and metrics.loss == pytest.approx(want_sum / want_count, rel=1e-5)
    assert trainer.step == 1 and trainer.tokens_seen == 4 * 32            # tokens_seen counts positions, masked or not


def test_masked_positions_do_not_reach_the_gradients(manifest):
    mask = np.ones((4, 32), dtype=np.bool_)
    mask[:, 16:] = False
    a, b = _trainer(manifest), _trainer(manifest)
    first = _batch(4, mask=mask)
    second = Batch(input_ids=first.input_ids.copy(), target_ids=first.target_ids.copy(), loss_mask=mask.copy())
    second.target_ids[:, 16:] = (second.target_ids[:, 16:] + 7) % 256       # other targets where the mask is off
    ma, mb = a.train_on([first]), b.train_on([second])
    assert ma.loss_sum == mb.loss_sum
    pa, pb = _params(a), _params(b)
    assert all(torch.equal(pa[k], pb[k]) for k in pa)


def test_z_loss_is_weight_times_mean_squared_logsumexp_and_changes_the_update(manifest):
    plain, reg = _trainer(manifest), _trainer(manifest, z_loss_weight=1e-2)
    batch = _batch(4, seed=3)
    _, count, lse_sq = _direct(reg, batch)
    mp, mr = plain.train_on([batch]), reg.train_on([batch])
    assert mr.z_loss_sum == pytest.approx(lse_sq, rel=1e-5) and mr.loss_sum == pytest.approx(mp.loss_sum, rel=1e-6)
    from research_b200.runtime.training import metrics_row

    reg.last_provenance = None
    row = metrics_row(reg, mr, reg.spec)
    assert row["z_loss"] == pytest.approx(1e-2 * lse_sq / count, rel=1e-5)
    assert row["total_loss"] == pytest.approx(row["loss"] + row["z_loss"], rel=1e-9) and row["lm_loss"] == row["loss"]
    pp, pr = _params(plain), _params(reg)
    assert any(not torch.equal(pp[k], pr[k]) for k in pp)


def test_accumulated_microbatches_equal_one_large_batch(manifest):
    big = _batch(8, seed=5)
    halves = [Batch(input_ids=big.input_ids[i:i + 4].copy(), target_ids=big.target_ids[i:i + 4].copy(),
                    loss_mask=big.loss_mask[i:i + 4].copy()) for i in (0, 4)]
    whole, split = _trainer(manifest, batch=8), _trainer(manifest, batch=4, accum=2)
    mw, ms = whole.train_on([big], diagnostics=True), split.train_on(halves, diagnostics=True)
    assert ms.token_count == mw.token_count == 256 and ms.loss_sum == pytest.approx(mw.loss_sum, rel=1e-6)
    assert ms.grad_norm == pytest.approx(mw.grad_norm, rel=1e-4)
    assert len(ms.microbatch_loss_sums) == 2 and sum(ms.microbatch_loss_sums) == pytest.approx(ms.loss_sum, rel=1e-6)
    pw, ps = _params(whole), _params(split)
    for k in pw:
        assert torch.allclose(pw[k], ps[k], atol=2e-6, rtol=1e-5), k


def test_uneven_masks_weigh_microbatches_by_their_token_counts(manifest):
    mask = np.ones((8, 32), dtype=np.bool_)
    mask[4:, 4:] = False                                                    # the second half carries 16 tokens only
    big = _batch(8, seed=6, mask=mask)
    halves = [Batch(input_ids=big.input_ids[i:i + 4].copy(), target_ids=big.target_ids[i:i + 4].copy(),
                    loss_mask=big.loss_mask[i:i + 4].copy()) for i in (0, 4)]
    whole, split = _trainer(manifest, batch=8), _trainer(manifest, batch=4, accum=2)
    whole.train_on([big])
    ms = split.train_on(halves)
    assert ms.microbatch_token_counts == [128.0, 16.0]
    pw, ps = _params(whole), _params(split)
    for k in pw:
        assert torch.allclose(pw[k], ps[k], atol=2e-6, rtol=1e-5), k        # a mean of means would not match


def test_gradient_clipping_scales_the_update_and_reports_the_unclipped_norm(manifest):
    free, tight = _trainer(manifest, clip=None, optimizer="adamw"), _trainer(manifest, clip=1e-3)
    batch = _batch(4, seed=8)
    mf, mt = free.train_on([batch], diagnostics=True), tight.train_on([batch], diagnostics=True)
    assert mt.grad_norm == pytest.approx(mf.grad_norm, rel=1e-5) and mf.grad_norm > 1e-3
    # AdamW's first step is sign-like: clipping leaves its direction, so compare second moments through a second step
    grads_free = torch.cat([e.param.main_grad.flatten() for e in free.store.entries])
    grads_tight = torch.cat([e.param.main_grad.flatten() for e in tight.store.entries])
    assert float(grads_free.norm()) == pytest.approx(mf.grad_norm, rel=1e-4)
    scale = 1e-3 / mf.grad_norm
    exp_avg = [st["mu"] for st in tight.optimizer.state.values() if "mu" in st]
    exp_free = [st["mu"] for st in free.optimizer.state.values() if "mu" in st]
    assert exp_avg and all(torch.allclose(a, b * scale, rtol=1e-3, atol=1e-12) for a, b in zip(exp_avg, exp_free))
    assert grads_tight.shape == grads_free.shape


def test_learning_rate_is_evaluated_at_the_old_step_count(manifest):
    trainer = _trainer(manifest, schedule={"peak_lr": 4e-3, "name": "constant", "warmup_steps": 4})
    lrs = [trainer.train_on([_batch(4, seed=s)]).lr for s in range(5)]
    assert lrs == pytest.approx([1e-3, 2e-3, 3e-3, 4e-3, 4e-3])
    assert trainer.optimizer.count == 5


def test_update_and_parameter_norms_describe_the_step(manifest):
    trainer = _trainer(manifest)
    before = _params(trainer)
    metrics = trainer.train_on([_batch(4, seed=9)], diagnostics=True)
    after = _params(trainer)
    delta = math.sqrt(sum(float((after[k] - before[k]).double().pow(2).sum()) for k in after))
    norm = math.sqrt(sum(float(after[k].double().pow(2).sum()) for k in after))
    assert metrics.update_norm == pytest.approx(delta, rel=1e-3)
    assert metrics.param_norm == pytest.approx(norm, rel=1e-3) or metrics.param_norm == pytest.approx(
        math.sqrt(sum(float(before[k].double().pow(2).sum()) for k in before)), rel=1e-3)


def test_moe_step_reports_router_statistics_and_moves_the_bias(manifest):
    trainer = _trainer(manifest, kind="trinity")
    bias = trainer.result.model.layers[1].mlp.expert_bias
    before = bias.detach().clone()
    metrics = trainer.train_on([_batch(4, seed=10)], diagnostics=True)
    assert metrics.moe_aux_loss is not None and metrics.aux_loss is not None
    assert metrics.router["router_load_min"] >= 0 and metrics.router["router_max_vio"] >= 0
    assert len(metrics.router_layers) == 1 and metrics.router_layers[0]["layer_index"] == 1
    layer = metrics.router_layers[0]
    assert float(layer["counts"].sum()) == 4 * 32 * 2 and layer["importance"].shape == (4,)     # tokens x top_k
    from research_b200.optim.diagnostics import router_layers_payload

    (row,) = router_layers_payload(metrics.router_layers)
    assert row["layer_index"] == 1 and "load_cv" in row and "importance_entropy" in row and row["experts_active"] == 4
    assert not torch.equal(bias.detach(), before) and abs(float(bias.sum())) < 1e-6     # SMEBU: centred update
    assert metrics.smebu["smebu_bias_norm"] > 0


def test_narrow_compute_precision_keeps_the_balance_bias_in_fp32_and_in_the_checkpoint(tmp_path, manifest):
    """With bf16 compute copies the expert bias that SMEBU moves is the fp32 master: the router reads it, the bf16
    copy follows it, the checkpoint stores it with its momentum, and a resumed run continues from it."""

    from research_b200.runtime.training import run_training
    from research_b200.services.checkpoints import read_array
    from tests.helpers import write_toml

    raw = tiny_raw_config(manifest, kind="trinity", run_id="bf", output_dir=(tmp_path / "runs").as_posix(), steps=4,
                          checkpoint_every=2, evals=True)
    raw["model"]["compute_dtype"] = "bfloat16"
    raw["training"]["precision"] = "bf16"
    seen = {}
    run_training(write_toml(raw, tmp_path / "bf.toml"), trainer_hook=lambda t: seen.setdefault("first", t))
    mlp = seen["first"].result.model.layers[1].mlp
    assert mlp.expert_bias.dtype == torch.bfloat16 and mlp.bias_master.dtype == torch.float32
    assert float(mlp.bias_master.abs().max()) > 0 and abs(float(mlp.bias_master.sum())) < 1e-6
    assert torch.equal(mlp.expert_bias.data, mlp.bias_master.to(torch.bfloat16))          # the copy follows the master
    layer = seen["first"].moe_balance.layers[0]
    assert layer.bias.data_ptr() == mlp.bias_master.data_ptr() and layer.momentum.dtype == torch.float32
    leaf = tmp_path / "runs" / "bf" / "checkpoints" / "000004" / "train"
    assert np.allclose(read_array(leaf / "model.layers.1.mlp.expert_bias"), mlp.bias_master.numpy(), atol=0)
    assert np.allclose(read_array(leaf / "moe_balance.layers.0.momentum"), layer.momentum.numpy(), atol=0)
    raw["training"]["target_tokens"] = 32 * 4 * 6
    before = mlp.bias_master.clone()
    run_training(write_toml(raw, tmp_path / "bf.toml"), resume=True,
                 trainer_hook=lambda t: seen.setdefault("second", t))
    resumed = seen["second"].result.model.layers[1].mlp
    assert not torch.equal(resumed.bias_master, before) and seen["second"].step == 6
    # full precision compute: the parameter itself is the fp32 bias, nothing to mirror
    plain = _trainer(manifest, kind="trinity")
    assert plain.result.model.layers[1].mlp.bias_master is None and plain.moe_balance.layers[0].entry is None


@pytest.mark.parametrize("kind, optimizer", [("decoder", "muon"), ("trinity", "dion")])
def test_bf16_compute_copies_through_the_whole_run_lifecycle(tmp_path, manifest, kind, optimizer):
    """fp32 masters with bf16 compute copies on the host path: preflight, train with checkpoints and evals, checkpoint
    eval, sampling and resume all work, and the saved leaves are the fp32 masters."""

    from research_b200.runtime.checkpoint_eval import evaluate_checkpoint
    from research_b200.runtime.preflight import run_preflight
    from research_b200.runtime.sampling import sample_checkpoint
    from research_b200.runtime.training import run_training
    from research_b200.services.checkpoints import read_array
    from tests.helpers import write_toml

    raw = tiny_raw_config(manifest, kind=kind, optimizer=optimizer, run_id="half", output_dir=(tmp_path / "runs").as_posix(),
                          steps=4, checkpoint_every=2, evals=True)
    raw["model"]["compute_dtype"] = "bfloat16"
    raw["training"]["precision"] = "bf16"
    cfg = write_toml(raw, tmp_path / "half.toml")
    report = run_preflight(cfg)
    assert report["model"]["compute_dtype"] == "bfloat16" and report["first_step"]["loss"] > 0
    seen = {}
    summary = run_training(cfg, trainer_hook=lambda t: seen.setdefault("t", t))
    trainer = seen["t"]
    assert summary.steps == 4 and math.isfinite(summary.final_loss)
    assert all(e.param.dtype == torch.bfloat16 for e in trainer.store.entries)
    run_dir = tmp_path / "runs" / "half"
    saved = read_array(run_dir / "checkpoints" / "000004" / "train" / "model.layers.0.attn.o.kernel")
    assert saved.dtype == np.float32
    roundtrip = torch.from_numpy(saved).to(torch.bfloat16).float().numpy()
    assert not np.array_equal(saved, roundtrip)                    # the master carries bits a bf16 copy cannot
    payload = evaluate_checkpoint(run_dir, "latest")
    assert payload["loss"] == pytest.approx(summary.final_eval_loss, rel=1e-3)
    sample = sample_checkpoint(run_dir, "best", prompt_ids=[1, 2, 3], max_new_tokens=4, top_k=1)
    assert len(sample["generated_ids"]) == 4
    raw["training"]["target_tokens"] = 32 * 4 * 6
    again = run_training(write_toml(raw, tmp_path / "half.toml"), resume=True)
    assert again.steps == 6 and math.isfinite(again.final_loss)
