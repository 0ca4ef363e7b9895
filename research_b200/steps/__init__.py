"""Train and eval steps, MoE load balancing."""

from research_b200._lazy import lazy_exports

__getattr__, __dir__, __all__ = lazy_exports(__name__, {
    "BatchStager": ("research_b200.steps.train", "BatchStager"),
    "EvalStep": ("research_b200.steps.eval", "EvalStep"),
    "MoeBalanceState": ("research_b200.steps.moe_balance", "MoeBalanceState"),
    "TrainStep": ("research_b200.steps.train", "TrainStep"),
    "apply_moe_balance_update": ("research_b200.steps.moe_balance", "apply_moe_balance_update"),
    "causal_lm_loss": ("research_b200.steps.eval", "causal_lm_loss"),
    "context_positions": ("research_b200.steps.train", "context_positions"),
    "init_moe_balance": ("research_b200.steps.moe_balance", "init_moe_balance"),
    "initialize_moe_balance_state": ("research_b200.steps.moe_balance", "init_moe_balance"),
    "local_batch_slices": ("research_b200.steps.train", "local_batch_slices"),
    "make_eval_step": ("research_b200.steps.eval", "EvalStep"),
    "make_train_step": ("research_b200.steps.train", "TrainStep"),
    "router_diagnostics": ("research_b200.steps.moe_balance", "router_diagnostics"),
})
