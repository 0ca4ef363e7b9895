"""Inference: checkpoint restore for evaluation and sampling, paged KV cache, prefill, decode, sampling."""

from research_b200._lazy import lazy_exports

__getattr__, __dir__, __all__ = lazy_exports(__name__, {
    "GenerationResult": ("research_b200.infer.generation", "GenerationResult"),
    "GraphedDecodeStep": ("research_b200.infer.generation", "GraphedDecodeStep"),
    "InferenceCheckpoint": ("research_b200.infer.checkpoint", "InferenceCheckpoint"),
    "InferenceRestore": ("research_b200.infer.checkpoint", "InferenceCheckpoint"),
    "KVCache": ("research_b200.infer.generation", "PagedKVCache"),
    "PagedKVCache": ("research_b200.infer.generation", "PagedKVCache"),
    "decode_one": ("research_b200.infer.generation", "decode_one"),
    "generate_tokens": ("research_b200.infer.generation", "generate_tokens"),
    "init_kv_cache": ("research_b200.infer.generation", "init_kv_cache"),
    "load_run_spec": ("research_b200.infer.checkpoint", "load_run_spec"),
    "make_decode_step": ("research_b200.infer.generation", "GraphedDecodeStep"),
    "prefill": ("research_b200.infer.generation", "prefill"),
    "restore_inference_checkpoint": ("research_b200.infer.checkpoint", "restore_inference_checkpoint"),
    "sample_next_token": ("research_b200.infer.generation", "sample_next_token"),
    "select_checkpoint": ("research_b200.infer.checkpoint", "select_checkpoint"),
})
