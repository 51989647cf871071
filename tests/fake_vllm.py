"""Minimal stand-ins for the vLLM objects the plugin touches (no vLLM import)."""
from __future__ import annotations

from types import SimpleNamespace


def make_vllm_config(model="meta-llama/Meta-Llama-3-8B", num_q_heads=32, num_kv_heads=8, head_size=128, block_size=128,
                     max_model_len=8192, max_num_seqs=8, rank=0, overrides=None, dtype=None, device_type="cuda",
                     mla=False, enforce_eager=True):
    import torch
    model_config = SimpleNamespace(
        model=model, is_deepseek_mla=mla, max_model_len=max_model_len, dtype=dtype or torch.bfloat16,
        enforce_eager=enforce_eager, get_num_attention_heads=lambda pc: num_q_heads,
        get_num_kv_heads=lambda pc: num_kv_heads, get_head_size=lambda: head_size,
        hf_text_config=SimpleNamespace(kv_lora_rank=512, qk_rope_head_dim=64) if mla else SimpleNamespace())
    extra = {"ucm_sparse_config": {"GSAOnDevice": dict(overrides or {})}}
    return SimpleNamespace(
        model_config=model_config, parallel_config=SimpleNamespace(rank=rank),
        device_config=SimpleNamespace(device_type=device_type), cache_config=SimpleNamespace(block_size=block_size),
        scheduler_config=SimpleNamespace(max_num_seqs=max_num_seqs),
        kv_transfer_config=SimpleNamespace(kv_connector_extra_config=extra))


class FakeRequest(SimpleNamespace):
    pass


def scheduler_output(num_scheduled_tokens, finished=(), resumed=()):
    return SimpleNamespace(num_scheduled_tokens=dict(num_scheduled_tokens), finished_req_ids=set(finished),
                           num_external_computed_tokens_per_req={},
                           scheduled_cached_reqs=SimpleNamespace(req_ids=[r for r, _ in resumed],
                                                                 resumed_from_preemption=[f for _, f in resumed]))
