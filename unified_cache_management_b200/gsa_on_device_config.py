"""Plugin configuration with the reference's keys.

Same fields and JSON format as ``GSAOnDeviceConfig``
(``ucm/sparse/gsa_on_device/gsa_on_device_config.py:36-285``) so existing per-model JSON files load
unchanged.  Keys the reference declares but never reads are honoured here with their documented
meaning: ``must_select_blocks`` (forced blocks), ``chunk_repre_method`` (block reduce: "max"
similarity = "min" distance, or "sum"), ``hash_bits``.  ESA/KVStar-style spellings are accepted by
``apply_overrides``.
"""
from __future__ import annotations

import json
from dataclasses import asdict, dataclass, field, fields
from typing import Any, Dict, List, Optional

_REPRE = ("max", "min", "sum")


@dataclass
class GSAOnDeviceConfig:
    model_name: str = "DummyModel"
    is_mla: bool = False
    hash_weight_type: str = "random"  # "random" or "fixed"
    num_hidden_layers: int = 36
    gpu_seq_len_threshold: int = 2048      # minimal seq_len to trigger retrieval
    gpu_concurrency_threshold: int = 4     # minimal number of long requests to trigger retrieval
    npu_seq_len_threshold: int = 2048
    npu_concurrency_threshold: int = 4
    chunk_size: int = 128
    chunk_repre_method: str = "max"
    head_dim: int = 128
    hash_bits: int = 128
    top_k_ratio_per_layer: List[float] = field(default_factory=lambda: [0.3] * 36)
    top_k_index_reuse: List[int] = field(default_factory=lambda: [-1] * 36)
    must_select_blocks: List[int] = field(default_factory=lambda: [0, -2, -1])
    hash_weight: Optional[List[List[float]]] = None
    kv_lora_rank: Optional[int] = None
    qk_rope_head_dim: Optional[int] = None
    hash_bits_kv_lora: Optional[int] = None
    hash_bits_qk_rope: Optional[int] = None
    hash_weight_kv_lora: Optional[List[List[float]]] = None
    hash_weight_qk_rope: Optional[List[List[float]]] = None
    vllm_hash_attention_topk: Optional[int] = None
    vllm_hash_attention_reduction_head_num: Optional[int] = None
    vllm_hash_attention_rollback_layers: List[int] = field(default_factory=list)
    vllm_hash_attention_skip_layers: List[bool] = field(default_factory=list)

    # ---- validation helpers shared by the two generators -------------------------------------
    def _common(self, model_name, hash_weight_type, num_hidden_layers, seq_len_threshold, chunk_size,
                chunk_repre_method, top_k_ratio_per_layer, top_k_index_reuse, must_select_blocks):
        if hash_weight_type not in ("random", "fixed"):
            raise ValueError(f"hash_weight_type should be either 'random' or 'fixed', but got {hash_weight_type}")
        if chunk_size % 128 != 0:
            raise ValueError(f"chunk_size should be divisible by 128, but got {chunk_size}")
        if chunk_repre_method not in _REPRE:
            raise ValueError(f"chunk_repre_method should be either 'max', 'min' or 'sum', but got {chunk_repre_method}")
        if len(top_k_ratio_per_layer) != num_hidden_layers:
            raise ValueError(f"top_k_ratio_per_layer length should be equal to num_hidden_layers={num_hidden_layers}, "
                             f"but got {len(top_k_ratio_per_layer)}")
        if len(top_k_index_reuse) != num_hidden_layers:
            raise ValueError(f"top_k_index_reuse length should be equal to num_hidden_layers={num_hidden_layers}, "
                             f"but got {len(top_k_index_reuse)}")
        self.model_name = model_name
        self.hash_weight_type = hash_weight_type
        self.num_hidden_layers = num_hidden_layers
        self.seq_len_threshold = seq_len_threshold
        self.chunk_size = chunk_size
        self.chunk_repre_method = chunk_repre_method
        self.top_k_ratio_per_layer = top_k_ratio_per_layer
        self.top_k_index_reuse = top_k_index_reuse
        self.must_select_blocks = must_select_blocks

    def generate_config_data(self, model_name, hash_weight_type, num_hidden_layers, seq_len_threshold, chunk_size,
                             chunk_repre_method, head_dim, hash_bits, top_k_ratio_per_layer, top_k_index_reuse,
                             must_select_blocks) -> None:
        self._common(model_name, hash_weight_type, num_hidden_layers, seq_len_threshold, chunk_size,
                     chunk_repre_method, top_k_ratio_per_layer, top_k_index_reuse, must_select_blocks)
        self.is_mla = False
        self.head_dim = head_dim
        self.hash_bits = hash_bits
        if hash_weight_type == "random":
            self.hash_weight = None

    def generate_mla_config_data(self, model_name, hash_weight_type, num_hidden_layers, seq_len_threshold,
                                 chunk_size, chunk_repre_method, kv_lora_rank, qk_rope_head_dim, hash_bits_kv_lora,
                                 hash_bits_qk_rope, top_k_ratio_per_layer, top_k_index_reuse,
                                 must_select_blocks) -> None:
        self._common(model_name, hash_weight_type, num_hidden_layers, seq_len_threshold, chunk_size,
                     chunk_repre_method, top_k_ratio_per_layer, top_k_index_reuse, must_select_blocks)
        self.is_mla = True
        self.head_dim = qk_rope_head_dim + kv_lora_rank
        self.hash_bits = hash_bits_qk_rope + hash_bits_kv_lora
        self.kv_lora_rank = kv_lora_rank
        self.qk_rope_head_dim = qk_rope_head_dim
        self.hash_bits_kv_lora = hash_bits_kv_lora
        self.hash_bits_qk_rope = hash_bits_qk_rope
        if hash_weight_type == "random":
            self.hash_weight = self.hash_weight_kv_lora = self.hash_weight_qk_rope = None

    def set_hash_weight(self, hash_weight: List[List[float]]) -> None:
        if self.hash_weight_type != "fixed":
            raise ValueError("hash_weight can only be set when hash_weight_type is 'fixed'")
        if len(hash_weight) != self.head_dim or len(hash_weight[0]) != self.hash_bits:
            raise ValueError(f"hash_weight shape should be ({self.head_dim}, {self.hash_bits}), "
                             f"but got ({len(hash_weight)}, {len(hash_weight[0])})")
        self.hash_weight = hash_weight

    def set_mla_hash_weight(self, hash_weight_kv_lora, hash_weight_qk_rope) -> None:
        if self.hash_weight_type != "fixed":
            raise ValueError("hash_weight can only be set when hash_weight_type is 'fixed'")
        if len(hash_weight_kv_lora) != self.kv_lora_rank or len(hash_weight_kv_lora[0]) != self.hash_bits_kv_lora:
            raise ValueError(f"hash_weight_kv_lora shape should be ({self.kv_lora_rank}, {self.hash_bits_kv_lora})")
        if len(hash_weight_qk_rope) != self.qk_rope_head_dim or len(hash_weight_qk_rope[0]) != self.hash_bits_qk_rope:
            raise ValueError(f"hash_weight_qk_rope shape should be ({self.qk_rope_head_dim}, {self.hash_bits_qk_rope})")
        self.hash_weight_kv_lora = hash_weight_kv_lora
        self.hash_weight_qk_rope = hash_weight_qk_rope

    # ---- derived settings used by the retrieval calls -------------------------------------------
    @property
    def reduce(self) -> str:
        """Block reduce for the kernels: max similarity = min distance."""
        return "sum" if self.chunk_repre_method == "sum" else "min"

    def apply_overrides(self, extra: Dict[str, Any], block_size: int) -> None:
        """Inline keys of ``ucm_sparse_config`` (ESA/KVStar spellings included)."""
        names = {f.name for f in fields(self)}
        for k, v in extra.items():
            if k in names:
                setattr(self, k, v)
        init_w, local_w = extra.get("init_window_sz"), extra.get("local_window_sz")
        if init_w is not None or local_w is not None:
            self.must_select_blocks = list(range(int(init_w or 0))) + [-(i + 1) for i in range(int(local_w or 0))][::-1]
        if self.chunk_repre_method not in _REPRE:
            raise ValueError(f"chunk_repre_method should be either 'max', 'min' or 'sum', but got {self.chunk_repre_method}")

    def to_json(self, file_path: str) -> None:
        with open(file_path, "w") as f:
            json.dump(asdict(self), f, indent=4)

    @classmethod
    def from_json(cls, file_path: str) -> "GSAOnDeviceConfig":
        with open(file_path, "r") as f:
            return cls(**json.load(f))
