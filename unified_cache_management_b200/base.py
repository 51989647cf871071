"""The sparse-plugin hook interface.

When the reference package is installed, ``UcmSparseBase`` / ``UcmSparseRole`` / ``INVALID_SLOT`` are
the reference's own objects (``ucm/sparse/base.py:36-322``), so the plugin in this package is a true
subclass for its factory and trampolines.  Otherwise a stand-in with the same hook names, argument
lists and default return values is defined here, so that the plugin can be driven without vLLM.
Nothing is imported from vLLM at module scope.
"""
from __future__ import annotations

import enum
from abc import ABC, abstractmethod
from typing import List, Optional, Tuple, Union

import torch

try:  # pragma: no cover - depends on the environment
    from ucm.sparse.base import (INVALID_SLOT, UcmSparseBase, UcmSparseCpuGpuBuffer, UcmSparseMetadata,
                                 UcmSparseRole)
    HAVE_REFERENCE_BASE = True
except Exception:  # noqa: BLE001 - any import problem means "not installed here"
    HAVE_REFERENCE_BASE = False
    INVALID_SLOT = -1

    class UcmSparseRole(enum.Enum):
        SCHEDULER = 0
        WORKER = 1

    class UcmSparseMetadata(ABC):  # noqa: B024
        """Metadata passed from the scheduler-side instance to the worker-side instance."""

    class UcmSparseCpuGpuBuffer:
        """A pinned host tensor with a device twin and explicit copies in both directions."""

        def __init__(self, *size, dtype: torch.dtype, device: torch.device, pin_memory: bool = True,
                     with_numpy: bool = True) -> None:
            pin = pin_memory and torch.cuda.is_available()
            self.cpu = torch.zeros(*size, dtype=dtype, device="cpu", pin_memory=pin)
            self.gpu = self.cpu.to(device)
            self.n = 0
            if with_numpy:
                if dtype == torch.bfloat16:
                    raise ValueError("bfloat16 tensors have no numpy view; pass with_numpy=False")
                self.np = self.cpu.numpy()

        def copy_to_gpu(self, n: Optional[int] = None) -> None:
            n = self.n if n is None else n
            if n > 0:
                self.gpu[:n].copy_(self.cpu[:n], non_blocking=True)

        def copy_to_cpu(self, n: Optional[int] = None) -> None:
            n = self.n if n is None else n
            if n > 0:
                self.cpu[:n].copy_(self.gpu[:n], non_blocking=True)

        def clear(self) -> None:
            self.n = 0

    class UcmSparseBase(ABC):
        """Hook ABI of a sparse-attention method (worker-side and scheduler-side)."""

        def __init__(self, vllm_config, role: UcmSparseRole):
            self._sparse_metadata: Optional[UcmSparseMetadata] = None
            self._vllm_config = vllm_config
            self._role = role

        @property
        def role(self) -> UcmSparseRole:
            return self._role

        # ---- worker side -----------------------------------------------------------------------
        def bind_sparse_metadata(self, sparse_metadata) -> None:
            self._sparse_metadata = sparse_metadata

        def clear_sparse_metadata(self) -> None:
            self._sparse_metadata = None

        def _get_sparse_metadata(self):
            return self._sparse_metadata

        def register_kv_caches(self, kv_caches):
            pass

        def execute_begin(self, scheduler_output):
            pass

        def execute_finished(self, logits_indices: torch.Tensor) -> torch.Tensor:
            return logits_indices

        def attention_begin(self, query, key, value, layer_name, forward_context, output=None, phase=None,
                            k_hash=None, decode_ql_nope=None, decode_q_pe=None) -> Tuple:
            return query, key, value, output

        def attention_finished(self, query, key, value, attn_output, layer_name, forward_context, phase=None) -> None:
            pass

        def update_states(self, scheduler_output) -> None:
            pass

        def ffn_begin(self, hidden_states, residual):
            return hidden_states, residual

        def ffn_finished(self, hidden_states, residual):
            return hidden_states, residual

        def layer_begin(self, positions, hidden_states, residual):
            return positions, hidden_states, residual

        def layer_finished(self, positions, hidden_states, residual):
            return positions, hidden_states, residual

        def request_finished_in_worker(self, request_id: Union[int, str]):
            pass

        # ---- scheduler side ----------------------------------------------------------------------
        @abstractmethod
        def request_begin(self, request_id: Union[int, str], prompt_token_ids: List[int]):
            raise NotImplementedError

        def request_finished_in_scheduler(self, request_id: Union[int, str]):
            pass

        def estimate_num_slots_sparsed(self, request) -> int:
            return INVALID_SLOT

        def update_state_after_alloc(self, request, num_blocks: int):
            pass

        def build_sparse_meta(self, scheduler_output, requests, input_batch, attn_metadata):
            pass

        def allocate_slots(self, kv_cache_manager, request, num_slots_sparsed):
            pass
