"""Per-request phase tracking for the on-device sparse plugin (host side, no GPU).

The plugin has to know, for every request scheduled in a step, whether the step is the request's first prefill chunk
(where a prefix-cache hit must be re-hashed), a later prefill chunk, or a decode step (where retrieval runs).  vLLM's
scheduler output does not say so directly; the reference derives it from a per-request flag it keeps across steps
(``is_prefill_flag``, ucm/sparse/gsa_on_device/gsa_on_device.py:1259-1380, 1407-1421).  Here the same decisions are a
small state machine with explicit transitions, so that they can be tested without a GPU:

    (unknown) --first chunk--> PREFILL --chunk that reaches the prompt's end--> DECODE --finished / preempted--> (unknown)

A request whose whole prompt fits one chunk goes (unknown) -> DECODE in a single step.  A request resumed after a
preemption is forgotten first and therefore starts again as a first prefill.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from enum import Enum
from typing import Dict, Hashable, Iterable, List, Mapping, Optional, Tuple


class Phase(Enum):
    PREFILL = "prefill"
    DECODE = "decode"


@dataclass(frozen=True)
class StepRole:
    """What one scheduled request does in this step."""
    first_prefill: bool   # the request was unknown before this step
    prefill: bool         # the step computes prompt tokens
    last_chunk: bool      # ... and reaches the end of the prompt: the next step decodes
    decode: bool          # the step decodes (retrieval applies)


@dataclass(frozen=True)
class PrefixLayout:
    """Tokens of a prompt that were NOT computed in the first chunk because a prefix cache (or an external store)
    already held their K/V: they occupy the first ``n_blocks`` blocks of the request, the last of them partly."""
    n_tokens: int
    n_blocks: int
    tail_tokens: int      # valid tokens in the last listed block (== block_size when it is full)

    @property
    def empty(self) -> bool:
        return self.n_tokens <= 0


def prefix_layout(num_prompt_tokens: int, query_len: int, block_size: int) -> PrefixLayout:
    """Layout of the prefix hit of a first prefill chunk that computes ``query_len`` of ``num_prompt_tokens`` tokens."""
    if not 0 <= query_len <= num_prompt_tokens:
        raise ValueError(f"query_len {query_len} outside [0, {num_prompt_tokens}]")
    if block_size <= 0:
        raise ValueError("block_size must be positive")
    n_tokens = num_prompt_tokens - query_len
    if n_tokens <= 0:
        return PrefixLayout(0, 0, 0)
    n_blocks = -(-n_tokens // block_size)
    return PrefixLayout(n_tokens, n_blocks, n_tokens - (n_blocks - 1) * block_size)


@dataclass
class PrefixHit:
    req_id: Hashable
    row: int              # the request's row in the step's batch
    layout: PrefixLayout


@dataclass
class StepPlan:
    """Everything the worker needs to know about a step before the forward pass starts."""
    num_reqs: int = 0
    decode_rows: List[int] = field(default_factory=list)     # batch rows of the decoding requests, in schedule order
    prefix_hits: List[PrefixHit] = field(default_factory=list)
    roles: Dict[Hashable, StepRole] = field(default_factory=dict)

    @property
    def has_decode(self) -> bool:
        return bool(self.decode_rows)

    @property
    def decode_only(self) -> bool:
        return self.has_decode and len(self.decode_rows) == self.num_reqs

    @property
    def total_prefix_tokens(self) -> int:
        return sum(h.layout.n_tokens for h in self.prefix_hits)

    @property
    def total_prefix_blocks(self) -> int:
        return sum(h.layout.n_blocks for h in self.prefix_hits)


class RequestPhaseTracker:
    """Remembers which phase every live request is in and turns a step's schedule into a ``StepPlan``."""

    def __init__(self) -> None:
        self._phase: Dict[Hashable, Phase] = {}

    def __contains__(self, req_id: Hashable) -> bool:
        return req_id in self._phase

    def __len__(self) -> int:
        return len(self._phase)

    def phase_of(self, req_id: Hashable) -> Optional[Phase]:
        return self._phase.get(req_id)

    def forget(self, req_id: Hashable) -> None:
        """The request finished, was aborted, or was preempted (it will come back as a new first prefill)."""
        self._phase.pop(req_id, None)

    def forget_many(self, req_ids: Iterable[Hashable]) -> None:
        for r in req_ids:
            self.forget(r)

    def advance(self, req_id: Hashable, num_computed_tokens: int, num_scheduled_tokens: int,
                num_prompt_tokens: int) -> StepRole:
        """Role of the request in the step being scheduled, and the transition the step causes."""
        before = self._phase.get(req_id)
        if before is Phase.DECODE:
            return StepRole(first_prefill=False, prefill=False, last_chunk=False, decode=True)
        first = before is None
        last = num_computed_tokens + num_scheduled_tokens >= num_prompt_tokens
        self._phase[req_id] = Phase.DECODE if last else Phase.PREFILL
        return StepRole(first_prefill=first, prefill=True, last_chunk=last, decode=False)

    def plan_step(self, num_scheduled_tokens: Mapping[Hashable, int], requests: Mapping[Hashable, object],
                  row_of: Mapping[Hashable, int], query_len_of_row, block_size: int,
                  external_tokens: Optional[Mapping[Hashable, int]] = None) -> StepPlan:
        """``requests[r]`` has ``num_computed_tokens`` and ``num_prompt_tokens``; ``row_of[r]`` is the request's batch
        row; ``query_len_of_row(row)`` the tokens it computes in this step; ``external_tokens[r]`` > 0 marks a prompt
        part of whose K/V came from a prefix cache or an external store."""
        plan = StepPlan(num_reqs=len(num_scheduled_tokens))
        external_tokens = external_tokens or {}
        for req_id, n_sched in num_scheduled_tokens.items():
            req = requests[req_id]
            role = self.advance(req_id, int(req.num_computed_tokens), int(n_sched), int(req.num_prompt_tokens))
            plan.roles[req_id] = role
            if role.decode:
                plan.decode_rows.append(int(row_of[req_id]))
            elif role.first_prefill and int(external_tokens.get(req_id, 0)) > 0:
                row = int(row_of[req_id])
                layout = prefix_layout(int(req.num_prompt_tokens), int(query_len_of_row(row)), block_size)
                if not layout.empty:
                    plan.prefix_hits.append(PrefixHit(req_id, row, layout))
        return plan


def prefix_slots(block_ids: "object", layout: PrefixLayout, block_size: int, token_index: "object"):
    """Slot of every prefix token: ``block_ids`` (tensor, the first ``layout.n_blocks`` entries of the request's
    block-table row) and ``token_index`` (tensor 0..n-1, int64) -> int64 tensor [layout.n_tokens]."""
    idx = token_index[: layout.n_tokens]
    blk = idx // block_size
    return block_ids.index_select(0, blk).to(idx.dtype) * block_size + (idx - blk * block_size)
