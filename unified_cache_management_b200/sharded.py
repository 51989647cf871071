"""Sequence-sharded retrieval for very long contexts: every rank scans its contiguous range of
logical blocks, emits its best k blocks as (score, global id) records, one all-gather brings the
records of all ranks into each GPU's own memory, and a merge kernel picks the global top-k.

The reference plugin has no context-parallel retrieval; the per-shard computation is the same scan
and selection as the unsharded path, and the result is identical to it (any member of the global
top-k is in its shard's local top-k; forced blocks carry score -1 so they survive the merge).

The collective is `torch.distributed.all_gather_into_tensor` (NCCL on GPUs): one message of
`B*Hout*k*8` bytes per rank, latency-bound.  The compute functions are parameters so that the plumbing
can be exercised with CPU ranks.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional, Sequence

import torch
import torch.distributed as dist


@dataclass
class ShardPlan:
    block_offset: int            # first logical block this rank holds
    blocks_per_rank: int
    seq_lens_local: torch.Tensor  # int32 [B]: tokens of each request inside this rank's range


def shard_plan(seq_lens_global: torch.Tensor, block_size: int, max_blocks_global: int, world: int, rank: int) -> ShardPlan:
    """Contiguous split of the logical block range [0, max_blocks_global) into `world` equal parts."""
    if max_blocks_global % world != 0:
        raise ValueError("max_blocks_global must be a multiple of the world size")
    per = max_blocks_global // world
    off = rank * per
    local = (seq_lens_global.to(torch.int64) - off * block_size).clamp(min=0, max=per * block_size).to(torch.int32)
    return ShardPlan(block_offset=off, blocks_per_rank=per, seq_lens_local=local)


def _default_candidates(*args, **kw):
    from . import ops
    return ops.topk_candidates(*args, **kw)


def _default_merge(*args, **kw):
    from . import ops
    return ops.merge_topk(*args, **kw)


def sharded_hamming_topk(codes_local, q_codes, block_table_local, seq_lens_global, k: int, block_size: int,
                         max_blocks_global: int, score_scale: float, *, group=None, reduce="sum",
                         reduce_kvhead: bool = False, must_select: Sequence[int] = (), sink_tokens: int = 0,
                         recent_tokens: int = 0, workspace=None, gather_buffer: Optional[torch.Tensor] = None,
                         send_buffer: Optional[torch.Tensor] = None, plan: Optional[ShardPlan] = None,
                         inputs_stable: bool = False, cache_append_only: bool = False, out_scores=None,
                         out_ids=None,
                         candidates_fn: Callable = _default_candidates, merge_fn: Callable = _default_merge):
    """Returns (scores float32 [B,Hout,k], global logical block ids int32 [B,Hout,k]), identical on
    every rank.  block_table_local is this rank's slice [B, max_blocks_global/world] of the table.
    ``send_buffer`` (int32 [2, B, Hout, min(k, blocks per rank)]) lets the local selection write its records
    straight into the message; ``gather_buffer`` (int32 [world*2, ...]) receives all ranks' messages; ``plan`` is
    a ``shard_plan`` result to reuse while the sequence lengths do not change; ``out_scores`` / ``out_ids`` receive
    the merged result."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    if plan is None:
        plan = shard_plan(seq_lens_global, block_size, max_blocks_global, world, rank)
    kl = min(k, plan.blocks_per_rank)
    extra = {}
    if candidates_fn is _default_candidates:
        extra["inputs_stable"] = inputs_stable
        extra["cache_append_only"] = cache_append_only
    direct = send_buffer is not None and candidates_fn is _default_candidates
    if direct:
        extra.update(out_scores=send_buffer[0].view(torch.float32), out_ids=send_buffer[1])
    sc, ids = candidates_fn(codes_local, q_codes, block_table_local, plan.seq_lens_local, seq_lens_global, kl,
                            plan.block_offset, score_scale, reduce=reduce, reduce_kvhead=reduce_kvhead,
                            must_select=must_select, sink_tokens=sink_tokens, recent_tokens=recent_tokens,
                            workspace=workspace, **extra)
    # one message per rank: [2, B, H, kl] int32 (float bits, then ids)
    send = send_buffer if direct else torch.stack((sc.view(torch.int32), ids))
    if gather_buffer is None:
        gather_buffer = torch.empty((world * 2,) + tuple(send.shape[1:]), dtype=torch.int32, device=send.device)
    dist.all_gather_into_tensor(gather_buffer, send, group=group)   # concatenation along dim 0
    gathered = gather_buffer.view((world, 2) + tuple(send.shape[1:]))
    cand_scores = gathered[:, 0].view(torch.float32)
    cand_ids = gathered[:, 1]
    if merge_fn is _default_merge:
        return merge_fn(cand_scores, cand_ids, k, out_scores=out_scores, out_ids=out_ids)
    return merge_fn(cand_scores, cand_ids, k)


def exchange_layout(world: int, rank: int, slab: int, seq: int):
    """Word offsets inside one rank's exchange buffer for step ``seq``: two parities, each
    [scores: world*slab | ids: world*slab | flags: world (padded to 64)].  Returns (scores_off, ids_off, flags_off,
    my_slice_off, words_per_parity): where a rank's records start and where THIS rank's slice and flag sit."""
    words = 2 * world * slab + 64
    base = (seq & 1) * words
    return base, base + world * slab, base + 2 * world * slab, rank * slab, words


class PeerExchange:
    """Gather buffers of all ranks mapped into each other's address space (torch symmetric memory), for the
    collective-free form of the sharded retrieval: every rank's selection kernel stores its records into all
    ranks' buffers over NVLink and publishes the step number; the merge kernel waits for all step numbers.

    Per rank and per step parity: scores float32 [world, B, H, kl], ids int32 [world, B, H, kl], flags int32 [world]
    (padded to 64 words).  Two parities alternate so that a rank that is one step ahead never overwrites records a
    slower rank still merges.  The step number is kept on the device (``state``: step word, arrival counter): both
    kernels read it there and the merge advances it, so a step captured in a CUDA graph stays correct when replayed."""

    def __init__(self, batch: int, heads: int, kl: int, device, group=None):
        import torch.distributed._symmetric_memory as symm_mem
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        if self.world > 8:
            raise ValueError("the peer exchange serves up to 8 ranks of one NVLink domain")
        self.shape = (self.world, batch, heads, kl)
        self.slab = batch * heads * kl                      # records of one rank
        self.words_per_parity = exchange_layout(self.world, self.rank, self.slab, 0)[4]
        self.buf = symm_mem.empty(2 * self.words_per_parity, dtype=torch.int32, device=device)
        self.buf.zero_()
        self.state = torch.zeros(2, dtype=torch.int32, device=device)   # step word, merge arrival counter
        self.handle = symm_mem.rendezvous(self.buf, self.group)
        self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
        torch.cuda.synchronize(device)
        dist.barrier(self.group)                            # every rank's flags are zero before any store
        self.seq = 0
        # pointer lists for the step forms: parity 0's ranks, then parity 1's
        self.step_ptrs = ([], [], [])
        for par in (0, 1):
            o_s, o_i, o_f, mine, _ = exchange_layout(self.world, self.rank, self.slab, par)
            self.step_ptrs[0].extend(p + 4 * (o_s + mine) for p in self.ptrs)
            self.step_ptrs[1].extend(p + 4 * (o_i + mine) for p in self.ptrs)
            self.step_ptrs[2].extend(p + 4 * (o_f + self.rank) for p in self.ptrs)

    def views(self, parity: int):
        """Local views (scores [world,B,H,kl] float32, ids, flags [world]) of one buffer parity."""
        o_s, o_i, o_f, _, _ = exchange_layout(self.world, self.rank, self.slab, parity)
        n = self.world * self.slab
        return (self.buf[o_s:o_s + n].view(torch.float32).view(self.shape), self.buf[o_i:o_i + n].view(self.shape),
                self.buf[o_f:o_f + self.world])

    def next_step(self):
        """By-value stepping with a host-side count (NOT for captured launches, and not to be mixed with the
        device-counted form on the same exchange): returns (seq, pointer lists for topk_candidates_p2p, local views
        for merge_topk_wait)."""
        self.seq += 1
        o_s, o_i, o_f, mine, _ = exchange_layout(self.world, self.rank, self.slab, self.seq)
        ps = [p + 4 * (o_s + mine) for p in self.ptrs]
        pi = [p + 4 * (o_i + mine) for p in self.ptrs]
        pf = [p + 4 * (o_f + self.rank) for p in self.ptrs]
        return self.seq, (ps, pi, pf), self.views(self.seq & 1)


def sharded_hamming_topk_p2p(codes_local, q_codes, block_table_local, seq_lens_global, k: int, block_size: int,
                             max_blocks_global: int, score_scale: float, exchange: PeerExchange, *, reduce="sum",
                             reduce_kvhead: bool = False, must_select: Sequence[int] = (), sink_tokens: int = 0,
                             recent_tokens: int = 0, workspace=None, plan: Optional[ShardPlan] = None,
                             status: Optional[torch.Tensor] = None, inputs_stable: bool = False,
                             cache_append_only: bool = False,
                             out_scores=None, out_ids=None):
    """``sharded_hamming_topk`` with the all-gather folded into the two kernels (see ``PeerExchange``): two launches
    per step and no collective call.  The step number is counted on the device, so the call may be captured in a
    CUDA graph and replayed (every rank must replay the same number of steps)."""
    from . import ops
    if plan is None:
        plan = shard_plan(seq_lens_global, block_size, max_blocks_global, exchange.world, exchange.rank)
    kl = min(k, plan.blocks_per_rank)
    if kl != exchange.shape[3]:
        raise ValueError("the exchange was sized for a different number of records per rank")
    ps, pi, pf = exchange.step_ptrs
    ops.topk_candidates_p2p_step(codes_local, q_codes, block_table_local, plan.seq_lens_local, seq_lens_global, kl,
                                 plan.block_offset, score_scale, ps, pi, pf, exchange.state[0:1], reduce=reduce,
                                 reduce_kvhead=reduce_kvhead, must_select=must_select, sink_tokens=sink_tokens,
                                 recent_tokens=recent_tokens, workspace=workspace, inputs_stable=inputs_stable,
                                 cache_append_only=cache_append_only)
    scores, ids, flags = exchange.views(0)
    return ops.merge_topk_wait_step(scores, ids, k, flags, exchange.words_per_parity, exchange.words_per_parity,
                                    exchange.state, status=status, out_scores=out_scores, out_ids=out_ids)
