"""CPU tests of the plugin's per-request phase tracking (chunked prefill, prefix hits, preemption)."""
from types import SimpleNamespace

import pytest
import torch

from unified_cache_management_b200.request_state import (Phase, RequestPhaseTracker, prefix_layout, prefix_slots)


def _req(prompt, computed):
    return SimpleNamespace(num_prompt_tokens=prompt, num_computed_tokens=computed)


def test_chunked_prefill_then_decode():
    t = RequestPhaseTracker()
    r = t.advance("a", 0, 512, 1300)
    assert (r.first_prefill, r.prefill, r.last_chunk, r.decode) == (True, True, False, False)
    assert t.phase_of("a") is Phase.PREFILL
    r = t.advance("a", 512, 512, 1300)
    assert (r.first_prefill, r.prefill, r.last_chunk, r.decode) == (False, True, False, False)
    r = t.advance("a", 1024, 276, 1300)          # the chunk that reaches the end of the prompt
    assert (r.first_prefill, r.prefill, r.last_chunk, r.decode) == (False, True, True, False)
    assert t.phase_of("a") is Phase.DECODE
    for step in range(3):
        r = t.advance("a", 1300 + step, 1, 1300)
        assert r.decode and not r.prefill


def test_prompt_that_fits_one_chunk_decodes_next_step():
    t = RequestPhaseTracker()
    r = t.advance("a", 0, 100, 100)
    assert r.first_prefill and r.last_chunk and not r.decode
    assert t.advance("a", 100, 1, 100).decode


def test_finished_and_preempted_requests_start_over():
    t = RequestPhaseTracker()
    t.advance("a", 0, 64, 64)
    assert t.advance("a", 64, 1, 64).decode
    t.forget("a")                                  # preempted: resumed later as a fresh prefill of prompt + output
    assert "a" not in t and len(t) == 0
    r = t.advance("a", 0, 70, 70)
    assert r.first_prefill and r.prefill
    t.forget("never seen")                         # harmless


@pytest.mark.parametrize("prompt,qlen,bs,want", [
    (1000, 1000, 128, (0, 0, 0)),                  # nothing cached
    (1000, 488, 128, (512, 4, 128)),               # hit ends on a block boundary
    (1000, 400, 128, (600, 5, 88)),                # hit ends inside the fifth block
    (130, 1, 128, (129, 2, 1)),                    # one token into the second block
    (16, 15, 16, (1, 1, 1)),
])
def test_prefix_layout(prompt, qlen, bs, want):
    lay = prefix_layout(prompt, qlen, bs)
    assert (lay.n_tokens, lay.n_blocks, lay.tail_tokens) == want
    assert lay.empty == (want[0] == 0)


def test_prefix_layout_rejects_bad_lengths():
    with pytest.raises(ValueError):
        prefix_layout(10, 11, 16)
    with pytest.raises(ValueError):
        prefix_layout(10, -1, 16)


def test_prefix_slots_follow_the_block_table():
    bs = 16
    lay = prefix_layout(100, 50, bs)               # 50 cached tokens: 3 full blocks + 2 tokens
    assert (lay.n_blocks, lay.tail_tokens) == (4, 2)
    row = torch.tensor([7, 3, 9, 1, 55, 66], dtype=torch.int32)
    slots = prefix_slots(row[: lay.n_blocks], lay, bs, torch.arange(4096, dtype=torch.int64))
    want = [int(row[p // bs]) * bs + p % bs for p in range(50)]
    assert slots.tolist() == want and slots.dtype == torch.int64


def test_plan_step_mixed_batch():
    """One step with a decoding request, a later prefill chunk, a first prefill with a prefix hit that ends inside a
    block, a first prefill without a hit, and a request resumed after preemption."""
    t = RequestPhaseTracker()
    bs = 128
    # history: d decodes, c is in the middle of its prompt, p was decoding and got preempted
    t.advance("d", 0, 300, 300)
    t.advance("c", 0, 256, 1000)
    t.advance("p", 0, 200, 200)
    t.forget("p")
    requests = {"d": _req(300, 310), "c": _req(1000, 256), "h": _req(1000, 600), "n": _req(64, 0), "p": _req(205, 0)}
    sched = {"d": 1, "c": 256, "h": 400, "n": 64, "p": 205}
    rows = {"d": 0, "c": 1, "h": 2, "n": 3, "p": 4}
    qlens = {0: 1, 1: 256, 2: 400, 3: 64, 4: 205}
    plan = t.plan_step(sched, requests, rows, lambda r: qlens[r], bs, external_tokens={"h": 600, "c": 0})
    assert plan.num_reqs == 5 and plan.decode_rows == [0] and plan.has_decode and not plan.decode_only
    assert [h.req_id for h in plan.prefix_hits] == ["h"]
    lay = plan.prefix_hits[0].layout
    assert (lay.n_tokens, lay.n_blocks, lay.tail_tokens) == (600, 5, 88)
    assert plan.total_prefix_tokens == 600 and plan.total_prefix_blocks == 5
    assert plan.roles["p"].first_prefill and plan.roles["p"].last_chunk      # resumed: starts over
    assert plan.roles["c"].prefill and not plan.roles["c"].first_prefill and not plan.roles["c"].last_chunk
    assert t.phase_of("h") is Phase.DECODE and t.phase_of("n") is Phase.DECODE and t.phase_of("c") is Phase.PREFILL
    # next step: everyone but c decodes
    sched2 = {"d": 1, "h": 1, "n": 1, "p": 1}
    plan2 = t.plan_step(sched2, requests, rows, lambda r: 1, bs)
    assert plan2.decode_only and plan2.decode_rows == [0, 2, 3, 4] and not plan2.prefix_hits
