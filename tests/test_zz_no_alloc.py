"""GPU test of the entry point for callers that cannot allocate device memory.

`ucmr_hamming_topk_static` keeps the scan -> selection scratch in an array inside the library instead of a
caller workspace (an engine whose KV-cache pool owns all free GPU memory has nothing to allocate from).
The test calls it through the C ABI twice in a row, on different inputs, and requires the outputs to be
bit-identical to the ordinary entry point's; the second call also shows that what the first one left in
the shared array does no harm.  It runs last on purpose: it touches nothing the other tests depend on and
must pass both alone in a fresh process and after everything else.
"""
import numpy as np
import pytest

from tests import helpers as H

pytestmark = pytest.mark.gpu


def _outputs(dev, B, Hout, k):
    import torch
    from unified_cache_management_b200 import ops
    z = lambda *s: torch.full(s, -7, dtype=torch.int32, device=dev)  # noqa: E731
    return ops.Retrieval(physical=z(B, Hout, k), logical=z(B, Hout, k), scores=z(B, Hout, k), valid_count=z(B),
                         new_seq_lens=z(B))


def test_static_scratch_matches_workspace_entry_point_twice(cuda_device):
    import torch
    from unified_cache_management_b200 import lib, ops
    dev = cuda_device
    assert lib.load_library().ucmr_static_workspace_capacity() == 4 << 20
    cases = [
        # (seed, B, Hkv, G, W, BS, max_blocks, k, mode, reduce_kvhead, forcing)
        (101, 4, 8, 4, 4, 128, 40, 6, "sum", False, dict(must_select=(0, -2, -1))),
        (202, 3, 4, 1, 4, 16, 70, 9, "min", True, dict(sink_tokens=16, recent_tokens=64)),
    ]
    for seed, B, Hkv, G, W, BS, mb, k, mode, red, forcing in cases:
        case = H.make_paged_case(seed, B, Hkv, G, W, BS, mb)
        args = (H.to_dev_i32(case["codes"], dev), H.to_dev_i32(case["q"], dev),
                H.to_dev_i32(case["block_table"], dev), H.to_dev_i32(case["seq_lens"], dev), k)
        want = ops.hamming_topk(*args, reduce=mode, reduce_kvhead=red, **forcing)
        got = ops.hamming_topk_static(*args, out=_outputs(dev, B, 1 if red else Hkv, k), reduce=mode,
                                      reduce_kvhead=red, **forcing)
        torch.cuda.synchronize()
        for name in ("physical", "logical", "scores", "valid_count", "new_seq_lens"):
            assert torch.equal(getattr(got, name), getattr(want, name)), (seed, name)


def test_static_scratch_rejects_oversized_shapes(cuda_device):
    import torch
    from unified_cache_management_b200 import lib, ops
    dev = cuda_device
    B, Hkv, mb = 8, 8, 32768                       # 8 * 8 * 32768 * 4 B = 8 MiB of scores > 4 MiB
    assert ops.workspace_bytes(B, Hkv, mb) > (4 << 20)
    codes = torch.zeros((4, 16, Hkv, 4), dtype=torch.int32, device=dev)
    q = torch.zeros((B, Hkv, 4), dtype=torch.int32, device=dev)
    bt = torch.zeros((B, mb), dtype=torch.int32, device=dev)
    sl = torch.full((B,), 16, dtype=torch.int32, device=dev)
    with pytest.raises(lib.UcmrError) as err:
        ops.hamming_topk_static(codes, q, bt, sl, 2, out=_outputs(dev, B, Hkv, 2))
    assert err.value.status == lib.UCMR_ERR_WORKSPACE
    assert "workspace" in str(err.value)
