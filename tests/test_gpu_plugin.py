"""GPU test of the GSAOnDevice plugin driven the way the patched vLLM drives it:
build_sparse_meta -> attention_begin (per layer) -> attention_finished -> execute_finished."""
from types import SimpleNamespace

import numpy as np
import pytest

from oracle import oracle as O
from tests import fake_vllm as F
from tests import helpers as H

pytestmark = pytest.mark.gpu


def _bf16_bits(t):
    import torch
    return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def test_prefill_then_decode_rewrites_and_restores_block_table(cuda_device):
    import torch
    from unified_cache_management_b200.base import UcmSparseRole
    from unified_cache_management_b200.gsa_on_device import GSAOnDevice
    dev = cuda_device
    BS, Hq, Hkv, D = 16, 8, 2, 128
    topk_tokens = 8 * BS
    cfg = F.make_vllm_config(block_size=BS, num_q_heads=Hq, num_kv_heads=Hkv, max_model_len=64 * BS, max_num_seqs=4,
                             overrides=dict(vllm_hash_attention_topk=topk_tokens, gpu_seq_len_threshold=topk_tokens,
                                            gpu_concurrency_threshold=2, vllm_hash_attention_rollback_layers=[0],
                                            vllm_hash_attention_skip_layers=[False, False, True]))
    plugin = GSAOnDevice(cfg, UcmSparseRole.WORKER)
    assert plugin.estimate_num_slots_sparsed(None) == -1

    n_req, NB, mb = 3, 200, 64
    lens = [40 * BS + 3, 25 * BS, 9 * BS + 1]
    rng = np.random.default_rng(0)
    perm = rng.permutation(NB)
    bt = np.zeros((n_req, mb), dtype=np.int32)
    off = 0
    for b, ln in enumerate(lens):
        n = -(-(ln + 1) // BS)
        bt[b, :n] = perm[off:off + n]
        off += n
    kv_caches = {f"model.layers.{i}.self_attn.attn": torch.zeros((2, NB, BS, Hkv, D), dtype=torch.bfloat16, device=dev)
                 for i in range(3)}
    plugin.initialize_kv_hash_cache_tensors(kv_caches, dev)
    assert kv_caches["model.layers.0.self_attn.attn"][1] is None            # rollback layer: no code cache
    k_hash = kv_caches["model.layers.1.self_attn.attn"][1]
    assert k_hash.shape == (NB, BS, Hkv, D // 16) and k_hash.dtype == torch.bfloat16

    requests = {f"r{b}": F.FakeRequest(num_computed_tokens=0, num_prompt_tokens=lens[b]) for b in range(n_req)}
    input_batch = SimpleNamespace(req_id_to_index={f"r{b}": b for b in range(n_req)})
    layer = "model.layers.1.self_attn.attn"

    # ---- step 1: prefill of all three prompts -------------------------------------------------------
    keys = [H.bf16_normal(rng, (ln, Hkv, D)) for ln in lens]
    key_all = torch.cat([H.bf16_to_dev(k, dev) for k in keys])
    slots = np.concatenate([bt[b, np.arange(ln) // BS].astype(np.int64) * BS + np.arange(ln) % BS
                            for b, ln in enumerate(lens)])
    qsl = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    meta = SimpleNamespace(seq_lens=torch.tensor(lens, dtype=torch.int32, device=dev),
                           block_table=torch.from_numpy(bt).to(dev), slot_mapping=torch.from_numpy(slots).to(dev),
                           query_start_loc=torch.from_numpy(qsl).to(dev))
    fc = SimpleNamespace(attn_metadata={layer: meta}, no_compile_layers={}, virtual_engine=0)
    so = F.scheduler_output({f"r{b}": lens[b] for b in range(n_req)})
    plugin.update_states(so)
    plugin.build_sparse_meta(so, requests, input_batch, {layer: meta})
    assert plugin.gsa_enabled and not plugin.has_decode                      # long enough, but no decode yet
    q_dummy = torch.zeros((sum(lens), Hq, D), dtype=torch.bfloat16, device=dev)
    plugin.attention_begin(q_dummy, key_all, key_all, layer, fc, k_hash=k_hash)
    plugin.attention_finished(q_dummy, key_all, key_all, None, layer, fc)
    plugin.execute_finished(None)
    torch.cuda.synchronize()
    r_bits = _bf16_bits(plugin.hash_encoder.hash_weights_bf16)
    codes_dev = k_hash.view(torch.int32).cpu().numpy().view(np.uint32)       # [NB,BS,Hkv,4]
    for b, ln in enumerate(lens):
        want, p64 = O.hash_encode(keys[b], r_bits)
        got = codes_dev.reshape(NB * BS, Hkv, 4)[slots[qsl[b]:qsl[b + 1]]]
        hard, soft = O.count_code_mismatches(got, p64)
        assert hard == 0

    # ---- step 2: decode of all three (one new token each) --------------------------------------------
    for r in requests.values():
        r.num_computed_tokens = r.num_prompt_tokens
    new_lens = [ln + 1 for ln in lens]
    new_keys = H.bf16_normal(rng, (n_req, Hkv, D))
    new_slots = np.array([bt[b, lens[b] // BS].astype(np.int64) * BS + lens[b] % BS for b in range(n_req)])
    q_bits = H.bf16_normal(rng, (n_req, Hq, D))
    bt_dev = torch.from_numpy(bt).to(dev)
    meta = SimpleNamespace(seq_lens=torch.tensor(new_lens, dtype=torch.int32, device=dev), block_table=bt_dev,
                           slot_mapping=torch.from_numpy(new_slots).to(dev),
                           query_start_loc=torch.arange(n_req + 1, dtype=torch.int32, device=dev))
    fc = SimpleNamespace(attn_metadata={layer: meta}, no_compile_layers={}, virtual_engine=0)
    so = F.scheduler_output({f"r{b}": 1 for b in range(n_req)})
    plugin.build_sparse_meta(so, requests, input_batch, {layer: meta})
    assert plugin.gsa_enabled and plugin.has_decode and plugin.decode_only
    kd = H.bf16_to_dev(new_keys, dev)
    plugin.attention_begin(H.bf16_to_dev(q_bits, dev), kd, kd, layer, fc, k_hash=k_hash)
    torch.cuda.synchronize()
    k = topk_tokens // BS
    sel = meta.block_table[:, :k].cpu().numpy()
    assert (meta.block_table[:, k:] == 0).all()
    new_seq = meta.seq_lens.cpu().numpy()

    # oracle on the cache contents as the device holds them now
    codes_now = k_hash.view(torch.int32).cpu().numpy().view(np.uint32)
    qm = O.group_mean_bf16(q_bits, Hkv)
    q_codes, _ = O.hash_encode(qm, r_bits)
    ref = O.hamming_topk(codes_now, q_codes, bt, np.array(new_lens), k, O.REDUCE_MIN, True, sink_tokens=BS,
                         recent_tokens=4 * BS)
    assert np.array_equal(sel, ref["physical"][:, 0, :])
    assert np.array_equal(new_seq, O.update_seq_lens(np.array(new_lens), topk_tokens, BS))

    # skip layer reuses the selection; attention_finished restores the original table and lengths
    layer2 = "model.layers.2.self_attn.attn"
    meta2 = SimpleNamespace(seq_lens=meta.seq_lens, block_table=meta.block_table, slot_mapping=meta.slot_mapping,
                            query_start_loc=meta.query_start_loc)
    fc2 = SimpleNamespace(attn_metadata={layer2: meta2}, no_compile_layers={}, virtual_engine=0)
    plugin.attention_begin(H.bf16_to_dev(q_bits, dev), kd, kd, layer2, fc2, k_hash=None)
    assert meta2.block_table is plugin.topk_block_table
    plugin.attention_finished(None, None, None, None, layer, fc)
    assert np.array_equal(meta.block_table.cpu().numpy(), bt)
    assert meta.seq_lens.cpu().tolist() == new_lens
    plugin.execute_finished(None)
    assert not plugin.gsa_enabled and not plugin.has_decode

    # finished requests drop their state; a resumed one starts as a prefill again
    so = F.scheduler_output({}, finished=["r0"], resumed=[("r1", True)])
    plugin.update_states(so)
    assert "r0" not in plugin.phases and "r1" not in plugin.phases and "r2" in plugin.phases


def test_prefix_cache_hit_rehashes_blocks_in_place(cuda_device):
    """First prefill of requests whose prefix is already in the K cache: the plugin hashes those blocks straight
    from the paged K cache (one request ends its prefix inside a block) and the scheduled tokens from `key`."""
    import torch
    from unified_cache_management_b200.base import UcmSparseRole
    from unified_cache_management_b200.gsa_on_device import GSAOnDevice
    dev = cuda_device
    BS, Hq, Hkv, D = 16, 8, 2, 128
    cfg = F.make_vllm_config(block_size=BS, num_q_heads=Hq, num_kv_heads=Hkv, max_model_len=32 * BS, max_num_seqs=4,
                             overrides=dict(vllm_hash_attention_topk=4 * BS, gpu_seq_len_threshold=4 * BS,
                                            gpu_concurrency_threshold=1, vllm_hash_attention_rollback_layers=[0],
                                            vllm_hash_attention_skip_layers=[False, False]))
    plugin = GSAOnDevice(cfg, UcmSparseRole.WORKER)
    NB, mb = 64, 32
    prompt = [5 * BS + 7, 4 * BS]
    prefix = [3 * BS + 4, 2 * BS]
    rng = np.random.default_rng(3)
    perm = rng.permutation(NB)
    bt = np.zeros((2, mb), dtype=np.int32)
    off = 0
    for b, ln in enumerate(prompt):
        n = -(-ln // BS)
        bt[b, :n] = perm[off:off + n]
        off += n
    layer = "model.layers.1.self_attn.attn"
    kv_bits = H.bf16_normal(rng, (2, NB, BS, Hkv, D))
    kv = H.bf16_to_dev(kv_bits, dev)
    kv_caches = {"model.layers.0.self_attn.attn": torch.zeros_like(kv), layer: kv}
    plugin.initialize_kv_hash_cache_tensors(kv_caches, dev)
    k_hash = kv_caches[layer][1]
    requests = {f"r{b}": F.FakeRequest(num_computed_tokens=prefix[b], num_prompt_tokens=prompt[b]) for b in range(2)}
    input_batch = SimpleNamespace(req_id_to_index={"r0": 0, "r1": 1})
    qlens = [prompt[b] - prefix[b] for b in range(2)]
    keys = [H.bf16_normal(rng, (q, Hkv, D)) for q in qlens]
    key_all = torch.cat([H.bf16_to_dev(k, dev) for k in keys])
    slots = np.concatenate([bt[b, np.arange(prefix[b], prompt[b]) // BS].astype(np.int64) * BS
                            + np.arange(prefix[b], prompt[b]) % BS for b in range(2)])
    qsl = np.concatenate([[0], np.cumsum(qlens)]).astype(np.int32)
    meta = SimpleNamespace(seq_lens=torch.tensor(prompt, dtype=torch.int32, device=dev),
                           block_table=torch.from_numpy(bt).to(dev), slot_mapping=torch.from_numpy(slots).to(dev),
                           query_start_loc=torch.from_numpy(qsl).to(dev))
    fc = SimpleNamespace(attn_metadata={layer: meta}, virtual_engine=0,
                         no_compile_layers={layer: SimpleNamespace(kv_cache=[kv_caches[layer]])})
    so = F.scheduler_output({"r0": qlens[0], "r1": qlens[1]})
    so.num_external_computed_tokens_per_req = {"r0": prefix[0], "r1": prefix[1]}
    plugin.update_states(so)
    plugin.build_sparse_meta(so, requests, input_batch, {layer: meta})
    assert plugin.has_pc_hit
    assert plugin.prefix_block_ids.cpu().tolist() == bt[0, :4].tolist() + bt[1, :2].tolist()
    assert plugin.prefix_block_tokens.cpu().tolist() == [BS, BS, BS, 4, BS, BS]
    q_dummy = torch.zeros((sum(qlens), Hq, D), dtype=torch.bfloat16, device=dev)
    plugin.attention_begin(q_dummy, key_all, key_all, layer, fc, k_hash=k_hash)
    torch.cuda.synchronize()
    r_bits = _bf16_bits(plugin.hash_encoder.hash_weights_bf16)
    codes = k_hash.view(torch.int32).cpu().numpy().view(np.uint32).reshape(NB * BS, Hkv, 4)
    k_rows = kv_bits[0].reshape(NB * BS, Hkv, D)
    touched = np.zeros(NB * BS, dtype=bool)
    for b in range(2):
        pos = np.arange(prompt[b])
        slot = bt[b, pos // BS].astype(np.int64) * BS + pos % BS
        src = np.concatenate([k_rows[slot[:prefix[b]]], keys[b]])
        _, p64 = O.hash_encode(src, r_bits)
        hard, _ = O.count_code_mismatches(codes[slot], p64)
        assert hard == 0
        touched[slot] = True
    assert (codes[~touched] == 0).all()     # nothing else was written (the code cache starts zeroed)


def test_mla_prefill_then_decode(cuda_device):
    """MLA (DeepSeek) branch: latent + rope codes side by side in 18-word rows; the decode step swaps in the selected
    block table, the shortened lengths and their scheduling metadata, and attention_finished swaps them back."""
    import torch
    from unified_cache_management_b200.base import UcmSparseRole
    from unified_cache_management_b200.gsa_on_device import GSAOnDevice
    dev = cuda_device
    BS, Hq, red = 64, 16, 2
    topk_tokens = 8 * BS
    cfg = F.make_vllm_config(model="deepseek-ai/DeepSeek-V2-Lite-Chat", mla=True, block_size=BS, num_q_heads=Hq,
                             num_kv_heads=1, head_size=576, max_model_len=64 * BS, max_num_seqs=4, enforce_eager=False,
                             overrides=dict(vllm_hash_attention_topk=topk_tokens, gpu_seq_len_threshold=topk_tokens,
                                            gpu_concurrency_threshold=1, vllm_hash_attention_rollback_layers=[0],
                                            vllm_hash_attention_skip_layers=[False, False, True]))
    plugin = GSAOnDevice(cfg, UcmSparseRole.WORKER)
    assert plugin.is_mla and plugin.hash_reduction_head_num == red
    n_req, NB, mb = 2, 120, 64
    lens = [30 * BS + 5, 17 * BS]
    rng = np.random.default_rng(11)
    perm = rng.permutation(NB)
    bt = np.zeros((n_req, mb), dtype=np.int32)
    off = 0
    for b, ln in enumerate(lens):
        n = -(-(ln + 1) // BS)
        bt[b, :n] = perm[off:off + n]
        off += n
    layers = [f"model.layers.{i}.self_attn.attn" for i in range(3)]
    kv_caches = {name: torch.zeros((NB, BS, 576), dtype=torch.bfloat16, device=dev) for name in layers}
    plugin.initialize_kv_hash_cache_tensors(kv_caches, dev)
    layer = layers[1]
    k_hash = kv_caches[layer][1]
    assert kv_caches[layers[0]][1] is None and k_hash.shape == (NB, BS, 36) and k_hash.dtype == torch.bfloat16
    requests = {f"r{b}": F.FakeRequest(num_computed_tokens=0, num_prompt_tokens=lens[b]) for b in range(n_req)}
    input_batch = SimpleNamespace(req_id_to_index={f"r{b}": b for b in range(n_req)})

    # ---- prefill ----------------------------------------------------------------------------------------
    T = sum(lens)
    nope = H.bf16_normal(rng, (T, 512))
    rope = H.bf16_normal(rng, (T, 1, 64))
    slots = np.concatenate([bt[b, np.arange(ln) // BS].astype(np.int64) * BS + np.arange(ln) % BS
                            for b, ln in enumerate(lens)])
    qsl = torch.from_numpy(np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)).to(dev)
    bt_dev = torch.from_numpy(bt).to(dev)
    meta = SimpleNamespace(decode=None, prefill=SimpleNamespace(query_start_loc=qsl, block_table=bt_dev, chunked_context=None),
                           slot_mapping=torch.from_numpy(slots).to(dev), query_start_loc=qsl)
    fc = SimpleNamespace(attn_metadata={layer: meta}, no_compile_layers={}, virtual_engine=0)
    so = F.scheduler_output({f"r{b}": lens[b] for b in range(n_req)})
    plugin.update_states(so)
    plugin.build_sparse_meta(so, requests, input_batch, {layer: meta})
    plugin.attention_begin(None, H.bf16_to_dev(nope, dev), H.bf16_to_dev(rope, dev), layer, fc, phase="prefill",
                           k_hash=k_hash)
    plugin.attention_finished(None, None, None, None, layer, fc, phase="prefill")
    plugin.execute_finished(None)
    torch.cuda.synchronize()
    rn = _bf16_bits(plugin.hash_encoder_nope.hash_weights_bf16)
    rr = _bf16_bits(plugin.hash_encoder_rope.hash_weights_bf16)
    codes = k_hash.view(torch.int32).cpu().numpy().view(np.uint32).reshape(NB * BS, 18)
    _, p64 = O.hash_encode(nope, rn)
    assert O.count_code_mismatches(codes[slots, :16], p64)[0] == 0
    _, p64 = O.hash_encode(rope[:, 0], rr)
    assert O.count_code_mismatches(codes[slots, 16:], p64)[0] == 0
    untouched = np.ones(NB * BS, dtype=bool)
    untouched[slots] = False
    assert (codes[untouched] == 0).all()

    # ---- decode -------------------------------------------------------------------------------------------
    for r in requests.values():
        r.num_computed_tokens = r.num_prompt_tokens
    new_lens = np.array([ln + 1 for ln in lens], dtype=np.int32)
    new_slots = np.array([bt[b, lens[b] // BS].astype(np.int64) * BS + lens[b] % BS for b in range(n_req)])
    new_nope, new_rope = H.bf16_normal(rng, (n_req, 512)), H.bf16_normal(rng, (n_req, 1, 64))
    q_nope, q_rope = H.bf16_normal(rng, (n_req, Hq, 512)), H.bf16_normal(rng, (n_req, Hq, 64))
    seq_dev = torch.from_numpy(new_lens).to(dev)
    plugin.mla_metadata_fn = lambda s, hq, hkv: (torch.full((4, 8), 7, dtype=torch.int32, device=dev),
                                                 torch.arange(s.numel() + 1, dtype=torch.int32, device=dev))
    topk_seq, topk_tiles, topk_splits = plugin.build_decode_hash(seq_dev)
    assert np.array_equal(topk_seq.cpu().numpy(), O.update_seq_lens(new_lens, topk_tokens, BS))
    tiles0 = torch.zeros((4, 8), dtype=torch.int32, device=dev)
    splits0 = torch.zeros((n_req + 1,), dtype=torch.int32, device=dev)
    topk_tiles, topk_splits, topk_seq = plugin.maybe_init_cudagraph_buffers_for_topk(n_req + 1, tiles0, topk_tiles,
                                                                                     topk_splits, topk_seq)
    dec = SimpleNamespace(block_table=bt_dev, seq_lens=seq_dev, topk_block_table=None, topk_seq_lens=topk_seq,
                          topk_tile_scheduler_metadata=topk_tiles, topk_num_splits=topk_splits,
                          tile_scheduler_metadata=tiles0, num_splits=splits0)
    meta = SimpleNamespace(decode=dec, prefill=None, slot_mapping=torch.from_numpy(new_slots).to(dev),
                           query_start_loc=torch.arange(n_req + 1, dtype=torch.int32, device=dev))
    fc = SimpleNamespace(attn_metadata={layer: meta}, no_compile_layers={}, virtual_engine=0)
    so = F.scheduler_output({f"r{b}": 1 for b in range(n_req)})
    plugin.build_sparse_meta(so, requests, input_batch, {layer: meta})
    assert plugin.gsa_enabled
    plugin.attention_begin(None, H.bf16_to_dev(new_nope, dev), H.bf16_to_dev(new_rope, dev), layer, fc, phase="decode",
                           k_hash=k_hash, decode_ql_nope=H.bf16_to_dev(q_nope, dev), decode_q_pe=H.bf16_to_dev(q_rope, dev))
    torch.cuda.synchronize()
    k = topk_tokens // BS
    assert dec.seq_lens is topk_seq and dec.tile_scheduler_metadata is topk_tiles and dec.num_splits is topk_splits
    sel = dec.block_table.cpu().numpy()
    assert sel.shape == (n_req, k)

    def pair_mean(x):   # heads h and h + Hq/red averaged: float32 sum, one rounding to bf16
        f = O.bf16_bits_to_f32(x).reshape(n_req, red, Hq // red, -1)
        return O.f32_to_bf16_bits((f.sum(axis=1, dtype=np.float32) / np.float32(red)).astype(np.float32))
    qn, _ = O.hash_encode(pair_mean(q_nope), rn)
    qr, _ = O.hash_encode(pair_mean(q_rope), rr)
    q_codes = np.concatenate([qn, qr], axis=-1)                             # [B, 8, 18]
    codes_now = k_hash.view(torch.int32).cpu().numpy().view(np.uint32).reshape(NB, BS, 1, 18)
    ref = O.hamming_topk(codes_now, q_codes, bt, new_lens, k, O.REDUCE_MIN, False, sink_tokens=BS,
                         recent_tokens=4 * BS)
    assert np.array_equal(sel, ref["physical"][:, 0, :])
    # the skip layer reuses the selection; attention_finished restores everything
    plugin.attention_finished(None, None, None, None, layer, fc, phase="decode")
    assert dec.block_table is bt_dev and dec.seq_lens is seq_dev and dec.tile_scheduler_metadata is tiles0
    assert dec.num_splits is splits0
    fc2 = SimpleNamespace(attn_metadata={layers[2]: meta}, no_compile_layers={}, virtual_engine=0)
    plugin.attention_begin(None, None, None, layers[2], fc2, phase="decode", k_hash=None)
    assert np.array_equal(dec.block_table.cpu().numpy(), sel)
    plugin.attention_finished(None, None, None, None, layers[2], fc2, phase="decode")
    assert dec.block_table is bt_dev


def test_mla_prefix_cache_hit_rehashes_latent_cache_in_place(cuda_device):
    """MLA with a prefix-cache hit: the hit's latent + rope vectors are hashed straight from the paged cache
    [NB, BS, 512 + 64] into the 18-word rows (one request ends its prefix inside a block)."""
    import torch
    from unified_cache_management_b200.base import UcmSparseRole
    from unified_cache_management_b200.gsa_on_device import GSAOnDevice
    dev = cuda_device
    BS = 64
    cfg = F.make_vllm_config(model="deepseek-ai/DeepSeek-V2-Lite-Chat", mla=True, block_size=BS, num_q_heads=16,
                             num_kv_heads=1, head_size=576, max_model_len=32 * BS, max_num_seqs=4,
                             overrides=dict(vllm_hash_attention_topk=4 * BS, gpu_seq_len_threshold=4 * BS,
                                            gpu_concurrency_threshold=1, vllm_hash_attention_rollback_layers=[0],
                                            vllm_hash_attention_skip_layers=[False, False]))
    plugin = GSAOnDevice(cfg, UcmSparseRole.WORKER)
    NB, mb = 40, 32
    prompt = [5 * BS + 7, 4 * BS]
    prefix = [3 * BS + 9, 2 * BS]
    rng = np.random.default_rng(21)
    perm = rng.permutation(NB)
    bt = np.zeros((2, mb), dtype=np.int32)
    off = 0
    for b, ln in enumerate(prompt):
        n = -(-ln // BS)
        bt[b, :n] = perm[off:off + n]
        off += n
    layer = "model.layers.1.self_attn.attn"
    kv_bits = H.bf16_normal(rng, (NB, BS, 576))
    kv = H.bf16_to_dev(kv_bits, dev)
    kv_caches = {"model.layers.0.self_attn.attn": torch.zeros_like(kv), layer: kv}
    plugin.initialize_kv_hash_cache_tensors(kv_caches, dev)
    k_hash = kv_caches[layer][1]
    requests = {f"r{b}": F.FakeRequest(num_computed_tokens=prefix[b], num_prompt_tokens=prompt[b]) for b in range(2)}
    input_batch = SimpleNamespace(req_id_to_index={"r0": 0, "r1": 1})
    qlens = [prompt[b] - prefix[b] for b in range(2)]
    T = sum(qlens)
    nope, rope = H.bf16_normal(rng, (T, 512)), H.bf16_normal(rng, (T, 1, 64))
    slots = np.concatenate([bt[b, np.arange(prefix[b], prompt[b]) // BS].astype(np.int64) * BS
                            + np.arange(prefix[b], prompt[b]) % BS for b in range(2)])
    qsl = torch.from_numpy(np.concatenate([[0], np.cumsum(qlens)]).astype(np.int32)).to(dev)
    bt_dev = torch.from_numpy(bt).to(dev)
    meta = SimpleNamespace(decode=None, prefill=SimpleNamespace(query_start_loc=qsl, block_table=bt_dev, chunked_context=None),
                           slot_mapping=torch.from_numpy(slots).to(dev), query_start_loc=qsl)
    fc = SimpleNamespace(attn_metadata={layer: meta}, virtual_engine=0,
                         no_compile_layers={layer: SimpleNamespace(kv_cache=[kv_caches[layer]])})
    so = F.scheduler_output({"r0": qlens[0], "r1": qlens[1]})
    so.num_external_computed_tokens_per_req = {"r0": prefix[0], "r1": prefix[1]}
    plugin.update_states(so)
    plugin.build_sparse_meta(so, requests, input_batch, {layer: meta})
    assert plugin.has_pc_hit and plugin.prefix_block_tokens.cpu().tolist() == [BS, BS, BS, 9, BS, BS]
    plugin.attention_begin(None, H.bf16_to_dev(nope, dev), H.bf16_to_dev(rope, dev), layer, fc, phase="prefill",
                           k_hash=k_hash)
    torch.cuda.synchronize()
    rn = _bf16_bits(plugin.hash_encoder_nope.hash_weights_bf16)
    rr = _bf16_bits(plugin.hash_encoder_rope.hash_weights_bf16)
    codes = k_hash.view(torch.int32).cpu().numpy().view(np.uint32).reshape(NB * BS, 18)
    rows = kv_bits.reshape(NB * BS, 576)
    touched = np.zeros(NB * BS, dtype=bool)
    o = 0
    for b in range(2):
        pos = np.arange(prompt[b])
        slot = bt[b, pos // BS].astype(np.int64) * BS + pos % BS
        src_n = np.concatenate([rows[slot[:prefix[b]], :512], nope[o:o + qlens[b]]])
        src_r = np.concatenate([rows[slot[:prefix[b]], 512:], rope[o:o + qlens[b], 0]])
        o += qlens[b]
        assert O.count_code_mismatches(codes[slot, :16], O.hash_encode(src_n, rn)[1])[0] == 0
        assert O.count_code_mismatches(codes[slot, 16:], O.hash_encode(src_r, rr)[1])[0] == 0
        touched[slot] = True
    assert (codes[~touched] == 0).all()


def test_reference_hamming_topk_module_interface(cuda_device):
    """cuda_hamming_topk / update_seq_lens with the reference's argument list."""
    import torch
    from unified_cache_management_b200 import hamming_topk as HT
    dev = cuda_device
    B, Hkv, W, BS, mb = 3, 4, 4, 16, 20
    case = H.make_paged_case(13, B, Hkv, 1, W, BS, mb)
    k_hash = H.to_dev_i32(case["codes"], dev).view(torch.bfloat16)           # the plugin stores codes as bf16
    q_hash = H.to_dev_i32(case["q"], dev).view(torch.bfloat16).unsqueeze(1)
    bt, sl = H.to_dev_i32(case["block_table"], dev), H.to_dev_i32(case["seq_lens"], dev)
    out = HT.cuda_hamming_topk(q_hash, k_hash, bt, sl, 6 * BS, BS, 2 * BS, False)
    torch.cuda.synchronize()
    ref = O.hamming_topk(case["codes"], case["q"], case["block_table"], case["seq_lens"], 6, O.REDUCE_MIN, True,
                         sink_tokens=BS, recent_tokens=2 * BS)
    assert np.array_equal(out.cpu().numpy(), ref["physical"][:, 0])
    with pytest.raises(AssertionError):
        HT.cuda_hamming_topk(q_hash, k_hash, bt, sl, 6 * BS + 1, BS, 2 * BS, False)
    with pytest.raises(AssertionError):
        HT.cuda_hamming_topk(q_hash, k_hash, bt, sl, 2 * BS, BS, 2 * BS, False)
    got = HT.update_seq_lens(sl, 6 * BS, BS).cpu().numpy()
    assert np.array_equal(got, O.update_seq_lens(case["seq_lens"], 6 * BS, BS))
    assert np.array_equal(HT.update_seq_lens(sl.cpu(), 6 * BS, BS).numpy(), got)
    assert HT.fake_hamming_topk(q_hash, k_hash, bt, sl, 6 * BS, BS, 2 * BS).shape == (B, 6)


def test_hash_encoder_interface(cuda_device):
    import torch
    from unified_cache_management_b200.hash_encoder import HashEncoder
    dev = cuda_device
    enc = HashEncoder(128, 128, torch.bfloat16, dev)
    w = enc.hash_weights
    assert w.dtype == torch.float32                                          # bf16 models keep a float32 master
    eye = (w.T @ w)
    assert torch.allclose(eye, torch.eye(128, device=dev), atol=1e-4)        # orthogonal projection
    with pytest.raises(ValueError):
        HashEncoder(128, 100, torch.bfloat16, dev)
    with pytest.raises(ValueError):
        enc.set_hash_weight(torch.zeros((64, 128), device=dev))
    with pytest.raises(ValueError):
        enc.compute_hash(torch.zeros((4, 64), dtype=torch.bfloat16, device=dev))
    rng = np.random.default_rng(1)
    x = H.bf16_normal(rng, (5, 7, 128))
    codes = enc.compute_hash(H.bf16_to_dev(x, dev))
    assert codes.shape == (5, 7, 16) and codes.dtype == torch.uint8
    _, p64 = O.hash_encode(x, _bf16_bits(enc.hash_weights_bf16))
    hard, _ = O.count_code_mismatches(codes.cpu().numpy().view("<u4"), p64)
    assert hard == 0
    pm = enc._unpack_hash(codes)
    assert pm.shape == (5, 7, 128) and set(pm.unique().tolist()) <= {-1.0, 1.0}
    assert torch.equal(pm > 0, torch.from_numpy(O.unpack_bits_u32(codes.cpu().numpy().view("<u4"))).to(dev))
