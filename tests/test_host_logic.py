"""CPU tests of the host-side mirror: config keys, model lookup, hook surface, role handling."""
import json
import os

import pytest

from tests import fake_vllm as F
from unified_cache_management_b200 import base
from unified_cache_management_b200.gsa_on_device_config import GSAOnDeviceConfig


def test_config_round_trip_and_validation(tmp_path):
    cfg = GSAOnDeviceConfig()
    assert cfg.must_select_blocks == [0, -2, -1] and cfg.chunk_repre_method == "max" and cfg.reduce == "min"
    cfg.generate_config_data("m", "random", 4, 2048, 128, "sum", 128, 128, [0.3] * 4, [-1] * 4, [0, -1])
    assert cfg.reduce == "sum"
    p = tmp_path / "c.json"
    cfg.to_json(str(p))
    again = GSAOnDeviceConfig.from_json(str(p))
    assert again.must_select_blocks == [0, -1] and again.num_hidden_layers == 4
    with pytest.raises(ValueError):
        cfg.generate_config_data("m", "learned", 4, 2048, 128, "sum", 128, 128, [0.3] * 4, [-1] * 4, [0])
    with pytest.raises(ValueError):
        cfg.generate_config_data("m", "random", 4, 2048, 100, "sum", 128, 128, [0.3] * 4, [-1] * 4, [0])
    with pytest.raises(ValueError):
        cfg.generate_config_data("m", "random", 4, 2048, 128, "median", 128, 128, [0.3] * 4, [-1] * 4, [0])
    with pytest.raises(ValueError):
        cfg.generate_config_data("m", "random", 4, 2048, 128, "sum", 128, 128, [0.3] * 3, [-1] * 4, [0])
    with pytest.raises(ValueError):
        cfg.set_hash_weight([[0.0]])
    cfg.apply_overrides({"init_window_sz": 1, "local_window_sz": 2, "vllm_hash_attention_topk": 4096}, 128)
    assert cfg.must_select_blocks == [0, -2, -1] and cfg.vllm_hash_attention_topk == 4096


# sha256 of json.dumps(parsed, sort_keys=True, separators=(",", ":")) of the reference's six per-model files
# (ucm/sparse/gsa_on_device/configs/*.json): the shipped files must parse to the same values.
_REFERENCE_CONFIG_DIGESTS = {
    "gsa_on_device_deepseek_r1_awq_config.json": "c720deaba07e98dfd800e845f21bb5bdf212d1847e30ba3b624fe0c5fc093b73",
    "gsa_on_device_deepseek_v2_lite_config.json": "6001244e3b7887374b2b77faaee07e37bb70c971dcbc6f95e9721f2463b5be7e",
    "gsa_on_device_qwen3_32B_config.json": "290541b311437409c8f10be10ef3cbe36df73fb35a4d75f8fefa70e9f1676251",
    "gsa_on_device_qwen3_4B_config.json": "b2da5f9dc1895d932cabba441ff91dd68c05638bbb5088cc2c6b217d1010a75d",
    "gsa_on_device_qwen3_coder_30B_A3B_config.json": "f76c044baa2ac3b2f5b4681eaffebb686191072941a0ec65b397d0f0ef5c42ac",
    "gsa_on_device_qwq_32B_config.json": "61743382310d630b70bd878107a5d0565965636bdb82bb6a7ecece46582bda35",
}
# per-model files this repository adds (the reference ships none for these models)
_ADDED_CONFIGS = {"gsa_on_device_llama3_8B_config.json", "gsa_on_device_llama3_70B_config.json"}


def _config_dir():
    return os.path.join(os.path.dirname(base.__file__), "configs")


def test_shipped_config_files_load():
    """Every key of the shipped per-model files is a field of the dataclass (same names as the reference)."""
    d = _config_dir()
    files = {f for f in os.listdir(d) if f.endswith(".json")}
    assert files == set(_REFERENCE_CONFIG_DIGESTS) | _ADDED_CONFIGS
    for f in files:
        cfg = GSAOnDeviceConfig.from_json(os.path.join(d, f))
        assert len(cfg.top_k_ratio_per_layer) == cfg.num_hidden_layers
        if cfg.vllm_hash_attention_topk is not None:   # the reference's QwQ file carries no vLLM keys
            assert cfg.vllm_hash_attention_topk % 128 == 0
            assert len(cfg.vllm_hash_attention_skip_layers) == cfg.num_hidden_layers


def test_shipped_config_values_are_the_reference_values():
    """The six files named like the reference's hold the reference's values: compared with the checkout when
    UCM_REFERENCE_ROOT points at one, and with the digests of its parsed files in any case."""
    import hashlib
    d = _config_dir()
    ref_root = os.environ.get("UCM_REFERENCE_ROOT")
    for name, digest in _REFERENCE_CONFIG_DIGESTS.items():
        with open(os.path.join(d, name)) as f:
            mine = json.load(f)
        canon = json.dumps(mine, sort_keys=True, separators=(",", ":")).encode()
        assert hashlib.sha256(canon).hexdigest() == digest, name
        if ref_root:
            ref_file = os.path.join(ref_root, "ucm", "sparse", "gsa_on_device", "configs", name)
            if os.path.exists(ref_file):
                with open(ref_file) as f:
                    assert json.load(f) == mine, name


def test_model_lookup():
    from unified_cache_management_b200.gsa_on_device import gsa_on_device_config_path_for_model
    assert gsa_on_device_config_path_for_model(F.make_vllm_config("Qwen/Qwen3-32B")).endswith("qwen3_32B_config.json")
    assert gsa_on_device_config_path_for_model(F.make_vllm_config("meta-llama/Meta-Llama-3-70B-Instruct")).endswith(
        "llama3_70B_config.json")
    with pytest.raises(ValueError):
        gsa_on_device_config_path_for_model(F.make_vllm_config("mistralai/Mixtral"))


def test_hook_surface_matches_reference_names():
    from unified_cache_management_b200.gsa_on_device import GSAOnDevice
    hooks = ["register_kv_caches", "execute_begin", "execute_finished", "attention_begin", "attention_finished",
             "update_states", "ffn_begin", "ffn_finished", "layer_begin", "layer_finished", "request_finished_in_worker",
             "request_begin", "request_finished_in_scheduler", "estimate_num_slots_sparsed", "update_state_after_alloc",
             "build_sparse_meta", "allocate_slots", "initialize_kv_hash_cache_tensors", "bind_sparse_metadata",
             "clear_sparse_metadata"]
    for h in hooks:
        assert callable(getattr(GSAOnDevice, h)), h
    assert base.INVALID_SLOT == -1
    assert {r.name for r in base.UcmSparseRole} == {"SCHEDULER", "WORKER"}
    import inspect
    sig = inspect.signature(GSAOnDevice.attention_begin)
    assert list(sig.parameters)[1:] == ["query", "key", "value", "layer_name", "forward_context", "output", "phase",
                                        "k_hash", "decode_ql_nope", "decode_q_pe"]


def test_scheduler_role_needs_no_device_buffers():
    from unified_cache_management_b200.gsa_on_device import GSAOnDevice
    plugin = GSAOnDevice(F.make_vllm_config("Qwen/Qwen3-4B", max_model_len=32768), base.UcmSparseRole.SCHEDULER)
    assert plugin.role == base.UcmSparseRole.SCHEDULER
    assert plugin.estimate_num_slots_sparsed(None) == base.INVALID_SLOT
    assert plugin.hash_topk_tokens == 2048 and plugin.seq_len_threshold == 2048
    plugin.request_begin("r", [1, 2, 3])
    plugin.request_finished_in_scheduler("r")
    with pytest.raises(ValueError):
        GSAOnDevice(F.make_vllm_config("Qwen/Qwen3-4B", device_type="npu"), base.UcmSparseRole.SCHEDULER)
    with pytest.raises(AssertionError):   # top-k budget above the context limit
        GSAOnDevice(F.make_vllm_config("Qwen/Qwen3-4B", max_model_len=1024), base.UcmSparseRole.SCHEDULER)


def test_peer_exchange_layout_keeps_slices_and_parities_apart():
    """Offsets of the collective-free exchange buffer: per parity scores / ids / flags do not overlap, ranks' slices
    are disjoint, and consecutive steps use different halves."""
    from unified_cache_management_b200.sharded import exchange_layout
    world, slab = 4, 96
    seen = {}
    for seq in (1, 2):
        for rank in range(world):
            o_s, o_i, o_f, mine, words = exchange_layout(world, rank, slab, seq)
            assert words == 2 * world * slab + 64 and o_s == (seq & 1) * words
            spans = [(o_s + mine, o_s + mine + slab), (o_i + mine, o_i + mine + slab), (o_f + rank, o_f + rank + 1)]
            for lo, hi in spans:
                assert o_s <= lo and hi <= o_s + words
                for (l2, h2) in seen.values():
                    assert hi <= l2 or h2 <= lo
            for n, sp in enumerate(spans):
                seen[(seq, rank, n)] = sp
    assert exchange_layout(world, 0, slab, 3)[0] == exchange_layout(world, 0, slab, 1)[0]


def test_reduce_mode_carries_the_inputs_stable_flag():
    from unified_cache_management_b200 import ops
    assert ops._mode("min", False) == 0 and ops._mode("sum", False) == 1
    assert ops._mode("sum", True) == 1 | 0x100 and ops._mode("min", True) == 0x100
    with open(os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "include", "ucmr.h")) as f:
        text = f.read()
    assert "#define UCMR_FLAG_INPUTS_STABLE 0x100" in text and "#define UCMR_FLAG_CACHE_APPEND_ONLY 0x200" in text
    assert ops._mode("sum", True, True) == 1 | 0x300
    with pytest.raises(ValueError):
        ops._mode("sum", False, True)
