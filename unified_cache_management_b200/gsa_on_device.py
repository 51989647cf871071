"""``GSAOnDevice`` sparse-attention plugin on the sm_100a retrieval kernels (CUDA; GQA and MLA models).

Drop-in for the reference plugin of the same name
(``ucm/sparse/gsa_on_device/gsa_on_device.py:99-1421``): same ``UcmSparseBase`` hooks with the same
side effects on ``attn_metadata.block_table`` / ``.seq_lens``, same config keys, same per-request
prefill/decode bookkeeping.  What changed is underneath:

* ``attention_begin`` caches the new tokens' key codes with ONE fused launch
  (encode + paged scatter on tcgen05; reference: Triton ``fused_hash_and_cache_kernel``);
* a decode step hashes the queries (group mean + encode, one launch) and retrieves with two launches
  (Hamming scan, exact top-k with block-table lookup; reference: scan kernel + torch min/topk/sort/
  gather), into persistent buffers, so the step is CUDA-graph friendly;
* nothing is imported from vLLM at module scope, and nothing else of the reference package is needed.

MLA models (DeepSeek: one latent kv head, 512-bit code of the latent + 64-bit code of the rope part per token)
follow the reference's CUDA MLA branch (gsa_on_device.py:221-233, 375-394, 426-455, 667-714, 1083-1096): two
encoders write side by side into 18-word cache rows, the decode step retrieves with the token-row scan, and the
FlashMLA scheduling metadata of the shortened sequences comes from vLLM's ``get_mla_metadata`` (imported when
first needed; ``mla_metadata_fn`` can be set instead).
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional, Union

import torch

from . import ops
from .base import INVALID_SLOT, UcmSparseBase, UcmSparseCpuGpuBuffer, UcmSparseMetadata, UcmSparseRole
from .gsa_on_device_config import GSAOnDeviceConfig
from .hamming_topk import update_seq_lens
from .hash_encoder import HashEncoder
from .request_state import RequestPhaseTracker, prefix_layout, prefix_slots

ReqType = Union[str, int]
_CONFIG_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "configs")


def cdiv(a: int, b: int) -> int:
    return -(-a // b)


def gsa_on_device_config_path_for_model(vllm_config, search_dirs: Optional[List[str]] = None) -> str:
    """Per-model JSON lookup by substrings of the model name (reference: gsa_on_device.py:46-96).
    ``UCM_GSA_ON_DEVICE_CONFIG`` or the ``config_path`` override wins."""
    env = os.environ.get("UCM_GSA_ON_DEVICE_CONFIG")
    if env:
        return env
    model = str(vllm_config.model_config.model).lower()
    rules = [
        (("deepseek", "r1"), (), "gsa_on_device_deepseek_r1_awq_config.json"),
        (("qwen3", "32b"), ("coder",), "gsa_on_device_qwen3_32B_config.json"),
        (("qwen3", "30b", "coder"), (), "gsa_on_device_qwen3_coder_30B_A3B_config.json"),
        (("qwen3", "4b"), (), "gsa_on_device_qwen3_4B_config.json"),
        (("qwq", "32b"), (), "gsa_on_device_qwq_32B_config.json"),
        (("deepseek", "v2"), (), "gsa_on_device_deepseek_v2_lite_config.json"),
        (("llama", "70b"), (), "gsa_on_device_llama3_70B_config.json"),
        (("llama", "8b"), (), "gsa_on_device_llama3_8B_config.json"),
    ]
    for must, must_not, fname in rules:
        if all(m in model for m in must) and not any(m in model for m in must_not):
            for d in (search_dirs or []) + [_CONFIG_DIR]:
                p = os.path.join(d, fname)
                if os.path.isfile(p):
                    return p
    raise ValueError(f"[GSAOnDevice] Unsupported model for gsa_on_device: {model}")


def _plugin_overrides(vllm_config) -> Dict:
    """Inline settings under kv_connector_extra_config['ucm_sparse_config']['GSAOnDevice']."""
    ktc = getattr(vllm_config, "kv_transfer_config", None)
    extra = getattr(ktc, "kv_connector_extra_config", None) if ktc is not None else None
    if isinstance(extra, dict):
        cfg = extra.get("ucm_sparse_config") or {}
        if isinstance(cfg, dict):
            return dict(cfg.get("GSAOnDevice") or {})
    return {}


class GSAOnDevice(UcmSparseBase):
    def __init__(self, vllm_config, role: UcmSparseRole):
        super().__init__(vllm_config, role)
        self.rank = vllm_config.parallel_config.rank
        self.is_mla = bool(getattr(vllm_config.model_config, "is_deepseek_mla", False))
        self.gsa_enabled = False
        if vllm_config.device_config.device_type != "cuda":
            raise ValueError(f"Unsupported device type: {vllm_config.device_config.device_type}")
        self.is_cuda = True
        self.device = torch.device(f"cuda:{self.rank}")

        # per tensor-parallel rank, as the reference reads them (gsa_on_device.py:118-123)
        self.num_q_heads = vllm_config.model_config.get_num_attention_heads(vllm_config.parallel_config)
        self.num_key_heads = vllm_config.model_config.get_num_kv_heads(vllm_config.parallel_config)
        self.block_size = vllm_config.cache_config.block_size

        overrides = _plugin_overrides(vllm_config)
        path = overrides.pop("config_path", None) or gsa_on_device_config_path_for_model(vllm_config)
        self.gsa_on_device_config = GSAOnDeviceConfig.from_json(path)
        self.gsa_on_device_config.apply_overrides(overrides, self.block_size)
        # the reference forces 1 sink block and 4 recent blocks (gsa_on_device.py:782-783); the config's
        # must_select_blocks list is used instead when this switch is on
        self.use_must_select_blocks = bool(overrides.get("use_must_select_blocks", False))

        cfg = self.gsa_on_device_config
        self.hash_topk_tokens = cfg.vllm_hash_attention_topk
        self.hash_rollback_layers = cfg.vllm_hash_attention_rollback_layers
        self.hash_skip_layers = cfg.vllm_hash_attention_skip_layers
        self.seq_len_threshold = cfg.gpu_seq_len_threshold
        self.concurrency_threshold = cfg.gpu_concurrency_threshold
        if self.hash_topk_tokens is None:
            # the reference's QwQ-32B file has no vLLM keys: its plugin stops at the comparison below with a
            # TypeError; say what is missing instead
            raise ValueError(f"{os.path.basename(path)} has no vllm_hash_attention_topk; set it (and the rollback / "
                             "skip layer lists) in ucm_sparse_config or in the file")
        assert self.seq_len_threshold >= self.hash_topk_tokens, \
            "seq_len_threshold must be larger than or equal to vllm_hash_attention_topk"
        assert self.hash_topk_tokens % self.block_size == 0, "vllm_hash_attention_topk must be divisible by block_size"
        assert self.hash_topk_tokens <= vllm_config.model_config.max_model_len, \
            "vllm_hash_attention_topk must be less than max_model_len"

        if role != UcmSparseRole.WORKER:
            return

        self.ori_seq_lens_decode = None
        self.ori_block_table_decode = None
        self.topk_block_table = None
        self.topk_seq_lens = None
        self.topk_seq_lens_qwen = None
        self.has_pc_hit = False
        self.has_decode = False
        self.decode_only = False
        self.phases = RequestPhaseTracker()   # which live request is prefilling / decoding
        self.step_plan = None
        self.num_reqs = 0

        self.max_batch_size = vllm_config.scheduler_config.max_num_seqs
        self.max_num_tokens = vllm_config.model_config.max_model_len
        self.decode_req_ids_buf = UcmSparseCpuGpuBuffer(self.max_batch_size, dtype=torch.int64, device=self.device,
                                                        pin_memory=True, with_numpy=True)
        max_block_per_seq = cdiv(self.max_num_tokens, self.block_size)
        self.max_block_per_seq = max_block_per_seq
        dev = self.device
        self.origin_tile_scheduler_metadata = None
        self.origin_num_splits = None
        self.mla_metadata_fn = None  # get_mla_metadata(seq_lens, num_q_heads, num_kv_heads); vLLM's when None
        if self.is_mla:
            self._init_mla(vllm_config, cfg, max_block_per_seq)
            self.init_for_pc()
            return
        self.full_block_table = torch.zeros((self.max_batch_size, max_block_per_seq), dtype=torch.int32, device=dev)
        self.full_seq_lens = torch.zeros((self.max_batch_size,), dtype=torch.int32, device=dev)
        self.head_dim = vllm_config.model_config.get_head_size()
        self.hash_encoder = HashEncoder(input_dim=self.head_dim, hash_bits=cfg.hash_bits or self.head_dim,
                                        dtype=vllm_config.model_config.dtype, device=dev)
        # persistent retrieval buffers (no allocation inside a step)
        self.topk_blocks = self.hash_topk_tokens // self.block_size
        self._workspace = ops.new_workspace(self.max_batch_size, self.num_key_heads, max_block_per_seq, dev, True)
        kb = min(self.topk_blocks, max_block_per_seq)
        self._retrieval = ops.Retrieval(
            physical=torch.zeros((self.max_batch_size, 1, kb), dtype=torch.int32, device=dev),
            logical=torch.zeros((self.max_batch_size, 1, kb), dtype=torch.int32, device=dev), scores=None,
            valid_count=torch.zeros((self.max_batch_size,), dtype=torch.int32, device=dev),
            new_seq_lens=torch.zeros((self.max_batch_size,), dtype=torch.int32, device=dev))
        self.init_for_pc()

    def _init_mla(self, vllm_config, cfg, max_block_per_seq):
        """Two encoders (latent and rope part), persistent retrieval buffers and, for CUDA-graph runs, the
        fixed-address copies of the shortened-sequence scheduling metadata (gsa_on_device.py:167-185, 210-233)."""
        dev = self.device
        hf = vllm_config.model_config.hf_text_config
        self.hash_reduction_head_num = cfg.vllm_hash_attention_reduction_head_num or 1
        self.kv_lora_rank = getattr(hf, "kv_lora_rank", None)
        self.qk_rope_head_dim = getattr(hf, "qk_rope_head_dim", None)
        if not self.kv_lora_rank or not self.qk_rope_head_dim:
            raise ValueError("MLA model config lacks kv_lora_rank / qk_rope_head_dim")
        dtype = vllm_config.model_config.dtype
        self.hash_encoder_nope = HashEncoder(input_dim=self.kv_lora_rank, hash_bits=self.kv_lora_rank, dtype=dtype,
                                             device=dev)
        self.hash_encoder_rope = HashEncoder(input_dim=self.qk_rope_head_dim, hash_bits=self.qk_rope_head_dim,
                                             dtype=dtype, device=dev)
        self.nope_words = self.kv_lora_rank // 32
        self.rope_words = self.qk_rope_head_dim // 32
        self.topk_blocks = self.hash_topk_tokens // self.block_size
        kb = min(self.topk_blocks, max_block_per_seq)
        self._workspace = ops.new_workspace(self.max_batch_size, 1, max_block_per_seq, dev, False)
        self._retrieval = ops.Retrieval(
            physical=torch.zeros((self.max_batch_size, 1, kb), dtype=torch.int32, device=dev),
            logical=torch.zeros((self.max_batch_size, 1, kb), dtype=torch.int32, device=dev), scores=None,
            valid_count=torch.zeros((self.max_batch_size,), dtype=torch.int32, device=dev),
            new_seq_lens=torch.zeros((self.max_batch_size,), dtype=torch.int32, device=dev))
        if not getattr(vllm_config.model_config, "enforce_eager", True):
            num_sms = torch.cuda.get_device_properties(dev).multi_processor_count
            self.cg_buf_topk_tile_scheduler_metadata = torch.zeros((num_sms, 8), device=dev, dtype=torch.int32)
            self.cg_buf_topk_num_splits = torch.empty((self.max_batch_size + 1,), device=dev, dtype=torch.int32)
            self.cg_buf_topk_seq_lens = torch.empty((self.max_batch_size + 1,), device=dev, dtype=torch.int32)

    # ---- prefix-cache bookkeeping buffers (gsa_on_device.py:333-360) ------------------------------
    def init_for_pc(self):
        self.prefix_slot_mapping_buf = torch.empty(self.max_num_tokens * self.max_batch_size, device=self.device,
                                                   dtype=torch.int64)
        self.prefix_block_ids_buf = torch.empty(cdiv(self.max_num_tokens * self.max_batch_size, self.block_size),
                                                device=self.device, dtype=torch.int32)
        self.prefix_block_tokens_buf = torch.empty_like(self.prefix_block_ids_buf)  # valid tokens per listed block
        self.token_idx_buf = torch.arange(self.max_num_tokens, device=self.device, dtype=torch.int64)

    # ---- hashing ---------------------------------------------------------------------------------
    @staticmethod
    def _fold_heads(x: torch.Tensor, fold: int) -> torch.Tensor:
        """[T, H, D] -> [T, H/fold, D]: heads h, h + H/fold, ... averaged (the MLA head reduction)."""
        if fold <= 1:
            return x
        t, h, d = x.shape
        return x.view(t, fold, h // fold, d).mean(dim=1)

    def hash_code(self, nope=None, rope=None, reduction_head_num: int = 1, query: Optional[torch.Tensor] = None):
        """Query codes, viewed as bf16 like the reference's (gsa_on_device.py:375-412).
        GQA: one code per kv head from the mean of its query group (the mean and the encode are one kernel).
        MLA: ``reduction_head_num`` = r folds heads h, h + H/r, ... into one, then the latent and the rope part go
        through their own encoders; returns the pair."""
        if self.is_mla:
            if nope is None or rope is None:
                raise ValueError("MLA mode requires `nope` and `rope`.")
            codes = (self.hash_encoder_nope.compute_hash(self._fold_heads(nope, reduction_head_num)),
                     self.hash_encoder_rope.compute_hash(self._fold_heads(rope, reduction_head_num)))
            return tuple(c.view(torch.bfloat16) for c in codes)
        if query is None:
            raise ValueError("GQA mode requires `query`.")
        hq, hkv = self.num_q_heads, self.num_key_heads
        if hq < hkv:      # fewer query heads than kv heads: every query head answers for hkv / hq kv heads
            query = torch.repeat_interleave(query, hkv // hq, dim=1)
        group = hq // hkv if hq > hkv else 1
        return self.hash_encoder.compute_hash_grouped(query, group).view(torch.bfloat16)

    def get_layer_attn_metadata(self, forward_context, layer_name: str):
        attn_meta = forward_context.attn_metadata
        return attn_meta[layer_name] if isinstance(attn_meta, dict) else attn_meta

    def get_layer_state(self, layer_name: str):
        """(rollback layer: dense attention, no code cache; skip layer: reuses the previous layer's selection) for a
        vLLM layer name such as ``model.layers.17.self_attn.attn`` (gsa_on_device.py:418-424)."""
        layer_id = int(layer_name.split(".")[2])
        skip = self.hash_skip_layers
        return layer_id in self.hash_rollback_layers, bool(skip[layer_id]) if layer_id < len(skip) else False

    def cache_k_hash_gqa_cuda(self, key, attn_metadata, k_hash, forward_context, layer_name):
        slot_mapping = attn_metadata.slot_mapping.flatten()
        n = slot_mapping.numel()
        self.hash_encoder.compute_hash_and_cache(key[:n], slot_mapping, k_hash, block_size=self.block_size)
        if self.has_pc_hit:
            # keys of the prefix-cache hit are already in the KV cache: hash those blocks into the code cache
            attn = forward_context.no_compile_layers[layer_name]
            kv_cache = attn.kv_cache[forward_context.virtual_engine]
            k_pool = kv_cache[0][0]
            # (reference: torch gather of the blocks, then compute_hash_and_cache with the prefix slot mapping,
            # gsa_on_device.py:574-588; here one kernel reads the blocks where they lie)
            self.hash_encoder.compute_hash_of_blocks(k_pool, self.prefix_block_ids, k_hash,
                                                     block_tokens=self.prefix_block_tokens)

    def _mla_code_cache_words(self, k_hash):
        """The MLA code cache [NB, BS, 36] bf16 as words [NB, BS, 1, 18]."""
        cw = ops.as_words(k_hash)
        return cw.unsqueeze(2) if cw.dim() == 3 else cw

    def cache_k_hash_mla_cuda(self, nope, rope, k_hash, attn_metadata, forward_context, layer_name):
        """Latent code to words [0, 16), rope code to words [16, 18) of each token's cache row: the reference
        hashes both and joins them with vLLM's concat_and_cache_mla (gsa_on_device.py:426-455)."""
        slot_mapping = attn_metadata.slot_mapping.flatten()
        n = slot_mapping.numel()
        cw = self._mla_code_cache_words(k_hash)
        enc_n, enc_r = self.hash_encoder_nope, self.hash_encoder_rope
        nope3 = nope.reshape(nope.shape[0], 1, nope.shape[-1])[:n]
        rope3 = rope.reshape(rope.shape[0], 1, rope.shape[-1])[:n]
        ops.hash_encode_and_cache(enc_n._as_bf16(nope3), slot_mapping, cw, enc_n.hash_weights_bf16, word_offset=0)
        ops.hash_encode_and_cache(enc_r._as_bf16(rope3), slot_mapping, cw, enc_r.hash_weights_bf16,
                                  word_offset=self.nope_words)
        if self.has_pc_hit:
            # the hit's latent + rope vectors are already in the paged cache [NB, BS, 512 + 64]
            attn = forward_context.no_compile_layers[layer_name]
            kv = attn.kv_cache[forward_context.virtual_engine][0]
            kv4 = kv.unsqueeze(2) if kv.dim() == 3 else kv
            ids = self.prefix_block_ids.to(torch.int32)
            ops.hash_encode_blocks(kv4[..., : self.kv_lora_rank], ids, cw, enc_n.hash_weights_bf16,
                                   block_tokens=self.prefix_block_tokens, word_offset=0)
            ops.hash_encode_blocks(kv4[..., self.kv_lora_rank:], ids, cw, enc_r.hash_weights_bf16,
                                   block_tokens=self.prefix_block_tokens, word_offset=self.nope_words)

    def update_decode_topk_mla_cuda(self, is_rollback_layer, is_skip_hash_layer, attn_metadata, decode_ql_nope,
                                    decode_q_pe, k_hash):
        """Reference: gsa_on_device.py:667-714.  The decode metadata carries the shortened sequence lengths and
        their FlashMLA scheduling data (built once per step by ``build_decode_hash``); this swaps them in
        together with the selected block table, ``attention_finished`` swaps them back."""
        if is_rollback_layer:
            return
        dec = attn_metadata.decode
        if is_skip_hash_layer:
            assert dec.topk_block_table is not None
            block_table = dec.topk_block_table
        else:
            q_nope_hash, q_rope_hash = self.hash_code(nope=decode_ql_nope, rope=decode_q_pe,
                                                      reduction_head_num=self.hash_reduction_head_num)
            q_hash = ops.as_words(torch.cat([q_nope_hash, q_rope_hash], dim=-1))       # [B, heads/r, 18]
            n = q_hash.shape[0]
            kb = self._retrieval.physical.shape[2]
            out = ops.Retrieval(physical=self._retrieval.physical[:n], logical=self._retrieval.logical[:n],
                                scores=None, valid_count=self._retrieval.valid_count[:n],
                                new_seq_lens=self._retrieval.new_seq_lens[:n])
            ops.hamming_topk(self._mla_code_cache_words(k_hash), q_hash, dec.block_table, dec.seq_lens, kb,
                             reduce=self.gsa_on_device_config.reduce, reduce_kvhead=False,
                             workspace=self._workspace, out=out, want_scores=False, inputs_stable=True, **self._forced())
            block_table = out.physical[:, 0, :]
            dec.topk_block_table = block_table
        self.ori_block_table_decode = dec.block_table
        self.ori_seq_lens_decode = dec.seq_lens
        self.origin_tile_scheduler_metadata = dec.tile_scheduler_metadata
        self.origin_num_splits = dec.num_splits
        dec.block_table = block_table
        dec.seq_lens = dec.topk_seq_lens
        dec.tile_scheduler_metadata = dec.topk_tile_scheduler_metadata
        dec.num_splits = dec.topk_num_splits

    def build_decode_hash(self, seq_lens):
        """Shortened sequence lengths of a decode step and FlashMLA's scheduling metadata for them
        (gsa_on_device.py:1083-1096); called by the patched FlashMLA metadata builder."""
        topk_seq_lens = update_seq_lens(seq_lens, topk_token=self.hash_topk_tokens, block_size=self.block_size)
        fn = self.mla_metadata_fn
        if fn is None:
            try:
                from vllm.attention.ops.flashmla import get_mla_metadata as fn
            except Exception as exc:  # the scheduling metadata is FlashMLA's own format: no stand-in
                raise RuntimeError("vLLM's FlashMLA ops (vllm.attention.ops.flashmla.get_mla_metadata) are needed "
                                   "for MLA decode metadata; set plugin.mla_metadata_fn otherwise") from exc
        topk_tile_scheduler_metadata, topk_num_splits = fn(topk_seq_lens, self.num_q_heads, 1)
        return topk_seq_lens, topk_tile_scheduler_metadata, topk_num_splits

    def maybe_init_cudagraph_buffers_for_topk(self, n, tile_scheduler_metadata, topk_tile_scheduler_metadata,
                                              topk_num_splits, topk_seq_lens):
        """The shortened-sequence scheduling metadata of the step, copied into the fixed-address buffers a CUDA-graph
        replay reads (gsa_on_device.py:1382-1405).  Returns views of those buffers."""
        def pinned(buf, src, rows):
            view = buf[:rows]
            view.copy_(src)
            return view

        meta = pinned(self.cg_buf_topk_tile_scheduler_metadata, topk_tile_scheduler_metadata,
                      tile_scheduler_metadata.size(0))
        splits = pinned(self.cg_buf_topk_num_splits, topk_num_splits, n)
        self.cg_buf_topk_num_splits[n:].fill_(topk_num_splits[-1])   # padding rows repeat the last offset
        lens = pinned(self.cg_buf_topk_seq_lens, topk_seq_lens, topk_seq_lens.size(0))
        return meta, splits, lens

    # ---- retrieval ---------------------------------------------------------------------------------
    # (inputs_stable in the retrieval calls: block table and lengths come from the step's attention metadata, built
    # before the forward pass; the kernel enqueued right before the scan is the query hashing, which writes neither)
    # (cache_append_only in a decode-only step: the key hashing before the scan wrote one new token per request, which
    # sits in the request's last block; a step with prefill chunks writes whole blocks and does not make the promise)
    def _forced(self):
        if self.use_must_select_blocks:
            return dict(must_select=tuple(self.gsa_on_device_config.must_select_blocks))
        return dict(sink_tokens=self.block_size, recent_tokens=self.block_size * 4)

    def update_decode_topk_gqa_cuda(self, query, k_hash, attn_metadata):
        n = self.num_reqs
        q_hash = self.hash_code(query=query[:n])
        kb = self._retrieval.physical.shape[2]
        out = ops.Retrieval(physical=self._retrieval.physical[:n], logical=self._retrieval.logical[:n], scores=None,
                            valid_count=self._retrieval.valid_count[:n], new_seq_lens=self._retrieval.new_seq_lens[:n])
        ops.hamming_topk(k_hash, q_hash, attn_metadata.block_table[:n], attn_metadata.seq_lens[:n], kb,
                         reduce=self.gsa_on_device_config.reduce, reduce_kvhead=self.num_key_heads > 1,
                         workspace=self._workspace, out=out, want_scores=False, inputs_stable=True,
                         cache_append_only=self.decode_only, **self._forced())
        block_table_decode = out.physical[:, 0, :]
        topk = kb
        if self.decode_only:
            self.new_block_table[:n, :topk] = block_table_decode
            self.new_block_table[:n, topk:] = 0
            attn_metadata.block_table = self.new_block_table
            self.new_seq_lens[:n] = self.topk_seq_lens_qwen
            attn_metadata.seq_lens = self.new_seq_lens
        else:
            ids = self.decode_req_ids
            self.new_block_table[ids, :topk] = block_table_decode[ids, :topk]
            self.new_block_table[ids, topk:] = 0
            attn_metadata.block_table = self.new_block_table
            self.new_seq_lens.index_copy_(0, ids, self.topk_seq_lens_qwen[ids])
            attn_metadata.seq_lens = self.new_seq_lens
        self.topk_block_table = attn_metadata.block_table
        self.topk_seq_lens = attn_metadata.seq_lens

    # ---- hooks ---------------------------------------------------------------------------------------
    def attention_begin(self, query, key, value, layer_name, forward_context, output=None, phase=None, k_hash=None,
                        decode_ql_nope=None, decode_q_pe=None):
        attn_metadata = self.get_layer_attn_metadata(forward_context, layer_name)
        is_rollback_layer, is_skip_hash_layer = self.get_layer_state(layer_name)
        # key codes are cached even while retrieval is off, so that it can switch on later
        if not is_rollback_layer and not is_skip_hash_layer:
            if self.is_mla:
                self.cache_k_hash_mla_cuda(key, value, k_hash, attn_metadata, forward_context, layer_name)
            else:
                self.cache_k_hash_gqa_cuda(key, attn_metadata, k_hash, forward_context, layer_name)
        if not self.gsa_enabled:
            return query, key, value, output
        if self.is_mla:
            if phase == "decode":
                self.update_decode_topk_mla_cuda(is_rollback_layer, is_skip_hash_layer, attn_metadata, decode_ql_nope,
                                                 decode_q_pe, k_hash)
            return query, key, value, output
        if self.has_decode and not is_rollback_layer:
            if is_skip_hash_layer:
                attn_metadata.block_table = self.topk_block_table  # reuse the previous layer's selection
                attn_metadata.seq_lens = self.topk_seq_lens
            else:
                self.update_decode_topk_gqa_cuda(query, k_hash, attn_metadata)
        return query, key, value, output

    def attention_finished(self, query, key, value, attn_output, layer_name, forward_context, phase=None) -> None:
        if not self.gsa_enabled:
            return
        attn_metadata = self.get_layer_attn_metadata(forward_context, layer_name)
        if self.is_mla:
            if phase == "decode":
                is_rollback_layer, _ = self.get_layer_state(layer_name)
                if not is_rollback_layer:
                    dec = attn_metadata.decode
                    dec.block_table = self.ori_block_table_decode
                    dec.seq_lens = self.ori_seq_lens_decode
                    dec.tile_scheduler_metadata = self.origin_tile_scheduler_metadata
                    dec.num_splits = self.origin_num_splits
            return
        if self.has_decode:
            is_rollback_layer, _ = self.get_layer_state(layer_name)
            if not is_rollback_layer:
                attn_metadata.block_table = self.ori_block_table_decode
                attn_metadata.seq_lens = self.ori_seq_lens_decode

    def request_begin(self, request_id: ReqType, prompt_token_ids: List[int]):
        pass

    def request_finished_in_scheduler(self, request_id: ReqType):
        pass

    def execute_begin(self, scheduler_output):
        pass

    def execute_finished(self, logits_indices: torch.Tensor):
        self.has_decode = False
        self.gsa_enabled = False
        self.decode_only = False
        self.has_pc_hit = False
        return logits_indices

    def estimate_num_slots_sparsed(self, request) -> int:
        return INVALID_SLOT

    def initialize_kv_hash_cache_tensors(self, kv_caches, device):
        """Pairs every layer's KV cache with its code cache: ``kv_caches[layer] = (kv_cache, khash_cache)``.  The code
        cache has the K cache's shape with the last dimension divided by 16 - one bit per key element, stored as bf16
        words like the reference's (gsa_on_device.py:1020-1032) - and is None for layers that never retrieve."""
        bits_per_word = torch.bfloat16.itemsize * 8
        for name in list(kv_caches):
            kv_cache = kv_caches[name]
            rollback, skip = self.get_layer_state(name)
            khash_cache = None
            if not (rollback or skip):
                k_shape = (kv_cache if self.is_mla else kv_cache[0]).shape
                khash_cache = torch.zeros(tuple(k_shape[:-1]) + (k_shape[-1] // bits_per_word,), dtype=torch.bfloat16,
                                          device=device)
            kv_caches[name] = (kv_cache, khash_cache)

    # ---- per-step bookkeeping (host) -------------------------------------------------------------------
    def rebuild_prefix_cache_info_for_req(self, block_table_row, num_prompt_tokens: int, qlen: int, block_size: int):
        """(prefix tokens, prefix blocks, their block ids, slot of every prefix token) of a first prefill chunk that
        computes ``qlen`` of the prompt's tokens (same return value as the reference's method of this name,
        gsa_on_device.py:1142-1174)."""
        layout = prefix_layout(num_prompt_tokens, qlen, block_size)
        if layout.empty:
            empty = block_table_row[:0]
            return 0, 0, empty, empty
        ids = block_table_row[: layout.n_blocks]
        return layout.n_tokens, layout.n_blocks, ids, prefix_slots(ids, layout, block_size, self.token_idx_buf)

    def get_seq_lens(self, attn_metadata):
        """Sequence lengths of the step (gsa_on_device.py:1211-1233); MLA metadata keeps them per phase."""
        if not self.is_mla:
            return getattr(attn_metadata, "seq_lens", None)
        dec = getattr(attn_metadata, "decode", None)
        if dec is not None:
            return getattr(dec, "seq_lens", None)
        pre = getattr(attn_metadata, "prefill", None)
        if pre is None:
            return None
        chunked = getattr(pre, "chunked_context", None)
        if chunked is not None:
            return getattr(chunked, "seq_lens", None)
        qsl = getattr(pre, "query_start_loc", None)
        if qsl is not None:
            return qsl[1:] - qsl[:-1]
        return getattr(pre, "seq_lens", None)

    def get_block_table_row(self, attn_metadata, req_row_id, qlen):
        """Block-table row of a request (gsa_on_device.py:1176-1209): MLA splits the table by phase."""
        if not self.is_mla:
            return attn_metadata.block_table[req_row_id]
        dec = getattr(attn_metadata, "decode", None)
        pre = getattr(attn_metadata, "prefill", None)
        num_decode_rows = int(dec.block_table.size(0)) if dec is not None else 0
        if qlen == 1 and dec is not None and req_row_id < num_decode_rows:
            return dec.block_table[req_row_id]
        if pre is not None:
            local = req_row_id - num_decode_rows
            if 0 <= local < int(pre.block_table.size(0)):
                return pre.block_table[local]
        raise RuntimeError(f"Failed to resolve MLA block_table row for request: req_row_id={req_row_id}, qlen={qlen}, "
                           f"num_decode_rows={num_decode_rows}")

    def prepare_cuda_decode_sparse_meta(self, attn_metadata, num_decodes):
        n = self.num_reqs
        self.full_seq_lens[:n].copy_(attn_metadata.seq_lens[:n], True)
        cols = attn_metadata.block_table.shape[1]
        self.full_block_table[:n, :cols].copy_(attn_metadata.block_table[:n], True)
        self.ori_seq_lens_decode = self.full_seq_lens[:n]
        self.ori_block_table_decode = self.full_block_table[:n, :cols]
        if not self.decode_only:
            self.decode_req_ids_buf.copy_to_gpu(num_decodes)
            self.decode_req_ids = self.decode_req_ids_buf.gpu[:num_decodes]
        self.topk_seq_lens_qwen = update_seq_lens(attn_metadata.seq_lens, topk_token=self.hash_topk_tokens,
                                                  block_size=self.block_size)
        self.new_block_table = attn_metadata.block_table
        self.new_seq_lens = attn_metadata.seq_lens

    def build_sparse_meta(self, scheduler_output, requests, input_batch, attn_metadata) -> Optional[UcmSparseMetadata]:
        self.num_reqs = len(scheduler_output.num_scheduled_tokens)
        if isinstance(attn_metadata, dict):
            attn_metadata = next(iter(attn_metadata.values()))
        seq_lens = self.get_seq_lens(attn_metadata)
        if seq_lens is None:
            return None
        # retrieval is on only when enough long requests run together (one host sync per step)
        num_long_reqs = int((seq_lens[: self.num_reqs] >= self.seq_len_threshold).sum().item())
        self.gsa_enabled = num_long_reqs >= self.concurrency_threshold

        q_lens = attn_metadata.query_start_loc[1:] - attn_metadata.query_start_loc[:-1]
        plan = self.phases.plan_step(
            scheduler_output.num_scheduled_tokens, requests, input_batch.req_id_to_index,
            lambda row: int(q_lens[row]), self.block_size,
            getattr(scheduler_output, "num_external_computed_tokens_per_req", None))
        self.step_plan = plan
        num_decodes = len(plan.decode_rows)
        self.decode_req_ids_buf.clear()
        self.decode_req_ids_buf.np[:num_decodes] = plan.decode_rows
        # prefix hits: their blocks are re-hashed in place by the first layer that sees them
        tok0 = blk0 = 0
        for hit in plan.prefix_hits:
            lay = hit.layout
            row = self.get_block_table_row(attn_metadata, hit.row, int(q_lens[hit.row]))
            ids = row[: lay.n_blocks]
            self.prefix_slot_mapping_buf[tok0: tok0 + lay.n_tokens] = prefix_slots(ids, lay, self.block_size,
                                                                                   self.token_idx_buf)
            self.prefix_block_ids_buf[blk0: blk0 + lay.n_blocks] = ids
            self.prefix_block_tokens_buf[blk0: blk0 + lay.n_blocks] = self.block_size
            self.prefix_block_tokens_buf[blk0 + lay.n_blocks - 1] = lay.tail_tokens
            tok0 += lay.n_tokens
            blk0 += lay.n_blocks
        self.has_pc_hit = bool(plan.prefix_hits)
        if self.has_pc_hit:
            self.prefix_slot_mapping = self.prefix_slot_mapping_buf[:tok0]
            self.prefix_block_ids = self.prefix_block_ids_buf[:blk0]
            self.prefix_block_tokens = self.prefix_block_tokens_buf[:blk0]
        if self.is_mla or not self.gsa_enabled:
            return None
        self.has_decode = plan.has_decode
        self.decode_only = plan.decode_only
        if self.has_decode:
            self.prepare_cuda_decode_sparse_meta(attn_metadata, num_decodes)
        return None

    def update_states(self, scheduler_output) -> None:
        """Finished requests are forgotten; so are requests resumed after a preemption, which start over as a first
        prefill (gsa_on_device.py:1407-1421)."""
        self.phases.forget_many(scheduler_output.finished_req_ids)
        cached = scheduler_output.scheduled_cached_reqs
        self.phases.forget_many(r for r, resumed in zip(cached.req_ids, cached.resumed_from_preemption) if resumed)

    def request_finished_in_worker(self, request_id: ReqType):
        self.phases.forget(request_id)
