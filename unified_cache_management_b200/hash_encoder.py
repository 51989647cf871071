"""``HashEncoder`` with the reference's interface, backed by the sm_100a encode kernels.

Mirrors ``ucm/sparse/gsa_on_device/hash_encoder.py`` (class at :373-724): same constructor
arguments, ``set_hash_weight`` / ``compute_hash`` / ``compute_hash_and_cache`` / ``_unpack_hash``,
same ``ValueError`` conditions, same packed layout (8 sign bits per uint8, LSB first).

Differences that follow from the B200 path: the projection runs as bf16 x bf16 with float32
accumulation on tensor cores, so the kernels read ``hash_weights_bf16`` (the float32 master copy
``hash_weights`` rounded once); inputs of another dtype are converted to bf16.  Only CUDA devices
are served: there is no Triton, NPU or CPU branch here.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import ops


class HashEncoder:
    def __init__(self, input_dim: int, hash_bits: int, dtype: torch.dtype, device: torch.device) -> None:
        self.input_dim = input_dim
        if hash_bits % 8 != 0:
            raise ValueError("hash_bits must be a multiple of 8")
        if hash_bits % 32 != 0:
            raise ValueError("hash_bits must be a multiple of 32 on this backend (codes are stored as 32-bit words)")
        self.hash_bits = hash_bits
        self.hash_numbers = hash_bits // 8  # uint8 numbers per code
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise ValueError(f"Unsupported device type: {self.device.type} (this backend is CUDA-only)")
        # the reference falls back to float32 weights for bf16 models because QR has no bf16 kernel
        # (hash_encoder.py:403-406); the master copy here is always float32
        self.dtype = torch.float32 if dtype == torch.bfloat16 else dtype
        self._init_hash_weights()
        self._init_bit_masks()

    def _init_hash_weights(self) -> None:
        # Haar-distributed orthogonal matrix: Gaussian -> QR -> fix the signs (hash_encoder.py:413-427)
        g = torch.normal(mean=0, std=2, size=(self.input_dim, self.hash_bits), dtype=torch.float32, device=self.device)
        q, r = torch.linalg.qr(g)
        self.hash_weights = (q * torch.sign(torch.diag(r))).to(self.dtype)
        self._refresh_bf16()

    def _refresh_bf16(self) -> None:
        self.hash_weights_bf16 = self.hash_weights.to(torch.bfloat16).contiguous()

    def set_hash_weight(self, hash_weights: torch.Tensor) -> None:
        if hash_weights.shape != (self.input_dim, self.hash_bits):
            raise ValueError(
                f"hash_weights shape {hash_weights.shape} does not match required shape {(self.input_dim, self.hash_bits)}")
        if hash_weights.dtype != self.dtype and hash_weights.dtype != torch.bfloat16:
            raise ValueError(f"hash_weights dtype {hash_weights.dtype} does not match required dtype {self.dtype}")
        if hash_weights.device != self.device:
            raise ValueError(f"hash_weights device {hash_weights.device} does not match required device {self.device}")
        self.hash_weights.copy_(hash_weights.to(self.dtype))
        self._refresh_bf16()

    def _init_bit_masks(self) -> None:
        self.bit_masks = torch.pow(2, torch.arange(8, dtype=torch.uint8, device=self.device))

    def _as_bf16(self, x: torch.Tensor) -> torch.Tensor:
        return x if x.dtype == torch.bfloat16 else x.to(torch.bfloat16)

    def compute_hash(self, x: torch.Tensor) -> torch.Tensor:
        """x (..., input_dim) -> uint8 (..., hash_bits // 8)."""
        if x.shape[-1] != self.input_dim:
            raise ValueError(f"x must be of shape (..., {self.input_dim}), but got {x.shape}")
        if x.device != self.device:
            raise ValueError(f"x device {x.device} does not match required device {self.device}")
        words = ops.hash_encode(self._as_bf16(x), self.hash_weights_bf16)
        return words.view(torch.uint8)

    def compute_hash_grouped(self, query: torch.Tensor, group: int) -> torch.Tensor:
        """[T, Hq, D] -> uint8 [T, Hq/group, hash_bits//8]: mean over each run of ``group`` heads
        (rounded to bf16 like ``query.view(T,Hkv,G,D).mean(2)``), then encode, in one launch."""
        words = ops.hash_encode_query(self._as_bf16(query), self.hash_weights_bf16, group_mean=group)
        return words.view(torch.uint8)

    def _reinterpret_cache_as_u8(self, cache: torch.Tensor) -> torch.Tensor:
        if cache.dtype == torch.uint8:
            if cache.shape[-1] != self.hash_numbers:
                raise ValueError(f"uint8 cache last dim mismatch: got {cache.shape[-1]}, expected {self.hash_numbers}")
            return cache
        if cache.dtype == torch.bfloat16:
            if cache.shape[-1] != self.hash_numbers // 2:
                raise ValueError(
                    f"bfloat16 cache last dim mismatch: got {cache.shape[-1]}, expected {self.hash_numbers // 2}")
            return cache.view(torch.uint8)
        if cache.dtype == torch.int32:
            if cache.shape[-1] != self.hash_numbers // 4:
                raise ValueError(f"int32 cache last dim mismatch: got {cache.shape[-1]}, expected {self.hash_numbers // 4}")
            return cache.view(torch.uint8)
        raise ValueError(f"unsupported k_hash_cache dtype {cache.dtype}, only uint8 / bfloat16 / int32 are supported")

    def compute_hash_and_cache(self, x: torch.Tensor, slot_mapping: torch.Tensor, k_hash_cache: torch.Tensor,
                               block_size: int = 128, **_unused_tile_hints) -> torch.Tensor:
        """Encode x [T,H,K] and write token t's codes into slot ``slot_mapping[t]`` of the paged cache
        [NB, BS, H, ?] (uint8, bf16 or int32 storage).  One launch.  Tile-size keywords of the Triton
        version are accepted and ignored."""
        if x.ndim != 3:
            raise ValueError(f"x must be [T,H,K], got {x.shape}")
        if slot_mapping.ndim != 1:
            raise ValueError(f"slot_mapping must be [T], got {slot_mapping.shape}")
        if k_hash_cache.ndim != 4:
            raise ValueError(f"k_hash_cache must be rank-4, got {k_hash_cache.shape}")
        if x.shape[-1] != self.input_dim:
            raise ValueError(f"x last dim must be {self.input_dim}, got {x.shape[-1]}")
        for name, t in (("x", x), ("slot_mapping", slot_mapping), ("k_hash_cache", k_hash_cache)):
            if t.device != self.device:
                raise ValueError(f"{name} device {t.device} does not match required device {self.device}")
        t_, h, _ = x.shape
        if slot_mapping.shape[0] != t_:
            raise ValueError(f"slot_mapping length {slot_mapping.shape[0]} != T {t_}")
        if k_hash_cache.shape[1] != block_size:
            raise ValueError(f"k_hash_cache.shape[1]={k_hash_cache.shape[1]} != block_size={block_size}")
        if k_hash_cache.shape[2] != h:
            raise ValueError(f"k_hash_cache.shape[2]={k_hash_cache.shape[2]} != H={h}")
        cache_u8 = self._reinterpret_cache_as_u8(k_hash_cache)
        ops.hash_encode_and_cache(self._as_bf16(x), slot_mapping, cache_u8, self.hash_weights_bf16)
        return k_hash_cache

    def compute_hash_of_blocks(self, k_cache: torch.Tensor, block_ids: torch.Tensor, k_hash_cache: torch.Tensor,
                               block_tokens: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Encode the keys of the listed blocks of the paged K cache [NB, BS, H, K] into the same blocks of the
        code cache, reading the blocks where they lie.  Same result as gathering the blocks and calling
        ``compute_hash_and_cache`` with their slot mapping (what the reference does on a prefix-cache hit,
        gsa_on_device.py:574-588); ``block_tokens[i]`` limits block i to its first tokens."""
        if k_cache.ndim != 4 or k_hash_cache.ndim != 4:
            raise ValueError("k_cache and k_hash_cache must be rank-4")
        if k_cache.shape[-1] != self.input_dim:
            raise ValueError(f"k_cache last dim must be {self.input_dim}, got {k_cache.shape[-1]}")
        if k_cache.dtype != torch.bfloat16:
            raise ValueError("the paged K cache must be bf16 (it is read in place)")
        if k_hash_cache.shape[1] != k_cache.shape[1] or k_hash_cache.shape[2] != k_cache.shape[2]:
            raise ValueError("k_hash_cache and k_cache disagree on block size or head count")
        cache_u8 = self._reinterpret_cache_as_u8(k_hash_cache)
        ops.hash_encode_blocks(k_cache, block_ids.to(torch.int32), cache_u8, self.hash_weights_bf16,
                               block_tokens=None if block_tokens is None else block_tokens.to(torch.int32))
        return k_hash_cache

    def _unpack_hash(self, packed_codes: torch.Tensor) -> torch.Tensor:
        """uint8 (..., hash_numbers) -> float16 (..., hash_bits) of +-1 (debug/analysis helper)."""
        if packed_codes.shape[-1] != self.hash_numbers:
            raise ValueError(f"packed_codes must be of shape (..., {self.hash_numbers}), but got {packed_codes.shape}")
        if packed_codes.device != self.device:
            raise ValueError(f"packed_codes device {packed_codes.device} does not match required device {self.device}")
        if packed_codes.dtype != torch.uint8:
            raise ValueError(f"packed_codes dtype {packed_codes.dtype} is not torch.uint8")
        bits = (packed_codes.unsqueeze(-1) & self.bit_masks) > 0
        return (bits.to(torch.float16) * 2 - 1).reshape(packed_codes.shape[:-1] + (self.hash_bits,))
