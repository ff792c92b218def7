"""Cache-shape / block-management surface of the reference's vLLM-v0 backend
(src/fused_turboquant/vllm_plugin/backend.py:51-188, cache_ops.py:20-82), without vLLM.

The arithmetic half of that backend (store + decode step) is ``PagedKVPool``; this module
keeps the shape contract and the block copy / swap operations, which are byte copies and
therefore independent of the slot layout.  Bit widths come from the same environment
variables the reference reads (TURBOQUANT_BITS, TURBOQUANT_V_BITS).
"""
from __future__ import annotations

import os
from typing import List, Tuple

import torch

from .paged import compute_compressed_elem_size, page_bytes


def _bits() -> tuple[int, int]:
    k = int(os.environ.get("TURBOQUANT_BITS", "4"))
    v_raw = os.environ.get("TURBOQUANT_V_BITS")
    return k, (int(v_raw) if v_raw else k)


def compressed_swap_blocks(src: torch.Tensor, dst: torch.Tensor, src_to_dst: torch.Tensor) -> None:
    """Copy whole blocks src[i] -> dst[j] for every (i, j) row of ``src_to_dst``
    (reference: cache_ops.py:20-38).  One indexed copy, no per-pair host loop; works across
    devices and for any block-major layout."""
    if src_to_dst.numel() == 0:
        return
    pairs = src_to_dst.reshape(-1, 2).long()
    dst.index_copy_(0, pairs[:, 1].to(dst.device), src.index_select(0, pairs[:, 0].to(src.device)).to(dst.device))


def compressed_copy_blocks(kv_caches: List[torch.Tensor], src_to_dsts: torch.Tensor) -> None:
    """Copy blocks inside every layer's cache (beam search / prefix caching; reference:
    cache_ops.py:41-61).  Caches of the v0 layout carry the K / V plane first
    ([2, num_blocks, ...]); pools of the page layout are block-major ([num_blocks, ...])."""
    if src_to_dsts.numel() == 0:
        return
    pairs = src_to_dsts.reshape(-1, 2).long()
    for cache in kv_caches:
        src, dst = pairs[:, 0].to(cache.device), pairs[:, 1].to(cache.device)
        dim = 1 if (cache.dim() == 5 and cache.shape[0] == 2) else 0
        cache.index_copy_(dim, dst, cache.index_select(dim, src))


class FusedTurboQuantBackend:
    """Shape contract and block management of the FUSED_TURBOQUANT backend."""

    name = "FUSED_TURBOQUANT"

    @staticmethod
    def get_name() -> str:
        return "FUSED_TURBOQUANT"

    @staticmethod
    def get_kv_cache_shape(num_blocks: int, block_size: int, num_kv_heads: int,
                           head_size: int) -> Tuple[int, ...]:
        """The reference's cache tensor: uint8 [2, num_blocks, block_size, Hkv, packed + 4], wide
        enough for the larger of K and V (backend.py:107-124)."""
        kb, vb = _bits()
        size = max(compute_compressed_elem_size(head_size, kb),
                   compute_compressed_elem_size(head_size, vb))
        return (2, num_blocks, block_size, num_kv_heads, size)

    @staticmethod
    def get_pool_shape(num_blocks: int, num_kv_heads: int, head_size: int) -> Tuple[int, ...]:
        """The page layout PagedKVPool uses: uint8 [num_blocks, Hkv, page_bytes], 16 tokens per
        block, no padding."""
        kb, vb = _bits()
        return (num_blocks, num_kv_heads, page_bytes(head_size, kb, vb))

    @staticmethod
    def swap_blocks(src_kv_cache: torch.Tensor, dst_kv_cache: torch.Tensor,
                    src_to_dst: torch.Tensor) -> None:
        compressed_swap_blocks(src_kv_cache, dst_kv_cache, src_to_dst)

    @staticmethod
    def copy_blocks(kv_caches: List[torch.Tensor], src_to_dsts: torch.Tensor) -> None:
        compressed_copy_blocks(kv_caches, src_to_dsts)

    @classmethod
    def is_available(cls) -> bool:
        from . import _lib
        return _lib.is_available()

    @classmethod
    def get_supported_head_sizes(cls) -> List[int]:
        """head_dim values the CUDA kernels are instantiated for (the reference also lists 512)."""
        return [64, 128, 256]

    @staticmethod
    def validate_configuration(head_size: int = 0, **kwargs) -> None:
        if head_size <= 0:
            return
        if (head_size & (head_size - 1)) != 0:
            raise ValueError(
                f"FUSED_TURBOQUANT (kind=rht) requires power-of-2 head_size for RHT, got {head_size}.")
        if head_size not in FusedTurboQuantBackend.get_supported_head_sizes():
            raise ValueError(f"head_size {head_size} has no sm_100a kernel (supported: 64, 128, 256)")
