"""Compressed KV cache for HF-style attention forwards, stored in a pre-allocated paged pool.

Mirrors ``CompressedKVCache`` of the reference (src/fused_turboquant/hf/fused_cache.py:140-360):
``store_compressed_key / store_compressed_value / store_compressed_kv``, ``get_compressed_key /
get_compressed_value``, ``decode_values``, ``get_seq_length``, ``reset``.  Where the reference
grows two tensors per layer with ``torch.cat`` on every step (fused_cache.py:194-222) and its
decode branch materialises dense K scores and dense V (fused_cache.py:576-624), this class writes
each new token once into a ``PagedKVPool`` and ``decode_attention`` runs the fused paged kernel.

Shapes follow HF: keys/values ``[batch, num_kv_heads, q_len, head_dim]``, every sequence of the
batch has the same length.  Capacity (``max_seq_len``) is fixed at construction; the pool is
allocated on the first store, when the batch size is known.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import kernels
from .paged import PagedKVPool, page_bytes
from .quantizer import CompressedTensor, TurboQuantMSE

_PAGE = 16


class CompressedKVCache:
    def __init__(self, quantizer: TurboQuantMSE, compress_v: bool = True, *, n_layers: int,
                 max_seq_len: int = 4096, quantizer_v: TurboQuantMSE | None = None):
        if not compress_v:
            raise ValueError("compress_v=False is not supported: keys and values share one pool")
        self.tq = quantizer
        self.tq_v = quantizer_v or quantizer
        if self.tq_v.head_dim != self.tq.head_dim:
            raise ValueError("key and value quantizers must agree on head_dim")
        self.compress_v = True
        self.n_layers = n_layers
        self.max_blocks = (max_seq_len + _PAGE - 1) // _PAGE
        self.max_seq_len = self.max_blocks * _PAGE
        self.pool: Optional[PagedKVPool] = None
        self.block_table: Optional[torch.Tensor] = None
        self._len = [0] * n_layers          # tokens stored per layer (host-side counters)
        self._k_pending: dict[int, torch.Tensor] = {}

    # ---- bookkeeping ---------------------------------------------------------------------
    def get_seq_length(self, layer_idx: int = 0) -> int:
        return self._len[layer_idx] if layer_idx < self.n_layers else 0

    def get_layer_quantizer(self, layer_idx: int) -> TurboQuantMSE:
        return self.tq

    def get_layer_quantizer_v(self, layer_idx: int) -> TurboQuantMSE:
        return self.tq_v

    def reset(self) -> None:
        self._len = [0] * self.n_layers
        self._k_pending.clear()

    def _ensure_pool(self, like: torch.Tensor) -> None:
        B, hkv, _, d = like.shape
        if self.pool is None:
            self.pool = PagedKVPool(B * self.max_blocks, hkv, d, self.tq.bits, self.tq_v.bits,
                                    self.n_layers, seed=self.tq.seed, device=like.device)
            # sequence b owns blocks [b * max_blocks, (b + 1) * max_blocks)
            self.block_table = torch.arange(B * self.max_blocks, dtype=torch.int32,
                                            device=like.device).view(B, self.max_blocks)
            self.batch = B
        elif B != self.batch or hkv != self.pool.num_kv_heads:
            raise ValueError("batch size / head count changed: call reset() and build a new cache")

    # ---- stores --------------------------------------------------------------------------
    def store_compressed_kv(self, key_states: torch.Tensor, value_states: torch.Tensor,
                            layer_idx: int) -> None:
        """Encode K and V of the new tokens in one launch and append them to the layer."""
        if key_states.shape != value_states.shape:
            raise ValueError("key_states and value_states must have the same shape")
        self._ensure_pool(key_states)
        B, hkv, q_len, d = key_states.shape
        start = self._len[layer_idx]
        if start + q_len > self.max_seq_len:
            raise RuntimeError(f"cache capacity {self.max_seq_len} exceeded")
        pos = torch.arange(start, start + q_len, device=key_states.device)
        slots = (self.block_table.long()[:, pos // _PAGE] * _PAGE + pos % _PAGE).reshape(-1)
        k = key_states.permute(0, 2, 1, 3).reshape(B * q_len, hkv, d)
        v = value_states.permute(0, 2, 1, 3).reshape(B * q_len, hkv, d)
        self.pool.store(k, v, slots, layer=layer_idx)
        self._len[layer_idx] = start + q_len

    def store_compressed_key(self, key_states: torch.Tensor, layer_idx: int) -> None:
        """Keys and values of a step are written together: the keys wait for their values."""
        self._k_pending[layer_idx] = key_states

    def store_compressed_value(self, value_states: torch.Tensor, layer_idx: int) -> None:
        if layer_idx not in self._k_pending:
            raise RuntimeError("store_compressed_key must be called before store_compressed_value")
        self.store_compressed_kv(self._k_pending.pop(layer_idx), value_states, layer_idx)

    # ---- fused decode --------------------------------------------------------------------
    def decode_attention(self, query_states: torch.Tensor, layer_idx: int,
                         scale: float | None = None) -> torch.Tensor:
        """Attention of one query token per sequence over everything stored in the layer.

        query_states: [B, Hq, 1, D] (not rotated); returns [B, Hq, 1, D] in the query's dtype.
        """
        B, hq, q_len, d = query_states.shape
        if q_len != 1:
            raise ValueError("decode_attention takes one query token per sequence")
        n = self._len[layer_idx]
        seq_lens = torch.full((B,), n, dtype=torch.int32, device=query_states.device)
        out = self.pool.decode_attention(query_states[:, :, 0], self.block_table, seq_lens,
                                         max(n, 1), scale, layer=layer_idx)
        return out.unsqueeze(2)

    # ---- contiguous views of the stored codes (the reference's dict format) -----------------
    def _gather(self, layer_idx: int, which: int) -> Optional[dict]:
        if self.pool is None or layer_idx >= self.n_layers or self._len[layer_idx] == 0:
            return None
        p = self.pool
        d, n = p.head_dim, self._len[layer_idx]
        pdk, pdv = d * p.key_bits // 8, d * p.value_bits // 8
        off_kn = _PAGE * pdk
        off_vc = off_kn + 2 * _PAGE
        off_vn = off_vc + _PAGE * pdv
        assert off_vn + 2 * _PAGE == page_bytes(d, p.key_bits, p.value_bits)
        pages = p.pool[layer_idx][self.block_table.long()]          # [B, blocks, Hkv, page]
        B, nblk, hkv, _ = pages.shape
        if which == 0:
            codes = pages[..., :off_kn].reshape(B, nblk, hkv, _PAGE, pdk)
            norms = pages[..., off_kn:off_vc]
        else:
            codes = pages[..., off_vc:off_vn].reshape(B, nblk, hkv, _PAGE, pdv)
            # value rows of page tokens with bit 1 set are stored with their halves exchanged
            swapped = torch.cat([codes[..., pdv // 2:], codes[..., :pdv // 2]], dim=-1)
            bit1 = (torch.arange(_PAGE, device=codes.device) & 2).bool().view(1, 1, 1, _PAGE, 1)
            codes = torch.where(bit1, swapped, codes)
            norms = pages[..., off_vn:]
        norms = norms.contiguous().view(torch.float16).reshape(B, nblk, hkv, _PAGE)
        codes = codes.permute(0, 2, 1, 3, 4).reshape(B, hkv, nblk * _PAGE, -1)[:, :, :n]
        norms = norms.permute(0, 2, 1, 3).reshape(B, hkv, nblk * _PAGE)[:, :, :n]
        return {"packed_indices": codes.contiguous(), "norms": norms.contiguous()}

    def get_compressed_key(self, layer_idx: int) -> Optional[dict]:
        return self._gather(layer_idx, 0)

    def get_compressed_value(self, layer_idx: int) -> Optional[dict]:
        return self._gather(layer_idx, 1)

    def decode_values(self, layer_idx: int) -> torch.Tensor:
        """Dense fp32 values [B, Hkv, kv_len, D] (the reference's unfused V path needs them)."""
        entry = self.get_compressed_value(layer_idx)
        ct = CompressedTensor(indices=entry["packed_indices"], norms=entry["norms"],
                              original_dim=self.tq_v.head_dim, bits=self.tq_v.bits)
        return self.tq_v.decode(ct)
