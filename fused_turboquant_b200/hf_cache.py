"""Compressed KV cache for HF-style attention forwards, stored in pre-allocated paged pools.

Drop-in for ``CompressedKVCache`` of the reference
(src/fused_turboquant/hf/fused_cache.py:140-360): same constructor ``(quantizer,
compress_v=True)``, same methods (``set_layer_quantizer[_v]``, ``get_layer_quantizer[_v]``,
``store_compressed_key / _value / _kv``, ``get_compressed_key / _value``, ``decode_values``,
``reset``) and, when ``transformers`` is importable, the same base class ``DynamicCache`` -- the
reference's patched forward stores through these methods and then calls ``DynamicCache.update``
with one-element dummy slices for the length bookkeeping (fused_cache.py:559-574); that keeps
working unchanged.

What differs is underneath.  The reference grows two tensors per layer with ``torch.cat`` on
every step (fused_cache.py:194-222) and its decode branch materialises dense K scores and dense
V (fused_cache.py:576-624).  Here a layer's K and V codes go, in one fused encode launch, into a
``PagedKVPool`` (one per layer, so layers may use different bit widths), and
``decode_attention`` runs the fused paged kernel over it.  ``get_compressed_key/value`` still
hand out the reference's contiguous dict format (a gather, for callers that want the codes).

Options beyond the reference's constructor are keyword-only: ``max_seq_len`` (capacity per
sequence, fixed), ``batch_size`` / ``num_kv_heads`` / ``n_layers`` / ``device`` (all four given:
every pool is allocated at construction, nothing is allocated inside a forward), ``quantizer_v``.
Sequences of a batch may have different lengths: ``store_compressed_kv(..., new_lens=...)``
appends only the first ``new_lens[b]`` of the ``q_len`` new tokens of sequence ``b`` (right-padded
prompts), and every later token of that sequence lands behind its own last one.
With ``compress_v=False`` (reference: fused_cache.py:559-570, 619-624) only keys are compressed;
values stay with the caller / ``DynamicCache.update`` and ``decode_attention`` takes them as
``full_values``.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import _trace, kernels
from .paged import PagedKVPool
from .quantizer import CompressedTensor, TurboQuantMSE

try:  # the reference's base class, when transformers is installed
    from transformers import DynamicCache as _Base
    _HAS_DYNAMIC_CACHE = True
except Exception:  # pragma: no cover - transformers missing or broken
    _Base = object
    _HAS_DYNAMIC_CACHE = False

logger = _trace.get_logger(__name__)
_PAGE = 16


class CompressedKVCache(_Base):
    def __init__(self, quantizer: TurboQuantMSE, compress_v: bool = True, *,
                 max_seq_len: int = 4096, batch_size: int | None = None,
                 num_kv_heads: int | None = None, n_layers: int | None = None, device=None,
                 quantizer_v: TurboQuantMSE | None = None):
        if _HAS_DYNAMIC_CACHE:
            super().__init__()
        self.tq = quantizer
        self._tq_v_default = quantizer_v
        if quantizer_v is not None:
            self._check_pair(quantizer, quantizer_v)
        self._layer_tq: dict[int, TurboQuantMSE] = {}
        self._layer_tq_v: dict[int, TurboQuantMSE] = {}
        self.compress_v = compress_v
        self.max_blocks = (max_seq_len + _PAGE - 1) // _PAGE
        self.max_seq_len = self.max_blocks * _PAGE
        self._pools: dict[int, PagedKVPool] = {}          # layer -> pool (compress_v layers)
        self._k_only: dict[int, Optional[dict]] = {}      # layer -> reference dict (K-only layers)
        self.block_table: Optional[torch.Tensor] = None
        self._lens: dict[int, torch.Tensor] = {}          # layer -> int32 [B] tokens stored
        self._max_len: dict[int, int] = {}                # layer -> host-side upper bound
        self._k_pending: dict[int, torch.Tensor] = {}
        self.batch: Optional[int] = None
        self._hkv: Optional[int] = None
        if None not in (batch_size, num_kv_heads, n_layers, device):
            like = torch.empty((batch_size, num_kv_heads, 0, quantizer.head_dim), device=device)
            for layer in range(n_layers):
                self._ensure_layer(layer, like)
            logger.info("CompressedKVCache: %d layers pre-allocated for batch %d x %d tokens",
                        n_layers, batch_size, self.max_seq_len)

    # ---- per-layer quantizers (reference: fused_cache.py:167-192) ---------------------------
    @staticmethod
    def _check_pair(tq_k: TurboQuantMSE, tq_v: TurboQuantMSE) -> None:
        if tq_v.head_dim != tq_k.head_dim:
            raise ValueError("key and value quantizers must agree on head_dim")
        if getattr(tq_v, "seed", None) != getattr(tq_k, "seed", None):
            raise ValueError("key and value quantizers must share the rotation seed: one sign table "
                             "serves the keys and the values of a pool")

    def set_layer_quantizer(self, layer_idx: int, tq: TurboQuantMSE) -> None:
        """Per-layer quantizer for K (and V, unless V is set separately); set before the layer's first store."""
        if layer_idx in self._pools or layer_idx in self._k_only:
            raise RuntimeError(f"layer {layer_idx} already holds tokens: reset() first")
        self._layer_tq[layer_idx] = tq

    def set_layer_quantizer_v(self, layer_idx: int, tq: TurboQuantMSE) -> None:
        if layer_idx in self._pools or layer_idx in self._k_only:
            raise RuntimeError(f"layer {layer_idx} already holds tokens: reset() first")
        self._check_pair(self.get_layer_quantizer(layer_idx), tq)
        self._layer_tq_v[layer_idx] = tq

    def get_layer_quantizer(self, layer_idx: int) -> TurboQuantMSE:
        return self._layer_tq.get(layer_idx, self.tq)

    def get_layer_quantizer_v(self, layer_idx: int) -> TurboQuantMSE:
        if layer_idx in self._layer_tq_v:
            return self._layer_tq_v[layer_idx]
        if layer_idx in self._layer_tq:
            return self._layer_tq[layer_idx]
        return self._tq_v_default or self.tq

    # ---- bookkeeping --------------------------------------------------------------------------
    def get_seq_length(self, layer_idx: int = 0, *args, **kwargs) -> int:
        """Tokens stored in the layer (longest sequence).  Falls back to DynamicCache's own count
        when nothing was stored through the compressed path."""
        n = self._max_len.get(layer_idx, 0)
        if n == 0 and _HAS_DYNAMIC_CACHE:
            try:
                return int(super().get_seq_length(layer_idx, *args, **kwargs))
            except Exception:
                return 0
        return n

    def seq_lens(self, layer_idx: int) -> Optional[torch.Tensor]:
        """int32 [B] tokens stored per sequence (device tensor), or None before the first store."""
        return self._lens.get(layer_idx)

    def reset(self):
        """Forget every stored token; pools stay allocated and are reused."""
        for t in self._lens.values():
            t.zero_()
        self._max_len.clear()
        self._k_only = {k: None for k in self._k_only}
        self._k_pending.clear()
        if _HAS_DYNAMIC_CACHE and hasattr(self, "layers"):
            self.layers.clear()

    def _ensure_layer(self, layer_idx: int, like: torch.Tensor) -> None:
        B, hkv, _, d = like.shape
        if self.batch is None:
            self.batch, self._hkv = B, hkv
            # sequence b owns blocks [b * max_blocks, (b + 1) * max_blocks) of every layer's pool
            self.block_table = torch.arange(B * self.max_blocks, dtype=torch.int32,
                                            device=like.device).view(B, self.max_blocks)
        elif B != self.batch or hkv != self._hkv:
            raise ValueError("batch size / head count changed: build a new cache")
        if layer_idx not in self._lens:
            self._lens[layer_idx] = torch.zeros(B, dtype=torch.int32, device=like.device)
        if self.compress_v and layer_idx not in self._pools:
            tq_k, tq_v = self.get_layer_quantizer(layer_idx), self.get_layer_quantizer_v(layer_idx)
            self._check_pair(tq_k, tq_v)
            self._pools[layer_idx] = PagedKVPool(B * self.max_blocks, hkv, d, tq_k.bits, tq_v.bits,
                                                 n_layers=1, seed=tq_k.seed, device=like.device)

    # ---- stores -------------------------------------------------------------------------------
    def _advance(self, layer_idx: int, q_len: int, new_lens, device):
        """Slots of the q_len new tokens of every sequence (-1 = padding), lengths updated."""
        start_max = self._max_len.get(layer_idx, 0)
        if start_max + q_len > self.max_seq_len:
            raise RuntimeError(f"cache capacity {self.max_seq_len} exceeded")
        lens = self._lens[layer_idx]
        t = torch.arange(q_len, device=device, dtype=torch.int32)
        pos = lens[:, None] + t[None, :]                                   # [B, q_len]
        blk = torch.gather(self.block_table.long(), 1, (pos // _PAGE).long())
        slots = blk * _PAGE + (pos % _PAGE).long()
        if new_lens is not None:
            nl = new_lens.to(device=device, dtype=torch.int32)
            slots = torch.where(t[None, :] < nl[:, None], slots, torch.full_like(slots, -1))
            lens += nl
        else:
            lens += q_len
        self._max_len[layer_idx] = start_max + q_len
        return slots.reshape(-1)

    def store_compressed_kv(self, key_states: torch.Tensor, value_states: torch.Tensor,
                            layer_idx: int, *, new_lens: torch.Tensor | None = None) -> None:
        """Encode K and V of the new tokens in one launch and append them to the layer
        (reference: fused_cache.py:274-331).  ``new_lens`` ([B], optional): valid new tokens per
        sequence; the rest of the q_len positions is padding and is not stored."""
        if not self.compress_v:
            self.store_compressed_key(key_states, layer_idx)
            return
        if key_states.shape != value_states.shape:
            raise ValueError("key_states and value_states must have the same shape")
        self._ensure_layer(layer_idx, key_states)
        B, hkv, q_len, d = key_states.shape
        slots = self._advance(layer_idx, q_len, new_lens, key_states.device)
        k = key_states.permute(0, 2, 1, 3).reshape(B * q_len, hkv, d)
        v = value_states.permute(0, 2, 1, 3).reshape(B * q_len, hkv, d)
        self._pools[layer_idx].store(k, v, slots, layer=0)

    def store_compressed_key(self, key_states: torch.Tensor, layer_idx: int):
        """Reference: fused_cache.py:226-243.  With compressed values the keys wait for their
        values (both go to the pool in one launch); K-only layers append to the contiguous dict."""
        if self.compress_v:
            self._k_pending[layer_idx] = key_states
            return
        self._ensure_layer(layer_idx, key_states)
        tq = self.get_layer_quantizer(layer_idx)
        ct = tq.encode(key_states)
        entry = {"packed_indices": ct.indices.view(*key_states.shape[:-1], -1),
                 "norms": ct.norms.view(*key_states.shape[:-1])}
        prev = self._k_only.get(layer_idx)
        if prev is not None:
            entry = {"packed_indices": torch.cat([prev["packed_indices"], entry["packed_indices"]], dim=2),
                     "norms": torch.cat([prev["norms"], entry["norms"]], dim=2)}
        self._k_only[layer_idx] = entry
        self._lens[layer_idx] += key_states.shape[2]
        self._max_len[layer_idx] = self._max_len.get(layer_idx, 0) + key_states.shape[2]

    def store_compressed_value(self, value_states: torch.Tensor, layer_idx: int):
        """Reference: fused_cache.py:252-265."""
        if not self.compress_v:
            raise RuntimeError("this cache was built with compress_v=False: values are not stored here")
        if layer_idx not in self._k_pending:
            raise RuntimeError("store_compressed_key must be called before store_compressed_value")
        self.store_compressed_kv(self._k_pending.pop(layer_idx), value_states, layer_idx)

    # ---- fused decode -------------------------------------------------------------------------
    def decode_attention(self, query_states: torch.Tensor, layer_idx: int,
                         scale: float | None = None, *, full_values: torch.Tensor | None = None
                         ) -> torch.Tensor:
        """Attention of one query token per sequence over everything stored in the layer
        (what the reference's decode branch computes, fused_cache.py:576-624).

        query_states: [B, Hq, 1, D] (not rotated); returns [B, Hq, 1, D] in the query's dtype.
        K-only caches (compress_v=False) need ``full_values`` [B, Hkv, kv_len, D].
        """
        B, hq, q_len, d = query_states.shape
        if q_len != 1:
            raise ValueError("decode_attention takes one query token per sequence")
        if self.compress_v:
            n = self._max_len.get(layer_idx, 0)
            out = self._pools[layer_idx].decode_attention(
                query_states[:, :, 0], self.block_table, self._lens[layer_idx], max(n, 1), scale,
                layer=0)
            return out.unsqueeze(2)
        if full_values is None:
            raise ValueError("compress_v=False: pass the uncompressed values as full_values")
        tq = self.get_layer_quantizer(layer_idx)
        entry = self._k_only[layer_idx]
        scale = (d ** -0.5) if scale is None else scale
        q_rot = kernels.rht(query_states.float().reshape(-1, d).contiguous(), tq.rotation.signs)
        scores = kernels.fused_qk_scores_rht(q_rot.view(B, hq, 1, d), entry["packed_indices"],
                                             entry["norms"], tq.quantizer.levels, scale, bits=tq.bits)
        w = torch.softmax(scores, dim=-1, dtype=torch.float32).to(query_states.dtype)
        hkv = full_values.shape[1]
        v = full_values[:, :, None].expand(B, hkv, hq // hkv, *full_values.shape[2:]) \
            .reshape(B, hq, *full_values.shape[2:])
        return torch.matmul(w, v.to(query_states.dtype))

    # ---- contiguous views of the stored codes (the reference's dict format) ---------------------
    def _gather(self, layer_idx: int, which: int) -> Optional[dict]:
        n = self._max_len.get(layer_idx, 0)
        if layer_idx not in self._pools or n == 0:
            return None
        p = self._pools[layer_idx]
        rows = [p.gather_sequence(0, self.block_table[b], n) for b in range(self.batch)]
        codes = torch.stack([r[2 * which] for r in rows])
        norms = torch.stack([r[2 * which + 1] for r in rows])
        return {"packed_indices": codes, "norms": norms}

    def get_compressed_key(self, layer_idx: int) -> Optional[dict]:
        if not self.compress_v:
            return self._k_only.get(layer_idx)
        return self._gather(layer_idx, 0)

    def get_compressed_value(self, layer_idx: int) -> Optional[dict]:
        return self._gather(layer_idx, 1) if self.compress_v else None

    def decode_values(self, layer_idx: int) -> torch.Tensor:
        """Dense fp32 values [B, Hkv, kv_len, D] (reference: fused_cache.py:333-346)."""
        tq = self.get_layer_quantizer_v(layer_idx)
        entry = self.get_compressed_value(layer_idx)
        ct = CompressedTensor(indices=entry["packed_indices"], norms=entry["norms"],
                              original_dim=tq.head_dim, bits=tq.bits)
        return tq.decode(ct)
