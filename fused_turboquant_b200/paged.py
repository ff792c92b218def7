"""Paged compressed KV pool: fused store and paged decode attention.

Plays the role of the reference's vLLM-v0 attention impl on its paged cache
(src/fused_turboquant/vllm_plugin/attention_impl.py:190-254 for the store,
:431-521 for the decode step, cache_ops.py:64-205 for the slot layout) with
the per-token Python loops replaced by two kernels.

Pool layout (per layer): u8 [num_blocks, Hkv, page_bytes]; a page holds the 16
tokens of one (block, head):  K codes | K norms fp16 | V codes | V norms fp16.
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib, _trace, codebook, kernels
from .kernels import _DT, _host_table, _ptr, _require_cuda, _stream

logger = _trace.get_logger(__name__)

PAGE_TOKENS = 16


def page_bytes(head_dim: int, bits_k: int, bits_v: int) -> int:
    n = int(_lib.load().ftq_page_bytes(head_dim, bits_k, bits_v))
    if n < 0:
        raise ValueError(f"unsupported head_dim={head_dim} / bits K={bits_k} V={bits_v}")
    return n


def compute_compressed_elem_size(head_dim: int, bits: int) -> int:
    """Bytes per (token, head) slot of the reference's v0 layout: packed codes + fp32 norm
    (reference: vllm_plugin/cache_ops.py:64-82)."""
    return kernels.packed_dim(head_dim, bits) + 4


class PagedKVPool:
    """Compressed paged KV cache for ``n_layers`` layers of one model shard."""

    def __init__(self, num_blocks: int, num_kv_heads: int, head_dim: int, key_bits: int = 4,
                 value_bits: int | None = None, n_layers: int = 1, seed: int = 42,
                 device="cuda"):
        value_bits = key_bits if value_bits is None else value_bits
        if head_dim < 1 or (head_dim & (head_dim - 1)) != 0:
            raise ValueError(f"head_dim must be a power of 2, got {head_dim}")
        for b in (key_bits, value_bits):
            if b not in (2, 3, 4):
                raise ValueError(f"bits must be 2, 3, or 4, got {b}")
        self.num_blocks, self.num_kv_heads, self.head_dim = num_blocks, num_kv_heads, head_dim
        self.key_bits, self.value_bits, self.n_layers = key_bits, value_bits, n_layers
        self.page_bytes = page_bytes(head_dim, key_bits, value_bits)
        self.signs = codebook.rht_signs(head_dim, seed)
        self.bounds_k, self.levels_k = codebook.codebook_f32(head_dim, key_bits)
        self.bounds_v, self.levels_v = codebook.codebook_f32(head_dim, value_bits)
        self.pool = torch.zeros((n_layers, num_blocks, num_kv_heads, self.page_bytes),
                                dtype=torch.uint8, device=device)
        logger.info("paged compressed KV pool: %d layers x %d blocks x %d KV heads, head_dim %d, "
                    "K%d/V%d, %d bytes per 16-token page (%.1f MiB)", n_layers, num_blocks,
                    num_kv_heads, head_dim, key_bits, value_bits, self.page_bytes,
                    self.pool.numel() / 2 ** 20)

    @property
    def layer_stride(self) -> int:
        return self.num_blocks * self.num_kv_heads * self.page_bytes

    def store(self, key: torch.Tensor, value: torch.Tensor, slot_mapping: torch.Tensor,
              layer: int | None = None) -> None:
        """Encode and scatter new tokens.

        key/value: [n_tokens, Hkv, D] (one layer, ``layer`` given) or
        [n_layers, n_tokens, Hkv, D] (all layers at once, ``layer`` None).
        slot_mapping: [n_tokens] int64, slot = block * 16 + offset; negative = skip.
        """
        _require_cuda(key, "key")
        if key.dtype not in _DT:
            key, value = key.float(), value.float()
        key, value = key.contiguous(), value.contiguous().to(key.dtype)
        sm = slot_mapping.to(device=key.device, dtype=torch.int64).contiguous()
        if layer is None:
            L, n_tokens = key.shape[0], key.shape[1]
            pool = self.pool
        else:
            L, n_tokens = 1, key.shape[0]
            pool = self.pool[layer]
        D, H = self.head_dim, self.num_kv_heads
        with torch.cuda.device(key.device), _trace.nvtx("ftq.store"):
            rc = _lib.load().ftq_paged_store(
                _ptr(key), _ptr(value), _DT[key.dtype], n_tokens, H, D, H * D, D, self.key_bits,
                self.value_bits, _lib.fptr(self.signs), _lib.fptr(self.bounds_k),
                _lib.fptr(self.bounds_v), _ptr(pool), self.num_blocks, _ptr(sm), L,
                n_tokens * H * D, self.layer_stride, _stream(key.device))
        _lib.check(rc, "ftq_paged_store")

    def workspace_bytes(self, batch: int, num_q_heads: int, max_seq_len: int,
                        n_layers: int = 1) -> int:
        return kernels.workspace_bytes(batch, num_q_heads, self.num_kv_heads, self.head_dim,
                                       max_seq_len, n_layers)

    def decode_attention(self, q: torch.Tensor, block_table: torch.Tensor,
                         seq_lens: torch.Tensor, max_seq_len: int, scale: float | None = None,
                         layer: int | None = None, out: torch.Tensor | None = None,
                         workspace: torch.Tensor | None = None) -> torch.Tensor:
        """One decode step of attention over the pool.

        q: [B, Hq, D] (``layer`` given) or [n_layers, B, Hq, D] (``layer`` None), not rotated.
        block_table: [B, max_blocks] int32; seq_lens: [B] int32.  Returns q-shaped output.
        No host synchronisation; graph-capturable when out/workspace are passed in.
        """
        _require_cuda(q, "q")
        if q.dtype not in _DT:
            q = q.float()
        q = q.contiguous()
        if layer is None:
            L, B, Hq, D = q.shape
            pool = self.pool
        else:
            L = 1
            B, Hq, D = q.shape
            pool = self.pool[layer]
        scale = (D ** -0.5) if scale is None else scale
        out = torch.empty_like(q) if out is None else out
        bt = block_table.to(device=q.device, dtype=torch.int32).contiguous()
        sl = seq_lens.to(device=q.device, dtype=torch.int32).contiguous()
        need = self.workspace_bytes(B, Hq, max_seq_len, L)
        ws = workspace if workspace is not None else kernels.get_workspace(q.device, need)
        with torch.cuda.device(q.device), _trace.nvtx("ftq.decode"):
            rc = _lib.load().ftq_paged_decode_attn(
                _ptr(q), _DT[q.dtype], _ptr(out), _DT[out.dtype], _ptr(pool), self.num_blocks,
                self.layer_stride, L, _ptr(bt), bt.shape[1], _ptr(sl), int(max_seq_len), B, Hq,
                self.num_kv_heads, D, self.key_bits, self.value_bits, _lib.fptr(self.levels_k),
                _lib.fptr(self.levels_v), _lib.fptr(self.signs), float(scale), _ptr(ws),
                ws.numel(), _stream(q.device))
        _lib.check(rc, "ftq_paged_decode_attn")
        self._last_decode = (ws, B, Hq, int(max_seq_len), L, q.device)
        return out

    def decode_status(self) -> int:
        """Status bits of this pool's last ``decode_attention`` call (0: nothing to report;
        1: a block id outside the pool was met, 2: a bounded wait inside a kernel ran out -- the
        rows concerned are NaN either way).  Copies one word back and synchronises the current
        stream; the kernels themselves never trap on such input."""
        last = getattr(self, "_last_decode", None)
        if last is None:
            return 0
        ws, B, Hq, max_seq_len, L, device = last
        bits = ctypes.c_int(0)
        with torch.cuda.device(device):
            rc = _lib.load().ftq_paged_decode_status(
                _ptr(ws), B, Hq, self.num_kv_heads, self.head_dim, max_seq_len, L, _stream(device),
                ctypes.byref(bits))
        if rc not in (0, -5):
            _lib.check(rc, "ftq_paged_decode_status")
        return int(bits.value)


    def gather_sequence(self, layer: int, block_row: torch.Tensor, seq_len: int):
        """Contiguous copy of one sequence's compressed K/V, in the reference's tensor format.

        block_row: [max_blocks] block ids of the sequence.  Returns
        (k_codes u8 [Hkv, S, pdk], k_norms f16 [Hkv, S], v_codes u8 [Hkv, S, pdv], v_norms f16
        [Hkv, S]) on the pool's device -- the arguments of the reference's
        ``flash_decode_compressed`` / ``get_compressed_key`` dict
        (kernels/triton_flash_decode.py:224-236, hf/fused_cache.py:333-346) for that sequence.
        Plain tensor indexing (a diagnostic / interop path, not the decode path).
        """
        S = int(seq_len)
        H, D = self.num_kv_heads, self.head_dim
        pdk, pdv = kernels.packed_dim(D, self.key_bits), kernels.packed_dim(D, self.value_bits)
        nb = (S + PAGE_TOKENS - 1) // PAGE_TOKENS
        ids = block_row[:nb].to(device=self.pool.device, dtype=torch.long)
        pages = self.pool[layer].index_select(0, ids)            # [nb, H, page_bytes]
        off_kn = PAGE_TOKENS * pdk
        off_vc = off_kn + 2 * PAGE_TOKENS
        off_vn = off_vc + PAGE_TOKENS * pdv

        def rows(lo, width):   # [nb, H, 16*width] -> [H, nb*16, width]
            x = pages[:, :, lo:lo + PAGE_TOKENS * width].reshape(nb, H, PAGE_TOKENS, width)
            return x.permute(1, 0, 2, 3).reshape(H, nb * PAGE_TOKENS, width)

        k_codes = rows(0, pdk)[:, :S].contiguous()
        v_raw = rows(off_vc, pdv)
        # V rows of page tokens with bit 1 set are stored with their halves exchanged
        swapped = torch.cat([v_raw[..., pdv // 2:], v_raw[..., :pdv // 2]], dim=-1)
        tok = torch.arange(nb * PAGE_TOKENS, device=pages.device)
        v_codes = torch.where(((tok & 2) != 0)[None, :, None], swapped, v_raw)[:, :S].contiguous()
        k_norms = rows(off_kn, 2).contiguous().view(torch.float16).reshape(H, -1)[:, :S].contiguous()
        v_norms = rows(off_vn, 2).contiguous().view(torch.float16).reshape(H, -1)[:, :S].contiguous()
        return k_codes, k_norms, v_codes, v_norms

    def continuation_attention(self, q: torch.Tensor, block_table: torch.Tensor,
                               seq_lens: torch.Tensor, max_seq_len: int, scale: float | None = None,
                               layer: int = 0) -> torch.Tensor:
        """Causal attention of ``q_len`` new tokens per sequence whose keys/values are already stored.

        q: [B, q_len, Hq, D]; seq_lens: [B] totals INCLUDING the new tokens.  Query i of a sequence
        attends positions < seq_len - q_len + i + 1.  Same device-side formulation as the reference's
        continuation chunk (vllm_plugin/v1_backend.py:1359-1384): the decode kernel run on one
        synthetic sequence per query with its own length; no host synchronisation.
        """
        B, q_len, Hq, D = q.shape
        synth_bt, synth_sl = synthetic_decode_batch(block_table, seq_lens, q_len)
        out = self.decode_attention(q.reshape(B * q_len, Hq, D), synth_bt, synth_sl, max_seq_len,
                                    scale, layer=layer)
        return out.view(B, q_len, Hq, D)


def synthetic_decode_batch(block_table: torch.Tensor, seq_lens: torch.Tensor, q_len: int):
    """Per-query block tables and lengths that turn a causal multi-query step into decode steps."""
    bt = block_table.repeat_interleave(q_len, dim=0)
    ar = torch.arange(q_len, device=seq_lens.device, dtype=seq_lens.dtype)
    sl = (seq_lens[:, None] - (q_len - 1) + ar[None, :]).reshape(-1)
    return bt, sl


def v0_store(kv_cache: torch.Tensor, key: torch.Tensor, value: torch.Tensor,
             slot_mapping: torch.Tensor, key_bits: int, value_bits: int, signs, bounds_k,
             bounds_v) -> None:
    """Encode K/V and write them in the reference's v0 layout
    kv_cache u8 [2, num_blocks, block_size, Hkv, packed_dim + 4]
    (reference: attention_impl.py:190-254; cache_ops.py:85-108)."""
    _require_cuda(key, "key")
    if key.dtype not in _DT:
        key, value = key.float(), value.float()
    key, value = key.contiguous(), value.contiguous().to(key.dtype)
    _, nb, bs, H, es = kv_cache.shape
    n_tokens, _, D = key.shape
    sm = slot_mapping.to(device=key.device, dtype=torch.int64).contiguous()
    with torch.cuda.device(key.device):
        rc = _lib.load().ftq_v0_store(
            _ptr(key), _ptr(value), _DT[key.dtype], n_tokens, H, D, H * D, D, key_bits, value_bits,
            _lib.fptr(_host_table(signs)), _lib.fptr(_host_table(bounds_k)),
            _lib.fptr(_host_table(bounds_v)), _ptr(kv_cache), nb, bs, es, _ptr(sm),
            _stream(key.device))
    _lib.check(rc, "ftq_v0_store")


def gather_compressed_kv_batched(kv_cache: torch.Tensor, block_tables: torch.Tensor,
                                 seq_lens: torch.Tensor, kv_type: int, packed_dim: int,
                                 max_seq_len: int):
    """Gather the v0 layout into contiguous tensors in one launch
    (reference: cache_ops.py:151-205): (packed [B,Hkv,max_seq_len,pd] u8, norms fp32 [B,Hkv,max_seq_len])."""
    _require_cuda(kv_cache, "kv_cache")
    _, nb, bs, H, es = kv_cache.shape
    B = block_tables.shape[0]
    bt = block_tables.to(device=kv_cache.device, dtype=torch.int32).contiguous()
    sl = seq_lens.to(device=kv_cache.device, dtype=torch.int32).contiguous()
    out_p = torch.empty((B, H, max_seq_len, packed_dim), dtype=torch.uint8, device=kv_cache.device)
    out_n = torch.empty((B, H, max_seq_len), dtype=torch.float32, device=kv_cache.device)
    with torch.cuda.device(kv_cache.device):
        rc = _lib.load().ftq_v0_gather(_ptr(kv_cache), nb, bs, H, es, kv_type, packed_dim,
                                       _ptr(bt), bt.shape[1], _ptr(sl), B, max_seq_len,
                                       _ptr(out_p), _ptr(out_n), _stream(kv_cache.device))
    _lib.check(rc, "ftq_v0_gather")
    return out_p, out_n
