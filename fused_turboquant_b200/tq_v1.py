"""vLLM-v1 "TURBOQUANT" slot format: the host side of the reference's in-kernel-rotation
backend, on libftq_b200.so.

  TurboQuantSlotConfig   <- BoundaryTurboQuantConfig / vLLM's TurboQuantConfig slot properties
                            (vllm_plugin/boundary_tq_config.py:21-81)
  midpoints_of           <- MatrixRotationStrategy.setup_layer (vllm_plugin/rotation/matrix.py:34-42)
  launch_store           <- HadamardStrategy.launch_store / _launch_rht
                            (vllm_plugin/rotation/hadamard.py:44-58, triton_inkernel_store.py:554-646),
                            with the optional value pre-rotation of v1_backend.py:727-740
  decode_attention       <- FusedTurboQuantV1Impl._decode_attention_offset_only
                            (vllm_plugin/v1_backend.py:975-1093)

The kv cache is the uint8 tensor ``[num_blocks, block_size, num_kv_heads, slot]`` vLLM allocates.
Tensors must live on a CUDA device; there is no CPU path.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from . import _lib
from .kernels import _DT, _host_table, _ptr, _require_cuda, _stream, rht


@dataclass(frozen=True)
class TurboQuantSlotConfig:
    """Slot layout of one (token, KV head): key codes | key norm f16 | value codes | scale f16 | zero f16.

    ``key_quant_bits == 8`` selects FP8 (e4m3) keys as vLLM's stock ``TurboQuantConfig`` does (the
    key field is ``head_dim`` bytes with no norm behind it) unless ``key_use_fp8_at_8bit`` is
    False: then the 8 bits are Lloyd-Max codes of a 256-entry table, one byte per coordinate plus
    the fp16 norm, as the reference's boundary layers store them
    (``BoundaryTurboQuantConfig(key_use_fp8_at_8bit=False)``, vllm_plugin/boundary_tq_config.py:26-35).
    """

    head_dim: int
    key_quant_bits: int       # 1..4: Lloyd-Max codes; 8: FP8 keys or 8-bit Lloyd-Max codes
    value_quant_bits: int     # 1, 2, 3, 4 or 8: per-vector uniform codes
    norm_correction: bool = True
    key_use_fp8_at_8bit: bool = True

    def __post_init__(self):
        if self.head_dim not in (64, 128, 256):
            raise ValueError(f"head_dim must be 64, 128 or 256, got {self.head_dim}")
        if self.key_quant_bits not in (1, 2, 3, 4, 8):
            raise ValueError(f"key_quant_bits must be 1, 2, 3, 4 or 8 (FP8), got {self.key_quant_bits}")
        if self.value_quant_bits not in (1, 2, 3, 4, 8):
            raise ValueError(f"value_quant_bits must be 1, 2, 3, 4 or 8, got {self.value_quant_bits}")

    @property
    def key_fp8(self) -> bool:
        return self.key_quant_bits == 8 and self.key_use_fp8_at_8bit

    @property
    def key_mse_bits(self) -> int:
        return 0 if self.key_fp8 else self.key_quant_bits

    @property
    def mse_bits(self) -> int:
        # (as in the reference: with FP8 keys the centroid table is sized for the values)
        return self.value_quant_bits if self.key_fp8 else self.key_quant_bits

    @property
    def n_centroids(self) -> int:
        return 2 ** self.mse_bits

    @property
    def effective_value_quant_bits(self) -> int:
        return self.value_quant_bits

    @property
    def key_packed_size(self) -> int:
        if self.key_fp8:
            return self.head_dim
        return math.ceil(self.head_dim * self.key_quant_bits / 8) + 2

    @property
    def value_data_bytes(self) -> int:
        if self.value_quant_bits == 8:
            return self.head_dim
        return math.ceil(self.head_dim * self.value_quant_bits / 8)

    @property
    def value_packed_size(self) -> int:
        return self.value_data_bytes + 4

    @property
    def slot_size(self) -> int:
        return self.key_packed_size + self.value_packed_size

    @property
    def slot_size_aligned(self) -> int:
        return self.slot_size + self.slot_size % 2


def midpoints_of(centroids: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """(sorted fp32 centroids, their midpoints) as the reference derives them per layer."""
    c, _ = centroids.to(torch.float32).sort()
    return c, (c[:-1] + c[1:]) / 2


KEY_BITS_MSE8 = 264   # FTQ_TQ_KEY_BITS_MSE8 of the C ABI: 8-bit Lloyd-Max key codes


def _key_bits(tq_config) -> int:
    """The C ABI's key_bits of a (possibly duck-typed) config: 8 bits that are not FP8 are 8-bit
    Lloyd-Max codes."""
    kb = int(tq_config.key_quant_bits)
    if kb == 8 and not getattr(tq_config, "key_fp8", True):
        return KEY_BITS_MSE8
    return kb


def _table_ptr(table, fp8: bool):
    # FP8 keys have no key codebook: whatever table the caller holds (the reference sizes it for the
    # values then) is not read
    return None if fp8 else _lib.fptr(_host_table(table))


def _cache_strides(kv_cache: torch.Tensor) -> tuple[int, int, int]:
    if kv_cache.dtype != torch.uint8:
        kv_cache = kv_cache.view(torch.uint8)
    if kv_cache.dim() != 4 or kv_cache.stride(3) != 1:
        raise ValueError("kv_cache must be [num_blocks, block_size, num_kv_heads, slot] with a dense last dim")
    return kv_cache.stride(0), kv_cache.stride(1), kv_cache.stride(2)


def launch_store(key: torch.Tensor, value: torch.Tensor, kv_cache: torch.Tensor,
                 slot_mapping: torch.Tensor, midpoints, tq_config: TurboQuantSlotConfig,
                 head_size: int | None = None, v_rotate: bool = False,
                 v_lloyd_max: bool = False) -> None:
    """Quantise ``key``/``value`` ``[N, Hkv, D]`` into the slots ``slot_mapping`` names (< 0: skipped,
    and so are slots beyond the cache's end).  ``key``/``value`` ``[L, N, Hkv, D]`` with a cache
    ``[L, num_blocks, block_size, Hkv, slot]`` stores all layers in one launch (same
    ``slot_mapping`` for every layer).

    ``v_lloyd_max`` (the reference's TURBOQUANT_V_LLOYD_MAX switch; 4-bit values only, ignored
    otherwise as in the reference): values become Lloyd-Max codes against the key midpoints, their
    norm goes into the scale field.  The reference rotates the values whenever that switch is on
    (vllm_plugin/v1_backend.py:736-740): pass ``v_rotate=True`` with it unless they already are.
    """
    _require_cuda(key, "key")
    _require_cuda(kv_cache, "kv_cache")
    layered = key.dim() == 4
    if layered != (kv_cache.dim() == 5):
        raise ValueError("key/value [L, N, Hkv, D] go with a cache [L, num_blocks, block_size, Hkv, slot]")
    n_layers = key.shape[0] if layered else 1
    if layered and kv_cache.shape[0] != n_layers:
        raise ValueError("key/value and kv_cache disagree on the number of layers")
    n, hkv, d = key.shape[-3:]
    if head_size is not None and head_size != d:
        raise ValueError(f"head_size {head_size} does not match key.shape[-1] {d}")
    if d != tq_config.head_dim:
        raise ValueError(f"key head size {d} does not match the config ({tq_config.head_dim})")
    if value.shape != key.shape:
        raise ValueError("key and value must have the same shape")
    if key.dtype not in _DT:
        key = key.float()
    if value.dtype != key.dtype:
        value = value.to(key.dtype)
    rotate_in_kernel = bool(v_rotate) and tq_config.value_quant_bits != 8
    if v_rotate and not rotate_in_kernel:
        # 8-bit values: rotate here (the kernel fuses the rotation for 1..4-bit values only)
        value = rht(value.float().contiguous(), None).to(key.dtype)
    if key.stride(-1) != 1 or value.stride() != key.stride():
        key, value = key.contiguous(), value.contiguous()
    if kv_cache.dtype != torch.uint8:
        kv_cache = kv_cache.view(torch.uint8)
    sb, sp, sh = _cache_strides(kv_cache[0] if layered else kv_cache)
    if kv_cache.shape[-1] < tq_config.slot_size:
        raise ValueError(f"kv_cache slots of {kv_cache.shape[-1]} bytes are smaller than {tq_config.slot_size}")
    sm = slot_mapping.to(device=key.device, dtype=torch.int64).contiguous()
    kb = _key_bits(tq_config)
    with torch.cuda.device(key.device):
        rc = _lib.load().ftq_tq_store_layers(
            _ptr(key), _ptr(value), _DT[key.dtype], n, hkv, d, key.stride(-3), key.stride(-2),
            kb, tq_config.value_quant_bits, int(rotate_in_kernel),
            int(bool(v_lloyd_max)), _table_ptr(midpoints, kb == 8), _ptr(kv_cache), sb, sp, sh,
            kv_cache.shape[-3], _ptr(sm), n_layers, key.stride(0) if layered else 0,
            kv_cache.stride(0) if layered else 0, kv_cache.shape[-4], _stream(key.device))
    _lib.check(rc, "ftq_tq_store_layers")


def decode_attention(query: torch.Tensor, kv_cache: torch.Tensor, block_table: torch.Tensor,
                     seq_lens: torch.Tensor, centroids, tq_config: TurboQuantSlotConfig, scale: float,
                     num_kv_splits: int = 8, kv_start_offset: torch.Tensor | None = None,
                     v_rotate: bool = False, mid_o: torch.Tensor | None = None,
                     output: torch.Tensor | None = None, lse: torch.Tensor | None = None,
                     out_dtype: torch.dtype | None = None, v_lloyd_max: bool = False,
                     prefix_output: torch.Tensor | None = None,
                     prefix_lse: torch.Tensor | None = None) -> torch.Tensor:
    """Decode attention of ``query`` ``[B, Hq, D]`` over the compressed cache; returns ``[B, Hq, D]``.

    All layers in one call: ``query`` ``[L, B, Hq, D]`` with ``kv_cache`` ``[L, num_blocks,
    block_size, Hkv, slot]`` (one allocation, every layer the same block table); ``mid_o``,
    ``output``, ``lse`` and the prefix tensors then carry the same leading ``L``.

    ``v_rotate``: the cache holds rotated values, the merged output is transformed back.
    ``v_lloyd_max``: 4-bit values are Lloyd-Max codes (see ``launch_store``).
    ``prefix_output`` ``[B, Hq, D]`` / ``prefix_lse`` ``[B, Hq]``: attention of the same queries
    over an uncompressed prefix ``[0, kv_start_offset)`` (the reference's deferred-prefill hybrid,
    vllm_plugin/v1_backend.py:1096-1277, computes it with SDPA); merged in by log-sum-exp.

    ``mid_o`` ``[B, Hq, num_kv_splits, D+1]`` fp32, ``output`` and ``lse`` ``[B, Hq]`` fp32 may be
    supplied (pre-allocated per layer, as the reference keeps them for CUDA-graph capture).
    """
    _require_cuda(query, "query")
    _require_cuda(kv_cache, "kv_cache")
    if kv_cache.dtype != torch.uint8:
        kv_cache = kv_cache.view(torch.uint8)
    n_layers, layer_stride, lead = 1, 0, ()
    if query.dim() == 4:
        if kv_cache.dim() != 5 or kv_cache.shape[0] != query.shape[0]:
            raise ValueError("a [L, B, Hq, D] query needs a [L, num_blocks, block_size, Hkv, slot] cache")
        n_layers, lead = query.shape[0], (query.shape[0],)
        layer_stride = kv_cache.stride(0)
        query = query.reshape(-1, *query.shape[2:])
        kv_cache = kv_cache[0]
    B, hq, d = query.shape
    B //= n_layers
    rows = B * n_layers
    if d != tq_config.head_dim:
        raise ValueError(f"query head size {d} does not match the config ({tq_config.head_dim})")
    if query.dtype not in _DT:
        query = query.float()
    query = query.contiguous()
    sb, sp, sh = _cache_strides(kv_cache)
    hkv = kv_cache.shape[2]
    dev = query.device
    bt = block_table.to(device=dev, dtype=torch.int32).contiguous()
    sl = seq_lens.to(device=dev, dtype=torch.int32).contiguous()
    ks = None if kv_start_offset is None else kv_start_offset.to(device=dev, dtype=torch.int32).contiguous()
    if mid_o is None:
        mid_o = torch.empty((rows, hq, num_kv_splits, d + 1), dtype=torch.float32, device=dev)
    elif mid_o.numel() != rows * hq * num_kv_splits * (d + 1) or mid_o.dtype != torch.float32 or \
            not mid_o.is_contiguous():
        raise ValueError("mid_o must be a contiguous fp32 [(L,) B, Hq, num_kv_splits, D+1] tensor")
    odt = out_dtype or query.dtype
    if output is None:
        output = torch.empty(lead + (B, hq, d), dtype=odt, device=dev)
    elif output.shape != lead + (B, hq, d) or not output.is_contiguous() or output.dtype not in _DT:
        raise ValueError("output must be a contiguous [(L,) B, Hq, D] tensor of a supported dtype")
    if lse is not None and (lse.dtype != torch.float32 or not lse.is_contiguous() or
                            lse.numel() != rows * hq or lse.device != dev):
        raise ValueError("lse must be a contiguous fp32 [(L,) B, Hq] tensor on the query's device")
    if (prefix_output is None) != (prefix_lse is None):
        raise ValueError("prefix_output and prefix_lse go together")
    if prefix_output is not None:
        _require_cuda(prefix_output, "prefix_output")
        if prefix_output.shape != lead + (B, hq, d) or prefix_lse.shape != lead + (B, hq):
            raise ValueError("prefix_output must be [(L,) B, Hq, D] and prefix_lse [(L,) B, Hq]")
        if prefix_output.dtype not in _DT:
            prefix_output = prefix_output.float()
        prefix_output = prefix_output.contiguous()
        prefix_lse = prefix_lse.to(device=dev, dtype=torch.float32).contiguous()
    kb = _key_bits(tq_config)
    with torch.cuda.device(dev):
        rc = _lib.load().ftq_tq_decode_layers(
            _ptr(query), _DT[query.dtype], B, hq, hkv, d, _ptr(kv_cache), sb, sp, sh,
            kv_cache.shape[1], _ptr(bt), bt.shape[1], _ptr(sl), _ptr(ks),
            kb, tq_config.value_quant_bits, int(tq_config.norm_correction),
            int(v_rotate), int(bool(v_lloyd_max)), _table_ptr(centroids, kb == 8), float(scale),
            num_kv_splits,
            _ptr(mid_o), _ptr(output), _DT[output.dtype], _ptr(lse), _ptr(prefix_output),
            _DT[prefix_output.dtype] if prefix_output is not None else 0, _ptr(prefix_lse),
            n_layers, layer_stride, kv_cache.shape[0], _stream(dev))
    _lib.check(rc, "ftq_tq_decode_layers")
    return output


def continuation_attention(query: torch.Tensor, kv_cache: torch.Tensor, block_table: torch.Tensor,
                           seq_lens: torch.Tensor, centroids, tq_config: TurboQuantSlotConfig,
                           scale: float, num_kv_splits: int = 8, v_rotate: bool = False,
                           v_lloyd_max: bool = False) -> torch.Tensor:
    """Causal attention of ``q_len`` new tokens per sequence that are already in the cache.

    query: [B, q_len, Hq, D]; seq_lens: [B] totals including the new tokens.  The reference's
    continuation chunk (vllm_plugin/v1_backend.py:1359-1384): one synthetic decode sequence per
    query with length ``cached_len + i + 1`` and the sequence's block table.
    """
    from .paged import synthetic_decode_batch
    B, q_len, hq, d = query.shape
    bt, sl = synthetic_decode_batch(block_table, seq_lens, q_len)
    out = decode_attention(query.reshape(B * q_len, hq, d), kv_cache, bt, sl, centroids, tq_config,
                           scale, num_kv_splits=num_kv_splits, v_rotate=v_rotate,
                           v_lloyd_max=v_lloyd_max)
    return out.view(B, q_len, hq, d)
