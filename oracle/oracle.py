"""numpy/ctypes front end of the CPU oracle (``ftq_oracle.c``).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by the smoke check and by the
benchmark's CPU arm.  The shipped package never imports this module.

Each function is a thin wrapper over the C restatement; the C file cites the
reference lines every step follows.  Arrays are numpy, C-contiguous; fp16 norms
travel as ``np.float16`` (bit patterns are what gets compared).
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libftq_oracle.so")
_lib = None


def build(force: bool = False) -> str:
    """Compile ``ftq_oracle.c`` into ``libftq_oracle.so`` next to it (gcc, no FMA contraction)."""
    src = os.path.join(_HERE, "ftq_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(
            ["gcc", "-O2", "-ffp-contract=off", "-fno-fast-math", "-fopenmp", "-fPIC", "-shared",
             "-o", _SO, src, "-lm"])
    return _SO


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_SO)
        _lib.ftq_oracle_f16_to_f32.restype = ctypes.c_float
        _lib.ftq_oracle_f32_to_f16.restype = ctypes.c_uint16
        _lib.ftq_oracle_f32_to_f16.argtypes = [ctypes.c_float]
        _lib.ftq_oracle_f16_to_f32.argtypes = [ctypes.c_uint16]
    return _lib


def _p(a: np.ndarray | None):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _c(a, dtype):
    return np.ascontiguousarray(a, dtype=dtype)


def packed_dim(d: int, bits: int) -> int:
    return {4: d // 2, 3: d * 3 // 8, 2: d // 4}[bits]


def set_threads(n: int) -> None:
    """Set the OpenMP thread count used by the oracle (benchmark CPU arm)."""
    omp = ctypes.CDLL("libgomp.so.1")
    omp.omp_set_num_threads(int(n))


def fwht(x: np.ndarray) -> np.ndarray:
    """Orthonormal FWHT over the last axis (no signs)."""
    x = _c(x, np.float32)
    d = x.shape[-1]
    y = np.empty_like(x)
    lib().ftq_oracle_rht(_p(x), None, _p(y), ctypes.c_int64(x.size // d), ctypes.c_int(d),
                         ctypes.c_int(0))
    return y


def rht(x: np.ndarray, signs: np.ndarray | None, inverse: bool = False) -> np.ndarray:
    x = _c(x, np.float32)
    d = x.shape[-1]
    s = None if signs is None else _c(signs, np.float32)
    y = np.empty_like(x)
    lib().ftq_oracle_rht(_p(x), _p(s), _p(y), ctypes.c_int64(x.size // d), ctypes.c_int(d),
                         ctypes.c_int(1 if inverse else 0))
    return y


def pack(idx: np.ndarray, bits: int) -> np.ndarray:
    idx = _c(idx, np.uint8)
    d = idx.shape[-1]
    pd = packed_dim(d, bits)
    flat = idx.reshape(-1, d)
    out = np.empty((flat.shape[0], pd), np.uint8)
    L = lib()
    for i in range(flat.shape[0]):
        L.ftq_oracle_pack(_p(flat[i]), _p(out[i]), ctypes.c_int(d), ctypes.c_int(bits))
    return out.reshape(*idx.shape[:-1], pd)


def unpack(packed: np.ndarray, d: int, bits: int) -> np.ndarray:
    packed = _c(packed, np.uint8)
    pd = packed.shape[-1]
    flat = packed.reshape(-1, pd)
    out = np.empty((flat.shape[0], d), np.uint8)
    L = lib()
    for i in range(flat.shape[0]):
        L.ftq_oracle_unpack(_p(flat[i]), _p(out[i]), ctypes.c_int(d), ctypes.c_int(bits))
    return out.reshape(*packed.shape[:-1], d)


def encode(x: np.ndarray, signs, boundaries, bits: int, norm_lanes: int = 8,
           return_normalized: bool = False):
    """``TurboQuantMSE._encode_unfused``: returns (packed u8 [..., pd], norms f16 [...])."""
    x = _c(x, np.float32)
    d = x.shape[-1]
    n = x.size // d
    pd = packed_dim(d, bits)
    s = None if signs is None else _c(signs, np.float32)
    b = _c(boundaries, np.float32)
    assert b.size == (1 << bits) + 1
    packed = np.empty((n, pd), np.uint8)
    norms = np.empty((n,), np.uint16)
    normalized = np.empty((n, d), np.float32) if return_normalized else None
    lib().ftq_oracle_encode(_p(x), ctypes.c_int64(n), ctypes.c_int(d), ctypes.c_int(bits), _p(s),
                            _p(b), _p(packed), _p(norms), ctypes.c_int(norm_lanes),
                            _p(normalized))
    out = (packed.reshape(*x.shape[:-1], pd), norms.view(np.float16).reshape(x.shape[:-1]))
    if return_normalized:
        return out + (normalized.reshape(x.shape),)
    return out


def decode_dense(packed, norms, levels, signs, bits: int, d: int) -> np.ndarray:
    """``TurboQuantMSE._decode_unfused``: dense fp32 [..., d]."""
    packed = _c(packed, np.uint8)
    norms16 = _c(norms, np.float16)
    n = norms16.size
    lv = _c(levels, np.float32)
    s = None if signs is None else _c(signs, np.float32)
    out = np.empty((n, d), np.float32)
    lib().ftq_oracle_decode_dense(_p(packed), _p(norms16.view(np.uint16)), ctypes.c_int64(n),
                                  ctypes.c_int(d), ctypes.c_int(bits), _p(lv), _p(s), _p(out))
    return out.reshape(*norms16.shape, d)


def qk_scores(q_rot, k_idx, k_norms, levels, scale: float, bits: int) -> np.ndarray:
    """``fused_qk_scores_rht`` for q_len == 1: q_rot [B,Hq,D] -> scores [B,Hq,S]."""
    q_rot = _c(q_rot, np.float32)
    k_idx = _c(k_idx, np.uint8)
    kn = _c(k_norms, np.float32)
    B, Hq, d = q_rot.shape
    _, Hkv, S, _ = k_idx.shape
    out = np.empty((B, Hq, S), np.float32)
    lib().ftq_oracle_qk_scores(_p(q_rot), _p(k_idx), _p(kn), _p(_c(levels, np.float32)),
                               ctypes.c_float(scale), ctypes.c_int(bits), ctypes.c_int(B),
                               ctypes.c_int(Hq), ctypes.c_int(Hkv), ctypes.c_int(S),
                               ctypes.c_int(d), _p(out))
    return out


def decode_attn(q, k_idx, k_norms, v_idx, v_norms, levels_k, levels_v, signs, scale: float,
                bits_k: int, bits_v: int, seq_lens=None) -> np.ndarray:
    """Composed unfused decode attention; q [B,Hq,D] in the ORIGINAL space -> out [B,Hq,D] fp32."""
    q = _c(q, np.float32)
    k_idx = _c(k_idx, np.uint8)
    v_idx = _c(v_idx, np.uint8)
    kn = _c(k_norms, np.float16)
    vn = _c(v_norms, np.float16)
    B, Hq, d = q.shape
    _, Hkv, S, _ = k_idx.shape
    sl = None if seq_lens is None else _c(seq_lens, np.int32)
    s = None if signs is None else _c(signs, np.float32)
    out = np.empty((B, Hq, d), np.float32)
    lib().ftq_oracle_decode_attn(_p(q), _p(k_idx), _p(kn.view(np.uint16)), _p(v_idx),
                                 _p(vn.view(np.uint16)), _p(_c(levels_k, np.float32)),
                                 _p(_c(levels_v, np.float32)), _p(s), ctypes.c_float(scale),
                                 ctypes.c_int(bits_k), ctypes.c_int(bits_v), _p(sl),
                                 ctypes.c_int(B), ctypes.c_int(Hq), ctypes.c_int(Hkv),
                                 ctypes.c_int(S), ctypes.c_int(d), _p(out))
    return out


def v0_write(kv_cache: np.ndarray, kv_type: int, packed, norms, slot_mapping) -> None:
    """Reference v0 paged write into kv_cache u8 [2, nb, bs, Hkv, pd+4] (in place)."""
    assert kv_cache.dtype == np.uint8 and kv_cache.flags.c_contiguous
    _, nb, bs, Hkv, es = kv_cache.shape
    packed = _c(packed, np.uint8)
    norms16 = _c(norms, np.float16)
    sm = _c(slot_mapping, np.int64)
    lib().ftq_oracle_v0_write(_p(kv_cache), ctypes.c_int64(nb), ctypes.c_int(bs),
                              ctypes.c_int(Hkv), ctypes.c_int(es), ctypes.c_int(kv_type),
                              _p(packed), ctypes.c_int(packed.shape[-1]),
                              _p(norms16.view(np.uint16)), _p(sm), ctypes.c_int64(sm.size))


def v0_gather(kv_cache: np.ndarray, kv_type: int, pd: int, block_tables, seq_lens,
              max_seq_len: int):
    """Reference v0 paged gather -> (packed [B,Hkv,max_seq_len,pd] u8, norms fp32 [B,Hkv,max_seq_len])."""
    _, nb, bs, Hkv, es = kv_cache.shape
    bt = _c(block_tables, np.int32)
    sl = _c(seq_lens, np.int32)
    B = bt.shape[0]
    out_p = np.empty((B, Hkv, max_seq_len, pd), np.uint8)
    out_n = np.empty((B, Hkv, max_seq_len), np.float32)
    lib().ftq_oracle_v0_gather(_p(kv_cache), ctypes.c_int64(nb), ctypes.c_int(bs),
                               ctypes.c_int(Hkv), ctypes.c_int(es), ctypes.c_int(kv_type),
                               ctypes.c_int(pd), _p(bt), ctypes.c_int(bt.shape[1]), _p(sl),
                               ctypes.c_int(B), ctypes.c_int(max_seq_len), _p(out_p), _p(out_n))
    return out_p, out_n


# ---------------------------------------------------------------- vLLM-v1 slot format

def tq_slot_bytes(d: int, key_bits: int, value_bits: int) -> int:
    """key codes + fp16 norm (key_bits 8 = FP8 keys: d bytes, no norm; 264 = 8-bit Lloyd-Max codes:
    d bytes + norm) + value codes + fp16 scale + fp16 zero, rounded up to even."""
    kbytes = d if key_bits == 8 else (d + 2 if key_bits == 264 else d * key_bits // 8 + 2)
    s = kbytes + (d if value_bits == 8 else d * value_bits // 8) + 4
    return s + s % 2


def tq_store(key, value, kv_cache: np.ndarray, slot_mapping, midpoints, key_bits: int,
             value_bits: int, return_rotated: bool = False, value_lloyd_max: bool = False,
             value_sum_order: int = 0):
    """The reference's in-kernel-rotation store into kv_cache [nb, block_size, Hkv, slot] (in place).

    value_lloyd_max: 4-bit values as Lloyd-Max codes of the key table (ignored for other widths);
    value_sum_order 1 adds the value's squares in the order of the CUDA store's fused rotation."""
    key, value = _c(key, np.float32), _c(value, np.float32)
    n, hkv, d = key.shape
    assert kv_cache.dtype == np.uint8 and kv_cache.flags.c_contiguous and kv_cache.ndim == 4
    sm = _c(slot_mapping, np.int64)
    mids = _c(np.zeros(1) if midpoints is None else midpoints, np.float32)   # (FP8 keys: unused)
    y = np.empty_like(key) if return_rotated else None
    st = kv_cache.strides
    lib().ftq_oracle_tq_store(_p(key), _p(value), ctypes.c_int64(n), ctypes.c_int(hkv),
                              ctypes.c_int(d), ctypes.c_int(key_bits), ctypes.c_int(value_bits),
                              _p(mids), _p(kv_cache), ctypes.c_int64(st[0]), ctypes.c_int64(st[1]),
                              ctypes.c_int64(st[2]), ctypes.c_int(kv_cache.shape[1]), _p(sm), _p(y),
                              ctypes.c_int(int(value_lloyd_max)), ctypes.c_int(int(value_sum_order)))
    return y


def tq_decode(q, kv_cache: np.ndarray, block_table, seq_lens, centroids, key_bits: int,
              value_bits: int, scale: float, splits: int, norm_correction: bool = False,
              kv_start=None, rotate_out: bool = False, value_lloyd_max: bool = False):
    """Split-KV decode over the slot format: returns (out [B,Hq,d], mid_o [B,Hq,splits,d+1], lse)."""
    q = _c(q, np.float32)
    B, Hq, d = q.shape
    hkv = kv_cache.shape[2]
    bt = _c(block_table, np.int32)
    sl = _c(seq_lens, np.int32)
    ks = None if kv_start is None else _c(kv_start, np.int32)
    cent = _c(np.zeros(1) if centroids is None else centroids, np.float32)   # (FP8 keys: unused)
    mid_o = np.empty((B, Hq, splits, d + 1), np.float32)
    out = np.empty((B, Hq, d), np.float32)
    lse = np.empty((B, Hq), np.float32)
    st = kv_cache.strides
    lib().ftq_oracle_tq_decode(_p(q), ctypes.c_int(B), ctypes.c_int(Hq), ctypes.c_int(hkv),
                               ctypes.c_int(d), _p(kv_cache), ctypes.c_int64(st[0]),
                               ctypes.c_int64(st[1]), ctypes.c_int64(st[2]),
                               ctypes.c_int(kv_cache.shape[1]), _p(bt), ctypes.c_int(bt.shape[1]),
                               _p(sl), _p(ks), ctypes.c_int(key_bits), ctypes.c_int(value_bits),
                               ctypes.c_int(int(norm_correction)), ctypes.c_int(int(rotate_out)),
                               _p(cent), ctypes.c_float(scale), ctypes.c_int(splits), _p(mid_o),
                               _p(out), _p(lse), ctypes.c_int(int(value_lloyd_max)))
    return out, mid_o, lse


def tq_merge_prefix(out, lse, out_prefix, lse_prefix):
    """Log-sum-exp merge of two attention results over disjoint key ranges
    (vllm_plugin/v1_backend.py:1267-1277): returns (out, lse)."""
    out, out_prefix = np.asarray(out, np.float64), np.asarray(out_prefix, np.float64)
    lse, lse_prefix = np.asarray(lse, np.float64), np.asarray(lse_prefix, np.float64)
    lmax = np.maximum(lse, lse_prefix)
    with np.errstate(invalid="ignore"):
        ep = np.where(np.isneginf(lmax), 0.0, np.exp(lse_prefix - lmax))
        eq = np.where(np.isneginf(lmax), 0.0, np.exp(lse - lmax))
    total = np.maximum(ep + eq, 1e-20)
    merged = out_prefix * (ep / total)[..., None] + out * (eq / total)[..., None]
    with np.errstate(divide="ignore"):
        return merged, lmax + np.log(ep + eq)
