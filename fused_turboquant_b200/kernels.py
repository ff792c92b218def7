"""The reference's kernel-level callables, backed by libftq_b200.so.

Same names, argument meaning and error behaviour as the functions the
reference's core / HF / vLLM-v0 code calls on CUDA tensors:

  fused_encode            <- triton_fused_encode      (kernels/triton_encode.py:150-209)
  fused_decode            <- triton_fused_decode      (kernels/triton_decode.py:104-155)
  rht                     <- triton_rht               (kernels/triton_rht.py:82-121)
  fused_qk_scores_rht     <- fused_qk_scores_rht      (kernels/triton_attention.py:158-225)
  flash_decode_compressed <- flash_decode_compressed  (kernels/triton_flash_decode.py:224-324)
  is_available            <- is_triton_available      (kernels/triton_rht.py:124)

The ``triton_*`` aliases at the bottom make the module importable in place of
the reference's.  Tensors must be CUDA tensors; the small tables (signs,
boundaries, levels) may live anywhere -- a host copy is cached per tensor.
Nothing here falls back to PyTorch or the CPU.
"""
from __future__ import annotations

import ctypes
import weakref

import numpy as np
import torch

from . import _lib

_DT = {torch.float32: _lib.F32, torch.float16: _lib.F16, torch.bfloat16: _lib.BF16}

# id(tensor) -> (weak reference, tensor version, host copy).  Keyed by identity: tensors compare
# element-wise, which rules them out as dictionary keys.
_table_cache: dict[int, tuple[weakref.ref, int, np.ndarray]] = {}
_workspaces: dict[tuple[int, int], torch.Tensor] = {}


def is_available() -> bool:
    return _lib.is_available()


def _host_table(t) -> np.ndarray | None:
    """fp32 host copy of a small table (cached while the tensor is alive and unmodified)."""
    if t is None:
        return None
    if isinstance(t, np.ndarray):
        return np.ascontiguousarray(t, dtype=np.float32)
    key = id(t)
    hit = _table_cache.get(key)
    if hit is not None and hit[0]() is t and hit[1] == t._version:
        return hit[2]
    arr = np.ascontiguousarray(t.detach().to(torch.float32).cpu().numpy())
    _table_cache[key] = (weakref.ref(t, lambda _r, k=key: _table_cache.pop(k, None)), t._version, arr)
    return arr


def _require_cuda(t: torch.Tensor, name: str) -> None:
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise RuntimeError(
            f"{name} must be a CUDA tensor: fused_turboquant_b200 has no CPU path "
            "(build libftq_b200.so and run on a B200)")


def _stream(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _ptr(t: torch.Tensor | None):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def packed_dim(head_dim: int, bits: int) -> int:
    if bits not in (2, 3, 4):
        raise ValueError(f"bits must be 2, 3, or 4, got {bits}")
    return head_dim * bits // 8


def workspace_bytes(B: int, Hq: int, Hkv: int, head_dim: int, max_seq_len: int,
                    n_layers: int = 1) -> int:
    return int(_lib.load().ftq_decode_workspace_bytes(B, Hq, Hkv, head_dim, max_seq_len, n_layers))


def get_workspace(device: torch.device, nbytes: int) -> torch.Tensor:
    """Per (device, stream) scratch buffer, grown on demand and reused across calls."""
    key = (device.index if device.index is not None else torch.cuda.current_device(),
           _stream(device))
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


# ------------------------------------------------------------------ encode

def fused_encode(x: torch.Tensor, signs, boundaries, bits: int):
    """RHT + norm + Lloyd-Max + pack in one launch -> (packed u8 (..., pd), norms f16 (...))."""
    _require_cuda(x, "x")
    if x.dtype not in _DT:
        x = x.float()
    d = x.shape[-1]
    lead = x.shape[:-1]
    pd = packed_dim(d, bits)
    x2 = x.contiguous().view(-1, d)
    n = x2.shape[0]
    packed = torch.empty((n, pd), dtype=torch.uint8, device=x.device)
    norms = torch.empty((n,), dtype=torch.float16, device=x.device)
    with torch.cuda.device(x.device):
        rc = _lib.load().ftq_encode(_ptr(x2), _DT[x2.dtype], n, d, d, bits,
                                    _lib.fptr(_host_table(signs)),
                                    _lib.fptr(_host_table(boundaries)), _ptr(packed), _ptr(norms),
                                    _stream(x.device))
    _lib.check(rc, "ftq_encode")
    return packed.view(*lead, pd), norms.view(lead)


def fused_decode(packed_indices: torch.Tensor, norms: torch.Tensor, levels, signs, bits: int,
                 original_dim: int) -> torch.Tensor:
    """unpack + dequant + denorm + inverse RHT -> fp32 (..., original_dim)."""
    _require_cuda(packed_indices, "packed_indices")
    d = original_dim
    pd = packed_dim(d, bits)
    p2 = packed_indices.contiguous().view(-1, pd)
    nflat = norms.contiguous().view(-1)
    if nflat.dtype not in (torch.float16, torch.float32):
        nflat = nflat.float()
    n = nflat.shape[0]
    out = torch.empty((n, d), dtype=torch.float32, device=packed_indices.device)
    with torch.cuda.device(out.device):
        rc = _lib.load().ftq_decode_dense(_ptr(p2), _ptr(nflat), _DT[nflat.dtype], n, d, bits,
                                          _lib.fptr(_host_table(levels)),
                                          _lib.fptr(_host_table(signs)), _ptr(out),
                                          _stream(out.device))
    _lib.check(rc, "ftq_decode_dense")
    return out.view(*norms.shape, d)


def rht(x: torch.Tensor, signs, inverse: bool = False) -> torch.Tensor:
    """Randomized Hadamard transform (forward or inverse), same shape and dtype out."""
    _require_cuda(x, "x")
    orig_dtype = x.dtype
    if x.dtype not in _DT:
        x = x.float()
    d = x.shape[-1]
    x2 = x.contiguous().view(-1, d)
    y = torch.empty_like(x2)
    with torch.cuda.device(x.device):
        rc = _lib.load().ftq_rht(_ptr(x2), _ptr(y), _DT[x2.dtype], x2.shape[0], d,
                                 _lib.fptr(_host_table(signs)), int(bool(inverse)),
                                 _stream(x.device))
    _lib.check(rc, "ftq_rht")
    y = y.view(x.shape)
    return y if y.dtype == orig_dtype else y.to(orig_dtype)


# --------------------------------------------------------------- attention

def fused_qk_scores_rht(q_rotated: torch.Tensor, key_indices: torch.Tensor,
                        key_norms: torch.Tensor, centroids, scale: float,
                        bits: int = 3) -> torch.Tensor:
    """Scores Q.K^T straight from packed keys -> fp32 [batch, n_q_heads, q_len, kv_len]."""
    _require_cuda(q_rotated, "q_rotated")
    B, Hq, q_len, d = q_rotated.shape
    _, Hkv, S, _ = key_indices.shape
    q = q_rotated.contiguous().float()
    ki = key_indices.contiguous()
    kn = key_norms.contiguous()
    if kn.dtype not in (torch.float16, torch.float32):
        kn = kn.float()
    out = torch.empty((B, Hq, q_len, S), dtype=torch.float32, device=q.device)
    with torch.cuda.device(q.device):
        rc = _lib.load().ftq_qk_scores(_ptr(q), _ptr(ki), _ptr(kn), _DT[kn.dtype],
                                       _lib.fptr(_host_table(centroids)), float(scale), bits, B,
                                       Hq, Hkv, q_len, S, d, _ptr(out), _stream(q.device))
    _lib.check(rc, "ftq_qk_scores")
    return out


def flash_decode_compressed(q_rotated: torch.Tensor, k_indices: torch.Tensor,
                            k_norms: torch.Tensor, v_indices: torch.Tensor,
                            v_norms: torch.Tensor, k_centroids, v_centroids, signs, scale: float,
                            bits_k: int = 4, bits_v: int = 4,
                            seq_lens: torch.Tensor | None = None, *, q_is_rotated: bool = True,
                            out_dtype: torch.dtype | None = None,
                            workspace: torch.Tensor | None = None) -> torch.Tensor:
    """QK + online softmax + V + inverse RHT in one split-KV pass.

    ``q_rotated`` is [batch, n_q_heads, 1, head_dim]; with ``q_is_rotated=False``
    the raw query is passed and the rotation is fused too.  Returns
    [batch, n_q_heads, 1, head_dim] in the original space (fp32 unless
    ``out_dtype`` says otherwise).  ``seq_lens`` is honoured.
    """
    _require_cuda(q_rotated, "q_rotated")
    B, Hq, q_len, d = q_rotated.shape
    if q_len != 1:
        raise ValueError("flash_decode_compressed handles one query token per sequence")
    _, Hkv, S, _ = k_indices.shape
    q = q_rotated.contiguous()
    if q.dtype not in _DT:
        q = q.float()
    out_dtype = out_dtype or torch.float32
    out = torch.empty((B, Hq, 1, d), dtype=out_dtype, device=q.device)
    ki, vi = k_indices.contiguous(), v_indices.contiguous()
    kn, vn = k_norms.contiguous().half(), v_norms.contiguous().half()
    sl = None if seq_lens is None else seq_lens.to(device=q.device, dtype=torch.int32).contiguous()
    need = workspace_bytes(B, Hq, Hkv, d, S, 1)
    ws = workspace if workspace is not None else get_workspace(q.device, need)
    with torch.cuda.device(q.device):
        rc = _lib.load().ftq_flash_decode(
            _ptr(q), _DT[q.dtype], int(bool(q_is_rotated)), _ptr(ki), _ptr(kn), _ptr(vi), _ptr(vn),
            _lib.fptr(_host_table(k_centroids)), _lib.fptr(_host_table(v_centroids)),
            _lib.fptr(_host_table(signs)), float(scale), bits_k, bits_v, _ptr(sl), B, Hq, Hkv, S,
            d, _ptr(out), _DT[out_dtype], _ptr(ws), ws.numel(), _stream(q.device))
    _lib.check(rc, "ftq_flash_decode")
    return out


# names the reference's modules export
triton_fused_encode = fused_encode
triton_fused_decode = fused_decode
triton_rht = rht
is_triton_available = is_available
