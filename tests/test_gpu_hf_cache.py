"""The HF-style compressed cache on the paged pool: a prefill and a few decode steps.

Stored codes must equal the oracle's encode of the concatenated keys / values byte for byte
(what the reference's torch.cat cache would hold), the fused decode step must match the oracle's
attention over everything stored (fp32: 2e-4 rel + 1e-4 abs; bf16: the 2e-3 / 1e-3 gate).
"""
import numpy as np
import pytest
import torch

from helpers import gate

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("d,bk,bv,G", [(128, 4, 4, 4), (64, 3, 3, 7), (256, 4, 2, 2)])
def test_prefill_then_decode_steps(oracle, tables, d, bk, bv, G):
    from fused_turboquant_b200 import TurboQuantMSE
    from fused_turboquant_b200.hf_cache import CompressedKVCache
    B, Hkv, n_layers, prefill, steps = 2, 2, 2, 37, 3
    rng = np.random.default_rng(d + bk)
    total = prefill + steps
    K = rng.standard_normal((n_layers, B, Hkv, total, d)).astype(np.float32)
    V = rng.standard_normal((n_layers, B, Hkv, total, d)).astype(np.float32)
    signs = tables[f"signs_d{d}"]
    cache = CompressedKVCache(TurboQuantMSE(d, bk, device="cuda"), n_layers=n_layers, max_seq_len=64,
                              quantizer_v=TurboQuantMSE(d, bv, device="cuda"))
    cu = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    assert cache.get_compressed_key(0) is None and cache.get_seq_length() == 0
    for layer in range(n_layers):
        cache.store_compressed_kv(cu(K[layer][:, :, :prefill]), cu(V[layer][:, :, :prefill]), layer)
    for s in range(steps):
        n = prefill + s + 1
        for layer in range(n_layers):
            # the two-call form of the reference's API
            cache.store_compressed_key(cu(K[layer][:, :, n - 1:n]), layer)
            cache.store_compressed_value(cu(V[layer][:, :, n - 1:n]), layer)
            assert cache.get_seq_length(layer) == n
            k_idx, k_n = oracle.encode(K[layer][:, :, :n], signs, tables[f"boundaries_d{d}_b{bk}"], bk)
            v_idx, v_n = oracle.encode(V[layer][:, :, :n], signs, tables[f"boundaries_d{d}_b{bv}"], bv)
            ek, ev = cache.get_compressed_key(layer), cache.get_compressed_value(layer)
            np.testing.assert_array_equal(ek["packed_indices"].cpu().numpy(), k_idx)
            np.testing.assert_array_equal(ev["packed_indices"].cpu().numpy(), v_idx)
            np.testing.assert_array_equal(ek["norms"].cpu().numpy().view(np.uint16), k_n.view(np.uint16))
            np.testing.assert_array_equal(ev["norms"].cpu().numpy().view(np.uint16), v_n.view(np.uint16))
            q = rng.standard_normal((B, Hkv * G, 1, d)).astype(np.float32)
            ref = oracle.decode_attn(q[:, :, 0], k_idx, k_n, v_idx, v_n, tables[f"levels_d{d}_b{bk}"],
                                     tables[f"levels_d{d}_b{bv}"], signs, d ** -0.5, bk, bv)
            out = cache.decode_attention(cu(q), layer)
            assert out.shape == (B, Hkv * G, 1, d)
            assert gate(out[:, :, 0].cpu().numpy(), ref, 2e-4, 1e-4) == 0
            qb = cu(q).bfloat16()
            ref_b = oracle.decode_attn(qb.float().cpu().numpy()[:, :, 0], k_idx, k_n, v_idx, v_n,
                                       tables[f"levels_d{d}_b{bk}"], tables[f"levels_d{d}_b{bv}"],
                                       signs, d ** -0.5, bk, bv)
            out_b = cache.decode_attention(qb, layer)
            assert out_b.dtype == torch.bfloat16
            ob = out_b[:, :, 0].float().cpu().numpy()
            ulp = np.abs(ref_b) * 2.0 ** -7 + 1e-30
            assert (np.abs(ob - ref_b) <= 1e-3 + 2e-3 * np.abs(ref_b) + ulp).all()
    # dense values for the unfused path, and reset
    dense = cache.decode_values(0)
    ref_dense = oracle.decode_dense(v_idx, v_n, tables[f"levels_d{d}_b{bv}"], signs, bv, d)
    assert dense.shape == (B, Hkv, total, d)
    cache.reset()
    assert cache.get_seq_length(0) == 0 and cache.get_compressed_value(1) is None
    np.testing.assert_allclose(dense.cpu().numpy(), oracle.decode_dense(
        *oracle.encode(V[0][:, :, :total], signs, tables[f"boundaries_d{d}_b{bv}"], bv),
        tables[f"levels_d{d}_b{bv}"], signs, bv, d), rtol=1e-6, atol=1e-30)
    del ref_dense


def test_capacity_and_argument_errors():
    from fused_turboquant_b200 import TurboQuantMSE
    from fused_turboquant_b200.hf_cache import CompressedKVCache
    tq = TurboQuantMSE(128, 4, device="cuda")
    cache = CompressedKVCache(tq, n_layers=1, max_seq_len=16)
    x = torch.zeros((1, 2, 17, 128), device="cuda")
    with pytest.raises(RuntimeError):
        cache.store_compressed_kv(x, x, 0)
    with pytest.raises(RuntimeError):
        cache.store_compressed_value(x[:, :, :1], 0)
    with pytest.raises(ValueError):       # one sign table per pool: the seeds must agree
        CompressedKVCache(tq, quantizer_v=TurboQuantMSE(128, 3, seed=7, device="cuda"))
    with pytest.raises(RuntimeError):     # K-only cache: values are not stored here
        CompressedKVCache(tq, compress_v=False).store_compressed_value(x[:, :, :1], 0)


def test_ragged_batch_preallocated_and_dynamic_cache_base(oracle, tables):
    """Right-padded prompts of different lengths, then decode steps: every sequence's tokens sit
    behind its own last one; all pools exist before the first store; the class is a
    transformers.DynamicCache when transformers is importable."""
    from fused_turboquant_b200 import TurboQuantMSE
    from fused_turboquant_b200.hf_cache import CompressedKVCache
    d, bits, B, Hkv, G, n_layers = 128, 4, 3, 2, 4, 2
    tq = TurboQuantMSE(d, bits, device="cuda")
    cache = CompressedKVCache(tq, max_seq_len=96, batch_size=B, num_kv_heads=Hkv, n_layers=n_layers,
                              device="cuda")
    try:
        from transformers import DynamicCache
        assert isinstance(cache, DynamicCache)
    except ImportError:
        pass
    assert len(cache._pools) == n_layers                       # allocated at construction
    before = torch.cuda.memory_allocated()
    rng = np.random.default_rng(3)
    lens = np.array([40, 7, 23])
    pad = int(lens.max())
    steps = 4
    K = rng.standard_normal((B, Hkv, pad + steps, d)).astype(np.float32)
    V = rng.standard_normal((B, Hkv, pad + steps, d)).astype(np.float32)
    cu = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    hist_k = [[K[b, :, :lens[b]]] for b in range(B)]
    hist_v = [[V[b, :, :lens[b]]] for b in range(B)]
    for layer in range(n_layers):
        cache.store_compressed_kv(cu(K[:, :, :pad]), cu(V[:, :, :pad]), layer,
                                  new_lens=torch.from_numpy(lens))
    for s in range(steps):
        for layer in range(n_layers):
            cache.store_compressed_kv(cu(K[:, :, pad + s:pad + s + 1]), cu(V[:, :, pad + s:pad + s + 1]), layer)
        for b in range(B):
            hist_k[b].append(K[b, :, pad + s:pad + s + 1])
            hist_v[b].append(V[b, :, pad + s:pad + s + 1])
    assert cache.seq_lens(0).cpu().tolist() == (lens + steps).tolist()
    q = rng.standard_normal((B, Hkv * G, 1, d)).astype(np.float32)
    out = cache.decode_attention(cu(q), 1)
    signs, bnd, lv = tables[f"signs_d{d}"], tables[f"boundaries_d{d}_b{bits}"], tables[f"levels_d{d}_b{bits}"]
    for b in range(B):
        kb = np.concatenate(hist_k[b], axis=1)[None]
        vb = np.concatenate(hist_v[b], axis=1)[None]
        k_idx, k_n = oracle.encode(kb, signs, bnd, bits)
        v_idx, v_n = oracle.encode(vb, signs, bnd, bits)
        ref = oracle.decode_attn(q[b:b + 1, :, 0], k_idx, k_n, v_idx, v_n, lv, lv, signs, d ** -0.5,
                                 bits, bits)
        assert gate(out[b:b + 1, :, 0].cpu().numpy(), ref, 2e-4, 1e-4) == 0, b
    # nothing but the step's own outputs / workspace was allocated after construction
    assert torch.cuda.memory_allocated() - before < 8 << 20


def test_keys_only_cache_matches_dense_attention(oracle, tables):
    """compress_v=False (reference: fused_cache.py:559-570, 619-624): compressed keys, the caller's
    own values."""
    from fused_turboquant_b200 import TurboQuantMSE
    from fused_turboquant_b200.hf_cache import CompressedKVCache
    d, bits, B, Hkv, G, S = 64, 3, 2, 2, 3, 29
    tq = TurboQuantMSE(d, bits, device="cuda")
    cache = CompressedKVCache(tq, compress_v=False)
    rng = np.random.default_rng(9)
    K = rng.standard_normal((B, Hkv, S, d)).astype(np.float32)
    V = rng.standard_normal((B, Hkv, S, d)).astype(np.float32)
    cu = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    cache.store_compressed_key(cu(K[:, :, :20]), 0)
    cache.store_compressed_kv(cu(K[:, :, 20:]), cu(V[:, :, 20:]), 0)       # stores the keys only
    assert cache.get_seq_length(0) == S and cache.get_compressed_value(0) is None
    signs = tables[f"signs_d{d}"]
    k_idx, k_n = oracle.encode(K, signs, tables[f"boundaries_d{d}_b{bits}"], bits)
    np.testing.assert_array_equal(cache.get_compressed_key(0)["packed_indices"].cpu().numpy(), k_idx)
    q = rng.standard_normal((B, Hkv * G, 1, d)).astype(np.float32)
    out = cache.decode_attention(cu(q), 0, full_values=cu(V))
    Kd = oracle.decode_dense(k_idx, k_n, tables[f"levels_d{d}_b{bits}"], signs, bits, d)
    Kx = np.repeat(Kd, G, axis=1)
    Vx = np.repeat(V, G, axis=1)
    sc = np.einsum("bhd,bhsd->bhs", q[:, :, 0], Kx) * d ** -0.5
    w = np.exp(sc - sc.max(-1, keepdims=True))
    w /= w.sum(-1, keepdims=True)
    ref = np.einsum("bhs,bhsd->bhd", w, Vx)
    assert gate(out[:, :, 0].cpu().numpy(), ref, 2e-4, 2e-4) == 0
