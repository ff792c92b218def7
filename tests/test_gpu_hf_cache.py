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
    with pytest.raises(ValueError):
        CompressedKVCache(tq, compress_v=False, n_layers=1)
