"""Pins the oracle's restatement of the vLLM-v1 slot-format path (store + split-KV decode) to
what the reference's own Triton kernels produced in interpreter mode (tests/golden/tq_v1.npz,
written by tests/golden/make_golden_tq_v1.py)."""
import numpy as np
import pytest

from helpers import tq_v1_compare_cache

CASES = ["d128_k4v4", "d128_k3v4_nc", "d64_k3v3_g7", "d256_k4v2", "d128_k2v8",
         "d128_k1v1_nc", "d64_k1v3", "d256_k3v1_nc",
         "d128_k4v4_nc_vlm", "d64_k4v4_vlm", "d128_k3v4_nc_vlm",   # _vlm: Lloyd-Max value codes
         "d128_k8v4", "d64_k8v2", "d256_k8v3"]                     # k8: FP8 (e4m3) keys


# 8-bit Lloyd-Max key codes (tq_v1_k8mse.npz): the fixtures' meta says 8 key bits like the FP8
# cases; the oracle and the C ABI tell the two apart by key_bits = 264
K8MSE = ["d128_k8mse_v4_nc", "d64_k8mse_v3", "d256_k8mse_v2_nc"]


def _case(golden, name):
    g = golden("tq_v1_k8mse.npz" if name in K8MSE else "tq_v1.npz")
    meta = [int(v) for v in g[f"{name}_meta"]]
    if name in K8MSE:
        meta[3] = 264
    return g, meta


@pytest.mark.parametrize("name", CASES + K8MSE)
def test_store_matches_reference_store_kernel(oracle, golden, name):
    g, (D, Hkv, G, kb, vb, nc, splits, bs, slot, nb) = _case(golden, name)
    assert slot == oracle.tq_slot_bytes(D, kb, vb)
    cache = np.zeros((nb, bs, Hkv, slot), np.uint8)
    vlm = name.endswith("_vlm")
    y = oracle.tq_store(g[f"{name}_K"], g[f"{name}_V"], cache, g[f"{name}_slot_mapping"],
                        g[f"{name}_midpoints"], kb, vb, return_rotated=True, value_lloyd_max=vlm)
    stats = tq_v1_compare_cache(cache, g[f"{name}_cache"], g[f"{name}_slot_mapping"],
                                g[f"{name}_kun"] if kb == 8 else y,
                                g[f"{name}_midpoints"], D, kb, vb, bs,
                                vy=g[f"{name}_vy"] if vlm else None)
    # FP8 keys: every byte the interpreter and the oracle disagree on is a subnormal or a tie
    assert stats["key_fp8_differ_unexplained"] == 0 and stats["key_fp8_vs_rne"] == 0, stats
    # (Lloyd-Max values: codes and norm are held to the same bar as the key's)
    assert stats["value_codes_differ_off_midpoint"] == 0 and stats["value_norm_max_ulp"] <= 1
    # value codes / scale / zero and every untouched byte: identical.  Key codes: identical except
    # where the rotated value sits on a midpoint (none expected in these fixtures); key norms:
    # at most one fp16 ulp (summation order of the squares is not fixed by the reference)
    assert stats["value_bytes_differ"] == 0 and stats["other_bytes_differ"] == 0
    assert stats["key_codes_differ_off_midpoint"] == 0
    assert stats["key_norm_max_ulp"] <= 1
    # the rotated unit key matches the torch restatement stored with the fixture
    sm = g[f"{name}_slot_mapping"]
    np.testing.assert_allclose(y[sm >= 0], g[f"{name}_y"][sm >= 0], atol=2e-6)


@pytest.mark.parametrize("name", CASES + K8MSE)
def test_decode_matches_reference_decode_kernels(oracle, golden, name):
    g, (D, Hkv, G, kb, vb, nc, splits, bs, slot, nb) = _case(golden, name)
    out, mid_o, lse = oracle.tq_decode(g[f"{name}_q"], g[f"{name}_cache"], g[f"{name}_block_table"],
                                       g[f"{name}_seq_lens"], g[f"{name}_centroids"], kb, vb,
                                       D ** -0.5, splits, norm_correction=bool(nc),
                                       kv_start=g[f"{name}_kv_start"],
                                       value_lloyd_max=name.endswith("_vlm"))
    ref = g[f"{name}_mid_o"]
    live = np.isfinite(ref[..., D])
    np.testing.assert_array_equal(np.isfinite(mid_o[..., D]), live)      # same empty splits
    np.testing.assert_allclose(mid_o[..., D][live], ref[..., D][live], rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(mid_o[..., :D][live], ref[..., :D][live], rtol=2e-4, atol=2e-5)
    assert np.all(mid_o[..., :D][~live] == 0)
    if f"{name}_out" in g.files:
        np.testing.assert_allclose(out, g[f"{name}_out"], rtol=2e-4, atol=2e-5)
        np.testing.assert_allclose(lse, g[f"{name}_lse"], rtol=1e-5, atol=1e-5)
    else:
        # kv_start > 0: the fixture has no merged output; merge the reference's partials here
        l = np.where(live, ref[..., D], -np.inf)
        w = np.exp(l - l.max(axis=-1, keepdims=True))
        merged = (w[..., None] * ref[..., :D]).sum(-2) / w.sum(-1)[..., None]
        np.testing.assert_allclose(out, merged, rtol=2e-4, atol=2e-5)
