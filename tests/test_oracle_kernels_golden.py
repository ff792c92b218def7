"""Pins the CPU oracle to outputs of the reference's own GPU kernels.

The fixtures in tests/golden/kernels_interp.npz were produced by executing the reference's
Triton kernels (fused encode, fused dense decode, RHT, fused QK scores, fused flash decode) in
Triton's interpreter mode on the inputs stored in the other fixture files; see
tests/golden/make_golden_kernels.py.
"""
import numpy as np
import pytest

DIMS = (64, 128, 256)
BITS = (2, 3, 4)
ATT_CASES = ["cfg1small", "d64_g7_k3v3", "d256_g2_k4v2"]


@pytest.mark.parametrize("bits", BITS)
@pytest.mark.parametrize("d", DIMS)
def test_reference_kernel_and_unfused_reference_agree_on_encode(golden, d, bits):
    # the fused kernel (norm = sqrt(sum + 1e-16)) and the unfused path give the same bytes here,
    # so one oracle serves both
    k, e = golden("kernels_interp.npz"), golden("encode.npz")
    np.testing.assert_array_equal(k[f"enc_d{d}_b{bits}_packed"], e[f"x32_d{d}_b{bits}_packed"])
    np.testing.assert_array_equal(k[f"enc_d{d}_b{bits}_norms"].view(np.uint16),
                                  e[f"x32_d{d}_b{bits}_norms"].view(np.uint16))


@pytest.mark.parametrize("bits", BITS)
@pytest.mark.parametrize("d", DIMS)
def test_oracle_encode_equals_reference_encode_kernel(oracle, golden, tables, d, bits):
    k, e = golden("kernels_interp.npz"), golden("encode.npz")
    packed, norms = oracle.encode(e[f"x32_d{d}"], tables[f"signs_d{d}"],
                                  tables[f"boundaries_d{d}_b{bits}"], bits)
    np.testing.assert_array_equal(packed, k[f"enc_d{d}_b{bits}_packed"])
    np.testing.assert_array_equal(norms.view(np.uint16), k[f"enc_d{d}_b{bits}_norms"].view(np.uint16))


@pytest.mark.parametrize("d,bits", [(64, 2), (128, 4), (256, 3)])
def test_oracle_dense_decode_equals_reference_decode_kernel(oracle, golden, tables, d, bits):
    k, e = golden("kernels_interp.npz"), golden("encode.npz")
    out = oracle.decode_dense(e[f"x32_d{d}_b{bits}_packed"], e[f"x32_d{d}_b{bits}_norms"],
                              tables[f"levels_d{d}_b{bits}"], tables[f"signs_d{d}"], bits, d)
    np.testing.assert_array_equal(out, k[f"dec_d{d}_b{bits}"])  # NaN rows (fp16 norm overflow) included


@pytest.mark.parametrize("d", DIMS)
def test_oracle_rht_equals_reference_rht_kernel(oracle, golden, tables, d):
    k, g = golden("kernels_interp.npz"), golden("fwht_kat.npz")
    y = oracle.rht(g[f"x_d{d}"], tables[f"signs_d{d}"])
    np.testing.assert_array_equal(y, k[f"rht_d{d}"])
    np.testing.assert_array_equal(oracle.rht(y, tables[f"signs_d{d}"], inverse=True), k[f"irht_d{d}"])


@pytest.mark.parametrize("name", ATT_CASES)
def test_oracle_scores_vs_reference_qk_kernel(oracle, golden, tables, name):
    k, g = golden("kernels_interp.npz"), golden("attention.npz")
    B, Hkv, G, S, d, bk, bv = (int(v) for v in g[f"{name}_meta"])
    s = oracle.qk_scores(g[f"{name}_q_rot"][:, :, 0, :], g[f"{name}_k_idx"],
                         g[f"{name}_k_norms"].astype(np.float32), tables[f"levels_d{d}_b{bk}"],
                         float(d) ** -0.5, bk)
    np.testing.assert_allclose(s, k[f"{name}_scores"][:, :, 0, :], rtol=1e-5, atol=2e-5)


@pytest.mark.parametrize("name", ATT_CASES)
def test_oracle_attention_vs_reference_flash_decode_kernel(oracle, golden, tables, name):
    k, g = golden("kernels_interp.npz"), golden("attention.npz")
    B, Hkv, G, S, d, bk, bv = (int(v) for v in g[f"{name}_meta"])
    out = oracle.decode_attn(g[f"{name}_q"][:, :, 0, :], g[f"{name}_k_idx"], g[f"{name}_k_norms"],
                             g[f"{name}_v_idx"], g[f"{name}_v_norms"], tables[f"levels_d{d}_b{bk}"],
                             tables[f"levels_d{d}_b{bv}"], tables[f"signs_d{d}"], float(d) ** -0.5,
                             bk, bv)
    # fp32 kernel vs double-accumulating oracle: far inside the 2e-3 / 1e-3 gate
    np.testing.assert_allclose(out, k[f"{name}_flash"][:, :, 0, :], rtol=2e-4, atol=2e-5)
