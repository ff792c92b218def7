"""Pins the CPU oracle (oracle/ftq_oracle.c) to outputs of the reference itself
(fixtures under tests/golden/, written by tests/golden/make_golden.py)."""
import numpy as np
import pytest

DIMS = (64, 128, 256)
BITS = (2, 3, 4)


def bf16_bits_to_f32(u16: np.ndarray) -> np.ndarray:
    return (u16.astype(np.uint32) << 16).view(np.float32)


def test_fwht_known_answer_d2(oracle, golden):
    # the reference's only known-answer test: fwht([1, 0]) == [1/sqrt2, 1/sqrt2]
    g = golden("fwht_kat.npz")
    y = oracle.fwht(g["x2"])
    np.testing.assert_array_equal(y, g["y2"])
    np.testing.assert_allclose(y, [2 ** -0.5, 2 ** -0.5], rtol=1e-7)


@pytest.mark.parametrize("d", DIMS)
def test_fwht_and_rht_match_reference_bitwise(oracle, golden, tables, d):
    g = golden("fwht_kat.npz")
    np.testing.assert_array_equal(oracle.fwht(g[f"x_d{d}"]), g[f"fwht_d{d}"])
    np.testing.assert_array_equal(oracle.rht(g[f"x_d{d}"], tables[f"signs_d{d}"]), g[f"rht_d{d}"])


@pytest.mark.parametrize("d", DIMS)
def test_rht_is_an_involution_and_keeps_norms(oracle, tables, d):
    rng = np.random.default_rng(d)
    x = rng.standard_normal((64, d)).astype(np.float32)
    s = tables[f"signs_d{d}"]
    y = oracle.rht(x, s)
    np.testing.assert_allclose(np.linalg.norm(y, axis=-1), np.linalg.norm(x, axis=-1), rtol=1e-5)
    np.testing.assert_allclose(oracle.rht(y, s, inverse=True), x, atol=1e-5)


@pytest.mark.parametrize("bits", BITS)
@pytest.mark.parametrize("d", DIMS)
def test_pack_roundtrip(oracle, d, bits):
    # includes 3-bit, which the reference's own tests leave out
    rng = np.random.default_rng(7 * d + bits)
    idx = rng.integers(0, 1 << bits, size=(33, d), dtype=np.uint8)
    p = oracle.pack(idx, bits)
    assert p.shape == (33, d * bits // 8)
    np.testing.assert_array_equal(oracle.unpack(p, d, bits), idx)


@pytest.mark.parametrize("bits", BITS)
@pytest.mark.parametrize("d", DIMS)
@pytest.mark.parametrize("kind", ["x32", "xbf"])
def test_encode_bit_exact_vs_reference(oracle, golden, tables, d, bits, kind):
    g = golden("encode.npz")
    x = g[f"x32_d{d}"] if kind == "x32" else bf16_bits_to_f32(g[f"xbf_d{d}"])
    packed, norms = oracle.encode(x, tables[f"signs_d{d}"], tables[f"boundaries_d{d}_b{bits}"], bits)
    np.testing.assert_array_equal(packed, g[f"{kind}_d{d}_b{bits}_packed"])
    np.testing.assert_array_equal(norms.view(np.uint16), g[f"{kind}_d{d}_b{bits}_norms"].view(np.uint16))


@pytest.mark.parametrize("bits", BITS)
@pytest.mark.parametrize("d", DIMS)
def test_decode_dense_vs_reference(oracle, golden, tables, d, bits):
    g, e = golden("decode_dense.npz"), golden("encode.npz")
    out = oracle.decode_dense(e[f"x32_d{d}_b{bits}_packed"], e[f"x32_d{d}_b{bits}_norms"],
                              tables[f"levels_d{d}_b{bits}"], tables[f"signs_d{d}"], bits, d)
    np.testing.assert_array_equal(out, g[f"d{d}_b{bits}"])


ATT_CASES = ["cfg1small", "d64_g7_k3v3", "d256_g2_k4v2"]


@pytest.mark.parametrize("name", ATT_CASES)
def test_attention_oracle_vs_reference(oracle, golden, tables, name):
    g = golden("attention.npz")
    B, Hkv, G, S, d, bk, bv = g[f"{name}_meta"]
    q = g[f"{name}_q"][:, :, 0, :]
    args = (q, g[f"{name}_k_idx"], g[f"{name}_k_norms"], g[f"{name}_v_idx"], g[f"{name}_v_norms"],
            tables[f"levels_d{d}_b{bk}"], tables[f"levels_d{d}_b{bv}"], tables[f"signs_d{d}"],
            float(d) ** -0.5, int(bk), int(bv))
    out = oracle.decode_attn(*args)
    ref = g[f"{name}_out_full"][:, :, 0, :]
    # fp32 reference vs double-accumulating oracle: far inside the 2e-3 / 1e-3 gate
    np.testing.assert_allclose(out, ref, rtol=2e-4, atol=2e-5)
    out_m = oracle.decode_attn(*args, seq_lens=g[f"{name}_seq_lens"])
    np.testing.assert_allclose(out_m, g[f"{name}_out_masked"][:, :, 0, :], rtol=2e-4, atol=2e-5)


@pytest.mark.parametrize("name", ATT_CASES)
def test_encode_of_attention_inputs_matches(oracle, golden, tables, name):
    g = golden("attention.npz")
    B, Hkv, G, S, d, bk, bv = g[f"{name}_meta"]
    for t, bits in (("K", bk), ("V", bv)):
        packed, norms = oracle.encode(g[f"{name}_{t}"], tables[f"signs_d{d}"],
                                      tables[f"boundaries_d{d}_b{bits}"], int(bits))
        np.testing.assert_array_equal(packed, g[f"{name}_{t.lower()}_idx"])
        np.testing.assert_array_equal(norms.view(np.uint16), g[f"{name}_{t.lower()}_norms"].view(np.uint16))


@pytest.mark.parametrize("name", ATT_CASES)
def test_qk_scores_rotated_space(oracle, golden, tables, name):
    g = golden("attention.npz")
    B, Hkv, G, S, d, bk, bv = g[f"{name}_meta"]
    s = oracle.qk_scores(g[f"{name}_q_rot"][:, :, 0, :], g[f"{name}_k_idx"],
                         g[f"{name}_k_norms"].astype(np.float32), tables[f"levels_d{d}_b{bk}"],
                         float(d) ** -0.5, int(bk))
    np.testing.assert_allclose(s, g[f"{name}_scores_rot"][:, :, 0, :], rtol=1e-4, atol=1e-4)
    # and the rotated-space scores agree with the decoded-space scores of the unfused path
    np.testing.assert_allclose(s, g[f"{name}_scores"][:, :, 0, :], rtol=1e-3, atol=2e-4)


def test_v0_layout_write_and_gather(oracle, golden):
    g = golden("v0_layout.npz")
    d, b, Hkv, bs, nb, es, n_tok = g["meta"]
    cache = np.zeros((2, nb, bs, Hkv, es), np.uint8)
    oracle.v0_write(cache, 0, g["packed"], g["norms"], g["slots"])
    np.testing.assert_array_equal(cache, g["cache"])
    gp, gn = oracle.v0_gather(cache, 0, d // 2, g["block_table"], np.array([n_tok], np.int32), 48)
    np.testing.assert_array_equal(gp, g["gathered_packed"])
    np.testing.assert_array_equal(gn, g["gathered_norms"])
    # negative slots are skipped
    cache2 = np.zeros_like(cache)
    slots = g["slots"].copy(); slots[::2] = -1
    oracle.v0_write(cache2, 0, g["packed"], g["norms"], slots)
    assert not np.array_equal(cache2, cache)
    keep = cache2.reshape(2, nb * bs, Hkv, es)[0, g["slots"][1::2]]
    np.testing.assert_array_equal(keep, cache.reshape(2, nb * bs, Hkv, es)[0, g["slots"][1::2]])


def test_slot_sizes_match_reference_tests():
    # reference tests/test_vllm_backend.py:28-43: 68 / 52 / 36 bytes at d=128, 36 at (64, 4)
    from fused_turboquant_b200.paged import compute_compressed_elem_size as ces
    assert (ces(128, 4), ces(128, 3), ces(128, 2), ces(64, 4)) == (68, 52, 36, 36)


def test_f16_conversion_matches_numpy(oracle):
    rng = np.random.default_rng(0)
    x = np.concatenate([rng.standard_normal(4000) * 10.0 ** rng.integers(-9, 6, 4000),
                        [0.0, -0.0, 65504.0, 65519.9, 65520.0, 1e-8, 5.96e-8, 2.98e-8, 6.1e-5]]
                       ).astype(np.float32)
    L = oracle.lib()
    got = np.array([L.ftq_oracle_f32_to_f16(float(v)) for v in x], np.uint16)
    with np.errstate(over="ignore"):
        np.testing.assert_array_equal(got, x.astype(np.float16).view(np.uint16))
    back = np.array([L.ftq_oracle_f16_to_f32(int(v)) for v in got], np.float32)
    np.testing.assert_array_equal(back, got.view(np.float16).astype(np.float32))
