"""GPU parity of the CUDA path against outputs of the reference's own GPU kernels.

Fixtures: tests/golden/kernels_interp.npz (the reference's Triton kernels executed in
interpreter mode; see tests/golden/make_golden_kernels.py).  Integer results must be equal
byte for byte; floating-point results are held to the tolerance written next to each check.
"""
import numpy as np
import pytest
import torch

from helpers import gate

pytestmark = pytest.mark.gpu

DIMS = (64, 128, 256)
BITS = (2, 3, 4)
ATT_CASES = ["cfg1small", "d64_g7_k3v3", "d256_g2_k4v2"]
cu = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("bits", BITS)
@pytest.mark.parametrize("d", DIMS)
def test_encode_equals_reference_encode_kernel(golden, tables, d, bits):
    from fused_turboquant_b200 import kernels
    k, e = golden("kernels_interp.npz"), golden("encode.npz")
    packed, norms = kernels.fused_encode(cu(e[f"x32_d{d}"]), tables[f"signs_d{d}"],
                                         tables[f"boundaries_d{d}_b{bits}"], bits)
    np.testing.assert_array_equal(packed.cpu().numpy(), k[f"enc_d{d}_b{bits}_packed"])
    np.testing.assert_array_equal(norms.cpu().numpy().view(np.uint16),
                                  k[f"enc_d{d}_b{bits}_norms"].view(np.uint16))
    # the bulk kernel takes over at 2048 vectors: tile the same rows and expect the same bytes
    reps = 2048 // e[f"x32_d{d}"].shape[0] + 1
    big = np.tile(e[f"x32_d{d}"], (reps, 1))
    packed2, norms2 = kernels.fused_encode(cu(big), tables[f"signs_d{d}"],
                                           tables[f"boundaries_d{d}_b{bits}"], bits)
    np.testing.assert_array_equal(packed2.cpu().numpy(), np.tile(k[f"enc_d{d}_b{bits}_packed"], (reps, 1)))
    np.testing.assert_array_equal(norms2.cpu().numpy().view(np.uint16),
                                  np.tile(k[f"enc_d{d}_b{bits}_norms"].view(np.uint16), reps))


@pytest.mark.parametrize("d,bits", [(64, 2), (128, 4), (256, 3)])
def test_dense_decode_equals_reference_decode_kernel(golden, tables, d, bits):
    from fused_turboquant_b200 import kernels
    k, e = golden("kernels_interp.npz"), golden("encode.npz")
    out = kernels.fused_decode(cu(e[f"x32_d{d}_b{bits}_packed"]), cu(e[f"x32_d{d}_b{bits}_norms"]),
                               tables[f"levels_d{d}_b{bits}"], tables[f"signs_d{d}"], bits, d)
    ref = k[f"dec_d{d}_b{bits}"]
    out = out.cpu().numpy()
    finite = np.isfinite(ref)
    np.testing.assert_array_equal(np.isfinite(out), finite)
    np.testing.assert_allclose(out[finite], ref[finite], rtol=1e-6, atol=1e-30)


@pytest.mark.parametrize("d", DIMS)
def test_rht_equals_reference_rht_kernel(golden, tables, d):
    from fused_turboquant_b200 import kernels
    k, g = golden("kernels_interp.npz"), golden("fwht_kat.npz")
    y = kernels.rht(cu(g[f"x_d{d}"]), tables[f"signs_d{d}"])
    np.testing.assert_array_equal(y.cpu().numpy(), k[f"rht_d{d}"])
    back = kernels.rht(y, tables[f"signs_d{d}"], inverse=True)
    np.testing.assert_array_equal(back.cpu().numpy(), k[f"irht_d{d}"])


@pytest.mark.parametrize("name", ATT_CASES)
def test_scores_and_attention_vs_reference_kernels(golden, tables, name):
    from fused_turboquant_b200 import kernels
    k, g = golden("kernels_interp.npz"), golden("attention.npz")
    B, Hkv, G, S, d, bk, bv = (int(v) for v in g[f"{name}_meta"])
    lk, lv = tables[f"levels_d{d}_b{bk}"], tables[f"levels_d{d}_b{bv}"]
    s = kernels.fused_qk_scores_rht(cu(g[f"{name}_q_rot"]), cu(g[f"{name}_k_idx"]),
                                    cu(g[f"{name}_k_norms"].astype(np.float32)), lk, d ** -0.5, bits=bk)
    np.testing.assert_allclose(s.cpu().numpy(), k[f"{name}_scores"], rtol=1e-4, atol=1e-4)
    # fp32 query: fp32 CUDA-core kernel, held to a tenth of the gate
    common = (cu(g[f"{name}_k_idx"]), cu(g[f"{name}_k_norms"]), cu(g[f"{name}_v_idx"]),
              cu(g[f"{name}_v_norms"]), lk, lv, tables[f"signs_d{d}"], d ** -0.5, bk, bv)
    out = kernels.flash_decode_compressed(cu(g[f"{name}_q_rot"]), *common)
    assert gate(out.cpu().numpy(), k[f"{name}_flash"], 2e-4, 1e-4) == 0
