"""GPU parity of the fused encode and the dense helpers, through the C ABI, against the oracle."""
import numpy as np
import pytest
import torch

from helpers import boundary_exempt

pytestmark = pytest.mark.gpu
DIMS = (64, 128, 256)
BITS = (2, 3, 4)


def _tables(tables, d, bits):
    return tables[f"signs_d{d}"], tables[f"boundaries_d{d}_b{bits}"], tables[f"levels_d{d}_b{bits}"]


def _unpack_codes(oracle, packed, d, bits):
    return oracle.unpack(packed, d, bits)


def _check_encode(oracle, x_t, x_np, signs, bounds, bits, d):
    """Codes bit-exact except coordinates within 1e-6 of a boundary; fp16 norms bit-exact."""
    from fused_turboquant_b200 import kernels
    packed, norms = kernels.fused_encode(x_t, signs, bounds, bits)
    rp, rn, normalized = oracle.encode(x_np, signs, bounds, bits, return_normalized=True)
    packed, norms = packed.cpu().numpy(), norms.cpu().numpy()
    assert packed.shape == rp.shape and norms.shape == rn.shape
    np.testing.assert_array_equal(norms.view(np.uint16), rn.view(np.uint16))
    if not np.array_equal(packed, rp):
        got = _unpack_codes(oracle, packed, d, bits)
        ref = _unpack_codes(oracle, rp, d, bits)
        bad = (got != ref) & ~boundary_exempt(normalized, bounds)
        assert bad.sum() == 0, f"{bad.sum()} code mismatches away from boundaries"
    return int((packed != rp).sum())


@pytest.mark.parametrize("bits", BITS)
@pytest.mark.parametrize("d", DIMS)
@pytest.mark.parametrize("kind", ["x32", "xbf"])
def test_encode_matches_golden_reference_outputs(golden, tables, d, bits, kind):
    """CUDA output == the reference's own output on the committed fixtures (bit for bit)."""
    from fused_turboquant_b200 import kernels
    g = golden("encode.npz")
    signs, bounds, _ = _tables(tables, d, bits)
    if kind == "x32":
        x = torch.from_numpy(g[f"x32_d{d}"]).cuda()
    else:
        x = torch.from_numpy(g[f"xbf_d{d}"].view(np.int16)).view(torch.bfloat16).cuda()
    packed, norms = kernels.fused_encode(x, signs, bounds, bits)
    np.testing.assert_array_equal(packed.cpu().numpy(), g[f"{kind}_d{d}_b{bits}_packed"])
    np.testing.assert_array_equal(norms.cpu().numpy().view(np.uint16),
                                  g[f"{kind}_d{d}_b{bits}_norms"].view(np.uint16))


@pytest.mark.parametrize("bits", BITS)
@pytest.mark.parametrize("d", DIMS)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_encode_vs_oracle_random(oracle, tables, d, bits, dtype):
    signs, bounds, _ = _tables(tables, d, bits)
    g = torch.Generator("cpu").manual_seed(1000 + d + bits)
    x = torch.randn(4099, d, generator=g)          # not a multiple of 4 vectors per warp
    x[:, :3] *= 20.0
    x = x.to(dtype)
    _check_encode(oracle, x.cuda(), x.float().numpy(), signs, bounds, bits, d)


@pytest.mark.parametrize("n", [0, 1, 3, 5, 33])
def test_encode_ragged_counts_and_shapes(oracle, tables, n):
    d, bits = 128, 4
    signs, bounds, _ = _tables(tables, d, bits)
    x = torch.randn(n, d, generator=torch.Generator("cpu").manual_seed(n))
    from fused_turboquant_b200 import kernels
    packed, norms = kernels.fused_encode(x.cuda(), signs, bounds, bits)
    assert packed.shape == (n, 64) and norms.shape == (n,)
    if n:
        _check_encode(oracle, x.cuda(), x.numpy(), signs, bounds, bits, d)
    # leading shape is kept, like the reference wrapper
    x4 = torch.randn(2, 3, 5, d).cuda()
    p4, n4 = kernels.fused_encode(x4, signs, bounds, bits)
    assert p4.shape == (2, 3, 5, 64) and n4.shape == (2, 3, 5)


def test_encode_config1_full_size(oracle, tables):
    """Benchmark configuration 1: K and V fp32 [1, 8, 1024, 128], 4 outlier channels per head x20, 4-bit."""
    d, bits = 128, 4
    signs, bounds, _ = _tables(tables, d, bits)
    g = torch.Generator("cpu").manual_seed(20251)
    kv = torch.randn(2, 1, 8, 1024, d, generator=g)
    for h in range(8):
        ch = torch.randperm(d, generator=g)[:4]
        kv[:, :, h, :, ch] *= 20.0
    flips = _check_encode(oracle, kv.cuda(), kv.numpy(), signs, bounds, bits, d)
    assert flips == 0


@pytest.mark.parametrize("bits", BITS)
@pytest.mark.parametrize("d", DIMS)
def test_dense_decode_and_roundtrip(oracle, golden, tables, d, bits):
    from fused_turboquant_b200 import TurboQuantMSE, kernels
    signs, bounds, levels = _tables(tables, d, bits)
    e, g = golden("encode.npz"), golden("decode_dense.npz")
    out = kernels.fused_decode(torch.from_numpy(e[f"x32_d{d}_b{bits}_packed"]).cuda(),
                               torch.from_numpy(e[f"x32_d{d}_b{bits}_norms"]).cuda(),
                               levels, signs, bits, d).cpu().numpy()
    # same operations in the same order as the reference: expected bit-identical, gate at 1e-6
    np.testing.assert_allclose(out, g[f"d{d}_b{bits}"], rtol=1e-6, atol=1e-30)
    # quality thresholds of the reference's tests (tests/test_quantizer.py:55-79)
    tq = TurboQuantMSE(d, bits, device="cuda")
    x = torch.randn(512, d, generator=torch.Generator("cpu").manual_seed(5)).cuda()
    y = tq.roundtrip(x)
    cos = torch.nn.functional.cosine_similarity(x, y, dim=-1).mean().item()
    assert cos > {4: 0.99, 3: 0.97, 2: 0.90}[bits]
    ct = tq.encode(x)
    assert ct.compression_ratio > 3


@pytest.mark.parametrize("d", DIMS)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_rht_forward_inverse(oracle, golden, tables, d, dtype):
    from fused_turboquant_b200 import kernels
    signs = tables[f"signs_d{d}"]
    x = torch.randn(257, d, generator=torch.Generator("cpu").manual_seed(d)).to(dtype)
    y = kernels.rht(x.cuda(), signs)
    assert y.dtype == dtype and y.shape == x.shape
    ref = oracle.rht(x.float().numpy(), signs)
    if dtype == torch.float32:
        np.testing.assert_array_equal(y.cpu().numpy(), ref)           # same op order: bit-exact
        g = golden("fwht_kat.npz")
        yk = kernels.rht(torch.from_numpy(g[f"x_d{d}"]).cuda(), signs)
        np.testing.assert_array_equal(yk.cpu().numpy(), g[f"rht_d{d}"])
        back = kernels.rht(y, signs, inverse=True).cpu().numpy()
        np.testing.assert_allclose(back, x.numpy(), atol=2e-5)
        np.testing.assert_array_equal(back, oracle.rht(ref, signs, inverse=True))
    else:
        np.testing.assert_array_equal(y.float().cpu().numpy(),
                                      torch.from_numpy(ref).to(dtype).float().numpy())
    # no signs = plain orthonormal FWHT
    y0 = kernels.rht(x.float().cuda(), None).cpu().numpy()
    np.testing.assert_array_equal(y0, oracle.fwht(x.float().numpy()))


def test_quantizer_api_errors_and_types(tables):
    from fused_turboquant_b200 import CompressedTensor, TurboQuantMSE
    with pytest.raises(ValueError):
        TurboQuantMSE(100, 4, device="cuda")
    with pytest.raises(ValueError):
        TurboQuantMSE(128, 5, device="cuda")
    tq = TurboQuantMSE(128, 3, device="cuda")
    ct = tq.encode(torch.randn(2, 4, 7, 128).cuda().half())
    assert isinstance(ct, CompressedTensor)
    assert ct.indices.dtype == torch.uint8 and ct.indices.shape == (2, 4, 7, 48)
    assert ct.norms.dtype == torch.float16 and ct.norms.shape == (2, 4, 7)
    assert tq.decode(ct).shape == (2, 4, 7, 128) and tq.decode(ct).dtype == torch.float32
    with pytest.raises(RuntimeError):
        tq.encode(torch.randn(4, 128))          # CPU tensor: no fallback
