"""The C-ABI library loads on a machine without a GPU and exports every symbol the header declares."""
import ctypes
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from fused_turboquant_b200 import _lib, build
    build.build()
    return _lib.load()


def header_symbols():
    text = open(os.path.join(ROOT, "include", "ftq_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ftq_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound(lib):
    from fused_turboquant_b200 import _lib
    syms = header_symbols()
    assert len(syms) >= 14
    for s in syms:
        assert hasattr(lib, s), f"{s} declared in ftq_b200.h but not exported"
    assert sorted(_lib.SIGNATURES) == syms, "ctypes signature table out of sync with the header"


def test_pure_host_entry_points(lib):
    assert lib.ftq_version() >= 100
    assert lib.ftq_last_error() == b"" or isinstance(lib.ftq_last_error(), bytes)
    assert [lib.ftq_packed_dim(128, b) for b in (4, 3, 2)] == [64, 48, 32]
    assert lib.ftq_packed_dim(128, 5) == -1
    # 16 * (pdk + pdv + 4): 2112 B at D=128 K4V4, 832 at D=64 K3V3, 3136 at D=256 K4V2
    assert lib.ftq_page_bytes(128, 4, 4) == 2112
    assert lib.ftq_page_bytes(64, 3, 3) == 832
    assert lib.ftq_page_bytes(256, 4, 2) == 3136
    assert lib.ftq_page_bytes(100, 4, 4) == -1
    assert lib.ftq_decode_workspace_bytes(64, 32, 8, 128, 8192, 1) > 0
    assert lib.ftq_decode_workspace_bytes(64, 32, 5, 128, 8192, 1) == 0     # Hq % Hkv != 0


def test_argument_errors_are_reported_before_any_gpu_work(lib):
    """Bad arguments return a negative status and a message; nothing is launched."""
    f32 = ctypes.POINTER(ctypes.c_float)
    signs = np.ones(128, np.float32)
    bounds = np.linspace(-1, 1, 17).astype(np.float32)
    fake = ctypes.c_void_p(0x1000)
    rc = lib.ftq_encode(fake, 0, 4, 128, 128, 5, signs.ctypes.data_as(f32), bounds.ctypes.data_as(f32),
                        fake, fake, None)
    assert rc == -1 and b"bits must be 2, 3, or 4" in lib.ftq_last_error()
    rc = lib.ftq_encode(fake, 0, 4, 96, 96, 4, signs.ctypes.data_as(f32), bounds.ctypes.data_as(f32),
                        fake, fake, None)
    assert rc == -2 and b"head_dim" in lib.ftq_last_error()
    bad = signs.copy(); bad[5] = 0.5
    rc = lib.ftq_encode(fake, 0, 4, 128, 128, 4, bad.ctypes.data_as(f32), bounds.ctypes.data_as(f32),
                        fake, fake, None)
    assert rc == -1 and b"signs[5]" in lib.ftq_last_error()
    rc = lib.ftq_encode(ctypes.c_void_p(0x1004), 0, 4, 128, 128, 4, signs.ctypes.data_as(f32),
                        bounds.ctypes.data_as(f32), fake, fake, None)
    assert rc == -1 and b"aligned" in lib.ftq_last_error()
    assert lib.ftq_encode(None, 0, 0, 128, 128, 4, None, bounds.ctypes.data_as(f32), None, None, None) == 0


def test_python_surface_validation_without_gpu():
    import torch
    from fused_turboquant_b200 import CompressedTensor, TurboQuantMSE, kernels
    with pytest.raises(ValueError, match="power of 2"):
        TurboQuantMSE(100, 4, device="cpu")
    with pytest.raises(ValueError, match="bits must be 2, 3, or 4"):
        TurboQuantMSE(128, 1, device="cpu")
    tq = TurboQuantMSE(128, 4, device="cpu")          # tables build on the host
    assert tq.quantizer.levels.shape == (16,) and tq.quantizer.boundaries.shape == (17,)
    assert tq.rotation.signs.abs().eq(1).all()
    lv = tq.quantizer.levels
    assert (lv[1:] > lv[:-1]).all()
    assert torch.allclose(lv, -lv.flip(0), atol=1e-6)         # symmetric codebook
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        tq.encode(torch.randn(2, 128))                        # no CPU fallback
    ct = CompressedTensor(torch.zeros(10, 64, dtype=torch.uint8), torch.zeros(10, dtype=torch.float16), 128, 4)
    assert abs(ct.compression_ratio - 256 / 66) < 1e-9
    assert kernels.triton_fused_encode is kernels.fused_encode
    assert kernels.packed_dim(128, 3) == 48


def test_tables_match_reference_fixtures(tables):
    from fused_turboquant_b200 import codebook
    for d in (64, 128, 256):
        np.testing.assert_array_equal(codebook.rht_signs(d, 42), tables[f"signs_d{d}"])
        for b in (2, 3, 4):
            bd, lv = codebook.codebook_f32(d, b)
            np.testing.assert_array_equal(bd, tables[f"boundaries_d{d}_b{b}"])
            np.testing.assert_array_equal(lv, tables[f"levels_d{d}_b{b}"])
    assert not np.array_equal(codebook.rht_signs(128, 42), codebook.rht_signs(128, 43))
    np.testing.assert_array_equal(codebook.rht_signs(128, 7), codebook.rht_signs(128, 7))
