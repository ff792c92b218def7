"""Shape contract and block copy / swap of the backend surface; mirrors the component tests of
the reference (tests/test_vllm_backend.py:28-109 there)."""
import pytest
import torch

from fused_turboquant_b200.backend import (FusedTurboQuantBackend, compressed_copy_blocks,
                                           compressed_swap_blocks)
from fused_turboquant_b200.paged import compute_compressed_elem_size


def test_compressed_elem_sizes():
    assert compute_compressed_elem_size(128, 4) == 68
    assert compute_compressed_elem_size(128, 3) == 52
    assert compute_compressed_elem_size(128, 2) == 36
    assert compute_compressed_elem_size(64, 4) == 36
    with pytest.raises(ValueError):
        compute_compressed_elem_size(128, 5)


def test_cache_shapes(monkeypatch):
    monkeypatch.setenv("TURBOQUANT_BITS", "4")
    monkeypatch.delenv("TURBOQUANT_V_BITS", raising=False)
    assert FusedTurboQuantBackend.get_kv_cache_shape(100, 16, 8, 128) == (2, 100, 16, 8, 68)
    monkeypatch.setenv("TURBOQUANT_BITS", "3")
    assert FusedTurboQuantBackend.get_kv_cache_shape(50, 16, 4, 128) == (2, 50, 16, 4, 52)
    monkeypatch.setenv("TURBOQUANT_V_BITS", "4")          # mixed bits: the wider slot wins
    assert FusedTurboQuantBackend.get_kv_cache_shape(50, 16, 4, 128) == (2, 50, 16, 4, 68)


def test_name_head_sizes_validation():
    assert FusedTurboQuantBackend.get_name() == "FUSED_TURBOQUANT"
    assert 128 in FusedTurboQuantBackend.get_supported_head_sizes()
    FusedTurboQuantBackend.validate_configuration(head_size=128)
    with pytest.raises(ValueError):
        FusedTurboQuantBackend.validate_configuration(head_size=96)
    with pytest.raises(ValueError):
        FusedTurboQuantBackend.validate_configuration(head_size=512)


def test_swap_and_copy_blocks():
    src = torch.randint(0, 255, (10, 16, 4, 68), dtype=torch.uint8)
    dst = torch.zeros_like(src)
    compressed_swap_blocks(src, dst, torch.tensor([[0, 5], [3, 7]]))
    assert torch.equal(dst[5], src[0]) and torch.equal(dst[7], src[3])
    assert dst[[0, 1, 2, 3, 4, 6, 8, 9]].abs().sum() == 0
    cache = torch.randint(0, 255, (2, 10, 16, 4, 68), dtype=torch.uint8)     # v0 layout
    pool = torch.randint(0, 255, (10, 4, 2112), dtype=torch.uint8)           # page layout
    c0, p0 = cache.clone(), pool.clone()
    compressed_copy_blocks([cache, pool], torch.tensor([[1, 8], [2, 9]]))
    assert torch.equal(cache[:, 8], c0[:, 1]) and torch.equal(cache[:, 9], c0[:, 2])
    assert torch.equal(pool[8], p0[1]) and torch.equal(pool[9], p0[2])
    assert torch.equal(cache[:, :8], c0[:, :8]) and torch.equal(pool[:8], p0[:8])
    compressed_copy_blocks([cache], torch.zeros(0, 2, dtype=torch.long))      # empty: no-op
