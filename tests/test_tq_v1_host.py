"""Host-side logic of the vLLM-v1 slot-format module and of the continuation helper (no GPU)."""
import numpy as np
import pytest
import torch

from fused_turboquant_b200 import tq_v1
from fused_turboquant_b200.paged import synthetic_decode_batch


@pytest.mark.parametrize("d,kb,vb,slot", [(128, 4, 4, 134), (128, 3, 4, 118), (64, 3, 3, 54),
                                          (256, 4, 2, 198), (128, 2, 8, 166), (128, 1, 1, 38),
                                          (64, 1, 3, 38), (256, 3, 1, 134), (128, 8, 4, 196),
                                          (64, 8, 2, 84), (256, 8, 3, 356)])
def test_slot_sizes_match_the_reference_kernels_fixture(golden, oracle, d, kb, vb, slot):
    cfg = tq_v1.TurboQuantSlotConfig(d, kb, vb)
    assert cfg.slot_size_aligned == slot == oracle.tq_slot_bytes(d, kb, vb)
    assert cfg.value_packed_size == cfg.value_data_bytes + 4
    if kb == 8:   # FP8 keys: one byte per coordinate, no norm, centroid table sized for the values
        assert cfg.key_fp8 and cfg.key_packed_size == d and cfg.key_mse_bits == 0
        assert cfg.n_centroids == 1 << vb
    else:
        assert cfg.key_packed_size == d * kb // 8 + 2
        assert cfg.n_centroids == 1 << kb and cfg.key_mse_bits == kb and not cfg.key_fp8
    g = golden("tq_v1.npz")
    names = {(128, 4, 4): "d128_k4v4", (128, 3, 4): "d128_k3v4_nc", (64, 3, 3): "d64_k3v3_g7",
             (256, 4, 2): "d256_k4v2", (128, 2, 8): "d128_k2v8", (128, 1, 1): "d128_k1v1_nc",
             (64, 1, 3): "d64_k1v3", (256, 3, 1): "d256_k3v1_nc", (128, 8, 4): "d128_k8v4",
             (64, 8, 2): "d64_k8v2", (256, 8, 3): "d256_k8v3"}
    assert int(g[f"{names[(d, kb, vb)]}_meta"][8]) == slot


def test_config_rejects_what_the_kernels_do_not_cover():
    for bad in [(96, 4, 4), (128, 0, 4), (128, 6, 4), (128, 4, 0), (128, 4, 5), (128, 5, 4)]:
        with pytest.raises(ValueError):
            tq_v1.TurboQuantSlotConfig(*bad)


def test_eight_bit_lloyd_max_keys_are_not_taken_for_fp8(golden):
    """8 key bits that are NOT FP8 (the reference's boundary layers) are 8-bit Lloyd-Max codes:
    another key_bits value at the C ABI, another slot size."""
    class Cfg:
        head_dim, key_quant_bits, value_quant_bits, norm_correction, key_fp8 = 128, 8, 4, True, False
    assert tq_v1._key_bits(Cfg()) == tq_v1.KEY_BITS_MSE8
    assert tq_v1._key_bits(tq_v1.TurboQuantSlotConfig(128, 8, 4)) == 8
    cfg = tq_v1.TurboQuantSlotConfig(128, 8, 4, key_use_fp8_at_8bit=False)
    assert tq_v1._key_bits(cfg) == tq_v1.KEY_BITS_MSE8
    assert not cfg.key_fp8 and cfg.key_mse_bits == 8 and cfg.n_centroids == 256
    assert cfg.key_packed_size == 130
    g = golden("tq_v1_k8mse.npz")
    for name, d, vb in (("d128_k8mse_v4_nc", 128, 4), ("d64_k8mse_v3", 64, 3), ("d256_k8mse_v2_nc", 256, 2)):
        c = tq_v1.TurboQuantSlotConfig(d, 8, vb, key_use_fp8_at_8bit=False)
        assert int(g[f"{name}_meta"][8]) == c.slot_size_aligned
        assert g[f"{name}_centroids"].shape == (256,) and g[f"{name}_midpoints"].shape == (255,)


def test_midpoints_follow_the_reference_recipe(golden):
    g = golden("tq_v1.npz")
    cent = torch.from_numpy(g["d128_k4v4_centroids"])
    c, m = tq_v1.midpoints_of(cent[torch.randperm(16, generator=torch.Generator().manual_seed(0))])
    np.testing.assert_array_equal(c.numpy(), g["d128_k4v4_centroids"])
    np.testing.assert_array_equal(m.numpy(), g["d128_k4v4_midpoints"])


def test_synthetic_decode_batch_is_causal():
    bt = torch.tensor([[5, 2, 9], [1, 4, 7]], dtype=torch.int32)
    sl = torch.tensor([40, 23], dtype=torch.int32)
    sbt, ssl = synthetic_decode_batch(bt, sl, 3)
    assert sbt.tolist() == [[5, 2, 9]] * 3 + [[1, 4, 7]] * 3
    assert ssl.tolist() == [38, 39, 40, 21, 22, 23] and ssl.dtype == torch.int32


def test_cpu_tensors_are_refused():
    cfg = tq_v1.TurboQuantSlotConfig(128, 4, 4)
    k = torch.zeros(2, 1, 128)
    cache = torch.zeros(1, 16, 1, 134, dtype=torch.uint8)
    with pytest.raises(RuntimeError):
        tq_v1.launch_store(k, k, cache, torch.zeros(2, dtype=torch.int64), torch.linspace(-1, 1, 15), cfg)
    with pytest.raises(RuntimeError):
        tq_v1.decode_attention(k, cache, torch.zeros(2, 1, dtype=torch.int32),
                               torch.ones(2, dtype=torch.int32), torch.linspace(-1, 1, 16), cfg, 0.1)
