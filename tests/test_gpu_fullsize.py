"""Parity at the full sizes of the benchmark configurations, through sampled oracle comparisons and size-independent
properties (determinism, independence of the physical page placement, independence of the
split-KV chunking)."""
import numpy as np
import pytest
import torch

from helpers import contiguous_from_pool, gate

pytestmark = pytest.mark.gpu


def _slots(bt, seq_lens, device):
    return torch.cat([bt[b, torch.arange(int(n), device=device) // 16].long() * 16 +
                      torch.arange(int(n), device=device) % 16 for b, n in enumerate(seq_lens)])


def test_encode_config3_layer_sampled_against_oracle(oracle, tables):
    """One layer of the config-3 prefill (64 x 8192 tokens x 8 heads, bf16, 1% channels x10):
    K encode of 4.2 M vectors; every 997th vector is checked bit for bit against the oracle."""
    from fused_turboquant_b200 import kernels
    d, bits = 128, 4
    signs, bounds = tables[f"signs_d{d}"], tables[f"boundaries_d{d}_b{bits}"]
    g = torch.Generator(device="cuda").manual_seed(3)
    n_tok, Hkv = 64 * 8192, 8
    x = torch.randn(n_tok, Hkv, d, device="cuda", generator=g)
    x = torch.where(torch.rand(Hkv, d, device="cuda", generator=g) < 0.01, x * 10.0, x).bfloat16()
    packed, norms = kernels.fused_encode(x, signs, bounds, bits)
    packed2, norms2 = kernels.fused_encode(x, signs, bounds, bits)
    assert torch.equal(packed, packed2) and torch.equal(norms, norms2)          # deterministic
    idx = torch.arange(0, n_tok * Hkv, 997, device="cuda")
    xs = x.view(-1, d)[idx].float().cpu().numpy()
    rp, rn = oracle.encode(xs, signs, bounds, bits)
    np.testing.assert_array_equal(packed.view(-1, d // 2)[idx].cpu().numpy(), rp)
    np.testing.assert_array_equal(norms.view(-1)[idx].cpu().numpy().view(np.uint16), rn.view(np.uint16))
    # size-independent check: norms of the codes' reconstruction track the input norms
    xn = x.float().norm(dim=-1).view(-1)[idx].cpu().numpy()
    np.testing.assert_allclose(norms.view(-1)[idx].float().cpu().numpy(), xn, rtol=2e-3)


@pytest.mark.parametrize("cfg", ["cfg3", "cfg2", "cfg5"])
def test_decode_full_config_sampled_and_invariants(oracle, tables, cfg):
    """One layer at the full batch/context of a benchmark configuration: sampled sequences against the
    oracle (2e-3 / 1e-3 gate on the fp32 result), bit-identical output under a different
    physical page placement, and agreement under a different split-KV chunking."""
    from fused_turboquant_b200 import PagedKVPool
    dev = torch.device("cuda")
    if cfg == "cfg3":
        B, Hq, Hkv, d, bk, bv = 64, 32, 8, 128, 4, 4
        seq_lens = np.full(B, 8192, np.int32)
    elif cfg == "cfg2":
        B, Hq, Hkv, d, bk, bv = 32, 14, 2, 64, 3, 3
        seq_lens = np.full(B, 4096, np.int32)
    else:
        B, Hq, Hkv, d, bk, bv = 256, 16, 8, 256, 4, 2
        rng = np.random.default_rng(5)
        seq_lens = np.floor(np.exp(rng.uniform(np.log(128), np.log(32768), B))).astype(np.int32)
    max_seq = int(seq_lens.max())
    max_blocks = (max_seq + 15) // 16
    n_blocks = int(((seq_lens + 15) // 16).sum())
    gcpu = torch.Generator("cpu").manual_seed(11)

    def table(perm):
        bt = np.zeros((B, max_blocks), np.int32)
        pos = 0
        for b in range(B):
            nb = (int(seq_lens[b]) + 15) // 16
            bt[b, :nb] = perm[pos:pos + nb]
            pos += nb
        return torch.from_numpy(bt).to(dev)

    perm1 = torch.randperm(n_blocks, generator=gcpu).numpy()
    perm2 = torch.randperm(n_blocks, generator=gcpu).numpy()
    pools, outs = [], []
    q = torch.randn(B, Hq, d, generator=gcpu).bfloat16().to(dev)
    sl = torch.from_numpy(seq_lens).to(dev)
    for perm in (perm1, perm2):
        bt = table(perm)
        pool = PagedKVPool(n_blocks, Hkv, d, bk, bv, n_layers=1, device=dev)
        gdev = torch.Generator(device=dev).manual_seed(77)       # same K/V for both placements
        b0 = 0
        while b0 < B:
            b1 = min(B, b0 + max(1, (1 << 17) // max_seq))
            n = int(seq_lens[b0:b1].sum())
            k = torch.randn(n, Hkv, d, device=dev, generator=gdev).bfloat16()
            v = torch.randn(n, Hkv, d, device=dev, generator=gdev).bfloat16()
            slots = _slots(bt[b0:b1], seq_lens[b0:b1], dev)
            pool.store(k, v, slots, layer=0)
            b0 = b1
        out = pool.decode_attention(q, bt, sl, max_seq, layer=0,
                                    out=torch.empty(B, Hq, d, dtype=torch.float32, device=dev))
        pools.append((pool, bt))
        outs.append(out)
    # physical placement does not matter: same tokens, same order, same arithmetic
    assert torch.equal(outs[0], outs[1])
    # a different chunking (longer max_seq_len hint) changes only the merge order
    pool, bt = pools[0]
    bt_wide = torch.cat([bt, torch.zeros(B, max_blocks, dtype=torch.int32, device=dev)], 1)
    out_c = pool.decode_attention(q, bt_wide, sl, 2 * max_seq, layer=0,
                                  out=torch.empty(B, Hq, d, dtype=torch.float32, device=dev))
    # (fp16 rounding of the softmax weights depends on the running maximum, hence on the chunking;
    # the two results agree far inside the 2e-3 / 1e-3 gate)
    diff = float((out_c - outs[0]).abs().max())
    assert gate(out_c.cpu().numpy(), outs[0].cpu().numpy(), 1e-3, 1e-4) == 0, diff
    # sampled sequences against the oracle (first, last, longest, shortest)
    sample = sorted({0, B - 1, int(seq_lens.argmax()), int(seq_lens.argmin())})
    pool_np = pool.pool[0].cpu().numpy()
    bt_np = bt.cpu().numpy()
    for b in sample:
        S = int(seq_lens[b])
        k_idx, k_n, v_idx, v_n = contiguous_from_pool(pool_np, bt_np[b:b + 1], seq_lens[b:b + 1], S,
                                                      d, bk, bv)
        ref = oracle.decode_attn(q[b:b + 1].float().cpu().numpy(), k_idx, k_n, v_idx, v_n,
                                 tables[f"levels_d{d}_b{bk}"], tables[f"levels_d{d}_b{bv}"],
                                 tables[f"signs_d{d}"], d ** -0.5, bk, bv)
        assert gate(outs[0][b:b + 1].cpu().numpy(), ref) == 0, (cfg, b)
