"""Device-side guards of the paged kernels: block ids and slots outside the cache.

The guards are exercised without ever producing an out-of-bounds address: the pool is allocated
with N blocks, the kernels are told it has N - 8, and the "bad" ids / slots lie in between, so a
missing guard would still touch allocated memory only (and show up as a wrong result).
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _filled_pool(d, bk, bv, Hkv, seq_lens, seed=0, extra_blocks=8):
    from fused_turboquant_b200 import PagedKVPool
    B = len(seq_lens)
    max_blocks = (max(seq_lens) + 15) // 16
    used = B * max_blocks
    pool = PagedKVPool(used + extra_blocks, Hkv, d, bk, bv, n_layers=1, device="cuda")
    rng = np.random.default_rng(seed)
    bt = rng.permutation(used).reshape(B, max_blocks).astype(np.int32)
    g = torch.Generator("cpu").manual_seed(seed)
    n_tok = int(sum(seq_lens))
    key = torch.randn(n_tok, Hkv, d, generator=g).bfloat16().cuda()
    val = torch.randn(n_tok, Hkv, d, generator=g).bfloat16().cuda()
    slots = np.array([int(bt[b, s // 16]) * 16 + s % 16 for b in range(B) for s in range(seq_lens[b])],
                     np.int64)
    pool.store(key, val, torch.from_numpy(slots).cuda(), layer=0)
    return pool, bt, key, val, slots, used


@pytest.mark.parametrize("d,G,bk,bv,qdtype", [
    (128, 4, 4, 4, torch.bfloat16),   # streaming tensor-core kernel
    (128, 8, 3, 3, torch.bfloat16),   # barrier-synchronised tensor-core kernel, two head halves
    (256, 2, 4, 2, torch.bfloat16),   # ... head_dim 256
    (128, 4, 4, 4, torch.float32),    # fp32 CUDA-core kernel
])
def test_block_id_outside_the_pool_poisons_only_its_sequence(d, G, bk, bv, qdtype):
    Hkv, seq_lens = 2, [700, 1300, 90]
    pool, bt, *_ , used = _filled_pool(d, bk, bv, Hkv, seq_lens)
    g = torch.Generator("cpu").manual_seed(5)
    q = torch.randn(len(seq_lens), Hkv * G, d, generator=g).to(qdtype).cuda()
    sl = torch.tensor(seq_lens, dtype=torch.int32).cuda()

    def run(table):
        out = torch.empty(q.shape, dtype=torch.float32, device="cuda")
        pool.decode_attention(q, torch.from_numpy(table).cuda(), sl, max(seq_lens), layer=0, out=out)
        torch.cuda.synchronize()
        return out.cpu().numpy()

    good = run(bt)
    assert np.isfinite(good).all()
    assert pool.decode_status() == 0
    # the kernels are told the pool ends 8 blocks early; sequence 1 names a block in that tail
    # (allocated, zero-filled, never written), everything else stays below the limit
    pool.num_blocks = used
    bad_bt = bt.copy()
    bad_bt[1, 3] = used + 2
    got = run(bad_bt)
    assert np.isnan(got[1]).all(), "a sequence with an out-of-range block id must come back as NaN"
    np.testing.assert_array_equal(got[0], good[0])
    np.testing.assert_array_equal(got[2], good[2])
    # ... and the call's status word says so (the next clean call clears it)
    assert pool.decode_status() == 1
    run(bt)
    assert pool.decode_status() == 0
    # negative ids are out of range too
    bad_bt[1, 3] = -1
    got = run(bad_bt)
    assert np.isnan(got[1]).all()
    np.testing.assert_array_equal(got[0], good[0])


def test_slot_outside_the_pool_is_skipped_by_the_store():
    d, bk, bv, Hkv = 128, 4, 3, 2
    pool, bt, key, val, slots, used = _filled_pool(d, bk, bv, Hkv, [40, 33])
    before = pool.pool.clone()
    pool.num_blocks = used               # the tail of 8 blocks is "outside" for the kernel
    pool.pool.zero_()
    bad = slots.copy()
    bad[5] = used * 16 + 3               # lands in the allocated tail if the guard were missing
    bad[17] = (used + 7) * 16 + 15
    pool.store(key, val, torch.from_numpy(bad).cuda(), layer=0)
    torch.cuda.synchronize()
    after = pool.pool.cpu().numpy()
    assert (after[0, used:] == 0).all(), "the store wrote beyond the block count it was given"
    # every other token landed where the unguarded run put it; the two dropped slots stay zero
    ref = before.cpu().numpy().copy()
    page = ref.shape[-1]
    from helpers import page_offsets, pd
    off_kn, off_vc, off_vn, _ = page_offsets(d, bk, bv)
    for tok in (5, 17):
        blk, t = int(slots[tok]) // 16, int(slots[tok]) % 16
        for h in range(Hkv):
            ref[0, blk, h, t * pd(d, bk):(t + 1) * pd(d, bk)] = 0
            ref[0, blk, h, off_kn + 2 * t:off_kn + 2 * t + 2] = 0
            ref[0, blk, h, off_vc + t * pd(d, bv):off_vc + (t + 1) * pd(d, bv)] = 0
            ref[0, blk, h, off_vn + 2 * t:off_vn + 2 * t + 2] = 0
    np.testing.assert_array_equal(after[0, :used], ref[0, :used])
    assert page == ref.shape[-1]


def test_gather_sequence_matches_the_host_restatement_of_the_layout():
    from helpers import contiguous_from_pool
    d, bk, bv, Hkv = 64, 3, 3, 2
    pool, bt, *_ = _filled_pool(d, bk, bv, Hkv, [50, 17])
    pool_np = pool.pool[0].cpu().numpy()
    for b, S in enumerate([50, 17]):
        kc, kn, vc, vn = pool.gather_sequence(0, torch.from_numpy(bt[b]).cuda(), S)
        rk, rkn, rv, rvn = contiguous_from_pool(pool_np, bt[b:b + 1], np.array([S]), S, d, bk, bv)
        np.testing.assert_array_equal(kc.cpu().numpy(), rk[0])
        np.testing.assert_array_equal(vc.cpu().numpy(), rv[0])
        np.testing.assert_array_equal(kn.cpu().numpy().view(np.uint16), rkn[0].view(np.uint16))
        np.testing.assert_array_equal(vn.cpu().numpy().view(np.uint16), rvn[0].view(np.uint16))


@pytest.mark.parametrize("d,G,bk,bv", [(128, 4, 4, 4), (128, 2, 4, 3), (64, 4, 4, 4)])
def test_many_short_items_per_cta(oracle, tables, d, G, bk, bv):
    """Hundreds of one- and two-page sequences (plus empty ones and a few long ones): every CTA of
    the streaming kernel runs many items in which most warps have no page at all, which is the
    path where a warp runs ahead of its published state and has to hand page requests back.
    All outputs against the oracle; two runs bit-identical."""
    from fused_turboquant_b200 import PagedKVPool
    rng = np.random.default_rng(d + bk + bv)
    B, Hkv = 700, 2
    seq_lens = rng.integers(1, 40, B).astype(np.int32)
    seq_lens[rng.integers(0, B, 25)] = 0
    seq_lens[[3, 77, 410]] = [1000, 555, 2049]
    max_seq = int(seq_lens.max())
    max_blocks = (max_seq + 15) // 16
    nblk = int(((seq_lens + 15) // 16).sum())
    perm = rng.permutation(nblk).astype(np.int32)
    bt = np.zeros((B, max_blocks), np.int32)
    pos = 0
    for b in range(B):
        nb = (int(seq_lens[b]) + 15) // 16
        bt[b, :nb] = perm[pos:pos + nb]
        pos += nb
    n_tok = int(seq_lens.sum())
    g = torch.Generator("cpu").manual_seed(1)
    key = torch.randn(n_tok, Hkv, d, generator=g).bfloat16()
    val = torch.randn(n_tok, Hkv, d, generator=g).bfloat16()
    q = torch.randn(B, Hkv * G, d, generator=g).bfloat16()
    slots = np.concatenate([bt[b, np.arange(seq_lens[b]) // 16].astype(np.int64) * 16 +
                            np.arange(seq_lens[b]) % 16 for b in range(B)])
    pool = PagedKVPool(nblk, Hkv, d, bk, bv, n_layers=1, device="cuda")
    pool.store(key.cuda(), val.cuda(), torch.from_numpy(slots).cuda(), layer=0)
    bt_d, sl_d = torch.from_numpy(bt).cuda(), torch.from_numpy(seq_lens).cuda()
    outs = [pool.decode_attention(q.cuda(), bt_d, sl_d, max_seq, layer=0,
                                  out=torch.empty(q.shape, dtype=torch.float32, device="cuda"))
            for _ in range(2)]
    torch.cuda.synchronize()
    assert torch.equal(outs[0], outs[1])
    got = outs[0].cpu().numpy()
    assert np.isfinite(got).all()
    assert (got[seq_lens == 0] == 0).all()                      # softmax over nothing
    ek, enk = oracle.encode(key.float().numpy(), pool.signs, pool.bounds_k, bk)
    ev, env = oracle.encode(val.float().numpy(), pool.signs, pool.bounds_v, bv)
    starts = np.concatenate([[0], np.cumsum(seq_lens)])
    bad = 0
    for b in list(range(0, B, 9)) + [3, 77, 410]:
        S = int(seq_lens[b])
        if S == 0:
            continue
        sl = slice(starts[b], starts[b] + S)
        tr = lambda a: np.ascontiguousarray(np.swapaxes(a[sl], 0, 1))[None]
        ref = oracle.decode_attn(q[b:b + 1].float().numpy(), tr(ek), tr(enk), tr(ev), tr(env),
                                 pool.levels_k, pool.levels_v, pool.signs, d ** -0.5, bk, bv)
        bad += int((np.abs(got[b:b + 1] - ref) > 1e-3 + 2e-3 * np.abs(ref)).sum())
    assert bad == 0
