"""Host logic of the multi-GPU paths, including a world_size-2 gloo run on CPU."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from fused_turboquant_b200 import sharding


def test_equal_sequence_shards_cover_the_batch():
    for batch, world in [(64, 8), (32, 4), (5, 2), (3, 4), (0, 2)]:
        got = [list(sharding.shard_sequences_equal(batch, world, r)) for r in range(world)]
        assert sum(got, []) == list(range(batch))
        assert max(len(g) for g in got) - min(len(g) for g in got) <= 1
    with pytest.raises(ValueError):
        sharding.shard_sequences_equal(8, 2, 2)


def test_lpt_balances_ragged_batches():
    rng = np.random.default_rng(5)
    lens = np.floor(np.exp(rng.uniform(np.log(128), np.log(32768), 256))).astype(int)
    for world in (1, 2, 4, 8):
        owned = sharding.shard_sequences_lpt(lens, world)
        assert sorted(sum(owned, [])) == list(range(256))
        loads = [int(lens[o].sum()) for o in owned]
        assert max(loads) - min(loads) <= lens.max()
        assert max(loads) <= 1.02 * (lens.sum() / world) + lens.max() / world
    assert sharding.shard_sequences_lpt([5, 5, 5], 2) == [[0, 2], [1]]       # deterministic ties


def test_kv_head_shards():
    kv, q = sharding.shard_kv_heads(8, 64, 8, 3)
    assert list(kv) == [3] and list(q) == list(range(24, 32))
    kv, q = sharding.shard_kv_heads(8, 32, 2, 1)
    assert list(kv) == [4, 5, 6, 7] and list(q) == list(range(16, 32))
    with pytest.raises(ValueError):
        sharding.shard_kv_heads(8, 64, 3, 0)
    with pytest.raises(ValueError):
        sharding.shard_kv_heads(8, 60, 2, 0)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        L, B, Hq, D = 2, 3, 8, 16
        full = torch.arange(L * B * Hq * D, dtype=torch.float32).view(L, B, Hq, D)
        _, qr = sharding.shard_kv_heads(4, Hq, world, rank)
        local = full[:, :, qr.start:qr.stop].contiguous()
        out = sharding.all_gather_heads(local)
        ok = torch.equal(out, full)
        # sequence sharding needs no exchange: every rank's slice is independent
        mine = sharding.shard_sequences_equal(7, world, rank)
        t = torch.tensor([float(len(mine))])
        dist.all_reduce(t)
        q.put((rank, bool(ok), float(t.item())))
    finally:
        dist.destroy_process_group()


def test_all_gather_heads_gloo_world2():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=60) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(r[0] for r in res) == [0, 1]
    assert all(r[1] for r in res), "gathered heads are out of order"
    assert all(r[2] == 7.0 for r in res)


def test_all_gather_requires_process_group():
    with pytest.raises(RuntimeError):
        sharding.all_gather_heads(torch.zeros(1, 2, 3))


def _absent_rank_worker(rank, world, port, q, done):
    """Rank 1 joins the group but never enters the collective; rank 0 must get an error, not hang."""
    import datetime
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    # (the rendezvous gets a generous limit -- a loaded machine starts the two interpreters many
    # seconds apart --, the short limit belongs to the group the collective runs on)
    dist.init_process_group("gloo", rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=180))
    short = dist.new_group(ranks=list(range(world)), backend="gloo",
                           timeout=datetime.timedelta(seconds=4))
    if rank == 1:
        done.wait(120)         # stays alive (a crashed peer is a different failure), skips the call
        os._exit(0)
    try:
        sharding.all_gather_heads(torch.zeros(1, 2, 2, 4), group=short)
        q.put("returned")
    except Exception as e:     # gloo reports the timeout as a RuntimeError / DistBackendError
        q.put(f"{type(e).__name__}: {e}"[:300])
    finally:
        done.set()
    os._exit(0)                # (no orderly teardown: the peer never reaches the shutdown barrier)


def test_all_gather_with_an_absent_rank_times_out_cleanly():
    ctx = mp.get_context("spawn")
    q, done = ctx.Queue(), ctx.Event()
    port = _free_port()
    procs = [ctx.Process(target=_absent_rank_worker, args=(r, 2, port, q, done)) for r in range(2)]
    for p in procs:
        p.start()
    msg = q.get(timeout=300)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert msg != "returned", "the collective returned although a rank never joined it"
    assert "Error" in msg or "Timed out" in msg or "timeout" in msg.lower(), msg


def test_mismatched_shard_counts_are_rejected_before_any_collective():
    # 8 KV heads cannot be split over 3 ranks; the host-side check fires on every rank
    for rank in range(3):
        with pytest.raises(ValueError):
            sharding.shard_kv_heads(8, 64, 3, rank)
    with pytest.raises(ValueError):
        sharding.shard_sequences_equal(10, 0, 0)
    with pytest.raises(ValueError):
        sharding.shard_sequences_lpt([1, 2, 3], 0)
