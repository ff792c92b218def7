"""Two-GPU check of KV-head sharding: every rank runs the paged decode on its own KV heads,
one NCCL all-gather assembles the output, which must equal the unsharded result bit for bit.
Skipped on boxes with fewer than two GPUs."""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _case():
    g = torch.Generator("cpu").manual_seed(21)
    B, Hkv, G, d, S = 3, 4, 4, 128, 150
    max_blocks = (S + 15) // 16
    bt = torch.randperm(B * max_blocks, generator=g).view(B, max_blocks).to(torch.int32)
    seq_lens = torch.tensor([S, 37, 96], dtype=torch.int32)
    n_tok = int(seq_lens.sum())
    key = torch.randn(n_tok, Hkv, d, generator=g).bfloat16()
    val = torch.randn(n_tok, Hkv, d, generator=g).bfloat16()
    q = torch.randn(B, Hkv * G, d, generator=g).bfloat16()
    slots = torch.cat([bt[b, torch.arange(int(n)) // 16].long() * 16 + torch.arange(int(n)) % 16
                       for b, n in enumerate(seq_lens)])
    return B, Hkv, G, d, S, bt, seq_lens, key, val, q, slots


def _run(pool_heads, kv_range, q_range, dev):
    from fused_turboquant_b200 import PagedKVPool
    B, Hkv, G, d, S, bt, seq_lens, key, val, q, slots = _case()
    pool = PagedKVPool(bt.numel(), pool_heads, d, 4, 3, device=dev)
    pool.store(key[:, kv_range].contiguous().to(dev), val[:, kv_range].contiguous().to(dev),
               slots.to(dev), layer=0)
    return pool.decode_attention(q[:, q_range].contiguous().to(dev), bt.to(dev), seq_lens.to(dev),
                                 S, layer=0)


def _worker(rank, world, port, ret):
    import torch.distributed as dist
    from fused_turboquant_b200 import sharding
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        B, Hkv, G = _case()[:3]
        kvr, qr = sharding.shard_kv_heads(Hkv, Hkv * G, world, rank)
        local = _run(len(kvr), slice(kvr.start, kvr.stop), slice(qr.start, qr.stop), dev)
        full = sharding.all_gather_heads(local)
        torch.cuda.synchronize()
        if rank == 0:
            ref = _run(Hkv, slice(0, Hkv), slice(0, Hkv * G), dev)
            ret.put(bool(torch.equal(full, ref)))
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_head_sharded_decode_matches_unsharded():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    ret = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, ret)) for r in range(2)]
    for p in procs:
        p.start()
    ok = ret.get(timeout=180)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert ok, "gathered head-sharded output differs from the unsharded one"
