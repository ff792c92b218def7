"""Multi-GPU partitioning of the decode path (one process per GPU).

The hot path shards without any data-path exchange along two axes:

  * sequences  -- every rank owns whole sequences (its own page pool and block
                  table); no collective at all.  Ragged batches are balanced by
                  token count (longest-processing-time first).
  * KV heads   -- rank r owns KV heads [r*Hkv/G, (r+1)*Hkv/G) and the query
                  heads of those groups; the softmax never crosses a KV head,
                  so the only exchange is one all-gather of the attention
                  output along the head axis.

The reference has no collective of its own (multi-GPU is vLLM's tensor
parallelism, which hands each rank its local heads:
src/fused_turboquant/vllm_plugin/v1_backend.py:292-315); this module is the
stand-alone equivalent for the benchmark and for callers outside vLLM.
"""
from __future__ import annotations

from typing import Sequence

import torch
import torch.distributed as dist

from . import _trace

logger = _trace.get_logger(__name__)


def shard_sequences_equal(batch: int, world_size: int, rank: int) -> range:
    """Contiguous, near-equal split of `batch` sequences."""
    if world_size <= 0 or not (0 <= rank < world_size):
        raise ValueError(f"bad rank {rank} / world_size {world_size}")
    base, rem = divmod(batch, world_size)
    start = rank * base + min(rank, rem)
    return range(start, start + base + (1 if rank < rem else 0))


def shard_sequences_lpt(seq_lens: Sequence[int], world_size: int) -> list[list[int]]:
    """Longest-processing-time-first assignment of sequences to ranks by token count.

    Returns, for every rank, the (sorted) list of sequence indices it owns.
    Deterministic: ties go to the lowest rank / lowest index.
    """
    if world_size <= 0:
        raise ValueError("world_size must be positive")
    order = sorted(range(len(seq_lens)), key=lambda i: (-int(seq_lens[i]), i))
    loads = [0] * world_size
    owned: list[list[int]] = [[] for _ in range(world_size)]
    for i in order:
        r = min(range(world_size), key=lambda k: (loads[k], k))
        owned[r].append(i)
        loads[r] += int(seq_lens[i])
    return [sorted(o) for o in owned]


def shard_kv_heads(num_kv_heads: int, num_q_heads: int, world_size: int,
                   rank: int) -> tuple[range, range]:
    """(kv head range, query head range) of `rank` under head sharding."""
    if num_kv_heads % world_size:
        raise ValueError(
            f"num_kv_heads={num_kv_heads} is not divisible by world_size={world_size}")
    if num_q_heads % num_kv_heads:
        raise ValueError("num_q_heads must be a multiple of num_kv_heads")
    per = num_kv_heads // world_size
    group = num_q_heads // num_kv_heads
    kv = range(rank * per, (rank + 1) * per)
    return kv, range(kv.start * group, kv.stop * group)


def all_gather_heads(out_local: torch.Tensor, group=None) -> torch.Tensor:
    """All-gather attention outputs along the head axis.

    out_local: [..., B, Hq_local, D] -> [..., B, Hq_local * world_size, D], rank-major
    in the head axis (the order shard_kv_heads assigns).  One collective
    (NCCL over NVLink on GPUs, gloo on CPU tensors).
    """
    if not dist.is_initialized():
        raise RuntimeError("torch.distributed is not initialised")
    world = dist.get_world_size(group)
    if world == 1:
        return out_local
    local = out_local.contiguous()
    flat = torch.empty((world * local.shape[0],) + tuple(local.shape[1:]), dtype=local.dtype,
                       device=local.device)
    with _trace.nvtx("ftq.all_gather"):
        dist.all_gather_into_tensor(flat, local, group=group)
    gathered = flat.view((world,) + tuple(local.shape))
    # [world, ..., B, Hl, D] -> [..., B, world, Hl, D] -> merge
    nd = local.dim()
    perm = list(range(1, nd - 1)) + [0, nd - 1, nd]
    g = gathered.permute(*perm)
    shape = list(local.shape)
    shape[-2] = shape[-2] * world
    return g.reshape(shape)
