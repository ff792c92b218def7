"""Times the vLLM-v1 slot-format path (fused store, split-KV decode) on one GPU.

    python -m fused_turboquant_b200.bench_tq_v1 [--shape qwen|llama] [--steps K] [--warmup W]

Synthetic data, one JSON line.  Shapes: ``qwen`` = 14 query / 2 KV heads, head_dim 64, 3-bit keys,
3-bit values, value rotation on, batch 32 x context 4096, 24 layer caches; ``llama`` = 32 / 8 heads,
head_dim 128, 4-bit keys and values, batch 64 x context 8192, 4 layer caches (each larger than L2);
``llama_k8v4`` = the same with FP8 keys.
Bytes counted: the slot bytes actually used (codes, norm, scale, zero; padding excluded) of every
attended (token, KV head), once per KV head, plus block ids, queries and outputs.
"""
from __future__ import annotations

import argparse
import json

import torch

from . import tq_v1

SHAPES = {
    "qwen": dict(Hq=14, Hkv=2, D=64, kb=3, vb=3, B=32, ctx=4096, layers=24, v_rotate=True),
    "llama": dict(Hq=32, Hkv=8, D=128, kb=4, vb=4, B=64, ctx=8192, layers=4, v_rotate=False),
    # vLLM's stock k8v4 preset: FP8 keys (fp32 kernel)
    "llama_k8v4": dict(Hq=32, Hkv=8, D=128, kb=8, vb=4, B=64, ctx=8192, layers=4, v_rotate=False),
}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--shape", default="llama", choices=sorted(SHAPES))
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--splits", type=int, default=0)
    args = ap.parse_args()
    w = SHAPES[args.shape]
    Hq, Hkv, D, kb, vb, B, ctx, L = (w[k] for k in ("Hq", "Hkv", "D", "kb", "vb", "B", "ctx", "layers"))
    dev = torch.device("cuda:0")
    gen = torch.Generator(device=dev).manual_seed(20252)
    cfg = tq_v1.TurboQuantSlotConfig(D, kb, vb, norm_correction=True)
    slot, bs = cfg.slot_size_aligned, 16
    blocks_per_seq = ctx // bs
    nb = B * blocks_per_seq
    cent = torch.sort(torch.randn(1 << min(kb, 4), generator=gen, device=dev) / D ** 0.5).values  # (FP8 keys: unused)
    cent, mids = tq_v1.midpoints_of(cent)
    caches, tables = [], []
    n_tok = B * ctx
    store_ms = []
    for layer in range(L):
        cache = torch.zeros((nb, bs, Hkv, slot), dtype=torch.uint8, device=dev)
        perm = torch.randperm(nb, generator=gen, device=dev)
        bt = perm.view(B, blocks_per_seq).to(torch.int32)
        pos = torch.arange(ctx, device=dev)
        slots = (bt.long()[:, pos // bs] * bs + pos % bs).reshape(-1)
        k = torch.randn((n_tok, Hkv, D), generator=gen, device=dev).bfloat16()
        v = torch.randn((n_tok, Hkv, D), generator=gen, device=dev).bfloat16()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        tq_v1.launch_store(k, v, cache, slots, mids, cfg, v_rotate=w["v_rotate"])
        e1.record()
        torch.cuda.synchronize()
        store_ms.append(e0.elapsed_time(e1))
        caches.append(cache)
        tables.append(bt)
        del k, v
    seq_lens = torch.full((B,), ctx, dtype=torch.int32, device=dev)
    q = torch.randn((L, B, Hq, D), generator=gen, device=dev).bfloat16()
    # smallest split count whose (sequence, KV head, split) items fill whole waves of the
    # persistent CTAs to >= 95 % (one CTA per SM with a 4-bit table, else two)
    slots = torch.cuda.get_device_properties(dev).multi_processor_count * (1 if 4 in (kb, vb) else 2)
    splits = args.splits
    if not splits:
        best = (0.0, 1)
        for s in range(1, 33):
            items = B * Hkv * s
            eff = items / (-(-items // slots) * slots)
            if eff > best[0] + 1e-9:
                best = (eff, s)
            if eff >= 0.95:
                break
        splits = best[1]
    mid_o = torch.empty((B, Hq, splits, D + 1), dtype=torch.float32, device=dev)
    out = torch.empty((B, Hq, D), dtype=torch.bfloat16, device=dev)

    def step():
        for layer in range(L):
            tq_v1.decode_attention(q[layer], caches[layer], tables[layer], seq_lens, cent, cfg,
                                   D ** -0.5, num_kv_splits=splits, v_rotate=w["v_rotate"],
                                   mid_o=mid_o, output=out)

    for _ in range(max(3, args.warmup)):
        step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    used = cfg.slot_size
    step_bytes = L * (B * ctx * Hkv * used + B * blocks_per_seq * 4 + 2 * B * Hq * D * 2)
    store_bytes = n_tok * Hkv * (2 * D * 2 + used)
    best_store = min(store_ms[1:]) if L > 1 else store_ms[0]
    print(json.dumps({
        "metric": "tq_v1_decode_attn_hbm_gbs", "value": step_bytes / ms / 1e6, "unit": "GB/s",
        "n_gpus": 1, "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.shape, **w, "splits": splits, "slot_bytes": slot,
                   "l2": "distinct layer caches, each step reads all of them"},
        "store": {"tokens_per_s": n_tok / best_store * 1e3, "ms": best_store,
                  "gbs": store_bytes / best_store / 1e6},
    }))


if __name__ == "__main__":
    main()
