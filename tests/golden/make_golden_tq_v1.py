"""Generates tq_v1.npz: the reference's vLLM-v1 ("TURBOQUANT" slot format) store and decode
kernels, executed on the CPU in Triton's interpreter mode.

    python tests/golden/make_golden_tq_v1.py --reference /path/to/reference

Per case (head_dim, key bits, value bits, norm correction, kv_start) the file holds the inputs
(K, V, q, slot mapping, block table, seq_lens, centroids, midpoints) and what the reference's
kernels wrote for them:

  {case}_cache     kv_cache bytes after `_launch_rht`              (vllm_plugin/triton_inkernel_store.py:554-646)
  {case}_mid_o     `_tq_decode_stage1_offset` partials [B,Hq,S,D+1] (vllm_plugin/triton_decode_offset.py:42-444)
  {case}_out       output of the stock stage-2 merge over them      (call as in vllm_plugin/v1_backend.py:1068-1085)
  {case}_y         the rotated unit key the store kernel bucketises, recomputed with torch ops
                   (used by the tests to tell a genuine code mismatch from a value sitting on a midpoint)
  {case}_kun       (FP8-key cases) the un-normalised rotated key the store kernel casts to e4m3, likewise
  {case}_vy        ("_vlm" cases) the unit value the store kernel bucketises, likewise; {case}_V then
                   holds the pre-rotated values the store kernel was given

The centroid tables come from the installed vLLM (`get_centroids`), as the reference obtains them;
the query rotation `q @ H` follows rotation/matrix.py:47-48.  Needs make_golden.py's environment.
"""
from __future__ import annotations

import argparse
import math
import os
import sys

os.environ["TRITON_INTERPRET"] = "1"

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))

# name, D, Hkv, group, key bits, value bits, norm_correction, seq_lens, kv_start, splits, block_size
CASES = [
    ("d128_k4v4", 128, 2, 4, 4, 4, 0, (70, 33), (0, 0), 4, 16),
    ("d128_k3v4_nc", 128, 2, 2, 3, 4, 1, (50, 64), (0, 0), 3, 16),
    ("d64_k3v3_g7", 64, 2, 7, 3, 3, 1, (45, 17), (0, 5), 4, 16),
    ("d256_k4v2", 256, 1, 2, 4, 2, 0, (37, 40), (0, 0), 2, 16),
    ("d128_k2v8", 128, 1, 4, 2, 8, 0, (21, 1), (3, 0), 2, 8),
    # 1-bit codes (reachable through the reference's bit-width overrides, v1_backend.py:466-491)
    ("d128_k1v1_nc", 128, 2, 4, 1, 1, 1, (40, 19), (0, 0), 3, 16),
    ("d64_k1v3", 64, 2, 2, 1, 3, 0, (30, 9), (0, 2), 2, 16),
    ("d256_k3v1_nc", 256, 1, 2, 3, 1, 1, (21, 18), (0, 0), 2, 8),
    # "_vlm": TURBOQUANT_V_LLOYD_MAX=1 -- values pre-rotated as v1_backend.py:736-740 does, stored
    # as 4-bit Lloyd-Max codes of the key table (3-bit keys: only 8 of the 16 codes occur)
    ("d128_k4v4_nc_vlm", 128, 2, 4, 4, 4, 1, (50, 23), (0, 0), 3, 16),
    ("d64_k4v4_vlm", 64, 2, 2, 4, 4, 0, (33, 12), (0, 4), 2, 16),
    ("d128_k3v4_nc_vlm", 128, 1, 2, 3, 4, 1, (20, 9), (0, 0), 2, 8),
    # key bits 8 = FP8 (e4m3) keys, vLLM's stock key_quant_bits == 8 (the e4nv variant a B200 takes)
    ("d128_k8v4", 128, 2, 4, 8, 4, 0, (45, 18), (0, 0), 3, 16),
    ("d64_k8v2", 64, 2, 2, 8, 2, 0, (27, 11), (0, 3), 2, 16),
    ("d256_k8v3", 256, 1, 2, 8, 3, 0, (19, 8), (0, 0), 2, 8),
]

# `--set k8mse` (written to tq_v1_k8mse.npz, own seed): key bits 8 = 8-bit Lloyd-Max codes, 256
# centroids, one byte per coordinate + the fp16 norm (BoundaryTurboQuantConfig with
# key_use_fp8_at_8bit = False, vllm_plugin/boundary_tq_config.py:26-35; store branch
# triton_inkernel_store.py:132-137)
CASES_K8MSE = [
    ("d128_k8mse_v4_nc", 128, 2, 4, 8, 4, 1, (45, 18), (0, 0), 3, 16),
    ("d64_k8mse_v3", 64, 2, 2, 8, 3, 0, (27, 11), (0, 3), 2, 16),
    ("d256_k8mse_v2_nc", 256, 1, 2, 8, 2, 1, (19, 8), (0, 0), 2, 8),
]


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of the reference repository")
    ap.add_argument("--set", default="main", choices=["main", "k8mse"],
                    help="main: tq_v1.npz; k8mse: the 8-bit Lloyd-Max key cases, tq_v1_k8mse.npz")
    args = ap.parse_args()
    k8mse = args.set == "k8mse"
    sys.path.insert(0, os.path.join(args.reference, "src"))
    from vllm.model_executor.layers.quantization.turboquant.centroids import get_centroids
    from vllm.v1.attention.ops.triton_decode_attention import _fwd_kernel_stage2

    from fused_turboquant.vllm_plugin.boundary_tq_config import BoundaryTurboQuantConfig
    from fused_turboquant.vllm_plugin.rotation.hadamard import _build_hadamard
    from fused_turboquant.vllm_plugin.triton_decode_offset import _tq_decode_stage1_offset
    import fused_turboquant.vllm_plugin.triton_inkernel_store as store_mod
    from fused_turboquant.vllm_plugin.triton_inkernel_store import _launch_rht

    # the e4b15 / e4nv choice asks the CUDA device for its capability: a B200 takes e4nv
    store_mod._use_fp8_e4b15 = lambda device: False

    torch.set_num_threads(1)
    gen = torch.Generator("cpu").manual_seed(20252 if k8mse else 20251)
    out = {}
    for name, D, Hkv, G, kb, vb, nc, seq_lens, kv_start, splits, bs in (CASES_K8MSE if k8mse else CASES):
        cfg = BoundaryTurboQuantConfig(head_dim=D, key_quant_bits=kb, value_quant_bits=vb,
                                       norm_correction=bool(nc), key_use_fp8_at_8bit=not k8mse)
        slot = cfg.key_packed_size + cfg.value_data_bytes + 4
        slot += slot % 2
        B, Hq = len(seq_lens), Hkv * G
        max_blocks = max((s + bs - 1) // bs for s in seq_lens)
        nb = B * max_blocks + 2
        perm = torch.randperm(nb, generator=gen)
        block_table = perm[:B * max_blocks].to(torch.int32).view(B, max_blocks)
        cent, _ = get_centroids(D, cfg.mse_bits).float().sort()   # (FP8 keys: sized for the values, unused)
        mids = (cent[:-1] + cent[1:]) / 2
        H = _build_hadamard(D, "cpu")

        # tokens of all sequences, plus two padding tokens (slot -1) that the store must skip
        K = torch.randn(sum(seq_lens) + 2, Hkv, D, generator=gen)
        V = torch.randn(sum(seq_lens) + 2, Hkv, D, generator=gen) * 1.5 + 0.25
        K[:, :, :3] *= 12.0
        V[5] = 0.75                       # a constant vector: scale clamps to 1e-8
        slots, pos = [], 0
        for b, s in enumerate(seq_lens):
            for t in range(s):
                slots.append(int(block_table[b, t // bs]) * bs + t % bs)
            pos += s
        slot_mapping = torch.tensor(slots[:7] + [-1] + slots[7:] + [-1], dtype=torch.int64)
        # rows 7 and the last one are the padding tokens: move K/V rows accordingly
        order = list(range(7)) + [len(slots)] + list(range(7, len(slots))) + [len(slots) + 1]
        K, V = K[order].contiguous(), V[order].contiguous()
        vlm = name.endswith("_vlm")
        if vlm:
            V = torch.einsum("nhd,de->nhe", V.float(), H).to(V.dtype).contiguous()
            vf = V.reshape(-1, D)
            vnorm = torch.sqrt((vf * vf).sum(-1, keepdim=True) + 1e-16)
            out[f"{name}_vy"] = (vf / (vnorm + 1e-8)).reshape(V.shape).numpy()
        os.environ["TURBOQUANT_V_LLOYD_MAX"] = "1" if vlm else "0"

        cache = torch.zeros(nb, bs, Hkv, slot, dtype=torch.uint8)
        _launch_rht(K, V, cache, slot_mapping, mids, cfg, D)

        q = torch.randn(B, Hq, D, generator=gen)
        q_rot = (q.float() @ H).contiguous()
        sl = torch.tensor(seq_lens, dtype=torch.int32)
        ks = torch.tensor(kv_start, dtype=torch.int32)
        mid_o = torch.zeros(B, Hq, splits, D + 1)
        scale = 1.0 / math.sqrt(D)
        BLOCK_D = 1 << (D - 1).bit_length()
        _tq_decode_stage1_offset[(B, Hq, splits)](
            q_rot, cache, block_table, sl, ks, cent, mid_o,
            q_rot.stride(0), q_rot.stride(1), cache.stride(0), cache.stride(1), cache.stride(2),
            block_table.stride(0), mid_o.stride(0), mid_o.stride(1), mid_o.stride(2),
            NUM_KV_HEADS=Hkv, HEAD_DIM=D, BLOCK_SIZE=bs, NUM_KV_SPLITS=splits, KV_GROUP_SIZE=G,
            # (the reference's call sites pass max(key_mse_bits, 2), v1_backend.py:1052 -- meant for
            # FP8 keys, whose key_mse_bits is 0, but it also turns 1 into 2, so that with 1-bit keys
            # its decode would read the store kernel's 1-bit codes as 2-bit ones; the 1-bit fixtures
            # are made with the kernel's own meaning of MSE_BITS = 1)
            MSE_BITS=2 if cfg.key_fp8 else kb, MSE_BYTES=0 if cfg.key_fp8 else cfg.key_packed_size - 2,
            KPS=cfg.key_packed_size, VQB=vb,
            VAL_DATA_BYTES=cfg.value_data_bytes, ATTN_SCALE=scale, BLOCK_D=BLOCK_D, BLOCK_KV=4,
            KEY_FP8=int(cfg.key_fp8), NORM_CORRECTION=nc, FP8_E4B15=0, V_LLOYD_MAX=int(vlm), num_warps=1, num_stages=1)
        o = torch.zeros(B, Hq, D)
        lse = torch.zeros(B, Hq)
        # the stock merge decides which splits exist from seq_lens alone; the reference only
        # calls it this way with kv_start = 0, so cases with an offset merge in the test instead
        if not any(kv_start):
            _fwd_kernel_stage2[(B, Hq)](
                mid_o, o, lse, sl, mid_o.stride(0), mid_o.stride(1), mid_o.stride(2),
                o.stride(0), o.stride(1), lse.stride(0),
                NUM_KV_SPLITS=splits, BLOCK_DV=BLOCK_D, Lv=D, num_warps=4, num_stages=2)
            out[f"{name}_out"] = o.numpy()
            out[f"{name}_lse"] = lse.numpy()

        kf = K.float().reshape(-1, D)
        norm = torch.sqrt((kf * kf).sum(-1, keepdim=True) + 1e-16)
        out[f"{name}_y"] = ((kf / (norm + 1e-8)) @ H).reshape(K.shape).numpy()
        if cfg.key_fp8:   # what the store kernel casts to FP8, recomputed with torch ops
            out[f"{name}_kun"] = (((kf / (norm + 1e-8)) @ H) * norm).reshape(K.shape).numpy()
        for k_, v_ in (("K", K), ("V", V), ("q", q), ("slot_mapping", slot_mapping),
                       ("block_table", block_table), ("seq_lens", sl), ("kv_start", ks),
                       ("centroids", cent), ("midpoints", mids), ("cache", cache),
                       ("mid_o", mid_o)):
            out[f"{name}_{k_}"] = v_.numpy()
        out[f"{name}_meta"] = np.array([D, Hkv, G, kb, vb, nc, splits, bs, slot, nb], np.int32)
        print(name, "slot", slot, flush=True)

    path = os.path.join(HERE, "tq_v1_k8mse.npz" if k8mse else "tq_v1.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path))


if __name__ == "__main__":
    main()
