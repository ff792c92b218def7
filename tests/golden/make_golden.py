"""Generates the golden fixtures in this directory by running the REFERENCE itself.

    python tests/golden/make_golden.py --reference /path/to/reference

Needs the reference checkout (imported from <reference>/src, CPU only); the
fixtures it writes are what travels: tests never import the reference.  Every
fixture stores the exact inputs next to the reference's outputs.

  tables.npz         generate_rht_signs(seed=42) and LloydMaxQuantizer tables for D x bits
  encode.npz         TurboQuantMSE._encode_unfused on fp32 and bf16-valued inputs (incl. edge rows)
  decode_dense.npz   TurboQuantMSE._decode_unfused of those codes
  attention.npz      composed unfused decode attention (decode K -> q.K^T*scale -> fp32 softmax ->
                     _fused_v_attention_fallback), with and without seq_lens masking, and the
                     rotated-space score formula of fused_qk_scores_rht evaluated with torch ops
  v0_layout.npz      write_compressed_to_slot / gather_compressed_kv_batched on a small paged cache
  fwht_kat.npz       the reference test-suite's known answers for fwht
"""
from __future__ import annotations

import argparse
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
DIMS = (64, 128, 256)
BITS = (2, 3, 4)


def edge_rows(d: int, gen: torch.Generator) -> torch.Tensor:
    """Rows that stress the arithmetic: zeros, one-hot, constants, outliers, tiny and huge scales."""
    rows = [torch.zeros(d), torch.ones(d), -torch.ones(d)]
    e = torch.zeros(d); e[3] = 1.0; rows.append(e)
    e = torch.zeros(d); e[d - 1] = -2.5; rows.append(e)
    r = torch.randn(d, generator=gen); r[:4] *= 20.0; rows.append(r)
    rows.append(torch.randn(d, generator=gen) * 1e-6)
    rows.append(torch.randn(d, generator=gen) * 1e4)
    rows.append(torch.randn(d, generator=gen) * 1e-30)
    alt = torch.ones(d); alt[1::2] = -1.0; rows.append(alt)
    return torch.stack(rows)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of the reference repository")
    args = ap.parse_args()
    sys.path.insert(0, os.path.join(args.reference, "src"))
    from fused_turboquant.core.hadamard import fwht, generate_rht_signs, randomized_hadamard
    from fused_turboquant.core.quantizer import CompressedTensor, TurboQuantMSE
    from fused_turboquant.kernels.triton_v_attention import _fused_v_attention_fallback
    from fused_turboquant.vllm_plugin.cache_ops import (
        compute_compressed_elem_size, gather_compressed_kv_batched, write_compressed_to_slot)

    torch.set_num_threads(1)
    gen = torch.Generator("cpu").manual_seed(20250)

    # ---- tables
    tables = {}
    tqs = {}
    for d in DIMS:
        tables[f"signs_d{d}"] = generate_rht_signs(d, seed=42).numpy()
        for b in BITS:
            tq = TurboQuantMSE(d, b, seed=42, device="cpu")
            tqs[(d, b)] = tq
            tables[f"boundaries_d{d}_b{b}"] = tq.quantizer.boundaries.numpy()
            tables[f"levels_d{d}_b{b}"] = tq.quantizer.levels.numpy()
    np.savez_compressed(os.path.join(HERE, "tables.npz"), **tables)

    # ---- fwht known answers (tests/test_hadamard.py:35-40 of the reference) + a random case
    kat = {"x2": np.array([1.0, 0.0], np.float32)}
    kat["y2"] = fwht(torch.tensor([1.0, 0.0])).numpy()
    for d in DIMS:
        x = torch.randn(5, d, generator=gen)
        kat[f"x_d{d}"] = x.numpy()
        kat[f"fwht_d{d}"] = fwht(x).numpy()
        kat[f"rht_d{d}"] = randomized_hadamard(x, generate_rht_signs(d, seed=42)).numpy()
    np.savez_compressed(os.path.join(HERE, "fwht_kat.npz"), **kat)

    # ---- encode / dense decode
    enc, dec = {}, {}
    for d in DIMS:
        x32 = torch.cat([torch.randn(38, d, generator=gen), edge_rows(d, gen)])
        xbf = torch.cat([torch.randn(38, d, generator=gen), edge_rows(d, gen)]).bfloat16()
        enc[f"x32_d{d}"] = x32.numpy()
        enc[f"xbf_d{d}"] = xbf.view(torch.int16).numpy().view(np.uint16)  # bf16 bit patterns
        for b in BITS:
            tq = tqs[(d, b)]
            for tag, x in (("x32", x32), ("xbf", xbf)):
                ct = tq._encode_unfused(x)
                enc[f"{tag}_d{d}_b{b}_packed"] = ct.indices.numpy()
                enc[f"{tag}_d{d}_b{b}_norms"] = ct.norms.numpy()
                if tag == "x32":
                    dec[f"d{d}_b{b}"] = tq._decode_unfused(ct).numpy()
    np.savez_compressed(os.path.join(HERE, "encode.npz"), **enc)
    np.savez_compressed(os.path.join(HERE, "decode_dense.npz"), **dec)

    # ---- composed decode attention (a reduced round-trip configuration and two mixed-bit cases)
    att = {}
    cases = [  # name, B, Hkv, group, S, D, bits_k, bits_v, outliers
        ("cfg1small", 1, 2, 4, 96, 128, 4, 4, True),
        ("d64_g7_k3v3", 2, 2, 7, 50, 64, 3, 3, False),
        ("d256_g2_k4v2", 2, 2, 2, 37, 256, 4, 2, False),
    ]
    for name, B, Hkv, G, S, d, bk, bv, outl in cases:
        K = torch.randn(B, Hkv, S, d, generator=gen)
        V = torch.randn(B, Hkv, S, d, generator=gen)
        if outl:
            for h in range(Hkv):
                ch = torch.randperm(d, generator=gen)[:4]
                K[:, h, :, ch] *= 20.0
                V[:, h, :, ch] *= 20.0
        q = torch.randn(B, Hkv * G, 1, d, generator=gen)
        scale = d ** -0.5
        tqk, tqv = tqs[(d, bk)], tqs[(d, bv)]
        ck, cv = tqk._encode_unfused(K), tqv._encode_unfused(V)
        Kd = tqk._decode_unfused(ck)
        Kr = Kd[:, :, None].expand(B, Hkv, G, S, d).reshape(B, Hkv * G, S, d)
        scores = torch.matmul(q, Kr.transpose(-1, -2)) * scale
        seq_lens = torch.tensor([S - 7 * i - 1 for i in range(B)], dtype=torch.int32)
        signs = tqk.rotation.signs
        for tag, sc in (("full", scores), ("masked", scores.clone())):
            if tag == "masked":
                for i in range(B):
                    sc[i, :, :, seq_lens[i]:] = float("-inf")
            w = torch.softmax(sc, dim=-1, dtype=torch.float32)
            out = _fused_v_attention_fallback(w, cv.indices, cv.norms, tqv.quantizer.levels, signs,
                                              d, bv, G)
            att[f"{name}_out_{tag}"] = out.numpy()
        # rotated-space score formula of the fused kernel, evaluated with torch ops
        q_rot = randomized_hadamard(q.float(), signs)
        from fused_turboquant.core.packing import unpack_2bit, unpack_3bit, unpack_nibbles
        unpack = {4: unpack_nibbles, 3: unpack_3bit, 2: unpack_2bit}[bk]
        cent = tqk.quantizer.levels[unpack(ck.indices, d).long()]          # [B,Hkv,S,d]
        centr = cent[:, :, None].expand(B, Hkv, G, S, d).reshape(B, Hkv * G, S, d)
        nr = ck.norms.float()[:, :, None].expand(B, Hkv, G, S).reshape(B, Hkv * G, S)
        att[f"{name}_scores_rot"] = (torch.einsum("bhqd,bhsd->bhqs", q_rot, centr) *
                                     nr[:, :, None, :] * scale).numpy()
        att[f"{name}_q_rot"] = q_rot.numpy()
        for k_, v_ in (("K", K), ("V", V), ("q", q), ("seq_lens", seq_lens),
                       ("k_idx", ck.indices), ("k_norms", ck.norms), ("v_idx", cv.indices),
                       ("v_norms", cv.norms), ("scores", scores)):
            att[f"{name}_{k_}"] = v_.numpy()
        att[f"{name}_meta"] = np.array([B, Hkv, G, S, d, bk, bv], np.int32)
    np.savez_compressed(os.path.join(HERE, "attention.npz"), **att)

    # ---- reference v0 paged layout
    v0 = {}
    d, b, Hkv, bs, nb = 128, 4, 2, 16, 6
    tq = tqs[(d, b)]
    es = compute_compressed_elem_size(d, b)
    n_tok = 40
    K = torch.randn(n_tok, Hkv, d, generator=gen)
    ck = tq._encode_unfused(K)
    perm = torch.randperm(nb, generator=gen)
    slots = torch.tensor([int(perm[t // bs]) * bs + t % bs for t in range(n_tok)])
    cache = torch.zeros(2, nb, bs, Hkv, es, dtype=torch.uint8)
    for t in range(n_tok):
        write_compressed_to_slot(cache, ck.indices[t], ck.norms[t], int(slots[t]), 0)
    bt = perm[:3].to(torch.int32).view(1, 3)
    gp, gn = gather_compressed_kv_batched(cache, bt, torch.tensor([n_tok]), 0, d // 2, 48)
    v0.update(K=K.numpy(), slots=slots.numpy(), cache=cache.numpy(), block_table=bt.numpy(),
              gathered_packed=gp.numpy(), gathered_norms=gn.numpy(),
              packed=ck.indices.numpy(), norms=ck.norms.numpy(),
              meta=np.array([d, b, Hkv, bs, nb, es, n_tok], np.int32))
    np.savez_compressed(os.path.join(HERE, "v0_layout.npz"), **v0)
    for f in sorted(os.listdir(HERE)):
        if f.endswith(".npz"):
            print(f, os.path.getsize(os.path.join(HERE, f)))


if __name__ == "__main__":
    main()
