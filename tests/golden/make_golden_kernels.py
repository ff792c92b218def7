"""Generates kernels_interp.npz by running the REFERENCE's own GPU kernels on the CPU.

    python tests/golden/make_golden_kernels.py --reference /path/to/reference

The reference's device code is written in Triton; Triton's interpreter mode
(TRITON_INTERPRET=1) executes those kernels on CPU tensors, program by program, so that the
outputs of the kernels themselves -- not of the reference's unfused PyTorch fallbacks -- can be
pinned without a GPU.  Inputs are the ones already stored in encode.npz / attention.npz /
fwht_kat.npz (written by make_golden.py, run that first); this file adds, for the same inputs:

  enc_d{D}_b{b}_packed / _norms   triton_fused_encode           (kernels/triton_encode.py)
  dec_d{D}_b{b}                   triton_fused_decode           (kernels/triton_decode.py)
  rht_d{D} / irht_d{D}            triton_rht forward / inverse  (kernels/triton_rht.py)
  {case}_scores                   fused_qk_scores_rht           (kernels/triton_attention.py)
  {case}_flash                    flash_decode_compressed       (kernels/triton_flash_decode.py)

Two things are adjusted at generation time only, neither touches kernel arithmetic: the QK
kernel's autotuner is given a single tile configuration (benchmarking candidates needs a GPU
driver), and `Tensor.is_cuda` reports True while flash_decode_compressed runs, because its
wrapper otherwise diverts CPU tensors to a fallback that cannot run without a GPU either.
"""
from __future__ import annotations

import argparse
import os
import sys

os.environ["TRITON_INTERPRET"] = "1"

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
DIMS = (64, 128, 256)
BITS = (2, 3, 4)
ATT_CASES = ("cfg1small", "d64_g7_k3v3", "d256_g2_k4v2")
DEC_CASES = ((64, 2), (128, 4), (256, 3))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of the reference repository")
    args = ap.parse_args()
    sys.path.insert(0, os.path.join(args.reference, "src"))
    import fused_turboquant.kernels.triton_attention as ta
    from fused_turboquant.kernels.triton_decode import triton_fused_decode
    from fused_turboquant.kernels.triton_encode import triton_fused_encode
    from fused_turboquant.kernels.triton_flash_decode import flash_decode_compressed
    from fused_turboquant.kernels.triton_rht import triton_rht

    ta._fused_qk_scores_kernel.configs = ta._fused_qk_scores_kernel.configs[1:2]  # BLOCK_S 64, BLOCK_D 64
    torch.set_num_threads(1)

    tables = np.load(os.path.join(HERE, "tables.npz"))
    enc = np.load(os.path.join(HERE, "encode.npz"))
    att = np.load(os.path.join(HERE, "attention.npz"))
    kat = np.load(os.path.join(HERE, "fwht_kat.npz"))
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a))
    out = {}

    for d in DIMS:
        signs = t(tables[f"signs_d{d}"])
        x = t(kat[f"x_d{d}"])
        y = triton_rht(x, signs)
        out[f"rht_d{d}"] = y.numpy()
        out[f"irht_d{d}"] = triton_rht(y, signs, inverse=True).numpy()
        for b in BITS:
            packed, norms = triton_fused_encode(t(enc[f"x32_d{d}"]), signs,
                                                t(tables[f"boundaries_d{d}_b{b}"]), b)
            out[f"enc_d{d}_b{b}_packed"] = packed.numpy()
            out[f"enc_d{d}_b{b}_norms"] = norms.numpy()
            print("encode", d, b, flush=True)
    for d, b in DEC_CASES:
        o = triton_fused_decode(t(enc[f"x32_d{d}_b{b}_packed"]), t(enc[f"x32_d{d}_b{b}_norms"]),
                                t(tables[f"levels_d{d}_b{b}"]), t(tables[f"signs_d{d}"]), b, d)
        out[f"dec_d{d}_b{b}"] = o.numpy()
        print("decode", d, b, flush=True)

    for name in ATT_CASES:
        B, Hkv, G, S, d, bk, bv = (int(v) for v in att[f"{name}_meta"])
        q_rot = t(att[f"{name}_q_rot"])
        k_idx, k_norms = t(att[f"{name}_k_idx"]), t(att[f"{name}_k_norms"])
        v_idx, v_norms = t(att[f"{name}_v_idx"]), t(att[f"{name}_v_norms"])
        lk, lv = t(tables[f"levels_d{d}_b{bk}"]), t(tables[f"levels_d{d}_b{bv}"])
        scale = d ** -0.5
        out[f"{name}_scores"] = ta.fused_qk_scores_rht(q_rot, k_idx, k_norms.float(), lk, scale,
                                                       bits=bk).numpy()
        torch.Tensor.is_cuda = property(lambda self: True)
        try:
            o = flash_decode_compressed(q_rot, k_idx, k_norms, v_idx, v_norms, lk, lv,
                                        t(tables[f"signs_d{d}"]), scale, bits_k=bk, bits_v=bv)
        finally:
            del torch.Tensor.is_cuda
        out[f"{name}_flash"] = o.numpy()
        print("attention", name, flush=True)

    path = os.path.join(HERE, "kernels_interp.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path))


if __name__ == "__main__":
    main()
