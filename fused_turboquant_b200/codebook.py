"""Host-side tables of the quantizer: RHT sign vector and Lloyd-Max codebook.

Both are tiny, computed once per (head_dim, bits, seed) and handed to the CUDA
kernels as inputs; they must be bit-identical to the reference's tables because
the codes are compared bit for bit.

  * signs     -- generate_rht_signs, src/fused_turboquant/core/hadamard.py:56-67
  * codebook  -- compute_lloyd_max_codebook, src/fused_turboquant/core/lloyd_max.py:24-88
"""
from __future__ import annotations

import math
from functools import lru_cache

import numpy as np


def rht_signs(dim: int, seed: int = 0) -> np.ndarray:
    """Seeded +-1 vector: torch's CPU generator, randint(0, 2) * 2 - 1, as fp32."""
    import torch

    gen = torch.Generator(device="cpu").manual_seed(seed)
    bits = torch.randint(0, 2, (dim,), generator=gen, dtype=torch.float32, device="cpu")
    return (bits * 2 - 1).numpy().astype(np.float32)


def _cell_means(grid: np.ndarray, pdf: np.ndarray, edges: np.ndarray) -> np.ndarray:
    """Weighted mean of the grid points of every cell [edges[i], edges[i+1]) (last cell closed)."""
    n = edges.size - 1
    lo = np.searchsorted(grid, edges[:-1], side="left")
    hi = np.searchsorted(grid, edges[1:], side="left")
    hi[-1] = np.searchsorted(grid, edges[-1], side="right")
    out = np.zeros(n)
    for i in range(n):
        w = pdf[lo[i]:hi[i]]
        tot = w.sum()
        if tot > 0:
            out[i] = np.multiply(grid[lo[i]:hi[i]], w).sum() / tot
        else:
            out[i] = (edges[i] + edges[i + 1]) / 2.0
    return out


@lru_cache(maxsize=64)
def lloyd_max_codebook(dim: int, bits: int, max_iterations: int = 300,
                       num_grid_points: int = 50000) -> tuple[np.ndarray, np.ndarray]:
    """Grid Lloyd-Max for the coordinate law of a random unit vector, pdf ~ (1-z^2)^((d-3)/2).

    Returns (boundaries[2^bits + 1], levels[2^bits]) in float64; callers cast to fp32.
    The grid spans +-6/sqrt(d) (clipped to +-1); the start is the equal-mass
    partition; every iteration sets interior boundaries to level midpoints and
    levels to cell means.
    """
    n_levels = 1 << bits
    sigma = 1.0 / math.sqrt(dim)
    lo, hi = max(-1.0, -6.0 * sigma), min(1.0, 6.0 * sigma)
    grid = np.linspace(lo, hi, num_grid_points)
    pdf = np.maximum(1.0 - grid**2, 0.0) ** ((dim - 3) / 2.0)
    pdf /= pdf.sum()

    edges = np.interp(np.linspace(0, 1, n_levels + 1), np.cumsum(pdf), grid)
    edges[0], edges[-1] = lo, hi
    levels = _cell_means(grid, pdf, edges)
    for _ in range(max_iterations):
        edges[1:-1] = (levels[:-1] + levels[1:]) / 2.0
        levels = _cell_means(grid, pdf, edges)
    edges.setflags(write=False)
    levels.setflags(write=False)
    return edges, levels


def codebook_f32(dim: int, bits: int, max_iterations: int = 300,
                 num_grid_points: int = 50000) -> tuple[np.ndarray, np.ndarray]:
    """(boundaries, levels) as contiguous fp32 arrays, the form the kernels take."""
    b, l = lloyd_max_codebook(dim, bits, max_iterations, num_grid_points)
    return np.ascontiguousarray(b, dtype=np.float32), np.ascontiguousarray(l, dtype=np.float32)
