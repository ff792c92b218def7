"""TurboQuantMSE on the B200 kernels: the reference's quantizer API
(src/fused_turboquant/core/quantizer.py:36-216) with every tensor operation
routed to libftq_b200.so.

The object owns the host tables (signs, boundaries, levels) and mirrors them
as device tensors for callers that read ``tq.rotation.signs`` /
``tq.quantizer.levels``.  encode/decode require CUDA tensors; there is no
unfused PyTorch branch.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from . import codebook, kernels


@dataclass
class CompressedTensor:
    """Packed codes + fp16 norms of a tensor of head vectors (reference: quantizer.py:36-51)."""

    indices: torch.Tensor
    norms: torch.Tensor
    original_dim: int
    bits: int

    @property
    def compression_ratio(self) -> float:
        original_bytes = self.norms.numel() * self.original_dim * 2
        compressed_bytes = self.indices.numel() + self.norms.numel() * 2
        if compressed_bytes == 0:
            return float("inf")
        return original_bytes / compressed_bytes


class _Rotation:
    """Holds the sign vector; forward/inverse call the RHT kernel (reference: hadamard.py:119-160)."""

    def __init__(self, dim: int, seed: int, device):
        self.dim = dim
        self.signs_host = codebook.rht_signs(dim, seed)
        self.signs = torch.from_numpy(self.signs_host).to(device)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return kernels.rht(x, self.signs_host, inverse=False)

    __call__ = forward

    def inverse(self, y: torch.Tensor) -> torch.Tensor:
        return kernels.rht(y, self.signs_host, inverse=True)

    def to(self, device):
        self.signs = self.signs.to(device)
        return self


class _Codebook:
    """boundaries / levels of the Lloyd-Max quantizer (reference: lloyd_max.py:91-141)."""

    def __init__(self, dim: int, bits: int, device, max_iterations: int, num_grid_points: int):
        self.dim, self.bits, self.num_levels = dim, bits, 1 << bits
        self.boundaries_host, self.levels_host = codebook.codebook_f32(
            dim, bits, max_iterations, num_grid_points)
        self.boundaries = torch.from_numpy(self.boundaries_host).to(device)
        self.levels = torch.from_numpy(self.levels_host).to(device)

    def to(self, device):
        self.boundaries = self.boundaries.to(device)
        self.levels = self.levels.to(device)
        return self


class TurboQuantMSE:
    """RHT + Lloyd-Max quantizer of head vectors.

        tq = TurboQuantMSE(head_dim=128, bits=4, device="cuda")
        ct = tq.encode(keys)      # (..., head_dim) -> CompressedTensor
        x  = tq.decode(ct)        # -> (..., head_dim) fp32
    """

    def __init__(self, head_dim: int, bits: int = 4, seed: int = 42, device="cuda",
                 max_iterations: int = 300, num_grid_points: int = 50000):
        if head_dim < 1 or (head_dim & (head_dim - 1)) != 0:
            raise ValueError(f"head_dim must be a power of 2, got {head_dim}")
        if bits not in (2, 3, 4):
            raise ValueError(f"bits must be 2, 3, or 4, got {bits}")
        self.head_dim, self.bits, self.device, self.seed = head_dim, bits, device, seed
        self.rotation = _Rotation(head_dim, seed, device)
        self.quantizer = _Codebook(head_dim, bits, device, max_iterations, num_grid_points)

    def encode(self, x: torch.Tensor) -> CompressedTensor:
        packed, norms = kernels.fused_encode(x, self.rotation.signs_host,
                                             self.quantizer.boundaries_host, self.bits)
        return CompressedTensor(indices=packed, norms=norms, original_dim=self.head_dim,
                                bits=self.bits)

    def decode(self, compressed: CompressedTensor) -> torch.Tensor:
        return kernels.fused_decode(compressed.indices, compressed.norms,
                                    self.quantizer.levels_host, self.rotation.signs_host,
                                    compressed.bits, compressed.original_dim)

    def roundtrip(self, x: torch.Tensor) -> torch.Tensor:
        return self.decode(self.encode(x))

    def to(self, device) -> "TurboQuantMSE":
        self.device = device
        self.rotation.to(device)
        self.quantizer.to(device)
        return self
