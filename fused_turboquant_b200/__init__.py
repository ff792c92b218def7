"""fused_turboquant_b200 -- B200-native (sm_100a) kernels for fused-turboquant's
KV encode and compressed-KV decode attention, behind the reference's surfaces.

Public names follow the reference package (src/fused_turboquant/__init__.py):
``TurboQuantMSE``, ``CompressedTensor`` and the kernel-level callables in
``fused_turboquant_b200.kernels``; ``PagedKVPool`` is the paged cache the vLLM
attention impl drives, ``hf_cache.CompressedKVCache`` the HF-style cache on top of it and
``tq_v1`` the vLLM-v1 slot-format store / decode.
"""
from .quantizer import CompressedTensor, TurboQuantMSE  # noqa: F401
from .paged import PagedKVPool  # noqa: F401
from . import kernels  # noqa: F401
from . import hf_cache, tq_v1  # noqa: F401

__version__ = "0.1.0"
