"""ftq_paged_decode_attn_static: paged decode attention for embedders that cannot allocate.

Collected last on purpose (file name), so a run that stops at the first failure has already
exercised everything else.  The entry point keeps its split-KV scratch in an array inside the
library, so a host whose device memory is fully owned by its own block manager -- or that is
entered where cudaMalloc is off limits -- can still run the decode step.  Checked here, through
the C ABI: same output as the workspace-taking entry point on two calls in a row (the scratch is
shared and not cleared between calls), and a clean error when the batch does not fit.
"""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _call(lib, static, q, out, pool, bt, sl, max_seq, ws=None):
    from fused_turboquant_b200 import _lib
    L, B, Hq, D = q.shape
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    args = [p(q), _lib.BF16, p(out), _lib.BF16, p(pool.pool), pool.num_blocks, pool.layer_stride, L,
            p(bt), bt.shape[1], p(sl), max_seq, B, Hq, pool.num_kv_heads, D, pool.key_bits,
            pool.value_bits, _lib.fptr(pool.levels_k), _lib.fptr(pool.levels_v),
            _lib.fptr(pool.signs), float(D) ** -0.5]
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    if static:
        return lib.ftq_paged_decode_attn_static(*args, stream)
    return lib.ftq_paged_decode_attn(*args, p(ws), ws.numel(), stream)


def test_static_scratch_entry_point_matches_workspace_entry_point():
    from fused_turboquant_b200 import PagedKVPool, _lib
    lib = _lib.load()
    dev = torch.device("cuda", 0)
    L, B, Hkv, G, D, bk, bv = 2, 4, 2, 4, 128, 4, 3
    seq_lens = np.array([900, 17, 300, 64], np.int32)
    max_seq = int(seq_lens.max())
    max_blocks = (max_seq + 15) // 16
    num_blocks = B * max_blocks
    g = torch.Generator("cpu").manual_seed(4242)
    bt = torch.randperm(num_blocks, generator=g).view(B, max_blocks).to(torch.int32)
    pool = PagedKVPool(num_blocks, Hkv, D, bk, bv, n_layers=L, device=dev)
    n_tok = int(seq_lens.sum())
    slots = torch.cat([bt[b, torch.arange(int(n)) // 16].long() * 16 + torch.arange(int(n)) % 16
                       for b, n in enumerate(seq_lens)])
    key = torch.randn(L, n_tok, Hkv, D, generator=g).bfloat16()
    val = torch.randn(L, n_tok, Hkv, D, generator=g).bfloat16()
    pool.store(key.to(dev), val.to(dev), slots.to(dev))
    bt_d, sl_d = bt.to(dev), torch.from_numpy(seq_lens).to(dev)
    ws = torch.empty(pool.workspace_bytes(B, Hkv * G, max_seq, L), dtype=torch.uint8, device=dev)
    assert ws.numel() <= 8 << 20

    for call in range(2):      # second call reuses the scratch the first one dirtied
        q = torch.randn(L, B, Hkv * G, D, generator=g).bfloat16().to(dev)
        want = torch.full_like(q, float("nan"))
        got = torch.full_like(q, float("nan"))
        assert _call(lib, False, q, want, pool, bt_d, sl_d, max_seq, ws) == 0, lib.ftq_last_error()
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info(dev)
        assert _call(lib, True, q, got, pool, bt_d, sl_d, max_seq) == 0, lib.ftq_last_error()
        torch.cuda.synchronize()
        if call == 1:   # (the first call may load the kernel's module; the second must be clean)
            assert torch.cuda.mem_get_info(dev)[0] == free_before, "the call changed free device memory"
        bits = ctypes.c_int(-1)
        assert lib.ftq_paged_decode_status(None, B, Hkv * G, Hkv, D, max_seq, L,
                                           ctypes.c_void_p(torch.cuda.current_stream().cuda_stream),
                                           ctypes.byref(bits)) == 0
        assert bits.value == 0
        a, b = got.float().cpu().numpy(), want.float().cpu().numpy()
        assert np.isfinite(a).all()
        # same gate the other decode tests use for bf16 outputs; in practice the bits agree
        assert (np.abs(a - b) <= 1e-3 + 2e-3 * np.abs(b)).all(), f"call {call}"
        assert np.array_equal(a, b), f"call {call}: outputs differ"


def test_static_scratch_rejects_a_batch_that_does_not_fit():
    from fused_turboquant_b200 import PagedKVPool, _lib
    lib = _lib.load()
    dev = torch.device("cuda", 0)
    L, B, Hkv, G, D = 1, 512, 8, 4, 128
    need = lib.ftq_decode_workspace_bytes(B, Hkv * G, Hkv, D, 64, L)
    assert need > 8 << 20
    pool = PagedKVPool(B * 4, Hkv, D, 4, 4, n_layers=L, device=dev)
    q = torch.zeros(L, B, Hkv * G, D, dtype=torch.bfloat16, device=dev)
    out = torch.zeros_like(q)
    bt = torch.arange(B * 4, dtype=torch.int32, device=dev).view(B, 4)
    sl = torch.full((B,), 64, dtype=torch.int32, device=dev)
    rc = _call(lib, True, q, out, pool, bt, sl, 64)
    assert rc == -4
    msg = lib.ftq_last_error().decode()
    assert "built-in scratch" in msg and str(need) in msg
