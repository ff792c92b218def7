"""The give-up path of the decode kernels' bounded waits, executed on purpose.

Every wait in device code has a poll limit; a wait that runs out marks the rows concerned NaN, sets
a bit in the call's status word and lets the kernel finish.  In the product library that path
only runs when a copy is lost, so this test uses the second library the build script makes
(`libftq_b200_waittest.so`): identical, except that in the head_dim-128 decode kernels warp 5 of
CTA 0 announces its first page copy to the mbarrier without issuing it, and the poll limit is 64.
Nothing faults, traps or spins without bound: the wait simply expires.
"""
import ctypes
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _test_lib():
    from fused_turboquant_b200 import _lib, build
    if not os.path.exists(build.TEST_LIB_PATH):
        pytest.skip("libftq_b200_waittest.so has not been built")
    lib = ctypes.CDLL(build.TEST_LIB_PATH)
    for name, (res, args) in _lib.SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    return lib


@pytest.mark.parametrize("G", [4, 8])   # streaming kernel / barrier-synchronised kernel
def test_an_expired_wait_poisons_its_rows_and_nothing_else(G):
    from fused_turboquant_b200 import PagedKVPool, _lib
    bad_lib, good_lib = _test_lib(), _lib.load()
    d, bk, bv, Hkv = 128, 4, 4, 2
    # equal lengths: every work item exists and is long enough for warp 5 to own a page of it,
    # whichever item CTA 0 draws first
    seq_lens = [4096, 4096, 4096]
    B = len(seq_lens)
    max_blocks = (max(seq_lens) + 15) // 16
    rng = np.random.default_rng(3)
    bt = torch.from_numpy(rng.permutation(B * max_blocks).reshape(B, max_blocks).astype(np.int32)).cuda()
    pool = PagedKVPool(B * max_blocks, Hkv, d, bk, bv, n_layers=1, device="cuda")
    g = torch.Generator("cpu").manual_seed(9)
    n_tok = sum(seq_lens)
    key = torch.randn(n_tok, Hkv, d, generator=g).bfloat16().cuda()
    val = torch.randn(n_tok, Hkv, d, generator=g).bfloat16().cuda()
    slots = torch.cat([bt[b, torch.arange(s, device="cuda") // 16].long() * 16 +
                       torch.arange(s, device="cuda") % 16 for b, s in enumerate(seq_lens)])
    pool.store(key, val, slots, layer=0)
    q = torch.randn(B, Hkv * G, d, generator=g).bfloat16().cuda()
    sl = torch.tensor(seq_lens, dtype=torch.int32).cuda()
    ws = torch.empty(pool.workspace_bytes(B, Hkv * G, max(seq_lens), 1), dtype=torch.uint8, device="cuda")
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    p = lambda t: ctypes.c_void_p(t.data_ptr())

    def run(lib):
        out = torch.full(q.shape, 7.0, dtype=torch.float32, device="cuda")
        rc = lib.ftq_paged_decode_attn(
            p(q), _lib.BF16, p(out), _lib.F32, p(pool.pool[0]), pool.num_blocks, pool.layer_stride, 1,
            p(bt), bt.shape[1], p(sl), max(seq_lens), B, Hkv * G, Hkv, d, bk, bv,
            _lib.fptr(pool.levels_k), _lib.fptr(pool.levels_v), _lib.fptr(pool.signs), d ** -0.5,
            p(ws), ws.numel(), stream)
        assert rc == 0, lib.ftq_last_error()
        bits = ctypes.c_int(-1)
        rc = lib.ftq_paged_decode_status(p(ws), B, Hkv * G, Hkv, d, max(seq_lens), 1, stream,
                                         ctypes.byref(bits))
        return out.cpu().numpy(), rc, bits.value

    good, rc, bits = run(good_lib)
    assert rc == 0 and bits == 0 and np.isfinite(good).all()

    got, rc, bits = run(bad_lib)          # returns: the wait gave up after its 64 polls
    assert rc == -5 and bits == 2, (rc, bits)
    # exactly one (sequence, KV head) unit -- the one whose chunk CTA 0 started with -- is
    # poisoned, all of its rows; every other unit is untouched by the lost copy
    units = got.reshape(B, Hkv, G, d)
    poisoned = np.isnan(units).any(axis=(2, 3))
    assert poisoned.sum() == 1, poisoned
    assert np.isnan(units[poisoned]).all()
    np.testing.assert_array_equal(units[~poisoned], good.reshape(B, Hkv, G, d)[~poisoned])

    again, rc, bits = run(good_lib)       # the context is as usable as before
    assert rc == 0 and bits == 0
    np.testing.assert_array_equal(again, good)
