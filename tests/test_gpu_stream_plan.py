"""The streaming decode kernel's launch protocol: the two-region split of the context, the
counters it clears itself (one workspace serving calls of different shapes, no initialisation),
and replays of a captured launch.
"""
import numpy as np
import pytest
import torch

from test_gpu_guards import _filled_pool

pytestmark = pytest.mark.gpu


def _oracle_bad(oracle, pool, key, val, q, seq_lens, got, d, bk, bv, which):
    """Elements of got[b] outside the gate, for the sequences in `which`."""
    ek, enk = oracle.encode(key.float().cpu().numpy(), pool.signs, pool.bounds_k, bk)
    ev, env = oracle.encode(val.float().cpu().numpy(), pool.signs, pool.bounds_v, bv)
    starts = np.concatenate([[0], np.cumsum(seq_lens)])
    bad = 0
    for b in which:
        S = int(seq_lens[b])
        sl = slice(starts[b], starts[b] + S)
        tr = lambda a: np.ascontiguousarray(np.swapaxes(a[sl], 0, 1))[None]
        ref = oracle.decode_attn(q[b:b + 1].float().cpu().numpy(), tr(ek), tr(enk), tr(ev), tr(env),
                                 pool.levels_k, pool.levels_v, pool.signs, d ** -0.5, bk, bv)
        bad += int((np.abs(got[b:b + 1] - ref) > 1e-3 + 2e-3 * np.abs(ref)).sum())
    return bad


def test_two_region_split_on_a_ragged_batch(oracle):
    """200 (sequence, KV head) units on 148 CTAs: one wave of whole-context items, the other 52
    units cut into shorter chunks -- among them sequences shorter than one chunk, sequences that
    end inside a chunk, and an empty one."""
    d, G, bk, bv, Hkv = 128, 4, 4, 4, 8
    rng = np.random.default_rng(11)
    seq_lens = rng.integers(1, 3000, 25).astype(np.int32)
    seq_lens[[0, 7, 19, 21, 24]] = [3000, 1, 0, 1537, 1024]
    pool, bt, key, val, _, _ = _filled_pool(d, bk, bv, Hkv, [int(s) for s in seq_lens], seed=3)
    g = torch.Generator("cpu").manual_seed(8)
    q = torch.randn(len(seq_lens), Hkv * G, d, generator=g).bfloat16().cuda()
    bt_d, sl_d = torch.from_numpy(bt).cuda(), torch.from_numpy(seq_lens).cuda()
    outs = [pool.decode_attention(q, bt_d, sl_d, int(seq_lens.max()), layer=0,
                                  out=torch.empty(q.shape, dtype=torch.float32, device="cuda"))
            for _ in range(2)]
    torch.cuda.synchronize()
    assert torch.equal(outs[0], outs[1])
    got = outs[0].cpu().numpy()
    assert np.isfinite(got).all()
    assert (got[19] == 0).all()
    which = [b for b in range(len(seq_lens)) if seq_lens[b] > 0]
    assert _oracle_bad(oracle, pool, key, val, q, seq_lens, got, d, bk, bv, which) == 0


def test_one_uninitialised_workspace_serves_calls_of_different_shapes():
    """The kernel clears the counters in the workspace tail itself: a workspace full of garbage
    works, and so does alternating between two batch shapes (different unit counts, different
    splits) on the same buffer."""
    d, G, bk, bv, Hkv = 128, 4, 4, 4, 4
    big, small = [5000, 3100, 4096, 77] * 12, [900, 33]
    pa, bta, *_ = _filled_pool(d, bk, bv, Hkv, big, seed=1)
    pb, btb, *_ = _filled_pool(d, bk, bv, Hkv, small, seed=2)
    g = torch.Generator("cpu").manual_seed(5)
    qa = torch.randn(len(big), Hkv * G, d, generator=g).bfloat16().cuda()
    qb = torch.randn(len(small), Hkv * G, d, generator=g).bfloat16().cuda()
    need = max(pa.workspace_bytes(len(big), Hkv * G, max(big), 1),
               pb.workspace_bytes(len(small), Hkv * G, max(small), 1))
    ws = torch.randint(0, 256, (need,), dtype=torch.uint8, device="cuda")
    ws[-4096:] = 0xFF            # the counter tail in particular

    def run(pool, q, bt, lens):
        out = torch.empty(q.shape, dtype=torch.float32, device="cuda")
        pool.decode_attention(q, torch.from_numpy(bt).cuda(), torch.tensor(lens, dtype=torch.int32).cuda(),
                              max(lens), layer=0, out=out, workspace=ws)
        return out

    a0 = run(pa, qa, bta, big)
    b0 = run(pb, qb, btb, small)
    a1 = run(pa, qa, bta, big)
    b1 = run(pb, qb, btb, small)
    torch.cuda.synchronize()
    # the reference result of each shape: a fresh, private workspace
    a_ref = pa.decode_attention(qa, torch.from_numpy(bta).cuda(), torch.tensor(big, dtype=torch.int32).cuda(),
                                max(big), layer=0, out=torch.empty(qa.shape, dtype=torch.float32, device="cuda"))
    b_ref = pb.decode_attention(qb, torch.from_numpy(btb).cuda(), torch.tensor(small, dtype=torch.int32).cuda(),
                                max(small), layer=0, out=torch.empty(qb.shape, dtype=torch.float32, device="cuda"))
    torch.cuda.synchronize()
    assert torch.isfinite(a_ref).all() and torch.isfinite(b_ref).all()
    assert torch.equal(a0, a_ref) and torch.equal(a1, a_ref)
    assert torch.equal(b0, b_ref) and torch.equal(b1, b_ref)


def test_replays_of_a_captured_decode_call():
    """A captured launch carries its epoch with it: every replay must still clear the counters
    before anybody counts on them.  Three replays with new queries against eager calls."""
    d, G, bk, bv, Hkv = 128, 4, 4, 4, 8
    lens = [4000, 2500, 8192, 100] * 10
    pool, bt, *_ = _filled_pool(d, bk, bv, Hkv, lens, seed=4)
    bt_d = torch.from_numpy(bt).cuda()
    sl_d = torch.tensor(lens, dtype=torch.int32).cuda()
    g = torch.Generator("cpu").manual_seed(6)
    qs = [torch.randn(len(lens), Hkv * G, d, generator=g).bfloat16().cuda() for _ in range(3)]
    eager = [pool.decode_attention(q, bt_d, sl_d, max(lens), layer=0) for q in qs]
    torch.cuda.synchronize()

    q_static = qs[0].clone()
    out_static = torch.empty_like(q_static)
    ws = torch.empty(pool.workspace_bytes(len(lens), Hkv * G, max(lens), 1), dtype=torch.uint8, device="cuda")
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        pool.decode_attention(q_static, bt_d, sl_d, max(lens), layer=0, out=out_static, workspace=ws)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        pool.decode_attention(q_static, bt_d, sl_d, max(lens), layer=0, out=out_static, workspace=ws)
    for i in (1, 2, 0, 2):
        q_static.copy_(qs[i])
        graph.replay()
        graph.replay()          # back to back: the second replay starts from the first one's leftovers
        torch.cuda.synchronize()
        assert torch.equal(out_static, eager[i]), f"replay with query set {i}"
