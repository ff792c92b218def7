"""GPU parity of the vLLM-v1 slot-format path (fused store, split-KV decode) against the
reference's own kernels (tests/golden/tq_v1.npz: their outputs in Triton's interpreter mode)
and against the oracle's restatement.

Bars: value codes, scale/zero and untouched bytes identical; key codes identical except where
the rotated value sits within 1e-6 of a midpoint; key norm within one fp16 ulp of the reference
kernel and identical to the oracle (same summation order); decode partials and outputs within
2e-4 relative + 2e-5 absolute in fp32, the 2e-3 / 1e-3 gate for 16-bit outputs.  Lloyd-Max value
codes ("_vlm") are held to the key codes' bar; FP8 keys ("k8") to the bar tests/helpers.py spells
out (identical to the oracle; identical to the reference kernel's bytes outside the three
situations in which Triton's interpreter mis-emulates the fp8 cast; identical to torch's
round-to-nearest-even cast away from ties).
"""
import numpy as np
import pytest
import torch

from helpers import gate, tq_v1_compare_cache

pytestmark = pytest.mark.gpu

CASES = ["d128_k4v4", "d128_k3v4_nc", "d64_k3v3_g7", "d256_k4v2", "d128_k2v8",
         "d128_k1v1_nc", "d64_k1v3", "d256_k3v1_nc",
         "d128_k4v4_nc_vlm", "d64_k4v4_vlm", "d128_k3v4_nc_vlm",   # _vlm: Lloyd-Max value codes
         "d128_k8v4", "d64_k8v2", "d256_k8v3"]                     # k8: FP8 (e4m3) keys
# 8-bit Lloyd-Max key codes (tq_v1_k8mse.npz; the reference's boundary layers): the fixtures' meta
# says 8 key bits like the FP8 cases; the oracle / helpers tell the two apart by key bits = 264,
# the host mirror by key_use_fp8_at_8bit
K8MSE = ["d128_k8mse_v4_nc", "d64_k8mse_v3", "d256_k8mse_v2_nc"]
cu = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _meta(g, name):
    return (int(v) for v in g[f"{name}_meta"])


def _case(golden, name):
    """(fixtures, meta with the oracle's key bits, host-mirror config) of a store / decode case."""
    from fused_turboquant_b200 import tq_v1
    mse8 = name in K8MSE
    g = golden("tq_v1_k8mse.npz" if mse8 else "tq_v1.npz")
    meta = [int(v) for v in g[f"{name}_meta"]]
    cfg = tq_v1.TurboQuantSlotConfig(meta[0], meta[3], meta[4], bool(meta[5]),
                                     key_use_fp8_at_8bit=not mse8)
    if mse8:
        meta[3] = 264
    return g, meta, cfg


@pytest.mark.parametrize("name", CASES + K8MSE)
def test_store_vs_reference_kernel_and_oracle(oracle, golden, name):
    from fused_turboquant_b200 import tq_v1
    g, (D, Hkv, G, kb, vb, nc, splits, bs, slot, nb), cfg = _case(golden, name)
    assert cfg.slot_size_aligned == slot
    cache = torch.zeros((nb, bs, Hkv, slot), dtype=torch.uint8, device="cuda")
    vlm = name.endswith("_vlm")    # (the fixture's V is already rotated for these cases)
    tq_v1.launch_store(cu(g[f"{name}_K"]), cu(g[f"{name}_V"]), cache, cu(g[f"{name}_slot_mapping"]),
                       g[f"{name}_midpoints"], cfg, D, v_lloyd_max=vlm)
    got = cache.cpu().numpy()
    st = tq_v1_compare_cache(got, g[f"{name}_cache"], g[f"{name}_slot_mapping"],
                             g[f"{name}_kun" if kb == 8 else f"{name}_y"],
                             g[f"{name}_midpoints"], D, kb, vb, bs, vy=g[f"{name}_vy"] if vlm else None)
    assert st["key_fp8_differ_unexplained"] == 0 and st["key_fp8_vs_rne"] == 0, st
    assert st["value_bytes_differ"] == 0 and st["other_bytes_differ"] == 0, st
    assert st["key_codes_differ_off_midpoint"] == 0 and st["key_norm_max_ulp"] <= 1, st
    assert st["value_codes_differ_off_midpoint"] == 0 and st["value_norm_max_ulp"] <= 1, st
    ref = np.zeros_like(got)
    oracle.tq_store(g[f"{name}_K"], g[f"{name}_V"], ref, g[f"{name}_slot_mapping"],
                    g[f"{name}_midpoints"], kb, vb, value_lloyd_max=vlm)
    np.testing.assert_array_equal(got, ref)


@pytest.mark.parametrize("name", CASES + K8MSE)
def test_decode_vs_reference_kernels(oracle, golden, name):
    from fused_turboquant_b200 import tq_v1
    g, (D, Hkv, G, kb, vb, nc, splits, bs, slot, nb), cfg = _case(golden, name)
    B, Hq = g[f"{name}_q"].shape[:2]
    mid_o = torch.empty((B, Hq, splits, D + 1), dtype=torch.float32, device="cuda")
    lse = torch.empty((B, Hq), dtype=torch.float32, device="cuda")
    out = tq_v1.decode_attention(cu(g[f"{name}_q"]), cu(g[f"{name}_cache"]), cu(g[f"{name}_block_table"]),
                                 cu(g[f"{name}_seq_lens"]), g[f"{name}_centroids"], cfg, D ** -0.5,
                                 num_kv_splits=splits, kv_start_offset=cu(g[f"{name}_kv_start"]),
                                 mid_o=mid_o, lse=lse, v_lloyd_max=name.endswith("_vlm"))
    ref = g[f"{name}_mid_o"]
    m = mid_o.cpu().numpy()
    live = np.isfinite(ref[..., D])
    np.testing.assert_array_equal(np.isfinite(m[..., D]), live)
    np.testing.assert_allclose(m[..., D][live], ref[..., D][live], rtol=1e-5, atol=2e-5)
    np.testing.assert_allclose(m[..., :D][live], ref[..., :D][live], rtol=2e-4, atol=2e-5)
    assert np.all(m[..., :D][~live] == 0)
    o_ref, _, lse_ref = oracle.tq_decode(g[f"{name}_q"], g[f"{name}_cache"], g[f"{name}_block_table"],
                                         g[f"{name}_seq_lens"], g[f"{name}_centroids"], kb, vb, D ** -0.5,
                                         splits, norm_correction=bool(nc), kv_start=g[f"{name}_kv_start"],
                                         value_lloyd_max=name.endswith("_vlm"))
    if f"{name}_out" in g.files:
        o_ref, lse_ref = g[f"{name}_out"], g[f"{name}_lse"]
    np.testing.assert_allclose(out.cpu().numpy(), o_ref, rtol=2e-4, atol=2e-5)
    np.testing.assert_allclose(lse.cpu().numpy(), lse_ref, rtol=1e-5, atol=2e-5)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("D,kb,vb,G,nc,lm", [
    (128, 4, 4, 4, True, False), (64, 2, 3, 7, False, False), (256, 3, 8, 2, True, False),
    (128, 3, 2, 8, False, False), (64, 1, 1, 4, True, False), (128, 1, 4, 2, False, False),
    (256, 4, 1, 2, True, False),
    # Lloyd-Max value codes (with the fused value rotation, as the reference always pairs them)
    (128, 4, 4, 4, True, True), (64, 4, 4, 7, False, True), (256, 3, 4, 2, True, True),
    # FP8 keys
    (128, 8, 4, 4, False, False), (64, 8, 8, 7, False, False), (256, 8, 2, 2, False, False)])
def test_store_then_decode_random_vs_oracle(oracle, D, kb, vb, G, nc, lm, dtype):
    """Ragged batch, 16-bit inputs, values kept in the rotated space, several splits."""
    from fused_turboquant_b200 import tq_v1
    rng = np.random.default_rng(D + kb + vb)
    Hkv, bs, splits = 2, 16, 5
    seq = [1, 37, 300, 129]
    B, Hq = len(seq), Hkv * G
    max_blocks = max((s + bs - 1) // bs for s in seq)
    nb = B * max_blocks + 3
    bt = rng.permutation(nb)[:B * max_blocks].astype(np.int32).reshape(B, max_blocks)
    slots = np.concatenate([[bt[b, t // bs] * bs + t % bs for t in range(s)] for b, s in enumerate(seq)])
    n = len(slots)
    K = torch.from_numpy(rng.standard_normal((n, Hkv, D)).astype(np.float32)).to(dtype)
    V = torch.from_numpy((rng.standard_normal((n, Hkv, D)) * 2 + 0.5).astype(np.float32)).to(dtype)
    q = torch.from_numpy(rng.standard_normal((B, Hq, D)).astype(np.float32)).to(dtype)
    cent = np.sort(rng.standard_normal(1 << min(kb, 4)).astype(np.float32)) / np.sqrt(D)   # (FP8 keys: unused)
    cent_t, mids_t = tq_v1.midpoints_of(torch.from_numpy(cent))
    cfg = tq_v1.TurboQuantSlotConfig(D, kb, vb, nc)
    slot = cfg.slot_size_aligned
    cache = torch.zeros((nb, bs, Hkv, slot), dtype=torch.uint8, device="cuda")
    tq_v1.launch_store(K.cuda(), V.cuda(), cache, torch.from_numpy(slots).cuda(), mids_t, cfg, v_rotate=True,
                       v_lloyd_max=lm)
    # oracle: values rotated first (plain Hadamard transform of the 16-bit inputs, kept in fp32 ->
    # the library rounds the rotated values back to the input dtype before quantising them)
    v_rot = torch.from_numpy(oracle.rht(V.float().numpy().reshape(-1, D), None)).to(dtype).float().numpy()
    ref = np.zeros((nb, bs, Hkv, slot), np.uint8)
    oracle.tq_store(K.float().numpy(), v_rot.reshape(n, Hkv, D), ref, slots, mids_t.numpy(), kb, vb,
                    value_lloyd_max=lm, value_sum_order=1)
    np.testing.assert_array_equal(cache.cpu().numpy(), ref)
    out = tq_v1.decode_attention(q.cuda(), cache, torch.from_numpy(bt).cuda(),
                                 torch.tensor(seq, dtype=torch.int32).cuda(), cent_t, cfg, D ** -0.5,
                                 num_kv_splits=splits, v_rotate=True, out_dtype=torch.float32, v_lloyd_max=lm)
    o_ref, _, _ = oracle.tq_decode(q.float().numpy(), ref, bt, np.array(seq, np.int32), cent_t.numpy(), kb, vb,
                                   D ** -0.5, splits, norm_correction=nc, rotate_out=True, value_lloyd_max=lm)
    # 16-bit queries take the tensor-core kernel where it exists (fp16 centroids / weights, fp32
    # accumulation): the north-star gate; 8-bit values, 1-bit codes and head_dim 256 stay on the
    # fp32 kernel
    if vb == 8 or D == 256 or 1 in (kb, vb) or lm or kb == 8:
        assert gate(out.cpu().numpy(), o_ref, 2e-4, 1e-4) == 0
    else:
        assert gate(out.cpu().numpy(), o_ref) == 0, np.abs(out.cpu().numpy() - o_ref).max()
    out16 = tq_v1.decode_attention(q.cuda(), cache, torch.from_numpy(bt).cuda(),
                                   torch.tensor(seq, dtype=torch.int32).cuda(), cent_t, cfg, D ** -0.5,
                                   num_kv_splits=splits, v_rotate=True, v_lloyd_max=lm)
    assert out16.dtype == dtype
    assert torch.equal(out16, out.to(dtype)) or gate(out16.float().cpu().numpy(), o_ref) <= out16.numel() // 500


@pytest.mark.parametrize("qdtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("name", ["d128_k4v4", "d128_k3v4_nc", "d64_k3v3_g7"])
def test_tensor_core_decode_vs_reference_fixture(oracle, golden, name, qdtype):
    """16-bit queries: the tensor-core stage 1 on the reference kernel's own cache bytes."""
    from fused_turboquant_b200 import tq_v1
    g = golden("tq_v1.npz")
    D, Hkv, G, kb, vb, nc, splits, bs, slot, nb = _meta(g, name)
    cfg = tq_v1.TurboQuantSlotConfig(D, kb, vb, bool(nc))
    q = cu(g[f"{name}_q"]).to(qdtype)
    B, Hq = q.shape[:2]
    mid_o = torch.empty((B, Hq, splits, D + 1), dtype=torch.float32, device="cuda")
    out = tq_v1.decode_attention(q, cu(g[f"{name}_cache"]), cu(g[f"{name}_block_table"]),
                                 cu(g[f"{name}_seq_lens"]), g[f"{name}_centroids"], cfg, D ** -0.5,
                                 num_kv_splits=splits, kv_start_offset=cu(g[f"{name}_kv_start"]),
                                 mid_o=mid_o, out_dtype=torch.float32)
    o_ref, m_ref, _ = oracle.tq_decode(q.float().cpu().numpy(), g[f"{name}_cache"], g[f"{name}_block_table"],
                                       g[f"{name}_seq_lens"], g[f"{name}_centroids"], kb, vb, D ** -0.5,
                                       splits, norm_correction=bool(nc), kv_start=g[f"{name}_kv_start"])
    m = mid_o.cpu().numpy()
    live = np.isfinite(m_ref[..., D])
    np.testing.assert_array_equal(np.isfinite(m[..., D]), live)
    assert np.all(m[..., :D][~live] == 0)
    np.testing.assert_allclose(m[..., D][live], m_ref[..., D][live], rtol=2e-3, atol=5e-3)
    # fp16 queries / weights on keys with x12 outlier channels: up to 2 elements in a thousand
    # sit just outside the 2e-3 / 1e-3 gate in fp32 (measured: 0-16 of 3 072-8 192 partial
    # elements, max |err| 2.8e-3; 0-3 of 1 024-2 048 output elements, max |err| 1.7e-3; all far
    # inside one bf16 ulp of the output)
    part, ref_part = m[..., :D][live], m_ref[..., :D][live]
    print(f"\n[tq tensor-core stage 1] {name} {qdtype}: partials outside 2e-3/1e-3: "
          f"{gate(part, ref_part)} of {part.size}, max |err| {np.abs(part - ref_part).max():.2e}; "
          f"outputs outside: {gate(out.cpu().numpy(), o_ref)} of {o_ref.size}, "
          f"max |err| {np.abs(out.cpu().numpy() - o_ref).max():.2e}")
    assert gate(part, ref_part) <= part.size // 300, gate(part, ref_part)
    assert np.abs(part - ref_part).max() < 4e-3
    o = out.cpu().numpy()
    assert gate(o, o_ref) <= o.size // 400, gate(o, o_ref)
    assert np.abs(o - o_ref).max() < 2.5e-3


def test_llama_shape_sampled(oracle):
    """32 query / 8 KV heads, head_dim 128, 4-bit keys and values, 16 sequences x 8192 tokens through
    shuffled block tables: the stored slots of sampled tokens and the decode output of sampled
    sequences against the oracle (both decode kernels)."""
    from fused_turboquant_b200 import tq_v1
    D, Hkv, G, kb, vb, bs, B, ctx = 128, 8, 4, 4, 4, 16, 16, 8192
    cfg = tq_v1.TurboQuantSlotConfig(D, kb, vb, norm_correction=True)
    slot = cfg.slot_size_aligned
    gen = torch.Generator(device="cuda").manual_seed(11)
    nblk = B * ctx // bs
    bt = torch.randperm(nblk, generator=gen, device="cuda").view(B, ctx // bs).to(torch.int32)
    pos = torch.arange(ctx, device="cuda")
    slots = (bt.long()[:, pos // bs] * bs + pos % bs).reshape(-1)
    K = torch.randn((B * ctx, Hkv, D), generator=gen, device="cuda").bfloat16()
    V = (torch.randn((B * ctx, Hkv, D), generator=gen, device="cuda") * 1.5 + 0.3).bfloat16()
    cent, mids = tq_v1.midpoints_of(torch.sort(torch.randn(16, generator=gen, device="cuda")).values / D ** 0.5)
    cache = torch.zeros((nblk, bs, Hkv, slot), dtype=torch.uint8, device="cuda")
    tq_v1.launch_store(K, V, cache, slots, mids, cfg)
    cache_np = cache.cpu().numpy()
    # stored bytes of 300 sampled tokens
    pick = torch.randperm(B * ctx, generator=gen, device="cuda")[:300].cpu().numpy()
    ref = np.zeros_like(cache_np)
    oracle.tq_store(K[pick].float().cpu().numpy(), V[pick].float().cpu().numpy(), ref, slots[pick].cpu().numpy(),
                    mids.cpu().numpy(), kb, vb)
    sl = slots[pick].cpu().numpy()
    np.testing.assert_array_equal(cache_np[sl // bs, sl % bs], ref[sl // bs, sl % bs])
    # decode of three sampled sequences, one of them cut short
    q = torch.randn((B, Hkv * G, D), generator=gen, device="cuda").bfloat16()
    seq = torch.full((B,), ctx, dtype=torch.int32, device="cuda")
    seq[5] = 4099
    sample = [0, 5, B - 1]
    o_ref, _, _ = oracle.tq_decode(q[sample].float().cpu().numpy(), cache_np, bt[sample].cpu().numpy(),
                                   seq[sample].cpu().numpy(), cent.cpu().numpy(), kb, vb, D ** -0.5, 4,
                                   norm_correction=True)
    for qq, tol in ((q, (2e-3, 1e-3)), (q.float(), (2e-4, 1e-4))):   # tensor-core / fp32 kernel
        out = tq_v1.decode_attention(qq, cache, bt, seq, cent, cfg, D ** -0.5, num_kv_splits=9,
                                     out_dtype=torch.float32)
        assert gate(out[sample].cpu().numpy(), o_ref, *tol) == 0


@pytest.mark.parametrize("qdtype", [torch.bfloat16, torch.float32])
def test_store_and_decode_are_graph_capturable(qdtype):
    """A decode step (store of the new token, attention with pre-allocated partials and output)
    replays from a CUDA graph with fresh inputs: no allocation and no host synchronisation
    inside the two calls -- what the reference needs from its per-layer buffers
    (vllm_plugin/v1_backend.py:1852-1866)."""
    from fused_turboquant_b200 import tq_v1
    dev = torch.device("cuda")
    B, Hkv, G, D, bs, splits = 4, 2, 4, 128, 16, 3
    cfg = tq_v1.TurboQuantSlotConfig(D, 4, 4, norm_correction=True)
    max_blocks = 20
    g = torch.Generator("cpu").manual_seed(9)
    bt = torch.randperm(B * max_blocks, generator=g).view(B, max_blocks).to(torch.int32).to(dev)
    cache = torch.zeros((B * max_blocks, bs, Hkv, cfg.slot_size_aligned), dtype=torch.uint8, device=dev)
    cent, mids = tq_v1.midpoints_of(torch.sort(torch.randn(16, generator=g)).values / D ** 0.5)
    ctx = 200
    kf = torch.randn(B * ctx, Hkv, D, generator=g).bfloat16().to(dev)
    slots = torch.cat([bt[b, torch.arange(ctx, device=dev) // bs].long() * bs +
                       torch.arange(ctx, device=dev) % bs for b in range(B)])
    tq_v1.launch_store(kf, kf, cache, slots, mids, cfg, v_rotate=True)
    k_new = torch.zeros(B, Hkv, D, dtype=torch.bfloat16, device=dev)
    v_new = torch.zeros_like(k_new)
    q = torch.zeros(B, Hkv * G, D, dtype=qdtype, device=dev)
    out = torch.zeros_like(q)
    mid_o = torch.zeros(B, Hkv * G, splits, D + 1, dtype=torch.float32, device=dev)
    lse = torch.zeros(B, Hkv * G, dtype=torch.float32, device=dev)
    slot_new = torch.zeros(B, dtype=torch.int64, device=dev)
    seq_lens = torch.zeros(B, dtype=torch.int32, device=dev)

    def step():
        tq_v1.launch_store(k_new, v_new, cache, slot_new, mids, cfg, v_rotate=True)
        tq_v1.decode_attention(q, cache, bt, seq_lens, cent, cfg, D ** -0.5, num_kv_splits=splits,
                               v_rotate=True, mid_o=mid_o, output=out, lse=lse)

    def set_inputs(pos, seed):
        gg = torch.Generator("cpu").manual_seed(seed)
        k_new.copy_(torch.randn(B, Hkv, D, generator=gg).bfloat16())
        v_new.copy_(torch.randn(B, Hkv, D, generator=gg).bfloat16())
        q.copy_(torch.randn(B, Hkv * G, D, generator=gg).to(qdtype))
        slot_new.copy_(bt[:, pos // bs].long() * bs + pos % bs)
        seq_lens.fill_(pos + 1)

    set_inputs(ctx, 1)
    step()                                   # warm-up outside the capture
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step()
    for i, pos in enumerate((ctx, ctx + 1, ctx + 2)):
        set_inputs(pos, 100 + i)
        graph.replay()
        got = out.clone()
        step()                               # same step, eagerly (the store rewrites the same slot)
        torch.cuda.synchronize()
        assert torch.equal(got, out), pos


@pytest.mark.parametrize("name", ["d128_k4v4", "d128_k8v4", "d64_k1v3"])
def test_cache_view_at_an_odd_halfword_offset(oracle, golden, name):
    """A cache that starts 2 bytes past a 4-byte boundary (a view into a larger buffer); the slots
    of the FP8-key case use a multiple of 4 bytes, the others 2 more."""
    from fused_turboquant_b200 import tq_v1
    g = golden("tq_v1.npz")
    D, Hkv, G, kb, vb, nc, splits, bs, slot, nb = _meta(g, name)
    cfg = tq_v1.TurboQuantSlotConfig(D, kb, vb, bool(nc))
    n = nb * bs * Hkv * slot
    buf = torch.zeros(n + 4, dtype=torch.uint8, device="cuda")
    cache = buf[2:2 + n].view(nb, bs, Hkv, slot)
    assert cache.data_ptr() % 4 == 2
    tq_v1.launch_store(cu(g[f"{name}_K"]), cu(g[f"{name}_V"]), cache, cu(g[f"{name}_slot_mapping"]),
                       g[f"{name}_midpoints"], cfg, D)
    aligned = torch.zeros((nb, bs, Hkv, slot), dtype=torch.uint8, device="cuda")
    tq_v1.launch_store(cu(g[f"{name}_K"]), cu(g[f"{name}_V"]), aligned, cu(g[f"{name}_slot_mapping"]),
                       g[f"{name}_midpoints"], cfg, D)
    assert torch.equal(cache, aligned)
    if name == "d128_k4v4":
        np.testing.assert_array_equal(cache.cpu().numpy(), g[f"{name}_cache"])
    assert int(buf[:2].sum()) == 0 and int(buf[2 + n:].sum()) == 0
    q = cu(g[f"{name}_q"]).bfloat16()
    args = (cu(g[f"{name}_block_table"]), cu(g[f"{name}_seq_lens"]), g[f"{name}_centroids"], cfg, D ** -0.5)
    out = tq_v1.decode_attention(q, cache, *args, num_kv_splits=splits, out_dtype=torch.float32)
    ref = tq_v1.decode_attention(q, aligned, *args, num_kv_splits=splits, out_dtype=torch.float32)
    # (the aligned copy runs the tensor-core kernel, the view the fp32 one)
    assert gate(out.cpu().numpy(), ref.cpu().numpy()) <= out.numel() // 300


@pytest.mark.parametrize("v_rotate", [False, True])
def test_prefix_hybrid_merge(oracle, golden, v_rotate):
    """Deferred-prefill hybrid: the first kv_start tokens are attended elsewhere (here: a dense
    fp32 softmax over random 'prefix' keys), the compressed rest by the decode kernel, and the two
    are merged by log-sum-exp inside the merge kernel.  One sequence has an empty compressed range,
    one an empty prefix (lse = -inf)."""
    from fused_turboquant_b200 import tq_v1
    g = golden("tq_v1.npz")
    name = "d128_k3v4_nc"
    D, Hkv, G, kb, vb, nc, splits, bs, slot, nb = _meta(g, name)
    cfg = tq_v1.TurboQuantSlotConfig(D, kb, vb, bool(nc))
    seq = g[f"{name}_seq_lens"]
    kv_start = np.array([int(seq[0]), 0], np.int32)        # sequence 0: nothing compressed is attended
    q = g[f"{name}_q"]
    B, Hq = q.shape[:2]
    rng = np.random.default_rng(5)
    out_p = rng.standard_normal((B, Hq, D)).astype(np.float32)
    lse_p = rng.standard_normal((B, Hq)).astype(np.float32) + 3.0
    lse_p[1, :3] = -np.inf                                  # no prefix for three heads of sequence 1
    out_p[1, :3] = 0.0
    lse = torch.empty((B, Hq), dtype=torch.float32, device="cuda")
    out = tq_v1.decode_attention(cu(q), cu(g[f"{name}_cache"]), cu(g[f"{name}_block_table"]), cu(seq),
                                 g[f"{name}_centroids"], cfg, D ** -0.5, num_kv_splits=splits,
                                 kv_start_offset=cu(kv_start), v_rotate=v_rotate, lse=lse,
                                 prefix_output=cu(out_p).bfloat16(), prefix_lse=cu(lse_p))
    o_ref, _, l_ref = oracle.tq_decode(q, g[f"{name}_cache"], g[f"{name}_block_table"], seq,
                                       g[f"{name}_centroids"], kb, vb, D ** -0.5, splits,
                                       norm_correction=bool(nc), kv_start=kv_start, rotate_out=v_rotate)
    o_ref[0], l_ref[0] = 0.0, -np.inf                       # (empty range: the oracle divides 0 / 0)
    out_p16 = torch.from_numpy(out_p).bfloat16().float().numpy()
    m_ref, ml_ref = oracle.tq_merge_prefix(o_ref, l_ref, out_p16, lse_p)
    np.testing.assert_allclose(out.cpu().numpy(), m_ref, rtol=2e-4, atol=2e-5)
    np.testing.assert_allclose(lse.cpu().numpy(), ml_ref, rtol=1e-5, atol=2e-5)
    np.testing.assert_allclose(out.cpu().numpy()[0], out_p16[0], rtol=1e-6, atol=1e-6)   # prefix only


def test_errors(golden):
    from fused_turboquant_b200 import tq_v1
    with pytest.raises(ValueError):
        tq_v1.TurboQuantSlotConfig(96, 4, 4)
    with pytest.raises(ValueError):
        tq_v1.TurboQuantSlotConfig(128, 5, 4)
    cfg = tq_v1.TurboQuantSlotConfig(128, 4, 4)
    assert (cfg.key_packed_size, cfg.value_packed_size, cfg.slot_size_aligned) == (66, 68, 134)
    k = torch.zeros((4, 2, 128), device="cuda")
    cache = torch.zeros((2, 16, 2, 100), dtype=torch.uint8, device="cuda")
    with pytest.raises(ValueError):
        tq_v1.launch_store(k, k, cache, torch.zeros(4, dtype=torch.int64), torch.linspace(-1, 1, 15), cfg)
    with pytest.raises(RuntimeError):
        tq_v1.launch_store(k.cpu(), k.cpu(), cache, torch.zeros(4, dtype=torch.int64), torch.linspace(-1, 1, 15), cfg)


@pytest.mark.parametrize("D,kb,vb,G,qdtype", [(128, 4, 4, 4, torch.bfloat16), (64, 3, 3, 7, torch.bfloat16),
                                               (128, 4, 4, 4, torch.float32), (256, 4, 2, 2, torch.bfloat16)])
def test_all_layers_in_one_call_equals_per_layer_calls(D, kb, vb, G, qdtype):
    """ftq_tq_decode_layers: the caches of L layers (one allocation, one block table) decoded in one
    call give, bit for bit, what L separate calls give; a block id outside the cache makes exactly
    the rows of its sequence NaN (the cache is a narrower view of its allocation, so nothing out
    of bounds is touched either way)."""
    from fused_turboquant_b200 import tq_v1
    L, B, Hkv, bs, splits = 3, 4, 2, 16, 4
    seq_lens = torch.tensor([200, 37, 512, 90], dtype=torch.int32, device="cuda")
    blocks_per_seq = 32
    nb = B * blocks_per_seq
    cfg = tq_v1.TurboQuantSlotConfig(D, kb, vb, norm_correction=True)
    g = torch.Generator(device="cuda").manual_seed(D + kb)
    big = torch.zeros((L, nb + 8, bs, Hkv, cfg.slot_size_aligned), dtype=torch.uint8, device="cuda")
    caches = big[:, :nb]                               # the kernels see nb blocks per layer
    bt = torch.randperm(nb, generator=g, device="cuda").view(B, blocks_per_seq).to(torch.int32)
    cent = torch.sort(torch.randn(1 << kb, generator=g, device="cuda") / D ** 0.5).values
    cent, mids = tq_v1.midpoints_of(cent)
    pos = torch.arange(512, device="cuda")
    slots = (bt.long()[:, pos // bs] * bs + pos % bs)
    slots = torch.where(pos[None, :] < seq_lens[:, None], slots, torch.full_like(slots, -1)).reshape(-1)
    for layer in range(L):
        k = torch.randn((B * 512, Hkv, D), generator=g, device="cuda").bfloat16()
        v = torch.randn((B * 512, Hkv, D), generator=g, device="cuda").bfloat16()
        tq_v1.launch_store(k, v, caches[layer], slots, mids, cfg)
    q = torch.randn((L, B, Hkv * G, D), generator=g, device="cuda").to(qdtype)
    lse = torch.empty((L, B, Hkv * G), dtype=torch.float32, device="cuda")
    one = tq_v1.decode_attention(q, caches, bt, seq_lens, cent, cfg, D ** -0.5, num_kv_splits=splits,
                                 lse=lse, out_dtype=torch.float32)
    assert one.shape == (L, B, Hkv * G, D) and torch.isfinite(one).all()
    for layer in range(L):
        lse1 = torch.empty((B, Hkv * G), dtype=torch.float32, device="cuda")
        per = tq_v1.decode_attention(q[layer], caches[layer], bt, seq_lens, cent, cfg, D ** -0.5,
                                     num_kv_splits=splits, lse=lse1, out_dtype=torch.float32)
        assert torch.equal(per, one[layer]) and torch.equal(lse1, lse[layer])
    bad = bt.clone()
    bad[2, 5] = nb + 3                                  # inside the allocation, outside the view
    got = tq_v1.decode_attention(q, caches, bad, seq_lens, cent, cfg, D ** -0.5, num_kv_splits=splits,
                                 out_dtype=torch.float32)
    assert torch.isnan(got[:, 2]).all()
    keep = [0, 1, 3]
    assert torch.equal(got[:, keep], one[:, keep])


@pytest.mark.parametrize("D,kb,vb,fp8", [(128, 4, 4, True), (64, 3, 3, True), (256, 8, 2, False), (128, 8, 8, True)])
def test_store_of_all_layers_in_one_call_equals_per_layer_calls(D, kb, vb, fp8):
    """[L, N, Hkv, D] keys / values into a [L, nb, bs, Hkv, slot] cache in one launch: the same bytes as
    one launch per layer (4-bit, 3-bit, 8-bit Lloyd-Max and FP8 keys)."""
    from fused_turboquant_b200 import tq_v1
    L, N, Hkv, bs, nb = 3, 150, 2, 16, 12
    cfg = tq_v1.TurboQuantSlotConfig(D, kb, vb, True, key_use_fp8_at_8bit=fp8)
    g = torch.Generator("cpu").manual_seed(D + kb)
    K = torch.randn(L, N, Hkv, D, generator=g).bfloat16().cuda()
    V = (torch.randn(L, N, Hkv, D, generator=g) * 1.3 - 0.2).bfloat16().cuda()
    n_cent = 256 if (kb == 8 and not fp8) else 1 << min(kb, 4)
    cent, mids = tq_v1.midpoints_of(torch.sort(torch.randn(n_cent, generator=g)).values / D ** 0.5)
    slots = torch.randperm(nb * bs, generator=g)[:N]
    slots[5] = -1
    one = torch.zeros((L, nb, bs, Hkv, cfg.slot_size_aligned), dtype=torch.uint8, device="cuda")
    tq_v1.launch_store(K, V, one, slots.cuda(), mids, cfg, v_rotate=vb != 8)
    per = torch.zeros_like(one)
    for l in range(L):
        tq_v1.launch_store(K[l], V[l], per[l], slots.cuda(), mids, cfg, v_rotate=vb != 8)
    assert torch.equal(one, per)
    assert one.any()


def test_store_skips_slots_beyond_the_cache():
    """A slot at or beyond num_blocks * block_size is dropped like a negative one.  The cache the
    call is given is a view of a larger allocation, so a missing guard would show as bytes
    written behind the view, not as an out-of-bounds write."""
    from fused_turboquant_b200 import tq_v1
    D, kb, vb, Hkv, bs, nb = 128, 4, 4, 2, 16, 6
    cfg = tq_v1.TurboQuantSlotConfig(D, kb, vb, True)
    g = torch.Generator("cpu").manual_seed(77)
    N = 40
    K = torch.randn(N, Hkv, D, generator=g).bfloat16().cuda()
    V = torch.randn(N, Hkv, D, generator=g).bfloat16().cuda()
    cent, mids = tq_v1.midpoints_of(torch.sort(torch.randn(16, generator=g)).values / D ** 0.5)
    big = torch.zeros((nb + 4, bs, Hkv, cfg.slot_size_aligned), dtype=torch.uint8, device="cuda")
    slots = torch.randperm(nb * bs, generator=g)[:N]
    good = big.clone()
    tq_v1.launch_store(K, V, good[:nb], slots.cuda(), mids, cfg)
    bad = slots.clone()
    bad[3] = nb * bs + 1            # inside `big`, outside the view the call is given
    bad[17] = (nb + 3) * bs + 15
    tq_v1.launch_store(K, V, big[:nb], bad.cuda(), mids, cfg)
    assert not big[nb:].any(), "the store wrote behind the cache it was given"
    want = good.clone()
    for tok in (3, 17):
        want[int(slots[tok]) // bs, int(slots[tok]) % bs] = 0
    assert torch.equal(big, want)
