"""numpy helpers shared by the tests: the page layout restated on the host, input generators."""
import numpy as np

PAGE = 16


def pd(d, bits):
    return d * bits // 8


def page_offsets(d, bk, bv):
    off_kn = PAGE * pd(d, bk)
    off_vc = off_kn + 2 * PAGE
    off_vn = off_vc + PAGE * pd(d, bv)
    return off_kn, off_vc, off_vn, off_vn + 2 * PAGE


def v_row(row, t):
    """V rows are stored with their halves exchanged for page tokens with bit 1 set."""
    if t & 2:
        h = row.shape[-1] // 2
        return np.concatenate([row[..., h:], row[..., :h]], axis=-1)
    return row


def pool_from_contiguous(k_idx, k_norms, v_idx, v_norms, block_table, num_blocks, d, bk, bv,
                         seq_lens=None, base=None):
    """Lay contiguous [B,Hkv,S,*] codes / fp16 norms out as pool u8 [num_blocks, Hkv, page_bytes].
    Slots of tokens beyond seq_len keep the bytes of `base` (zeros when None)."""
    B, Hkv, S, _ = k_idx.shape
    off_kn, off_vc, off_vn, pbytes = page_offsets(d, bk, bv)
    pool = np.zeros((num_blocks, Hkv, pbytes), np.uint8) if base is None else base.copy()
    kn = np.ascontiguousarray(k_norms, np.float16).view(np.uint16)
    vn = np.ascontiguousarray(v_norms, np.float16).view(np.uint16)
    for b in range(B):
        n = S if seq_lens is None else int(seq_lens[b])
        for s in range(n):
            blk, t = int(block_table[b, s // PAGE]), s % PAGE
            for h in range(Hkv):
                page = pool[blk, h]
                page[t * pd(d, bk):(t + 1) * pd(d, bk)] = k_idx[b, h, s]
                page[off_kn + 2 * t:off_kn + 2 * t + 2] = np.frombuffer(kn[b, h, s].tobytes(), np.uint8)
                page[off_vc + t * pd(d, bv):off_vc + (t + 1) * pd(d, bv)] = v_row(v_idx[b, h, s], t)
                page[off_vn + 2 * t:off_vn + 2 * t + 2] = np.frombuffer(vn[b, h, s].tobytes(), np.uint8)
    return pool


def contiguous_from_pool(pool, block_table, seq_lens, S, d, bk, bv):
    """Inverse of pool_from_contiguous (positions >= seq_len stay zero)."""
    B = block_table.shape[0]
    Hkv = pool.shape[1]
    off_kn, off_vc, off_vn, _ = page_offsets(d, bk, bv)
    k_idx = np.zeros((B, Hkv, S, pd(d, bk)), np.uint8)
    v_idx = np.zeros((B, Hkv, S, pd(d, bv)), np.uint8)
    k_n = np.zeros((B, Hkv, S), np.uint16)
    v_n = np.zeros((B, Hkv, S), np.uint16)
    for b in range(B):
        for s in range(int(seq_lens[b])):
            blk, t = int(block_table[b, s // PAGE]), s % PAGE
            for h in range(Hkv):
                page = pool[blk, h]
                k_idx[b, h, s] = page[t * pd(d, bk):(t + 1) * pd(d, bk)]
                v_idx[b, h, s] = v_row(page[off_vc + t * pd(d, bv):off_vc + (t + 1) * pd(d, bv)], t)
                k_n[b, h, s] = page[off_kn + 2 * t:off_kn + 2 * t + 2].view(np.uint16)[0]
                v_n[b, h, s] = page[off_vn + 2 * t:off_vn + 2 * t + 2].view(np.uint16)[0]
    return k_idx, k_n.view(np.float16), v_idx, v_n.view(np.float16)


def shuffled_block_table(rng, B, max_blocks, num_blocks):
    perm = rng.permutation(num_blocks)[:B * max_blocks]
    return perm.reshape(B, max_blocks).astype(np.int32)


def boundary_exempt(normalized, boundaries, tol=1e-6):
    """Mask of coordinates whose normalised rotated value lies within tol of a decision boundary."""
    dist = np.abs(normalized[..., None] - np.asarray(boundaries, np.float32)[None, :]).min(-1)
    return dist <= tol


def gate(out, ref, rtol=2e-3, atol=1e-3):
    """Number of elements violating |out - ref| <= atol + rtol * |ref|."""
    out = np.asarray(out, np.float64)
    ref = np.asarray(ref, np.float64)
    return int((np.abs(out - ref) > atol + rtol * np.abs(ref)).sum())


def tq_v1_compare_cache(cache, ref, slot_mapping, y, midpoints, d, key_bits, value_bits, block_size,
                        vy=None):
    """Compare two kv caches in the vLLM-v1 slot format ([nb, block_size, Hkv, slot] uint8).

    Returns counts: value-region bytes that differ, bytes that differ outside written slots, key
    codes that differ although the rotated value `y` ([n_tokens, Hkv, d]) is farther than 1e-6
    from every midpoint, and the largest key-norm distance in fp16 ulps.  With `vy` (the unit
    values of a Lloyd-Max value cache, 4-bit codes) the value codes and the value norm are compared
    the same way (`value_codes_differ_off_midpoint`, `value_norm_max_ulp`) and `value_bytes_differ`
    counts the zero-point field only.  `key_bits == 8` means FP8 (e4m3) keys: `y` must then be the
    un-normalised rotated key the store casts.  Triton's interpreter -- the fixtures' source --
    emulates the fp32 -> e4m3 cast unfaithfully in three situations, which a GPU's conversion
    instruction (round to nearest even; what the oracle and the CUDA store do) does not share:
    it truncates in e4m3's subnormal range (|x| < 2^-6), rounds ties away from zero, and loses the
    carry when the mantissa rounds up to the next power of two (1.95 becomes 1.0 instead of 2.0).
    `key_fp8_differ_unexplained` counts key bytes that differ outside those three situations;
    `key_fp8_vs_rne` counts bytes of `cache` that differ from torch's round-to-nearest-even cast
    of `y` although `y` is farther than 1e-6 (relative) from the tie between the two candidates.
    """
    key_mse8 = key_bits == 264          # 8-bit Lloyd-Max codes: one byte per coordinate + norm
    if key_mse8:
        key_bits = 8
    key_fp8 = key_bits == 8 and not key_mse8
    mse = d * key_bits // 8
    kps = mse + (0 if key_fp8 else 2)
    vdb = d if value_bits == 8 else d * value_bits // 8
    used = kps + vdb + 4
    hkv = cache.shape[2]
    written = np.zeros(cache.shape[:3], bool)
    stats = dict(value_bytes_differ=0, other_bytes_differ=0, key_codes_differ_off_midpoint=0,
                 key_codes_differ=0, key_norm_max_ulp=0, value_codes_differ_off_midpoint=0,
                 value_norm_max_ulp=0, key_fp8_differ=0, key_fp8_differ_unexplained=0,
                 key_fp8_vs_rne=0)
    mids = np.asarray(midpoints, np.float32)
    for tok, slot in enumerate(np.asarray(slot_mapping)):
        if slot < 0:
            continue
        blk, off = int(slot) // block_size, int(slot) % block_size
        written[blk, off, :] = True
        for h in range(hkv):
            a, b = cache[blk, off, h], ref[blk, off, h]
            if vy is None:
                stats["value_bytes_differ"] += int((a[kps:used] != b[kps:used]).sum())
            else:
                stats["value_bytes_differ"] += int((a[used - 2:used] != b[used - 2:used]).sum())
                va = int(a[kps + vdb]) | (int(a[kps + vdb + 1]) << 8)
                vb_ = int(b[kps + vdb]) | (int(b[kps + vdb + 1]) << 8)
                stats["value_norm_max_ulp"] = max(stats["value_norm_max_ulp"], abs(va - vb_))
                ca = np.unpackbits(a[kps:kps + vdb], bitorder="little").reshape(d, 4)
                cb = np.unpackbits(b[kps:kps + vdb], bitorder="little").reshape(d, 4)
                vdiff = (ca != cb).any(axis=1)
                vnear = np.abs(vy[tok, h][:, None] - mids[None, :]).min(axis=1) < 1e-6
                stats["value_codes_differ_off_midpoint"] += int((vdiff & ~vnear).sum())
            stats["other_bytes_differ"] += int((a[used:] != b[used:]).sum())
            if key_fp8:
                import torch
                f8 = lambda u: torch.from_numpy(u.copy()).view(torch.float8_e4m3fn).float().numpy().astype(np.float64)
                val = y[tok, h].astype(np.float64)
                fa = f8(a[:mse])
                near_tie = lambda fo: np.abs(val - (fa + fo) / 2) <= 1e-6 * np.abs(val)
                diff = a[:mse] != b[:mse]
                if diff.any():
                    small = np.abs(val) < 2.0 ** -6
                    carry = ((a[:mse] & 7) == 0) & (a[:mse].astype(np.int32) - b[:mse] == 8)
                    stats["key_fp8_differ"] += int(diff.sum())
                    stats["key_fp8_differ_unexplained"] += int(
                        (diff & ~near_tie(f8(b[:mse])) & ~small & ~carry).sum())
                rne = torch.from_numpy(y[tok, h].copy()).clamp(-448, 448).to(torch.float8_e4m3fn) \
                    .view(torch.uint8).numpy()
                d2 = a[:mse] != rne
                if d2.any():
                    stats["key_fp8_vs_rne"] += int((d2 & ~near_tie(f8(rne))).sum())
                continue
            na = int(a[mse]) | (int(a[mse + 1]) << 8)
            nb_ = int(b[mse]) | (int(b[mse + 1]) << 8)
            stats["key_norm_max_ulp"] = max(stats["key_norm_max_ulp"], abs(na - nb_))
            if (a[:mse] != b[:mse]).any():
                bits = np.unpackbits(a[:mse], bitorder="little").reshape(d, key_bits)
                bits_r = np.unpackbits(b[:mse], bitorder="little").reshape(d, key_bits)
                diff = (bits != bits_r).any(axis=1)
                stats["key_codes_differ"] += int(diff.sum())
                near = np.abs(y[tok, h][:, None] - mids[None, :]).min(axis=1) < 1e-6
                stats["key_codes_differ_off_midpoint"] += int((diff & ~near).sum())
    stats["other_bytes_differ"] += int((cache[~written] != ref[~written]).sum())
    return stats
