// Split-KV decode attention over compressed K/V (fp32 arithmetic) + merge.
//
// One query token per sequence.  A CTA owns (sequence, KV head, KV chunk): it
// stages the chunk's pages into shared memory with cp.async (page ids come
// from the block table, or the pages are cut from contiguous tensors), scores
// every key in the ROTATED space against all query heads of the GQA group, so
// each packed byte is fetched once per KV head, runs an online softmax, and
// accumulates V in the rotated space.  The chunk's (max, sum, accumulator) go
// to a caller-provided workspace; the merge kernel combines the chunks and
// applies the inverse rotation once per (sequence, query head).
//
// Arithmetic follows the reference's fused formulation
// (src/fused_turboquant/kernels/triton_flash_decode.py:33-324):
//   score = knorm * scale * sum_d q_rot[d] * C_k[code_k[d]]
//   acc  += exp(score - m) * vnorm * C_v[code_v[:]]      (with the m rescale)
//   out   = inverse_rht(acc / l)
// and additionally fuses the query rotation (hf/fused_cache.py:579-581) and the
// page-table walk (vllm_plugin/cache_ops.py:151-205).
#pragma once

#include <math.h>

#include "ftq_common.cuh"

namespace ftq {

// How the tensor-core decode kernels cut the (layer, sequence, KV head) units into work items: up
// to three regions of consecutive units, each with its own chunk length -- few long chunks for
// the units that fill whole waves of the grid, shorter ones for the rest, sized so that the last
// wave has an item for every CTA (the longer ones first: the CTAs that arrive last get the short
// ones).  Items are numbered region by region: item = r.first_item + (unit - r.first_unit) *
// r.chunks + chunk.  A unit owns row_chunks chunk rows of the partials buffer whatever its region.
struct SplitRegion {
    int first_unit, first_item, chunks, chunk_tokens;
    FastDiv div_chunks;
};
struct SplitPlan {
    SplitRegion r[3];
    int n_regions, row_chunks, total_items;
};
__host__ __device__ __forceinline__ const SplitRegion& region_of_item(const SplitPlan& s, int item) {
    int k = 0;
    if (s.n_regions > 1 && item >= s.r[1].first_item) k = 1;
    if (s.n_regions > 2 && item >= s.r[2].first_item) k = 2;
    return s.r[k];
}
__host__ __device__ __forceinline__ const SplitRegion& region_of_unit(const SplitPlan& s, int unit) {
    int k = 0;
    if (s.n_regions > 1 && unit >= s.r[1].first_unit) k = 1;
    if (s.n_regions > 2 && unit >= s.r[2].first_unit) k = 2;
    return s.r[k];
}

struct AttnParams {
    const void* q;              // [L*B, Hq, D]
    // paged source
    const uint8_t* pool;        // [L][num_blocks, Hkv, page_bytes]
    int64_t pool_layer_stride;  // bytes
    const int32_t* block_table; // [B, max_blocks]
    int max_blocks;
    // contiguous source
    const uint8_t* k_codes;     // [B, Hkv, S, pdk]
    const uint16_t* k_norms;    // [B, Hkv, S]
    const uint8_t* v_codes;
    const uint16_t* v_norms;
    int S;
    const int32_t* seq_lens;    // [B] or nullptr
    int B, Hq, Hkv;
    float scale;
    int q_is_rotated;
    int q_dtype;                // kF32 / kF16 / kBF16
    int cp16;                   // contiguous source: every span 16-byte aligned
    int chunk_tokens, n_chunks, n_hpass;
    float* partials;            // [L*B*Hq][row_chunks][D + 4]
    // Tensor-core kernels: how the (layer, sequence, KV head) units are cut into work items (see
    // SplitPlan).  The fp32 kernels use one split for all units: n_chunks / chunk_tokens above.
    SplitPlan split;
    // Counters of the tensor-core path.  work_counter[0] = next work item.  The barrier-synchronised
    // kernel has the host zero it before the launch.  The streaming kernel clears its counters
    // itself: CTA 0 zeroes work_counter[0] (tickets), work_counter[1] (CTAs that have left) and
    // the unit counters, then stores `epoch` (unique per launch, never 0) into the 64-bit word at
    // work_counter + 2; everybody checks for it before the first atomic on a counter, and the
    // last CTA to leave stores 0 there, so that a replay of the same launch does not find its
    // own epoch.
    // work_counter[4] is the call's status word (kStatus* bits, cleared with the counters): what
    // the kernels of this call met; the host reads it on request (ftq_paged_decode_status).
    // nullptr for the contiguous entry points.
    int* work_counter;
    // streaming tensor-core kernel: it finishes the split-KV merge itself
    int* unit_counter;          // [n_units = L*B*Hkv] chunks delivered per unit
    int n_units;
    unsigned long long epoch;
    void* out;                  // [L*B, Hq, D]
    int out_dtype;
    int64_t num_blocks;         // block ids are checked against it
    FastDiv div_chunks, div_hkv, div_b;  // divisions by n_chunks, Hkv, B
    Codebook lk, lv;
    SignBits signs;
    float rsqrt_d;
    // tensor-core path: V centroids pre-multiplied by v_scale before the fp16 rounding
    // (lv_scaled), undone through the weights (inv_v_scale)
    Codebook lv_scaled;
    float inv_v_scale;
};

constexpr int kStatusWord = 4;         // index into AttnParams::work_counter
constexpr int kStatusBadBlock = 1;     // a block id outside [0, num_blocks) was met (its rows are NaN)
constexpr int kStatusWaitExpired = 2;  // a bounded wait of a kernel ran out (its rows are NaN)

__device__ __forceinline__ void cp_async_16(void* smem, const void* gmem, int src_bytes) {
    const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem),
                 "r"(src_bytes));
}
__device__ __forceinline__ void cp_async_4(void* smem, const void* gmem, int src_bytes) {
    const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;\n" ::"r"(s), "l"(gmem),
                 "r"(src_bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

// Copy `valid` of `total` bytes (both multiples of CP) into shared memory, zero-filling the rest.
template <int CP>
__device__ __forceinline__ void stage_span(uint8_t* dst, const uint8_t* src, int total, int valid,
                                           int tid, int nthreads) {
    for (int off = tid * CP; off < total; off += nthreads * CP) {
        int nb = valid - off;
        nb = nb < 0 ? 0 : (nb > CP ? CP : nb);
        // a zero-byte copy still needs a valid, aligned source address
        const uint8_t* s = nb > 0 ? src + off : src;
        if constexpr (CP == 16) cp_async_16(dst + off, s, nb);
        else cp_async_4(dst + off, s, nb);
    }
}

// A lane's slice of one packed vector: NB bytes starting at p (shared memory).
template <int NB>
__device__ __forceinline__ void load_code_bytes(const uint8_t* p, uint32_t (&w)[(NB + 3) / 4]) {
    if constexpr (NB == 16) {
        const uint4 v = *reinterpret_cast<const uint4*>(p);
        w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w;
    } else if constexpr (NB == 8) {
        const uint2 v = *reinterpret_cast<const uint2*>(p);
        w[0] = v.x; w[1] = v.y;
    } else if constexpr (NB % 4 == 0) {
#pragma unroll
        for (int i = 0; i < NB / 4; i++) w[i] = reinterpret_cast<const uint32_t*>(p)[i];
    } else if constexpr (NB == 6) {
        const uint16_t* h = reinterpret_cast<const uint16_t*>(p);
        w[0] = static_cast<uint32_t>(h[0]) | (static_cast<uint32_t>(h[1]) << 16);
        w[1] = h[2];
    } else if constexpr (NB == 3) {
        w[0] = static_cast<uint32_t>(p[0]) | (static_cast<uint32_t>(p[1]) << 8) |
               (static_cast<uint32_t>(p[2]) << 16);
    } else if constexpr (NB == 2) {
        w[0] = *reinterpret_cast<const uint16_t*>(p);
    } else {
        static_assert(NB == 1, "unsupported slice size");
        w[0] = p[0];
    }
}

// Code j of a little-endian stream of BITS-wide codes held in w[].
template <int BITS, int NWORDS>
__device__ __forceinline__ uint32_t extract_code(const uint32_t (&w)[NWORDS], int j) {
    const int off = j * BITS;
    const int lo = off >> 5, sh = off & 31;
    constexpr uint32_t mask = (1u << BITS) - 1u;
    if (sh + BITS <= 32) return (w[lo] >> sh) & mask;
    return __funnelshift_r(w[lo], w[lo + 1 < NWORDS ? lo + 1 : lo], sh) & mask;
}

constexpr int kTilePages = 4;
constexpr int kAttnThreads = 128;

template <int D>
struct AttnCfg {
    static constexpr int E = D / kOctet;
    static constexpr int GH = 64 / E;  // query heads per pass: 8 / 4 / 2 for D = 64 / 128 / 256
};

// PAGED: pages come from the pool through the block table; otherwise they are
// cut from contiguous [B,Hkv,S,*] tensors (cp.async granule 16 bytes when every
// span is 16-byte aligned, p.cp16, else 4).
template <int D, int BK, int BV, bool PAGED>
__global__ void __launch_bounds__(kAttnThreads)
attn_split_kernel(const AttnParams p) {
    constexpr int E = AttnCfg<D>::E;
    constexpr int GH = AttnCfg<D>::GH;
    constexpr int PDK = packed_dim(D, BK), PDV = packed_dim(D, BV);
    constexpr int NBK = PDK / kOctet, NBV = PDV / kOctet;  // bytes per lane per vector
    constexpr int OFF_KN = kPageTokens * PDK;
    constexpr int OFF_VC = OFF_KN + 2 * kPageTokens;
    constexpr int OFF_VN = OFF_VC + kPageTokens * PDV;
    constexpr int PAGE_BYTES = OFF_VN + 2 * kPageTokens;
    constexpr int TILE_BYTES = kTilePages * PAGE_BYTES;
    constexpr int ROW = D + 4;  // floats per partial row: acc[D], m, l, pad, pad

    // the tile ring doubles as the cross-warp merge area once the loop is over
    constexpr int MERGE_BYTES = 4 * GH * (D + 2) * 4;
    constexpr int RING_BYTES =
        ((2 * TILE_BYTES > MERGE_BYTES ? 2 * TILE_BYTES : MERGE_BYTES) + 15) / 16 * 16;

    extern __shared__ __align__(16) uint8_t smem_raw[];
    uint8_t* tiles = smem_raw;                                   // RING_BYTES
    float* qs = reinterpret_cast<float*>(smem_raw + RING_BYTES);      // [GH][D]
    float* lutk = qs + GH * D;
    float* lutv = lutk + kMaxLevels;

    const int tid = threadIdx.x;
    const int lane = tid & 31, warp = tid >> 5;
    const int t = lane & 7, o = lane >> 3;

    const int chunk = blockIdx.x;
    const int hkv = blockIdx.y / p.n_hpass;
    const int hp = blockIdx.y - hkv * p.n_hpass;
    const int lb = blockIdx.z;
    const int layer = lb / p.B;
    const int b = lb - layer * p.B;
    const int group = p.Hq / p.Hkv;
    const int h0 = hp * GH;
    const int nh = min(GH, group - h0);

    int seq_len = p.seq_lens ? p.seq_lens[b] : p.S;
    if (!PAGED) seq_len = min(seq_len, p.S);
    const int t0 = chunk * p.chunk_tokens;
    const int t1 = min(seq_len, t0 + p.chunk_tokens);
    float* prow = p.partials +
                  ((static_cast<int64_t>(lb) * p.Hq + hkv * group + h0) * p.n_chunks + chunk) * ROW;
    const int64_t prow_head_stride = static_cast<int64_t>(p.n_chunks) * ROW;
    if (t0 >= t1) {
        if (tid < nh) {
            prow[tid * prow_head_stride + D] = -INFINITY;
            prow[tid * prow_head_stride + D + 1] = 0.f;
        }
        return;
    }

    const uint8_t* pool = PAGED ? p.pool + layer * p.pool_layer_stride : nullptr;
    const int32_t* btab = PAGED ? p.block_table + static_cast<int64_t>(b) * p.max_blocks : nullptr;
    const int64_t cbase = (static_cast<int64_t>(b) * p.Hkv + hkv) * p.S;

    bool bad_block = false;  // (every thread walks the same block ids)
    auto issue_tile = [&](int ti, int buf) {
        uint8_t* dst = tiles + buf * TILE_BYTES;
#pragma unroll
        for (int pi = 0; pi < kTilePages; pi++) {
            const int ts = t0 + ti * (kTilePages * kPageTokens) + pi * kPageTokens;
            if (ts >= t1) break;
            uint8_t* pd = dst + pi * PAGE_BYTES;
            if constexpr (PAGED) {
                // a block id outside the pool is never dereferenced: block 0 stands in and the
                // chunk's result is replaced by NaN below
                int64_t blk = btab[ts / kPageTokens];
                if (static_cast<uint64_t>(blk) >= static_cast<uint64_t>(p.num_blocks)) {
                    blk = 0;
                    bad_block = true;
                }
                const uint8_t* src = pool + (blk * p.Hkv + hkv) * PAGE_BYTES;
                stage_span<16>(pd, src, PAGE_BYTES, PAGE_BYTES, tid, kAttnThreads);
            } else {
                const int ntok = min(kPageTokens, t1 - ts);
                if (p.cp16) {
                    stage_span<16>(pd, p.k_codes + (cbase + ts) * PDK, kPageTokens * PDK,
                                   ntok * PDK, tid, kAttnThreads);
                    stage_span<16>(pd + OFF_VC, p.v_codes + (cbase + ts) * PDV, kPageTokens * PDV,
                                   ntok * PDV, tid, kAttnThreads);
                } else {
                    stage_span<4>(pd, p.k_codes + (cbase + ts) * PDK, kPageTokens * PDK,
                                  ntok * PDK, tid, kAttnThreads);
                    stage_span<4>(pd + OFF_VC, p.v_codes + (cbase + ts) * PDV, kPageTokens * PDV,
                                  ntok * PDV, tid, kAttnThreads);
                }
                if (tid < 2 * kPageTokens) {
                    const int tk = tid & (kPageTokens - 1);
                    const bool isv = tid >= kPageTokens;
                    const uint16_t* nsrc = isv ? p.v_norms : p.k_norms;
                    const uint16_t val = tk < ntok ? nsrc[cbase + ts + tk] : uint16_t(0);
                    reinterpret_cast<uint16_t*>(pd + (isv ? OFF_VN : OFF_KN))[tk] = val;
                }
            }
        }
        cp_async_commit();
    };

    const int n_tiles = (t1 - t0 + kTilePages * kPageTokens - 1) / (kTilePages * kPageTokens);
    issue_tile(0, 0);

    // ---- prologue: tables and the rotated, pre-scaled queries of this pass
    if (tid < kMaxLevels) {
        lutk[tid] = p.lk.v[tid];
        lutv[tid] = p.lv.v[tid];
    }
    {
        const int hh = warp * 4 + o;  // one octet rotates one query head (GH <= 8 < 16 octets)
        const bool hv = hh < nh;
        const int64_t qoff =
            (static_cast<int64_t>(lb) * p.Hq + hkv * group + h0 + (hv ? hh : 0)) * D;
        float a[E];
#pragma unroll
        for (int i = 0; i < E / 8; i++) {
            float tmp[8];
            const int64_t eo = qoff + 8 * (t + 8 * i);
            if (p.q_dtype == kF32) load8<float>(static_cast<const float*>(p.q) + eo, tmp);
            else if (p.q_dtype == kBF16)
                load8<__nv_bfloat16>(static_cast<const __nv_bfloat16*>(p.q) + eo, tmp);
            else load8<__half>(static_cast<const __half*>(p.q) + eo, tmp);
#pragma unroll
            for (int c = 0; c < 8; c++) {
                const uint32_t m = p.q_is_rotated ? 0u : sign_mask(p.signs, load_coord(t, 8 * i + c));
                a[8 * i + c] = __uint_as_float(__float_as_uint(tmp[c]) ^ m);
            }
        }
        if (p.q_is_rotated) {
            if (hh < GH) {
#pragma unroll
                for (int r = 0; r < E; r++)
                    qs[hh * D + load_coord(t, r)] = hv ? a[r] * p.scale : 0.f;
            }
        } else {
            octet_fwht<E>(a, lane);
            if (hh < GH) {
#pragma unroll
                for (int k = 0; k < E; k++)
                    qs[hh * D + t + 8 * k] = hv ? a[k] * p.rsqrt_d * p.scale : 0.f;
            }
        }
    }
    __syncthreads();

    float qr[GH][E];
#pragma unroll
    for (int h = 0; h < GH; h++)
#pragma unroll
        for (int r = 0; r < E; r++) qr[h][r] = qs[h * D + t * E + r];

    float m_run[GH], l_run[GH], acc[GH][E];
#pragma unroll
    for (int h = 0; h < GH; h++) {
        m_run[h] = -INFINITY;
        l_run[h] = 0.f;
#pragma unroll
        for (int r = 0; r < E; r++) acc[h][r] = 0.f;
    }

    // ---- main loop over 64-token tiles, double buffered
    for (int ti = 0; ti < n_tiles; ti++) {
        if (ti + 1 < n_tiles) {
            issue_tile(ti + 1, (ti + 1) & 1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();

        const int ts = t0 + ti * (kTilePages * kPageTokens) + warp * kPageTokens;
        if (ts < t1) {  // warp-uniform
            const int ntok = min(kPageTokens, t1 - ts);
            const uint8_t* page = tiles + (ti & 1) * TILE_BYTES + warp * PAGE_BYTES;

            float sc[4][GH];
#pragma unroll
            for (int step = 0; step < 4; step++) {
                const int tk = step * 4 + o;
                uint32_t w[(NBK + 3) / 4];
                load_code_bytes<NBK>(page + tk * PDK + t * NBK, w);
                const float kn =
                    __half2float(reinterpret_cast<const __half*>(page + OFF_KN)[tk]);
                float kv[E];
#pragma unroll
                for (int r = 0; r < E; r++) kv[r] = lutk[extract_code<BK>(w, r)];
#pragma unroll
                for (int h = 0; h < GH; h++) {
                    float d = 0.f;
#pragma unroll
                    for (int r = 0; r < E; r++) d = fmaf(qr[h][r], kv[r], d);
                    d += __shfl_xor_sync(0xffffffffu, d, 1);
                    d += __shfl_xor_sync(0xffffffffu, d, 2);
                    d += __shfl_xor_sync(0xffffffffu, d, 4);
                    sc[step][h] = tk < ntok ? d * kn : -INFINITY;
                }
            }

            float wp[4][GH];
#pragma unroll
            for (int h = 0; h < GH; h++) {
                float mx = fmaxf(fmaxf(sc[0][h], sc[1][h]), fmaxf(sc[2][h], sc[3][h]));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
                const float m_new = fmaxf(m_run[h], mx);  // finite: token 0 of the page is valid
                const float corr = m_run[h] == -INFINITY ? 0.f : __expf(m_run[h] - m_new);
                m_run[h] = m_new;
                float ls = 0.f;
#pragma unroll
                for (int step = 0; step < 4; step++) {
                    const float pe = sc[step][h] == -INFINITY ? 0.f : __expf(sc[step][h] - m_new);
                    ls += pe;
                    wp[step][h] = pe;
                }
                l_run[h] = l_run[h] * corr + ls;
#pragma unroll
                for (int r = 0; r < E; r++) acc[h][r] *= corr;
            }

#pragma unroll
            for (int step = 0; step < 4; step++) {
                const int tk = step * 4 + o;
                uint32_t w[(NBV + 3) / 4];
                // pool pages store a V row with its halves exchanged for tokens with bit 1 set
                const int vt = PAGED ? (t ^ ((tk & 2) << 1)) : t;
                load_code_bytes<NBV>(page + OFF_VC + tk * PDV + vt * NBV, w);
                const float vn = tk < ntok
                    ? __half2float(reinterpret_cast<const __half*>(page + OFF_VN)[tk]) : 0.f;
                float vv[E];
#pragma unroll
                for (int r = 0; r < E; r++) vv[r] = lutv[extract_code<BV>(w, r)];
#pragma unroll
                for (int h = 0; h < GH; h++) {
                    const float wgt = tk < ntok ? wp[step][h] * vn : 0.f;
#pragma unroll
                    for (int r = 0; r < E; r++) acc[h][r] = fmaf(wgt, vv[r], acc[h][r]);
                }
            }
        }
        __syncthreads();
    }

    // ---- combine the 4 octets of each warp, then the 4 warps through shared memory
#pragma unroll
    for (int h = 0; h < GH; h++) {
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 8);
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 16);
#pragma unroll
        for (int r = 0; r < E; r++) {
            acc[h][r] += __shfl_xor_sync(0xffffffffu, acc[h][r], 8);
            acc[h][r] += __shfl_xor_sync(0xffffffffu, acc[h][r], 16);
        }
    }
    float* wacc = reinterpret_cast<float*>(tiles);   // [4][GH][D]   (tiles are free now)
    float* wm = wacc + 4 * GH * D;                   // [4][GH]
    float* wl = wm + 4 * GH;                         // [4][GH]
    if (o == 0) {
#pragma unroll
        for (int h = 0; h < GH; h++) {
#pragma unroll
            for (int r = 0; r < E; r++) wacc[(warp * GH + h) * D + t * E + r] = acc[h][r];
            if (t == 0) {
                wm[warp * GH + h] = m_run[h];
                wl[warp * GH + h] = l_run[h];
            }
        }
    }
    __syncthreads();
    for (int idx = tid; idx < nh * D; idx += kAttnThreads) {
        const int h = idx / D, d = idx - h * D;
        float M = -INFINITY;
#pragma unroll
        for (int w2 = 0; w2 < 4; w2++) M = fmaxf(M, wm[w2 * GH + h]);
        float a = 0.f, l = 0.f;
#pragma unroll
        for (int w2 = 0; w2 < 4; w2++) {
            const float mw = wm[w2 * GH + h];
            if (mw != -INFINITY) {
                const float f = __expf(mw - M);
                a = fmaf(wacc[(w2 * GH + h) * D + d], f, a);
                l = fmaf(wl[w2 * GH + h], f, l);
            }
        }
        prow[h * prow_head_stride + d] = a;
        if (d == 0) {
            if (bad_block) {
                M = __int_as_float(0x7fc00000);
                if (h == 0 && p.work_counter) atomicOr(p.work_counter + kStatusWord, kStatusBadBlock);
            }
            prow[h * prow_head_stride + D] = M;
            prow[h * prow_head_stride + D + 1] = l;
        }
    }
}

// Merge the chunk partials of one (layer, sequence, query head), normalise,
// rotate back to the original space (inverse_randomized_hadamard,
// core/hadamard.py:93-100) and store.  One octet per output vector.
template <int D, typename OT>
__global__ void __launch_bounds__(128)
attn_merge_kernel(const float* __restrict__ partials, OT* __restrict__ out,
                  const int32_t* __restrict__ seq_lens, int S, int B, int Hq, int n_chunks,
                  int chunk_tokens, int64_t n_vec, SignBits signs, float rsqrt_d, int Hkv,
                  const SplitPlan split) {
    constexpr int E = D / kOctet;
    constexpr int ROW = D + 4;
    const int lane = threadIdx.x & 31;
    const int t = lane & 7;
    const int64_t v = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 3;
    const bool valid = v < n_vec;
    int nc = 0;
    if (valid) {
        const int b = static_cast<int>((v / Hq) % B);
        const int len = seq_lens ? (S > 0 ? min(seq_lens[b], S) : seq_lens[b]) : S;
        // the unit's region tells how many chunks it was cut into (split.n_regions == 0: one
        // split for all units, n_chunks / chunk_tokens)
        int ncr = n_chunks, ct = chunk_tokens;
        if (split.n_regions > 0) {
            const int unit = static_cast<int>((v / Hq) * Hkv + (v % Hq) / (Hq / Hkv));
            const SplitRegion& rg = region_of_unit(split, unit);
            ncr = rg.chunks;
            ct = rg.chunk_tokens;
        }
        nc = min(ncr, (len + ct - 1) / ct);
    }
    const float* rows =
        partials + (valid ? v : 0) * (split.n_regions > 0 ? split.row_chunks : n_chunks) * ROW;
    float M = -INFINITY;
    for (int c = 0; c < nc; c++) M = fmaxf(M, rows[c * ROW + D]);
    float a[E];
#pragma unroll
    for (int r = 0; r < E; r++) a[r] = 0.f;
    float L = 0.f;
    for (int c = 0; c < nc; c++) {
        const float mc = rows[c * ROW + D];
        if (mc == -INFINITY) continue;
        const float f = __expf(mc - M);
        L = fmaf(rows[c * ROW + D + 1], f, L);
#pragma unroll
        for (int i = 0; i < E / 8; i++) {
            float tmp[8];
            load8<float>(rows + c * ROW + 8 * (t + 8 * i), tmp);
#pragma unroll
            for (int cc = 0; cc < 8; cc++) a[8 * i + cc] = fmaf(tmp[cc], f, a[8 * i + cc]);
        }
    }
    const float inv = L > 0.f ? 1.f / L : 0.f;
#pragma unroll
    for (int r = 0; r < E; r++) a[r] *= inv;
    octet_fwht<E>(a, lane);
    if (valid) {
#pragma unroll
        for (int k = 0; k < E; k++) {
            const float r = a[k] * rsqrt_d;
            out[v * D + t + 8 * k] =
                from_float<OT>(__uint_as_float(__float_as_uint(r) ^ sign_mask(signs, t + 8 * k)));
        }
    }
}

}  // namespace ftq
