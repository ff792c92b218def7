// vLLM-v1 slot format, decode stage 1 on the tensor cores.
//
// Same result as tq_split_kernel (ftq_tq_v1.cuh) -- the reference's
// `_tq_decode_stage1_offset` (src/fused_turboquant/vllm_plugin/triton_decode_offset.py:42-444)
// for all query heads of a GQA group at once, partials in the reference's
// [B, Hq, splits, D+1] layout -- with the structure of the page-layout kernel
// (ftq_attn_mma.cuh): persistent CTAs loop over (split, KV head, sequence) items, every warp
// walks 16-token pages with its own online-softmax state, `S = K.Q^T` and `O^T = V^T.P^T` run
// on m16n8k16 fp16 MMAs (fp32 accumulate) with the query heads as the N dimension.
//
// What differs from the page-layout kernel:
//  * Pages do not exist in this cache: the 16 slots of a page are token-major, 134-byte-ish
//    records that start on 2-byte boundaries, so no bulk copy can fetch them.  A warp copies
//    the 16 slots of its next page as they are -- aligned 32-bit words, consecutive lanes on
//    consecutive words of a slot -- into registers one page ahead and from there into 16 rows of
//    its page buffer; the fragment loads shift by a row's start offset (0 or 2 bytes).
//  * Values are uniform codes: value = code * scale + zero.  The value table returns the (centred)
//    fp16 integers of a byte's (or index's) two codes, the per-token scale is folded into the softmax
//    weight and sum(p * zero) is one more scalar accumulator per head (added to every
//    coordinate of the output at the end).
//  * Norm correction (re-normalising a key's centroid vector to unit length) needs
//    sum_d c[code]^2 per token: two extra MMAs per k-block multiply the key tile with itself
//    (its own fragments are valid B operands); the diagonal holds the sums in fp32.
//
// Centroids, integer codes, queries and weights are fp16 operands; everything else is fp32.
#pragma once

#include "ftq_attn_mma.cuh"
#include "ftq_tq_v1.cuh"

namespace ftq {

template <int D, int KB, int VB, int NH>
struct TqMmaCfg {
    static_assert(VB != 8, "8-bit values take the fp32 kernel");
    static constexpr int NKB = D / 16, NMT = D / 32;
    static constexpr int PDK = D * KB / 8, PDV = D * VB / 8;
    static constexpr int KSB = PDK / 4, VSB = PDV / 8;  // slice bytes per lane
    static constexpr int IWK = 2 * KB, IWV = 2 * VB;
    static constexpr bool BYTE = KB == 4 || VB == 4;
    static constexpr int WARPS = BYTE ? 16 : 8;
    static constexpr int THREADS = 32 * WARPS;
    static constexpr int CTAS_PER_SM = BYTE ? 1 : 2;
    // Page buffer of a warp: 16 rows, row t = the aligned 32-bit words that cover token t's slot
    // (the slot itself starts at byte 0 or 2 of the row), then the 16 alignment bits and the 16
    // slot addresses the copy loop reads.
    static constexpr int USED = PDK + 2 + PDV + 4;             // bytes of a slot that carry data
    static constexpr int NWR = (USED + 2) / 4;                 // words per row (USED = 2 mod 4)
    static constexpr int ROWB = (4 * NWR + 15) / 16 * 16;
    static constexpr int OFF_MIS = kPageTokens * ROWB;         // u32: bit t = slot t starts 2 bytes in
    static constexpr int OFF_AL = OFF_MIS + 16;                // u64[16]: aligned slot addresses | mis
    static constexpr int PAGE_BYTES = OFF_AL + kPageTokens * 8 + 16;
    static constexpr int NCOPY = (kPageTokens * NWR + 31) / 32;  // words per lane and page
    static constexpr int TKS = KB == 4 ? 0 : (1 << IWK) * 128;
    static constexpr int TVS = VB == 4 ? 0 : (1 << IWV) * 128;
    static constexpr int SMALL_ALIGN = TKS > TVS ? TKS : TVS;
    static constexpr int SMALL_BYTES = TKS + TVS + SMALL_ALIGN;
    static constexpr int STATE_F4 = NH * NMT;
    static constexpr int XCHG_BYTES = WARPS * (32 * STATE_F4 * 16 + NH * 3 * 4 * 4);
    static constexpr int BUF_BYTES =
        (WARPS * PAGE_BYTES > XCHG_BYTES ? WARPS * PAGE_BYTES : XCHG_BYTES) + 16;
    static constexpr int QS_BYTES = 8 * (D + 16) * 4;
    // [slack up to the 64 KB boundary][64 KB byte table][small tables | queries | buffers]
    static constexpr int REST_BYTES = SMALL_BYTES + QS_BYTES + BUF_BYTES + 64;
    static constexpr int SMEM_BYTES = (BYTE ? 2 * 65536 : 0) + REST_BYTES;
};

template <int D, int KB, int VB, int NH>
__global__ void __launch_bounds__(TqMmaCfg<D, KB, VB, NH>::THREADS, TqMmaCfg<D, KB, VB, NH>::CTAS_PER_SM)
tq_mma_kernel(const TqDecodeParams p, int n_items) {
    using C = TqMmaCfg<D, KB, VB, NH>;
    constexpr int NKB = C::NKB, NMT = C::NMT, WARPS = C::WARPS, THREADS = C::THREADS;
    constexpr int E = D / kOctet;
    constexpr int PDK = C::PDK, PDV = C::PDV;
    using Regs = PageRegs<C::KSB, C::VSB>;

    extern __shared__ __align__(16) uint8_t smem_raw[];
    const uint32_t sbase = static_cast<uint32_t>(__cvta_generic_to_shared(smem_raw));
    uint32_t window = 0, rest = sbase;
    if constexpr (C::BYTE) {
        window = (sbase + 65535u) & ~65535u;
        rest = window + 65536u;
    }
    auto gptr = [&](uint32_t saddr) { return smem_raw + (saddr - sbase); };
    uint32_t tk_small = 0, tv_small = 0, cur = rest;
    if constexpr (C::SMALL_ALIGN > 0) {
        cur = (rest + C::SMALL_ALIGN - 1) & ~static_cast<uint32_t>(C::SMALL_ALIGN - 1);
        if (C::TKS >= C::TVS) { tk_small = cur; tv_small = cur + C::TKS; }
        else { tv_small = cur; tk_small = cur + C::TVS; }
        cur += C::TKS + C::TVS;
    }
    cur = (cur + 15u) & ~15u;
    float* qs = reinterpret_cast<float*>(gptr(cur));            // [8][D + 16]
    const uint32_t bufs = (cur + C::QS_BYTES + 15u) & ~15u;     // page buffers / merge exchange area
    float4* xchg = reinterpret_cast<float4*>(gptr(bufs));       // [WARPS][NH][NMT][32]
    float* xml = reinterpret_cast<float*>(gptr(bufs + WARPS * 32 * C::STATE_F4 * 16));  // [WARPS][NH][3][4]

    const int tid = threadIdx.x;
    const int lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, tg = lane & 3;
    const bool odd = g & 1;
    const int group = p.Hq / p.Hkv;  // <= 4 * NH
    const uint32_t sel_plo = odd ? 0x1044u : 0x4410u;
    const uint32_t sel_phi = odd ? 0x3244u : 0x4432u;

    // ---- once per CTA: key centroid table and the table of value codes.  The codes are centred
    // (code - (2^VB - 1) / 2, exact in fp16) and the zero point moved accordingly: the weighted sums
    // of `code * scale` and of `zero` would otherwise be two large numbers of opposite sign, and
    // the fp16 rounding of the weights would be paid on their magnitude instead of the value's
    // (4-bit codes are centred on 8, not 7.5: the arithmetic dequantisation subtracts 1024 + centre
    // in fp16, where only integers exist at that magnitude)
    constexpr float kCtr = VB == 4 ? 8.f : 0.5f * ((1 << VB) - 1);
    if constexpr (C::BYTE) {
        uint32_t* tb = reinterpret_cast<uint32_t*>(gptr(window));
        for (int i = tid; i < 256 * 64; i += THREADS) {
            const int e = i >> 6, col = i & 63;
            if (col < 32) {
                if constexpr (KB == 4) {
                    const __half2 h = __floats2half2_rn(p.centroids.v[e & 15], p.centroids.v[e >> 4]);
                    tb[i] = *reinterpret_cast<const uint32_t*>(&h);
                }
            }
            // (columns 32..63 of a row are free: 4-bit value codes are dequantised arithmetically)
        }
    }
    if constexpr (KB != 4) {
        uint32_t* t = reinterpret_cast<uint32_t*>(gptr(tk_small));
        for (int i = tid; i < (1 << C::IWK) * 32; i += THREADS) {
            const int e = i >> 5;
            const __half2 h = __floats2half2_rn(p.centroids.v[e & ((1 << KB) - 1)], p.centroids.v[e >> KB]);
            t[i] = *reinterpret_cast<const uint32_t*>(&h);
        }
    }
    if constexpr (VB != 4) {
        uint32_t* t = reinterpret_cast<uint32_t*>(gptr(tv_small));
        for (int i = tid; i < (1 << C::IWV) * 32; i += THREADS) {
            const int e = i >> 5;
            const __half2 h = __floats2half2_rn(static_cast<float>(e & ((1 << VB) - 1)) - kCtr,
                                                static_cast<float>(e >> VB) - kCtr);
            t[i] = *reinterpret_cast<const uint32_t*>(&h);
        }
    }
    const uint32_t lk_lane = (KB == 4 ? window : tk_small) | (lane * 4);
    const uint32_t lv_lane = (VB == 4 ? (window | 128u) : tv_small) | (lane * 4);
    __syncthreads();

    auto qs_index = [](int head, int coord) {
        return head * (D + 16) + (coord / (D / 4)) * (D / 4 + 4) + coord % (D / 4);
    };
    struct Item { int sid, hkv, b, bs, layer, t0, t1, n_pages; };
    auto item_info = [&](int item) {
        Item it;
        it.sid = item % p.splits;
        const int r = item / p.splits;
        it.hkv = r % p.Hkv;
        it.b = r / p.Hkv;   // (layer, sequence) row
        it.layer = static_cast<int>(fast_div(static_cast<uint32_t>(it.b), p.div_bseq));
        it.bs = it.b - it.layer * p.B_seq;
        const int seq_len = p.seq_lens[it.bs];
        const int kv_start = p.kv_start ? p.kv_start[it.bs] : 0;
        const int split_len = (seq_len - kv_start + p.splits - 1) / p.splits;
        it.t0 = kv_start + split_len * it.sid;
        it.t1 = min(it.t0 + split_len, seq_len);
        it.n_pages = it.t1 > it.t0 ? (it.t1 - it.t0 + kPageTokens - 1) / kPageTokens : 0;
        return it;
    };
    auto mid_row = [&](const Item& it, int h) {
        return p.mid_o + ((static_cast<int64_t>(it.b) * p.Hq + it.hkv * group + h) * p.splits + it.sid) *
                             (D + 1);
    };
    constexpr int NRED = (NH * NMT <= WARPS) ? NH * NMT : WARPS;

    const uint32_t my_page = bufs + warp * C::PAGE_BYTES;

    for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
        const Item cur_it = item_info(item);
        const int hkv = cur_it.hkv, t0 = cur_it.t0, t1 = cur_it.t1, n_pages = cur_it.n_pages;
        if (n_pages == 0) {  // neutral partial (CTA-uniform): zeros and lse = -inf
            for (int idx = tid; idx < group * (D + 1); idx += THREADS) {
                const int h = idx / (D + 1), d = idx - h * (D + 1);
                mid_row(cur_it, h)[d] = d == D ? -INFINITY : 0.f;
            }
            continue;
        }
        // ---- prologue: rotate (no signs) and pre-scale the queries of the group; scores are
        // kept in the base-2 exponent domain
        if (warp < 2) {
            const int t8 = lane & 7, o = lane >> 3;
            const int hh = warp * 4 + o;
            const bool hv = hh < group;
            const int64_t qoff = (static_cast<int64_t>(cur_it.b) * p.Hq + hkv * group + (hv ? hh : 0)) * D;
            float a[E];
#pragma unroll
            for (int i = 0; i < E / 8; i++) {
                float tmp[8];
                const int64_t eo = qoff + 8 * (t8 + 8 * i);
                if (p.q_dtype == kF32) load8<float>(static_cast<const float*>(p.q) + eo, tmp);
                else if (p.q_dtype == kBF16)
                    load8<__nv_bfloat16>(static_cast<const __nv_bfloat16*>(p.q) + eo, tmp);
                else load8<__half>(static_cast<const __half*>(p.q) + eo, tmp);
#pragma unroll
                for (int c = 0; c < 8; c++) a[8 * i + c] = tmp[c];
            }
            octet_fwht<E>(a, lane);
#pragma unroll
            for (int k = 0; k < E; k++)
                qs[qs_index(hh, t8 + 8 * k)] = hv ? a[k] * p.rsqrt_d * (p.scale * kLog2e) : 0.f;
        }
        __syncthreads();  // queries visible; the buffers are free (last item's merge is over)

        uint32_t qb[NH][NKB][2];
#pragma unroll
        for (int hh = 0; hh < NH; hh++)
#pragma unroll
            for (int kb = 0; kb < NKB; kb++) {
                const float4 q4 = *reinterpret_cast<const float4*>(
                    qs + qs_index(4 * hh + (g >> 1), (D / 4) * tg + 4 * kb));
                const __half2 lo = __floats2half2_rn(q4.x, q4.y);
                const __half2 hi = __floats2half2_rn(q4.z, q4.w);
                qb[hh][kb][0] = *reinterpret_cast<const uint32_t*>(&lo);
                qb[hh][kb][1] = *reinterpret_cast<const uint32_t*>(&hi);
            }

        float m_run[NH], l_run[NH], z_run[NH], oacc[NH][NMT][4];
#pragma unroll
        for (int hh = 0; hh < NH; hh++) {
            m_run[hh] = -INFINITY;
            l_run[hh] = 0.f;
            z_run[hh] = 0.f;
#pragma unroll
            for (int mt = 0; mt < NMT; mt++)
#pragma unroll
                for (int i = 0; i < 4; i++) oacc[hh][mt][i] = 0.f;
        }

        const int32_t* btab = p.block_table + static_cast<int64_t>(cur_it.bs) * p.max_blocks;
        const uint8_t* const kv_layer = p.kv_cache + cur_it.layer * p.cache_layer_stride;
        bool bad_block = false;   // a block id outside the cache: block 0 stands in, lse becomes NaN
        // ---- staging, one page ahead, in registers.  The 16 slots of a page are copied word by
        // word: lane l takes the words l, l + 32, ... of the list (token 0 words 0..NWR-1, token 1
        // ...), so that a load instruction reads consecutive words of one or two slots.  Slots
        // start on 2-byte boundaries; the words are taken from the 4-byte boundary at or 2 bytes
        // before the start (both inside the cache: slots are even-sized and the cache is 4-byte
        // aligned), except that the last, half-used word of a slot that starts ON a boundary is
        // fetched as 16 bits (nothing past the slot is read).  Nothing is realigned here: the
        // fragment loads below shift by the row's start offset.
        // Slots of 24+ words are copied one token per load instruction (lane = word; words 32, 33
        // of all 16 tokens in one more instruction), shorter ones as a flat list of words.
        constexpr int NWR = C::NWR;
        constexpr bool ROWMODE = NWR >= 24;
        constexpr int REM = ROWMODE && NWR > 32 ? NWR - 32 : 0;
        static_assert(REM * kPageTokens <= 32, "slot too long for the copy loop");
        constexpr int NCOPY = ROWMODE ? kPageTokens + (REM ? 1 : 0) : C::NCOPY;
        uint32_t raw[NCOPY];
        uint32_t mis_next = 0u;
        // (token, word) that copy step i handles in this lane; word < 0: nothing
        auto copy_slot = [&](int i, int& tok, int& w) {
            if constexpr (ROWMODE) {
                if (i < kPageTokens) {
                    tok = i;
                    w = lane < (NWR < 32 ? NWR : 32) ? lane : -1;
                } else {
                    tok = lane / (REM ? REM : 1);
                    w = tok < kPageTokens ? 32 + lane % (REM ? REM : 1) : -1;
                }
            } else {
                const int f = 32 * i + lane;
                tok = f / NWR;
                w = f < kPageTokens * NWR ? f - tok * NWR : -1;
            }
        };
        auto prefetch = [&](int pg) {
            if (pg >= n_pages) return;  // warp-uniform
            // tokens past the end of the range re-read the last valid slot (their weight is zero)
            const int pos = min(t0 + pg * kPageTokens + (lane & 15), t1 - 1);
            const uint32_t blk = fast_div(static_cast<uint32_t>(pos), p.div_block);
            const uint32_t off = static_cast<uint32_t>(pos) - blk * p.block_size;
            int64_t id = btab[blk];
            if (p.num_blocks > 0 && static_cast<uint64_t>(id) >= static_cast<uint64_t>(p.num_blocks)) {
                id = 0;
                bad_block = true;
            }
            const uint8_t* sp = kv_layer + id * p.stride_block +
                                off * p.stride_pos + hkv * p.stride_head;
            const uint32_t m = static_cast<uint32_t>(reinterpret_cast<uintptr_t>(sp) >> 1) & 1u;
            mis_next = __ballot_sync(0xffffffffu, m != 0u) & 0xffffu;
            __syncwarp();  // the address list of the previous prefetch has been read by every lane
            if (lane < 16) {
                const unsigned long long entry = (reinterpret_cast<uintptr_t>(sp) - 2 * m) | m;
                asm volatile("st.shared.b64 [%0], %1;\n" ::"r"(my_page + C::OFF_AL + 8 * lane), "l"(entry));
            }
            __syncwarp();
#pragma unroll
            for (int i = 0; i < NCOPY; i++) {
                int tok, w;
                copy_slot(i, tok, w);
                uint32_t v = 0u;
                if (w >= 0) {
                    unsigned long long entry;
                    asm volatile("ld.shared.b64 %0, [%1];\n" : "=l"(entry) : "r"(my_page + C::OFF_AL + 8 * tok));
                    const uint8_t* al = reinterpret_cast<const uint8_t*>(entry & ~3ull);
                    // (streaming loads: a slot is read once per decode step)
                    if (w == NWR - 1 && !(entry & 1ull))
                        v = __ldcs(reinterpret_cast<const uint16_t*>(al + 4 * w));
                    else
                        v = __ldcs(reinterpret_cast<const uint32_t*>(al + 4 * w));
                }
                raw[i] = v;
            }
        };
        // write the prefetched words into the warp's page buffer (rows of ROWB bytes)
        auto scatter = [&]() {
#pragma unroll
            for (int i = 0; i < NCOPY; i++) {
                int tok, w;
                copy_slot(i, tok, w);
                if (w >= 0)
                    asm volatile("st.shared.b32 [%0], %1;\n" ::"r"(my_page + tok * C::ROWB + 4 * w), "r"(raw[i]));
            }
            if (lane == 0) asm volatile("st.shared.b32 [%0], %1;\n" ::"r"(my_page + C::OFF_MIS), "r"(mis_next));
        };
        // SB bytes at byte address `addr` (any alignment) of the page buffer -> ceil(SB/4) words
        auto lds_bytes = [&](uint32_t addr, auto sb_tag, uint32_t* out) {
            constexpr int SB = decltype(sb_tag)::value;
            constexpr int NW = (SB + 3) / 4;
            const uint32_t base = addr & ~3u, sh = 8u * (addr & 3u);
            uint32_t wds[NW + 1];
            if constexpr (SB == 16) {  // rows and 16-byte slices keep `base` 16-byte aligned
                const uint4 q4 = lds128(base);
                wds[0] = q4.x; wds[1] = q4.y; wds[2] = q4.z; wds[3] = q4.w;
                wds[4] = lds32(base + 16);
            } else {
#pragma unroll
                for (int j = 0; j <= NW; j++) wds[j] = lds32(base + 4 * j);
            }
#pragma unroll
            for (int j = 0; j < NW; j++) out[j] = __funnelshift_r(wds[j], wds[j + 1], sh);
        };
        auto lds_half = [&](uint32_t addr) {
            unsigned short h;
            asm volatile("ld.shared.u16 %0, [%1];\n" : "=h"(h) : "r"(addr));
            return __half2float(__ushort_as_half(h));
        };
        // every lane copies its slices of the staged page into registers (same fragment maps as
        // the page-layout kernel: K slice tg of tokens rho(g), rho(g)+2; V slice g of tokens
        // 4tg .. 4tg+3 in lane-rotated order) together with the scalars of its two score rows
        float kn_a, kn_b, vs_a, vs_b, vz_a, vz_b;
        auto read_page = [&](Regs& r) {
            const uint32_t mis = lds32(my_page + C::OFF_MIS);
            const int ktok = 4 * (g >> 1) + (g & 1);
            const uint32_t rowa = my_page + ktok * C::ROWB + 2u * ((mis >> ktok) & 1u);
            const uint32_t rowb = my_page + (ktok + 2) * C::ROWB + 2u * ((mis >> (ktok + 2)) & 1u);
            lds_bytes(rowa + C::KSB * tg, std::integral_constant<int, C::KSB>{}, r.k[0]);
            lds_bytes(rowb + C::KSB * tg, std::integral_constant<int, C::KSB>{}, r.k[1]);
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int tk = 4 * tg + ((j + tg) & 3);
                const uint32_t row = my_page + tk * C::ROWB + 2u * ((mis >> tk) & 1u);
                lds_bytes(row + PDK + 2 + C::VSB * g, std::integral_constant<int, C::VSB>{}, r.v[j]);
            }
            kn_a = lds_half(rowa + PDK);
            kn_b = lds_half(rowb + PDK);
            vs_a = lds_half(rowa + PDK + 2 + PDV);
            vs_b = lds_half(rowb + PDK + 2 + PDV);
            vz_a = lds_half(rowa + PDK + 4 + PDV);
            vz_b = lds_half(rowb + PDK + 4 + PDV);
        };

        prefetch(warp);
        for (int pg = warp; pg < n_pages; pg += WARPS) {
            __syncwarp();  // the previous page's fragments are in registers: the buffer is free
            scatter();
            __syncwarp();
            prefetch(pg + WARPS);
            Regs r;
            read_page(r);

            // ---- S = K.Q^T (two accumulator chains per head half) and, for the norm correction,
            // the key tile times itself: its diagonal is sum_d c^2 per token
            float c[NH][2][4], cna[4], cnb[4];
#pragma unroll
            for (int i = 0; i < 4; i++) cna[i] = cnb[i] = 0.f;
#pragma unroll
            for (int hh = 0; hh < NH; hh++)
#pragma unroll
                for (int z = 0; z < 2; z++)
#pragma unroll
                    for (int i = 0; i < 4; i++) c[hh][z][i] = 0.f;
#pragma unroll
            for (int kb = 0; kb < NKB; kb++) {
                const uint32_t a0 = lut32(entry_addr<C::IWK>(r.k[0], 2 * kb, lk_lane));
                const uint32_t a1 = lut32(entry_addr<C::IWK>(r.k[1], 2 * kb, lk_lane));
                const uint32_t a2 = lut32(entry_addr<C::IWK>(r.k[0], 2 * kb + 1, lk_lane));
                const uint32_t a3 = lut32(entry_addr<C::IWK>(r.k[1], 2 * kb + 1, lk_lane));
#pragma unroll
                for (int hh = 0; hh < NH; hh++)
                    mma_16816(c[hh][kb & 1], a0, a1, a2, a3, qb[hh][kb][0], qb[hh][kb][1]);
                if (p.norm_correction) {  // CTA-uniform
                    mma_16816(cna, a0, a1, a2, a3, a0, a2);  // columns = the tokens of rows 0..7
                    mma_16816(cnb, a0, a1, a2, a3, a1, a3);  // columns = the tokens of rows 8..15
                }
            }

            // ---- online softmax per head (4*hh + tg) over the page's 16 tokens
            const int ntok = min(kPageTokens, t1 - t0 - pg * kPageTokens);
            const int tokA = 4 * (g >> 1) + (g & 1);
            const bool okA = tokA < ntok, okB = tokA + 2 < ntok;
            float kna = kn_a, knb = kn_b;
            if (p.norm_correction) {
                // (row g, column g) of the first product is held by lane (g, g >> 1), element g & 1;
                // (row g + 8, column g) of the second one by the same lane, element 2 + (g & 1)
                const float da = odd ? cna[1] : cna[0];
                const float db = odd ? cnb[3] : cnb[2];
                const int src = (lane & ~3) | (g >> 1);
                kna *= rsqrtf(__shfl_sync(0xffffffffu, da, src) + 1e-16f);
                knb *= rsqrtf(__shfl_sync(0xffffffffu, db, src) + 1e-16f);
            }
            const float vsa = okA ? vs_a : 0.f;
            const float vsb = okB ? vs_b : 0.f;
            const float vza = okA ? fmaf(kCtr, vsa, vz_a) : 0.f;
            const float vzb = okB ? fmaf(kCtr, vsb, vz_b) : 0.f;
            uint32_t pb[NH][2][2];
#pragma unroll
            for (int hh = 0; hh < NH; hh++) {
                const float sa = okA ? (c[hh][0][0] + c[hh][1][0]) * kna : -INFINITY;
                const float sb = okB ? (c[hh][0][2] + c[hh][1][2]) * knb : -INFINITY;
                float mx = fmaxf(sa, sb);
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
                if (__any_sync(0xffffffffu, mx > m_run[hh])) {
                    const float m_new = fmaxf(m_run[hh], mx);  // finite: the page's first token is valid
                    const float corr = fast_exp2(m_run[hh] - m_new);
                    l_run[hh] *= corr;
                    z_run[hh] *= corr;
#pragma unroll
                    for (int mt = 0; mt < NMT; mt++)
#pragma unroll
                        for (int i = 0; i < 4; i++) oacc[hh][mt][i] *= corr;
                    m_run[hh] = m_new;
                }
                const float pa = fast_exp2(sa - m_run[hh]);
                const float pbv = fast_exp2(sb - m_run[hh]);
                l_run[hh] += pa + pbv;
                z_run[hh] = fmaf(pa, vza, fmaf(pbv, vzb, z_run[hh]));
                const uint32_t ha = __half_as_ushort(__float2half_rn(pa * vsa));
                const uint32_t hb = __half_as_ushort(__float2half_rn(pbv * vsb));
                uint32_t t0w = movmatrix_trans(__byte_perm(ha, 0u, 0x1010u));
                uint32_t t1w = movmatrix_trans(__byte_perm(hb, 0u, 0x1010u));
                if (tg & 2) { const uint32_t x = t0w; t0w = t1w; t1w = x; }
                {
                    const uint32_t sh = (tg & 1) * 16;
                    const uint32_t lo = __funnelshift_r(t0w, t1w, sh);
                    const uint32_t hi = __funnelshift_r(t1w, t0w, sh);
                    t0w = lo;
                    t1w = hi;
                }
                pb[hh][0][0] = __byte_perm(t0w, 0u, sel_plo);
                pb[hh][0][1] = __byte_perm(t0w, 0u, sel_phi);
                pb[hh][1][0] = __byte_perm(t1w, 0u, sel_plo);
                pb[hh][1][1] = __byte_perm(t1w, 0u, sel_phi);
            }

            // ---- O^T += V^T.P^T with the integer value codes as the A operand
            if constexpr (VB == 4) {
                // 4-bit codes are turned into fp16 arithmetically, no look-up: a nibble or-ed into
                // the mantissa of 1024.0 (0x6400) is 1024 + code (or 1024 + 16 * code one nibble
                // up), and one packed subtract / multiply-add centres it exactly.  A 32-bit word
                // (coordinates 0..7 of the lane's slice) yields the pairs (0,4) (1,5) (2,6) (3,7):
                // two m-tiles whose rows hold other coordinates than the table version's -- the
                // write-out below knows.
                const uint32_t kMagic = 0x64006400u;
                const __half2 kSubLo = __floats2half2_rn(1024.f + kCtr, 1024.f + kCtr);
                const __half2 kMulHi = __floats2half2_rn(0.0625f, 0.0625f);
                const __half2 kSubHi = __floats2half2_rn(-(64.f + kCtr), -(64.f + kCtr));
                auto dq = [&](uint32_t w, uint32_t (&t)[4]) {
                    const uint32_t w8 = w >> 8;
                    const uint32_t x0 = (w & 0x000F000Fu) | kMagic, x1 = (w & 0x00F000F0u) | kMagic;
                    const uint32_t x2 = (w8 & 0x000F000Fu) | kMagic, x3 = (w8 & 0x00F000F0u) | kMagic;
                    const __half2 h0 = __hsub2(*reinterpret_cast<const __half2*>(&x0), kSubLo);
                    const __half2 h1 = __hfma2(*reinterpret_cast<const __half2*>(&x1), kMulHi, kSubHi);
                    const __half2 h2 = __hsub2(*reinterpret_cast<const __half2*>(&x2), kSubLo);
                    const __half2 h3 = __hfma2(*reinterpret_cast<const __half2*>(&x3), kMulHi, kSubHi);
                    t[0] = *reinterpret_cast<const uint32_t*>(&h0);
                    t[1] = *reinterpret_cast<const uint32_t*>(&h1);
                    t[2] = *reinterpret_cast<const uint32_t*>(&h2);
                    t[3] = *reinterpret_cast<const uint32_t*>(&h3);
                };
#pragma unroll
                for (int ks = 0; ks < 2; ks++)
#pragma unroll
                    for (int wd = 0; wd < NMT / 2; wd++) {
                        uint32_t ta[4], tb4[4];
                        dq(r.v[2 * ks][wd], ta);
                        dq(r.v[2 * ks + 1][wd], tb4);
#pragma unroll
                        for (int hh = 0; hh < NH; hh++) {
                            mma_16816(oacc[hh][2 * wd], ta[0], ta[1], tb4[0], tb4[1], pb[hh][ks][0], pb[hh][ks][1]);
                            mma_16816(oacc[hh][2 * wd + 1], ta[2], ta[3], tb4[2], tb4[3], pb[hh][ks][0], pb[hh][ks][1]);
                        }
                    }
            } else
#pragma unroll
            for (int ks = 0; ks < 2; ks++)
#pragma unroll
                for (int mt = 0; mt < NMT; mt++) {
                    const uint32_t a0 = lut32(entry_addr<C::IWV>(r.v[2 * ks], 2 * mt, lv_lane));
                    const uint32_t a1 = lut32(entry_addr<C::IWV>(r.v[2 * ks], 2 * mt + 1, lv_lane));
                    const uint32_t a2 = lut32(entry_addr<C::IWV>(r.v[2 * ks + 1], 2 * mt, lv_lane));
                    const uint32_t a3 = lut32(entry_addr<C::IWV>(r.v[2 * ks + 1], 2 * mt + 1, lv_lane));
#pragma unroll
                    for (int hh = 0; hh < NH; hh++)
                        mma_16816(oacc[hh][mt], a0, a1, a2, a3, pb[hh][ks][0], pb[hh][ks][1]);
                }
        }

        // ---- fold the warps' states: every warp publishes (m, l, z, O), NRED warps reduce
#pragma unroll
        for (int hh = 0; hh < NH; hh++) {
#pragma unroll
            for (int m = 4; m < 32; m <<= 1) {
                l_run[hh] += __shfl_xor_sync(0xffffffffu, l_run[hh], m);
                z_run[hh] += __shfl_xor_sync(0xffffffffu, z_run[hh], m);
            }
        }
        // every warp is done with its page buffer: the area becomes the exchange area
        const bool any_bad = __syncthreads_or(bad_block) != 0;
#pragma unroll
        for (int hh = 0; hh < NH; hh++) {
#pragma unroll
            for (int mt = 0; mt < NMT; mt++)
                xchg[((warp * NH + hh) * NMT + mt) * 32 + lane] = make_float4(
                    oacc[hh][mt][0], oacc[hh][mt][1], oacc[hh][mt][2], oacc[hh][mt][3]);
            if (g == 0) {
                xml[((warp * NH + hh) * 3 + 0) * 4 + tg] = m_run[hh];
                xml[((warp * NH + hh) * 3 + 1) * 4 + tg] = l_run[hh];
                xml[((warp * NH + hh) * 3 + 2) * 4 + tg] = z_run[hh];
            }
        }
        __syncthreads();
        if (warp < NRED) {
            for (int j = tid; j < NH * NMT * 32; j += NRED * 32) {
                const int ln = j & 31, mt = (j >> 5) % NMT, hh = j / (32 * NMT);
                const int tg_ = ln & 3, g_ = ln >> 2;
                float M = -INFINITY;
#pragma unroll
                for (int w2 = 0; w2 < WARPS; w2++)
                    M = fmaxf(M, xml[((w2 * NH + hh) * 3 + 0) * 4 + tg_]);
                float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
                float l = 0.f, z = 0.f;
#pragma unroll
                for (int w2 = 0; w2 < WARPS; w2++) {
                    const float mw = xml[((w2 * NH + hh) * 3 + 0) * 4 + tg_];
                    if (mw != -INFINITY) {
                        const float f = fast_exp2(mw - M);
                        const float4 o = xchg[((w2 * NH + hh) * NMT + mt) * 32 + ln];
                        a.x = fmaf(o.x, f, a.x);
                        a.y = fmaf(o.y, f, a.y);
                        a.z = fmaf(o.z, f, a.z);
                        a.w = fmaf(o.w, f, a.w);
                        l = fmaf(xml[((w2 * NH + hh) * 3 + 1) * 4 + tg_], f, l);
                        z = fmaf(xml[((w2 * NH + hh) * 3 + 2) * 4 + tg_], f, z);
                    }
                }
                const int h = 4 * hh + tg_;
                if (h < group) {
                    // partial = (sum p * (code * scale + zero)) / sum p, lse in natural-log units
                    const float inv = 1.f / l;
                    float* dst = mid_row(cur_it, h);
                    if constexpr (VB == 4) {
                        // rows of the arithmetic dequantisation: m-tile pair (2w, 2w + 1) covers
                        // coordinates 8w..8w+7 of the slice as (0,4 | 1,5) and (2,6 | 3,7)
                        float* o4 = dst + (D / 8) * g_ + 8 * (mt >> 1) + 2 * (mt & 1);
                        o4[0] = (a.x + z) * inv;
                        o4[4] = (a.y + z) * inv;
                        o4[1] = (a.z + z) * inv;
                        o4[5] = (a.w + z) * inv;
                    } else {
                        float* o4 = dst + (D / 8) * g_ + 4 * mt;
                        o4[0] = (a.x + z) * inv;
                        o4[1] = (a.y + z) * inv;
                        o4[2] = (a.z + z) * inv;
                        o4[3] = (a.w + z) * inv;
                    }
                    if (g_ == 0 && mt == 0)
                        dst[D] = any_bad ? __int_as_float(0x7fc00000) : M * kLn2 + logf(l);
                }
            }
        }
    }
}

}  // namespace ftq
