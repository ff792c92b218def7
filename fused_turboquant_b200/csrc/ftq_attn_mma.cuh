// Paged split-KV decode attention on the tensor cores (barrier-synchronised form;
// ftq_attn_stream.cuh holds the streaming form of the same arithmetic): whole
// 16-token pages arrive in a per-warp ring by 1-D bulk copies (TMA), every lane
// copies its slices to registers, the codes are dequantised through a
// bank-conflict-free shared-memory table and feed warp-level m16n8k16 fp16 MMAs
// (fp32 accumulate).  With a GQA
// group of G query heads the products are skinny GEMMs (G x D x tokens), so the
// per-element work no longer grows with G and every packed byte is dequantised
// exactly once per KV head.
//
// Same mathematics as attn_split_kernel (ftq_attn.cuh), i.e. the fused
// formulation of src/fused_turboquant/kernels/triton_flash_decode.py:33-324 in the
// reference; centroids, the rotated query and the softmax weights are rounded
// to fp16 before the MMAs, accumulation is fp32.  The V centroids are multiplied
// by a host-chosen factor in [1, 2) before the rounding (and the weights divided
// by it): a common rounding bias of the centroids would otherwise add up over
// all coordinates into one output element through the inverse rotation.
//
// Work split: persistent CTAs (one per SM when a 4-bit byte table is in use --
// 16 warps, or 8 where 16 page rings do not fit beside the table -- else two per
// SM with 8 warps) loop over work items
// (KV chunk, KV head, sequence x layer); the dequantisation tables are built once
// per CTA.  Within an item each warp walks pages warp, warp+W, ... with its own
// online-softmax state; the states are merged pairwise (registers + a small
// shared exchange area) and warp 0 writes one partial row per query head (same
// workspace format as attn_split_kernel, so attn_merge_kernel finishes both).
//
// Tables: an entry holds the fp16 centroids of two adjacent codes, replicated
// for the 32 lanes so that bank = lane (no conflicts whatever the codes are).
// 4-bit codes index by byte: the table occupies a 64 KB-aligned window with
// 256-byte rows, so that the address is one byte-permute -- the code byte
// dropped into bits 8..15 of the lane's base address.  3- and 2-bit codes use
// 128-byte rows in a table aligned to its own size (shift + and/or).
//
// Fragment maps for one 16-token page (lane = 4*g + tg), query heads handled in
// halves of 4 (NH = 1 for a GQA group <= 4, else 2):
//   S = K.Q^T :  A = K [16 tokens x 16 coords]: rows g / g+8 = page tokens rho(g) / rho(g)+2,
//                    k-block kb covers coordinates (D/4)*tg + 4*kb + {0..3}
//                B = Q^T[16 coords x 8]: column n = head n>>1 (each head twice)
//                C[token][head tg]  (columns 2tg and 2tg+1 are the same head)
//   the weights p*vnorm are rounded to fp16 and transposed with movmatrix, which
//   hands lane (g, tg) the weights of head g>>1 for page tokens 4tg .. 4tg+3;
//   O^T = V^T.P^T with reduction index k = (token, parity of d), so that the fp16
//   pair a table lookup returns, (V[t,d], V[t,d+1]), is directly an A register:
//                A[row = d-pair][k = (token, parity)] = V[token][2*pair + parity]
//                B[k = (token, parity)][n = (head n>>1, parity n&1)] = p or 0
//                C[d-pair][(head tg, parity)]: lane (g,tg) owns O[head tg][(D/8)g .. +D/8)
//   so a lane dequantises the K slices (D/4 coordinates) of two tokens and the V
//   slices (D/8 coordinates) of four tokens per page, all contiguous bytes, every
//   code exactly once per KV head.
#pragma once

#include <type_traits>

#include "ftq_attn.cuh"

namespace ftq {

constexpr float kLog2e = 1.4426950408889634f, kLn2 = 0.6931471805599453f;
constexpr int kMmaMaxChunkPages = 1024;  // block ids of one chunk are staged in shared memory

// (not volatile: a pure function of its operands, so the compiler may interleave the MMAs
// with the table lookups of later k-blocks)
__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                          uint32_t a3, uint32_t b0, uint32_t b1) {
    asm(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.b32 %0, [%1];\n" : "=r"(v) : "r"(addr));
    return v;
}
// Lookup in a dequantisation table: the tables never change after the CTA-wide barrier that
// follows their construction and every address derives from page data read after that barrier,
// so the load may be scheduled freely (not volatile).
__device__ __forceinline__ uint32_t lut32(uint32_t addr) {
    uint32_t v;
    asm("ld.shared.b32 %0, [%1];\n" : "=r"(v) : "r"(addr));
    return v;
}

__device__ __forceinline__ uint2 lut64(uint32_t addr) {
    uint2 v;
    asm("ld.shared.v2.b32 {%0,%1}, [%2];\n" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}

#ifndef FTQ_LAZY_SLACK
#define FTQ_LAZY_SLACK 3
#endif
// slack of the lazy reference maximum of the online softmax (base-2 exponent units)
constexpr float kLazyMaxSlack = static_cast<float>(FTQ_LAZY_SLACK);
// m16n8k16 with a zero accumulator input (saves clearing the accumulators of every page)
__device__ __forceinline__ void mma_16816_z(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                            uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%10,%10,%10,%10};\n"
        : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}

__device__ __forceinline__ uint32_t f2h_sat(float x) {
    unsigned short h;
    asm("cvt.rn.satfinite.f16.f32 %0, %1;\n" : "=h"(h) : "f"(x));
    return h;
}

// ---- mbarrier + bulk-copy (TMA, 1-D, no multicast) helpers; all addresses are shared-window
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::
            "r"(dst), "l"(src), "r"(bytes), "r"(bar)
        : "memory");
}
// The same copy with an L2 policy: KV pages are read once per decode step, so L2 is told to drop
// them first (measured on B200: +1.5 % on the Llama-shaped K4V4 batch).
__device__ __forceinline__ uint64_t l2_evict_first_policy() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;\n" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ void bulk_g2s_hint(uint32_t dst, const void* src, uint32_t bytes,
                                              uint32_t bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;\n" ::
            "r"(dst), "l"(src), "r"(bytes), "r"(bar), "l"(policy)
        : "memory");
}
// Bounded wait: gives up after kMbarSpinLimit polls (each poll may itself block for a
// hardware-defined slice) and reports failure instead of hanging the SM.
// FTQ_TEST_WAIT_EXPIRY (only the test library of build.py defines it): warp 5 of CTA 0 announces its
// first page copy to the mbarrier but does not issue it, and the poll limit is small -- the wait
// runs out, which is the one way to execute the give-up path (NaN rows, status word) on purpose.
#ifdef FTQ_TEST_WAIT_EXPIRY
constexpr int kMbarSpinLimit = 1 << 6;
#else
constexpr int kMbarSpinLimit = 1 << 20;
#endif
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (int i = 0; i < kMbarSpinLimit; i++) {
        uint32_t ok;
        asm volatile(
            "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
            "selp.u32 %0, 1, 0, p;\n}\n"
            : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
    }
    return false;
}
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.b32 {%0,%1}, [%2];\n" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}

// Load slice `idx` (SB bytes each, slices back to back starting at the 4-byte aligned shared
// address `row`) of a staged page into ceil(SB/4) words.  Slices whose size is not a multiple
// of 4 are cut out of the enclosing aligned chunk with funnel shifts.
template <int SB>
__device__ __forceinline__ void lds_slice(uint32_t row, int idx, uint32_t (&w)[(SB + 3) / 4]) {
    if constexpr (SB % 16 == 0) {
#pragma unroll
        for (int i = 0; i < SB / 16; i++) {
            const uint4 v = lds128(row + idx * SB + 16 * i);
            w[4 * i] = v.x; w[4 * i + 1] = v.y; w[4 * i + 2] = v.z; w[4 * i + 3] = v.w;
        }
    } else if constexpr (SB % 8 == 0) {
#pragma unroll
        for (int i = 0; i < SB / 8; i++) {
            const uint2 v = lds64(row + idx * SB + 8 * i);
            w[2 * i] = v.x; w[2 * i + 1] = v.y;
        }
    } else if constexpr (SB % 4 == 0) {
#pragma unroll
        for (int i = 0; i < SB / 4; i++) w[i] = lds32(row + idx * SB + 4 * i);
    } else if constexpr (SB == 6) {
        const uint32_t c = row + (idx >> 1) * 12;
        const uint32_t x0 = lds32(c), x1 = lds32(c + 4), x2 = lds32(c + 8);
        const bool odd = idx & 1;
        w[0] = odd ? __funnelshift_r(x1, x2, 16) : x0;
        w[1] = odd ? (x2 >> 16) : (x1 & 0xffffu);
    } else if constexpr (SB == 3) {
        const uint32_t c = row + (idx >> 2) * 12;
        const uint32_t x0 = lds32(c), x1 = lds32(c + 4), x2 = lds32(c + 8);
        const int q = idx & 3;
        const uint32_t lo = q == 0 ? x0 : (q == 1 ? __funnelshift_r(x0, x1, 24)
                                                  : (q == 2 ? __funnelshift_r(x1, x2, 16) : (x2 >> 8)));
        w[0] = lo & 0xffffffu;
    } else {
        static_assert(SB == 2, "unsupported slice size");
        const uint32_t x = lds32(row + (idx >> 1) * 4);
        w[0] = (idx & 1) ? (x >> 16) : (x & 0xffffu);
    }
}

// Shared-memory byte offset (entry * 128) of the table entry for code pair `pair`
// of a slice: bits [pair*IW, pair*IW + IW) of the little-endian stream in w[].
template <int IW, int NW>
__device__ __forceinline__ uint32_t pair_index(const uint32_t (&w)[NW], int pair) {
    constexpr uint32_t mask = ((1u << IW) - 1u) << 7;
    const int bo = pair * IW;
    const int j = bo >> 5, sh = bo & 31;
    uint32_t x;
    if (sh + IW <= 32) x = sh >= 7 ? (w[j] >> (sh - 7)) : (w[j] << (7 - sh));
    else x = __funnelshift_r(w[j], w[j + 1 < NW ? j + 1 : j], sh - 7);
    return x & mask;
}

// Shared-memory address of the table entry for code pair `pair` of a slice.
//   IW == 8 (4-bit): lane_base = window | table half | lane*4; the code byte becomes byte 1.
//   IW  < 8        : lane_base = table | lane*4; entry * 128 is or-ed in.
template <int IW, int NW>
__device__ __forceinline__ uint32_t entry_addr(const uint32_t (&w)[NW], int pair, uint32_t lane_base) {
    if constexpr (IW == 8) {
        const int j = pair >> 2, k = pair & 3;
        return __byte_perm(w[j], lane_base, 0x7604u | (static_cast<uint32_t>(k) << 4));
    } else {
        return lane_base | pair_index<IW>(w, pair);
    }
}

template <int D, int BK, int BV, int NH>
struct MmaCfg {
    static constexpr int NKB = D / 16;                  // k-blocks of K.Q^T
    static constexpr int NMT = D / 32;                  // m-tiles of O^T
    static constexpr int PDK = packed_dim(D, BK), PDV = packed_dim(D, BV);
    static constexpr int KSB = PDK / 4, VSB = PDV / 8;  // slice bytes per lane
    static constexpr int IWK = 2 * BK, IWV = 2 * BV;    // table index width (two codes)
    static constexpr bool BYTE = BK == 4 || BV == 4;    // a 64 KB byte-indexed window is used
    static constexpr int OFF_KN = kPageTokens * PDK;
    static constexpr int OFF_VC = OFF_KN + 2 * kPageTokens;
    static constexpr int OFF_VN = OFF_VC + kPageTokens * PDV;
    static constexpr int PAGE_BYTES = OFF_VN + 2 * kPageTokens;
    // small (non-byte) tables, each aligned to its own size
    static constexpr int TKS = BK == 4 ? 0 : (1 << IWK) * 128;
    // 2-bit values next to 4-bit keys: the upper half of every row of the key's byte window holds,
    // 16 times, the FOUR centroids of a value byte (8 bytes), so one byte-permute + one 8-byte
    // load dequantise four codes (instead of shift/and + two 4-byte loads)
    static constexpr bool V2BYTE = BK == 4 && BV == 2;
    static constexpr int TVS = (BV == 4 || V2BYTE) ? 0 : (1 << IWV) * 128;
    static constexpr int SMALL_ALIGN = TKS > TVS ? TKS : TVS;
    static constexpr int SMALL_BYTES = TKS + TVS + SMALL_ALIGN;  // incl. alignment slack
    static constexpr int STATE_F4 = NH * NMT;                    // float4 items per lane
    // per-warp ring of pages staged by bulk copies (TMA), one mbarrier per buffer
    static constexpr int RING = 2;
    static constexpr int BASE_A = SMALL_BYTES + 8 * (D + 16) * 4 + kMmaMaxChunkPages * 4 + 64;
    // Shared memory needed with `w` warps.  Two groups of objects are placed first-fit around the
    // 64 KB table window.  With one head half the merge exchange area (every warp's (O, m, l))
    // gets its own space when it fits (`sep`), so that the first pages of the NEXT item can
    // already be copied into the ring while the merge runs; otherwise it aliases the ring
    // (idle during the merge).
    __host__ __device__ static constexpr int xchg_bytes(int w) {
        return w * (32 * STATE_F4 * 16 + NH * 2 * 4 * 4);
    }
    __host__ __device__ static constexpr int total_w(int w, bool sep) {
        const int xchg = xchg_bytes(w), ring = w * RING * PAGE_BYTES, bars = w * RING * 8 + 256;
        const int a = BASE_A + (sep ? xchg + 16 : 0);
        const int b = ((sep || ring > xchg) ? ring : xchg) + bars;
        if (!BYTE) return a + b;
        // objects are placed first-fit before / after the 64 KB-aligned table window
        const int mn = a < b ? a : b;
        const int worst = (65536 + b > mn + a + b) ? 65536 + b : mn + a + b;
        return 65536 + worst;
    }
    // head_dim 256 keeps the query fragments in shared memory (one 8-byte load per k-block and
    // page) instead of 32 registers, which lets it run 16 warps per SM like head_dim 128
    // wherever 16 page rings fit next to the byte table
#ifndef FTQ_W16
#define FTQ_W16 16
#endif
    static constexpr int WARPS = (BYTE && total_w(FTQ_W16, false) <= 227 * 1024) ? FTQ_W16 : 8;
    // (an 8-warp CTA that owns its SM has 255 registers per thread and keeps them in registers)
    static constexpr bool QSMEM = D == 256 && !(BYTE && WARPS == 8);
    static constexpr int THREADS = 32 * WARPS;
    static constexpr int CTAS_PER_SM = BYTE ? 1 : 2;
    static constexpr int XCHG_BYTES = xchg_bytes(WARPS);
    static constexpr int RING_BYTES = WARPS * RING * PAGE_BYTES;
    static constexpr int BARS = WARPS * RING * 8 + 256;
    __host__ __device__ static constexpr int total(bool sep) { return total_w(WARPS, sep); }
    static constexpr bool SEP = NH == 1 && total(true) <= 227 * 1024;
    static constexpr int GROUP_A = BASE_A + (SEP ? XCHG_BYTES + 16 : 0);
    static constexpr int GROUP_B = ((SEP || RING_BYTES > XCHG_BYTES) ? RING_BYTES : XCHG_BYTES) + BARS;
    static constexpr int SMEM_BYTES = total(SEP);
};

// One page worth of packed data in registers (per lane).
template <int KSB, int VSB>
struct PageRegs {
    uint32_t k[2][(KSB + 3) / 4];  // K slice tg of page tokens rho(g), rho(g) + 2
    uint32_t v[4][(VSB + 3) / 4];  // V slice g of page tokens 4tg .. 4tg+3
    uint2 kn, vn;                  // fp16 norms of page tokens 4(g>>1) .. 4(g>>1)+3
};

__device__ __forceinline__ float half_bits_to_float(uint32_t h16) {
    return __half2float(__ushort_as_half(static_cast<unsigned short>(h16)));
}

// 2^x, one MUFU (flushes denormal results to zero; exp2(-inf) = 0)
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
    uint32_t d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(d) : "r"(a));
    return d;
}

template <int D, int BK, int BV, bool SHARED_LUT, int NH>
__global__ void __launch_bounds__(MmaCfg<D, BK, BV, NH>::THREADS, MmaCfg<D, BK, BV, NH>::CTAS_PER_SM)
attn_mma_kernel(const AttnParams p, int n_items) {
    using C = MmaCfg<D, BK, BV, NH>;
    constexpr int NKB = C::NKB, NMT = C::NMT, WARPS = C::WARPS, THREADS = C::THREADS;
    constexpr int E = D / kOctet;
    constexpr int ROW = D + 4;
    using Regs = PageRegs<C::KSB, C::VSB>;

    extern __shared__ __align__(16) uint8_t smem_raw[];
    const uint32_t sbase = static_cast<uint32_t>(__cvta_generic_to_shared(smem_raw));
    // ---- carve shared memory (addresses in the shared window): the byte table needs a
    // 64 KB-aligned window; the other objects go first-fit before or after it
    uint32_t window = 0, free0 = sbase, end0 = sbase, free1 = sbase;
    if constexpr (C::BYTE) {
        window = (sbase + 65535u) & ~65535u;
        end0 = window;
        free1 = window + 65536u;
    }
    auto take = [&](uint32_t bytes, uint32_t align) {
        uint32_t a = (free0 + align - 1) & ~(align - 1);
        if (a + bytes <= end0) { free0 = a + bytes; return a; }
        a = (free1 + align - 1) & ~(align - 1);
        free1 = a + bytes;
        return a;
    };
    auto gptr = [&](uint32_t saddr) { return smem_raw + (saddr - sbase); };
    // group A: small tables, queries, block ids
    const uint32_t grp_a = take(C::GROUP_A, 16);
    uint32_t tk_small = 0, tv_small = 0, cur = grp_a;
    if constexpr (C::SMALL_ALIGN > 0) {
        cur = (grp_a + C::SMALL_ALIGN - 1) & ~static_cast<uint32_t>(C::SMALL_ALIGN - 1);
        if (C::TKS >= C::TVS) { tk_small = cur; tv_small = cur + C::TKS; }
        else { tv_small = cur; tk_small = cur + C::TVS; }
        cur += C::TKS + C::TVS;
        if (SHARED_LUT) tv_small = tk_small;
    }
    cur = (cur + 15u) & ~15u;
    float* qs = reinterpret_cast<float*>(gptr(cur));                  // [8][D + 16]
    int32_t* sblk = reinterpret_cast<int32_t*>(qs + 8 * (D + 16));    // block ids of the chunk
    // group B: page ring + mbarriers
    const uint32_t grp_b = take(C::GROUP_B, 128);
    const uint32_t bars = grp_b;                              // [WARPS][RING] x 8 bytes
    const uint32_t ring = (grp_b + WARPS * C::RING * 8 + 127u) & ~127u;
    // merge exchange area: own space after the block ids, or aliasing the ring
    const uint32_t xaddr = C::SEP ? ((cur + 8 * (D + 16) * 4 + kMmaMaxChunkPages * 4 + 15u) & ~15u) : ring;
    float4* xchg = reinterpret_cast<float4*>(gptr(xaddr));  // [WARPS][NH][NMT][32]
    float* xml = reinterpret_cast<float*>(gptr(xaddr + WARPS * 32 * C::STATE_F4 * 16));  // [WARPS][NH][2][4]

    const int tid = threadIdx.x;
    const int lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, tg = lane & 3;
    const bool odd = g & 1;
    const int group = p.Hq / p.Hkv;  // <= 4 * NH
    // byte selectors (source 4 = a zero byte): a lane's own fp16 of a packed pair, and the
    // placement of a weight in the low (even g) or high (odd g) half of a B register
    uint32_t sel_own = odd ? 0x4432u : 0x4410u;
    uint32_t sel_plo = odd ? 0x1044u : 0x4410u;
    uint32_t sel_phi = odd ? 0x3244u : 0x4432u;
    // Lane constants of the page reads: byte offset of the key row rho(g) and of the norm quad;
    // per value register j the row of page token 4tg + ((j + tg) & 3) (plus the slice where
    // slices are whole words) and the slice index otherwise (slice g, halves exchanged for tokens
    // with bit 1 set).  (The streaming kernel pins these in registers; here that measured no gain.)
    uint32_t koff = (4 * (g >> 1) + (g & 1)) * MmaCfg<D, BK, BV, NH>::PDK;
    uint32_t noff = MmaCfg<D, BK, BV, NH>::OFF_KN + 8 * (g >> 1);
    uint32_t vrow[4];
    int vidx[4];
#pragma unroll
    for (int j = 0; j < 4; j++) {
        using CC = MmaCfg<D, BK, BV, NH>;
        const int u = (j + tg) & 3;
        const int slice = g ^ ((u & 2) << 1);
        vrow[j] = CC::OFF_VC + (4 * tg + u) * CC::PDV + (CC::VSB % 4 == 0 ? slice * CC::VSB : 0);
        vidx[j] = CC::VSB % 4 == 0 ? 0 : slice;
    }

    // ---- once per CTA: dequantisation tables
    if constexpr (C::BYTE) {
        uint32_t* tb = reinterpret_cast<uint32_t*>(gptr(window));
        for (int i = tid; i < 256 * 64; i += THREADS) {
            const int e = i >> 6, col = i & 63;
            if (col < 32) {
                if constexpr (BK == 4) {
                    const __half2 h = __floats2half2_rn(p.lk.v[e & 15], p.lk.v[e >> 4]);
                    tb[i] = *reinterpret_cast<const uint32_t*>(&h);
                }
            } else if constexpr (BV == 4 && !SHARED_LUT) {
                const __half2 h = __floats2half2_rn(p.lv_scaled.v[e & 15], p.lv_scaled.v[e >> 4]);
                tb[i] = *reinterpret_cast<const uint32_t*>(&h);
            } else if constexpr (C::V2BYTE) {
                const int sh = 4 * (col & 1);  // word 0: codes 0, 1 of the byte; word 1: codes 2, 3
                const __half2 h = __floats2half2_rn(p.lv_scaled.v[(e >> sh) & 3],
                                                    p.lv_scaled.v[(e >> (sh + 2)) & 3]);
                tb[i] = *reinterpret_cast<const uint32_t*>(&h);
            }
        }
    }
    if constexpr (BK != 4) {
        uint32_t* t = reinterpret_cast<uint32_t*>(gptr(tk_small));
        for (int i = tid; i < (1 << C::IWK) * 32; i += THREADS) {
            const int e = i >> 5;
            const __half2 h = __floats2half2_rn(p.lk.v[e & ((1 << BK) - 1)], p.lk.v[e >> BK]);
            t[i] = *reinterpret_cast<const uint32_t*>(&h);
        }
    }
    if constexpr (BV != 4 && !SHARED_LUT && !C::V2BYTE) {
        uint32_t* t = reinterpret_cast<uint32_t*>(gptr(tv_small));
        for (int i = tid; i < (1 << C::IWV) * 32; i += THREADS) {
            const int e = i >> 5;
            const __half2 h = __floats2half2_rn(p.lv_scaled.v[e & ((1 << BV) - 1)], p.lv_scaled.v[e >> BV]);
            t[i] = *reinterpret_cast<const uint32_t*>(&h);
        }
    }
    const uint32_t lk_lane = (BK == 4 ? window : tk_small) | (lane * 4);
    const uint32_t lv_lane =
        C::V2BYTE ? (window | 128u | ((lane & 15) * 8))
                  : ((BV == 4 ? (window | (SHARED_LUT ? 0u : 128u)) : tv_small) | (lane * 4));

    // ---- once per CTA: one mbarrier per ring buffer (a single arrival + the copy's bytes)
    if (lane == 0) {
#pragma unroll
        for (int r = 0; r < C::RING; r++) mbar_init(bars + (warp * C::RING + r) * 8, 1);
    }
    mbar_fence_init();
    __syncthreads();
    uint32_t phase = 0;   // bit r = parity the next wait on ring buffer r expects
    int ring_it = 0;      // pages this warp has taken from its ring so far (buffer = ring_it % RING)
    bool primed = false;  // the first RING pages of the current item were requested early
    bool stalled = false; // a bulk copy never arrived: stop waiting, poison the result

    // rotated queries in shared memory: head rows of D + 16 floats, each quarter of a row
    // padded by 4, so that the 16 distinct float4 a fragment load touches are 2-way at worst
    auto qs_index = [](int head, int coord) {
        return head * (D + 16) + (coord / (D / 4)) * (D / 4 + 4) + coord % (D / 4);
    };
    // ---- persistent loop over work items
    struct Item { int chunk, hkv, lb, layer, b, t0, t1, n_pages; };
    auto item_info = [&](int item) {
        Item it;
        // (items are numbered region by region: see SplitPlan)
        const SplitRegion& rg = region_of_item(p.split, item);
        const int j = item - rg.first_item;
        it.chunk = j % rg.chunks;
        const int rest = rg.first_unit + j / rg.chunks;
        const int ct = rg.chunk_tokens;
        it.hkv = rest % p.Hkv;
        it.lb = rest / p.Hkv;
        it.layer = it.lb / p.B;
        it.b = it.lb - it.layer * p.B;
        it.t0 = it.chunk * ct;
        it.t1 = min(p.seq_lens[it.b], it.t0 + ct);
        it.n_pages = (it.t1 - it.t0 + kPageTokens - 1) / kPageTokens;
        return it;
    };
    const int64_t prow_head_stride = static_cast<int64_t>(p.split.row_chunks) * ROW;
    auto partial_row = [&](const Item& it) {
        return p.partials +
               ((static_cast<int64_t>(it.lb) * p.Hq + it.hkv * group) * p.split.row_chunks + it.chunk) * ROW;
    };
    // Work items are handed out by a global counter (zeroed by the host before the launch), one
    // at a time and in index order, so that CTAs that drew short items come back for more: with
    // ragged batches a fixed item-to-CTA assignment leaves most SMs idle while a few finish long
    // sequences.  Thread 0 draws a CTA's NEXT item at the start of the current one (everybody
    // learns it at the item's first barrier, early enough to request its first pages before the
    // merge); items without tokens get their (-inf, 0) rows on the spot.
    __shared__ int s_next[2];  // written in alternation: a slot is read before its next write's barrier
    __shared__ int s_bad[2];   // item (by parity of its place in this CTA's sequence) saw a bad block id
    int ticket = n_items;  // thread 0: counter value drawn for the next item
    auto draw_ticket = [&]() {
        if (tid == 0) ticket = atomicAdd(p.work_counter, 1);
    };
    // thread 0 only: first item with tokens at or after ticket t (further tickets drawn on demand)
    auto resolve_ticket = [&](int t) {
        while (true) {
            if (t >= n_items) return n_items;
            const Item it = item_info(t);
            if (it.t0 < it.t1) return t;
            float* prow = partial_row(it);
            for (int h = 0; h < group; h++) {
                prow[h * prow_head_stride + D] = -INFINITY;
                prow[h * prow_head_stride + D + 1] = 0.f;
            }
            t = atomicAdd(p.work_counter, 1);
        }
    };
    // item prologue, run by warps [w0, w0 + nw): block ids of the chunk and the rotated,
    // pre-scaled queries (8 octets of the first two warps rotate the at most 8 heads)
    // (a block id outside [0, num_blocks) is never dereferenced: block 0 stands in for it and
    // flag `bad_slot` of s_bad makes the item's result NaN)
    auto prologue = [&](const Item& it, int w0, int nw, int bad_slot) {
        const int32_t* btab =
            p.block_table + static_cast<int64_t>(it.b) * p.max_blocks + it.t0 / kPageTokens;
        for (int i = tid - w0 * 32; i < it.n_pages; i += nw * 32) {
            const int32_t id = btab[i];
            const bool ok = static_cast<uint32_t>(id) < static_cast<uint64_t>(p.num_blocks);
            if (!ok) {
                s_bad[bad_slot] = 1;
                atomicOr(p.work_counter + kStatusWord, kStatusBadBlock);
            }
            sblk[i] = ok ? id : 0;
        }
        if (warp - w0 < 2) {  // warp-uniform
            const int t8 = lane & 7, o = lane >> 3;
            const int hh = (warp - w0) * 4 + o;
            const bool hv = hh < group;
            const int64_t qoff =
                (static_cast<int64_t>(it.lb) * p.Hq + it.hkv * group + (hv ? hh : 0)) * D;
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
                for (int c = 0; c < 8; c++)
                    a[8 * i + c] = __uint_as_float(
                        __float_as_uint(tmp[c]) ^ sign_mask(p.signs, load_coord(t8, 8 * i + c)));
            }
            octet_fwht<E>(a, lane);
#pragma unroll
            for (int k = 0; k < E; k++)
                qs[qs_index(hh, t8 + 8 * k)] = hv ? a[k] * p.rsqrt_d * (p.scale * kLog2e) : 0.f;
        }
    };
    // warps that fold the per-warp states into the partial rows; when at least two warps are
    // left over they run the next item's prologue at the same time
    constexpr int NRED = (NH * NMT <= WARPS - 2) ? NH * NMT : WARPS;

#ifdef FTQ_TEST_WAIT_EXPIRY
    bool test_drop = blockIdx.x == 0 && warp == 5;
#endif
    draw_ticket();
    if (tid == 0) {
        s_next[1] = resolve_ticket(ticket);
        s_bad[0] = 0;
        s_bad[1] = 0;
    }
    __syncthreads();
    int item = s_next[1];
    int slot = 0;
    if (item < n_items) prologue(item_info(item), 0, WARPS, 0);
    while (item < n_items) {
        const Item cur = item_info(item);
        const int hkv = cur.hkv, layer = cur.layer;
        const int t0 = cur.t0, t1 = cur.t1, n_pages = cur.n_pages;
        // reserve this CTA's next item now: everybody knows it after the barrier, in time for the
        // early page requests at the end of the main loop
        if (tid == 0) { draw_ticket(); s_next[slot] = resolve_ticket(ticket); }
        __syncthreads();  // prologue of this item visible; ring and exchange area free
        const bool bad_item = s_bad[slot] != 0;   // (s_bad[slot ^ 1] collects the next item's)
        const int next = s_next[slot];
        slot ^= 1;

        // Q^T fragments: column n = g is head 4*hh + (g >> 1); k-block kb covers coordinates
        // (D/4)*tg + 4*kb + {0,1} (b0) and + {2,3} (b1)
        uint32_t qb[C::QSMEM ? 1 : NH][C::QSMEM ? 1 : NKB][2];
        // shared-memory copy of the fragments (QSMEM): [hh][kb][lane] x 8 bytes, in place of the
        // fp32 queries, which nobody reads again before the next item's prologue rewrites them
        const uint32_t qfrag = static_cast<uint32_t>(__cvta_generic_to_shared(qs));
        if constexpr (!C::QSMEM) {
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
        } else {
            constexpr int NE = NH * NKB * 32, PER = (NE + THREADS - 1) / THREADS;
            uint2 frag[PER];
#pragma unroll
            for (int i = 0; i < PER; i++) {
                const int e = tid + i * THREADS;
                const int ln = e & 31, kb = (e >> 5) % NKB, hh = (e >> 5) / NKB;
                if (e < NE) {
                    const float4 q4 = *reinterpret_cast<const float4*>(
                        qs + qs_index(4 * hh + (ln >> 3), (D / 4) * (ln & 3) + 4 * kb));
                    const __half2 lo = __floats2half2_rn(q4.x, q4.y);
                    const __half2 hi = __floats2half2_rn(q4.z, q4.w);
                    frag[i] = make_uint2(*reinterpret_cast<const uint32_t*>(&lo),
                                         *reinterpret_cast<const uint32_t*>(&hi));
                }
            }
            __syncthreads();
#pragma unroll
            for (int i = 0; i < PER; i++) {
                const int e = tid + i * THREADS;
                if (e < NE) reinterpret_cast<uint2*>(qs)[e] = frag[i];
            }
            __syncthreads();
        }

        // page address = head_base + block id * blk_stride (one 32 x 32 -> 64 bit multiply-add)
        const uint8_t* head_base =
            p.pool + layer * p.pool_layer_stride + static_cast<int64_t>(hkv) * C::PAGE_BYTES;
        const uint32_t blk_stride = static_cast<uint32_t>(p.Hkv) * C::PAGE_BYTES;

        // per lane: softmax state of head 4*hh + tg, O[head][(D/8)*g .. + D/8)
        float m_run[NH], l_run[NH], oacc[NH][NMT][4];
#pragma unroll
        for (int hh = 0; hh < NH; hh++) {
            m_run[hh] = -INFINITY;
            l_run[hh] = 0.f;
#pragma unroll
            for (int mt = 0; mt < NMT; mt++)
#pragma unroll
                for (int i = 0; i < 4; i++) oacc[hh][mt][i] = 0.f;
        }

        const uint32_t my_bars = bars + warp * C::RING * 8;
        const uint32_t my_ring = ring + warp * C::RING * C::PAGE_BYTES;
        // lane 0 starts the bulk copy of page pg into ring buffer rb (contiguous PAGE_BYTES)
        const uint64_t page_policy = l2_evict_first_policy();   // (pages are read once per step)
        auto issue_page = [&](int pg, int rb) {
            const uint8_t* page =
                head_base + static_cast<uint64_t>(static_cast<uint32_t>(sblk[pg])) * blk_stride;
            mbar_expect_tx(my_bars + rb * 8, C::PAGE_BYTES);
#ifdef FTQ_TEST_WAIT_EXPIRY
            if (test_drop) {   // (see kMbarSpinLimit)
                test_drop = false;
                return;
            }
#endif
            bulk_g2s_hint(my_ring + rb * C::PAGE_BYTES, page, C::PAGE_BYTES, my_bars + rb * 8, page_policy);
        };
        // same, for the first pages of a later item, whose block ids are not staged yet
        auto issue_page_of = [&](const Item& it2, int pg, int rb) {
            int32_t blk = p.block_table[static_cast<int64_t>(it2.b) * p.max_blocks +
                                        it2.t0 / kPageTokens + pg];
            if (static_cast<uint32_t>(blk) >= static_cast<uint64_t>(p.num_blocks)) blk = 0;
            const uint8_t* page = p.pool + it2.layer * p.pool_layer_stride +
                                  static_cast<uint64_t>(static_cast<uint32_t>(blk)) * blk_stride +
                                  static_cast<int64_t>(it2.hkv) * C::PAGE_BYTES;
            mbar_expect_tx(my_bars + rb * 8, C::PAGE_BYTES);
            bulk_g2s_hint(my_ring + rb * C::PAGE_BYTES, page, C::PAGE_BYTES, my_bars + rb * 8, page_policy);
        };
        // every lane copies its slices of the staged page into registers
        auto read_page = [&](Regs& r, int rb) {
            const uint32_t page = my_ring + rb * C::PAGE_BYTES;
            lds_slice<C::KSB>(page + koff, tg, r.k[0]);
            lds_slice<C::KSB>(page + koff + 2 * C::PDK, tg, r.k[1]);
            // register j holds page token 4tg + ((j + tg) & 3): the four lanes of a quad then read
            // rows of alternating parity in one instruction (2-way instead of 4-way bank conflict);
            // the P.V k-slots of a lane may hold its tokens in any order as long as the weights
            // follow (see the rotation of the transposed weights below).  The pool stores a V row
            // with its two halves exchanged for tokens with bit 1 set, so that the four rows a quad
            // reads in one instruction fall into distinct bank groups.
#pragma unroll
            for (int j = 0; j < 4; j++) {
                if constexpr (C::VSB % 4 == 0) lds_slice<C::VSB>(page + vrow[j], 0, r.v[j]);
                else lds_slice<C::VSB>(page + vrow[j], vidx[j], r.v[j]);
            }
            r.kn = lds64(page + noff);
            r.vn = lds64(page + noff + (C::OFF_VN - C::OFF_KN));
        };

        // S = K.Q^T of one page (two accumulator chains per head half)
        auto qk_scores = [&](const Regs& r, float (&c)[NH][2][4]) {
#pragma unroll
            for (int kb = 0; kb < NKB; kb++) {
                const uint32_t a0 = lut32(entry_addr<C::IWK>(r.k[0], 2 * kb, lk_lane));
                const uint32_t a1 = lut32(entry_addr<C::IWK>(r.k[1], 2 * kb, lk_lane));
                const uint32_t a2 = lut32(entry_addr<C::IWK>(r.k[0], 2 * kb + 1, lk_lane));
                const uint32_t a3 = lut32(entry_addr<C::IWK>(r.k[1], 2 * kb + 1, lk_lane));
#pragma unroll
                for (int hh = 0; hh < NH; hh++) {
                    uint32_t b0, b1;
                    if constexpr (C::QSMEM) {
                        const uint2 qv = lds64(qfrag + ((hh * NKB + kb) * 32 + lane) * 8);
                        b0 = qv.x; b1 = qv.y;
                    } else {
                        b0 = qb[hh][kb][0]; b1 = qb[hh][kb][1];
                    }
                    // (the first MMA of each of the two accumulator chains starts from zero)
                    if (kb < 2) mma_16816_z(c[hh][kb & 1], a0, a1, a2, a3, b0, b1);
                    else mma_16816(c[hh][kb & 1], a0, a1, a2, a3, b0, b1);
                }
            }
        };

        // online softmax per head (4*hh + tg) over the page's scores (base-2 exponent domain:
        // the queries carry log2(e)); the weights p * vnorm are rounded to fp16 and transposed
        // into the B operand of P.V.  FULL = all 16 tokens of the page are valid.
        auto softmax_update = [&](auto full_tag, const Regs& r, int pg, const float (&c)[NH][2][4],
                                  uint32_t (&pb)[NH][2][2]) {
            constexpr bool FULL = decltype(full_tag)::value;
            bool okA = true, okB = true;
            if constexpr (!FULL) {
                const int ntok = t1 - t0 - pg * kPageTokens;
                const int tokA = 4 * (g >> 1) + (g & 1);  // rows g, g+8 of S: tokens tokA, tokA + 2
                okA = tokA < ntok;
                okB = tokA + 2 < ntok;
            }
            const float kna = half_bits_to_float(__byte_perm(r.kn.x, 0u, sel_own));
            const float knb = half_bits_to_float(__byte_perm(r.kn.y, 0u, sel_own));
            float vna = half_bits_to_float(__byte_perm(r.vn.x, 0u, sel_own)) * p.inv_v_scale;
            float vnb = half_bits_to_float(__byte_perm(r.vn.y, 0u, sel_own)) * p.inv_v_scale;
            if constexpr (!FULL) {
                vna = okA ? vna : 0.f;
                vnb = okB ? vnb : 0.f;
            }
#pragma unroll
            for (int hh = 0; hh < NH; hh++) {
                float sa = (c[hh][0][0] + c[hh][1][0]) * kna;
                float sb = (c[hh][0][2] + c[hh][1][2]) * knb;
                if constexpr (!FULL) {
                    sa = okA ? sa : -INFINITY;
                    sb = okB ? sb : -INFINITY;
                }
                // Lazy reference maximum: the cross-lane maximum and the rescale run only when a
                // score exceeds the reference by more than kLazyMaxSlack (always on the first
                // page of an item, where it is -inf); weights stay below 2^kLazyMaxSlack.
                const float mloc = fmaxf(sa, sb);
                if (__any_sync(0xffffffffu, mloc > m_run[hh] + kLazyMaxSlack)) {
                    float mx = mloc;
                    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
                    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
                    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
                    const float m_new = fmaxf(m_run[hh], mx);  // finite: page token 0 is valid
                    const float corr = fast_exp2(m_run[hh] - m_new);  // 1 if unchanged, 0 from -inf
                    l_run[hh] *= corr;
#pragma unroll
                    for (int mt = 0; mt < NMT; mt++)
#pragma unroll
                        for (int i = 0; i < 4; i++) oacc[hh][mt][i] *= corr;
                    m_run[hh] = m_new;
                }
                const float pa = fast_exp2(sa - m_run[hh]);  // exp2(-inf) = 0 for masked tokens
                const float pbv = fast_exp2(sb - m_run[hh]);
                l_run[hh] += pa + pbv;
                const uint32_t ha = f2h_sat(pa * vna);
                const uint32_t hb = f2h_sat(pbv * vnb);
                // M[token row][column n], both columns of a head equal; transposed, lane (g, tg)
                // receives head g>>1, page tokens 4tg, 4tg+1 (first) and 4tg+2, 4tg+3 (second)
                uint32_t t0w = movmatrix_trans(__byte_perm(ha, 0u, 0x1010u));
                uint32_t t1w = movmatrix_trans(__byte_perm(hb, 0u, 0x1010u));
                // rotate the four 16-bit weights by tg positions to match the V register order
                if (tg & 2) { const uint32_t x = t0w; t0w = t1w; t1w = x; }
                {
                    const uint32_t sh = (tg & 1) * 16;
                    const uint32_t lo = __funnelshift_r(t0w, t1w, sh);
                    const uint32_t hi = __funnelshift_r(t1w, t0w, sh);
                    t0w = lo;
                    t1w = hi;
                }
                // column n = (head, parity): an even g keeps the weight in the low half (parity 0
                // rows of the k index), an odd g in the high half; the other half is zero
                pb[hh][0][0] = __byte_perm(t0w, 0u, sel_plo);
                pb[hh][0][1] = __byte_perm(t0w, 0u, sel_phi);
                pb[hh][1][0] = __byte_perm(t1w, 0u, sel_plo);
                pb[hh][1][1] = __byte_perm(t1w, 0u, sel_phi);
            }
        };

        // O^T += V^T.P^T : rows = d-pairs (D/16)*g + 2*mt + {0,1}, k = (token, parity)
        auto pv_accum = [&](const uint32_t (&v)[4][(C::VSB + 3) / 4], const uint32_t (&pb)[NH][2][2]) {
#pragma unroll
            for (int ks = 0; ks < 2; ks++)
#pragma unroll
                for (int mt = 0; mt < NMT; mt++) {
                    uint32_t a0, a1, a2, a3;
                    if constexpr (C::V2BYTE) {
                        // byte mt of a token's slice = its d-pairs 2mt and 2mt + 1
                        const uint2 lo = lut64(entry_addr<8>(v[2 * ks], mt, lv_lane));
                        const uint2 hi = lut64(entry_addr<8>(v[2 * ks + 1], mt, lv_lane));
                        a0 = lo.x; a1 = lo.y; a2 = hi.x; a3 = hi.y;
                    } else {
                        a0 = lut32(entry_addr<C::IWV>(v[2 * ks], 2 * mt, lv_lane));
                        a1 = lut32(entry_addr<C::IWV>(v[2 * ks], 2 * mt + 1, lv_lane));
                        a2 = lut32(entry_addr<C::IWV>(v[2 * ks + 1], 2 * mt, lv_lane));
                        a3 = lut32(entry_addr<C::IWV>(v[2 * ks + 1], 2 * mt + 1, lv_lane));
                    }
#pragma unroll
                    for (int hh = 0; hh < NH; hh++)
                        mma_16816(oacc[hh][mt], a0, a1, a2, a3, pb[hh][ks][0], pb[hh][ks][1]);
                }
        };

        // ---- main loop: the warp's pages; RING bulk copies stay in flight during the math.
        // Software pipeline: K.Q^T of page i+1 and P.V of page i are independent and sit in one
        // straight-line block, so their look-ups and MMAs overlap each other's latencies.
        {
            // (a warp whose wait has run out requests nothing any more: the mbarrier of the lost
            // copy never completes its phase, and arriving on it again would be an error)
            if (lane == 0 && !primed && !stalled) {
                // (when the exchange area aliases the ring, the previous item's merge wrote it
                // with ordinary stores)
                asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
#pragma unroll
                for (int r = 0; r < C::RING; r++)
                    if (warp + r * WARPS < n_pages) issue_page(warp + r * WARPS, (ring_it + r) % C::RING);
            }
            // stage page pg into registers and re-arm its ring buffer
            auto fetch = [&](Regs& r, int pg) {
                const int rb = ring_it % C::RING;
                ring_it++;
                if (!stalled && !mbar_wait(my_bars + rb * 8, (phase >> rb) & 1u)) stalled = true;
                phase ^= 1u << rb;
                read_page(r, rb);
                __syncwarp();  // every lane has its slices: the buffer may be refilled
                const int nxt = pg + C::RING * WARPS;
                if (lane == 0 && nxt < n_pages && !stalled) issue_page(nxt, rb);
            };
            // all pages but possibly the last one of the chunk are full (warp-uniform branch)
            auto softmax_page = [&](const Regs& r, int pg2, const float (&c2)[NH][2][4],
                                    uint32_t (&pb2)[NH][2][2]) {
                if ((pg2 + 1) * kPageTokens <= t1 - t0) softmax_update(std::true_type{}, r, pg2, c2, pb2);
                else softmax_update(std::false_type{}, r, pg2, c2, pb2);
            };
            Regs ra, rb_;
            uint32_t pba[NH][2][2], pbb[NH][2][2];
            float c[NH][2][4];
            int pg = warp;
            // (two head halves already give the scheduler independent work and the extra live
            // registers would spill: plain order there)
            constexpr bool kPipelined = (NH == 1 || (D == 256 && !C::QSMEM)) && !C::QSMEM && WARPS <= 16;
            if constexpr (!kPipelined) {
                for (; pg < n_pages; pg += WARPS) {
                    fetch(ra, pg);
                    qk_scores(ra, c);
                    softmax_page(ra, pg, c, pba);
                    pv_accum(ra.v, pba);
                }
            } else if (pg < n_pages) {
                fetch(ra, pg);
                qk_scores(ra, c);
                softmax_page(ra, pg, c, pba);
                while (true) {
                    // ra / pba hold page pg, scores done, P.V pending
                    if (pg + WARPS >= n_pages) { pv_accum(ra.v, pba); break; }
                    fetch(rb_, pg + WARPS);
                    qk_scores(rb_, c);
                    pv_accum(ra.v, pba);
                    softmax_page(rb_, pg + WARPS, c, pbb);
                    pg += WARPS;
                    if (pg + WARPS >= n_pages) { pv_accum(rb_.v, pbb); break; }
                    fetch(ra, pg + WARPS);
                    qk_scores(ra, c);
                    pv_accum(rb_.v, pbb);
                    softmax_page(ra, pg + WARPS, c, pba);
                    pg += WARPS;
                }
            }
        }

        // ---- this warp's ring is drained: request the first pages of the next item now, so that
        // they arrive while the merge below runs (only when the merge has its own exchange area)
        primed = false;
        if constexpr (C::SEP) {
            if (next < n_items) {
                const Item nx = item_info(next);
                if (lane == 0 && !stalled) {
#pragma unroll
                    for (int r = 0; r < C::RING; r++)
                        if (warp + r * WARPS < nx.n_pages)
                            issue_page_of(nx, warp + r * WARPS, (ring_it + r) % C::RING);
                }
                primed = true;
            }
        }

        // ---- fold the warps' states: every warp publishes (m, l, O), NRED warps reduce
#pragma unroll
        for (int hh = 0; hh < NH; hh++) {
            l_run[hh] += __shfl_xor_sync(0xffffffffu, l_run[hh], 4);
            l_run[hh] += __shfl_xor_sync(0xffffffffu, l_run[hh], 8);
            l_run[hh] += __shfl_xor_sync(0xffffffffu, l_run[hh], 16);
        }
        // a warp whose copy never arrived poisons its state (NaN propagates to the output)
        if (stalled) {
#pragma unroll
            for (int hh = 0; hh < NH; hh++) m_run[hh] = __int_as_float(0x7fc00000);
            if (lane == 0) atomicOr(p.work_counter + kStatusWord, kStatusWaitExpired);
        }
        __syncthreads();  // every warp is done with the ring: it becomes the exchange area
#pragma unroll
        for (int hh = 0; hh < NH; hh++) {
#pragma unroll
            for (int mt = 0; mt < NMT; mt++)
                xchg[((warp * NH + hh) * NMT + mt) * 32 + lane] = make_float4(
                    oacc[hh][mt][0], oacc[hh][mt][1], oacc[hh][mt][2], oacc[hh][mt][3]);
            if (g == 0) {
                xml[((warp * NH + hh) * 2 + 0) * 4 + tg] = m_run[hh];
                xml[((warp * NH + hh) * 2 + 1) * 4 + tg] = l_run[hh];
            }
        }
        __syncthreads();
        if (warp < NRED) {
            float* prow = partial_row(cur);
            for (int j = tid; j < NH * NMT * 32; j += NRED * 32) {
                const int ln = j & 31, mt = (j >> 5) % NMT, hh = j / (32 * NMT);
                const int tg_ = ln & 3, g_ = ln >> 2;
                float M = -INFINITY;
                bool nan = bad_item;
#pragma unroll
                for (int w2 = 0; w2 < WARPS; w2++) {
                    const float mw = xml[((w2 * NH + hh) * 2 + 0) * 4 + tg_];
                    nan |= mw != mw;   // (fmaxf drops a NaN operand)
                    M = fmaxf(M, mw);
                }
                float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
                float l = 0.f;
#pragma unroll
                for (int w2 = 0; w2 < WARPS; w2++) {
                    const float mw = xml[((w2 * NH + hh) * 2 + 0) * 4 + tg_];
                    if (mw != -INFINITY) {  // (NaN compares unequal: poison goes through)
                        const float f = fast_exp2(mw - M);
                        const float4 o = xchg[((w2 * NH + hh) * NMT + mt) * 32 + ln];
                        a.x = fmaf(o.x, f, a.x);
                        a.y = fmaf(o.y, f, a.y);
                        a.z = fmaf(o.z, f, a.z);
                        a.w = fmaf(o.w, f, a.w);
                        l = fmaf(xml[((w2 * NH + hh) * 2 + 1) * 4 + tg_], f, l);
                    }
                }
                const int h = 4 * hh + tg_;
                if (h < group) {
                    float* dst = prow + h * prow_head_stride;
                    *reinterpret_cast<float4*>(dst + (D / 8) * g_ + 4 * mt) = a;
                    if (g_ == 0 && mt == 0) {
                        // the partial rows carry natural-log maxima; NaN marks a poisoned item
                        dst[D] = nan ? __int_as_float(0x7fc00000) : M * kLn2;
                        dst[D + 1] = l;
                    }
                }
            }
        }
        if constexpr (NRED < WARPS) {
            if (warp >= NRED && next < n_items) prologue(item_info(next), NRED, WARPS - NRED, slot);
        } else {
            __syncthreads();
            if (next < n_items) prologue(item_info(next), 0, WARPS, slot);
        }
        if (tid == 0) s_bad[slot ^ 1] = 0;  // this item's flag: free for the item after next
        item = next;
    }
}

}  // namespace ftq
