// Paged split-KV decode attention, streaming form of the tensor-core kernel.
//
// Same arithmetic, tables, page layout and fragment maps as attn_mma_kernel
// (ftq_attn_mma.cuh: the fused formulation of
// src/fused_turboquant/kernels/triton_flash_decode.py:33-324 of the reference with
// the query rotation of hf/fused_cache.py:579-581 and the page-table walk of
// vllm_plugin/cache_ops.py:151-205 folded in).  What differs is the control
// structure: there is no CTA-wide barrier after the set-up.
//
//   * Every warp runs one continuous stream of pages that crosses work-item
//     boundaries: its two-deep ring of 1-D bulk copies (TMA, no multicast) is
//     refilled the moment a page has been copied to registers, whichever item
//     the next page belongs to.
//   * The page -> warp map of an item depends on its page count only (so the
//     order of every sum, hence every output bit, is independent of timing and
//     of which CTA runs the item): pages are dealt round-robin, except that
//     warps 0 and 1, the service warps, sit out the first SKIP rounds.
//   * When a warp has consumed its pages of item number s (s counts the items
//     of this CTA) it publishes its (m, l, O) state in shared memory and moves
//     on.  Warp 0 then waits for the W states, folds them in warp order and
//     writes the chunk's partial row; warp 1 prepares item s + 2 (next ticket
//     from the global counter, block ids, rotated query fragments) into the
//     metadata buffer item s has released.  Their smaller share of pages pays
//     for that.  Item metadata is double buffered; a warp can never be more
//     than two items ahead of the slowest one.
//   * The split-KV merge is part of the kernel: the CTA that delivers the last
//     chunk of a (layer, sequence, KV head) unit (a counter per unit) merges
//     the unit's partial rows, applies the inverse rotation
//     (core/hadamard.py:93-100) and stores the output (warp 0, right after the
//     fold).  No CTA ever waits for another CTA's work.
//   * The kernel clears its own counters: CTA 0 zeroes them and publishes the
//     launch's epoch, everybody checks for the epoch before the first atomic
//     on a counter (the first two items of a CTA are fixed, so that check is
//     long satisfied when it comes), the last CTA to leave takes the epoch out
//     again.  The launch is a programmatic dependent of whatever kernel
//     precedes it in the stream: the tables are built before
//     griddepcontrol.wait, global memory is touched only after it.
//   * The online softmax keeps a lazy reference maximum: the cross-lane maximum
//     and the rescale run only when some score exceeds the reference by more
//     than kLazyMaxSlack (base-2 exponent units); weights stay below
//     2^kLazyMaxSlack and are converted to fp16 with saturation.
//
// Every wait (mbarrier, shared-memory flags, epoch) is bounded; a wait that runs
// out marks the warp's state with NaN, which reaches the output instead of a
// hang, sets a bit in the call's status word, and the warp requests no further
// pages (the lost copy's mbarrier must not be arrived on again).
// Block ids outside [0, num_blocks) are never dereferenced: the item is
// computed on block 0 and its result replaced by NaN.
#pragma once

#include "ftq_attn_mma.cuh"

namespace ftq {

constexpr int kStreamMaxChunkPages = 512;   // 8192 tokens
constexpr int kFlagSpinLimit = 1 << 22;

template <int D, int BK, int BV, int NH>
struct StreamCfg {
    using M = MmaCfg<D, BK, BV, NH>;
    static constexpr int NKB = M::NKB, NMT = M::NMT;
    static constexpr bool BYTE = M::BYTE;
    static constexpr int PAGE_BYTES = M::PAGE_BYTES;
    static constexpr int RING = 2;
    static constexpr bool QSMEM = D == 256;                       // query fragments stay in shared memory
    static constexpr int QFRAG_BYTES = NH * NKB * 32 * 8;         // per metadata buffer
    static constexpr int QS_BYTES = 2 * 8 * (D + 16) * 4;         // fp32 rotated queries (2 scratch blocks)
    static constexpr int CTL_BYTES = 256 + 2 * 32 * 4;            // control words + per-warp addresses
    static constexpr int SBLK_BYTES = 2 * kStreamMaxChunkPages * 4;
    static constexpr int MISC_BYTES =
        M::SMALL_BYTES + CTL_BYTES + SBLK_BYTES + QS_BYTES + 2 * QFRAG_BYTES + 64;
    static constexpr int RING_W = RING * PAGE_BYTES + RING * 8;   // pages + their mbarriers
    static constexpr int XCHG_W = 32 * M::STATE_F4 * 16 + NH * 2 * 4 * 4;
    static constexpr int LIMIT = 227 * 1024;
    // rounds of an item's page deal that the two service warps sit out (their share of the
    // pages shrinks by what their service work costs; measured optimum)
#ifdef FTQ_SERVICE_SKIP
    static constexpr int SKIP = FTQ_SERVICE_SKIP;
#else
    static constexpr int SKIP = 7;
#endif
    // service warps: 2 = warp 0 folds and finishes units, warp 1 prepares; 1 = warp 0 does both
#ifdef FTQ_SERVICE_WARPS
    static constexpr int NSVC = FTQ_SERVICE_WARPS;
#else
    static constexpr int NSVC = 2;
#endif

    // First-fit placement (the same walk the kernel does): objects go before or after the
    // 64 KB-aligned table window.  Returns the bytes needed from `base`, or -1.
    __host__ __device__ static constexpr int plan(int warps, int base) {
        long long window = 0, free0 = base, end0 = base, free1 = base;
        if (BYTE) {
            window = (static_cast<long long>(base) + 65535) / 65536 * 65536;
            end0 = window;
            free1 = window + 65536;
        }
        const int sizes[3] = {MISC_BYTES, RING_W, XCHG_W};
        for (int kind = 0; kind < 3; kind++) {
            const int n = kind == 0 ? 1 : warps;
            for (int i = 0; i < n; i++) {
                const long long a0 = (free0 + 127) / 128 * 128;
                if (a0 + sizes[kind] <= end0) { free0 = a0 + sizes[kind]; continue; }
                const long long a1 = (free1 + 127) / 128 * 128;
                free1 = a1 + sizes[kind];
            }
        }
        const long long end = free1 > free0 ? free1 : free0;
        return static_cast<int>(end - base);
    }
    __host__ __device__ static constexpr int need(int warps) {
        int worst = 0;
        const int bases[5] = {0, 16, 1024, 2048, 4096};
        for (int i = 0; i < 5; i++) {
            const int n = plan(warps, bases[i]);
            worst = n > worst ? n : worst;
        }
        return worst + 128;
    }
    // one CTA per SM around a 64 KB byte table (16 warps when their rings and exchange slots fit
    // beside it, else 8); two 8-warp CTAs per SM with the small tables of 3- and 2-bit codes
    static constexpr int CTAS_PER_SM = BYTE ? 1 : 2;
    static constexpr int LIMIT_CTA = BYTE ? LIMIT : LIMIT / 2 - 1024;
    static constexpr int WARPS = (BYTE && need(16) <= LIMIT_CTA) ? 16 : 8;
    static constexpr int THREADS = 32 * WARPS;
    static constexpr int SMEM_BYTES = need(WARPS);
    static constexpr bool FITS = SMEM_BYTES <= LIMIT_CTA;
};

// Merge the chunk partials of one (layer, sequence, KV head) unit: normalise, rotate back
// (inverse_randomized_hadamard, core/hadamard.py:93-100) and store.  One warp; one octet per
// query head, four heads per pass.  Rows may have been written by other CTAs of this launch:
// they are read past L1.
template <int D>
__device__ __forceinline__ void stream_merge_unit(const AttnParams& p, int lb, int hkv, int group,
                                                  int nc, bool poison, int lane) {
    constexpr int E = D / kOctet;
    constexpr int ROW = D + 4;
    const int t = lane & 7, o = lane >> 3;
    for (int h0 = 0; h0 < group; h0 += 4) {
        const int h = h0 + o;
        const bool valid = h < group;
        const int64_t v = static_cast<int64_t>(lb) * p.Hq + hkv * group + (valid ? h : 0);
        const float* rows = p.partials + v * p.split.row_chunks * ROW;
        float M = -INFINITY;
        bool nan = poison;
        for (int c = 0; c < nc; c++) {
            const float mc = __ldcg(rows + c * ROW + D);
            nan |= mc != mc;  // (fmaxf drops a NaN operand)
            M = fmaxf(M, mc);
        }
        float a[E];
#pragma unroll
        for (int r = 0; r < E; r++) a[r] = 0.f;
        float L = 0.f;
        for (int c = 0; c < nc; c++) {
            const float mc = __ldcg(rows + c * ROW + D);
            if (mc == -INFINITY || mc != mc) continue;
            const float f = __expf(mc - M);
            L = fmaf(__ldcg(rows + c * ROW + D + 1), f, L);
#pragma unroll
            for (int i = 0; i < E / 8; i++) {
                const float4 x = __ldcg(reinterpret_cast<const float4*>(rows + c * ROW + 8 * (t + 8 * i)));
                const float4 y = __ldcg(reinterpret_cast<const float4*>(rows + c * ROW + 8 * (t + 8 * i)) + 1);
                a[8 * i + 0] = fmaf(x.x, f, a[8 * i + 0]);
                a[8 * i + 1] = fmaf(x.y, f, a[8 * i + 1]);
                a[8 * i + 2] = fmaf(x.z, f, a[8 * i + 2]);
                a[8 * i + 3] = fmaf(x.w, f, a[8 * i + 3]);
                a[8 * i + 4] = fmaf(y.x, f, a[8 * i + 4]);
                a[8 * i + 5] = fmaf(y.y, f, a[8 * i + 5]);
                a[8 * i + 6] = fmaf(y.z, f, a[8 * i + 6]);
                a[8 * i + 7] = fmaf(y.w, f, a[8 * i + 7]);
            }
        }
        float inv = L > 0.f ? 1.f / L : 0.f;
        if (nan) inv = __int_as_float(0x7fc00000);
#pragma unroll
        for (int r = 0; r < E; r++) a[r] *= inv;
        octet_fwht<E>(a, lane);
        if (valid) {
#pragma unroll
            for (int k = 0; k < E; k++) {
                const float r = a[k] * p.rsqrt_d;
                const float s = __uint_as_float(__float_as_uint(r) ^ sign_mask(p.signs, t + 8 * k));
                const int64_t idx = v * D + t + 8 * k;
                if (p.out_dtype == kBF16) static_cast<__nv_bfloat16*>(p.out)[idx] = __float2bfloat16_rn(s);
                else if (p.out_dtype == kF16) static_cast<__half*>(p.out)[idx] = __float2half_rn(s);
                else static_cast<float*>(p.out)[idx] = s;
            }
        }
    }
}

// Control words in shared memory (ints)
enum : int {
    kCtlReady = 0,      // highest item number whose metadata is complete
    kCtlReduced = 1,    // highest item number whose published states have been consumed
    kCtlItem = 2,       // [2] global item index (n_items: the stream has ended)
    kCtlPages = 4,      // [2]
    kCtlTokens = 6,     // [2] tokens of the chunk
    kCtlArrived = 8,    // [2] states published so far by items using this buffer (never reset)
    kCtlBad = 10,       // [2] a block id was out of range
    kCtlBase = 12,      // [2] x u64: pool address of (block 0, KV head) of the item's layer
    kCtlLayout = 16,    // set-up failed (shared-memory plan does not fit)
    kCtlChunk = 18,     // [2] the item's chunk index,
    kCtlHkv = 20,       // [2] KV head,
    kCtlLb = 22,        // [2] layer * B + sequence,
    kCtlSeqLen = 24,    // [2] and the sequence's length
    kCtlRingAddr = 64,  // [32] shared-window address of a warp's ring
    kCtlXchgAddr = 96,  // [32] ... of its exchange slot
};

template <int D, int BK, int BV, bool SHARED_LUT, int NH>
__global__ void __launch_bounds__(StreamCfg<D, BK, BV, NH>::THREADS, StreamCfg<D, BK, BV, NH>::CTAS_PER_SM)
attn_stream_kernel(const AttnParams p, int n_items) {
    using S = StreamCfg<D, BK, BV, NH>;
    using C = MmaCfg<D, BK, BV, NH>;
    constexpr int NKB = C::NKB, NMT = C::NMT, WARPS = S::WARPS, THREADS = S::THREADS;
    constexpr int E = D / kOctet;
    constexpr int ROW = D + 4;
    constexpr int PAGE_BYTES = C::PAGE_BYTES;
    using Regs = PageRegs<C::KSB, C::VSB>;

    extern __shared__ __align__(16) uint8_t smem_raw[];
    const uint32_t sbase = static_cast<uint32_t>(__cvta_generic_to_shared(smem_raw));
    uint32_t window = 0, free0 = sbase, end0 = sbase, free1 = sbase;
    if constexpr (C::BYTE) {
        window = (sbase + 65535u) & ~65535u;
        end0 = window;
        free1 = window + 65536u;
    }
    auto take = [&](uint32_t bytes) {
        uint32_t a = (free0 + 127u) & ~127u;
        if (a + bytes <= end0) { free0 = a + bytes; return a; }
        a = (free1 + 127u) & ~127u;
        free1 = a + bytes;
        return a;
    };
    auto gptr = [&](uint32_t saddr) { return smem_raw + (saddr - sbase); };

    // the next kernel of the stream may start its own set-up as soon as every CTA got here
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
    const int g = lane >> 2, tg = lane & 3;
    const bool odd = g & 1;
    const int group = p.Hq / p.Hkv;  // <= 4 * NH
    uint32_t sel_own = odd ? 0x4432u : 0x4410u;
    uint32_t sel_plo = odd ? 0x1044u : 0x4410u;
    uint32_t sel_phi = odd ? 0x3244u : 0x4432u;
    asm volatile("" : "+r"(sel_own), "+r"(sel_plo), "+r"(sel_phi));

    // ---- misc block: small tables, control words, block ids, query scratch and fragments
    const uint32_t misc = take(S::MISC_BYTES);
    uint32_t tk_small = 0, tv_small = 0, cur = misc;
    if constexpr (C::SMALL_ALIGN > 0) {
        cur = (misc + C::SMALL_ALIGN - 1) & ~static_cast<uint32_t>(C::SMALL_ALIGN - 1);
        if (C::TKS >= C::TVS) { tk_small = cur; tv_small = cur + C::TKS; }
        else { tv_small = cur; tk_small = cur + C::TVS; }
        cur += C::TKS + C::TVS;
        if (SHARED_LUT) tv_small = tk_small;
    }
    cur = (cur + 15u) & ~15u;
    volatile int* ctl = reinterpret_cast<volatile int*>(gptr(cur));
    cur += S::CTL_BYTES;
    int32_t* sblk = reinterpret_cast<int32_t*>(gptr(cur));           // [2][kStreamMaxChunkPages]
    cur += S::SBLK_BYTES;
    float* qs = reinterpret_cast<float*>(gptr(cur));                  // [8][D + 16]
    cur += S::QS_BYTES;
    const uint32_t qfrag = cur;                                       // [2][NH][NKB][32] x 8 bytes
    uint2* qfrag_g = reinterpret_cast<uint2*>(gptr(cur));

    // per-warp rings and exchange slots (thread 0 walks the placement for everybody)
    if (tid == 0) {
        for (int w = 0; w < WARPS; w++) ctl[kCtlRingAddr + w] = static_cast<int>(take(S::RING_W));
        for (int w = 0; w < WARPS; w++) ctl[kCtlXchgAddr + w] = static_cast<int>(take(S::XCHG_W));
        const uint32_t end = free1 > free0 ? free1 : free0;
        ctl[kCtlLayout] = end > sbase + S::SMEM_BYTES ? 1 : 0;
        ctl[kCtlReady] = 1;   // items 0 and 1 are prepared before the barrier that opens the stream
        ctl[kCtlReduced] = -1;
        ctl[kCtlArrived] = 0;
        ctl[kCtlArrived + 1] = 0;
    }

    // ---- once per CTA: dequantisation tables (same contents as attn_mma_kernel's)
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
                const int sh = 4 * (col & 1);
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
    // (pinning these two as well made the compiler spill in the page loop)
    const uint32_t lk_lane = (BK == 4 ? window : tk_small) | (lane * 4);
    const uint32_t lv_lane =
        C::V2BYTE ? (window | 128u | ((lane & 15) * 8))
                  : ((BV == 4 ? (window | (SHARED_LUT ? 0u : 128u)) : tv_small) | (lane * 4));
    // Everything up to here touched shared memory only.  From here on the kernel reads and writes
    // global memory that the kernel before it in the stream may still be using (the workspace).
    asm volatile("griddepcontrol.wait;\n" ::: "memory");
    unsigned long long* epoch_word = reinterpret_cast<unsigned long long*>(p.work_counter + 2);
    if (blockIdx.x == 0) {
        for (int i = tid; i < p.n_units; i += THREADS) p.unit_counter[i] = 0;
        if (tid == 0) {
            p.work_counter[0] = 0;
            p.work_counter[1] = 0;
            p.work_counter[kStatusWord] = 0;
        }
    }
    __syncthreads();
    if (blockIdx.x == 0 && tid == 0) {
        __threadfence();
        asm volatile("st.release.gpu.global.u64 [%0], %1;\n" ::"l"(epoch_word), "l"(p.epoch) : "memory");
    }
    if (ctl[kCtlLayout]) return;  // cannot happen for a configuration the launcher accepts
    const uint32_t my_ring = static_cast<uint32_t>(ctl[kCtlRingAddr + warp]);
    const uint32_t my_bars = my_ring + S::RING * PAGE_BYTES;
    float4* my_xchg = reinterpret_cast<float4*>(gptr(static_cast<uint32_t>(ctl[kCtlXchgAddr + warp])));
    if (lane == 0) {
#pragma unroll
        for (int r = 0; r < S::RING; r++) mbar_init(my_bars + r * 8, 1);
    }
    mbar_fence_init();

    auto qs_index = [](int head, int coord) {
        return head * (D + 16) + (coord / (D / 4)) * (D / 4 + 4) + coord % (D / 4);
    };
    struct Item { int chunk, hkv, lb, layer, b, t0, t1, n_pages, seq_len; };
    auto item_info = [&](int item) {
        Item it;
        // (items are numbered region by region: see SplitPlan)
        const SplitRegion& rg = region_of_item(p.split, item);
        const int j = item - rg.first_item;
        const int q = static_cast<int>(fast_div(static_cast<uint32_t>(j), rg.div_chunks));
        it.chunk = j - q * rg.chunks;
        const int rest = rg.first_unit + q;
        const int ct = rg.chunk_tokens;
        it.lb = static_cast<int>(fast_div(static_cast<uint32_t>(rest), p.div_hkv));
        it.hkv = rest - it.lb * p.Hkv;
        it.layer = static_cast<int>(fast_div(static_cast<uint32_t>(it.lb), p.div_b));
        it.b = it.lb - it.layer * p.B;
        it.seq_len = p.seq_lens[it.b];
        it.t0 = it.chunk * ct;
        it.t1 = min(it.seq_len, it.t0 + ct);
        it.n_pages = (it.t1 - it.t0 + kPageTokens - 1) / kPageTokens;
        return it;
    };
    const int64_t prow_head_stride = static_cast<int64_t>(p.split.row_chunks) * ROW;
    const uint32_t blk_stride = static_cast<uint32_t>(p.Hkv) * PAGE_BYTES;

    // bounded polls of a shared-memory word (all lanes read the same word)
    auto wait_ge = [&](int word, int value) {
        for (int i = 0; i < kFlagSpinLimit; i++) {
            if (ctl[word] >= value) { __threadfence_block(); return true; }
            __nanosleep(40);
        }
        return false;
    };

    // ---- metadata of one item (run by a whole warp): resolve the ticket to the next item with
    // tokens, stage its block ids, rotate and pre-scale its queries into MMA fragments
    bool stalled = false;   // a bounded wait of this warp ran out: its results are replaced by NaN
    // states that must have been published in buffer seq & 1 once item number seq is complete
    auto arrivals_due = [&](int seq) { return WARPS * ((seq >> 1) + 1); };
    // the counters are valid once CTA 0 has published this launch's epoch (checked before a warp's
    // first atomic on any of them; by then it has normally been there for a long time)
    bool epoch_seen = false;
    auto await_epoch = [&]() {
        if (epoch_seen) return;
        epoch_seen = true;
        for (int i = 0; i < kFlagSpinLimit; i++) {
            unsigned long long v;
            asm volatile("ld.acquire.gpu.global.u64 %0, [%1];\n" : "=l"(v) : "l"(epoch_word) : "memory");
            if (v == p.epoch) return;
            __nanosleep(100);
        }
        stalled = true;
    };
    // work items: the first two of a CTA are fixed, the rest are drawn from the counter
    auto draw_item = [&]() {
        await_epoch();
        int t = 0;
        if (lane == 0) t = 2 * static_cast<int>(gridDim.x) + atomicAdd(p.work_counter, 1);
        return __shfl_sync(0xffffffffu, t, 0);
    };

    // `qsw` is a scratch row block for the fp32 rotated queries (two exist, so that two warps
    // can run this at start-up).  With wait_seq >= 0 the buffer still belongs to item number
    // wait_seq: nothing is written before every warp has published that item and the fold
    // service has read its fields.
    auto prepare = [&](int buf, int ticket, float* qsw, int wait_seq) {
        // (every lane walks the same tickets; lane 0 draws and writes)
        int item = ticket;
        Item it{};
        while (item < n_items) {
            it = item_info(item);
            if (it.t0 < it.t1) break;
            if (it.chunk == 0) {
                // a sequence without tokens: its outputs are zero (softmax over nothing)
                for (int h = 0; h < group; h++) {
                    const int64_t v = static_cast<int64_t>(it.lb) * p.Hq + it.hkv * group + h;
                    for (int d = lane; d < D; d += 32) {
                        if (p.out_dtype == kBF16)
                            static_cast<__nv_bfloat16*>(p.out)[v * D + d] = __float2bfloat16_rn(0.f);
                        else if (p.out_dtype == kF16)
                            static_cast<__half*>(p.out)[v * D + d] = __float2half_rn(0.f);
                        else static_cast<float*>(p.out)[v * D + d] = 0.f;
                    }
                }
            }
            item = draw_item();
        }
        if (wait_seq >= 0) {
            if (!stalled && !wait_ge(kCtlArrived + buf, arrivals_due(wait_seq))) stalled = true;
            if (!stalled && !wait_ge(kCtlReduced, wait_seq)) stalled = true;
        }
        if (item >= n_items) {
            if (lane == 0) {
                ctl[kCtlItem + buf] = n_items;
                ctl[kCtlPages + buf] = 0;
                ctl[kCtlTokens + buf] = 0;
                ctl[kCtlBad + buf] = 0;
            }
            __syncwarp();
            return;
        }
        const int32_t* btab =
            p.block_table + static_cast<int64_t>(it.b) * p.max_blocks + it.t0 / kPageTokens;
        bool bad = false;
        for (int i = lane; i < it.n_pages; i += 32) {
            const int32_t id = btab[i];
            const bool ok = static_cast<uint32_t>(id) < static_cast<uint32_t>(p.num_blocks);
            bad |= !ok;
            sblk[buf * kStreamMaxChunkPages + i] = ok ? id : 0;
        }
        bad = __any_sync(0xffffffffu, bad);
        if (bad) {
            await_epoch();   // (the status word is cleared with the counters)
            if (lane == 0) atomicOr(p.work_counter + kStatusWord, kStatusBadBlock);
        }
        const int t8 = lane & 7, o = lane >> 3;
#pragma unroll
        for (int pass = 0; pass < NH; pass++) {
            const int hh = pass * 4 + o;
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
                for (int c2 = 0; c2 < 8; c2++)
                    a[8 * i + c2] = __uint_as_float(
                        __float_as_uint(tmp[c2]) ^ sign_mask(p.signs, load_coord(t8, 8 * i + c2)));
            }
            octet_fwht<E>(a, lane);
#pragma unroll
            for (int k = 0; k < E; k++)
                qsw[qs_index(hh, t8 + 8 * k)] = hv ? a[k] * p.rsqrt_d * (p.scale * kLog2e) : 0.f;
        }
        __syncwarp();
        // fragments: column n = g is head 4*hh + (g >> 1); k-block kb covers coordinates
        // (D/4)*tg + 4*kb + {0,1} (b0) and + {2,3} (b1)
#pragma unroll 4
        for (int i2 = 0; i2 < NH * NKB; i2++) {
            const int hh = i2 / NKB, kb = i2 % NKB;
            const float4 q4 = *reinterpret_cast<const float4*>(
                qsw + qs_index(4 * hh + (lane >> 3), (D / 4) * (lane & 3) + 4 * kb));
            const __half2 lo = __floats2half2_rn(q4.x, q4.y);
            const __half2 hi = __floats2half2_rn(q4.z, q4.w);
            qfrag_g[(buf * NH * NKB + i2) * 32 + lane] =
                make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
        }
        if (lane == 0) {
            ctl[kCtlItem + buf] = item;
            ctl[kCtlPages + buf] = it.n_pages;
            ctl[kCtlTokens + buf] = it.t1 - it.t0;
            ctl[kCtlBad + buf] = bad ? 1 : 0;
            ctl[kCtlChunk + buf] = it.chunk;
            ctl[kCtlHkv + buf] = it.hkv;
            ctl[kCtlLb + buf] = it.lb;
            ctl[kCtlSeqLen + buf] = it.seq_len;
            const uint8_t* base = p.pool + it.layer * p.pool_layer_stride +
                                  static_cast<int64_t>(it.hkv) * PAGE_BYTES;
            *reinterpret_cast<volatile unsigned long long*>(const_cast<int*>(ctl + kCtlBase + 2 * buf)) =
                reinterpret_cast<unsigned long long>(base);
        }
        __syncwarp();
    };

    // ---- the first two items of this CTA: blockIdx.x (warp 0) and blockIdx.x + gridDim.x
    // (warp 1); everybody may start on them after the barrier
    if (warp < 2) {
        const int t = static_cast<int>(blockIdx.x) + warp * static_cast<int>(gridDim.x);
        prepare(warp, t, qs + warp * (8 * (D + 16)), -1);
        __threadfence_block();
    }
    __syncthreads();

    // ---- per-warp stream state (all warp-uniform)
    int gseq = 0;                       // item the next page request belongs to
    int cseq = 0;                       // item number the arithmetic state belongs to
    bool g_end = ctl[kCtlItem + 0] >= n_items;
    bool deferred = false;              // a request was handed back: later ones must not overtake it

    // Pages of an item are dealt round-robin, except that the two service warps (warp 0 folds
    // the published states and finishes units, warp 1 prepares the item after next, see below)
    // sit out the first SKIP rounds.  Warp w's pages: w - NSVC, then steps of W - NSVC while the
    // page lies in the first SKIP - 1 rounds, steps of W after that; a service warp starts at
    // (W - NSVC) * SKIP + w.  The map depends on nothing but the page count, so the order of
    // every floating-point sum is fixed.
    constexpr int NSVC = S::NSVC;
    constexpr int WC = S::SKIP > 0 ? WARPS - NSVC : WARPS;
    constexpr int THR = S::SKIP > 0 ? WC * (S::SKIP - 1) : 0;
    const int g_first = S::SKIP > 0 ? (warp < NSVC ? WC * S::SKIP + warp : warp - NSVC) : warp;
    const uint64_t page_policy = l2_evict_first_policy();
#ifdef FTQ_TEST_WAIT_EXPIRY
    bool test_drop = blockIdx.x == 0 && warp == 5;   // (see kMbarSpinLimit)
#endif
    int g_next = g_first;                                   // next page of item gseq for this warp
    int g_lim = g_end ? 0 : ctl[kCtlPages + 0];             // its page count (0: nothing to take)
    // request the next page of the stream into ring buffer rb; returns its index within item
    // gseq, -1 at the end of the stream, -2 when the request is handed back
    auto grab = [&](int rb) {
        int pg = g_next;
        if (pg < g_lim) {
            g_next += pg < THR ? WC : WARPS;
        } else {
            // this warp's pages of item gseq are used up (or nothing may be taken)
            pg = deferred ? -2 : -1;
            while (!g_end && !deferred) {
                if (g_next < g_lim) {
                    pg = g_next;
                    g_next += pg < THR ? WC : WARPS;
                    break;
                }
                // Item gseq + 1 is prepared once every warp has published its state of item
                // gseq - 1: only wait for it once this warp has done so (cseq >= gseq);
                // otherwise hand the decision back to the consumer.
                if (gseq > cseq) { pg = -2; deferred = true; break; }
                gseq++;
                g_next = g_first;
                if (!stalled && !wait_ge(kCtlReady, gseq)) stalled = true;
                g_end = ctl[kCtlItem + (gseq & 1)] >= n_items;
                g_lim = g_end ? 0 : ctl[kCtlPages + (gseq & 1)];
            }
            if (pg < 0) g_lim = 0;   // end / handed back: the fast check above must keep failing
        }
        // (a warp whose wait has run out requests nothing any more: the mbarrier of the lost copy
        // never completes its phase, and arriving on it again would be an error)
        if (pg >= 0 && lane == 0 && !stalled) {
            const int buf = gseq & 1;
            const unsigned long long base =
                *reinterpret_cast<volatile unsigned long long*>(const_cast<int*>(ctl + kCtlBase + 2 * buf));
            const uint8_t* page = reinterpret_cast<const uint8_t*>(base) +
                static_cast<uint64_t>(static_cast<uint32_t>(sblk[buf * kStreamMaxChunkPages + pg])) * blk_stride;
            mbar_expect_tx(my_bars + rb * 8, PAGE_BYTES);
#ifdef FTQ_TEST_WAIT_EXPIRY
            if (!test_drop)
#endif
            bulk_g2s_hint(my_ring + rb * PAGE_BYTES, page, PAGE_BYTES, my_bars + rb * 8, page_policy);
        }
#ifdef FTQ_TEST_WAIT_EXPIRY
        if (pg >= 0) test_drop = false;
#endif
        return pg;
    };

    // ---- per-item arithmetic state
    int ntok_item = ctl[kCtlTokens + 0];
    uint32_t qb[S::QSMEM ? 1 : NH][S::QSMEM ? 1 : NKB][2];
    uint32_t qf_item = qfrag;  // fragment base of the current item (QSMEM)
    float m_run[NH], l_run[NH], oacc[NH][NMT][4];
    auto load_ctx = [&](int seq) {
        const int buf = seq & 1;
        ntok_item = ctl[kCtlTokens + buf];
        qf_item = qfrag + buf * S::QFRAG_BYTES;
        if constexpr (!S::QSMEM) {
#pragma unroll
            for (int hh = 0; hh < NH; hh++)
#pragma unroll
                for (int kb = 0; kb < NKB; kb++) {
                    const uint2 v = lds64(qf_item + ((hh * NKB + kb) * 32 + lane) * 8);
                    qb[hh][kb][0] = v.x;
                    qb[hh][kb][1] = v.y;
                }
        }
    };
    auto reset_state = [&]() {
#pragma unroll
        for (int hh = 0; hh < NH; hh++) {
            m_run[hh] = -INFINITY;
            l_run[hh] = 0.f;
#pragma unroll
            for (int mt = 0; mt < NMT; mt++)
#pragma unroll
                for (int i = 0; i < 4; i++) oacc[hh][mt][i] = 0.f;
        }
    };

    // a lane's slices of a staged page: keys + both norm vectors, and values
    // Lane constants of the page reads (like the table bases and byte selectors above) are made
    // opaque to the compiler -- an empty asm that "modifies" them: left alone it recomputes them
    // for every page rather than spend registers on them, ~25 instructions per page (measured +4 %).
    uint32_t koff = (4 * (g >> 1) + (g & 1)) * C::PDK;   // key row rho(g)
    uint32_t noff = C::OFF_KN + 8 * (g >> 1);
    asm volatile("" : "+r"(koff), "+r"(noff));
    auto read_keys = [&](Regs& r, uint32_t page) {
        lds_slice<C::KSB>(page + koff, tg, r.k[0]);
        lds_slice<C::KSB>(page + koff + 2 * C::PDK, tg, r.k[1]);
        r.kn = lds64(page + noff);
        r.vn = lds64(page + noff + (C::OFF_VN - C::OFF_KN));
    };
    // this lane's four value slices inside a page: register j holds page token 4tg + ((j + tg) & 3),
    // slice g with its halves exchanged for tokens with bit 1 set (the rotation by tg and the
    // exchanged halves keep the quad's reads conflict-free).  vrow = byte offset of the token's
    // row (plus the slice where slices are whole words), vidx = slice index otherwise.
    uint32_t vrow[4];
    int vidx[4];
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const int u = (j + tg) & 3;
        const int slice = g ^ ((u & 2) << 1);
        vrow[j] = C::OFF_VC + (4 * tg + u) * C::PDV + (C::VSB % 4 == 0 ? slice * C::VSB : 0);
        vidx[j] = C::VSB % 4 == 0 ? 0 : slice;
        asm volatile("" : "+r"(vrow[j]));
        if constexpr (C::VSB % 4 != 0) asm volatile("" : "+r"(vidx[j]));
    }
    auto read_values = [&](Regs& r, uint32_t page) {
#pragma unroll
        for (int j = 0; j < 4; j++) {
            if constexpr (C::VSB % 4 == 0) lds_slice<C::VSB>(page + vrow[j], 0, r.v[j]);
            else lds_slice<C::VSB>(page + vrow[j], vidx[j], r.v[j]);
        }
    };

    // S = K.Q^T of one page (two accumulator chains per head half, the first MMA of a chain
    // starts from zero)
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
                if constexpr (S::QSMEM) {
                    const uint2 qv = lds64(qf_item + ((hh * NKB + kb) * 32 + lane) * 8);
                    b0 = qv.x; b1 = qv.y;
                } else {
                    b0 = qb[hh][kb][0]; b1 = qb[hh][kb][1];
                }
                if (kb < 2) mma_16816_z(c[hh][kb & 1], a0, a1, a2, a3, b0, b1);
                else mma_16816(c[hh][kb & 1], a0, a1, a2, a3, b0, b1);
            }
        }
    };

    // online softmax with a lazy reference maximum; the weights p * vnorm are rounded to fp16
    // and transposed into the B operand of P.V.  FULL = all 16 tokens of the page are valid.
    auto softmax_update = [&](auto full_tag, const Regs& r, int pg, const float (&c)[NH][2][4],
                              uint32_t (&pb)[NH][2][2]) {
        constexpr bool FULL = decltype(full_tag)::value;
        bool okA = true, okB = true;
        if constexpr (!FULL) {
            const int ntok = ntok_item - pg * kPageTokens;
            const int tokA = 4 * (g >> 1) + (g & 1);
            okA = tokA < ntok;
            okB = tokA + 2 < ntok;
        }
        const float kna = half_bits_to_float(__byte_perm(r.kn.x, 0u, sel_own));
        const float knb = half_bits_to_float(__byte_perm(r.kn.y, 0u, sel_own));
        // (the factor that undoes the scaling of the value centroids is applied once per item,
        // when the state is published)
        float vna = half_bits_to_float(__byte_perm(r.vn.x, 0u, sel_own));
        float vnb = half_bits_to_float(__byte_perm(r.vn.y, 0u, sel_own));
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
            const float mloc = fmaxf(sa, sb);
            // the reference moves only when a score leaves the slack above it (always on the
            // first page of an item, where it is -inf)
            if (__any_sync(0xffffffffu, mloc > m_run[hh] + kLazyMaxSlack)) {
                float mx = mloc;
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
                const float m_new = fmaxf(m_run[hh], mx);  // finite: page token 0 is valid
                const float corr = fast_exp2(m_run[hh] - m_new);
                l_run[hh] *= corr;
#pragma unroll
                for (int mt = 0; mt < NMT; mt++)
#pragma unroll
                    for (int i = 0; i < 4; i++) oacc[hh][mt][i] *= corr;
                m_run[hh] = m_new;
            }
            const float pa = fast_exp2(sa - m_run[hh]);
            const float pbv = fast_exp2(sb - m_run[hh]);
            l_run[hh] += pa + pbv;
            const uint32_t ha = f2h_sat(pa * vna);
            const uint32_t hb = f2h_sat(pbv * vnb);
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
    };

    auto pv_accum = [&](const uint32_t (&v)[4][(C::VSB + 3) / 4], const uint32_t (&pb)[NH][2][2]) {
#pragma unroll
        for (int ks = 0; ks < 2; ks++)
#pragma unroll
            for (int mt = 0; mt < NMT; mt++) {
                uint32_t a0, a1, a2, a3;
                if constexpr (C::V2BYTE) {
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

    // ---- fold service for item number seq (warp 0, after it has published its own state): fold
    // the W states in warp order, write the chunk's partial row, and finish the unit when this
    // was its last chunk
    auto serve_fold = [&](int seq) {
        const int buf = seq & 1;
        if (!stalled && !wait_ge(kCtlArrived + buf, arrivals_due(seq))) stalled = true;
        const bool bad = ctl[kCtlBad + buf] != 0 || stalled;
        const int chunk = ctl[kCtlChunk + buf], hkv = ctl[kCtlHkv + buf], lb = ctl[kCtlLb + buf];
        const int seq_len = ctl[kCtlSeqLen + buf];
        float* prow = p.partials +
            ((static_cast<int64_t>(lb) * p.Hq + hkv * group) * p.split.row_chunks + chunk) * ROW;
        // lane (g, tg) folds what it would own as a compute lane: O[head 4hh + tg][(D/8)g ..)
        float M[NH];
        bool nan = bad;
#pragma unroll
        for (int hh = 0; hh < NH; hh++) M[hh] = -INFINITY;
#pragma unroll 4
        for (int w2 = 0; w2 < WARPS; w2++) {
            const float* xm = reinterpret_cast<const float*>(
                gptr(static_cast<uint32_t>(ctl[kCtlXchgAddr + w2]) + 32 * C::STATE_F4 * 16));
#pragma unroll
            for (int hh = 0; hh < NH; hh++) {
                const float mw = xm[(hh * 2 + 0) * 4 + tg];
                nan |= mw != mw;
                M[hh] = fmaxf(M[hh], mw);
            }
        }
        float4 acc[NH][NMT];
        float l[NH];
#pragma unroll
        for (int hh = 0; hh < NH; hh++) {
            l[hh] = 0.f;
#pragma unroll
            for (int mt = 0; mt < NMT; mt++) acc[hh][mt] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll 2
        for (int w2 = 0; w2 < WARPS; w2++) {
            const uint32_t xa = static_cast<uint32_t>(ctl[kCtlXchgAddr + w2]);
            const float* xm = reinterpret_cast<const float*>(gptr(xa + 32 * C::STATE_F4 * 16));
            const float4* xo = reinterpret_cast<const float4*>(gptr(xa));
#pragma unroll
            for (int hh = 0; hh < NH; hh++) {
                const float mw = xm[(hh * 2 + 0) * 4 + tg];
                if (mw != -INFINITY) {   // (uniform over the warp: a state is empty for all heads)
                    const float f = fast_exp2(mw - M[hh]);
                    l[hh] = fmaf(xm[(hh * 2 + 1) * 4 + tg], f, l[hh]);
#pragma unroll
                    for (int mt = 0; mt < NMT; mt++) {
                        const float4 o = xo[(hh * NMT + mt) * 32 + lane];
                        acc[hh][mt].x = fmaf(o.x, f, acc[hh][mt].x);
                        acc[hh][mt].y = fmaf(o.y, f, acc[hh][mt].y);
                        acc[hh][mt].z = fmaf(o.z, f, acc[hh][mt].z);
                        acc[hh][mt].w = fmaf(o.w, f, acc[hh][mt].w);
                    }
                }
            }
        }
        __syncwarp();
        __threadfence_block();
        if (lane == 0) ctl[kCtlReduced] = seq;   // the exchange slots may be rewritten
#pragma unroll
        for (int hh = 0; hh < NH; hh++) {
            const int h = 4 * hh + tg;
            if (h < group) {
                float* dst = prow + h * prow_head_stride;
#pragma unroll
                for (int mt = 0; mt < NMT; mt++)
                    *reinterpret_cast<float4*>(dst + (D / 8) * g + 4 * mt) = acc[hh][mt];
                if (g == 0) {
                    dst[D] = nan ? __int_as_float(0x7fc00000) : M[hh] * kLn2;  // natural-log maxima
                    dst[D + 1] = l[hh];
                }
            }
        }
        // has every chunk of this (layer, sequence, KV head) unit been delivered?
        const SplitRegion& rg = region_of_unit(p.split, lb * p.Hkv + hkv);
        const int nc = min(rg.chunks, (seq_len + rg.chunk_tokens - 1) / rg.chunk_tokens);
        bool last = true;
        if (nc > 1) {
            __threadfence();
            __syncwarp();
            int old = 0;
            await_epoch();
            if (lane == 0) old = atomicAdd(p.unit_counter + lb * p.Hkv + hkv, 1);
            last = __shfl_sync(0xffffffffu, old, 0) == nc - 1;
            if (last) __threadfence();
        } else {
            __threadfence_block();   // the row was written by this warp alone
            __syncwarp();
        }
        if (last) stream_merge_unit<D>(p, lb, hkv, group, nc, false, lane);
    };

    // ---- prepare service for item number seq (warp 1, after it has published its own state):
    // once every warp is done with item seq, its metadata buffer takes item seq + 2
    auto serve_prepare = [&](int seq) {
        const int t = draw_item();
        prepare(seq & 1, t, qs, seq);
        __threadfence_block();
        if (lane == 0) ctl[kCtlReady] = seq + 2;
    };

    // publish this warp's state of item number seq, then serve the item if it is this warp's turn
    auto finish_item = [&](int seq) {
#pragma unroll
        for (int hh = 0; hh < NH; hh++) {
            l_run[hh] += __shfl_xor_sync(0xffffffffu, l_run[hh], 4);
            l_run[hh] += __shfl_xor_sync(0xffffffffu, l_run[hh], 8);
            l_run[hh] += __shfl_xor_sync(0xffffffffu, l_run[hh], 16);
        }
        if (!stalled && !wait_ge(kCtlReduced, seq - 1)) stalled = true;
        float* xml = reinterpret_cast<float*>(my_xchg + 32 * C::STATE_F4);
#pragma unroll
        for (int hh = 0; hh < NH; hh++) {
            if (m_run[hh] != -INFINITY) {  // (warp-uniform per head half: the reference is shared)
#pragma unroll
                for (int mt = 0; mt < NMT; mt++)
                    my_xchg[(hh * NMT + mt) * 32 + lane] = make_float4(
                        oacc[hh][mt][0] * p.inv_v_scale, oacc[hh][mt][1] * p.inv_v_scale,
                        oacc[hh][mt][2] * p.inv_v_scale, oacc[hh][mt][3] * p.inv_v_scale);
            }
            if (g == 0) {
                xml[(hh * 2 + 0) * 4 + tg] = stalled ? __int_as_float(0x7fc00000) : m_run[hh];
                xml[(hh * 2 + 1) * 4 + tg] = l_run[hh];
            }
        }
        __syncwarp();
        __threadfence_block();
        if (lane == 0) atomicAdd(const_cast<int*>(ctl + kCtlArrived + (seq & 1)), 1);
        if (warp == 0) serve_fold(seq);
        if (warp == NSVC - 1) serve_prepare(seq);
    };

    auto softmax_page = [&](const Regs& r, int pg2, const float (&c2)[NH][2][4],
                            uint32_t (&pb2)[NH][2][2]) {
        if ((pg2 + 1) * kPageTokens <= ntok_item) softmax_update(std::true_type{}, r, pg2, c2, pb2);
        else softmax_update(std::false_type{}, r, pg2, c2, pb2);
    };

    // ---- prime the ring, then consume the stream.  The ring is a FIFO of two pages: (pgA, tagA)
    // describe the page consumed next, (pgB, tagB) the one after it; tag = the page's item number,
    // or the negative result of grab (-1: the stream has ended, -2: request handed back).
    int pgA = grab(0), tagA = pgA < 0 ? pgA : gseq;
    int pgB = grab(1), tagB = pgB < 0 ? pgB : gseq;
    reset_state();
    int want = -3;         // item number whose query fragments / token count are loaded (-3: none)

    // Software pipeline (one head half): K.Q^T of a page and P.V of the page before it are
    // independent and sit in one straight-line block.  One register set serves both: the
    // values of a page are read from its ring buffer only after P.V of the page before has
    // consumed the value registers, and the buffer is released after that read.
    constexpr bool kPipelined = NH == 1 && !S::QSMEM;
    Regs r;
    uint32_t pb[NH][2][2];
    float c[NH][2][4];
    bool pending = false;  // P.V of the previous page (values and weights in registers) is due
    int n = 0;             // pages fetched so far: ring buffer n & 1, mbarrier parity (n >> 1) & 1
    for (;;) {
        const int par = n & 1;
        bool first = false;
        if (tagA != want) {
            // rare path: item boundary, empty ring or end of stream (one copy of all of it)
            if constexpr (kPipelined) {
                if (pending) {
                    pv_accum(r.v, pb);
                    pending = false;
                }
            }
            // publish the finished items: up to the page's item; everything consumed when the
            // ring ran dry two items ahead of the published state (-2) or the stream ended (-1)
            const int target = tagA == -2 ? gseq + 1 : (tagA == -1 ? gseq : tagA);
            while (cseq < target) {
                finish_item(cseq);
                cseq++;
                reset_state();
            }
            if (tagA == -1) break;
            if (tagA == -2) {
                // refill the (empty) ring in stream order, starting with this buffer
                want = -3;
                deferred = false;
                pgA = grab(par);
                tagA = pgA < 0 ? pgA : gseq;
                pgB = grab(par ^ 1);
                tagB = pgB < 0 ? pgB : gseq;
                continue;
            }
            load_ctx(cseq);
            want = cseq;
            first = true;
        }
        const int sp = pgA;
        const uint32_t page = my_ring + par * PAGE_BYTES;
        if (!stalled && !mbar_wait(my_bars + par * 8, (n >> 1) & 1)) stalled = true;
        read_keys(r, page);
        if constexpr (kPipelined) {
            if (first) {
                // first page of an item: nothing to overlap with (generic softmax: rare path)
                qk_scores(r, c);
                read_values(r, page);
                __syncwarp();  // every lane has its slices: the buffer may be refilled
                pgA = pgB;
                tagA = tagB;
                pgB = grab(par);
                tagB = pgB < 0 ? pgB : gseq;
                softmax_update(std::false_type{}, r, sp, c, pb);
                pending = true;
            } else {
                qk_scores(r, c);
                pv_accum(r.v, pb);
                read_values(r, page);
                __syncwarp();
                pgA = pgB;
                tagA = tagB;
                pgB = grab(par);
                tagB = pgB < 0 ? pgB : gseq;
                softmax_page(r, sp, c, pb);
            }
        } else {
            read_values(r, page);
            __syncwarp();
            pgA = pgB;
            tagA = tagB;
            pgB = grab(par);
            tagB = pgB < 0 ? pgB : gseq;
            qk_scores(r, c);
            softmax_page(r, sp, c, pb);
            pv_accum(r.v, pb);
        }
        n++;
    }
    // the last CTA to leave takes the epoch out of the workspace: a replay of this very launch
    // (a captured graph) must not find its own epoch there before CTA 0 has cleared the counters
    if (stalled) {
        await_epoch();
        if (lane == 0) atomicOr(p.work_counter + kStatusWord, kStatusWaitExpired);
    }
    __syncthreads();
    if (warp == 0) {
        await_epoch();
        if (lane == 0 && atomicAdd(p.work_counter + 1, 1) == static_cast<int>(gridDim.x) - 1) {
            __threadfence();
            asm volatile("st.release.gpu.global.u64 [%0], %1;\n" ::"l"(epoch_word), "l"(0ull) : "memory");
        }
    }
}

}  // namespace ftq
