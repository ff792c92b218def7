// Instantiates the split-KV decode attention kernels for one head_dim (FTQ_D).
#include "ftq_attn_stream.cuh"
#include "ftq_launch.h"

#ifndef FTQ_D
#error "compile with -DFTQ_D=64, 128 or 256"
#endif
#define FTQ_CAT2(a, b) a##b
#define FTQ_CAT(a, b) FTQ_CAT2(a, b)

namespace ftq {

template <int BK, int BV, bool PAGED>
static cudaError_t run_split(const AttnParams& p, int n_lb, cudaStream_t stream) {
    constexpr int D = FTQ_D;
    constexpr int GH = AttnCfg<D>::GH;
    constexpr int page = kPageTokens * (packed_dim(D, BK) + packed_dim(D, BV) + 4);
    constexpr int merge = 4 * GH * (D + 2) * 4;
    constexpr int ring = ((2 * kTilePages * page > merge ? 2 * kTilePages * page : merge) + 15) / 16 * 16;
    constexpr int smem = ring + (GH * D + 2 * kMaxLevels) * 4;
    static_assert(smem <= 48 * 1024, "shared memory budget");
    const dim3 grid(p.n_chunks, p.Hkv * p.n_hpass, n_lb);
    attn_split_kernel<D, BK, BV, PAGED><<<grid, kAttnThreads, smem, stream>>>(p);
    return cudaGetLastError();
}

template <int BK, bool PAGED>
static cudaError_t by_bv(int bv, const AttnParams& p, int n_lb, cudaStream_t stream) {
    switch (bv) {
        case 2: return run_split<BK, 2, PAGED>(p, n_lb, stream);
        case 3: return run_split<BK, 3, PAGED>(p, n_lb, stream);
        case 4: return run_split<BK, 4, PAGED>(p, n_lb, stream);
    }
    return cudaErrorInvalidValue;
}

template <bool PAGED>
static cudaError_t by_bk(int bk, int bv, const AttnParams& p, int n_lb, cudaStream_t stream) {
    switch (bk) {
        case 2: return by_bv<2, PAGED>(bv, p, n_lb, stream);
        case 3: return by_bv<3, PAGED>(bv, p, n_lb, stream);
        case 4: return by_bv<4, PAGED>(bv, p, n_lb, stream);
    }
    return cudaErrorInvalidValue;
}

cudaError_t FTQ_CAT(launch_attn_split_d, FTQ_D)(int bits_k, int bits_v, bool paged,
                                                const AttnParams& p, int n_lb,
                                                cudaStream_t stream) {
    return paged ? by_bk<true>(bits_k, bits_v, p, n_lb, stream)
                 : by_bk<false>(bits_k, bits_v, p, n_lb, stream);
}

// The streaming kernel (no CTA-wide barriers, merge included) serves the configurations in
// which it was measured faster than the barrier-synchronised one: a 4-bit byte table (one CTA
// per SM) with one head half (GQA group <= 4) -- 16 warps at head_dim 64 / 128, 8 warps at
// head_dim 256 (16 rings and exchange slots do not fit beside the table there).  Measured on
// B200: +20 % on the Llama-shaped K4V4 batch, +5 % on the ragged head_dim-256 K4V2 batch.  With
// 3- and 2-bit codes (two 8-warp CTAs per SM, or one 16-warp CTA) and with two head halves it
// measured 0-17 % slower; those keep attn_mma_kernel + the merge launch.
template <int BK, int BV, int NH>
constexpr bool use_stream_kernel() {
    using S = StreamCfg<FTQ_D, BK, BV, NH>;
#if defined(FTQ_NO_STREAM)
    return false;
#elif defined(FTQ_ALL_STREAM)
    return S::FITS;
#else
    return S::FITS && S::BYTE && NH == 1 && (S::WARPS == 16 || FTQ_D == 256);
#endif
}

template <int BK, int BV, bool SHARED, int NH>
static cudaError_t run_mma_nh(const AttnParams& p, int n_lb, cudaStream_t stream, bool* merged) {
    constexpr int D = FTQ_D;
    if constexpr (use_stream_kernel<BK, BV, NH>()) {
        using S = StreamCfg<D, BK, BV, NH>;
        auto kern = attn_stream_kernel<D, BK, BV, SHARED, NH>;
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             S::SMEM_BYTES);
        if (e != cudaSuccess) return e;
        const int64_t items = p.split.total_items;
        const int64_t slots = static_cast<int64_t>(sm_count()) * S::CTAS_PER_SM;
        const unsigned grid = static_cast<unsigned>(items < slots ? items : slots);
        // One node per call: the kernel clears its own counters.  Programmatic stream
        // serialisation lets the set-up of this launch (tables in shared memory) run while the
        // kernel before it in the stream drains; the kernel waits for that kernel's completion
        // (griddepcontrol.wait) before it touches anything in global memory.
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3(grid);
        cfg.blockDim = dim3(S::THREADS);
        cfg.dynamicSmemBytes = S::SMEM_BYTES;
        cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
#ifdef FTQ_NO_PDL
        attr[0].val.programmaticStreamSerializationAllowed = 0;
#else
        attr[0].val.programmaticStreamSerializationAllowed = 1;
#endif
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        *merged = true;
        return cudaLaunchKernelEx(&cfg, kern, p, static_cast<int>(items));
    } else {
    *merged = false;
    using C = MmaCfg<D, BK, BV, NH>;
    static_assert(C::SMEM_BYTES <= 227 * 1024, "shared memory budget");
    auto kern = attn_mma_kernel<D, BK, BV, SHARED, NH>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         C::SMEM_BYTES);
    if (e != cudaSuccess) return e;
    const int64_t items = p.split.total_items;
    const int64_t slots = static_cast<int64_t>(sm_count()) * C::CTAS_PER_SM;
    const unsigned grid = static_cast<unsigned>(items < slots ? items : slots);
    e = cudaMemsetAsync(p.work_counter, 0, 256, stream);   // this kernel counts from a zeroed word
    if (e != cudaSuccess) return e;
    kern<<<grid, C::THREADS, C::SMEM_BYTES, stream>>>(p, static_cast<int>(items));
    return cudaGetLastError();
    }
}

template <int BK, int BV, bool SHARED>
static cudaError_t run_mma(const AttnParams& p, int n_lb, cudaStream_t stream, bool* merged) {
    return p.Hq / p.Hkv <= 4 ? run_mma_nh<BK, BV, SHARED, 1>(p, n_lb, stream, merged)
                             : run_mma_nh<BK, BV, SHARED, 2>(p, n_lb, stream, merged);
}

// FTQ_ONLY_BITS=<b> (a development aid, never set by the build script) instantiates the
// tensor-core kernels for bits_k = bits_v = b only, which cuts the compile time of an experiment.
template <int BK>
static cudaError_t mma_by_bv(int bv, bool shared_lut, const AttnParams& p, int n_lb,
                             cudaStream_t stream, bool* merged) {
#ifdef FTQ_ONLY_BITS
    if (BK != FTQ_ONLY_BITS || bv != FTQ_ONLY_BITS) return cudaErrorInvalidValue;
    if constexpr (BK == FTQ_ONLY_BITS) {
        return shared_lut ? run_mma<BK, BK, true>(p, n_lb, stream, merged)
                          : run_mma<BK, BK, false>(p, n_lb, stream, merged);
    }
#else
    if (shared_lut && bv == BK) return run_mma<BK, BK, true>(p, n_lb, stream, merged);
    switch (bv) {
        case 2: return run_mma<BK, 2, false>(p, n_lb, stream, merged);
        case 3: return run_mma<BK, 3, false>(p, n_lb, stream, merged);
        case 4: return run_mma<BK, 4, false>(p, n_lb, stream, merged);
    }
#endif
    return cudaErrorInvalidValue;
}

cudaError_t FTQ_CAT(launch_attn_mma_d, FTQ_D)(int bits_k, int bits_v, bool shared_lut,
                                              const AttnParams& p, int n_lb, cudaStream_t stream,
                                              bool* merged) {
    switch (bits_k) {
        case 2: return mma_by_bv<2>(bits_v, shared_lut, p, n_lb, stream, merged);
        case 3: return mma_by_bv<3>(bits_v, shared_lut, p, n_lb, stream, merged);
        case 4: return mma_by_bv<4>(bits_v, shared_lut, p, n_lb, stream, merged);
    }
    return cudaErrorInvalidValue;
}

// CTAs per SM of the streaming kernel where launch_attn_mma picks it for this configuration, 0
// where it picks the barrier-synchronised kernel (the host plans the split of the context
// differently for the two)
template <int BK, int BV, int NH>
static constexpr int stream_ctas() {
    return use_stream_kernel<BK, BV, NH>() ? StreamCfg<FTQ_D, BK, BV, NH>::CTAS_PER_SM : 0;
}
template <int BK>
static int stream_ctas_by_bv(int bv, int nh) {
#ifdef FTQ_ONLY_BITS
    if (BK != FTQ_ONLY_BITS || bv != FTQ_ONLY_BITS) return 0;
    return nh == 1 ? stream_ctas<BK, BK, 1>() : stream_ctas<BK, BK, 2>();
#else
    switch (bv) {
        case 2: return nh == 1 ? stream_ctas<BK, 2, 1>() : stream_ctas<BK, 2, 2>();
        case 3: return nh == 1 ? stream_ctas<BK, 3, 1>() : stream_ctas<BK, 3, 2>();
        case 4: return nh == 1 ? stream_ctas<BK, 4, 1>() : stream_ctas<BK, 4, 2>();
    }
    return 0;
#endif
}
int FTQ_CAT(attn_mma_stream_ctas_d, FTQ_D)(int bits_k, int bits_v, int group) {
    const int nh = group <= 4 ? 1 : 2;
    switch (bits_k) {
        case 2: return stream_ctas_by_bv<2>(bits_v, nh);
        case 3: return stream_ctas_by_bv<3>(bits_v, nh);
        case 4: return stream_ctas_by_bv<4>(bits_v, nh);
    }
    return 0;
}

cudaError_t FTQ_CAT(launch_attn_merge_d, FTQ_D)(int out_dtype, const float* partials, void* out,
                                                const int32_t* seq_lens, int S, int B, int Hq,
                                                int n_chunks, int chunk_tokens, int64_t n_vec,
                                                const SignBits& signs, float rsqrt_d, int Hkv,
                                                const SplitPlan& split, cudaStream_t stream) {
    constexpr int D = FTQ_D;
    const unsigned grid = static_cast<unsigned>((n_vec + 15) / 16);
    switch (out_dtype) {
        case kF32:
            attn_merge_kernel<D, float><<<grid, 128, 0, stream>>>(
                partials, static_cast<float*>(out), seq_lens, S, B, Hq, n_chunks, chunk_tokens,
                n_vec, signs, rsqrt_d, Hkv, split);
            break;
        case kF16:
            attn_merge_kernel<D, __half><<<grid, 128, 0, stream>>>(
                partials, static_cast<__half*>(out), seq_lens, S, B, Hq, n_chunks, chunk_tokens,
                n_vec, signs, rsqrt_d, Hkv, split);
            break;
        case kBF16:
            attn_merge_kernel<D, __nv_bfloat16><<<grid, 128, 0, stream>>>(
                partials, static_cast<__nv_bfloat16*>(out), seq_lens, S, B, Hq, n_chunks,
                chunk_tokens, n_vec, signs, rsqrt_d, Hkv, split);
            break;
        default:
            return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

}  // namespace ftq
