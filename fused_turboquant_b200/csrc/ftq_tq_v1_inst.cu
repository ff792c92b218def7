// Instantiates the vLLM-v1 slot-format kernels for one head_dim (FTQ_D).  FTQ_TQ_PART selects
// what this object holds, so that the halves compile in parallel: 0 = the store kernels,
// 1 = the decode kernels (fp32 split, tensor-core split, merge); undefined = both.
#include "ftq_launch.h"
#include "ftq_tq_v1.cuh"
#include "ftq_tq_v1_launch.h"
#if !defined(FTQ_TQ_PART) || FTQ_TQ_PART == 0
#define FTQ_TQ_STORE 1
#endif
#if !defined(FTQ_TQ_PART) || FTQ_TQ_PART == 1
#define FTQ_TQ_DECODE 1
#endif
#if FTQ_D != 256 && defined(FTQ_TQ_DECODE)
#include "ftq_tq_v1_mma.cuh"
#endif

#ifndef FTQ_D
#error "compile with -DFTQ_D=64, 128 or 256"
#endif
#define FTQ_CAT2(a, b) a##b
#define FTQ_CAT(a, b) FTQ_CAT2(a, b)

namespace ftq {

#ifdef FTQ_TQ_STORE
template <int KB, int VB, typename T, bool K8M>
static cudaError_t store_run(const TqStoreParams& p, int value_mode, int64_t n_vec,
                             const TqTable<K8M>& t8, cudaStream_t stream) {
    const int64_t want = (n_vec + 31) / 32;  // 8 warps x 4 vectors per CTA pass
    const int layers = value_mode >> 8;      // (the launcher packs the layer count above the flags)
    const int64_t cap = (static_cast<int64_t>(sm_count()) * 8 + layers - 1) / layers;
    const dim3 gx(static_cast<unsigned>(want < 1 ? 1 : (want < cap ? want : cap)), layers);
    const bool rotate_v = (value_mode & kTqRotateValues) != 0;
    if constexpr (VB == 4 && KB != 8) {
        if (value_mode & kTqLloydMaxValues) {
            if (rotate_v) tq_store_kernel<FTQ_D, KB, VB, T, true, true><<<gx, 256, 0, stream>>>(p, n_vec, t8);
            else tq_store_kernel<FTQ_D, KB, VB, T, false, true><<<gx, 256, 0, stream>>>(p, n_vec, t8);
            return cudaGetLastError();
        }
    }
    if constexpr (VB != 8) {
        if (rotate_v) {
            tq_store_kernel<FTQ_D, KB, VB, T, true, false, K8M><<<gx, 256, 0, stream>>>(p, n_vec, t8);
            return cudaGetLastError();
        }
    } else if (rotate_v) {
        return cudaErrorInvalidValue;  // 8-bit values are rotated by the caller
    }
    tq_store_kernel<FTQ_D, KB, VB, T, false, false, K8M><<<gx, 256, 0, stream>>>(p, n_vec, t8);
    return cudaGetLastError();
}

template <int KB, int VB, bool K8M>
static cudaError_t store_by_dtype(int dtype, const TqStoreParams& p, int vmode, int64_t n_vec,
                                  const TqTable<K8M>& t8, cudaStream_t s) {
    switch (dtype) {
        case kF32: return store_run<KB, VB, float, K8M>(p, vmode, n_vec, t8, s);
        case kF16: return store_run<KB, VB, __half, K8M>(p, vmode, n_vec, t8, s);
        case kBF16: return store_run<KB, VB, __nv_bfloat16, K8M>(p, vmode, n_vec, t8, s);
    }
    return cudaErrorInvalidValue;
}

template <int KB, bool K8M = false>
static cudaError_t store_by_vb(int vb, int dtype, const TqStoreParams& p, int vmode, int64_t n_vec,
                               const TqTable<K8M>& t8, cudaStream_t s) {
    switch (vb) {
        case 1: return store_by_dtype<KB, 1, K8M>(dtype, p, vmode, n_vec, t8, s);
        case 2: return store_by_dtype<KB, 2, K8M>(dtype, p, vmode, n_vec, t8, s);
        case 3: return store_by_dtype<KB, 3, K8M>(dtype, p, vmode, n_vec, t8, s);
        case 4: return store_by_dtype<KB, 4, K8M>(dtype, p, vmode, n_vec, t8, s);
        case 8: return store_by_dtype<KB, 8, K8M>(dtype, p, vmode, n_vec, t8, s);
    }
    return cudaErrorInvalidValue;
}

cudaError_t FTQ_CAT(launch_tq_store_d, FTQ_D)(int kb, int vb, int dtype, const TqStoreParams& p,
                                             int value_mode, int64_t n_vec, const TqTable256* mid8,
                                             cudaStream_t stream) {
    const TqNoTable none{};
    switch (kb) {
        case 1: return store_by_vb<1>(vb, dtype, p, value_mode, n_vec, none, stream);
        case 2: return store_by_vb<2>(vb, dtype, p, value_mode, n_vec, none, stream);
        case 3: return store_by_vb<3>(vb, dtype, p, value_mode, n_vec, none, stream);
        case 4: return store_by_vb<4>(vb, dtype, p, value_mode, n_vec, none, stream);
        case 8:   // 8-bit Lloyd-Max codes with a table, FP8 keys without
            return mid8 ? store_by_vb<8, true>(vb, dtype, p, value_mode, n_vec, *mid8, stream)
                        : store_by_vb<8>(vb, dtype, p, value_mode, n_vec, none, stream);
    }
    return cudaErrorInvalidValue;
}

#endif  // FTQ_TQ_STORE

#ifdef FTQ_TQ_DECODE
template <int KB, int VB, bool K8M>
static cudaError_t split_run(const TqDecodeParams& p, const TqTable<K8M>& t8, cudaStream_t stream) {
    constexpr int smem = tq_split_smem_bytes<FTQ_D>(KB, VB, K8M);
    static_assert(smem <= 48 * 1024, "tile does not fit the default shared-memory carve-out");
    const dim3 grid(p.splits, p.Hkv * p.n_hpass, p.B);
    tq_split_kernel<FTQ_D, KB, VB, K8M><<<grid, kAttnThreads, smem, stream>>>(p, t8);
    return cudaGetLastError();
}

template <int KB, bool K8M = false>
static cudaError_t split_by_vb(int vb, const TqDecodeParams& p, const TqTable<K8M>& t8,
                               cudaStream_t s) {
    switch (vb) {
        case 1: return split_run<KB, 1, K8M>(p, t8, s);
        case 2: return split_run<KB, 2, K8M>(p, t8, s);
        case 3: return split_run<KB, 3, K8M>(p, t8, s);
        case 4: return split_run<KB, 4, K8M>(p, t8, s);
        case 8: return split_run<KB, 8, K8M>(p, t8, s);
    }
    return cudaErrorInvalidValue;
}

cudaError_t FTQ_CAT(launch_tq_split_d, FTQ_D)(int kb, int vb, const TqDecodeParams& p,
                                             const TqTable256* cent8, cudaStream_t stream) {
    const TqNoTable none{};
    switch (kb) {
        case 1: return split_by_vb<1>(vb, p, none, stream);
        case 2: return split_by_vb<2>(vb, p, none, stream);
        case 3: return split_by_vb<3>(vb, p, none, stream);
        case 4: return split_by_vb<4>(vb, p, none, stream);
        case 8:   // 8-bit Lloyd-Max codes with a table, FP8 keys without
            return cent8 ? split_by_vb<8, true>(vb, p, *cent8, stream)
                         : split_by_vb<8>(vb, p, none, stream);
    }
    return cudaErrorInvalidValue;
}

#if FTQ_D != 256
template <int KB, int VB, int NH>
static cudaError_t mma_run(const TqDecodeParams& p, int n_items, cudaStream_t stream) {
    using C = TqMmaCfg<FTQ_D, KB, VB, NH>;
    static_assert(C::SMEM_BYTES <= 227 * 1024, "shared memory budget");
    auto kern = tq_mma_kernel<FTQ_D, KB, VB, NH>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
    if (e != cudaSuccess) return e;
    const int64_t slots = static_cast<int64_t>(sm_count()) * C::CTAS_PER_SM;
    const unsigned gx = static_cast<unsigned>(n_items < slots ? n_items : slots);
    kern<<<gx, C::THREADS, C::SMEM_BYTES, stream>>>(p, n_items);
    return cudaGetLastError();
}

template <int KB, int VB>
static cudaError_t mma_by_nh(int nh, const TqDecodeParams& p, int n_items, cudaStream_t s) {
    return nh == 1 ? mma_run<KB, VB, 1>(p, n_items, s) : mma_run<KB, VB, 2>(p, n_items, s);
}

template <int KB>
static cudaError_t mma_by_vb(int vb, int nh, const TqDecodeParams& p, int n_items, cudaStream_t s) {
    switch (vb) {
        case 2: return mma_by_nh<KB, 2>(nh, p, n_items, s);
        case 3: return mma_by_nh<KB, 3>(nh, p, n_items, s);
        case 4: return mma_by_nh<KB, 4>(nh, p, n_items, s);
    }
    return cudaErrorInvalidValue;
}
#endif

// Tensor-core stage 1 (16-bit queries, GQA group <= 8, value_bits != 8, head_dim 64 / 128).
cudaError_t FTQ_CAT(launch_tq_mma_d, FTQ_D)(int kb, int vb, int nh, const TqDecodeParams& p,
                                           int n_items, cudaStream_t stream) {
#if FTQ_D != 256
    switch (kb) {
        case 2: return mma_by_vb<2>(vb, nh, p, n_items, stream);
        case 3: return mma_by_vb<3>(vb, nh, p, n_items, stream);
        case 4: return mma_by_vb<4>(vb, nh, p, n_items, stream);
    }
#endif
    return cudaErrorInvalidValue;
}

cudaError_t FTQ_CAT(launch_tq_merge_d, FTQ_D)(int out_dtype, const TqMergeParams& p,
                                             cudaStream_t stream) {
    const unsigned grid = static_cast<unsigned>((p.n_rows + 15) / 16);  // 128 threads = 16 rows
    switch (out_dtype) {
        case kF32: tq_merge_kernel<FTQ_D, float><<<grid, 128, 0, stream>>>(p); break;
        case kF16: tq_merge_kernel<FTQ_D, __half><<<grid, 128, 0, stream>>>(p); break;
        case kBF16: tq_merge_kernel<FTQ_D, __nv_bfloat16><<<grid, 128, 0, stream>>>(p); break;
        default: return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

#endif  // FTQ_TQ_DECODE

}  // namespace ftq
