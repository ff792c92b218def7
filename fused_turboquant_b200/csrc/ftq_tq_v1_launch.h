// Launchers of the vLLM-v1 slot-format kernels (ftq_tq_v1_inst.cu, one object per head_dim).
#pragma once

#include <cuda_runtime.h>

#include "ftq_tq_v1.cuh"

namespace ftq {

// kb = 8 with a table (mid8 / cent8 not NULL) = 8-bit Lloyd-Max key codes, without = FP8 keys.
// value_mode of the store launchers
constexpr int kTqRotateValues = 1;    // Hadamard-transform the values in the kernel
constexpr int kTqLloydMaxValues = 2;  // 4-bit values: Lloyd-Max codes against the key midpoints
// bits 8.. of value_mode: the number of layers stored by the launch (grid y; at least 1)

#define FTQ_DECLARE_TQ_LAUNCHERS(DD)                                                              \
    cudaError_t launch_tq_store_d##DD(int kb, int vb, int dtype, const TqStoreParams& p,          \
                                      int value_mode, int64_t n_vec, const TqTable256* mid8,      \
                                      cudaStream_t stream);                                       \
    cudaError_t launch_tq_split_d##DD(int kb, int vb, const TqDecodeParams& p,                    \
                                      const TqTable256* cent8, cudaStream_t stream);              \
    cudaError_t launch_tq_mma_d##DD(int kb, int vb, int nh, const TqDecodeParams& p, int n_items,   \
                                    cudaStream_t stream);                                         \
    cudaError_t launch_tq_merge_d##DD(int out_dtype, const TqMergeParams& p, cudaStream_t stream);

FTQ_DECLARE_TQ_LAUNCHERS(64)
FTQ_DECLARE_TQ_LAUNCHERS(128)
FTQ_DECLARE_TQ_LAUNCHERS(256)

}  // namespace ftq
