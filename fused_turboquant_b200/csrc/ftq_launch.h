// Host-side launchers, one translation unit per head_dim (compiled with
// -DFTQ_D=64|128|256) so the template instantiations build in parallel.
#pragma once

#include <cuda_runtime.h>

#include "ftq_attn.cuh"
#include "ftq_encode2.cuh"

namespace ftq {

#define FTQ_DECLARE_LAUNCHERS(DD)                                                              \
    cudaError_t launch_encode_d##DD(int bits, int dtype, const EncodeSource& src,               \
                                    const EncodeSink& sink, const EncodeTables& tab,            \
                                    const Encode2Tables* tab2, int64_t n_vec, int n_layers,     \
                                    cudaStream_t stream);                                       \
    cudaError_t launch_attn_split_d##DD(int bits_k, int bits_v, bool paged, const AttnParams& p, \
                                        int n_lb, cudaStream_t stream);                         \
    cudaError_t launch_attn_mma_d##DD(int bits_k, int bits_v, bool shared_lut, const AttnParams& p, \
                                      int n_lb, cudaStream_t stream, bool* merged);            \
    int attn_mma_stream_ctas_d##DD(int bits_k, int bits_v, int group);                          \
    cudaError_t launch_attn_merge_d##DD(int out_dtype, const float* partials, void* out,        \
                                        const int32_t* seq_lens, int S, int B, int Hq,          \
                                        int n_chunks, int chunk_tokens, int64_t n_vec,          \
                                        const SignBits& signs, float rsqrt_d, int Hkv,          \
                                        const SplitPlan& split, cudaStream_t stream);

FTQ_DECLARE_LAUNCHERS(64)
FTQ_DECLARE_LAUNCHERS(128)
FTQ_DECLARE_LAUNCHERS(256)

// number of SMs of the current device (cached per device)
int sm_count();

}  // namespace ftq
