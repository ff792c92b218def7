// Instantiates the fused encode kernel for one head_dim (FTQ_D).
#include "ftq_launch.h"

#ifndef FTQ_D
#error "compile with -DFTQ_D=64, 128 or 256"
#endif
#define FTQ_CAT2(a, b) a##b
#define FTQ_CAT(a, b) FTQ_CAT2(a, b)

namespace ftq {

// Throughput kernel (needs the table quantizer; see ftq_encode2.cuh).
template <int BITS, typename T>
static cudaError_t run2(const EncodeSource& src, const EncodeSink& sink, const Encode2Tables& tab,
                        int64_t n_vec, int n_layers, cudaStream_t stream) {
    // 16 warps per SM: two CTAs of 8 warps, or one of 16 where two transpose areas would not
    // fit next to two copies of the quantiser table (head_dim 256); a warp pass = 8 vectors
    constexpr int threads = encode2_threads(FTQ_D);
    constexpr int ctas_per_sm = 512 / threads;
    constexpr int smem = encode2_smem_bytes(FTQ_D, threads / 32);
    auto kern = encode2_kernel<FTQ_D, BITS, T>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    const int64_t want = (n_vec + threads / 4 - 1) / (threads / 4);
    const int64_t cap = static_cast<int64_t>(sm_count()) * ctas_per_sm;   // persistent grid
    const unsigned gx = static_cast<unsigned>(want < 1 ? 1 : (want < cap ? want : cap));
    kern<<<dim3(gx, n_layers), threads, smem, stream>>>(src, sink, tab, n_vec);
    return cudaGetLastError();
}

template <int BITS, typename T>
static cudaError_t run(const EncodeSource& src, const EncodeSink& sink, const EncodeTables& tab,
                       const Encode2Tables* tab2, int64_t n_vec, int n_layers,
                       cudaStream_t stream) {
    if (tab2) return run2<BITS, T>(src, sink, *tab2, n_vec, n_layers, stream);
    constexpr int threads = 256;                       // 8 warps, 32 vectors per CTA pass
    const int64_t want = (n_vec + 31) / 32;
    const int64_t cap = static_cast<int64_t>(sm_count()) * 8;  // persistent-style grid
    const unsigned gx = static_cast<unsigned>(want < 1 ? 1 : (want < cap ? want : cap));
    encode_kernel<FTQ_D, BITS, T><<<dim3(gx, n_layers), threads, 0, stream>>>(src, sink, tab, n_vec);
    return cudaGetLastError();
}

template <int BITS>
static cudaError_t by_dtype(int dtype, const EncodeSource& src, const EncodeSink& sink,
                            const EncodeTables& tab, const Encode2Tables* tab2, int64_t n_vec,
                            int n_layers, cudaStream_t stream) {
    switch (dtype) {
        case kF32: return run<BITS, float>(src, sink, tab, tab2, n_vec, n_layers, stream);
        case kF16: return run<BITS, __half>(src, sink, tab, tab2, n_vec, n_layers, stream);
        case kBF16:
            return run<BITS, __nv_bfloat16>(src, sink, tab, tab2, n_vec, n_layers, stream);
    }
    return cudaErrorInvalidValue;
}

cudaError_t FTQ_CAT(launch_encode_d, FTQ_D)(int bits, int dtype, const EncodeSource& src,
                                            const EncodeSink& sink, const EncodeTables& tab,
                                            const Encode2Tables* tab2, int64_t n_vec, int n_layers,
                                            cudaStream_t stream) {
    switch (bits) {
        case 2: return by_dtype<2>(dtype, src, sink, tab, tab2, n_vec, n_layers, stream);
        case 3: return by_dtype<3>(dtype, src, sink, tab, tab2, n_vec, n_layers, stream);
        case 4: return by_dtype<4>(dtype, src, sink, tab, tab2, n_vec, n_layers, stream);
    }
    return cudaErrorInvalidValue;
}

}  // namespace ftq
