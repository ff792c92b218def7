// Dense helpers on the quantizer API: standalone randomized Hadamard
// transform, dense dequantisation, and attention scores from packed keys.
// They share the octet butterfly of ftq_common.cuh with the encode kernel.
#pragma once

#include "ftq_common.cuh"

namespace ftq {

// Read the 8 codes of coordinate run g (coordinates 8g .. 8g+7) of one packed vector.
template <int BITS>
__device__ __forceinline__ uint32_t load_run(const uint8_t* vec, int g) {
    if constexpr (BITS == 4) {
        return *reinterpret_cast<const uint32_t*>(vec + 4 * g);
    } else if constexpr (BITS == 2) {
        return *reinterpret_cast<const uint16_t*>(vec + 2 * g);
    } else {
        const uint8_t* p = vec + 3 * g;
        return static_cast<uint32_t>(p[0]) | (static_cast<uint32_t>(p[1]) << 8) |
               (static_cast<uint32_t>(p[2]) << 16);
    }
}

// ------------------------------------------------------------------- RHT
// forward: y = fwht(x * signs) * D^-1/2 ; inverse: y = fwht(x) * D^-1/2 * signs
// (core/hadamard.py:70-100 of the reference).
template <int D, typename T>
__global__ void __launch_bounds__(256)
rht_kernel(const T* __restrict__ x, T* __restrict__ y, SignBits signs, float rsqrt_d, int inverse,
           int64_t n_vec) {
    constexpr int E = D / kOctet;
    const int lane = threadIdx.x & 31;
    const int t = lane & 7;
    const int sub = lane >> 3;
    const int64_t warp = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int64_t n_warps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;

    for (int64_t base = warp * 4; base < n_vec; base += n_warps * 4) {
        const int64_t v = base + sub;
        const bool valid = v < n_vec;
        float a[E];
#pragma unroll
        for (int i = 0; i < E / 8; i++) {
            float tmp[8];
            if (valid) {
                load8<T>(x + v * D + 8 * (t + 8 * i), tmp);
            } else {
#pragma unroll
                for (int c = 0; c < 8; c++) tmp[c] = 0.f;
            }
#pragma unroll
            for (int c = 0; c < 8; c++) {
                const uint32_t m = inverse ? 0u : sign_mask(signs, load_coord(t, 8 * i + c));
                a[8 * i + c] = __uint_as_float(__float_as_uint(tmp[c]) ^ m);
            }
        }
        octet_fwht<E>(a, lane);
        if (valid) {
#pragma unroll
            for (int k = 0; k < E; k++) {
                float r = __fmul_rn(a[k], rsqrt_d);
                if (inverse) r = __uint_as_float(__float_as_uint(r) ^ sign_mask(signs, t + 8 * k));
                y[v * D + t + 8 * k] = from_float<T>(r);
            }
        }
    }
}

// --------------------------------------------------------- dense dequant
// out = fwht(levels[code] * norm) * D^-1/2 * signs  (core/quantizer.py:191-205).
template <int D, int BITS, typename NormT>
__global__ void __launch_bounds__(256)
decode_dense_kernel(const uint8_t* __restrict__ packed, const NormT* __restrict__ norms,
                    float* __restrict__ out, Codebook levels, SignBits signs, float rsqrt_d,
                    int64_t n_vec) {
    constexpr int E = D / kOctet;
    constexpr int PD = packed_dim(D, BITS);
    __shared__ float lut[kMaxLevels];
    if (threadIdx.x < kMaxLevels) lut[threadIdx.x] = levels.v[threadIdx.x];
    __syncthreads();

    const int lane = threadIdx.x & 31;
    const int t = lane & 7;
    const int sub = lane >> 3;
    const int64_t warp = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int64_t n_warps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;

    for (int64_t base = warp * 4; base < n_vec; base += n_warps * 4) {
        const int64_t v = base + sub;
        const bool valid = v < n_vec;
        const float nf = valid ? to_float<NormT>(norms[v]) : 0.f;
        float a[E];
#pragma unroll
        for (int i = 0; i < E / 8; i++) {
            const uint32_t w = valid ? load_run<BITS>(packed + v * PD, t + 8 * i) : 0u;
#pragma unroll
            for (int c = 0; c < 8; c++)
                a[8 * i + c] = __fmul_rn(lut[(w >> (BITS * c)) & ((1u << BITS) - 1u)], nf);
        }
        octet_fwht<E>(a, lane);
        if (valid) {
#pragma unroll
            for (int k = 0; k < E; k++) {
                const float r = __fmul_rn(a[k], rsqrt_d);
                out[v * D + t + 8 * k] =
                    __uint_as_float(__float_as_uint(r) ^ sign_mask(signs, t + 8 * k));
            }
        }
    }
}

// -------------------------------------------------------------- QK scores
// out[b,hq,tq,s] = norm[b,hkv,s] * scale * sum_d q_rot[b,hq,tq,d] * levels[code[b,hkv,s,d]]
// (kernels/triton_attention.py:47-152).  grid = (ceil(S / 64), B * Hkv); an octet
// scores one key against every query row of its KV head, so the packed key is
// read once per KV head.
template <int D, int BITS, typename NormT>
__global__ void __launch_bounds__(128)
qk_scores_kernel(const float* __restrict__ q_rot, const uint8_t* __restrict__ k_codes,
                 const NormT* __restrict__ k_norms, float* __restrict__ out, Codebook levels,
                 float scale, int Hq, int Hkv, int q_len, int S) {
    constexpr int E = D / kOctet;
    constexpr int PD = packed_dim(D, BITS);
    extern __shared__ float smem[];
    float* lut = smem;            // [16]
    float* qs = smem + kMaxLevels;  // [rows][D]
    const int group = Hq / Hkv;
    const int rows = group * q_len;
    const int bh = blockIdx.y;
    const int b = bh / Hkv, hkv = bh % Hkv;
    if (threadIdx.x < kMaxLevels) lut[threadIdx.x] = levels.v[threadIdx.x];
    // query rows of this KV head are contiguous: [b, hkv*group .. +group, q_len, D]
    const float* qsrc = q_rot + (static_cast<int64_t>(b) * Hq + hkv * group) * q_len * D;
    for (int i = threadIdx.x; i < rows * D; i += blockDim.x) qs[i] = qsrc[i];
    __syncthreads();

    const int lane = threadIdx.x & 31;
    const int t = lane & 7;
    const int oct = threadIdx.x >> 3;  // 16 octets per CTA
    // uniform trip count for the whole CTA: the shuffles below need full warps
    for (int s0 = blockIdx.x * 64; s0 < min(S, (blockIdx.x + 1) * 64); s0 += 16) {
        const int s = s0 + oct;
        const bool valid = s < S;
        const int64_t tok = (static_cast<int64_t>(b) * Hkv + hkv) * S + (valid ? s : 0);
        float kv[E];
#pragma unroll
        for (int i = 0; i < E / 8; i++) {
            const uint32_t w = load_run<BITS>(k_codes + tok * PD, t + 8 * i);
#pragma unroll
            for (int c = 0; c < 8; c++) kv[8 * i + c] = lut[(w >> (BITS * c)) & ((1u << BITS) - 1u)];
        }
        const float nf = to_float<NormT>(k_norms[tok]);
        for (int r = 0; r < rows; r++) {
            float acc = 0.f;
#pragma unroll
            for (int i = 0; i < E / 8; i++)
#pragma unroll
                for (int c = 0; c < 8; c++)
                    acc = fmaf(qs[r * D + 8 * (t + 8 * i) + c], kv[8 * i + c], acc);
            acc += __shfl_xor_sync(0xffffffffu, acc, 1);
            acc += __shfl_xor_sync(0xffffffffu, acc, 2);
            acc += __shfl_xor_sync(0xffffffffu, acc, 4);
            if (t == 0 && valid) {
                const int hq = hkv * group + r / q_len;
                const int tq = r % q_len;
                out[((static_cast<int64_t>(b) * Hq + hq) * q_len + tq) * S + s] = nf * acc * scale;
            }
        }
    }
}

}  // namespace ftq
