// Shared device helpers for the fused-turboquant sm_100a kernels.
//
// Lane layout used by every kernel that runs the Hadamard butterfly
// ("octet layout"): 8 lanes cooperate on one head vector of D coordinates,
// each lane holding E = D/8 values in registers.
//
//   load layout   : lane t, register r = c + 8*i  <->  coordinate 8*(t + 8*i) + c
//                   (a lane owns whole runs of 8 consecutive coordinates, so a
//                   bf16 row is read with one 16-byte load per run)
//   final layout  : lane l, register k            <->  coordinate l + 8*k
//
// The butterfly stages run in the order h = 1, 2, 4, ... (the order of
// core/hadamard.py:38-48 of the reference, which fixes the rounding).  Stages
// on coordinate bits held in registers are plain in-lane add/sub.  The three
// stages on bits held in the lane id are done by first exchanging that lane
// bit with an already-finished register bit (half of the registers cross the
// lane boundary, one shuffle each) and then running the stage in-lane.  That
// exchange is what turns the load layout into the final layout, and the final
// layout is exactly what the norm needs: lane l's registers are the terms of
// running sum l of the 8-way strided reduction.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace ftq {

constexpr int kOctet = 8;          // lanes per head vector
constexpr int kPageTokens = 16;    // tokens per page
constexpr int kMaxLevels = 16;

enum : int { kF32 = 0, kF16 = 1, kBF16 = 2 };

__host__ __device__ constexpr int packed_dim(int d, int bits) { return d * bits / 8; }

// ---------------------------------------------------------------- tables

// Small per-call tables, passed by value as kernel parameters (they live in
// the constant bank; no device allocation, no extra load latency).
struct SignBits {
    uint32_t w[8];  // bit i of the concatenation = 1 when signs[i] is -1 (D <= 256)
};

struct Codebook {
    float v[kMaxLevels];  // levels[0 .. 2^bits)  or interior boundaries [1 .. 2^bits) at v[0..]
};

// ---------------------------------------------------------------- loads

__device__ __forceinline__ float bf16_lo(uint32_t u) { return __uint_as_float(u << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t u) { return __uint_as_float(u & 0xffff0000u); }

// Load 8 consecutive elements starting at p (16-byte aligned for 2-byte types,
// 32-byte aligned for fp32) and widen to fp32.
template <typename T>
__device__ __forceinline__ void load8(const T* p, float (&o)[8]);

template <>
__device__ __forceinline__ void load8<float>(const float* p, float (&o)[8]) {
    const float4 a = __ldg(reinterpret_cast<const float4*>(p));
    const float4 b = __ldg(reinterpret_cast<const float4*>(p) + 1);
    o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w;
    o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
}

template <>
__device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float (&o)[8]) {
    const uint4 a = __ldg(reinterpret_cast<const uint4*>(p));
    o[0] = bf16_lo(a.x); o[1] = bf16_hi(a.x);
    o[2] = bf16_lo(a.y); o[3] = bf16_hi(a.y);
    o[4] = bf16_lo(a.z); o[5] = bf16_hi(a.z);
    o[6] = bf16_lo(a.w); o[7] = bf16_hi(a.w);
}

template <>
__device__ __forceinline__ void load8<__half>(const __half* p, float (&o)[8]) {
    const uint4 a = __ldg(reinterpret_cast<const uint4*>(p));
    const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const __half2 h = *reinterpret_cast<const __half2*>(&w[j]);
        const float2 f = __half22float2(h);
        o[2 * j] = f.x;
        o[2 * j + 1] = f.y;
    }
}

template <typename T>
__device__ __forceinline__ T from_float(float f);
template <>
__device__ __forceinline__ float from_float<float>(float f) { return f; }
template <>
__device__ __forceinline__ __half from_float<__half>(float f) { return __float2half_rn(f); }
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float f) {
    return __float2bfloat16_rn(f);
}

template <typename T>
__device__ __forceinline__ float to_float(T v);
template <>
__device__ __forceinline__ float to_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_float<__half>(__half v) { return __half2float(v); }
template <>
__device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) {
    return __bfloat162float(v);
}

// ------------------------------------------------------------- division by a launch constant
// floor(n / d) for 0 <= n < 2^31 as one wide multiply and a shift: mul = ceil(2^sh / d) with
// sh = 31 + ceil(log2 d) fits in 32 bits, and n * (mul * d - 2^sh) < 2^sh keeps the floor exact.
struct FastDiv {
    uint32_t d, mul, sh;
};
inline FastDiv make_fastdiv(uint32_t d) {
    FastDiv f;
    f.d = d;
    uint32_t l = 0;
    while ((1ull << l) < d) l++;
    f.sh = 31 + l;
    f.mul = static_cast<uint32_t>(((1ull << f.sh) + d - 1) / d);
    return f;
}
__host__ __device__ __forceinline__ uint32_t fast_div(uint32_t n, const FastDiv& f) {
    return static_cast<uint32_t>((static_cast<uint64_t>(n) * f.mul) >> f.sh);
}

// ------------------------------------------------------------- butterfly

// Sign of coordinate `coord` as a 0 / 0x80000000 mask.
__device__ __forceinline__ uint32_t sign_mask(const SignBits& s, int coord) {
    return ((s.w[coord >> 5] >> (coord & 31)) & 1u) << 31;
}

// In-lane stage on register-index bit B: for every pair (r, r | 1<<B) the low
// register gets a + b and the high one a - b (plain fp32 add/sub, one rounding each).
template <int E, int B>
__device__ __forceinline__ void stage_inlane(float (&v)[E]) {
#pragma unroll
    for (int r = 0; r < E; r++) {
        if ((r & (1 << B)) == 0) {
            const float a = v[r];
            const float b = v[r | (1 << B)];
            v[r] = __fadd_rn(a, b);
            v[r | (1 << B)] = __fsub_rn(a, b);
        }
    }
}

// Exchange lane-id bit LB with register-index bit RB: the value at
// (lane bit x, register bit y) moves to (lane bit y, register bit x).
// Half of the registers travel; one shuffle per travelling register.
template <int E, int LB, int RB>
__device__ __forceinline__ void swap_lane_reg(float (&v)[E], int lane) {
    const bool hi = (lane >> LB) & 1;
#pragma unroll
    for (int r = 0; r < E; r++) {
        if ((r & (1 << RB)) == 0) {
            const int r1 = r | (1 << RB);
            const float send = hi ? v[r] : v[r1];
            const float recv = __shfl_xor_sync(0xffffffffu, send, 1 << LB);
            if (hi) v[r] = recv; else v[r1] = recv;
        }
    }
}

// Unnormalised Walsh-Hadamard butterfly over D = 8*E coordinates spread over an
// octet of lanes; input in the load layout, output in the final layout.
template <int E>
__device__ __forceinline__ void octet_fwht(float (&v)[E], int lane) {
    stage_inlane<E, 0>(v);            // h = 1
    stage_inlane<E, 1>(v);            // h = 2
    stage_inlane<E, 2>(v);            // h = 4
    swap_lane_reg<E, 0, 0>(v, lane);  // coordinate bit 3 <-> bit 0
    stage_inlane<E, 0>(v);            // h = 8
    swap_lane_reg<E, 1, 1>(v, lane);  // bit 4 <-> bit 1
    stage_inlane<E, 1>(v);            // h = 16
    swap_lane_reg<E, 2, 2>(v, lane);  // bit 5 <-> bit 2
    stage_inlane<E, 2>(v);            // h = 32
    if constexpr (E >= 16) stage_inlane<E, 3>(v);  // h = 64
    if constexpr (E >= 32) stage_inlane<E, 4>(v);  // h = 128
}

// Coordinate held by (lane t, register r) in the load layout.
__device__ __forceinline__ constexpr int load_coord(int t, int r) {
    return 8 * (t + 8 * (r >> 3)) + (r & 7);
}

}  // namespace ftq
