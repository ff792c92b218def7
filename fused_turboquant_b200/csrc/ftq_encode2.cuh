// Fused KV encode, throughput version.  Same arithmetic, bit for bit, as
// encode_kernel (ftq_encode.cuh) -- which restates TurboQuantMSE._encode_unfused of
// the reference (src/fused_turboquant/core/quantizer.py:137-160) -- with the
// instruction count cut to what the B200 issue slots allow:
//
//  * every lane carries TWO vectors packed into 64-bit register pairs and runs
//    the butterfly, scaling, squares, running sums and the division on
//    Blackwell's packed fp32 instructions (add/sub/mul/fma .f32x2, round to
//    nearest, each half an ordinary IEEE operation);
//  * the lane<->register transposition between butterfly stage h=4 and h=8
//    goes once through shared memory (conflict-free) instead of three rounds of
//    shuffles and selects;
//  * y / denom is q = y*r refined twice with exact FMA residuals (r the correctly
//    rounded reciprocal), which yields the correctly rounded quotient that
//    __fdiv_rn returns;
//  * bucketisation is one table lookup: x is mapped to one of 257 cells of
//    [-1, 1] with a single FMA (monotone in x); a cell contains at most one
//    decision boundary (checked on the host), so
//    code = codes below the cell + [x > boundary in the cell], the comparison
//    done as a saturating FMA; codes are accumulated into the packed word in
//    floating point (exact below 2^24).
#pragma once

#include "ftq_encode.cuh"

namespace ftq {

constexpr int kQuantCells = 257;
constexpr float kCellScale = 128.0f;                 // cells per unit of x
constexpr float kCellMagic = 98304.0f + 128.0f;      // 1.5 * 2^16 + scale: ulp = 2^-7
constexpr float kStepScale = 1.2676506002282294e30f; // 2^100

struct QuantCell {
    float neg_thr_scaled;  // -boundary * 2^100, or -FLT_MAX when the cell holds no boundary
    float base;            // number of interior boundaries in lower cells
};

struct Encode2Tables {
    SignBits signs;
    float rsqrt_d;
    QuantCell cells[kQuantCells];
};

typedef unsigned long long u64;

__device__ __forceinline__ u64 pk2(float lo, float hi) {
    u64 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void upk2(u64 v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ u64 add2(u64 a, u64 b) {
    u64 r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ u64 sub2(u64 a, u64 b) {
    u64 r;
    asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ u64 mul2(u64 a, u64 b) {
    u64 r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ u64 fma2(u64 a, u64 b, u64 c) {
    u64 r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
__device__ __forceinline__ float fma_sat(float a, float b, float c) {
    float r;
    asm("fma.rn.sat.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}

// Raw (not yet widened) run of 8 consecutive elements, so that the next iteration's loads can
// be in flight while the current vectors are processed.
template <typename T> struct Raw8 { uint4 v; };
template <> struct Raw8<float> { float4 a, b; };

template <typename T>
__device__ __forceinline__ void load_raw8(const T* p, Raw8<T>& r) {
    r.v = __ldg(reinterpret_cast<const uint4*>(p));
}
template <>
__device__ __forceinline__ void load_raw8<float>(const float* p, Raw8<float>& r) {
    r.a = __ldg(reinterpret_cast<const float4*>(p));
    r.b = __ldg(reinterpret_cast<const float4*>(p) + 1);
}
template <typename T>
__device__ __forceinline__ void widen8(const Raw8<T>& r, float (&o)[8]);
template <>
__device__ __forceinline__ void widen8<float>(const Raw8<float>& r, float (&o)[8]) {
    o[0] = r.a.x; o[1] = r.a.y; o[2] = r.a.z; o[3] = r.a.w;
    o[4] = r.b.x; o[5] = r.b.y; o[6] = r.b.z; o[7] = r.b.w;
}
template <>
__device__ __forceinline__ void widen8<__nv_bfloat16>(const Raw8<__nv_bfloat16>& r, float (&o)[8]) {
    o[0] = bf16_lo(r.v.x); o[1] = bf16_hi(r.v.x);
    o[2] = bf16_lo(r.v.y); o[3] = bf16_hi(r.v.y);
    o[4] = bf16_lo(r.v.z); o[5] = bf16_hi(r.v.z);
    o[6] = bf16_lo(r.v.w); o[7] = bf16_hi(r.v.w);
}
template <>
__device__ __forceinline__ void widen8<__half>(const Raw8<__half>& r, float (&o)[8]) {
    const uint32_t w[4] = {r.v.x, r.v.y, r.v.z, r.v.w};
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[j]));
        o[2 * j] = f.x;
        o[2 * j + 1] = f.y;
    }
}

template <typename T>
__device__ __forceinline__ void zero_raw8(Raw8<T>& r) { r.v = make_uint4(0u, 0u, 0u, 0u); }
template <>
__device__ __forceinline__ void zero_raw8<float>(Raw8<float>& r) {
    r.a = make_float4(0.f, 0.f, 0.f, 0.f);
    r.b = r.a;
}
// 16-bit inputs: flip the signs on the packed pairs (mask bits 15 / 31), then widen.
template <typename T>
__device__ __forceinline__ void widen8_signed(const Raw8<T>& r, const uint32_t* sg, float (&o)[8]) {
    Raw8<T> f;
    f.v = make_uint4(r.v.x ^ sg[0], r.v.y ^ sg[1], r.v.z ^ sg[2], r.v.w ^ sg[3]);
    widen8<T>(f, o);
}

// In-lane butterfly stage on register-index bit B of packed pairs.
template <int E, int B>
__device__ __forceinline__ void stage2(u64 (&p)[E]) {
#pragma unroll
    for (int r = 0; r < E; r++) {
        if ((r & (1 << B)) == 0) {
            const u64 a = p[r], b = p[r | (1 << B)];
            p[r] = add2(a, b);
            p[r | (1 << B)] = sub2(a, b);
        }
    }
}

// Transpose slot of one pair of vectors (A, B): [run m = coordinate / 8][element c][A, B],
// runs 20 floats apart, so that the 16-byte stores of an octet (lanes = consecutive runs) and
// the 8-byte loads of a half warp (lanes = consecutive elements, second octet 16 banks on)
// cover all 32 banks without conflicts.
constexpr int kRunStride = 20;
__host__ __device__ constexpr int encode2_slot_floats(int D) {
    const int s = (D / 8) * kRunStride;
    return s % 32 == 16 ? s : s + 16;
}
__host__ __device__ constexpr int encode2_smem_bytes(int D, int warps) {
    return warps * 4 * encode2_slot_floats(D) * 4;  // dynamic part (the table is static)
}

__host__ __device__ constexpr int encode2_threads(int D) { return D >= 256 ? 512 : 256; }

template <int D, int BITS, typename T>
__global__ void __launch_bounds__(encode2_threads(D), 512 / encode2_threads(D))
encode2_kernel(EncodeSource src, EncodeSink sink, const Encode2Tables tab, int64_t n_vec) {
    constexpr int E = D / kOctet;
    constexpr int NCH = E / 8;
    constexpr int SLOT = encode2_slot_floats(D);
    constexpr int NW = BITS == 2 ? (E + 15) / 16 : E / 8;  // packed words per lane
    constexpr int IPW = BITS == 2 ? 16 : 8;                 // items per word
    constexpr int CPF = 24 / BITS;                          // codes per fp32 accumulator
    constexpr int FPW = (IPW + CPF - 1) / CPF;              // accumulators per word
    constexpr bool NARROW = sizeof(T) == 2;                 // bf16 / fp16 input

    // the quantiser table is a static array: its shared-memory offset is then an immediate of
    // the load and the per-element address is one bit-select (cell row | lane column)
    __shared__ __align__(128) float2 lut[kQuantCells * 16];            // [257][16]
    extern __shared__ __align__(16) uint8_t smem_raw[];
    float* tbuf = reinterpret_cast<float*>(smem_raw);                  // [warps][4][SLOT]

    const int tid = threadIdx.x;
    const int lane = tid & 31, wip = tid >> 5;
    const int t = lane & 7, sub = lane >> 3;
    for (int i = tid; i < kQuantCells * 16; i += blockDim.x)
        lut[i] = make_float2(tab.cells[i >> 4].neg_thr_scaled, tab.cells[i >> 4].base);
    __syncthreads();
    const uint32_t lut_col = (lane & 15) * 8;
    float* slot = tbuf + (wip * 4 + sub) * SLOT;

    const int64_t warp = (static_cast<int64_t>(blockIdx.x) * blockDim.x + tid) >> 5;
    const int64_t n_warps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
    const T* xbase = static_cast<const T*>(src.base) + blockIdx.y * src.layer_stride;
    const int64_t sink_layer = blockIdx.y * sink.layer_stride;

    // sign masks in the load layout: per element for fp32 input; for 16-bit input one mask per
    // packed pair of elements (bits 15 and 31), applied before the values are widened
    constexpr int NSGN = NARROW ? E / 2 : E;
    uint32_t sgn[NSGN];
#pragma unroll
    for (int r = 0; r < NSGN; r++) {
        if constexpr (NARROW)
            sgn[r] = (sign_mask(tab.signs, load_coord(t, 2 * r)) >> 16) |
                     sign_mask(tab.signs, load_coord(t, 2 * r + 1));
        else
            sgn[r] = sign_mask(tab.signs, load_coord(t, r));
    }
    const u64 scale2 = pk2(tab.rsqrt_d, tab.rsqrt_d);
    const u64 cs2 = pk2(kCellScale, kCellScale), cm2 = pk2(kCellMagic, kCellMagic);
    const TransposeConsts<BITS> tc = transpose_consts<BITS>(lane);

    // the two vectors of this lane for the group starting at `base`: issue their loads (zeros
    // stand in for vectors past the end) and fetch the slots their codes go to
    Raw8<T> rawA[NCH], rawB[NCH];
    int64_t slotA = -1, slotB = -1;
    auto issue_loads = [&](int64_t base) {
        const int64_t vA = base + sub, vB = base + 4 + sub;
        slotA = load_slot(sink, vA, vA < n_vec);
        slotB = load_slot(sink, vB, vB < n_vec);
        if (vA < n_vec) {
            const int64_t o = fast_div(static_cast<uint32_t>(vA), src.div_inner);
            const T* row = xbase + o * src.outer_stride + (vA - o * src.n_inner) * src.inner_stride;
#pragma unroll
            for (int i = 0; i < NCH; i++) load_raw8<T>(row + 8 * (t + 8 * i), rawA[i]);
        } else {
#pragma unroll
            for (int i = 0; i < NCH; i++) zero_raw8<T>(rawA[i]);
        }
        if (vB < n_vec) {
            const int64_t o = fast_div(static_cast<uint32_t>(vB), src.div_inner);
            const T* row = xbase + o * src.outer_stride + (vB - o * src.n_inner) * src.inner_stride;
#pragma unroll
            for (int i = 0; i < NCH; i++) load_raw8<T>(row + 8 * (t + 8 * i), rawB[i]);
        } else {
#pragma unroll
            for (int i = 0; i < NCH; i++) zero_raw8<T>(rawB[i]);
        }
    };
    if (warp * 8 < n_vec) issue_loads(warp * 8);

    for (int64_t base = warp * 8; base < n_vec; base += n_warps * 8) {
        const int64_t vA = base + sub, vB = base + 4 + sub;
        const bool okA = vA < n_vec, okB = vB < n_vec;
        const int64_t cur_slotA = slotA, cur_slotB = slotB;
        u64 p[E];
#pragma unroll
        for (int i = 0; i < NCH; i++) {
            float a[8], b[8];
            if constexpr (NARROW) {
                widen8_signed<T>(rawA[i], &sgn[4 * i], a);
                widen8_signed<T>(rawB[i], &sgn[4 * i], b);
            } else {
                widen8<T>(rawA[i], a);
                widen8<T>(rawB[i], b);
#pragma unroll
                for (int c = 0; c < 8; c++) {
                    a[c] = __uint_as_float(__float_as_uint(a[c]) ^ sgn[8 * i + c]);
                    b[c] = __uint_as_float(__float_as_uint(b[c]) ^ sgn[8 * i + c]);
                }
            }
#pragma unroll
            for (int c = 0; c < 8; c++) p[8 * i + c] = pk2(a[c], b[c]);
        }
        // next group's loads fly while this one is processed (16-bit inputs: 4 registers per run)
        if constexpr (NARROW) {
            if (base + n_warps * 8 < n_vec) issue_loads(base + n_warps * 8);
        }
        // stages h = 1, 2, 4 on the coordinates inside a run
        stage2<E, 0>(p);
        stage2<E, 1>(p);
        stage2<E, 2>(p);

        // lane <-> register transposition through shared memory, both vectors at once:
        // (lane t, register c + 8i) = coordinate 8(t + 8i) + c   ->   (lane l, register k) = l + 8k
        __syncwarp();
#pragma unroll
        for (int i = 0; i < NCH; i++) {
            float* run = slot + (t + 8 * i) * kRunStride;
#pragma unroll
            for (int c = 0; c < 8; c += 2) {
                ulonglong2 v2;
                v2.x = p[8 * i + c];
                v2.y = p[8 * i + c + 1];
                *reinterpret_cast<ulonglong2*>(run + 2 * c) = v2;
            }
        }
        __syncwarp();
#pragma unroll
        for (int k = 0; k < E; k++)
            p[k] = *reinterpret_cast<const u64*>(slot + k * kRunStride + 2 * t);

        // stages h = 8, 16, ... : register bits 0.. of the new layout
        stage2<E, 0>(p);
        stage2<E, 1>(p);
        stage2<E, 2>(p);
        if constexpr (E >= 16) stage2<E, 3>(p);
        if constexpr (E >= 32) stage2<E, 4>(p);

        // scale, 8-way strided sum of squares (lane l = running sum l), ordered octet sum
        u64 acc = pk2(0.f, 0.f);
#pragma unroll
        for (int k = 0; k < E; k++) {
            p[k] = mul2(p[k], scale2);
            // the squares are rounded on their own (scalar mul.rn): a packed multiply feeding a
            // packed add may be contracted into a fused multiply-add, which changes the norm
            float ya, yb;
            upk2(p[k], ya, yb);
            acc = add2(acc, pk2(__fmul_rn(ya, ya), __fmul_rn(yb, yb)));
        }
        u64 s = __shfl_sync(0xffffffffu, acc, 0, 8);
#pragma unroll
        for (int l = 1; l < 8; l++) s = add2(s, __shfl_sync(0xffffffffu, acc, l, 8));
        float sA, sB;
        upk2(s, sA, sB);
        const float normA = __fsqrt_rn(sA), normB = __fsqrt_rn(sB);
        const float dA = __fadd_rn(normA, 1e-8f), dB = __fadd_rn(normB, 1e-8f);
        const u64 r2 = pk2(__frcp_rn(dA), __frcp_rn(dB));
        const u64 nd2 = pk2(-dA, -dB);

        // normalise, bucketise, accumulate the packed words in floating point
        u64 wf[NW * FPW];
#pragma unroll
        for (int i = 0; i < NW * FPW; i++) wf[i] = pk2(0.f, 0.f);
#pragma unroll
        for (int k = 0; k < E; k++) {
            u64 q = mul2(p[k], r2);
            u64 e = fma2(nd2, q, p[k]);
            q = fma2(e, r2, q);
            e = fma2(nd2, q, p[k]);
            q = fma2(e, r2, q);
            // cell = floor((x + 1) * 128 rounded to 1/128); row = cell * 128 bytes
            const u64 cv = fma2(q, cs2, cm2);
            float cA, cB, qA, qB;
            upk2(cv, cA, cB);
            upk2(q, qA, qB);
            float2 eA, eB;
            {
                const uint32_t oA = (__float_as_uint(cA) & 0xFF80u) | lut_col;
                const uint32_t oB = (__float_as_uint(cB) & 0xFF80u) | lut_col;
                eA = *reinterpret_cast<const float2*>(reinterpret_cast<const uint8_t*>(lut) + oA);
                eB = *reinterpret_cast<const float2*>(reinterpret_cast<const uint8_t*>(lut) + oB);
            }
            const float stA = fma_sat(qA, kStepScale, eA.x);
            const float stB = fma_sat(qB, kStepScale, eB.x);
            const u64 code = add2(pk2(eA.y, eB.y), pk2(stA, stB));
            // position of code k inside its word (see encode_kernel)
            const int word = BITS == 2 ? (k >> 4) : (k >> 3);
            const int pos = BITS == 2 ? (((k >> 1) & 7) | ((k & 1) << 3)) : (k & 7);
            const int fi = word * FPW + pos / CPF;
            const float sc = static_cast<float>(1u << (BITS * (pos % CPF)));
            wf[fi] = fma2(code, pk2(sc, sc), wf[fi]);
        }
        uint32_t wA[NW], wB[NW];
#pragma unroll
        for (int i = 0; i < NW; i++) {
            float a0, b0;
            upk2(wf[i * FPW], a0, b0);
            wA[i] = __float2uint_rn(a0);
            wB[i] = __float2uint_rn(b0);
            if constexpr (FPW == 2) {
                float a1, b1;
                upk2(wf[i * FPW + 1], a1, b1);
                wA[i] |= __float2uint_rn(a1) << (BITS * CPF);
                wB[i] |= __float2uint_rn(b1) << (BITS * CPF);
            }
        }
        emit_vector<D, BITS>(wA, normA, okA, vA, cur_slotA, sink, sink_layer, lane, tc);
        emit_vector<D, BITS>(wB, normB, okB, vB, cur_slotB, sink, sink_layer, lane, tc);
        if constexpr (!NARROW) {
            if (base + n_warps * 8 < n_vec) issue_loads(base + n_warps * 8);
        }
    }
}

}  // namespace ftq
