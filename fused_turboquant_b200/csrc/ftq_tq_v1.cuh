// vLLM-v1 "TURBOQUANT" slot format: fused store and split-KV decode attention.
//
// Slot of one (token, KV head), at kv_cache + block*stride_block + pos*stride_pos +
// head*stride_head (slots are only 2-byte aligned: their size is rounded up to even):
//     [key codes (D*kb/8) | key norm fp16 | value codes (D*vb/8, or D for 8 bits) |
//      value scale fp16 | value zero fp16]
//
// Store  = the reference's in-kernel-rotation store
//          (src/fused_turboquant/vllm_plugin/triton_inkernel_store.py:365-440 and 39-330):
//          norm of the RAW key, normalise, Hadamard butterfly without signs, * 1/sqrt(D),
//          code = #{midpoints <= y}, pack; values: per-vector min/max uniform quantisation,
//          q = int((v - min) / scale + 0.5), scale and min stored as fp16.
// Decode = `_tq_decode_stage1_offset` (vllm_plugin/triton_decode_offset.py:42-444) for all query
//          heads of a GQA group at once (each slot is read once per KV head, not once per query
//          head), writing the same [B, Hq, splits, D+1] partials (acc / l, lse), followed by a
//          merge kernel with the semantics of the stock stage-2 kernel the reference launches
//          (vllm_plugin/v1_backend.py:1068-1085) and, optionally, the Hadamard transform that
//          maps an output accumulated over rotated values back (v1_backend.py:1088-1092).
//
// Key "bits" = 8 selects FP8 keys (vLLM's stock TurboQuantConfig: key_quant_bits == 8;
// triton_inkernel_store.py:80-91, triton_decode_offset.py:175-194): the key field is D bytes of
// e4m3 (rotated key * norm, round to nearest even, saturating, as the cvt instruction the
// reference's cast compiles to) with no norm behind it; score = sum(q_rot * k) * scale.
//
// The order in which the key's squares are added is not fixed by the reference (a Triton
// reduction); here: 8 running sums in register order, combined pairwise over the octet.
#pragma once

#include <cuda_fp8.h>

#include <cfloat>
#include <type_traits>

#include "ftq_attn.cuh"
#include "ftq_encode2.cuh"

namespace ftq {

constexpr int kTqMaxMid = 15;  // key codes of 1..4 bits

// 8-bit Lloyd-Max key codes (256 centroids, one byte per coordinate + the fp16 norm; the
// reference's BoundaryTurboQuantConfig with key_use_fp8_at_8bit = False,
// vllm_plugin/boundary_tq_config.py:26-35): the kernels are instantiated with KB = 8 and K8M =
// true and get their table -- 255 midpoints for the store, 256 centroids for the decode -- as a
// second kernel parameter (1 KB of constant bank, no device allocation); everybody else passes
// an empty struct.
constexpr int kTqKeyBitsMse8 = 264;  // the host-side key_bits value that selects it
struct TqTable256 { float v[256]; };
struct TqNoTable { int unused; };
template <bool K8M> using TqTable = std::conditional_t<K8M, TqTable256, TqNoTable>;

struct TqStoreParams {
    const void* key;       // [n_tokens, Hkv, D], strides in elements
    const void* value;
    int64_t token_stride, head_stride;
    int Hkv;
    FastDiv div_hkv;
    uint8_t* kv_cache;
    int64_t stride_block, stride_pos, stride_head;  // bytes
    int block_size;
    FastDiv div_block;
    const int64_t* slot_mapping;
    float midpoints[kTqMaxMid];
    float rsqrt_d;  // 1.0f / sqrtf(D), as the reference computes it
    // layers in one launch (blockIdx.y = layer): element / byte distances between the layers'
    // key / value tensors and caches; every layer uses the same slot_mapping
    int64_t kv_layer_stride, cache_layer_stride;
    // slots at or beyond it (a stale or corrupt mapping) are skipped like negative ones
    int64_t slot_limit;
};

__host__ __device__ constexpr int tq_value_bytes(int d, int vb) { return vb == 8 ? d : d * vb / 8; }

__device__ __forceinline__ void store_u32_as_halves(uint8_t* dst, uint32_t w) {
    reinterpret_cast<uint16_t*>(dst)[0] = static_cast<uint16_t>(w);
    reinterpret_cast<uint16_t*>(dst)[1] = static_cast<uint16_t>(w >> 16);
}

// 1-bit codes of a vector in the butterfly's output layout (lane l of the octet, register k =
// coordinate l + 8k; bit k of `mine` is this lane's code of register k): byte k of the packed
// codes is the octet's ballot of register k (coordinate 8k + j in bit j, as
// triton_inkernel_store.py:138-146 packs them).  Called by all 32 lanes.
template <int E>
__device__ __forceinline__ void emit_bits1(uint32_t mine, uint8_t* dst, bool store, int lane) {
    const int t = lane & 7, sub = lane >> 3;
    uint32_t wd[E / 4];
#pragma unroll
    for (int i = 0; i < E / 4; i++) wd[i] = 0u;
#pragma unroll
    for (int k = 0; k < E; k++) {
        const uint32_t b = (__ballot_sync(0xffffffffu, (mine >> k) & 1u) >> (8 * sub)) & 0xffu;
        wd[k >> 2] |= b << (8 * (k & 3));
    }
#pragma unroll
    for (int j = 0; j < E / 4; j++)
        if (store && t == j) store_u32_as_halves(dst + 4 * j, wd[j]);
}

// code = number of midpoints <= y, found as the reference finds it (binary search on `y >= mid`,
// triton_inkernel_store.py:92-100; the midpoints are strictly ascending, checked on the host):
// bit LVL of the code is decided by one comparison against the midpoint that the bits above it
// select.  tq_pick builds that midpoint with a tree of selects over the known bits (2^k - 1 selects
// for the k-th bit from the top), so a 4-bit code costs 4 compares + 11 selects instead of 15
// compares + 15 adds.
template <int KB, int LVL, int DEPTH, int PREFIX>
__device__ __forceinline__ float tq_pick(const bool (&bit)[4], const float (&m)[kTqMaxMid]) {
    if constexpr (DEPTH == KB - 1 - LVL) {
        return m[(PREFIX << (LVL + 1)) | ((1 << LVL) - 1)];
    } else {
        return bit[KB - 1 - DEPTH] ? tq_pick<KB, LVL, DEPTH + 1, PREFIX * 2 + 1>(bit, m)
                                   : tq_pick<KB, LVL, DEPTH + 1, PREFIX * 2>(bit, m);
    }
}
template <int KB, int LVL>
__device__ __forceinline__ void tq_search_level(float y, bool (&bit)[4], const float (&m)[kTqMaxMid]) {
    bit[LVL] = y >= tq_pick<KB, LVL, 0, 0>(bit, m);
    if constexpr (LVL > 0) tq_search_level<KB, LVL - 1>(y, bit, m);
}
// ORs the code of y, shifted left by `shift`, into w (one predicated OR per bit).
template <int KB>
__device__ __forceinline__ void tq_or_code(float y, const float (&m)[kTqMaxMid], uint32_t& w, int shift) {
    bool bit[4] = {false, false, false, false};
    tq_search_level<KB, KB - 1>(y, bit, m);
#pragma unroll
    for (int b = 0; b < KB; b++)
        if (bit[b]) w |= 1u << (shift + b);
}

// Round a value the way a tensor of the input dtype would hold it.
template <typename T>
__device__ __forceinline__ float round_as(float v);
template <> __device__ __forceinline__ float round_as<float>(float v) { return v; }
template <> __device__ __forceinline__ float round_as<__half>(float v) {
    return __half2float(__float2half_rn(v));
}
template <> __device__ __forceinline__ float round_as<__nv_bfloat16>(float v) {
    return __bfloat162float(__float2bfloat16_rn(v));
}

// ROTV: the values are Hadamard-transformed (no signs, * 1/sqrt(D), rounded to the input dtype)
// before they are quantised, i.e. the cache keeps them in the rotated space
// (src/fused_turboquant/vllm_plugin/v1_backend.py:727-740 does this with a matrix product).
// LMV (4-bit values only): Lloyd-Max value codes (TURBOQUANT_V_LLOYD_MAX,
// triton_inkernel_store.py:159-203): the value is normalised like the key (norm = sqrt(sum + 1e-16),
// v / (norm + 1e-8)), bucketised against the KEY midpoints, packed as 4-bit codes; the norm goes
// where the scale would and the zero point is 0.  The squares are added in register order per
// lane, then pairwise over the octet -- in whichever layout the values sit (after the fused
// rotation: lane l holds the coordinates l + 8k).
template <int D, int KB, int VB, typename T, bool ROTV, bool LMV = false, bool K8M = false>
__global__ void __launch_bounds__(256)
tq_store_kernel(const TqStoreParams p, int64_t n_vec, const TqTable<K8M> t8) {
    static_assert(!K8M || KB == 8, "the 256-entry table belongs to 8-bit keys");
    static_assert(!ROTV || VB != 8, "rotated 8-bit values are rotated by the caller");
    static_assert(!LMV || VB == 4, "Lloyd-Max value codes are 4-bit");
    constexpr int E = D / kOctet;
    constexpr int NCH = E / 8;
    constexpr bool KBYTE = KB == 8;             // one byte per coordinate: FP8 or an 8-bit code
    constexpr bool KFP8 = KBYTE && !K8M;
    static_assert(!(KBYTE && LMV), "Lloyd-Max value codes use a 4-bit key codebook");
    constexpr int MSE = D * KB / 8;                      // (8-bit keys: D bytes)
    constexpr int KPS = MSE + (KFP8 ? 0 : 2);
    constexpr int VDB = tq_value_bytes(D, VB);
    constexpr int VMAX = (1 << VB) - 1;
    constexpr int NMID = KBYTE ? 0 : (1 << KB) - 1;
    constexpr int NW = KB == 2 ? (E + 15) / 16 : E / 8;  // (unused for 1-bit codes and 8-bit keys)
    constexpr int KT = (KB == 1 || KBYTE) ? 2 : KB;      // transposition constants: 2..4 bits only
    constexpr int VT = (ROTV && VB != 1) ? VB : 4;

    const int lane = threadIdx.x & 31;
    const int t = lane & 7, sub = lane >> 3;
    const int64_t warp = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int64_t n_warps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
    const TransposeConsts<KT> tc = transpose_consts<KT>(lane);
    const TransposeConsts<VT> tcv = transpose_consts<VT>(lane);
    (void)tc;
    (void)tcv;
    // 8-bit codes: the 255 midpoints in shared memory (lanes search at different places)
    __shared__ float smid[K8M ? 256 : 1];
    if constexpr (K8M) {
        for (int i = threadIdx.x; i < 256; i += blockDim.x) smid[i] = i < 255 ? t8.v[i] : FLT_MAX;
        __syncthreads();
    }
    // code = number of midpoints <= y (what the reference's binary search returns,
    // triton_inkernel_store.py:92-100, for strictly ascending midpoints)
    auto code8 = [&](float yv) {
        uint32_t idx = 0;
#pragma unroll
        for (int step = 128; step >= 1; step >>= 1)
            if (yv >= smid[K8M ? idx + step - 1 : 0]) idx += step;
        return idx;
    };
    (void)code8;

    for (int64_t base = warp * 4; base < n_vec; base += n_warps * 4) {
        const int64_t v = base + sub;
        const bool valid = v < n_vec;
        const uint32_t token = valid ? fast_div(static_cast<uint32_t>(v), p.div_hkv) : 0u;
        const int head = valid ? static_cast<int>(static_cast<uint32_t>(v) - token * p.Hkv) : 0;
        // (requested here, looked at only after the key's arithmetic: the warp does not wait for it)
        const int64_t slot = valid ? p.slot_mapping[token] : -1;
        const int64_t row_off = blockIdx.y * p.kv_layer_stride +
                                static_cast<int64_t>(token) * p.token_stride + head * p.head_stride;

        // ---- key: raw norm, normalise, butterfly, midpoint search
        float y[E];
#pragma unroll
        for (int i = 0; i < NCH; i++) {
            float tmp[8];
            if (valid) {
                load8<T>(static_cast<const T*>(p.key) + row_off + 8 * (t + 8 * i), tmp);
            } else {
#pragma unroll
                for (int c = 0; c < 8; c++) tmp[c] = 0.f;
            }
#pragma unroll
            for (int c = 0; c < 8; c++) y[8 * i + c] = tmp[c];
        }
        float s = 0.f;
#pragma unroll
        for (int r = 0; r < E; r++) s = __fadd_rn(s, __fmul_rn(y[r], y[r]));
        s = __fadd_rn(s, __shfl_xor_sync(0xffffffffu, s, 1));
        s = __fadd_rn(s, __shfl_xor_sync(0xffffffffu, s, 2));
        s = __fadd_rn(s, __shfl_xor_sync(0xffffffffu, s, 4));
        const float norm = __fsqrt_rn(__fadd_rn(s, 1e-16f));
        const float den = __fadd_rn(norm, 1e-8f);
#pragma unroll
        for (int r = 0; r < E; r++) y[r] = __fdiv_rn(y[r], den);
        octet_fwht<E>(y, lane);  // -> (lane l, register k) = coordinate l + 8k

        // negative = padding (triton_inkernel_store.py:398-399); a slot at or beyond the cache's
        // end is dropped the same way instead of being written out of bounds
        const bool store = valid && static_cast<uint64_t>(slot) < static_cast<uint64_t>(p.slot_limit);
        uint8_t* dst = nullptr;
        if (store) {
            int64_t blk, off;
            if (slot < (1ll << 31)) {
                const uint32_t b32 = fast_div(static_cast<uint32_t>(slot), p.div_block);
                blk = b32;
                off = static_cast<uint32_t>(slot) - b32 * p.block_size;
            } else {
                blk = slot / p.block_size;
                off = slot - blk * p.block_size;
            }
            dst = p.kv_cache + blockIdx.y * p.cache_layer_stride + blk * p.stride_block +
                  off * p.stride_pos + head * p.stride_head;
        }

        if constexpr (KBYTE) {
            // lane l holds the coordinates l + 8k: neighbouring lanes trade bytes so that each
            // stores 16-bit pairs (the even lane those of even k, the odd lane those of odd k)
            const bool odd = lane & 1;
#pragma unroll
            for (int k = 0; k < E; k += 2) {
                uint32_t a, b;
                if constexpr (KFP8) {
                    a = __nv_cvt_float_to_fp8(__fmul_rn(__fmul_rn(y[k], p.rsqrt_d), norm),
                                              __NV_SATFINITE, __NV_E4M3);
                    b = __nv_cvt_float_to_fp8(__fmul_rn(__fmul_rn(y[k + 1], p.rsqrt_d), norm),
                                              __NV_SATFINITE, __NV_E4M3);
                } else {
                    a = code8(__fmul_rn(y[k], p.rsqrt_d));
                    b = code8(__fmul_rn(y[k + 1], p.rsqrt_d));
                }
                const uint32_t recv = __shfl_xor_sync(0xffffffffu, odd ? a : b, 1);
                const uint32_t pair = odd ? (recv | (b << 8)) : (a | (recv << 8));
                const int coord = odd ? t - 1 + 8 * (k + 1) : t + 8 * k;
                if (store) *reinterpret_cast<uint16_t*>(dst + coord) = static_cast<uint16_t>(pair);
            }
        }
        uint32_t w[NW];
#pragma unroll
        for (int i = 0; i < NW; i++) w[i] = 0u;
#pragma unroll
        for (int k = 0; k < (KBYTE ? 0 : E); k++) {
            const float yv = __fmul_rn(y[k], p.rsqrt_d);
            constexpr int SB = KBYTE ? 1 : KB;  // (8-bit keys were stored above)
            if constexpr (KB == 1) {
                tq_or_code<SB>(yv, p.midpoints, w[0], k);
            } else if constexpr (KB == 2) {
                const int pos = ((k >> 1) & 7) | ((k & 1) << 3);
                tq_or_code<SB>(yv, p.midpoints, w[k >> 4], 2 * pos);
            } else {
                tq_or_code<SB>(yv, p.midpoints, w[k >> 3], KB * (k & 7));
            }
        }
        if constexpr (KB == 1) emit_bits1<E>(w[0], dst, store, lane);
#pragma unroll
        for (int i = 0; i < ((KB == 1 || KBYTE) ? 0 : NW); i++) {
            const uint32_t o = octet_transpose_items<KT>(w[i], tc);
            if constexpr (KB == 3) {
                const int g0 = (4 * t) / 3;
                const uint32_t lo = __shfl_sync(0xffffffffu, o, g0, 8);
                const uint32_t hi = __shfl_sync(0xffffffffu, o, g0 + 1, 8);
                const uint64_t cat = (static_cast<uint64_t>(hi) << 24) | lo;
                const uint32_t word = static_cast<uint32_t>(cat >> (8 * ((4 * t) % 3)));
                if (store && t < 6) store_u32_as_halves(dst + 4 * (6 * i + t), word);
            } else {
                const int widx = t + 8 * i;
                if (store && widx < MSE / 4) store_u32_as_halves(dst + 4 * widx, o);
            }
        }
        if (!KFP8 && store && t == 0)
            *reinterpret_cast<__half*>(dst + MSE) = __float2half_rn(norm);

        // ---- value: per-vector uniform quantisation; a lane owns runs of 8 consecutive coordinates
        float vv[E];
#pragma unroll
        for (int i = 0; i < NCH; i++) {
            float tmp[8];
            if (valid) {
                load8<T>(static_cast<const T*>(p.value) + row_off + 8 * (t + 8 * i), tmp);
            } else {
#pragma unroll
                for (int c = 0; c < 8; c++) tmp[c] = 0.f;
            }
#pragma unroll
            for (int c = 0; c < 8; c++) vv[8 * i + c] = tmp[c];
        }
        if constexpr (ROTV) {
            octet_fwht<E>(vv, lane);
#pragma unroll
            for (int k = 0; k < E; k++) vv[k] = round_as<T>(__fmul_rn(vv[k], p.rsqrt_d));
        }
        float mn = INFINITY, mx = -INFINITY;
#pragma unroll
        for (int k = 0; k < E; k++) {
            mn = fminf(mn, vv[k]);
            mx = fmaxf(mx, vv[k]);
        }
#pragma unroll
        for (int m = 1; m < 8; m <<= 1) {
            mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, m));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, m));
        }
        float scale = __fdiv_rn(__fsub_rn(mx, mn), static_cast<float>(VMAX));
        scale = scale > 1e-8f ? scale : 1e-8f;
        float vden = 1.f;
        if constexpr (LMV) {
            float s2 = 0.f;
#pragma unroll
            for (int r = 0; r < E; r++) s2 = __fadd_rn(s2, __fmul_rn(vv[r], vv[r]));
            s2 = __fadd_rn(s2, __shfl_xor_sync(0xffffffffu, s2, 1));
            s2 = __fadd_rn(s2, __shfl_xor_sync(0xffffffffu, s2, 2));
            s2 = __fadd_rn(s2, __shfl_xor_sync(0xffffffffu, s2, 4));
            scale = __fsqrt_rn(__fadd_rn(s2, 1e-16f));  // the norm takes the scale's place
            vden = __fadd_rn(scale, 1e-8f);
            mn = 0.f;                                    // ... and the zero point is 0
        }
        auto vcode = [&](float x) -> uint32_t {
            if constexpr (LMV) {
                uint32_t c = 0;
                tq_or_code<(KBYTE ? 1 : KB)>(__fdiv_rn(x, vden), p.midpoints, c, 0);
                return c;
            } else {
                const float f = __fadd_rn(__fdiv_rn(__fsub_rn(x, mn), scale), 0.5f);
                return static_cast<uint32_t>(min(max(__float2int_rz(f), 0), VMAX));
            }
        };
        if constexpr (!ROTV) {
#pragma unroll
            for (int i = 0; i < NCH; i++) {
                uint32_t q[8];
#pragma unroll
                for (int c = 0; c < 8; c++) q[c] = vcode(vv[8 * i + c]);
                const int run = t + 8 * i;  // coordinates 8*run .. 8*run + 7
                if (!store) continue;
                uint8_t* vd = dst + KPS;
                if constexpr (VB == 8) {
#pragma unroll
                    for (int c = 0; c < 8; c += 2)
                        reinterpret_cast<uint16_t*>(vd + 8 * run)[c >> 1] =
                            static_cast<uint16_t>(q[c] | (q[c + 1] << 8));
                } else {
                    uint32_t word = 0;
#pragma unroll
                    for (int c = 0; c < 8; c++) word |= q[c] << (VB * c);
                    if constexpr (VB == 4) {
                        store_u32_as_halves(vd + 4 * run, word);
                    } else if constexpr (VB == 1) {
                        vd[run] = static_cast<uint8_t>(word);
                    } else if constexpr (VB == 2) {
                        *reinterpret_cast<uint16_t*>(vd + 2 * run) = static_cast<uint16_t>(word);
                    } else {
                        vd[3 * run] = static_cast<uint8_t>(word);
                        vd[3 * run + 1] = static_cast<uint8_t>(word >> 8);
                        vd[3 * run + 2] = static_cast<uint8_t>(word >> 16);
                    }
                }
            }
        } else {
            // rotated values sit in the butterfly's output layout (lane l, register k = coordinate
            // l + 8k): pack and transpose them exactly like the key codes
            constexpr int NWV = VB == 2 ? (E + 15) / 16 : E / 8;
            uint32_t wv[NWV];
#pragma unroll
            for (int i = 0; i < NWV; i++) wv[i] = 0u;
#pragma unroll
            for (int k = 0; k < E; k++) {
                const uint32_t code = vcode(vv[k]);
                if constexpr (VB == 1) {
                    wv[0] |= code << k;
                } else if constexpr (VB == 2) {
                    const int pos = ((k >> 1) & 7) | ((k & 1) << 3);
                    wv[k >> 4] |= code << (2 * pos);
                } else {
                    wv[k >> 3] |= code << (VB * (k & 7));
                }
            }
            uint8_t* vd = dst + KPS;
            if constexpr (VB == 1) emit_bits1<E>(wv[0], vd, store, lane);
#pragma unroll
            for (int i = 0; i < (VB == 1 ? 0 : NWV); i++) {
                const uint32_t o = octet_transpose_items<VT>(wv[i], tcv);
                if constexpr (VB == 3) {
                    const int g0 = (4 * t) / 3;
                    const uint32_t lo = __shfl_sync(0xffffffffu, o, g0, 8);
                    const uint32_t hi = __shfl_sync(0xffffffffu, o, g0 + 1, 8);
                    const uint64_t cat = (static_cast<uint64_t>(hi) << 24) | lo;
                    const uint32_t word = static_cast<uint32_t>(cat >> (8 * ((4 * t) % 3)));
                    if (store && t < 6) store_u32_as_halves(vd + 4 * (6 * i + t), word);
                } else {
                    const int widx = t + 8 * i;
                    if (store && widx < VDB / 4) store_u32_as_halves(vd + 4 * widx, o);
                }
            }
        }
        if (store && t == 0) {
            *reinterpret_cast<__half*>(dst + KPS + VDB) = __float2half_rn(scale);
            *reinterpret_cast<__half*>(dst + KPS + VDB + 2) = __float2half_rn(mn);
        }
    }
}

// ------------------------------------------------------------------ decode

struct TqDecodeParams {
    const void* q;  // [B, Hq, D], original space
    int q_dtype;
    // B counts (layer, sequence) rows: q / mid_o / out are stacked [n_layers * B_seq, ...]; row r
    // reads the cache of layer r / B_seq and the block table / lengths of sequence r % B_seq
    int B, Hq, Hkv;
    int B_seq;
    FastDiv div_bseq;
    int64_t cache_layer_stride;  // bytes between the caches of consecutive layers
    int64_t num_blocks;          // block ids are checked against it (<= 0: not checked)
    const uint8_t* kv_cache;
    int64_t stride_block, stride_pos, stride_head;
    int block_size;
    FastDiv div_block;
    const int32_t* block_table;
    int max_blocks;
    const int32_t* seq_lens;
    const int32_t* kv_start;  // nullable
    int norm_correction;
    int value_lloyd_max;  // 4-bit values are Lloyd-Max codes of the key table, scale slot = norm
    float scale;
    int splits, n_hpass;
    float rsqrt_d;
    Codebook centroids;
    float* mid_o;  // [B, Hq, splits, D + 1]
};

constexpr int kTqTileTokens = 64;

// Row stride (bytes) of a staged tile whose rows hold `bytes` of codes read in lane slices of `nb`
// bytes: one alignment unit of padding when that lowers the bank-conflict degree of the
// token-per-thread stores that fill the tile (degree = gcd(stride in words, 32)).
__host__ __device__ constexpr int tq_gcd(int a, int b) { return b == 0 ? a : tq_gcd(b, a % b); }
__host__ __device__ constexpr int tq_row_stride(int bytes, int nb) {
    const int unit = nb % 16 == 0 ? 16 : (nb % 8 == 0 ? 8 : 4);
    return tq_gcd((bytes + unit) / 4, 32) < tq_gcd(bytes / 4, 32) ? bytes + unit : bytes;
}

template <int D, int KB, int VB, bool K8M = false>
__global__ void __launch_bounds__(kAttnThreads)
tq_split_kernel(const TqDecodeParams p, const TqTable<K8M> t8) {
    static_assert(!K8M || KB == 8, "the 256-entry table belongs to 8-bit keys");
    constexpr int E = AttnCfg<D>::E;
    constexpr int GH = AttnCfg<D>::GH;
    constexpr bool KFP8 = KB == 8 && !K8M;   // D bytes of e4m3, no norm field
    constexpr int MSE = D * KB / 8;
    constexpr int NU = KFP8 ? 0 : 1;  // 16-bit units of the key norm
    constexpr int VDB = tq_value_bytes(D, VB);
    constexpr int NBK = MSE / kOctet, NBV = VDB / kOctet;
    constexpr int SLOT_U16 = (MSE + 2 * NU + VDB + 4) / 2;

    // tile buffers; once the loop is over the K/V areas double as the cross-warp merge area
    constexpr int KROW = tq_row_stride(MSE, NBK), VROW = tq_row_stride(VDB, NBV);
    constexpr int TILE_BYTES = kTqTileTokens * (KROW + VROW);
    constexpr int MERGE_BYTES = 4 * GH * (D + 2) * 4;
    constexpr int BUF_BYTES = ((TILE_BYTES > MERGE_BYTES ? TILE_BYTES : MERGE_BYTES) + 15) / 16 * 16;
    extern __shared__ __align__(16) uint8_t smem_raw[];
    uint8_t* kbuf = smem_raw;                               // [64][KROW]
    uint8_t* vbuf = smem_raw + kTqTileTokens * KROW;        // [64][VROW]
    float* meta = reinterpret_cast<float*>(smem_raw + BUF_BYTES);   // [3][64]: key norm, value scale, zero
    const uint8_t** slots = reinterpret_cast<const uint8_t**>(meta + 3 * kTqTileTokens);  // [64]
    float* qs = reinterpret_cast<float*>(slots + kTqTileTokens);    // [GH][D]
    float* lut = qs + GH * D;                                       // [16], 8-bit key codes: [256]

    const int tid = threadIdx.x;
    const int lane = tid & 31, warp = tid >> 5;
    const int t = lane & 7, o = lane >> 3;
    const int sid = blockIdx.x;
    const int hkv = blockIdx.y / p.n_hpass;
    const int hp = blockIdx.y - hkv * p.n_hpass;
    const int b = blockIdx.z;
    const int group = p.Hq / p.Hkv;
    const int h0 = hp * GH;
    const int nh = min(GH, group - h0);

    const int layer = static_cast<int>(fast_div(static_cast<uint32_t>(b), p.div_bseq));
    const int bs = b - layer * p.B_seq;   // sequence (block table / length row)
    const uint8_t* const kv_layer = p.kv_cache + layer * p.cache_layer_stride;
    const int seq_len = p.seq_lens[bs];
    const int kv_start = p.kv_start ? p.kv_start[bs] : 0;
    const int eff = seq_len - kv_start;
    const int split_len = (eff + p.splits - 1) / p.splits;
    const int t0 = kv_start + split_len * sid;
    const int t1 = min(t0 + split_len, seq_len);
    float* mo = p.mid_o + ((static_cast<int64_t>(b) * p.Hq + hkv * group + h0) * p.splits + sid) * (D + 1);
    const int64_t mo_head_stride = static_cast<int64_t>(p.splits) * (D + 1);
    if (t0 >= t1) {  // neutral partial: zeros and lse = -inf
        for (int idx = tid; idx < nh * (D + 1); idx += kAttnThreads) {
            const int h = idx / (D + 1), d = idx - h * (D + 1);
            mo[h * mo_head_stride + d] = d == D ? -INFINITY : 0.f;
        }
        return;
    }

    // ---- prologue: centroids and the rotated (no signs), pre-scaled queries of this pass
    if constexpr (K8M) {
        for (int i = tid; i < 256; i += kAttnThreads) lut[i] = t8.v[i];
    } else {
        if (tid < kMaxLevels) lut[tid] = p.centroids.v[tid];
    }
    {
        const int hh = warp * 4 + o;
        const bool hv = hh < nh;
        const int64_t qoff = (static_cast<int64_t>(b) * p.Hq + hkv * group + h0 + (hv ? hh : 0)) * D;
        float a[E];
#pragma unroll
        for (int i = 0; i < E / 8; i++) {
            float tmp[8];
            const int64_t eo = qoff + 8 * (t + 8 * i);
            if (p.q_dtype == kF32) load8<float>(static_cast<const float*>(p.q) + eo, tmp);
            else if (p.q_dtype == kBF16)
                load8<__nv_bfloat16>(static_cast<const __nv_bfloat16*>(p.q) + eo, tmp);
            else load8<__half>(static_cast<const __half*>(p.q) + eo, tmp);
#pragma unroll
            for (int c = 0; c < 8; c++) a[8 * i + c] = tmp[c];
        }
        octet_fwht<E>(a, lane);
        if (hh < GH) {
#pragma unroll
            for (int k = 0; k < E; k++)
                qs[hh * D + t + 8 * k] = hv ? a[k] * p.rsqrt_d * p.scale : 0.f;
        }
    }
    __syncthreads();

    // queries and accumulators as pairs of adjacent coordinates: the dot products and the value
    // accumulation run on Blackwell's packed fp32 FMA (two independent IEEE FMAs per instruction)
    constexpr int EP = E / 2;
    u64 qr[GH][EP];
#pragma unroll
    for (int h = 0; h < GH; h++)
#pragma unroll
        for (int i = 0; i < EP; i++)
            qr[h][i] = pk2(qs[h * D + t * E + 2 * i], qs[h * D + t * E + 2 * i + 1]);

    float m_run[GH], l_run[GH];
    u64 acc[GH][EP];
#pragma unroll
    for (int h = 0; h < GH; h++) {
        m_run[h] = -INFINITY;
        l_run[h] = 0.f;
#pragma unroll
        for (int i = 0; i < EP; i++) acc[h][i] = pk2(0.f, 0.f);
    }

    const int32_t* btab = p.block_table + static_cast<int64_t>(bs) * p.max_blocks;
    // address of the slot of position `pos` (this CTA's KV head); a block id outside the cache
    // is never dereferenced (block 0 stands in, the partial's lse becomes NaN)
    bool bad_block = false;
    auto slot_ptr = [&](int pos) {
        const uint32_t pg = fast_div(static_cast<uint32_t>(pos), p.div_block);
        const uint32_t off = static_cast<uint32_t>(pos) - pg * p.block_size;
        int64_t id = btab[pg];
        if (p.num_blocks > 0 && static_cast<uint64_t>(id) >= static_cast<uint64_t>(p.num_blocks)) {
            id = 0;
            bad_block = true;
        }
        return kv_layer + id * p.stride_block + off * p.stride_pos + hkv * p.stride_head;
    };
    // put 16-bit unit j of a slot where the math reads it: key codes / value codes / scalars
    auto place_u16 = [&](int tk, int j, uint32_t v) {
        if (j < MSE / 2) {
            reinterpret_cast<uint16_t*>(kbuf)[tk * (KROW / 2) + j] = static_cast<uint16_t>(v);
        } else if (NU && j == MSE / 2) {
            meta[tk] = __half2float(__ushort_as_half(static_cast<uint16_t>(v)));
        } else if (j < MSE / 2 + NU + VDB / 2) {
            reinterpret_cast<uint16_t*>(vbuf)[tk * (VROW / 2) + j - MSE / 2 - NU] = static_cast<uint16_t>(v);
        } else if (j < SLOT_U16) {
            meta[(j - (MSE / 2 + NU + VDB / 2) + 1) * kTqTileTokens + tk] =
                __half2float(__ushort_as_half(static_cast<uint16_t>(v)));
        }
    };

    // Staging with a register prefetch: two threads per token (warps 0-1 the first half of the
    // slot, warps 2-3 the second) load the slot as ALIGNED 32-bit words -- a slot starts on a
    // 2-byte boundary, so the words are shifted by 16 bits for every other slot and the first /
    // last unit is fetched on its own rather than touching bytes outside the slot.  The loads of
    // tile i+1 are issued before the math of tile i and consumed after it.
    constexpr int USED = MSE + 2 * NU + VDB + 4;     // bytes of a slot that are read
    constexpr int NWORDS = (USED + 2 + 3) / 4;       // aligned words covering them at either alignment
    constexpr int HW = (NWORDS + 1) / 2;             // words per thread
    constexpr bool PREFETCH = HW <= 34;
    uint32_t raw[PREFETCH ? HW + 1 : 1];
    int raw_mis = 0;
    const int ld_tk = tid & (kTqTileTokens - 1), ld_m0 = (tid >> 6) * HW;
    auto prefetch = [&](int ts) {
        if constexpr (PREFETCH) {
            const bool live = ts + ld_tk < t1;
            const uint8_t* sp = live ? slot_ptr(ts + ld_tk) : kv_layer;
            raw_mis = static_cast<int>(reinterpret_cast<uintptr_t>(sp) >> 1) & 1;
            const uint8_t* al = sp - 2 * raw_mis;
#pragma unroll
            for (int i = 0; i <= HW; i++) {
                const int m = ld_m0 + i;
                // the slot occupies bytes [lo, hi) of the aligned range: a word that is only half
                // inside is fetched as that half, one that is outside not at all
                const int lo = 2 * raw_mis, hi = lo + USED, b0 = 4 * m;
                uint32_t v = 0u;
                if (live && b0 < hi) {
                    if (b0 < lo)
                        v = static_cast<uint32_t>(__ldcs(reinterpret_cast<const uint16_t*>(al + b0 + 2))) << 16;
                    else if (b0 + 4 > hi)
                        v = __ldcs(reinterpret_cast<const uint16_t*>(al + b0));
                    else
                        v = __ldcs(reinterpret_cast<const uint32_t*>(al + b0));
                }
                raw[i] = v;
            }
        }
    };
    if constexpr (PREFETCH) prefetch(t0);

    for (int ts = t0; ts < t1; ts += kTqTileTokens) {
        const int ntile = min(kTqTileTokens, t1 - ts);
        if constexpr (PREFETCH) {
#pragma unroll
            for (int i = 0; i < HW; i++) {
                const int m = ld_m0 + i;  // word m of the slot = 16-bit units 2m, 2m + 1
                const uint32_t w = raw_mis ? __funnelshift_r(raw[i], raw[i + 1], 16) : raw[i];
                if (m < MSE / 4) {
                    reinterpret_cast<uint32_t*>(kbuf)[ld_tk * (KROW / 4) + m] = w;
                } else if (m < NWORDS) {
                    place_u16(ld_tk, 2 * m, w & 0xffffu);
                    place_u16(ld_tk, 2 * m + 1, w >> 16);
                }
            }
            __syncthreads();
            if (ts + kTqTileTokens < t1) prefetch(ts + kTqTileTokens);
        } else {
            // wide slots: plain staging, 8 loads per thread in flight
            if (tid < ntile) slots[tid] = slot_ptr(ts + tid);
            __syncthreads();
            for (int base = tid; base < ntile * SLOT_U16; base += kAttnThreads * 8) {
                uint16_t v[8];
#pragma unroll
                for (int u = 0; u < 8; u++) {
                    const int idx = base + u * kAttnThreads;
                    const int tk = idx / SLOT_U16, j = idx - tk * SLOT_U16;
                    v[u] = idx < ntile * SLOT_U16
                               ? __ldcs(reinterpret_cast<const uint16_t*>(slots[tk]) + j) : uint16_t(0);
                }
#pragma unroll
                for (int u = 0; u < 8; u++) {
                    const int idx = base + u * kAttnThreads;
                    if (idx >= ntile * SLOT_U16) break;
                    const int tk = idx / SLOT_U16;
                    place_u16(tk, idx - tk * SLOT_U16, v[u]);
                }
            }
            __syncthreads();
        }

        const int tw = warp * 16;  // this warp's 16 tokens of the tile
        if (tw < ntile) {          // warp-uniform
            float sc[4][GH];
#pragma unroll
            for (int step = 0; step < 4; step++) {
                const int tk = tw + step * 4 + o;
                uint32_t w[(NBK + 3) / 4];
                load_code_bytes<NBK>(kbuf + tk * KROW + t * NBK, w);
                u64 kv[EP];
                u64 cn2 = pk2(0.f, 0.f);
#pragma unroll
                for (int i = 0; i < EP; i++) {
                    if constexpr (KFP8) {
                        const __half2_raw h2 = __nv_cvt_fp8x2_to_halfraw2(
                            static_cast<__nv_fp8x2_storage_t>((w[i >> 1] >> (16 * (i & 1))) & 0xffffu),
                            __NV_E4M3);
                        const float2 f2 = __half22float2(__half2(h2));
                        kv[i] = pk2(f2.x, f2.y);
                    } else {
                        kv[i] = pk2(lut[extract_code<KB>(w, 2 * i)], lut[extract_code<KB>(w, 2 * i + 1)]);
                        cn2 = fma2(kv[i], kv[i], cn2);
                    }
                }
                float kn = KFP8 ? 1.f : meta[tk];
                if (!KFP8 && p.norm_correction) {  // re-normalise the centroid vector to unit length
                    float c0, c1;
                    upk2(cn2, c0, c1);
                    float cn = c0 + c1;
                    cn += __shfl_xor_sync(0xffffffffu, cn, 1);
                    cn += __shfl_xor_sync(0xffffffffu, cn, 2);
                    cn += __shfl_xor_sync(0xffffffffu, cn, 4);
                    kn *= 1.0f / sqrtf(cn + 1e-16f);
                }
#pragma unroll
                for (int h = 0; h < GH; h++) {
                    u64 d2 = pk2(0.f, 0.f);
#pragma unroll
                    for (int i = 0; i < EP; i++) d2 = fma2(qr[h][i], kv[i], d2);
                    float d0, d1;
                    upk2(d2, d0, d1);
                    float d = d0 + d1;
                    d += __shfl_xor_sync(0xffffffffu, d, 1);
                    d += __shfl_xor_sync(0xffffffffu, d, 2);
                    d += __shfl_xor_sync(0xffffffffu, d, 4);
                    sc[step][h] = tk < ntile ? d * kn : -INFINITY;
                }
            }
            float wp[4][GH];
#pragma unroll
            for (int h = 0; h < GH; h++) {
                float mx = fmaxf(fmaxf(sc[0][h], sc[1][h]), fmaxf(sc[2][h], sc[3][h]));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
                const float m_new = fmaxf(m_run[h], mx);  // finite: the warp's first token is valid
                const float corr = m_run[h] == -INFINITY ? 0.f : __expf(m_run[h] - m_new);
                m_run[h] = m_new;
                float ls = 0.f;
#pragma unroll
                for (int step = 0; step < 4; step++) {
                    const float pe = sc[step][h] == -INFINITY ? 0.f : __expf(sc[step][h] - m_new);
                    ls += pe;
                    wp[step][h] = pe;
                }
                l_run[h] = l_run[h] * corr + ls;
                const u64 corr2 = pk2(corr, corr);
#pragma unroll
                for (int i = 0; i < EP; i++) acc[h][i] = mul2(acc[h][i], corr2);
            }
#pragma unroll
            for (int step = 0; step < 4; step++) {
                const int tk = tw + step * 4 + o;
                const bool ok = tk < ntile;
                uint32_t w[(NBV + 3) / 4];
                load_code_bytes<NBV>(vbuf + tk * VROW + t * NBV, w);
                // (slots past the end of the tile hold stale bytes: keep them out of the arithmetic)
                const float vs = ok ? meta[kTqTileTokens + tk] : 0.f;
                const float vz = ok ? meta[2 * kTqTileTokens + tk] : 0.f;
                u64 vv[EP];
                bool lm = false;
                if constexpr (VB == 4) lm = p.value_lloyd_max != 0;
                if (lm) {
                    // values[d] = centroid[code] * norm, the centroid vector re-normalised to unit
                    // length under norm correction (triton_decode_offset.py:399-423)
                    u64 cn2 = pk2(0.f, 0.f);
#pragma unroll
                    for (int i = 0; i < EP; i++) {
                        vv[i] = pk2(lut[extract_code<VB>(w, 2 * i)], lut[extract_code<VB>(w, 2 * i + 1)]);
                        cn2 = fma2(vv[i], vv[i], cn2);
                    }
                    float vn = vs;
                    if (p.norm_correction) {
                        float c0, c1;
                        upk2(cn2, c0, c1);
                        float cn = c0 + c1;
                        cn += __shfl_xor_sync(0xffffffffu, cn, 1);
                        cn += __shfl_xor_sync(0xffffffffu, cn, 2);
                        cn += __shfl_xor_sync(0xffffffffu, cn, 4);
                        vn *= 1.0f / sqrtf(cn + 1e-16f);
                    }
                    const u64 vn2 = pk2(vn, vn);
#pragma unroll
                    for (int i = 0; i < EP; i++) vv[i] = mul2(vv[i], vn2);
                } else {
                    const u64 vs2 = pk2(vs, vs), vz2 = pk2(vz, vz);
#pragma unroll
                    for (int i = 0; i < EP; i++)
                        vv[i] = fma2(pk2(static_cast<float>(extract_code<VB>(w, 2 * i)),
                                         static_cast<float>(extract_code<VB>(w, 2 * i + 1))), vs2, vz2);
                }
#pragma unroll
                for (int h = 0; h < GH; h++) {
                    const float wgt = ok ? wp[step][h] : 0.f;
                    const u64 wgt2 = pk2(wgt, wgt);
#pragma unroll
                    for (int i = 0; i < EP; i++) acc[h][i] = fma2(wgt2, vv[i], acc[h][i]);
                }
            }
        }
        __syncthreads();
    }

    // ---- combine the 4 octets of each warp, then the 4 warps through shared memory
#pragma unroll
    for (int h = 0; h < GH; h++) {
        // octets of a warp share m_run (the max was reduced over the warp), so sums just add
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 8);
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 16);
#pragma unroll
        for (int i = 0; i < EP; i++) {
            acc[h][i] = add2(acc[h][i], __shfl_xor_sync(0xffffffffu, acc[h][i], 8));
            acc[h][i] = add2(acc[h][i], __shfl_xor_sync(0xffffffffu, acc[h][i], 16));
        }
    }
    float* wacc = reinterpret_cast<float*>(smem_raw);  // [4][GH][D]
    float* wm = wacc + 4 * GH * D;                     // [4][GH]
    float* wl = wm + 4 * GH;                           // [4][GH]
    if (o == 0) {
#pragma unroll
        for (int h = 0; h < GH; h++) {
#pragma unroll
            for (int i = 0; i < EP; i++)
                *reinterpret_cast<u64*>(wacc + (warp * GH + h) * D + t * E + 2 * i) = acc[h][i];
            if (t == 0) {
                wm[warp * GH + h] = m_run[h];
                wl[warp * GH + h] = l_run[h];
            }
        }
    }
    const bool any_bad = __syncthreads_or(bad_block) != 0;
    for (int idx = tid; idx < nh * D; idx += kAttnThreads) {
        const int h = idx / D, d = idx - h * D;
        float M = -INFINITY;
#pragma unroll
        for (int w2 = 0; w2 < 4; w2++) M = fmaxf(M, wm[w2 * GH + h]);
        float a = 0.f, l = 0.f;
#pragma unroll
        for (int w2 = 0; w2 < 4; w2++) {
            const float mw = wm[w2 * GH + h];
            if (mw != -INFINITY) {
                const float f = __expf(mw - M);
                a = fmaf(wacc[(w2 * GH + h) * D + d], f, a);
                l = fmaf(wl[w2 * GH + h], f, l);
            }
        }
        const float safe_l = l > 0.f ? l : 1.f;
        mo[h * mo_head_stride + d] = a / safe_l;
        if (d == 0)
            mo[h * mo_head_stride + D] = any_bad ? __int_as_float(0x7fc00000) : M + logf(safe_l);
    }
}

template <int D>
constexpr int tq_split_smem_bytes(int kb, int vb, bool k8m = false) {
    const int mse = D * kb / 8, vdb = tq_value_bytes(D, vb);
    const int tile = kTqTileTokens * (tq_row_stride(mse, mse / kOctet) + tq_row_stride(vdb, vdb / kOctet));
    const int merge = 4 * AttnCfg<D>::GH * (D + 2) * 4;
    const int buf = ((tile > merge ? tile : merge) + 15) / 16 * 16;
    return buf + 3 * kTqTileTokens * 4 + kTqTileTokens * 8 + AttnCfg<D>::GH * D * 4 +
           (k8m ? 256 : kMaxLevels) * 4;
}

struct TqMergeParams {
    const float* mid_o;  // [n_rows, splits, D + 1]
    void* out;           // [n_rows, D]
    float* lse;          // [n_rows], nullable
    int64_t n_rows;
    int splits;
    int rotate;
    float rsqrt_d;
    // Attention over an uncompressed prefix of the same rows, computed elsewhere (nullable):
    // merged in by log-sum-exp as vllm_plugin/v1_backend.py:1267-1277 does.
    const void* prefix_out;   // [n_rows, D] of prefix_dtype, original space
    int prefix_dtype;
    const float* prefix_lse;  // [n_rows]
};

// Merge the split partials of 4 (sequence, query head) rows per warp: softmax-weighted by lse,
// optionally Hadamard-transform the result, optionally merge a prefix result in, cast and store.
// mid_o rows with lse = -inf are skipped.
template <int D, typename OT>
__global__ void __launch_bounds__(128)
tq_merge_kernel(const TqMergeParams p) {
    const float* __restrict__ mid_o = p.mid_o;
    OT* __restrict__ out = static_cast<OT*>(p.out);
    float* __restrict__ lse_out = p.lse;
    const int64_t n_rows = p.n_rows;
    const int splits = p.splits, rotate = p.rotate;
    const float rsqrt_d = p.rsqrt_d;
    constexpr int E = D / kOctet;
    const int lane = threadIdx.x & 31;
    const int t = lane & 7;
    const int64_t row = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) / 8;
    const bool valid = row < n_rows;
    const float* base = mid_o + (valid ? row : 0) * static_cast<int64_t>(splits) * (D + 1);
    float M = -INFINITY;
    for (int s = 0; s < splits; s++) M = fmaxf(M, base[static_cast<int64_t>(s) * (D + 1) + D]);
    float a[E];
#pragma unroll
    for (int r = 0; r < E; r++) a[r] = 0.f;
    float l = 0.f;
    for (int s = 0; s < splits; s++) {
        const float* ps = base + static_cast<int64_t>(s) * (D + 1);
        const float ls = ps[D];
        if (ls == -INFINITY) continue;
        const float f = __expf(ls - M);
        l += f;
#pragma unroll
        for (int r = 0; r < E; r++) a[r] = fmaf(ps[load_coord(t, r)], f, a[r]);
    }
    const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
    for (int r = 0; r < E; r++) a[r] *= inv;
    if (rotate) {
        octet_fwht<E>(a, lane);
#pragma unroll
        for (int k = 0; k < E; k++) a[k] *= rsqrt_d;
    }
    if (!valid) return;
    float lse = l > 0.f ? M + logf(l) : -INFINITY;
    float w_own = 1.f, w_pre = 0.f;
    const bool prefix = p.prefix_out != nullptr;
    if (prefix) {
        const float lp = p.prefix_lse[row];
        const float lmax = fmaxf(lp, lse);
        if (lmax == -INFINITY) {  // nothing attended on either side
            w_own = 0.f;
        } else {
            const float ep = __expf(lp - lmax), eq = __expf(lse - lmax);
            const float total = fmaxf(ep + eq, 1e-20f);
            w_pre = ep / total;
            w_own = eq / total;
            lse = lmax + logf(ep + eq);
        }
    }
    OT* orow = out + row * D;
#pragma unroll
    for (int r = 0; r < E; r++) {
        const int coord = rotate ? t + 8 * r : load_coord(t, r);
        float v = a[r];
        if (prefix) {
            const int64_t at = row * D + coord;
            const float pv = p.prefix_dtype == kF32 ? static_cast<const float*>(p.prefix_out)[at]
                             : p.prefix_dtype == kF16
                                 ? __half2float(static_cast<const __half*>(p.prefix_out)[at])
                                 : __bfloat162float(static_cast<const __nv_bfloat16*>(p.prefix_out)[at]);
            v = pv * w_pre + v * w_own;
        }
        if constexpr (sizeof(OT) == 4) orow[coord] = v;
        else if constexpr (std::is_same<OT, __half>::value) orow[coord] = __float2half_rn(v);
        else orow[coord] = __float2bfloat16_rn(v);
    }
    if (lse_out && t == 0) lse_out[row] = lse;
}

}  // namespace ftq
