// Fused KV encode for sm_100a: sign flip -> Hadamard butterfly -> L2 norm ->
// normalise -> Lloyd-Max bucketise -> bit-pack -> store (contiguous, paged pool
// or the reference's v0 slot layout), one pass over the input, no scratch memory.
//
// The arithmetic restates TurboQuantMSE._encode_unfused of the reference
// (src/fused_turboquant/core/quantizer.py:137-160) operation for operation, so
// that the packed codes and the fp16 norms come out bit-identical:
//   y      = fwht(x * signs) * fp32(D^-1/2)            core/hadamard.py:38-48,90
//   norm   = sqrt(sum_l (sum_k y[l+8k]^2))             the order torch.norm uses on CPU:
//                                                      8 strided running sums, then left to right
//   n      = y / (norm + 1e-8)                         IEEE division
//   code   = clamp(#{boundaries < n} - 1, 0, 2^b-1)    core/lloyd_max.py:131-132
//   packed = pack_{nibbles,3bit,2bit}(code)            core/packing.py:14-103
//   norm16 = fp16(norm), round to nearest even
// No fused multiply-add may touch y or the sum of squares: every add, multiply,
// divide and square root below is an explicitly rounded intrinsic.
#pragma once

#include "ftq_common.cuh"

namespace ftq {

struct EncodeTables {
    SignBits signs;
    float bounds[kMaxLevels - 1];  // interior boundaries b[1] .. b[2^bits - 1]
    float rsqrt_d;                 // fp32(D ** -0.5)
};

// Where the vectors come from: vector v = (outer, inner) with inner < n_inner.
struct EncodeSource {
    const void* base;
    int n_inner;           // vectors per outer index (Hkv for [tokens, Hkv, D]; 1 for flat rows)
    int64_t outer_stride;  // elements
    int64_t inner_stride;  // elements
    int64_t layer_stride;  // elements, blockIdx.y advances by this
    FastDiv div_inner;     // division by n_inner (filled in by the dispatcher)
};

enum : int { kSinkFlat = 0, kSinkPaged = 1, kSinkV0 = 2 };

// Where the codes and the norm of vector v go.
struct EncodeSink {
    int mode;
    // flat: codes at codes + v * pd, norm (fp16) at norms + v
    uint8_t* codes;
    uint16_t* norms;
    // paged pool / v0 layout: token = v / Hkv, head = v % Hkv, slot = slot_mapping[token]
    const int64_t* slot_mapping;
    int64_t slot_limit;     // slots at or beyond it (a stale or corrupt mapping) are skipped
    int Hkv;
    FastDiv div_hkv;        // division by Hkv (filled in by the dispatcher)
    int64_t page_bytes;     // paged: bytes per (block, head) page
    int codes_off;          // paged: offset of this tensor's codes inside the page
    int norms_off;          // paged: offset of this tensor's fp16 norms inside the page
    int swap_halves;        // paged: store the row's two halves exchanged for tokens with bit 1 set
    int block_size;         // v0: tokens per block
    int elem_size;          // v0: bytes per (token, head) slot
    int64_t plane_off;      // v0: byte offset of the K or V plane
    int64_t layer_stride;   // bytes, blockIdx.y advances by this
};

// Transposition of an 8-lane x (items per word) matrix of BITS-wide items: afterwards lane j
// holds the items that had in-word position j, ordered by source lane.  Three exchange rounds
// (partner lane ^ 1, ^ 2, ^ 4).  In a round with item distance s the sender rotates its word
// by s (left if it is the upper lane of the pair, right otherwise), so that the items the
// partner wants already sit where the partner puts them: the receiver merges with one
// bit-select.  Rounds whose distance is a whole number of bytes are a single byte-permute of
// (own word, partner's word) instead.  For 3-bit items bits 24..31 carry junk between the
// rounds (never selected into the low 24 bits) and are cleared at the end.
template <int BITS>
struct TransposeConsts {
    uint32_t a[3];  // rotate-left amount of the sender, or the byte-permute selector
    uint32_t b[3];  // bits the receiver keeps of its own word (unused for byte-permute rounds)
};

template <int BITS>
__device__ __forceinline__ TransposeConsts<BITS> transpose_consts(int lane) {
    constexpr uint32_t m[3] = {BITS == 4 ? 0x0F0F0F0Fu : BITS == 3 ? 0x001C71C7u : 0x33333333u,
                               BITS == 4 ? 0x00FF00FFu : BITS == 3 ? 0x0003F03Fu : 0x0F0F0F0Fu,
                               BITS == 4 ? 0x0000FFFFu : BITS == 3 ? 0x00000FFFu : 0x00FF00FFu};
    TransposeConsts<BITS> c;
#pragma unroll
    for (int j = 0; j < 3; j++) {
        const int s = BITS << j;
        const bool upper = (lane >> j) & 1;
        if (s == 8) {
            c.a[j] = upper ? 0x3715u : 0x6240u;
            c.b[j] = 0u;
        } else if (s == 16) {
            c.a[j] = upper ? 0x3276u : 0x5410u;
            c.b[j] = 0u;
        } else {
            c.a[j] = upper ? s : 32 - s;
            c.b[j] = upper ? (m[j] << s) : m[j];
        }
    }
    return c;
}

template <int BITS>
__device__ __forceinline__ uint32_t octet_transpose_items(uint32_t w, const TransposeConsts<BITS>& c) {
#pragma unroll
    for (int j = 0; j < 3; j++) {
        const int s = BITS << j;
        if (s == 8 || s == 16) {
            const uint32_t p = __shfl_xor_sync(0xffffffffu, w, 1 << j);
            w = __byte_perm(w, p, c.a[j]);
        } else {
            const uint32_t p = __shfl_xor_sync(0xffffffffu, __funnelshift_l(w, w, c.a[j]), 1 << j);
            w = (w & c.b[j]) | (p & ~c.b[j]);
        }
    }
    if constexpr (BITS == 3) w &= 0x00FFFFFFu;
    return w;
}

// Slot of the token that vector v belongs to (paged pool / v0 layout); loaded ahead of the
// arithmetic so that the store at the end does not wait for it.
__device__ __forceinline__ int64_t load_slot(const EncodeSink& sink, int64_t v, bool valid) {
    if (sink.mode == kSinkFlat || !valid) return -1;
    // (the value is not looked at before emit_vector: a compare here would make the warp wait for
    // the load before the arithmetic instead of after it)
    return sink.slot_mapping[fast_div(static_cast<uint32_t>(v), sink.div_hkv)];
}

// Store one encoded vector: `w` holds this lane's codes (coordinates l + 8k) packed as
// octet_transpose_items expects; the octet transposes them so that every lane owns whole
// output words, then writes codes and norm to the sink.  `slot` is load_slot(sink, v, valid).
// Must be called by all 32 lanes.
template <int D, int BITS, int NW>
__device__ __forceinline__ void emit_vector(const uint32_t (&w)[NW], float norm, bool valid,
                                            int64_t v, int64_t slot, const EncodeSink& sink,
                                            int64_t sink_layer, int lane,
                                            const TransposeConsts<BITS>& tc) {
    constexpr int PD = packed_dim(D, BITS);
    const int t = lane & 7;
    // destination of this vector
    uint8_t* dst = nullptr;
    bool store = valid;
    int rot = 0;  // word rotation inside the row (half swap of the paged V rows)
    if (sink.mode == kSinkFlat) {
        dst = sink.codes + v * PD;
    } else if (valid) {
        const uint32_t token = fast_div(static_cast<uint32_t>(v), sink.div_hkv);
        const int head = static_cast<int>(static_cast<uint32_t>(v) - token * sink.Hkv);
        // negative = padding (the reference's `slot < 0` skip, triton_inkernel_store.py:398-399);
        // a slot at or beyond the cache's end is dropped the same way instead of being written
        // out of bounds (one unsigned compare covers both)
        if (static_cast<uint64_t>(slot) >= static_cast<uint64_t>(sink.slot_limit)) {
            store = false;
        } else if (sink.mode == kSinkPaged) {
            // slot >= 0 here; pages per layer and bytes per page both fit 32 bits
            const uint32_t blk = static_cast<uint32_t>(static_cast<uint64_t>(slot) / kPageTokens);
            const int off = static_cast<int>(static_cast<uint64_t>(slot) % kPageTokens);
            uint8_t* page = sink.codes + sink_layer +
                            static_cast<uint64_t>(blk * sink.Hkv + head) *
                                static_cast<uint32_t>(sink.page_bytes);
            dst = page + sink.codes_off + off * PD;
            if (sink.swap_halves && (off & 2)) rot = PD / 8;
            if (t == 0)
                *reinterpret_cast<__half*>(page + sink.norms_off + 2 * off) =
                    __float2half_rn(norm);
        } else {
            const int64_t blk = slot / sink.block_size;
            const int64_t off = slot - blk * sink.block_size;
            dst = sink.codes + sink.plane_off +
                  ((blk * sink.block_size + off) * sink.Hkv + head) * sink.elem_size;
            if (t == 0) *reinterpret_cast<float*>(dst + PD) = __half2float(__float2half_rn(norm));
        }
    }
    if (sink.mode == kSinkFlat && valid && t == 0)
        reinterpret_cast<__half*>(sink.norms)[v] = __float2half_rn(norm);

    // transpose across the octet so that every lane owns whole output words
#pragma unroll
    for (int i = 0; i < NW; i++) {
        const uint32_t o = octet_transpose_items<BITS>(w[i], tc);
        if constexpr (BITS == 3) {
            // lane j holds the 24-bit group j of row i; regroup 8 x 3 bytes into 6 words
            const int g0 = (4 * t) / 3;
            const uint32_t lo = __shfl_sync(0xffffffffu, o, g0, 8);
            const uint32_t hi = __shfl_sync(0xffffffffu, o, g0 + 1, 8);
            const uint64_t cat = (static_cast<uint64_t>(hi) << 24) | lo;
            const uint32_t word = static_cast<uint32_t>(cat >> (8 * ((4 * t) % 3)));
            if (store && t < 6) {
                int widx = 6 * i + t;
                widx = widx + rot < PD / 4 ? widx + rot : widx + rot - PD / 4;
                reinterpret_cast<uint32_t*>(dst)[widx] = word;
            }
        } else {
            int widx = t + 8 * i;
            if (store && widx < PD / 4) {
                widx = widx + rot < PD / 4 ? widx + rot : widx + rot - PD / 4;
                reinterpret_cast<uint32_t*>(dst)[widx] = o;
            }
        }
    }
}

template <int D, int BITS, typename T>
__global__ void __launch_bounds__(256)
encode_kernel(EncodeSource src, EncodeSink sink, EncodeTables tab, int64_t n_vec) {
    constexpr int E = D / kOctet;          // values per lane
    constexpr int NCH = E / 8;             // 8-coordinate runs per lane
    constexpr int PD = packed_dim(D, BITS);
    constexpr int NLEV = 1 << BITS;
    // words of packed items per lane before the transpose
    constexpr int NW = BITS == 2 ? (E + 15) / 16 : E / 8;

    const int lane = threadIdx.x & 31;
    const int t = lane & 7;
    const int sub = lane >> 3;  // which of the warp's 4 vectors
    const int64_t warp = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int64_t n_warps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;

    const T* xbase = static_cast<const T*>(src.base) + blockIdx.y * src.layer_stride;
    const int64_t sink_layer = blockIdx.y * sink.layer_stride;

    // Per-lane sign masks in the load layout (same for every vector).
    uint32_t sgn[E];
#pragma unroll
    for (int r = 0; r < E; r++) sgn[r] = sign_mask(tab.signs, load_coord(t, r));
    const TransposeConsts<BITS> tc = transpose_consts<BITS>(lane);

    for (int64_t base = warp * 4; base < n_vec; base += n_warps * 4) {
        const int64_t v = base + sub;
        const bool valid = v < n_vec;
        const int64_t slot = load_slot(sink, v, valid);
        const int64_t outer = valid ? fast_div(static_cast<uint32_t>(v), src.div_inner) : 0;
        const int inner = valid ? static_cast<int>(v - outer * src.n_inner) : 0;
        const T* row = xbase + outer * src.outer_stride + inner * src.inner_stride;

        float y[E];
#pragma unroll
        for (int i = 0; i < NCH; i++) {
            float tmp[8];
            if (valid) {
                load8<T>(row + 8 * (t + 8 * i), tmp);
            } else {
#pragma unroll
                for (int c = 0; c < 8; c++) tmp[c] = 0.f;
            }
#pragma unroll
            for (int c = 0; c < 8; c++)
                y[8 * i + c] = __uint_as_float(__float_as_uint(tmp[c]) ^ sgn[8 * i + c]);
        }

        octet_fwht<E>(y, lane);

        // scale, then the 8-way strided sum of squares (lane l = running sum l)
        float acc = 0.f;
#pragma unroll
        for (int k = 0; k < E; k++) {
            y[k] = __fmul_rn(y[k], tab.rsqrt_d);
            acc = __fadd_rn(acc, __fmul_rn(y[k], y[k]));
        }
        float s = __shfl_sync(0xffffffffu, acc, 0, 8);
#pragma unroll
        for (int l = 1; l < 8; l++) s = __fadd_rn(s, __shfl_sync(0xffffffffu, acc, l, 8));
        const float norm = __fsqrt_rn(s);
        const float denom = __fadd_rn(norm, 1e-8f);

        // bucketise and pack this lane's codes (coordinates l + 8k)
        uint32_t w[NW];
#pragma unroll
        for (int i = 0; i < NW; i++) w[i] = 0u;
#pragma unroll
        for (int k = 0; k < E; k++) {
            const float nv = __fdiv_rn(y[k], denom);
            uint32_t code = 0;
#pragma unroll
            for (int j = 0; j < NLEV - 1; j++) code += (tab.bounds[j] < nv) ? 1u : 0u;
            if constexpr (BITS == 2) {
                const int pos = ((k >> 1) & 7) | ((k & 1) << 3);
                w[k >> 4] |= code << (2 * pos);
            } else {
                w[k >> 3] |= code << (BITS * (k & 7));
            }
        }

        emit_vector<D, BITS>(w, norm, valid, v, slot, sink, sink_layer, lane, tc);
    }
}

}  // namespace ftq
