/*
 * ftq_oracle.c -- CPU restatement of the fused-turboquant hot path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the CUDA library is
 * compared against; nothing in the shipped package may call it.  It is also
 * the CPU arm of the benchmark (timed with OpenMP over the host cores).
 *
 * Every function restates, in plain scalar C, one step of the reference's
 * unfused PyTorch path (paths are relative to the reference project root):
 *
 *   fwht / randomized_hadamard        src/fused_turboquant/core/hadamard.py:23-100
 *   LloydMaxQuantizer.quantize        src/fused_turboquant/core/lloyd_max.py:121-137
 *   pack_nibbles / pack_3bit / pack_2bit (+unpack)
 *                                     src/fused_turboquant/core/packing.py:14-128
 *   TurboQuantMSE._encode_unfused     src/fused_turboquant/core/quantizer.py:137-160
 *   TurboQuantMSE._decode_unfused     src/fused_turboquant/core/quantizer.py:191-205
 *   decode attention (composed)       scores = q . decode(K)^T * scale, fp32 softmax,
 *                                     out = w . decode(V), as hf/fused_cache.py:576-624 and
 *                                     kernels/triton_v_attention.py:247-285 compose it
 *   paged write / gather (v0 layout)  src/fused_turboquant/vllm_plugin/cache_ops.py:85-205
 *
 * Parity status: PINNED.  The encode/decode/pack functions are checked
 * bit-for-bit against outputs of the reference itself (the .npz files
 * under tests/golden/, produced by tests/golden/make_golden.py which imports
 * the reference), and against outputs of the reference's own Triton kernels
 * executed in interpreter mode (tests/golden/make_golden_kernels.py ->
 * kernels_interp.npz): fused encode, fused dense decode, RHT, QK scores, flash
 * decode.
 *
 * Build with:  gcc -O2 -ffp-contract=off -fno-fast-math -fopenmp -shared -fPIC
 * (-ffp-contract=off matters: a fused multiply-add changes rounding and the
 * codes / fp16 norms would no longer be bit-exact).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define FTQ_MAX_D 8192

/* ---------------------------------------------------------------- helpers */

int ftq_oracle_packed_dim(int d, int bits) {
    /* core/packing.py: 4-bit d/2, 3-bit 3d/8, 2-bit d/4 */
    if (bits == 4) return d / 2;
    if (bits == 3) return d * 3 / 8;
    if (bits == 2) return d / 4;
    return -1;
}

/* fp32 -> fp16 bits, round to nearest even (what Tensor.half() does). */
uint16_t ftq_oracle_f32_to_f16(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t absx = x & 0x7fffffffu;
    if (absx >= 0x7f800000u) { /* inf / nan */
        return (uint16_t)(sign | 0x7c00u | ((absx > 0x7f800000u) ? 0x200u : 0u));
    }
    if (absx >= 0x477ff000u) { /* >= 65520 rounds to inf */
        return (uint16_t)(sign | 0x7c00u);
    }
    if (absx < 0x33000001u) { /* < 2^-25 (+1ulp): rounds to zero */
        return (uint16_t)sign;
    }
    int32_t exp = (int32_t)(absx >> 23) - 127;
    uint32_t man = (absx & 0x7fffffu) | 0x800000u;
    uint32_t half;
    if (exp < -14) { /* subnormal half */
        int shift = -14 - exp + 13; /* bits dropped from the 24-bit significand */
        uint32_t q = man >> shift;
        uint32_t rem = man & ((1u << shift) - 1u);
        uint32_t halfway = 1u << (shift - 1);
        if (rem > halfway || (rem == halfway && (q & 1u))) q++;
        half = q;
    } else {
        uint32_t q = ((uint32_t)(exp + 15) << 10) | ((man >> 13) & 0x3ffu);
        uint32_t rem = man & 0x1fffu;
        if (rem > 0x1000u || (rem == 0x1000u && (q & 1u))) q++;
        half = q; /* a carry out of the mantissa bumps the exponent, as it should */
    }
    return (uint16_t)(sign | half);
}

float ftq_oracle_f16_to_f32(uint16_t h) {
    uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1fu;
    uint32_t man = h & 0x3ffu;
    uint32_t x;
    if (exp == 0) {
        if (man == 0) {
            x = sign;
        } else {
            int e = -1;
            do { man <<= 1; e++; } while (!(man & 0x400u));
            x = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3ffu) << 13);
        }
    } else if (exp == 31) {
        x = sign | 0x7f800000u | (man << 13);
    } else {
        x = sign | ((exp + 112u) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &x, 4);
    return f;
}

/* ------------------------------------------------------------------ FWHT */

/* core/hadamard.py:38-48 -- stages h = 1, 2, 4, ...; in each block of 2h the
 * low half becomes a+b and the high half a-b; then one multiply by d^-1/2. */
void ftq_oracle_fwht(float *x, int d) {
    for (int h = 1; h < d; h <<= 1) {
        for (int base = 0; base < d; base += 2 * h) {
            for (int j = 0; j < h; j++) {
                float a = x[base + j];
                float b = x[base + h + j];
                x[base + j] = a + b;
                x[base + h + j] = a - b;
            }
        }
    }
    float s = (float)pow((double)d, -0.5);
    for (int i = 0; i < d; i++) x[i] = x[i] * s;
}

/* core/hadamard.py:70-100.  forward: fwht(x*signs); inverse: fwht(y)*signs.
 * signs may be NULL (all +1). */
void ftq_oracle_rht(const float *x, const float *signs, float *y, int64_t n, int d,
                    int inverse) {
#pragma omp parallel for schedule(static)
    for (int64_t v = 0; v < n; v++) {
        float buf[FTQ_MAX_D];
        const float *xi = x + v * d;
        float *yo = y + v * d;
        if (!inverse) {
            for (int i = 0; i < d; i++) buf[i] = signs ? xi[i] * signs[i] : xi[i];
            ftq_oracle_fwht(buf, d);
            for (int i = 0; i < d; i++) yo[i] = buf[i];
        } else {
            for (int i = 0; i < d; i++) buf[i] = xi[i];
            ftq_oracle_fwht(buf, d);
            for (int i = 0; i < d; i++) yo[i] = signs ? buf[i] * signs[i] : buf[i];
        }
    }
}

/* ------------------------------------------------------------- pack/unpack */

/* core/packing.py:14-31, 50-64, 85-103 */
void ftq_oracle_pack(const uint8_t *idx, uint8_t *out, int d, int bits) {
    if (bits == 4) {
        for (int i = 0; i < d / 2; i++)
            out[i] = (uint8_t)((idx[2 * i + 1] << 4) | idx[2 * i]);
    } else if (bits == 2) {
        for (int i = 0; i < d / 4; i++)
            out[i] = (uint8_t)(idx[4 * i] | (idx[4 * i + 1] << 2) | (idx[4 * i + 2] << 4) |
                               (idx[4 * i + 3] << 6));
    } else { /* 3-bit: 8 codes -> 24-bit little-endian stream */
        for (int g = 0; g < d / 8; g++) {
            uint32_t w = 0;
            for (int j = 0; j < 8; j++) w |= (uint32_t)(idx[8 * g + j] & 7u) << (3 * j);
            out[3 * g] = (uint8_t)(w & 0xff);
            out[3 * g + 1] = (uint8_t)((w >> 8) & 0xff);
            out[3 * g + 2] = (uint8_t)((w >> 16) & 0xff);
        }
    }
}

/* core/packing.py:34-47, 67-82, 106-128 */
void ftq_oracle_unpack(const uint8_t *in, uint8_t *idx, int d, int bits) {
    if (bits == 4) {
        for (int i = 0; i < d / 2; i++) {
            idx[2 * i] = in[i] & 0x0f;
            idx[2 * i + 1] = (in[i] >> 4) & 0x0f;
        }
    } else if (bits == 2) {
        for (int i = 0; i < d / 4; i++)
            for (int j = 0; j < 4; j++) idx[4 * i + j] = (in[i] >> (2 * j)) & 3;
    } else {
        for (int g = 0; g < d / 8; g++) {
            uint32_t w = (uint32_t)in[3 * g] | ((uint32_t)in[3 * g + 1] << 8) |
                         ((uint32_t)in[3 * g + 2] << 16);
            for (int j = 0; j < 8; j++) idx[8 * g + j] = (w >> (3 * j)) & 7u;
        }
    }
}

/* ----------------------------------------------------------------- encode */

/* torch.norm(rot, dim=-1) on the CPU builds of torch this was pinned against
 * reduces a contiguous fp32 row with `lanes` running sums (lane l adds
 * sq[l], sq[l+lanes], ... in order, each square rounded on its own), then adds
 * the lanes left to right and takes one sqrt.  lanes = 8 reproduces it
 * exactly (0 mismatches over 600k rows at d = 64/128/256). */
static float norm_like_torch(const float *y, int d, int lanes) {
    float acc[16] = {0.0f};
    if (lanes < 1 || lanes > 16) lanes = 8;
    int body = d - (d % lanes);
    for (int k = 0; k < body; k += lanes)
        for (int l = 0; l < lanes; l++) {
            float sq = y[k + l] * y[k + l];
            acc[l] = acc[l] + sq;
        }
    float s = acc[0];
    for (int l = 1; l < lanes; l++) s = s + acc[l];
    for (int k = body; k < d; k++) {
        float sq = y[k] * y[k];
        s = s + sq;
    }
    return sqrtf(s);
}

/* core/lloyd_max.py:131-132: bucketize(x, boundaries) - 1, clamped.
 * bucketize(right=False) = number of boundaries strictly below x. */
static inline uint8_t quantize_one(float x, const float *boundaries, int nb, int levels) {
    int c = 0;
    for (int i = 0; i < nb; i++) c += (boundaries[i] < x) ? 1 : 0;
    c -= 1;
    if (c < 0) c = 0;
    if (c > levels - 1) c = levels - 1;
    return (uint8_t)c;
}

/* core/quantizer.py:137-160.  x: [n, d] fp32 (bf16/fp16 callers widen first,
 * exactly as x.float() does).  Outputs packed [n, packed_dim] u8 and
 * norms [n] as fp16 bit patterns.  If `normalized_out` is non-NULL it receives
 * the normalised rotated coordinates [n, d] (used by tests to find elements
 * that sit within 1e-6 of a decision boundary). */
void ftq_oracle_encode(const float *x, int64_t n, int d, int bits, const float *signs,
                       const float *boundaries, uint8_t *packed, uint16_t *norms_f16,
                       int norm_lanes, float *normalized_out) {
    const int levels = 1 << bits;
    const int nb = levels + 1;
    const int pd = ftq_oracle_packed_dim(d, bits);
#pragma omp parallel for schedule(static)
    for (int64_t v = 0; v < n; v++) {
        float y[FTQ_MAX_D];
        uint8_t idx[FTQ_MAX_D];
        const float *xi = x + v * d;
        for (int i = 0; i < d; i++) y[i] = signs ? xi[i] * signs[i] : xi[i];
        ftq_oracle_fwht(y, d);
        float norm = norm_like_torch(y, d, norm_lanes);
        float denom = norm + 1e-8f;
        for (int i = 0; i < d; i++) {
            float nv = y[i] / denom;
            if (normalized_out) normalized_out[v * d + i] = nv;
            idx[i] = quantize_one(nv, boundaries, nb, levels);
        }
        ftq_oracle_pack(idx, packed + v * pd, d, bits);
        norms_f16[v] = ftq_oracle_f32_to_f16(norm);
    }
}

/* core/quantizer.py:191-205: unpack -> levels[idx] * float(norm) -> fwht -> *signs */
void ftq_oracle_decode_dense(const uint8_t *packed, const uint16_t *norms_f16, int64_t n, int d,
                             int bits, const float *levels, const float *signs, float *out) {
    const int pd = ftq_oracle_packed_dim(d, bits);
#pragma omp parallel for schedule(static)
    for (int64_t v = 0; v < n; v++) {
        float y[FTQ_MAX_D];
        uint8_t idx[FTQ_MAX_D];
        ftq_oracle_unpack(packed + v * pd, idx, d, bits);
        float nf = ftq_oracle_f16_to_f32(norms_f16[v]);
        for (int i = 0; i < d; i++) y[i] = levels[idx[i]] * nf;
        ftq_oracle_fwht(y, d);
        for (int i = 0; i < d; i++) out[v * d + i] = signs ? y[i] * signs[i] : y[i];
    }
}

/* --------------------------------------------------------- decode attention */

/* kernels/triton_attention.py:145-152 (what fused_qk_scores_rht returns):
 * score[b,hq,s] = norm[b,hkv,s] * sum_d q_rot[b,hq,d] * C[idx[b,hkv,s,d]] * scale
 * q_rot: [B,Hq,D] fp32 already rotated; k_norms fp32 [B,Hkv,S]. */
void ftq_oracle_qk_scores(const float *q_rot, const uint8_t *k_idx, const float *k_norms,
                          const float *levels, float scale, int bits, int B, int Hq, int Hkv,
                          int S, int d, float *scores) {
    const int pd = ftq_oracle_packed_dim(d, bits);
    const int group = Hq / Hkv;
#pragma omp parallel for collapse(2) schedule(static)
    for (int b = 0; b < B; b++)
        for (int hq = 0; hq < Hq; hq++) {
            uint8_t idx[FTQ_MAX_D];
            int hkv = hq / group;
            const float *q = q_rot + ((int64_t)b * Hq + hq) * d;
            for (int s = 0; s < S; s++) {
                int64_t t = ((int64_t)b * Hkv + hkv) * S + s;
                ftq_oracle_unpack(k_idx + t * pd, idx, d, bits);
                float acc = 0.0f;
                for (int i = 0; i < d; i++) acc += q[i] * levels[idx[i]];
                scores[((int64_t)b * Hq + hq) * S + s] = k_norms[t] * acc * scale;
            }
        }
}

/* Composed decode attention for one query token per sequence, restating the
 * reference's unfused path: dense-decode K and V into the ORIGINAL space
 * (_decode_unfused), scores = q . K^T * scale over s < seq_len, softmax in fp32,
 * out = w . V.  q is NOT rotated here.  K/V contiguous [B,Hkv,S,pd]; norms are
 * fp16 bit patterns [B,Hkv,S]; seq_lens may be NULL (all S).  out [B,Hq,D] fp32.
 * Accumulations run in double so the result is a tight target for the fp32
 * GPU kernel (the reference itself accumulates in fp32; the difference is
 * orders of magnitude inside the 2e-3 / 1e-3 gate). */
void ftq_oracle_decode_attn(const float *q, const uint8_t *k_idx, const uint16_t *k_norms,
                            const uint8_t *v_idx, const uint16_t *v_norms,
                            const float *levels_k, const float *levels_v, const float *signs,
                            float scale, int bits_k, int bits_v, const int32_t *seq_lens, int B,
                            int Hq, int Hkv, int S, int d, float *out) {
    const int pdk = ftq_oracle_packed_dim(d, bits_k);
    const int pdv = ftq_oracle_packed_dim(d, bits_v);
    const int group = Hq / Hkv;
#pragma omp parallel for collapse(2) schedule(dynamic, 1)
    for (int b = 0; b < B; b++)
        for (int hkv = 0; hkv < Hkv; hkv++) {
            int len = seq_lens ? seq_lens[b] : S;
            if (len > S) len = S;
            int64_t base = ((int64_t)b * Hkv + hkv) * S;
            float *kd = (float *)malloc((size_t)(len > 0 ? len : 1) * d * sizeof(float));
            float *vd = (float *)malloc((size_t)(len > 0 ? len : 1) * d * sizeof(float));
            double *w = (double *)malloc((size_t)(len > 0 ? len : 1) * sizeof(double));
            uint8_t idx[FTQ_MAX_D];
            float y[FTQ_MAX_D];
            for (int s = 0; s < len; s++) {
                ftq_oracle_unpack(k_idx + (base + s) * pdk, idx, d, bits_k);
                float nf = ftq_oracle_f16_to_f32(k_norms[base + s]);
                for (int i = 0; i < d; i++) y[i] = levels_k[idx[i]] * nf;
                ftq_oracle_fwht(y, d);
                for (int i = 0; i < d; i++) kd[(int64_t)s * d + i] = signs ? y[i] * signs[i] : y[i];
                ftq_oracle_unpack(v_idx + (base + s) * pdv, idx, d, bits_v);
                nf = ftq_oracle_f16_to_f32(v_norms[base + s]);
                for (int i = 0; i < d; i++) y[i] = levels_v[idx[i]] * nf;
                ftq_oracle_fwht(y, d);
                for (int i = 0; i < d; i++) vd[(int64_t)s * d + i] = signs ? y[i] * signs[i] : y[i];
            }
            for (int g = 0; g < group; g++) {
                int hq = hkv * group + g;
                const float *qv = q + ((int64_t)b * Hq + hq) * d;
                float *o = out + ((int64_t)b * Hq + hq) * d;
                if (len <= 0) {
                    for (int i = 0; i < d; i++) o[i] = 0.0f;
                    continue;
                }
                double m = -INFINITY;
                for (int s = 0; s < len; s++) {
                    double acc = 0.0;
                    for (int i = 0; i < d; i++) acc += (double)qv[i] * (double)kd[(int64_t)s * d + i];
                    w[s] = (double)(float)(acc * (double)scale);
                    if (w[s] > m) m = w[s];
                }
                double l = 0.0;
                for (int s = 0; s < len; s++) { w[s] = exp(w[s] - m); l += w[s]; }
                for (int i = 0; i < d; i++) {
                    double acc = 0.0;
                    for (int s = 0; s < len; s++) acc += w[s] * (double)vd[(int64_t)s * d + i];
                    o[i] = (float)(acc / l);
                }
            }
            free(kd); free(vd); free(w);
        }
}

/* ------------------------------------------------------------ paged layouts */

/* Reference v0 paged layout (vllm_plugin/backend.py:107-124, cache_ops.py:85-108):
 * kv_cache u8 [2, num_blocks, block_size, Hkv, packed_dim+4]; plane 0 = K, 1 = V;
 * each slot = packed codes followed by the norm widened to 4 fp32 bytes.
 * Tokens whose slot is negative are skipped (attention_impl.py:217-220). */
void ftq_oracle_v0_write(uint8_t *kv_cache, int64_t num_blocks, int block_size, int Hkv,
                         int elem_size, int kv_type, const uint8_t *packed, int pd,
                         const uint16_t *norms_f16, const int64_t *slot_mapping, int64_t n_tokens) {
    for (int64_t t = 0; t < n_tokens; t++) {
        int64_t slot = slot_mapping[t];
        if (slot < 0) continue;
        int64_t blk = slot / block_size, off = slot % block_size;
        for (int h = 0; h < Hkv; h++) {
            uint8_t *dst = kv_cache +
                (((((int64_t)kv_type * num_blocks + blk) * block_size + off) * Hkv + h) * elem_size);
            memcpy(dst, packed + (t * Hkv + h) * pd, (size_t)pd);
            float nf = ftq_oracle_f16_to_f32(norms_f16[t * Hkv + h]);
            memcpy(dst + pd, &nf, 4);
        }
    }
}

/* cache_ops.py:151-205: walk the block table, copy slot bytes, reinterpret the
 * 4 norm bytes as fp32; positions >= seq_len stay zero. */
void ftq_oracle_v0_gather(const uint8_t *kv_cache, int64_t num_blocks, int block_size, int Hkv,
                          int elem_size, int kv_type, int pd, const int32_t *block_tables,
                          int max_blocks, const int32_t *seq_lens, int B, int max_seq_len,
                          uint8_t *out_packed, float *out_norms) {
    memset(out_packed, 0, (size_t)B * Hkv * max_seq_len * pd);
    memset(out_norms, 0, (size_t)B * Hkv * max_seq_len * sizeof(float));
    for (int b = 0; b < B; b++)
        for (int pos = 0; pos < seq_lens[b]; pos++) {
            int64_t blk = block_tables[(int64_t)b * max_blocks + pos / block_size];
            int off = pos % block_size;
            for (int h = 0; h < Hkv; h++) {
                const uint8_t *src = kv_cache +
                    (((((int64_t)kv_type * num_blocks + blk) * block_size + off) * Hkv + h) * elem_size);
                int64_t o = ((int64_t)b * Hkv + h) * max_seq_len + pos;
                memcpy(out_packed + o * pd, src, (size_t)pd);
                memcpy(out_norms + o, src + pd, 4);
            }
        }
}

/* ============================================================================
 * vLLM-v1 "TURBOQUANT" slot format: in-kernel-rotation store and split-KV decode.
 *
 * Restates the reference's Triton kernels
 *   _fused_store_rht + _bucketize_pack_norm_v_store
 *       src/fused_turboquant/vllm_plugin/triton_inkernel_store.py:365-440, 39-330
 *   _tq_decode_stage1_offset
 *       src/fused_turboquant/vllm_plugin/triton_decode_offset.py:42-444
 * and the stock stage-2 merge they are followed by (call site
 * src/fused_turboquant/vllm_plugin/v1_backend.py:1068-1085).
 *
 * Slot of one (token, KV head):  [key codes | key norm f16 | value codes | scale f16 | zero f16]
 * at kv_cache + block*stride_block + pos*stride_pos + head*stride_head.
 *
 * Parity status: PINNED against tests/golden/tq_v1.npz, which holds what those kernels
 * wrote when executed in Triton's interpreter mode (tests/golden/make_golden_tq_v1.py).
 * One degree of freedom is not fixed by the reference: the order in which `tl.sum`
 * adds the squares of the key.  This file (and the CUDA kernel) add them in "octet order":
 * 8 running sums over the coordinates 8(t+8i)+c (t = sum index, c then i ascending),
 * combined pairwise (t^1, t^2, t^4).  A different order moves the norm by an ulp at most,
 * which can flip a code only where the rotated value sits within ~1e-7 of a midpoint.
 * ==========================================================================*/

static float tq_key_norm_sq(const float *k, int d) {
    float lane[8];
    for (int t = 0; t < 8; t++) {
        float s = 0.0f;
        for (int i = 0; i < d / 64; i++)
            for (int c = 0; c < 8; c++) {
                float v = k[8 * (t + 8 * i) + c];
                float sq = v * v;
                s = s + sq;
            }
        lane[t] = s;
    }
    for (int m = 1; m < 8; m <<= 1) {
        float nxt[8];
        for (int t = 0; t < 8; t++) nxt[t] = lane[t] + lane[t ^ m];
        memcpy(lane, nxt, sizeof(lane));
    }
    return lane[0];
}

/* Sum of squares in the order the CUDA store adds them when the vector sits in the butterfly's
 * output layout (after the fused value rotation): lane l of the octet owns the coordinates
 * l + 8k, k ascending, then the lanes are combined pairwise. */
static float tq_norm_sq_rotated_layout(const float *v, int d) {
    float lane[8];
    for (int l = 0; l < 8; l++) {
        float s = 0.0f;
        for (int k = 0; k < d / 8; k++) {
            float sq = v[l + 8 * k] * v[l + 8 * k];
            s = s + sq;
        }
        lane[l] = s;
    }
    for (int m = 1; m < 8; m <<= 1) {
        float nxt[8];
        for (int t = 0; t < 8; t++) nxt[t] = lane[t] + lane[t ^ m];
        memcpy(lane, nxt, sizeof(lane));
    }
    return lane[0];
}

static void tq_pack_bits(const int *idx, uint8_t *out, int d, int bits) {
    if (bits == 8) {
        for (int i = 0; i < d; i++) out[i] = (uint8_t)idx[i];
        return;
    }
    if (bits == 1) { /* coordinate 8k + j in bit j of byte k (triton_inkernel_store.py:138-146) */
        for (int k = 0; k < d / 8; k++) {
            unsigned b = 0;
            for (int j = 0; j < 8; j++) b |= (unsigned)(idx[8 * k + j] & 1) << j;
            out[k] = (uint8_t)b;
        }
        return;
    }
    uint8_t tmp[FTQ_MAX_D];
    for (int i = 0; i < d; i++) tmp[i] = (uint8_t)idx[i];
    ftq_oracle_pack(tmp, out, d, bits);
}

/* fp32 -> FP8 e4m3 (1-4-3, bias 7, no infinities, 0x7f = NaN): round to nearest even, finite
 * overflow saturates to +-448 -- the semantics of the conversion instruction that the reference's
 * `.to(tl.float8e4nv)` (triton_inkernel_store.py:84-87) compiles to on a GPU. */
static uint8_t f32_to_e4m3(float x) {
    uint8_t sign = signbit(x) ? 0x80 : 0;
    if (isnan(x)) return (uint8_t)(sign | 0x7f);
    double a = fabs((double)x);
    if (a >= 464.0) return (uint8_t)(sign | 0x7e); /* 464 = halfway to the absent 512: saturate */
    int e;
    int q; /* value = q * 2^(e-3) with q in [8, 16), or a subnormal multiple of 2^-9 */
    if (a < 0.015625) { /* below 2^-6: multiples of 2^-9 */
        double r = nearbyint(a * 512.0); /* default rounding mode: to nearest even */
        q = (int)r;
        if (q == 8) return (uint8_t)(sign | 0x08);
        return (uint8_t)(sign | q);
    }
    double m = frexp(a, &e); /* a = m * 2^e, m in [0.5, 1) */
    q = (int)nearbyint(m * 16.0); /* in [8, 16] */
    e -= 1;                       /* a ~ (q / 8) * 2^e */
    if (q == 16) { q = 8; e += 1; }
    int be = e + 7;
    if (be > 15 || (be == 15 && q - 8 > 6)) return (uint8_t)(sign | 0x7e);
    return (uint8_t)(sign | (be << 3) | (q - 8));
}
static float e4m3_to_f32(uint8_t b) {
    int be = (b >> 3) & 0xf, m = b & 7;
    float v;
    if (be == 0xf && m == 7) return NAN;
    if (be == 0) v = ldexpf((float)m, -9);
    else v = ldexpf((float)(8 + m), be - 7 - 3);
    return (b & 0x80) ? -v : v;
}

static void put_f16(uint8_t *dst, float v) {
    uint16_t h = ftq_oracle_f32_to_f16(v);
    dst[0] = (uint8_t)(h & 0xff);
    dst[1] = (uint8_t)(h >> 8);
}
static float get_f16(const uint8_t *src) {
    return ftq_oracle_f16_to_f32((uint16_t)(src[0] | (src[1] << 8)));
}

/* key/value: [n_tokens, Hkv, d] fp32 contiguous.  y_out (nullable): the rotated unit keys.
 * value_lloyd_max (4-bit values only, otherwise ignored: triton_inkernel_store.py:159-203): the
 * value is normalised like the key, bucketised against the key midpoints, its norm stored in the
 * scale field, zero point 0.  value_sum_order: 0 = squares added in the key's order, 1 = in the
 * order of the CUDA store's fused value rotation (the reference leaves the order open). */
void ftq_oracle_tq_store(const float *key, const float *value, int64_t n_tokens, int Hkv, int d,
                         int key_bits, int value_bits, const float *midpoints, uint8_t *kv_cache,
                         int64_t stride_block, int64_t stride_pos, int64_t stride_head,
                         int block_size, const int64_t *slot_mapping, float *y_out,
                         int value_lloyd_max, int value_sum_order) {
    /* key_bits 264 = 8-bit Lloyd-Max codes (256 centroids, one byte per coordinate + norm:
     * triton_inkernel_store.py:132-137, boundary_tq_config.py:26-35); 8 = FP8 keys */
    const int key_mse8 = key_bits == 264;
    if (key_mse8) key_bits = 8;
    const int key_fp8 = key_bits == 8 && !key_mse8; /* d bytes of e4m3(y * norm), no norm field */
    const int n_cent = key_fp8 ? 1 : 1 << key_bits;
    const int mse_bytes = d * key_bits / 8;
    const int kps = mse_bytes + (key_fp8 ? 0 : 2);
    const int vdb = value_bits == 8 ? d : d * value_bits / 8;
    const int vmax = (1 << value_bits) - 1;
    const float rs = 1.0f / sqrtf((float)d);
    for (int64_t tok = 0; tok < n_tokens; tok++) {
        const int64_t slot = slot_mapping[tok];
        if (slot < 0) continue;
        for (int h = 0; h < Hkv; h++) {
            const float *k = key + (tok * Hkv + h) * d;
            const float *v = value + (tok * Hkv + h) * d;
            uint8_t *dst = kv_cache + (slot / block_size) * stride_block +
                           (slot % block_size) * stride_pos + (int64_t)h * stride_head;
            /* keys: norm of the raw vector, normalise, Hadamard (no signs), midpoint search */
            float norm = sqrtf(tq_key_norm_sq(k, d) + 1e-16f);
            float y[FTQ_MAX_D];
            float den = norm + 1e-8f;
            for (int i = 0; i < d; i++) y[i] = k[i] / den;
            for (int hh = 1; hh < d; hh <<= 1)
                for (int base = 0; base < d; base += 2 * hh)
                    for (int j = 0; j < hh; j++) {
                        float a = y[base + j], b = y[base + hh + j];
                        y[base + j] = a + b;
                        y[base + hh + j] = a - b;
                    }
            int idx[FTQ_MAX_D];
            for (int i = 0; i < d; i++) {
                y[i] = y[i] * rs;
                int c = 0;
                for (int j = 0; j < n_cent - 1; j++) c += (y[i] >= midpoints[j]) ? 1 : 0;
                idx[i] = c;
            }
            if (y_out) memcpy(y_out + (tok * Hkv + h) * d, y, sizeof(float) * d);
            if (key_fp8) {
                for (int i = 0; i < d; i++) {
                    float un = y[i] * norm;
                    dst[i] = f32_to_e4m3(un);
                }
            } else {
                tq_pack_bits(idx, dst, d, key_bits);
                put_f16(dst + mse_bytes, norm);
            }
            if (value_lloyd_max && value_bits == 4) {
                float vn = sqrtf((value_sum_order ? tq_norm_sq_rotated_layout(v, d)
                                                  : tq_key_norm_sq(v, d)) + 1e-16f);
                float vden = vn + 1e-8f;
                for (int i = 0; i < d; i++) {
                    float u = v[i] / vden;
                    int c = 0;
                    for (int j = 0; j < n_cent - 1; j++) c += (u >= midpoints[j]) ? 1 : 0;
                    idx[i] = c;
                }
                tq_pack_bits(idx, dst + kps, d, 4);
                put_f16(dst + kps + vdb, vn);
                put_f16(dst + kps + vdb + 2, 0.0f);
                continue;
            }
            /* values: per-vector uniform quantisation */
            float mn = v[0], mx = v[0];
            for (int i = 1; i < d; i++) {
                mn = v[i] < mn ? v[i] : mn;
                mx = v[i] > mx ? v[i] : mx;
            }
            float scale = (mx - mn) / (float)vmax;
            if (!(scale > 1e-8f)) scale = 1e-8f;
            for (int i = 0; i < d; i++) {
                float t = (v[i] - mn) / scale;
                t = t + 0.5f;
                int q = (int)t;
                idx[i] = q < 0 ? 0 : (q > vmax ? vmax : q);
            }
            tq_pack_bits(idx, dst + kps, d, value_bits);
            put_f16(dst + kps + vdb, scale);
            put_f16(dst + kps + vdb + 2, mn);
        }
    }
}

static int tq_code(const uint8_t *p, int i, int bits) {
    if (bits == 8) return p[i];
    int bo = i * bits;
    uint32_t w = (uint32_t)p[bo >> 3] | ((uint32_t)p[(bo >> 3) + 1] << 8);
    return (int)((w >> (bo & 7)) & ((1u << bits) - 1u));
}

/* q: [B, Hq, d] fp32 in the ORIGINAL space (rotated here with the plain Hadamard transform, as
 * rotation/matrix.py:47-48 does with a matrix product).  mid_o: [B, Hq, splits, d+1], out: [B, Hq, d],
 * lse: [B, Hq] (each nullable).  rotate_out != 0 applies the Hadamard transform to the merged output
 * (values stored in the rotated space, v1_backend.py:1088-1092). */
void ftq_oracle_tq_decode(const float *q, int B, int Hq, int Hkv, int d, const uint8_t *kv_cache,
                          int64_t stride_block, int64_t stride_pos, int64_t stride_head,
                          int block_size, const int32_t *block_table, int max_blocks,
                          const int32_t *seq_lens, const int32_t *kv_start, int key_bits,
                          int value_bits, int norm_correction, int rotate_out,
                          const float *centroids, float scale, int splits, float *mid_o,
                          float *out, float *lse, int value_lloyd_max) {
    const int v_lm = value_lloyd_max && value_bits == 4; /* triton_decode_offset.py:399-423 */
    const int group = Hq / Hkv;
    const int key_mse8 = key_bits == 264; /* 8-bit Lloyd-Max codes: the generic MSE branch */
    if (key_mse8) key_bits = 8;
    const int key_fp8 = key_bits == 8 && !key_mse8; /* triton_decode_offset.py:175-194 */
    const int mse_bytes = d * key_bits / 8;
    const int kps = mse_bytes + (key_fp8 ? 0 : 2);
    const int vdb = value_bits == 8 ? d : d * value_bits / 8;
#pragma omp parallel for collapse(2) schedule(dynamic)
    for (int b = 0; b < B; b++)
        for (int hq = 0; hq < Hq; hq++) {
            const int hk = hq / group;
            float qr[FTQ_MAX_D];
            memcpy(qr, q + ((int64_t)b * Hq + hq) * d, sizeof(float) * d);
            ftq_oracle_fwht(qr, d);
            const int seq_len = seq_lens[b];
            const int start = kv_start ? kv_start[b] : 0;
            const int eff = seq_len - start;
            const int split_len = (eff + splits - 1) / splits;
            double M = -INFINITY, L = 0.0, O[FTQ_MAX_D];
            for (int i = 0; i < d; i++) O[i] = 0.0;
            for (int s = 0; s < splits; s++) {
                const int s0 = start + split_len * s;
                const int s1 = s0 + split_len < seq_len ? s0 + split_len : seq_len;
                double m = -INFINITY, l = 0.0, acc[FTQ_MAX_D];
                for (int i = 0; i < d; i++) acc[i] = 0.0;
                for (int pos = s0; pos < s1; pos++) {
                    const int64_t blk = block_table[(int64_t)b * max_blocks + pos / block_size];
                    const uint8_t *slot = kv_cache + blk * stride_block +
                                          (int64_t)(pos % block_size) * stride_pos +
                                          (int64_t)hk * stride_head;
                    double dot = 0.0, cn = 0.0, sc;
                    if (key_fp8) {
                        for (int i = 0; i < d; i++) dot += (double)qr[i] * (double)e4m3_to_f32(slot[i]);
                        sc = dot * (double)scale;
                    } else {
                        for (int i = 0; i < d; i++) {
                            const double c = centroids[tq_code(slot, i, key_bits)];
                            dot += (double)qr[i] * c;
                            cn += c * c;
                        }
                        if (norm_correction) dot *= 1.0 / sqrt(cn + 1e-16);
                        sc = (double)get_f16(slot + mse_bytes) * dot * (double)scale;
                    }
                    double vs = get_f16(slot + kps + vdb), vz = get_f16(slot + kps + vdb + 2);
                    if (v_lm) { /* value = centroid[code] * norm, re-normalised under norm correction */
                        double vcn = 0.0;
                        for (int i = 0; i < d; i++) {
                            const double c = centroids[tq_code(slot + kps, i, 4)];
                            vcn += c * c;
                        }
                        if (norm_correction) vs *= 1.0 / sqrt(vcn + 1e-16);
                        vz = 0.0;
                    }
                    const double mn = sc > m ? sc : m;
                    const double corr = exp(m - mn), p = exp(sc - mn);
                    for (int i = 0; i < d; i++)
                        acc[i] = acc[i] * corr +
                                 p * ((v_lm ? (double)centroids[tq_code(slot + kps, i, 4)]
                                            : (double)tq_code(slot + kps, i, value_bits)) * vs + vz);
                    l = l * corr + p;
                    m = mn;
                }
                const double safe_l = l > 0.0 ? l : 1.0;
                const double lse_s = s0 < s1 ? m + log(safe_l) : -INFINITY;
                if (mid_o) {
                    float *mo = mid_o + (((int64_t)b * Hq + hq) * splits + s) * (d + 1);
                    for (int i = 0; i < d; i++) mo[i] = (float)(acc[i] / safe_l);
                    mo[d] = (float)lse_s;
                }
                if (s0 < s1) { /* merge as the stage-2 kernel does, on (acc / l, lse) */
                    const double Mn = lse_s > M ? lse_s : M;
                    const double old = exp(M - Mn), w = exp(lse_s - Mn);
                    for (int i = 0; i < d; i++) O[i] = O[i] * old + w * (acc[i] / safe_l);
                    L = L * old + w;
                    M = Mn;
                }
            }
            if (out) {
                float res[FTQ_MAX_D];
                for (int i = 0; i < d; i++) res[i] = (float)(O[i] / L);
                if (rotate_out) ftq_oracle_fwht(res, d);
                memcpy(out + ((int64_t)b * Hq + hq) * d, res, sizeof(float) * d);
            }
            if (lse) lse[(int64_t)b * Hq + hq] = (float)(M + log(L));
        }
}
