/*
 * ftq_b200.h -- C ABI of libftq_b200.so: fused-turboquant's KV encode and
 * compressed-KV decode attention as hand-written CUDA for NVIDIA B200 (sm_100a).
 *
 * Conventions
 *  - Every entry point returns 0 (FTQ_OK) or a negative ftq_status;
 *    ftq_last_error() returns the message of the last failure on the calling thread.
 *  - Pointers named *_host are host memory (small tables, read during the
 *    call); every other pointer is device memory on the current device.
 *  - No entry point allocates, frees or synchronises, except
 *    where its comment says otherwise.  Work is enqueued on `stream`
 *    (a cudaStream_t passed as void*; NULL = the legacy default stream).
 *  - Tensors are dense row-major unless a stride argument says otherwise.
 *  - head_dim must be 64, 128 or 256; bits must be 2, 3 or 4.
 *  - Packed code formats are the reference's (core/packing.py:14-128):
 *    4-bit: byte = code[2i] | code[2i+1] << 4; 2-bit: 4 codes per byte, LSB
 *    first; 3-bit: 8 codes -> 24-bit little-endian stream.  Norms are IEEE fp16.
 *
 * Reference citations are paths inside the sudy-super/fused-turboquant project.
 */
#ifndef FTQ_B200_H
#define FTQ_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
    FTQ_OK = 0,
    FTQ_ERR_INVALID = -1,     /* bad argument (shape, bits, alignment, NULL) */
    FTQ_ERR_UNSUPPORTED = -2, /* valid request this build has no kernel for  */
    FTQ_ERR_CUDA = -3,        /* a CUDA runtime call failed                  */
    FTQ_ERR_WORKSPACE = -4,   /* caller workspace missing or too small       */
    FTQ_ERR_DEVICE = -5       /* a kernel reported a problem (ftq_paged_decode_status) */
} ftq_status;

typedef enum { FTQ_F32 = 0, FTQ_F16 = 1, FTQ_BF16 = 2 } ftq_dtype;

/* Tokens per page of the paged KV pool (fixed). */
#define FTQ_PAGE_TOKENS 16

/* Library version (major*10000 + minor*100 + patch). */
int ftq_version(void);

/* Message of the last error raised on this thread ("" if none). */
const char *ftq_last_error(void);

/* Bytes of packed codes per vector: head_dim*bits/8; -1 if unsupported.
 * Mirrors the packed_dim arithmetic of kernels/triton_encode.py:176-183. */
int ftq_packed_dim(int head_dim, int bits);

/* ------------------------------------------------------------------ encode */

/*
 * Fused encode: y = FWHT(x * signs) / sqrt(D); norm = ||y||2;
 * code = #{interior boundaries < y/(norm+1e-8)}; pack; norm -> fp16.
 * Replaces triton_fused_encode (kernels/triton_encode.py:150-209) and is
 * bit-exact with TurboQuantMSE._encode_unfused (core/quantizer.py:137-160).
 *   x            [n_vec, head_dim] of `dtype`, rows `row_stride` elements apart,
 *                each row 16-byte aligned
 *   signs_host   [head_dim] floats, each exactly +1 or -1; NULL = all +1
 *   boundaries_host [2^bits + 1] ascending (LloydMaxQuantizer.boundaries)
 *   packed       [n_vec, packed_dim] u8 out;  norms_f16 [n_vec] out
 */
int ftq_encode(const void *x, int dtype, int64_t n_vec, int head_dim, int64_t row_stride,
               int bits, const float *signs_host, const float *boundaries_host,
               uint8_t *packed, uint16_t *norms_f16, void *stream);

/*
 * Dense dequantisation: unpack -> levels[code] * norm -> FWHT -> * signs.
 * Replaces triton_fused_decode (kernels/triton_decode.py:104-155);
 * same arithmetic as TurboQuantMSE._decode_unfused (core/quantizer.py:191-205).
 *   norms: fp16 ([n_vec]) when norms_dtype == FTQ_F16, fp32 when FTQ_F32.
 *   out   [n_vec, head_dim] fp32
 */
int ftq_decode_dense(const uint8_t *packed, const void *norms, int norms_dtype, int64_t n_vec,
                     int head_dim, int bits, const float *levels_host, const float *signs_host,
                     float *out, void *stream);

/*
 * Randomized Hadamard transform, forward (FWHT(x*signs)) or inverse
 * (FWHT(x)*signs), output dtype = input dtype.
 * Replaces triton_rht (kernels/triton_rht.py:82-121); arithmetic of
 * randomized_hadamard / inverse_randomized_hadamard (core/hadamard.py:70-100).
 */
int ftq_rht(const void *x, void *y, int dtype, int64_t n_vec, int head_dim,
            const float *signs_host, int inverse, void *stream);

/* ------------------------------------------------------- attention (dense) */

/*
 * Scores from packed keys: out[b,hq,t,s] = norm[b,hkv,s] * scale *
 * sum_d q_rot[b,hq,t,d] * levels[code[b,hkv,s,d]],  hkv = hq / (Hq/Hkv).
 * Replaces fused_qk_scores_rht (kernels/triton_attention.py:158-225).
 *   q_rot [B,Hq,q_len,D] fp32 (already rotated); k_codes [B,Hkv,S,packed_dim];
 *   k_norms [B,Hkv,S] fp16 or fp32 (norms_dtype); out [B,Hq,q_len,S] fp32.
 */
int ftq_qk_scores(const float *q_rot, const uint8_t *k_codes, const void *k_norms,
                  int norms_dtype, const float *levels_host, float scale, int bits, int B, int Hq,
                  int Hkv, int q_len, int S, int head_dim, float *out, void *stream);

/*
 * Bytes of caller workspace ftq_flash_decode / ftq_paged_decode_attn need for
 * a batch of B sequences (per layer) whose longest context is max_seq_len.
 */
size_t ftq_decode_workspace_bytes(int B, int Hq, int Hkv, int head_dim, int max_seq_len,
                                  int n_layers);

/*
 * Single-pass decode attention over CONTIGUOUS compressed K/V (one query
 * token per sequence): rotated-space Q.K, online softmax, V accumulation,
 * inverse rotation of the output.  Fills the slot of flash_decode_compressed
 * (kernels/triton_flash_decode.py:224-324); unlike the reference it honours
 * seq_lens.
 *   q [B,Hq,D] of q_dtype; q_is_rotated != 0 means q is already RHT-rotated
 *   (the reference's calling convention), 0 means the kernel rotates it.
 *   k_codes [B,Hkv,S,pdk], k_norms [B,Hkv,S] fp16, same for v.
 *   seq_lens [B] int32 device or NULL (= S everywhere).
 *   out [B,Hq,D] of out_dtype, in the ORIGINAL (un-rotated) space.
 *   workspace: device scratch of ftq_decode_workspace_bytes(B,Hq,Hkv,D,S,1) bytes.
 */
int ftq_flash_decode(const void *q, int q_dtype, int q_is_rotated, const uint8_t *k_codes,
                     const uint16_t *k_norms, const uint8_t *v_codes, const uint16_t *v_norms,
                     const float *levels_k_host, const float *levels_v_host,
                     const float *signs_host, float scale, int bits_k, int bits_v,
                     const int32_t *seq_lens, int B, int Hq, int Hkv, int S, int head_dim,
                     void *out, int out_dtype, void *workspace, size_t workspace_bytes,
                     void *stream);

/* ------------------------------------------------------------- paged pool */

/*
 * Page layout of the paged KV pool (one pool per layer):
 *   pool u8 [num_blocks, Hkv, page_bytes]; a (block, head) page holds 16 tokens:
 *     [ K codes 16 x pdk | K norms 16 x fp16 | V codes 16 x pdv | V norms 16 x fp16 ]
 *   page_bytes = 16 * (pdk + pdv + 4); every sub-array starts 16-byte aligned.
 *   K rows and all norms are in token order.  A V row (pdv bytes) is stored with its two
 *   halves exchanged when the token's offset in the page has bit 1 set (tokens 2, 3, 6, 7,
 *   10, 11, 14, 15): the decode kernel reads four rows per instruction and this spreads them
 *   over the shared-memory banks.  The bytes themselves are the reference's packed codes.
 * The pool plays the role of the kv_cache tensor whose shape the backend
 * defines (vllm_plugin/backend.py:107-124); slots hold the same code bytes
 * and fp16 norms the reference stores, grouped per (block, head) so that one
 * page is a single contiguous span.
 */
int64_t ftq_page_bytes(int head_dim, int bits_k, int bits_v);

/*
 * Fused encode + scatter of new K and V vectors into the paged pool.
 * Replaces FusedTurboQuantImpl._compress_and_write_to_cache
 * (vllm_plugin/attention_impl.py:190-254): tq.encode(K), tq_v.encode(V), then
 * the per-token slot writes; tokens with slot_mapping < 0 are skipped.
 *   key, value   [n_tokens, Hkv, D] of `dtype`; token_stride / head_stride in elements
 *   slot_mapping [n_tokens] int64 device: slot = block * 16 + offset
 *   n_layers > 1 batches layers: key/value/pool advance by *_layer_stride
 *   (elements for key/value, bytes for the pool); slot_mapping is shared.
 */
int ftq_paged_store(const void *key, const void *value, int dtype, int64_t n_tokens, int Hkv,
                    int head_dim, int64_t token_stride, int64_t head_stride, int bits_k,
                    int bits_v, const float *signs_host, const float *boundaries_k_host,
                    const float *boundaries_v_host, uint8_t *pool, int64_t num_blocks,
                    const int64_t *slot_mapping, int n_layers, int64_t kv_layer_stride,
                    int64_t pool_layer_stride, void *stream);

/*
 * Paged decode attention, one query token per sequence, straight from the
 * packed pool through the block table (no gather, no dense K/V).
 * Replaces FusedTurboQuantImpl._forward_decode (vllm_plugin/attention_impl.py:431-521:
 * gather_compressed_kv_batched -> randomized_hadamard(q) -> fused_qk_scores_rht ->
 * softmax -> gather + decode V -> matmul) with one split-KV kernel plus a merge.
 *   q   [n_layers, B, Hq, D] of q_dtype, NOT rotated (rotation is fused)
 *   out [n_layers, B, Hq, D] of out_dtype, original space
 *   block_table [B, max_blocks] int32 device; seq_lens [B] int32 device
 *   (both shared by all layers); pool advances pool_layer_stride bytes per layer.
 *   max_seq_len: upper bound on seq_lens (host value; sizes the grid).
 *   workspace: ftq_decode_workspace_bytes(B,Hq,Hkv,D,max_seq_len,n_layers) bytes.
 */
int ftq_paged_decode_attn(const void *q, int q_dtype, void *out, int out_dtype,
                          const uint8_t *pool, int64_t num_blocks, int64_t pool_layer_stride,
                          int n_layers, const int32_t *block_table, int max_blocks,
                          const int32_t *seq_lens, int max_seq_len, int B, int Hq, int Hkv,
                          int head_dim, int bits_k, int bits_v, const float *levels_k_host,
                          const float *levels_v_host, const float *signs_host, float scale,
                          void *workspace, size_t workspace_bytes, void *stream);

/* ------------------------------------------- decode without a workspace */

/* Size of the scratch array built into the library (bytes, per GPU). */
#define FTQ_STATIC_SCRATCH_BYTES (8u << 20)

/*
 * ftq_paged_decode_attn for callers that cannot provide a workspace because
 * they cannot allocate device memory at all: engines that gave the whole
 * device to their own block manager, code entered where cudaMalloc is not
 * permitted or would stall every stream, hosts that forbid allocation after
 * start-up.  It has no counterpart in the reference (which allocates freely
 * through torch); it exists only for such embedders.
 *
 * Same arguments and results as ftq_paged_decode_attn, minus the workspace:
 * the split-KV partials go to an 8 MiB array that is part of the library
 * image.  Consequences to know about:
 *   - every GPU that loads the library holds those 8 MiB until the process ends;
 *   - a batch whose partials exceed FTQ_STATIC_SCRATCH_BYTES
 *     (ftq_decode_workspace_bytes tells) is rejected with FTQ_ERR_WORKSPACE;
 *   - all calls on one GPU share the array and it keeps whatever the last call
 *     left (every partial row that is read is written first by the same call,
 *     and the counters in its tail are cleared at the start of every call,
 *     by the kernel itself or by a memset node), so two calls that may run at the same time on one GPU
 *     (different streams) corrupt each other: serialise them;
 *   - the device that owns q / out / pool must be the current device of the
 *     calling thread: the size check and the scratch address are per device;
 *   - the first call on each device looks up the array's device address
 *     (one cudaGetSymbolAddress, no allocation); make that first call outside
 *     any stream capture.
 * The call itself allocates nothing and frees nothing.
 */
int ftq_paged_decode_attn_static(const void *q, int q_dtype, void *out, int out_dtype,
                                 const uint8_t *pool, int64_t num_blocks,
                                 int64_t pool_layer_stride, int n_layers,
                                 const int32_t *block_table, int max_blocks,
                                 const int32_t *seq_lens, int max_seq_len, int B, int Hq, int Hkv,
                                 int head_dim, int bits_k, int bits_v, const float *levels_k_host,
                                 const float *levels_v_host, const float *signs_host, float scale,
                                 void *stream);

/*
 * What the kernels of the LAST ftq_paged_decode_attn call on `workspace` met
 * (`workspace` NULL: the last ftq_paged_decode_attn_static call on the current
 * device).  The shape arguments are that call's: they locate the status word
 * in the workspace tail.  *status_bits (may be NULL) receives
 *   FTQ_STATUS_BAD_BLOCK_ID   a block-table id outside [0, num_blocks); the id
 *                             was not dereferenced, the (sequence, KV head)
 *                             rows it belongs to are NaN;
 *   FTQ_STATUS_WAIT_EXPIRED   a bounded wait inside a kernel ran out; the rows
 *                             concerned are NaN.
 * Returns FTQ_OK when no bit is set, FTQ_ERR_DEVICE otherwise.  Copies four
 * bytes back and SYNCHRONISES `stream`: meant for a host that wants to know
 * without scanning the output for NaN, at a point where it can afford a sync.
 * No counterpart in the reference (its Triton kernels do not check ids).
 */
#define FTQ_STATUS_BAD_BLOCK_ID 1
#define FTQ_STATUS_WAIT_EXPIRED 2
int ftq_paged_decode_status(const void *workspace, int B, int Hq, int Hkv, int head_dim,
                            int max_seq_len, int n_layers, void *stream, int *status_bits);

/* ------------------------------------------- reference v0 layout adaptors */

/*
 * Same fused encode, written into the reference's own v0 paged layout
 * kv_cache u8 [2, num_blocks, block_size, Hkv, packed_dim + 4] (plane 0 = K,
 * 1 = V; slot = codes then the norm widened to 4 fp32 bytes), as
 * compute_compressed_elem_size / write_compressed_to_slot define it
 * (vllm_plugin/cache_ops.py:64-108).  Requires bits_k == bits_v or
 * elem_size >= max(pdk, pdv) + 4; `elem_size` is the last dimension.
 */
int ftq_v0_store(const void *key, const void *value, int dtype, int64_t n_tokens, int Hkv,
                 int head_dim, int64_t token_stride, int64_t head_stride, int bits_k, int bits_v,
                 const float *signs_host, const float *boundaries_k_host,
                 const float *boundaries_v_host, uint8_t *kv_cache, int64_t num_blocks,
                 int block_size, int elem_size, const int64_t *slot_mapping, void *stream);

/*
 * Gather from the v0 layout into contiguous tensors, the job of
 * gather_compressed_kv_batched (vllm_plugin/cache_ops.py:151-205), without the
 * per-token host loop: out_codes [B,Hkv,max_seq_len,pd] u8 (zero beyond
 * seq_len), out_norms [B,Hkv,max_seq_len] fp32.
 */
int ftq_v0_gather(const uint8_t *kv_cache, int64_t num_blocks, int block_size, int Hkv,
                  int elem_size, int kv_type, int packed_dim, const int32_t *block_tables,
                  int max_blocks, const int32_t *seq_lens, int B, int max_seq_len,
                  uint8_t *out_codes, float *out_norms, void *stream);

/* ---------------------------------------------------------------------------
 * vLLM-v1 "TURBOQUANT" slot format (the reference's in-kernel-rotation backend).
 *
 * kv_cache is the uint8 tensor [num_blocks, block_size, Hkv, slot] vLLM allocates
 * (src/fused_turboquant/vllm_plugin/v1_backend.py:149-261); the three byte strides
 * are passed explicitly, so any slot padding works.  They and the base address must
 * be even.  A slot holds
 *     [key codes D*kb/8 | key norm f16 | value codes D*vb/8 (D for vb = 8) | scale f16 | zero f16]
 * (vllm_plugin/boundary_tq_config.py:66-81; ftq_tq_slot_bytes returns its size rounded
 * up to even).  Supported: head_dim 64/128/256, key_bits 1/2/3/4 (Lloyd-Max codes) or 8,
 * which selects FP8 keys as vLLM's stock TurboQuantConfig does (key_quant_bits == 8;
 * triton_inkernel_store.py:80-91): the key field is then D bytes of e4m3 (rotated key * norm,
 * round to nearest even, saturating) with NO norm field, and midpoints_host / centroids_host
 * may be NULL; value_bits 1/2/3/4/8 (per-vector uniform codes; 4-bit values optionally
 * Lloyd-Max codes).  key_bits = FTQ_TQ_KEY_BITS_MSE8 selects the reference's 8-bit
 * Lloyd-Max key codes (256 centroids, its boundary layers: BoundaryTurboQuantConfig with
 * key_use_fp8_at_8bit = False, vllm_plugin/boundary_tq_config.py:26-35; store branch
 * triton_inkernel_store.py:132-137): the key field is D code bytes + the fp16 norm,
 * midpoints_host holds 255 and centroids_host 256 ascending entries; such caches are decoded
 * by the fp32 kernel, and Lloyd-Max value codes are not available with them.
 */
#define FTQ_TQ_KEY_BITS_MSE8 264
int ftq_tq_slot_bytes(int head_dim, int key_bits, int value_bits);

/*
 * Replaces RotationStrategy.launch_store -> _launch_rht -> _fused_store_rht
 * (vllm_plugin/rotation/hadamard.py:44-58, triton_inkernel_store.py:554-646 and 365-440):
 * per (token, KV head): norm of the raw key, key / (norm + 1e-8), Hadamard butterfly
 * without signs, * 1/sqrt(D), code = number of midpoints <= y, pack, fp16 norm; value:
 * min/max, scale = max((max - min) / (2^vb - 1), 1e-8), code = int((v - min) / scale + 0.5),
 * pack, fp16 scale and min.  Tokens with slot_mapping[token] < 0 are skipped.
 * key/value: [n_tokens, Hkv, head_dim] of `dtype`, strides in elements, rows 16-byte aligned.
 * midpoints_host: 2^key_bits - 1 floats, ascending.  rotate_values != 0 keeps the values in the
 * rotated space (TURBOQUANT_V_ROTATE, v1_backend.py:727-740): they are Hadamard-transformed in
 * the kernel (no signs, * 1/sqrt(D), rounded to `dtype` as the reference's tensor would be) before
 * they are quantised; not available for value_bits = 8 (FTQ_ERR_UNSUPPORTED: rotate them first,
 * e.g. with ftq_rht and no signs).  value_lloyd_max != 0 (TURBOQUANT_V_LLOYD_MAX,
 * triton_inkernel_store.py:159-203; 4-bit values only, ignored for other widths as in the
 * reference): the (rotated) value is normalised like the key, bucketised against the KEY
 * midpoints and packed as 4-bit codes; its norm is stored where the scale would be, the zero
 * point is 0.
 */
int ftq_tq_store(const void *key, const void *value, int dtype, int64_t n_tokens, int Hkv,
                 int head_dim, int64_t token_stride, int64_t head_stride, int key_bits,
                 int value_bits, int rotate_values, int value_lloyd_max,
                 const float *midpoints_host, uint8_t *kv_cache, int64_t stride_block,
                 int64_t stride_pos, int64_t stride_head, int block_size,
                 const int64_t *slot_mapping, void *stream);

/*
 * ftq_tq_store for the caches of n_layers layers in ONE launch: key / value are
 * [n_layers, n_tokens, Hkv, head_dim] (kv_layer_stride elements between layers), the caches
 * lie cache_layer_stride bytes apart and every layer uses the same slot_mapping (vLLM gives all
 * layers the same one).  The reference stores per layer (v1_backend.py:727-760); small models
 * are launch-bound that way.  num_blocks > 0 additionally skips every slot at or beyond
 * num_blocks * block_size (a stale or corrupt mapping) like a negative one, instead of writing
 * out of bounds.  With n_layers = 1, strides 0, num_blocks = 0 this is ftq_tq_store.
 */
int ftq_tq_store_layers(const void *key, const void *value, int dtype, int64_t n_tokens, int Hkv,
                        int head_dim, int64_t token_stride, int64_t head_stride, int key_bits,
                        int value_bits, int rotate_values, int value_lloyd_max,
                        const float *midpoints_host, uint8_t *kv_cache, int64_t stride_block,
                        int64_t stride_pos, int64_t stride_head, int block_size,
                        const int64_t *slot_mapping, int n_layers, int64_t kv_layer_stride,
                        int64_t cache_layer_stride, int64_t num_blocks, void *stream);

/*
 * Replaces _decode_attention_offset_only (vllm_plugin/v1_backend.py:975-1093): query
 * rotation q @ H, _tq_decode_stage1_offset (vllm_plugin/triton_decode_offset.py:42-444)
 * and the stage-2 merge, in two launches.  q: [B, Hq, head_dim] of q_dtype in the original
 * space.  Attends positions [kv_start_offset[b], seq_lens[b]) (kv_start_offset may be NULL = 0),
 * split into num_kv_splits ranges exactly as the reference splits them.  mid_o
 * (caller-provided, [B, Hq, num_kv_splits, head_dim + 1] fp32) receives the same partials
 * the reference's stage 1 writes (acc / l and lse; zeros and -inf for an empty range).
 * out: [B, Hq, head_dim] of out_dtype; lse (nullable): [B, Hq] fp32.  norm_correction:
 * re-normalise each key's centroid vector to unit length.  rotate_output: apply the
 * Hadamard transform to the merged output (values were stored in the rotated space).
 * value_lloyd_max: 4-bit values are Lloyd-Max codes of the key table scaled by the stored norm
 * (triton_decode_offset.py:399-423; re-normalised under norm_correction); ignored for other widths.
 * centroids_host: 2^key_bits floats, ascending.  prefix_out / prefix_lse (both or neither;
 * [B, Hq, head_dim] of prefix_dtype in the original space, [B, Hq] fp32): the attention of the same
 * queries over an uncompressed prefix [0, kv_start_offset[b]) computed by the caller; it is merged
 * in by log-sum-exp, with the weights of _decode_attention_hybrid (v1_backend.py:1267-1277), after
 * the output rotation; lse then receives the merged value.  No allocation, no host synchronisation.
 */
int ftq_tq_decode(const void *q, int q_dtype, int B, int Hq, int Hkv, int head_dim,
                  const uint8_t *kv_cache, int64_t stride_block, int64_t stride_pos,
                  int64_t stride_head, int block_size, const int32_t *block_table,
                  int max_blocks, const int32_t *seq_lens, const int32_t *kv_start_offset,
                  int key_bits, int value_bits, int norm_correction, int rotate_output,
                  int value_lloyd_max, const float *centroids_host, float scale,
                  int num_kv_splits, float *mid_o, void *out, int out_dtype, float *lse,
                  const void *prefix_out, int prefix_dtype, const float *prefix_lse,
                  void *stream);

/*
 * ftq_tq_decode over the caches of n_layers layers in ONE call (two launches in total): q, mid_o,
 * out, lse and the prefix tensors are stacked along a leading layer axis ([n_layers * B, ...] rows,
 * layer-major), layer i's cache starts cache_layer_stride bytes (even) after layer i - 1's, and
 * every layer uses the same block_table / seq_lens / kv_start_offset rows (vLLM gives all layers
 * of a request the same block ids).  The reference launches once per layer
 * (vllm_plugin/v1_backend.py:1030-1085); small layers (a 0.5 B model moves 14 MB per layer) are
 * launch-bound that way, which is what this entry point removes.  n_layers * B <= 65535.
 * num_blocks > 0 additionally checks every block id the kernels read against [0, num_blocks): an
 * id outside is never dereferenced, and the (sequence, head) rows it belongs to come back as NaN.
 * With n_layers = 1, cache_layer_stride = 0, num_blocks = 0 this is ftq_tq_decode.
 */
int ftq_tq_decode_layers(const void *q, int q_dtype, int B, int Hq, int Hkv, int head_dim,
                         const uint8_t *kv_cache, int64_t stride_block, int64_t stride_pos,
                         int64_t stride_head, int block_size, const int32_t *block_table,
                         int max_blocks, const int32_t *seq_lens, const int32_t *kv_start_offset,
                         int key_bits, int value_bits, int norm_correction, int rotate_output,
                         int value_lloyd_max, const float *centroids_host, float scale,
                         int num_kv_splits, float *mid_o, void *out, int out_dtype, float *lse,
                         const void *prefix_out, int prefix_dtype, const float *prefix_lse,
                         int n_layers, int64_t cache_layer_stride, int64_t num_blocks,
                         void *stream);

#ifdef __cplusplus
}
#endif
#endif /* FTQ_B200_H */
