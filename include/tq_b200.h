/*
 * tq_b200.h -- C ABI of libtq_b200.so: TurboQuant+ KV-cache compression on NVIDIA B200 (sm_100a).
 *
 * Every entry point is extern "C", takes plain pointers and sizes, returns TQ_OK (0) or a
 * negative TQ_ERR_* code, and (except the create/destroy pair and the *_sync helpers) neither
 * allocates nor synchronises: work is enqueued on the cudaStream_t passed as `stream`
 * (a void* here so that the header needs no CUDA include).  Pointers named *_dev are device
 * pointers owned by the caller; pointers in tq_quantizer_desc are host pointers that are read
 * during tq_quantizer_create only.  A status of TQ_OK means the launch was accepted;
 * asynchronous faults surface at the caller's next synchronisation.
 *
 * The reference project (TheTom/turboquant_plus) is pure Python/NumPy and has no FFI; each
 * declaration cites the reference function (file:line inside that project) whose arithmetic
 * the entry point replaces.
 */
#ifndef TQ_B200_H
#define TQ_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TQ_OK 0
#define TQ_ERR_INVALID (-1)      /* bad argument (null pointer, negative size, bad enum)       */
#define TQ_ERR_UNSUPPORTED (-2)  /* combination not built (e.g. WHT mode with d != 128)        */
#define TQ_ERR_ALIGN (-3)        /* a device pointer or stride is not aligned as documented    */
#define TQ_ERR_CUDA (-4)         /* a CUDA runtime call failed; see tq_last_error()            */
#define TQ_ERR_TOO_LARGE (-5)    /* size beyond a documented maximum or workspace too small    */
#define TQ_ERR_DEVICE (-6)       /* the device is not an sm_100 part / no kernel image         */

/* element types of caller buffers */
#define TQ_F32 0
#define TQ_F16 1
#define TQ_F64 2
#define TQ_BF16 3

/* rotation kinds */
#define TQ_ROT_DENSE 0 /* d x d orthogonal matrix: turboquant/rotation.py:25-50             */
#define TQ_ROT_WHT 1   /* D2 (H/sqrt d) D1 with +-1 sign vectors: turboquant/rotation.py:75-185 */

/* cache formats (per tensor, per layer) */
#define TQ_FMT_TURBO2 2  /* 2-bit PolarQuant + fp32 scale: 36 B / 128-d vector            */
#define TQ_FMT_TURBO3 3  /* 3-bit: 52 B                                                   */
#define TQ_FMT_TURBO4 4  /* 4-bit: 68 B                                                   */
#define TQ_FMT_Q8_0 8    /* int8 + fp16 scale per 32 values: 136 B                        */
#define TQ_FMT_PROD2 18  /* 1-bit PolarQuant + 1-bit QJL sketch + 2 fp32: 40 B (K only)   */
#define TQ_FMT_PROD3 19  /* 2-bit + 1-bit QJL: 56 B (K only)                              */
#define TQ_FMT_PROD4 20  /* 3-bit + 1-bit QJL: 72 B (K only)                              */

const char* tq_version(void);
const char* tq_error_string(int code);
/* message of the last failure on the calling thread ("" if none) */
const char* tq_last_error(void);

/* ------------------------------------------------------------------------------------------
 * Quantizer constants.  Mirrors the state a reference quantizer object holds after
 * construction: PolarQuant.__init__ (turboquant/polar_quant.py:46-54: rotation, centroids),
 * QJL.__init__ (turboquant/qjl.py:50-70: S) and TurboQuant.__init__
 * (turboquant/turboquant.py:57-77: PolarQuant(b-1) + QJL(seed+1000)).  The constants are
 * passed in, never generated here, so that they can be exported from the reference.
 * ------------------------------------------------------------------------------------------ */
typedef struct tq_quantizer tq_quantizer;

typedef struct tq_quantizer_desc {
  int32_t d;               /* vector dimension; WHT mode needs d == 128, dense mode 1..1024     */
  int32_t bits;            /* PolarQuant bit width, 1..4 (number of centroids = 1 << bits)      */
  int32_t rotation;        /* TQ_ROT_DENSE or TQ_ROT_WHT                                        */
  int32_t norm_correction; /* turboquant/polar_quant.py:109-112                                 */
  const double* rot;       /* dense: d*d row-major, y = rot @ x                                 */
  const double* signs1;    /* WHT: d values of +-1 applied before the transform                 */
  const double* signs2;    /* WHT: d values of +-1 applied after the transform                  */
  const double* centroids; /* 1 << bits sorted values                                           */
  int32_t qjl;             /* 0: none; 1: residual sketch present (kind follows `rotation`)     */
  const double* qjl_s;     /* dense: d*d row-major S, z = sign(S r)                             */
  const double* qjl_signs1;/* WHT: S = D2' (H/sqrt d) D1'                                       */
  const double* qjl_signs2;
} tq_quantizer_desc;

/* Allocates a few hundred KB of device memory on the current device and uploads the constants. */
int tq_quantizer_create(const tq_quantizer_desc* desc, tq_quantizer** out);
int tq_quantizer_destroy(tq_quantizer* q);

/* ------------------------------------------------------------------------------------------
 * tq_quantize: PolarQuant.quantize (turboquant/polar_quant.py:56-85), and, when the quantizer
 * has a QJL stage and out_qjl_dev is given, TurboQuant.quantize
 * (turboquant/turboquant.py:79-100 = polar_quant.py:121-132 + qjl.py:72-94).
 *
 *   x_dev          n vectors of d values, row stride ld (elements), type x_dtype.
 *                  WHT mode: TQ_F32 / TQ_F16 / TQ_BF16, rows 16-byte aligned.
 *                  dense mode: TQ_F32 / TQ_F16 / TQ_F64.
 *   out_packed_dev n * (d*bits/8) bytes, per vector the MSB-first bit stream of
 *                  utils.pack_indices (turboquant/utils.py:71-98); needs d*bits % 8 == 0; or NULL
 *   out_idx_dev    n * d bytes, one index per byte; or NULL
 *   out_norm_dev   n floats, ||x||_2; or NULL
 *   out_scale_dev  n floats, the factor dequantization multiplies centroids by:
 *                  ||x|| / ||centroids[idx]|| with norm correction, else ||x||; or NULL
 *   out_qjl_dev    n * ceil(d/8) bytes, utils.pack_bits order (turboquant/utils.py:20-49); or NULL
 *   out_rnorm_dev  n floats, ||residual||_2; or NULL
 * ------------------------------------------------------------------------------------------ */
int tq_quantize(const tq_quantizer* q, const void* x_dev, int32_t x_dtype, int64_t ld, int64_t n,
                uint8_t* out_packed_dev, uint8_t* out_idx_dev, float* out_norm_dev,
                float* out_scale_dev, uint8_t* out_qjl_dev, float* out_rnorm_dev, void* stream);

/* ------------------------------------------------------------------------------------------
 * tq_dequantize: PolarQuant.dequantize (turboquant/polar_quant.py:87-119) plus, when qjl_dev is
 * given, QJL.dequantize (turboquant/qjl.py:96-134) summed as in TurboQuant.dequantize
 * (turboquant/turboquant.py:102-124).  Exactly one of packed_dev / idx_dev is given.
 * out_dtype: TQ_F32, TQ_F16 or (dense mode) TQ_F64; out row stride = d.
 * ------------------------------------------------------------------------------------------ */
int tq_dequantize(const tq_quantizer* q, const uint8_t* packed_dev, const uint8_t* idx_dev,
                  const float* norm_dev, const uint8_t* qjl_dev, const float* rnorm_dev,
                  float shrinkage, int64_t n, void* out_dev, int32_t out_dtype, void* stream);

/* ------------------------------------------------------------------------------------------
 * tq_quantize_residual: PolarQuant.quantize_and_residual (turboquant/polar_quant.py:121-132) in one
 * launch, dense mode, fp64 arithmetic: indices (one per byte; or NULL), norms (or NULL) and
 * x - dequantize(indices, norms) as fp64 rows of stride ld_res elements.  x may be a column slice of
 * a wider matrix (row stride ld), and so may the residual: the two sub-vector quantizers of
 * OutlierTurboQuant.quantize (turboquant/outlier.py:110-150) write the halves of one residual
 * matrix, which tq_qjl_quantize then sketches.
 * tq_dequantize_strided: PolarQuant.dequantize into (accumulate = 0) or added onto (accumulate = 1)
 * a column slice of fp64 rows of stride ld_out: the scatter-and-add of OutlierTurboQuant.dequantize
 * (turboquant/outlier.py:180-208).
 * ------------------------------------------------------------------------------------------ */
int tq_quantize_residual(const tq_quantizer* q, const void* x_dev, int32_t x_dtype, int64_t ld, int64_t n,
                         uint8_t* out_idx_dev, float* out_norm_dev, double* out_residual_dev,
                         int64_t ld_res, void* stream);
int tq_dequantize_strided(const tq_quantizer* q, const uint8_t* idx_dev, const float* norm_dev, int64_t n,
                          double* out_dev, int64_t ld_out, int32_t accumulate, void* stream);

/* ------------------------------------------------------------------------------------------
 * tq_requantize: temporal decay of stored codes, requantize_3to2 of
 * benchmarks/temporal_decay_prototype.py:93-125 for any source / destination widths (dst <= src):
 * old tokens are re-coded with fewer bits without leaving the rotated domain.  Both quantizers are
 * sign-WHT mode with the same sign vectors (same seed).
 *   packed_src_dev  n * 16*bits_src bytes, the packed index stream tq_quantize writes
 *   scale_src_dev   n floats, the factor that multiplies the source centroids (out_scale_dev of
 *                   tq_quantize: norm / ||centroids[idx]||, the prototype's dequantize_3bit); with
 *                   scale_is_norm != 0 the vector norms instead, divided by ||centroids[idx]|| here
 *   packed_dst_dev  n * 16*bits_dst bytes
 *   norm_dst_dev    n floats, the norm of the source reconstruction (the prototype's recon_norm); or NULL
 *   scale_dst_dev   n floats, the prototype's corrected_norm: recon_norm / ||centroids_dst[idx_dst]||
 * ------------------------------------------------------------------------------------------ */
int tq_requantize(const tq_quantizer* src_q, const tq_quantizer* dst_q, const uint8_t* packed_src_dev,
                  const float* scale_src_dev, int32_t scale_is_norm, int64_t n, uint8_t* packed_dst_dev,
                  float* norm_dst_dev, float* scale_dst_dev, void* stream);

/* ------------------------------------------------------------------------------------------
 * Primitives with their own reference functions.
 * ------------------------------------------------------------------------------------------ */
/* utils.pack_indices (turboquant/utils.py:71-98): count indices (one per byte) -> MSB-first
 * stream of ceil(count*bits/8) bytes, bits in 1..4; bits in 5..8 copies the bytes. */
int tq_pack_indices(const uint8_t* idx_dev, int64_t count, int32_t bits, uint8_t* out_dev, void* stream);
/* inverse (the reference has none; the decode path needs it) */
int tq_unpack_indices(const uint8_t* packed_dev, int64_t count, int32_t bits, uint8_t* out_dev, void* stream);
/* utils.pack_bits / unpack_bits (turboquant/utils.py:20-68): rows of d int8 signs (+1 -> bit 1,
 * MSB first) <-> rows of ceil(d/8) bytes. */
int tq_pack_bits(const int8_t* signs_dev, int64_t rows, int32_t d, uint8_t* out_dev, void* stream);
int tq_unpack_bits(const uint8_t* packed_dev, int64_t rows, int32_t d, int8_t* out_dev, void* stream);
/* rotation.fast_walsh_hadamard_transform / apply_fast_rotation{,_batch,_transpose}
 * (turboquant/rotation.py:99-185) in fp64: rows of d values are zero-padded to n (power of two,
 * <= 4096), multiplied by signs1 (or not, if NULL), transformed, scaled 1/sqrt(n), multiplied by
 * signs2 (or not), cropped to d. */
int tq_sign_wht_f64(const double* x_dev, int64_t rows, int32_t d, int32_t n, const double* signs1_dev,
                    const double* signs2_dev, double* out_dev, void* stream);
/* codebook.nearest_centroid_indices (turboquant/codebook.py:121-134): index = number of fp64
 * midpoints strictly below the value. out: one int64 per value. */
int tq_nearest_centroid_f64(const double* values_dev, int64_t count, const double* centroids_dev,
                            int32_t n_centroids, int64_t* out_dev, void* stream);

/* QJL.quantize (turboquant/qjl.py:72-94) on its own, fp64 arithmetic, any d: bits of sign(S r) in
 * utils.pack_bits order (zero counts as +1) and ||r||_2.  Needs a dense-mode quantizer created
 * with qjl_s (its rot may be NULL).  r dtype TQ_F64 / TQ_F32 / TQ_F16. */
int tq_qjl_quantize(const tq_quantizer* q, const void* r_dev, int32_t dtype, int64_t n,
                    uint8_t* out_bits_dev, float* out_norm_dev, void* stream);
/* QJL.dequantize (turboquant/qjl.py:96-134): shrinkage * sqrt(pi/2)/sqrt(d) * ||r|| * S^T z. */
int tq_qjl_dequantize(const tq_quantizer* q, const uint8_t* bits_dev, const float* rnorm_dev,
                      float shrinkage, int64_t n, void* out_dev, int32_t out_dtype, void* stream);

/* ------------------------------------------------------------------------------------------
 * Paged compressed cache.  New surface: the reference's KVCacheCompressor
 * (turboquant/kv_cache.py:69-165) only has bulk compress/decompress; its docstring names a
 * streaming compress_token (kv_cache.py:65-66) that is never defined.  One layer's cache is a
 * byte pool of `num_pages` pages; page p, KV head h starts at p*page_stride + h*head_stride and
 * holds `page_tokens` tokens as consecutive arrays (offsets in the layout struct):
 *   K indices [page_tokens][d*bits/8] | K scale f32[page_tokens] | (K QJL bits [page_tokens][d/8]
 *   | K residual scale f32[page_tokens]) | V indices | V scale
 * q8_0 tensors hold int8 [page_tokens][d] | fp16 scales [page_tokens][d/32].
 * ------------------------------------------------------------------------------------------ */
typedef struct tq_cache_layout {
  int32_t d, page_tokens, num_kv_heads, k_format, v_format;
  int32_t k_idx_bytes, v_idx_bytes;       /* per token                                         */
  int32_t k_idx_off, k_scale_off, k_qjl_off, k_rscale_off, v_idx_off, v_scale_off;
  int32_t record_bytes;                   /* one (page, head) record, multiple of 128          */
  int64_t head_stride, page_stride;       /* bytes                                             */
} tq_cache_layout;

/* Fills every field from (d, page_tokens, num_kv_heads, k_format, v_format); d must be 128 and
 * page_tokens a multiple of 32 in 32..256. */
int tq_cache_layout_init(tq_cache_layout* layout, int32_t d, int32_t page_tokens, int32_t num_kv_heads,
                         int32_t k_format, int32_t v_format);

/* Quantize-on-append: k_dev, v_dev are [n_tokens][num_kv_heads][d] (dtype TQ_F32/TQ_F16/TQ_BF16),
 * slot_dev[t] = page*page_tokens + offset of token t (negative: skip the token).
 * kq / vq hold the constants of the K and V tensors (ignored for q8_0 tensors, may be NULL). */
int tq_cache_append(const tq_quantizer* kq, const tq_quantizer* vq, const tq_cache_layout* layout,
                    uint8_t* pool_dev, const void* k_dev, const void* v_dev, int32_t dtype,
                    int64_t n_tokens, const int64_t* slot_dev, void* stream);

/* Bookkeeping of a decode step in one launch (new surface; the reference appends in Python): for every sequence b
 * the slot of its next token, block_table[b][seq_lens[b] / page_tokens] * page_tokens + seq_lens[b] % page_tokens,
 * written `copies` times -- slots_dev[c][b] = slot + c * copy_stride, for layers whose pages follow one another in one
 * pool -- and seq_lens[b] incremented.  A sequence whose block-table row is full gets slot -1 (tq_cache_append skips
 * it) and keeps its length. */
int tq_decode_step_slots(const int32_t* block_table_dev, int32_t max_pages_per_seq, int32_t* seq_lens_dev,
                         int32_t page_tokens, int32_t batch, int32_t copies, int64_t copy_stride,
                         int64_t* slots_dev, void* stream);

/* Stores rows that were quantized elsewhere (tq_quantize with a dense-mode quantizer, whose
 * kernel does not address pages) into the records of a paged cache: which = 0 writes the K
 * arrays, 1 the V arrays.  packed_dev [n_tokens][num_kv_heads][idx_bytes], scale_dev
 * [n_tokens][num_kv_heads] (the out_scale of tq_quantize); PROD formats also take the sign sketch
 * [n_tokens][num_kv_heads][d/8] and residual scales = ||r|| * sqrt(pi/2)/sqrt(d).  Same new
 * surface as tq_cache_append (the reference has no paged cache). */
int tq_cache_store(const tq_cache_layout* layout, uint8_t* pool_dev, int32_t which,
                   const uint8_t* packed_dev, const float* scale_dev, const uint8_t* qjl_dev,
                   const float* rscale_dev, int64_t n_tokens, const int64_t* slot_dev, void* stream);

/* ------------------------------------------------------------------------------------------
 * Wire / on-disk block formats of the reference's documents (its llama.cpp fork's cache types;
 * docs/papers/block-size-experiment.md:25-37, docs/papers/turbo4-resurrection.md:125-138,169,208):
 *   turbo3: fp16 norm | qs[B/4] (low two index bits, element j in bits 2(j%4) of byte j/4) | signs[B/8]
 *           (third index bit, element j in bit j%8 of byte j/8); B = 32, 64 or 128 elements per block
 *   turbo2: fp16 norm | qs[B/4]
 *   turbo4: fp16 norm | fp16 rnorm (unused, written as 0) | qs[64] nibbles, element j in bits 4(j%2)
 *           of byte j/2; 128 elements per block
 * The norm of every block of a 128-element vector is the cache's scale (||x|| / ||centroids[idx]||)
 * rounded to fp16.  Blocks are laid out [n_tokens][num_kv_heads][128 / block_elems][block bytes] for
 * the tokens at slot_dev[t] (negative: skipped); which = 0 converts the K tensor, 1 the V tensor.
 * tq_block_bytes: bytes of one block, or -1 for a combination that does not exist.
 * ------------------------------------------------------------------------------------------ */
int64_t tq_block_bytes(int32_t format, int32_t block_elems);
int tq_cache_export_blocks(const tq_cache_layout* layout, const uint8_t* pool_dev, int32_t which,
                           const int64_t* slot_dev, int64_t n_tokens, int32_t block_elems,
                           uint8_t* out_dev, void* stream);
int tq_cache_import_blocks(const tq_cache_layout* layout, uint8_t* pool_dev, int32_t which,
                           const int64_t* slot_dev, int64_t n_tokens, int32_t block_elems,
                           const uint8_t* in_dev, void* stream);

/* tq_requantize on the records of paged caches: the K (which = 0) or V (which = 1) codes of the tokens at
 * src_slot_dev[t] of one cache are re-quantized into the records at dst_slot_dev[t] of a cache with a narrower
 * format (same KV heads, quantizers of the same seed); negative slots are skipped.  Old pages of a sequence move
 * to a pool that costs fewer bytes per token; tq_decode_attn_lse + tq_attn_merge then attend over both pools. */
int tq_cache_requantize(const tq_quantizer* src_q, const tq_quantizer* dst_q, const tq_cache_layout* src_layout,
                        const uint8_t* src_pool_dev, const int64_t* src_slot_dev,
                        const tq_cache_layout* dst_layout, uint8_t* dst_pool_dev, const int64_t* dst_slot_dev,
                        int32_t which, int64_t n_tokens, void* stream);

/* Scratch for tq_decode_attn (split partials + rotated queries), bytes; 256-byte aligned buffer. */
int64_t tq_decode_workspace_bytes(int32_t batch, int32_t num_q_heads, int32_t num_kv_heads,
                                  int32_t max_pages_per_seq);
/* A workspace must be initialised once after it is allocated (or be zero-filled): its last 256 KB hold
 * the per-(sequence, KV head) tickets with which the last split to finish elects itself to merge the
 * others, and a status word.  Every call that runs to completion leaves the tickets at zero again; after a
 * call whose status reads 1 (below) re-initialise the workspace before it is used again.  Enqueues one memset. */
int tq_decode_workspace_init(void* workspace_dev, int64_t workspace_bytes, void* stream);
/* After a synchronisation: 0 if every tq_decode_attn / tq_prefill_attn that used this workspace since the
 * previous tq_decode_status_sync finished cleanly, 1 if a bounded wait inside one of those kernels gave up
 * (results of the calls since then are invalid).  The kernels only ever set the word; this call copies it to
 * the host (4 bytes, synchronous) and, when it was set, clears it. */
int tq_decode_status_sync(void* workspace_dev, int64_t workspace_bytes, int32_t* status_out);
/* Self-test of the give-up path (new surface; the reference has no device code): enqueues a one-warp kernel that
 * waits on a barrier nothing arrives at, with a limit of 2^20 SM clocks (about half a millisecond) instead of the
 * attention kernels' 2^30, gives up, and raises this workspace's status word the way those kernels do.  The
 * kernel returns normally and the context stays usable; tq_decode_status_sync then reads 1 once. */
int tq_selftest_wait_gives_up(void* workspace_dev, int64_t workspace_bytes, void* stream);

/* Decode attention straight off the packed cache: for every sequence b and query head h,
 * softmax(q k^T * scale) v over the first seq_lens[b] cached tokens of KV head
 * h / (num_q_heads/num_kv_heads), with k and v the dequantized cache contents -- the
 * dequantize-then-attend computation of the reference's tests (tests/test_kv_cache.py:73-89,
 * 128-131) without materialising the dequantized cache.  Queries are rotated once by the K
 * rotation (and projected by S for PROD formats), scores are taken against centroid values, V is
 * accumulated in its rotated space and un-rotated once per output row.
 *   q_dev [batch][num_q_heads][d] (TQ_F16/TQ_BF16/TQ_F32); out_dev same shape, out_dtype likewise
 *   block_table_dev [batch][max_pages_per_seq] int32 page numbers; seq_lens_dev [batch] int32
 *   scale <= 0 selects 1/sqrt(d). */
int tq_decode_attn(const tq_quantizer* kq, const tq_quantizer* vq, const tq_cache_layout* layout,
                   const uint8_t* pool_dev, const int32_t* block_table_dev, int32_t max_pages_per_seq,
                   const int32_t* seq_lens_dev, const void* q_dev, int32_t q_dtype, int32_t batch,
                   int32_t num_q_heads, float scale, void* workspace_dev, int64_t workspace_bytes,
                   void* out_dev, int32_t out_dtype, void* stream);

/* tq_decode_attn with its launches selectable: phases bit 0 = the dense-rotation query kernel (only
 * launched when the K quantizer has a dense rotation; sign-WHT rotations are applied inside the
 * attention kernel), bit 1 = the attention kernel (split attention, merge by the last split to finish,
 * un-rotation).  3 is tq_decode_attn.  Lets a caller re-run the attention kernel alone (timing, or
 * many layers that share one rotated query); bits run in order against the same workspace.
 * TQ_DECODE_OVERLAP (bit 3) launches the attention kernel with programmatic stream serialization:
 * it may start while the preceding kernel of the stream is still running, and until that kernel has
 * completed it only reads the cache pages, the block table and the sequence lengths (queries are read,
 * the workspace and the output written, afterwards).  Set it only when the preceding kernel writes none of
 * those three -- e.g. the attention call of another layer; after a tq_cache_append into the same pool launch
 * without it. */
#define TQ_DECODE_OVERLAP 8
/* TQ_DECODE_OVERLAP_Q (bits 3 and 6): TQ_DECODE_OVERLAP for a call whose queries the preceding kernel does not
 * write either -- a chain of attention calls whose queries were all produced beforehand (the layers of a
 * benchmark step, the calls over the old and the recent part of a sequence that tq_attn_merge joins).  The
 * kernel then reads its queries and streams its pages while the preceding kernel is still finishing, and waits for
 * it only before its first write (split partials, tickets, output).  Honoured by the kernel for PolarQuant K and V
 * with <= 4 query heads per KV head and a sign-WHT K rotation; elsewhere it means TQ_DECODE_OVERLAP. */
#define TQ_DECODE_OVERLAP_Q (8 | 64)
/* TQ_DECODE_OVERLAP_APPEND (bits 3, 6 and 7): for the attention call that follows the append of the step's new token.
 * The caller states that, of everything this call reads, the preceding kernel writes at most the last cached position
 * of each sequence (slot seq_lens[b] - 1): not the queries, not the block table, not the sequence lengths, no other
 * page.  The kernel then streams every page but the last of each sequence while that kernel is still running,
 * fetches the last page once it has completed, and writes afterwards.  (tq_cache_append and tq_quantize let their
 * dependents start early for this.)  Honoured where TQ_DECODE_OVERLAP_Q is; elsewhere the call runs in stream order. */
#define TQ_DECODE_OVERLAP_APPEND (8 | 64 | 128)
/* TQ_DECODE_CHAIN_HEAD (bit 8): a hint without any effect on the result.  Attention calls launched with
 * TQ_DECODE_OVERLAP_Q follow this call in the stream (it is the first of a chain: the first layer of a decode step
 * whose queries all exist beforehand): the kernel then takes the form those calls take, whose CTAs leave room on
 * an SM for the CTAs of the next call.  Not combined with TQ_DECODE_OVERLAP_APPEND. */
#define TQ_DECODE_CHAIN_HEAD 256
/* TQ_DECODE_SPARSE_V (bit 4): sparse V as in the reference's docs/papers/sparse-v-dequant.md:64-84 -- the V
 * dequantization and accumulation are skipped where the attention weight exp(score - running max) is below 1e-6;
 * here per 16-token tile of a warp (skipped when every weight of the tile, for every query head of the group, is
 * below the threshold).  The weights still count in the softmax denominator.  Off by default: results then differ
 * from dense attention by at most (number of skipped positions) x 1e-6 relative to the largest weight. */
#define TQ_DECODE_SPARSE_V 16
/* TQ_DECODE_NO_DEQUANT (bit 5): measurement only, the "no-dequant ceiling" of the reference's
 * docs/decode-speed-hardware-analysis.md:25-41 -- the kernel copies the same records, runs the same barriers,
 * tensor-core instructions, softmax and merges, but feeds the packed words to the tensor cores instead of
 * looking centroids up.  The outputs are meaningless; the run time is what the kernel would cost if
 * dequantization were free.  Honoured by the kernel for turbo3 K and V with <= 4 query heads per KV head on
 * 128-token pages; other shapes ignore the bit. */
#define TQ_DECODE_NO_DEQUANT 32
int tq_decode_attn_phases(const tq_quantizer* kq, const tq_quantizer* vq, const tq_cache_layout* layout,
                          const uint8_t* pool_dev, const int32_t* block_table_dev,
                          int32_t max_pages_per_seq, const int32_t* seq_lens_dev, const void* q_dev,
                          int32_t q_dtype, int32_t batch, int32_t num_q_heads, float scale,
                          void* workspace_dev, int64_t workspace_bytes, void* out_dev, int32_t out_dtype,
                          int32_t phases, void* stream);

/* tq_decode_attn_phases that also returns, per (sequence, query head), the natural logarithm of the softmax
 * denominator sum_t exp(scale * q.k_t) over the attended tokens (-inf for an empty sequence), and tq_attn_merge,
 * which joins the outputs of two calls over disjoint parts of a sequence: out = (e^la a + e^lb b) / (e^la + e^lb),
 * lse_out = log(e^la + e^lb) (or NULL); rows = batch * num_q_heads rows of 128; out may be one of the inputs.
 * Together they attend over a sequence whose old pages live in another cache at fewer bits (temporal decay,
 * benchmarks/temporal_decay_prototype.py) -- new surface, the reference never runs attention over its caches. */
int tq_decode_attn_lse(const tq_quantizer* kq, const tq_quantizer* vq, const tq_cache_layout* layout,
                       const uint8_t* pool_dev, const int32_t* block_table_dev, int32_t max_pages_per_seq,
                       const int32_t* seq_lens_dev, const void* q_dev, int32_t q_dtype, int32_t batch,
                       int32_t num_q_heads, float scale, void* workspace_dev, int64_t workspace_bytes,
                       void* out_dev, int32_t out_dtype, int32_t phases, float* lse_dev, void* stream);
int tq_attn_merge(const void* out_a_dev, const float* lse_a_dev, const void* out_b_dev, const float* lse_b_dev,
                  int64_t rows, int32_t dtype, void* out_dev, float* lse_out_dev, void* stream);

/* Chunked-prefill attention over the packed cache on the tcgen05 tensor cores: a chunk of
 * `chunk_tokens` new tokens per sequence, whose K/V rows have already been appended, attends
 * causally to the cache: query i of sequence b sits at position kv_lens[b] - chunk_tokens + i and
 * sees the cached tokens 0 .. that position.  Per (sequence, query, head) this is again the
 * reference tests' dequantize-then-attend (tests/test_kv_cache.py:73-89) restricted to the visible
 * prefix; the reference has no chunked or masked variant of its own.
 *   q_dev, out_dev [batch][chunk_tokens][num_q_heads][d]; K and V formats turbo2/3/4; 128-token pages.
 *   The page range of a row block is split over several CTAs when the grid would otherwise not fill
 *   the GPU; the last split to finish folds the partials (ticket, as in tq_decode_attn).
 *   workspace_dev: tq_prefill_workspace_bytes(...) bytes, 256-byte aligned, initialised once with
 *   tq_decode_workspace_init (or zero-filled); same tail layout as the decode workspace, so one
 *   buffer of the larger size serves both; tq_decode_status_sync reads its status word. */
int64_t tq_prefill_workspace_bytes(int32_t batch, int32_t chunk_tokens, int32_t num_q_heads,
                                   int32_t num_kv_heads, int32_t max_pages_per_seq);
int tq_prefill_attn(const tq_quantizer* kq, const tq_quantizer* vq, const tq_cache_layout* layout,
                    const uint8_t* pool_dev, const int32_t* block_table_dev, int32_t max_pages_per_seq,
                    const int32_t* kv_lens_dev, const void* q_dev, int32_t q_dtype, int32_t batch,
                    int32_t chunk_tokens, int32_t num_q_heads, float scale, void* workspace_dev,
                    int64_t workspace_bytes, void* out_dev, int32_t out_dtype, void* stream);

/* ------------------------------------------------------------------------------------------
 * tq_decode_attn_static: tq_decode_attn for callers that cannot allocate device memory.
 * (No counterpart in the reference, which has neither an attention kernel nor device memory.)
 *
 * Who this is for: code that holds device pointers to its inputs and outputs but has no way to
 * obtain a scratch buffer -- a plugin loaded into a serving process whose memory pool already owns
 * all of HBM, a loop that cannot afford the device-wide synchronisation cudaMalloc brings, or a
 * foreign-language host that binds this header and owns no allocator.  Instead of a
 * caller-provided workspace, the split partials and rotated queries go to an array compiled into
 * the library: TQ_DECODE_STATIC_SCRATCH_BYTES (8 MiB) per GPU that loads the library, held until
 * the process exits.  The call itself allocates and frees nothing.
 *
 *   - Shapes whose scratch need (tq_decode_workspace_bytes) exceeds 8 MiB are refused with
 *     TQ_ERR_TOO_LARGE and a message naming both numbers; nothing is launched.  Batch 1 with
 *     32 query heads over 256 pages needs about 0.7 MB; batch 256 with 32 heads does not fit.
 *   - The first call on each device looks up the array's device address (one
 *     cudaGetSymbolAddress, with that device current).  Make that first call before any stream
 *     capture begins on the device.
 *   - All calls on a device share the one array, and it keeps whatever the previous call left.
 *     The kernels do not depend on old contents (every call first clears, with an asynchronous
 *     memset on `stream`, the ticket counters it is going to use, and every partial that is read
 *     was written in the same call), but two calls that overlap on the GPU -- different streams,
 *     or different host threads -- race on it.  Issue calls that use this entry point on one
 *     stream per device, or order them with events.
 *   - tq_decode_static_status_sync reads (and clears) the array's status word the way
 *     tq_decode_status_sync does for a caller-owned workspace: 0 after clean calls, 1 if a bounded
 *     wait inside the kernel gave up since the previous read.  It synchronises (a 4-byte copy).
 *   - Arguments and results are those of tq_decode_attn without workspace_dev/workspace_bytes;
 *     the outputs are bit-identical to tq_decode_attn on the same inputs.
 * ------------------------------------------------------------------------------------------ */
#define TQ_DECODE_STATIC_SCRATCH_BYTES (8 * 1024 * 1024)
int tq_decode_attn_static(const tq_quantizer* kq, const tq_quantizer* vq, const tq_cache_layout* layout,
                          const uint8_t* pool_dev, const int32_t* block_table_dev,
                          int32_t max_pages_per_seq, const int32_t* seq_lens_dev, const void* q_dev,
                          int32_t q_dtype, int32_t batch, int32_t num_q_heads, float scale,
                          void* out_dev, int32_t out_dtype, void* stream);
/* Status word of the built-in scratch array of the current device (no counterpart in the reference). */
int tq_decode_static_status_sync(int32_t* status_out);

#ifdef __cplusplus
}
#endif
#endif /* TQ_B200_H */
