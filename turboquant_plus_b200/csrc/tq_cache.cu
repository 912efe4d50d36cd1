// Quantize-on-append into the paged cache (dispatch over the per-tensor formats).
#include "tq_internal.cuh"

// Slots of the next token of every sequence, for a decode step: sequence b appends at position seq_lens[b], which the
// block table maps to a page.  One launch instead of a chain of elementwise tensor operations in front of the append.
__global__ void k_decode_step_slots(const int32_t* __restrict__ block_table, int32_t max_pages, int32_t* seq_lens,
                                    int32_t page_tokens, int32_t batch, int32_t copies, int64_t copy_stride,
                                    int64_t* __restrict__ slots) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= batch) return;
  const int pos = seq_lens[b];
  const int pg = pos / page_tokens;
  int64_t slot = -1;   // a sequence whose block-table row is full (or whose length is negative) appends nothing
  if (pos >= 0 && pg < max_pages) slot = (int64_t)block_table[(int64_t)b * max_pages + pg] * page_tokens + (pos - pg * page_tokens);
  for (int c = 0; c < copies; ++c) slots[(int64_t)c * batch + b] = slot < 0 ? -1 : slot + c * copy_stride;
  if (slot >= 0) seq_lens[b] = pos + 1;
}

extern "C" int tq_decode_step_slots(const int32_t* block_table_dev, int32_t max_pages_per_seq, int32_t* seq_lens_dev,
                                    int32_t page_tokens, int32_t batch, int32_t copies, int64_t copy_stride,
                                    int64_t* slots_dev, void* stream) {
  TQ_REQUIRE(batch >= 0 && copies >= 1 && page_tokens >= 1 && max_pages_per_seq >= 1, TQ_ERR_INVALID, "bad sizes");
  if (batch == 0) return TQ_OK;
  TQ_REQUIRE(block_table_dev && seq_lens_dev && slots_dev, TQ_ERR_INVALID, "tq_decode_step_slots: null buffer");
  k_decode_step_slots<<<(batch + 127) / 128, 128, 0, (cudaStream_t)stream>>>(block_table_dev, max_pages_per_seq, seq_lens_dev,
                                                                            page_tokens, batch, copies, copy_stride, slots_dev);
  return tq_launch_check("k_decode_step_slots");
}

extern "C" int tq_cache_append(const tq_quantizer* kq, const tq_quantizer* vq, const tq_cache_layout* L,
                               uint8_t* pool_dev, const void* k_dev, const void* v_dev, int32_t dtype, int64_t n_tokens,
                               const int64_t* slot_dev, void* stream) {
  TQ_REQUIRE(L && pool_dev, TQ_ERR_INVALID, "tq_cache_append: layout or pool missing");
  TQ_REQUIRE(n_tokens >= 0, TQ_ERR_INVALID, "n_tokens must be >= 0");
  if (n_tokens == 0) return TQ_OK;
  TQ_REQUIRE(k_dev && v_dev && slot_dev, TQ_ERR_INVALID, "tq_cache_append: k, v or slot mapping missing");
  TQ_REQUIRE(tq_aligned(pool_dev, 128), TQ_ERR_ALIGN, "cache pool must be 128-byte aligned");
  cudaStream_t st = (cudaStream_t)stream;
  const int H = L->num_kv_heads;
  // PolarQuant K and V from 16-bit rows: both tensors in one launch while launches are short enough for their fixed
  // cost to matter (measured: 6.0 vs 5.7 G vectors/s at 65,536 vectors per tensor, 7.6 vs 8.1 at 1,048,576)
  if (n_tokens * H <= 131072 && kq && vq && L->k_format >= TQ_FMT_TURBO2 && L->k_format <= TQ_FMT_TURBO4 && L->v_format == L->k_format &&
      kq->rotation == TQ_ROT_WHT && vq->rotation == TQ_ROT_WHT && kq->d == TQ_D && vq->d == TQ_D &&
      kq->bits == L->k_format && vq->bits == L->v_format) {
    TqQuantDst dk, dv;
    memset(&dk, 0, sizeof(dk));
    dk.slots = slot_dev;
    dk.page_stride = L->page_stride;
    dk.head_stride = L->head_stride;
    dk.page_tokens = L->page_tokens;
    dk.heads = H;
    dv = dk;
    dk.idx = pool_dev + L->k_idx_off;
    dk.scale = reinterpret_cast<float*>(pool_dev + L->k_scale_off);
    dv.idx = pool_dev + L->v_idx_off;
    dv.scale = reinterpret_cast<float*>(pool_dev + L->v_scale_off);
    int rc = TQ_OK;
    if (tq_quantize_mma_try_pair(kq->fast, k_dev, dk, vq->fast, v_dev, dv, dtype, TQ_D, n_tokens * H, st, &rc)) return rc;
  }
  for (int which = 0; which < 2; ++which) {
    const int fmt = which == 0 ? L->k_format : L->v_format;
    const tq_quantizer* q = which == 0 ? kq : vq;
    const void* x = which == 0 ? k_dev : v_dev;
    const int idx_off = which == 0 ? L->k_idx_off : L->v_idx_off;
    const int sc_off = which == 0 ? L->k_scale_off : L->v_scale_off;
    if (fmt == TQ_FMT_Q8_0) {
      int rc = tq_q8_0_append_launch(x, dtype, n_tokens, H, pool_dev + idx_off, pool_dev + sc_off, slot_dev,
                                     L->page_tokens, L->page_stride, L->head_stride, st);
      if (rc != TQ_OK) return rc;
      continue;
    }
    const bool prod = fmt >= TQ_FMT_PROD2;
    const int bits = prod ? fmt - 17 : fmt;
    TQ_REQUIRE(q, TQ_ERR_INVALID, "tq_cache_append: quantizer missing for a turbo/prod tensor");
    TQ_REQUIRE(q->d == TQ_D && q->bits == bits, TQ_ERR_INVALID,
               "quantizer (d=%d, bits=%d) does not match cache format %d", q->d, q->bits, fmt);
    TQ_REQUIRE(!prod || q->qjl, TQ_ERR_INVALID, "PROD cache format needs a quantizer with a QJL stage");
    TQ_REQUIRE(q->rotation == TQ_ROT_WHT, TQ_ERR_UNSUPPORTED,
               "quantize-on-append is built for WHT-mode quantizers (dense mode: quantize, then tq_cache_store)");
    TqQuantDst dst;
    memset(&dst, 0, sizeof(dst));
    dst.idx = pool_dev + idx_off;
    dst.scale = reinterpret_cast<float*>(pool_dev + sc_off);
    if (prod) {
      dst.qjl = pool_dev + L->k_qjl_off;
      dst.rnorm = reinterpret_cast<float*>(pool_dev + L->k_rscale_off);
      dst.rscale_const = 1;
    }
    dst.slots = slot_dev;
    dst.page_stride = L->page_stride;
    dst.head_stride = L->head_stride;
    dst.page_tokens = L->page_tokens;
    dst.heads = H;
    int rc = tq_quantize_wht_launch(q->fast, x, dtype, TQ_D, n_tokens * H, dst, prod, st);
    if (rc != TQ_OK) return rc;
  }
  return TQ_OK;
}
