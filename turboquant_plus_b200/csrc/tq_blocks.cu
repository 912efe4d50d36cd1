// Wire / on-disk codec between the paged cache records and the block formats the reference's documents describe
// for its llama.cpp fork (docs/papers/block-size-experiment.md:25-37, docs/papers/turbo4-resurrection.md:125-138,
// 169, 208):
//   turbo3, storage block of B in {32, 64, 128} elements:  fp16 norm | qs[B/4] | signs[B/8]
//       index of element j = ((qs[j/4] >> ((j%4)*2)) & 3) | (signs[j/8] & (1 << (j%8)) ? 4 : 0)
//       (14 bytes per 32, 50 bytes per 128); every block of one 128-element rotation group carries the same norm,
//       which is the corrected norm ||x|| / ||centroids[idx]|| -- the scale the cache stores
//   turbo2:  fp16 norm | qs[B/4]                      index = (qs[j/4] >> ((j%4)*2)) & 3
//   turbo4, one block per 128 elements, 68 bytes:  fp16 norm | fp16 rnorm (left over from the QJL era, written as 0)
//       | qs[64]                                      index = (qs[j/2] >> ((j%2)*4)) & 15
// The reference tree holds no code for these structs (they live in the fork), so the byte layouts follow the
// documents' extraction expressions and sizes.  The sign vectors of the rotation are not part of a block: caches
// interoperate only between quantizers built with the same signs.
//
// One thread converts 32 elements of one vector: 4*bits bytes (whole words) of the MSB-first index stream on the
// cache side, one storage block (or a quarter / half of one) on the block side.  Pure bit shuffling in registers,
// bound by HBM.
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/tq_b200.h"
#include "tq_internal.cuh"

namespace {

__host__ __device__ inline int blk_bytes(int bits, int B) {
  if (bits == 4) return 4 + B / 2;
  return 2 + B / 4 + (bits == 3 ? B / 8 : 0);
}

struct BlkArgs {
  uint8_t* pool;         // cache pool (read for export, written for import)
  uint8_t* blocks;       // [n_tokens][heads][128/B][block bytes]
  const int64_t* slots;
  int64_t n_tokens, page_stride, head_stride;
  int32_t heads, page_tokens, bits, B, idx_off, scale_off;
};

__device__ __forceinline__ uint32_t bswap32(uint32_t x) { return __byte_perm(x, 0, 0x0123); }

// BITS is a template parameter and every loop is unrolled, so the 32 indices of a thread live in registers; the
// cache side moves as BITS aligned words (4*BITS bytes at a multiple of 4*BITS), the block side as halfwords
// (blocks start on even addresses only: 14- and 50-byte blocks).
template <bool EXPORT, int BITS>
__global__ void __launch_bounds__(256) k_cache_blocks(const BlkArgs a) {
  const int64_t total = a.n_tokens * a.heads * 4;
  const int bb = blk_bytes(BITS, a.B), per_vec = (TQ_D / a.B) * bb;
  constexpr int HDR = BITS == 4 ? 4 : 2;
  for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < total; i += (int64_t)gridDim.x * 256) {
    const int sub = (int)(i & 3);
    const int64_t vec = i >> 2, tok = vec / a.heads;
    const int head = (int)(vec - tok * a.heads);
    const int64_t slot = a.slots[tok];
    const int e0 = 32 * sub, blk = e0 / a.B, e = e0 % a.B;
    uint16_t* bp = reinterpret_cast<uint16_t*>(a.blocks + vec * per_vec + (size_t)blk * bb);
    uint16_t* qs = bp + HDR / 2 + (BITS == 4 ? e / 4 : e / 8);          // 16 (nibbles) or 8 bytes of this thread
    uint16_t* sg = bp + HDR / 2 + a.B / 8 + e / 16;                      // turbo3: 4 bytes of high bits
    if (slot < 0) {
      if (EXPORT) {  // a skipped token leaves zero blocks
        if (e == 0) { bp[0] = 0; if (BITS == 4) bp[1] = 0; }
#pragma unroll
        for (int k = 0; k < (BITS == 4 ? 8 : 4); ++k) qs[k] = 0;
        if (BITS == 3) { sg[0] = 0; sg[1] = 0; }
      }
      continue;
    }
    const int64_t page = slot / a.page_tokens;
    const int off = (int)(slot - page * a.page_tokens);
    uint8_t* rec = a.pool + page * a.page_stride + (int64_t)head * a.head_stride;
    uint32_t* stream = reinterpret_cast<uint32_t*>(rec + a.idx_off + (size_t)off * (16 * BITS)) + sub * BITS;
    float* scale = reinterpret_cast<float*>(rec + a.scale_off) + off;
    uint32_t idx[32];
    if (EXPORT) {
      uint32_t w[BITS];
#pragma unroll
      for (int k = 0; k < BITS; ++k) w[k] = bswap32(stream[k]);       // 32*BITS bits, first index in the top bits
#pragma unroll
      for (int k = 0; k < 32; ++k) {
        const int start = k * BITS, wi = start >> 5, o = start & 31;
        uint32_t m;
        if (o + BITS <= 32) m = w[wi] >> (32 - BITS - o);
        else m = __funnelshift_l(w[wi + 1 < BITS ? wi + 1 : wi], w[wi], o + BITS - 32);
        idx[k] = m & ((1u << BITS) - 1u);
      }
      if (e == 0) {
        const __half hs = __float2half_rn(*scale);
        bp[0] = *reinterpret_cast<const uint16_t*>(&hs);
        if (BITS == 4) bp[1] = 0;
      }
      if (BITS == 4) {
#pragma unroll
        for (int k = 0; k < 8; ++k)
          qs[k] = (uint16_t)(idx[4 * k] | (idx[4 * k + 1] << 4) | (idx[4 * k + 2] << 8) | (idx[4 * k + 3] << 12));
      } else {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          uint32_t v = 0;
#pragma unroll
          for (int j = 0; j < 8; ++j) v |= (idx[8 * k + j] & 3u) << (2 * j);
          qs[k] = (uint16_t)v;
        }
        if (BITS == 3) {
#pragma unroll
          for (int k = 0; k < 2; ++k) {
            uint32_t v = 0;
#pragma unroll
            for (int j = 0; j < 16; ++j) v |= ((idx[16 * k + j] >> 2) & 1u) << j;
            sg[k] = (uint16_t)v;
          }
        }
      }
    } else {
      if (BITS == 4) {
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint32_t v = qs[k];
#pragma unroll
          for (int j = 0; j < 4; ++j) idx[4 * k + j] = (v >> (4 * j)) & 15u;
        }
      } else {
        uint32_t hi = 0;
        if (BITS == 3) hi = (uint32_t)sg[0] | ((uint32_t)sg[1] << 16);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const uint32_t v = qs[k];
#pragma unroll
          for (int j = 0; j < 8; ++j) idx[8 * k + j] = ((v >> (2 * j)) & 3u) | (((hi >> (8 * k + j)) & 1u) << 2);
        }
      }
      uint32_t w[BITS];
#pragma unroll
      for (int k = 0; k < BITS; ++k) w[k] = 0;
#pragma unroll
      for (int k = 0; k < 32; ++k) {
        const int start = k * BITS, wi = start >> 5, o = start & 31;
        if (o + BITS <= 32) {
          w[wi] |= idx[k] << (32 - BITS - o);
        } else {
          w[wi] |= idx[k] >> (o + BITS - 32);
          if (wi + 1 < BITS) w[wi + 1] |= idx[k] << (64 - BITS - o);
        }
      }
#pragma unroll
      for (int k = 0; k < BITS; ++k) stream[k] = bswap32(w[k]);
      if (sub == 0) {
        const uint16_t raw = *reinterpret_cast<const uint16_t*>(a.blocks + vec * per_vec);
        *scale = __half2float(*reinterpret_cast<const __half*>(&raw));
      }
    }
  }
}

int run_blocks(bool exp, const tq_cache_layout* L, uint8_t* pool, int32_t which, const int64_t* slot_dev,
               int64_t n_tokens, int32_t block_elems, uint8_t* blocks, void* stream) {
  TQ_REQUIRE(L, TQ_ERR_INVALID, "block codec: layout is null");
  TQ_REQUIRE(which == 0 || which == 1, TQ_ERR_INVALID, "which must be 0 (K) or 1 (V)");
  TQ_REQUIRE(n_tokens >= 0, TQ_ERR_INVALID, "n_tokens must be >= 0");
  TQ_REQUIRE(n_tokens == 0 || (pool && slot_dev), TQ_ERR_INVALID, "block codec: null argument");
  const int fmt = which == 0 ? L->k_format : L->v_format;
  TQ_REQUIRE(fmt == TQ_FMT_TURBO2 || fmt == TQ_FMT_TURBO3 || fmt == TQ_FMT_TURBO4, TQ_ERR_UNSUPPORTED,
             "block formats exist for turbo2 / turbo3 / turbo4 tensors, got format %d", fmt);
  const int bits = fmt == TQ_FMT_TURBO2 ? 2 : fmt == TQ_FMT_TURBO3 ? 3 : 4;
  TQ_REQUIRE(block_elems == 32 || block_elems == 64 || block_elems == 128, TQ_ERR_INVALID,
             "storage block must hold 32, 64 or 128 elements, got %d", block_elems);
  TQ_REQUIRE(bits != 4 || block_elems == 128, TQ_ERR_UNSUPPORTED, "turbo4 blocks hold 128 elements");
  if (n_tokens == 0) return TQ_OK;
  TQ_REQUIRE(blocks, TQ_ERR_INVALID, "block codec: block buffer is null");
  TQ_REQUIRE(tq_aligned(blocks, 2) && tq_aligned(pool, 128), TQ_ERR_ALIGN, "block codec: misaligned buffer");
  BlkArgs a;
  a.pool = pool;
  a.blocks = blocks;
  a.slots = slot_dev;
  a.n_tokens = n_tokens;
  a.page_stride = L->page_stride;
  a.head_stride = L->head_stride;
  a.heads = L->num_kv_heads;
  a.page_tokens = L->page_tokens;
  a.bits = bits;
  a.B = block_elems;
  a.idx_off = which == 0 ? L->k_idx_off : L->v_idx_off;
  a.scale_off = which == 0 ? L->k_scale_off : L->v_scale_off;
  const int64_t total = n_tokens * L->num_kv_heads * 4;
  int64_t g = (total + 255) / 256;
  const int64_t cap = (int64_t)tq_num_sms() * 16;
  if (g > cap) g = cap;
#define TQ_BLK(E, B_) k_cache_blocks<E, B_><<<(int)g, 256, 0, (cudaStream_t)stream>>>(a)
  if (exp) {
    if (bits == 2) TQ_BLK(true, 2); else if (bits == 3) TQ_BLK(true, 3); else TQ_BLK(true, 4);
  } else {
    if (bits == 2) TQ_BLK(false, 2); else if (bits == 3) TQ_BLK(false, 3); else TQ_BLK(false, 4);
  }
#undef TQ_BLK
  return tq_launch_check("k_cache_blocks");
}

}  // namespace

extern "C" int64_t tq_block_bytes(int32_t format, int32_t block_elems) {
  const int bits = format == TQ_FMT_TURBO2 ? 2 : format == TQ_FMT_TURBO3 ? 3 : format == TQ_FMT_TURBO4 ? 4 : 0;
  if (!bits || (block_elems != 32 && block_elems != 64 && block_elems != 128) || (bits == 4 && block_elems != 128))
    return -1;
  return blk_bytes(bits, block_elems);
}

extern "C" int tq_cache_export_blocks(const tq_cache_layout* layout, const uint8_t* pool_dev, int32_t which,
                                      const int64_t* slot_dev, int64_t n_tokens, int32_t block_elems,
                                      uint8_t* out_dev, void* stream) {
  return run_blocks(true, layout, const_cast<uint8_t*>(pool_dev), which, slot_dev, n_tokens, block_elems, out_dev, stream);
}

extern "C" int tq_cache_import_blocks(const tq_cache_layout* layout, uint8_t* pool_dev, int32_t which,
                                      const int64_t* slot_dev, int64_t n_tokens, int32_t block_elems,
                                      const uint8_t* in_dev, void* stream) {
  return run_blocks(false, layout, pool_dev, which, slot_dev, n_tokens, block_elems, const_cast<uint8_t*>(in_dev), stream);
}
