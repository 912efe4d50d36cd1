// Temporal decay: re-quantize stored PolarQuant codes to a narrower codebook without leaving the rotated domain
// (requantize_3to2 of benchmarks/temporal_decay_prototype.py:93-125, for any pair of widths 1..4 bits).
//
// Per vector: values = centroids_src[idx] * scale_src; recon = ||values||; unit = values / recon (values themselves when
// recon <= 1e-10); idx_dst = number of destination midpoints <= unit (np.digitize: a tie goes to the upper cell);
// scale_dst = recon / ||centroids_dst[idx_dst]|| (recon itself when that norm is <= 1e-10).  Source and destination
// share the rotation, so no transform runs: the kernel streams (16*bits_src + 4) bytes in and (16*bits_dst + 8) out
// per vector and is bound by HBM.
//
// Layout of the work: 8 lanes per vector, 16 coordinates per lane (2*bits bytes of the MSB-first index stream, which
// start on a 2-byte boundary and are read as halfwords), 4 vectors per warp; the two sums of squares are reduced over the 8 lanes with shuffles.
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include "../../include/tq_b200.h"
#include "tq_internal.cuh"

namespace {

struct RqTables {
  float cent_src[16];
  float cent_dst[16];
  float mid_dst[15];
  int32_t bits_src, bits_dst;
};

// Where vector v lives.  Flat: row v of a dense (n, 16*bits) stream and entry v of a scale array.  Paged: vector
// v = (token, head) of a cache pool, the token's place given by a slot (page * page_tokens + offset; negative = skip).
struct RqSide {
  uint8_t* base;          // flat: index stream; paged: pool + offset of the index array inside a record
  float* scale;           // flat: scale array;  paged: pool + offset of the scale array inside a record (as bytes)
  const int64_t* slots;   // null: flat
  int64_t page_stride, head_stride;
  int32_t heads, page_tokens;
};

template <int BITS>
__device__ __forceinline__ bool rq_locate(const RqSide& S, int64_t v, uint8_t*& idx, float*& scale) {
  if (!S.slots) {
    idx = S.base + v * (16 * BITS);
    scale = S.scale + v;
    return true;
  }
  const int64_t tok = v / S.heads, slot = S.slots[tok];
  if (slot < 0) return false;
  const int head = (int)(v - tok * S.heads);
  const int64_t page = slot / S.page_tokens, off = slot - page * S.page_tokens;
  const int64_t rec = page * S.page_stride + (int64_t)head * S.head_stride;
  idx = S.base + rec + off * (16 * BITS);
  scale = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(S.scale) + rec) + off;
  return true;
}

__device__ __forceinline__ float rq_sum8(float v) {
  v += __shfl_xor_sync(0xffffffffu, v, 1);
  v += __shfl_xor_sync(0xffffffffu, v, 2);
  v += __shfl_xor_sync(0xffffffffu, v, 4);
  return v;
}

template <int BS, int BD>
__global__ void __launch_bounds__(256) k_requantize(const RqTables T, const RqSide src, const RqSide dst, int64_t n,
                                                    int scale_is_norm, float* __restrict__ norm_dst) {
  // codebooks in shared memory: the lanes of a warp look up different entries, which the constant bank serialises
  __shared__ float s_src[16], s_dst[16];
  if (threadIdx.x < 16) {
    s_src[threadIdx.x] = T.cent_src[threadIdx.x];
    s_dst[threadIdx.x] = T.cent_dst[threadIdx.x];
  }
  __syncthreads();
  float mid[(1 << BD) - 1];
#pragma unroll
  for (int i = 0; i < (1 << BD) - 1; ++i) mid[i] = T.mid_dst[i];
  const int lane = threadIdx.x & 31, sub = lane & 7;
  const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t v0 = warp * 4; v0 < n; v0 += nwarps * 4) {  // n is uniform, so whole warps leave together
    const int64_t v = v0 + (lane >> 3);
    uint8_t *sp = nullptr, *dp = nullptr;
    float *ssc = nullptr, *dsc = nullptr;
    const bool ok = v < n && rq_locate<BS>(src, v, sp, ssc) && rq_locate<BD>(dst, v, dp, dsc);
    // this lane's 16 fields: BS halfwords of the big-endian stream, first coordinate in the top bits
    uint64_t word = 0;
    if (ok) {
      const uint16_t* p = reinterpret_cast<const uint16_t*>(sp + sub * 2 * BS);
#pragma unroll
      for (int i = 0; i < BS; ++i) word = (word << 16) | (uint64_t)__byte_perm((uint32_t)p[i], 0, 0x4401);
    }
    float sc = ok ? *ssc : 0.f;
    float val[16], ss = 0.f;
#pragma unroll
    for (int k = 0; k < 16; ++k) {
      const uint32_t m = (uint32_t)(word >> (BS * (15 - k))) & ((1u << BS) - 1u);
      val[k] = s_src[m];
      ss = fmaf(val[k], val[k], ss);
    }
    if (scale_is_norm) {  // the prototype's dequantize_3bit: norm / ||centroids[idx]||
      const float cn0 = sqrtf(rq_sum8(ss));
      sc = cn0 > 1e-10f ? sc / cn0 : sc;
    }
    ss = 0.f;
#pragma unroll
    for (int k = 0; k < 16; ++k) {
      val[k] *= sc;
      ss = fmaf(val[k], val[k], ss);
    }
    float recon = sqrtf(rq_sum8(ss));
    const bool tiny = !(recon > 1e-10f);
    const float inv = tiny ? 1.f : 1.f / recon;
    if (tiny) recon = 0.f;
    uint64_t out = 0;
    float cc = 0.f;
#pragma unroll
    for (int k = 0; k < 16; ++k) {
      const float u = tiny ? val[k] : val[k] * inv;
      int m = 0;
#pragma unroll
      for (int b = 0; b < (1 << BD) - 1; ++b) m += (mid[b] <= u) ? 1 : 0;
      out = (out << BD) | (uint64_t)m;
      const float c = s_dst[m];
      cc = fmaf(c, c, cc);
    }
    const float cn = sqrtf(rq_sum8(cc));
    if (ok) {
      uint16_t* q = reinterpret_cast<uint16_t*>(dp + sub * 2 * BD);
#pragma unroll
      for (int i = 0; i < BD; ++i)
        q[i] = (uint16_t)__byte_perm((uint32_t)(out >> (16 * (BD - 1 - i))), 0, 0x4401);
      if (sub == 0) {
        if (norm_dst) norm_dst[v] = recon;
        *dsc = cn > 1e-10f ? recon / cn : recon;
      }
    }
  }
}

}  // namespace

static int rq_launch(const tq_quantizer* src_q, const tq_quantizer* dst_q, const RqSide& src, const RqSide& dst, int64_t n,
                     int32_t scale_is_norm, float* norm_dst_dev, void* stream) {
  TQ_REQUIRE(src_q && dst_q, TQ_ERR_INVALID, "tq_requantize: quantizer is null");
  TQ_REQUIRE(src_q->rotation == TQ_ROT_WHT && dst_q->rotation == TQ_ROT_WHT, TQ_ERR_UNSUPPORTED,
             "tq_requantize works on sign-WHT (d = 128) codes");
  TQ_REQUIRE(memcmp(src_q->fast.s1, dst_q->fast.s1, sizeof(src_q->fast.s1)) == 0 &&
                 memcmp(src_q->fast.s2, dst_q->fast.s2, sizeof(src_q->fast.s2)) == 0,
             TQ_ERR_INVALID, "tq_requantize: source and destination must share the rotation (same sign vectors)");
  TQ_REQUIRE(dst_q->bits <= src_q->bits, TQ_ERR_INVALID, "tq_requantize: destination width %d exceeds source width %d",
             dst_q->bits, src_q->bits);
  RqTables T;
  memset(&T, 0, sizeof(T));
  T.bits_src = src_q->bits;
  T.bits_dst = dst_q->bits;
  for (int i = 0; i < (1 << T.bits_src); ++i) T.cent_src[i] = src_q->fast.cent[i];
  for (int i = 0; i < (1 << T.bits_dst); ++i) T.cent_dst[i] = dst_q->fast.cent[i];
  for (int i = 0; i + 1 < (1 << T.bits_dst); ++i) T.mid_dst[i] = dst_q->fast.bnd[i];
  const int64_t warps = (n + 3) / 4;
  const int64_t want = (warps + 7) / 8;
  const int64_t cap = (int64_t)tq_num_sms() * 8;
  const int grid = (int)(want < cap ? want : cap);
#define TQ_RQ(S, D_) \
  k_requantize<S, D_><<<grid, 256, 0, (cudaStream_t)stream>>>(T, src, dst, n, scale_is_norm ? 1 : 0, norm_dst_dev)
  switch (T.bits_src * 8 + T.bits_dst) {
    case 4 * 8 + 4: TQ_RQ(4, 4); break;
    case 4 * 8 + 3: TQ_RQ(4, 3); break;
    case 4 * 8 + 2: TQ_RQ(4, 2); break;
    case 4 * 8 + 1: TQ_RQ(4, 1); break;
    case 3 * 8 + 3: TQ_RQ(3, 3); break;
    case 3 * 8 + 2: TQ_RQ(3, 2); break;
    case 3 * 8 + 1: TQ_RQ(3, 1); break;
    case 2 * 8 + 2: TQ_RQ(2, 2); break;
    case 2 * 8 + 1: TQ_RQ(2, 1); break;
    default: TQ_RQ(1, 1); break;
  }
#undef TQ_RQ
  return tq_launch_check("k_requantize");
}

extern "C" int tq_requantize(const tq_quantizer* src_q, const tq_quantizer* dst_q, const uint8_t* packed_src_dev,
                             const float* scale_src_dev, int32_t scale_is_norm, int64_t n, uint8_t* packed_dst_dev,
                             float* norm_dst_dev, float* scale_dst_dev, void* stream) {
  TQ_REQUIRE(n >= 0, TQ_ERR_INVALID, "tq_requantize: n must be >= 0");
  if (n == 0) return TQ_OK;
  TQ_REQUIRE(packed_src_dev && scale_src_dev && packed_dst_dev && scale_dst_dev, TQ_ERR_INVALID,
             "tq_requantize: null buffer");
  TQ_REQUIRE(tq_aligned(packed_src_dev, 2) && tq_aligned(packed_dst_dev, 2), TQ_ERR_ALIGN,
             "tq_requantize: index streams must be 2-byte aligned");
  RqSide src, dst;
  memset(&src, 0, sizeof(src));
  memset(&dst, 0, sizeof(dst));
  src.base = const_cast<uint8_t*>(packed_src_dev);
  src.scale = const_cast<float*>(scale_src_dev);
  dst.base = packed_dst_dev;
  dst.scale = scale_dst_dev;
  return rq_launch(src_q, dst_q, src, dst, n, scale_is_norm, norm_dst_dev, stream);
}

extern "C" int tq_cache_requantize(const tq_quantizer* src_q, const tq_quantizer* dst_q, const tq_cache_layout* src_layout,
                                   const uint8_t* src_pool_dev, const int64_t* src_slot_dev,
                                   const tq_cache_layout* dst_layout, uint8_t* dst_pool_dev, const int64_t* dst_slot_dev,
                                   int32_t which, int64_t n_tokens, void* stream) {
  TQ_REQUIRE(src_layout && dst_layout, TQ_ERR_INVALID, "tq_cache_requantize: layout is null");
  TQ_REQUIRE(which == 0 || which == 1, TQ_ERR_INVALID, "which must be 0 (K) or 1 (V)");
  TQ_REQUIRE(n_tokens >= 0, TQ_ERR_INVALID, "n_tokens must be >= 0");
  TQ_REQUIRE(n_tokens == 0 || (src_pool_dev && dst_pool_dev && src_slot_dev && dst_slot_dev), TQ_ERR_INVALID,
             "tq_cache_requantize: null argument");
  TQ_REQUIRE(src_layout->num_kv_heads == dst_layout->num_kv_heads, TQ_ERR_INVALID,
             "tq_cache_requantize: the caches differ in KV heads");
  const int sf = which == 0 ? src_layout->k_format : src_layout->v_format;
  const int df = which == 0 ? dst_layout->k_format : dst_layout->v_format;
  TQ_REQUIRE(sf >= TQ_FMT_TURBO2 && sf <= TQ_FMT_TURBO4 && df >= TQ_FMT_TURBO2 && df <= TQ_FMT_TURBO4, TQ_ERR_UNSUPPORTED,
             "tq_cache_requantize converts turbo2 / turbo3 / turbo4 tensors, got formats %d -> %d", sf, df);
  TQ_REQUIRE(src_q && dst_q && src_q->bits == sf && dst_q->bits == df, TQ_ERR_INVALID,
             "tq_cache_requantize: quantizer widths do not match the cache formats");
  if (n_tokens == 0) return TQ_OK;
  RqSide src, dst;
  src.base = const_cast<uint8_t*>(src_pool_dev) + (which == 0 ? src_layout->k_idx_off : src_layout->v_idx_off);
  src.scale = reinterpret_cast<float*>(const_cast<uint8_t*>(src_pool_dev) +
                                       (which == 0 ? src_layout->k_scale_off : src_layout->v_scale_off));
  src.slots = src_slot_dev;
  src.page_stride = src_layout->page_stride;
  src.head_stride = src_layout->head_stride;
  src.heads = src_layout->num_kv_heads;
  src.page_tokens = src_layout->page_tokens;
  dst.base = dst_pool_dev + (which == 0 ? dst_layout->k_idx_off : dst_layout->v_idx_off);
  dst.scale = reinterpret_cast<float*>(dst_pool_dev + (which == 0 ? dst_layout->k_scale_off : dst_layout->v_scale_off));
  dst.slots = dst_slot_dev;
  dst.page_stride = dst_layout->page_stride;
  dst.head_stride = dst_layout->head_stride;
  dst.heads = dst_layout->num_kv_heads;
  dst.page_tokens = dst_layout->page_tokens;
  return rq_launch(src_q, dst_q, src, dst, n_tokens * src_layout->num_kv_heads, 0, nullptr, stream);
}
