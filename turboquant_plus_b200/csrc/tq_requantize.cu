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

__device__ __forceinline__ float rq_sum8(float v) {
  v += __shfl_xor_sync(0xffffffffu, v, 1);
  v += __shfl_xor_sync(0xffffffffu, v, 2);
  v += __shfl_xor_sync(0xffffffffu, v, 4);
  return v;
}

template <int BS, int BD>
__global__ void __launch_bounds__(256) k_requantize(const RqTables T, const uint8_t* __restrict__ src,
                                                    const float* __restrict__ scale_src, int64_t n,
                                                    int scale_is_norm, uint8_t* __restrict__ dst,
                                                    float* __restrict__ norm_dst, float* __restrict__ scale_dst) {
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
    const bool ok = v < n;
    // this lane's 16 fields: BS halfwords of the big-endian stream, first coordinate in the top bits
    uint64_t word = 0;
    if (ok) {
      const uint16_t* p = reinterpret_cast<const uint16_t*>(src + v * (16 * BS) + sub * 2 * BS);
#pragma unroll
      for (int i = 0; i < BS; ++i) word = (word << 16) | (uint64_t)__byte_perm((uint32_t)p[i], 0, 0x4401);
    }
    float sc = ok ? scale_src[v] : 0.f;
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
      uint16_t* q = reinterpret_cast<uint16_t*>(dst + v * (16 * BD) + sub * 2 * BD);
#pragma unroll
      for (int i = 0; i < BD; ++i)
        q[i] = (uint16_t)__byte_perm((uint32_t)(out >> (16 * (BD - 1 - i))), 0, 0x4401);
      if (sub == 0) {
        if (norm_dst) norm_dst[v] = recon;
        scale_dst[v] = cn > 1e-10f ? recon / cn : recon;
      }
    }
  }
}

}  // namespace

extern "C" int tq_requantize(const tq_quantizer* src_q, const tq_quantizer* dst_q, const uint8_t* packed_src_dev,
                             const float* scale_src_dev, int32_t scale_is_norm, int64_t n, uint8_t* packed_dst_dev,
                             float* norm_dst_dev, float* scale_dst_dev, void* stream) {
  TQ_REQUIRE(src_q && dst_q, TQ_ERR_INVALID, "tq_requantize: quantizer is null");
  TQ_REQUIRE(src_q->rotation == TQ_ROT_WHT && dst_q->rotation == TQ_ROT_WHT, TQ_ERR_UNSUPPORTED,
             "tq_requantize works on sign-WHT (d = 128) codes");
  TQ_REQUIRE(memcmp(src_q->fast.s1, dst_q->fast.s1, sizeof(src_q->fast.s1)) == 0 &&
                 memcmp(src_q->fast.s2, dst_q->fast.s2, sizeof(src_q->fast.s2)) == 0,
             TQ_ERR_INVALID, "tq_requantize: source and destination must share the rotation (same sign vectors)");
  TQ_REQUIRE(dst_q->bits <= src_q->bits, TQ_ERR_INVALID, "tq_requantize: destination width %d exceeds source width %d",
             dst_q->bits, src_q->bits);
  TQ_REQUIRE(n >= 0, TQ_ERR_INVALID, "tq_requantize: n must be >= 0");
  if (n == 0) return TQ_OK;
  TQ_REQUIRE(packed_src_dev && scale_src_dev && packed_dst_dev && scale_dst_dev, TQ_ERR_INVALID,
             "tq_requantize: null buffer");
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
  TQ_REQUIRE(tq_aligned(packed_src_dev, 2) && tq_aligned(packed_dst_dev, 2), TQ_ERR_ALIGN,
             "tq_requantize: index streams must be 2-byte aligned");
#define TQ_RQ(S, D_)                                                                                              \
  k_requantize<S, D_><<<grid, 256, 0, (cudaStream_t)stream>>>(T, packed_src_dev, scale_src_dev, n,              \
                                                               scale_is_norm ? 1 : 0, packed_dst_dev, norm_dst_dev, \
                                                               scale_dst_dev)
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
