// Dequantize kernels (API parity and debugging; the attention kernels never materialise this).
#include "tq_internal.cuh"

// ------------------------------------------------------------------------------------------
// d = 128, WHT rotation: x_hat = D1 (H/sqrt d) D2 (scale * centroids[idx])  [+ QJL term]
// ------------------------------------------------------------------------------------------
template <int BITS>
__device__ __forceinline__ void tq_unpack16(const uint8_t* p, uint32_t (&idx)[16]) {
  // p points at 2*BITS bytes holding 16 indices MSB first
  uint32_t w0 = 0, w1 = 0;
#pragma unroll
  for (int j = 0; j < BITS; ++j) {
    w0 = (w0 << 8) | p[j];
    w1 = (w1 << 8) | p[BITS + j];
  }
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    idx[k] = (w0 >> (BITS * (7 - k))) & ((1u << BITS) - 1);
    idx[8 + k] = (w1 >> (BITS * (7 - k))) & ((1u << BITS) - 1);
  }
}

template <typename Tout> struct TqStore16;
template <> struct TqStore16<float> {
  static __device__ __forceinline__ void store(float* p, const float (&x)[16]) {
    float4* p4 = reinterpret_cast<float4*>(p);
#pragma unroll
    for (int i = 0; i < 4; ++i) p4[i] = make_float4(x[4 * i], x[4 * i + 1], x[4 * i + 2], x[4 * i + 3]);
  }
};
template <> struct TqStore16<__half> {
  static __device__ __forceinline__ void store(__half* p, const float (&x)[16]) {
    uint4* p4 = reinterpret_cast<uint4*>(p);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      uint4 v;
      __half2* h = reinterpret_cast<__half2*>(&v);
#pragma unroll
      for (int j = 0; j < 4; ++j) h[j] = __floats2half2_rn(x[8 * i + 2 * j], x[8 * i + 2 * j + 1]);
      p4[i] = v;
    }
  }
};

template <typename Tout, int BITS>
__global__ void __launch_bounds__(256) k_dequantize_wht(const TqFast f, const uint8_t* __restrict__ packed,
                                                        const uint8_t* __restrict__ idx_u8,
                                                        const float* __restrict__ norm,
                                                        const uint8_t* __restrict__ qjl,
                                                        const float* __restrict__ rnorm, float shrink, int64_t n,
                                                        Tout* __restrict__ out) {
  __shared__ float lut[16];
  if (threadIdx.x < 16) lut[threadIdx.x] = f.cent[threadIdx.x];
  __syncthreads();
  const int lane = threadIdx.x & 31, sub = lane & 7;
  const uint32_t b1 = tq_lane_bits16(f.s1, sub), b2 = tq_lane_bits16(f.s2, sub);
  const uint32_t bj1 = tq_lane_bits16(f.j1, sub), bj2 = tq_lane_bits16(f.j2, sub);
  for (int64_t v = ((int64_t)blockIdx.x * 256 + threadIdx.x) >> 3; v < (n + 3) / 4 * 4;
       v += (int64_t)gridDim.x * 32) {
    const bool ok = v < n;
    uint32_t idx[16];
    if (ok) {
      if (packed) {
        tq_unpack16<BITS>(packed + v * (16 * BITS) + sub * 2 * BITS, idx);
      } else {
        const uint4 w = *reinterpret_cast<const uint4*>(idx_u8 + v * TQ_D + sub * 16);
        const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
        for (int k = 0; k < 16; ++k) idx[k] = (ww[k >> 2] >> (8 * (k & 3))) & ((1u << BITS) - 1);
      }
    } else {
#pragma unroll
      for (int k = 0; k < 16; ++k) idx[k] = 0;
    }
    float y[16];
    float cc = 0.f;
#pragma unroll
    for (int k = 0; k < 16; ++k) {
      y[k] = lut[idx[k]];
      cc = fmaf(y[k], y[k], cc);
    }
    cc = tq_sum8(cc);
    float sc = ok ? norm[v] : 0.f;
    if (f.norm_correction) {
      float cn = sqrtf(cc);
      cn = cn > 1e-10f ? cn : 1.0f;
      sc = sc / cn;
    }
    sc *= TQ_RSQRT_D;
#pragma unroll
    for (int k = 0; k < 16; ++k) y[k] = tq_flip(y[k] * sc, b2, k);
    tq_wht16_regs(y);
    tq_wht128_lanes(y, sub);
#pragma unroll
    for (int k = 0; k < 16; ++k) y[k] = tq_flip(y[k], b1, k);
    if (qjl) {
      // shrinkage * sqrt(pi/2)/sqrt(d) * ||r|| * S^T z, S^T = J1 (H/sqrt d) J2
      const uint32_t zb = ok ? (((uint32_t)qjl[v * 16 + sub * 2] << 8) | qjl[v * 16 + sub * 2 + 1]) : 0u;
      const float g = ok ? shrink * (1.2533141373155001f * TQ_RSQRT_D) * rnorm[v] * TQ_RSQRT_D : 0.f;
      float z[16];
#pragma unroll
      for (int k = 0; k < 16; ++k) z[k] = tq_flip(((zb >> (15 - k)) & 1u) ? g : -g, bj2, k);
      tq_wht16_regs(z);
      tq_wht128_lanes(z, sub);
#pragma unroll
      for (int k = 0; k < 16; ++k) y[k] += tq_flip(z[k], bj1, k);
    }
    if (ok) TqStore16<Tout>::store(out + v * TQ_D + sub * 16, y);
  }
}

// ------------------------------------------------------------------------------------------
// any d, dense rotation, fp64: x_hat = norm * R^T yhat' + shrink * sqrt(pi/2)/sqrt(d) * gamma * S^T z
// ------------------------------------------------------------------------------------------
constexpr int DV = 8;

template <typename T> __device__ __forceinline__ T tq_from_double(double v);
template <> __device__ __forceinline__ double tq_from_double<double>(double v) { return v; }
template <> __device__ __forceinline__ float tq_from_double<float>(double v) { return (float)v; }
template <> __device__ __forceinline__ __half tq_from_double<__half>(double v) { return __float2half_rn((float)v); }

__device__ __forceinline__ double tq_as_double(double v) { return v; }
__device__ __forceinline__ double tq_as_double(float v) { return (double)v; }
__device__ __forceinline__ double tq_as_double(__half v) { return (double)__half2float(v); }

template <typename Tout>
__global__ void __launch_bounds__(128) k_dequantize_dense(const double* __restrict__ rot, const double* __restrict__ s,
                                                          const double* __restrict__ cent, int d, int bits,
                                                          int norm_correction, const uint8_t* __restrict__ packed,
                                                          const uint8_t* __restrict__ idx_u8,
                                                          const float* __restrict__ norm,
                                                          const uint8_t* __restrict__ qjl,
                                                          const float* __restrict__ rnorm, double shrink, int64_t n,
                                                          Tout* __restrict__ out, int64_t ld_out, int accumulate) {
  extern __shared__ __align__(16) double sm[];
  double* ys = sm;                    // [d][DV]
  double* zs = sm + (size_t)d * DV;   // [d][DV] (QJL signs scaled), only when qjl
  __shared__ double s_red[DV];
  const int tid = threadIdx.x;
  const int64_t v0 = (int64_t)blockIdx.x * DV;
  const int nv = (int)((n - v0) < DV ? (n - v0) : DV);
  if (tid < DV) s_red[tid] = 0.0;
  __syncthreads();
  double part[DV];
#pragma unroll
  for (int v = 0; v < DV; ++v) part[v] = 0.0;
  const int bpv = d * bits / 8, rb = (d + 7) / 8;
  for (int i = tid; i < d * DV; i += 128) {
    const int v = i % DV, k = i / DV;
    double c = 0.0, z = 0.0;
    if (v < nv) {
      uint32_t m;
      if (packed) {
        m = 0;
        for (int r = 0; r < bits; ++r) {
          const int pos = k * bits + r;
          m = (m << 1) | ((packed[(v0 + v) * bpv + (pos >> 3)] >> (7 - (pos & 7))) & 1u);
        }
      } else {
        m = idx_u8[(v0 + v) * d + k];
      }
      c = cent[m];
      if (qjl) z = ((qjl[(v0 + v) * rb + (k >> 3)] >> (7 - (k & 7))) & 1u) ? 1.0 : -1.0;
    }
    ys[i] = c;
    if (qjl) zs[i] = z;
#pragma unroll
    for (int vv = 0; vv < DV; ++vv)
      if (vv == v) part[vv] += c * c;
  }
#pragma unroll
  for (int v = 0; v < DV; ++v) atomicAdd(&s_red[v], part[v]);
  __syncthreads();
  const double qc = shrink * 1.2533141373155001 / sqrt((double)d);  // turboquant/qjl.py:131-132
  for (int j = tid; j < d; j += 128) {
    double acc[DV], acz[DV];
#pragma unroll
    for (int v = 0; v < DV; ++v) acc[v] = 0.0, acz[v] = 0.0;
    for (int k = 0; k < d; ++k) {
      const double r = __ldg(rot + (size_t)k * d + j);
      const double2* yv = reinterpret_cast<const double2*>(ys + (size_t)k * DV);
#pragma unroll
      for (int h = 0; h < DV / 2; ++h) {
        const double2 p = yv[h];
        acc[2 * h] = fma(r, p.x, acc[2 * h]);
        acc[2 * h + 1] = fma(r, p.y, acc[2 * h + 1]);
      }
      if (qjl) {
        const double sv = __ldg(s + (size_t)k * d + j);
        const double2* zv = reinterpret_cast<const double2*>(zs + (size_t)k * DV);
#pragma unroll
        for (int h = 0; h < DV / 2; ++h) {
          const double2 p = zv[h];
          acz[2 * h] = fma(sv, p.x, acz[2 * h]);
          acz[2 * h + 1] = fma(sv, p.y, acz[2 * h + 1]);
        }
      }
    }
#pragma unroll
    for (int v = 0; v < DV; ++v) {
      if (v < nv) {
        double cn = 1.0;
        if (norm_correction) {
          cn = sqrt(s_red[v]);
          cn = cn > 1e-10 ? cn : 1.0;
        }
        double r = (acc[v] / cn) * (double)norm[v0 + v];
        if (qjl) r += acz[v] * (qc * (double)rnorm[v0 + v]);
        Tout* o = out + (v0 + v) * ld_out + j;
        *o = accumulate ? tq_from_double<Tout>(tq_as_double(*o) + r) : tq_from_double<Tout>(r);
      }
    }
  }
}

extern "C" int tq_dequantize(const tq_quantizer* q, const uint8_t* packed_dev, const uint8_t* idx_dev,
                             const float* norm_dev, const uint8_t* qjl_dev, const float* rnorm_dev, float shrinkage,
                             int64_t n, void* out_dev, int32_t out_dtype, void* stream) {
  TQ_REQUIRE(q, TQ_ERR_INVALID, "tq_dequantize: quantizer is null");
  TQ_REQUIRE(q->rotation == TQ_ROT_WHT || q->rot, TQ_ERR_INVALID, "tq_dequantize: quantizer was created without a rotation");
  TQ_REQUIRE(n >= 0, TQ_ERR_INVALID, "tq_dequantize: n must be >= 0");
  if (n == 0) return TQ_OK;
  TQ_REQUIRE((packed_dev != nullptr) != (idx_dev != nullptr), TQ_ERR_INVALID,
             "tq_dequantize: give exactly one of packed / unpacked indices");
  TQ_REQUIRE(norm_dev && out_dev, TQ_ERR_INVALID, "tq_dequantize: norms or output missing");
  TQ_REQUIRE((qjl_dev != nullptr) == (rnorm_dev != nullptr), TQ_ERR_INVALID,
             "tq_dequantize: QJL bits and residual norms go together");
  TQ_REQUIRE(!qjl_dev || q->qjl, TQ_ERR_INVALID, "tq_dequantize: quantizer has no QJL stage");
  TQ_REQUIRE(!packed_dev || (q->d * q->bits) % 8 == 0, TQ_ERR_UNSUPPORTED, "packed input needs d*bits % 8 == 0");
  cudaStream_t st = (cudaStream_t)stream;
  if (q->rotation == TQ_ROT_WHT) {
    TQ_REQUIRE(tq_aligned(out_dev, 16) && (!idx_dev || tq_aligned(idx_dev, 16)), TQ_ERR_ALIGN,
               "tq_dequantize: buffers must be 16-byte aligned");
    const int64_t groups = (n + 3) / 4;
    const int64_t cap = (int64_t)tq_num_sms() * 16;
    const int64_t want = (groups + 7) / 8;
    const int grid = (int)(want < cap ? want : cap);
#define TQ_DQ(T, B) \
  k_dequantize_wht<T, B><<<grid, 256, 0, st>>>(q->fast, packed_dev, idx_dev, norm_dev, qjl_dev, rnorm_dev, shrinkage, n, (T*)out_dev)
#define TQ_DQB(T)            \
  switch (q->bits) {         \
    case 1: TQ_DQ(T, 1); break; \
    case 2: TQ_DQ(T, 2); break; \
    case 3: TQ_DQ(T, 3); break; \
    default: TQ_DQ(T, 4); break; \
  }
    if (out_dtype == TQ_F32) {
      TQ_DQB(float)
    } else if (out_dtype == TQ_F16) {
      TQ_DQB(__half)
    } else {
      tq_set_error("WHT dequantize writes fp32 or fp16, got dtype %d", out_dtype);
      return TQ_ERR_UNSUPPORTED;
    }
#undef TQ_DQB
#undef TQ_DQ
    return tq_launch_check("k_dequantize_wht");
  }
  const size_t smem = (size_t)q->d * DV * 8 * (qjl_dev ? 2 : 1);
  const int grid = (int)((n + DV - 1) / DV);
#define TQ_DD(T)                                                                                                     \
  do {                                                                                                               \
    if (smem > 48 * 1024)                                                                                            \
      TQ_CUDA(cudaFuncSetAttribute(k_dequantize_dense<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));  \
    k_dequantize_dense<T><<<grid, 128, smem, st>>>(q->rot, q->s, q->cent64, q->d, q->bits, q->norm_correction,      \
                                                   packed_dev, idx_dev, norm_dev, qjl_dev, rnorm_dev,               \
                                                   (double)shrinkage, n, (T*)out_dev, (int64_t)q->d, 0);            \
  } while (0)
  switch (out_dtype) {
    case TQ_F64: TQ_DD(double); break;
    case TQ_F32: TQ_DD(float); break;
    case TQ_F16: TQ_DD(__half); break;
    default:
      tq_set_error("dense dequantize writes fp64, fp32 or fp16, got dtype %d", out_dtype);
      return TQ_ERR_UNSUPPORTED;
  }
#undef TQ_DD
  return tq_launch_check("k_dequantize_dense");
}

extern "C" int tq_dequantize_strided(const tq_quantizer* q, const uint8_t* idx_dev, const float* norm_dev, int64_t n,
                                     double* out_dev, int64_t ld_out, int32_t accumulate, void* stream) {
  TQ_REQUIRE(q, TQ_ERR_INVALID, "tq_dequantize_strided: quantizer is null");
  TQ_REQUIRE(q->rotation == TQ_ROT_DENSE && q->rot, TQ_ERR_UNSUPPORTED,
             "tq_dequantize_strided: needs a dense-mode quantizer with a rotation");
  TQ_REQUIRE(n >= 0, TQ_ERR_INVALID, "tq_dequantize_strided: n must be >= 0");
  if (n == 0) return TQ_OK;
  TQ_REQUIRE(idx_dev && norm_dev && out_dev, TQ_ERR_INVALID, "tq_dequantize_strided: null buffer");
  TQ_REQUIRE(ld_out >= q->d, TQ_ERR_INVALID, "tq_dequantize_strided: row stride %lld smaller than d", (long long)ld_out);
  TQ_REQUIRE(tq_aligned(out_dev, 8), TQ_ERR_ALIGN, "tq_dequantize_strided: output rows must be 8-byte aligned");
  const size_t smem = (size_t)q->d * DV * 8;
  const int grid = (int)((n + DV - 1) / DV);
  if (smem > 48 * 1024)
    TQ_CUDA(cudaFuncSetAttribute(k_dequantize_dense<double>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  k_dequantize_dense<double><<<grid, 128, smem, (cudaStream_t)stream>>>(
      q->rot, q->s, q->cent64, q->d, q->bits, q->norm_correction, nullptr, idx_dev, norm_dev, nullptr, nullptr, 1.0, n,
      out_dev, ld_out, accumulate ? 1 : 0);
  return tq_launch_check("k_dequantize_dense");
}
