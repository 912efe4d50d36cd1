// Stand-alone QJL stage (turboquant/qjl.py:72-134) for any d, fp64 like the reference, and the
// scatter of already-quantized rows into a paged cache.
#include "tq_internal.cuh"

namespace {
constexpr int QV = 8;  // vectors per CTA

template <typename T> __device__ __forceinline__ double to_d(T v);
template <> __device__ __forceinline__ double to_d<float>(float v) { return (double)v; }
template <> __device__ __forceinline__ double to_d<double>(double v) { return v; }
template <> __device__ __forceinline__ double to_d<__half>(__half v) { return (double)__half2float(v); }

template <typename Tin>
__global__ void __launch_bounds__(128) k_qjl_quantize(const double* __restrict__ s_t, int d, const Tin* __restrict__ r,
                                                      int64_t n, uint8_t* __restrict__ out_bits,
                                                      float* __restrict__ out_norm) {
  extern __shared__ __align__(16) double sm[];
  double* rs = sm;  // [d][QV]
  uint8_t* sb = reinterpret_cast<uint8_t*>(sm + (size_t)d * QV);  // [QV][d]
  __shared__ double s_red[QV];
  const int tid = threadIdx.x;
  const int64_t v0 = (int64_t)blockIdx.x * QV;
  const int nv = (int)((n - v0) < QV ? (n - v0) : QV);
  if (tid < QV) s_red[tid] = 0.0;
  double part = 0.0;  // stride 128 is a multiple of QV: a thread always sees the same vector
  for (int i = tid; i < d * QV; i += 128) {
    const int v = i % QV, k = i / QV;
    const double x = v < nv ? to_d<Tin>(r[(v0 + v) * d + k]) : 0.0;
    rs[i] = x;
    part += x * x;
  }
  __syncthreads();
  atomicAdd(&s_red[tid % QV], part);
  __syncthreads();
  if (tid < nv && out_norm) out_norm[v0 + tid] = (float)sqrt(s_red[tid]);
  for (int j = tid; j < d; j += 128) {
    double acc[QV];
#pragma unroll
    for (int v = 0; v < QV; ++v) acc[v] = 0.0;
    for (int k = 0; k < d; ++k) {
      const double sv = __ldg(s_t + (size_t)k * d + j);
      const double2* rv = reinterpret_cast<const double2*>(rs + (size_t)k * QV);
#pragma unroll
      for (int h = 0; h < QV / 2; ++h) {
        const double2 p = rv[h];
        acc[2 * h] = fma(sv, p.x, acc[2 * h]);
        acc[2 * h + 1] = fma(sv, p.y, acc[2 * h + 1]);
      }
    }
#pragma unroll
    for (int v = 0; v < QV; ++v) sb[v * d + j] = acc[v] < 0.0 ? 0 : 1;  // zero -> +1: turboquant/qjl.py:89-90
  }
  __syncthreads();
  const int rb = (d + 7) / 8;
  for (int i = tid; i < nv * rb; i += 128) {
    const int v = i / rb, o = i - v * rb;
    uint32_t byte = 0;
    for (int bit = 0; bit < 8; ++bit) {
      const int e = o * 8 + bit;
      byte = (byte << 1) | (e < d ? sb[v * d + e] : 0u);
    }
    out_bits[v0 * rb + i] = (uint8_t)byte;
  }
}

template <typename T> __device__ __forceinline__ T from_d(double v);
template <> __device__ __forceinline__ double from_d<double>(double v) { return v; }
template <> __device__ __forceinline__ float from_d<float>(double v) { return (float)v; }
template <> __device__ __forceinline__ __half from_d<__half>(double v) { return __float2half_rn((float)v); }

template <typename Tout>
__global__ void __launch_bounds__(128) k_qjl_dequantize(const double* __restrict__ s, int d,
                                                        const uint8_t* __restrict__ bits,
                                                        const float* __restrict__ rnorm, double shrink, int64_t n,
                                                        Tout* __restrict__ out) {
  extern __shared__ __align__(16) double sm[];
  double* zs = sm;  // [d][QV]
  const int tid = threadIdx.x;
  const int64_t v0 = (int64_t)blockIdx.x * QV;
  const int nv = (int)((n - v0) < QV ? (n - v0) : QV);
  const int rb = (d + 7) / 8;
  for (int i = tid; i < d * QV; i += 128) {
    const int v = i % QV, k = i / QV;
    zs[i] = v < nv ? (((bits[(v0 + v) * rb + (k >> 3)] >> (7 - (k & 7))) & 1u) ? 1.0 : -1.0) : 0.0;
  }
  __syncthreads();
  const double qc = shrink * 1.2533141373155001 / sqrt((double)d);  // sqrt(pi/2)/sqrt(d): turboquant/qjl.py:32,131
  for (int j = tid; j < d; j += 128) {
    double acc[QV];
#pragma unroll
    for (int v = 0; v < QV; ++v) acc[v] = 0.0;
    for (int k = 0; k < d; ++k) {
      const double sv = __ldg(s + (size_t)k * d + j);  // (S^T z)_j = sum_k S[k][j] z_k
      const double2* zv = reinterpret_cast<const double2*>(zs + (size_t)k * QV);
#pragma unroll
      for (int h = 0; h < QV / 2; ++h) {
        const double2 p = zv[h];
        acc[2 * h] = fma(sv, p.x, acc[2 * h]);
        acc[2 * h + 1] = fma(sv, p.y, acc[2 * h + 1]);
      }
    }
#pragma unroll
    for (int v = 0; v < QV; ++v)
      if (v < nv) out[(v0 + v) * d + j] = from_d<Tout>(acc[v] * (qc * (double)rnorm[v0 + v]));
  }
}

// rows [n_tokens][heads][row_bytes] -> record arrays of a paged cache; one thread per 4 bytes
__global__ void k_cache_scatter(const uint8_t* __restrict__ src, int row_bytes, int64_t n_tokens, int heads,
                                uint8_t* __restrict__ dst_base, const int64_t* __restrict__ slots, int page_tokens,
                                int64_t page_stride, int64_t head_stride) {
  const int wpr = row_bytes / 4;
  const int64_t total = n_tokens * heads * wpr;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = i / wpr;
    const int w = (int)(i - row * wpr);
    const int64_t tok = row / heads;
    const int head = (int)(row - tok * heads);
    const int64_t slot = slots[tok];
    if (slot < 0) continue;
    const int64_t page = slot / page_tokens;
    const int within = (int)(slot - page * page_tokens);
    uint8_t* d = dst_base + page * page_stride + head * head_stride + (int64_t)within * row_bytes + w * 4;
    *reinterpret_cast<uint32_t*>(d) = *reinterpret_cast<const uint32_t*>(src + row * row_bytes + w * 4);
  }
}
}  // namespace

extern "C" int tq_qjl_quantize(const tq_quantizer* q, const void* r_dev, int32_t dtype, int64_t n,
                               uint8_t* out_bits_dev, float* out_norm_dev, void* stream) {
  TQ_REQUIRE(q && q->s_t, TQ_ERR_INVALID, "tq_qjl_quantize: needs a dense-mode quantizer with a QJL matrix");
  TQ_REQUIRE(n >= 0, TQ_ERR_INVALID, "n must be >= 0");
  if (n == 0) return TQ_OK;
  TQ_REQUIRE(r_dev && out_bits_dev, TQ_ERR_INVALID, "null buffer");
  const size_t smem = (size_t)q->d * QV * 8 + (size_t)q->d * QV + 16;
  const int grid = (int)((n + QV - 1) / QV);
  cudaStream_t st = (cudaStream_t)stream;
#define TQ_QQ(T)                                                                                               \
  do {                                                                                                         \
    if (smem > 48 * 1024)                                                                                      \
      TQ_CUDA(cudaFuncSetAttribute(k_qjl_quantize<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
    k_qjl_quantize<T><<<grid, 128, smem, st>>>(q->s_t, q->d, (const T*)r_dev, n, out_bits_dev, out_norm_dev);  \
  } while (0)
  switch (dtype) {
    case TQ_F64: TQ_QQ(double); break;
    case TQ_F32: TQ_QQ(float); break;
    case TQ_F16: TQ_QQ(__half); break;
    default:
      tq_set_error("tq_qjl_quantize accepts fp64, fp32 or fp16 input, got dtype %d", dtype);
      return TQ_ERR_UNSUPPORTED;
  }
#undef TQ_QQ
  return tq_launch_check("k_qjl_quantize");
}

extern "C" int tq_qjl_dequantize(const tq_quantizer* q, const uint8_t* bits_dev, const float* rnorm_dev,
                                 float shrinkage, int64_t n, void* out_dev, int32_t out_dtype, void* stream) {
  TQ_REQUIRE(q && q->s, TQ_ERR_INVALID, "tq_qjl_dequantize: needs a dense-mode quantizer with a QJL matrix");
  TQ_REQUIRE(n >= 0, TQ_ERR_INVALID, "n must be >= 0");
  if (n == 0) return TQ_OK;
  TQ_REQUIRE(bits_dev && rnorm_dev && out_dev, TQ_ERR_INVALID, "null buffer");
  const size_t smem = (size_t)q->d * QV * 8;
  const int grid = (int)((n + QV - 1) / QV);
  cudaStream_t st = (cudaStream_t)stream;
#define TQ_QD(T)                                                                                                 \
  do {                                                                                                           \
    if (smem > 48 * 1024)                                                                                        \
      TQ_CUDA(cudaFuncSetAttribute(k_qjl_dequantize<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
    k_qjl_dequantize<T><<<grid, 128, smem, st>>>(q->s, q->d, bits_dev, rnorm_dev, (double)shrinkage, n, (T*)out_dev); \
  } while (0)
  switch (out_dtype) {
    case TQ_F64: TQ_QD(double); break;
    case TQ_F32: TQ_QD(float); break;
    case TQ_F16: TQ_QD(__half); break;
    default:
      tq_set_error("tq_qjl_dequantize writes fp64, fp32 or fp16, got dtype %d", out_dtype);
      return TQ_ERR_UNSUPPORTED;
  }
#undef TQ_QD
  return tq_launch_check("k_qjl_dequantize");
}

extern "C" int tq_cache_store(const tq_cache_layout* L, uint8_t* pool_dev, int32_t which, const uint8_t* packed_dev,
                              const float* scale_dev, const uint8_t* qjl_dev, const float* rscale_dev,
                              int64_t n_tokens, const int64_t* slot_dev, void* stream) {
  TQ_REQUIRE(L && pool_dev && slot_dev, TQ_ERR_INVALID, "tq_cache_store: null argument");
  TQ_REQUIRE(which == 0 || which == 1, TQ_ERR_INVALID, "which must be 0 (K) or 1 (V)");
  TQ_REQUIRE(n_tokens >= 0, TQ_ERR_INVALID, "n_tokens must be >= 0");
  if (n_tokens == 0) return TQ_OK;
  TQ_REQUIRE(packed_dev && scale_dev, TQ_ERR_INVALID, "indices and scales are required");
  const int fmt = which == 0 ? L->k_format : L->v_format;
  TQ_REQUIRE(fmt != TQ_FMT_Q8_0, TQ_ERR_UNSUPPORTED, "tq_cache_store handles turbo/prod tensors; q8_0 goes through tq_cache_append");
  const bool prod = fmt >= TQ_FMT_PROD2;
  TQ_REQUIRE(!prod || (qjl_dev && rscale_dev), TQ_ERR_INVALID, "PROD format needs the sign sketch and residual scales");
  TQ_REQUIRE(tq_aligned(packed_dev, 4) && tq_aligned(pool_dev, 128), TQ_ERR_ALIGN, "buffers must be aligned");
  cudaStream_t st = (cudaStream_t)stream;
  const int H = L->num_kv_heads;
  auto go = [&](const void* src, int row_bytes, int off) {
    const int64_t total = n_tokens * H * (row_bytes / 4);
    int64_t g = (total + 255) / 256;
    const int64_t cap = (int64_t)tq_num_sms() * 16;
    if (g > cap) g = cap;
    k_cache_scatter<<<(int)g, 256, 0, st>>>((const uint8_t*)src, row_bytes, n_tokens, H, pool_dev + off, slot_dev,
                                            L->page_tokens, L->page_stride, L->head_stride);
  };
  go(packed_dev, which == 0 ? L->k_idx_bytes : L->v_idx_bytes, which == 0 ? L->k_idx_off : L->v_idx_off);
  go(scale_dev, 4, which == 0 ? L->k_scale_off : L->v_scale_off);
  if (prod) {
    go(qjl_dev, TQ_D / 8, L->k_qjl_off);
    go(rscale_dev, 4, L->k_rscale_off);
  }
  return tq_launch_check("k_cache_scatter");
}
