// Stand-alone primitives: bit packing, the fp64 sign * Walsh-Hadamard rotation for any power-of-two
// size, and the nearest-centroid search.
#include "tq_internal.cuh"

__global__ void k_pack_indices(const uint8_t* __restrict__ idx, int64_t count, int bits, uint8_t* __restrict__ out,
                               int64_t out_bytes) {
  for (int64_t o = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; o < out_bytes; o += (int64_t)gridDim.x * blockDim.x) {
    uint32_t byte = 0;
    for (int bit = 0; bit < 8; ++bit) {
      const int64_t pos = o * 8 + bit, e = pos / bits;
      const int r = (int)(pos - e * bits);
      const uint32_t b = e < count ? ((idx[e] >> (bits - 1 - r)) & 1u) : 0u;
      byte = (byte << 1) | b;
    }
    out[o] = (uint8_t)byte;
  }
}

__global__ void k_unpack_indices(const uint8_t* __restrict__ packed, int64_t count, int bits, uint8_t* __restrict__ out) {
  for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < count; e += (int64_t)gridDim.x * blockDim.x) {
    uint32_t m = 0;
    for (int r = 0; r < bits; ++r) {
      const int64_t pos = e * bits + r;
      m = (m << 1) | ((packed[pos >> 3] >> (7 - (int)(pos & 7))) & 1u);
    }
    out[e] = (uint8_t)m;
  }
}

__global__ void k_copy_bytes(const uint8_t* __restrict__ in, int64_t count, uint8_t* __restrict__ out) {
  for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < count; e += (int64_t)gridDim.x * blockDim.x)
    out[e] = in[e];
}

__global__ void k_pack_bits(const int8_t* __restrict__ s, int64_t rows, int d, uint8_t* __restrict__ out) {
  const int rb = (d + 7) / 8;
  for (int64_t o = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; o < rows * rb; o += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = o / rb;
    const int c = (int)(o - row * rb);
    uint32_t byte = 0;
    for (int bit = 0; bit < 8; ++bit) {
      const int e = c * 8 + bit;
      byte = (byte << 1) | ((e < d && s[row * d + e] > 0) ? 1u : 0u);
    }
    out[o] = (uint8_t)byte;
  }
}

__global__ void k_unpack_bits(const uint8_t* __restrict__ p, int64_t rows, int d, int8_t* __restrict__ out) {
  const int rb = (d + 7) / 8;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < rows * d; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = i / d;
    const int e = (int)(i - row * d);
    out[i] = ((p[row * rb + (e >> 3)] >> (7 - (e & 7))) & 1u) ? 1 : -1;
  }
}

static inline int grid_for(int64_t work, int block) {
  int64_t g = (work + block - 1) / block;
  const int64_t cap = (int64_t)tq_num_sms() * 32;
  if (g > cap) g = cap;
  if (g < 1) g = 1;
  return (int)g;
}

extern "C" int tq_pack_indices(const uint8_t* idx_dev, int64_t count, int32_t bits, uint8_t* out_dev, void* stream) {
  TQ_REQUIRE(bits >= 1 && bits <= 8, TQ_ERR_INVALID, "bit_width must be 1-8, got %d", bits);
  TQ_REQUIRE(count >= 0, TQ_ERR_INVALID, "count must be >= 0");
  if (count == 0) return TQ_OK;
  TQ_REQUIRE(idx_dev && out_dev, TQ_ERR_INVALID, "null buffer");
  cudaStream_t st = (cudaStream_t)stream;
  if (bits > 4) {
    k_copy_bytes<<<grid_for(count, 256), 256, 0, st>>>(idx_dev, count, out_dev);
  } else {
    const int64_t ob = (count * bits + 7) / 8;
    k_pack_indices<<<grid_for(ob, 256), 256, 0, st>>>(idx_dev, count, bits, out_dev, ob);
  }
  return tq_launch_check("k_pack_indices");
}

extern "C" int tq_unpack_indices(const uint8_t* packed_dev, int64_t count, int32_t bits, uint8_t* out_dev, void* stream) {
  TQ_REQUIRE(bits >= 1 && bits <= 8, TQ_ERR_INVALID, "bit_width must be 1-8, got %d", bits);
  TQ_REQUIRE(count >= 0, TQ_ERR_INVALID, "count must be >= 0");
  if (count == 0) return TQ_OK;
  TQ_REQUIRE(packed_dev && out_dev, TQ_ERR_INVALID, "null buffer");
  cudaStream_t st = (cudaStream_t)stream;
  if (bits > 4)
    k_copy_bytes<<<grid_for(count, 256), 256, 0, st>>>(packed_dev, count, out_dev);
  else
    k_unpack_indices<<<grid_for(count, 256), 256, 0, st>>>(packed_dev, count, bits, out_dev);
  return tq_launch_check("k_unpack_indices");
}

extern "C" int tq_pack_bits(const int8_t* signs_dev, int64_t rows, int32_t d, uint8_t* out_dev, void* stream) {
  TQ_REQUIRE(rows >= 0 && d >= 1, TQ_ERR_INVALID, "bad shape");
  if (rows == 0) return TQ_OK;
  TQ_REQUIRE(signs_dev && out_dev, TQ_ERR_INVALID, "null buffer");
  k_pack_bits<<<grid_for(rows * ((d + 7) / 8), 256), 256, 0, (cudaStream_t)stream>>>(signs_dev, rows, d, out_dev);
  return tq_launch_check("k_pack_bits");
}

extern "C" int tq_unpack_bits(const uint8_t* packed_dev, int64_t rows, int32_t d, int8_t* out_dev, void* stream) {
  TQ_REQUIRE(rows >= 0 && d >= 1, TQ_ERR_INVALID, "bad shape");
  if (rows == 0) return TQ_OK;
  TQ_REQUIRE(packed_dev && out_dev, TQ_ERR_INVALID, "null buffer");
  k_unpack_bits<<<grid_for(rows * d, 256), 256, 0, (cudaStream_t)stream>>>(packed_dev, rows, d, out_dev);
  return tq_launch_check("k_unpack_bits");
}

// One CTA per row; the row lives in shared memory for all log2(n) butterfly stages.
__global__ void __launch_bounds__(256) k_sign_wht_f64(const double* __restrict__ x, int64_t rows, int d, int n,
                                                      const double* __restrict__ s1, const double* __restrict__ s2,
                                                      double* __restrict__ out) {
  extern __shared__ double buf[];
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      double v = i < d ? x[row * d + i] : 0.0;
      if (s1) v *= s1[i];
      buf[i] = v;
    }
    __syncthreads();
    for (int h = 1; h < n; h <<= 1) {
      for (int p = threadIdx.x; p < n / 2; p += blockDim.x) {
        const int i = ((p / h) * 2 * h) + (p % h);
        const double a = buf[i], b = buf[i + h];
        buf[i] = a + b;
        buf[i + h] = a - b;
      }
      __syncthreads();
    }
    const double sc = sqrt((double)n);
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
      double v = buf[i] / sc;
      if (s2) v *= s2[i];
      out[row * d + i] = v;
    }
    __syncthreads();
  }
}

extern "C" int tq_sign_wht_f64(const double* x_dev, int64_t rows, int32_t d, int32_t n, const double* signs1_dev,
                               const double* signs2_dev, double* out_dev, void* stream) {
  TQ_REQUIRE(n >= 1 && (n & (n - 1)) == 0, TQ_ERR_INVALID, "Input length must be a positive power of 2, got %d", n);
  TQ_REQUIRE(n <= 4096, TQ_ERR_TOO_LARGE, "transform size %d beyond the maximum 4096", n);
  TQ_REQUIRE(d >= 1 && d <= n && rows >= 0, TQ_ERR_INVALID, "bad shape");
  if (rows == 0) return TQ_OK;
  TQ_REQUIRE(x_dev && out_dev, TQ_ERR_INVALID, "null buffer");
  const int64_t cap = (int64_t)tq_num_sms() * 8;
  const int grid = (int)(rows < cap ? rows : cap);
  k_sign_wht_f64<<<grid, 256, (size_t)n * 8, (cudaStream_t)stream>>>(x_dev, rows, d, n, signs1_dev, signs2_dev, out_dev);
  return tq_launch_check("k_sign_wht_f64");
}

__global__ void k_nearest_centroid_f64(const double* __restrict__ v, int64_t count, const double* __restrict__ c, int nc,
                                       int64_t* __restrict__ out) {
  extern __shared__ double bnd[];
  for (int i = threadIdx.x; i < nc - 1; i += blockDim.x) bnd[i] = (c[i] + c[i + 1]) / 2.0;
  __syncthreads();
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (int64_t)gridDim.x * blockDim.x) {
    const double x = v[i];
    // lower-bound binary search: number of boundaries strictly below x
    int lo = 0, hi = nc - 1;
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      if (bnd[mid] < x) lo = mid + 1;
      else hi = mid;
    }
    out[i] = lo;
  }
}

extern "C" int tq_nearest_centroid_f64(const double* values_dev, int64_t count, const double* centroids_dev,
                                       int32_t n_centroids, int64_t* out_dev, void* stream) {
  TQ_REQUIRE(n_centroids >= 1 && n_centroids <= 4096, TQ_ERR_INVALID, "n_centroids must be in 1..4096");
  TQ_REQUIRE(count >= 0, TQ_ERR_INVALID, "count must be >= 0");
  if (count == 0) return TQ_OK;
  TQ_REQUIRE(values_dev && centroids_dev && out_dev, TQ_ERR_INVALID, "null buffer");
  k_nearest_centroid_f64<<<grid_for(count, 256), 256, (size_t)n_centroids * 8, (cudaStream_t)stream>>>(
      values_dev, count, centroids_dev, n_centroids, out_dev);
  return tq_launch_check("k_nearest_centroid_f64");
}
