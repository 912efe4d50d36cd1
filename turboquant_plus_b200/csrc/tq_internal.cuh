// Internal declarations shared by the translation units of libtq_b200.so.
#pragma once
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include "tq_b200.h"

#define TQ_D 128            // the only dimension of the fast (WHT / cache / attention) path
#define TQ_SQRT_D 11.313708498984761f
#define TQ_RSQRT_D 0.08838834764831845f

// Constants of one quantizer in the form the d = 128 kernels consume; passed by value as a
// kernel parameter (lives in the constant bank, uniform reads).
struct TqFast {
  uint32_t s1[4], s2[4];   // rotation sign bits, bit e set => element e multiplied by -1
  uint32_t j1[4], j2[4];   // QJL sign-WHT sign bits
  float cent[16];          // centroids rounded to fp32
  float bnd[15];           // fp64 midpoints rounded to fp32
  float lut_alpha;         // cent16[i] = fp16(lut_alpha * cent[i]); chosen to minimise the fp16 rounding error
  uint16_t cent16[16];
  int32_t bits;
  int32_t norm_correction;
  int32_t symmetric;       // bnd[i] == -bnd[n-2-i] in fp32 and the codebook likewise
  int32_t has_qjl;
};

struct tq_quantizer {
  int32_t d, bits, rotation, norm_correction, qjl, device;
  TqFast fast;               // valid when rotation == TQ_ROT_WHT
  // dense mode, device memory (fp64): R row-major, its transpose, S, its transpose
  double *rot, *rot_t, *s, *s_t;
  double* cent64;            // 1 << bits
  double* bnd64;             // (1 << bits) - 1
  float* rot32;              // R row-major in fp32 (query / output rotation of the attention path)
  float* rot32_t;
  float* s32;                // S row-major fp32
  float* s32_t;
  double host_cent[16];
};

void tq_set_error(const char* fmt, ...);
int tq_cuda_fail(cudaError_t e, const char* what);

#define TQ_CUDA(call)                                            \
  do {                                                           \
    cudaError_t e__ = (call);                                    \
    if (e__ != cudaSuccess) return tq_cuda_fail(e__, #call);     \
  } while (0)

#define TQ_REQUIRE(cond, code, ...)  \
  do {                               \
    if (!(cond)) {                   \
      tq_set_error(__VA_ARGS__);     \
      return (code);                 \
    }                                \
  } while (0)

static inline bool tq_aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

int tq_launch_check(const char* what);
int tq_num_sms();

// ---- device helpers ---------------------------------------------------------------------
__device__ __forceinline__ float tq_flip(float v, uint32_t bits16, int k) {
  // multiply v by -1 when bit k of bits16 is set
  return __int_as_float(__float_as_int(v) ^ ((bits16 << (31 - k)) & 0x80000000u));
}

// 16-element natural-order Walsh-Hadamard butterflies held in registers (strides 1,2,4,8)
__device__ __forceinline__ void tq_wht16_regs(float (&x)[16]) {
#pragma unroll
  for (int h = 1; h < 16; h <<= 1) {
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      if ((i & h) == 0) {
        float a = x[i], b = x[i + h];
        x[i] = a + b;
        x[i + h] = a - b;
      }
    }
  }
}

// strides 16, 32, 64 across the 8 lanes that share one 128-element vector (lane l holds
// elements 16*l .. 16*l+15)
__device__ __forceinline__ void tq_wht128_lanes(float (&x)[16], int sub) {
#pragma unroll
  for (int bit = 1; bit < 8; bit <<= 1) {
    const float sgn = (sub & bit) ? -1.0f : 1.0f;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      float v = __shfl_xor_sync(0xffffffffu, x[i], bit);
      x[i] = fmaf(sgn, x[i], v);
    }
  }
}

__device__ __forceinline__ float tq_sum8(float v) {
  v += __shfl_xor_sync(0xffffffffu, v, 1);
  v += __shfl_xor_sync(0xffffffffu, v, 2);
  v += __shfl_xor_sync(0xffffffffu, v, 4);
  return v;
}

__device__ __forceinline__ uint32_t tq_lane_bits16(const uint32_t (&m)[4], int sub) {
  return (m[sub >> 1] >> ((sub & 1) * 16)) & 0xffffu;
}

template <typename T> struct TqLoad16;
template <> struct TqLoad16<float> {
  static __device__ __forceinline__ void load(const float* p, float (&x)[16]) {
    const float4* p4 = reinterpret_cast<const float4*>(p);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float4 v = __ldg(p4 + i);
      x[4 * i] = v.x; x[4 * i + 1] = v.y; x[4 * i + 2] = v.z; x[4 * i + 3] = v.w;
    }
  }
};
template <> struct TqLoad16<__half> {
  static __device__ __forceinline__ void load(const __half* p, float (&x)[16]) {
    const uint4* p4 = reinterpret_cast<const uint4*>(p);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      uint4 v = __ldg(p4 + i);
      const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 f = __half22float2(h[j]);
        x[8 * i + 2 * j] = f.x; x[8 * i + 2 * j + 1] = f.y;
      }
    }
  }
};
template <> struct TqLoad16<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&x)[16]) {
    const uint4* p4 = reinterpret_cast<const uint4*>(p);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      uint4 v = __ldg(p4 + i);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 f = __bfloat1622float2(h[j]);
        x[8 * i + 2 * j] = f.x; x[8 * i + 2 * j + 1] = f.y;
      }
    }
  }
};

// Where the d = 128 quantize kernel puts its results: plain arrays (slots == nullptr, one
// "page" of unlimited size) or the records of a paged cache.
struct TqQuantDst {
  uint8_t* idx;     // packed indices: dst(v) = idx + page*page_stride + head*head_stride + within*idx_bytes
  float* norm;      // ||x||            (plain arrays only; nullptr in cache mode)
  float* scale;     // dequantization factor
  uint8_t* qjl;     // packed sign sketch
  float* rnorm;     // residual norm (plain arrays) / residual scale (cache mode)
  uint8_t* idx_u8;  // unpacked indices (plain arrays only)
  const int64_t* slots;
  int64_t page_stride, head_stride;
  int32_t page_tokens;  // 0 => plain arrays
  int32_t heads;        // vectors per token in the input
  int32_t rscale_const; // cache mode: store rnorm * sqrt(pi/2)/sqrt(d) so that attention needs one multiply
};

// address of vector v's record field (elem_bytes per token and head) in plain arrays or in a paged cache;
// ok = false when the token's slot is negative (skip it)
// The part of that address that every field of the record shares: byte offset of (page, head) and the token's
// position inside the page; field address = base + offset + within * elem_bytes.
__device__ __forceinline__ int64_t tq_dst_record(const TqQuantDst& dst, int64_t v, int64_t& within, bool& ok);

__device__ __forceinline__ uint8_t* tq_dst_ptr(uint8_t* base, const TqQuantDst& dst, int64_t v, int32_t elem_bytes,
                                               bool& ok) {
  int64_t within;
  const int64_t off = tq_dst_record(dst, v, within, ok);
  return base + off + within * elem_bytes;
}

__device__ __forceinline__ int64_t tq_dst_record(const TqQuantDst& dst, int64_t v, int64_t& within64, bool& ok) {
  if (dst.page_tokens == 0) {
    within64 = v;
    return 0;
  }
  // 32-bit arithmetic whenever the numbers allow it (64-bit division costs ~100 instructions)
  int64_t tok;
  int32_t head;
  if ((dst.heads & (dst.heads - 1)) == 0) {
    const int sh = 31 - __clz(dst.heads);
    tok = v >> sh;
    head = (int32_t)(v & (dst.heads - 1));
  } else if (v < 0x7fffffffLL) {
    const uint32_t v32 = (uint32_t)v, h32 = (uint32_t)dst.heads;
    const uint32_t t32 = v32 / h32;
    tok = t32;
    head = (int32_t)(v32 - t32 * h32);
  } else {
    tok = v / dst.heads;
    head = (int32_t)(v - tok * dst.heads);
  }
  const int64_t slot = dst.slots ? dst.slots[tok] : tok;
  if (slot < 0) {
    ok = false;
    within64 = 0;
    return 0;
  }
  int64_t page;
  int32_t within;
  if ((dst.page_tokens & (dst.page_tokens - 1)) == 0) {
    const int sh = 31 - __clz(dst.page_tokens);
    page = slot >> sh;
    within = (int32_t)(slot & (dst.page_tokens - 1));
  } else if (slot < 0x7fffffffLL) {
    const uint32_t pg = (uint32_t)slot / (uint32_t)dst.page_tokens;
    page = pg;
    within = (int32_t)((uint32_t)slot - pg * (uint32_t)dst.page_tokens);
  } else {
    page = slot / dst.page_tokens;
    within = (int32_t)(slot - page * dst.page_tokens);
  }
  within64 = within;
  return page * dst.page_stride + head * dst.head_stride;
}

int tq_quantize_wht_launch(const TqFast& f, const void* x, int32_t dtype, int64_t ld, int64_t n,
                           const TqQuantDst& dst, bool want_qjl, cudaStream_t st);
bool tq_quantize_mma_try(const TqFast& f, const void* x, int32_t dtype, int64_t ld, int64_t n, const TqQuantDst& dst,
                         bool want_qjl, cudaStream_t st, int* rc);
bool tq_quantize_mma_try_pair(const TqFast& f0, const void* x0, const TqQuantDst& d0, const TqFast& f1, const void* x1,
                              const TqQuantDst& d1, int32_t dtype, int64_t ld, int64_t n, cudaStream_t st, int* rc);
int tq_q8_0_append_launch(const void* x, int32_t dtype, int64_t n_tokens, int32_t heads, uint8_t* q_base,
                          uint8_t* scale_base, const int64_t* slots, int32_t page_tokens,
                          int64_t page_stride, int64_t head_stride, cudaStream_t st);
