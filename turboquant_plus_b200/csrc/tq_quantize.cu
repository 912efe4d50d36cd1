// Quantize kernels: norm extraction, rotation, nearest Lloyd-Max centroid, bit packing and the
// optional 1-bit QJL sketch of the residual.
//
//   k_quantize_wht   d = 128, sign * Walsh-Hadamard rotation in registers + warp shuffles, fp32.
//                    Eight lanes share a vector (16 consecutive elements each); a warp handles
//                    four vectors per iteration.  Output is the packed stream the cache stores.
//   k_quantize_dense any d <= 1024, dense d x d rotation in fp64 -- the reference's own
//                    arithmetic (turboquant/polar_quant.py:56-85 runs an fp64 GEMM), used where
//                    index-exact agreement with the reference classes matters more than speed.
//   k_q8_0_append    int8 + fp16 scale per 32 values.
#include "tq_internal.cuh"

// ------------------------------------------------------------------------------------------
// d = 128, WHT rotation
//
// The integer ALU pipe of an SM runs at half the FP32 rate, so everything that can be phrased as fp32
// arithmetic is: sign flips are multiplications by +-1, threshold tests produce 0.0f / 1.0f that are summed,
// the index is assembled as a float, and eight 3-bit indices are packed by an exact fp32 Horner sum
// (< 2^24) that is turned into an integer once per group.
// ------------------------------------------------------------------------------------------
template <typename Tin, int BITS, bool SYM, bool QJL>
__global__ void __launch_bounds__(256) k_quantize_wht(const TqFast f, const Tin* __restrict__ x, int64_t ld, int64_t n,
                                                      const TqQuantDst dst) {
  // a dependent kernel launched with programmatic stream serialization may start now (it waits for this grid's
  // completion itself before it touches what this grid writes); without such a dependent this does nothing
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  constexpr int NC = 1 << BITS, HALF = NC / 2;
  constexpr int IDXB = 16 * BITS;              // packed bytes per vector
  constexpr int GS = BITS == 4 ? 4 : 8;        // indices per fp32 Horner group (GS * BITS <= 24 bits)
  constexpr int NG = 16 / GS;
  constexpr float RADIX = (float)(1 << BITS);
  __shared__ __align__(16) uint8_t st_idx[8][4][IDXB];
  __shared__ __align__(16) uint8_t st_q[8][4][16];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, sub = lane & 7, vi = lane >> 3;
  const uint32_t b1 = tq_lane_bits16(f.s1, sub), b2 = tq_lane_bits16(f.s2, sub);
  const bool need_c = QJL || (dst.scale != nullptr && f.norm_correction);
  // sign1 as +-1.0f factors, pinned in registers (opaque to the compiler, or it recomputes them from the
  // bit mask for every vector on the half-rate integer pipe)
  float sg1[16];
#pragma unroll
  for (int k = 0; k < 16; ++k) {
    sg1[k] = ((b1 >> k) & 1u) ? -1.0f : 1.0f;
    asm volatile("" : "+f"(sg1[k]));
  }
  // sign2 never touches the values when the codebook is symmetric: negating a coordinate mirrors its index
  // (i -> 2^b - 1 - i), which is an XOR of the packed word with a per-lane constant.  (A coordinate exactly on a
  // boundary then takes the upper instead of the lower index on mirrored lanes.)
  uint32_t flip0 = 0, flip1 = 0;
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    if ((b2 >> k) & 1u) flip0 |= ((1u << BITS) - 1) << (BITS * (7 - k));
    if ((b2 >> (8 + k)) & 1u) flip1 |= ((1u << BITS) - 1) << (BITS * (7 - k));
  }

  for (int64_t base = ((int64_t)blockIdx.x * 8 + warp) * 4; base < n; base += (int64_t)gridDim.x * 32) {
    const int64_t v = base + vi;
    const bool ok = v < n;
    float u[16];
    if (ok) {
      TqLoad16<Tin>::load(x + v * ld + sub * 16, u);
    } else {
#pragma unroll
      for (int k = 0; k < 16; ++k) u[k] = 0.f;
    }
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < 16; ++k) ss = fmaf(u[k], u[k], ss);
    ss = tq_sum8(ss);
    const float nrm = sqrtf(ss);
    const float safe = nrm > 0.f ? nrm : 1.0f;  // turboquant/polar_quant.py:74
#pragma unroll
    for (int k = 0; k < 16; ++k) u[k] *= sg1[k];
    tq_wht16_regs(u);
    tq_wht128_lanes(u, sub);
    // sg2 * u = y * safe * sqrt(d) with y the rotated unit vector.
    // Magnitude threshold tests on the FP32 pipe: step(a > b) = sat(sat(a * BIGS - b * BIG) * 2^16) with BIG = 2^40 and
    // BIGS = BIG / (safe * sqrt d).  The inner FMA is exact up to one rounding, so it is positive exactly when
    // a * BIGS > b * BIG, and a positive result is at least 2^-10 (operands near 2^37 carry 48 exact product
    // bits; 2^-12 for the smallest 4-bit boundary), which the second saturating multiply turns into 1.  Compared with testing a > b * safe * sqrt d
    // this moves a decision only for coordinates within a few 1e-8 relative of a boundary.
    const float ts = safe * TQ_SQRT_D;
    constexpr float BIG = 1099511627776.0f;  // 2^40
    const float bigs = BIG / ts;
    float NB[NC - 1];                        // -b_j * BIG
#pragma unroll
    for (int j = 0; j < NC - 1; ++j) NB[j] = -f.bnd[j] * BIG;

    float c[16];
    float cc = 0.f;
    float wf[NG];
#pragma unroll
    for (int gq = 0; gq < NG; ++gq) wf[gq] = 0.f;
#pragma unroll
    for (int k = 0; k < 16; ++k) {
      if (!SYM) u[k] = tq_flip(u[k], b2, k);
      float idxf, cm;
      if (SYM) {
        // magnitude level m = #positive boundaries below |u|, sign from the centre boundary
        const float a = fabsf(u[k]);
        float m = 0.f;
        cm = f.cent[HALF];
#pragma unroll
        for (int j = 1; j < HALF; ++j) {
          const float p = __saturatef(__saturatef(fmaf(a, bigs, NB[HALF - 1 + j])) * 65536.0f);
          m += p;
          if (need_c) cm = fmaf(p, f.cent[HALF + j] - f.cent[HALF + j - 1], cm);
        }
        // the centre boundary is (almost) zero, where the 2^-10 argument does not hold: plain comparison
        const float sgn = u[k] > f.bnd[HALF - 1] * ts ? 1.0f : -1.0f;
        idxf = fmaf(sgn, m + 0.5f, (float)HALF - 0.5f);  // HALF + m or HALF - 1 - m
        cm *= sgn;
      } else {
        idxf = 0.f;
        cm = f.cent[0];
#pragma unroll
        for (int j = 0; j < NC - 1; ++j) {
          const float p = u[k] > f.bnd[j] * ts ? 1.0f : 0.0f;  // arbitrary codebook: plain comparisons
          idxf += p;
          if (need_c) cm = fmaf(p, f.cent[j + 1] - f.cent[j], cm);
        }
      }
      c[k] = cm;
      if (need_c) cc = fmaf(cm, cm, cc);
      wf[k / GS] = fmaf(wf[k / GS], RADIX, idxf);  // exact: below 2^24
    }
    float invn = 1.0f;
    if (need_c) {
      cc = tq_sum8(cc);
      if (f.norm_correction) {
        float cn = sqrtf(cc);
        cn = cn > 1e-10f ? cn : 1.0f;  // turboquant/polar_quant.py:110-111
        invn = 1.0f / cn;
      }
    }
    // integers out of the Horner sums (exact: the sums are whole numbers below 2^24)
    uint32_t wi[NG];
#pragma unroll
    for (int gq = 0; gq < NG; ++gq) wi[gq] = __float2uint_rn(wf[gq]);
    uint32_t w0, w1;  // 8 indices each, MSB first
    if (BITS == 4) {
      w0 = (wi[0] << 16) | wi[1 % NG];
      w1 = (wi[2 % NG] << 16) | wi[3 % NG];
    } else {
      w0 = wi[0];
      w1 = wi[1 % NG];
    }
    if (SYM && nrm > 0.f) {  // a zero vector keeps the index of the value 0 on every lane
      w0 ^= flip0;
      w1 ^= flip1;
    }
    if (dst.idx) {
      uint8_t* s = &st_idx[warp][vi][sub * 2 * BITS];
#pragma unroll
      for (int j = 0; j < BITS; ++j) {
        s[j] = (uint8_t)(w0 >> (8 * (BITS - 1 - j)));
        s[BITS + j] = (uint8_t)(w1 >> (8 * (BITS - 1 - j)));
      }
    }
    if (dst.idx_u8 && ok) {
      uint32_t o4[4] = {0, 0, 0, 0};
#pragma unroll
      for (int k = 0; k < 16; ++k) {
        const uint32_t wsrc = k < 8 ? w0 : w1;
        const uint32_t id = (wsrc >> (BITS * (7 - (k & 7)))) & ((1u << BITS) - 1);
        o4[k >> 2] |= id << (8 * (k & 3));
      }
      *reinterpret_cast<uint4*>(dst.idx_u8 + v * TQ_D + sub * 16) = make_uint4(o4[0], o4[1], o4[2], o4[3]);
    }

    float rn = 0.f;
    if (QJL) {
      // residual in the rotated domain, scaled like u: E = (y - yhat') * safe * sqrt(d)
      const float cs = invn * ts;
      float ee = 0.f;
#pragma unroll
      for (int k = 0; k < 16; ++k) {
        u[k] = fmaf(-c[k], cs, u[k]);
        ee = fmaf(u[k], u[k], ee);
      }
      ee = tq_sum8(ee);
      rn = nrm > 0.f ? sqrtf(ee) * TQ_RSQRT_D : 0.f;  // ||r|| = ||x|| * ||y - yhat'||
      // r ~ D1 H D2 E, then S r ~ J2 H J1 r  (positive factors dropped: only signs are kept)
      const uint32_t m12 = b1 ^ tq_lane_bits16(f.j1, sub);
      const uint32_t bj2 = tq_lane_bits16(f.j2, sub);
      if (!SYM) {  // symmetric codebooks never applied sign2, so there is nothing to undo
#pragma unroll
        for (int k = 0; k < 16; ++k) u[k] = tq_flip(u[k], b2, k);
      }
      tq_wht16_regs(u);
      tq_wht128_lanes(u, sub);
#pragma unroll
      for (int k = 0; k < 16; ++k) u[k] = tq_flip(u[k], m12, k);
      tq_wht16_regs(u);
      tq_wht128_lanes(u, sub);
      uint32_t bits = 0;
#pragma unroll
      for (int k = 0; k < 16; ++k) {
        const float t = tq_flip(u[k], bj2, k);
        bits |= (t < 0.f ? 0u : 1u) << (15 - k);  // zero counts as +1: turboquant/qjl.py:89-90
      }
      if (!(nrm > 0.f)) bits = 0xffffu;  // zero input -> zero residual -> all +1
      if (dst.qjl) {
        st_q[warp][vi][sub * 2] = (uint8_t)(bits >> 8);
        st_q[warp][vi][sub * 2 + 1] = (uint8_t)bits;
      }
    }
    __syncwarp();
    // coalesced 16-byte stores of the staged bytes
    if (dst.idx && lane < 4 * BITS) {
      const int vv = lane / BITS, ch = lane - vv * BITS;
      if (base + vv < n) {
        bool good = true;
        uint8_t* p = tq_dst_ptr(dst.idx, dst, base + vv, IDXB, good);
        if (good) *reinterpret_cast<uint4*>(p + ch * 16) = *reinterpret_cast<const uint4*>(&st_idx[warp][vv][ch * 16]);
      }
    }
    if (QJL && dst.qjl && lane < 4) {
      if (base + lane < n) {
        bool good = true;
        uint8_t* p = tq_dst_ptr(dst.qjl, dst, base + lane, 16, good);
        if (good) *reinterpret_cast<uint4*>(p) = *reinterpret_cast<const uint4*>(&st_q[warp][lane][0]);
      }
    }
    if (ok && sub == 0) {
      bool good = true;
      if (dst.norm) dst.norm[v] = nrm;
      if (dst.scale) {
        float* p = reinterpret_cast<float*>(tq_dst_ptr(reinterpret_cast<uint8_t*>(dst.scale), dst, v, 4, good));
        if (good) *p = nrm * invn;
      }
      if (QJL && dst.rnorm) {
        good = true;
        float* p = reinterpret_cast<float*>(tq_dst_ptr(reinterpret_cast<uint8_t*>(dst.rnorm), dst, v, 4, good));
        // sqrt(pi/2)/sqrt(d): turboquant/qjl.py:32,131
        if (good) *p = dst.rscale_const ? rn * (1.2533141373155001f * TQ_RSQRT_D) : rn;
      }
    }
    __syncwarp();
  }
}

template <typename Tin, int BITS, bool SYM>
static int launch_wht3(const TqFast& f, const Tin* x, int64_t ld, int64_t n, const TqQuantDst& dst, bool qjl,
                       cudaStream_t st) {
  const int64_t tiles = (n + 31) / 32;
  const int64_t cap = (int64_t)tq_num_sms() * 8;
  const int grid = (int)(tiles < cap ? tiles : cap);
  if (qjl)
    k_quantize_wht<Tin, BITS, SYM, true><<<grid, 256, 0, st>>>(f, x, ld, n, dst);
  else
    k_quantize_wht<Tin, BITS, SYM, false><<<grid, 256, 0, st>>>(f, x, ld, n, dst);
  return tq_launch_check("k_quantize_wht");
}

template <typename Tin>
static int launch_wht2(const TqFast& f, const Tin* x, int64_t ld, int64_t n, const TqQuantDst& dst, bool qjl,
                       cudaStream_t st) {
#define TQ_CASE(B)                                                        \
  case B:                                                                 \
    return f.symmetric ? launch_wht3<Tin, B, true>(f, x, ld, n, dst, qjl, st) \
                       : launch_wht3<Tin, B, false>(f, x, ld, n, dst, qjl, st);
  switch (f.bits) {
    TQ_CASE(1)
    TQ_CASE(2)
    TQ_CASE(3)
    TQ_CASE(4)
  }
#undef TQ_CASE
  tq_set_error("bits %d out of range", f.bits);
  return TQ_ERR_INVALID;
}

int tq_quantize_wht_launch(const TqFast& f, const void* x, int32_t dtype, int64_t ld, int64_t n, const TqQuantDst& dst,
                           bool want_qjl, cudaStream_t st) {
  if (n == 0) return TQ_OK;
  TQ_REQUIRE(tq_aligned(x, 16), TQ_ERR_ALIGN, "input rows must be 16-byte aligned");
  int rc = TQ_OK;  // 16-bit inputs into a packed stream: Hadamard transform on the tensor cores
  if (tq_quantize_mma_try(f, x, dtype, ld, n, dst, want_qjl, st, &rc)) return rc;
  switch (dtype) {
    case TQ_F32:
      TQ_REQUIRE(ld % 4 == 0, TQ_ERR_ALIGN, "fp32 row stride must be a multiple of 4 elements");
      return launch_wht2<float>(f, (const float*)x, ld, n, dst, want_qjl, st);
    case TQ_F16:
      TQ_REQUIRE(ld % 8 == 0, TQ_ERR_ALIGN, "fp16 row stride must be a multiple of 8 elements");
      return launch_wht2<__half>(f, (const __half*)x, ld, n, dst, want_qjl, st);
    case TQ_BF16:
      TQ_REQUIRE(ld % 8 == 0, TQ_ERR_ALIGN, "bf16 row stride must be a multiple of 8 elements");
      return launch_wht2<__nv_bfloat16>(f, (const __nv_bfloat16*)x, ld, n, dst, want_qjl, st);
    default:
      tq_set_error("WHT quantize accepts fp32, fp16 or bf16 input, got dtype %d", dtype);
      return TQ_ERR_UNSUPPORTED;
  }
}

// ------------------------------------------------------------------------------------------
// any d, dense rotation, fp64
// ------------------------------------------------------------------------------------------
// NumPy's pairwise float summation (what np.linalg.norm(x, axis=1) runs for each contiguous row):
// fewer than 8 terms are added in order, up to 128 terms use 8 interleaved accumulators combined
// as ((r0+r1)+(r2+r3))+((r4+r5)+(r6+r7)), longer rows are split in halves (a multiple of 8).
// The square and the add are kept as separately rounded operations (no FMA contraction), as on the host.
__device__ __forceinline__ float tq_add_rn(float a, float b) { return __fadd_rn(a, b); }
__device__ __forceinline__ double tq_add_rn(double a, double b) { return __dadd_rn(a, b); }
__device__ __forceinline__ float tq_sq_rn(float a) { return __fmul_rn(a, a); }
__device__ __forceinline__ double tq_sq_rn(double a) { return __dmul_rn(a, a); }

template <typename A>
__device__ A tq_pairwise_sq(const double* xs, int stride, int n) {
  if (n < 8) {
    A r = (A)0;  // adding the first term to +0 gives the first term
    for (int i = 0; i < n; ++i) r = tq_add_rn(r, tq_sq_rn((A)xs[(size_t)i * stride]));
    return r;
  }
  if (n <= 128) {
    A r[8];
    for (int j = 0; j < 8; ++j) r[j] = tq_sq_rn((A)xs[(size_t)j * stride]);
    int i = 8;
    for (; i < n - (n % 8); i += 8)
      for (int j = 0; j < 8; ++j) r[j] = tq_add_rn(r[j], tq_sq_rn((A)xs[(size_t)(i + j) * stride]));
    A res = tq_add_rn(tq_add_rn(tq_add_rn(r[0], r[1]), tq_add_rn(r[2], r[3])),
                      tq_add_rn(tq_add_rn(r[4], r[5]), tq_add_rn(r[6], r[7])));
    for (; i < n; ++i) res = tq_add_rn(res, tq_sq_rn((A)xs[(size_t)i * stride]));
    return res;
  }
  int n2 = n / 2;
  n2 -= n2 % 8;
  return tq_add_rn(tq_pairwise_sq<A>(xs, stride, n2), tq_pairwise_sq<A>(xs + (size_t)n2 * stride, stride, n - n2));
}

template <typename T> __device__ __forceinline__ double tq_to_double(T v);
template <> __device__ __forceinline__ double tq_to_double<float>(float v) { return (double)v; }
template <> __device__ __forceinline__ double tq_to_double<double>(double v) { return v; }
template <> __device__ __forceinline__ double tq_to_double<__half>(__half v) { return (double)__half2float(v); }

struct TqDenseArgs {
  const double *rot, *rot_t, *s_t, *cent, *bnd;
  int32_t d, bits, norm_correction;
  uint8_t *out_packed, *out_idx;
  float *out_norm, *out_scale, *out_rnorm;
  uint8_t* out_qjl;
  double* out_res;  // x - dequantize(quantize(x)), fp64 rows of stride ld_res; or null
  int64_t ld_res;
};

constexpr int TV = 8;  // vectors per CTA

template <typename Tin, bool WIDE>
__global__ void __launch_bounds__(128) k_quantize_dense(const TqDenseArgs a, const Tin* __restrict__ x, int64_t ld,
                                                        int64_t n) {
  extern __shared__ __align__(16) double sm[];
  const int d = a.d, tid = threadIdx.x;
  double* xs = sm;                  // [d][TV] original values
  double* ws = sm + (size_t)d * TV; // [d][TV] work: normalised input, then centroid vector, then residual
  __shared__ double s_norm[TV], s_red[TV];
  __shared__ float s_normf[TV];
  uint8_t* s_idx = reinterpret_cast<uint8_t*>(ws + (size_t)d * TV);  // [TV][d]
  const int64_t v0 = (int64_t)blockIdx.x * TV;
  const int nv = (int)((n - v0) < TV ? (n - v0) : TV);

  for (int i = tid; i < d * TV; i += 128) {
    const int v = i / d, k = i - v * d;
    xs[(size_t)k * TV + v] = v < nv ? tq_to_double<Tin>(x[(v0 + v) * ld + k]) : 0.0;
  }
  __syncthreads();
  if (tid < TV) {
    // the reference takes the norm in the input's own precision (fp32 input -> fp32 arithmetic)
    // Same shape as NumPy's add.reduce (first term + pairwise sum of the rest).  SIMD builds of NumPy
    // order the partial sums differently, so the norm agrees to an ulp or two, not bit for bit.
    double nrm;
    if (WIDE) {
      const double s0 = tq_sq_rn(xs[tid]);
      nrm = sqrt(d > 1 ? tq_add_rn(s0, tq_pairwise_sq<double>(xs + TV + tid, TV, d - 1)) : s0);
    } else {
      const float x0 = (float)xs[tid];
      const float s0 = tq_sq_rn(x0);
      nrm = (double)sqrtf(d > 1 ? tq_add_rn(s0, tq_pairwise_sq<float>(xs + TV + tid, TV, d - 1)) : s0);
    }
    s_norm[tid] = nrm;
    s_normf[tid] = (float)nrm;
    s_red[tid] = 0.0;
  }
  __syncthreads();
  for (int i = tid; i < d * TV; i += 128) {
    const int v = i % TV;
    const double nrm = s_norm[v];
    const double safe = nrm > 0.0 ? nrm : 1.0;
    // x / safe_norm in the input's precision (turboquant/polar_quant.py:75)
    ws[i] = WIDE ? xs[i] / safe : (double)((float)xs[i] / (float)safe);
  }
  __syncthreads();
  const int nb = (1 << a.bits) - 1;
  double local_cc[TV];
#pragma unroll
  for (int v = 0; v < TV; ++v) local_cc[v] = 0.0;
  // y_j = sum_k R[j][k] xn[k]; thread j streams column j of R^T (coalesced across threads)
  for (int j = tid; j < d; j += 128) {
    double acc[TV];
#pragma unroll
    for (int v = 0; v < TV; ++v) acc[v] = 0.0;
    for (int k = 0; k < d; ++k) {
      const double r = __ldg(a.rot_t + (size_t)k * d + j);
      const double2* xv = reinterpret_cast<const double2*>(ws + (size_t)k * TV);
#pragma unroll
      for (int h = 0; h < TV / 2; ++h) {
        const double2 p = xv[h];
        acc[2 * h] = fma(r, p.x, acc[2 * h]);
        acc[2 * h + 1] = fma(r, p.y, acc[2 * h + 1]);
      }
    }
#pragma unroll
    for (int v = 0; v < TV; ++v) {
      int m = 0;
      for (int b = 0; b < nb; ++b) m += (a.bnd[b] < acc[v]) ? 1 : 0;  // searchsorted, side='left'
      s_idx[v * d + j] = (uint8_t)m;
      const double c = a.cent[m];
      local_cc[v] += c * c;
    }
  }
#pragma unroll
  for (int v = 0; v < TV; ++v) atomicAdd(&s_red[v], local_cc[v]);
  __syncthreads();  // every thread is done reading ws (normalised input)

  // outputs that only need the indices
  if (a.out_idx)
    for (int i = tid; i < nv * d; i += 128) a.out_idx[v0 * d + i] = s_idx[i];
  if (a.out_packed) {
    const int bpv = d * a.bits / 8;
    for (int i = tid; i < nv * bpv; i += 128) {
      const int v = i / bpv, o = i - v * bpv;
      uint32_t byte = 0;
      for (int bit = 0; bit < 8; ++bit) {
        const int pos = o * 8 + bit, e = pos / a.bits, r = pos - e * a.bits;
        byte = (byte << 1) | ((s_idx[v * d + e] >> (a.bits - 1 - r)) & 1u);
      }
      a.out_packed[v0 * bpv + i] = (uint8_t)byte;
    }
  }
  if (tid < nv) {
    if (a.out_norm) a.out_norm[v0 + tid] = s_normf[tid];
    double cn = sqrt(s_red[tid]);
    cn = cn > 1e-10 ? cn : 1.0;
    if (a.out_scale) a.out_scale[v0 + tid] = (float)(a.norm_correction ? (double)s_normf[tid] / cn : (double)s_normf[tid]);
  }
  if (a.out_qjl == nullptr && a.out_rnorm == nullptr && a.out_res == nullptr) return;

  // ---- residual + QJL: x_hat = norm * R^T yhat', r = x - x_hat, z = sign(S r) ----
  for (int i = tid; i < d * TV; i += 128) {
    const int k = i / TV, v = i - k * TV;
    double c = a.cent[s_idx[v * d + k]];
    if (a.norm_correction) {
      double cn = sqrt(s_red[v]);
      cn = cn > 1e-10 ? cn : 1.0;
      c = c / cn;
    }
    ws[i] = c;
  }
  __syncthreads();
  double racc[TV];
#pragma unroll
  for (int v = 0; v < TV; ++v) racc[v] = 0.0;
  // x_hat_unit[j] = sum_k R[k][j] yhat'[k]  (row k of R is contiguous in j)
  // results for all j of this thread are needed after ws is overwritten -> two passes over j-stripes,
  // each storing into xs (xs[j] is only touched by the thread that owns j)
  for (int j = tid; j < d; j += 128) {
    double acc[TV];
#pragma unroll
    for (int v = 0; v < TV; ++v) acc[v] = 0.0;
    for (int k = 0; k < d; ++k) {
      const double r = __ldg(a.rot + (size_t)k * d + j);
      const double2* yv = reinterpret_cast<const double2*>(ws + (size_t)k * TV);
#pragma unroll
      for (int h = 0; h < TV / 2; ++h) {
        const double2 p = yv[h];
        acc[2 * h] = fma(r, p.x, acc[2 * h]);
        acc[2 * h + 1] = fma(r, p.y, acc[2 * h + 1]);
      }
    }
#pragma unroll
    for (int v = 0; v < TV; ++v) {
      // x_hat = x_hat_unit * norm, residual = x - x_hat.  The norm is the one that is returned and stored (fp32):
      // the residual is then exactly x - dequantize(indices, norms) for the norms the caller holds, which is how
      // turboquant/polar_quant.py:121-132 defines it (for fp64 inputs the reference's own norm has 29 more bits;
      // norms are carried in fp32 here, 6e-8 relative)
      const double res = xs[(size_t)j * TV + v] - acc[v] * (double)s_normf[v];
      xs[(size_t)j * TV + v] = res;
      racc[v] += res * res;
      if (a.out_res && v < nv) a.out_res[(v0 + v) * a.ld_res + j] = res;
    }
  }
  if (tid < TV) s_red[tid] = 0.0;
  __syncthreads();
#pragma unroll
  for (int v = 0; v < TV; ++v) atomicAdd(&s_red[v], racc[v]);
  __syncthreads();
  if (tid < nv && a.out_rnorm) a.out_rnorm[v0 + tid] = (float)sqrt(s_red[tid]);
  if (a.out_qjl == nullptr) return;
  // p_j = sum_k S[j][k] r[k]; sign bit per j into s_idx (1 => +1)
  for (int j = tid; j < d; j += 128) {
    double acc[TV];
#pragma unroll
    for (int v = 0; v < TV; ++v) acc[v] = 0.0;
    for (int k = 0; k < d; ++k) {
      const double r = __ldg(a.s_t + (size_t)k * d + j);
      const double2* rv = reinterpret_cast<const double2*>(xs + (size_t)k * TV);
#pragma unroll
      for (int h = 0; h < TV / 2; ++h) {
        const double2 p = rv[h];
        acc[2 * h] = fma(r, p.x, acc[2 * h]);
        acc[2 * h + 1] = fma(r, p.y, acc[2 * h + 1]);
      }
    }
#pragma unroll
    for (int v = 0; v < TV; ++v) s_idx[v * d + j] = acc[v] < 0.0 ? 0 : 1;  // zero -> +1 (qjl.py:89-90)
  }
  __syncthreads();
  const int rb = (d + 7) / 8;
  for (int i = tid; i < nv * rb; i += 128) {
    const int v = i / rb, o = i - v * rb;
    uint32_t byte = 0;
    for (int bit = 0; bit < 8; ++bit) {
      const int e = o * 8 + bit;
      byte = (byte << 1) | (e < d ? s_idx[v * d + e] : 0u);
    }
    a.out_qjl[v0 * rb + i] = (uint8_t)byte;
  }
}

static int launch_dense(const tq_quantizer* q, const void* x, int32_t dtype, int64_t ld, int64_t n, TqDenseArgs& a,
                        cudaStream_t st) {
  if (n == 0) return TQ_OK;
  const size_t smem = (size_t)q->d * TV * 8 * 2 + (size_t)q->d * TV + 16;
  const int grid = (int)((n + TV - 1) / TV);
#define TQ_DENSE(T, W)                                                                                             \
  do {                                                                                                             \
    if (smem > 48 * 1024)                                                                                          \
      TQ_CUDA(cudaFuncSetAttribute(k_quantize_dense<T, W>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
    k_quantize_dense<T, W><<<grid, 128, smem, st>>>(a, (const T*)x, ld, n);                                        \
  } while (0)
  switch (dtype) {
    case TQ_F32: TQ_DENSE(float, false); break;
    case TQ_F16: TQ_DENSE(__half, false); break;
    case TQ_F64: TQ_DENSE(double, true); break;
    default:
      tq_set_error("dense quantize accepts fp32, fp16 or fp64 input, got dtype %d", dtype);
      return TQ_ERR_UNSUPPORTED;
  }
#undef TQ_DENSE
  return tq_launch_check("k_quantize_dense");
}

extern "C" int tq_quantize(const tq_quantizer* q, const void* x_dev, int32_t x_dtype, int64_t ld, int64_t n,
                           uint8_t* out_packed_dev, uint8_t* out_idx_dev, float* out_norm_dev, float* out_scale_dev,
                           uint8_t* out_qjl_dev, float* out_rnorm_dev, void* stream) {
  TQ_REQUIRE(q, TQ_ERR_INVALID, "tq_quantize: quantizer is null");
  TQ_REQUIRE(q->rotation == TQ_ROT_WHT || q->rot, TQ_ERR_INVALID, "tq_quantize: quantizer was created without a rotation");
  TQ_REQUIRE(n >= 0, TQ_ERR_INVALID, "tq_quantize: n must be >= 0");
  if (n == 0) return TQ_OK;
  TQ_REQUIRE(x_dev, TQ_ERR_INVALID, "tq_quantize: x is null");
  TQ_REQUIRE(ld >= q->d, TQ_ERR_INVALID, "tq_quantize: row stride %lld smaller than d", (long long)ld);
  const bool want_qjl = out_qjl_dev != nullptr || out_rnorm_dev != nullptr;
  TQ_REQUIRE(!want_qjl || q->qjl, TQ_ERR_INVALID, "tq_quantize: QJL outputs requested from a quantizer without a QJL stage");
  TQ_REQUIRE(!out_packed_dev || (q->d * q->bits) % 8 == 0, TQ_ERR_UNSUPPORTED,
             "per-vector packed output needs d*bits to be a multiple of 8");
  cudaStream_t st = (cudaStream_t)stream;
  if (q->rotation == TQ_ROT_WHT) {
    TQ_REQUIRE(!out_packed_dev || tq_aligned(out_packed_dev, 16), TQ_ERR_ALIGN, "packed output must be 16-byte aligned");
    TQ_REQUIRE(!out_idx_dev || tq_aligned(out_idx_dev, 16), TQ_ERR_ALIGN, "index output must be 16-byte aligned");
    TQ_REQUIRE(!out_qjl_dev || tq_aligned(out_qjl_dev, 16), TQ_ERR_ALIGN, "QJL output must be 16-byte aligned");
    TqQuantDst dst;
    memset(&dst, 0, sizeof(dst));
    dst.idx = out_packed_dev;
    dst.idx_u8 = out_idx_dev;
    dst.norm = out_norm_dev;
    dst.scale = out_scale_dev;
    dst.qjl = out_qjl_dev;
    dst.rnorm = out_rnorm_dev;
    dst.heads = 1;
    return tq_quantize_wht_launch(q->fast, x_dev, x_dtype, ld, n, dst, want_qjl, st);
  }
  TqDenseArgs a;
  memset(&a, 0, sizeof(a));
  a.rot = q->rot;
  a.rot_t = q->rot_t;
  a.s_t = q->s_t;
  a.cent = q->cent64;
  a.bnd = q->bnd64;
  a.d = q->d;
  a.bits = q->bits;
  a.norm_correction = q->norm_correction;
  a.out_packed = out_packed_dev;
  a.out_idx = out_idx_dev;
  a.out_norm = out_norm_dev;
  a.out_scale = out_scale_dev;
  a.out_qjl = out_qjl_dev;
  a.out_rnorm = out_rnorm_dev;
  return launch_dense(q, x_dev, x_dtype, ld, n, a, st);
}

extern "C" int tq_quantize_residual(const tq_quantizer* q, const void* x_dev, int32_t x_dtype, int64_t ld, int64_t n,
                                    uint8_t* out_idx_dev, float* out_norm_dev, double* out_residual_dev,
                                    int64_t ld_res, void* stream) {
  TQ_REQUIRE(q, TQ_ERR_INVALID, "tq_quantize_residual: quantizer is null");
  TQ_REQUIRE(q->rotation == TQ_ROT_DENSE && q->rot, TQ_ERR_UNSUPPORTED,
             "tq_quantize_residual: needs a dense-mode quantizer with a rotation");
  TQ_REQUIRE(n >= 0, TQ_ERR_INVALID, "tq_quantize_residual: n must be >= 0");
  if (n == 0) return TQ_OK;
  TQ_REQUIRE(x_dev && out_residual_dev, TQ_ERR_INVALID, "tq_quantize_residual: null buffer");
  TQ_REQUIRE(ld >= q->d && ld_res >= q->d, TQ_ERR_INVALID, "tq_quantize_residual: row strides %lld / %lld smaller than d",
             (long long)ld, (long long)ld_res);
  TQ_REQUIRE(tq_aligned(out_residual_dev, 8), TQ_ERR_ALIGN, "tq_quantize_residual: residual rows must be 8-byte aligned");
  TqDenseArgs a;
  memset(&a, 0, sizeof(a));
  a.rot = q->rot;
  a.rot_t = q->rot_t;
  a.cent = q->cent64;
  a.bnd = q->bnd64;
  a.d = q->d;
  a.bits = q->bits;
  a.norm_correction = q->norm_correction;
  a.out_idx = out_idx_dev;
  a.out_norm = out_norm_dev;
  a.out_res = out_residual_dev;
  a.ld_res = ld_res;
  return launch_dense(q, x_dev, x_dtype, ld, n, a, (cudaStream_t)stream);
}

// ------------------------------------------------------------------------------------------
// q8_0: per 32 values an fp16 scale d = max|x|/127 and int8 round-half-away(x / d)
// ------------------------------------------------------------------------------------------
template <typename Tin>
__global__ void __launch_bounds__(256) k_q8_0_append(const Tin* __restrict__ x, int64_t n_vec, int32_t heads,
                                                     uint8_t* q_base, uint8_t* scale_base,
                                                     const int64_t* __restrict__ slots, int32_t page_tokens,
                                                     int64_t page_stride, int64_t head_stride) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // see k_quantize_wht
  const int lane = threadIdx.x & 31, sub = lane & 7;
  const int64_t v = ((int64_t)blockIdx.x * 256 + threadIdx.x) >> 3;
  const bool ok = v < n_vec;
  float u[16];
  if (ok) {
    TqLoad16<Tin>::load(x + v * TQ_D + sub * 16, u);
  } else {
#pragma unroll
    for (int k = 0; k < 16; ++k) u[k] = 0.f;
  }
  float amax = 0.f;
#pragma unroll
  for (int k = 0; k < 16; ++k) amax = fmaxf(amax, fabsf(u[k]));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));  // a 32-value block spans two lanes
  const float dd = amax / 127.0f;
  const float id = dd > 0.f ? 1.0f / dd : 0.f;
  uint32_t w[4] = {0, 0, 0, 0};
#pragma unroll
  for (int k = 0; k < 16; ++k) {
    const int qv = (int)roundf(u[k] * id);
    w[k >> 2] |= ((uint32_t)(qv & 0xff)) << (8 * (k & 3));
  }
  if (!ok) return;
  const int64_t tok = v / heads;
  const int32_t head = (int32_t)(v - tok * heads);
  const int64_t slot = slots ? slots[tok] : tok;
  if (slot < 0) return;
  const int64_t page = slot / page_tokens;
  const int32_t within = (int32_t)(slot - page * page_tokens);
  const int64_t rec = page * page_stride + head * head_stride;
  *reinterpret_cast<uint4*>(q_base + rec + (int64_t)within * TQ_D + sub * 16) = make_uint4(w[0], w[1], w[2], w[3]);
  if ((sub & 1) == 0)
    *reinterpret_cast<__half*>(scale_base + rec + (int64_t)within * 8 + (sub >> 1) * 2) = __float2half_rn(dd);
}

int tq_q8_0_append_launch(const void* x, int32_t dtype, int64_t n_tokens, int32_t heads, uint8_t* q_base,
                          uint8_t* scale_base, const int64_t* slots, int32_t page_tokens, int64_t page_stride,
                          int64_t head_stride, cudaStream_t st) {
  const int64_t n_vec = n_tokens * heads;
  if (n_vec == 0) return TQ_OK;
  TQ_REQUIRE(tq_aligned(x, 16), TQ_ERR_ALIGN, "input must be 16-byte aligned");
  const int grid = (int)((n_vec * 8 + 255) / 256);
  switch (dtype) {
    case TQ_F32:
      k_q8_0_append<float><<<grid, 256, 0, st>>>((const float*)x, n_vec, heads, q_base, scale_base, slots, page_tokens,
                                                  page_stride, head_stride);
      break;
    case TQ_F16:
      k_q8_0_append<__half><<<grid, 256, 0, st>>>((const __half*)x, n_vec, heads, q_base, scale_base, slots,
                                                   page_tokens, page_stride, head_stride);
      break;
    case TQ_BF16:
      k_q8_0_append<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)x, n_vec, heads, q_base, scale_base,
                                                          slots, page_tokens, page_stride, head_stride);
      break;
    default:
      tq_set_error("q8_0 append accepts fp32, fp16 or bf16 input, got dtype %d", dtype);
      return TQ_ERR_UNSUPPORTED;
  }
  return tq_launch_check("k_q8_0_append");
}
