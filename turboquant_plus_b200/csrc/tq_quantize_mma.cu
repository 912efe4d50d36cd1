// d = 128 sign-WHT quantizer with the Hadamard transform on the tensor cores.
//
//   k_quantize_mma<Tin, BITS, NORMC>   Tin = __half, __nv_bfloat16 or float, symmetric codebook, packed output.
//
// H128 = H8 (x) H16 (element e = 16 i + j).  A warp takes 16 vectors at a time:
//   * the 16 x 128 tile is copied to shared memory with 16-byte asynchronous copies (double buffered) and read
//     back as MMA operands with ldmatrix (rows padded to 272 bytes so that the eight rows of a matrix fall into
//     different bank groups);
//   * for each i, one m16n8k16 MMA per 8 output columns contracts the 16 inputs x[v][16 i + j'] with
//     sign1[16 i + j'] * H16[j'][j].  Inputs are 16-bit, the matrix entries are +-1: every product is exact and
//     the sums are accumulated in fp32;
//   * the 16 output columns are dealt to the two n-tiles so that thread (g, t) holds, for vectors g and g + 8 and
//     for every i, the four consecutive columns j = 4 t .. 4 t + 3: the 8-point transform over i is three butterfly
//     stages in its own registers (the last one negated, so that the sign bit alone decides the centre boundary);
//   * ||x|| is taken from the transformed values (||H x||^2 = 128 ||x||^2), magnitudes are compared against the
//     positive boundaries scaled by ||x|| sqrt(d) (two tests for 3 bits), sign2 mirrors the index by an XOR, eight
//     indices at a time are packed by an exact fp32 Horner sum, and the norm correction comes from a
//     population-count histogram of the magnitude levels;
//   * a 4 x 4 transpose of words inside each quad of lanes leaves every lane with 32 consecutive indices of its
//     vector, which it stores as the reference's most-significant-bit-first stream (turboquant/utils.py pack_indices
//     order, the layout the cache keeps).
//   * fp32 inputs are split into three bf16 terms (8 + 8 + 8 significant bits, by truncation: the split is exact)
//     that go through the same MMAs one after the other into one fp32 accumulator; products with +-1 stay exact.
//   * QJLS (PROD keys with a 2..4-bit PolarQuant stage): the residual against the chosen centroids is formed in place
//     in the rotated domain, its norm taken, and sign(S r) computed as two more 128-point transforms in the same
//     register layout (element 16 i + 4 t + c of lane t: the bits of i and c are butterflies in registers, the two
//     bits of t two lane exchanges), with the sign flips in between from a lane-indexed table in shared memory.
// Everything else (1-bit PolarQuant stages, asymmetric codebooks, unpacked output) stays with k_quantize_wht.
#include "tq_internal.cuh"

namespace {

constexpr int QM_THREADS = 128;
constexpr int QM_WARPS = 4;
constexpr int QM_ROWS = 16;
// bytes between the rows of a staged tile: 16-bit rows 256 + 16 (the eight rows of an ldmatrix fall into different bank
// groups), fp32 rows 512 + 32 (rows g = 0..3 of a half-warp's 8-byte loads start 8 banks apart)
template <typename T> constexpr int qm_rowb() { return sizeof(T) == 4 ? 544 : 272; }

template <typename T> struct QmIn;
template <> struct QmIn<__half> {
  static constexpr uint32_t ONE = 0x3C00u, MINUS = 0xBC00u;
  // c = a . b (zero accumulator)
  static __device__ __forceinline__ void mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(0.f));
  }
};
template <> struct QmIn<__nv_bfloat16> {
  static constexpr uint32_t ONE = 0x3F80u, MINUS = 0xBF80u;
  static __device__ __forceinline__ void mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(0.f));
  }
  // c += a . b
  static __device__ __forceinline__ void mma_acc(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
};
template <> struct QmIn<float> : QmIn<__nv_bfloat16> {};   // fp32 rows are fed as bf16 terms

// (x0, x1) = hi + mid + lo, each term a pair of bf16 values obtained by truncation: every term keeps the eight leading
// significant bits of what is left, so three terms hold all 24 and every subtraction is exact.  Low half = x0.
__device__ __forceinline__ void qm_split3(float x0, float x1, uint32_t& hi, uint32_t& mid, uint32_t& lo) {
  const uint32_t u0 = __float_as_uint(x0), u1 = __float_as_uint(x1);
  hi = __byte_perm(u0, u1, 0x7632);
  const float r0 = x0 - __uint_as_float(u0 & 0xffff0000u), r1 = x1 - __uint_as_float(u1 & 0xffff0000u);
  const uint32_t v0 = __float_as_uint(r0), v1 = __float_as_uint(r1);
  mid = __byte_perm(v0, v1, 0x7632);
  const float s0 = r0 - __uint_as_float(v0 & 0xffff0000u), s1 = r1 - __uint_as_float(v1 & 0xffff0000u);
  lo = __byte_perm(__float_as_uint(s0), __float_as_uint(s1), 0x7632);
}

__device__ __forceinline__ uint32_t qm_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint32_t qm_bit(const uint32_t (&m)[4], int e) { return (m[e >> 5] >> (e & 31)) & 1u; }
// 1.0f when a > b, else 0.0f, in one instruction
__device__ __forceinline__ float qm_gt(float a, float b) {
  float d;
  asm("set.gt.f32.f32 %0, %1, %2;" : "=f"(d) : "f"(a), "f"(b));
  return d;
}

// packed fp32 arithmetic (two operations per instruction); operands are register pairs as the MMA leaves them
__device__ __forceinline__ float2 qm_add2(float2 a, float2 b) {
  float2 d;
  asm("{\n .reg .b64 ra, rb, rd;\n mov.b64 ra, {%2, %3};\n mov.b64 rb, {%4, %5};\n add.rn.f32x2 rd, ra, rb;\n mov.b64 {%0, %1}, rd;\n}\n"
      : "=f"(d.x), "=f"(d.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
  return d;
}
__device__ __forceinline__ float2 qm_sub2(float2 a, float2 b) {
  float2 d;
  asm("{\n .reg .b64 ra, rb, rd;\n mov.b64 ra, {%2, %3};\n mov.b64 rb, {%4, %5};\n sub.rn.f32x2 rd, ra, rb;\n mov.b64 {%0, %1}, rd;\n}\n"
      : "=f"(d.x), "=f"(d.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
  return d;
}
__device__ __forceinline__ float2 qm_mul2(float2 a, float2 b) {
  float2 d;
  asm("{\n .reg .b64 ra, rb, rd;\n mov.b64 ra, {%2, %3};\n mov.b64 rb, {%4, %5};\n mul.rn.f32x2 rd, ra, rb;\n mov.b64 {%0, %1}, rd;\n}\n"
      : "=f"(d.x), "=f"(d.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
  return d;
}
__device__ __forceinline__ float2 qm_fma2(float2 a, float2 b, float2 c) {
  float2 d;
  asm("{\n .reg .b64 ra, rb, rc, rd;\n mov.b64 ra, {%2, %3};\n mov.b64 rb, {%4, %5};\n mov.b64 rc, {%6, %7};\n"
      " fma.rn.f32x2 rd, ra, rb, rc;\n mov.b64 {%0, %1}, rd;\n}\n"
      : "=f"(d.x), "=f"(d.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y), "f"(c.x), "f"(c.y));
  return d;
}
__device__ __forceinline__ float2 qm_dup(float v) { return make_float2(v, v); }

// `tile`: the CTA's staging memory, QM_WARPS x 2 buffers of QM_ROWS rows of qm_rowb<Tin>() bytes, then 4 KB for the
// B operands of the MMAs
template <typename Tin, int BITS, bool NORMC, bool QJLS = false>
__device__ __forceinline__ void qm_body(const TqFast& f, const Tin* __restrict__ x, int64_t ld, int64_t n,
                                        const TqQuantDst& dst, uint8_t* tile) {
  // a dependent kernel launched with programmatic stream serialization may start now (it waits for this grid's
  // completion itself before it touches what this grid writes); without such a dependent this does nothing
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  constexpr int QM_ROWB = qm_rowb<Tin>();
  constexpr int BUFB = QM_ROWS * QM_ROWB;                      // bytes of one staged tile
  constexpr int CHUNKS = (int)(TQ_D * sizeof(Tin) / 16);       // 16-byte chunks per row
  constexpr int NC = 1 << BITS, HALF = NC / 2, NT = HALF - 1;  // NT positive boundaries
  constexpr int IDXB = 16 * BITS;
  constexpr float RADIX = (float)NC;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;

  // B operands: rows k = 2t, 2t+1 (register 0) and 2t+8, 2t+9 (register 1) of sign1 * H16.  The 16 output columns
  // are dealt to the two n-tiles so that the accumulator columns of lane t (2t, 2t+1 of each tile) are the four
  // consecutive outputs j = 4t .. 4t+3.
  // They depend on the lane only: the warps write them to shared memory once ([i][lane] x 16 bytes, two values of i
  // per warp) and every warp reads the four words of a step just before its two MMAs -- 32 registers less per thread,
  // a fifth CTA per SM.
  uint8_t* bsm = tile + QM_WARPS * 2 * BUFB;
  {
#pragma unroll
    for (int ii = 0; ii < 8 / QM_WARPS; ++ii) {
      const int i = warp * (8 / QM_WARPS) + ii;
      uint32_t b4[4];
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int col = 4 * (g >> 1) + 2 * nt + (g & 1);  // this lane's B column g of tile nt is output j = col
          uint32_t r = 0;
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int k = 2 * t + 8 * h + e;
            const uint32_t neg = qm_bit(f.s1, 16 * i + k) ^ (uint32_t)(__popc(k & col) & 1);
            r |= (neg ? QmIn<Tin>::MINUS : QmIn<Tin>::ONE) << (16 * e);
          }
          b4[2 * nt + h] = r;
        }
      *reinterpret_cast<uint4*>(bsm + (i * 32 + lane) * 16) = make_uint4(b4[0], b4[1], b4[2], b4[3]);
    }
  }
  // QJL stage: +-1 factors of sign1 ^ j1 for this lane's 32 elements, [i][lane] x (c = 0..3), and the j2 flips as a
  // mask word in the order the sketch bits are gathered (i, then c, most significant first)
  float4* m12f = reinterpret_cast<float4*>(bsm + 8 * 32 * 16);
  uint32_t j2w = 0;
  if constexpr (QJLS) {
    {
#pragma unroll
      for (int ii = 0; ii < 8 / QM_WARPS; ++ii) {
        const int i = warp * (8 / QM_WARPS) + ii;
        float v4[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) v4[c] = (qm_bit(f.s1, 16 * i + 4 * t + c) ^ qm_bit(f.j1, 16 * i + 4 * t + c)) ? -1.0f : 1.0f;
        m12f[i * 32 + lane] = make_float4(v4[0], v4[1], v4[2], v4[3]);
      }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int c = 0; c < 4; ++c) j2w = (j2w << 1) | qm_bit(f.j2, 16 * i + 4 * t + c);
  }
  __syncthreads();
  const uint4* bfr4 = reinterpret_cast<const uint4*>(bsm) + lane;
  // sign2 mirrors an index (i -> 2^b - 1 - i): an XOR of the packed word.  Word tp of this lane packs, most
  // significant first, the elements 16 (2 tp + (k >> 2)) + 4 t + (k & 3), k = 0..7.
  uint32_t flip[4];
#pragma unroll
  for (int tp = 0; tp < 4; ++tp) {
    uint32_t m = 0;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const int e = 16 * (2 * tp + (k >> 2)) + 4 * t + (k & 3);
      if (qm_bit(f.s2, e)) m |= (uint32_t)(NC - 1) << (BITS * (7 - k));
    }
    flip[tp] = m;
  }
  float bnd[NT > 0 ? NT : 1], dsq[NT > 0 ? NT : 1];  // positive boundaries; steps of the squared centroids
#pragma unroll
  for (int j = 0; j < NT; ++j) {
    bnd[j] = f.bnd[HALF + j];
    dsq[j] = f.cent[HALF + j + 1] * f.cent[HALF + j + 1] - f.cent[HALF + j] * f.cent[HALF + j];
  }
  const float c0sq = f.cent[HALF] * f.cent[HALF];
  // QJL stage: the chosen centroid's magnitude from the test results.  3 bits (levels 2 p2 + p1): c4 + p2 (c6 - c4) +
  // p1 ((c5 - c4) + p2 ((c7 - c6) - (c5 - c4))); otherwise the first magnitude and the steps between neighbours.
  float cst[HALF > 3 ? HALF : 4];
  if constexpr (BITS == 3) {
    cst[0] = f.cent[4];
    cst[1] = f.cent[6] - f.cent[4];
    cst[2] = f.cent[5] - f.cent[4];
    cst[3] = (f.cent[7] - f.cent[6]) - (f.cent[5] - f.cent[4]);
  } else {
    cst[0] = f.cent[HALF];
#pragma unroll
    for (int j = 0; j < NT; ++j) cst[1 + j] = f.cent[HALF + j + 1] - f.cent[HALF + j];
  }
  const uint32_t zero_idx = 0.f > f.bnd[HALF - 1] ? HALF : HALF - 1;   // index of the value 0

  const int64_t ntiles = (n + QM_ROWS - 1) / QM_ROWS;
  const int64_t stride = (int64_t)gridDim.x * QM_WARPS;
  int64_t ti = (int64_t)blockIdx.x * QM_WARPS + warp;
  uint8_t* wtile = tile + (size_t)warp * 2 * BUFB;
  // a lane copies the same 16-byte chunk of rows row0, row0 + RSTEP, ... of every tile
  constexpr int RSTEP = 32 / CHUNKS;
  const int row0 = lane / CHUNKS;
  const uint8_t* xlane = reinterpret_cast<const uint8_t*>(x + (int64_t)row0 * ld) + (lane % CHUNKS) * 16;
  const int64_t row_step = (int64_t)RSTEP * ld * (int64_t)sizeof(Tin), tile_step = (int64_t)QM_ROWS * ld * (int64_t)sizeof(Tin);
  const uint32_t slane = qm_smem(wtile) + row0 * QM_ROWB + (lane % CHUNKS) * 16;
  auto issue = [&](int64_t tile_i, int buf) {
    const int64_t v0 = tile_i * QM_ROWS;
    const uint8_t* src = xlane + tile_i * tile_step;
    const uint32_t sdst = slane + buf * BUFB;
    if (v0 + QM_ROWS <= n) {   // a whole tile (all but the last one): no row tests
#pragma unroll
      for (int r2 = 0; r2 < QM_ROWS / RSTEP; ++r2) {
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(sdst + r2 * RSTEP * QM_ROWB), "l"(src) : "memory");
        src += row_step;
      }
    } else {
#pragma unroll
      for (int r2 = 0; r2 < QM_ROWS / RSTEP; ++r2) {
        if (v0 + row0 + r2 * RSTEP < n)
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(sdst + r2 * RSTEP * QM_ROWB), "l"(src) : "memory");
        src += row_step;
      }
    }
  };
  if (ti < ntiles) issue(ti, 0);
  asm volatile("cp.async.commit_group;" ::: "memory");

  for (int it = 0; ti < ntiles; ti += stride, ++it) {
    if (ti + stride < ntiles) issue(ti + stride, (it + 1) & 1);
    asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group 1;" ::: "memory");
    __syncwarp();
    const int64_t v0 = ti * QM_ROWS;

    // ---- 16-point stage on the tensor cores ----
    float acc[8][2][4];
    if constexpr (sizeof(Tin) == 4) {
      // thread (g, t): rows g and g + 8, columns 16 i + 2t, + 1 (registers 0, 1) and 16 i + 2t + 8, + 9 (2, 3)
      const uint8_t* abase = wtile + (it & 1) * BUFB + g * QM_ROWB + 8 * t;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float2 x0 = *reinterpret_cast<const float2*>(abase + 64 * i);
        const float2 x1 = *reinterpret_cast<const float2*>(abase + 8 * QM_ROWB + 64 * i);
        const float2 x2 = *reinterpret_cast<const float2*>(abase + 64 * i + 32);
        const float2 x3 = *reinterpret_cast<const float2*>(abase + 8 * QM_ROWB + 64 * i + 32);
        uint32_t a[3][4];
        qm_split3(x0.x, x0.y, a[0][0], a[1][0], a[2][0]);
        qm_split3(x1.x, x1.y, a[0][1], a[1][1], a[2][1]);
        qm_split3(x2.x, x2.y, a[0][2], a[1][2], a[2][2]);
        qm_split3(x3.x, x3.y, a[0][3], a[1][3], a[2][3]);
        const uint4 b4 = bfr4[32 * i];
        const uint32_t bfr[2][2] = {{b4.x, b4.y}, {b4.z, b4.w}};
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
          QmIn<Tin>::mma(acc[i][nt], a[0], bfr[nt][0], bfr[nt][1]);
          QmIn<Tin>::mma_acc(acc[i][nt], a[1], bfr[nt][0], bfr[nt][1]);
          QmIn<Tin>::mma_acc(acc[i][nt], a[2], bfr[nt][0], bfr[nt][1]);
        }
      }
    } else {
      const uint32_t abase = qm_smem(wtile + (it & 1) * BUFB) + ((lane & 7) + 8 * ((lane >> 3) & 1)) * QM_ROWB + 16 * (lane >> 4);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        uint32_t a[4];
        asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                     : "=r"(a[0]), "=r"(a[1]), "=r"(a[2]), "=r"(a[3])
                     : "r"(abase + 32 * i));
        const uint4 b4 = bfr4[32 * i];
        QmIn<Tin>::mma(acc[i][0], a, b4.x, b4.y);
        QmIn<Tin>::mma(acc[i][1], a, b4.z, b4.w);
      }
    }
    // ---- 8-point stage over i, in registers ----
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int r = 0; r < 4; r += 2)   // register pairs (r, r + 1): two butterflies per instruction
#pragma unroll
        for (int h = 1; h < 8; h <<= 1)
#pragma unroll
          for (int i = 0; i < 8; ++i)
            if ((i & h) == 0) {
              const float2 a = make_float2(acc[i][nt][r], acc[i][nt][r + 1]);
              const float2 b = make_float2(acc[i + h][nt][r], acc[i + h][nt][r + 1]);
              float2 lo, hi;
              if (h < 4) {
                lo = qm_add2(a, b);
                hi = qm_sub2(a, b);
              } else {
                // The last stage produces the NEGATED transform, (-a) - b and b - a: "sign bit clear" then means
                // value <= 0 for every nonzero value and for zeros that arise by cancellation (x - x = +0), which is
                // how the reference decides the centre boundary (not above it -> lower index).  A zero formed from
                // two zero inputs can come out as -0 and take the upper of the two central indices; it sits exactly
                // on the boundary.
                const float2 na = qm_mul2(a, qm_dup(-1.0f));
                lo = qm_sub2(na, b);
                hi = qm_add2(b, na);
              }
              acc[i][nt][r] = lo.x; acc[i][nt][r + 1] = lo.y;
              acc[i + h][nt][r] = hi.x; acc[i + h][nt][r + 1] = hi.y;
            }

    // ---- the lane's two vectors: rows g (registers 0,1) and g + 8 (registers 2,3) ----
#pragma unroll
    for (int vs = 0; vs < 2; ++vs) {
      const int64_t v = v0 + g + 8 * vs;
      const bool ok = v < n;
      float2 ss2 = make_float2(0.f, 0.f);
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
          const float2 y = make_float2(acc[i][nt][2 * vs], acc[i][nt][2 * vs + 1]);
          ss2 = qm_fma2(y, y, ss2);
        }
      float ss = ss2.x + ss2.y;
      ss += __shfl_xor_sync(0xffffffffu, ss, 1);
      ss += __shfl_xor_sync(0xffffffffu, ss, 2);
      const float nrm = sqrtf(ss) * TQ_RSQRT_D;          // ||H x|| = sqrt(d) ||x||
      const float safe = nrm > 0.f ? nrm : 1.0f;          // turboquant/polar_quant.py:74
      const float ts = safe * TQ_SQRT_D;                  // the values are y * ||x|| * sqrt(d), y the rotated unit vector
      float thr[NT > 0 ? NT : 1];
#pragma unroll
      for (int j = 0; j < NT; ++j) thr[j] = bnd[j] * ts;
      const float d31 = BITS == 3 ? thr[2] - thr[0] : 0.f;

      float2 cc2 = make_float2(0.f, 0.f);
      uint32_t w[4];
#pragma unroll
      for (int tp = 0; tp < 4; ++tp) {
        // Coordinates in pairs (the two columns of an accumulator row), digits in two Horner chains of radix
        // RADIX^2 -- the even and the odd digits of a word -- joined at the end: every sum stays a half-integer
        // below 2^23, exact in fp32.
        constexpr int HG = BITS == 4 ? 4 : 8;              // digits per exact fp32 Horner sum (<= 24 bits)
        float2 ch[8 / HG];
#pragma unroll
        for (int q = 0; q < 8 / HG; ++q) ch[q] = make_float2(0.f, 0.f);
#pragma unroll
        for (int k = 0; k < 8; k += 2) {
          // minus the transformed values of elements k and k + 1 of the word
          const float2 nu = make_float2(acc[2 * tp + (k >> 2)][(k >> 1) & 1][2 * vs], acc[2 * tp + (k >> 2)][(k >> 1) & 1][2 * vs + 1]);
          const float a0 = fabsf(nu.x), a1 = fabsf(nu.y);
          float2 m5;                                       // magnitude level + 1/2
          if constexpr (BITS == 3) {
            // two tests instead of three: against the middle boundary, then against the lower or the upper one
            // (picked arithmetically; the upper one is thr[0] + d31, within an ulp of thr[2])
            const float2 p2 = make_float2(qm_gt(a0, thr[1]), qm_gt(a1, thr[1]));
            const float2 th = qm_fma2(p2, qm_dup(d31), qm_dup(thr[0]));
            const float2 p1 = make_float2(qm_gt(a0, th.x), qm_gt(a1, th.y));
            m5 = qm_fma2(p2, qm_dup(2.0f), qm_add2(p1, qm_dup(0.5f)));
          } else {
            m5 = make_float2(0.5f, 0.5f);
#pragma unroll
            for (int j = 0; j < NT; ++j) {
              const float2 p = make_float2(qm_gt(a0, thr[j]), qm_gt(a1, thr[j]));
              m5 = qm_add2(m5, p);
              if (NORMC && BITS == 4) cc2 = qm_fma2(p, qm_dup(dsq[j]), cc2);
            }
          }
          // index = HALF - 1/2 + sign * m5, sign = -1 where the value is <= 0, i.e. where nu's sign bit is clear
          const float2 digit = make_float2(__int_as_float(__float_as_int(m5.x) | (~__float_as_int(nu.x) & 0x80000000)),
                                           __int_as_float(__float_as_int(m5.y) | (~__float_as_int(nu.y) & 0x80000000)));
          ch[k / HG] = qm_fma2(ch[k / HG], qm_dup(RADIX * RADIX), digit);
        }
        float wf[8 / HG];
#pragma unroll
        for (int q = 0; q < 8 / HG; ++q) wf[q] = fmaf(ch[q].x, RADIX, ch[q].y);
        // + (HALF - 1/2) in every digit turns the signed digits into indices; the sums are whole numbers < 2^24
        if constexpr (BITS == 4) {
          constexpr float OFF = 7.5f * 4369.0f;            // 4369 = (16^4 - 1) / 15
          w[tp] = (__float2uint_rn(wf[0] + OFF) << 16) | __float2uint_rn(wf[1] + OFF);
        } else {
          constexpr float OFF = ((float)HALF - 0.5f) * (float)(((1u << (8 * BITS)) - 1) / (NC - 1));
          w[tp] = __float2uint_rn(wf[0] + OFF);
        }
        // a zero vector takes the index of the value 0 in every coordinate (no mirroring either): the upper central
        // index when the centre boundary, a midpoint of two fp64 centroids, has come out a hair below zero
        constexpr uint32_t ONES = (uint32_t)(((1ull << (8 * BITS)) - 1) / (NC - 1));   // bit 0 of every field
        w[tp] = nrm > 0.f ? (w[tp] ^ flip[tp]) : ONES * zero_idx;
      }
      float invn = 1.0f;
      float cc = cc2.x + cc2.y;
      if (NORMC && BITS != 4) {
        // ||c[idx]||^2 from a histogram of magnitude levels: field = [s | low], level m = s ? low : ~low, and
        // n_j = #{m >= j} is a population count over the packed words (mirroring an index keeps its level)
        constexpr uint32_t M0 = (uint32_t)(((1ull << (8 * BITS)) - 1) / (NC - 1));  // bit 0 of every field
        uint32_t n1 = 0, n2 = 0, n3 = 0;
#pragma unroll
        for (int tp = 0; tp < 4; ++tp) {
          const uint32_t sneg = ~(w[tp] >> (BITS - 1)) & M0;               // fields with s = 0
          const uint32_t xw = w[tp] ^ (sneg * (uint32_t)(HALF - 1));        // low bits complemented there
          if (BITS == 3) {
            const uint32_t b0 = xw & M0, b1 = (xw >> 1) & M0;
            n1 += __popc(b0 | b1);
            n2 += __popc(b1);
            n3 += __popc(b0 & b1);
          } else {
            n1 += __popc(xw & M0);
          }
        }
        cc = (float)n1 * dsq[0];
        if (BITS == 3) cc = fmaf((float)n2, dsq[1], fmaf((float)n3, dsq[2], cc));
      }
      if (NORMC) {
        cc += __shfl_xor_sync(0xffffffffu, cc, 1);
        cc += __shfl_xor_sync(0xffffffffu, cc, 2);
        float cn = sqrtf(fmaf((float)TQ_D, c0sq, cc));
        cn = cn > 1e-10f ? cn : 1.0f;                      // turboquant/polar_quant.py:110-111
        invn = 1.0f / cn;
      }
      // ---- 4 x 4 transpose inside the quad: afterwards w[s] is the word lane s packed for this lane ----
      {
        const bool b0 = t & 1, b1 = t & 2;
#pragma unroll
        for (int jb = 0; jb < 4; jb += 2) {
          const uint32_t send = b0 ? w[jb] : w[jb + 1];
          const uint32_t recv = __shfl_xor_sync(0xffffffffu, send, 1);
          if (b0) w[jb] = recv; else w[jb + 1] = recv;
        }
#pragma unroll
        for (int jb = 0; jb < 2; ++jb) {
          const uint32_t send = b1 ? w[jb] : w[jb + 2];
          const uint32_t recv = __shfl_xor_sync(0xffffffffu, send, 2);
          if (b1) w[jb] = recv; else w[jb + 2] = recv;
        }
      }
      // w[s] = [run(2t, s) | run(2t+1, s)], run(i, s) = the indices of elements 16 i + 4 s .. + 3 (4 BITS bits).
      // This lane's 32 consecutive elements are run(2t,0..3) run(2t+1,0..3): 32 BITS bits, most significant first.
      constexpr int RW = 4 * BITS;
      bool good = ok;
      int64_t within = 0;
      const int64_t rec_off = ok ? tq_dst_record(dst, v, within, good) : 0;
      if (good && dst.idx) {
        {
          uint8_t* p = dst.idx + rec_off + within * IDXB + 4 * BITS * t;
          if (BITS == 3) {
            const uint32_t h0 = w[0] >> RW, h1 = w[1] >> RW, h2 = w[2] >> RW, h3 = w[3] >> RW;
            const uint32_t l0 = w[0] & 0xfffu, l1 = w[1] & 0xfffu, l2 = w[2] & 0xfffu, l3 = w[3] & 0xfffu;
            uint32_t* p32 = reinterpret_cast<uint32_t*>(p);
            p32[0] = __byte_perm((h0 << 20) | (h1 << 8) | (h2 >> 4), 0, 0x0123);
            p32[1] = __byte_perm((h2 << 28) | (h3 << 16) | (l0 << 4) | (l1 >> 8), 0, 0x0123);
            p32[2] = __byte_perm((l1 << 24) | (l2 << 12) | l3, 0, 0x0123);
          } else if (BITS == 2) {
            // 8-bit runs: bytes h0 h1 h2 h3 l0 l1 l2 l3 in memory order
            const uint32_t a01 = __byte_perm(w[0], w[1], 0x4051), a23 = __byte_perm(w[2], w[3], 0x4051);  // bytes h h l l
            *reinterpret_cast<uint2*>(p) = make_uint2(__byte_perm(a01, a23, 0x5410), __byte_perm(a01, a23, 0x7632));
          } else {
            // 16-bit runs: big-endian halves h0 h1 h2 h3 l0 l1 l2 l3
            *reinterpret_cast<uint4*>(p) = make_uint4(__byte_perm(w[0], w[1], 0x6723), __byte_perm(w[2], w[3], 0x6723),
                                                      __byte_perm(w[0], w[1], 0x4501), __byte_perm(w[2], w[3], 0x4501));
          }
        }
      }
      if (ok && t == 0) {
        if (dst.norm) dst.norm[v] = nrm;
        if (dst.scale && good) *reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(dst.scale) + rec_off + within * 4) = nrm * invn;
      }
      if constexpr (QJLS) {
        // ---- residual in the rotated domain, in place (negated like the values): -(u - c * cs), cs = ts / ||c|| ----
        const float cs = invn * ts;
        float2 ee2 = make_float2(0.f, 0.f);
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
          for (int nt = 0; nt < 2; ++nt) {
            const float2 nu = make_float2(acc[i][nt][2 * vs], acc[i][nt][2 * vs + 1]);
            const float a0 = fabsf(nu.x), a1 = fabsf(nu.y);
            float2 cm;                                     // magnitude of the chosen centroid
            if constexpr (BITS == 3) {
              const float2 p2 = make_float2(qm_gt(a0, thr[1]), qm_gt(a1, thr[1]));
              const float2 th = qm_fma2(p2, qm_dup(d31), qm_dup(thr[0]));
              const float2 p1 = make_float2(qm_gt(a0, th.x), qm_gt(a1, th.y));
              // level 2 p2 + p1: c4, c5, c6, c7
              const float2 base = qm_fma2(p2, qm_dup(cst[1]), qm_dup(cst[0]));
              const float2 slope = qm_fma2(p2, qm_dup(cst[3]), qm_dup(cst[2]));
              cm = qm_fma2(p1, slope, base);
            } else {
              cm = qm_dup(cst[0]);
#pragma unroll
              for (int j = 0; j < NT; ++j) {
                const float2 p = make_float2(qm_gt(a0, thr[j]), qm_gt(a1, thr[j]));
                cm = qm_fma2(p, qm_dup(cst[1 + j]), cm);
              }
            }
            // the centroid carries the value's sign; the registers hold minus the value
            cm.x = __int_as_float(__float_as_int(cm.x) | (~__float_as_int(nu.x) & 0x80000000));
            cm.y = __int_as_float(__float_as_int(cm.y) | (~__float_as_int(nu.y) & 0x80000000));
            const float2 r = qm_fma2(cm, qm_dup(cs), nu);
            ee2 = qm_fma2(r, r, ee2);
            acc[i][nt][2 * vs] = r.x;
            acc[i][nt][2 * vs + 1] = r.y;
          }
        float ee = ee2.x + ee2.y;
        ee += __shfl_xor_sync(0xffffffffu, ee, 1);
        ee += __shfl_xor_sync(0xffffffffu, ee, 2);
        const float rn = nrm > 0.f ? sqrtf(ee) * TQ_RSQRT_D : 0.f;   // ||r|| = ||x|| * ||y - yhat'||
        // ---- sign(S r), S r ~ J2 H J1 D1 H E (positive factors dropped): two transforms with the flips between ----
        auto wht = [&]() {
#pragma unroll
          for (int i = 0; i < 8; ++i)
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {   // element bit 0: the two columns of a register pair
              const float a = acc[i][nt][2 * vs], b = acc[i][nt][2 * vs + 1];
              acc[i][nt][2 * vs] = a + b;
              acc[i][nt][2 * vs + 1] = a - b;
            }
#pragma unroll
          for (int i = 0; i < 8; ++i) {        // bit 1: the two n-tiles
            const float2 a = make_float2(acc[i][0][2 * vs], acc[i][0][2 * vs + 1]);
            const float2 b = make_float2(acc[i][1][2 * vs], acc[i][1][2 * vs + 1]);
            const float2 s = qm_add2(a, b), d = qm_sub2(a, b);
            acc[i][0][2 * vs] = s.x; acc[i][0][2 * vs + 1] = s.y;
            acc[i][1][2 * vs] = d.x; acc[i][1][2 * vs + 1] = d.y;
          }
#pragma unroll
          for (int m = 1; m <= 2; m <<= 1) {   // bits 2, 3: the lanes of the quad
            const float2 sg = qm_dup((t & m) ? -1.0f : 1.0f);
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
              for (int nt = 0; nt < 2; ++nt) {
                const float2 own = make_float2(acc[i][nt][2 * vs], acc[i][nt][2 * vs + 1]);
                const float2 oth = make_float2(__shfl_xor_sync(0xffffffffu, own.x, m), __shfl_xor_sync(0xffffffffu, own.y, m));
                const float2 r = qm_fma2(own, sg, oth);   // bit clear: own + other; bit set: other - own
                acc[i][nt][2 * vs] = r.x;
                acc[i][nt][2 * vs + 1] = r.y;
              }
          }
#pragma unroll
          for (int h = 1; h < 8; h <<= 1)      // bits 4-6: the eight blocks
#pragma unroll
            for (int i = 0; i < 8; ++i)
              if ((i & h) == 0)
#pragma unroll
                for (int nt = 0; nt < 2; ++nt) {
                  const float2 a = make_float2(acc[i][nt][2 * vs], acc[i][nt][2 * vs + 1]);
                  const float2 b = make_float2(acc[i + h][nt][2 * vs], acc[i + h][nt][2 * vs + 1]);
                  const float2 s = qm_add2(a, b), d = qm_sub2(a, b);
                  acc[i][nt][2 * vs] = s.x; acc[i][nt][2 * vs + 1] = s.y;
                  acc[i + h][nt][2 * vs] = d.x; acc[i + h][nt][2 * vs + 1] = d.y;
                }
        };
        wht();
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float4 s4 = m12f[i * 32 + lane];
          const float2 a = qm_mul2(make_float2(acc[i][0][2 * vs], acc[i][0][2 * vs + 1]), make_float2(s4.x, s4.y));
          const float2 b = qm_mul2(make_float2(acc[i][1][2 * vs], acc[i][1][2 * vs + 1]), make_float2(s4.z, s4.w));
          acc[i][0][2 * vs] = a.x; acc[i][0][2 * vs + 1] = a.y;
          acc[i][1][2 * vs] = b.x; acc[i][1][2 * vs + 1] = b.y;
        }
        wht();
        // sketch bit = 1 where j2 * (S r) >= 0 (turboquant/qjl.py:89-90).  The registers hold minus the projection:
        // its sign bit is the sketch bit before the j2 flip, which is an XOR of the gathered word.  (A projection
        // that is exactly zero, of a nonzero residual, takes the bit its zero's sign gives.)
        uint32_t sk = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
          for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int c = 0; c < 2; ++c) sk = __funnelshift_l(__float_as_uint(acc[i][nt][2 * vs + c]), sk, 1);
        sk ^= j2w;
        if (!(nrm > 0.f)) sk = 0xffffffffu;   // zero input -> zero residual -> all +1
        // Lane t holds, for every block i, the nibble of elements 16 i + 4 t .. + 3 (nibble 4 i + t of the sketch).
        // Bytes 4 t .. 4 t + 3 of the sketch are the nibbles of blocks 2 t and 2 t + 1 from all four lanes: byte t
        // (from the top) of every lane's word.
        const int quad = lane & ~3;
        uint32_t xb[4];
#pragma unroll
        for (int s = 0; s < 4; ++s) xb[s] = (__shfl_sync(0xffffffffu, sk, quad + s) >> (24 - 8 * t)) & 0xffu;
        const uint32_t b0 = ((xb[0] >> 4) << 4) | (xb[1] >> 4), b1 = ((xb[2] >> 4) << 4) | (xb[3] >> 4);
        const uint32_t b2 = ((xb[0] & 15) << 4) | (xb[1] & 15), b3 = ((xb[2] & 15) << 4) | (xb[3] & 15);
        if (good && dst.qjl)
          *reinterpret_cast<uint32_t*>(dst.qjl + rec_off + within * 16 + 4 * t) = b0 | (b1 << 8) | (b2 << 16) | (b3 << 24);
        if (ok && t == 0 && good && dst.rnorm)   // sqrt(pi/2)/sqrt(d): turboquant/qjl.py:32,131
          *reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(dst.rnorm) + rec_off + within * 4) =
              dst.rscale_const ? rn * (1.2533141373155001f * TQ_RSQRT_D) : rn;
      }
    }
    __syncwarp();  // every lane is done with this buffer before the copies of the tile after next land in it
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
}

// staging memory of one CTA (tiles + B operands): 16-bit rows fit the static limit, fp32 rows (72 KB) are dynamic
// (the QJL stage adds 4 KB of sign factors and keeps more values live: one CTA less per SM)
template <typename Tin, bool QJLS = false> constexpr int qm_tile_bytes() {
  return QM_WARPS * 2 * QM_ROWS * qm_rowb<Tin>() + 8 * 32 * 16 + (QJLS ? 8 * 32 * 16 : 0);
}
template <typename Tin, bool QJLS = false> constexpr int qm_ctas_per_sm() { return (sizeof(Tin) == 4 ? 3 : 5) - (QJLS ? 1 : 0); }
template <typename Tin, bool QJLS = false> __device__ __forceinline__ uint8_t* qm_tile() {
  if constexpr (sizeof(Tin) == 4) {
    extern __shared__ __align__(16) uint8_t qm_dyn[];
    return qm_dyn;
  } else {
    __shared__ __align__(16) uint8_t qm_static[qm_tile_bytes<Tin, QJLS>()];
    return qm_static;
  }
}

template <typename Tin, int BITS, bool NORMC, bool QJLS = false>
__global__ void __launch_bounds__(QM_THREADS, qm_ctas_per_sm<Tin, QJLS>()) k_quantize_mma(const TqFast f, const Tin* __restrict__ x,
                                                                                         int64_t ld, int64_t n, const TqQuantDst dst) {
  qm_body<Tin, BITS, NORMC, QJLS>(f, x, ld, n, dst, qm_tile<Tin, QJLS>());
}

// Two tensors of the same shape in one launch (the K and V rows of a cache append): blockIdx.y picks the job.
struct QmJob {
  TqFast f;
  const void* x;
  TqQuantDst dst;
};
template <typename Tin, int BITS, bool NORMC>
__global__ void __launch_bounds__(QM_THREADS, qm_ctas_per_sm<Tin>()) k_quantize_mma_pair(const __grid_constant__ QmJob j0,
                                                                                        const __grid_constant__ QmJob j1, int64_t ld,
                                                                                        int64_t n) {
  uint8_t* tile = qm_tile<Tin>();
  if (blockIdx.y == 0) qm_body<Tin, BITS, NORMC>(j0.f, reinterpret_cast<const Tin*>(j0.x), ld, n, j0.dst, tile);
  else qm_body<Tin, BITS, NORMC>(j1.f, reinterpret_cast<const Tin*>(j1.x), ld, n, j1.dst, tile);
}

// dynamic shared memory of a launch (0 for 16-bit rows); raises the kernel's limit once per device
template <typename Tin, auto kernel, bool QJLS = false>
int qm_dyn_smem(size_t* bytes) {
  *bytes = 0;
  if constexpr (sizeof(Tin) == 4) {
    *bytes = qm_tile_bytes<Tin, QJLS>();
    static thread_local int configured_dev = -1;  // one per kernel: the kernel is a template argument
    int dev = 0;
    TQ_CUDA(cudaGetDevice(&dev));
    if (configured_dev != dev) {
      TQ_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, qm_tile_bytes<Tin, QJLS>()));
      configured_dev = dev;
    }
  }
  return TQ_OK;
}

template <typename Tin, int BITS>
int launch_mma(const TqFast& f, const Tin* x, int64_t ld, int64_t n, const TqQuantDst& dst, bool want_qjl, cudaStream_t st) {
  const int64_t tiles = (n + QM_ROWS - 1) / QM_ROWS;
  const int64_t ctas = (tiles + QM_WARPS - 1) / QM_WARPS;
  size_t smem = 0;
  if constexpr (BITS == 4) {
    if (want_qjl) return TQ_ERR_UNSUPPORTED;   // not offered by qm_serves: seven tests and their centroid steps spill
  } else if (want_qjl) {   // the residual needs the norm correction whether or not the scale is stored
    const int64_t capq = (int64_t)tq_num_sms() * qm_ctas_per_sm<Tin, true>();
    const int gridq = (int)(ctas < capq ? ctas : capq);
    if (f.norm_correction) {
      const int rc = qm_dyn_smem<Tin, k_quantize_mma<Tin, BITS, true, true>, true>(&smem);
      if (rc != TQ_OK) return rc;
      k_quantize_mma<Tin, BITS, true, true><<<gridq, QM_THREADS, smem, st>>>(f, x, ld, n, dst);
    } else {
      const int rc = qm_dyn_smem<Tin, k_quantize_mma<Tin, BITS, false, true>, true>(&smem);
      if (rc != TQ_OK) return rc;
      k_quantize_mma<Tin, BITS, false, true><<<gridq, QM_THREADS, smem, st>>>(f, x, ld, n, dst);
    }
    return tq_launch_check("k_quantize_mma");
  }
  const int64_t cap = (int64_t)tq_num_sms() * qm_ctas_per_sm<Tin>();
  const int grid = (int)(ctas < cap ? ctas : cap);
  if (f.norm_correction && dst.scale) {
    const int rc = qm_dyn_smem<Tin, k_quantize_mma<Tin, BITS, true>>(&smem);
    if (rc != TQ_OK) return rc;
    k_quantize_mma<Tin, BITS, true><<<grid, QM_THREADS, smem, st>>>(f, x, ld, n, dst);
  } else {
    const int rc = qm_dyn_smem<Tin, k_quantize_mma<Tin, BITS, false>>(&smem);
    if (rc != TQ_OK) return rc;
    k_quantize_mma<Tin, BITS, false><<<grid, QM_THREADS, smem, st>>>(f, x, ld, n, dst);
  }
  return tq_launch_check("k_quantize_mma");
}

template <typename Tin, int BITS>
int launch_mma_pair(const QmJob& j0, const QmJob& j1, int64_t ld, int64_t n, bool normc, cudaStream_t st) {
  const int64_t tiles = (n + QM_ROWS - 1) / QM_ROWS;
  const int64_t ctas = (tiles + QM_WARPS - 1) / QM_WARPS;
  const int64_t cap = (int64_t)tq_num_sms() * qm_ctas_per_sm<Tin>() / 2;  // two jobs share the SMs
  dim3 grid((unsigned)(ctas < cap ? ctas : cap), 2);
  size_t smem = 0;
  if (normc) {
    const int rc = qm_dyn_smem<Tin, k_quantize_mma_pair<Tin, BITS, true>>(&smem);
    if (rc != TQ_OK) return rc;
    k_quantize_mma_pair<Tin, BITS, true><<<grid, QM_THREADS, smem, st>>>(j0, j1, ld, n);
  } else {
    const int rc = qm_dyn_smem<Tin, k_quantize_mma_pair<Tin, BITS, false>>(&smem);
    if (rc != TQ_OK) return rc;
    k_quantize_mma_pair<Tin, BITS, false><<<grid, QM_THREADS, smem, st>>>(j0, j1, ld, n);
  }
  return tq_launch_check("k_quantize_mma_pair");
}

bool qm_serves(const TqFast& f, int32_t dtype, int64_t ld, const TqQuantDst& dst, bool want_qjl) {
  if (!f.symmetric || !dst.idx || dst.idx_u8) return false;
  if (!want_qjl && (dst.qjl || dst.rnorm)) return false;
  if (want_qjl && f.bits == 4) return false;   // 5-bit PROD: the butterfly kernel
  if (dst.qjl && !tq_aligned(dst.qjl, 4)) return false;
  if (dtype != TQ_F16 && dtype != TQ_BF16 && dtype != TQ_F32) return false;
  // rows must start on 16-byte boundaries (1-bit codebooks have no magnitude levels to test)
  return f.bits >= 2 && f.bits <= 4 && ld % (dtype == TQ_F32 ? 4 : 8) == 0;
}

}  // namespace

// K and V of one append in a single launch, when both take this kernel with the same template arguments.
bool tq_quantize_mma_try_pair(const TqFast& f0, const void* x0, const TqQuantDst& d0, const TqFast& f1, const void* x1,
                              const TqQuantDst& d1, int32_t dtype, int64_t ld, int64_t n, cudaStream_t st, int* rc) {
  if (!qm_serves(f0, dtype, ld, d0, false) || !qm_serves(f1, dtype, ld, d1, false)) return false;
  if (f0.bits != f1.bits || (f0.norm_correction && d0.scale) != (f1.norm_correction && d1.scale)) return false;
  if (!tq_aligned(x0, 16) || !tq_aligned(x1, 16) || n == 0) return false;
  QmJob j0, j1;
  j0.f = f0; j0.x = x0; j0.dst = d0;
  j1.f = f1; j1.x = x1; j1.dst = d1;
  const bool normc = f0.norm_correction && d0.scale;
#define TQ_CASE(B)                                                                              \
  case B:                                                                                       \
    *rc = dtype == TQ_F16    ? launch_mma_pair<__half, B>(j0, j1, ld, n, normc, st)             \
          : dtype == TQ_BF16 ? launch_mma_pair<__nv_bfloat16, B>(j0, j1, ld, n, normc, st)      \
                             : launch_mma_pair<float, B>(j0, j1, ld, n, normc, st);             \
    return true;
  switch (f0.bits) {
    TQ_CASE(2)
    TQ_CASE(3)
    TQ_CASE(4)
  }
#undef TQ_CASE
  return false;
}

// Returns true when this kernel serves the request (rc then holds the launch status).
bool tq_quantize_mma_try(const TqFast& f, const void* x, int32_t dtype, int64_t ld, int64_t n, const TqQuantDst& dst,
                         bool want_qjl, cudaStream_t st, int* rc) {
  if (!qm_serves(f, dtype, ld, dst, want_qjl)) return false;
#define TQ_CASE(B)                                                                                           \
  case B:                                                                                                    \
    *rc = dtype == TQ_F16    ? launch_mma<__half, B>(f, (const __half*)x, ld, n, dst, want_qjl, st)               \
          : dtype == TQ_BF16 ? launch_mma<__nv_bfloat16, B>(f, (const __nv_bfloat16*)x, ld, n, dst, want_qjl, st) \
                             : launch_mma<float, B>(f, (const float*)x, ld, n, dst, want_qjl, st);                \
    return true;
  switch (f.bits) {
    TQ_CASE(2)
    TQ_CASE(3)
    TQ_CASE(4)
  }
#undef TQ_CASE
  return false;
}
