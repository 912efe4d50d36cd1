// Decode attention straight off the packed paged cache, and quantize-on-append.
//
//   k_prepare_queries  rotates each query once by the K rotation (and projects it by the QJL matrix
//                      for PROD formats), folds in softmax scale * log2(e) and the fp16 LUT factor.
//   k_decode_attn      grid (split, kv head, sequence).  A CTA walks its range of pages; each page
//                      record (packed K | K scales | packed V | V scales) is brought into shared memory
//                      with one bulk async copy (cp.async.bulk + mbarrier, 3 stages).  Eight warps
//                      take 16 tokens each per page: pairs of packed indices are turned into fp16
//                      centroid pairs through a lane-replicated (bank-conflict-free) table, fed to
//                      mma.sync.m16n8k16 as the A operand (tokens on M, the <= 8 query heads of the
//                      GQA group on N), softmax is kept online in the log2 domain, the probabilities
//                      are transposed in registers (movmatrix) and multiply V^T tiles dequantized the
//                      same way.  tcgen05 is deliberately not used here: with 4..8 query rows the
//                      work per byte is tiny and the cost is the dequantization ALU, not the MMA.
//   k_decode_combine   merges the split partials (deterministic order) and rotates the output back
//                      from V's rotated space.
#include "tq_internal.cuh"

namespace {

constexpr int ATT_THREADS = 256;
constexpr int ATT_WARPS = 8;
constexpr int ATT_STAGES = 3;
constexpr int MAX_G = 8;  // query heads per KV head handled by one N=8 MMA tile
constexpr uint32_t WAIT_TRIES = 1u << 22;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(dst)),
               "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: gives up after WAIT_TRIES polls and reports it instead of spinning forever.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity) {
  for (uint32_t i = 0; i < WAIT_TRIES; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  return false;
}

__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
  uint32_t d;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
  return d;
}
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

struct AttnParams {
  const uint8_t* pool;
  const int32_t* block_table;
  const int32_t* seq_lens;
  const float* qrot;   // [B][Hq][128]  K-rotated, pre-scaled queries
  const float* qproj;  // [B][Hq][128]  S-projected queries (PROD), pre-scaled
  float* part_o;       // [B][Hq][S][128]
  float* part_ml;      // [B][Hq][S][2]
  int32_t* status;
  int32_t max_pages, batch, hq, hkv, group, chunk_pages, num_splits;
  tq_cache_layout L;
};

// Pair table: entry (ia << BITS | ib) holds half2(alpha*c[ia], alpha*c[ib]).  Tables of <= 64 entries
// are replicated per lane (word index = entry*32 + lane) so that every lookup hits its own bank.
template <int BITS> struct PairLut {
  static constexpr int ENTRIES = 1 << (2 * BITS);
  static constexpr bool REPL = ENTRIES <= 64;
  static constexpr int WORDS = REPL ? ENTRIES * 32 : ENTRIES;
  static __device__ __forceinline__ void fill(uint32_t* lut, const TqFast& f, int tid, int nthreads) {
    for (int i = tid; i < WORDS; i += nthreads) {
      const int e = REPL ? (i >> 5) : i;
      const uint32_t lo = f.cent16[e >> BITS], hi = f.cent16[e & ((1 << BITS) - 1)];
      lut[i] = lo | (hi << 16);
    }
  }
  static __device__ __forceinline__ uint32_t get(const uint32_t* lut, uint32_t field, int lane) {
    return REPL ? lut[field * 32 + lane] : lut[field];
  }
};

// field p (2*BITS bits wide, counted from the most significant end) of a big-endian word array
template <int BITS, int NW>
__device__ __forceinline__ uint32_t be_field(const uint32_t (&w)[NW], int p) {
  constexpr int FB = 2 * BITS;
  const int start = p * FB, k = start >> 5, o = start & 31;
  if (o + FB <= 32) return (w[k] >> (32 - FB - o)) & ((1u << FB) - 1);
  return __funnelshift_l(w[k + 1 < NW ? k + 1 : k], w[k], o) >> (32 - FB);
}

template <int KB, int VB>
__global__ void __launch_bounds__(ATT_THREADS, 2) k_decode_attn(const AttnParams P, const TqFast fk, const TqFast fv) {
  extern __shared__ __align__(128) uint8_t smem[];
  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int seq_len = P.seq_lens[b];
  const int PT = P.L.page_tokens;
  const int n_pages = (seq_len + PT - 1) / PT;
  const int page_lo = split * P.chunk_pages;
  if (page_lo >= n_pages) return;
  const int page_hi = min(n_pages, page_lo + P.chunk_pages);
  const int np = page_hi - page_lo;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
  const uint32_t rec = (uint32_t)P.L.record_bytes;
  uint8_t* stage0 = smem;
  uint32_t* lutk = reinterpret_cast<uint32_t*>(smem + (size_t)ATT_STAGES * rec);
  uint32_t* lutv = lutk + PairLut<KB>::WORDS;
  uint64_t* bars = reinterpret_cast<uint64_t*>(lutv + PairLut<VB>::WORDS);
  __shared__ int s_fail;

  if (tid == 0) {
    for (int s = 0; s < ATT_STAGES; ++s) mbar_init(&bars[s], 1);
    s_fail = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  PairLut<KB>::fill(lutk, fk, tid, ATT_THREADS);
  PairLut<VB>::fill(lutv, fv, tid, ATT_THREADS);
  __syncthreads();

  const int32_t* bt = P.block_table + (size_t)b * P.max_pages;
  auto issue = [&](int i) {
    const int64_t page = bt[page_lo + i];
    const uint8_t* src = P.pool + page * P.L.page_stride + (int64_t)kvh * P.L.head_stride;
    uint64_t* bar = &bars[i % ATT_STAGES];
    mbar_expect_tx(bar, rec);
    bulk_g2s(stage0 + (size_t)(i % ATT_STAGES) * rec, src, rec, bar);
  };
  if (tid == 0) {
    issue(0);
    if (np > 1) issue(1);
  }

  // query fragments (B operand): head g, dims 32t + 4j + {0,1} and {2,3}; hi/lo fp16 split
  uint32_t qh[8][2], ql[8][2];
  {
    const bool hv = g < P.group;
    const float* qp = P.qrot + ((size_t)b * P.hq + (size_t)kvh * P.group + (hv ? g : 0)) * TQ_D + 32 * t;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float4 v = hv ? *reinterpret_cast<const float4*>(qp + 4 * j) : make_float4(0.f, 0.f, 0.f, 0.f);
      const __half2 h0 = __floats2half2_rn(v.x, v.y), h1 = __floats2half2_rn(v.z, v.w);
      const float2 f0 = __half22float2(h0), f1 = __half22float2(h1);
      qh[j][0] = *reinterpret_cast<const uint32_t*>(&h0);
      qh[j][1] = *reinterpret_cast<const uint32_t*>(&h1);
      ql[j][0] = pack_h2(v.x - f0.x, v.y - f0.y);
      ql[j][1] = pack_h2(v.z - f1.x, v.w - f1.y);
    }
  }

  float o[8][4];
#pragma unroll
  for (int j = 0; j < 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

  constexpr int KIDXB = 16 * KB, VIDXB = 16 * VB;
  constexpr int KW = KB;  // 32-bit words per thread chunk (32 dims * KB bits / 32)
  const int tiles_per_page = PT / 16;

  for (int i = 0; i < np; ++i) {
    if (tid == 0 && i + 2 < np) issue(i + 2);
    if (!mbar_wait_bounded(&bars[i % ATT_STAGES], (uint32_t)((i / ATT_STAGES) & 1))) s_fail = 1;
    const uint8_t* st = stage0 + (size_t)(i % ATT_STAGES) * rec;
    const int valid = min(PT, seq_len - (page_lo + i) * PT);  // tokens of this page that exist

    for (int tile = warp; tile < tiles_per_page; tile += ATT_WARPS) {
      const int tb = tile * 16;
      if (tb >= valid) break;
      // ---------------- S = K_tile (16 tokens x 128) . q^T ----------------
      float s[4] = {0.f, 0.f, 0.f, 0.f};
      {
        uint32_t w0[KW], w1[KW];
        const uint32_t* p0 = reinterpret_cast<const uint32_t*>(st + P.L.k_idx_off + (tb + g) * KIDXB + t * (KIDXB / 4));
        const uint32_t* p1 = p0 + 8 * (KIDXB / 4);
#pragma unroll
        for (int k = 0; k < KW; ++k) {
          w0[k] = __byte_perm(p0[k], 0, 0x0123);
          w1[k] = __byte_perm(p1[k], 0, 0x0123);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const uint32_t a0 = PairLut<KB>::get(lutk, be_field<KB, KW>(w0, 2 * j), lane);
          const uint32_t a1 = PairLut<KB>::get(lutk, be_field<KB, KW>(w1, 2 * j), lane);
          const uint32_t a2 = PairLut<KB>::get(lutk, be_field<KB, KW>(w0, 2 * j + 1), lane);
          const uint32_t a3 = PairLut<KB>::get(lutk, be_field<KB, KW>(w1, 2 * j + 1), lane);
          mma16816(s, a0, a1, a2, a3, qh[j][0], qh[j][1]);
          mma16816(s, a0, a1, a2, a3, ql[j][0], ql[j][1]);
        }
      }
      const float* ksc = reinterpret_cast<const float*>(st + P.L.k_scale_off);
      const float* vsc = reinterpret_cast<const float*>(st + P.L.v_scale_off);
      const bool ok0 = tb + g < valid, ok1 = tb + g + 8 < valid;
      const float ks0 = ksc[tb + g], ks1 = ksc[tb + g + 8];
      s[0] = ok0 ? s[0] * ks0 : -INFINITY;
      s[1] = ok0 ? s[1] * ks0 : -INFINITY;
      s[2] = ok1 ? s[2] * ks1 : -INFINITY;
      s[3] = ok1 ? s[3] * ks1 : -INFINITY;
      // ---------------- online softmax (log2 domain), heads 2t and 2t+1 ----------------
      float mx0 = fmaxf(s[0], s[2]), mx1 = fmaxf(s[1], s[3]);
#pragma unroll
      for (int sh = 4; sh < 32; sh <<= 1) {
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, sh));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, sh));
      }
      const float mn0 = fmaxf(m_run[0], mx0), mn1 = fmaxf(m_run[1], mx1);  // finite: token tb is valid
      const float r0 = fast_exp2(m_run[0] - mn0), r1 = fast_exp2(m_run[1] - mn1);
      m_run[0] = mn0;
      m_run[1] = mn1;
      const float p00 = fast_exp2(s[0] - mn0), p01 = fast_exp2(s[1] - mn1);
      const float p10 = fast_exp2(s[2] - mn0), p11 = fast_exp2(s[3] - mn1);
      l_run[0] = l_run[0] * r0 + p00 + p10;
      l_run[1] = l_run[1] * r1 + p01 + p11;
      if (__any_sync(0xffffffffu, (r0 != 1.0f) || (r1 != 1.0f))) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          o[j][0] *= r0; o[j][1] *= r1; o[j][2] *= r0; o[j][3] *= r1;
        }
      }
      // probabilities * V scale, as fp16, transposed into the B-operand layout (tokens on K)
      const float vs0 = ok0 ? vsc[tb + g] : 0.f, vs1 = ok1 ? vsc[tb + g + 8] : 0.f;
      const uint32_t pb0 = movmatrix_trans(pack_h2(p00 * vs0, p01 * vs0));
      const uint32_t pb1 = movmatrix_trans(pack_h2(p10 * vs1, p11 * vs1));
      // ---------------- O^T += V_tile^T . P^T ----------------
      {
        uint32_t h[4][8];  // half2 (dim 16g+2jj, dim 16g+2jj+1) for tokens tb + {2t, 2t+1, 2t+8, 2t+9}
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          const int tok = tb + 2 * t + (q4 & 1) + (q4 >> 1) * 8;
          const uint8_t* pv = st + P.L.v_idx_off + tok * VIDXB + g * (2 * VB);
          uint32_t w[2];
          if (VB == 3) {
            const uint16_t* ph = reinterpret_cast<const uint16_t*>(pv);
            const uint32_t a = ph[0], bb = ph[1], c = ph[2];
            w[0] = __byte_perm(a, bb, 0x0145);
            w[1] = __byte_perm(c, 0, 0x0144);
          } else if (VB == 2) {
            w[0] = __byte_perm(*reinterpret_cast<const uint32_t*>(pv), 0, 0x0123);
            w[1] = 0;
          } else if (VB == 4) {
            const uint2 v2 = *reinterpret_cast<const uint2*>(pv);
            w[0] = __byte_perm(v2.x, 0, 0x0123);
            w[1] = __byte_perm(v2.y, 0, 0x0123);
          } else {  // VB == 1
            w[0] = __byte_perm((uint32_t)*reinterpret_cast<const uint16_t*>(pv), 0, 0x0144);
            w[1] = 0;
          }
#pragma unroll
          for (int jj = 0; jj < 8; ++jj) h[q4][jj] = PairLut<VB>::get(lutv, be_field<VB, 2>(w, jj), lane);
        }
#pragma unroll
        for (int jj = 0; jj < 8; ++jj) {
          const uint32_t a0 = __byte_perm(h[0][jj], h[1][jj], 0x5410);
          const uint32_t a1 = __byte_perm(h[0][jj], h[1][jj], 0x7632);
          const uint32_t a2 = __byte_perm(h[2][jj], h[3][jj], 0x5410);
          const uint32_t a3 = __byte_perm(h[2][jj], h[3][jj], 0x7632);
          mma16816(o[jj], a0, a1, a2, a3, pb0, pb1);
        }
      }
    }
    __syncthreads();  // every warp is done with this stage before it is refilled
  }

  // ---------------- merge the eight warps, write the split partial ----------------
  // l is still per thread (tokens g and g+8 only): sum over the 8 lanes that share t
#pragma unroll
  for (int sh = 4; sh < 32; sh <<= 1) {
    l_run[0] += __shfl_xor_sync(0xffffffffu, l_run[0], sh);
    l_run[1] += __shfl_xor_sync(0xffffffffu, l_run[1], sh);
  }
  float* so = reinterpret_cast<float*>(smem);            // [warp][head 8][dim 128]
  float* sml = so + ATT_WARPS * MAX_G * TQ_D;            // [warp][head 8][2]
#pragma unroll
  for (int jj = 0; jj < 8; ++jj) {
    const int d0 = 16 * g + 2 * jj;
    float* base = so + (size_t)warp * MAX_G * TQ_D;
    base[(2 * t) * TQ_D + d0] = o[jj][0];
    base[(2 * t + 1) * TQ_D + d0] = o[jj][1];
    base[(2 * t) * TQ_D + d0 + 1] = o[jj][2];
    base[(2 * t + 1) * TQ_D + d0 + 1] = o[jj][3];
  }
  if (g == 0) {
    sml[(warp * MAX_G + 2 * t) * 2] = m_run[0];
    sml[(warp * MAX_G + 2 * t) * 2 + 1] = l_run[0];
    sml[(warp * MAX_G + 2 * t + 1) * 2] = m_run[1];
    sml[(warp * MAX_G + 2 * t + 1) * 2 + 1] = l_run[1];
  }
  __syncthreads();
  for (int e = tid; e < P.group * TQ_D; e += ATT_THREADS) {
    const int head = e >> 7, dim = e & 127;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < ATT_WARPS; ++w) M = fmaxf(M, sml[(w * MAX_G + head) * 2]);
    float acc = 0.f, L = 0.f;
#pragma unroll
    for (int w = 0; w < ATT_WARPS; ++w) {
      const float mw = sml[(w * MAX_G + head) * 2];
      const float f = mw == -INFINITY ? 0.f : fast_exp2(mw - M);
      acc = fmaf(so[((size_t)w * MAX_G + head) * TQ_D + dim], f, acc);
      L = fmaf(sml[(w * MAX_G + head) * 2 + 1], f, L);
    }
    const size_t slot = ((size_t)b * P.hq + (size_t)kvh * P.group + head) * P.num_splits + split;
    P.part_o[slot * TQ_D + dim] = acc;
    if (dim == 0) {
      P.part_ml[slot * 2] = M;
      P.part_ml[slot * 2 + 1] = L;
    }
  }
  if (tid == 0 && s_fail) atomicExch(P.status, 1);
}

// ------------------------------------------------------------------------------------------
// 128-point sign*WHT of a vector held in shared memory by a 128-thread block
__device__ __forceinline__ float wht128_block(float v, float* buf, int j) {
  buf[j] = v;
  __syncthreads();
#pragma unroll
  for (int h = 1; h < TQ_D; h <<= 1) {
    const float a = buf[j], bb = buf[j ^ h];
    __syncthreads();
    buf[j] = (j & h) ? bb - a : a + bb;
    __syncthreads();
  }
  return buf[j] * TQ_RSQRT_D;
}

__device__ __forceinline__ float sign_of(const uint32_t (&m)[4], int j) { return ((m[j >> 5] >> (j & 31)) & 1u) ? -1.f : 1.f; }

template <typename Tq>
__global__ void __launch_bounds__(128) k_prepare_queries(const Tq* __restrict__ q, int64_t rows, float qscale,
                                                         int k_dense, const float* __restrict__ rot_t,
                                                         const TqFast fk, int prod, const float* __restrict__ s_t,
                                                         float* __restrict__ qrot, float* __restrict__ qproj,
                                                         int32_t* status) {
  __shared__ float xs[TQ_D], buf[TQ_D];
  const int j = threadIdx.x;
  if (blockIdx.x == 0 && j == 0) *status = 0;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const float x = (float)q[row * TQ_D + j];
    xs[j] = x;
    __syncthreads();
    float y;
    if (k_dense) {
      y = 0.f;
#pragma unroll 8
      for (int k = 0; k < TQ_D; ++k) y = fmaf(__ldg(rot_t + k * TQ_D + j), xs[k], y);  // (R x)_j
    } else {
      y = wht128_block(x * sign_of(fk.s1, j), buf, j) * sign_of(fk.s2, j);
    }
    qrot[row * TQ_D + j] = y * (qscale / fk.lut_alpha);
    if (prod) {
      float z;
      if (k_dense) {
        z = 0.f;
#pragma unroll 8
        for (int k = 0; k < TQ_D; ++k) z = fmaf(__ldg(s_t + k * TQ_D + j), xs[k], z);  // (S x)_j
      } else {
        __syncthreads();
        z = wht128_block(x * sign_of(fk.j1, j), buf, j) * sign_of(fk.j2, j);
      }
      qproj[row * TQ_D + j] = z * qscale;
    }
    __syncthreads();
  }
}

template <typename To>
__global__ void __launch_bounds__(128) k_decode_combine(const float* __restrict__ part_o,
                                                        const float* __restrict__ part_ml,
                                                        const int32_t* __restrict__ seq_lens, int hq, int num_splits,
                                                        int chunk_pages, int page_tokens, int v_dense,
                                                        const float* __restrict__ rot, const TqFast fv,
                                                        To* __restrict__ out) {
  __shared__ float ys[TQ_D], buf[TQ_D];
  const int j = threadIdx.x;
  const int64_t row = blockIdx.x;
  const int b = (int)(row / hq);
  const int n_pages = (seq_lens[b] + page_tokens - 1) / page_tokens;
  const int ns = (n_pages + chunk_pages - 1) / chunk_pages;
  float M = -INFINITY;
  for (int s = 0; s < ns; ++s) M = fmaxf(M, part_ml[(row * num_splits + s) * 2]);
  float acc = 0.f, L = 0.f;
  for (int s = 0; s < ns; ++s) {
    const float f = exp2f(part_ml[(row * num_splits + s) * 2] - M);
    acc = fmaf(part_o[(row * num_splits + s) * TQ_D + j], f, acc);
    L = fmaf(part_ml[(row * num_splits + s) * 2 + 1], f, L);
  }
  const float y = ns > 0 ? acc / (L * fv.lut_alpha) : 0.f;  // attention output in V's rotated space
  float x;
  if (v_dense) {
    ys[j] = y;
    __syncthreads();
    x = 0.f;
#pragma unroll 8
    for (int k = 0; k < TQ_D; ++k) x = fmaf(__ldg(rot + k * TQ_D + j), ys[k], x);  // (R^T y)_j
  } else {
    x = wht128_block(y * sign_of(fv.s2, j), buf, j) * sign_of(fv.s1, j);  // D1 (H/sqrt d) D2 y
  }
  out[row * TQ_D + j] = (To)x;
}

struct SplitPlan {
  int chunk_pages, num_splits;
};

SplitPlan plan_splits(int batch, int hkv, int max_pages) {
  const int slots = 2 * tq_num_sms();
  const long items = (long)batch * hkv;
  SplitPlan p;
  if (max_pages < 1) max_pages = 1;
  if (items >= slots) {
    p.chunk_pages = max_pages < 32 ? max_pages : 32;
  } else {
    const int s = (int)((slots + items - 1) / items);
    p.chunk_pages = (max_pages + s - 1) / s;
    if (p.chunk_pages < 1) p.chunk_pages = 1;
  }
  p.num_splits = (max_pages + p.chunk_pages - 1) / p.chunk_pages;
  return p;
}

struct WsLayout {
  size_t qrot, qproj, part_o, part_ml, status, total;
};

WsLayout ws_layout(int batch, int hq, int num_splits) {
  WsLayout w;
  size_t off = 0;
  auto take = [&](size_t bytes) {
    size_t o = off;
    off += (bytes + 255) & ~(size_t)255;
    return o;
  };
  const size_t rows = (size_t)batch * hq;
  w.qrot = take(rows * TQ_D * 4);
  w.qproj = take(rows * TQ_D * 4);
  w.part_o = take(rows * num_splits * TQ_D * 4);
  w.part_ml = take(rows * num_splits * 2 * 4);
  w.status = take(256);
  w.total = off;
  return w;
}

int fmt_bits(int fmt) { return (fmt >= TQ_FMT_TURBO2 && fmt <= TQ_FMT_TURBO4) ? fmt : 0; }

template <int KB, int VB>
int launch_attn(const AttnParams& P, const TqFast& fk, const TqFast& fv, cudaStream_t st) {
  const size_t smem = (size_t)ATT_STAGES * P.L.record_bytes + (size_t)(PairLut<KB>::WORDS + PairLut<VB>::WORDS) * 4 + 64;
  const size_t merge = (size_t)ATT_WARPS * MAX_G * (TQ_D + 2) * 4;
  const size_t need = smem > merge ? smem : merge;
  TQ_REQUIRE(need <= 227 * 1024, TQ_ERR_TOO_LARGE, "page record of %d bytes does not fit the shared-memory pipeline",
             P.L.record_bytes);
  TQ_CUDA(cudaFuncSetAttribute(k_decode_attn<KB, VB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)need));
  dim3 grid(P.num_splits, P.hkv, P.batch);
  k_decode_attn<KB, VB><<<grid, ATT_THREADS, need, st>>>(P, fk, fv);
  return tq_launch_check("k_decode_attn");
}

}  // namespace

extern "C" int64_t tq_decode_workspace_bytes(int32_t batch, int32_t num_q_heads, int32_t num_kv_heads,
                                             int32_t max_pages_per_seq) {
  if (batch < 1 || num_q_heads < 1 || num_kv_heads < 1 || max_pages_per_seq < 1) return TQ_ERR_INVALID;
  const SplitPlan p = plan_splits(batch, num_kv_heads, max_pages_per_seq);
  return (int64_t)ws_layout(batch, num_q_heads, p.num_splits).total;
}

extern "C" int tq_decode_status_sync(const void* workspace_dev, int64_t workspace_bytes, int32_t* status_out) {
  TQ_REQUIRE(workspace_dev && status_out && workspace_bytes >= 256, TQ_ERR_INVALID, "bad workspace");
  TQ_CUDA(cudaMemcpy(status_out, (const uint8_t*)workspace_dev + workspace_bytes - 256, 4, cudaMemcpyDeviceToHost));
  return TQ_OK;
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

extern "C" int tq_decode_attn(const tq_quantizer* kq, const tq_quantizer* vq, const tq_cache_layout* L,
                              const uint8_t* pool_dev, const int32_t* block_table_dev, int32_t max_pages_per_seq,
                              const int32_t* seq_lens_dev, const void* q_dev, int32_t q_dtype, int32_t batch,
                              int32_t num_q_heads, float scale, void* workspace_dev, int64_t workspace_bytes,
                              void* out_dev, int32_t out_dtype, void* stream) {
  return tq_decode_attn_phases(kq, vq, L, pool_dev, block_table_dev, max_pages_per_seq, seq_lens_dev, q_dev, q_dtype,
                               batch, num_q_heads, scale, workspace_dev, workspace_bytes, out_dev, out_dtype, 7, stream);
}

extern "C" int tq_decode_attn_phases(const tq_quantizer* kq, const tq_quantizer* vq, const tq_cache_layout* L,
                                     const uint8_t* pool_dev, const int32_t* block_table_dev,
                                     int32_t max_pages_per_seq, const int32_t* seq_lens_dev, const void* q_dev,
                                     int32_t q_dtype, int32_t batch, int32_t num_q_heads, float scale,
                                     void* workspace_dev, int64_t workspace_bytes, void* out_dev, int32_t out_dtype,
                                     int32_t phases, void* stream) {
  TQ_REQUIRE(kq && vq && L, TQ_ERR_INVALID, "tq_decode_attn: quantizers or layout missing");
  TQ_REQUIRE(batch >= 0 && num_q_heads >= 1 && max_pages_per_seq >= 1, TQ_ERR_INVALID, "bad sizes");
  if (batch == 0) return TQ_OK;
  TQ_REQUIRE(pool_dev && block_table_dev && seq_lens_dev && q_dev && out_dev && workspace_dev, TQ_ERR_INVALID,
             "tq_decode_attn: null buffer");
  TQ_REQUIRE(L->d == TQ_D && kq->d == TQ_D && vq->d == TQ_D, TQ_ERR_UNSUPPORTED, "decode attention is built for d == 128");
  TQ_REQUIRE(num_q_heads % L->num_kv_heads == 0, TQ_ERR_INVALID, "num_q_heads must be a multiple of num_kv_heads");
  const int group = num_q_heads / L->num_kv_heads;
  TQ_REQUIRE(group <= MAX_G, TQ_ERR_UNSUPPORTED, "at most %d query heads per KV head, got %d", MAX_G, group);
  TQ_REQUIRE(batch <= 65535 && L->num_kv_heads <= 65535, TQ_ERR_TOO_LARGE, "batch and KV heads are grid dimensions (<= 65535)");
  TQ_REQUIRE(tq_aligned(pool_dev, 128) && tq_aligned(workspace_dev, 256) && tq_aligned(q_dev, 16) && tq_aligned(out_dev, 16),
             TQ_ERR_ALIGN, "pool (128), workspace (256), q and out (16) must be aligned");
  const int kb = fmt_bits(L->k_format), vb = fmt_bits(L->v_format);
  TQ_REQUIRE(kb && vb, TQ_ERR_UNSUPPORTED, "decode attention: K format %d / V format %d not built yet", L->k_format,
             L->v_format);
  TQ_REQUIRE(kq->bits == kb && vq->bits == vb, TQ_ERR_INVALID, "quantizer bit widths do not match the cache formats");
  const SplitPlan plan = plan_splits(batch, L->num_kv_heads, max_pages_per_seq);
  const WsLayout w = ws_layout(batch, num_q_heads, plan.num_splits);
  TQ_REQUIRE((int64_t)w.total <= workspace_bytes, TQ_ERR_TOO_LARGE, "workspace of %lld bytes is smaller than the %lld needed",
             (long long)workspace_bytes, (long long)w.total);
  cudaStream_t st = (cudaStream_t)stream;
  uint8_t* ws = (uint8_t*)workspace_dev;
  // the status word sits in the last 256 bytes of the caller's buffer
  int32_t* status = reinterpret_cast<int32_t*>(ws + workspace_bytes - 256);
  if (scale <= 0.f) scale = TQ_RSQRT_D;
  const float qscale = scale * 1.4426950408889634f;
  const int64_t rows = (int64_t)batch * num_q_heads;
  const int pgrid = (int)(rows < 4096 ? rows : 4096);
  const int k_dense = kq->rotation == TQ_ROT_DENSE, v_dense = vq->rotation == TQ_ROT_DENSE;
  float* qrot = reinterpret_cast<float*>(ws + w.qrot);
  float* qproj = reinterpret_cast<float*>(ws + w.qproj);
#define TQ_PREP(T)                                                                                                  \
  k_prepare_queries<T><<<pgrid, 128, 0, st>>>((const T*)q_dev, rows, qscale, k_dense, kq->rot32_t, kq->fast, 0,     \
                                              kq->s32_t, qrot, qproj, status)
  int rc = TQ_OK;
  if (phases & 1) {
    switch (q_dtype) {
      case TQ_F16: TQ_PREP(__half); break;
      case TQ_BF16: TQ_PREP(__nv_bfloat16); break;
      case TQ_F32: TQ_PREP(float); break;
      default:
        tq_set_error("queries must be fp16, bf16 or fp32, got dtype %d", q_dtype);
        return TQ_ERR_UNSUPPORTED;
    }
    rc = tq_launch_check("k_prepare_queries");
    if (rc != TQ_OK) return rc;
  }
#undef TQ_PREP

  AttnParams P;
  memset(&P, 0, sizeof(P));
  P.pool = pool_dev;
  P.block_table = block_table_dev;
  P.seq_lens = seq_lens_dev;
  P.qrot = qrot;
  P.qproj = qproj;
  P.part_o = reinterpret_cast<float*>(ws + w.part_o);
  P.part_ml = reinterpret_cast<float*>(ws + w.part_ml);
  P.status = status;
  P.max_pages = max_pages_per_seq;
  P.batch = batch;
  P.hq = num_q_heads;
  P.hkv = L->num_kv_heads;
  P.group = group;
  P.chunk_pages = plan.chunk_pages;
  P.num_splits = plan.num_splits;
  P.L = *L;
#define TQ_ATT(K, V) \
  if (kb == K && vb == V) rc = launch_attn<K, V>(P, kq->fast, vq->fast, st);
  if (phases & 2) {
    rc = TQ_ERR_UNSUPPORTED;
    TQ_ATT(2, 2) TQ_ATT(2, 3) TQ_ATT(2, 4) TQ_ATT(3, 2) TQ_ATT(3, 3) TQ_ATT(3, 4) TQ_ATT(4, 2) TQ_ATT(4, 3) TQ_ATT(4, 4)
    if (rc != TQ_OK) return rc;
  }
#undef TQ_ATT
  if (!(phases & 4)) return TQ_OK;

#define TQ_COMB(T)                                                                                             \
  k_decode_combine<T><<<(unsigned)rows, 128, 0, st>>>(P.part_o, P.part_ml, seq_lens_dev, num_q_heads,          \
                                                      plan.num_splits, plan.chunk_pages, L->page_tokens, v_dense, \
                                                      vq->rot32, vq->fast, (T*)out_dev)
  switch (out_dtype) {
    case TQ_F16: TQ_COMB(__half); break;
    case TQ_BF16: TQ_COMB(__nv_bfloat16); break;
    case TQ_F32: TQ_COMB(float); break;
    default:
      tq_set_error("output must be fp16, bf16 or fp32, got dtype %d", out_dtype);
      return TQ_ERR_UNSUPPORTED;
  }
#undef TQ_COMB
  return tq_launch_check("k_decode_combine");
}

// ------------------------------------------------------------------------------------------
// Decode attention for callers that may not allocate device memory.
//
// The split partials and rotated queries of tq_decode_attn normally live in a buffer the caller
// allocates.  Some callers cannot do that: a plugin that runs inside another runtime which has
// already handed every byte of HBM to its own pool, a latency-bound serving loop in which
// cudaMalloc's implicit device-wide synchronisation is not acceptable, or a host language binding
// that has raw pointers to inputs and outputs but no allocator of its own.  For them the scratch is
// this fixed array, part of the library image: every GPU that loads the library holds
// TQ_STATIC_SCRATCH_BYTES of it until the process exits.
//
// In host code `g_static_scratch` is only a handle for the symbol, not an address the GPU can use;
// the device address comes from cudaGetSymbolAddress, looked up once per device below.
// ------------------------------------------------------------------------------------------
#include <mutex>

#define TQ_STATIC_SCRATCH_BYTES TQ_DECODE_STATIC_SCRATCH_BYTES  // 8 MiB, stated in tq_b200.h
#define TQ_STATIC_MAX_DEVICES 64

static __device__ __align__(256) unsigned char g_static_scratch[TQ_STATIC_SCRATCH_BYTES];
static void* g_static_scratch_addr[TQ_STATIC_MAX_DEVICES];  // device address of the array, per device
static std::mutex g_static_scratch_mutex;

// Device address of g_static_scratch on the current device (set-up on the first call per device).
static int static_scratch_for_current_device(void** out) {
  int dev = -1;
  TQ_CUDA(cudaGetDevice(&dev));
  TQ_REQUIRE(dev >= 0 && dev < TQ_STATIC_MAX_DEVICES, TQ_ERR_UNSUPPORTED, "device ordinal %d beyond %d", dev,
             TQ_STATIC_MAX_DEVICES);
  std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
  if (g_static_scratch_addr[dev] == nullptr) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress((void**)&p, g_static_scratch);
    if (e != cudaSuccess) return tq_cuda_fail(e, "cudaGetSymbolAddress(g_static_scratch)");
    TQ_REQUIRE(p != nullptr && tq_aligned(p, 256), TQ_ERR_CUDA, "static scratch has no usable device address");
    g_static_scratch_addr[dev] = p;
  }
  *out = g_static_scratch_addr[dev];
  return TQ_OK;
}

extern "C" int tq_decode_attn_static(const tq_quantizer* kq, const tq_quantizer* vq, const tq_cache_layout* L,
                                     const uint8_t* pool_dev, const int32_t* block_table_dev,
                                     int32_t max_pages_per_seq, const int32_t* seq_lens_dev, const void* q_dev,
                                     int32_t q_dtype, int32_t batch, int32_t num_q_heads, float scale, void* out_dev,
                                     int32_t out_dtype, void* stream) {
  TQ_REQUIRE(L, TQ_ERR_INVALID, "tq_decode_attn_static: layout missing");
  TQ_REQUIRE(batch >= 0 && num_q_heads >= 1 && max_pages_per_seq >= 1, TQ_ERR_INVALID, "bad sizes");
  if (batch == 0) return TQ_OK;
  const int64_t need = tq_decode_workspace_bytes(batch, num_q_heads, L->num_kv_heads, max_pages_per_seq);
  TQ_REQUIRE(need > 0, TQ_ERR_INVALID, "bad sizes");
  TQ_REQUIRE(need <= TQ_STATIC_SCRATCH_BYTES, TQ_ERR_TOO_LARGE,
             "tq_decode_attn_static: this shape needs %lld bytes of scratch, the built-in array holds %d "
             "(batch %d x %d query heads x %d pages); use tq_decode_attn with a caller-owned workspace",
             (long long)need, TQ_STATIC_SCRATCH_BYTES, batch, num_q_heads, max_pages_per_seq);
  void* scratch = nullptr;
  int rc = static_scratch_for_current_device(&scratch);
  if (rc != TQ_OK) return rc;
  // Nothing in the scratch has to start at zero: the query kernel resets the status word, and every
  // partial that the merge kernel reads is written by the attention kernel of the same call.
  return tq_decode_attn_phases(kq, vq, L, pool_dev, block_table_dev, max_pages_per_seq, seq_lens_dev, q_dev, q_dtype,
                               batch, num_q_heads, scale, scratch, TQ_STATIC_SCRATCH_BYTES, out_dev, out_dtype, 7,
                               stream);
}
