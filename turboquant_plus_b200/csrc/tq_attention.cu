// Decode attention straight off the packed paged cache.
//
//   k_decode_attn<KK,VK>  grid (split, kv head, sequence), 256 threads, 2 CTAs per SM.
//     prologue  the CTA's <= 8 query heads are rotated by the K rotation (one warp per head: sign,
//               128-point Walsh-Hadamard in registers + shuffles, sign) and, for PROD keys, projected by
//               the QJL sign-WHT; scale * log2(e) and the fp16 table factor are folded in.  Dense
//               rotations are applied by k_prepare_queries beforehand instead.
//     main loop the CTA walks its range of pages; each (page, head) record (packed K | K scales |
//               [sign sketch | residual scales] | packed V | V scales) arrives in shared memory through one
//               bulk async copy (cp.async.bulk + mbarrier, 3 stages, bounded waits).  Eight warps take 16
//               tokens each: 2b-bit index *pairs* become fp16 centroid pairs through a lane-replicated
//               (bank-conflict-free) table whose address is one shift + one logic op, and feed
//               mma.sync.m16n8k16 as the A operand (tokens on M, query heads of the GQA group on N, query
//               split into hi+lo fp16).  q8_0 operands are int8 -> fp16 by byte permute + one subtract.
//               Softmax is online in the log2 domain; probabilities * V scale are transposed in registers
//               (movmatrix) and multiply V^T tiles dequantized the same way; O stays in V's rotated space.
//     epilogue  the CTA stores its split partial; the last CTA of a (sequence, kv head) to finish -- a
//               ticket taken with one atomicAdd, nobody waits -- merges the splits in fixed order, rotates
//               back (WHT per warp, or dense) and writes the output.  One launch per call in WHT mode.
//   tcgen05 is deliberately not used here: with 4..8 query rows the MMA work is a few percent of the tensor
//   pipe; the cost is forming the operands.
#include <mutex>

#include "tq_internal.cuh"

namespace {

constexpr int ATT_THREADS = 256;
constexpr int ATT_WARPS = 8;
constexpr int ATT_STAGES = 3;
constexpr int MAX_G = 8;  // query heads per KV head handled by one N=8 MMA tile
constexpr long long WAIT_CYCLES = 1LL << 30;  // ~0.5 s at the SM clock: upper bound of any single wait
// Sparse V (docs/papers/sparse-v-dequant.md:64-84 of the reference: "if (attn_weight < 1e-6f) continue;" before the V
// dequantization of a position, the weight being exp(score - running max)): here the unit is a 16-token tile of one
// warp -- the tile's V lookups and MMAs are skipped when every weight in it, for every head, is below the threshold.
// The weights still enter the softmax denominators.
constexpr float SPARSE_V_TAU = 1e-6f;
constexpr int MAX_TICKETS = 65536;                    // (sequence, kv head) pairs per call
constexpr size_t TAIL_BYTES = (size_t)MAX_TICKETS * 4 + 256;  // tickets + status word at the end of a workspace

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
// Bounded wait: polls until the phase completes or WAIT_CYCLES SM clocks have passed, then gives up and
// reports it instead of spinning forever.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  while (clock64() - t0 < WAIT_CYCLES)
    if (mbar_try_wait(bar, parity)) return true;
  return false;
}

// Barrier `id` over one 256-thread group.  id 0 with a 256-thread CTA is the block barrier; a 512-thread CTA runs
// two independent groups on ids 1 and 2.
__device__ __forceinline__ void group_sync(int id) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "n"(ATT_THREADS) : "memory");
}

__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  // volatile on purpose: a warp-collective instruction must not be sunk into, or speculated out of,
  // code that only some lanes execute
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
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
  uint32_t v;
  // not volatile: the tables are constant while the main loop runs, so loads may be hoisted and batched
  asm("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint32_t hsub2_u32(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("sub.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
__device__ __forceinline__ uint32_t hmul2_u32(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

// Optional per-CTA phase stamps (debug builds with -DTQ_PHASE_TIMING): globaltimer at kernel entry, main-loop
// entry, main-loop exit, partial written, kernel exit.
#ifdef TQ_PHASE_TIMING
__device__ unsigned long long g_phase_log[8192 * 16];
__device__ __forceinline__ void phase_stamp(int slot) {
  if ((threadIdx.x & 255) == 0) {
    unsigned long long tns;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(tns));
    const int per = blockDim.x >> 8;  // 256-thread groups per CTA, each stamps its own row
    const int cta = blockIdx.x * per + (threadIdx.x >> 8) + gridDim.x * per * (blockIdx.y + gridDim.y * blockIdx.z);
    if (cta < 8192) {
      g_phase_log[cta * 16 + slot] = tns;
      if (slot == 0) {
        unsigned smid;
        asm volatile("mov.u32 %0, %smid;" : "=r"(smid));
        g_phase_log[cta * 16 + 15] = smid;
      }
    }
  }
}
#define PHASE_STAMP(s) phase_stamp(s)
#else
#define PHASE_STAMP(s)
#endif

struct AttnParams {
  const uint8_t* pool;
  const int32_t* block_table;
  const int32_t* seq_lens;
  const void* q;       // raw queries [B][Hq][128] (q_dtype), used when the rotation is applied in the prologue
  const float* qrot;   // [B][Hq][128] rotated, pre-scaled queries (dense rotations only)
  const float* qproj;  // [B][Hq][128] S-projected queries (dense PROD only)
  float* part_o;       // [B][Hq][S][128]
  float* part_ml;      // [B][Hq][S][2]
  int32_t* tickets;    // [B*Hkv], zero between calls
  int32_t* status;
  void* out;           // [B][Hq][128] (out_dtype)
  float* lse;          // [B][Hq] natural log of the softmax denominator (with the maximum folded in); or null
  const float* v_rot;  // dense V rotation, row-major fp32 (nullptr: sign-WHT or identity)
  float qscale;        // softmax scale * log2(e)
  int32_t q_dtype, out_dtype;
  int32_t k_pre;       // 1: queries come rotated from qrot/qproj
  int32_t k_ident, v_ident;  // identity rotation (q8_0 tensors)
  int32_t max_pages, batch, hq, hkv, group, chunk_pages, num_splits;
  int32_t stages;      // 2 or 3 page records in flight per CTA
  int32_t overlap;     // launched with programmatic stream serialization: see TQ_DECODE_OVERLAP
  int32_t sparse_v;    // skip the V work of a 16-token tile whose weights are all below SPARSE_V_TAU: TQ_DECODE_SPARSE_V
  tq_cache_layout L;
};

// ---- kinds ------------------------------------------------------------------------------------
// KK / VK: 2,3,4 = turbo bits; 8 = q8_0; 18,19,20 = PROD with 1,2,3 PolarQuant bits + sign sketch.
template <int KIND> struct Kind {
  static constexpr bool Q8 = KIND == 8;
  static constexpr bool PROD = KIND >= 18;
  static constexpr int BITS = Q8 ? 0 : (PROD ? KIND - 17 : KIND);
};

// Pair table: entry (ia << BITS | ib) holds half2(alpha*c[ia], alpha*c[ib]).  Tables of <= 64 entries are
// replicated per lane (byte address = entry*128 + lane*4) so that every lookup hits its own bank; the table is
// aligned to its size so that the address is (field bits) | (lane base).
template <int BITS> struct PairLut {
  static constexpr int ENTRIES = BITS ? (1 << (2 * BITS)) : 0;
  static constexpr bool REPL = ENTRIES <= 64;
  static constexpr int SHIFT = REPL ? 7 : 2;
  static constexpr int BYTES = BITS ? ENTRIES << SHIFT : 0;
};

template <int BITS>
__device__ __forceinline__ void lut_fill(uint8_t* lut, const uint16_t* c16, int tid, int nthreads = ATT_THREADS) {
  using T = PairLut<BITS>;
  if (T::REPL) {
    // entry e occupies 128 bytes (one word per lane): eight 16-byte stores of the same value
    for (int i = tid; i < T::ENTRIES * 8; i += nthreads) {
      const int e = i >> 3;
      const uint32_t v = (uint32_t)c16[e >> BITS] | ((uint32_t)c16[e & ((1 << BITS) - 1)] << 16);
      reinterpret_cast<uint4*>(lut)[i] = make_uint4(v, v, v, v);
    }
  } else {
    uint32_t* w = reinterpret_cast<uint32_t*>(lut);
    for (int e = tid; e < T::ENTRIES; e += nthreads)
      w[e] = (uint32_t)c16[e >> BITS] | ((uint32_t)c16[e & ((1 << BITS) - 1)] << 16);
  }
}

// (field p of width FB bits, counted from the most significant end of a big-endian word array) << SH
template <int FB, int SH, int NW>
__device__ __forceinline__ uint32_t field_off(const uint32_t (&w)[NW], int p) {
  constexpr uint32_t MASK = ((1u << FB) - 1) << SH;
  const int start = p * FB, k = start >> 5, o = start & 31;
  if (o + FB <= 32) {
    const int sr = 32 - FB - o;
    const uint32_t v = sr > SH ? (w[k] >> (sr - SH)) : (sr < SH ? (w[k] << (SH - sr)) : w[k]);
    return v & MASK;
  }
  // the field straddles words k and k+1: in the 64-bit value (w[k] : w[k+1]) it sits 64 - o - FB bits above the
  // low end, so one funnel shift by sr puts it at bit SH.  o > 32 - FB gives sr < 32 - SH: the 5-bit count is exact.
  const int sr = 64 - o - FB - SH;
  return __funnelshift_r(w[k + 1 < NW ? k + 1 : k], w[k], sr) & MASK;
}

__device__ __forceinline__ float load_q(const void* q, int dtype, size_t i) {
  if (dtype == TQ_F16) return __half2float(reinterpret_cast<const __half*>(q)[i]);
  if (dtype == TQ_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(q)[i]);
  return reinterpret_cast<const float*>(q)[i];
}
__device__ __forceinline__ void store_out(void* out, int dtype, size_t i, float v) {
  if (dtype == TQ_F16) reinterpret_cast<__half*>(out)[i] = __float2half_rn(v);
  else if (dtype == TQ_BF16) reinterpret_cast<__nv_bfloat16*>(out)[i] = __float2bfloat16_rn(v);
  else reinterpret_cast<float*>(out)[i] = v;
}

// 128-point sign * Walsh-Hadamard of one vector held by a warp: lane l has elements 4l..4l+3.
// y = post (H/sqrt d) pre x, signs as bit masks (bit e set => -1).
__device__ __forceinline__ void warp_wht128(float (&x)[4], const uint32_t (&pre)[4], const uint32_t (&post)[4], int lane) {
  const uint32_t pb = (pre[lane >> 3] >> ((lane & 7) * 4)) & 0xfu, qb = (post[lane >> 3] >> ((lane & 7) * 4)) & 0xfu;
#pragma unroll
  for (int k = 0; k < 4; ++k) x[k] = ((pb >> k) & 1u) ? -x[k] : x[k];
  float a = x[0] + x[1], b = x[0] - x[1], c = x[2] + x[3], d = x[2] - x[3];
  x[0] = a + c; x[1] = b + d; x[2] = a - c; x[3] = b - d;
#pragma unroll
  for (int bit = 1; bit < 32; bit <<= 1) {
    const float sgn = (lane & bit) ? -1.0f : 1.0f;
#pragma unroll
    for (int k = 0; k < 4; ++k) x[k] = fmaf(sgn, x[k], __shfl_xor_sync(0xffffffffu, x[k], bit));
  }
#pragma unroll
  for (int k = 0; k < 4; ++k) x[k] = (((qb >> k) & 1u) ? -x[k] : x[k]) * TQ_RSQRT_D;
}

// Fold of the split partials of one head by one warp (see finish_splits).  A round covers 64 splits: lane j
// fetches (max, sum) of splits s0 + j and s0 + 32 + j, twenty 16-byte loads per lane go out before anything
// waits, the warp agrees on the maximum, then the rows are accumulated in split order.
template <int HALVES, bool V_Q8>
__device__ __forceinline__ void fold_splits(const AttnParams& P, float v_alpha, float* qbuf, size_t row0, int ns, int warp) {
  const int lane = threadIdx.x & 31;
  if (warp >= HALVES * P.group) return;
  const int head = warp % P.group, half = warp / P.group;
  constexpr int ROW_LANES = 32 / HALVES;
  const int chunk = lane & (ROW_LANES - 1), parity = lane / ROW_LANES;
  const int col4 = half * 16 + chunk;                      // 16-byte column of the 128-float row
  const size_t base = (row0 + head) * P.num_splits;
  const float4* rows = reinterpret_cast<const float4*>(P.part_o + base * TQ_D) + col4;
  float M = -INFINITY, Lsum = 0.f;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  constexpr int NB = 20, BATCHES = (64 + HALVES * NB - 1) / (HALVES * NB);
  for (int s0 = 0; s0 < ns; s0 += 64) {
    float4 ov[NB];
#pragma unroll
    for (int u = 0; u < NB; ++u) {
      const int j = HALVES * u + parity;                   // split s0 + j
      ov[u] = s0 + j < ns ? __ldcg(rows + (size_t)(s0 + j) * (TQ_D / 4)) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    const float2* mlp = reinterpret_cast<const float2*>(P.part_ml) + base + s0 + lane;
    const float2 ml0 = s0 + lane < ns ? __ldcg(mlp) : make_float2(-INFINITY, 0.f);
    const float2 ml1 = s0 + 32 + lane < ns ? __ldcg(mlp + 32) : make_float2(-INFINITY, 0.f);
    float Mn = fmaxf(ml0.x, ml1.x);
#pragma unroll
    for (int sh = 1; sh < 32; sh <<= 1) Mn = fmaxf(Mn, __shfl_xor_sync(0xffffffffu, Mn, sh));
    Mn = fmaxf(Mn, M);                                     // finite: split s0 exists
    const float r = fast_exp2(M - Mn);
    const float f0 = fast_exp2(ml0.x - Mn), f1 = fast_exp2(ml1.x - Mn);  // 0 for the lanes without a split
    float lf = fmaf(ml0.y, f0, ml1.y * f1);
#pragma unroll
    for (int sh = 1; sh < 32; sh <<= 1) lf += __shfl_xor_sync(0xffffffffu, lf, sh);
    Lsum = fmaf(Lsum, r, lf);
    acc.x *= r; acc.y *= r; acc.z *= r; acc.w *= r;
    M = Mn;
#pragma unroll
    for (int k = 0; k < BATCHES; ++k) {
      if (k > 0) {
        if (s0 + HALVES * NB * k >= ns) break;
#pragma unroll
        for (int u = 0; u < NB; ++u) {
          const int j = HALVES * (NB * k + u) + parity;
          ov[u] = (j < 64 && s0 + j < ns) ? __ldcg(rows + (size_t)(s0 + j) * (TQ_D / 4)) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
      }
#pragma unroll
      for (int u = 0; u < NB; ++u) {
        const int jb = HALVES * (NB * k + u);              // lane-independent part of the split number
        if (jb >= 64) break;
        const float fu = __shfl_sync(0xffffffffu, jb < 32 ? f0 : f1, (jb + parity) & 31);
        acc.x = fmaf(ov[u].x, fu, acc.x); acc.y = fmaf(ov[u].y, fu, acc.y);
        acc.z = fmaf(ov[u].z, fu, acc.z); acc.w = fmaf(ov[u].w, fu, acc.w);
      }
    }
  }
  if (HALVES == 2) {
    acc.x += __shfl_xor_sync(0xffffffffu, acc.x, 16); acc.y += __shfl_xor_sync(0xffffffffu, acc.y, 16);
    acc.z += __shfl_xor_sync(0xffffffffu, acc.z, 16); acc.w += __shfl_xor_sync(0xffffffffu, acc.w, 16);
  }
  PHASE_STAMP(12);
  // M and Lsum are in the log2 domain of the scaled scores: ln sum exp(score) = ln 2 (M + log2 Lsum)
  if (P.lse && half == 0 && lane == 0) P.lse[row0 + head] = (M + log2f(Lsum)) * 0.6931471805599453f;
  // attention output in V's rotated space
  const float inv = 1.0f / (Lsum * (V_Q8 ? 1.0f : v_alpha));
  if (parity == 0)
    reinterpret_cast<float4*>(qbuf + head * TQ_D)[col4] = make_float4(acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv);
}

// Tail shared by the decode kernels, entered by the whole CTA after its split partial has been written:
// take a ticket; the last CTA of a (sequence, kv head) folds all splits in a fixed order, un-rotates and stores.
// One thread publishes the CTA's writes (the block barrier orders the other threads' stores before its
// release), so the rest of the CTA does not execute a device-wide fence.
template <bool V_Q8>
__device__ __forceinline__ void finish_splits(const AttnParams& P, const uint32_t (&vs1)[4], const uint32_t (&vs2)[4],
                                              float v_alpha, float* qbuf, uint8_t* stage0, volatile int* s_flags,
                                              size_t row0, int ns, int b, int kvh, int tid = threadIdx.x, int bar_id = 0) {
  const int lane = tid & 31, warp = tid >> 5;
  group_sync(bar_id);
  if (tid == 0) {
    if (s_flags[0]) atomicExch(P.status, 1);
    __threadfence();
    const int prev = atomicAdd(&P.tickets[b * P.hkv + kvh], 1);
    if (prev == ns - 1) {
      P.tickets[b * P.hkv + kvh] = 0;  // leave the counter at zero for the next call
      s_flags[1] = 1;
      __threadfence();
    }
  }
  group_sync(bar_id);
  PHASE_STAMP(3);
  if (!s_flags[1]) return;
  // Warp (half, head) folds the splits of one head.  With at most four heads there are two warps per head and each
  // takes 64 of the 128 dims: lanes 0..15 then read even splits, lanes 16..31 odd ones (16 bytes each), and one
  // lane exchange joins the two at the end; with more heads a warp takes the whole row and every split.
  if (2 * P.group <= ATT_WARPS) fold_splits<2, V_Q8>(P, v_alpha, qbuf, row0, ns, warp);
  else fold_splits<1, V_Q8>(P, v_alpha, qbuf, row0, ns, warp);
  group_sync(bar_id);
  PHASE_STAMP(13);
  if (P.v_rot) {  // dense rotation: x = R^T y
    for (int e = tid; e < P.group * TQ_D; e += ATT_THREADS) {
      const int head = e >> 7, j = e & 127;
      float x = 0.f;
#pragma unroll 8
      for (int k = 0; k < TQ_D; ++k) x = fmaf(__ldg(P.v_rot + k * TQ_D + j), qbuf[head * TQ_D + k], x);
      store_out(P.out, P.out_dtype, (row0 + head) * TQ_D + j, x);
    }
  } else if (warp < P.group) {
    float x[4];
    const float4 v = *reinterpret_cast<const float4*>(qbuf + warp * TQ_D + 4 * lane);
    x[0] = v.x; x[1] = v.y; x[2] = v.z; x[3] = v.w;
    if (!P.v_ident) warp_wht128(x, vs2, vs1, lane);  // R^T = D1 (H/sqrt d) D2
#pragma unroll
    for (int k = 0; k < 4; ++k) store_out(P.out, P.out_dtype, (row0 + warp) * TQ_D + 4 * lane + k, x[k]);
  }
}

// shared-memory carve-up, identical on host and device
template <int KK, int VK> struct SmemPlan {
  static constexpr int LK = PairLut<Kind<KK>::BITS>::BYTES;
  static constexpr int LV = PairLut<Kind<VK>::BITS>::BYTES;
  static constexpr int LS = Kind<KK>::PROD ? PairLut<1>::BYTES : 0;
  static constexpr int ALIGN = (LK > LV ? LK : LV) > 512 ? (LK > LV ? LK : LV) : 512;  // largest table
  // order tables by size so that each stays aligned to its own size
  static constexpr int OFF_BIG = 0;
  static constexpr int OFF_SMALL = LK > LV ? LK : LV;
  static constexpr int OFF_K = LK >= LV ? OFF_BIG : OFF_SMALL;
  static constexpr int OFF_V = LK >= LV ? OFF_SMALL : OFF_BIG;
  static constexpr int OFF_S = LK + LV;
  static constexpr int OFF_Q = ((OFF_S + LS + 127) / 128) * 128;  // float qbuf[2][8][128]
  static constexpr int OFF_BAR = OFF_Q + 2 * MAX_G * TQ_D * 4;
  static constexpr int OFF_PL = OFF_BAR + 128;  // PROD: lo halves of the projected-query fragments, uint2[8][32]
  static constexpr int OFF_STAGE = OFF_PL + (Kind<KK>::PROD ? 2048 : 0);
  static size_t bytes(int record_bytes, int nstages) {
    const size_t stages = (size_t)nstages * record_bytes;
    const size_t merge = (size_t)ATT_WARPS * MAX_G * (TQ_D + 2) * 4;
    return (size_t)ALIGN + OFF_STAGE + (stages > merge ? stages : merge);
  }
};

template <int KK, int VK>
__global__ void __launch_bounds__(ATT_THREADS, 2) k_decode_attn(const AttnParams P, const TqFast fk, const TqFast fv) {
  using KT = Kind<KK>;
  using VT = Kind<VK>;
  using SP = SmemPlan<KK, VK>;
  constexpr int KB = KT::BITS, VB = VT::BITS;
  extern __shared__ __align__(128) uint8_t smem_raw[];
  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
  PHASE_STAMP(0);
  const int seq_len = P.seq_lens[b];
  const int PT = P.L.page_tokens;
  const int n_pages = (seq_len + PT - 1) / PT;
  const int page_lo = split * P.chunk_pages;
  const size_t row0 = (size_t)b * P.hq + (size_t)kvh * P.group;  // first query / output row of this CTA
  if (n_pages == 0 && split == 0) {  // empty sequence: zeros
    for (int e = tid; e < P.group * TQ_D; e += ATT_THREADS) store_out(P.out, P.out_dtype, row0 * TQ_D + e, 0.f);
    if (P.lse && tid < P.group) P.lse[row0 + tid] = -INFINITY;
    return;
  }
  if (page_lo >= n_pages) return;
  const int page_hi = min(n_pages, page_lo + P.chunk_pages);
  const int np = page_hi - page_lo;
  const int ns = (n_pages + P.chunk_pages - 1) / P.chunk_pages;  // splits of this sequence that run

  // align the carve-up to the largest table
  const uint32_t raw = smem_u32(smem_raw);
  uint8_t* sm = smem_raw + (((raw + SP::ALIGN - 1) & ~(uint32_t)(SP::ALIGN - 1)) - raw);
  float* qbuf = reinterpret_cast<float*>(sm + SP::OFF_Q);
  uint64_t* bars = reinterpret_cast<uint64_t*>(sm + SP::OFF_BAR);
  volatile int* s_flags = reinterpret_cast<volatile int*>(sm + SP::OFF_BAR + 64);  // [0] wait failed, [1] this CTA merges
  uint8_t* stage0 = sm + SP::OFF_STAGE;
  const uint32_t rec = (uint32_t)P.L.record_bytes;
  const int NS = P.stages;

  const int32_t* bt = P.block_table + (size_t)b * P.max_pages;
  auto issue = [&](int i) {
    const int64_t page = bt[page_lo + i];
    const uint8_t* src = P.pool + page * P.L.page_stride + (int64_t)kvh * P.L.head_stride;
    uint64_t* bar = &bars[i % NS];
    mbar_expect_tx(bar, rec);
    bulk_g2s(stage0 + (size_t)(i % NS) * rec, src, rec, bar);
  };
  if (tid == 0) {
    for (int s = 0; s < ATT_STAGES; ++s) mbar_init(&bars[s], 1);
    s_flags[0] = 0;
    s_flags[1] = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    issue(0);
    if (NS > 2 && np > 1) issue(1);
  }
  if constexpr (KB > 0) lut_fill<KB>(sm + SP::OFF_K, fk.cent16, tid);
  if constexpr (VB > 0) lut_fill<VB>(sm + SP::OFF_V, fv.cent16, tid);
  if (KT::PROD) {
    uint32_t* w = reinterpret_cast<uint32_t*>(sm + SP::OFF_S);
    for (int i = tid; i < PairLut<1>::BYTES / 4; i += ATT_THREADS) {
      const int e = i >> 5;  // (bit_a << 1) | bit_b, bit 1 => +1.0
      w[i] = ((e & 2) ? 0x3C00u : 0xBC00u) | (((e & 1) ? 0x3C00u : 0xBC00u) << 16);
    }
  }
  PHASE_STAMP(5);
  // ---- prologue: rotated / projected queries into qbuf[0] (K rotation) and qbuf[1] (QJL projection) ----
  if (warp < P.group) {
    float x[4], y[4];
    const size_t row = row0 + warp;
    if (P.k_pre) {
      const float4 v = *reinterpret_cast<const float4*>(P.qrot + row * TQ_D + 4 * lane);
      x[0] = v.x; x[1] = v.y; x[2] = v.z; x[3] = v.w;
      if (KT::PROD) {
        const float4 u = *reinterpret_cast<const float4*>(P.qproj + row * TQ_D + 4 * lane);
        y[0] = u.x; y[1] = u.y; y[2] = u.z; y[3] = u.w;
      }
    } else {
#pragma unroll
      for (int k = 0; k < 4; ++k) x[k] = y[k] = load_q(P.q, P.q_dtype, row * TQ_D + 4 * lane + k);
      if (!P.k_ident) {
        warp_wht128(x, fk.s1, fk.s2, lane);
        if (KT::PROD) warp_wht128(y, fk.j1, fk.j2, lane);
      }
      const float sk = P.qscale / (KT::Q8 ? 1.0f : fk.lut_alpha);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        x[k] *= sk;
        y[k] *= P.qscale;
      }
    }
    *reinterpret_cast<float4*>(qbuf + warp * TQ_D + 4 * lane) = make_float4(x[0], x[1], x[2], x[3]);
    if (KT::PROD) *reinterpret_cast<float4*>(qbuf + (MAX_G + warp) * TQ_D + 4 * lane) = make_float4(y[0], y[1], y[2], y[3]);
  }
  PHASE_STAMP(6);
  __syncthreads();
  PHASE_STAMP(7);

  // query fragments (B operand) of head g, hi/lo fp16 split
  uint32_t qh[8][2], ql[8][2], ph[KT::PROD ? 8 : 1][2];
  {
    const bool hv = g < P.group;
    const float* qp = qbuf + (hv ? g : 0) * TQ_D;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      // dims this thread supplies in k-step j: 32t + 4j .. +3 (packed formats), or, for q8_0 keys, the
      // thread's 8 dims of block j/2: 32(j/2) + 8t + 4(j%2) .. +3
      const int dq = KT::Q8 ? 32 * (j >> 1) + 8 * t + 4 * (j & 1) : 32 * t + 4 * j;
      float4 v = hv ? *reinterpret_cast<const float4*>(qp + dq) : make_float4(0.f, 0.f, 0.f, 0.f);
      const __half2 h0 = __floats2half2_rn(v.x, v.y), h1 = __floats2half2_rn(v.z, v.w);
      const float2 f0 = __half22float2(h0), f1 = __half22float2(h1);
      qh[j][0] = *reinterpret_cast<const uint32_t*>(&h0);
      qh[j][1] = *reinterpret_cast<const uint32_t*>(&h1);
      ql[j][0] = pack_h2(v.x - f0.x, v.y - f0.y);
      ql[j][1] = pack_h2(v.z - f1.x, v.w - f1.y);
      if constexpr (KT::PROD) {
        float4 u = hv ? *reinterpret_cast<const float4*>(qp + MAX_G * TQ_D + dq) : make_float4(0.f, 0.f, 0.f, 0.f);
        const __half2 e0 = __floats2half2_rn(u.x, u.y), e1 = __floats2half2_rn(u.z, u.w);
        const float2 r0 = __half22float2(e0), r1 = __half22float2(e1);
        ph[j][0] = *reinterpret_cast<const uint32_t*>(&e0);
        ph[j][1] = *reinterpret_cast<const uint32_t*>(&e1);
        // the lo halves live in shared memory (registers are spent on qh, ql, ph and the O accumulators);
        // a fragment depends on the lane only, so warp 0 writes it for everybody
        if (warp == 0)
          reinterpret_cast<uint2*>(sm + SP::OFF_PL)[j * 32 + lane] =
              make_uint2(pack_h2(u.x - r0.x, u.y - r0.y), pack_h2(u.z - r1.x, u.w - r1.y));
      }
    }
  }
  if constexpr (KT::PROD) __syncthreads();
  const uint32_t lk_base = smem_u32(sm + SP::OFF_K) + (PairLut<KB>::REPL ? lane * 4 : 0);
  const uint32_t lv_base = smem_u32(sm + SP::OFF_V) + (PairLut<VB>::REPL ? lane * 4 : 0);
  const uint32_t ls_base = smem_u32(sm + SP::OFF_S) + lane * 4;

  PHASE_STAMP(1);
  float o[8][4];
#pragma unroll
  for (int j = 0; j < 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

  constexpr int KIDXB = KT::Q8 ? TQ_D : 16 * KB;  // K bytes per token
  constexpr int VIDXB = VT::Q8 ? TQ_D : 16 * VB;
  constexpr int KW = KT::Q8 ? 8 : KB;             // 32-bit words per thread chunk (32 dims)
  const int tiles_per_page = PT / 16;

  for (int i = 0; i < np; ++i) {
    if (tid == 0 && i + NS - 1 < np) issue(i + NS - 1);
    // once a wait has given up the CTA stops waiting (and stops trusting the data): it only drains
    if (!s_flags[0] && !mbar_wait_bounded(&bars[i % NS], (uint32_t)((i / NS) & 1))) s_flags[0] = 1;
    const uint8_t* st = stage0 + (size_t)(i % NS) * rec;
    const int valid = min(PT, seq_len - (page_lo + i) * PT);  // tokens of this page that exist

    for (int tile = warp; tile < tiles_per_page; tile += ATT_WARPS) {
      const int tb = tile * 16;
      if (tb >= valid) break;
      const bool ok0 = tb + g < valid, ok1 = tb + g + 8 < valid;
      // ---------------- S = K_tile (16 tokens x 128) . q^T ----------------
      float s[4] = {0.f, 0.f, 0.f, 0.f};
      {
        uint32_t w0[KW], w1[KW];
        const uint32_t* p0 = reinterpret_cast<const uint32_t*>(st + P.L.k_idx_off + (tb + g) * KIDXB + t * (KIDXB / 4));
        const uint32_t* p1 = p0 + 8 * (KIDXB / 4);
        if constexpr (KT::Q8) {
          // int8 -> fp16 exactly: (b ^ 0x80) | 0x6400 is 1024 + (b + 128); subtract 1152.  A 32-value block has
          // one scale, so k-steps 2b and 2b+1 cover block b (thread t supplies its dims 8t..8t+7) and the
          // block's partial scores are scaled in fp32 afterwards -- the operands carry no rounding.
          const uint8_t* q0 = st + P.L.k_idx_off + (tb + g) * TQ_D + 8 * t;
          const uint8_t* q1 = q0 + 8 * TQ_D;
          const uint2 sc0 = *reinterpret_cast<const uint2*>(st + P.L.k_scale_off + (tb + g) * 8);
          const uint2 sc1 = *reinterpret_cast<const uint2*>(st + P.L.k_scale_off + (tb + g + 8) * 8);
          const uint32_t scw0[2] = {sc0.x, sc0.y}, scw1[2] = {sc1.x, sc1.y};
#pragma unroll
          for (int blk = 0; blk < 4; ++blk) {
            const uint2 u0 = *reinterpret_cast<const uint2*>(q0 + 32 * blk);
            const uint2 u1 = *reinterpret_cast<const uint2*>(q1 + 32 * blk);
            const uint32_t x0[2] = {u0.x ^ 0x80808080u, u0.y ^ 0x80808080u};
            const uint32_t x1[2] = {u1.x ^ 0x80808080u, u1.y ^ 0x80808080u};
            float sb[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int h2 = 0; h2 < 2; ++h2) {
              const int j = 2 * blk + h2;
              const uint32_t a0 = hsub2_u32(__byte_perm(x0[h2], 0x64646464u, 0x4140), 0x64806480u);
              const uint32_t a2 = hsub2_u32(__byte_perm(x0[h2], 0x64646464u, 0x4342), 0x64806480u);
              const uint32_t a1 = hsub2_u32(__byte_perm(x1[h2], 0x64646464u, 0x4140), 0x64806480u);
              const uint32_t a3 = hsub2_u32(__byte_perm(x1[h2], 0x64646464u, 0x4342), 0x64806480u);
              mma16816(sb, a0, a1, a2, a3, qh[j][0], qh[j][1]);
              mma16816(sb, a0, a1, a2, a3, ql[j][0], ql[j][1]);
            }
            const __half2 hs0 = *reinterpret_cast<const __half2*>(&scw0[blk >> 1]);
            const __half2 hs1 = *reinterpret_cast<const __half2*>(&scw1[blk >> 1]);
            const float f0 = (blk & 1) ? __high2float(hs0) : __low2float(hs0);
            const float f1 = (blk & 1) ? __high2float(hs1) : __low2float(hs1);
            s[0] = fmaf(sb[0], f0, s[0]); s[1] = fmaf(sb[1], f0, s[1]);
            s[2] = fmaf(sb[2], f1, s[2]); s[3] = fmaf(sb[3], f1, s[3]);
          }
        } else {
#pragma unroll
          for (int k = 0; k < KW; ++k) {
            w0[k] = __byte_perm(p0[k], 0, 0x0123);
            w1[k] = __byte_perm(p1[k], 0, 0x0123);
          }
          constexpr int SH = PairLut<KB>::SHIFT;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const uint32_t a0 = lds32(field_off<2 * KB, SH, KW>(w0, 2 * j) | lk_base);
            const uint32_t a1 = lds32(field_off<2 * KB, SH, KW>(w1, 2 * j) | lk_base);
            const uint32_t a2 = lds32(field_off<2 * KB, SH, KW>(w0, 2 * j + 1) | lk_base);
            const uint32_t a3 = lds32(field_off<2 * KB, SH, KW>(w1, 2 * j + 1) | lk_base);
            mma16816(s, a0, a1, a2, a3, qh[j][0], qh[j][1]);
            mma16816(s, a0, a1, a2, a3, ql[j][0], ql[j][1]);
          }
        }
      }
      if (!KT::Q8) {
        const float* ksc = reinterpret_cast<const float*>(st + P.L.k_scale_off);
        const float ks0 = ksc[tb + g], ks1 = ksc[tb + g + 8];
        s[0] *= ks0; s[1] *= ks0; s[2] *= ks1; s[3] *= ks1;
      }
      if constexpr (KT::PROD) {
        // + sqrt(pi/2)/sqrt(d) * ||r|| * <S q, z>: the sign sketch as +-1 fp16 operands
        float s2[4] = {0.f, 0.f, 0.f, 0.f};
        uint32_t z0[1], z1[1];
        const uint32_t* pz = reinterpret_cast<const uint32_t*>(st + P.L.k_qjl_off + (tb + g) * 16 + t * 4);
        z0[0] = __byte_perm(pz[0], 0, 0x0123);
        z1[0] = __byte_perm(pz[8 * 4], 0, 0x0123);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const uint32_t a0 = lds32(field_off<2, 7, 1>(z0, 2 * j) | ls_base);
          const uint32_t a1 = lds32(field_off<2, 7, 1>(z1, 2 * j) | ls_base);
          const uint32_t a2 = lds32(field_off<2, 7, 1>(z0, 2 * j + 1) | ls_base);
          const uint32_t a3 = lds32(field_off<2, 7, 1>(z1, 2 * j + 1) | ls_base);
          mma16816(s2, a0, a1, a2, a3, ph[j][0], ph[j][1]);
          const uint2 lo = reinterpret_cast<const uint2*>(sm + SP::OFF_PL)[j * 32 + lane];
          mma16816(s2, a0, a1, a2, a3, lo.x, lo.y);
        }
        const float* rsc = reinterpret_cast<const float*>(st + P.L.k_rscale_off);
        const float r0 = rsc[tb + g], r1 = rsc[tb + g + 8];
        s[0] = fmaf(s2[0], r0, s[0]); s[1] = fmaf(s2[1], r0, s[1]);
        s[2] = fmaf(s2[2], r1, s[2]); s[3] = fmaf(s2[3], r1, s[3]);
      }
      s[0] = ok0 ? s[0] : -INFINITY;
      s[1] = ok0 ? s[1] : -INFINITY;
      s[2] = ok1 ? s[2] : -INFINITY;
      s[3] = ok1 ? s[3] : -INFINITY;
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
      if (P.sparse_v && !__any_sync(0xffffffffu, fmaxf(fmaxf(p00, p01), fmaxf(p10, p11)) >= SPARSE_V_TAU)) continue;
      // probabilities (* V scale), as fp16, transposed into the B-operand layout (tokens on K)
      float vs0 = 1.0f, vs1 = 1.0f;
      if (!VT::Q8) {
        const float* vsc = reinterpret_cast<const float*>(st + P.L.v_scale_off);
        vs0 = ok0 ? vsc[tb + g] : 0.f;
        vs1 = ok1 ? vsc[tb + g + 8] : 0.f;
      }
      const uint32_t pb0 = movmatrix_trans(pack_h2(p00 * vs0, p01 * vs0));
      const uint32_t pb1 = movmatrix_trans(pack_h2(p10 * vs1, p11 * vs1));
      // ---------------- O^T += V_tile^T . P^T ----------------
      // thread (g, t): dims 16g .. 16g+15 of tokens tb + {2t, 2t+1, 2t+8, 2t+9}
      if constexpr (VT::Q8) {
        uint32_t x[4][4], sc2[2];
        const uint16_t* vsc = reinterpret_cast<const uint16_t*>(st + P.L.v_scale_off);
        uint32_t scl[4];
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          const int tok = tb + 2 * t + (q4 & 1) + (q4 >> 1) * 8;
          const uint4 v = *reinterpret_cast<const uint4*>(st + P.L.v_idx_off + tok * TQ_D + g * 16);
          x[q4][0] = v.x ^ 0x80808080u; x[q4][1] = v.y ^ 0x80808080u;
          x[q4][2] = v.z ^ 0x80808080u; x[q4][3] = v.w ^ 0x80808080u;
          scl[q4] = tok < valid ? vsc[tok * 4 + (g >> 1)] : 0u;  // a stale scale must not meet p = 0
        }
        sc2[0] = scl[0] | (scl[1] << 16);
        sc2[1] = scl[2] | (scl[3] << 16);
#pragma unroll
        for (int jj = 0; jj < 8; ++jj) {
          const uint32_t sel = (jj & 1) ? 0x4342 : 0x4140;
          const uint32_t h0 = hsub2_u32(__byte_perm(x[0][jj >> 1], 0x64646464u, sel), 0x64806480u);
          const uint32_t h1 = hsub2_u32(__byte_perm(x[1][jj >> 1], 0x64646464u, sel), 0x64806480u);
          const uint32_t h2 = hsub2_u32(__byte_perm(x[2][jj >> 1], 0x64646464u, sel), 0x64806480u);
          const uint32_t h3 = hsub2_u32(__byte_perm(x[3][jj >> 1], 0x64646464u, sel), 0x64806480u);
          const uint32_t a0 = hmul2_u32(__byte_perm(h0, h1, 0x5410), sc2[0]);
          const uint32_t a1 = hmul2_u32(__byte_perm(h0, h1, 0x7632), sc2[0]);
          const uint32_t a2 = hmul2_u32(__byte_perm(h2, h3, 0x5410), sc2[1]);
          const uint32_t a3 = hmul2_u32(__byte_perm(h2, h3, 0x7632), sc2[1]);
          mma16816(o[jj], a0, a1, a2, a3, pb0, pb1);
        }
      } else {
        uint32_t h[4][8];  // half2 (dim 16g+2jj, dim 16g+2jj+1) per token
        constexpr int SH = PairLut<VB>::SHIFT;
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          const int tok = tb + 2 * t + (q4 & 1) + (q4 >> 1) * 8;
          const uint8_t* pv = st + P.L.v_idx_off + tok * VIDXB + g * (2 * VB);
          uint32_t w[2];
          if constexpr (VB == 3) {
            const uint16_t* phw = reinterpret_cast<const uint16_t*>(pv);
            const uint32_t a = phw[0], bb = phw[1], c = phw[2];
            w[0] = __byte_perm(a, bb, 0x0145);
            w[1] = __byte_perm(c, 0, 0x0144);
          } else if constexpr (VB == 2) {
            w[0] = __byte_perm(*reinterpret_cast<const uint32_t*>(pv), 0, 0x0123);
            w[1] = 0;
          } else {
            const uint2 v2 = *reinterpret_cast<const uint2*>(pv);
            w[0] = __byte_perm(v2.x, 0, 0x0123);
            w[1] = __byte_perm(v2.y, 0, 0x0123);
          }
#pragma unroll
          for (int jj = 0; jj < 8; ++jj) h[q4][jj] = lds32(field_off<2 * VB, SH, 2>(w, jj) | lv_base);
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

  PHASE_STAMP(2);
  // ---------------- merge the eight warps, write the split partial ----------------
  // l is still per thread (tokens g and g+8 only): sum over the 8 lanes that share t
#pragma unroll
  for (int sh = 4; sh < 32; sh <<= 1) {
    l_run[0] += __shfl_xor_sync(0xffffffffu, l_run[0], sh);
    l_run[1] += __shfl_xor_sync(0xffffffffu, l_run[1], sh);
  }
  float* so = reinterpret_cast<float*>(stage0);   // [warp][head 8][dim 128]
  float* sml = so + ATT_WARPS * MAX_G * TQ_D;     // [warp][head 8][2]
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
    float acc = 0.f, Lsum = 0.f;
#pragma unroll
    for (int w = 0; w < ATT_WARPS; ++w) {
      const float mw = sml[(w * MAX_G + head) * 2];
      const float f = mw == -INFINITY ? 0.f : fast_exp2(mw - M);
      acc = fmaf(so[((size_t)w * MAX_G + head) * TQ_D + dim], f, acc);
      Lsum = fmaf(sml[(w * MAX_G + head) * 2 + 1], f, Lsum);
    }
    const size_t slot = (row0 + head) * P.num_splits + split;
    P.part_o[slot * TQ_D + dim] = acc;
    if (dim == 0) {
      P.part_ml[slot * 2] = M;
      P.part_ml[slot * 2 + 1] = Lsum;
    }
  }
  finish_splits<VT::Q8>(P, fv.s1, fv.s2, fv.lut_alpha, qbuf, stage0, s_flags, row0, ns, b, kvh);
  PHASE_STAMP(4);
}

// ------------------------------------------------------------------------------------------
// Decode attention, PolarQuant K and V, at most four query heads per KV head (the GQA shape of every decode
// workload this library is measured on).  Same pipeline and the same split / ticket protocol as k_decode_attn;
// what changes is how the 8 columns of the MMA tiles are spent:
//   * S = K q^T: columns 0..3 carry the fp16 "hi" halves of the four query heads, columns 4..7 the "lo" halves,
//     so one m16n8k16 per 16 dims instead of two; the halves meet through one lane exchange (lane ^ 2), after
//     which thread (g, t) owns one token (g + 8 (t >> 1)) and two heads (2 (t & 1), + 1).
//   * O^T += V^T P^T: a k-slot pair is (token, dim parity) instead of (token, token'), column n is
//     (head n >> 1, parity n & 1), and the P operand is p on the matching parity, 0 on the other.  A pair-table
//     word (two dims of one token) is then an A-operand register as it comes: no re-pairing permutes, 32 dims per
//     MMA, and O takes 16 accumulator registers per thread: o[blk] = head t, dims 16 g + 4 blk .. + 3.
//   * the running maxima are only reduced across the warp when some score exceeds them.
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ void load_q4(const void* q, int dtype, size_t i, float (&x)[4]) {
  if (dtype == TQ_F16) {
    const uint2 u = *reinterpret_cast<const uint2*>(reinterpret_cast<const __half*>(q) + i);
    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&u.x));
    const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&u.y));
    x[0] = a.x; x[1] = a.y; x[2] = b.x; x[3] = b.y;
  } else if (dtype == TQ_BF16) {
    const uint2 u = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(q) + i);
    x[0] = __uint_as_float(u.x << 16); x[1] = __uint_as_float(u.x & 0xffff0000u);
    x[2] = __uint_as_float(u.y << 16); x[3] = __uint_as_float(u.y & 0xffff0000u);
  } else {
    const float4 v = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(q) + i);
    x[0] = v.x; x[1] = v.y; x[2] = v.z; x[3] = v.w;
  }
}

// What the kernel needs of a quantizer, packed into 80 bytes so that the whole parameter block is six 64-byte
// lines: parameters live in the constant bank, every line misses once per launch, and the misses of one warp
// are serial.  The warps therefore touch one line each before anything else happens.
struct AttnQuant {
  uint32_t s1[4], s2[4];
  uint16_t cent16[16];
  float alpha;
  uint32_t pad[3];
};
static_assert(sizeof(AttnQuant) == 80, "AttnQuant layout");

constexpr int G4_HEADS = 4;
constexpr int G4_HSTRIDE = TQ_D + 4;  // floats between heads in the warp-merge buffer: 16-byte stores stay conflict-free

// One CTA per SM runs TWO independent 256-thread groups (own split, own pipeline, own barrier), sharing only the
// pair tables.  Two separate 256-thread CTAs on one SM did the same work, but the warp schedulers favoured the
// CTA that arrived first: it finished its pages in 9.7 us, its neighbour in 12.6 us, and the SM idled at half
// occupancy in between.  Warps of one CTA have the same age and progress together.
constexpr int G4_GROUPS = 2;
constexpr int G4_THREADS = G4_GROUPS * ATT_THREADS;

// bytes of one group's private shared memory: query buffer, barriers, pipeline stages (or the warp-merge buffer)
template <int KB, int VB>
constexpr size_t g4_group_bytes(int record_bytes, int nstages) {
  using SP = SmemPlan<KB, VB>;
  const size_t stages = (size_t)nstages * record_bytes;
  const size_t merge = (size_t)ATT_WARPS * G4_HEADS * (TQ_D + 4 + 2) * 4;
  return (((size_t)(SP::OFF_STAGE - SP::OFF_Q) + (stages > merge ? stages : merge)) + 127) / 128 * 128;
}

template <int KB, int VB, bool SPARSE>
__global__ void __launch_bounds__(G4_THREADS, 1) k_decode_attn_g4(const __grid_constant__ AttnParams P, const __grid_constant__ AttnQuant fk,
                                                                    const __grid_constant__ AttnQuant fv) {
  using SP = SmemPlan<KB, VB>;
  extern __shared__ __align__(128) uint8_t smem_raw[];
  const int grp = threadIdx.x >> 8;              // which of the CTA's two groups
  // groups are numbered (kv head, split) so that an odd number of splits does not leave half a CTA empty
  const int gidx = G4_GROUPS * blockIdx.x + grp, b = blockIdx.y;
  const bool exists = gidx < P.num_splits * P.hkv;
  const int kvh = exists ? gidx / P.num_splits : 0, split = exists ? gidx % P.num_splits : P.num_splits;
  const int tid = threadIdx.x & 255, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
  const int bar_id = 1 + grp;
  PHASE_STAMP(0);
  {  // one parameter line per warp, all misses in flight together
    const uint32_t* pp = reinterpret_cast<const uint32_t*>(&P);
    uint32_t touch;
    if (warp < 4) touch = pp[min(16 * warp, (int)(sizeof(AttnParams) / 4) - 1)];
    else if (warp < 6) touch = warp == 4 ? fk.s1[0] : fk.pad[2];
    else touch = warp == 6 ? fv.s1[0] : fv.pad[2];
    asm volatile("" ::"r"(touch));
  }
  PHASE_STAMP(14);
  // Programmatic dependent launch: let the next kernel in the stream start its own prologue as soon as SMs free
  // up.  Everything this kernel does before griddepcontrol.wait below reads only the cache, the block table and
  // the sequence lengths; queries are read, and the workspace and the output written, after the wait, i.e.
  // after the preceding kernel has completed and its writes are visible.  Both instructions do nothing in a
  // launch without the attribute.
  if (P.overlap) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int PT = P.L.page_tokens;
  const int page_lo = split * P.chunk_pages;
  const size_t row0 = (size_t)b * P.hq + (size_t)kvh * P.group;
  const int32_t* bt = P.block_table + (size_t)b * P.max_pages;
  const uint32_t raw = smem_u32(smem_raw);
  uint8_t* sm = smem_raw + (((raw + SP::ALIGN - 1) & ~(uint32_t)(SP::ALIGN - 1)) - raw);
  const uint32_t rec = (uint32_t)P.L.record_bytes;
  const int NS = P.stages;
  uint8_t* smg = sm + (size_t)grp * g4_group_bytes<KB, VB>(rec, NS);   // this group's private part
  float* qbuf = reinterpret_cast<float*>(smg + SP::OFF_Q);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smg + SP::OFF_BAR);
  volatile int* s_flags = reinterpret_cast<volatile int*>(smg + SP::OFF_BAR + 64);
  uint8_t* stage0 = smg + SP::OFF_STAGE;
  constexpr int PRODUCER = ATT_THREADS - 32;  // lane 0 of the last warp issues every bulk copy

  auto issue = [&](int i, int64_t page) {
    const uint8_t* src = P.pool + page * P.L.page_stride + (int64_t)kvh * P.L.head_stride;
    uint64_t* bar = &bars[i % NS];
    mbar_expect_tx(bar, rec);
    bulk_g2s(stage0 + (size_t)(i % NS) * rec, src, rec, bar);
  };

  // The warps take different roles so that their global-load latencies (and their instruction fetches, which are
  // cold in every launch) overlap: the producer sends the first pages on their way as early as it can, the first
  // `group` warps rotate one query head each, the others fill the pair tables.
  const int seq_len = P.seq_lens[b];
  int pg_ahead = 0;  // producer: block-table entry of the page issued in the next iteration
  float x[4] = {0.f, 0.f, 0.f, 0.f};
  if (tid == PRODUCER) {
    int pg_next[ATT_STAGES];
#pragma unroll
    for (int i = 0; i < ATT_STAGES; ++i) pg_next[i] = bt[min(page_lo + i, P.max_pages - 1)];
    for (int s = 0; s < ATT_STAGES; ++s) mbar_init(&bars[s], 1);
    s_flags[0] = 0;
    s_flags[1] = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    const int my_pages = min((seq_len + PT - 1) / PT, page_lo + P.chunk_pages) - page_lo;
    if (my_pages > 0) {
      issue(0, pg_next[0]);
      if (NS > 2) {
        if (my_pages > 1) issue(1, pg_next[1]);
        pg_ahead = pg_next[2];
      } else {
        pg_ahead = pg_next[1];
      }
    }
  } else if (warp < P.group) {
    if (P.overlap) asm volatile("griddepcontrol.wait;" ::: "memory");
    if (P.k_pre) load_q4(P.qrot, TQ_F32, (row0 + warp) * TQ_D + 4 * lane, x);
    else load_q4(P.q, P.q_dtype, (row0 + warp) * TQ_D + 4 * lane, x);
    if (!P.k_pre) {
      warp_wht128(x, fk.s1, fk.s2, lane);
      const float sk = P.qscale / fk.alpha;
#pragma unroll
      for (int k = 0; k < 4; ++k) x[k] *= sk;
    }
    // 16-byte chunk c = 8 t + j of head h sits at 8 t + (j ^ (t + 4 (h & 1))): the fragment reads below (fixed j,
    // all t and h) then touch every bank group instead of one
    const int tq = lane >> 3, jq = lane & 7;
    *reinterpret_cast<float4*>(qbuf + warp * TQ_D + 4 * (8 * tq + (jq ^ (tq + 4 * (warp & 1))))) =
        make_float4(x[0], x[1], x[2], x[3]);
  }
  __syncwarp();
  if (warp >= P.group) {
    const int fh = ATT_THREADS - 32 * P.group;   // table-filling threads per group; both groups share the work
    lut_fill<KB>(sm + SP::OFF_K, fk.cent16, grp * fh + tid - 32 * P.group, G4_GROUPS * fh);
    lut_fill<VB>(sm + SP::OFF_V, fv.cent16, grp * fh + tid - 32 * P.group, G4_GROUPS * fh);
  }
  PHASE_STAMP(5);
  // every thread waits before it can touch the workspace or the output (the query warps already have)
  if (P.overlap) asm volatile("griddepcontrol.wait;" ::: "memory");
  const int n_pages = (seq_len + PT - 1) / PT;
  if (n_pages == 0 && split == 0) {  // empty sequence: zeros (split 0 exists for every kv head)
    for (int e = tid; e < P.group * TQ_D; e += ATT_THREADS) store_out(P.out, P.out_dtype, row0 * TQ_D + e, 0.f);
    if (P.lse && tid < P.group) P.lse[row0 + tid] = -INFINITY;
  }
  const int np = min(n_pages, page_lo + P.chunk_pages) - page_lo;
  const int ns = (n_pages + P.chunk_pages - 1) / P.chunk_pages;
  PHASE_STAMP(6);
  __syncthreads();               // the only CTA-wide barrier: tables, query buffers and mbarriers are ready
  if (np <= 0) return;           // this group has no pages (its split lies beyond the sequence)
  PHASE_STAMP(7);

  // B operand of S = K q^T: column g is head g & 3, hi half for g < 4, lo half otherwise
  uint32_t qf[8][2];
  {
    const int head = g & 3;
    const bool hv = head < P.group, lo = g >= 4;
    const float* qp = qbuf + (hv ? head : 0) * TQ_D + 32 * t;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float4 v = hv ? *reinterpret_cast<const float4*>(qp + 4 * (j ^ (t + 4 * (head & 1)))) : make_float4(0.f, 0.f, 0.f, 0.f);
      const __half2 h0 = __floats2half2_rn(v.x, v.y), h1 = __floats2half2_rn(v.z, v.w);
      const float2 f0 = __half22float2(h0), f1 = __half22float2(h1);
      qf[j][0] = lo ? pack_h2(v.x - f0.x, v.y - f0.y) : *reinterpret_cast<const uint32_t*>(&h0);
      qf[j][1] = lo ? pack_h2(v.z - f1.x, v.w - f1.y) : *reinterpret_cast<const uint32_t*>(&h1);
    }
  }
  const uint32_t lk_base = smem_u32(sm + SP::OFF_K) + (PairLut<KB>::REPL ? lane * 4 : 0);
  const uint32_t lv_base = smem_u32(sm + SP::OFF_V) + (PairLut<VB>::REPL ? lane * 4 : 0);
  // P operand: this thread's column is (head g >> 1, parity g & 1); the owner of p[token][head] is lane
  // 4 (token & 7) + 2 (token >> 3) + (head >> 1), half (head & 1) of its packed pair
  const int src0 = 16 * (t & 1) + 2 * (t >> 1) + (g >> 2);            // token 4t; token 4t + i is 4 i lanes further
  const uint32_t psel = ((g >> 1) & 1) ? ((g & 1) ? 0x3244u : 0x4432u) : ((g & 1) ? 0x1044u : 0x4410u);
  const int rsrc = (lane & ~3) | (t >> 1);                             // a lane that tracks head t's running maximum
  const bool upper = t >= 2;                                           // keeps token g + 8 after the exchange

  PHASE_STAMP(1);
  float o[4][4];
#pragma unroll
  for (int j = 0; j < 4; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

  constexpr int KIDXB = 16 * KB, VIDXB = 16 * VB, KW = KB;
  constexpr float MAX_SLACK = 4.0f;
  const int tiles_per_page = PT / 16;
  // byte offsets inside a page record that do not depend on the tile
  const uint32_t k_off = P.L.k_idx_off + g * KIDXB + t * (KIDXB / 4);
  const uint32_t v_off = P.L.v_idx_off + 4 * t * VIDXB + g * (2 * VB);
  const uint32_t ks_off = P.L.k_scale_off + 4 * (g + (upper ? 8 : 0));
  const uint32_t vs_off = P.L.v_scale_off + 4 * (g + (upper ? 8 : 0));

  for (int i = 0; i < np; ++i) {
    if (tid == PRODUCER && i + NS - 1 < np) {
      issue(i + NS - 1, pg_ahead);
      pg_ahead = bt[min(page_lo + i + NS, P.max_pages - 1)];
    }
    if (!s_flags[0] && !mbar_wait_bounded(&bars[i % NS], (uint32_t)((i / NS) & 1))) s_flags[0] = 1;
    const uint8_t* st = stage0 + (size_t)(i % NS) * rec;
    const int valid = min(PT, seq_len - (page_lo + i) * PT);

    for (int tile = warp; tile < tiles_per_page; tile += ATT_WARPS) {
      const int tb = tile * 16;
      if (tb >= valid) break;
      // ---------------- S = K_tile (16 tokens x 128) . [q_hi | q_lo] ----------------
      const float ks = *reinterpret_cast<const float*>(st + ks_off + 4 * tb);
      float sa[4] = {0.f, 0.f, 0.f, 0.f}, sb[4] = {0.f, 0.f, 0.f, 0.f};
      {
        uint32_t w0[KW], w1[KW];
        const uint32_t* p0 = reinterpret_cast<const uint32_t*>(st + k_off + tb * KIDXB);
        const uint32_t* p1 = p0 + 8 * (KIDXB / 4);
#pragma unroll
        for (int k = 0; k < KW; ++k) {
          w0[k] = __byte_perm(p0[k], 0, 0x0123);
          w1[k] = __byte_perm(p1[k], 0, 0x0123);
        }
        constexpr int SH = PairLut<KB>::SHIFT;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const uint32_t a0 = lds32(field_off<2 * KB, SH, KW>(w0, 2 * j) | lk_base);
          const uint32_t a1 = lds32(field_off<2 * KB, SH, KW>(w1, 2 * j) | lk_base);
          const uint32_t a2 = lds32(field_off<2 * KB, SH, KW>(w0, 2 * j + 1) | lk_base);
          const uint32_t a3 = lds32(field_off<2 * KB, SH, KW>(w1, 2 * j + 1) | lk_base);
          if (j & 1) mma16816(sb, a0, a1, a2, a3, qf[j][0], qf[j][1]);
          else mma16816(sa, a0, a1, a2, a3, qf[j][0], qf[j][1]);
        }
      }
      // the V words and both scales of this tile are fetched here, ahead of the softmax arithmetic that separates
      // them from their use: the loads then wait under it instead of in front of the table lookups
      uint32_t vw[4][2];
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) {
        const uint8_t* pv = st + v_off + tb * VIDXB + q4 * VIDXB;
        if constexpr (VB == 3) {
          const uint16_t* phw = reinterpret_cast<const uint16_t*>(pv);
          const uint32_t a = phw[0], bb = phw[1], c = phw[2];
          vw[q4][0] = __byte_perm(a, bb, 0x0145);
          vw[q4][1] = __byte_perm(c, 0, 0x0144);
        } else if constexpr (VB == 2) {
          vw[q4][0] = __byte_perm(*reinterpret_cast<const uint32_t*>(pv), 0, 0x0123);
          vw[q4][1] = 0;
        } else {
          const uint2 v2 = *reinterpret_cast<const uint2*>(pv);
          vw[q4][0] = __byte_perm(v2.x, 0, 0x0123);
          vw[q4][1] = __byte_perm(v2.y, 0, 0x0123);
        }
      }
      const float vs_raw = *reinterpret_cast<const float*>(st + vs_off + 4 * tb);
      // hi + lo: the partner lane (t ^ 2) holds the other half of the same heads
      const float give0 = upper ? sa[0] + sb[0] : sa[2] + sb[2], give1 = upper ? sa[1] + sb[1] : sa[3] + sb[3];
      const float keep0 = upper ? sa[2] + sb[2] : sa[0] + sb[0], keep1 = upper ? sa[3] + sb[3] : sa[1] + sb[1];
      const int tok = tb + g + (upper ? 8 : 0);
      const bool ok = tok < valid;
      float sc0 = (keep0 + __shfl_xor_sync(0xffffffffu, give0, 2)) * ks;
      float sc1 = (keep1 + __shfl_xor_sync(0xffffffffu, give1, 2)) * ks;
      sc0 = ok ? sc0 : -INFINITY;
      sc1 = ok ? sc1 : -INFINITY;
      // ---------------- online softmax (log2 domain), heads 2(t&1) and 2(t&1)+1 ----------------
      // The running maxima move only when a score exceeds them by more than 2^MAX_SLACK: probabilities then stay
      // below 2^MAX_SLACK (far inside fp16 and fp32 range) and almost every tile skips the warp reduction and the
      // rescaling of O.  The normalised result is the same up to rounding.
      if (__any_sync(0xffffffffu, (sc0 > m0 + MAX_SLACK) || (sc1 > m1 + MAX_SLACK))) {
        float mx0 = sc0, mx1 = sc1;
#pragma unroll
        for (int sh = 2; sh < 32; sh <<= 1) {
          mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, sh));
          mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, sh));
        }
        const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);  // finite: token tb is valid
        const float r0 = fast_exp2(m0 - mn0), r1 = fast_exp2(m1 - mn1);
        m0 = mn0;
        m1 = mn1;
        l0 *= r0;
        l1 *= r1;
        const float ra = __shfl_sync(0xffffffffu, r0, rsrc), rb = __shfl_sync(0xffffffffu, r1, rsrc);
        const float r = (t & 1) ? rb : ra;                        // O of this thread belongs to head t
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          o[j][0] *= r; o[j][1] *= r; o[j][2] *= r; o[j][3] *= r;
        }
      }
      const float p0 = fast_exp2(sc0 - m0), p1 = fast_exp2(sc1 - m1);
      l0 += p0;
      l1 += p1;
      // a template parameter, not a run-time flag: the possible jump keeps the V loads below it from being issued early
      if (SPARSE && !__any_sync(0xffffffffu, fmaxf(p0, p1) >= SPARSE_V_TAU)) continue;
      const float vs = ok ? vs_raw : 0.f;
      const uint32_t hp = pack_h2(p0 * vs, p1 * vs);
      uint32_t pb[4];
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) pb[q4] = __byte_perm(__shfl_sync(0xffffffffu, hp, src0 + 4 * q4), 0, psel);
      // ---------------- O^T += V_tile^T . P^T : tokens tb + 4t .. 4t+3, dims 16g .. 16g+15 ----------------
      uint32_t h[4][8];
      constexpr int SHV = PairLut<VB>::SHIFT;
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) {
#pragma unroll
        for (int jj = 0; jj < 8; ++jj) h[q4][jj] = lds32(field_off<2 * VB, SHV, 2>(vw[q4], jj) | lv_base);
      }
#pragma unroll
      for (int u = 0; u < 2; ++u) {
#pragma unroll
        for (int blk = 0; blk < 4; ++blk)
          mma16816(o[blk], h[2 * u][2 * blk], h[2 * u][2 * blk + 1], h[2 * u + 1][2 * blk], h[2 * u + 1][2 * blk + 1],
                   pb[2 * u], pb[2 * u + 1]);
      }
    }
    group_sync(bar_id);  // every warp of the group is done with this stage before it is refilled
  }

  PHASE_STAMP(2);
  // ---------------- merge the eight warps, write the split partial ----------------
#pragma unroll
  for (int sh = 2; sh < 32; sh <<= 1) {
    l0 += __shfl_xor_sync(0xffffffffu, l0, sh);
    l1 += __shfl_xor_sync(0xffffffffu, l1, sh);
  }
  float* so = reinterpret_cast<float*>(stage0);                    // [warp][head 4][G4_HSTRIDE]
  float* sml = so + ATT_WARPS * G4_HEADS * G4_HSTRIDE;             // [warp][head 4][2]
#pragma unroll
  for (int blk = 0; blk < 4; ++blk)
    *reinterpret_cast<float4*>(so + (size_t)(warp * G4_HEADS + t) * G4_HSTRIDE + 16 * g + 4 * blk) =
        make_float4(o[blk][0], o[blk][1], o[blk][2], o[blk][3]);
  if (g == 0 && t < 2) {
    *reinterpret_cast<float4*>(sml + (warp * G4_HEADS + 2 * t) * 2) = make_float4(m0, l0, m1, l1);
  }
  group_sync(bar_id);
  for (int e = tid; e < P.group * TQ_D; e += ATT_THREADS) {
    const int head = e >> 7, dim = e & 127;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < ATT_WARPS; ++w) M = fmaxf(M, sml[(w * G4_HEADS + head) * 2]);
    float acc = 0.f, Lsum = 0.f;
#pragma unroll
    for (int w = 0; w < ATT_WARPS; ++w) {
      const float mw = sml[(w * G4_HEADS + head) * 2];
      const float f = mw == -INFINITY ? 0.f : fast_exp2(mw - M);
      acc = fmaf(so[(size_t)(w * G4_HEADS + head) * G4_HSTRIDE + dim], f, acc);
      Lsum = fmaf(sml[(w * G4_HEADS + head) * 2 + 1], f, Lsum);
    }
    const size_t slot = (row0 + head) * P.num_splits + split;
    P.part_o[slot * TQ_D + dim] = acc;
    if (dim == 0) {
      P.part_ml[slot * 2] = M;
      P.part_ml[slot * 2 + 1] = Lsum;
    }
  }
  PHASE_STAMP(11);
  finish_splits<false>(P, fv.s1, fv.s2, fv.alpha, qbuf, stage0, s_flags, row0, ns, b, kvh, tid, bar_id);
  PHASE_STAMP(4);
}

// ------------------------------------------------------------------------------------------
// dense rotations of the queries (the d x d matrix is too large to apply once per CTA)
template <typename Tq>
__global__ void __launch_bounds__(128) k_prepare_queries(const Tq* __restrict__ q, int64_t rows, float qscale,
                                                         const float* __restrict__ rot_t, float alpha, int prod,
                                                         const float* __restrict__ s_t, float* __restrict__ qrot,
                                                         float* __restrict__ qproj) {
  __shared__ float xs[TQ_D];
  const int j = threadIdx.x;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    xs[j] = (float)q[row * TQ_D + j];
    __syncthreads();
    float y = 0.f;
#pragma unroll 8
    for (int k = 0; k < TQ_D; ++k) y = fmaf(__ldg(rot_t + k * TQ_D + j), xs[k], y);  // (R x)_j
    qrot[row * TQ_D + j] = y * (qscale / alpha);
    if (prod) {
      float z = 0.f;
#pragma unroll 8
      for (int k = 0; k < TQ_D; ++k) z = fmaf(__ldg(s_t + k * TQ_D + j), xs[k], z);  // (S x)_j
      qproj[row * TQ_D + j] = z * qscale;
    }
    __syncthreads();
  }
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
  size_t qrot, qproj, part_o, part_ml, total;
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
  w.total = off + TAIL_BYTES;  // tickets and the status word live at the very end of the caller's buffer
  return w;
}

template <int KK, int VK>
int launch_attn(const AttnParams& P, const TqFast& fk, const TqFast& fv, cudaStream_t st) {
  const size_t need = SmemPlan<KK, VK>::bytes(P.L.record_bytes, P.stages);
  TQ_REQUIRE(need <= 113 * 1024, TQ_ERR_TOO_LARGE, "page record of %d bytes does not fit the shared-memory pipeline",
             P.L.record_bytes);
  static thread_local int configured_dev = -1;  // per instantiation
  int dev = 0;
  TQ_CUDA(cudaGetDevice(&dev));
  if (configured_dev != dev) {
    TQ_CUDA(cudaFuncSetAttribute(k_decode_attn<KK, VK>, cudaFuncAttributeMaxDynamicSharedMemorySize, 113 * 1024));
    configured_dev = dev;
  }
  dim3 grid(P.num_splits, P.hkv, P.batch);
  k_decode_attn<KK, VK><<<grid, ATT_THREADS, need, st>>>(P, fk, fv);
  return tq_launch_check("k_decode_attn");
}

template <int KB, int VB, bool SPARSE>
int launch_attn_g4(const AttnParams& P, const TqFast& fk, const TqFast& fv, cudaStream_t st) {
  using SP = SmemPlan<KB, VB>;
  const size_t need = (size_t)SP::ALIGN + SP::OFF_Q + G4_GROUPS * g4_group_bytes<KB, VB>(P.L.record_bytes, P.stages);
  constexpr size_t LIMIT = 220 * 1024;  // one CTA per SM
  TQ_REQUIRE(need <= LIMIT, TQ_ERR_TOO_LARGE, "page record of %d bytes does not fit the shared-memory pipeline",
             P.L.record_bytes);
  static thread_local int configured_dev = -1;  // per instantiation
  int dev = 0;
  TQ_CUDA(cudaGetDevice(&dev));
  if (configured_dev != dev) {
    TQ_CUDA(cudaFuncSetAttribute(k_decode_attn_g4<KB, VB, SPARSE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)LIMIT));
    configured_dev = dev;
  }
  AttnQuant ak, av;
  memset(&ak, 0, sizeof(ak));
  memset(&av, 0, sizeof(av));
  memcpy(ak.s1, fk.s1, 16); memcpy(ak.s2, fk.s2, 16); memcpy(ak.cent16, fk.cent16, 32); ak.alpha = fk.lut_alpha;
  memcpy(av.s1, fv.s1, 16); memcpy(av.s2, fv.s2, 16); memcpy(av.cent16, fv.cent16, 32); av.alpha = fv.lut_alpha;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3((P.num_splits * P.hkv + G4_GROUPS - 1) / G4_GROUPS, P.batch);
  cfg.blockDim = dim3(G4_THREADS);
  cfg.dynamicSmemBytes = need;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = P.overlap ? 1 : 0;
  TQ_CUDA(cudaLaunchKernelEx(&cfg, k_decode_attn_g4<KB, VB, SPARSE>, P, ak, av));
  return tq_launch_check("k_decode_attn_g4");
}

bool fmt_ok(int fmt, bool is_k) {
  if (fmt >= TQ_FMT_TURBO2 && fmt <= TQ_FMT_TURBO4) return true;
  if (fmt == TQ_FMT_Q8_0) return true;
  return is_k && fmt >= TQ_FMT_PROD2 && fmt <= TQ_FMT_PROD4;
}

}  // namespace

#ifdef TQ_PHASE_TIMING
extern "C" int tq_debug_phase_log(void* host_out, long long bytes) {
  return cudaMemcpyFromSymbol(host_out, g_phase_log, (size_t)bytes) == cudaSuccess ? 0 : -1;
}
#endif

extern "C" int64_t tq_decode_workspace_bytes(int32_t batch, int32_t num_q_heads, int32_t num_kv_heads,
                                             int32_t max_pages_per_seq) {
  if (batch < 1 || num_q_heads < 1 || num_kv_heads < 1 || max_pages_per_seq < 1) return TQ_ERR_INVALID;
  const SplitPlan p = plan_splits(batch, num_kv_heads, max_pages_per_seq);
  return (int64_t)ws_layout(batch, num_q_heads, p.num_splits).total;
}

extern "C" int tq_decode_workspace_init(void* workspace_dev, int64_t workspace_bytes, void* stream) {
  TQ_REQUIRE(workspace_dev && workspace_bytes >= (int64_t)TAIL_BYTES, TQ_ERR_INVALID,
             "workspace must hold at least %lld bytes", (long long)TAIL_BYTES);
  TQ_CUDA(cudaMemsetAsync((uint8_t*)workspace_dev + workspace_bytes - TAIL_BYTES, 0, TAIL_BYTES, (cudaStream_t)stream));
  return TQ_OK;
}

extern "C" int tq_decode_status_sync(const void* workspace_dev, int64_t workspace_bytes, int32_t* status_out) {
  TQ_REQUIRE(workspace_dev && status_out && workspace_bytes >= 256, TQ_ERR_INVALID, "bad workspace");
  TQ_CUDA(cudaMemcpy(status_out, (const uint8_t*)workspace_dev + workspace_bytes - 256, 4, cudaMemcpyDeviceToHost));
  return TQ_OK;
}

extern "C" int tq_decode_attn(const tq_quantizer* kq, const tq_quantizer* vq, const tq_cache_layout* L,
                              const uint8_t* pool_dev, const int32_t* block_table_dev, int32_t max_pages_per_seq,
                              const int32_t* seq_lens_dev, const void* q_dev, int32_t q_dtype, int32_t batch,
                              int32_t num_q_heads, float scale, void* workspace_dev, int64_t workspace_bytes,
                              void* out_dev, int32_t out_dtype, void* stream) {
  return tq_decode_attn_phases(kq, vq, L, pool_dev, block_table_dev, max_pages_per_seq, seq_lens_dev, q_dev, q_dtype,
                               batch, num_q_heads, scale, workspace_dev, workspace_bytes, out_dev, out_dtype, 3, stream);
}

static int decode_impl(const tq_quantizer* kq, const tq_quantizer* vq, const tq_cache_layout* L,
                       const uint8_t* pool_dev, const int32_t* block_table_dev, int32_t max_pages_per_seq,
                       const int32_t* seq_lens_dev, const void* q_dev, int32_t q_dtype, int32_t batch,
                       int32_t num_q_heads, float scale, void* workspace_dev, int64_t workspace_bytes, void* out_dev,
                       int32_t out_dtype, int32_t phases, float* lse_dev, void* stream) {
  TQ_REQUIRE(L, TQ_ERR_INVALID, "tq_decode_attn: layout missing");
  TQ_REQUIRE(batch >= 0 && num_q_heads >= 1 && max_pages_per_seq >= 1, TQ_ERR_INVALID, "bad sizes");
  if (batch == 0) return TQ_OK;
  TQ_REQUIRE(pool_dev && block_table_dev && seq_lens_dev && q_dev && out_dev && workspace_dev, TQ_ERR_INVALID,
             "tq_decode_attn: null buffer");
  TQ_REQUIRE(L->d == TQ_D, TQ_ERR_UNSUPPORTED, "decode attention is built for d == 128");
  TQ_REQUIRE(fmt_ok(L->k_format, true) && fmt_ok(L->v_format, false), TQ_ERR_UNSUPPORTED,
             "decode attention: K format %d / V format %d unknown", L->k_format, L->v_format);
  const bool k_q8 = L->k_format == TQ_FMT_Q8_0, v_q8 = L->v_format == TQ_FMT_Q8_0;
  const bool k_prod = L->k_format >= TQ_FMT_PROD2;
  TQ_REQUIRE(k_q8 || kq, TQ_ERR_INVALID, "tq_decode_attn: K quantizer missing");
  TQ_REQUIRE(v_q8 || vq, TQ_ERR_INVALID, "tq_decode_attn: V quantizer missing");
  TQ_REQUIRE(num_q_heads % L->num_kv_heads == 0, TQ_ERR_INVALID, "num_q_heads must be a multiple of num_kv_heads");
  const int group = num_q_heads / L->num_kv_heads;
  TQ_REQUIRE(group <= MAX_G, TQ_ERR_UNSUPPORTED, "at most %d query heads per KV head, got %d", MAX_G, group);
  TQ_REQUIRE(batch <= 65535 && L->num_kv_heads <= 65535 && (int64_t)batch * L->num_kv_heads <= MAX_TICKETS,
             TQ_ERR_TOO_LARGE, "batch x KV heads beyond %d", MAX_TICKETS);
  TQ_REQUIRE(tq_aligned(pool_dev, 128) && tq_aligned(workspace_dev, 256) && tq_aligned(q_dev, 16) && tq_aligned(out_dev, 16),
             TQ_ERR_ALIGN, "pool (128), workspace (256), q and out (16) must be aligned");
  TQ_REQUIRE(workspace_bytes % 256 == 0, TQ_ERR_ALIGN, "workspace size must be a multiple of 256 bytes");
  TQ_REQUIRE(q_dtype == TQ_F16 || q_dtype == TQ_BF16 || q_dtype == TQ_F32, TQ_ERR_UNSUPPORTED,
             "queries must be fp16, bf16 or fp32, got dtype %d", q_dtype);
  TQ_REQUIRE(out_dtype == TQ_F16 || out_dtype == TQ_BF16 || out_dtype == TQ_F32, TQ_ERR_UNSUPPORTED,
             "output must be fp16, bf16 or fp32, got dtype %d", out_dtype);
  if (!k_q8) {
    const int kb = k_prod ? L->k_format - 17 : L->k_format;
    TQ_REQUIRE(kq->d == TQ_D && kq->bits == kb, TQ_ERR_INVALID, "K quantizer bit width does not match the cache format");
    TQ_REQUIRE(!k_prod || kq->qjl, TQ_ERR_INVALID, "PROD cache format needs a K quantizer with a QJL stage");
  }
  if (!v_q8) TQ_REQUIRE(vq->d == TQ_D && vq->bits == L->v_format, TQ_ERR_INVALID,
                        "V quantizer bit width does not match the cache format");
  const SplitPlan plan = plan_splits(batch, L->num_kv_heads, max_pages_per_seq);
  const WsLayout w = ws_layout(batch, num_q_heads, plan.num_splits);
  TQ_REQUIRE((int64_t)w.total <= workspace_bytes, TQ_ERR_TOO_LARGE, "workspace of %lld bytes is smaller than the %lld needed",
             (long long)workspace_bytes, (long long)w.total);
  cudaStream_t st = (cudaStream_t)stream;
  uint8_t* ws = (uint8_t*)workspace_dev;
  if (scale <= 0.f) scale = TQ_RSQRT_D;
  const float qscale = scale * 1.4426950408889634f;
  const int64_t rows = (int64_t)batch * num_q_heads;
  const bool k_dense = !k_q8 && kq->rotation == TQ_ROT_DENSE, v_dense = !v_q8 && vq->rotation == TQ_ROT_DENSE;
  float* qrot = reinterpret_cast<float*>(ws + w.qrot);
  float* qproj = reinterpret_cast<float*>(ws + w.qproj);
  int rc = TQ_OK;
  if ((phases & 1) && k_dense) {
    const int pgrid = (int)(rows < 4096 ? rows : 4096);
#define TQ_PREP(T)                                                                                              \
  k_prepare_queries<T><<<pgrid, 128, 0, st>>>((const T*)q_dev, rows, qscale, kq->rot32_t, kq->fast.lut_alpha,   \
                                              k_prod ? 1 : 0, kq->s32_t, qrot, qproj)
    if (q_dtype == TQ_F16) TQ_PREP(__half);
    else if (q_dtype == TQ_BF16) TQ_PREP(__nv_bfloat16);
    else TQ_PREP(float);
#undef TQ_PREP
    rc = tq_launch_check("k_prepare_queries");
    if (rc != TQ_OK) return rc;
  }
  if (!(phases & 2)) return TQ_OK;

  AttnParams P;
  memset(&P, 0, sizeof(P));
  P.pool = pool_dev;
  P.block_table = block_table_dev;
  P.seq_lens = seq_lens_dev;
  P.q = q_dev;
  P.qrot = qrot;
  P.qproj = qproj;
  P.part_o = reinterpret_cast<float*>(ws + w.part_o);
  P.part_ml = reinterpret_cast<float*>(ws + w.part_ml);
  P.tickets = reinterpret_cast<int32_t*>(ws + workspace_bytes - TAIL_BYTES);
  P.status = reinterpret_cast<int32_t*>(ws + workspace_bytes - 256);
  P.out = out_dev;
  P.lse = lse_dev;
  P.v_rot = v_dense ? vq->rot32 : nullptr;
  P.qscale = qscale;
  P.q_dtype = q_dtype;
  P.out_dtype = out_dtype;
  P.k_pre = k_dense ? 1 : 0;
  P.k_ident = k_q8 ? 1 : 0;
  P.v_ident = v_q8 ? 1 : 0;
  P.max_pages = max_pages_per_seq;
  P.batch = batch;
  P.hq = num_q_heads;
  P.hkv = L->num_kv_heads;
  P.group = group;
  P.chunk_pages = plan.chunk_pages;
  P.num_splits = plan.num_splits;
  P.stages = L->record_bytes > 24 * 1024 ? 2 : 3;
  P.overlap = (phases & TQ_DECODE_OVERLAP) ? 1 : 0;
  P.sparse_v = (phases & TQ_DECODE_SPARSE_V) ? 1 : 0;
  P.L = *L;
  TqFast none;
  memset(&none, 0, sizeof(none));
  none.lut_alpha = 1.0f;
  const TqFast& fk = k_q8 ? none : kq->fast;
  const TqFast& fv = v_q8 ? none : vq->fast;
  rc = TQ_ERR_UNSUPPORTED;
  tq_set_error("decode attention: K format %d with V format %d is not instantiated", L->k_format, L->v_format);
  // PolarQuant K and V with at most four query heads per KV head take the kernel specialised for that shape
  const bool g4 = group <= G4_HEADS && !k_q8 && !v_q8 && !k_prod;
#define TQ_ATT_G4(K, V) \
  if (g4 && L->k_format == K && L->v_format == V)               \
    rc = P.sparse_v ? launch_attn_g4<K, V, true>(P, fk, fv, st) : launch_attn_g4<K, V, false>(P, fk, fv, st);
  TQ_ATT_G4(2, 2) TQ_ATT_G4(2, 3) TQ_ATT_G4(2, 4) TQ_ATT_G4(3, 2) TQ_ATT_G4(3, 3) TQ_ATT_G4(3, 4) TQ_ATT_G4(4, 2)
  TQ_ATT_G4(4, 3) TQ_ATT_G4(4, 4)
#undef TQ_ATT_G4
  if (g4) return rc;
#define TQ_ATT(K, V) \
  if (L->k_format == K && L->v_format == V) rc = launch_attn<K, V>(P, fk, fv, st);
  TQ_ATT(2, 2) TQ_ATT(2, 3) TQ_ATT(2, 4) TQ_ATT(3, 2) TQ_ATT(3, 3) TQ_ATT(3, 4) TQ_ATT(4, 2) TQ_ATT(4, 3) TQ_ATT(4, 4)
  TQ_ATT(8, 2) TQ_ATT(8, 3) TQ_ATT(8, 4) TQ_ATT(8, 8)
  TQ_ATT(18, 2) TQ_ATT(18, 3) TQ_ATT(19, 2) TQ_ATT(19, 3) TQ_ATT(19, 4) TQ_ATT(20, 3) TQ_ATT(20, 4)
#undef TQ_ATT
  return rc;
}

extern "C" int tq_decode_attn_phases(const tq_quantizer* kq, const tq_quantizer* vq, const tq_cache_layout* L,
                                     const uint8_t* pool_dev, const int32_t* block_table_dev,
                                     int32_t max_pages_per_seq, const int32_t* seq_lens_dev, const void* q_dev,
                                     int32_t q_dtype, int32_t batch, int32_t num_q_heads, float scale,
                                     void* workspace_dev, int64_t workspace_bytes, void* out_dev, int32_t out_dtype,
                                     int32_t phases, void* stream) {
  return decode_impl(kq, vq, L, pool_dev, block_table_dev, max_pages_per_seq, seq_lens_dev, q_dev, q_dtype, batch,
                     num_q_heads, scale, workspace_dev, workspace_bytes, out_dev, out_dtype, phases, nullptr, stream);
}

extern "C" int tq_decode_attn_lse(const tq_quantizer* kq, const tq_quantizer* vq, const tq_cache_layout* L,
                                  const uint8_t* pool_dev, const int32_t* block_table_dev, int32_t max_pages_per_seq,
                                  const int32_t* seq_lens_dev, const void* q_dev, int32_t q_dtype, int32_t batch,
                                  int32_t num_q_heads, float scale, void* workspace_dev, int64_t workspace_bytes,
                                  void* out_dev, int32_t out_dtype, int32_t phases, float* lse_dev, void* stream) {
  TQ_REQUIRE(lse_dev, TQ_ERR_INVALID, "tq_decode_attn_lse: lse buffer is null");
  return decode_impl(kq, vq, L, pool_dev, block_table_dev, max_pages_per_seq, seq_lens_dev, q_dev, q_dtype, batch,
                     num_q_heads, scale, workspace_dev, workspace_bytes, out_dev, out_dtype, phases, lse_dev, stream);
}

// out = (e^la a + e^lb b) / (e^la + e^lb) per row: joins the attention outputs of two disjoint parts of one sequence
// (say, old pages kept at fewer bits in another cache) from their log-sum-exps.  One warp per 128-wide row.
template <typename T>
__global__ void __launch_bounds__(256) k_attn_merge(const T* a, const float* la, const T* b, const float* lb,
                                                    int64_t rows, T* out, float* lse_out) {  // out may be a or b
  const int lane = threadIdx.x & 31;
  const int64_t row = ((int64_t)blockIdx.x * 256 + threadIdx.x) >> 5;
  if (row >= rows) return;
  const float x = la[row], y = lb[row], m = fmaxf(x, y);
  float wa = 0.5f, wb = 0.5f, l = m;
  if (m == -INFINITY) { wa = wb = 0.f; }   // both parts empty: zeros
  else {
    const float ea = __expf(x - m), eb = __expf(y - m);
    wa = ea / (ea + eb);
    wb = eb / (ea + eb);
    l = m + logf(ea + eb);
  }
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int64_t i = row * TQ_D + 4 * lane + k;
    const float av = wa == 0.f ? 0.f : (float)a[i] * wa, bv = wb == 0.f ? 0.f : (float)b[i] * wb;
    out[i] = (T)(av + bv);
  }
  if (lse_out && lane == 0) lse_out[row] = l;
}

extern "C" int tq_attn_merge(const void* out_a_dev, const float* lse_a_dev, const void* out_b_dev,
                             const float* lse_b_dev, int64_t rows, int32_t dtype, void* out_dev, float* lse_out_dev,
                             void* stream) {
  TQ_REQUIRE(rows >= 0, TQ_ERR_INVALID, "tq_attn_merge: rows must be >= 0");
  if (rows == 0) return TQ_OK;
  TQ_REQUIRE(out_a_dev && lse_a_dev && out_b_dev && lse_b_dev && out_dev, TQ_ERR_INVALID, "tq_attn_merge: null buffer");
  const int grid = (int)((rows * 32 + 255) / 256);
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == TQ_F32)
    k_attn_merge<float><<<grid, 256, 0, st>>>((const float*)out_a_dev, lse_a_dev, (const float*)out_b_dev, lse_b_dev, rows,
                                              (float*)out_dev, lse_out_dev);
  else if (dtype == TQ_F16)
    k_attn_merge<__half><<<grid, 256, 0, st>>>((const __half*)out_a_dev, lse_a_dev, (const __half*)out_b_dev, lse_b_dev,
                                               rows, (__half*)out_dev, lse_out_dev);
  else if (dtype == TQ_BF16)
    k_attn_merge<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)out_a_dev, lse_a_dev,
                                                      (const __nv_bfloat16*)out_b_dev, lse_b_dev, rows,
                                                      (__nv_bfloat16*)out_dev, lse_out_dev);
  else {
    tq_set_error("tq_attn_merge: outputs must be fp16, bf16 or fp32, got dtype %d", dtype);
    return TQ_ERR_UNSUPPORTED;
  }
  return tq_launch_check("k_attn_merge");
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
  // What must start at zero: the ticket counters at the end of the array.  The array is zero when the
  // library is loaded, and every call leaves its counters at zero again (the CTA that takes the last
  // ticket resets it), so nothing is cleared here.  Partials are written before they are read.
  return tq_decode_attn_phases(kq, vq, L, pool_dev, block_table_dev, max_pages_per_seq, seq_lens_dev, q_dev, q_dtype,
                               batch, num_q_heads, scale, scratch, TQ_STATIC_SCRATCH_BYTES, out_dev, out_dtype, 3,
                               stream);
}
