// Pieces shared by the decode-attention kernels (tq_attention.cu: any format pair; tq_decode_g4.cu: PolarQuant
// K and V with at most four query heads per KV head): PTX wrappers, the kernel parameter block, the pair tables,
// and the split merge that both kernels end with.
#pragma once
#include "tq_internal.cuh"

namespace tqatt {


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
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, long long limit = WAIT_CYCLES) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  while (clock64() - t0 < limit)
    if (mbar_try_wait(bar, parity)) return true;
  return false;
}

// Barrier `id` over one 256-thread group.  id 0 with a 256-thread CTA is the block barrier; a 512-thread CTA runs
// two independent groups on ids 1 and 2.
template <int NT = ATT_THREADS>
__device__ __forceinline__ void group_sync(int id) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "n"(NT) : "memory");
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
__device__ __forceinline__ float fast_log2(float x) {
  float y;
  asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
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
  int32_t nodeq;       // measurement variant without table lookups (results meaningless): TQ_DECODE_NO_DEQUANT
  int32_t q_early;     // the preceding kernel does not write the queries: they are read before the dependency wait
  int32_t tail_late;   // the preceding kernel may write the last cached position of a sequence: its page is fetched
                       // after the dependency wait, every other page before (TQ_DECODE_OVERLAP_APPEND)
  int32_t chain_head;  // attention calls with TQ_DECODE_OVERLAP_Q follow this one (TQ_DECODE_CHAIN_HEAD)
  int32_t kv_div;      // CTAs (grid.y entries) per KV head of the cache: hkv and group describe the query-head groups
                       // that a CTA serves, kv_div of which share a KV head (specialised kernel, groups of 5..16 heads)
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
template <bool V_Q8, int NT = ATT_THREADS>
__device__ __forceinline__ void finish_splits(const AttnParams& P, const uint32_t (&vs1)[4], const uint32_t (&vs2)[4],
                                              float v_alpha, float* qbuf, uint8_t* stage0, volatile int* s_flags,
                                              size_t row0, int ns, int b, int kvh, int tid = threadIdx.x, int bar_id = 0) {
  const int lane = tid & 31, warp = tid >> 5;
  group_sync<NT>(bar_id);
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
  group_sync<NT>(bar_id);
  if (!s_flags[1]) return;
  // Warp (half, head) folds the splits of one head.  With at most four heads there are two warps per head and each
  // takes 64 of the 128 dims: lanes 0..15 then read even splits, lanes 16..31 odd ones (16 bytes each), and one
  // lane exchange joins the two at the end; with more heads a warp takes the whole row and every split.
  if (2 * P.group <= NT / 32) fold_splits<2, V_Q8>(P, v_alpha, qbuf, row0, ns, warp);
  else fold_splits<1, V_Q8>(P, v_alpha, qbuf, row0, ns, warp);
  group_sync<NT>(bar_id);
  if (P.v_rot) {  // dense rotation: x = R^T y
    for (int e = tid; e < P.group * TQ_D; e += NT) {
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

// Split plan shared by the launchers and the workspace sizing.
struct SplitPlan {
  int chunk_pages, num_splits;
};

}  // namespace tqatt

// tq_decode_g4.cu: launches the kernel specialised for PolarQuant K and V, <= 4 query heads per KV head, 128-token
// pages in the layout tq_cache_layout_init produces.  Returns false (nothing launched) when the call is not of that
// shape; otherwise *rc is the launch status.
bool tq_decode_g4_try(const tqatt::AttnParams& P, const TqFast& fk, const TqFast& fv, cudaStream_t st, int* rc);
