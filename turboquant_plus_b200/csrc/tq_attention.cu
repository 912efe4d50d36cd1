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

#include "tq_attention.cuh"

namespace {

using namespace tqatt;

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
  const int PT = P.L.page_tokens;
  // a length beyond the block-table row (or a negative one) is clamped: page numbers are only ever read from the
  // row's max_pages entries, and the split count stays inside the plan the workspace was sized for
  const int seq_len = min(max(P.seq_lens[b], 0), P.max_pages * PT);
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
  __syncthreads();

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
      // The running reference is the maximum of score + log2(V scale), not of the score alone: the P operand of the
      // second product is p * (V scale) in fp16 and then never exceeds 1 whatever the norms of the values are (a
      // higher reference scales p, the softmax sums and O alike; the final division removes it).
      float vs0 = 1.0f, vs1 = 1.0f, lv0 = 0.f, lv1 = 0.f;
      if (!VT::Q8) {
        const float* vsc = reinterpret_cast<const float*>(st + P.L.v_scale_off);
        vs0 = ok0 ? vsc[tb + g] : 0.f;     // a stale scale must not meet p = 0
        vs1 = ok1 ? vsc[tb + g + 8] : 0.f;
        lv0 = fmaxf(fast_log2(vs0), -100.0f);   // zero vectors have scale 0
        lv1 = fmaxf(fast_log2(vs1), -100.0f);
      }
      float mx0 = fmaxf(s[0] + lv0, s[2] + lv1), mx1 = fmaxf(s[1] + lv0, s[3] + lv1);
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
      // the threshold of the sparse-V option is relative to the largest weight, i.e. to the score maximum
      if (P.sparse_v && !__any_sync(0xffffffffu, fmaxf(fmaxf(p00 * vs0, p01 * vs0), fmaxf(p10 * vs1, p11 * vs1)) >= SPARSE_V_TAU)) continue;
      // probabilities (* V scale), as fp16, transposed into the B-operand layout (tokens on K)
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

bool fmt_ok(int fmt, bool is_k) {
  if (fmt >= TQ_FMT_TURBO2 && fmt <= TQ_FMT_TURBO4) return true;
  if (fmt == TQ_FMT_Q8_0) return true;
  return is_k && fmt >= TQ_FMT_PROD2 && fmt <= TQ_FMT_PROD4;
}

}  // namespace

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

// The give-up path of the bounded waits, run on purpose where it is harmless: one warp waits on an mbarrier that
// nothing ever arrives at, with a limit of 2^20 clocks (about half a millisecond) instead of the kernels' 2^30, gives up,
// raises the workspace's status word exactly as the attention kernels do, and returns.  Nothing hangs and nothing
// faults: the context stays usable, which is what the test after it checks.
__global__ void k_selftest_wait_gives_up(int32_t* status) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    tqatt::mbar_init(&bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();
  const bool done = tqatt::mbar_wait_bounded(&bar, 0, 1LL << 20);
  if (!__all_sync(0xffffffffu, done) && threadIdx.x == 0) atomicExch(status, 1);
}

extern "C" int tq_selftest_wait_gives_up(void* workspace_dev, int64_t workspace_bytes, void* stream) {
  TQ_REQUIRE(workspace_dev && workspace_bytes >= 256, TQ_ERR_INVALID, "bad workspace");
  int32_t* word = reinterpret_cast<int32_t*>((uint8_t*)workspace_dev + workspace_bytes - 256);
  k_selftest_wait_gives_up<<<1, 32, 0, (cudaStream_t)stream>>>(word);
  return tq_launch_check("k_selftest_wait_gives_up");
}

extern "C" int tq_decode_status_sync(void* workspace_dev, int64_t workspace_bytes, int32_t* status_out) {
  TQ_REQUIRE(workspace_dev && status_out && workspace_bytes >= 256, TQ_ERR_INVALID, "bad workspace");
  uint8_t* word = (uint8_t*)workspace_dev + workspace_bytes - 256;
  TQ_CUDA(cudaMemcpy(status_out, word, 4, cudaMemcpyDeviceToHost));
  // the word is only ever set by the kernels; reading it is what clears it
  if (*status_out != 0) TQ_CUDA(cudaMemset(word, 0, 4));
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
  P.nodeq = (phases & TQ_DECODE_NO_DEQUANT) ? 1 : 0;
  // queries come from the preceding kernel when the K rotation is dense (k_prepare_queries writes them)
  P.q_early = ((phases & TQ_DECODE_OVERLAP_Q) == TQ_DECODE_OVERLAP_Q && !k_dense) ? 1 : 0;
  // After an append only the specialised kernel knows to fetch the page of the new token late; everything else runs
  // in stream order.
  const bool after_append = (phases & TQ_DECODE_OVERLAP_APPEND) == TQ_DECODE_OVERLAP_APPEND;
  P.tail_late = after_append && P.q_early && !P.sparse_v ? 1 : 0;
  if (after_append && !P.tail_late) P.overlap = P.q_early = 0;
  P.chain_head = (phases & TQ_DECODE_CHAIN_HEAD) ? 1 : 0;
  P.kv_div = 1;
  P.L = *L;
  TqFast none;
  memset(&none, 0, sizeof(none));
  none.lut_alpha = 1.0f;
  const TqFast& fk = k_q8 ? none : kq->fast;
  const TqFast& fv = v_q8 ? none : vq->fast;
  rc = TQ_ERR_UNSUPPORTED;
  tq_set_error("decode attention: K format %d with V format %d is not instantiated", L->k_format, L->v_format);
  // PolarQuant K and V with at most four query heads per KV head on 128-token pages take the kernel specialised
  // for that shape (tq_decode_g4.cu)
  if (tq_decode_g4_try(P, fk, fv, st, &rc)) return rc;
  if (after_append) P.overlap = P.q_early = P.tail_late = 0;   // the general kernel: stream order
  rc = TQ_ERR_UNSUPPORTED;
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
  // What must start at zero: the ticket counters of this call's (sequence, KV head) pairs at the end of the
  // array.  A clean call leaves them at zero, but a caller cannot re-initialise this array the way it can a
  // workspace of its own, so they are cleared here on the stream (an asynchronous memset: no allocation, no
  // synchronisation); a call that was torn down half-way then cannot mislead the next one.  Partials are written
  // before they are read.
  uint8_t* tail = (uint8_t*)scratch + TQ_STATIC_SCRATCH_BYTES - TAIL_BYTES;
  // (up to four counters per (sequence, KV head): groups of more than four query heads are dealt to several CTAs)
  const size_t counters = (size_t)batch * L->num_kv_heads * 4;
  TQ_CUDA(cudaMemsetAsync(tail, 0, (counters < (size_t)MAX_TICKETS ? counters : (size_t)MAX_TICKETS) * 4, (cudaStream_t)stream));
  return tq_decode_attn_phases(kq, vq, L, pool_dev, block_table_dev, max_pages_per_seq, seq_lens_dev, q_dev, q_dtype,
                               batch, num_q_heads, scale, scratch, TQ_STATIC_SCRATCH_BYTES, out_dev, out_dtype, 3,
                               stream);
}

extern "C" int tq_decode_static_status_sync(int32_t* status_out) {
  TQ_REQUIRE(status_out, TQ_ERR_INVALID, "tq_decode_static_status_sync: status_out is null");
  void* scratch = nullptr;
  int rc = static_scratch_for_current_device(&scratch);
  if (rc != TQ_OK) return rc;
  return tq_decode_status_sync(scratch, TQ_STATIC_SCRATCH_BYTES, status_out);
}
