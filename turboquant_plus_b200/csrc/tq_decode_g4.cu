// Decode attention for at most four query heads per KV head on 128-token pages: the shape of the headline workload
// (Llama-3-8B: 32 query / 8 KV heads, turbo3 K and V) and of the other decode configurations (q8_0 keys with turbo2
// values, PROD keys -- PolarQuant + QJL sign sketch -- with turbo3 values).  Same pipeline and the same split /
// ticket protocol as k_decode_attn (tq_attention.cu); what changes is how the 8 columns of the MMA tiles are
// spent, and that everything the page loop needs is a compile-time constant:
//   * S = K q^T: columns 0..3 carry the fp16 "hi" halves of the four query heads, columns 4..7 the "lo" halves,
//     so one m16n8k16 per 16 dims instead of two; the halves meet through one lane exchange (lane ^ 2), after
//     which thread (g, t) owns one token (g + 8 (t >> 1)) and two heads (2 (t & 1), + 1).
//   * O^T += V^T P^T: a k-slot pair is (token, dim parity) instead of (token, token'), column n is
//     (head n >> 1, parity n & 1), and the P operand is p on the matching parity, 0 on the other.  A pair-table
//     word (two dims of one token) is then an A-operand register as it comes: no re-pairing permutes, 32 dims per
//     MMA, and O takes 16 accumulator registers per thread: o[blk] = head t, dims 16 g + 4 blk .. + 3.
//   * the running maxima are only reduced across the warp when some score exceeds them.
//   * page size (128 tokens = one 16-token tile per warp and page), pipeline depth (3 records) and every offset
//     inside a record are template constants; record bytes are read through 32-bit shared-memory addresses with
//     immediate offsets; only the last page of a sequence runs the variant that masks tokens past the end.
//   * q8_0 operands are int8 -> fp16 by byte permute + one subtract (exact), the per-block scales applied to the
//     partial scores of each 32-dim block in fp32 (keys) or to the operand pairs (values); the sign sketch of PROD
//     keys becomes +-1 operands by one shift and one logic op per pair (dims d and d + 16 of a 32-bit word pair up,
//     so that their bits land on the two fp16 sign positions together), against the S-projected query.
#include "tq_attention.cuh"

namespace {

using namespace tqatt;

// What the kernel needs of a quantizer, packed into 112 bytes so that the whole parameter block is a handful of
// 64-byte lines: parameters live in the constant bank, every line misses once per launch, and the misses of one
// warp are serial.  The warps therefore touch one line each before anything else happens.
struct AttnQuant {
  uint32_t s1[4], s2[4];   // rotation signs
  uint32_t j1[4], j2[4];   // QJL sign-WHT signs (PROD keys)
  uint16_t cent16[16];
  float alpha;
  uint32_t pad[3];
};
static_assert(sizeof(AttnQuant) == 112, "AttnQuant layout");

constexpr int G4_HEADS = 4;
constexpr int G4_HSTRIDE = TQ_D + 4;  // floats between heads in the warp-merge buffer: 16-byte stores stay conflict-free
constexpr int G4_PT = 128;            // tokens per page

// One 256-thread CTA per (KV head, split), two CTAs per SM.  (One 512-thread CTA running two such groups keeps the
// two in step inside a single launch and is 3 % faster there at 32K tokens; but in a chain of launches with
// programmatic dependent launch the half-SM CTAs of the next call take the place of finished ones one by one, so
// that one CTA's latency-bound prologue and tail run under the other's page loop: 11.4 against 13.2 us per call.)

constexpr int up128(int x) { return (x + 127) / 128 * 128; }


// Record layout of a (page, head) for 128-token pages, as tq_cache_layout_init lays it out, and the carve-up of
// the CTA's shared memory: the two pair tables, the query buffer(s), the mbarriers and flags, and the pipeline stages
// (reused as the warp-merge buffer after the page loop).
// KK / VK: 2,3,4 = turbo bits; 8 = q8_0; 18,19,20 = PROD with 1,2,3 PolarQuant bits + sign sketch (keys only).
template <int KK, int VK, int NW = ATT_WARPS> struct G4 {
  using KT = Kind<KK>;
  using VT = Kind<VK>;
  static constexpr int KB = KT::BITS, VB = VT::BITS;
  static constexpr int KIDXB = KT::Q8 ? TQ_D : 16 * KB, VIDXB = VT::Q8 ? TQ_D : 16 * VB;  // index bytes per token
  static constexpr int KSCB = KT::Q8 ? 8 : 4, VSCB = VT::Q8 ? 8 : 4;                      // scale bytes per token
  static constexpr int K_IDX = 0;
  static constexpr int K_SCALE = K_IDX + G4_PT * KIDXB;
  static constexpr int K_QJL = K_SCALE + G4_PT * KSCB;        // PROD keys: sign sketch, then residual scales
  static constexpr int K_RSCALE = K_QJL + G4_PT * 16;
  static constexpr int V_IDX = KT::PROD ? K_RSCALE + G4_PT * 4 : K_QJL;
  static constexpr int V_SCALE = V_IDX + G4_PT * VIDXB;
  static constexpr int REC = V_SCALE + G4_PT * VSCB;
  static constexpr int LK = PairLut<KB>::BYTES, LV = PairLut<VB>::BYTES;
  static constexpr int ALIGN = (LK > LV ? LK : LV) > 512 ? (LK > LV ? LK : LV) : 512;  // largest table
  static constexpr int OFF_K = LK >= LV ? 0 : LV;   // the larger table first: each stays aligned to its own size
  static constexpr int OFF_V = LK >= LV ? LK : 0;
  static constexpr int OFF_GROUPS = up128(LK + LV);
  static constexpr int G_Q = 0;                                   // float [4 heads][128] (PROD: + the projected queries)
  static constexpr int G_BAR = G_Q + (KT::PROD ? 2 : 1) * G4_HEADS * TQ_D * 4;   // 3 mbarriers, two flag words at + 64
  static constexpr int G_STAGE = G_BAR + 128;
  // page records in flight: 3 (4 and 5 measured: no faster); 2 for the four-warp CTAs, four of which share an SM
  static constexpr int NS = NW == 4 ? 2 : 3;
  static constexpr int MERGE = NW * G4_HEADS * (G4_HSTRIDE + 2) * 4;
  static constexpr int GROUP_BYTES = up128(G_STAGE + (NS * REC > MERGE ? NS * REC : MERGE));
  static constexpr int SMEM = ALIGN + OFF_GROUPS + GROUP_BYTES;
};

// ---- shared-memory loads through 32-bit addresses with immediate offsets ----------------------------------------
// Not volatile: the compiler may schedule and combine them.  What keeps a load of a pipeline stage behind the wait
// for that stage is a data dependency: the stage address is formed from a value the wait produces.
template <int OFF> __device__ __forceinline__ uint32_t lds_u32(uint32_t a) {
  uint32_t v;
  asm("ld.shared.u32 %0, [%1+%2];" : "=r"(v) : "r"(a), "n"(OFF));
  return v;
}
template <int OFF> __device__ __forceinline__ uint32_t lds_u16(uint32_t a) {
  uint16_t v;
  asm("ld.shared.u16 %0, [%1+%2];" : "=h"(v) : "r"(a), "n"(OFF));
  return v;
}
template <int OFF> __device__ __forceinline__ float lds_f32(uint32_t a) {
  float v;
  asm("ld.shared.f32 %0, [%1+%2];" : "=f"(v) : "r"(a), "n"(OFF));
  return v;
}
template <int OFF> __device__ __forceinline__ uint2 lds_u64(uint32_t a) {
  uint2 v;
  asm("ld.shared.v2.u32 {%0,%1}, [%2+%3];" : "=r"(v.x), "=r"(v.y) : "r"(a), "n"(OFF));
  return v;
}
template <int OFF> __device__ __forceinline__ uint4 lds_u128(uint32_t a) {
  uint4 v;
  asm("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4+%5];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a), "n"(OFF));
  return v;
}

// One row chunk of K indices (a thread's 32 dims of one token: 4 KB bytes at a 4 KB-byte-aligned address) as
// big-endian words: word k holds stream bits 32 k .. 32 k + 31, first bit in the most significant position.
template <int KB, int OFF> __device__ __forceinline__ void load_k_words(uint32_t a, uint32_t (&w)[KB]) {
  if constexpr (KB == 1) {
    w[0] = __byte_perm(lds_u32<OFF>(a), 0, 0x0123);
  } else if constexpr (KB == 2) {
    const uint2 v = lds_u64<OFF>(a);
    w[0] = __byte_perm(v.x, 0, 0x0123);
    w[1] = __byte_perm(v.y, 0, 0x0123);
  } else if constexpr (KB == 3) {
    w[0] = __byte_perm(lds_u32<OFF>(a), 0, 0x0123);
    w[1] = __byte_perm(lds_u32<OFF + 4>(a), 0, 0x0123);
    w[2] = __byte_perm(lds_u32<OFF + 8>(a), 0, 0x0123);
  } else {
    const uint4 v = lds_u128<OFF>(a);
    w[0] = __byte_perm(v.x, 0, 0x0123);
    w[1] = __byte_perm(v.y, 0, 0x0123);
    w[2] = __byte_perm(v.z, 0, 0x0123);
    w[3] = __byte_perm(v.w, 0, 0x0123);
  }
}

// A thread's 16 dims of one V token (2 VB bytes at byte offset 2 VB g of the token's row) as two big-endian words.
// Three-bit rows put that chunk on a 2-byte boundary: two aligned words that cover it are loaded from `a` (the
// chunk's address rounded down to 4 bytes) and the six bytes are picked out with selectors that depend on whether
// the chunk starts the word (even g) or sits in its upper half (odd g).
template <int VB, int OFF> __device__ __forceinline__ void load_v_words(uint32_t a, uint32_t sel0, uint32_t sel1, uint32_t (&w)[2]) {
  if constexpr (VB == 2) {
    w[0] = __byte_perm(lds_u32<OFF>(a), 0, 0x0123);
    w[1] = 0;
  } else if constexpr (VB == 3) {
    const uint32_t x0 = lds_u32<OFF>(a), x1 = lds_u32<OFF + 4>(a);
    w[0] = __byte_perm(x0, x1, sel0);
    w[1] = __byte_perm(x0, x1, sel1);
  } else {
    const uint2 v = lds_u64<OFF>(a);
    w[0] = __byte_perm(v.x, 0, 0x0123);
    w[1] = __byte_perm(v.y, 0, 0x0123);
  }
}

// Per-thread state of the page loop.
struct G4State {
  float o[4][4];
  float m0, m1, l0, l1;
};

// What a thread needs to find its part of a page record: byte offsets inside the record of the data of its warp's
// tile (tokens 16 warp .. + 15), and the lane roles of the two exchanges.
struct G4Thr {
  uint32_t k_thr;    // K indices (or int8 values) of row g: its 32 dims (q8_0: its 8 dims of block 0)
  uint32_t ks_thr;   // K scale of the token this thread keeps after the exchange (PROD, q8_0: of row g)
  uint32_t z_thr;    // PROD: sign-sketch word of row g; residual scales follow at rs_thr
  uint32_t rs_thr;
  uint32_t v_thr;    // V indices of token t, dims 16 g .. (rounded down to 4 bytes; q8_0: the 16 int8 values)
  uint32_t vs_thr;   // V scale of the kept token (q8_0: fp16 scale of token t, block g >> 1)
  uint32_t vsel0, vsel1;
  uint32_t psel;
  int src0, rsrc;
  bool upper;
  int t, tok_in_page, vtok_in_page;
};

__device__ __forceinline__ uint32_t s8x2_to_h2(uint32_t biased, uint32_t sel) {
  // two int8 values, stored as value ^ 0x80 = value + 128, as exact fp16: (b | 0x6400) is 1024 + b; subtract 1152
  return hsub2_u32(__byte_perm(biased, 0x64646464u, sel), 0x64806480u);
}

// Scores of one 16-token tile against the four heads (hi halves in columns 0-3, lo halves in 4-7), per thread the
// MMA accumulator fragment (rows g and g + 8, columns 2t and 2t + 1).  LUT keys return raw sums (the caller applies
// the K scale of the row it keeps); q8_0 and PROD keys return finished scores of both rows.
template <int KK, int VK, bool NODEQ, int TOK0>
__device__ __forceinline__ void g4_scores(float (&s)[4], uint32_t st, const G4Thr& T, const uint32_t (&qf)[8][2],
                                          const uint32_t (&qp)[Kind<KK>::PROD ? 8 : 1][2], uint32_t lk_base) {
  using C = G4<KK, VK>;
  using KT = Kind<KK>;
  constexpr int KB = KT::BITS;
  s[0] = s[1] = s[2] = s[3] = 0.f;
  if constexpr (KT::Q8) {
    // a 32-value block has one scale: k-steps 2b and 2b+1 cover block b (this thread supplies its dims 8t .. 8t+7 of
    // the block), and the block's partial scores are scaled in fp32 -- the operands carry no rounding
    const uint2 sc0 = lds_u64<TOK0 * C::KSCB>(st + T.ks_thr), sc1 = lds_u64<(TOK0 + 8) * C::KSCB>(st + T.ks_thr);
    const uint32_t scw0[2] = {sc0.x, sc0.y}, scw1[2] = {sc1.x, sc1.y};
#pragma unroll
    for (int blk = 0; blk < 4; ++blk) {
      uint2 u0, u1;
      constexpr int R0 = TOK0 * TQ_D, R1 = (TOK0 + 8) * TQ_D;   // rows g and g + 8 of this tile
      if (blk == 0) { u0 = lds_u64<R0>(st + T.k_thr); u1 = lds_u64<R1>(st + T.k_thr); }
      if (blk == 1) { u0 = lds_u64<R0 + 32>(st + T.k_thr); u1 = lds_u64<R1 + 32>(st + T.k_thr); }
      if (blk == 2) { u0 = lds_u64<R0 + 64>(st + T.k_thr); u1 = lds_u64<R1 + 64>(st + T.k_thr); }
      if (blk == 3) { u0 = lds_u64<R0 + 96>(st + T.k_thr); u1 = lds_u64<R1 + 96>(st + T.k_thr); }
      const uint32_t x0[2] = {u0.x ^ 0x80808080u, u0.y ^ 0x80808080u};
      const uint32_t x1[2] = {u1.x ^ 0x80808080u, u1.y ^ 0x80808080u};
      float sb[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int h2 = 0; h2 < 2; ++h2) {
        const int j = 2 * blk + h2;
        mma16816(sb, s8x2_to_h2(x0[h2], 0x4140), s8x2_to_h2(x1[h2], 0x4140), s8x2_to_h2(x0[h2], 0x4342),
                 s8x2_to_h2(x1[h2], 0x4342), qf[j][0], qf[j][1]);
      }
      const __half2 hs0 = *reinterpret_cast<const __half2*>(&scw0[blk >> 1]);
      const __half2 hs1 = *reinterpret_cast<const __half2*>(&scw1[blk >> 1]);
      const float f0 = (blk & 1) ? __high2float(hs0) : __low2float(hs0);
      const float f1 = (blk & 1) ? __high2float(hs1) : __low2float(hs1);
      s[0] = fmaf(sb[0], f0, s[0]); s[1] = fmaf(sb[1], f0, s[1]);
      s[2] = fmaf(sb[2], f1, s[2]); s[3] = fmaf(sb[3], f1, s[3]);
    }
  } else {
    uint32_t w0[KB], w1[KB];
    load_k_words<KB, TOK0 * C::KIDXB>(st + T.k_thr, w0);
    load_k_words<KB, (TOK0 + 8) * C::KIDXB>(st + T.k_thr, w1);
    constexpr int SH = PairLut<KB>::SHIFT;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      uint32_t a0, a1, a2, a3;
      if constexpr (NODEQ) {
        a0 = w0[j % KB]; a1 = w1[j % KB]; a2 = w0[(j + 1) % KB]; a3 = w1[(j + 1) % KB];
      } else {
        a0 = lds32(field_off<2 * KB, SH, KB>(w0, 2 * j) | lk_base);
        a1 = lds32(field_off<2 * KB, SH, KB>(w1, 2 * j) | lk_base);
        a2 = lds32(field_off<2 * KB, SH, KB>(w0, 2 * j + 1) | lk_base);
        a3 = lds32(field_off<2 * KB, SH, KB>(w1, 2 * j + 1) | lk_base);
      }
      mma16816(s, a0, a1, a2, a3, qf[j][0], qf[j][1]);
    }
    if constexpr (KT::PROD) {
      // + sqrt(pi/2)/sqrt(d) * ||r|| * <S q, z>: the sign sketch as +-1 operands.  Word t of a row holds its 32 dims
      // 32t .. 32t+31, first dim in the most significant bit; dims i and i + 16 form a pair, so that after a shift by
      // i their bits sit on the sign positions of the two fp16 halves (bit set = +1).
      const uint32_t z0 = __byte_perm(lds_u32<TOK0 * 16>(st + T.z_thr), 0, 0x0123);
      const uint32_t z1 = __byte_perm(lds_u32<(TOK0 + 8) * 16>(st + T.z_thr), 0, 0x0123);
      float s2[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const uint32_t a0 = (~(z0 << (2 * j)) & 0x80008000u) | 0x3C003C00u;
        const uint32_t a1 = (~(z1 << (2 * j)) & 0x80008000u) | 0x3C003C00u;
        const uint32_t a2 = (~(z0 << (2 * j + 1)) & 0x80008000u) | 0x3C003C00u;
        const uint32_t a3 = (~(z1 << (2 * j + 1)) & 0x80008000u) | 0x3C003C00u;
        mma16816(s2, a0, a1, a2, a3, qp[j][0], qp[j][1]);
      }
      const float k0 = lds_f32<TOK0 * 4>(st + T.ks_thr), k1 = lds_f32<TOK0 * 4 + 32>(st + T.ks_thr);
      const float r0 = lds_f32<TOK0 * 4>(st + T.rs_thr), r1 = lds_f32<TOK0 * 4 + 32>(st + T.rs_thr);
      s[0] = fmaf(s2[0], r0, s[0] * k0); s[1] = fmaf(s2[1], r0, s[1] * k0);
      s[2] = fmaf(s2[2], r1, s[2] * k1); s[3] = fmaf(s2[3], r1, s[3] * k1);
    }
  }
}

// One 16-token tile of one warp: scores against the four query heads, online softmax, O^T += V^T P^T.
//   st      shared-memory address of the page record
//   MASKED  the page may end inside or before this tile (`valid` tokens of the page exist)
//   NODEQ   measurement variant: the table lookups are left out and the packed words themselves are fed to the
//           tensor cores (copies, barriers, MMAs, softmax and merges as in the real kernel; results meaningless)
//   TOK0    first token of the tile relative to the warp's first tile of the page (a multiple of 16)
template <int KK, int VK, bool MASKED, bool SPARSE, bool NODEQ, int TOK0>
__device__ __forceinline__ void g4_tile(G4State& S, uint32_t st, const G4Thr& T, const uint32_t (&qf)[8][2],
                                        const uint32_t (&qp)[Kind<KK>::PROD ? 8 : 1][2], uint32_t lk_base, uint32_t lv_base,
                                        int valid) {
  using C = G4<KK, VK>;
  using KT = Kind<KK>;
  using VT = Kind<VK>;
  constexpr int VB = VT::BITS;
  constexpr bool K_LUT = !KT::Q8 && !KT::PROD;   // raw sums, one scale per row
  constexpr float MAX_SLACK = 4.0f;
  const int t = T.t;
  // ---------------- S = K_tile (16 tokens x 128) . [q_hi | q_lo] ----------------
  float ks = 1.0f;
  if constexpr (K_LUT) ks = lds_f32<TOK0 * 4>(st + T.ks_thr);
  float s[4];
  g4_scores<KK, VK, NODEQ, TOK0>(s, st, T, qf, qp, lk_base);
  // the V words and scale of this tile are fetched here, ahead of the softmax arithmetic that separates them from
  // their use: the loads then wait under it instead of in front of the table lookups
  uint32_t vw[4][VT::Q8 ? 4 : 2];
  uint32_t vsc16[4];   // q8_0 values: fp16 block scale of the thread's four tokens, both halves alike
  float vs_raw = 1.0f;
  if constexpr (VT::Q8) {
#pragma unroll
    for (int q4 = 0; q4 < 4; ++q4) {
      uint4 v;
      uint32_t sc;
      if (q4 == 0) { v = lds_u128<TOK0 * TQ_D>(st + T.v_thr); sc = lds_u16<TOK0 * C::VSCB>(st + T.vs_thr); }
      if (q4 == 1) { v = lds_u128<(TOK0 + 4) * TQ_D>(st + T.v_thr); sc = lds_u16<(TOK0 + 4) * C::VSCB>(st + T.vs_thr); }
      if (q4 == 2) { v = lds_u128<(TOK0 + 8) * TQ_D>(st + T.v_thr); sc = lds_u16<(TOK0 + 8) * C::VSCB>(st + T.vs_thr); }
      if (q4 == 3) { v = lds_u128<(TOK0 + 12) * TQ_D>(st + T.v_thr); sc = lds_u16<(TOK0 + 12) * C::VSCB>(st + T.vs_thr); }
      vw[q4][0] = v.x ^ 0x80808080u; vw[q4][1] = v.y ^ 0x80808080u;
      vw[q4][2] = v.z ^ 0x80808080u; vw[q4][3] = v.w ^ 0x80808080u;
      if constexpr (MASKED) sc = (T.vtok_in_page + TOK0 + 4 * q4 < valid) ? sc : 0u;   // a stale scale must not meet p = 0
      vsc16[q4] = __byte_perm(sc, 0, 0x1010);
    }
  } else {
    load_v_words<VB, TOK0 * C::VIDXB>(st + T.v_thr, T.vsel0, T.vsel1, vw[0]);
    load_v_words<VB, (TOK0 + 4) * C::VIDXB>(st + T.v_thr, T.vsel0, T.vsel1, vw[1]);
    load_v_words<VB, (TOK0 + 8) * C::VIDXB>(st + T.v_thr, T.vsel0, T.vsel1, vw[2]);
    load_v_words<VB, (TOK0 + 12) * C::VIDXB>(st + T.v_thr, T.vsel0, T.vsel1, vw[3]);
    vs_raw = lds_f32<TOK0 * 4>(st + T.vs_thr);
  }
  constexpr int SHV = PairLut<VB>::SHIFT;
  auto v_half = [&](uint32_t (&h)[2][8], int u) {
#pragma unroll
    for (int q2 = 0; q2 < 2; ++q2) {
#pragma unroll
      for (int jj = 0; jj < 8; ++jj) {
        if constexpr (VT::Q8) {
          h[q2][jj] = hmul2_u32(s8x2_to_h2(vw[2 * u + q2][jj >> 1], (jj & 1) ? 0x4342 : 0x4140), vsc16[2 * u + q2]);
        } else if constexpr (NODEQ) {
          h[q2][jj] = vw[2 * u + q2][jj & 1] ^ (uint32_t)jj;
        } else {
          h[q2][jj] = lds32(field_off<2 * VB, SHV, 2>(vw[2 * u + q2], jj) | lv_base);
        }
      }
    }
  };
  // hi + lo: the partner lane (t ^ 2) holds the other half of the same heads
  const bool upper = T.upper;
  const float give0 = upper ? s[0] : s[2], give1 = upper ? s[1] : s[3];
  const float keep0 = upper ? s[2] : s[0], keep1 = upper ? s[3] : s[1];
  const float sum0 = keep0 + __shfl_xor_sync(0xffffffffu, give0, 2);
  const float sum1 = keep1 + __shfl_xor_sync(0xffffffffu, give1, 2);
  // ---------------- online softmax (log2 domain), heads 2(t&1) and 2(t&1)+1 ----------------
  // The running maxima move only when a score exceeds them by more than 2^MAX_SLACK, so that almost every tile skips
  // the warp reduction and the rescaling of O.  What is tracked is the maximum of score + log2(V scale), not of the
  // score alone: the P operand of the second product is p * (V scale) in fp16, and with this reference it never
  // exceeds 2^MAX_SLACK whatever the norms of the values are (a reference that is too high only scales p, the
  // softmax sums and O by the same factor, which the final division removes).
  bool ok = true;
  float vs = vs_raw;
  float d0 = fmaf(sum0, ks, -S.m0), d1 = fmaf(sum1, ks, -S.m1);   // score - running reference
  if constexpr (MASKED) {
    ok = T.tok_in_page + TOK0 < valid;
    vs = ok ? vs_raw : 0.f;                                       // a stale scale must not meet p = 0
    d0 = ok ? d0 : -INFINITY;
    d1 = ok ? d1 : -INFINITY;
  }
  const float lvs = VT::Q8 ? 0.f : fmaxf(fast_log2(vs), -100.0f);  // zero vectors have scale 0
  if (__any_sync(0xffffffffu, (d0 + lvs > MAX_SLACK) || (d1 + lvs > MAX_SLACK))) {
    float sc0 = sum0 * ks, sc1 = sum1 * ks;
    if constexpr (MASKED) {
      sc0 = ok ? sc0 : -INFINITY;
      sc1 = ok ? sc1 : -INFINITY;
    }
    float mx0 = sc0 + lvs, mx1 = sc1 + lvs;
#pragma unroll
    for (int sh = 2; sh < 32; sh <<= 1) {
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, sh));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, sh));
    }
    const float mn0 = fmaxf(S.m0, mx0), mn1 = fmaxf(S.m1, mx1);  // finite: the tile's first token exists
    const float r0 = fast_exp2(S.m0 - mn0), r1 = fast_exp2(S.m1 - mn1);
    S.m0 = mn0;
    S.m1 = mn1;
    S.l0 *= r0;
    S.l1 *= r1;
    d0 = sc0 - mn0;
    d1 = sc1 - mn1;
    const float ra = __shfl_sync(0xffffffffu, r0, T.rsrc), rb = __shfl_sync(0xffffffffu, r1, T.rsrc);
    const float r = (t & 1) ? rb : ra;                        // O of this thread belongs to head t
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      S.o[j][0] *= r; S.o[j][1] *= r; S.o[j][2] *= r; S.o[j][3] *= r;
    }
  }
  const float p0 = fast_exp2(d0), p1 = fast_exp2(d1);
  S.l0 += p0;
  S.l1 += p1;
  // a template parameter, not a run-time flag: the possible jump keeps the V loads below it from being issued early
  // (the threshold is applied to p * V scale, the token's weight in the output relative to the largest one)
  if (SPARSE && !__any_sync(0xffffffffu, fmaxf(p0, p1) * vs >= SPARSE_V_TAU)) return;
  const uint32_t hp = pack_h2(p0 * vs, p1 * vs);
  uint32_t pb[4];
#pragma unroll
  for (int q4 = 0; q4 < 4; ++q4)
    pb[q4] = __byte_perm(__shfl_sync(0xffffffffu, hp, T.src0 + 16 * (q4 & 1) + 2 * (q4 >> 1)), 0, T.psel);
  // ---------------- O^T += V_tile^T . P^T : tokens t, t+4, t+8, t+12 of the tile, dims 16g .. 16g+15 ----------------
  // (neighbouring lanes read neighbouring token rows: rows are 16 VB bytes apart, which spreads a quad of lanes over
  // the shared-memory banks; a stride of four rows put lanes t and t+2 on the same banks)
  // two halves of eight tokens: the table words of one half (16 registers) are live at a time, which leaves the
  // compiler room to keep more loads in flight (all four token rows at once: 5 % slower at 256K tokens; forming
  // the first half ahead of the softmax arithmetic: no gain)
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    uint32_t h[2][8];
    v_half(h, u);
#pragma unroll
    for (int blk = 0; blk < 4; ++blk)
      mma16816(S.o[blk], h[0][2 * blk], h[0][2 * blk + 1], h[1][2 * blk], h[1][2 * blk + 1], pb[2 * u], pb[2 * u + 1]);
  }
}

// the warp's tiles of one page: tile TT covers tokens 16 (warp + NW TT) .. + 15
template <int KK, int VK, bool SPARSE, bool NODEQ, int NW, int TT>
__device__ __forceinline__ void g4_page(G4State& S, uint32_t st, const G4Thr& T, const uint32_t (&qf)[8][2],
                                        const uint32_t (&qp)[Kind<KK>::PROD ? 8 : 1][2], uint32_t lk_base, uint32_t lv_base,
                                        bool full, int last_valid, int warp) {
  constexpr int TOK0 = 16 * NW * TT;
  if (full) g4_tile<KK, VK, false, SPARSE, NODEQ, TOK0>(S, st, T, qf, qp, lk_base, lv_base, G4_PT);
  else if (16 * warp + TOK0 < last_valid) g4_tile<KK, VK, true, SPARSE, NODEQ, TOK0>(S, st, T, qf, qp, lk_base, lv_base, last_valid);
  if constexpr (TT + 1 < ATT_WARPS / NW) g4_page<KK, VK, SPARSE, NODEQ, NW, TT + 1>(S, st, T, qf, qp, lk_base, lv_base, full, last_valid, warp);
}

// NW warps per CTA: 8 (two CTAs per SM), or 4 (four per SM, two tiles per warp and page) for chains of calls that may
// overlap completely: the CTAs of two consecutive calls then share an SM four at a time, each in a phase of its own,
// and the SM's warps are in a page loop 80 % of the time instead of 67 %.
// TAIL: the call follows the append of the step's token (TQ_DECODE_OVERLAP_APPEND).  A template parameter, so that the
// page loop of every other instantiation carries nothing for it.
template <int KK, int VK, bool SPARSE, bool NODEQ, int NW, bool TAIL = false>
__global__ void __launch_bounds__(32 * NW, 16 / NW) k_decode_attn_g4(const __grid_constant__ AttnParams P, const __grid_constant__ AttnQuant fk,
                                                                      const __grid_constant__ AttnQuant fv) {
  using C = G4<KK, VK, NW>;
  constexpr int NT = 32 * NW;          // threads
  constexpr int G4_NS = C::NS;
  using KT = Kind<KK>;
  using VT = Kind<VK>;
  constexpr int KB = KT::BITS, VB = VT::BITS;
  extern __shared__ __align__(128) uint8_t smem_raw[];
  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
  constexpr int bar_id = 0;
  {  // one parameter line per warp, all misses in flight together
    const uint32_t* pp = reinterpret_cast<const uint32_t*>(&P);
    uint32_t touch;
    if (warp < 4) touch = pp[min(16 * warp, (int)(sizeof(AttnParams) / 4) - 1)];
    else if (warp < 6) touch = warp == 4 ? fk.s1[0] : fk.pad[2];   // first and last word of the 112-byte blocks
    else touch = warp == 6 ? fv.s1[0] : fv.pad[2];
    asm volatile("" ::"r"(touch));
  }
  // Programmatic dependent launch: let the next kernel in the stream start as soon as SMs free up.  Everything
  // this kernel does before its griddepcontrol.wait reads only the cache, the block table and the sequence
  // lengths -- and, when the caller says that the preceding kernel does not write the queries either (q_early),
  // the queries.  What comes after the wait runs after the preceding kernel has completed and its writes are
  // visible: the workspace and the output are only ever touched there.  Without q_early the wait stands in front of
  // the query load; with it, in front of the first write (after the page loop).  Both instructions do nothing in a
  // launch without the attribute.
  if (P.overlap) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int page_lo = split * P.chunk_pages;
  const size_t row0 = (size_t)b * P.hq + (size_t)kvh * P.group;
  const int32_t* bt = P.block_table + (size_t)b * P.max_pages;
  const uint32_t raw = smem_u32(smem_raw);
  uint8_t* sm = smem_raw + (((raw + C::ALIGN - 1) & ~(uint32_t)(C::ALIGN - 1)) - raw);
  uint8_t* smg = sm + C::OFF_GROUPS;
  float* qbuf = reinterpret_cast<float*>(smg + C::G_Q);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smg + C::G_BAR);
  volatile int* s_flags = reinterpret_cast<volatile int*>(smg + C::G_BAR + 64);
  uint8_t* stage0 = smg + C::G_STAGE;
  constexpr int PRODUCER = NT - 32;  // lane 0 of the last warp issues every bulk copy
  // kvh names a group of query heads; kv_div of them share a KV head of the cache
  const uint8_t* pool_head = P.pool + (int64_t)(P.kv_div == 1 ? kvh : kvh / P.kv_div) * P.L.head_stride;

  auto issue = [&](int stage, int64_t page) {
    uint64_t* bar = &bars[stage];
    mbar_expect_tx(bar, C::REC);
    bulk_g2s(stage0 + stage * C::REC, pool_head + page * P.L.page_stride, C::REC, bar);
  };

  // The warps take different roles so that their global-load latencies (and their instruction fetches, which are
  // cold in every launch) overlap: the producer sends the first pages on their way as early as it can, the first
  // `group` warps rotate one query head each, the others fill the pair tables.
  // A length beyond the block-table row (or a negative one) is clamped: page numbers are only ever read from the
  // row's max_pages entries and the split count stays inside the plan the workspace was sized for.
  const int seq_len = min(max(P.seq_lens[b], 0), P.max_pages * G4_PT);
  const int n_pages = (seq_len + G4_PT - 1) / G4_PT;
  const int np = min(n_pages, page_lo + P.chunk_pages) - page_lo;   // pages of this CTA (<= 0: none)
  int pg_ahead = 0;  // producer: block-table entry of the page issued in the next iteration
  float x[4] = {0.f, 0.f, 0.f, 0.f}, y[4] = {0.f, 0.f, 0.f, 0.f};
  if (tid == PRODUCER) {   // (with four warps and four heads this warp rotates a query as well, afterwards)
    int pg_next[G4_NS];
#pragma unroll
    for (int i = 0; i < G4_NS; ++i) pg_next[i] = bt[min(page_lo + i, P.max_pages - 1)];
#pragma unroll
    for (int s = 0; s < G4_NS; ++s) mbar_init(&bars[s], 1);
    s_flags[0] = 0;
    s_flags[1] = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
#pragma unroll
    for (int s = 0; s < G4_NS - 1; ++s)
      if (np > s) {
        // after an append the last page of the sequence is what the preceding kernel writes: it is fetched once that
        // kernel has completed (the wait costs nothing when it already has), every other page right away
        if (TAIL && page_lo + s == n_pages - 1) asm volatile("griddepcontrol.wait;" ::: "memory");
        issue(s, pg_next[s]);
      }
    pg_ahead = pg_next[G4_NS - 1];
  }
  if (warp < P.group && (tid != PRODUCER || NW == 4)) {
    if (P.overlap && !P.q_early) asm volatile("griddepcontrol.wait;" ::: "memory");
    if (P.k_pre) {   // dense rotations: rotated (and, for PROD keys, projected) queries come from k_prepare_queries
      load_q4(P.qrot, TQ_F32, (row0 + warp) * TQ_D + 4 * lane, x);
      if constexpr (KT::PROD) load_q4(P.qproj, TQ_F32, (row0 + warp) * TQ_D + 4 * lane, y);
    } else {
      load_q4(P.q, P.q_dtype, (row0 + warp) * TQ_D + 4 * lane, x);
      if constexpr (KT::PROD) {
#pragma unroll
        for (int k = 0; k < 4; ++k) y[k] = x[k];
        warp_wht128(y, fk.j1, fk.j2, lane);
      }
      if (!KT::Q8) warp_wht128(x, fk.s1, fk.s2, lane);   // q8_0 tensors are stored unrotated
      const float sk = P.qscale / fk.alpha;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        x[k] *= sk;
        y[k] *= P.qscale;
      }
    }
    // 16-byte chunk c = 8 t + j of head h sits at 8 t + (j ^ (t + 4 (h & 1))): the fragment reads below (fixed j,
    // all t and h) then touch every bank group instead of one
    const int tq = lane >> 3, jq = lane & 7;
    *reinterpret_cast<float4*>(qbuf + warp * TQ_D + 4 * (8 * tq + (jq ^ (tq + 4 * (warp & 1))))) =
        make_float4(x[0], x[1], x[2], x[3]);
    if constexpr (KT::PROD)   // projected queries: plain rows behind the rotated ones
      *reinterpret_cast<float4*>(qbuf + (G4_HEADS + warp) * TQ_D + 4 * lane) = make_float4(y[0], y[1], y[2], y[3]);
  }
  __syncwarp();
  if (NW == 4) {   // every warp may have rotated a query: all of them fill the tables afterwards
    if constexpr (KB > 0) lut_fill<KB>(sm + C::OFF_K, fk.cent16, tid, NT);
    if constexpr (VB > 0) lut_fill<VB>(sm + C::OFF_V, fv.cent16, tid, NT);
  } else if (warp >= P.group) {
    const int fh = NT - 32 * P.group;   // table-filling threads
    if constexpr (KB > 0) lut_fill<KB>(sm + C::OFF_K, fk.cent16, tid - 32 * P.group, fh);
    if constexpr (VB > 0) lut_fill<VB>(sm + C::OFF_V, fv.cent16, tid - 32 * P.group, fh);
  }
  if (P.overlap && !P.q_early) asm volatile("griddepcontrol.wait;" ::: "memory");   // the query warps already have
  if (n_pages == 0 && split == 0) {  // empty sequence: zeros (split 0 exists for every kv head)
    if (P.overlap && P.q_early) asm volatile("griddepcontrol.wait;" ::: "memory");
    for (int e = tid; e < P.group * TQ_D; e += NT) store_out(P.out, P.out_dtype, row0 * TQ_D + e, 0.f);
    if (P.lse && tid < P.group) P.lse[row0 + tid] = -INFINITY;
  }
  const int ns = (n_pages + P.chunk_pages - 1) / P.chunk_pages;
  __syncthreads();               // tables, query buffer and mbarriers are ready
  if (np <= 0) return;           // this CTA has no pages (its split lies beyond the sequence)

  // B operand of S = K q^T: column g is head g & 3, hi half for g < 4, lo half otherwise
  uint32_t qf[8][2], qp[KT::PROD ? 8 : 1][2];
  {
    const int head = g & 3;
    const bool hv = head < P.group, lo = g >= 4;
    const float* qh = qbuf + (hv ? head : 0) * TQ_D;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      // dims this thread supplies in k-step j: 32t + 4j .. +3 (packed formats), or, for q8_0 keys, its 8 dims of
      // block j/2: 32(j/2) + 8t + 4(j%2) .. +3; as the 16-byte chunk (row, col) of the staged query
      const int crow = KT::Q8 ? (j >> 1) : t, ccol = KT::Q8 ? 2 * t + (j & 1) : j;
      float4 v = hv ? *reinterpret_cast<const float4*>(qh + 4 * (8 * crow + (ccol ^ (crow + 4 * (head & 1)))))
                    : make_float4(0.f, 0.f, 0.f, 0.f);
      const __half2 h0 = __floats2half2_rn(v.x, v.y), h1 = __floats2half2_rn(v.z, v.w);
      const float2 f0 = __half22float2(h0), f1 = __half22float2(h1);
      qf[j][0] = lo ? pack_h2(v.x - f0.x, v.y - f0.y) : *reinterpret_cast<const uint32_t*>(&h0);
      qf[j][1] = lo ? pack_h2(v.z - f1.x, v.w - f1.y) : *reinterpret_cast<const uint32_t*>(&h1);
      if constexpr (KT::PROD) {
        // sign-sketch operands pair dims i and i + 16 of the thread's 32 (i = 2j for the first register of the
        // k-step, 2j + 1 for the second), dim i + 16 in the low half
        const float* ph = qh + G4_HEADS * TQ_D + 32 * t;
        const float a0 = hv ? ph[16 + 2 * j] : 0.f, a1 = hv ? ph[2 * j] : 0.f;
        const float b0 = hv ? ph[16 + 2 * j + 1] : 0.f, b1 = hv ? ph[2 * j + 1] : 0.f;
        const __half2 e0 = __floats2half2_rn(a0, a1), e1 = __floats2half2_rn(b0, b1);
        const float2 r0 = __half22float2(e0), r1 = __half22float2(e1);
        qp[j][0] = lo ? pack_h2(a0 - r0.x, a1 - r0.y) : *reinterpret_cast<const uint32_t*>(&e0);
        qp[j][1] = lo ? pack_h2(b0 - r1.x, b1 - r1.y) : *reinterpret_cast<const uint32_t*>(&e1);
      }
    }
    if constexpr (!KT::PROD) qp[0][0] = qp[0][1] = 0u;
  }
  const uint32_t lk_base = smem_u32(sm + C::OFF_K) + (PairLut<KB>::REPL ? lane * 4 : 0);
  const uint32_t lv_base = smem_u32(sm + C::OFF_V) + (PairLut<VB>::REPL ? lane * 4 : 0);
  // P operand: this thread's column is (head g >> 1, parity g & 1); the owner of p[token][head] is lane
  // 4 (token & 7) + 2 (token >> 3) + (head >> 1), half (head & 1) of its packed pair
  const int src0 = 4 * t + (g >> 2);                                  // token t; token 4 i + t: + 16 (i & 1) + 2 (i >> 1)
  const uint32_t psel = ((g >> 1) & 1) ? ((g & 1) ? 0x3244u : 0x4432u) : ((g & 1) ? 0x1044u : 0x4410u);
  const int rsrc = (lane & ~3) | (t >> 1);                             // a lane that tracks head t's running maximum
  const bool upper = t >= 2;                                           // keeps token g + 8 after the exchange

  G4State S;
#pragma unroll
  for (int j = 0; j < 4; ++j) S.o[j][0] = S.o[j][1] = S.o[j][2] = S.o[j][3] = 0.f;
  S.m0 = S.m1 = -INFINITY;
  S.l0 = S.l1 = 0.f;

  // byte offsets inside a page record of what this thread reads in its warp's tile (tokens 16 warp .. + 15)
  G4Thr T;
  T.t = t;
  T.upper = upper;
  T.src0 = src0;
  T.rsrc = rsrc;
  T.psel = psel;
  T.tok_in_page = 16 * warp + g + (upper ? 8 : 0);
  T.vtok_in_page = 16 * warp + t;
  T.k_thr = C::K_IDX + (16 * warp + g) * C::KIDXB + (KT::Q8 ? 8 * t : t * (C::KIDXB / 4));
  // the row this thread keeps (packed keys: the scale is applied after the exchange), or row g (q8_0 and PROD keys
  // finish the scores of both rows before the exchange)
  T.ks_thr = C::K_SCALE + C::KSCB * ((KT::Q8 || KT::PROD) ? 16 * warp + g : T.tok_in_page);
  T.z_thr = C::K_QJL + (16 * warp + g) * 16 + 4 * t;
  T.rs_thr = C::K_RSCALE + 4 * (16 * warp + g);
  const uint32_t v_chunk = C::V_IDX + (16 * warp + t) * C::VIDXB + g * (VT::Q8 ? 16 : 2 * VB);
  T.v_thr = v_chunk & ~3u;
  T.vs_thr = VT::Q8 ? C::V_SCALE + (16 * warp + t) * C::VSCB + 2 * (g >> 1) : C::V_SCALE + 4 * T.tok_in_page;
  const bool v_odd = (v_chunk & 2u) != 0;
  T.vsel0 = v_odd ? 0x2345u : 0x0123u;
  T.vsel1 = v_odd ? 0x6744u : 0x4544u;
  const uint32_t stage_addr = smem_u32(stage0);
  // pages 0 .. np-2 of the CTA are full; the last one is full unless the sequence ends inside it
  const int last_valid = seq_len - (page_lo + np - 1) * G4_PT;          // >= 1
  const int n_full = last_valid >= G4_PT ? np : np - 1;

  int stage = 0;
  uint32_t parity = 0;
  for (int i = 0; i < np; ++i) {
    if (tid == PRODUCER && i + G4_NS - 1 < np) {
      if (TAIL && page_lo + i + G4_NS - 1 == n_pages - 1) asm volatile("griddepcontrol.wait;" ::: "memory");
      issue(stage == 0 ? G4_NS - 1 : stage - 1, pg_ahead);            // the stage the page before this one has left
      pg_ahead = bt[min(page_lo + i + G4_NS, P.max_pages - 1)];
    }
    // (the page the preceding kernel writes is only fetched once that kernel has completed: the bounded wait for it
    // starts then, however long that kernel runs)
    if (TAIL && page_lo + i == n_pages - 1) asm volatile("griddepcontrol.wait;" ::: "memory");
    if (!s_flags[0] && !mbar_wait_bounded(&bars[stage], parity)) s_flags[0] = 1;
    // the stage address carries a value the wait above produced (always zero), so that no load of the stage can
    // be scheduled ahead of the wait
    uint32_t dep;
    asm volatile("mov.u32 %0, 0;" : "=r"(dep)::"memory");
    const uint32_t st = stage_addr + stage * C::REC + dep;
    g4_page<KK, VK, SPARSE, NODEQ, NW, 0>(S, st, T, qf, qp, lk_base, lv_base, i < n_full, last_valid, warp);
    group_sync<NT>(bar_id);  // every warp is done with this stage before it is refilled
    if (++stage == G4_NS) {
      stage = 0;
      parity ^= 1u;
    }
  }
  // from here on the workspace and the output are written
  if (P.overlap && P.q_early) asm volatile("griddepcontrol.wait;" ::: "memory");
  // ---------------- merge the eight warps, write the split partial ----------------
#pragma unroll
  for (int sh = 2; sh < 32; sh <<= 1) {
    S.l0 += __shfl_xor_sync(0xffffffffu, S.l0, sh);
    S.l1 += __shfl_xor_sync(0xffffffffu, S.l1, sh);
  }
  float* so = reinterpret_cast<float*>(stage0);                    // [warp][head 4][G4_HSTRIDE]
  float* sml = so + NW * G4_HEADS * G4_HSTRIDE;                    // [warp][head 4][2]
#pragma unroll
  for (int blk = 0; blk < 4; ++blk)
    *reinterpret_cast<float4*>(so + (size_t)(warp * G4_HEADS + t) * G4_HSTRIDE + 16 * g + 4 * blk) =
        make_float4(S.o[blk][0], S.o[blk][1], S.o[blk][2], S.o[blk][3]);
  if (g == 0 && t < 2) {
    *reinterpret_cast<float4*>(sml + (warp * G4_HEADS + 2 * t) * 2) = make_float4(S.m0, S.l0, S.m1, S.l1);
  }
  group_sync<NT>(bar_id);
  {
    // thread (head, DPT consecutive dims): 4 heads x 128 dims over the CTA's threads; the warps' rows are added in
    // warp order
    constexpr int DPT = G4_HEADS * TQ_D / NT;     // 2 or 4
    const int head = tid / (TQ_D / DPT), dim = DPT * (tid % (TQ_D / DPT));
    if (head < P.group) {
      float mw[NW], M = -INFINITY;
#pragma unroll
      for (int w = 0; w < NW; ++w) {
        mw[w] = sml[(w * G4_HEADS + head) * 2];
        M = fmaxf(M, mw[w]);
      }
      float a[DPT], Lsum = 0.f;
#pragma unroll
      for (int k = 0; k < DPT; ++k) a[k] = 0.f;
#pragma unroll
      for (int w = 0; w < NW; ++w) {
        const float f = mw[w] == -INFINITY ? 0.f : fast_exp2(mw[w] - M);
        const float* v = so + (size_t)(w * G4_HEADS + head) * G4_HSTRIDE + dim;
#pragma unroll
        for (int k = 0; k < DPT; ++k) a[k] = fmaf(v[k], f, a[k]);
        Lsum = fmaf(sml[(w * G4_HEADS + head) * 2 + 1], f, Lsum);
      }
      const size_t slot = (row0 + head) * P.num_splits + split;
#pragma unroll
      for (int k = 0; k < DPT; k += 2)
        *reinterpret_cast<float2*>(P.part_o + slot * TQ_D + dim + k) = make_float2(a[k], a[k + 1]);
      if (dim == 0) *reinterpret_cast<float2*>(P.part_ml + slot * 2) = make_float2(M, Lsum);
    }
  }
  finish_splits<VT::Q8, NT>(P, fv.s1, fv.s2, fv.alpha, qbuf, stage0, s_flags, row0, ns, b, kvh, tid, bar_id);
}

template <int KK, int VK, bool SPARSE, bool NODEQ, int NW = ATT_WARPS, bool TAIL = false>
int launch_attn_g4(const AttnParams& P, const TqFast& fk, const TqFast& fv, cudaStream_t st) {
  using C = G4<KK, VK, NW>;
  static_assert((16 / NW) * (C::SMEM + 1024) <= 228 * 1024, "CTAs of the specialised decode kernel per SM");
  static thread_local int configured_dev = -1;  // per instantiation
  int dev = 0;
  TQ_CUDA(cudaGetDevice(&dev));
  if (configured_dev != dev) {
    TQ_CUDA(cudaFuncSetAttribute(k_decode_attn_g4<KK, VK, SPARSE, NODEQ, NW, TAIL>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM));
    configured_dev = dev;
  }
  AttnQuant ak, av;
  memset(&ak, 0, sizeof(ak));
  memset(&av, 0, sizeof(av));
  memcpy(ak.s1, fk.s1, 16); memcpy(ak.s2, fk.s2, 16); memcpy(ak.j1, fk.j1, 16); memcpy(ak.j2, fk.j2, 16);
  memcpy(ak.cent16, fk.cent16, 32); ak.alpha = fk.lut_alpha;
  memcpy(av.s1, fv.s1, 16); memcpy(av.s2, fv.s2, 16); memcpy(av.cent16, fv.cent16, 32); av.alpha = fv.lut_alpha;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(P.num_splits, P.hkv, P.batch);
  cfg.blockDim = dim3(32 * NW);
  cfg.dynamicSmemBytes = C::SMEM;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = P.overlap ? 1 : 0;
  TQ_CUDA(cudaLaunchKernelEx(&cfg, k_decode_attn_g4<KK, VK, SPARSE, NODEQ, NW, TAIL>, P, ak, av));
  return tq_launch_check("k_decode_attn_g4");
}

template <int KK, int VK>
bool layout_matches(const tq_cache_layout& L) {
  using C = G4<KK, VK>;
  if (Kind<KK>::PROD && (L.k_qjl_off != C::K_QJL || L.k_rscale_off != C::K_RSCALE)) return false;
  return L.page_tokens == G4_PT && L.k_idx_off == C::K_IDX && L.k_scale_off == C::K_SCALE && L.v_idx_off == C::V_IDX &&
         L.v_scale_off == C::V_SCALE && L.record_bytes == C::REC && L.k_idx_bytes == C::KIDXB && L.v_idx_bytes == C::VIDXB;
}

}  // namespace

bool tq_decode_g4_try(const tqatt::AttnParams& P_in, const TqFast& fk, const TqFast& fv, cudaStream_t st, int* rc) {
  const int kf = P_in.L.k_format, vf = P_in.L.v_format;
  tqatt::AttnParams P = P_in;
  if (P.group > G4_HEADS) {
    // 5..16 query heads per KV head: the group is dealt to 2..4 CTAs of up to four heads each, which run side by side
    // over the same pages (one of them brings a page in from HBM, the others find it in L2).  Query heads of a KV
    // head are neighbours, so a CTA's first row is still (grid.y index) * (heads per CTA); only the cache head differs.
    // This pays in a chain of calls (8 heads, 32K tokens: 16.7 us per call against 25.6 for the general kernel, which
    // has no early-start form); a call on its own is served better by the general kernel (25.6 against 28.2 us), whose
    // CTAs dequantize a page once for all eight heads.
    if (!((P.q_early || P.chain_head) && !P.tail_late)) return false;
    const int parts = (P.group + G4_HEADS - 1) / G4_HEADS;
    if (P.group > 4 * G4_HEADS || P.group % parts != 0 || (int64_t)P.hkv * parts > 65535 ||
        (int64_t)P.batch * P.hkv * parts > MAX_TICKETS)
      return false;
    P.group /= parts;
    P.hkv *= parts;
    P.kv_div = parts;
  }
  // The four-warp form pays in a chain of attention calls, where the CTAs of consecutive calls share an SM in
  // different phases: calls launched with TQ_DECODE_OVERLAP_Q, and the call in front of them when the caller says so
  // (TQ_DECODE_CHAIN_HEAD).  A call that follows an append overlaps only its start with that short kernel: it takes
  // the eight-warp form, which is the faster one for a call on its own.
  const bool chain = (P.q_early || P.chain_head) && !P.tail_late;
  // PolarQuant K and V: every pair of widths, with the sparse-V and the measurement variants
#define TQ_ATT_G4(K, V)                                                                                              \
  if (kf == K && vf == V) {                                                                                          \
    if (!layout_matches<K, V>(P.L)) return false;                                                                    \
    if (P.nodeq && K == 3 && V == 3) *rc = launch_attn_g4<3, 3, false, true>(P, fk, fv, st);                         \
    else if (P.sparse_v && chain) *rc = launch_attn_g4<K, V, true, false, 4>(P, fk, fv, st);                         \
    else if (P.sparse_v) *rc = launch_attn_g4<K, V, true, false>(P, fk, fv, st);                                     \
    else if (P.tail_late) *rc = launch_attn_g4<K, V, false, false, ATT_WARPS, true>(P, fk, fv, st);                  \
    else if (chain) *rc = launch_attn_g4<K, V, false, false, 4>(P, fk, fv, st);                                      \
    else *rc = launch_attn_g4<K, V, false, false>(P, fk, fv, st);                                                    \
    return true;                                                                                                     \
  }
  TQ_ATT_G4(2, 2) TQ_ATT_G4(2, 3) TQ_ATT_G4(2, 4) TQ_ATT_G4(3, 2) TQ_ATT_G4(3, 3) TQ_ATT_G4(3, 4) TQ_ATT_G4(4, 2)
  TQ_ATT_G4(4, 3) TQ_ATT_G4(4, 4)
#undef TQ_ATT_G4
  // q8_0 and PROD keys (the sparse-V option of these pairs runs the general kernel)
  if (P.sparse_v) return false;
#define TQ_ATT_G4X(K, V)                                                                                   \
  if (kf == K && vf == V) {                                                                                \
    if (!layout_matches<K, V>(P.L)) return false;                                                          \
    /* the four-warp form where four CTAs with two page records each fit an SM */                         \
    if constexpr (4 * (G4<K, V, 4>::SMEM + 1024) <= 228 * 1024) {                                          \
      if (chain) {                                                                                         \
        *rc = launch_attn_g4<K, V, false, false, 4>(P, fk, fv, st);                                        \
        return true;                                                                                       \
      }                                                                                                    \
    }                                                                                                      \
    if (P.tail_late) *rc = launch_attn_g4<K, V, false, false, ATT_WARPS, true>(P, fk, fv, st);             \
    else *rc = launch_attn_g4<K, V, false, false>(P, fk, fv, st);                                          \
    return true;                                                                                           \
  }
  TQ_ATT_G4X(8, 2) TQ_ATT_G4X(8, 3) TQ_ATT_G4X(8, 4) TQ_ATT_G4X(8, 8)
  TQ_ATT_G4X(18, 2) TQ_ATT_G4X(18, 3) TQ_ATT_G4X(19, 2) TQ_ATT_G4X(19, 3) TQ_ATT_G4X(19, 4) TQ_ATT_G4X(20, 3) TQ_ATT_G4X(20, 4)
#undef TQ_ATT_G4X
  return false;
}
