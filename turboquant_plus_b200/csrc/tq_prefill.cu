// Chunked-prefill attention over the packed paged cache on the 5th-generation tensor cores (tcgen05).
//
// One CTA = 128 rows of (query token, query head) pairs that share a KV head; row r is lane r of tensor memory.
// Per 128-token page: the packed page record arrives by a bulk async copy; producer warps turn the K and V indices
// (2b-bit pairs -> fp16 centroid pairs through a lane-replicated table) into unswizzled tcgen05 operand tiles in
// shared memory (K-major for K, MN-major for V); S = Q K^T and O += P V run as tcgen05.mma with the rotated queries
// (fp16 hi + lo halves), S, P and O all in tensor memory; the row warps do the online softmax between the two
// products.  The kernel, its roles, its tensor-memory map and its hand-offs are described above k_prefill_attn2.
// Every wait is bounded in time; a CTA that gives up sets the status word and still frees its tensor memory.
#include <type_traits>
#include "tq_internal.cuh"

namespace {

constexpr int PF_ROWS = 128;
constexpr long long PF_WAIT_CYCLES = 1LL << 30;

__device__ __forceinline__ uint32_t sptr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ bool pf_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  // the hint lets the hardware keep the thread suspended for up to that many nanoseconds before the instruction returns
  // false: a waiting role then spends few issue slots on polling
  asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n selp.u32 %0, 1, 0, p;\n}\n"
               : "=r"(ok) : "r"(sptr(bar)), "r"(parity), "r"(20000u) : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool pf_wait(uint64_t* bar, uint32_t parity) {
  if (pf_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  while (clock64() - t0 < PF_WAIT_CYCLES)
    if (pf_try_wait(bar, parity)) return true;
  return false;
}

// shared-memory matrix descriptor, no swizzle: start address, leading-dimension and stride byte offsets (16-byte
// units), descriptor version 1.  K-major operand: LBO = distance between 8-element K chunks, SBO = distance
// between 8-row groups.  MN-major operand: LBO = distance between 8-row K groups, SBO = between 8-element N chunks.
__device__ __forceinline__ uint64_t umma_desc(uint32_t addr, uint32_t lbo, uint32_t sbo) {
  return (uint64_t)((addr >> 4) & 0x3fff) | ((uint64_t)((lbo >> 4) & 0x3fff) << 16) |
         ((uint64_t)((sbo >> 4) & 0x3fff) << 32) | ((uint64_t)1 << 46);
}
// instruction descriptor, kind::f16: fp32 accumulator, fp16 A and B, A K-major, B major as given, N, M
__device__ __forceinline__ uint32_t umma_idesc(int m, int n, bool b_mn_major) {
  return (1u << 4) | ((b_mn_major ? 1u : 0u) << 16) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
__device__ __forceinline__ void umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t acc) {
  asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n"
               ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(acc) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(sptr(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t addr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
        "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
        "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(addr) : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t addr, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(addr) : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// sixteen columns into v[OFF .. OFF + 15], no wait: the caller waits once for all of its loads
template <int OFF, int N>
__device__ __forceinline__ void tmem_ld16_nowait(uint32_t addr, uint32_t (&v)[N]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(v[OFF]), "=r"(v[OFF + 1]), "=r"(v[OFF + 2]), "=r"(v[OFF + 3]), "=r"(v[OFF + 4]), "=r"(v[OFF + 5]),
        "=r"(v[OFF + 6]), "=r"(v[OFF + 7]), "=r"(v[OFF + 8]), "=r"(v[OFF + 9]), "=r"(v[OFF + 10]), "=r"(v[OFF + 11]),
        "=r"(v[OFF + 12]), "=r"(v[OFF + 13]), "=r"(v[OFF + 14]), "=r"(v[OFF + 15])
      : "r"(addr) : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t addr, const uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      ::"r"(addr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
        "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]) : "memory");
}
__device__ __forceinline__ float pf_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// two fp32 operations per instruction (sm_100 packed fp32), and the three-input maximum
__device__ __forceinline__ float2 pf_mul2(float2 a, float2 b) {
  float2 d;
  asm("{\n .reg .b64 ra, rb, rd;\n mov.b64 ra, {%2, %3};\n mov.b64 rb, {%4, %5};\n mul.rn.f32x2 rd, ra, rb;\n mov.b64 {%0, %1}, rd;\n}\n"
      : "=f"(d.x), "=f"(d.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
  return d;
}
__device__ __forceinline__ float2 pf_add2(float2 a, float2 b) {
  float2 d;
  asm("{\n .reg .b64 ra, rb, rd;\n mov.b64 ra, {%2, %3};\n mov.b64 rb, {%4, %5};\n add.rn.f32x2 rd, ra, rb;\n mov.b64 {%0, %1}, rd;\n}\n"
      : "=f"(d.x), "=f"(d.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
  return d;
}
__device__ __forceinline__ float pf_max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ uint32_t pf_pack(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ uint32_t pf_lds(uint32_t addr) {
  uint32_t v;
  asm("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}

// 128-point sign * Walsh-Hadamard of a row, y = post (H/sqrt d) pre x, held by two threads, 64 elements each (thread `half` has elements 64 half ... 64 half + 63):
// a 64-point transform in registers, then the last butterfly through `xs` ([element][row] floats, 64 KB of shared
// memory that nothing else uses meanwhile).  Called by all 256 row threads (named barrier 2).
constexpr int PF_HALF = TQ_D / 2;
__device__ __forceinline__ void rows_sync() { asm volatile("bar.sync 2, 256;" ::: "memory"); }
__device__ __forceinline__ void row_wht128_pair(float (&x)[PF_HALF], const uint32_t (&pre)[4], const uint32_t (&post)[4],
                                                int half, float* xs, int r) {
  const uint32_t pre0 = half ? pre[2] : pre[0], pre1 = half ? pre[3] : pre[1];
  const uint32_t post0 = half ? post[2] : post[0], post1 = half ? post[3] : post[1];
#pragma unroll
  for (int e = 0; e < PF_HALF; ++e) x[e] = (((e < 32 ? pre0 : pre1) >> (e & 31)) & 1u) ? -x[e] : x[e];
#pragma unroll
  for (int h = 1; h < PF_HALF; h <<= 1) {
#pragma unroll
    for (int i = 0; i < PF_HALF; ++i) {
      if ((i & h) == 0) {
        const float a = x[i], b = x[i + h];
        x[i] = a + b;
        x[i + h] = a - b;
      }
    }
  }
#pragma unroll
  for (int e = 0; e < PF_HALF; ++e) xs[(PF_HALF * half + e) * PF_ROWS + r] = x[e];
  rows_sync();
#pragma unroll
  for (int e = 0; e < PF_HALF; ++e) {
    const float y = xs[(PF_HALF * (half ^ 1) + e) * PF_ROWS + r];
    const float z = half ? y - x[e] : x[e] + y;
    x[e] = ((((e < 32 ? post0 : post1) >> (e & 31)) & 1u) ? -z : z) * TQ_RSQRT_D;
  }
}

struct PrefillParams {
  const uint8_t* pool;
  const int32_t* block_table;
  const int32_t* kv_lens;   // cached tokens per sequence, the chunk's own tokens included
  const void* q;            // [B][Tq][Hq][128]
  void* out;                // same shape
  const float* k_rot_t;     // dense K rotation transposed (R x)_j = sum_k rot_t[k][j] x_k, or nullptr
  const float* v_rot;       // dense V rotation row-major (R^T y)_j = sum_k rot[k][j] y_k, or nullptr
  int32_t* status;
  float qscale;             // softmax scale * log2(e)
  int32_t q_dtype, out_dtype;
  int32_t max_pages, batch, tq, hq, hkv, group;
  // split of the page range over several CTAs (flash-decoding style), merged by the last CTA to finish
  float* part_o;            // [slot][16 four-element groups][2 halves][128 rows][4]
  float* part_ml;           // [slot][128 rows][2]
  int32_t* tickets;         // [(b * hkv + kvh) * row_blocks + rb], zero between calls
  int32_t chunk_pages, num_splits, row_blocks;
  tq_cache_layout L;
};

template <int BITS> struct PfLut {
  static constexpr int ENTRIES = 1 << (2 * BITS);
  static constexpr bool REPL = ENTRIES <= 64;
  static constexpr int SHIFT = REPL ? 7 : 2;
  static constexpr int BYTES = ENTRIES << SHIFT;
};

// One token's packed indices (16*BITS bytes at `src`) -> 128 fp16 values written as sixteen 16-byte rows of the
// operand tile: chunk c (dims 8c..8c+7) goes to tile + c*128 (+ the token's row offset, already in `dst`).
// SCALED: every pair is multiplied by `scale2` (one fp16 factor in both halves) on its way to the tile.
template <int BITS, bool SCALED = false>
__device__ __forceinline__ void pf_dequant_token(const uint8_t* src, uint8_t* dst, uint32_t lut_base, uint32_t scale2 = 0) {
  constexpr int SH = PfLut<BITS>::SHIFT;
  constexpr uint32_t MASK = ((1u << (2 * BITS)) - 1) << SH;
  constexpr int NW = 4 * BITS;  // 32-bit words per token
  const uint4* s4 = reinterpret_cast<const uint4*>(src);
  uint32_t w[NW];
#pragma unroll
  for (int i = 0; i < BITS; ++i) {
    const uint4 v = s4[i];
    w[4 * i] = __byte_perm(v.x, 0, 0x0123);
    w[4 * i + 1] = __byte_perm(v.y, 0, 0x0123);
    w[4 * i + 2] = __byte_perm(v.z, 0, 0x0123);
    w[4 * i + 3] = __byte_perm(v.w, 0, 0x0123);
  }
#pragma unroll
  for (int c = 0; c < 16; ++c) {
    uint32_t o4[4];
#pragma unroll
    for (int p = 0; p < 4; ++p) {
      const int start = (4 * c + p) * 2 * BITS, k = start >> 5, o = start & 31;
      uint32_t f;
      if (o + 2 * BITS <= 32) {
        const int sr = 32 - 2 * BITS - o;
        f = sr > SH ? (w[k] >> (sr - SH)) : (sr < SH ? (w[k] << (SH - sr)) : w[k]);
      } else {
        f = __funnelshift_l(w[k + 1 < NW ? k + 1 : k], w[k], o) >> (32 - 2 * BITS - SH);
      }
      o4[p] = pf_lds((f & MASK) | lut_base);   // the table starts on a multiple of its size: one logic instruction
      if constexpr (SCALED) asm("mul.f16x2 %0, %0, %1;" : "+r"(o4[p]) : "r"(scale2));
    }
    *reinterpret_cast<uint4*>(dst + c * 128) = make_uint4(o4[0], o4[1], o4[2], o4[3]);
  }
}


// ------------------------------------------------------------------------------------------
// k_prefill_attn2: the work split over specialised warps (one CTA per SM, 544 threads):
//   warps 0-7  rows: two threads per row r = lane r of tensor memory (warps w and w + 4 reach the same 32 lanes), one
//              per half of a page's 128 score columns: reads S, online softmax (the halves exchange their maxima
//              through shared memory), writes P, rescales its half of O (lazily: only when the row maximum grows by
//              more than 2^4); both threads share the query rotation, the split partial, the merge and the output
//              (64 elements each; query and output rows pass through shared memory and the partials are laid out
//              by warp, so that every global access of a warp covers whole lines);
//   warps 8-11 K producers: thread t dequantizes the K row of token t of the page into a double-buffered operand tile
//              and copies its scale; they wait for the score MMA of page i - 2 only, one page ahead of
//   warps 12-15 V producers: the V row of token t times its V scale; their tile is free after the product of page
//              i - 2; one of them issues the bulk copies of the page records;
//   warp 16    one lane issues every tcgen05.mma: S_{i+1} = Q K_{i+1}^T is queued before O += P_i V_i, so the
//              tensor core works on the next page while the row warps are in the softmax of this one.
// (With one warp per row quarter and one per token quarter -- nine warps -- a page took 4,350 cycles.  Seventeen warps
// alone changed nothing: the time went into executed instructions -- a causal mask evaluated on every page, scalar
// fp32 arithmetic, polling loops -- and into the K producers waiting for the product of page i - 2 when the score MMA
// was all they needed.  Now ~3,300 cycles, against 1,536 of tensor work; the shared-memory pipe is the next limit.)
// Tensor memory, all 512 columns: Q hi 0-63 | Q lo 64-127 | S0 128-255 | S1 256-383 | O 384-511 (fp32, accumulated
// by the MMAs across pages).  P overlays the first 64 columns of its S buffer.  Hand-offs are mbarriers (counts in
// brackets): k_ready/v_ready [128 producer arrivals], s_full/o_done [tcgen05.commit], p_ready [128 row arrivals];
// buffer b of page i completes each of them for the (i >> 1)-th time, which fixes the parity to wait for.  Every
// wait is bounded; a role that gives up raises the CTA's fail flag, the others see it or run out of time
// themselves, and the tensor memory is released on every path.
// ------------------------------------------------------------------------------------------
constexpr int PF2_THREADS = 544;
constexpr float PF2_SLACK = 4.0f;

template <int KB, int VB> struct PfSmem2 {
  static constexpr int ALIGN = 8192;                    // each table starts on a multiple of its size (at most 8 KB)
  static constexpr int OFF_K = 0;
  static constexpr int OFF_V = 8192;
  static constexpr int OFF_BAR = 16384;              // 12 mbarriers, tensor-memory base, fail flag, 4 exchange mbarriers
  static constexpr int OFF_SC = OFF_BAR + 256;          // float K scales[4 slots][128 tokens], then the row halves'
                                                        // exchange area float[2 buffers][2 halves][128 rows], then
                                                        // their parts of the row sum float[2 halves][128 rows]
  static constexpr int OFF_KT = OFF_SC + 5120;          // K operand tiles, 2 x 32 KB
  static constexpr int OFF_VT = OFF_KT + 65536;         // V operand tiles
  static constexpr int OFF_ST = OFF_VT + 65536;         // two page records
  static size_t bytes(int record_bytes) { return (size_t)ALIGN + OFF_ST + 2 * (size_t)record_bytes; }
};

__device__ __forceinline__ void pf_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(sptr(bar)) : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t addr, const uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(addr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
        "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]),
        "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]),
        "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31]) : "memory");
}
// bounded wait whose verdict is the same in every lane of the warp (warp-collective tcgen05 instructions follow)
__device__ __forceinline__ bool pf_wait_warp(uint64_t* bar, uint32_t parity) {
  return __all_sync(0xffffffffu, pf_wait(bar, parity));
}
// AND of a predicate over the 128 V producer threads (named barrier 1)
__device__ __forceinline__ bool producers_all(bool ok) {
  uint32_t r;
  asm volatile("{\n .reg .pred p, q;\n setp.ne.b32 p, %1, 0;\n bar.red.and.pred q, 1, 128, p;\n selp.u32 %0, 1, 0, q;\n}\n"
               : "=r"(r) : "r"((uint32_t)ok) : "memory");
  return r != 0;
}

template <int KB, int VB>
__global__ void __launch_bounds__(PF2_THREADS, 1) k_prefill_attn2(const PrefillParams P, const TqFast fk, const TqFast fv) {
  using SP = PfSmem2<KB, VB>;
  extern __shared__ __align__(128) uint8_t smem_raw[];
  const int rb = blockIdx.x / P.num_splits, split = blockIdx.x - rb * P.num_splits, kvh = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int PT = P.L.page_tokens;  // 128 (checked on the host)
  const int kv_len = P.kv_lens[b];
  const int nrows = P.tq * P.group;
  const int rtid = tid & 127;                        // row (warps 0-7) or token (warps 8-15) this thread serves
  const int row = rb * PF_ROWS + rtid;
  const bool is_row = tid < 256, is_prod = tid >= 256 && tid < 512;
  const bool is_prim = tid < 128;                    // the row thread that stages the query and writes the output
  const int hf = (tid >> 7) & 1;                     // row threads: half of a page's columns; producers: 0 = K, 1 = V
  const bool row_ok = is_row && row < nrows;
  const int qi = row_ok ? row / P.group : 0, hl = row_ok ? row - qi * P.group : 0;
  const int pos = row_ok ? kv_len - P.tq + qi : -1;
  const int last_row = min(nrows, (rb + 1) * PF_ROWS) - 1;
  const int pos_max = kv_len - P.tq + last_row / P.group;
  const int np_all = min(P.max_pages, pos_max >= 0 ? pos_max / PT + 1 : 0);
  const int ns = np_all > 0 ? (np_all + P.chunk_pages - 1) / P.chunk_pages : 1;
  if (split >= ns) return;                           // nothing to do, and no tensor memory taken yet
  const int page_lo = split * P.chunk_pages;
  const int np = max(0, min(np_all, page_lo + P.chunk_pages) - page_lo);

  const uint32_t raw = sptr(smem_raw);
  uint8_t* sm = smem_raw + (((raw + SP::ALIGN - 1) & ~(uint32_t)(SP::ALIGN - 1)) - raw);
  uint64_t* bars = reinterpret_cast<uint64_t*>(sm + SP::OFF_BAR);
  uint64_t *rec_full = bars, *k_ready = bars + 2, *v_ready = bars + 4, *s_full = bars + 6, *p_ready = bars + 8,
           *o_done = bars + 10;
  uint64_t* xbar = bars + 16;   // one per row quarter: both halves' maxima of a page are in shared memory [64 arrivals]
  uint32_t* tbase = reinterpret_cast<uint32_t*>(sm + SP::OFF_BAR + 96);
  volatile int* fail = reinterpret_cast<volatile int*>(sm + SP::OFF_BAR + 104);
  float* scales = reinterpret_cast<float*>(sm + SP::OFF_SC);
  uint8_t* ktile = sm + SP::OFF_KT;
  uint8_t* vtile = sm + SP::OFF_VT;
  uint8_t* stage0 = sm + SP::OFF_ST;
  const uint32_t rec = (uint32_t)P.L.record_bytes;
  const int32_t* bt = P.block_table + (size_t)b * P.max_pages;

  auto issue = [&](int i) {
    const int64_t page = bt[page_lo + i];
    const uint8_t* src = P.pool + page * P.L.page_stride + (int64_t)kvh * P.L.head_stride;
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(sptr(&rec_full[i & 1])), "r"(rec) : "memory");
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     sptr(stage0 + (size_t)(i & 1) * rec)), "l"(src), "r"(rec), "r"(sptr(&rec_full[i & 1])) : "memory");
  };
  if (tid == 256) {
    for (int i = 0; i < 2; ++i) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(sptr(&rec_full[i])) : "memory");
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 128;" ::"r"(sptr(&k_ready[i])) : "memory");
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 128;" ::"r"(sptr(&v_ready[i])) : "memory");
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(sptr(&s_full[i])) : "memory");
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 256;" ::"r"(sptr(&p_ready[i])) : "memory");
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(sptr(&o_done[i])) : "memory");
    }
    for (int i = 0; i < 4; ++i)
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 64;" ::"r"(sptr(&xbar[i])) : "memory");
    *fail = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    if (np > 0) issue(0);
    if (np > 1) issue(1);
  }
  if (warp == 0) {  // tensor memory: all 512 columns of the SM (one CTA per SM)
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(sptr(tbase)), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (!is_prim) {
    // table fill by the 416 threads that do not rotate a query
    for (int i = tid - 128; i < PfLut<KB>::BYTES / 16; i += PF2_THREADS - 128) {
      if (PfLut<KB>::REPL) {
        const int e = i >> 3;
        const uint32_t v = (uint32_t)fk.cent16[e >> KB] | ((uint32_t)fk.cent16[e & ((1 << KB) - 1)] << 16);
        reinterpret_cast<uint4*>(sm + SP::OFF_K)[i] = make_uint4(v, v, v, v);
      } else {
        uint32_t v[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const int e = 4 * i + k;
          v[k] = (uint32_t)fk.cent16[e >> KB] | ((uint32_t)fk.cent16[e & ((1 << KB) - 1)] << 16);
        }
        reinterpret_cast<uint4*>(sm + SP::OFF_K)[i] = make_uint4(v[0], v[1], v[2], v[3]);
      }
    }
    for (int i = tid - 128; i < PfLut<VB>::BYTES / 16; i += PF2_THREADS - 128) {
      if (PfLut<VB>::REPL) {
        const int e = i >> 3;
        const uint32_t v = (uint32_t)fv.cent16[e >> VB] | ((uint32_t)fv.cent16[e & ((1 << VB) - 1)] << 16);
        reinterpret_cast<uint4*>(sm + SP::OFF_V)[i] = make_uint4(v, v, v, v);
      } else {
        uint32_t v[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const int e = 4 * i + k;
          v[k] = (uint32_t)fv.cent16[e >> VB] | ((uint32_t)fv.cent16[e & ((1 << VB) - 1)] << 16);
        }
        reinterpret_cast<uint4*>(sm + SP::OFF_V)[i] = make_uint4(v[0], v[1], v[2], v[3]);
      }
    }
  }

  // ---- prologue (row warps): this row's query, rotated by the K rotation, scaled, fp16 hi + lo into tensor memory;
  // each of the row's two threads holds one half of its elements ----
  float o[PF_HALF];
  if (is_row) {
    // The rows come in through shared memory: read directly, a thread's own half row would put the lanes of a load
    // 256 or 512 bytes apart (one line per lane and instruction); staged, a warp reads whole rows.  Row stride: the
    // row plus 16 bytes, so that the 16-byte accesses of consecutive rows fall into different banks.
    {
      const int esz = P.q_dtype == TQ_F32 ? 4 : 2;
      const int cpr = TQ_D * esz / 16, stride = TQ_D * esz + 16;   // 16-byte chunks per row
      uint8_t* stg = ktile;                                        // the operand tiles are not in use yet
#pragma unroll 8
      for (int it = 0; it < cpr / 2; ++it) {
        const int c = it * 256 + tid, r = c / cpr, w = c - r * cpr;
        const int grow = rb * PF_ROWS + r;
        uint4 val = make_uint4(0u, 0u, 0u, 0u);
        if (grow < nrows) {
          const int gq = grow / P.group, gh = grow - gq * P.group;
          const size_t off = ((((size_t)b * P.tq + gq) * P.hq + (size_t)kvh * P.group + gh) * TQ_D) * esz + w * 16;
          val = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(P.q) + off);
        }
        *reinterpret_cast<uint4*>(stg + r * stride + w * 16) = val;
      }
      rows_sync();
      const uint8_t* mine = stg + rtid * stride + hf * PF_HALF * esz;
      if (P.q_dtype == TQ_F32) {
#pragma unroll
        for (int e = 0; e < PF_HALF; e += 4) {
          const float4 v = *reinterpret_cast<const float4*>(mine + e * 4);
          o[e] = v.x; o[e + 1] = v.y; o[e + 2] = v.z; o[e + 3] = v.w;
        }
      } else {
#pragma unroll
        for (int e = 0; e < PF_HALF; e += 8) {
          const uint4 w4 = *reinterpret_cast<const uint4*>(mine + e * 2);
          const uint32_t ww[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const float2 f = P.q_dtype == TQ_F16 ? __half22float2(*reinterpret_cast<const __half2*>(&ww[k]))
                                                 : __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&ww[k]));
            o[e + 2 * k] = f.x; o[e + 2 * k + 1] = f.y;
          }
        }
      }
      rows_sync();   // the staged rows are read: the exchange area of the rotation below is the same memory
    }
    float* xs = reinterpret_cast<float*>(ktile);  // [k][row], 64 KB: the operand tiles are not in use yet
    if (P.k_rot_t) {
      // dense rotation: the rows staged transposed, then this thread's 64 elements of y = R x
#pragma unroll
      for (int k = 0; k < PF_HALF; ++k) xs[(PF_HALF * hf + k) * PF_ROWS + rtid] = o[k];
      rows_sync();
#pragma unroll
      for (int j = 0; j < PF_HALF; ++j) o[j] = 0.f;
      for (int k = 0; k < TQ_D; ++k) {
        const float xv = xs[k * PF_ROWS + rtid];
        const float4* rr = reinterpret_cast<const float4*>(P.k_rot_t + (size_t)k * TQ_D + PF_HALF * hf);
#pragma unroll
        for (int j = 0; j < PF_HALF; j += 4) {
          const float4 r4 = __ldg(rr + (j >> 2));
          o[j] = fmaf(r4.x, xv, o[j]); o[j + 1] = fmaf(r4.y, xv, o[j + 1]);
          o[j + 2] = fmaf(r4.z, xv, o[j + 2]); o[j + 3] = fmaf(r4.w, xv, o[j + 3]);
        }
      }
    } else {
      row_wht128_pair(o, fk.s1, fk.s2, hf, xs, rtid);
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();  // tensor-memory base, tables and barriers visible; the dense staging area is free again
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tb = *tbase;
  const uint32_t TQc = 0, TQLc = 64, TSc = 128, TOc = 384;   // S buffer b at TSc + 128 b; P overlays its first 64 columns

  if (is_row) {
    // =========================== row warps ===========================
    const uint32_t tm = tb + ((uint32_t)((warp & 3) * 32) << 16);  // this warp's 32 lanes
    float* xch = scales + 512;                                     // [buffer][half][row]
    {
      const float sk = P.qscale / fk.lut_alpha;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t u[16], ul[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const float a = o[32 * c + 2 * j] * sk, bq = o[32 * c + 2 * j + 1] * sk;
          const __half2 h = __floats2half2_rn(a, bq);
          const float2 hv = __half22float2(h);
          u[j] = *reinterpret_cast<const uint32_t*>(&h);
          ul[j] = pf_pack(a - hv.x, bq - hv.y);
        }
        tmem_st16(tm + TQc + 32 * hf + 16 * c, u);
        tmem_st16(tm + TQLc + 32 * hf + 16 * c, ul);
      }
      asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    }
    asm volatile("bar.sync 3, 288;" ::: "memory");   // with the MMA warp: the queries are in tensor memory

    float m_run = -INFINITY, l_run = 0.f;   // l_run: this half's part of the row sum
    for (int i = 0; i < np; ++i) {
      if (*fail) break;
      const int bf = i & 1;
      const uint32_t ph = (uint32_t)((i >> 1) & 1);
      if (!pf_wait_warp(&s_full[bf], ph)) { *fail = 1; break; }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const float4* ksc4 = reinterpret_cast<const float4*>(scales + (i & 3) * PF_ROWS + 64 * hf);
      const uint32_t ts = tm + TSc + 128 * bf;
      const int t0 = (page_lo + i) * PT;
      // a page that every row of this warp sees completely needs no causal mask (rows without a query count as
      // seeing everything: nothing of theirs is stored)
      const bool masked = !__all_sync(0xffffffffu, !row_ok || t0 + PT - 1 <= pos);
      // pass 1: this half's scaled scores into registers, row maximum
      float sv[64];
      float mx = -INFINITY;
      uint32_t raw[64];   // the four loads fly together; each score replaces its raw value (same registers)
      tmem_ld16_nowait<0>(ts + 64 * hf, raw);
      tmem_ld16_nowait<16>(ts + 64 * hf + 16, raw);
      tmem_ld16_nowait<32>(ts + 64 * hf + 32, raw);
      tmem_ld16_nowait<48>(ts + 64 * hf + 48, raw);
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      auto pass1 = [&](auto masked_c) {   // two copies behind a warp-uniform branch: only the diagonal pages pay for the mask
        constexpr bool MASKED = decltype(masked_c)::value;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const uint32_t* v = raw + 16 * c;
#pragma unroll
          for (int j = 0; j < 16; j += 4) {
            const float4 k4 = ksc4[4 * c + (j >> 2)];
            float2 x01 = pf_mul2(make_float2(__uint_as_float(v[j]), __uint_as_float(v[j + 1])), make_float2(k4.x, k4.y));
            float2 x23 = pf_mul2(make_float2(__uint_as_float(v[j + 2]), __uint_as_float(v[j + 3])), make_float2(k4.z, k4.w));
            if (MASKED) {
              const int tt = t0 + 64 * hf + 16 * c + j;
              x01.x = tt <= pos ? x01.x : -INFINITY;
              x01.y = tt + 1 <= pos ? x01.y : -INFINITY;
              x23.x = tt + 2 <= pos ? x23.x : -INFINITY;
              x23.y = tt + 3 <= pos ? x23.y : -INFINITY;
            }
            sv[16 * c + j] = x01.x; sv[16 * c + j + 1] = x01.y;
            sv[16 * c + j + 2] = x23.x; sv[16 * c + j + 3] = x23.y;
            mx = pf_max3(mx, x01.x, x01.y);
            mx = pf_max3(mx, x23.x, x23.y);
          }
        }
      };
      if (masked) pass1(std::true_type{}); else pass1(std::false_type{});
      // the other half's maximum: both threads of a row then take the same decisions below.  (The arrival also tells
      // the other half that this one has read its scores: the P columns that half writes overlay them.)
      xch[(bf * 2 + hf) * PF_ROWS + rtid] = mx;
      pf_arrive(&xbar[warp & 3]);
      if (!pf_wait_warp(&xbar[warp & 3], (uint32_t)(i & 1))) { *fail = 1; break; }
      mx = fmaxf(mx, xch[(bf * 2 + (hf ^ 1)) * PF_ROWS + rtid]);
      // The row maximum moves only when it grows by more than 2^PF2_SLACK (probabilities stay below 2^PF2_SLACK).
      // O lives in tensor memory and is being accumulated by the MMAs: a rescale waits for the product of the
      // page before, multiplies the row in place, and only then lets this page's product start (p_ready below).
      float resc = 1.0f;
      if (i == 0) {
        // the reference starts PF2_SLACK above the first page's maximum: a later page then moves it only when it
        // beats that maximum by 2^(2 PF2_SLACK), which is rare -- and every move stalls the row on the tensor core
        m_run = mx + PF2_SLACK;
      } else if (mx > m_run + PF2_SLACK) {
        resc = pf_exp2(m_run - mx);   // m_run == -inf (nothing seen yet) gives 0: the row of O is zero anyway
        m_run = mx;
        l_run *= resc;
      }
      if (i > 0 && __any_sync(0xffffffffu, resc != 1.0f)) {
        if (!pf_wait_warp(&o_done[(i - 1) & 1], (uint32_t)(((i - 1) >> 1) & 1))) { *fail = 1; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
        for (int c = 0; c < 2; ++c) {   // this half's 64 columns of O
          uint32_t v[32];
          tmem_ld32(tm + TOc + 64 * hf + 32 * c, v);
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) * resc);
          tmem_st32(tm + TOc + 64 * hf + 32 * c, v);
        }
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      }
      // pass 2: probabilities (masked scores are -inf and give 0), row sum, P as packed fp16 (the V scales are in the
      // V operand tile)
      const float m_use = m_run == -INFINITY ? 0.f : m_run;
      const float2 nm2 = make_float2(-m_use, -m_use);
      float2 ls2 = make_float2(0.f, 0.f);
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t u[16];
#pragma unroll
        for (int j = 0; j < 32; j += 2) {
          float2 p = pf_add2(make_float2(sv[32 * c + j], sv[32 * c + j + 1]), nm2);
          p.x = pf_exp2(p.x);
          p.y = pf_exp2(p.y);
          ls2 = pf_add2(ls2, p);
          u[j >> 1] = pf_pack(p.x, p.y);
        }
        tmem_st16(ts + 32 * hf + 16 * c, u);  // P overlays S columns 0-63, which the first half has consumed
      }
      l_run += ls2.x + ls2.y;
      asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      pf_arrive(&p_ready[bf]);
    }
    // this thread's half of the accumulated row of O, once the last product has completed
    scales[(8 + hf) * PF_ROWS + rtid] = l_run;   // the halves' parts of the row sum
#pragma unroll
    for (int j = 0; j < PF_HALF; ++j) o[j] = 0.f;
    if (np > 0 && !*fail) {
      if (!pf_wait_warp(&o_done[(np - 1) & 1], (uint32_t)(((np - 1) >> 1) & 1))) {
        *fail = 1;
      } else {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t v[32];
          tmem_ld32(tm + TOc + PF_HALF * hf + 32 * c, v);
#pragma unroll
          for (int j = 0; j < 32; ++j) o[32 * c + j] = __uint_as_float(v[j]);
        }
      }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();  // every role is done with tensor memory
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tb), "r"(512u) : "memory");
    l_run = scales[8 * PF_ROWS + rtid] + scales[9 * PF_ROWS + rtid];
    // A CTA that gave up a wait reports it, writes no partial and merges nothing, but still takes its ticket below:
    // the counter of its (sequence, KV head, row block) then returns to zero like after a clean call, and a later
    // call on the same workspace cannot elect its merger too early.
    const bool failed = *fail != 0;   // stable: every role has passed the barrier above
    if (failed && tid == 0) atomicExch(P.status, 1);
    if (failed && ns <= 1) return;
    // ---- split partial / merge by the last split / epilogue: the 256 row threads only ----
    if (ns > 1) {
      const size_t slot0 = (((size_t)b * P.hkv + kvh) * P.row_blocks + rb) * P.num_splits;
      if (!failed) {
        // partial of a slot: [16 four-element groups][half][128 rows] float4 -- a warp's stores and loads are contiguous
        float4* po = reinterpret_cast<float4*>(P.part_o + (slot0 + split) * PF_ROWS * TQ_D) + hf * PF_ROWS + rtid;
#pragma unroll
        for (int j = 0; j < PF_HALF; j += 4) po[(j >> 2) * 2 * PF_ROWS] = make_float4(o[j], o[j + 1], o[j + 2], o[j + 3]);
        if (is_prim) reinterpret_cast<float2*>(P.part_ml)[(slot0 + split) * PF_ROWS + rtid] = make_float2(m_run, l_run);
      }
      __threadfence();
      rows_sync();
      if (tid == 0) {
        int* tk = P.tickets + ((size_t)b * P.hkv + kvh) * P.row_blocks + rb;
        const int prev = atomicAdd(tk, 1);
        int last = 0;
        if (prev == ns - 1) {
          *tk = 0;  // zero again for the next call
          last = 1;
        }
        *fail = last;  // reuse the flag word as "this CTA merges"
      }
      rows_sync();
      if (!*fail || failed) return;
      __threadfence();
      float M = -INFINITY;
      for (int s_i = 0; s_i < ns; ++s_i)
        M = fmaxf(M, __ldcg(reinterpret_cast<const float2*>(P.part_ml) + (slot0 + s_i) * PF_ROWS + rtid).x);
#pragma unroll
      for (int j = 0; j < PF_HALF; ++j) o[j] = 0.f;
      l_run = 0.f;
      for (int s_i = 0; s_i < ns; ++s_i) {
        const float2 ml = __ldcg(reinterpret_cast<const float2*>(P.part_ml) + (slot0 + s_i) * PF_ROWS + rtid);
        const float f = ml.x == -INFINITY ? 0.f : exp2f(ml.x - M);
        l_run = fmaf(ml.y, f, l_run);
        const float4* po = reinterpret_cast<const float4*>(P.part_o + (slot0 + s_i) * PF_ROWS * TQ_D) + hf * PF_ROWS + rtid;
#pragma unroll
        for (int j = 0; j < PF_HALF; j += 4) {
          const float4 v = __ldcg(po + (j >> 2) * 2 * PF_ROWS);
          o[j] = fmaf(v.x, f, o[j]); o[j + 1] = fmaf(v.y, f, o[j + 1]);
          o[j + 2] = fmaf(v.z, f, o[j + 2]); o[j + 3] = fmaf(v.w, f, o[j + 3]);
        }
      }
    }
    {
      const float inv = l_run > 0.f ? 1.0f / (l_run * fv.lut_alpha) : 0.f;
#pragma unroll
      for (int j = 0; j < PF_HALF; ++j) o[j] *= inv;
      float* ys = reinterpret_cast<float*>(ktile);  // [k][row]; the operand tiles are idle by now
      if (P.v_rot) {
#pragma unroll
        for (int k = 0; k < PF_HALF; ++k) ys[(PF_HALF * hf + k) * PF_ROWS + rtid] = o[k];
        rows_sync();
#pragma unroll
        for (int j = 0; j < PF_HALF; ++j) o[j] = 0.f;
        for (int k = 0; k < TQ_D; ++k) {
          const float yv = ys[k * PF_ROWS + rtid];
          const float4* rr = reinterpret_cast<const float4*>(P.v_rot + (size_t)k * TQ_D + PF_HALF * hf);
#pragma unroll
          for (int j = 0; j < PF_HALF; j += 4) {
            const float4 r4 = __ldg(rr + (j >> 2));
            o[j] = fmaf(r4.x, yv, o[j]); o[j + 1] = fmaf(r4.y, yv, o[j + 1]);
            o[j + 2] = fmaf(r4.z, yv, o[j + 2]); o[j + 3] = fmaf(r4.w, yv, o[j + 3]);
          }
        }
      } else {
        row_wht128_pair(o, fv.s2, fv.s1, hf, ys, rtid);  // R^T = D1 (H/sqrt d) D2
      }
      // The rows leave through shared memory like they came in: staged, a warp writes whole rows.
      rows_sync();   // the exchange area of the rotation is read: the staging below is the same memory
      {
        const int esz = P.out_dtype == TQ_F32 ? 4 : 2;
        const int cpr = TQ_D * esz / 16, stride = TQ_D * esz + 16;
        uint8_t* stg = ktile;
        uint8_t* mine = stg + rtid * stride + hf * PF_HALF * esz;
        if (P.out_dtype == TQ_F32) {
#pragma unroll
          for (int j = 0; j < PF_HALF; j += 4)
            *reinterpret_cast<float4*>(mine + j * 4) = make_float4(o[j], o[j + 1], o[j + 2], o[j + 3]);
        } else if (P.out_dtype == TQ_F16) {
#pragma unroll
          for (int j = 0; j < PF_HALF; j += 8)
            *reinterpret_cast<uint4*>(mine + j * 2) = make_uint4(pf_pack(o[j], o[j + 1]), pf_pack(o[j + 2], o[j + 3]),
                                                                 pf_pack(o[j + 4], o[j + 5]), pf_pack(o[j + 6], o[j + 7]));
        } else {
#pragma unroll
          for (int j = 0; j < PF_HALF; j += 8) {
            uint32_t w[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const __nv_bfloat162 h = __floats2bfloat162_rn(o[j + 2 * k], o[j + 2 * k + 1]);
              w[k] = *reinterpret_cast<const uint32_t*>(&h);
            }
            *reinterpret_cast<uint4*>(mine + j * 2) = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
        rows_sync();
#pragma unroll 8
        for (int it = 0; it < cpr / 2; ++it) {
          const int c = it * 256 + tid, r = c / cpr, w = c - r * cpr;
          const int grow = rb * PF_ROWS + r;
          if (grow < nrows) {
            const int gq = grow / P.group, gh = grow - gq * P.group;
            const size_t off = ((((size_t)b * P.tq + gq) * P.hq + (size_t)kvh * P.group + gh) * TQ_D) * esz + w * 16;
            *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(P.out) + off) =
                *reinterpret_cast<const uint4*>(stg + r * stride + w * 16);
          }
        }
      }
    }
    return;
  }

  if (is_prod) {
    // =========================== producer warps ===========================
    const uint32_t lk_base = sptr(sm + SP::OFF_K) + (PfLut<KB>::REPL ? lane * 4 : 0);
    const uint32_t lv_base = sptr(sm + SP::OFF_V) + (PfLut<VB>::REPL ? lane * 4 : 0);
    const uint32_t tile_row = (uint32_t)(rtid >> 3) * 2048 + (uint32_t)(rtid & 7) * 16;  // token rtid inside an operand tile
    if (hf == 0) {
      // K producers.  The K tile of buffer bf is free once S of page i - 2 is complete, and so is the scale slot
      // i & 3 (the rows finished page i - 4 long before): they run one page ahead of the V producers, whose tile is
      // free only after the product of page i - 2, and S of the next page is ready before the rows ask for it.
      for (int i = 0; i < np; ++i) {
        const int bf = i & 1;
        if (*fail) break;
        if (i >= 2 && !pf_wait(&s_full[bf], (uint32_t)(((i - 2) >> 1) & 1))) { *fail = 1; break; }
        if (!pf_wait(&rec_full[bf], (uint32_t)((i >> 1) & 1))) { *fail = 1; break; }
        const uint8_t* st = stage0 + (size_t)bf * rec;
        pf_dequant_token<KB>(st + P.L.k_idx_off + rtid * (16 * KB), ktile + bf * 32768 + tile_row, lk_base);
        scales[(i & 3) * PF_ROWS + rtid] = reinterpret_cast<const float*>(st + P.L.k_scale_off)[rtid];
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        pf_arrive(&k_ready[bf]);   // also: this thread has read its part of the record
      }
    } else {
      // V producers; one of them refills a record's stage once both groups have read it
      for (int i = 0; i < np; ++i) {
        const int bf = i & 1;
        const uint32_t ph = (uint32_t)((i >> 1) & 1);
        bool ok = !*fail;
        if (ok && i >= 2) ok = pf_wait(&o_done[bf], (uint32_t)(((i - 2) >> 1) & 1));
        if (ok) ok = pf_wait(&rec_full[bf], ph);
        if (!producers_all(ok)) {  // the 128 V producers go on or give up together (they share a named barrier below)
          *fail = 1;
          break;
        }
        const uint8_t* st = stage0 + (size_t)bf * rec;
        // The token's V scale goes into its row of the operand tile (fp16 product, rounding 2^-11 per element), so
        // that the P operand is the bare probability, bounded by 2^(2 PF2_SLACK) whatever the norms of the values
        // are; a token past the end of the sequence may hold anything: its row is zeroed (its P is zero too, but
        // 0 x inf would not be).  Scales beyond the fp16 range saturate.
        const float vsc = (page_lo + i) * PT + rtid < kv_len ? reinterpret_cast<const float*>(st + P.L.v_scale_off)[rtid] : 0.f;
        const __half2 s2 = __float2half2_rn(fminf(vsc, 65504.0f));
        pf_dequant_token<VB, true>(st + P.L.v_idx_off + rtid * (16 * VB), vtile + bf * 32768 + tile_row, lv_base,
                                   *reinterpret_cast<const uint32_t*>(&s2));
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        pf_arrive(&v_ready[bf]);
        asm volatile("bar.sync 1, 128;" ::: "memory");   // every V producer has read this record
        if (tid == 384 && i + 2 < np) {
          if (!pf_wait(&k_ready[bf], ph)) { *fail = 1; } else { issue(i + 2); }   // ... and every K producer
        }
      }
    }
    asm volatile("bar.sync 5, 256;" ::: "memory");   // both groups have left their loops: no copy will be issued any more
    if (*fail && tid == 256) {  // copies in flight get the same bounded time before the CTA leaves
      for (int st_i = 0; st_i < 2; ++st_i) pf_wait(&rec_full[st_i], 0), pf_wait(&rec_full[st_i], 1);
    }
  } else {
    // =========================== MMA warp ===========================
    asm volatile("bar.sync 3, 288;" ::: "memory");
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (lane == 0 && np > 0) {
      const uint32_t idesc_s = umma_idesc(128, 128, false), idesc_o = umma_idesc(128, 128, true);
      auto qk = [&](int i) {   // S_i = Q K_i^T (fp16 hi and lo halves of Q), into S buffer i & 1
        const int bf = i & 1;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint64_t kd = umma_desc(sptr(ktile + bf * 32768) + ks * 256, 128, 2048);
          umma_ts(tb + TSc + 128 * bf, tb + TQc + ks * 8, kd, idesc_s, ks > 0);
          umma_ts(tb + TSc + 128 * bf, tb + TQLc + ks * 8, kd, idesc_s, 1);
        }
        umma_commit(&s_full[bf]);
      };
      bool okay = pf_wait(&k_ready[0], 0);
      if (okay) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        qk(0);
      }
      for (int i = 0; okay && i < np; ++i) {
        if (*fail) break;
        const int bf = i & 1;
        const uint32_t ph = (uint32_t)((i >> 1) & 1);
        if (i + 1 < np) {
          if (!pf_wait(&k_ready[(i + 1) & 1], (uint32_t)(((i + 1) >> 1) & 1))) { okay = false; break; }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          qk(i + 1);
        }
        if (!pf_wait(&p_ready[bf], ph) || !pf_wait(&v_ready[bf], ph)) { okay = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)   // O += P_i V_i: P from tensor memory, V tile MN-major, N = 128
          umma_ts(tb + TOc, tb + TSc + 128 * bf + ks * 8, umma_desc(sptr(vtile + bf * 32768) + ks * 4096, 2048, 128),
                  idesc_o, (i > 0 || ks > 0) ? 1u : 0u);
        umma_commit(&o_done[bf]);
      }
      if (!okay) *fail = 1;
    }
    __syncwarp();
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();  // matches the row warps' barrier before the tensor memory is released
}

}  // namespace

template <int KB, int VB>
static int launch_prefill(const PrefillParams& P, const TqFast& fk, const TqFast& fv, cudaStream_t st) {
  const size_t need = PfSmem2<KB, VB>::bytes(P.L.record_bytes);
  constexpr size_t LIMIT = 220 * 1024;  // one CTA per SM (it also takes all 512 tensor-memory columns)
  TQ_REQUIRE(need <= LIMIT, TQ_ERR_TOO_LARGE, "page record of %d bytes does not fit the prefill pipeline",
             P.L.record_bytes);
  static thread_local int configured_dev = -1;
  int dev = 0;
  TQ_CUDA(cudaGetDevice(&dev));
  if (configured_dev != dev) {
    TQ_CUDA(cudaFuncSetAttribute(k_prefill_attn2<KB, VB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)LIMIT));
    configured_dev = dev;
  }
  dim3 grid(P.row_blocks * P.num_splits, P.hkv, P.batch);
  k_prefill_attn2<KB, VB><<<grid, PF2_THREADS, need, st>>>(P, fk, fv);
  return tq_launch_check("k_prefill_attn2");
}

struct PfPlan {
  int row_blocks, chunk_pages, num_splits;
  size_t part_o, part_ml, total;
};
static const size_t PF_TAIL = 65536 * 4 + 256;  // tickets + status word, at the end of the workspace
static const long PF_CTA_COST_PAGES = 16;  // prologue, partial and merge of a CTA, in units of one page of the main loop

static PfPlan pf_plan(int batch, int chunk_tokens, int hq, int hkv, int max_pages) {
  PfPlan p;
  p.row_blocks = (chunk_tokens * (hq / hkv) + PF_ROWS - 1) / PF_ROWS;
  const long base = (long)p.row_blocks * hkv * batch;
  const int slots = tq_num_sms();  // one CTA per SM
  const int cap = max_pages / 8 > 1 ? max_pages / 8 : 1;  // at least eight pages per split
  // splits per row block: the count that minimises (waves of CTAs) x (pages per split + fixed cost of a CTA)
  int s = 1;
  long best = -1;
  for (int c = 1; c <= cap && c <= 64; ++c) {
    const long waves = (base * c + slots - 1) / slots;
    const long cost = waves * ((max_pages + c - 1) / c + PF_CTA_COST_PAGES);
    if (best < 0 || cost < best) {
      best = cost;
      s = c;
    }
  }
  p.chunk_pages = (max_pages + s - 1) / s;
  p.num_splits = (max_pages + p.chunk_pages - 1) / p.chunk_pages;
  const size_t slots_total = (size_t)base * p.num_splits;
  p.part_o = 0;
  p.part_ml = slots_total * PF_ROWS * TQ_D * 4;
  p.total = p.part_ml + slots_total * PF_ROWS * 2 * 4 + PF_TAIL;
  p.total = (p.total + 255) & ~(size_t)255;
  return p;
}

extern "C" int64_t tq_prefill_workspace_bytes(int32_t batch, int32_t chunk_tokens, int32_t num_q_heads,
                                              int32_t num_kv_heads, int32_t max_pages_per_seq) {
  if (batch < 1 || chunk_tokens < 1 || num_q_heads < 1 || num_kv_heads < 1 || max_pages_per_seq < 1 ||
      num_q_heads % num_kv_heads)
    return TQ_ERR_INVALID;
  return (int64_t)pf_plan(batch, chunk_tokens, num_q_heads, num_kv_heads, max_pages_per_seq).total;
}

extern "C" int tq_prefill_attn(const tq_quantizer* kq, const tq_quantizer* vq, const tq_cache_layout* L,
                               const uint8_t* pool_dev, const int32_t* block_table_dev, int32_t max_pages_per_seq,
                               const int32_t* kv_lens_dev, const void* q_dev, int32_t q_dtype, int32_t batch,
                               int32_t chunk_tokens, int32_t num_q_heads, float scale, void* workspace_dev,
                               int64_t workspace_bytes, void* out_dev, int32_t out_dtype, void* stream) {
  TQ_REQUIRE(kq && vq && L, TQ_ERR_INVALID, "tq_prefill_attn: quantizers or layout missing");
  TQ_REQUIRE(batch >= 0 && chunk_tokens >= 1 && num_q_heads >= 1 && max_pages_per_seq >= 1, TQ_ERR_INVALID, "bad sizes");
  if (batch == 0) return TQ_OK;
  TQ_REQUIRE(pool_dev && block_table_dev && kv_lens_dev && q_dev && out_dev && workspace_dev, TQ_ERR_INVALID,
             "tq_prefill_attn: null buffer");
  TQ_REQUIRE(workspace_bytes % 256 == 0 && tq_aligned(workspace_dev, 256), TQ_ERR_ALIGN,
             "workspace must be 256-byte aligned and a multiple of 256 bytes");
  TQ_REQUIRE(L->d == TQ_D && L->page_tokens == 128, TQ_ERR_UNSUPPORTED,
             "prefill attention is built for d == 128 and 128-token pages");
  TQ_REQUIRE(L->k_format >= TQ_FMT_TURBO2 && L->k_format <= TQ_FMT_TURBO4 && L->v_format >= TQ_FMT_TURBO2 &&
                 L->v_format <= TQ_FMT_TURBO4,
             TQ_ERR_UNSUPPORTED, "prefill attention is built for turbo2/3/4 K and V, got %d / %d", L->k_format, L->v_format);
  TQ_REQUIRE(kq->d == TQ_D && vq->d == TQ_D && kq->bits == L->k_format && vq->bits == L->v_format, TQ_ERR_INVALID,
             "quantizer bit widths do not match the cache formats");
  TQ_REQUIRE(num_q_heads % L->num_kv_heads == 0, TQ_ERR_INVALID, "num_q_heads must be a multiple of num_kv_heads");
  TQ_REQUIRE(q_dtype == TQ_F16 || q_dtype == TQ_BF16 || q_dtype == TQ_F32, TQ_ERR_UNSUPPORTED, "bad query dtype %d", q_dtype);
  TQ_REQUIRE(out_dtype == TQ_F16 || out_dtype == TQ_BF16 || out_dtype == TQ_F32, TQ_ERR_UNSUPPORTED, "bad output dtype %d", out_dtype);
  TQ_REQUIRE(tq_aligned(pool_dev, 128) && tq_aligned(q_dev, 16) && tq_aligned(out_dev, 16), TQ_ERR_ALIGN,
             "pool (128), q and out (16) must be aligned");
  TQ_REQUIRE(batch <= 65535 && L->num_kv_heads <= 65535, TQ_ERR_TOO_LARGE, "batch and KV heads are grid dimensions");
  PrefillParams P;
  memset(&P, 0, sizeof(P));
  P.pool = pool_dev;
  P.block_table = block_table_dev;
  P.kv_lens = kv_lens_dev;
  P.q = q_dev;
  P.out = out_dev;
  P.k_rot_t = kq->rotation == TQ_ROT_DENSE ? kq->rot32_t : nullptr;
  P.v_rot = vq->rotation == TQ_ROT_DENSE ? vq->rot32 : nullptr;
  P.status = reinterpret_cast<int32_t*>((uint8_t*)workspace_dev + workspace_bytes - 256);
  if (scale <= 0.f) scale = TQ_RSQRT_D;
  P.qscale = scale * 1.4426950408889634f;
  P.q_dtype = q_dtype;
  P.out_dtype = out_dtype;
  P.max_pages = max_pages_per_seq;
  P.batch = batch;
  P.tq = chunk_tokens;
  P.hq = num_q_heads;
  P.hkv = L->num_kv_heads;
  P.group = num_q_heads / L->num_kv_heads;
  const PfPlan plan = pf_plan(batch, chunk_tokens, num_q_heads, L->num_kv_heads, max_pages_per_seq);
  TQ_REQUIRE((int64_t)plan.total <= workspace_bytes, TQ_ERR_TOO_LARGE,
             "prefill workspace of %lld bytes is smaller than the %lld needed (tq_prefill_workspace_bytes)",
             (long long)workspace_bytes, (long long)plan.total);
  TQ_REQUIRE((int64_t)batch * L->num_kv_heads * plan.row_blocks <= 65536, TQ_ERR_TOO_LARGE,
             "batch x KV heads x row blocks beyond 65536");
  P.part_o = reinterpret_cast<float*>((uint8_t*)workspace_dev + plan.part_o);
  P.part_ml = reinterpret_cast<float*>((uint8_t*)workspace_dev + plan.part_ml);
  P.tickets = reinterpret_cast<int32_t*>((uint8_t*)workspace_dev + workspace_bytes - PF_TAIL);
  P.chunk_pages = plan.chunk_pages;
  P.num_splits = plan.num_splits;
  P.row_blocks = plan.row_blocks;
  P.L = *L;
  cudaStream_t st = (cudaStream_t)stream;
  int rc = TQ_ERR_UNSUPPORTED;
#define TQ_PF(K, V) \
  if (L->k_format == K && L->v_format == V) rc = launch_prefill<K, V>(P, kq->fast, vq->fast, st);
  TQ_PF(2, 2) TQ_PF(3, 3) TQ_PF(4, 4) TQ_PF(3, 2) TQ_PF(4, 2) TQ_PF(4, 3)
#undef TQ_PF
  if (rc == TQ_ERR_UNSUPPORTED) tq_set_error("prefill attention: K format %d with V format %d is not instantiated", L->k_format, L->v_format);
  return rc;
}
