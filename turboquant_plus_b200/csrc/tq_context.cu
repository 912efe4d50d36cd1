// Quantizer constants, error reporting and the paged-cache layout arithmetic.
#include <math.h>
#include <stdarg.h>
#include <stdlib.h>

#include <vector>

#include "tq_internal.cuh"

static thread_local char g_err[512] = "";

void tq_set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

int tq_cuda_fail(cudaError_t e, const char* what) {
  tq_set_error("CUDA error %d (%s) in %s", (int)e, cudaGetErrorString(e), what);
  return (e == cudaErrorNoKernelImageForDevice || e == cudaErrorInvalidDeviceFunction) ? TQ_ERR_DEVICE
                                                                                       : TQ_ERR_CUDA;
}

int tq_launch_check(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return tq_cuda_fail(e, what);
  return TQ_OK;
}

int tq_num_sms() {
  static thread_local int cached_dev = -1, cached = 0;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 148;
  if (dev != cached_dev) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached = n;
    cached_dev = dev;
  }
  return cached;
}

extern "C" const char* tq_version(void) { return "tq_b200 0.1 (sm_100a)"; }

extern "C" const char* tq_error_string(int code) {
  switch (code) {
    case TQ_OK: return "ok";
    case TQ_ERR_INVALID: return "invalid argument";
    case TQ_ERR_UNSUPPORTED: return "unsupported combination";
    case TQ_ERR_ALIGN: return "misaligned pointer or stride";
    case TQ_ERR_CUDA: return "CUDA runtime error";
    case TQ_ERR_TOO_LARGE: return "size beyond the supported maximum";
    case TQ_ERR_DEVICE: return "no kernel image for this device (needs sm_100a)";
    default: return "unknown error";
  }
}

extern "C" const char* tq_last_error(void) { return g_err; }

static bool is_pm1(const double* v, int n) {
  for (int i = 0; i < n; ++i)
    if (v[i] != 1.0 && v[i] != -1.0) return false;
  return true;
}

static void sign_bits(const double* v, uint32_t (&out)[4]) {
  for (int w = 0; w < 4; ++w) out[w] = 0;
  for (int e = 0; e < TQ_D; ++e)
    if (v[e] < 0) out[e >> 5] |= 1u << (e & 31);
}

template <typename T>
static int upload(T** dst, const std::vector<T>& src) {
  TQ_CUDA(cudaMalloc((void**)dst, src.size() * sizeof(T)));
  TQ_CUDA(cudaMemcpy(*dst, src.data(), src.size() * sizeof(T), cudaMemcpyHostToDevice));
  return TQ_OK;
}

static int upload_matrix(const double* m, int d, double** dev, double** dev_t, float** dev32, float** dev32_t) {
  std::vector<double> a(m, m + (size_t)d * d), t((size_t)d * d);
  std::vector<float> a32((size_t)d * d), t32((size_t)d * d);
  for (int i = 0; i < d; ++i)
    for (int j = 0; j < d; ++j) {
      t[(size_t)j * d + i] = a[(size_t)i * d + j];
      a32[(size_t)i * d + j] = (float)a[(size_t)i * d + j];
      t32[(size_t)j * d + i] = (float)a[(size_t)i * d + j];
    }
  int rc;
  if ((rc = upload(dev, a)) != TQ_OK) return rc;
  if ((rc = upload(dev_t, t)) != TQ_OK) return rc;
  if (dev32 && (rc = upload(dev32, a32)) != TQ_OK) return rc;
  if (dev32_t && (rc = upload(dev32_t, t32)) != TQ_OK) return rc;
  return TQ_OK;
}

extern "C" int tq_quantizer_destroy(tq_quantizer* q) {
  if (!q) return TQ_OK;
  void* ptrs[] = {q->rot, q->rot_t, q->s, q->s_t, q->cent64, q->bnd64, q->rot32, q->rot32_t, q->s32, q->s32_t};
  for (void* p : ptrs)
    if (p) cudaFree(p);
  free(q);
  return TQ_OK;
}

extern "C" int tq_quantizer_create(const tq_quantizer_desc* desc, tq_quantizer** out) {
  TQ_REQUIRE(desc && out, TQ_ERR_INVALID, "tq_quantizer_create: null argument");
  *out = nullptr;
  TQ_REQUIRE(desc->bits >= 1 && desc->bits <= 4, TQ_ERR_INVALID, "bits must be 1..4, got %d", desc->bits);
  TQ_REQUIRE(desc->centroids, TQ_ERR_INVALID, "centroids missing");
  TQ_REQUIRE(desc->rotation == TQ_ROT_DENSE || desc->rotation == TQ_ROT_WHT, TQ_ERR_INVALID,
             "rotation kind %d unknown", desc->rotation);
  const int nc = 1 << desc->bits;
  for (int i = 1; i < nc; ++i)
    TQ_REQUIRE(desc->centroids[i] > desc->centroids[i - 1], TQ_ERR_INVALID, "centroids must be strictly increasing");
  if (desc->rotation == TQ_ROT_WHT) {
    TQ_REQUIRE(desc->d == TQ_D, TQ_ERR_UNSUPPORTED, "WHT mode is built for d == 128, got d = %d", desc->d);
    TQ_REQUIRE(desc->signs1 && desc->signs2, TQ_ERR_INVALID, "WHT mode needs signs1 and signs2");
    TQ_REQUIRE(is_pm1(desc->signs1, TQ_D) && is_pm1(desc->signs2, TQ_D), TQ_ERR_INVALID, "signs must be +-1");
    if (desc->qjl) {
      TQ_REQUIRE(desc->qjl_signs1 && desc->qjl_signs2, TQ_ERR_INVALID, "WHT mode QJL needs qjl_signs1/2");
      TQ_REQUIRE(is_pm1(desc->qjl_signs1, TQ_D) && is_pm1(desc->qjl_signs2, TQ_D), TQ_ERR_INVALID,
                 "qjl signs must be +-1");
    }
  } else {
    TQ_REQUIRE(desc->d >= 1 && desc->d <= 1024, TQ_ERR_UNSUPPORTED, "dense mode supports d in 1..1024, got %d", desc->d);
    TQ_REQUIRE(desc->rot || desc->qjl, TQ_ERR_INVALID, "dense mode needs rot (or only a QJL matrix)");
    if (desc->qjl) TQ_REQUIRE(desc->qjl_s, TQ_ERR_INVALID, "dense mode QJL needs qjl_s");
  }
  tq_quantizer* q = (tq_quantizer*)calloc(1, sizeof(tq_quantizer));
  TQ_REQUIRE(q, TQ_ERR_INVALID, "out of host memory");
  q->d = desc->d;
  q->bits = desc->bits;
  q->rotation = desc->rotation;
  q->norm_correction = desc->norm_correction ? 1 : 0;
  q->qjl = desc->qjl ? 1 : 0;
  cudaError_t e = cudaGetDevice(&q->device);
  if (e != cudaSuccess) {
    free(q);
    return tq_cuda_fail(e, "cudaGetDevice");
  }
  std::vector<double> c(desc->centroids, desc->centroids + nc), b(nc - 1);
  for (int i = 0; i < nc - 1; ++i) b[i] = (c[i] + c[i + 1]) / 2.0;  // turboquant/codebook.py:133
  for (int i = 0; i < nc; ++i) q->host_cent[i] = c[i];

  TqFast& f = q->fast;
  memset(&f, 0, sizeof(f));
  f.bits = desc->bits;
  f.norm_correction = q->norm_correction;
  f.has_qjl = q->qjl;
  for (int i = 0; i < nc; ++i) f.cent[i] = (float)c[i];
  for (int i = 0; i < nc - 1; ++i) f.bnd[i] = (float)b[i];
  // symmetric codebook: positive boundaries mirror negative ones, centre boundary is (almost) zero
  bool sym = fabs(b[nc / 2 - 1]) < 1e-12;
  for (int i = 0; i < nc; ++i) sym = sym && (f.cent[i] == -f.cent[nc - 1 - i]);
  for (int i = 0; i < nc - 1; ++i)
    if (i != nc / 2 - 1) sym = sym && (f.bnd[i] == -f.bnd[nc - 2 - i]);
  f.symmetric = sym ? 1 : 0;
  // The attention kernels feed centroids to the tensor cores as fp16.  A common factor alpha in
  // [1, 2) is picked so that alpha * c_i all round to fp16 with the smallest worst relative error
  // (the factor is divided out of the query / output once), instead of taking alpha = 1.
  {
    double best = 1e30;
    float best_a = 1.0f;
    for (int i = 0; i < 65536; ++i) {
      const float a = 1.0f + (float)i / 65536.0f;
      double worst = 0.0;
      for (int k = 0; k < nc; ++k) {
        const double want = (double)a * c[k];
        const double got = (double)__half2float(__float2half_rn((float)want));
        const double rel = want != 0.0 ? fabs(got / want - 1.0) : 0.0;
        if (rel > worst) worst = rel;
      }
      if (worst < best) {
        best = worst;
        best_a = a;
      }
    }
    f.lut_alpha = best_a;
    for (int k = 0; k < nc; ++k) {
      const __half h = __float2half_rn((float)((double)best_a * c[k]));
      f.cent16[k] = *reinterpret_cast<const uint16_t*>(&h);
    }
  }

  int rc = TQ_OK;
  if (desc->rotation == TQ_ROT_WHT) {
    sign_bits(desc->signs1, f.s1);
    sign_bits(desc->signs2, f.s2);
    if (desc->qjl) {
      sign_bits(desc->qjl_signs1, f.j1);
      sign_bits(desc->qjl_signs2, f.j2);
    }
  } else {
    if (desc->rot) rc = upload_matrix(desc->rot, q->d, &q->rot, &q->rot_t, &q->rot32, &q->rot32_t);
    if (rc == TQ_OK && desc->qjl) rc = upload_matrix(desc->qjl_s, q->d, &q->s, &q->s_t, &q->s32, &q->s32_t);
  }
  if (rc == TQ_OK) rc = upload(&q->cent64, c);
  if (rc == TQ_OK) rc = upload(&q->bnd64, b);
  if (rc != TQ_OK) {
    tq_quantizer_destroy(q);
    return rc;
  }
  *out = q;
  return TQ_OK;
}

// ------------------------------------------------------------------------------------------
static int fmt_idx_bits(int fmt) {
  switch (fmt) {
    case TQ_FMT_TURBO2: return 2;
    case TQ_FMT_TURBO3: return 3;
    case TQ_FMT_TURBO4: return 4;
    case TQ_FMT_PROD2: return 1;
    case TQ_FMT_PROD3: return 2;
    case TQ_FMT_PROD4: return 3;
    default: return -1;
  }
}

static inline int32_t up128(int32_t v) { return (v + 127) & ~127; }

extern "C" int tq_cache_layout_init(tq_cache_layout* L, int32_t d, int32_t page_tokens, int32_t num_kv_heads,
                                    int32_t k_format, int32_t v_format) {
  TQ_REQUIRE(L, TQ_ERR_INVALID, "layout is null");
  TQ_REQUIRE(d == TQ_D, TQ_ERR_UNSUPPORTED, "the paged cache is built for d == 128, got %d", d);
  TQ_REQUIRE(page_tokens >= 32 && page_tokens <= 256 && page_tokens % 32 == 0, TQ_ERR_INVALID,
             "page_tokens must be a multiple of 32 in 32..256, got %d", page_tokens);
  TQ_REQUIRE(num_kv_heads >= 1, TQ_ERR_INVALID, "num_kv_heads must be >= 1");
  const bool k_q8 = k_format == TQ_FMT_Q8_0, v_q8 = v_format == TQ_FMT_Q8_0;
  TQ_REQUIRE(k_q8 || fmt_idx_bits(k_format) > 0, TQ_ERR_INVALID, "unknown K format %d", k_format);
  TQ_REQUIRE(v_q8 || (fmt_idx_bits(v_format) > 0 && v_format < TQ_FMT_PROD2), TQ_ERR_INVALID,
             "V format %d must be turbo2/3/4 or q8_0", v_format);
  memset(L, 0, sizeof(*L));
  L->d = d;
  L->page_tokens = page_tokens;
  L->num_kv_heads = num_kv_heads;
  L->k_format = k_format;
  L->v_format = v_format;
  int32_t off = 0;
  L->k_idx_bytes = k_q8 ? d : d * fmt_idx_bits(k_format) / 8;
  L->k_idx_off = off;
  off = up128(off + page_tokens * L->k_idx_bytes);
  L->k_scale_off = off;
  off = up128(off + page_tokens * (k_q8 ? (d / 32) * 2 : 4));
  L->k_qjl_off = L->k_rscale_off = -1;
  if (k_format >= TQ_FMT_PROD2 && k_format <= TQ_FMT_PROD4) {
    L->k_qjl_off = off;
    off = up128(off + page_tokens * (d / 8));
    L->k_rscale_off = off;
    off = up128(off + page_tokens * 4);
  }
  L->v_idx_bytes = v_q8 ? d : d * fmt_idx_bits(v_format) / 8;
  L->v_idx_off = off;
  off = up128(off + page_tokens * L->v_idx_bytes);
  L->v_scale_off = off;
  off = up128(off + page_tokens * (v_q8 ? (d / 32) * 2 : 4));
  L->record_bytes = off;
  L->head_stride = off;
  L->page_stride = (int64_t)off * num_kv_heads;
  return TQ_OK;
}
