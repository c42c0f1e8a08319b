/*
 * TEST INFRASTRUCTURE ONLY -- CPU oracle for the tensor-ash GEMM hot path.
 *
 * A plain-C restatement of the reference's own CPU test fixtures and of the
 * shader arithmetic that has no CPU twin.  Nothing in the product library
 * links, loads or calls this file: only the test suite, the smoke check and
 * the benchmark's CPU-baseline leg do, as the checker / reported baseline.
 *
 * Pinning: every function that has a known-answer test in the reference is
 * checked against those vectors by tests/test_oracle_golden.py (LCG range and
 * determinism, cpu_bmm 2x2 cases, f16 encodings and RNE ties, the 4x4/tile-2
 * pack layout, the C smoke-test results, split-K route answers).
 *
 * Each function cites the reference file:line it follows (paths relative to
 * the reference project root).
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define TAO_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------ */
/* Deterministic inputs: tools/test-support/src/lib.rs:9-55            */
/* ------------------------------------------------------------------ */

static inline uint64_t lcg_seed(uint64_t seed) {
  return (seed * 0x9E3779B97F4A7C15ull) | 1ull;
}
static inline uint64_t lcg_step(uint64_t s) {
  return s * 6364136223846793005ull + 1442695040888963407ull;
}

/* fill_det (lib.rs:9-18): uniform [-1, 1) from the top 24 bits. */
TAO_API void tao_fill_det(float *out, size_t n, uint64_t seed) {
  uint64_t s = lcg_seed(seed);
  for (size_t i = 0; i < n; ++i) {
    s = lcg_step(s);
    uint32_t bits = (uint32_t)(s >> 40);
    out[i] = (float)bits / (float)(1u << 24) * 2.0f - 1.0f;
  }
}

/* LcgRng (lib.rs:26-55): new / next_u64 / range_u32, state passed by pointer. */
TAO_API uint64_t tao_lcg_new(uint64_t seed) { return lcg_seed(seed); }
TAO_API uint64_t tao_lcg_next(uint64_t *state) {
  *state = lcg_step(*state);
  return *state;
}
TAO_API uint32_t tao_lcg_range_u32(uint64_t *state, uint32_t lo, uint32_t hi) {
  if (lo == hi) return lo;
  uint64_t span = (uint64_t)(hi - lo) + 1;
  return lo + (uint32_t)(tao_lcg_next(state) % span);
}

/* Normal inputs for the batched-GEMM and weight configurations.  The reference
 * has no normal generator; this one is Box-Muller over the fill_det LCG stream
 * (two draws per pair, u1 in (0,1], u2 in [0,1)), evaluated in f64 and rounded
 * once to f32, so every consumer of this library gets the same bits. */
TAO_API void tao_fill_normal(float *out, size_t n, uint64_t seed, double sigma) {
  uint64_t s = lcg_seed(seed);
  const double two_pi = 6.283185307179586476925286766559;
  for (size_t i = 0; i < n; i += 2) {
    s = lcg_step(s);
    double u1 = ((double)(uint32_t)(s >> 40) + 1.0) / 16777216.0;
    s = lcg_step(s);
    double u2 = (double)(uint32_t)(s >> 40) / 16777216.0;
    double r = sqrt(-2.0 * log(u1));
    out[i] = (float)(sigma * r * cos(two_pi * u2));
    if (i + 1 < n) out[i + 1] = (float)(sigma * r * sin(two_pi * u2));
  }
}

/* ------------------------------------------------------------------ */
/* f32 <-> f16, round-to-nearest-even: src/dtype.rs:42-112             */
/* ------------------------------------------------------------------ */

static inline uint32_t f32_bits(float v) { uint32_t b; memcpy(&b, &v, 4); return b; }
static inline float bits_f32(uint32_t b) { float v; memcpy(&v, &b, 4); return v; }

TAO_API uint16_t tao_f32_to_f16_bits(float value) {
  uint32_t bits = f32_bits(value);
  uint16_t sign = (uint16_t)((bits >> 16) & 0x8000u);
  int32_t exp = (int32_t)((bits >> 23) & 0xffu);
  uint32_t mant = bits & 0x007fffffu;
  if (exp == 0xff) return (uint16_t)(sign | 0x7c00u | (mant ? 0x0200u : 0u));
  int32_t unb = exp - 127;
  if (unb >= 16) return (uint16_t)(sign | 0x7c00u);
  if (unb >= -14) {
    uint32_t half_exp = (uint32_t)(unb + 15) << 10;
    uint32_t m10 = mant >> 13, rest = mant & 0x1fffu;
    uint32_t out = (uint32_t)sign | half_exp | m10;
    if (rest > 0x1000u || (rest == 0x1000u && (m10 & 1u))) out += 1;
    return (uint16_t)out;
  }
  if (unb >= -25) {
    uint32_t full = mant | 0x00800000u;
    uint32_t shift = (uint32_t)(-14 - unb) + 13;
    uint32_t m10 = full >> shift, rest = full & ((1u << shift) - 1u);
    uint32_t halfway = 1u << (shift - 1);
    uint32_t out = (uint32_t)sign | m10;
    if (rest > halfway || (rest == halfway && (m10 & 1u))) out += 1;
    return (uint16_t)out;
  }
  return sign;
}

/* src/dtype.rs:87-105.  IEEE binary16 decode, which is what the device's own f16 loads do.
 * On subnormal halves the reference's host decode normalises with a shift one too large
 * (leading_zeros() - 21 on a 10-bit field, dtype.rs:95-97), returning a wrong value for the
 * 1023 * 2 patterns below 2^-14; tao_f16_bits_to_f32_reference restates that behaviour
 * exactly, and this function is the IEEE decode the parity tests check tensors against. */
static float tao_decode_half(uint16_t h, uint32_t field_bias) {
  uint32_t sign = ((uint32_t)(h & 0x8000u)) << 16;
  uint32_t exp = (h >> 10) & 0x1fu, mant = h & 0x03ffu, out;
  if (exp == 0 && mant == 0) out = sign;
  else if (exp == 0) {
    uint32_t shift = (uint32_t)__builtin_clz(mant) - field_bias;
    uint32_t m = (mant << (shift + 1)) & 0x03ffu;
    uint32_t e = 127 - 15 - shift;
    out = sign | (e << 23) | (m << 13);
  } else if (exp == 0x1f) out = mant ? (sign | 0x7fc00000u | (mant << 13)) : (sign | 0x7f800000u);
  else out = sign | ((exp + 127 - 15) << 23) | (mant << 13);
  return bits_f32(out);
}

TAO_API float tao_f16_bits_to_f32(uint16_t h) { return tao_decode_half(h, 22); }

TAO_API float tao_f16_bits_to_f32_reference(uint16_t h) { return tao_decode_half(h, 21); }

TAO_API float tao_round_via_f16(float v) { return tao_f16_bits_to_f32(tao_f32_to_f16_bits(v)); }

TAO_API void tao_round_via_f16_array(float *x, size_t n) {
#pragma omp parallel for schedule(static)
  for (size_t i = 0; i < n; ++i) x[i] = tao_round_via_f16(x[i]);
}

TAO_API void tao_f32_to_f16_array(const float *x, uint16_t *out, size_t n) {
#pragma omp parallel for schedule(static)
  for (size_t i = 0; i < n; ++i) out[i] = tao_f32_to_f16_bits(x[i]);
}

/* ------------------------------------------------------------------ */
/* cpu_bmm: tools/test-support/src/lib.rs:57-135                       */
/* ------------------------------------------------------------------ */

/* Per output element: f64 accumulation over k ascending, one cast to f32,
 * then alpha * acc, then + C when accumulate.  A/B broadcast when
 * a_batched/b_batched is 0.  The loops run i,k,j over an f64 row buffer
 * (cache friendly); every element's sum is still k = 0,1,2,... in f64, so the
 * result is bit-identical to the reference's i,j,k order.  threads <= 0 uses
 * every core; threads == 1 is the reference's single-threaded form. */
TAO_API void tao_cpu_bmm(const float *a, const float *b, float *c, uint32_t batch, uint32_t m,
                         uint32_t n, uint32_t k, float alpha, int accumulate, int a_batched,
                         int b_batched, int threads) {
  size_t mk = (size_t)m * k, kn = (size_t)k * n, mn = (size_t)m * n;
  long rows = (long)batch * (long)m;
#ifdef _OPENMP
  int nt = threads > 0 ? threads : omp_get_max_threads();
#else
  int nt = 1;
  (void)threads;
#endif
#pragma omp parallel num_threads(nt)
  {
    double *acc = (double *)malloc(sizeof(double) * n);
#pragma omp for schedule(dynamic, 8)
    for (long r = 0; r < rows; ++r) {
      size_t bi = (size_t)(r / m), i = (size_t)(r % m);
      const float *ap = a + (a_batched ? bi * mk : 0) + i * k;
      const float *bp = b + (b_batched ? bi * kn : 0);
      float *cp = c + bi * mn + i * n;
      for (uint32_t j = 0; j < n; ++j) acc[j] = 0.0;
      for (uint32_t kk = 0; kk < k; ++kk) {
        double av = (double)ap[kk];
        const float *brow = bp + (size_t)kk * n;
        for (uint32_t j = 0; j < n; ++j) acc[j] += av * (double)brow[j];
      }
      for (uint32_t j = 0; j < n; ++j) {
        float scaled = alpha * (float)acc[j];
        cp[j] = accumulate ? cp[j] + scaled : scaled;
      }
    }
    free(acc);
  }
}

/* One output element of the same GEMM (f64 accumulate, f32 cast, alpha):
 * used for sampled validation at sizes where a full oracle pass is too slow,
 * following the bench-time check of tools/ml-bench/src/bench/commands.rs:225-273. */
TAO_API float tao_cpu_dot(const float *a_row, const float *b_col0, uint32_t k, uint32_t ldb,
                          float alpha) {
  double acc = 0.0;
  for (uint32_t kk = 0; kk < k; ++kk) acc += (double)a_row[kk] * (double)b_col0[(size_t)kk * ldb];
  return alpha * (float)acc;
}

/* ------------------------------------------------------------------ */
/* Fused epilogue reference: tests/correctness/epilogue.rs:9-47,       */
/* batched bias tests/common/mod.rs:63-84, order from                  */
/* shaders/matmul_epilogue_common.glsl:14-21                           */
/* ------------------------------------------------------------------ */

static double activate64(double x, int act) {
  switch (act) {
    case 1: return x > 0.0 ? x : 0.0;
    case 2: return x / (1.0 + exp(-x));
    case 3: {
      const double k0 = 0.7978845608028654;
      return 0.5 * x * (1.0 + tanh(k0 * (x + 0.044715 * x * x * x)));
    }
    default: return x;
  }
}

TAO_API double tao_activate(double x, int act) { return activate64(x, act); }

/* c holds alpha*(A@B)(+C_old) on entry.  bias may be NULL; bias_batched picks
 * [B,N] (one row per batch) over [N].  binary: 0 none, 1 x += beta*d, 2 x *= d. */
TAO_API void tao_cpu_epilogue(float *c, uint32_t batch, uint32_t m, uint32_t n, const float *bias,
                              int bias_batched, int act, int binary, const float *d, float beta) {
  size_t mn = (size_t)m * n;
#pragma omp parallel for schedule(static)
  for (long r = 0; r < (long)batch * (long)m; ++r) {
    size_t bi = (size_t)(r / m);
    float *row = c + (size_t)r * n;
    const float *drow = d ? d + (size_t)r * n : NULL;
    const float *brow = bias ? bias + (bias_batched ? bi * n : 0) : NULL;
    for (uint32_t j = 0; j < n; ++j) {
      double x = (double)row[j];
      if (brow) x += (double)brow[j];
      x = activate64(x, act);
      if (binary == 1) x += (double)beta * (double)drow[j];
      else if (binary == 2) x *= (double)drow[j];
      row[j] = (float)x;
    }
  }
  (void)mn;
}

/* tolerance(k) = 8*k*eps: tools/test-support/src/lib.rs:157-162 */
TAO_API float tao_tolerance(uint32_t k) { return 8.0f * (float)k * 1.1920928955078125e-7f; }

/* max_abs_err: lib.rs:137-155.  Non-finite difference reports +inf. */
TAO_API float tao_max_abs_err(const float *a, const float *b, size_t n, size_t *idx_out) {
  float m = 0.0f;
  size_t idx = 0;
  for (size_t i = 0; i < n; ++i) {
    float e = fabsf(a[i] - b[i]);
    if (!isfinite(e)) { if (idx_out) *idx_out = i; return INFINITY; }
    if (e > m) { m = e; idx = i; }
  }
  if (idx_out) *idx_out = idx;
  return m;
}

/* ------------------------------------------------------------------ */
/* Packed f16-weight layout: src/matmul/api.rs:317-344                 */
/* ------------------------------------------------------------------ */
TAO_API int tao_pack_f16w_row_tiles(const float *src, float *out, size_t k, size_t n,
                                    size_t tile_n) {
  if (tile_n == 0 || n % tile_n != 0) return -1;
  size_t tiles = n / tile_n;
  for (size_t t = 0; t < tiles; ++t)
    for (size_t ki = 0; ki < k; ++ki)
      memcpy(out + (t * k + ki) * tile_n, src + ki * n + t * tile_n, tile_n * sizeof(float));
  return 0;
}

/* f16w_row_tile_n: src/pipeline/routing.rs:10-41 (k16 rule -> 32, else 64). */
TAO_API uint32_t tao_f16w_row_tile_n(uint32_t k, uint32_t n) {
  int k16 = (k >= 4096) || (n <= 512) || (k >= 2048 && n <= 2048);
  if (k16 || (n % 64) != 0) return 32;
  return 64;
}

/* ------------------------------------------------------------------ */
/* Two-stage split-K in shader arithmetic (f32):                       */
/* partition shaders/matmul_splitk2_kernel.glsl:138-142, per-thread    */
/* ascending-k fma :163-190, alpha at store :197-215, ordered plane    */
/* sum shaders/matmul_f32_splitk2_reduce.comp:54-59.                   */
/* ------------------------------------------------------------------ */
TAO_API void tao_splitk_bounds(uint32_t k, uint32_t splits, uint32_t id, uint32_t *lo,
                               uint32_t *hi) {
  uint32_t per = k / splits, rem = k % splits;
  uint32_t l = id * per + (id < rem ? id : rem);
  *lo = l;
  *hi = l + per + (id < rem ? 1u : 0u);
}

/* Emulates both stages in f32: plane[s] = alpha * fma-chain over [lo,hi),
 * c = ((0 + p0) + p1) + ...  Single matrix (batch handled by the caller). */
TAO_API void tao_splitk2_f32(const float *a, const float *b, float *c, uint32_t m, uint32_t n,
                             uint32_t k, uint32_t splits, float alpha) {
#pragma omp parallel for schedule(static)
  for (long i = 0; i < (long)m; ++i) {
    for (uint32_t j = 0; j < n; ++j) {
      float total = 0.0f;
      for (uint32_t s = 0; s < splits; ++s) {
        uint32_t lo, hi;
        tao_splitk_bounds(k, splits, s, &lo, &hi);
        float acc = 0.0f;
        for (uint32_t kk = lo; kk < hi; ++kk)
          acc = fmaf(a[(size_t)i * k + kk], b[(size_t)kk * n + j], acc);
        total += (alpha == 1.0f) ? acc : alpha * acc;
      }
      c[(size_t)i * n + j] = total;
    }
  }
}

static uint64_t cdiv(uint64_t a, uint64_t b) { return a / b + (a % b != 0); }
static uint64_t sat_mul(uint64_t a, uint64_t b) {
  uint64_t r;
  return __builtin_mul_overflow(a, b, &r) ? UINT64_MAX : r;
}

/* default_num_k_splits: src/executor/splitk2.rs:94-122 (saturating tile count) */
TAO_API uint32_t tao_default_num_k_splits(uint32_t batch, uint32_t m, uint32_t n, uint32_t k,
                                          uint32_t tile_m, uint32_t tile_n) {
  if (tile_m == 0 || tile_n == 0) return 1;
  uint64_t tiles = sat_mul(sat_mul(cdiv(m, tile_m), cdiv(n, tile_n)), batch ? batch : 1);
  if (tiles == 0) return 1;
  uint64_t raw = cdiv(64, tiles);
  if (raw < 1) raw = 1;
  uint64_t max_splits = (uint64_t)k / 32;
  if (max_splits < 1) max_splits = 1;
  return (uint32_t)(raw < max_splits ? raw : max_splits);
}

/* heuristic_splits: src/executor/splitk2.rs:48-83.  Returns 0 for "none". */
TAO_API uint32_t tao_heuristic_splits(uint32_t batch, uint32_t m, uint32_t n, uint32_t k) {
  if (batch == 0 || m <= 1 || n <= 1 || k < 1024) return 0;
  int use_m128 = m >= 128 && n >= 128;
  uint32_t tile = use_m128 ? 128 : 64;
  uint64_t tiles = sat_mul(sat_mul(batch, cdiv(m, tile)), cdiv(n, tile));
  uint64_t target;
  uint32_t min_k_per_split;
  if (use_m128) {
    uint32_t min_k;
    if (tiles == 1) min_k = 1024;
    else if (tiles <= 4) min_k = 2048;
    else if (tiles <= 16) min_k = 4096;
    else return 0;
    if (k < min_k) return 0;
    target = (tiles >= 9 && k >= 8192) ? 128 : 64;
    min_k_per_split = 128;
  } else {
    if (tiles > 4) return 0;
    target = 128;
    min_k_per_split = 64;
  }
  uint64_t wanted = cdiv(target, tiles);
  uint32_t max_splits = k / min_k_per_split;
  if (use_m128 && tiles == 1 && max_splits < 16) max_splits = 16;
  static const uint32_t cand[5] = {64, 32, 16, 8, 4};
  for (int i = 0; i < 5; ++i)
    if ((uint64_t)cand[i] <= wanted && cand[i] <= max_splits) return cand[i];
  return 0;
}

/* ------------------------------------------------------------------ */
/* Row GEMV in shader arithmetic: shaders/matmul_row_bda_kernel.glsl   */
/* :252-267 (slice s walks k = s, s+KSLICES, ... with fma; slices are  */
/* summed in order 0..KSLICES-1).  Used for the bit-level GEMV claim;  */
/* the f64 cpu_bmm above stays the tolerance oracle.                   */
/* ------------------------------------------------------------------ */
TAO_API void tao_row_gemv_f32(const float *a, const float *b, float *c, uint32_t n, uint32_t k,
                              uint32_t kslices) {
#pragma omp parallel for schedule(static)
  for (long j = 0; j < (long)n; ++j) {
    float total = 0.0f;
    for (uint32_t s = 0; s < kslices; ++s) {
      float acc = 0.0f;
      for (uint32_t kk = s; kk < k; kk += kslices) acc = fmaf(a[kk], b[(size_t)kk * n + j], acc);
      total += acc;
    }
    c[j] = total;
  }
}

/* ------------------------------------------------------------------ */
/* Model-op references                                                 */
/* ------------------------------------------------------------------ */

/* RMSNorm: tests/correctness/decoder.rs:80-90 (f64 mean of squares). */
TAO_API void tao_cpu_rmsnorm(const float *x, const float *w, float *out, uint32_t rows,
                             uint32_t cols, float eps) {
  for (uint32_t r = 0; r < rows; ++r) {
    double ss = 0.0;
    for (uint32_t j = 0; j < cols; ++j) ss += (double)x[(size_t)r * cols + j] * x[(size_t)r * cols + j];
    double inv = 1.0 / sqrt(ss / cols + (double)eps);
    for (uint32_t j = 0; j < cols; ++j)
      out[(size_t)r * cols + j] = (float)((double)x[(size_t)r * cols + j] * inv * (double)w[j]);
  }
}

/* LayerNorm: include/tensor_ash.h:187-191 (population variance). */
TAO_API void tao_cpu_layernorm(const float *x, const float *w, const float *b, float *out,
                               uint32_t rows, uint32_t cols, float eps) {
  for (uint32_t r = 0; r < rows; ++r) {
    const float *xr = x + (size_t)r * cols;
    double mean = 0.0, var = 0.0;
    for (uint32_t j = 0; j < cols; ++j) mean += xr[j];
    mean /= cols;
    for (uint32_t j = 0; j < cols; ++j) var += ((double)xr[j] - mean) * ((double)xr[j] - mean);
    var /= cols;
    double inv = 1.0 / sqrt(var + (double)eps);
    for (uint32_t j = 0; j < cols; ++j)
      out[(size_t)r * cols + j] = (float)(((double)xr[j] - mean) * inv * (double)w[j] + (double)b[j]);
  }
}

/* Masked row softmax: include/tensor_ash.h:69-76,169-182; masked columns are
 * exactly 0.  mask_kind 0 full, 1 prefix, 2 causal. */
TAO_API void tao_cpu_softmax_rows(const float *x, float *out, uint32_t rows, uint32_t cols,
                                  float scale, uint32_t mask_kind, uint32_t valid_or_prefix,
                                  uint32_t rows_per_group) {
  for (uint32_t r = 0; r < rows; ++r) {
    uint32_t valid = cols;
    if (mask_kind == 1) valid = valid_or_prefix < cols ? valid_or_prefix : cols;
    else if (mask_kind == 2) {
      uint64_t v = (uint64_t)valid_or_prefix + (rows_per_group ? r % rows_per_group : 0) + 1;
      valid = v < cols ? (uint32_t)v : cols;
    }
    const float *xr = x + (size_t)r * cols;
    float *orow = out + (size_t)r * cols;
    double mx = -INFINITY, sum = 0.0;
    for (uint32_t j = 0; j < valid; ++j) { double v = (double)xr[j] * scale; if (v > mx) mx = v; }
    for (uint32_t j = 0; j < valid; ++j) sum += exp((double)xr[j] * scale - mx);
    for (uint32_t j = 0; j < cols; ++j)
      orow[j] = j < valid ? (float)(exp((double)xr[j] * scale - mx) / sum) : 0.0f;
  }
}

/* Interleaved-pair RoPE: shaders/op_rope_body.glsl:129-134; table is
 * [T_max, rot_dim/2, 2] (cos, sin); lanes >= rot_dim pass through. */
TAO_API void tao_cpu_rope(const float *x, const float *table, float *out, uint32_t tokens,
                          uint32_t heads, uint32_t head_dim, uint32_t rot_dim, uint32_t pos_base) {
  uint32_t half = rot_dim / 2;
  for (uint32_t t = 0; t < tokens; ++t)
    for (uint32_t h = 0; h < heads; ++h) {
      const float *xv = x + ((size_t)t * heads + h) * head_dim;
      float *ov = out + ((size_t)t * heads + h) * head_dim;
      const float *tab = table + (size_t)(pos_base + t) * half * 2;
      float tmp[1024];
      for (uint32_t i = 0; i < head_dim; ++i) tmp[i] = xv[i];
      for (uint32_t i = 0; i < half; ++i) {
        double x0 = tmp[2 * i], x1 = tmp[2 * i + 1];
        double c = tab[2 * i], s = tab[2 * i + 1];
        ov[2 * i] = (float)(x0 * c - x1 * s);
        ov[2 * i + 1] = (float)(x0 * s + x1 * c);
      }
      for (uint32_t i = rot_dim; i < head_dim; ++i) ov[i] = tmp[i];
    }
}

/* Argmax with "largest index wins ties": tests/correctness/token_loop.rs:15-22,
 * shaders/op_argmax_f32.comp:51-75. */
TAO_API uint32_t tao_cpu_argmax(const float *x, uint32_t n) {
  uint32_t best = 0;
  for (uint32_t i = 1; i < n; ++i)
    if (x[i] >= x[best]) best = i;
  return best;
}

/* Causal flash-attention reference: tests/correctness/flash.rs:14-62.
 * q [H, T_q, dh], kt [H_kv, dh, T_max], v [H_kv, T_max, dh], out [H, T_q, dh];
 * row i sees positions < min(kv_len, pos_base + i + 1); all-masked rows -> 0. */
TAO_API void tao_cpu_flash(const float *q, const float *kt, const float *v, float *out,
                           uint32_t heads, uint32_t kv_heads, uint32_t t_q, uint32_t dh,
                           uint32_t t_max, uint32_t kv_len, uint32_t pos_base, float scale) {
  uint32_t group = heads / kv_heads;
#pragma omp parallel for schedule(dynamic, 4)
  for (long hi = 0; hi < (long)heads * (long)t_q; ++hi) {
    uint32_t h = (uint32_t)(hi / t_q), i = (uint32_t)(hi % t_q);
    uint32_t kvh = h / group;
    uint64_t lim = (uint64_t)pos_base + i + 1;
    uint32_t valid = lim < kv_len ? (uint32_t)lim : kv_len;
    const float *qr = q + ((size_t)h * t_q + i) * dh;
    float *orow = out + ((size_t)h * t_q + i) * dh;
    if (valid == 0) { for (uint32_t d = 0; d < dh; ++d) orow[d] = 0.0f; continue; }
    double *s = (double *)malloc(sizeof(double) * valid);
    double mx = -INFINITY;
    for (uint32_t p = 0; p < valid; ++p) {
      double acc = 0.0;
      for (uint32_t d = 0; d < dh; ++d)
        acc += (double)qr[d] * (double)kt[((size_t)kvh * dh + d) * t_max + p];
      s[p] = acc * (double)scale;
      if (s[p] > mx) mx = s[p];
    }
    double sum = 0.0;
    for (uint32_t p = 0; p < valid; ++p) { s[p] = exp(s[p] - mx); sum += s[p]; }
    for (uint32_t d = 0; d < dh; ++d) {
      double acc = 0.0;
      for (uint32_t p = 0; p < valid; ++p) acc += s[p] * (double)v[((size_t)kvh * t_max + p) * dh + d];
      orow[d] = (float)(acc / sum);
    }
    free(s);
  }
}

/* Single-row GQA decode attention: tests/correctness/attn_decode.rs:16-56.
 * q [H_kv, group, dh] -> out same; attends positions [0, kv_len). */
TAO_API void tao_cpu_attn_decode(const float *q, const float *kt, const float *v, float *out,
                                 uint32_t kv_heads, uint32_t group, uint32_t dh, uint32_t t_max,
                                 uint32_t kv_len, float scale) {
  tao_cpu_flash(q, kt, v, out, kv_heads * group, kv_heads, 1, dh, t_max, kv_len,
                kv_len ? kv_len - 1 : 0, scale);
}

TAO_API int tao_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
