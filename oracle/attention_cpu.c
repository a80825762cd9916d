/* CPU oracle for the attention forward: TEST INFRASTRUCTURE, not part of the product.
 *
 * Only the tests, the smoke check and the CPU-baseline leg of the benchmark may load this
 * file's library; the product path (libflashfwd_b200.so) never does and has no CPU fallback.
 *
 * It restates, in plain C, the arithmetic of the reference's attention_forward_cpu
 * (src/main.cu:159-268 of the reference) so that it can travel to machines where the reference
 * sources are absent. The restatement is pinned: tests compare it bit for bit with the
 * reference function itself (compiled from the reference sources into oracle/_ref/) and with
 * golden vectors generated from that function.
 *
 * Arithmetic followed, step by step (reference line numbers):
 *   1. scores[i][j] = (sum_k float(half(q_ik * k_jk))) * scale: every product is rounded to
 *      fp16 (the host `__half` operator*), summed sequentially over k in fp32     (:189-197)
 *   2. ALiBi: scores[i][j] -= slope[h] * |i - j|                                     (:200-207)
 *   3. causal: j > i -> -inf (:210-218); window: |i - j| > w -> -inf when w >= 0     (:220-229)
 *   4. row max, expf(s - max), fp32 sum in j order, p = e / sum                      (:232-252)
 *   5. out[i][k] = half(sum_j float(half(p_ij) * v_jk)): normalised p rounded to fp16, every
 *      product rounded to fp16, summed sequentially over j in fp32                   (:255-263)
 *
 * Two deliberate differences, neither of which changes a single output bit for finite inputs:
 *   - masked keys are skipped instead of carried as -inf: exp(-inf - max) is +0, half(+0) * v
 *     is +-0, and adding +-0 to an fp32 sum that started at +0 leaves it unchanged;
 *   - the j loop is vectorised ACROSS keys (8 independent sums), never across k, so each
 *     sum still adds its products in the reference's k order.
 * The window here is two-sided (left, right) because the library's ABI is; the reference's
 * symmetric window is left == right == w.
 *
 * Dropout (oracle_attention_forward_dropout): the reference's CPU function has none, and the
 * reference skips its check when dropout is on (src/main.cu:103), so this part is NOT pinned by
 * the reference. It restates what the reference's kernel does to P (src/flash_forward.h:248-265:
 * after the softmax, drop with probability p, else scale by 1/(1-p)) on top of the steps above,
 * with the library's documented keep rule (Philox-4x32-10, see include/flash_forward_b200.h).
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#if defined(__AVX2__) && defined(__F16C__)
#include <immintrin.h>
#define ORACLE_SIMD 1
#else
#define ORACLE_SIMD 0
#endif

/* ---- fp16 <-> fp32, round to nearest even, IEEE subnormals (what __float2half does on the host) ---- */
static inline float h2f(uint16_t h) {
  uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1f;
  uint32_t man = h & 0x3ffu;
  uint32_t bits;
  if (exp == 0) {
    if (man == 0) {
      bits = sign;
    } else {
      int e = -1;
      do { man <<= 1; ++e; } while (!(man & 0x400u));
      bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3ffu) << 13);
    }
  } else if (exp == 31) {
    bits = sign | 0x7f800000u | (man << 13);
  } else {
    bits = sign | ((exp + 112) << 23) | (man << 13);
  }
  float f;
  memcpy(&f, &bits, 4);
  return f;
}

static inline uint16_t f2h(float f) {
  uint32_t x;
  memcpy(&x, &f, 4);
  uint32_t sign = (x >> 16) & 0x8000u;
  uint32_t ax = x & 0x7fffffffu;
  if (ax >= 0x7f800000u) return (uint16_t)(sign | 0x7c00u | ((ax > 0x7f800000u) ? 0x200u : 0));
  if (ax >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u);       /* rounds to >= 65520 -> inf */
  if (ax < 0x33000001u) return (uint16_t)sign;                    /* <= 2^-25 -> 0 (ties to even) */
  int exp = (int)(ax >> 23) - 127;
  uint32_t man = (ax & 0x7fffffu) | 0x800000u;
  int shift = (exp < -14) ? (13 + (-14 - exp)) : 13;
  uint32_t half_man = man >> shift;
  uint32_t rem = man & ((1u << shift) - 1);
  uint32_t halfway = 1u << (shift - 1);
  if (rem > halfway || (rem == halfway && (half_man & 1))) ++half_man;
  uint32_t res;
  if (exp < -14) {
    res = half_man; /* subnormal; a carry into bit 10 is the smallest normal, encoded correctly */
  } else {
    res = ((uint32_t)(exp + 15) << 10) + (half_man - 0x400u); /* carry propagates into the exponent */
  }
  return (uint16_t)(sign | res);
}

static inline float round_h(float x) { return h2f(f2h(x)); }

/* ---- one head, a list of query rows ----
 * Kt: keys transposed to fp32 [d][N]; Vf: values as fp32 [N][d]; Qh: fp16 queries [N][d].
 * scratch: N floats. out: fp16 [nrows][d] when packed != 0, else written at out[row*d]. */
typedef struct {
  const uint16_t* Qh;
  const float* Kt;
  const float* Vf;
  int N, d;
  float scale;
  int causal, wl, wr;
  float slope;
  int use_alibi;
  /* dropout: keep_thr in 0..255 (256 = off), the head's index in the flattened (batch, head) axis */
  unsigned keep_thr;
  uint64_t seed;
  unsigned bh;
} HeadCtx;

/* Philox-4x32 with 10 rounds (Salmon, Moraes, Dror, Shaw 2011), written from the published description. */
static void philox4x32_10(uint32_t k0, uint32_t k1, uint32_t c[4]) {
  for (int r = 0; r < 10; ++r) {
    const uint64_t p0 = (uint64_t)0xD2511F53u * c[0];
    const uint64_t p1 = (uint64_t)0xCD9E8D57u * c[2];
    const uint32_t n0 = (uint32_t)(p1 >> 32) ^ c[1] ^ k0;
    const uint32_t n1 = (uint32_t)p1;
    const uint32_t n2 = (uint32_t)(p0 >> 32) ^ c[3] ^ k1;
    const uint32_t n3 = (uint32_t)p0;
    c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
}

/* key column j of query row i of head bh is kept when byte (j % 16) of the block's 16 random bytes is below keep_thr */
static int dropout_keep(uint64_t seed, unsigned bh, int i, int j, unsigned keep_thr) {
  uint32_t c[4] = {(uint32_t)(j / 16), (uint32_t)i, bh, 0u};
  philox4x32_10((uint32_t)seed, (uint32_t)(seed >> 32), c);
  const unsigned t = (unsigned)(j % 16);
  const unsigned byte = (c[t / 4] >> (8 * (t % 4))) & 0xffu;
  return byte < keep_thr;
}

static void attend_row(const HeadCtx* c, int i, float* s, float* acc, uint16_t* out_row) {
  const int N = c->N, d = c->d;
  int lo = 0, hi = N - 1;
  if (c->wl >= 0 && i - c->wl > lo) lo = i - c->wl;
  if (c->wr >= 0 && i + c->wr < hi) hi = i + c->wr;
  if (c->causal && i < hi) hi = i;
  const int n = hi - lo + 1;
  if (n <= 0) { /* nothing visible: the reference would produce NaN; never reached by its masks */
    for (int k = 0; k < d; ++k) out_row[k] = f2h(NAN);
    return;
  }
  /* step 1 */
  for (int j = 0; j < n; ++j) s[j] = 0.0f;
  for (int k = 0; k < d; ++k) {
    const float q = h2f(c->Qh[(size_t)i * d + k]);
    const float* kt = c->Kt + (size_t)k * N + lo;
    int j = 0;
#if ORACLE_SIMD
    const __m256 qv = _mm256_set1_ps(q);
    for (; j + 8 <= n; j += 8) {
      __m256 prod = _mm256_mul_ps(qv, _mm256_loadu_ps(kt + j));
      prod = _mm256_cvtph_ps(_mm256_cvtps_ph(prod, _MM_FROUND_TO_NEAREST_INT | _MM_FROUND_NO_EXC));
      _mm256_storeu_ps(s + j, _mm256_add_ps(_mm256_loadu_ps(s + j), prod));
    }
#endif
    for (; j < n; ++j) s[j] += round_h(q * kt[j]);
  }
  for (int j = 0; j < n; ++j) s[j] = s[j] * c->scale;
  /* step 2 */
  if (c->use_alibi) {
    for (int j = 0; j < n; ++j) s[j] -= c->slope * (float)abs(i - (lo + j));
  }
  /* step 4 (step 3 is the [lo, hi] range) */
  float mx = -INFINITY;
  for (int j = 0; j < n; ++j) mx = fmaxf(mx, s[j]);
  float sum = 0.0f;
  for (int j = 0; j < n; ++j) {
    s[j] = expf(s[j] - mx);
    sum += s[j];
  }
  if (c->keep_thr < 256u) { /* dropout on the normalised probabilities */
    const float keep_scale = c->keep_thr ? 256.0f / (float)c->keep_thr : 0.0f;
    for (int j = 0; j < n; ++j)
      s[j] = dropout_keep(c->seed, c->bh, i, lo + j, c->keep_thr) ? round_h(s[j] / sum * keep_scale) : 0.0f;
  } else {
    for (int j = 0; j < n; ++j) s[j] = round_h(s[j] / sum);
  }
  /* step 5 */
  for (int k = 0; k < d; ++k) acc[k] = 0.0f;
  for (int j = 0; j < n; ++j) {
    const float pj = s[j];
    const float* v = c->Vf + (size_t)(lo + j) * d;
    int k = 0;
#if ORACLE_SIMD
    const __m256 pv = _mm256_set1_ps(pj);
    for (; k + 8 <= d; k += 8) {
      __m256 prod = _mm256_mul_ps(pv, _mm256_loadu_ps(v + k));
      prod = _mm256_cvtph_ps(_mm256_cvtps_ph(prod, _MM_FROUND_TO_NEAREST_INT | _MM_FROUND_NO_EXC));
      _mm256_storeu_ps(acc + k, _mm256_add_ps(_mm256_loadu_ps(acc + k), prod));
    }
#endif
    for (; k < d; ++k) acc[k] += round_h(pj * v[k]);
  }
  for (int k = 0; k < d; ++k) out_row[k] = f2h(acc[k]);
}

static int prepare_head(const uint16_t* Kh, const uint16_t* Vh, int N, int d, float** Kt, float** Vf) {
  *Kt = (float*)malloc((size_t)N * d * sizeof(float));
  *Vf = (float*)malloc((size_t)N * d * sizeof(float));
  if (!*Kt || !*Vf) { free(*Kt); free(*Vf); return -1; }
  for (int j = 0; j < N; ++j)
    for (int k = 0; k < d; ++k) {
      (*Kt)[(size_t)k * N + j] = h2f(Kh[(size_t)j * d + k]);
      (*Vf)[(size_t)j * d + k] = h2f(Vh[(size_t)j * d + k]);
    }
  return 0;
}

/* Attention of selected query rows of ONE head. q, k, v: fp16 [N][d] of that head. rows: nrows
 * indices in [0, N). out: fp16 [nrows][d]. window_left/right < 0 mean unbounded. slope is the
 * head's ALiBi slope (ignored unless use_alibi). Returns 0, or -1 when out of memory. */
int oracle_attention_rows(const uint16_t* q, const uint16_t* k, const uint16_t* v, float scale, int N, int d,
                          int causal, int window_left, int window_right, int use_alibi, float slope,
                          const int* rows, int nrows, uint16_t* out) {
  float *Kt, *Vf;
  if (prepare_head(k, v, N, d, &Kt, &Vf) != 0) return -1;
  float* s = (float*)malloc((size_t)N * sizeof(float));
  float* acc = (float*)malloc((size_t)d * sizeof(float));
  if (!s || !acc) { free(s); free(acc); free(Kt); free(Vf); return -1; }
  HeadCtx c = {q, Kt, Vf, N, d, scale, causal, window_left, window_right, slope, use_alibi, 256u, 0, 0};
  for (int r = 0; r < nrows; ++r) attend_row(&c, rows[r], s, acc, out + (size_t)r * d);
  free(s); free(acc); free(Kt); free(Vf);
  return 0;
}

/* ---- whole tensors, heads spread over threads ---- */
typedef struct {
  const uint16_t *Q, *K, *V;
  uint16_t* O;
  int BH, H, N, d;
  float scale;
  int causal, wl, wr;
  const float* slopes;
  volatile int* next;
  int err;
  unsigned keep_thr;
  uint64_t seed;
} Job;

static void* worker(void* arg) {
  Job* jb = (Job*)arg;
  const size_t hs = (size_t)jb->N * jb->d;
  float* s = (float*)malloc((size_t)jb->N * sizeof(float));
  float* acc = (float*)malloc((size_t)jb->d * sizeof(float));
  if (!s || !acc) { jb->err = -1; free(s); free(acc); return NULL; }
  for (;;) {
    int bh = __sync_fetch_and_add(jb->next, 1);
    if (bh >= jb->BH) break;
    float *Kt, *Vf;
    if (prepare_head(jb->K + bh * hs, jb->V + bh * hs, jb->N, jb->d, &Kt, &Vf) != 0) { jb->err = -1; break; }
    HeadCtx c = {jb->Q + bh * hs, Kt, Vf, jb->N, jb->d, jb->scale, jb->causal, jb->wl, jb->wr,
                 jb->slopes ? jb->slopes[bh % jb->H] : 0.0f, jb->slopes != NULL, jb->keep_thr, jb->seed, (unsigned)bh};
    for (int i = 0; i < jb->N; ++i) attend_row(&c, i, s, acc, jb->O + bh * hs + (size_t)i * jb->d);
    free(Kt); free(Vf);
  }
  free(s); free(acc);
  return NULL;
}

static int run_jobs(const uint16_t* q, const uint16_t* k, const uint16_t* v, uint16_t* out, int B, int H, int N, int d,
                    float scale, int causal, int window_left, int window_right, const float* alibi_slopes, int nthreads,
                    unsigned keep_thr, uint64_t seed) {
  if (nthreads < 1) nthreads = 1;
  if (nthreads > 256) nthreads = 256;
  volatile int next = 0;
  Job jobs[256];
  pthread_t th[256];
  for (int t = 0; t < nthreads; ++t) {
    Job j = {q, k, v, out, B * H, H, N, d, scale, causal, window_left, window_right, alibi_slopes, &next, 0, keep_thr, seed};
    jobs[t] = j;
  }
  if (nthreads == 1) {
    worker(&jobs[0]);
    return jobs[0].err;
  }
  for (int t = 0; t < nthreads; ++t) pthread_create(&th[t], NULL, worker, &jobs[t]);
  int err = 0;
  for (int t = 0; t < nthreads; ++t) { pthread_join(th[t], NULL); if (jobs[t].err) err = -1; }
  return err;
}

/* Attention of whole [B][H][N][d] fp16 tensors, one head at a time per thread.
 * alibi_slopes: H floats or NULL. Returns 0 or -1. */
int oracle_attention_forward(const uint16_t* q, const uint16_t* k, const uint16_t* v, uint16_t* out, int B, int H,
                             int N, int d, float scale, int causal, int window_left, int window_right,
                             const float* alibi_slopes, int nthreads) {
  return run_jobs(q, k, v, out, B, H, N, d, scale, causal, window_left, window_right, alibi_slopes, nthreads, 256u, 0);
}

/* The same with dropout: keep_thr = round(256 * (1 - p)) in 0..255, seed as given to the library. */
int oracle_attention_forward_dropout(const uint16_t* q, const uint16_t* k, const uint16_t* v, uint16_t* out, int B,
                                     int H, int N, int d, float scale, int causal, int window_left, int window_right,
                                     const float* alibi_slopes, int nthreads, unsigned keep_thr, uint64_t seed) {
  return run_jobs(q, k, v, out, B, H, N, d, scale, causal, window_left, window_right, alibi_slopes, nthreads, keep_thr,
                  seed);
}

/* The raw generator, for known-answer tests. ctr is read and overwritten with the output. */
void oracle_philox4x32_10(uint32_t k0, uint32_t k1, uint32_t* ctr) { philox4x32_10(k0, k1, ctr); }

/* The keep decision alone, for tests of the mask's statistics. */
int oracle_dropout_keep(uint64_t seed, unsigned bh, int row, int col, unsigned keep_thr) {
  return dropout_keep(seed, bh, row, col, keep_thr);
}

/* max and mean absolute difference of two fp16 arrays, compared in fp32 (the acceptance metric);
 * also counts NaNs in `a`. */
void oracle_abs_error(const uint16_t* a, const uint16_t* b, size_t n, double* max_abs, double* mean_abs,
                      long long* nan_count) {
  double mx = 0, sum = 0;
  long long nans = 0;
  for (size_t i = 0; i < n; ++i) {
    float x = h2f(a[i]), y = h2f(b[i]);
    if (x != x) { ++nans; continue; }
    double e = fabs((double)x - (double)y);
    if (e > mx) mx = e;
    sum += e;
  }
  *max_abs = mx;
  *mean_abs = n ? sum / (double)n : 0;
  *nan_count = nans;
}

int oracle_uses_simd(void) { return ORACLE_SIMD; }
