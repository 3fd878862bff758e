/* C restatement of the reference engine's MoE expert arithmetic.  TEST INFRASTRUCTURE ONLY:
 * it is the checker for large parity cases and the timed CPU baseline; the shipped library
 * never links or calls it.
 *
 * Decode formulas follow the reference kernels:
 *   Q4_K / Q6_K      kogarashi kernels/native.cu:26-40, 52-82
 *   NVFP4 linear     tsumuji kernels/include/decode.cuh:148-173, decode/gemv.cu:97-107,149-157
 *   NVFP4 tiled      hayate cu/glm53/math.cuh:41-49, dense.cuh:26-37,61-73
 *   block FP8        hayate cu/glm53/math.cuh:17-22,40, dense.cuh:38-41
 * The work split (rows of all selected experts concatenated, claimed in chunks by a pool of
 * threads; one dispatch for gate/up/SwiGLU and one for down) follows the reference CPU expert
 * path, hayate crates/kernels/src/cpu/glm53.rs:760-967 and crates/models/src/glm53/
 * cpu_experts.rs:142-393.  The reference has no CPU kernel for Q4_K / Q6_K or for the linear
 * NVFP4 layout; for those formats this is a restatement of the GPU decode formulas.
 * Parity of this file: pinned through tests/test_oracle_golden.py against oracle/formats.py,
 * which in turn is pinned on the reference's known-answer vectors.
 */
#include <math.h>
#include <omp.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

enum { FMT_F32 = 0, FMT_F16 = 1, FMT_Q4K = 12, FMT_Q6K = 14, FMT_BF16 = 30,
       FMT_NVFP4_LINEAR = 100, FMT_NVFP4_TILED = 101, FMT_FP8_BLOCK = 102 };

static float fp8_table[256];
static int tables_ready = 0;
static const float e2m1_table[16] = {0.f, .5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f,
                                     -0.f, -.5f, -1.f, -1.5f, -2.f, -3.f, -4.f, -6.f};

static void init_tables(void) {
  if (tables_ready) return;
  for (int b = 0; b < 256; ++b) {
    int e = (b >> 3) & 15, m = b & 7;
    float v = (e == 15 && m == 7) ? NAN : e ? ldexpf(1.f + m / 8.f, e - 7) : ldexpf((float)m, -9);
    fp8_table[b] = (b & 128) ? -v : v;
  }
  tables_ready = 1;
}

static inline float half_to_float(uint16_t h) {
  uint32_t s = (uint32_t)(h >> 15) << 31, e = (h >> 10) & 31, m = h & 1023, u;
  if (e == 0) {
    if (!m) u = s;
    else { int sh = 0; while (!(m & 1024)) { m <<= 1; ++sh; } u = s | ((uint32_t)(113 - sh) << 23) | ((m & 1023) << 13); }
  } else if (e == 31) u = s | 0x7f800000u | (m << 13);
  else u = s | ((e + 112) << 23) | (m << 13);
  float f; memcpy(&f, &u, 4); return f;
}
static inline float bf16_to_float(uint16_t b) { uint32_t u = (uint32_t)b << 16; float f; memcpy(&f, &u, 4); return f; }
static inline float bf16_round(float x) {
  uint32_t u; memcpy(&u, &x, 4); u = (u + 0x7fffu + ((u >> 16) & 1u)) & 0xffff0000u; memcpy(&x, &u, 4); return x;
}

/* One matrix [n rows, k cols].  `w` is the payload, `aux` the scale area where the format keeps
 * it apart (linear NVFP4: e4m3 [n][k/16]; block FP8: float [ceil(n/128)][ceil(k/128)]);
 * `gscale` multiplies the row sum (linear NVFP4 global scale), `rounded` rounds each decoded
 * weight to bf16 (Hayate FP8 / shared-expert path). */
typedef struct { int fmt; const uint8_t* w; const uint8_t* aux; float gscale; int n, k; int rounded; } Mat;

static void decode_row(const Mat* m, int r, float* out) {
  const int k = m->k;
  switch (m->fmt) {
    case FMT_F32: memcpy(out, m->w + (size_t)r * k * 4, (size_t)k * 4); break;
    case FMT_F16: { const uint16_t* p = (const uint16_t*)m->w + (size_t)r * k; for (int i = 0; i < k; ++i) out[i] = half_to_float(p[i]); } break;
    case FMT_BF16: { const uint16_t* p = (const uint16_t*)m->w + (size_t)r * k; for (int i = 0; i < k; ++i) out[i] = bf16_to_float(p[i]); } break;
    case FMT_Q4K: {
      const uint8_t* row = m->w + (size_t)r * (k / 256) * 144;
      for (int b = 0; b < k / 256; ++b) {
        const uint8_t* bl = row + b * 144; const uint8_t* sc = bl + 4;
        uint16_t hd, hm; memcpy(&hd, bl, 2); memcpy(&hm, bl + 2, 2);
        const float d = half_to_float(hd), dm = half_to_float(hm);
        for (int g = 0; g < 8; ++g) {
          int scale = g < 4 ? (sc[g] & 63) : ((sc[g + 4] & 15) | ((sc[g - 4] >> 6) << 4));
          int mi = g < 4 ? (sc[g + 4] & 63) : ((sc[g + 4] >> 4) | ((sc[g] >> 6) << 4));
          const float ds = d * (float)scale, mm = dm * (float)mi;
          const uint8_t* q = bl + 16 + (g / 2) * 32; const int sh = (g & 1) * 4;
          float* o = out + b * 256 + g * 32;
          for (int l = 0; l < 32; ++l) o[l] = ds * (float)((q[l] >> sh) & 15) - mm;
        }
      }
    } break;
    case FMT_Q6K: {
      const uint8_t* row = m->w + (size_t)r * (k / 256) * 210;
      for (int b = 0; b < k / 256; ++b) {
        const uint8_t* bl = row + b * 210; const int8_t* sc = (const int8_t*)(bl + 192);
        uint16_t hd; memcpy(&hd, bl + 208, 2); const float d = half_to_float(hd);
        for (int n = 0; n < 2; ++n) for (int g = 0; g < 4; ++g) for (int l = 0; l < 32; ++l) {
          int q = ((bl[n * 64 + l + (g & 1) * 32] >> ((g / 2) * 4)) & 15) | (((bl[128 + n * 32 + l] >> (g * 2)) & 3) << 4);
          out[b * 256 + n * 128 + g * 32 + l] = (d * (float)sc[n * 8 + l / 16 + g * 2]) * (float)(q - 32);
        }
      }
    } break;
    case FMT_NVFP4_LINEAR: {
      const uint8_t* c = m->w + (size_t)r * (k / 2); const uint8_t* s = m->aux + (size_t)r * (k / 16);
      for (int i = 0; i < k; i += 2) {
        const float sf = fp8_table[s[i / 16]];
        out[i] = e2m1_table[c[i / 2] & 15] * sf; out[i + 1] = e2m1_table[c[i / 2] >> 4] * sf;
      }
    } break;
    case FMT_NVFP4_TILED: {
      const int n = m->n, cols = (k / 16 + 3) / 4 * 4;
      const uint8_t* scales = m->w + (size_t)n * k / 2;
      float global; memcpy(&global, scales + (size_t)((n + 127) / 128 * 128) * cols, 4);
      const uint8_t* c = m->w + (size_t)r * (k / 2);
      for (int sc = 0; sc < k / 16; ++sc) {
        size_t at = ((size_t)(r / 128) * (cols / 4) + sc / 4) * 512 + (r % 32) * 16 + (r % 128 / 32) * 4 + sc % 4;
        const float mult = fp8_table[scales[at]] * global;
        for (int i = 0; i < 16; i += 2) {
          float a = e2m1_table[c[sc * 8 + i / 2] & 15] * mult, b = e2m1_table[c[sc * 8 + i / 2] >> 4] * mult;
          out[sc * 16 + i] = m->rounded ? bf16_round(a) : a; out[sc * 16 + i + 1] = m->rounded ? bf16_round(b) : b;
        }
      }
    } break;
    case FMT_FP8_BLOCK: {
      const float* s = (const float*)m->aux + (size_t)(r / 128) * ((k + 127) / 128);
      const uint8_t* p = m->w + (size_t)r * k;
      for (int i = 0; i < k; ++i) { float v = fp8_table[p[i]] * s[i / 128]; out[i] = m->rounded ? bf16_round(v) : v; }
    } break;
    default: memset(out, 0, (size_t)k * 4);
  }
}

/* ---- AVX2 + FMA row products for the two GGUF formats of the decode benchmark -------------------------------------
 * The timed CPU baseline uses them when the host has AVX2 and FMA (the reference's CPU expert pool is AVX2 code on
 * pinned threads: engines/hayate/crates/kernels/src/cpu_experts.rs:73-78); the parity checks keep the scalar loops
 * above.  A row is multiplied while it is decoded: per 32-column sub-block sum(q x) and sum(x) in eight float lanes,
 * then ds * sum(q x) - dmin m * sum(x) (Q4_K) or d sc * sum((q - 32) x) (Q6_K) in float32. */
#include <immintrin.h>
static int simd_enabled = 0;
void cpu_set_simd(int on) { simd_enabled = on && __builtin_cpu_supports("avx2") && __builtin_cpu_supports("fma"); }
int cpu_simd(void) { return simd_enabled; }

__attribute__((target("avx2,fma"))) static inline float hsum8(__m256 v) {
  __m128 lo = _mm256_castps256_ps128(v), hi = _mm256_extractf128_ps(v, 1);
  lo = _mm_add_ps(lo, hi);
  lo = _mm_add_ps(lo, _mm_movehl_ps(lo, lo));
  lo = _mm_add_ss(lo, _mm_shuffle_ps(lo, lo, 1));
  return _mm_cvtss_f32(lo);
}
__attribute__((target("avx2,fma"))) static float q4k_row_dot_avx2(const uint8_t* row, const float* x, int k) {
  float total = 0.f;
  const __m256i mask = _mm256_set1_epi32(15);
  for (int b = 0; b < k / 256; ++b) {
    const uint8_t* bl = row + b * 144; const uint8_t* sc = bl + 4;
    uint16_t hd, hm; memcpy(&hd, bl, 2); memcpy(&hm, bl + 2, 2);
    const float d = half_to_float(hd), dm = half_to_float(hm);
    for (int p = 0; p < 4; ++p) {                       /* 32 bytes: low nibbles sub-block 2p, high nibbles 2p + 1 */
      const uint8_t* q = bl + 16 + p * 32;
      const float* x0 = x + b * 256 + p * 64; const float* x1 = x0 + 32;
      __m256 q0 = _mm256_setzero_ps(), q1 = _mm256_setzero_ps(), s0 = _mm256_setzero_ps(), s1 = _mm256_setzero_ps();
      for (int l = 0; l < 32; l += 8) {
        const __m256i w = _mm256_cvtepu8_epi32(_mm_loadl_epi64((const __m128i*)(q + l)));
        const __m256 lo = _mm256_cvtepi32_ps(_mm256_and_si256(w, mask)), hi = _mm256_cvtepi32_ps(_mm256_srli_epi32(w, 4));
        const __m256 a = _mm256_loadu_ps(x0 + l), c = _mm256_loadu_ps(x1 + l);
        q0 = _mm256_fmadd_ps(lo, a, q0); s0 = _mm256_add_ps(s0, a);
        q1 = _mm256_fmadd_ps(hi, c, q1); s1 = _mm256_add_ps(s1, c);
      }
      for (int h = 0; h < 2; ++h) {
        const int g = 2 * p + h;
        const int scale = g < 4 ? (sc[g] & 63) : ((sc[g + 4] & 15) | ((sc[g - 4] >> 6) << 4));
        const int mi = g < 4 ? (sc[g + 4] & 63) : ((sc[g + 4] >> 4) | ((sc[g] >> 6) << 4));
        total += d * (float)scale * hsum8(h ? q1 : q0) - dm * (float)mi * hsum8(h ? s1 : s0);
      }
    }
  }
  return total;
}
__attribute__((target("avx2,fma"))) static float q6k_row_dot_avx2(const uint8_t* row, const float* x, int k) {
  float total = 0.f;
  const __m256i m4 = _mm256_set1_epi32(15), m2 = _mm256_set1_epi32(3), off = _mm256_set1_epi32(32);
  for (int b = 0; b < k / 256; ++b) {
    const uint8_t* bl = row + b * 210; const int8_t* sc = (const int8_t*)(bl + 192);
    uint16_t hd; memcpy(&hd, bl + 208, 2); const float d = half_to_float(hd);
    for (int n = 0; n < 2; ++n)
      for (int g = 0; g < 4; ++g)
        for (int half = 0; half < 2; ++half) {          /* 16 columns = one scale */
          const uint8_t* ql = bl + n * 64 + (g & 1) * 32 + half * 16; const uint8_t* qh = bl + 128 + n * 32 + half * 16;
          const float* xs = x + b * 256 + n * 128 + g * 32 + half * 16;
          __m256 acc = _mm256_setzero_ps();
          for (int l = 0; l < 16; l += 8) {
            __m256i lo = _mm256_cvtepu8_epi32(_mm_loadl_epi64((const __m128i*)(ql + l)));
            __m256i hi = _mm256_cvtepu8_epi32(_mm_loadl_epi64((const __m128i*)(qh + l)));
            lo = _mm256_and_si256(_mm256_srli_epi32(lo, (g / 2) * 4), m4);
            hi = _mm256_slli_epi32(_mm256_and_si256(_mm256_srli_epi32(hi, g * 2), m2), 4);
            const __m256 qv = _mm256_cvtepi32_ps(_mm256_sub_epi32(_mm256_or_si256(lo, hi), off));
            acc = _mm256_fmadd_ps(qv, _mm256_loadu_ps(xs + l), acc);
          }
          total += d * (float)sc[n * 8 + half + g * 2] * hsum8(acc);
        }
  }
  return total;
}
/* one row of a quantized matrix times one activation row, through the AVX2 path when it is on and has the format */
static int simd_row_dot(const Mat* m, int r, const float* x, float* out) {
  if (!simd_enabled) return 0;
  if (m->fmt == FMT_Q4K) { *out = q4k_row_dot_avx2(m->w + (size_t)r * (m->k / 256) * 144, x, m->k); return 1; }
  if (m->fmt == FMT_Q6K) { *out = q6k_row_dot_avx2(m->w + (size_t)r * (m->k / 256) * 210, x, m->k); return 1; }
  return 0;
}

/* dot of a decoded row with ntok activation rows; float partial sums in 16 lanes (vectorisable)
 * or double when f64 is set. */
static void row_dots(const float* w, const float* x, int k, int ntok, int ldx, double* out, int f64) {
  for (int t = 0; t < ntok; ++t) {
    const float* xt = x + (size_t)t * ldx;
    if (f64) { double s = 0; for (int i = 0; i < k; ++i) s += (double)w[i] * (double)xt[i]; out[t] = s; }
    else {
      float acc[16] = {0};
      for (int i = 0; i < k; i += 16) for (int j = 0; j < 16; ++j) acc[j] += w[i + j] * xt[i + j];
      float s = 0; for (int j = 0; j < 16; ++j) s += acc[j];
      out[t] = s;
    }
  }
}

/* y[t][r] = gscale * sum_k W[r][k] x[t][k]; rows are split over `threads` OpenMP threads. */
void cpu_matvec(int fmt, const void* w, const void* aux, float gscale, int rounded, int n, int k,
                const float* x, int ntok, float* y, int f64, int threads) {
  init_tables();
  Mat m = {fmt, (const uint8_t*)w, (const uint8_t*)aux, gscale, n, k, rounded};
#pragma omp parallel num_threads(threads)
  {
    float* buf = (float*)malloc((size_t)k * 4);
    double dots[64];
#pragma omp for schedule(dynamic, 64)
    for (int r = 0; r < n; ++r) {
      decode_row(&m, r, buf);
      for (int t0 = 0; t0 < ntok; t0 += 64) {
        int nt = ntok - t0 < 64 ? ntok - t0 : 64;
        row_dots(buf, x + (size_t)t0 * k, k, nt, k, dots, f64);
        for (int t = 0; t < nt; ++t) y[(size_t)(t0 + t) * n + r] = (float)(dots[t] * (double)gscale);
      }
    }
    free(buf);
  }
}

void cpu_decode(int fmt, const void* w, const void* aux, int rounded, int n, int k, float* out) {
  init_tables();
  Mat m = {fmt, (const uint8_t*)w, (const uint8_t*)aux, 1.f, n, k, rounded};
#pragma omp parallel for
  for (int r = 0; r < n; ++r) decode_row(&m, r, out + (size_t)r * k);
}

/* ---- Kogarashi-shaped whole layer for `tokens` tokens (softmax top-k router, GGML weights,
 * optional shared expert with a sigmoid gate), two dispatches like the reference CPU expert
 * path: (1) gate/up/SwiGLU rows of every (token, slot) pair and of the shared expert,
 * (2) down rows; then the combine.  Weights of an expert are decoded once per row and applied
 * to every token that selected it. */
typedef struct {
  int hidden, inter, experts, topk, tokens;
  const float* router;                       /* [E][H] */
  const uint8_t *gate, *up, *down;           /* ggml [k, rows, E] */
  int gate_ty, up_ty, down_ty;
  const uint8_t *sh_gate, *sh_up, *sh_down;  /* nullable */
  const float* sh_inp;                       /* [H] */
  const float* n;                            /* [T][H] */
  float* x;                                  /* [T][H] in/out */
  float* logits; int* ids; float* prob;      /* [T][E], [T][k], [T][k] */
} KogarashiCpu;

static size_t row_bytes(int ty, int k) { return ty == FMT_Q4K ? (size_t)k / 256 * 144 : ty == FMT_Q6K ? (size_t)k / 256 * 210 : ty == FMT_F32 ? (size_t)k * 4 : (size_t)k * 2; }

void cpu_route_softmax_topk(const float* logits, int tokens, int experts, int topk, int* ids, float* prob) {
  for (int t = 0; t < tokens; ++t) {
    float* v = (float*)malloc((size_t)experts * 4); memcpy(v, logits + (size_t)t * experts, (size_t)experts * 4);
    for (int s = 0; s < topk; ++s) {
      int best = 0; for (int e = 1; e < experts; ++e) if (v[e] > v[best]) best = e;
      ids[t * topk + s] = best; prob[t * topk + s] = v[best]; v[best] = -INFINITY;
    }
    float mx = prob[t * topk], z = 0;
    for (int s = 0; s < topk; ++s) z += expf(prob[t * topk + s] - mx);
    for (int s = 0; s < topk; ++s) prob[t * topk + s] = expf(prob[t * topk + s] - mx) / z;
    free(v);
  }
}

int cpu_kogarashi_layer(const KogarashiCpu* L, int threads) {
  init_tables();
  const int H = L->hidden, F = L->inter, E = L->experts, K = L->topk, T = L->tokens;
  const int shared = L->sh_gate != NULL;
  cpu_matvec(FMT_F32, L->router, NULL, 1.f, 0, E, H, L->n, T, L->logits, 0, threads);
  cpu_route_softmax_topk(L->logits, T, E, K, L->ids, L->prob);
  /* expert -> list of (token, slot) */
  int* count = (int*)calloc((size_t)E + 1, sizeof(int));
  for (int a = 0; a < T * K; ++a) ++count[L->ids[a]];
  int* start = (int*)malloc(((size_t)E + 1) * sizeof(int)); start[0] = 0;
  for (int e = 0; e < E; ++e) start[e + 1] = start[e] + count[e];
  int* fill = (int*)calloc((size_t)E, sizeof(int));
  int* assign = (int*)malloc((size_t)T * K * sizeof(int));
  for (int a = 0; a < T * K; ++a) { int e = L->ids[a]; assign[start[e] + fill[e]++] = a; }
  int nact = 0; int* active = (int*)malloc((size_t)E * sizeof(int));
  for (int e = 0; e < E; ++e) if (count[e]) active[nact++] = e;
  const int slots = K + shared;
  float* ff = (float*)malloc((size_t)T * slots * F * 4);      /* [T][slots][F] */
  float* dn = (float*)malloc((size_t)T * slots * H * 4);      /* [T][slots][H] */
  const size_t grow = row_bytes(L->gate_ty, H), urow = row_bytes(L->up_ty, H), drow = row_bytes(L->down_ty, F);
  const int groups = nact + shared;
  /* dispatch 1: gate/up/SwiGLU */
#pragma omp parallel num_threads(threads)
  {
    float* wg = (float*)malloc((size_t)H * 4); float* wu = (float*)malloc((size_t)H * 4);
#pragma omp for schedule(dynamic, 128) collapse(2)
    for (int gi = 0; gi < groups; ++gi) for (int r = 0; r < F; ++r) {
      const int is_sh = gi == nact; const int e = is_sh ? 0 : active[gi];
      Mat mg = {L->gate_ty, is_sh ? L->sh_gate : L->gate + (size_t)e * F * grow, NULL, 1.f, F, H, 0};
      Mat mu = {L->up_ty, is_sh ? L->sh_up : L->up + (size_t)e * F * urow, NULL, 1.f, F, H, 0};
      const int cnt = is_sh ? T : count[e];
      const int simd = simd_enabled && (mg.fmt == FMT_Q4K || mg.fmt == FMT_Q6K);
      if (!simd) { decode_row(&mg, r, wg); decode_row(&mu, r, wu); }
      for (int i = 0; i < cnt; ++i) {
        const int a = is_sh ? -1 : assign[start[e] + i]; const int t = is_sh ? i : a / K, s = is_sh ? K : a % K;
        double g, u;
        float gs, us;
        if (simd && simd_row_dot(&mg, r, L->n + (size_t)t * H, &gs) && simd_row_dot(&mu, r, L->n + (size_t)t * H, &us)) { g = gs; u = us; }
        else { row_dots(wg, L->n + (size_t)t * H, H, 1, H, &g, 0); row_dots(wu, L->n + (size_t)t * H, H, 1, H, &u, 0); }
        const float gf = (float)g; ff[((size_t)t * slots + s) * F + r] = gf * (1.f / (1.f + expf(-gf))) * (float)u;
      }
    }
    free(wg); free(wu);
  }
  /* dispatch 2: down */
#pragma omp parallel num_threads(threads)
  {
    float* wd = (float*)malloc((size_t)F * 4);
#pragma omp for schedule(dynamic, 128) collapse(2)
    for (int gi = 0; gi < groups; ++gi) for (int r = 0; r < H; ++r) {
      const int is_sh = gi == nact; const int e = is_sh ? 0 : active[gi];
      Mat md = {L->down_ty, is_sh ? L->sh_down : L->down + (size_t)e * H * drow, NULL, 1.f, H, F, 0};
      const int cnt = is_sh ? T : count[e];
      const int simd = simd_enabled && (md.fmt == FMT_Q4K || md.fmt == FMT_Q6K);
      if (!simd) decode_row(&md, r, wd);
      for (int i = 0; i < cnt; ++i) {
        const int a = is_sh ? -1 : assign[start[e] + i]; const int t = is_sh ? i : a / K, s = is_sh ? K : a % K;
        double v;
        float vs;
        if (simd && simd_row_dot(&md, r, ff + ((size_t)t * slots + s) * F, &vs)) v = vs;
        else row_dots(wd, ff + ((size_t)t * slots + s) * F, F, 1, F, &v, 0);
        dn[((size_t)t * slots + s) * H + r] = (float)v;
      }
    }
    free(wd);
  }
  /* combine (native.cu:113-117) */
  for (int t = 0; t < T; ++t) {
    float sg = 0.f;
    if (shared) { double d; row_dots(L->sh_inp, L->n + (size_t)t * H, H, 1, H, &d, 0); sg = 1.f / (1.f + expf(-(float)d)); }
    for (int i = 0; i < H; ++i) {
      float v = 0; for (int s = 0; s < K; ++s) v = fmaf(L->prob[t * K + s], dn[((size_t)t * slots + s) * H + i], v);
      L->x[(size_t)t * H + i] += v + (shared ? sg * dn[((size_t)t * slots + K) * H + i] : 0.f);
    }
  }
  free(count); free(start); free(fill); free(assign); free(active); free(ff); free(dn);
  return 0;
}

int cpu_max_threads(void) { return omp_get_max_threads(); }

/* ---- FP8 prefill layer on the CPU (timed baseline of the prefill workload) -----------------------------------------
 * Block-FP8 weights (e4m3 payload [E][n][k], float32 scale per 128 x 128 block), activations quantized to e4m3 per token
 * and 128 channels, SwiGLU product rounded to bf16 and quantized the same way, float32 rows combined in slot order:
 * the layer of oracle/layers.py `fp8_forward`, with float32 sums instead of float64.  A weight row is decoded once and
 * multiplied with every row routed to its expert.  The reference's own CPU expert pool (hayate crates/kernels/src/cpu/
 * glm53.rs, cpu_experts.rs:142-393) handles block-FP8 the same way: dequantize a row, fused multiply-adds in float32. */
typedef struct {
  int hidden, inter, experts, topk, tokens;
  const uint8_t* gate; const uint8_t* up; const uint8_t* down;       /* [E][n][k] */
  const float* gate_s; const float* up_s; const float* down_s;       /* [E][n/128][k/128] */
  const float* x; const float* logits; float* out; int* ids; float* prob;
} Fp8Cpu;

/* round to nearest even onto the e4m3 grid (saturating at 448), as a table search over the 127 positive codes */
static uint8_t e4m3_encode(float v) {
  const float a = fabsf(v) > 448.f ? 448.f : fabsf(v);
  int lo = 0, hi = 126;                                   /* fp8_table[0 .. 126] ascends from 0 to 448 */
  while (lo < hi) { const int mid = (lo + hi + 1) / 2; if (fp8_table[mid] <= a) lo = mid; else hi = mid - 1; }
  int code = lo;
  if (lo < 126) {
    const float below = a - fp8_table[lo], above = fp8_table[lo + 1] - a;
    if (above < below || (above == below && (lo & 1))) code = lo + 1;
  }
  return (uint8_t)(code | (v < 0 || (v == 0 && signbit(v)) ? 128 : 0));
}
/* rows [n][k] float32 -> their e4m3 dequantization in place (what the GEMM multiplies with) */
static void act_quantize_dequant(float* rows, int n, int k, int threads) {
#pragma omp parallel for num_threads(threads) schedule(static)
  for (int r = 0; r < n; ++r)
    for (int b = 0; b < k / 128; ++b) {
      float* g = rows + (size_t)r * k + b * 128;
      float amax = 0.f;
      for (int i = 0; i < 128; ++i) amax = fmaxf(amax, fabsf(g[i]));
      const float scale = amax == 0.f ? 1.f : amax / 448.f, inv = 1.f / scale;
      for (int i = 0; i < 128; ++i) g[i] = fp8_table[e4m3_encode(g[i] * inv)] * scale;
    }
}
static void fp8_row(const uint8_t* p, const float* s, int k, float* out) {      /* one weight row: payload and its row of block scales */
  for (int b = 0; b < k / 128; ++b) {
    const float sc = s[b];
    for (int i = 0; i < 128; ++i) out[b * 128 + i] = fp8_table[p[b * 128 + i]] * sc;
  }
}
static float dot_f32(const float* a, const float* b, int k) {
  float acc[16] = {0};
  for (int i = 0; i < k; i += 16) for (int j = 0; j < 16; ++j) acc[j] += a[i + j] * b[i + j];
  float v = 0; for (int j = 0; j < 16; ++j) v += acc[j];
  return v;
}

int cpu_fp8_layer(const Fp8Cpu* L, int threads) {
  init_tables();
  const int H = L->hidden, F = L->inter, E = L->experts, K = L->topk, T = L->tokens;
  cpu_route_softmax_topk(L->logits, T, E, K, L->ids, L->prob);
  int* count = (int*)calloc((size_t)E + 1, sizeof(int));
  for (int a = 0; a < T * K; ++a) ++count[L->ids[a]];
  int* start = (int*)malloc(((size_t)E + 1) * sizeof(int)); start[0] = 0;
  for (int e = 0; e < E; ++e) start[e + 1] = start[e] + count[e];
  int* fill = (int*)calloc((size_t)E, sizeof(int));
  int* assign = (int*)malloc((size_t)T * K * sizeof(int));
  for (int a = 0; a < T * K; ++a) { const int e = L->ids[a]; assign[start[e] + fill[e]++] = a; }
  float* xq = (float*)malloc((size_t)T * H * 4);
  memcpy(xq, L->x, (size_t)T * H * 4);
  act_quantize_dequant(xq, T, H, threads);
  float* hh = (float*)malloc((size_t)T * K * F * 4);                 /* SwiGLU products, one row per assignment */
  float* y = (float*)malloc((size_t)T * K * H * 4);                  /* down rows, one per assignment */
#pragma omp parallel num_threads(threads)
  {
    float* wg = (float*)malloc((size_t)H * 4); float* wu = (float*)malloc((size_t)H * 4);
#pragma omp for schedule(dynamic, 64) collapse(2)
    for (int e = 0; e < E; ++e) for (int r = 0; r < F; ++r) {
      if (!count[e]) continue;
      fp8_row(L->gate + ((size_t)e * F + r) * H, L->gate_s + ((size_t)e * (F / 128) + r / 128) * (H / 128), H, wg);
      fp8_row(L->up + ((size_t)e * F + r) * H, L->up_s + ((size_t)e * (F / 128) + r / 128) * (H / 128), H, wu);
      for (int i = 0; i < count[e]; ++i) {
        const int a = assign[start[e] + i];
        const float* xt = xq + (size_t)(a / K) * H;
        const float g = dot_f32(wg, xt, H), u = dot_f32(wu, xt, H);
        hh[(size_t)a * F + r] = bf16_round(g / (1.f + expf(-g)) * u);
      }
    }
    free(wg); free(wu);
  }
  act_quantize_dequant(hh, T * K, F, threads);
#pragma omp parallel num_threads(threads)
  {
    float* wd = (float*)malloc((size_t)F * 4);
#pragma omp for schedule(dynamic, 64) collapse(2)
    for (int e = 0; e < E; ++e) for (int r = 0; r < H; ++r) {
      if (!count[e]) continue;
      fp8_row(L->down + ((size_t)e * H + r) * F, L->down_s + ((size_t)e * (H / 128) + r / 128) * (F / 128), F, wd);
      for (int i = 0; i < count[e]; ++i) {
        const int a = assign[start[e] + i];
        y[(size_t)a * H + r] = dot_f32(wd, hh + (size_t)a * F, F);
      }
    }
    free(wd);
  }
#pragma omp parallel for num_threads(threads) schedule(static)
  for (int t = 0; t < T; ++t)
    for (int i = 0; i < H; ++i) {
      float v = 0.f;
      for (int s2 = 0; s2 < K; ++s2) v = fmaf(L->prob[t * K + s2], y[((size_t)t * K + s2) * H + i], v);
      L->out[(size_t)t * H + i] = v;
    }
  free(count); free(start); free(fill); free(assign); free(xq); free(hh); free(y);
  return 0;
}


/* ---- Hayate-shaped whole layer on NVFP4 images: the reference's CPU expert path --------------------------------------
 * The one CPU implementation of this path that the reference has (hayate crates/kernels/src/cpu/glm53.rs:192-260 row
 * products, :700-760 work on a range of rows, :760-967 the pool; crates/models/src/glm53/cpu_experts.rs:142-393 the two
 * dispatches).  What it does, restated: activations bf16 -> float32 once, with a second copy in which every 16 columns
 * are stored as their 8 even then their 8 odd columns (the low and the high nibbles of the 8 weight bytes); a weight row
 * is never decoded to memory: per 16-column block the nibbles go through a 16-entry table of 2 * e2m1 to integers, then
 * floats, the block's sum for every activation row (at most four share one pass over the weights) is multiplied by the
 * block's e4m3 scale, and the row total by global * 0.5; gate and up rows of one expert are produced together and leave
 * as swiglu(bf16(g), bf16(u)); rows are claimed 128 at a time by whichever thread is free.  Around it, for a whole
 * layer: the router projection and selection (cu/glm53/decode.cu:18-31), the shared expert with bf16-rounded weights
 * (decode.cu:44-45, 52) and the sum in ascending expert id with a bf16 rounding per add (decode.cu:55-59). */
typedef struct {
  int hidden, inter, experts, topk, tokens;
  float scale;
  const uint16_t* router;                    /* bf16 [E][H] */
  const float* bias;                         /* [E], selection only */
  const uint8_t* images;                     /* [E][3 * stride]: gate | up | down, NVFP4 with tiled scales */
  size_t stride;
  const uint8_t* shared;                     /* [3 * stride], nullable */
  const uint16_t* x;                         /* bf16 [T][H] */
  uint16_t* out;                             /* bf16 [T][H] */
  float* logits; int* ids; float* weights;   /* [T][E], [T][k], [T][k] */
} HayateCpu;

static inline uint16_t bf16_bits(float x) { uint32_t u; x = bf16_round(x); memcpy(&u, &x, 4); return (uint16_t)(u >> 16); }

/* every 16 columns: even columns, then odd columns */
static void split_even_odd(const float* x, float* out, int k) {
  for (int c = 0; c < k; c += 16)
    for (int i = 0; i < 8; ++i) { out[c + i] = x[c + 2 * i]; out[c + 8 + i] = x[c + 2 * i + 1]; }
}

/* one NVFP4 matrix: scales in 128 x 4 tiles behind the codes (Hayate), or `linear`: e4m3 [n][k/16] given apart (Tsumuji) */
typedef struct { const uint8_t* codes; const uint8_t* scales; float global; int n, k, cols, linear; } Nv4;
static Nv4 nv4_view(const uint8_t* image, int n, int k) {
  Nv4 m; m.codes = image; m.n = n; m.k = k; m.cols = (k / 16 + 3) / 4 * 4; m.linear = 0;
  m.scales = image + (size_t)n * k / 2;
  memcpy(&m.global, m.scales + (size_t)((n + 127) / 128 * 128) * m.cols, 4);
  return m;
}
static inline uint8_t nv4_scale(const Nv4* m, int r, int block) {
  if (m->linear) return m->scales[(size_t)r * (m->k / 16) + block];
  return m->scales[((size_t)(r / 128) * (m->cols / 4) + block / 4) * 512 + (r % 32) * 16 + (r % 128 / 32) * 4 + block % 4];
}

/* One weight row times `rows` (<= 4) activation rows given in even/odd order at stride k.  ROUNDED: every weight is
 * rounded to bf16 after its two scales are applied (the shared expert), so the scale cannot be taken out of the sum. */
__attribute__((target("avx2,fma"))) static void nv4_row_avx2(const Nv4* m, int r, const float* xs, int rows, int rounded, float* out) {
  const __m128i table = _mm_setr_epi8(0, 1, 2, 3, 4, 6, 8, 12, 0, -1, -2, -3, -4, -6, -8, -12);
  const __m128i low = _mm_set1_epi8(15);
  const uint8_t* codes = m->codes + (size_t)r * (m->k / 2);
  __m256 acc[4] = {_mm256_setzero_ps(), _mm256_setzero_ps(), _mm256_setzero_ps(), _mm256_setzero_ps()};
  for (int b = 0; b < m->k / 16; ++b) {
    const __m128i bytes = _mm_loadl_epi64((const __m128i*)(codes + b * 8));
    const __m128i even = _mm_shuffle_epi8(table, _mm_and_si128(bytes, low));
    const __m128i odd = _mm_shuffle_epi8(table, _mm_and_si128(_mm_srli_epi16(bytes, 4), low));
    __m256 we = _mm256_cvtepi32_ps(_mm256_cvtepi8_epi32(even)), wo = _mm256_cvtepi32_ps(_mm256_cvtepi8_epi32(odd));
    const float s = fp8_table[nv4_scale(m, r, b)];
    if (rounded) {
      const __m256 mult = _mm256_set1_ps(s * m->global * 0.5f);
      const __m256i half = _mm256_set1_epi32(0x7fff), one = _mm256_set1_epi32(1), keep = _mm256_set1_epi32((int)0xffff0000u);
      __m256i ue = _mm256_castps_si256(_mm256_mul_ps(we, mult)), uo = _mm256_castps_si256(_mm256_mul_ps(wo, mult));
      ue = _mm256_and_si256(_mm256_add_epi32(ue, _mm256_add_epi32(half, _mm256_and_si256(_mm256_srli_epi32(ue, 16), one))), keep);
      uo = _mm256_and_si256(_mm256_add_epi32(uo, _mm256_add_epi32(half, _mm256_and_si256(_mm256_srli_epi32(uo, 16), one))), keep);
      we = _mm256_castsi256_ps(ue); wo = _mm256_castsi256_ps(uo);
      for (int t = 0; t < rows; ++t) {
        const float* x = xs + (size_t)t * m->k + b * 16;
        acc[t] = _mm256_fmadd_ps(we, _mm256_loadu_ps(x), acc[t]);
        acc[t] = _mm256_fmadd_ps(wo, _mm256_loadu_ps(x + 8), acc[t]);
      }
    } else {
      const __m256 sv = _mm256_set1_ps(s);
      for (int t = 0; t < rows; ++t) {
        const float* x = xs + (size_t)t * m->k + b * 16;
        const __m256 block = _mm256_fmadd_ps(wo, _mm256_loadu_ps(x + 8), _mm256_mul_ps(we, _mm256_loadu_ps(x)));
        acc[t] = _mm256_fmadd_ps(sv, block, acc[t]);
      }
    }
  }
  for (int t = 0; t < rows; ++t) out[t] = hsum8(acc[t]) * (rounded ? 1.f : m->global * 0.5f);
}
/* the same sums without vector instructions */
static void nv4_row_scalar(const Nv4* m, int r, const float* xs, int rows, int rounded, float* out) {
  static const int twice[16] = {0, 1, 2, 3, 4, 6, 8, 12, 0, -1, -2, -3, -4, -6, -8, -12};
  const uint8_t* codes = m->codes + (size_t)r * (m->k / 2);
  float total[4] = {0, 0, 0, 0};
  for (int b = 0; b < m->k / 16; ++b) {
    const float s = fp8_table[nv4_scale(m, r, b)];
    for (int t = 0; t < rows; ++t) {
      const float* x = xs + (size_t)t * m->k + b * 16;
      float block = 0.f;
      for (int i = 0; i < 8; ++i) {
        float we = (float)twice[codes[b * 8 + i] & 15], wo = (float)twice[codes[b * 8 + i] >> 4];
        if (rounded) { we = bf16_round(we * (s * m->global * 0.5f)); wo = bf16_round(wo * (s * m->global * 0.5f)); }
        block += we * x[i] + wo * x[8 + i];
      }
      total[t] += rounded ? block : s * block;
    }
  }
  for (int t = 0; t < rows; ++t) out[t] = total[t] * (rounded ? 1.f : m->global * 0.5f);
}
static inline void nv4_row(const Nv4* m, int r, const float* xs, int rows, int rounded, float* out) {
  if (simd_enabled) nv4_row_avx2(m, r, xs, rows, rounded, out); else nv4_row_scalar(m, r, xs, rows, rounded, out);
}

static inline float hayate_swiglu(float gate, float up) {     /* math.cuh:31-34 on bf16 inputs */
  gate = gate < 10.f ? gate : 10.f;
  up = up < -10.f ? -10.f : up > 10.f ? 10.f : up;
  return bf16_round(bf16_round(gate / (1.f + expf(-gate))) * up);
}

/* a group of at most four activation rows that meet the same expert image */
typedef struct { const uint8_t* image; int rounded; int rows; int first; } HayateJob;   /* first: index of its rows in the row buffers */

int cpu_hayate_layer(const HayateCpu* L, int threads) {
  init_tables();
  const int H = L->hidden, F = L->inter, E = L->experts, K = L->topk, T = L->tokens;
  if (H % 16 || F % 16 || K > 32 || K > E || T < 1) return -1;
  const int per_token = K + (L->shared ? 1 : 0);
  /* activations: float32, and the even/odd copy */
  float* xf = (float*)malloc((size_t)T * H * 4);
  float* xs = (float*)malloc((size_t)T * H * 4);
  for (size_t i = 0; i < (size_t)T * H; ++i) xf[i] = bf16_to_float(L->x[i]);
  for (int t = 0; t < T; ++t) split_even_odd(xf + (size_t)t * H, xs + (size_t)t * H, H);
  /* router projection and selection */
#pragma omp parallel for num_threads(threads) schedule(static)
  for (int e = 0; e < E; ++e)
    for (int t = 0; t < T; ++t) {
      float acc[16] = {0};
      const uint16_t* w = L->router + (size_t)e * H; const float* x = xf + (size_t)t * H;
      for (int i = 0; i < H; i += 16) for (int j = 0; j < 16; ++j) acc[j] += bf16_to_float(w[i + j]) * x[i + j];
      float s = 0; for (int j = 0; j < 16; ++j) s += acc[j];
      L->logits[(size_t)t * E + e] = s;
    }
  for (int t = 0; t < T; ++t) {
    const float* lg = L->logits + (size_t)t * E;
    int* ids = L->ids + (size_t)t * K; float* w = L->weights + (size_t)t * K;
    float total = 0.f;
    for (int s = 0; s < K; ++s) {
      int best = -1; float key = 0.f, score = 0.f;
      for (int e = 0; e < E; ++e) {
        int taken = 0; for (int q = 0; q < s; ++q) taken |= ids[q] == e;
        if (taken) continue;
        const float sc = 1.f / (1.f + expf(-lg[e])), v = sc + L->bias[e];
        if (best < 0 || v > key) { best = e; key = v; score = sc; }
      }
      ids[s] = best; w[s] = score; total += score;
    }
    for (int s = 0; s < K; ++s) w[s] = w[s] / (total + 1e-20f) * L->scale;
  }
  /* jobs: per expert the (token, slot) pairs that chose it, four at a time; the shared expert takes every token */
  const int pairs = T * per_token;
  int* pair_of_row = (int*)malloc((size_t)pairs * sizeof(int));        /* row buffer index -> token * per_token + slot */
  HayateJob* jobs = (HayateJob*)malloc((size_t)pairs * sizeof(HayateJob));
  int njobs = 0, nrows = 0;
  for (int e = 0; e <= E; ++e) {
    if (e == E && !L->shared) break;
    int open = 0;
    for (int t = 0; t < T; ++t)
      for (int s = 0; s < per_token; ++s) {
        const int hit = e == E ? s == K : (s < K && L->ids[(size_t)t * K + s] == e);
        if (!hit) continue;
        if (!open) { jobs[njobs].image = e == E ? L->shared : L->images + (size_t)e * 3 * L->stride; jobs[njobs].rounded = e == E;
                     jobs[njobs].rows = 0; jobs[njobs].first = nrows; ++njobs; }
        pair_of_row[nrows++] = t * per_token + s;
        open = ++jobs[njobs - 1].rows < 4;
      }
  }
  float* in = (float*)malloc((size_t)nrows * H * 4);        /* even/odd activations of every job row */
  float* act = (float*)malloc((size_t)nrows * F * 4);
  float* acts = (float*)malloc((size_t)nrows * F * 4);
  float* y = (float*)malloc((size_t)nrows * H * 4);
  for (int r = 0; r < nrows; ++r) memcpy(in + (size_t)r * H, xs + (size_t)(pair_of_row[r] / per_token) * H, (size_t)H * 4);
  /* dispatch 1: gate and up rows together, 128 rows per claim */
  const int chunks1 = (F + 127) / 128, chunks2 = (H + 127) / 128;
#pragma omp parallel for num_threads(threads) schedule(dynamic, 1)
  for (int item = 0; item < njobs * chunks1; ++item) {
    const HayateJob* j = jobs + item / chunks1;
    const Nv4 gate = nv4_view(j->image, F, H), up = nv4_view(j->image + L->stride, F, H);
    const int r0 = item % chunks1 * 128, r1 = r0 + 128 < F ? r0 + 128 : F;
    float g[4], u[4];
    for (int r = r0; r < r1; ++r) {
      nv4_row(&gate, r, in + (size_t)j->first * H, j->rows, j->rounded, g);
      nv4_row(&up, r, in + (size_t)j->first * H, j->rows, j->rounded, u);
      for (int m = 0; m < j->rows; ++m) act[(size_t)(j->first + m) * F + r] = hayate_swiglu(bf16_round(g[m]), bf16_round(u[m]));
    }
  }
  for (int r = 0; r < nrows; ++r) split_even_odd(act + (size_t)r * F, acts + (size_t)r * F, F);
  /* dispatch 2: down rows */
#pragma omp parallel for num_threads(threads) schedule(dynamic, 1)
  for (int item = 0; item < njobs * chunks2; ++item) {
    const HayateJob* j = jobs + item / chunks2;
    const Nv4 down = nv4_view(j->image + 2 * L->stride, H, F);
    const int r0 = item % chunks2 * 128, r1 = r0 + 128 < H ? r0 + 128 : H;
    float d[4];
    for (int r = r0; r < r1; ++r) {
      nv4_row(&down, r, acts + (size_t)j->first * F, j->rows, j->rounded, d);
      for (int m = 0; m < j->rows; ++m) y[(size_t)(j->first + m) * H + r] = bf16_round(d[m]);
    }
  }
  /* sum per token: routed experts in ascending expert id, a bf16 rounding after every add, the shared expert last */
  int* row_of_pair = (int*)malloc((size_t)pairs * sizeof(int));
  for (int r = 0; r < nrows; ++r) row_of_pair[pair_of_row[r]] = r;
#pragma omp parallel for num_threads(threads) schedule(static)
  for (int t = 0; t < T; ++t) {
    int order[32];
    const int* ids = L->ids + (size_t)t * K;
    for (int i = 0; i < K; ++i) { int v = i, q = i; while (q && ids[order[q - 1]] > ids[v]) { order[q] = order[q - 1]; --q; } order[q] = v; }
    for (int c = 0; c < H; ++c) {
      float acc = 0.f;
      for (int i = 0; i < K; ++i) {
        const int s = order[i];
        acc = bf16_round(acc + bf16_round(y[(size_t)row_of_pair[t * per_token + s] * H + c] * L->weights[(size_t)t * K + s]));
      }
      if (L->shared) acc = bf16_round(acc + y[(size_t)row_of_pair[t * per_token + K] * H + c]);
      L->out[(size_t)t * H + c] = bf16_bits(acc);
    }
  }
  free(row_of_pair); free(y); free(acts); free(act); free(in); free(jobs); free(pair_of_row); free(xs); free(xf);
  return 0;
}


/* ---- Tsumuji-shaped whole layer: NVFP4 experts in the linear layout, float32 activations --------------------------
 * The reference has no CPU code for this layout; the arithmetic is that of its kernels (tsumuji kernels/decode/
 * gemv.cu:97-107, 149-157: block sums times the e4m3 scale, the row total times the matrix's global scale,
 * silu(g) * u without clamps in float32; ops.cu:148-200 the router; ops.cu:217-223 the weighted sum plus the gated
 * shared expert), run with the work split of the CPU expert path above. */
typedef struct {
  int hidden, inter, experts, topk, tokens;
  const uint16_t* router;                    /* bf16 [E + 1][H]; row E = shared gate */
  const uint8_t* blocks;                     /* [E][27/16 * F * H] */
  const float* gs;                           /* [E][3] */
  const uint16_t* shared_gu;                 /* bf16 [2F][H] */
  const uint16_t* shared_down;               /* bf16 [H][F] */
  const float* x;                            /* [T][H] */
  float* out;                                /* [T][H] */
  float* logits;                             /* [T][E + 1]; input when given_logits */
  int given_logits;
  int* ids; float* w; float* shared_gate;    /* [T][k], [T][k], [T] */
} TsumujiCpu;

static float bf16_row_dot(const uint16_t* w, const float* x, int k) {
  float acc[16] = {0};
  for (int i = 0; i < k; i += 16) for (int j = 0; j < 16; ++j) acc[j] += bf16_to_float(w[i + j]) * x[i + j];
  float s = 0; for (int j = 0; j < 16; ++j) s += acc[j];
  return s;
}

int cpu_tsumuji_layer(const TsumujiCpu* L, int threads) {
  init_tables();
  const int H = L->hidden, F = L->inter, E = L->experts, K = L->topk, T = L->tokens;
  if (H % 16 || F % 16 || K > 32 || K > E || T < 1) return -1;
  const size_t FH = (size_t)F * H, stride = FH * 27 / 16;
  if (!L->given_logits) {
#pragma omp parallel for num_threads(threads) schedule(static)
    for (int e = 0; e <= E; ++e)
      for (int t = 0; t < T; ++t) L->logits[(size_t)t * (E + 1) + e] = bf16_row_dot(L->router + (size_t)e * H, L->x + (size_t)t * H, H);
  }
#pragma omp parallel for num_threads(threads) schedule(static)
  for (int t = 0; t < T; ++t) {
    const float* lg = L->logits + (size_t)t * (E + 1);
    int* ids = L->ids + (size_t)t * K; float* w = L->w + (size_t)t * K;
    float top = lg[0]; for (int e = 1; e < E; ++e) top = lg[e] > top ? lg[e] : top;
    double all = 0; for (int e = 0; e < E; ++e) all += (double)expf(lg[e] - top);
    double chosen = 0;
    for (int s = 0; s < K; ++s) {
      int best = -1; float key = 0.f;
      for (int e = 0; e < E; ++e) {
        int taken = 0; for (int q = 0; q < s; ++q) taken |= ids[q] == e;
        if (taken) continue;
        const float v = expf(lg[e] - top);
        if (best < 0 || v > key) { best = e; key = v; }
      }
      ids[s] = best; w[s] = key / (float)all; chosen += (double)w[s];
    }
    for (int s = 0; s < K; ++s) w[s] = w[s] / (float)chosen;
    L->shared_gate[t] = 1.f / (1.f + expf(-lg[E]));
  }
  /* per expert the (token, slot) pairs that chose it, four rows per pass over the weights */
  const int pairs = T * K;
  int* pair_of_row = (int*)malloc((size_t)pairs * sizeof(int));
  int* row_of_pair = (int*)malloc((size_t)pairs * sizeof(int));
  HayateJob* jobs = (HayateJob*)malloc((size_t)pairs * sizeof(HayateJob));   /* image = the expert's block; rounded = expert id */
  int njobs = 0, nrows = 0;
  for (int e = 0; e < E; ++e) {
    int open = 0;
    for (int t = 0; t < T; ++t)
      for (int s = 0; s < K; ++s) {
        if (L->ids[(size_t)t * K + s] != e) continue;
        if (!open) { jobs[njobs].image = L->blocks + (size_t)e * stride; jobs[njobs].rounded = e; jobs[njobs].rows = 0; jobs[njobs].first = nrows; ++njobs; }
        row_of_pair[t * K + s] = nrows; pair_of_row[nrows++] = t * K + s;
        open = ++jobs[njobs - 1].rows < 4;
      }
  }
  float* in = (float*)malloc((size_t)(nrows + T) * H * 4);       /* even/odd activations: job rows, then one row per token */
  float* act = (float*)malloc((size_t)(nrows + T) * F * 4);
  float* acts = (float*)malloc((size_t)nrows * F * 4);
  float* y = (float*)malloc((size_t)(nrows + T) * H * 4);
  for (int r = 0; r < nrows; ++r) split_even_odd(L->x + (size_t)(pair_of_row[r] / K) * H, in + (size_t)r * H, H);
  const int chunks1 = (F + 127) / 128, chunks2 = (H + 127) / 128;
  /* dispatch 1: routed gate / up rows, and the shared expert's (dense bf16, natural column order) */
#pragma omp parallel for num_threads(threads) schedule(dynamic, 1)
  for (int item = 0; item < (njobs + T) * chunks1; ++item) {
    const int r0 = item % chunks1 * 128, r1 = r0 + 128 < F ? r0 + 128 : F;
    if (item / chunks1 >= njobs) {
      const int t = item / chunks1 - njobs;
      for (int r = r0; r < r1; ++r) {
        const float g = bf16_row_dot(L->shared_gu + (size_t)r * H, L->x + (size_t)t * H, H);
        const float u = bf16_row_dot(L->shared_gu + (size_t)(F + r) * H, L->x + (size_t)t * H, H);
        act[(size_t)(nrows + t) * F + r] = g / (1.f + expf(-g)) * u;
      }
      continue;
    }
    const HayateJob* j = jobs + item / chunks1;
    const float* gs = L->gs + (size_t)j->rounded * 3;
    const Nv4 gate = {j->image, j->image + FH * 3 / 2, gs[0], F, H, 0, 1}, up = {j->image + FH / 2, j->image + FH * 3 / 2 + FH / 16, gs[1], F, H, 0, 1};
    float g[4], u[4];
    for (int r = r0; r < r1; ++r) {
      nv4_row(&gate, r, in + (size_t)j->first * H, j->rows, 0, g);
      nv4_row(&up, r, in + (size_t)j->first * H, j->rows, 0, u);
      for (int m = 0; m < j->rows; ++m) act[(size_t)(j->first + m) * F + r] = g[m] / (1.f + expf(-g[m])) * u[m];
    }
  }
  for (int r = 0; r < nrows; ++r) split_even_odd(act + (size_t)r * F, acts + (size_t)r * F, F);
  /* dispatch 2: down rows */
#pragma omp parallel for num_threads(threads) schedule(dynamic, 1)
  for (int item = 0; item < (njobs + T) * chunks2; ++item) {
    const int r0 = item % chunks2 * 128, r1 = r0 + 128 < H ? r0 + 128 : H;
    if (item / chunks2 >= njobs) {
      const int t = item / chunks2 - njobs;
      for (int r = r0; r < r1; ++r) y[(size_t)(nrows + t) * H + r] = bf16_row_dot(L->shared_down + (size_t)r * F, act + (size_t)(nrows + t) * F, F);
      continue;
    }
    const HayateJob* j = jobs + item / chunks2;
    const Nv4 down = {j->image + FH, j->image + FH * 3 / 2 + FH / 8, L->gs[(size_t)j->rounded * 3 + 2], H, F, 0, 1};
    float d[4];
    for (int r = r0; r < r1; ++r) {
      nv4_row(&down, r, acts + (size_t)j->first * F, j->rows, 0, d);
      for (int m = 0; m < j->rows; ++m) y[(size_t)(j->first + m) * H + r] = d[m];
    }
  }
  /* out = sum over slots (slot order) of w * y, plus gate * shared */
#pragma omp parallel for num_threads(threads) schedule(static)
  for (int t = 0; t < T; ++t)
    for (int c = 0; c < H; ++c) {
      float acc = 0.f;
      for (int s = 0; s < K; ++s) acc = fmaf(L->w[(size_t)t * K + s], y[(size_t)row_of_pair[t * K + s] * H + c], acc);
      L->out[(size_t)t * H + c] = fmaf(L->shared_gate[t], y[(size_t)(nrows + t) * H + c], acc);
    }
  free(y); free(acts); free(act); free(in); free(jobs); free(row_of_pair); free(pair_of_row);
  return 0;
}
