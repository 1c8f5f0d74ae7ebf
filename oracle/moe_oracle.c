/* Plain-C restatement of the reference's batch-1 MoE decode layer and int8 GEMV.
 * TEST AND BASELINE INFRASTRUCTURE ONLY: linked by tests/ and timed by the bench's CPU-baseline
 * leg; the product library never calls it.
 *
 * It follows the reference's CUDA kernels row by row, with one OpenMP thread per block of rows
 * standing in for a warp (paths are within the reference project):
 *   rmsnorm of x                kernels/drama.cu:180-200  (stage_x_norm)
 *   int8 row dot                kernels/drama.cu:70-102   (dot_q8: per 128-group scale)
 *   bf16 row dot                kernels/drama.cu:105-133  (dot_bf16)
 *   int4 row dot                kernels/drama.cu:137-169  (dot_q4: scale * sum(q x) + min * sum(x))
 *   router + softmax + top-k    kernels/drama.cu:371-435  (k_router_topk; ties to the lower index)
 *   gate/up + SwiGLU            kernels/drama.cu:475-518  (k_moe_gate_up_q4)
 *   down + combine              kernels/drama.cu:521-585  (k_moe_down_q4)
 * Parity of this file is pinned through tests/test_oracle_c.py against the numpy oracle, which is
 * itself pinned against outputs of the reference's PyTorch code (tests/golden).
 *
 * Build: gcc -O3 -fopenmp -shared -fPIC -o oracle/libmoe_oracle.so oracle/moe_oracle.c -lm
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#if defined(__x86_64__) && defined(__GNUC__)
#define CLONES __attribute__((target_clones("avx512f", "avx2", "default")))
#else
#define CLONES
#endif

static float half_to_float(uint16_t h) {
  const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1f, man = h & 0x3ffu, bits;
  if (exp == 0) {
    if (man == 0) {
      bits = sign;
    } else {
      int e = -1;
      do {
        ++e;
        man <<= 1;
      } while (!(man & 0x400u));
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

static float bf16_to_float(uint16_t b) {
  const uint32_t bits = (uint32_t)b << 16;
  float f;
  memcpy(&f, &bits, 4);
  return f;
}

static float silu(float x) { return x / (1.f + expf(-x)); }
static float sigmoidf_(float x) { return 1.f / (1.f + expf(-x)); }

/* xh = x * rsqrt(mean(x^2) + eps) * nw, or a copy of x when nw is NULL. */
static void rmsnorm(const float* x, const float* nw, float eps, int k, float* xh) {
  if (!nw) {
    memcpy(xh, x, (size_t)k * 4);
    return;
  }
  float ss = 0.f;
  for (int i = 0; i < k; ++i) ss += x[i] * x[i];
  const float inv = 1.f / sqrtf(ss / (float)k + eps);
  for (int i = 0; i < k; ++i) xh[i] = x[i] * inv * nw[i];
}

CLONES static float dot_q8(const int8_t* w, const uint16_t* s, const float* x, int k) {
  float acc = 0.f;
  for (int g = 0; g < k / 128; ++g) {
    float d = 0.f;
    for (int i = 0; i < 128; ++i) d += (float)w[g * 128 + i] * x[g * 128 + i];
    acc += d * half_to_float(s[g]);
  }
  return acc;
}

CLONES static float dot_bf16(const uint16_t* w, const float* x, int k) {
  float acc = 0.f;
  for (int i = 0; i < k; ++i) acc += bf16_to_float(w[i]) * x[i];
  return acc;
}

/* xs[g] = sum of x over the 64-wide group g. */
CLONES static float dot_q4(const uint8_t* q, const uint16_t* sm, const float* x, const float* xs, int k) {
  float acc = 0.f;
  for (int g = 0; g < k / 64; ++g) {
    float qx = 0.f;
    for (int i = 0; i < 32; ++i) {
      const uint8_t b = q[g * 32 + i];
      qx += (float)(b & 15) * x[g * 64 + 2 * i] + (float)(b >> 4) * x[g * 64 + 2 * i + 1];
    }
    acc += half_to_float(sm[2 * g]) * qx + half_to_float(sm[2 * g + 1]) * xs[g];
  }
  return acc;
}

static void group_sums(const float* x, int k, float* xs) {
  for (int g = 0; g < k / 64; ++g) {
    float s = 0.f;
    for (int i = 0; i < 64; ++i) s += x[g * 64 + i];
    xs[g] = s;
  }
}

/* y[n] = W[n] . rmsnorm?(x) (+ res[n]). kernels/drama.cu:222-240. */
int orc_gemv_q8(const int8_t* w, const uint16_t* s, const float* x, const float* res, float* y, int n, int k,
                const float* nw, float eps) {
  float* xh = (float*)malloc((size_t)k * 4);
  if (!xh) return -1;
  rmsnorm(x, nw, eps, k, xh);
#pragma omp parallel for schedule(static)
  for (int r = 0; r < n; ++r) {
    const float d = dot_q8(w + (size_t)r * k, s + (size_t)r * (k / 128), xh, k);
    y[r] = d + (res ? res[r] : 0.f);
  }
  free(xh);
  return 0;
}

/* Softmax over e logits, top-k (ties to the lower index), renormalised weights.
 * kernels/drama.cu:397-431. */
void orc_route(const float* logits, int e, int topk, int* idx, float* wts) {
  float m = -INFINITY, z = 0.f;
  float* p = (float*)malloc((size_t)e * 4);
  for (int i = 0; i < e; ++i) m = logits[i] > m ? logits[i] : m;
  for (int i = 0; i < e; ++i) z += (p[i] = expf(logits[i] - m));
  for (int i = 0; i < e; ++i) p[i] /= z;
  float total = 0.f;
  for (int k = 0; k < topk; ++k) {
    int bi = -1;
    float bv = -2.f;
    for (int i = 0; i < e; ++i)
      if (p[i] > bv) bv = p[i], bi = i; /* strict: the first (lowest) index wins a tie */
    idx[k] = bi;
    wts[k] = bv;
    total += bv;
    p[bi] = -1.f;
  }
  for (int k = 0; k < topk; ++k) wts[k] /= total;
  free(p);
}

typedef struct {
  const uint16_t* router; /* bf16 [e + 1, h] */
  const float* post_norm; /* f32 [h] */
  const uint8_t* gu_q;    /* [e, 2i, h/2] */
  const uint16_t* gu_sm;  /* [e, 2i, h/64, 2] */
  const uint8_t* d_q;     /* [e, h, i/2] */
  const uint16_t* d_sm;   /* [e, h, i/64, 2] */
  const int8_t* sgu_q;    /* [2i, h] */
  const uint16_t* sgu_s;  /* [2i, h/128] */
  const int8_t* sd_q;     /* [h, i] */
  const uint16_t* sd_s;   /* [h, i/128] */
  int e, h, i, topk;
  float eps;
} orc_layer;

/* One decode layer in place: x <- x + moe(rmsnorm(x)). Writes idx/wts (topk entries) when non-NULL.
 * src/engine.rs:959-1042 with x == res == y. */
int orc_moe_decode_layer(const orc_layer* L, float* x, int* idx_out, float* wts_out) {
  const int h = L->h, ii = L->i, e = L->e, topk = L->topk;
  float* xh = (float*)malloc((size_t)h * 4);
  float* xs = (float*)malloc((size_t)(h / 64) * 4);
  float* logits = (float*)malloc((size_t)(e + 1) * 4);
  float* act = (float*)malloc((size_t)(topk + 1) * ii * 4);
  float* as = (float*)malloc((size_t)topk * (ii / 64) * 4);
  int* idx = (int*)malloc((size_t)topk * 4);
  float* wts = (float*)malloc((size_t)topk * 4);
  if (!xh || !xs || !logits || !act || !as || !idx || !wts) return -1;
  rmsnorm(x, L->post_norm, L->eps, h, xh);
  group_sums(xh, h, xs);
#pragma omp parallel for schedule(static)
  for (int r = 0; r <= e; ++r) logits[r] = dot_bf16(L->router + (size_t)r * h, xh, h);
  orc_route(logits, e, topk, idx, wts);
  const float sg = sigmoidf_(logits[e]);
  /* gate/up + SwiGLU: (topk + 1) x i outputs */
#pragma omp parallel for schedule(static)
  for (int t = 0; t < (topk + 1) * ii; ++t) {
    const int k = t / ii, j = t % ii;
    float g, u;
    if (k == topk) {
      g = dot_q8(L->sgu_q + (size_t)j * h, L->sgu_s + (size_t)j * (h / 128), xh, h);
      u = dot_q8(L->sgu_q + (size_t)(ii + j) * h, L->sgu_s + (size_t)(ii + j) * (h / 128), xh, h);
    } else {
      const uint8_t* q = L->gu_q + (size_t)idx[k] * 2 * ii * (h / 2);
      const uint16_t* sm = L->gu_sm + (size_t)idx[k] * 2 * ii * (h / 64) * 2;
      g = dot_q4(q + (size_t)j * (h / 2), sm + (size_t)j * (h / 64) * 2, xh, xs, h);
      u = dot_q4(q + (size_t)(ii + j) * (h / 2), sm + (size_t)(ii + j) * (h / 64) * 2, xh, xs, h);
    }
    act[t] = silu(g) * u;
  }
  for (int k = 0; k < topk; ++k) group_sums(act + (size_t)k * ii, ii, as + (size_t)k * (ii / 64));
  /* down + combine */
#pragma omp parallel for schedule(static)
  for (int n = 0; n < h; ++n) {
    float acc = 0.f;
    for (int k = 0; k < topk; ++k) {
      const size_t row = (size_t)idx[k] * h + n;
      acc += wts[k] * dot_q4(L->d_q + row * (ii / 2), L->d_sm + row * (ii / 64) * 2, act + (size_t)k * ii,
                             as + (size_t)k * (ii / 64), ii);
    }
    const float sh = dot_q8(L->sd_q + (size_t)n * ii, L->sd_s + (size_t)n * (ii / 128), act + (size_t)topk * ii, ii);
    x[n] = x[n] + sg * sh + acc;
  }
  if (idx_out) memcpy(idx_out, idx, (size_t)topk * 4);
  if (wts_out) memcpy(wts_out, wts, (size_t)topk * 4);
  free(xh), free(xs), free(logits), free(act), free(as), free(idx), free(wts);
  return 0;
}

/* Overrides the thread count the environment chose (a launcher may pin OMP_NUM_THREADS to 1). */
void orc_set_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

int orc_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
