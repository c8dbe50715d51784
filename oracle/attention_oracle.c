/*
 * TEST INFRASTRUCTURE -- CPU oracle for the hot path. Not part of the product:
 * only tests/, __graft_entry__.smoke() and bench.py's cpu_baseline / reference
 * arm may load this file's library. The product path (libptxb200.so) never
 * calls it and has no CPU fallback.
 *
 * Plain-C restatement of the reference's CPU checkers:
 *   fab_cpu_ref   test/gpu/blackwell/flash_attention_defs.jl:967-976
 *                 inputs rounded to bf16, widened to fp32;
 *                 scores = (Q K^T) * sm_scale; rmax = rowmax(scores);
 *                 ex = exp(scores - rmax); O = (ex / rowsum(ex)) V   (fp32)
 *   fam_cpu_ref   test/gpu/ampere/flash_attention.jl:284-299
 *                 the same with scores[r,c] = -Inf for c > r (causal)
 *   _ghb_cpu_ref  test/gpu/blackwell/gemm_highperf_blackwell.jl:224-228
 *   bf16_gemm_ref test/setup.jl:225-234
 *                 inputs rounded to bf16, fp32 matrix product
 *
 * PARITY PINNING: the reference holds no golden output vectors for this path --
 * its tests compare GPU results with these CPU formulas on seeded random inputs
 * under a tolerance -- and the reference itself (Julia) cannot run where this
 * oracle was written. The oracle is therefore pinned against (a) fixtures
 * produced by an independent float64 implementation (tests/golden/), and (b) the
 * reference's exact known-answer constants (descriptor bit patterns, probe
 * values), not against reference-produced outputs: "parity unpinned" in the
 * strict sense for the floating-point outputs.
 *
 * Inputs are bf16 bit patterns (uint16_t), i.e. already quantised, row-major:
 * Q, K, V as (BH, S, D); O as fp32 (BH, S, D). A, Bt as (M,K), (N,K); C fp32 (M,N).
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#if defined(__GNUC__) && defined(__x86_64__)
#define ORACLE_CLONES __attribute__((target_clones("avx512f", "avx2,fma", "default")))
#else
#define ORACLE_CLONES
#endif

static inline float bf16_to_f32(uint16_t h) {
  uint32_t u = (uint32_t)h << 16;
  float f;
  memcpy(&f, &u, sizeof f);
  return f;
}

/* fp32 -> bf16 bits, round to nearest even (what Julia's BFloat16(x) does). */
uint16_t oracle_f32_to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, sizeof u);
  if ((u & 0x7F800000u) == 0x7F800000u && (u & 0x007FFFFFu) != 0) return (uint16_t)((u >> 16) | 0x0040u); /* NaN */
  u += 0x7FFFu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}

void oracle_round_bf16(const float* in, uint16_t* out, size_t n) {
  for (size_t i = 0; i < n; ++i) out[i] = oracle_f32_to_bf16(in[i]);
}

#define LANES 16

/* dot product of two fp32 vectors of length d (d % 16 == 0), 16 partial sums */
ORACLE_CLONES
static float dot_f32(const float* a, const float* b, int d) {
  float acc[LANES];
  for (int l = 0; l < LANES; ++l) acc[l] = 0.0f;
  for (int i = 0; i < d; i += LANES)
    for (int l = 0; l < LANES; ++l) acc[l] += a[i + l] * b[i + l];
  float s = 0.0f;
  for (int l = 0; l < LANES; ++l) s += acc[l];
  return s;
}

ORACLE_CLONES
static void axpy_f32(float* y, const float* x, float a, int d) {
  for (int i = 0; i < d; ++i) y[i] += a * x[i];
}

/* One (batch, head) slice. kf, vf: widened K and V (S x D). scratch: S floats. */
ORACLE_CLONES
static void attention_slice(const float* qf, const float* kf, const float* vf, float* o, int S, int D,
                            float sm_scale, int causal, int row_begin, int row_end, float* scratch) {
  for (int r = row_begin; r < row_end; ++r) {
    const int ncols = causal ? r + 1 : S;
    const float* q = qf + (size_t)r * D;
    float rmax = -INFINITY;
    for (int c = 0; c < ncols; ++c) {
      const float s = dot_f32(q, kf + (size_t)c * D, D) * sm_scale;
      scratch[c] = s;
      if (s > rmax) rmax = s;
    }
    float sum = 0.0f;
    for (int c = 0; c < ncols; ++c) {
      const float e = expf(scratch[c] - rmax);
      scratch[c] = e;
      sum += e;
    }
    float* orow = o + (size_t)r * D;
    for (int i = 0; i < D; ++i) orow[i] = 0.0f;
    const float inv = 1.0f / sum;
    for (int c = 0; c < ncols; ++c) axpy_f32(orow, vf + (size_t)c * D, scratch[c] * inv, D);
  }
}

/*
 * O[bh] = softmax(Q[bh] K[bh]^T * sm_scale (+ causal mask)) V[bh] for bh in
 * [0, BH). Returns 0, or -1 on a bad argument / allocation failure.
 * nthreads <= 0: use every core OpenMP offers.
 */
int oracle_attention_fwd(const uint16_t* q, const uint16_t* k, const uint16_t* v, float* o, int BH,
                         int S, int D, float sm_scale, int causal, int nthreads) {
  if (!q || !k || !v || !o || BH <= 0 || S <= 0 || D <= 0 || D % LANES != 0) return -1;
  const size_t slice = (size_t)S * D;
  int failed = 0;
#ifdef _OPENMP
  if (nthreads > 0) omp_set_num_threads(nthreads);
#endif
  for (int bh = 0; bh < BH && !failed; ++bh) {
    float* qf = (float*)malloc(slice * sizeof(float));
    float* kf = (float*)malloc(slice * sizeof(float));
    float* vf = (float*)malloc(slice * sizeof(float));
    if (!qf || !kf || !vf) { free(qf); free(kf); free(vf); return -1; }
    for (size_t i = 0; i < slice; ++i) {
      qf[i] = bf16_to_f32(q[bh * slice + i]);
      kf[i] = bf16_to_f32(k[bh * slice + i]);
      vf[i] = bf16_to_f32(v[bh * slice + i]);
    }
#pragma omp parallel
    {
      float* scratch = (float*)malloc((size_t)S * sizeof(float));
      if (!scratch) {
#pragma omp atomic write
        failed = 1;
      } else {
#pragma omp for schedule(dynamic, 16)
        for (int r0 = 0; r0 < S; r0 += 16) {
          const int r1 = r0 + 16 < S ? r0 + 16 : S;
          attention_slice(qf, kf, vf, o + bh * slice, S, D, sm_scale, causal, r0, r1, scratch);
        }
        free(scratch);
      }
    }
    free(qf); free(kf); free(vf);
  }
  return failed ? -1 : 0;
}

/* C[M,N] = A[M,K] * Bt[N,K]^T, bf16 inputs widened to fp32, fp32 accumulation. */
int oracle_gemm(const uint16_t* a, const uint16_t* bt, float* c, int M, int N, int K, int nthreads) {
  if (!a || !bt || !c || M <= 0 || N <= 0 || K <= 0 || K % LANES != 0) return -1;
  float* af = (float*)malloc((size_t)M * K * sizeof(float));
  float* bf = (float*)malloc((size_t)N * K * sizeof(float));
  if (!af || !bf) { free(af); free(bf); return -1; }
  for (size_t i = 0; i < (size_t)M * K; ++i) af[i] = bf16_to_f32(a[i]);
  for (size_t i = 0; i < (size_t)N * K; ++i) bf[i] = bf16_to_f32(bt[i]);
#ifdef _OPENMP
  if (nthreads > 0) omp_set_num_threads(nthreads);
#endif
#pragma omp parallel for schedule(static)
  for (int m = 0; m < M; ++m)
    for (int n = 0; n < N; ++n) c[(size_t)m * N + n] = dot_f32(af + (size_t)m * K, bf + (size_t)n * K, K);
  free(af); free(bf);
  return 0;
}

int oracle_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
