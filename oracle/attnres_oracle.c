/*
 * C port of the AttnRes read oracle.  TEST INFRASTRUCTURE ONLY: it is linked by
 * the tests and by the benchmark's CPU-baseline leg, never by the shipped
 * library, and the CUDA path has no fallback to it.
 *
 * Restates validation/oracle.py:5-19 of the reference (forward) and the
 * closed-form gradient its kernels implement
 * (src/attnres/_kernels/fixed_tail.py:606-864): BF16 storage, FP32 element
 * arithmetic; sums are carried in double so the result does not depend on the
 * summation order.  Rows are independent and are split over OpenMP threads.
 *
 * Parity status: pinned against tests/golden/reference_oracle.npz (vectors
 * produced by the reference oracle itself).
 *
 * Layouts (all contiguous): values [S,N,D], query [R], upstream/out [N,D],
 * dv [S,N,D], dq [R]; BF16 tensors are passed as uint16 bit patterns.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

static inline float bf16_to_float(uint16_t bits) {
  uint32_t w = (uint32_t)bits << 16;
  float f;
  memcpy(&f, &w, sizeof f);
  return f;
}

/* Round to nearest even, NaN kept quiet. */
static inline uint16_t float_to_bf16(float f) {
  uint32_t w;
  memcpy(&w, &f, sizeof w);
  if ((w & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((w >> 16) | 0x0040u);
  w += 0x7fffu + ((w >> 16) & 1u);
  return (uint16_t)(w >> 16);
}

int attnres_oracle_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* Per-row softmax over sources: fills logit[s], prob[s], inv_rms[s]. */
static void row_weights(const uint16_t* values, const float* q, int S, int64_t N, int D, int R,
                        float eps, float scale, int64_t n, float* logit, float* prob,
                        float* inv_rms) {
  const int tail0 = D - R;
  float top = -INFINITY;
  for (int s = 0; s < S; ++s) {
    const uint16_t* row = values + ((int64_t)s * N + n) * D;
    double ss = 0.0;
    for (int r = 0; r < R; ++r) {
      const float t = bf16_to_float(row[tail0 + r]);
      ss += (double)(t * t);
    }
    const float ir = 1.0f / sqrtf((float)(ss / R) + eps);
    double dot = 0.0;
    for (int r = 0; r < R; ++r) {
      const float k = bf16_to_float(row[tail0 + r]) * ir;
      dot += (double)(k * q[r]);
    }
    inv_rms[s] = ir;
    logit[s] = (float)dot * scale;
    if (logit[s] > top) top = logit[s];
  }
  double denom = 0.0;
  for (int s = 0; s < S; ++s) {
    prob[s] = expf(logit[s] - top);
    denom += prob[s];
  }
  for (int s = 0; s < S; ++s) prob[s] = (float)(prob[s] / denom);
}

void attnres_oracle_forward(const uint16_t* values, const uint16_t* query, int S, int64_t N,
                            int D, int R, float eps, float scale, uint16_t* out) {
  float* q = (float*)malloc(sizeof(float) * (size_t)R);
  for (int r = 0; r < R; ++r) q[r] = bf16_to_float(query[r]);
#pragma omp parallel
  {
    float* logit = (float*)malloc(sizeof(float) * (size_t)S * 3);
    float* prob = logit + S;
    float* inv_rms = prob + S;
    double* acc = (double*)malloc(sizeof(double) * (size_t)D);
#pragma omp for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
      row_weights(values, q, S, N, D, R, eps, scale, n, logit, prob, inv_rms);
      for (int d = 0; d < D; ++d) acc[d] = 0.0;
      for (int s = 0; s < S; ++s) {
        const uint16_t* row = values + ((int64_t)s * N + n) * D;
        for (int d = 0; d < D; ++d) acc[d] += (double)(prob[s] * bf16_to_float(row[d]));
      }
      for (int d = 0; d < D; ++d) out[n * D + d] = float_to_bf16((float)acc[d]);
    }
    free(acc);
    free(logit);
  }
  free(q);
}

void attnres_oracle_backward(const uint16_t* values, const uint16_t* query,
                             const uint16_t* upstream, int S, int64_t N, int D, int R, float eps,
                             float scale, uint16_t* dv, uint16_t* dq) {
  const int tail0 = D - R;
  float* q = (float*)malloc(sizeof(float) * (size_t)R);
  for (int r = 0; r < R; ++r) q[r] = bf16_to_float(query[r]);
  int threads = attnres_oracle_threads();
  double* dq_all = (double*)calloc((size_t)threads * (size_t)R, sizeof(double));
#pragma omp parallel
  {
#ifdef _OPENMP
    double* dq_mine = dq_all + (size_t)omp_get_thread_num() * (size_t)R;
#else
    double* dq_mine = dq_all;
#endif
    float* logit = (float*)malloc(sizeof(float) * (size_t)S * 4);
    float* prob = logit + S;
    float* inv_rms = prob + S;
    float* dw = inv_rms + S;
#pragma omp for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
      row_weights(values, q, S, N, D, R, eps, scale, n, logit, prob, inv_rms);
      const uint16_t* g = upstream + n * D;
      double delta = 0.0;
      for (int s = 0; s < S; ++s) {
        const uint16_t* row = values + ((int64_t)s * N + n) * D;
        double sum = 0.0;
        for (int d = 0; d < D; ++d) sum += (double)(bf16_to_float(row[d]) * bf16_to_float(g[d]));
        dw[s] = (float)sum;
        delta += (double)prob[s] * sum;
      }
      for (int s = 0; s < S; ++s) {
        const uint16_t* row = values + ((int64_t)s * N + n) * D;
        uint16_t* grow = dv + ((int64_t)s * N + n) * D;
        const float dz = prob[s] * (dw[s] - (float)delta);
        const float ir = inv_rms[s];
        for (int d = 0; d < tail0; ++d) grow[d] = float_to_bf16(prob[s] * bf16_to_float(g[d]));
        for (int r = 0; r < R; ++r) {
          const float k = bf16_to_float(row[tail0 + r]) * ir;
          const float direct = prob[s] * bf16_to_float(g[tail0 + r]);
          const float routed = ir * (scale * dz * q[r] - k * dz * logit[s] / (float)R);
          grow[tail0 + r] = float_to_bf16(direct + routed);
          dq_mine[r] += (double)(scale * dz * k);
        }
      }
    }
    free(logit);
  }
  for (int r = 0; r < R; ++r) {
    double total = 0.0;
    for (int t = 0; t < threads; ++t) total += dq_all[(size_t)t * (size_t)R + r];
    dq[r] = float_to_bf16((float)total);
  }
  free(dq_all);
  free(q);
}
