/* TEST INFRASTRUCTURE — CPU oracle for the cleandl_b200 kernels.  Never linked into or called by
 * the product library; only tests, the smoke check and the bench's cpu_baseline leg use it.
 *
 * Each function restates, in plain C with f64 arithmetic, the f64 reference that clean-lm's own
 * GPU integration tests compare against (the reference has no other host implementation):
 *   oracle_matmul        crates/cleandl/tests/matmul.rs:89-118
 *   oracle_rmsnorm_fwd   crates/cleandl/tests/norm.rs:97-130 (RmsNorm branch)
 *   oracle_attention     crates/cleandl/tests/attention.rs:357-514 (dense layout, no softcap)
 * oracle_rmsnorm_bwd has no counterpart in the reference (its tree holds only the call sites,
 * crates/sky-1/src/training/model/decoder.rs:599-607); it is the analytic derivative of the forward.
 *
 * PARITY UNPINNED: the reference ships no golden vectors (its tests draw inputs from Rust RNG
 * streams at run time) and cannot be compiled here (no Rust toolchain, un-vendored
 * dependencies), so this oracle is checked against an independent float64 implementation
 * (tests/golden/make_golden.py) instead of against reference outputs.
 *
 * Inputs are f32 arrays holding values already rounded to the storage type (bf16), packed
 * row-major.  Build: gcc -O3 -fopenmp -shared -fPIC cpu_ref.c -o liboracle.so -lm
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* out[b,i,j] = alpha * sum_k a[b,i,k] b[b,k,j] + beta * c[b,i,j];  bound = |alpha| sum |a b| + |beta c|. */
void oracle_matmul(const float* a, const float* b, const float* c, float alpha, float beta,
                   int64_t batch, int64_t m, int64_t k, int64_t n, float* out, float* bound) {
#pragma omp parallel
  {
    double* sum = (double*)malloc(sizeof(double) * (size_t)n);
    double* abs_ = (double*)malloc(sizeof(double) * (size_t)n);
#pragma omp for collapse(2) schedule(static)
    for (int64_t bi = 0; bi < batch; ++bi) {
      for (int64_t i = 0; i < m; ++i) {
        for (int64_t j = 0; j < n; ++j) {
          sum[j] = 0.0;
          abs_[j] = 0.0;
        }
        const float* arow = a + (bi * m + i) * k;
        for (int64_t kk = 0; kk < k; ++kk) {
          const double av = (double)arow[kk];
          const float* brow = b + (bi * k + kk) * n;
          if (bound) {
            for (int64_t j = 0; j < n; ++j) {
              const double p = av * (double)brow[j];
              sum[j] += p;
              abs_[j] += fabs(p);
            }
          } else {
            for (int64_t j = 0; j < n; ++j) sum[j] += av * (double)brow[j];
          }
        }
        for (int64_t j = 0; j < n; ++j) {
          double value = (double)alpha * sum[j];
          double bd = fabs((double)alpha) * abs_[j];
          if (c) {
            const double cv = (double)beta * (double)c[(bi * m + i) * n + j];
            value += cv;
            bd += fabs(cv);
          }
          out[(bi * m + i) * n + j] = (float)value;
          if (bound) bound[(bi * m + i) * n + j] = (float)bd;
        }
      }
    }
    free(sum);
    free(abs_);
  }
}

/* y = x * r_inv * scale + bias with r_inv = 1 / sqrt(mean(x^2) + eps), all in f64. */
void oracle_rmsnorm_fwd(const float* x, const float* scale, const float* bias, float eps,
                        int64_t rows, int64_t cols, float* y, float* r_inv) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r) {
    const float* row = x + r * cols;
    double var = 0.0;
    for (int64_t c = 0; c < cols; ++c) var += (double)row[c] * (double)row[c];
    var /= (double)cols;
    const double ri = 1.0 / sqrt(var + (double)eps);
    if (r_inv) r_inv[r] = (float)ri;
    for (int64_t c = 0; c < cols; ++c) {
      double v = (double)row[c] * ri;
      if (scale) v *= (double)scale[c];
      if (bias) v += (double)bias[c];
      y[r * cols + c] = (float)v;
    }
  }
}

/* dx = r g - r^3 x mean(g x) (+ residual),  g = dy * scale;  dscale[j] += sum_i dy x r.
 * r is recomputed from x in f64 (the device kernel is handed the forward's f32 r_inv). */
void oracle_rmsnorm_bwd(const float* x, const float* dy, const float* residual, const float* scale,
                        float eps, int64_t rows, int64_t cols, float* dx, double* dscale_accum) {
  for (int64_t r = 0; r < rows; ++r) {
    const float* xr = x + r * cols;
    const float* dr = dy + r * cols;
    double var = 0.0, dot = 0.0;
    for (int64_t c = 0; c < cols; ++c) {
      var += (double)xr[c] * (double)xr[c];
      dot += (double)dr[c] * (double)scale[c] * (double)xr[c];
    }
    var /= (double)cols;
    const double ri = 1.0 / sqrt(var + (double)eps);
    const double cm = dot / (double)cols;
    for (int64_t c = 0; c < cols; ++c) {
      const double g = (double)dr[c] * (double)scale[c];
      double v = ri * g - ri * ri * ri * (double)xr[c] * cm;
      if (residual) v += (double)residual[r * cols + c];
      dx[r * cols + c] = (float)v;
      dscale_accum[c] += (double)dr[c] * (double)xr[c] * ri;
    }
  }
}

/* Dense [B, S, H, D] attention forward (+ backward when d_out != NULL), per (batch, head) in f64.
 * Causal mask aligned to the bottom right: query i sees keys j <= i + sk - sq.  Rows with no
 * visible key give out = 0 and lse = -inf.  dk/dv accumulate over the query heads of a group. */
void oracle_attention(const float* q, const float* k, const float* v, const float* d_out,
                      int64_t batch, int64_t sq, int64_t sk, int64_t hq, int64_t hk, int64_t d,
                      float scale_f, int causal, float* out, float* lse, float* dq, float* dk,
                      float* dv) {
  const double scale = (double)scale_f;
  const int64_t group = hq / hk;
  double* dk_acc = NULL;
  double* dv_acc = NULL;
  if (d_out) {
    dk_acc = (double*)calloc((size_t)(batch * sk * hk * d), sizeof(double));
    dv_acc = (double*)calloc((size_t)(batch * sk * hk * d), sizeof(double));
  }
#pragma omp parallel
  {
    double* s = (double*)malloc(sizeof(double) * (size_t)sk);
    double* p = (double*)malloc(sizeof(double) * (size_t)sk);
    double* o = (double*)malloc(sizeof(double) * (size_t)d);
    double* dqr = (double*)malloc(sizeof(double) * (size_t)d);
    /* One (batch, kv head) per task so that dk/dv accumulation needs no atomics. */
#pragma omp for collapse(2) schedule(dynamic)
    for (int64_t b = 0; b < batch; ++b) {
      for (int64_t kh = 0; kh < hk; ++kh) {
        for (int64_t h = kh * group; h < (kh + 1) * group; ++h) {
          for (int64_t i = 0; i < sq; ++i) {
            const float* qi = q + ((b * sq + i) * hq + h) * d;
            int64_t lo = 0, hi = sk;
            if (causal) {
              const int64_t center = i + sk - sq;
              hi = center + 1 < sk ? center + 1 : sk;
              if (hi < 0) hi = 0;
            }
            if (hi <= lo) { lo = 0; hi = 0; }
            double mx = -INFINITY;
            for (int64_t j = lo; j < hi; ++j) {
              const float* kj = k + ((b * sk + j) * hk + kh) * d;
              double acc = 0.0;
              for (int64_t x = 0; x < d; ++x) acc += (double)qi[x] * (double)kj[x];
              s[j] = scale * acc;
              if (s[j] > mx) mx = s[j];
            }
            double sum = 0.0;
            for (int64_t j = lo; j < hi; ++j) sum += exp(s[j] - mx);
            const double l = (lo == hi) ? -INFINITY : mx + log(sum);
            for (int64_t x = 0; x < d; ++x) o[x] = 0.0;
            for (int64_t j = lo; j < hi; ++j) {
              p[j] = exp(s[j] - l);
              const float* vj = v + ((b * sk + j) * hk + kh) * d;
              for (int64_t x = 0; x < d; ++x) o[x] += p[j] * (double)vj[x];
            }
            float* oi = out + ((b * sq + i) * hq + h) * d;
            for (int64_t x = 0; x < d; ++x) oi[x] = (float)o[x];
            if (lse) lse[(b * hq + h) * sq + i] = (float)l;
            if (d_out) {
              const float* doi = d_out + ((b * sq + i) * hq + h) * d;
              double dpsum = 0.0;
              for (int64_t x = 0; x < d; ++x) {
                dpsum += (double)doi[x] * o[x];
                dqr[x] = 0.0;
              }
              for (int64_t j = lo; j < hi; ++j) {
                const float* kj = k + ((b * sk + j) * hk + kh) * d;
                const float* vj = v + ((b * sk + j) * hk + kh) * d;
                double dp = 0.0;
                for (int64_t x = 0; x < d; ++x) dp += (double)doi[x] * (double)vj[x];
                const double dqk = p[j] * (dp - dpsum) * scale;
                double* dkj = dk_acc + ((b * sk + j) * hk + kh) * d;
                double* dvj = dv_acc + ((b * sk + j) * hk + kh) * d;
                for (int64_t x = 0; x < d; ++x) {
                  dvj[x] += p[j] * (double)doi[x];
                  dqr[x] += dqk * (double)kj[x];
                  dkj[x] += dqk * (double)qi[x];
                }
              }
              float* dqi = dq + ((b * sq + i) * hq + h) * d;
              for (int64_t x = 0; x < d; ++x) dqi[x] = (float)dqr[x];
            }
          }
        }
      }
    }
    free(s);
    free(p);
    free(o);
    free(dqr);
  }
  if (d_out) {
    const int64_t n = batch * sk * hk * d;
    for (int64_t i = 0; i < n; ++i) {
      dk[i] = (float)dk_acc[i];
      dv[i] = (float)dv_acc[i];
    }
    free(dk_acc);
    free(dv_acc);
  }
}
