/*
 * CPU oracle for the mograd training hot path.  TEST INFRASTRUCTURE ONLY:
 * the shipped library never links, loads or calls anything in this file; it
 * exists so that the CUDA kernels can be checked against an independent
 * restatement of the reference's arithmetic, and so that the benchmark can
 * time "the same maths on the host cores" next to the GPU number.
 *
 * The reference (jjvraw/mograd) is pure Mojo and cannot be built without the
 * Mojo/MAX toolchain, so each routine here restates the reference algorithm
 * and cites the file:line it follows.  All tensors are float32 in memory
 * (callers round through bf16 first when the GPU path is bf16); all
 * arithmetic is float64 so that the oracle is the more accurate side of
 * every comparison.  The oracle is pinned against the reference's own
 * known-answer vectors by tests/test_oracle_kat.py.
 *
 * Build: make -C oracle   (gcc -O3 -march=native -fopenmp -shared -fPIC)
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORC_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------------ */
/* matmul_bias_bt forward:  Y[m,n] = sum_k A[m,k] * W[n,k] + bias[n]          */
/* Contract: mograd/runtime/gpu/kernels/__init__.mojo:770-799 ("a @ b.T +    */
/* bias", bias broadcast over the last axis).  bias may be NULL.             */
/* ------------------------------------------------------------------------ */
ORC_API void orc_matmul_bias_bt(const float* a, const float* w, const float* bias, float* y,
                                int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldw, int64_t ldy) {
  /* 4 x 4 output blocks share their operand loads; every output is still one float64 dot product over k. */
  const int64_t MB = (M + 3) / 4, NB = (N + 3) / 4;
#pragma omp parallel for schedule(static) collapse(2)
  for (int64_t mb = 0; mb < MB; ++mb) {
    for (int64_t nb = 0; nb < NB; ++nb) {
      const int64_t m0 = mb * 4, n0 = nb * 4;
      const int64_t mr = M - m0 < 4 ? M - m0 : 4, nr = N - n0 < 4 ? N - n0 : 4;
      if (mr == 4 && nr == 4) {
        const float *a0 = a + m0 * lda, *a1 = a0 + lda, *a2 = a1 + lda, *a3 = a2 + lda;
        const float *w0 = w + n0 * ldw, *w1 = w0 + ldw, *w2 = w1 + ldw, *w3 = w2 + ldw;
        double c00 = 0, c01 = 0, c02 = 0, c03 = 0, c10 = 0, c11 = 0, c12 = 0, c13 = 0;
        double c20 = 0, c21 = 0, c22 = 0, c23 = 0, c30 = 0, c31 = 0, c32 = 0, c33 = 0;
#pragma omp simd reduction(+ : c00, c01, c02, c03, c10, c11, c12, c13, c20, c21, c22, c23, c30, c31, c32, c33)
        for (int64_t k = 0; k < K; ++k) {
          const double x0 = a0[k], x1 = a1[k], x2 = a2[k], x3 = a3[k];
          const double v0 = w0[k], v1 = w1[k], v2 = w2[k], v3 = w3[k];
          c00 += x0 * v0; c01 += x0 * v1; c02 += x0 * v2; c03 += x0 * v3;
          c10 += x1 * v0; c11 += x1 * v1; c12 += x1 * v2; c13 += x1 * v3;
          c20 += x2 * v0; c21 += x2 * v1; c22 += x2 * v2; c23 += x2 * v3;
          c30 += x3 * v0; c31 += x3 * v1; c32 += x3 * v2; c33 += x3 * v3;
        }
        const double c[4][4] = {{c00, c01, c02, c03}, {c10, c11, c12, c13}, {c20, c21, c22, c23}, {c30, c31, c32, c33}};
        for (int i = 0; i < 4; ++i)
          for (int j = 0; j < 4; ++j)
            y[(m0 + i) * ldy + n0 + j] = (float)(c[i][j] + (bias ? (double)bias[n0 + j] : 0.0));
      } else {
        for (int64_t m = m0; m < m0 + mr; ++m)
          for (int64_t n = n0; n < n0 + nr; ++n) {
            const float* ar = a + m * lda;
            const float* wr = w + n * ldw;
            double acc = 0.0;
#pragma omp simd reduction(+ : acc)
            for (int64_t k = 0; k < K; ++k) acc += (double)ar[k] * (double)wr[k];
            if (bias) acc += (double)bias[n];
            y[m * ldy + n] = (float)acc;
          }
      }
    }
  }
}

/* ------------------------------------------------------------------------ */
/* Linear backward as the reference's gradient rules compose it:            */
/*   dX = dY @ W          (matmul_grad, mograd/grad.mojo:180-183)            */
/*   dW = (X^T @ dY)^T    (matmul_grad + transpose_grad, grad.mojo:186-187)  */
/*   db = sum_rows dY     (add_grad + expand_grad, grad.mojo:126-127,278-288)*/
/* Any output pointer may be NULL.                                          */
/* ------------------------------------------------------------------------ */
ORC_API void orc_matmul_bias_bt_bwd(const float* dy, const float* x, const float* w, float* dx, float* dw,
                                    float* db, int64_t M, int64_t N, int64_t K, int64_t lddy, int64_t ldx,
                                    int64_t ldw, int64_t lddx, int64_t lddw) {
  /* dX and dW: four output rows share every load of the streamed operand; float64 accumulators per row. */
  if (dx) {
#pragma omp parallel
    {
      double* acc = (double*)malloc(sizeof(double) * (size_t)K * 4);
      double *q0 = acc, *q1 = acc + K, *q2 = acc + 2 * K, *q3 = acc + 3 * K;
#pragma omp for schedule(static)
      for (int64_t mb = 0; mb < (M + 3) / 4; ++mb) {
        const int64_t m0 = mb * 4, mr = M - m0 < 4 ? M - m0 : 4;
        for (int64_t k = 0; k < 4 * K; ++k) acc[k] = 0.0;
        for (int64_t n = 0; n < N; ++n) {
          const double g0 = (double)dy[m0 * lddy + n];
          const double g1 = mr > 1 ? (double)dy[(m0 + 1) * lddy + n] : 0.0;
          const double g2 = mr > 2 ? (double)dy[(m0 + 2) * lddy + n] : 0.0;
          const double g3 = mr > 3 ? (double)dy[(m0 + 3) * lddy + n] : 0.0;
          const float* wr = w + n * ldw;
#pragma omp simd
          for (int64_t k = 0; k < K; ++k) {
            const double wv = (double)wr[k];
            q0[k] += g0 * wv;
            q1[k] += g1 * wv;
            q2[k] += g2 * wv;
            q3[k] += g3 * wv;
          }
        }
        for (int64_t i = 0; i < mr; ++i)
          for (int64_t k = 0; k < K; ++k) dx[(m0 + i) * lddx + k] = (float)acc[i * K + k];
      }
      free(acc);
    }
  }
  if (dw) {
#pragma omp parallel
    {
      double* acc = (double*)malloc(sizeof(double) * (size_t)K * 4);
      double *q0 = acc, *q1 = acc + K, *q2 = acc + 2 * K, *q3 = acc + 3 * K;
#pragma omp for schedule(static)
      for (int64_t nb = 0; nb < (N + 3) / 4; ++nb) {
        const int64_t n0 = nb * 4, nr = N - n0 < 4 ? N - n0 : 4;
        for (int64_t k = 0; k < 4 * K; ++k) acc[k] = 0.0;
        for (int64_t m = 0; m < M; ++m) {
          const float* dr = dy + m * lddy + n0;
          const double g0 = (double)dr[0];
          const double g1 = nr > 1 ? (double)dr[1] : 0.0;
          const double g2 = nr > 2 ? (double)dr[2] : 0.0;
          const double g3 = nr > 3 ? (double)dr[3] : 0.0;
          const float* xr = x + m * ldx;
#pragma omp simd
          for (int64_t k = 0; k < K; ++k) {
            const double xv = (double)xr[k];
            q0[k] += g0 * xv;
            q1[k] += g1 * xv;
            q2[k] += g2 * xv;
            q3[k] += g3 * xv;
          }
        }
        for (int64_t i = 0; i < nr; ++i)
          for (int64_t k = 0; k < K; ++k) dw[(n0 + i) * lddw + k] = (float)acc[i * K + k];
      }
      free(acc);
    }
  }
  if (db) {
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
      double acc = 0.0;
      for (int64_t m = 0; m < M; ++m) acc += (double)dy[m * lddy + n];
      db[n] = (float)acc;
    }
  }
}

/* ------------------------------------------------------------------------ */
/* LayerNorm forward: y = (x - mean) / sqrt(mean((x-mean)^2) + eps) * g + b  */
/* Definition: mograd/nn/modules/normalization.mojo:17-27 (biased variance,  */
/* last axis).  mean_out / rstd_out (one per row) may be NULL.               */
/* ------------------------------------------------------------------------ */
ORC_API void orc_layer_norm_fwd(const float* x, const float* gamma, const float* beta, float* y, float* mean_out,
                                float* rstd_out, int64_t rows, int64_t cols, double eps) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r) {
    const float* xr = x + r * cols;
    double mu = 0.0;
    for (int64_t c = 0; c < cols; ++c) mu += (double)xr[c];
    mu /= (double)cols;
    double var = 0.0;
    for (int64_t c = 0; c < cols; ++c) {
      const double d = (double)xr[c] - mu;
      var += d * d;
    }
    var /= (double)cols;
    const double rstd = 1.0 / sqrt(var + eps);
    for (int64_t c = 0; c < cols; ++c)
      y[r * cols + c] = (float)(((double)xr[c] - mu) * rstd * (double)gamma[c] + (double)beta[c]);
    if (mean_out) mean_out[r] = (float)mu;
    if (rstd_out) rstd_out[r] = (float)rstd;
  }
}

/* ------------------------------------------------------------------------ */
/* LayerNorm backward, the algebra of                                       */
/* mograd/runtime/gpu/kernels/normalization.mojo:126-170:                    */
/*   xhat = (x-mu)*rstd; c1 = mean(dy*g); c2 = mean(dy*g*xhat);              */
/*   dx = rstd*(dy*g - c1 - xhat*c2); dgamma = sum_rows dy*xhat;             */
/*   dbeta = sum_rows dy.   (mu/rstd recomputed from x, var = E[x^2]-mu^2    */
/*   clamped at 0 as the kernel does.)                                       */
/* ------------------------------------------------------------------------ */
ORC_API void orc_layer_norm_bwd(const float* dy, const float* x, const float* gamma, float* dx, float* dgamma,
                                float* dbeta, int64_t rows, int64_t cols, double eps) {
  double* dg = (double*)calloc((size_t)cols, sizeof(double));
  double* db = (double*)calloc((size_t)cols, sizeof(double));
#pragma omp parallel
  {
    double* dg_l = (double*)calloc((size_t)cols, sizeof(double));
    double* db_l = (double*)calloc((size_t)cols, sizeof(double));
#pragma omp for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
      const float* xr = x + r * cols;
      const float* dyr = dy + r * cols;
      double sx = 0.0, sx2 = 0.0;
      for (int64_t c = 0; c < cols; ++c) {
        sx += (double)xr[c];
        sx2 += (double)xr[c] * (double)xr[c];
      }
      const double n = (double)cols;
      const double mu = sx / n;
      double var = sx2 / n - mu * mu;
      if (var < 0.0) var = 0.0;
      const double rstd = 1.0 / sqrt(var + eps);
      double c1 = 0.0, c2 = 0.0;
      for (int64_t c = 0; c < cols; ++c) {
        const double xhat = ((double)xr[c] - mu) * rstd;
        const double dyg = (double)dyr[c] * (double)gamma[c];
        c1 += dyg;
        c2 += dyg * xhat;
      }
      c1 /= n;
      c2 /= n;
      for (int64_t c = 0; c < cols; ++c) {
        const double xhat = ((double)xr[c] - mu) * rstd;
        const double dyv = (double)dyr[c];
        dx[r * cols + c] = (float)(rstd * (dyv * (double)gamma[c] - c1 - xhat * c2));
        dg_l[c] += dyv * xhat;
        db_l[c] += dyv;
      }
    }
#pragma omp critical
    {
      for (int64_t c = 0; c < cols; ++c) {
        dg[c] += dg_l[c];
        db[c] += db_l[c];
      }
    }
    free(dg_l);
    free(db_l);
  }
  for (int64_t c = 0; c < cols; ++c) {
    dgamma[c] = (float)dg[c];
    dbeta[c] = (float)db[c];
  }
  free(dg);
  free(db);
}

/* ------------------------------------------------------------------------ */
/* Cross-entropy, dense float labels (the reference's form):                */
/*   loss = -(1/N) sum_r sum_c label[r,c]*(x[r,c] - max_r - log sum exp)     */
/* mograd/runtime/gpu/kernels/cross_entropy.mojo:14-77 (+ sum_rows :155-177) */
/*   dlogits = (softmax(x) - label) * upstream / N   (cross_entropy.mojo:    */
/*   185-241).  ldx / ldl are row strides in elements.  dlogits may be NULL. */
/* ------------------------------------------------------------------------ */
ORC_API double orc_cross_entropy_dense(const float* logits, const float* labels, float* dlogits, int64_t N,
                                       int64_t C, int64_t ldx, int64_t ldl, int64_t lddx, double upstream) {
  double total = 0.0;
#pragma omp parallel for schedule(static) reduction(+ : total)
  for (int64_t r = 0; r < N; ++r) {
    const float* xr = logits + r * ldx;
    const float* lr = labels + r * ldl;
    double mx = -INFINITY;
    for (int64_t c = 0; c < C; ++c)
      if ((double)xr[c] > mx) mx = (double)xr[c];
    double se = 0.0;
    for (int64_t c = 0; c < C; ++c) se += exp((double)xr[c] - mx);
    const double lse = log(se);
    double row = 0.0;
    for (int64_t c = 0; c < C; ++c) row += ((double)xr[c] - mx - lse) * (double)lr[c];
    total += -row / (double)N;
    if (dlogits) {
      const double g = upstream / (double)N;
      for (int64_t c = 0; c < C; ++c)
        dlogits[r * lddx + c] = (float)((exp((double)xr[c] - mx) / se - (double)lr[c]) * g);
    }
  }
  return total;
}

/* Same arithmetic with the one-hot label given as a class index per row     */
/* (label[r,c] = (c == idx[r])), which is what the reference's train loop    */
/* builds with one_hot().cast() (examples/tinyshakespear/train.mojo:38-41).  */
/* row_lse (natural log, includes the max) may be NULL.                      */
ORC_API double orc_cross_entropy_index(const float* logits, const int64_t* idx, float* dlogits, float* row_lse,
                                       int64_t N, int64_t C, int64_t ldx, int64_t lddx, double upstream) {
  double total = 0.0;
#pragma omp parallel for schedule(static) reduction(+ : total)
  for (int64_t r = 0; r < N; ++r) {
    const float* xr = logits + r * ldx;
    double mx = -INFINITY;
    for (int64_t c = 0; c < C; ++c)
      if ((double)xr[c] > mx) mx = (double)xr[c];
    double se = 0.0;
    for (int64_t c = 0; c < C; ++c) se += exp((double)xr[c] - mx);
    const double lse = log(se);
    const int64_t t = idx[r];
    total += -((double)xr[t] - mx - lse) / (double)N;
    if (row_lse) row_lse[r] = (float)(mx + lse);
    if (dlogits) {
      const double g = upstream / (double)N;
      for (int64_t c = 0; c < C; ++c)
        dlogits[r * lddx + c] = (float)((exp((double)xr[c] - mx) / se - (c == t ? 1.0 : 0.0)) * g);
    }
  }
  return total;
}

/* ------------------------------------------------------------------------ */
/* Attention forward, float64, naive O(S^2): restates ref_sdpa_f64,          */
/* tests/kernels/attention/harness.mojo:58-109.  Q/K/V are BSHD, O is BHSD,  */
/* LSE is (B,H,S) natural log, softmax is max-subtracted, causal keeps       */
/* j <= i.  mask (B,H,S,S additive) may be NULL.                             */
/* ------------------------------------------------------------------------ */
ORC_API void orc_sdpa_fwd(const float* q, const float* k, const float* v, const float* mask, float* out,
                          float* lse, int64_t B, int64_t S, int64_t H, int64_t D, double scale, int causal) {
#pragma omp parallel
  {
    double* sc = (double*)malloc(sizeof(double) * (size_t)S);
#pragma omp for schedule(dynamic, 1) collapse(2)
    for (int64_t bh = 0; bh < B * H; ++bh) {
      for (int64_t i = 0; i < S; ++i) {
        const int64_t b = bh / H, h = bh % H;
        const int64_t j_end = causal ? (i + 1) : S;
        const float* qi = q + ((b * S + i) * H + h) * D;
        double row_max = -1e300;
        for (int64_t j = 0; j < j_end; ++j) {
          const float* kj = k + ((b * S + j) * H + h) * D;
          double s = 0.0;
          for (int64_t d = 0; d < D; ++d) s += (double)qi[d] * (double)kj[d];
          s *= scale;
          if (mask) s += (double)mask[(bh * S + i) * S + j];
          sc[j] = s;
          if (s > row_max) row_max = s;
        }
        double denom = 0.0;
        for (int64_t j = 0; j < j_end; ++j) {
          sc[j] = exp(sc[j] - row_max);
          denom += sc[j];
        }
        for (int64_t d = 0; d < D; ++d) {
          double acc = 0.0;
          for (int64_t j = 0; j < j_end; ++j) acc += sc[j] * (double)v[((b * S + j) * H + h) * D + d];
          out[(bh * S + i) * D + d] = (float)(acc / denom);
        }
        if (lse) lse[bh * S + i] = (float)(row_max + log(denom));
      }
    }
    free(sc);
  }
}

/* ------------------------------------------------------------------------ */
/* Attention backward, float64: restates ref_sdpa_bwd_f64,                   */
/* tests/kernels/attention/harness.mojo:112-175.  dO is BHSD; dQ/dK/dV BSHD. */
/* ds = p*(dp - delta)*scale, dq += ds*k, dk += ds*q, dv += p*dO, with       */
/* delta = sum_d dO*O recomputed from p and v.                               */
/* Parallelised over (b,h); every (b,h) owns its slice of dQ/dK/dV.          */
/* o_saved (BHSD, may be NULL): when given, delta = sum_d dO*o_saved, i.e.   */
/* the forward output as it was STORED, which is what the reference's GPU    */
/* kernels use (flash_attn_bwd_delta_kernel,                                 */
/* mograd/runtime/gpu/kernels/attention/nvidia_bwd.mojo:784-836); with NULL  */
/* delta comes from the exact recomputed output as in the harness.           */
/* ------------------------------------------------------------------------ */
ORC_API void orc_sdpa_bwd(const float* q, const float* k, const float* v, const float* dy, const float* mask,
                          const float* o_saved, float* dq, float* dk, float* dv, int64_t B, int64_t S, int64_t H,
                          int64_t D, double scale, int causal) {
#pragma omp parallel
  {
    double* p = (double*)malloc(sizeof(double) * (size_t)S);
    double* dqa = (double*)malloc(sizeof(double) * (size_t)(S * D));
    double* dka = (double*)malloc(sizeof(double) * (size_t)(S * D));
    double* dva = (double*)malloc(sizeof(double) * (size_t)(S * D));
    double* od = (double*)malloc(sizeof(double) * (size_t)D);
#pragma omp for schedule(dynamic, 1)
    for (int64_t bh = 0; bh < B * H; ++bh) {
      const int64_t b = bh / H, h = bh % H;
      memset(dqa, 0, sizeof(double) * (size_t)(S * D));
      memset(dka, 0, sizeof(double) * (size_t)(S * D));
      memset(dva, 0, sizeof(double) * (size_t)(S * D));
      for (int64_t i = 0; i < S; ++i) {
        const int64_t j_end = causal ? (i + 1) : S;
        const float* qi = q + ((b * S + i) * H + h) * D;
        const float* dyi = dy + (bh * S + i) * D;
        double row_max = -1e300;
        for (int64_t j = 0; j < j_end; ++j) {
          const float* kj = k + ((b * S + j) * H + h) * D;
          double s = 0.0;
          for (int64_t d = 0; d < D; ++d) s += (double)qi[d] * (double)kj[d];
          s *= scale;
          if (mask) s += (double)mask[(bh * S + i) * S + j];
          p[j] = s;
          if (s > row_max) row_max = s;
        }
        double denom = 0.0;
        for (int64_t j = 0; j < j_end; ++j) {
          p[j] = exp(p[j] - row_max);
          denom += p[j];
        }
        for (int64_t j = 0; j < j_end; ++j) p[j] /= denom;
        for (int64_t d = 0; d < D; ++d) od[d] = 0.0;
        for (int64_t j = 0; j < j_end; ++j) {
          const float* vj = v + ((b * S + j) * H + h) * D;
          for (int64_t d = 0; d < D; ++d) od[d] += p[j] * (double)vj[d];
        }
        double delta = 0.0;
        if (o_saved) {
          const float* oi = o_saved + (bh * S + i) * D;
          for (int64_t d = 0; d < D; ++d) delta += (double)dyi[d] * (double)oi[d];
        } else {
          for (int64_t d = 0; d < D; ++d) delta += (double)dyi[d] * od[d];
        }
        for (int64_t j = 0; j < j_end; ++j) {
          const float* kj = k + ((b * S + j) * H + h) * D;
          const float* vj = v + ((b * S + j) * H + h) * D;
          double dp = 0.0;
          for (int64_t d = 0; d < D; ++d) dp += (double)dyi[d] * (double)vj[d];
          const double ds = p[j] * (dp - delta) * scale;
          for (int64_t d = 0; d < D; ++d) {
            dqa[i * D + d] += ds * (double)kj[d];
            dka[j * D + d] += ds * (double)qi[d];
            dva[j * D + d] += p[j] * (double)dyi[d];
          }
        }
      }
      for (int64_t s = 0; s < S; ++s)
        for (int64_t d = 0; d < D; ++d) {
          const int64_t o = ((b * S + s) * H + h) * D + d;
          dq[o] = (float)dqa[s * D + d];
          dk[o] = (float)dka[s * D + d];
          dv[o] = (float)dva[s * D + d];
        }
    }
    free(p);
    free(dqa);
    free(dka);
    free(dva);
    free(od);
  }
}

/* ------------------------------------------------------------------------ */
/* Elementwise helpers the train-step oracle needs (callers of the hot path: */
/* relu / relu_grad mograd/runtime/gpu/kernels/elementwise.mojo, embedding   */
/* gather / scatter_add mograd/runtime/gpu/kernels/gather_scatter.mojo:14-71)*/
/* ------------------------------------------------------------------------ */
ORC_API void orc_relu(const float* x, float* y, int64_t n) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) y[i] = x[i] > 0.f ? x[i] : 0.f;
}

/* dx = dy where the forward input was > 0, else 0 */
ORC_API void orc_relu_grad(const float* x, const float* dy, float* dx, int64_t n) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) dx[i] = x[i] > 0.f ? dy[i] : 0.f;
}

ORC_API void orc_embedding_fwd(const float* table, const int64_t* idx, float* out, int64_t T, int64_t d) {
#pragma omp parallel for schedule(static)
  for (int64_t t = 0; t < T; ++t) memcpy(out + t * d, table + idx[t] * d, sizeof(float) * (size_t)d);
}

ORC_API void orc_embedding_bwd(const float* dout, const int64_t* idx, float* dtable, int64_t T, int64_t V,
                               int64_t d) {
  double* acc = (double*)calloc((size_t)(V * d), sizeof(double));
  for (int64_t t = 0; t < T; ++t)
    for (int64_t c = 0; c < d; ++c) acc[idx[t] * d + c] += (double)dout[t * d + c];
  for (int64_t i = 0; i < V * d; ++i) dtable[i] = (float)acc[i];
  free(acc);
}

/* Round-to-nearest-even float32 -> bfloat16 -> float32, so both sides of a  */
/* bf16 comparison consume identical inputs.                                 */
ORC_API void orc_round_bf16(const float* x, float* y, int64_t n) {
  for (int64_t i = 0; i < n; ++i) {
    uint32_t u;
    memcpy(&u, x + i, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) {
      u |= 0x00400000u; /* quiet NaN */
      u &= 0xffff0000u;
    } else {
      u += 0x7fffu + ((u >> 16) & 1u);
      u &= 0xffff0000u;
    }
    memcpy(y + i, &u, 4);
  }
}
