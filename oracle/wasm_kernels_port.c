/*
 * CPU oracle for the quantized matrix-product path of fluidaudio-web.
 *
 * TEST INFRASTRUCTURE ONLY. This file is the checker the CUDA backend is compared
 * against; nothing in the shipped package links, imports or calls it.
 *
 * Pinning status: PINNED to outputs of the reference itself.  The four kernels restated here ship
 * compiled as src/gpu/wasm-kernels.wasm; oracle/wasm_exec.py executes that module through the host
 * calling convention of src/gpu/wasm-context.js, tests/golden/gen_wasm_golden.py stores what it returns
 * on the reference gate's seeded cases plus ragged / partial-block / grouped-convolution cases, and
 * tests/test_oracle_pinned.py requires this file to reproduce every stored array bit for bit (and
 * re-executes the module live where a reference checkout is present).  The JavaScript half (bias,
 * activation, residual, glue ops) has no compiled form to execute; it stays pinned to the closed-form
 * expectations of scripts/wasm-verify.mjs and the seeded cases of scripts/backend-conformance.mjs
 * restated in tests/test_oracle.py.
 *
 * It restates, operation by operation and in the same order, the reference's own
 * CPU implementation of the path:
 *   - the Rust->wasm32+simd128 kernels in rust/wasm-kernels/src/lib.rs
 *     (matmul_f32 :59-94, conv1d_f32 :99-138, matmul_int8 :143-162,
 *      matmul_nbits :169-203), and
 *   - the JavaScript half that wraps them, src/gpu/wasm-context.js
 *     (activations :12-38, bias/act epilogue :290-305, residual add :151-154,
 *      and the plain-JS glue ops :308-343, 363-563, 632-685).
 *
 * Arithmetic rules that make the restatement bit-faithful:
 *   - wasm32 simd128 without relaxed-simd has no fused multiply-add: every a*b+c
 *     is an f32 multiply followed by a separately rounded f32 add.  Build this file
 *     with -ffp-contract=off (the Makefile does); lanes of a v128 are independent,
 *     so vector width does not change any result.
 *   - JavaScript arithmetic on Float32Array elements is IEEE double: `let acc = 0;
 *     acc += x[i]*y[i]` accumulates in f64 and rounds once when stored back into a
 *     Float32Array.  Every glue op below therefore uses `double` exactly where the
 *     JS uses a plain `let`.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define ORACLE_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------------- */
/* rust/wasm-kernels/src/lib.rs                                               */
/* ------------------------------------------------------------------------- */

/* lib.rs:59-94.  Per row i: zero the C row, then for k ascending
 * C[i,j] = C[i,j] + A[i,k]*B[k,j] for every j (mul and add rounded separately). */
ORACLE_API void wk_matmul_f32(const float *a, const float *b, float *c, size_t m, size_t k, size_t n) {
  for (size_t i = 0; i < m; i++) {
    float *crow = c + i * n;
    for (size_t j = 0; j < n; j++) crow[j] = 0.0f;
    const float *arow = a + i * k;
    for (size_t kk = 0; kk < k; kk++) {
      const float aik = arow[kk];
      const float *brow = b + kk * n;
      for (size_t j = 0; j < n; j++) {
        float p = aik * brow[j];
        crow[j] = crow[j] + p;
      }
    }
  }
}

/* Same arithmetic as wk_matmul_f32 with rows spread over OpenMP threads (rows are
 * independent, so results are bit-identical).  Used for the timed CPU baseline. */
ORACLE_API void wk_matmul_f32_mt(const float *a, const float *b, float *c, size_t m, size_t k, size_t n) {
#pragma omp parallel for schedule(static)
  for (long i = 0; i < (long)m; i++) wk_matmul_f32(a + (size_t)i * k, b, c + (size_t)i * n, 1, k, n);
}

/* lib.rs:99-138.  Direct 1-D conv, zero weights skipped (:120). */
ORACLE_API void wk_conv1d_f32(const float *x, const float *w, float *y, size_t cout, size_t cin, size_t l, size_t lout,
                              size_t k, size_t stride, size_t pad_left, size_t dilation, size_t groups) {
  size_t cin_g = cin / groups, cout_g = cout / groups;
  for (size_t co = 0; co < cout; co++) {
    size_t g = co / cout_g;
    float *yrow = y + co * lout;
    for (size_t t = 0; t < lout; t++) yrow[t] = 0.0f;
    for (size_t cig = 0; cig < cin_g; cig++) {
      size_t ci = g * cin_g + cig;
      const float *xrow = x + ci * l;
      size_t wbase = (co * cin_g + cig) * k;
      for (size_t kk = 0; kk < k; kk++) {
        float wv = w[wbase + kk];
        if (wv == 0.0f) continue;
        size_t off = kk * dilation;
        for (size_t t = 0; t < lout; t++) {
          size_t src = t * stride + off;
          if (src >= pad_left) {
            size_t xi = src - pad_left;
            if (xi < l) {
              float p = xrow[xi] * wv;
              yrow[t] = yrow[t] + p;
            }
          }
        }
      }
    }
  }
}

/* lib.rs:143-162.  Loop order i, j, k; acc += a*(f32)q sequential in k; then *scale[j].
 * wq byte index k*n + j, reinterpreted as int8. */
ORACLE_API void wk_matmul_int8(const float *a, const uint8_t *wq, const float *scale, float *y, size_t m, size_t n,
                               size_t k) {
  for (size_t i = 0; i < m; i++) {
    const float *arow = a + i * k;
    float *yrow = y + i * n;
    for (size_t j = 0; j < n; j++) {
      float acc = 0.0f;
      for (size_t kk = 0; kk < k; kk++) {
        int8_t q = (int8_t)wq[kk * n + j];
        float p = arow[kk] * (float)q;
        acc = acc + p;
      }
      yrow[j] = acc * scale[j];
    }
  }
}

/* Same per-output operation sequence as wk_matmul_int8 (k ascending, one f32
 * accumulator per output) with the loops interchanged to i, k, j so the weight
 * row is read contiguously; bit-identical results, used for larger parity cases
 * and the multithreaded CPU baseline.  Needs `acc` scratch of n floats per row. */
static void int8_row_kj(const float *arow, const uint8_t *wq, const float *scale, float *yrow, size_t n, size_t k,
                        size_t j0, size_t j1) {
  for (size_t j = j0; j < j1; j++) yrow[j] = 0.0f;
  for (size_t kk = 0; kk < k; kk++) {
    const float av = arow[kk];
    const int8_t *wrow = (const int8_t *)(wq + kk * n);
    for (size_t j = j0; j < j1; j++) {
      float p = av * (float)wrow[j];
      yrow[j] = yrow[j] + p;
    }
  }
  for (size_t j = j0; j < j1; j++) yrow[j] = yrow[j] * scale[j];
}
/* Work items are (row, block of 512 columns): outputs are independent, so few-row products (token-by-token
 * decoding) spread over the threads as well. */
ORACLE_API void wk_matmul_int8_kj(const float *a, const uint8_t *wq, const float *scale, float *y, size_t m, size_t n,
                                  size_t k) {
  const long cb = 512, nb = (long)((n + cb - 1) / cb);
#pragma omp parallel for schedule(static)
  for (long w = 0; w < (long)m * nb; w++) {
    const size_t i = (size_t)(w / nb), j0 = (size_t)(w % nb) * cb, j1 = j0 + cb < n ? j0 + cb : n;
    int8_row_kj(a + i * k, wq, scale, y + i * n, n, k, j0, j1);
  }
}
/* The reference loop order itself, rows over OpenMP threads (timed CPU baseline). */
ORACLE_API void wk_matmul_int8_mt(const float *a, const uint8_t *wq, const float *scale, float *y, size_t m, size_t n,
                                  size_t k) {
#pragma omp parallel for schedule(static)
  for (long i = 0; i < (long)m; i++) wk_matmul_int8(a + (size_t)i * k, wq, scale, y + (size_t)i * n, 1, n, k);
}

/* lib.rs:181-199: one output element.  w=(q-zp)*scale then acc += a*w; the t loop
 * stops at kk>=k (partial last block). */
static inline float nbits_one(const float *arow, const uint8_t *bq_row, const float *sc_row, const uint8_t *zp_row,
                              size_t k, size_t nblk, size_t blocksize) {
  float acc = 0.0f;
  for (size_t blk = 0; blk < nblk; blk++) {
    float scale = sc_row[blk];
    uint8_t zbyte = zp_row[blk / 2]; /* packed int4 zero-point, even blk = low nibble */
    float zpv = (float)((blk & 1) == 0 ? (zbyte & 0x0f) : (zbyte >> 4));
    size_t blk_base = blk * blocksize;
    const uint8_t *bq_blk = bq_row + blk * 16;
    for (size_t t = 0; t < blocksize; t++) {
      size_t kk = blk_base + t;
      if (kk >= k) break;
      uint8_t byte = bq_blk[t / 2];
      float q = (float)((t & 1) == 0 ? (byte & 0x0f) : (byte >> 4));
      float d = q - zpv;
      float wv = d * scale;
      float p = arow[kk] * wv;
      acc = acc + p;
    }
  }
  return acc;
}
/* lib.rs:169-203.  Loop order j (output column), i (row), blk, t. */
ORACLE_API void wk_matmul_nbits(const float *a, const uint8_t *bq, const float *scales, const uint8_t *zp, float *y,
                                size_t m, size_t n, size_t k, size_t nblk, size_t zpb, size_t blocksize) {
  for (size_t j = 0; j < n; j++)
    for (size_t i = 0; i < m; i++)
      y[i * n + j] = nbits_one(a + i * k, bq + j * nblk * 16, scales + j * nblk, zp + j * zpb, k, nblk, blocksize);
}
/* Output columns over OpenMP threads; identical arithmetic (timed CPU baseline). */
ORACLE_API void wk_matmul_nbits_mt(const float *a, const uint8_t *bq, const float *scales, const uint8_t *zp, float *y,
                                   size_t m, size_t n, size_t k, size_t nblk, size_t zpb, size_t blocksize) {
#pragma omp parallel for schedule(static)
  for (long j = 0; j < (long)n; j++)
    for (size_t i = 0; i < m; i++)
      y[i * n + (size_t)j] = nbits_one(a + i * k, bq + (size_t)j * nblk * 16, scales + (size_t)j * nblk,
                                       zp + (size_t)j * zpb, k, nblk, blocksize);
}

/* ------------------------------------------------------------------------- */
/* src/gpu/wasm-context.js — activations and epilogues (f64 math, f32 store)  */
/* ------------------------------------------------------------------------- */

/* Activation codes follow src/gpu/kernels/actf.js:24
 * (none 0, gelu 1, tanh 2, relu 3, silu 4, gelu_erf 5). */
static double clampd(double v, double lo, double hi) { return v < lo ? lo : (v > hi ? hi : v); }
static double js_gelu_tanh(double x) { /* wasm-context.js:12-15 */
  double t = clampd(0.7978845608028654 * (x + 0.044715 * x * x * x), -20.0, 20.0);
  return 0.5 * x * (1 + tanh(t));
}
static double js_erf_a(double x) { /* wasm-context.js:16-20 (Abramowitz-Stegun 7.1.26) */
  double t = 1 / (1 + 0.3275911 * fabs(x));
  double y = 1 - ((((1.061405429 * t - 1.453152027) * t + 1.421413741) * t - 0.284496736) * t + 0.254829592) * t *
                     exp(-x * x);
  return x >= 0 ? y : -y;
}
static double js_gelu_erf(double x) { return 0.5 * x * (1 + js_erf_a(x * 0.70710678118654752)); } /* :21 */
static double js_silu(double x) { return x / (1 + exp(-clampd(x, -30.0, 30.0))); }                   /* :22 */
ORACLE_API double js_apply_act(double v, int act) { /* wasm-context.js:23-38 */
  switch (act) {
    case 1: return js_gelu_tanh(v);
    case 2: return tanh(v);
    case 3: return v > 0 ? v : 0;
    case 4: return js_silu(v);
    case 5: return js_gelu_erf(v);
    default: return v;
  }
}

/* wasm-context.js:290-297: out[i,j] = act(out[i,j] + bias[j]); skipped entirely
 * when there is no bias and act is none. */
ORACLE_API void js_bias_act_columns(float *out, size_t M, size_t N, const float *bias, int act) {
  if (!bias && act == 0) return;
  for (size_t i = 0; i < M; i++)
    for (size_t j = 0; j < N; j++) {
      double v = (double)out[i * N + j] + (bias ? (double)bias[j] : 0.0);
      out[i * N + j] = (float)js_apply_act(v, act);
    }
}
/* wasm-context.js:298-305: per-row bias (conv outputs). */
ORACLE_API void js_bias_act_rows(float *out, size_t R, size_t C, const float *bias, int act) {
  if (!bias && act == 0) return;
  for (size_t r = 0; r < R; r++)
    for (size_t c = 0; c < C; c++) {
      double v = (double)out[r * C + c] + (bias ? (double)bias[r] : 0.0);
      out[r * C + c] = (float)js_apply_act(v, act);
    }
}
/* wasm-context.js:151-154: out[i] += add[i] on Float32Array elements. */
ORACLE_API void js_residual_add(float *out, const float *add, size_t n) {
  for (size_t i = 0; i < n; i++) out[i] = (float)((double)out[i] + (double)add[i]);
}

/* ------------------------------------------------------------------------- */
/* src/gpu/wasm-context.js — glue ops used by the encoder / decoder forwards  */
/* ------------------------------------------------------------------------- */

/* :308-326 */
ORACLE_API void js_layernorm(const float *x, const float *gamma, const float *beta, float *out, size_t R, size_t C,
                             double eps) {
  for (size_t r = 0; r < R; r++) {
    double mean = 0;
    for (size_t j = 0; j < C; j++) mean += x[r * C + j];
    mean /= (double)C;
    double v = 0;
    for (size_t j = 0; j < C; j++) {
      double d = x[r * C + j] - mean;
      v += d * d;
    }
    v /= (double)C;
    double inv = 1 / sqrt(v + eps);
    for (size_t j = 0; j < C; j++) out[r * C + j] = (float)((x[r * C + j] - mean) * inv * gamma[j] + beta[j]);
  }
}
/* :327-343.  e is stored to f32 before the sum reads the double; the divide reads
 * the f32 back. */
ORACLE_API void js_softmax(const float *x, float *out, size_t R, size_t C) {
  for (size_t r = 0; r < R; r++) {
    double mx = -INFINITY;
    for (size_t j = 0; j < C; j++) mx = fmax(mx, (double)x[r * C + j]);
    double s = 0;
    for (size_t j = 0; j < C; j++) {
      double e = exp((double)x[r * C + j] - mx);
      out[r * C + j] = (float)e;
      s += e;
    }
    for (size_t j = 0; j < C; j++) out[r * C + j] = (float)((double)out[r * C + j] / s);
  }
}
/* :363-373.  b broadcasts over rows when it has one row. op 0 add, 1 mul. */
ORACLE_API void js_ewise(const float *a, const float *b, float *out, size_t R, size_t C, int b_rows_is_one, int op) {
  for (size_t i = 0; i < R * C; i++) {
    double bv = b_rows_is_one ? b[i % C] : b[i];
    out[i] = (float)(op == 1 ? (double)a[i] * bv : (double)a[i] + bv);
  }
}
/* :380-384 */
ORACLE_API void js_scale(const float *x, float *out, size_t n, double s) {
  for (size_t i = 0; i < n; i++) out[i] = (float)((double)x[i] * s);
}
/* :396-405 */
ORACLE_API void js_silu_op(const float *x, float *out, size_t n) {
  for (size_t i = 0; i < n; i++) out[i] = (float)js_silu(x[i]);
}
ORACLE_API void js_relu_op(const float *x, float *out, size_t n) {
  for (size_t i = 0; i < n; i++) out[i] = x[i] > 0 ? x[i] : 0.0f;
}
/* :428-434: x[2C,T] -> a * sigmoid(b) */
ORACLE_API void js_glu(const float *x, float *out, size_t C, size_t T) {
  for (size_t c = 0; c < C; c++)
    for (size_t t = 0; t < T; t++)
      out[c * T + t] = (float)((double)x[c * T + t] * (1 / (1 + exp(-(double)x[(c + C) * T + t]))));
}
/* :435-441 */
ORACLE_API void js_transpose(const float *x, float *out, size_t R, size_t C) {
  for (size_t r = 0; r < R; r++)
    for (size_t c = 0; c < C; c++) out[c * R + r] = x[r * C + c];
}
/* :442-448 */
ORACLE_API void js_slice_cols(const float *x, float *out, size_t R, size_t C, size_t col0, size_t width) {
  for (size_t r = 0; r < R; r++)
    for (size_t j = 0; j < width; j++) out[r * width + j] = x[r * C + col0 + j];
}
/* :449-452 */
ORACLE_API void js_set_cols(float *dst, size_t dst_cols, const float *src, size_t src_rows, size_t src_cols,
                            size_t col0) {
  for (size_t r = 0; r < src_rows; r++)
    for (size_t j = 0; j < src_cols; j++) dst[r * dst_cols + col0 + j] = src[r * src_cols + j];
}
/* :462-482 */
ORACLE_API void js_bmm_qk(const float *q, const float *b, const float *qb, float *out, size_t q_rows, size_t b_rows,
                          size_t H, size_t HD, size_t W, int b_shared) {
  size_t T = q_rows / W, Tb = b_shared ? b_rows : b_rows / W, stride = H * HD;
  for (size_t w = 0; w < W; w++)
    for (size_t h = 0; h < H; h++) {
      size_t ho = h * HD;
      for (size_t i = 0; i < T; i++) {
        size_t qBase = (w * T + i) * stride + ho, oBase = ((w * H + h) * T + i) * Tb;
        for (size_t j = 0; j < Tb; j++) {
          size_t bBase = (b_shared ? j : w * Tb + j) * stride + ho;
          double acc = 0;
          for (size_t d = 0; d < HD; d++)
            acc += ((double)q[qBase + d] + (qb ? (double)qb[ho + d] : 0.0)) * (double)b[bBase + d];
          out[oBase + j] = (float)acc;
        }
      }
    }
}
/* :484-500 */
ORACLE_API void js_bmm_pv(const float *p, const float *v, float *out, size_t p_rows, size_t v_rows, size_t H, size_t HD,
                          size_t W) {
  size_t Tk = v_rows / W, Tq = p_rows / (W * H), stride = H * HD;
  for (size_t w = 0; w < W; w++)
    for (size_t i = 0; i < Tq; i++)
      for (size_t c = 0; c < stride; c++) {
        size_t h = c / HD, pBase = ((w * H + h) * Tq + i) * Tk;
        double acc = 0;
        for (size_t j = 0; j < Tk; j++) acc += (double)p[pBase + j] * (double)v[(w * Tk + j) * stride + c];
        out[(w * Tq + i) * stride + c] = (float)acc;
      }
}
/* :525-538 (rows = H*t) and :539-551 (H = 1) */
ORACLE_API void js_rel_shift_b(const float *x, float *out, size_t rows, size_t H) {
  size_t t = rows / H, p = 2 * t - 1, twoT = 2 * t;
  for (size_t h = 0; h < H; h++)
    for (size_t i = 0; i < t; i++)
      for (size_t j = 0; j < t; j++) {
        size_t f = t + i * p + j, col = f % twoT;
        out[(h * t + i) * t + j] = col == 0 ? 0.0f : x[(h * t + f / twoT) * p + (col - 1)];
      }
}
/* :552-563 */
ORACLE_API void js_sub_reshape(const float *x, float *out, size_t C, size_t Tsub, size_t F) {
  size_t CF = C * F;
  for (size_t idx = 0; idx < Tsub * CF; idx++) {
    size_t ho = idx / CF, rem = idx % CF, c = rem / F, wo = rem % F;
    out[idx] = x[c * (Tsub * F) + ho * F + wo];
  }
}
/* :632-685 */
ORACLE_API void js_conv2d(const float *x, const float *w, const float *bias, float *out, size_t cout, size_t cin,
                          size_t h, size_t W_, size_t kh, size_t kw, size_t strideH, size_t strideW, long padTop,
                          long padBottom, long padLeft, long padRight, size_t groups, int act) {
  size_t Ho = (size_t)(((long)h + padTop + padBottom - (long)kh) / (long)strideH) + 1;
  size_t Wo = (size_t)(((long)W_ + padLeft + padRight - (long)kw) / (long)strideW) + 1;
  size_t cinG = cin / groups, coutG = cout / groups;
#pragma omp parallel for schedule(static)
  for (long co_ = 0; co_ < (long)cout; co_++) {
    size_t co = (size_t)co_, g = co / coutG;
    for (size_t ho = 0; ho < Ho; ho++)
      for (size_t wo = 0; wo < Wo; wo++) {
        double acc = bias ? (double)bias[co] : 0.0;
        for (size_t ci = 0; ci < cinG; ci++) {
          size_t rc = g * cinG + ci;
          for (size_t khh = 0; khh < kh; khh++) {
            long hi = (long)(ho * strideH + khh) - padTop;
            if (hi < 0 || hi >= (long)h) continue;
            for (size_t kww = 0; kww < kw; kww++) {
              long wi = (long)(wo * strideW + kww) - padLeft;
              if (wi < 0 || wi >= (long)W_) continue;
              acc += (double)x[rc * h * W_ + (size_t)hi * W_ + (size_t)wi] *
                     (double)w[((co * cinG + ci) * kh + khh) * kw + kww];
            }
          }
        }
        out[co * Ho * Wo + ho * Wo + wo] = (float)js_apply_act(acc, act);
      }
  }
}

/* ------------------------------------------------------------------------- */
/* Integer restatement for the int8-activation mode                           */
/* ------------------------------------------------------------------------- */

/* Exact int32 product of int8 activations [M,K] and int8 weights stored in the
 * reference's byte order (index k*N+n, lib.rs:141-142).  Not in the reference
 * (which never quantises activations); it is the checker for the accumulators
 * the tensor-core kernel produces in its integer mode. */
ORACLE_API void int8_gemm_i32(const int8_t *aq, const uint8_t *wq, int32_t *acc, size_t m, size_t n, size_t k) {
#pragma omp parallel for schedule(static)
  for (long i = 0; i < (long)m; i++) {
    int32_t *row = acc + (size_t)i * n;
    for (size_t j = 0; j < n; j++) row[j] = 0;
    for (size_t kk = 0; kk < k; kk++) {
      int32_t av = aq[(size_t)i * k + kk];
      const int8_t *wrow = (const int8_t *)(wq + kk * n);
      for (size_t j = 0; j < n; j++) row[j] += av * (int32_t)wrow[j];
    }
  }
}

/* ------------------------------------------------------------------------- */
/* Seeded inputs of scripts/backend-conformance.mjs:46-54 (mulberry32)        */
/* ------------------------------------------------------------------------- */

static double mulberry32_next(uint32_t *seed) {
  uint32_t s = *seed;
  s = s + 0x6d2b79f5u;
  *seed = s;
  uint32_t t = (s ^ (s >> 15)) * (1u | s);
  t = (t + ((t ^ (t >> 7)) * (61u | t))) ^ t;
  return (double)(t ^ (t >> 14)) / 4294967296.0;
}
/* mkData: Float32Array.from(rand() - 0.5) */
ORACLE_API void mulberry32_fill_f32(uint32_t *seed, float *out, size_t n) {
  for (size_t i = 0; i < n; i++) out[i] = (float)(mulberry32_next(seed) - 0.5);
}
/* mkBytes: floor(rand()*256) */
ORACLE_API void mulberry32_fill_u8(uint32_t *seed, uint8_t *out, size_t n) {
  for (size_t i = 0; i < n; i++) out[i] = (uint8_t)floor(mulberry32_next(seed) * 256.0);
}

/* Thread count of the OpenMP variants (the timed CPU baseline); n <= 0 leaves it unchanged. */
ORACLE_API void oracle_set_num_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

ORACLE_API int oracle_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
