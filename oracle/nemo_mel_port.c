/* CPU restatement of the reference's NeMo-style log-mel front end: TEST INFRASTRUCTURE ONLY.
 *
 * Follows src/engines/asr-nemotron/nemotron-mel.js (class JsPreprocessor, which
 * src/engines/asr-parakeet/parakeet-mel.js wraps with logGuard 2^-24 + per-feature normalisation), step for step:
 *   :66-110  createMelFilterbank     slaney scale, slaney norm, Float32Array [nMels][257]
 *   :131-141 createPaddedHannWindow  symmetric Hann of 400 in doubles, centred in 512
 *   :158-189 precomputeTwiddles      cos/sin(-2 pi i / N) in doubles, bit-reversal table
 *   :191-357 fft                     in-place radix-2 decimation in time, doubles
 *   :451-573 computeRawMel           pre-emphasis rounded to f32, 256 zeros either side, per frame: one 256-point
 *                                    complex FFT of the windowed frame, real-spectrum reconstruction, power stored as
 *                                    f32, filterbank sum in a double over each filter's non-zero span, log(. + guard)
 *   :586-620 normalizeFeatures       per mel row over featuresLen = floor(N/160) frames: mean, variance with N-1,
 *                                    (x - mean) / (sqrt(var) + 1e-5), sums in doubles
 * JavaScript numbers are doubles; values stored into a Float32Array are rounded to f32 at that point.
 *
 * Pinning: this code path is plain JavaScript in the reference (no compiled form ships), and no JavaScript
 * runtime exists on the build machines, so it cannot be executed: parity unpinned for this file.  It is checked
 * against an independent numpy formulation (rfft-based) of the same pipeline in tests/test_mel_oracle.py.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define EXPORT __attribute__((visibility("default")))

enum { SR = 16000, N_FFT = 512, WIN = 400, HOP = 160, NBINS = 257 };
static const double PREEMPH = 0.97;

static double hz_to_mel(double f) { return f >= 1000.0 ? 15.0 + log(f / 1000.0) / (log(6.4) / 27.0) : f / (200.0 / 3); }
static double mel_to_hz(double m) { return m >= 15.0 ? 1000.0 * exp((log(6.4) / 27.0) * (m - 15.0)) : m * (200.0 / 3); }

/* fb: [nMels][257] f32; bounds: [nMels][2] (first non-zero bin, one past the last). */
EXPORT void mel_filterbank(int nMels, float *fb, int32_t *bounds) {
  double allf[NBINS];
  for (int i = 0; i < NBINS; i++) allf[i] = (8000.0 * i) / (NBINS - 1);
  int np = nMels + 2;
  double *pts = (double *)malloc(sizeof(double) * np), *diff = (double *)malloc(sizeof(double) * (np - 1));
  double mmin = hz_to_mel(0.0), mmax = hz_to_mel(8000.0);
  for (int i = 0; i < np; i++) pts[i] = mel_to_hz(mmin + ((mmax - mmin) * i) / (np - 1));
  for (int i = 0; i < np - 1; i++) diff[i] = pts[i + 1] - pts[i];
  for (int m = 0; m < nMels; m++) {
    double enorm = 2.0 / (pts[m + 2] - pts[m]);
    int start = -1, end = -1;
    for (int k = 0; k < NBINS; k++) {
      double down = (allf[k] - pts[m]) / diff[m], up = (pts[m + 2] - allf[k]) / diff[m + 1];
      double v = fmax(0.0, fmin(down, up)) * enorm;
      fb[m * NBINS + k] = (float)v;
      if (fb[m * NBINS + k] > 0) {
        if (start < 0) start = k;
        end = k;
      }
    }
    if (start < 0) { start = 0; end = -1; }
    bounds[2 * m] = start;
    bounds[2 * m + 1] = end + 1;
  }
  free(pts);
  free(diff);
}

EXPORT void mel_hann_window(double *w) {
  memset(w, 0, sizeof(double) * N_FFT);
  for (int n = 0; n < WIN; n++) w[((N_FFT - WIN) >> 1) + n] = 0.5 * (1 - cos((2 * M_PI * n) / (WIN - 1)));
}

EXPORT void mel_twiddles(int N, double *c, double *s) {
  for (int i = 0; i < N / 2; i++) {
    double a = (-2 * M_PI * i) / N;
    c[i] = cos(a);
    s[i] = sin(a);
  }
}

static void fft_inplace(double *re, double *im, int N, const double *twc, const double *tws) {
  int bits = 0;
  while ((1 << bits) < N) bits++;
  for (int i = 0; i < N; i++) {
    int x = i, r = 0;
    for (int b = 0; b < bits; b++) { r = (r << 1) | (x & 1); x >>= 1; }
    if (i < r) {
      double t = re[i]; re[i] = re[r]; re[r] = t;
      t = im[i]; im[i] = im[r]; im[r] = t;
    }
  }
  /* The reference unrolls the first three stages with the constants 1, -i and sqrt(1/2); the table entries they
   * stand for are equal to those constants, so one loop serves every stage. */
  for (int len = 2; len <= N; len <<= 1) {
    int half = len >> 1, step = N / len;
    for (int i = 0; i < N; i += len)
      for (int k = 0; k < half; k++) {
        double wc = twc[k * step], ws = tws[k * step];
        if (len == 2) { wc = 1; ws = 0; }
        if (len == 4 && k == 1) { wc = 0; ws = -1; }
        if (len == 8) {
          const double r = M_SQRT1_2;
          if (k == 1) { wc = r; ws = -r; }
          if (k == 2) { wc = 0; ws = -1; }
          if (k == 3) { wc = -r; ws = -r; }
        }
        int p = i + k, q = p + half;
        double tr = re[q] * wc - im[q] * ws, ti = re[q] * ws + im[q] * wc;
        re[q] = re[p] - tr; im[q] = im[p] - ti;
        re[p] += tr; im[p] += ti;
      }
  }
}

/* raw: [nMels][nFrames] with nFrames = N/160 + 1 (for N >= 1); returns featuresLen = floor(N/160). */
EXPORT int mel_compute_raw(const float *audio, int N, int nMels, double logGuard, float *raw, int *nFramesOut) {
  if (N <= 0) { *nFramesOut = 0; return 0; }
  const int pad = N_FFT >> 1, paddedLen = N + 2 * pad;
  const int nFrames = (paddedLen - N_FFT) / HOP + 1, featLen = N / HOP;
  *nFramesOut = nFrames;
  if (featLen == 0) return 0;
  double *padded = (double *)calloc(paddedLen, sizeof(double));
  padded[pad] = (double)audio[0];
  for (int i = 1; i < N; i++) padded[pad + i] = (double)(float)((double)audio[i] - PREEMPH * (double)audio[i - 1]);
  float *fb = (float *)malloc(sizeof(float) * nMels * NBINS);
  int32_t *bounds = (int32_t *)malloc(sizeof(int32_t) * nMels * 2);
  mel_filterbank(nMels, fb, bounds);
  double win[N_FFT], twc[N_FFT / 2], tws[N_FFT / 2], hc[N_FFT / 4], hs[N_FFT / 4];
  mel_hann_window(win);
  mel_twiddles(N_FFT, twc, tws);
  mel_twiddles(N_FFT / 2, hc, hs);
  const int halfN = N_FFT >> 1, quarterN = halfN >> 1;
  double re[N_FFT / 2], im[N_FFT / 2];
  float power[NBINS];
  for (int t = 0; t < nFrames; t++) {
    const int off = t * HOP;
    for (int k = 0; k < halfN; k++) {
      re[k] = padded[off + 2 * k] * win[2 * k];
      im[k] = padded[off + 2 * k + 1] * win[2 * k + 1];
    }
    fft_inplace(re, im, halfN, hc, hs);
    double z0r = re[0], z0i = im[0];
    power[0] = (float)((z0r + z0i) * (z0r + z0i));
    power[halfN] = (float)((z0r - z0i) * (z0r - z0i));
    for (int k = 1; k < quarterN; k++) {
      double rk = re[k], ik = im[k], rnk = re[halfN - k], ink = im[halfN - k];
      double xeR = 0.5 * (rk + rnk), xeI = 0.5 * (ik - ink), xoR = 0.5 * (ik + ink), xoI = -0.5 * (rk - rnk);
      double wc = twc[k], ws = tws[k];
      double tr = xoR * wc - xoI * ws, ti = xoR * ws + xoI * wc;
      double xkR = xeR + tr, xkI = xeI + ti;
      power[k] = (float)(xkR * xkR + xkI * xkI);
      double xnR = xeR - tr, xnI = xeI - ti;
      power[halfN - k] = (float)(xnR * xnR + xnI * xnI);
    }
    power[quarterN] = (float)(re[quarterN] * re[quarterN] + im[quarterN] * im[quarterN]);
    for (int m = 0; m < nMels; m++) {
      double v = 0;
      for (int k = bounds[2 * m]; k < bounds[2 * m + 1]; k++) v += (double)power[k] * (double)fb[m * NBINS + k];
      raw[(size_t)m * nFrames + t] = (float)log(v + logGuard);
    }
  }
  free(padded);
  free(fb);
  free(bounds);
  return featLen;
}

/* features: [nMels][featLen] from raw [nMels][nFrames]. */
EXPORT void mel_normalize(const float *raw, int nMels, int nFrames, int featLen, float *features) {
  for (int m = 0; m < nMels; m++) {
    const float *src = raw + (size_t)m * nFrames;
    float *dst = features + (size_t)m * featLen;
    double sum = 0;
    for (int t = 0; t < featLen; t++) sum += src[t];
    double mean = sum / featLen, var = 0;
    for (int t = 0; t < featLen; t++) {
      double d = src[t] - mean;
      var += d * d;
    }
    double inv = featLen > 1 ? 1.0 / (sqrt(var / (featLen - 1)) + 1e-5) : 0;
    for (int t = 0; t < featLen; t++) dst[t] = (float)((src[t] - mean) * inv);
  }
}
