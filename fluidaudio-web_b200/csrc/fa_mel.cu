// NeMo-style log-mel front end on the GPU, for whole batches of equal-length windows.
//
// The reference computes log-mel on the host (a worker thread per window): ParakeetMel.process
// (src/engines/asr-parakeet/parakeet-mel.js:16-21) = JsPreprocessor.computeRawMel + normalizeFeatures
// (src/engines/asr-nemotron/nemotron-mel.js:451-573, 586-620).  Same pipeline here, same arithmetic types:
//   pre-emphasis 0.97 rounded to f32 | 256 zeros either side | per frame (hop 160): 512 samples x symmetric Hann(400)
//   centred in the frame, in doubles | one 256-point complex FFT (radix 2, decimation in time, doubles) of the
//   even/odd samples + real-spectrum reconstruction | power stored as f32 | slaney filterbank (f32 weights) summed in
//   a double over each filter's non-zero span | log(. + guard) stored as f32 | per mel row over floor(N/160) frames:
//   mean, variance with N-1, (x - mean) / (sqrt(var) + 1e-5), sums in doubles.
// Doubles are affordable here (48k frames of 256-point FFTs are ~1 GFLOP per 32-window batch; the kernel is paced by
// shared-memory traffic and instruction issue, not by the FP64 pipe) and they keep the result within rounding of the
// reference's.  Multiplies and adds are kept separate (no fused multiply-add)
// where the JavaScript has them separate.
//
// One warp transforms one frame (three stages in registers, five in shared memory: see k_mel_raw); the filterbank,
// window and twiddle tables are built on the host in doubles with the reference's formulas, once per context and
// mel count.
#include <cmath>

#include "fa_internal.cuh"

namespace {

constexpr int kNfft = 512, kHalf = 256, kQuarter = 128, kBins = 257, kHop = 160, kWin = 400;
constexpr int kWarps = 8, kFramesPerWarp = 4;
constexpr int kStageTw = 8 + 16 + 32 + 64 + 128;  // twiddles of the five shared-memory stages, stage by stage

// Shared-memory layout of a frame's 256 complex points: one spare double after every 16.  With it the 64-bit stores
// that follow the register stages (a lane owns 8 consecutive points: stride 8) and the butterflies of the stages
// with 16 or more points per half touch every bank once per half-warp; without it the strided stores were 16-way
// conflicts and shared-memory wavefronts paced the kernel.
constexpr int kPadLen = kHalf + kHalf / 16;
__device__ __forceinline__ int pad16(int i) { return i + (i >> 4); }

struct MelTables {
  const float *fbt;      // [maxSpan][nMels]: weight j of filter m's non-zero span (a warp reads one j of 32 filters at once)
  const int *bounds;     // [nMels][2]
  int maxSpan;
  const double *win;     // [512]
  const double *twc, *tws;  // cos/sin(-2 pi i / 512), i < 256
  const double *sc, *ss;    // per stage with 8, 16, .. 128 butterflies per group: cos/sin(-2 pi k / (2 * half)), k < half
};

__device__ __forceinline__ double padded_sample(const float *audio, int N, int i) {  // i: index into the padded signal
  const int j = i - kHalf;
  if (j < 0 || j >= N) return 0.0;
  if (j == 0) return (double)audio[0];
  return (double)(float)__dsub_rn((double)audio[j], __dmul_rn(0.97, (double)audio[j - 1]));
}

// One radix-2 butterfly of the reference's transform: q <- p - w q, p <- p + w q, multiplies and adds separate.
__device__ __forceinline__ void butterfly(double &rp, double &ip, double &rq, double &iq, double wc, double ws) {
  const double tr = __dsub_rn(__dmul_rn(rq, wc), __dmul_rn(iq, ws));
  const double ti = __dadd_rn(__dmul_rn(rq, ws), __dmul_rn(iq, wc));
  rq = __dsub_rn(rp, tr);
  iq = __dsub_rn(ip, ti);
  rp = __dadd_rn(rp, tr);
  ip = __dadd_rn(ip, ti);
}

// raw[w][m][t] = log(mel power + guard), t < nFrames.
// One warp transforms one frame.  A lane reads the 8 points that land (bit-reversed) on positions 8*lane .. 8*lane+7 -
// for each of the 8 a warp reads one permuted run of 32 consecutive input pairs - and runs the first three stages on
// them in registers (with the exact constants 1, -i and sqrt(1/2) the reference uses there); the other five stages
// go through shared memory.  Every butterfly is the same arithmetic on the same operands as a stage-by-stage
// transform, so the result does not depend on this schedule.
__global__ void __launch_bounds__(32 * kWarps) k_mel_raw(const float *__restrict__ audio, int N, int nFrames, int nMels,
                                                         double guard, MelTables tb, float *__restrict__ raw) {
  __shared__ double re_s[kWarps][kPadLen], im_s[kWarps][kPadLen];
  __shared__ float pw_s[kWarps][kBins + 3];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, w = blockIdx.y;
  double *re = re_s[warp], *im = im_s[warp];
  float *power = pw_s[warp];
  const float *au = audio + (size_t)w * N;
  const int src_lo = (int)(__brev((unsigned)lane) >> 27);  // the low five bits of the source index of this lane's points
  const double w0c = tb.sc[0], w0s = tb.ss[0];              // the table's own (1, -0) for k = 0
  fa_grid_dep_sync();
  for (int f = 0; f < kFramesPerWarp; f++) {
    const int t = (blockIdx.x * kWarps + warp) * kFramesPerWarp + f;
    if (t >= nFrames) break;  // warp-uniform
    const int off = t * kHop;
    double xr[8], xi[8];
#pragma unroll
    for (int c = 0; c < 8; c++) {
      const int k = (int)((__brev((unsigned)c) >> 29) << 5) | src_lo, idx = 2 * k;  // k = 8-bit reversal of 8*lane + c
      xr[c] = __dmul_rn(padded_sample(au, N, off + idx), tb.win[idx]);
      xi[c] = __dmul_rn(padded_sample(au, N, off + idx + 1), tb.win[idx + 1]);
    }
    const double r2 = 0.70710678118654752440;
    // groups of 2: w = 1
    butterfly(xr[0], xi[0], xr[1], xi[1], 1.0, 0.0);
    butterfly(xr[2], xi[2], xr[3], xi[3], 1.0, 0.0);
    butterfly(xr[4], xi[4], xr[5], xi[5], 1.0, 0.0);
    butterfly(xr[6], xi[6], xr[7], xi[7], 1.0, 0.0);
    // groups of 4: k = 0 from the table, k = 1 is -i
    butterfly(xr[0], xi[0], xr[2], xi[2], w0c, w0s);
    butterfly(xr[1], xi[1], xr[3], xi[3], 0.0, -1.0);
    butterfly(xr[4], xi[4], xr[6], xi[6], w0c, w0s);
    butterfly(xr[5], xi[5], xr[7], xi[7], 0.0, -1.0);
    // groups of 8
    butterfly(xr[0], xi[0], xr[4], xi[4], w0c, w0s);
    butterfly(xr[1], xi[1], xr[5], xi[5], r2, -r2);
    butterfly(xr[2], xi[2], xr[6], xi[6], 0.0, -1.0);
    butterfly(xr[3], xi[3], xr[7], xi[7], -r2, -r2);
#pragma unroll
    for (int c = 0; c < 8; c++) {
      re[pad16(8 * lane + c)] = xr[c];
      im[pad16(8 * lane + c)] = xi[c];
    }
    __syncwarp();
    int tw_off = 0;
    for (int half = 8; half <= kQuarter; half <<= 1) {
#pragma unroll
      for (int i = 0; i < kQuarter / 32; i++) {
        const int bf = lane + 32 * i, grp = bf / half, k = bf - grp * half;
        const int p = pad16(grp * 2 * half + k), q = pad16(grp * 2 * half + k + half);
        double rp = re[p], ip = im[p], rq = re[q], iq = im[q];
        butterfly(rp, ip, rq, iq, tb.sc[tw_off + k], tb.ss[tw_off + k]);
        re[q] = rq;
        im[q] = iq;
        re[p] = rp;
        im[p] = ip;
      }
      tw_off += half;
      __syncwarp();
    }
    // spectrum of the 512 real samples from the 256-point transform of (even, odd) pairs; power as f32
    if (lane == 0) {
      const double z0r = re[0], z0i = im[0];
      const double s = __dadd_rn(z0r, z0i), d = __dsub_rn(z0r, z0i);
      power[0] = (float)__dmul_rn(s, s);
      power[kHalf] = (float)__dmul_rn(d, d);
      const double rq = re[pad16(kQuarter)], iq = im[pad16(kQuarter)];
      power[kQuarter] = (float)__dadd_rn(__dmul_rn(rq, rq), __dmul_rn(iq, iq));
    }
#pragma unroll
    for (int i = 0; i < kQuarter / 32; i++) {
      const int k = lane + 32 * i;
      if (k >= 1) {
        const double rk = re[pad16(k)], ik = im[pad16(k)], rnk = re[pad16(kHalf - k)], ink = im[pad16(kHalf - k)];
        const double xeR = __dmul_rn(0.5, __dadd_rn(rk, rnk)), xeI = __dmul_rn(0.5, __dsub_rn(ik, ink));
        const double xoR = __dmul_rn(0.5, __dadd_rn(ik, ink)), xoI = __dmul_rn(-0.5, __dsub_rn(rk, rnk));
        const double wc = tb.twc[k], ws = tb.tws[k];
        const double tr = __dsub_rn(__dmul_rn(xoR, wc), __dmul_rn(xoI, ws));
        const double ti = __dadd_rn(__dmul_rn(xoR, ws), __dmul_rn(xoI, wc));
        const double xkR = __dadd_rn(xeR, tr), xkI = __dadd_rn(xeI, ti);
        power[k] = (float)__dadd_rn(__dmul_rn(xkR, xkR), __dmul_rn(xkI, xkI));
        const double xnR = __dsub_rn(xeR, tr), xnI = __dsub_rn(xeI, ti);
        power[kHalf - k] = (float)__dadd_rn(__dmul_rn(xnR, xnR), __dmul_rn(xnI, xnI));
      }
    }
    __syncwarp();
    for (int m = lane; m < nMels; m += 32) {
      const int k0 = tb.bounds[2 * m], n = tb.bounds[2 * m + 1] - k0;
      double v = 0.0;
      for (int j = 0; j < n; j++) v = __dadd_rn(v, __dmul_rn((double)power[k0 + j], (double)tb.fbt[(size_t)j * nMels + m]));
      raw[((size_t)w * nMels + m) * nFrames + t] = (float)log(v + guard);
    }
    __syncwarp();
  }
}

// stats[w][m] = {mean, 1 / (sqrt(var) + 1e-5)} over the first featLen frames of raw[w][m][:]
__global__ void __launch_bounds__(256) k_mel_stats(const float *__restrict__ raw, int nFrames, int featLen, double *__restrict__ stats) {
  __shared__ double red[8];
  fa_grid_dep_sync();
  const float *row = raw + (size_t)blockIdx.x * nFrames;
  auto block_sum = [&](double v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    double t = 0.0;
    for (int i = 0; i < 8; i++) t += red[i];
    return t;
  };
  double s = 0.0;
  for (int t = threadIdx.x; t < featLen; t += blockDim.x) s += (double)row[t];
  const double mean = block_sum(s) / (double)featLen;
  double v = 0.0;
  for (int t = threadIdx.x; t < featLen; t += blockDim.x) {
    const double d = (double)row[t] - mean;
    v += d * d;
  }
  const double var = block_sum(v);
  if (threadIdx.x == 0) {
    stats[2 * blockIdx.x] = mean;
    stats[2 * blockIdx.x + 1] = featLen > 1 ? 1.0 / (sqrt(var / (double)(featLen - 1)) + 1e-5) : 0.0;
  }
}

// out[w][t][m] (time-major, what the encoder's front end reads) = (raw[w][m][t] - mean) * inv, or raw as is
__global__ void __launch_bounds__(256) k_mel_apply(const float *__restrict__ raw, const double *__restrict__ stats, int nMels,
                                                   int nFrames, int outLen, float *__restrict__ out) {
  __shared__ float tile[32][33];
  fa_grid_dep_sync();
  const int w = blockIdx.z, m0 = blockIdx.y * 32, t0 = blockIdx.x * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  for (int r = ty; r < 32; r += 8) {
    const int m = m0 + r, t = t0 + tx;
    float v = 0.f;
    if (m < nMels && t < outLen) {
      const float x = raw[((size_t)w * nMels + m) * nFrames + t];
      v = stats ? (float)(((double)x - stats[2 * ((size_t)w * nMels + m)]) * stats[2 * ((size_t)w * nMels + m) + 1]) : x;
    }
    tile[r][tx] = v;
  }
  __syncthreads();
  for (int r = ty; r < 32; r += 8) {
    const int t = t0 + r, m = m0 + tx;
    if (t < outLen && m < nMels) out[((size_t)w * outLen + t) * nMels + m] = tile[tx][r];
  }
}

double hz_to_mel(double f) { return f >= 1000.0 ? 15.0 + std::log(f / 1000.0) / (std::log(6.4) / 27.0) : f / (200.0 / 3); }
double mel_to_hz(double m) { return m >= 15.0 ? 1000.0 * std::exp((std::log(6.4) / 27.0) * (m - 15.0)) : m * (200.0 / 3); }

}  // namespace

// Tables of one mel count: [maxSpan i32, pad | bounds i32 nMels*2 | fbt f32 maxSpan*nMels | (8-byte aligned) win 512 |
// twc 256 | tws 256 | sc 248 | ss 248 doubles], built with the formulas of nemotron-mel.js:66-110 (filterbank),
// :131-141 (window), :158-171 (twiddles).  The filterbank is kept as each filter's non-zero span, transposed; the
// stage twiddles are the reference's cos/sin(-2 pi i / 256) table read at i = k * (128 / half), stage by stage.
static int mel_tables(fa_ctx *ctx, int nMels, MelTables *out) {
  auto it = ctx->mel_tables.find(nMels);
  if (it == ctx->mel_tables.end()) {
    std::vector<float> fb((size_t)nMels * kBins);
    std::vector<int> bnd((size_t)nMels * 2);
    std::vector<double> allf(kBins), pts(nMels + 2), diff(nMels + 1);
    for (int i = 0; i < kBins; i++) allf[i] = (8000.0 * i) / (kBins - 1);
    const double mmin = hz_to_mel(0.0), mmax = hz_to_mel(8000.0);
    for (int i = 0; i < nMels + 2; i++) pts[i] = mel_to_hz(mmin + ((mmax - mmin) * i) / (nMels + 1));
    for (int i = 0; i < nMels + 1; i++) diff[i] = pts[i + 1] - pts[i];
    int max_span = 1;
    for (int m = 0; m < nMels; m++) {
      const double enorm = 2.0 / (pts[m + 2] - pts[m]);
      int start = -1, end = -1;
      for (int k = 0; k < kBins; k++) {
        const double down = (allf[k] - pts[m]) / diff[m], up = (pts[m + 2] - allf[k]) / diff[m + 1];
        const float v = (float)(std::fmax(0.0, std::fmin(down, up)) * enorm);
        fb[(size_t)m * kBins + k] = v;
        if (v > 0) {
          if (start < 0) start = k;
          end = k;
        }
      }
      if (start < 0) { start = 0; end = -1; }
      bnd[2 * m] = start;
      bnd[2 * m + 1] = end + 1;
      max_span = std::max(max_span, end + 1 - start);
    }
    const size_t b_n = (size_t)nMels * 2, fbt_n = (size_t)max_span * nMels;
    const size_t off_d = round_up(8 + b_n * 4 + fbt_n * 4, 8), total = off_d + (size_t)(512 + 256 + 256 + 2 * kStageTw) * 8;
    std::vector<unsigned char> host(total, 0);
    ((int *)host.data())[0] = max_span;
    int *bounds = (int *)(host.data() + 8);
    float *fbt = (float *)(host.data() + 8 + b_n * 4);
    double *win = (double *)(host.data() + off_d), *twc = win + 512, *tws = twc + 256, *sc = tws + 256, *ss = sc + kStageTw;
    for (size_t i = 0; i < b_n; i++) bounds[i] = bnd[i];
    for (int m = 0; m < nMels; m++)
      for (int j = 0; j < bnd[2 * m + 1] - bnd[2 * m]; j++) fbt[(size_t)j * nMels + m] = fb[(size_t)m * kBins + bnd[2 * m] + j];
    for (int n = 0; n < kWin; n++) win[((kNfft - kWin) >> 1) + n] = 0.5 * (1 - std::cos((2 * M_PI * n) / (kWin - 1)));
    for (int i = 0; i < 256; i++) { const double a = (-2 * M_PI * i) / 512; twc[i] = std::cos(a); tws[i] = std::sin(a); }
    double hc[128], hs[128];
    for (int i = 0; i < 128; i++) { const double a = (-2 * M_PI * i) / 256; hc[i] = std::cos(a); hs[i] = std::sin(a); }
    for (int half = 8, o = 0; half <= 128; o += half, half <<= 1)
      for (int k = 0; k < half; k++) { sc[o + k] = hc[k * (128 / half)]; ss[o + k] = hs[k * (128 / half)]; }
    FA_REQUIRE(ctx, !ctx->capturing, "logMelWindows: the tables of a mel count are built on first use, which must not happen "
                                     "inside a recording; run the sequence once eagerly before fa_graph_begin");
    void *dev = nullptr;
    FA_TRY(fa_block_acquire_global(ctx, round_up(total, 256), &dev));
    FA_CHECK_CUDA(ctx, cudaMemcpyAsync(dev, host.data(), total, cudaMemcpyHostToDevice, ctx->stream));
    FA_CHECK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));  // the host vector goes away
    it = ctx->mel_tables.emplace(nMels, dev).first;
    ctx->mel_spans[nMels] = max_span;
  }
  const unsigned char *base = (const unsigned char *)it->second;
  const int max_span = ctx->mel_spans[nMels];
  const size_t b_n = (size_t)nMels * 2, off_d = round_up(8 + b_n * 4 + (size_t)max_span * nMels * 4, 8);
  out->maxSpan = max_span;
  out->bounds = (const int *)(base + 8);
  out->fbt = (const float *)(base + 8 + b_n * 4);
  out->win = (const double *)(base + off_d);
  out->twc = out->win + 512;
  out->tws = out->twc + 256;
  out->sc = out->tws + 256;
  out->ss = out->sc + kStageTw;
  return FA_OK;
}

extern "C" int fa_log_mel_windows(fa_ctx *ctx, const fa_tensor *audio, int n_mels, double log_guard, int normalize,
                                  fa_tensor **out) {
  if (!ctx || !out) return fa_fail(ctx, FA_ERR_INVALID, "logMelWindows: NULL argument");
  FA_REQUIRE(ctx, fa_valid(ctx, audio), "logMelWindows: unknown tensor handle");
  FA_REQUIRE(ctx, audio->storage == FA_F32, "logMelWindows: audio must be f32 storage");
  FA_REQUIRE(ctx, n_mels >= 1 && n_mels <= 256, "logMelWindows: n_mels=%d is outside 1..256", n_mels);
  const int W = audio->rows, N = audio->cols;
  FA_REQUIRE(ctx, W >= 1 && N >= kHop, "logMelWindows: %d windows of %d samples (at least %d samples needed)", W, N, kHop);
  FA_CHECK_CUDA(ctx, cudaSetDevice(ctx->device));
  FA_TRY(fa_touch_f32(ctx, audio));
  const int nFrames = N / kHop + 1, featLen = N / kHop, outLen = normalize ? featLen : nFrames;
  MelTables tb;
  FA_TRY(mel_tables(ctx, n_mels, &tb));
  void *raw = nullptr, *stats = nullptr;
  size_t rb = 0, sb = 0;
  FA_TRY(fa_block_acquire(ctx, (size_t)W * n_mels * nFrames * 4, &raw, &rb));
  fa_tensor *y = nullptr;
  int rc = fa_tensor_new(ctx, W, outLen * n_mels, FA_F32, true, &y);
  if (rc == FA_OK && normalize) rc = fa_block_acquire(ctx, (size_t)W * n_mels * 16, &stats, &sb);
  if (rc == FA_OK) {
    {
      LaunchScope ls(ctx, "mel_raw");
      fa_launch_dep(ctx, k_mel_raw, dim3(ceil_div(nFrames, kWarps * kFramesPerWarp), W), dim3(32 * kWarps), 0,
                    (const float *)audio->dptr, N, nFrames, n_mels, log_guard, tb, (float *)raw);
    }
    if (normalize) {
      LaunchScope ls(ctx, "mel_stats");
      fa_launch_dep(ctx, k_mel_stats, dim3(W * n_mels), dim3(256), 0, (const float *)raw, nFrames, featLen, (double *)stats);
    }
    {
      LaunchScope ls(ctx, "mel_apply");
      fa_launch_dep(ctx, k_mel_apply, dim3(ceil_div(outLen, 32), ceil_div(n_mels, 32), W), dim3(256), 0, (const float *)raw,
                    (const double *)stats, n_mels, nFrames, outLen, (float *)y->dptr);
    }
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) rc = fa_fail(ctx, FA_ERR_CUDA, "launch logMelWindows: %s", cudaGetErrorString(e));
  }
  fa_block_release(ctx, raw);
  if (stats) fa_block_release(ctx, stats);
  if (rc != FA_OK) {
    if (y) fa_free_tensor(ctx, y);
    return rc;
  }
  *out = y;
  return FA_OK;
}
