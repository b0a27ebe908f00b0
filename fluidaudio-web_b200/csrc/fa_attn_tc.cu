// Attention products (bmmQK / bmmPV, src/gpu/kernels/attention.js:14-146) on the tensor cores.
//
// Each (window, head) pair is one small product; all of them go through ONE launch of the batched
// tcgen05 GEMM (fa_gemm_tc.cu).  The operands are cut out of the head-strided [T, H*HD] projections and
// written as f16 in the GEMM's box-contiguous layouts by the pack kernels below:
//   QK^T : streamed ("weight") side = keys  b[j, h*HD + d]   -> Wp[batch][j/128][d/64][j%128][d%64]
//          row ("activation") side  = q + qb                  -> Ap[batch][d/64][i][d%64]
//   P@V  : streamed side = V transposed  v[j, h*HD + d]       -> Wp[batch][d/128][j/64][d%128][j%64]
//          row side      = probabilities p[(batch*Tq + i), j] -> Ap[batch][j/64][i][j%64]
// Accumulation is f32 in TMEM; only the operands are rounded to f16.
#include "fa_internal.cuh"

namespace {

// rows r of src[(w*T + r) * S + h*HD + d] (+ addv[h*HD + d]) -> Ap[batch][d/64][r][d%64], d zero padded.
// Grid (row groups of 8, K chunks, batch = w*H + h): a warp packs one 64-wide chunk of one row, so the only
// division left is the one per thread that splits the batch index.
__global__ void __launch_bounds__(256) k_pack_act_heads(const float *__restrict__ src, const float *__restrict__ addv,
                                                        const float *__restrict__ addv2, __half *__restrict__ dst,
                                                        __half *__restrict__ dst2, int T, int S, int H, int HD, int nch) {
  fa_grid_dep_sync();
  // dst2 (optional): the same rows with a second bias vector - the content and the positional query of
  // relative-position attention (q + u, q + v) from one read of q
  const int pr = threadIdx.x & 31, r = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (r >= T) return;
  const int c = blockIdx.y, batch = blockIdx.z, w = batch / H, h = batch - w * H, d = c * 64 + pr * 2;
  float x = 0.f, y = 0.f, x2 = 0.f, y2 = 0.f;
  const float *row = src + ((size_t)w * T + r) * S + h * HD;
  if (d + 1 < HD) {
    const float2 v = *(const float2 *)(row + d);
    x = x2 = v.x, y = y2 = v.y;
    if (addv) {
      const float2 a = *(const float2 *)(addv + h * HD + d);
      x += a.x, y += a.y;
    }
    if (dst2 && addv2) {
      const float2 a = *(const float2 *)(addv2 + h * HD + d);
      x2 += a.x, y2 += a.y;
    }
  } else if (d < HD) {
    x = x2 = row[d];
    if (addv) x += addv[h * HD + d];
    if (dst2 && addv2) x2 += addv2[h * HD + d];
  }
  const size_t o = (((size_t)batch * nch + c) * T + r) * 32 + pr;
  ((__half2 *)dst)[o] = __floats2half2_rn(x, y);
  if (dst2) ((__half2 *)dst2)[o] = __floats2half2_rn(x2, y2);
}

// keys: src[(wsrc*Tb + j) * S + h*HD + d] -> Wp[batch][j/128][d/64][j%128][d%64]; rows j >= Tb and d >= HD zero.
// Grid (16 row groups of 8 per 128-row tile, tiles_n * nch, batch).
__global__ void __launch_bounds__(256) k_pack_w_heads(const float *__restrict__ src, __half *__restrict__ dst, int Tb, int S,
                                                      int H, int HD, int tiles_n, int nch, int w_shared) {
  fa_grid_dep_sync();
  const int pr = threadIdx.x & 31, jr = blockIdx.x * 8 + (threadIdx.x >> 5);
  const int tn = blockIdx.y / nch, c = blockIdx.y - tn * nch, batch = blockIdx.z;
  const int w = w_shared ? 0 : batch / H, h = batch % H, j = tn * 128 + jr, d = c * 64 + pr * 2;
  float x = 0.f, y = 0.f;
  if (j < Tb) {
    const float *row = src + ((size_t)w * Tb + j) * S + h * HD;
    if (d + 1 < HD) {
      const float2 v = *(const float2 *)(row + d);
      x = v.x, y = v.y;
    } else if (d < HD) {
      x = row[d];
    }
  }
  ((__half2 *)dst)[((((size_t)batch * tiles_n + tn) * nch + c) * 128 + jr) * 32 + pr] = __floats2half2_rn(x, y);
}

// probabilities: p[(batch*Tq + r) * Tk + j] -> Ap[batch][j/64][r][j%64], j zero padded
__global__ void k_pack_act_probs(const float *__restrict__ p, __half *__restrict__ dst, int Tq, int Tk, int nch,
                                 unsigned total) {
  fa_grid_dep_sync();
  for (unsigned i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
    const int pr = i & 31;
    unsigned t = i >> 5;
    const int r = t % Tq;
    t /= Tq;
    const int c = t % nch, batch = t / nch;
    const int j = c * 64 + pr * 2;
    const float *row = p + ((size_t)batch * Tq + r) * Tk;
    float x = j < Tk ? row[j] : 0.f, y = j + 1 < Tk ? row[j + 1] : 0.f;
    ((__half2 *)dst)[i] = __floats2half2_rn(x, y);
  }
}

// values transposed: v[(w*Tk + j) * S + h*HD + d] -> Wp[batch][d/128][j/64][d%128][j%64].
// One CTA per (batch, 64-key chunk): the 64 x HD slab goes through shared memory.
__global__ void __launch_bounds__(256) k_pack_w_vT(const float *__restrict__ v, __half *__restrict__ dst, int Tk, int S,
                                                   int H, int HD, int tiles_n, int nch) {
  fa_grid_dep_sync();
  extern __shared__ float tile[];  // [64 keys][HD + 1]
  const int batch = blockIdx.x / nch, c = blockIdx.x % nch;
  const int w = batch / H, h = batch % H, ldt = HD + 1;
  for (int jj = threadIdx.x >> 5; jj < 64; jj += 8) {  // a warp per key row, lanes along the head dimension
    const int j = c * 64 + jj;
    const float *row = v + ((size_t)w * Tk + (j < Tk ? j : Tk - 1)) * S + h * HD;
    for (int d = threadIdx.x & 31; d < HD; d += 32) tile[jj * ldt + d] = j < Tk ? row[d] : 0.f;
  }
  __syncthreads();
  // dst rows: for each d (padded to tiles_n*128), 64 keys = 32 half2
  for (int e = threadIdx.x; e < tiles_n * 128 * 32; e += 256) {
    const int pr = e & 31, dr = e >> 5;  // dr = d within [0, tiles_n*128)
    const int tn = dr >> 7, dl = dr & 127;
    float x = 0.f, y = 0.f;
    if (dr < HD) {
      x = tile[(pr * 2) * ldt + dr];
      y = tile[(pr * 2 + 1) * ldt + dr];
    }
    const size_t o = ((((size_t)batch * tiles_n + tn) * nch + c) * 128 + dl) * 32 + pr;
    ((__half2 *)dst)[o] = __floats2half2_rn(x, y);
  }
}

// softmax over j of ac[i][j] + bd[i][T-1-i+j] (the rel-shifted positional scores, see k_rel_shift_b),
// written straight into the packed f16 row operand of the P@V product: Ap[batch][j/64][i][j%64], the
// K tail zero filled.  One warp per score row, the row held in registers (T <= 256).
__global__ void k_softmax_shift_pack(const float *__restrict__ ac, const float *__restrict__ bd, __half *__restrict__ dst,
                                     int rows, int T, int nch) {
  fa_grid_dep_sync();
  const int warps = blockDim.x >> 5, lane = threadIdx.x & 31, P = 2 * T - 1;
  for (int r = blockIdx.x * warps + (threadIdx.x >> 5); r < rows; r += gridDim.x * warps) {
    const int batch = r / T, i = r - batch * T;
    const float *a = ac + (size_t)r * T;
    const float *b = bd + (size_t)r * P + (T - 1 - i);
    float v[8];
    float mx = -INFINITY;
#pragma unroll
    for (int u = 0; u < 8; u++) {
      const int j = lane + 32 * u;
      v[u] = j < T ? a[j] + b[j] : -INFINITY;
      mx = fmaxf(mx, v[u]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float s = 0.f;
#pragma unroll
    for (int u = 0; u < 8; u++) {
      v[u] = lane + 32 * u < T ? expf(v[u] - mx) : 0.f;
      s += v[u];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    const float inv = 1.0f / s;
#pragma unroll
    for (int u = 0; u < 8; u++) {
      const int j = lane + 32 * u;
      if (j < nch * 64) dst[(((size_t)batch * nch + (j >> 6)) * T + i) * 64 + (j & 63)] = __float2half_rn(v[u] * inv);
    }
  }
}

int grid_for(fa_ctx *ctx, size_t n) {
  size_t g = (n + 255) / 256, cap = (size_t)ctx->sm_count * 16;
  return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}

struct Block {
  fa_ctx *ctx;
  void *p = nullptr;
  size_t bytes = 0;
  explicit Block(fa_ctx *c) : ctx(c) {}
  int get(size_t need) { return fa_block_acquire(ctx, need, &p, &bytes); }
  ~Block() {
    if (p) fa_block_release(ctx, p);
  }
};

}  // namespace

static bool qk_shape_ok(fa_ctx *ctx, int T, int Tb, int H, int HD, int W, size_t *a_halves, size_t *w_halves, int b_shared) {
  const long long batches = (long long)W * H;
  if (!fa_tc_available(ctx) || HD < 64 || T < 32 || Tb < 32 || T > 256 || batches * T * Tb * HD < (1ll << 22)) return false;
  const int nch = ceil_div(HD, 64), tiles_n = ceil_div(Tb, 128);
  const int wb = b_shared ? H : (int)batches;  // shared keys (the positional table) are packed once per head
  *a_halves = (size_t)batches * nch * T * 64;
  *w_halves = (size_t)wb * tiles_n * nch * 128 * 64;
  return !(*a_halves / 2 >= (1ull << 31) || *w_halves / 2 >= (1ull << 31) || batches > 65535 || tiles_n * nch > 65535);
}

// Packed per-head keys of `b`.  b_cache (may be NULL): the tensor behind `b` when the keys are shared; its packed
// copy is kept on the tensor across calls (the projected positional table of a layer never changes between steps).
static int pack_keys(fa_ctx *ctx, const float *b, fa_tensor *b_cache, int Tb, int H, int HD, int W, int b_shared,
                     size_t w_halves, Block &wp, const __half **wpk) {
  const long long batches = (long long)W * H;
  const int S = H * HD, nch = ceil_div(HD, 64), tiles_n = ceil_div(Tb, 128);
  const int wb = b_shared ? H : (int)batches;
  const bool cacheable = b_shared && b_cache && !b_cache->view;
  const bool cached = cacheable && b_cache->hk16_valid && b_cache->hk_kind == 0 && b_cache->hk_Tb == Tb && b_cache->hk_H == H && b_cache->hk_HD == HD;
  if (cached) {
    *wpk = (const __half *)b_cache->hk16;
    return FA_OK;
  }
  if (cacheable && !ctx->capturing) {  // (a block taken while recording belongs to the recording)
    if (b_cache->hk16 && b_cache->hk16_bytes < w_halves * 2) {
      fa_block_release(ctx, b_cache->hk16);
      b_cache->hk16 = nullptr;
    }
    if (!b_cache->hk16) FA_TRY(fa_block_acquire(ctx, w_halves * 2, &b_cache->hk16, &b_cache->hk16_bytes));
    b_cache->hk_kind = 0, b_cache->hk_Tb = Tb, b_cache->hk_H = H, b_cache->hk_HD = HD;
    b_cache->hk16_valid = true;
    *wpk = (const __half *)b_cache->hk16;
  } else {
    FA_TRY(wp.get(w_halves * 2));
    *wpk = (const __half *)wp.p;
  }
  {
    LaunchScope ls(ctx, "attn_pack_k");
    // with shared keys the source has a single "window" (w = 0 for every packed batch h)
    fa_launch_dep(ctx, k_pack_w_heads, dim3(16, tiles_n * nch, (unsigned)wb), dim3(256), 0, b, (__half *)*wpk, Tb, S, H, HD,
                  tiles_n, nch, 0);
  }
  FA_LAUNCH_CHECK(ctx, "attn_pack_k");
  return FA_OK;
}

// out[((w*H+h)*T + i)*Tb + j] = packed queries x packed keys, one (w, h) per batch
static int qk_gemm(fa_ctx *ctx, const __half *ap, const __half *wpk, float *out, int T, int Tb, int H, int HD, int W,
                   int b_shared) {
  TcEpilogue ep;
  ep.batches = W * H;
  ep.w_batch_mod = b_shared ? H : 0;
  ep.o_div = 1;
  ep.o_hi = (long long)T * Tb;
  ep.o_lo = 0;
  ep.ldc = Tb;
  return fa_tc_gemm_f16(ctx, ap, wpk, out, T, Tb, HD, ep);
}

int fa_tc_bmm_qk(fa_ctx *ctx, const float *q, const float *b, fa_tensor *b_cache, const float *qb, float *out, int T, int Tb,
                 int H, int HD, int W, int b_shared, bool *done) {
  *done = false;
  size_t a_halves = 0, w_halves = 0;
  if (!qk_shape_ok(ctx, T, Tb, H, HD, W, &a_halves, &w_halves, b_shared)) return FA_OK;
  const int S = H * HD, nch = ceil_div(HD, 64);
  Block ap(ctx), wp(ctx);
  FA_TRY(ap.get(a_halves * 2));
  {
    LaunchScope ls(ctx, "attn_pack_q");
    fa_launch_dep(ctx, k_pack_act_heads, dim3(ceil_div(T, 8), nch, (unsigned)(W * H)), dim3(256), 0, q, qb, (const float *)nullptr,
                  (__half *)ap.p, (__half *)nullptr, T, S, H, HD, nch);
  }
  FA_LAUNCH_CHECK(ctx, "attn_pack_q");
  const __half *wpk = nullptr;
  FA_TRY(pack_keys(ctx, b, b_cache, Tb, H, HD, W, b_shared, w_halves, wp, &wpk));
  FA_TRY(qk_gemm(ctx, (const __half *)ap.p, wpk, out, T, Tb, H, HD, W, b_shared));
  *done = true;
  return FA_OK;
}

static bool pv_shape_ok(fa_ctx *ctx, int Tq, int Tk, int H, int HD, int W) {
  const long long batches = (long long)W * H;
  if (!fa_tc_available(ctx) || HD < 64 || HD > 160 || Tq < 32 || Tk < 32 || Tq > 256 || batches * Tq * Tk * HD < (1ll << 22))
    return false;
  const int nch = ceil_div(Tk, 64), tiles_n = ceil_div(HD, 128);
  const size_t a_halves = (size_t)batches * nch * Tq * 64, w_halves = (size_t)batches * tiles_n * nch * 128 * 64;
  return a_halves / 2 < (1ull << 31) && w_halves / 2 < (1ull << 31);
}

// P@V with the probabilities already in packed f16 form (p16 == nullptr: pack them from the f32 tensor p).
static int pv_core(fa_ctx *ctx, const float *p, const __half *p16, const float *v, float *out, __half *out16, int Tq, int Tk,
                   int H, int HD, int W) {
  const long long batches = (long long)W * H;
  const int S = H * HD, nch = ceil_div(Tk, 64), tiles_n = ceil_div(HD, 128);
  const size_t a_halves = (size_t)batches * nch * Tq * 64, w_halves = (size_t)batches * tiles_n * nch * 128 * 64;
  Block ap(ctx), wp(ctx);
  FA_TRY(wp.get(w_halves * 2));
  if (!p16) {
    FA_TRY(ap.get(a_halves * 2));
    {
      LaunchScope ls(ctx, "attn_pack_p");
      fa_launch_dep(ctx, k_pack_act_probs, dim3(grid_for(ctx, a_halves / 2)), dim3(256), 0, p, (__half *)ap.p, Tq, Tk, nch,
                                                                            (unsigned)(a_halves / 2));
    }
    FA_LAUNCH_CHECK(ctx, "attn_pack_p");
    p16 = (const __half *)ap.p;
  }
  {
    LaunchScope ls(ctx, "attn_pack_v");
    fa_launch_dep(ctx, k_pack_w_vT, dim3((unsigned)(batches * nch)), dim3(256), (size_t)64 * (HD + 1) * 4, v, (__half *)wp.p, Tk, S, H, HD,
                                                                                          tiles_n, nch);
  }
  FA_LAUNCH_CHECK(ctx, "attn_pack_v");
  TcEpilogue ep;
  ep.batches = (int)batches;
  ep.o_div = H;  // out[(w*Tq + i)*S + h*HD + d]
  ep.o_hi = (long long)Tq * S;
  ep.o_lo = HD;
  ep.ldc = S;
  ep.out16 = out16;  // the context feeds the output projection: hand it over already packed
  ep.o16_rows = W * Tq;
  ep.o16_row_hi = Tq;
  ep.o16_col_lo = HD;
  return fa_tc_gemm_f16(ctx, p16, (const __half *)wp.p, out, Tq, HD, Tk, ep);
}

int fa_tc_bmm_pv(fa_ctx *ctx, const float *p, const float *v, float *out, __half *out16, int Tq, int Tk, int H, int HD,
                 int W, bool *done) {
  *done = false;
  if (!pv_shape_ok(ctx, Tq, Tk, H, HD, W)) return FA_OK;
  FA_TRY(pv_core(ctx, p, nullptr, v, out, out16, Tq, Tk, H, HD, W));
  *done = true;
  return FA_OK;
}

// Fused rel-pos self-attention (the optional attnFused member, src/gpu/compute.d.ts:247-248; op sequence
// of src/engines/asr-parakeet/raw-encoder.js:335-341): content scores and positional scores on the
// batched tensor-core GEMM, then ONE pass that shifts, adds, normalises and emits the probabilities as
// the packed f16 operand of the P@V product - the [W*H*T, T] probability tensor is never stored in f32.
int fa_tc_attn_fused(fa_ctx *ctx, const float *q, const float *k, const float *v, const float *pos, fa_tensor *pos_cache,
                     const float *pbu, const float *pbv, float *out, __half *out16, int T, int H, int HD, int W, bool *done) {
  *done = false;
  const int P = 2 * T - 1;
  const long long batches = (long long)W * H;
  if (!pv_shape_ok(ctx, T, T, H, HD, W) || batches * T * P >= (1ll << 31)) return FA_OK;
  Block ac(ctx), bd(ctx), pr(ctx);
  FA_TRY(ac.get((size_t)batches * T * T * 4));
  FA_TRY(bd.get((size_t)batches * T * P * 4));
  // one read of q gives both packed queries; the layer's own keys are packed per call, the positional keys once
  size_t a_halves = 0, wk_halves = 0, wp_halves = 0, a2 = 0;
  if (!qk_shape_ok(ctx, T, T, H, HD, W, &a_halves, &wk_halves, 0) || !qk_shape_ok(ctx, T, P, H, HD, W, &a2, &wp_halves, 1))
    return FA_OK;
  const int S = H * HD, nchq = ceil_div(HD, 64);
  Block qu(ctx), qv(ctx), wk(ctx), wpos(ctx);
  FA_TRY(qu.get(a_halves * 2));
  FA_TRY(qv.get(a_halves * 2));
  {
    LaunchScope ls(ctx, "attn_pack_q");
    fa_launch_dep(ctx, k_pack_act_heads, dim3(ceil_div(T, 8), nchq, (unsigned)batches), dim3(256), 0, q, pbu, pbv, (__half *)qu.p,
                  (__half *)qv.p, T, S, H, HD, nchq);
  }
  FA_LAUNCH_CHECK(ctx, "attn_pack_q");
  const __half *kk = nullptr, *kp = nullptr;
  FA_TRY(pack_keys(ctx, k, nullptr, T, H, HD, W, 0, wk_halves, wk, &kk));
  FA_TRY(qk_gemm(ctx, (const __half *)qu.p, kk, (float *)ac.p, T, T, H, HD, W, 0));
  FA_TRY(pack_keys(ctx, pos, pos_cache, P, H, HD, W, 1, wp_halves, wpos, &kp));
  FA_TRY(qk_gemm(ctx, (const __half *)qv.p, kp, (float *)bd.p, T, P, H, HD, W, 1));
  const int nch = ceil_div(T, 64);
  FA_TRY(pr.get((size_t)batches * nch * T * 64 * 2));
  {
    LaunchScope ls(ctx, "attn_softmax_shift_pack");
    const int rows = (int)(batches * T);
    int grid = ceil_div(rows, 8);
    if (grid > ctx->sm_count * 16) grid = ctx->sm_count * 16;
    fa_launch_dep(ctx, k_softmax_shift_pack, dim3(grid), dim3(256), 0, (const float *)ac.p, (const float *)bd.p, (__half *)pr.p, rows, T, nch);
  }
  FA_LAUNCH_CHECK(ctx, "attn_softmax_shift_pack");
  FA_TRY(pv_core(ctx, nullptr, (const __half *)pr.p, v, out, out16, T, T, H, HD, W));
  *done = true;
  return FA_OK;
}
