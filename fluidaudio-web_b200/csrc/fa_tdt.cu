// Batched greedy TDT decoding (prediction network + joint) for many encoder windows at once.
//
// The reference decodes one window at a time on a CPU core, in Rust compiled to wasm
// (rust/parakeet-decoder/src/lib.rs: predict :150-156, compute_predproj :159-175, joint_tail :179-227,
// decode_proj :288-319), and names that stage as the cost right after the encoder
// (src/engines/asr-parakeet/pipeline.js:38-40).  Its own GPU form runs the whole loop of a window in one workgroup
// (src/engines/asr-parakeet/gpu-decoder.js).  Windows are independent, so here they advance in LOCK-STEP, one joint
// evaluation per window per round, and every product of a round is a matrix product over all windows:
//
//   joint in   J[w]   = relu(proj[w, t_w] + predproj[w]) * out_scale      (gather at each window's own frame t_w)
//   logits     OUT    = J @ out_q + out_b      int8 out-matrix [640][8198], three int8 digits per activation row on
//                                              kind::i8 (exact integer sums, f32-grade result)
//   pick       argmax over the 8193 tokens and the 5 durations; emit / commit the candidate state / advance t_w
//   predict    G0 = [embed[tok] | H0] @ [W0;R0]^T + b  -> cell -> (NH0, NC0);  G1 = [NH0 | H1] @ [W1;R1]^T + b -> cell
//   predproj   = NH1 @ pred_w + pred_b         f32 weights on kind::tf32 with value + residue planes (f32-grade)
//
// The prediction network is evaluated for every window in every round: for a window that did not emit, its inputs
// (committed state, last token) are unchanged, so the result is the same as the cached one the reference keeps.
// A round is recorded once and replayed; the host looks at a device counter of finished windows every few rounds.
// Gate nonlinearities are the crate's own exp / tanh approximations (lib.rs:49-68), evaluated with separate
// multiplies and adds, so that the only difference from the reference is the summation order inside the products.
#include "fa_internal.cuh"

namespace {

constexpr int HID = 640, VOCAB = 8193, LOGITS = 8198, BLANK = VOCAB - 1, MAX_SYMBOLS = 10;

__device__ __forceinline__ float t_floorf(float x) {
  const float i = (float)(int)x;
  return i > x ? __fsub_rn(i, 1.0f) : i;
}
__device__ __forceinline__ float t_ldexpf(float x, int e) {
  float r = x;
  int n = e;
  while (n > 30) { r = __fmul_rn(r, 1073741824.0f); n -= 30; }
  while (n < -30) { r = __fmul_rn(r, 9.313225746154785e-10f); n += 30; }
  return __fmul_rn(r, __uint_as_float((unsigned)(127 + n) << 23));
}
__device__ __forceinline__ float t_expf(float x) {
  const float xc = x > 30.0f ? 30.0f : (x < -30.0f ? -30.0f : x);
  const float t = __fmul_rn(xc, 1.4426950408889634f);
  const float fl = t_floorf(t);
  const float fr = __fsub_rn(t, fl);
  float p = __fmul_rn(fr, 0.0096181f);
  p = __fmul_rn(fr, __fadd_rn(0.0555041f, p));
  p = __fmul_rn(fr, __fadd_rn(0.2402265f, p));
  p = __fmul_rn(fr, __fadd_rn(0.6931472f, p));
  p = __fadd_rn(1.0f, p);
  return t_ldexpf(p, (int)fl);
}
__device__ __forceinline__ float t_sigmoid(float x) { return __fdiv_rn(1.0f, __fadd_rn(1.0f, t_expf(-x))); }
__device__ __forceinline__ float t_tanhf(float x) {
  const float e = t_expf(__fmul_rn(2.0f, x));
  return __fdiv_rn(__fsub_rn(e, 1.0f), __fadd_rn(e, 1.0f));
}

// J[w][n] = relu(proj[w*T + t_w][n] + predproj[w][n]) * scale[n]; finished windows produce zeros.
__global__ void __launch_bounds__(256) k_tdt_joint_in(const float *__restrict__ proj, const int *__restrict__ t, int T,
                                                      const float *__restrict__ predproj, const float *__restrict__ scale,
                                                      float *__restrict__ J) {
  const int w = blockIdx.x, tw = t[w];
  for (int n = threadIdx.x; n < HID; n += blockDim.x) {
    float v = 0.0f;
    if (tw < T) {
      v = __fadd_rn(proj[((size_t)w * T + tw) * HID + n], predproj[(size_t)w * HID + n]);
      v = v > 0.0f ? v : 0.0f;
      if (scale) v = __fmul_rn(v, scale[n]);
    }
    J[(size_t)w * HID + n] = v;
  }
}

// One block per window: first-maximum over tokens and durations (the reference scans upwards with a strict >),
// then the TDT bookkeeping of decode_proj (lib.rs:300-316) and, on an emission, the commit of the candidate state.
__global__ void __launch_bounds__(256) k_tdt_pick(const float *__restrict__ logits, int ld, int T, int cap, int *__restrict__ t,
                                                  int *__restrict__ emitted, int *__restrict__ last_tok, int *__restrict__ counts,
                                                  int *__restrict__ ids, int *__restrict__ frames, float *__restrict__ xh0,
                                                  float *__restrict__ xh1, const float *__restrict__ nh1, float *__restrict__ c0,
                                                  float *__restrict__ c1, const float *__restrict__ nc0, const float *__restrict__ nc1,
                                                  int *__restrict__ done_count) {
  __shared__ float sv[8];
  __shared__ int si[8];
  __shared__ int s_tok;
  const int w = blockIdx.x, tw = t[w];
  if (tw >= T) return;  // this window finished in an earlier round (block-uniform)
  const float *row = logits + (size_t)w * ld;
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < VOCAB; i += blockDim.x) {
    const float v = row[i];
    if (v > bv) { bv = v; bi = i; }  // ascending i per thread: keeps the first maximum
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
  }
  if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = bv; si[threadIdx.x >> 5] = bi; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int k = 1; k < 8; k++)
      if (sv[k] > bv || (sv[k] == bv && si[k] < bi)) { bv = sv[k]; bi = si[k]; }
    const int tok = bi == 0x7fffffff ? 0 : bi;  // every logit NaN or -inf: the reference's scan leaves index 0
    int step = 0;
    float dv = -INFINITY;
    for (int i = VOCAB; i < LOGITS; i++)
      if (row[i] > dv) { dv = row[i]; step = i - VOCAB; }
    int em = emitted[w], n_out = counts[w], tn = tw;
    if (tok != BLANK) {
      if (n_out < cap) { ids[(size_t)w * cap + n_out] = tok; frames[(size_t)w * cap + n_out] = tw; }
      n_out++;
      em++;
      last_tok[w] = tok;
      counts[w] = n_out;
    }
    if (step > 0) { tn += step; em = 0; }
    else if (tok == BLANK || em >= MAX_SYMBOLS) { tn += 1; em = 0; }
    t[w] = tn;
    emitted[w] = em;
    if (tn >= T) atomicAdd(done_count, 1);
    s_tok = tok;
  }
  __syncthreads();
  if (s_tok != BLANK) {  // commit_state: H = NH, C = NC (H0 / H1 live in the right halves of the two LSTM inputs)
    for (int n = threadIdx.x; n < HID; n += blockDim.x) {
      xh0[(size_t)w * 2 * HID + HID + n] = xh1[(size_t)w * 2 * HID + n];  // NH0 is the left half of layer 1's input
      xh1[(size_t)w * 2 * HID + HID + n] = nh1[(size_t)w * HID + n];
      c0[(size_t)w * HID + n] = nc0[(size_t)w * HID + n];
      c1[(size_t)w * HID + n] = nc1[(size_t)w * HID + n];
    }
  }
}

// xh0[w][0:640] = embed[last_tok[w]]
__global__ void __launch_bounds__(256) k_tdt_embed(const float *__restrict__ embed, const int *__restrict__ last_tok,
                                                   float *__restrict__ xh0) {
  const int w = blockIdx.x;
  const float *e = embed + (size_t)last_tok[w] * HID;
  for (int n = threadIdx.x; n < HID; n += blockDim.x) xh0[(size_t)w * 2 * HID + n] = e[n];
}

// ONNX iofc gates G [W][2560] (bias already added) and the committed cell state -> candidate cell and hidden state.
// nh goes out with row pitch nh_ld (layer 0 writes the left half of layer 1's input).
__global__ void __launch_bounds__(256) k_tdt_cell(const float *__restrict__ G, const float *__restrict__ c, float *__restrict__ nc,
                                                  float *__restrict__ nh, int nh_ld, int W) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= W * HID) return;
  const int w = i / HID, g = i - w * HID;
  const float *gr = G + (size_t)w * 4 * HID;
  const float zi = gr[g], zo = gr[HID + g], zf = gr[2 * HID + g], zc = gr[3 * HID + g];
  const float cc = __fadd_rn(__fmul_rn(t_sigmoid(zf), c[i]), __fmul_rn(t_sigmoid(zi), t_tanhf(zc)));
  nc[i] = cc;
  nh[(size_t)w * nh_ld + g] = __fmul_rn(t_sigmoid(zo), t_tanhf(cc));
}

__global__ void k_fill_int(int *p, int n, int v) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) p[i] = v;
}

}  // namespace

struct fa_tdt {
  fa_tensor *embed = nullptr, *wr[2] = {nullptr, nullptr}, *bsum[2] = {nullptr, nullptr}, *pred_w = nullptr, *pred_b = nullptr;
  fa_tensor *out_b = nullptr, *out_scale = nullptr, *ones = nullptr, *out_w = nullptr;
  fa_bytes *out_q = nullptr;
};

static void tdt_release(fa_ctx *ctx, fa_tdt *d) {
  fa_tensor *ts[] = {d->embed, d->wr[0], d->wr[1], d->bsum[0], d->bsum[1], d->pred_w, d->pred_b, d->out_b, d->out_scale, d->ones, d->out_w};
  for (fa_tensor *t : ts)
    if (t) fa_free_tensor(ctx, t);
  if (d->out_q) fa_free_bytes(ctx, d->out_q);
  delete d;
}

extern "C" int fa_tdt_create(fa_ctx *ctx, const float *embed, const float *l0w, const float *l0r, const float *l0b,
                             const float *l1w, const float *l1r, const float *l1b, const float *pred_w, const float *pred_b,
                             const float *out_w, const float *out_b, const int8_t *out_q, const float *out_scale, fa_tdt **out) {
  if (!ctx || !out) return fa_fail(ctx, FA_ERR_INVALID, "tdtCreate: NULL argument");
  FA_REQUIRE(ctx, embed && l0w && l0r && l0b && l1w && l1r && l1b && pred_w && pred_b && out_b, "tdtCreate: NULL weight pointer");
  FA_REQUIRE(ctx, (out_q && out_scale) || out_w, "tdtCreate: needs the out matrix as int8 rows + scales or as f32");
  fa_tdt *d = new fa_tdt();
  int rc = fa_upload_f32(ctx, embed, VOCAB, HID, &d->embed);
  // LSTM weights [4*HID][HID] (row = gate output) as one [2*HID][4*HID] right-hand matrix per layer: rows 0..639
  // multiply the layer input, rows 640..1279 the committed hidden state
  const float *lw[2] = {l0w, l1w}, *lr[2] = {l0r, l1r}, *lb[2] = {l0b, l1b};
  std::vector<float> tmp((size_t)2 * HID * 4 * HID), bs(4 * HID);
  for (int l = 0; l < 2 && rc == FA_OK; l++) {
    for (int g = 0; g < 4 * HID; g++)
      for (int k = 0; k < HID; k++) {
        tmp[(size_t)k * 4 * HID + g] = lw[l][(size_t)g * HID + k];
        tmp[(size_t)(HID + k) * 4 * HID + g] = lr[l][(size_t)g * HID + k];
      }
    for (int g = 0; g < 4 * HID; g++) bs[g] = lb[l][g] + lb[l][4 * HID + g];  // lib.rs:139: b[g] + b[4*HID + g] first
    rc = fa_upload_f32(ctx, tmp.data(), 2 * HID, 4 * HID, &d->wr[l]);
    if (rc == FA_OK) rc = fa_upload_f32(ctx, bs.data(), 1, 4 * HID, &d->bsum[l]);
  }
  if (rc == FA_OK) rc = fa_upload_f32(ctx, pred_w, HID, HID, &d->pred_w);
  if (rc == FA_OK) rc = fa_upload_f32(ctx, pred_b, 1, HID, &d->pred_b);
  if (rc == FA_OK) rc = fa_upload_f32(ctx, out_b, 1, LOGITS, &d->out_b);
  if (rc == FA_OK && out_q) {
    std::vector<float> one(LOGITS, 1.0f);
    rc = fa_upload_bytes(ctx, out_q, (size_t)HID * LOGITS, &d->out_q);
    if (rc == FA_OK) rc = fa_upload_f32(ctx, out_scale, 1, HID, &d->out_scale);
    if (rc == FA_OK) rc = fa_upload_f32(ctx, one.data(), 1, LOGITS, &d->ones);
  } else if (rc == FA_OK) {
    rc = fa_upload_f32(ctx, out_w, HID, LOGITS, &d->out_w);
  }
  if (rc != FA_OK) {
    const std::string msg = ctx->err;
    tdt_release(ctx, d);
    ctx->err = msg;
    return rc;
  }
  *out = d;
  return FA_OK;
}

extern "C" int fa_tdt_free(fa_ctx *ctx, fa_tdt *d) {
  if (!ctx) return fa_fail(ctx, FA_ERR_INVALID, "tdtFree: NULL context");
  if (d) tdt_release(ctx, d);
  return FA_OK;
}

namespace {

struct TdtState {
  fa_tensor *xh0 = nullptr, *xh1 = nullptr, *c0 = nullptr, *c1 = nullptr, *nc0 = nullptr, *nc1 = nullptr, *nh1 = nullptr,
            *predproj = nullptr, *J = nullptr;
  void *ints = nullptr;  // t, emitted, last_tok, counts [W each], done_count, then ids and frames [W*cap each]
  size_t ints_bytes = 0;
};

// predict(last_tok) + compute_predproj for every window, from the committed state
int tdt_predict(fa_ctx *ctx, fa_tdt *d, TdtState &s, int W, const int *last_tok) {
  {
    LaunchScope ls(ctx, "tdt_embed");
    k_tdt_embed<<<W, 256, 0, ctx->stream>>>((const float *)d->embed->dptr, last_tok, (float *)s.xh0->dptr);
  }
  fa_tensor *g = nullptr;
  FA_TRY(fa_matmul(ctx, s.xh0, d->wr[0], d->bsum[0], FA_ACT_NONE, nullptr, &g));
  {
    LaunchScope ls(ctx, "tdt_cell");
    k_tdt_cell<<<ceil_div(W * HID, 256), 256, 0, ctx->stream>>>((const float *)g->dptr, (const float *)s.c0->dptr,
                                                                 (float *)s.nc0->dptr, (float *)s.xh1->dptr, 2 * HID, W);
  }
  FA_TRY(fa_free_tensor(ctx, g));
  FA_TRY(fa_matmul(ctx, s.xh1, d->wr[1], d->bsum[1], FA_ACT_NONE, nullptr, &g));
  {
    LaunchScope ls(ctx, "tdt_cell");
    k_tdt_cell<<<ceil_div(W * HID, 256), 256, 0, ctx->stream>>>((const float *)g->dptr, (const float *)s.c1->dptr,
                                                                 (float *)s.nc1->dptr, (float *)s.nh1->dptr, HID, W);
  }
  FA_TRY(fa_free_tensor(ctx, g));
  fa_tensor *pp = nullptr;
  FA_TRY(fa_matmul(ctx, s.nh1, d->pred_w, d->pred_b, FA_ACT_NONE, nullptr, &pp));
  FA_CHECK_CUDA(ctx, cudaMemcpyAsync(s.predproj->dptr, pp->dptr, (size_t)W * HID * 4, cudaMemcpyDeviceToDevice, ctx->stream));
  FA_TRY(fa_free_tensor(ctx, pp));
  FA_LAUNCH_CHECK(ctx, "tdt_predict");
  return FA_OK;
}

int tdt_round(fa_ctx *ctx, fa_tdt *d, TdtState &s, const fa_tensor *proj, int W, int T, int cap) {
  int *t = (int *)s.ints, *emitted = t + W, *last_tok = t + 2 * W, *counts = t + 3 * W, *done = t + 4 * W;
  int *ids = done + 4, *frames = ids + (size_t)W * cap;
  {
    LaunchScope ls(ctx, "tdt_joint_in");
    k_tdt_joint_in<<<W, 256, 0, ctx->stream>>>((const float *)proj->dptr, t, T, (const float *)s.predproj->dptr,
                                               d->out_scale ? (const float *)d->out_scale->dptr : nullptr, (float *)s.J->dptr);
  }
  fa_tensor *logits = nullptr;
  if (d->out_q)
    FA_TRY(fa_matmul_int8(ctx, s.J, d->out_q, d->ones, LOGITS, HID, d->out_b, FA_ACT_NONE, &logits));
  else
    FA_TRY(fa_matmul(ctx, s.J, d->out_w, d->out_b, FA_ACT_NONE, nullptr, &logits));
  {
    LaunchScope ls(ctx, "tdt_pick");
    k_tdt_pick<<<W, 256, 0, ctx->stream>>>((const float *)logits->dptr, LOGITS, T, cap, t, emitted, last_tok, counts, ids, frames,
                                           (float *)s.xh0->dptr, (float *)s.xh1->dptr, (const float *)s.nh1->dptr,
                                           (float *)s.c0->dptr, (float *)s.c1->dptr, (const float *)s.nc0->dptr,
                                           (const float *)s.nc1->dptr, done);
  }
  FA_TRY(fa_free_tensor(ctx, logits));
  FA_LAUNCH_CHECK(ctx, "tdt_round");
  return tdt_predict(ctx, d, s, W, last_tok);
}

}  // namespace

extern "C" int fa_tdt_decode_proj(fa_ctx *ctx, fa_tdt *d, const fa_tensor *proj, int W, int T, int cap, int32_t *ids_host,
                                  int32_t *frames_host, int32_t *counts_host, int *rounds_out) {
  if (!ctx || !d || !ids_host || !frames_host || !counts_host) return fa_fail(ctx, FA_ERR_INVALID, "tdtDecodeProj: NULL argument");
  FA_REQUIRE(ctx, fa_valid(ctx, proj), "tdtDecodeProj: unknown tensor handle");
  FA_REQUIRE(ctx, W >= 1 && T >= 1 && cap >= 1, "tdtDecodeProj: W=%d T=%d cap=%d", W, T, cap);
  FA_REQUIRE(ctx, proj->storage == FA_F32 && proj->rows == W * T && proj->cols == HID,
             "tdtDecodeProj: frames are [%d,%d], expected f32 [%d,%d]", proj->rows, proj->cols, W * T, HID);
  FA_REQUIRE(ctx, !ctx->capturing, "tdtDecodeProj: not allowed while recording (it reads results back)");
  FA_CHECK_CUDA(ctx, cudaSetDevice(ctx->device));
  FA_TRY(fa_touch_f32(ctx, proj));
  int arena = -1;
  FA_TRY(fa_push_arena(ctx, &arena));
  TdtState s;
  const int saved_limbs = ctx->int8_limbs;
  ctx->int8_limbs = 3;  // f32-grade activations for the joint's int8 product: token picks follow the f32 reference
  fa_graph *graph = nullptr;
  int rc = FA_OK, rounds = 0;
  auto alloc = [&](int r, int c, fa_tensor **t) { return rc == FA_OK ? (rc = fa_alloc(ctx, r, c, t)) : rc; };
  alloc(W, 2 * HID, &s.xh0), alloc(W, 2 * HID, &s.xh1), alloc(W, HID, &s.c0), alloc(W, HID, &s.c1), alloc(W, HID, &s.nc0),
      alloc(W, HID, &s.nc1), alloc(W, HID, &s.nh1), alloc(W, HID, &s.predproj), alloc(W, HID, &s.J);
  const size_t n_int = (size_t)4 * W + 4 + (size_t)2 * W * cap;
  if (rc == FA_OK) rc = fa_block_acquire(ctx, n_int * 4, &s.ints, &s.ints_bytes);
  int *t = (int *)s.ints, *last_tok = t + 2 * W, *done = t + 4 * W;
  if (rc == FA_OK) {
    // decode_proj :290-294: zero state, last token = blank, predict + predproj once
    fa_tensor *z[] = {s.xh0, s.xh1, s.c0, s.c1, s.nc0, s.nc1, s.nh1};
    for (fa_tensor *x : z) cudaMemsetAsync(x->dptr, 0, (size_t)x->rows * x->cols * 4, ctx->stream);
    cudaMemsetAsync(s.ints, 0, n_int * 4, ctx->stream);
    k_fill_int<<<ceil_div(W, 256), 256, 0, ctx->stream>>>(last_tok, W, BLANK);
    rc = tdt_predict(ctx, d, s, W, last_tok);
  }
  // one round eagerly (first-use caches of the weights), then the round as a recorded batch, replayed
  if (rc == FA_OK) rc = tdt_round(ctx, d, s, proj, W, T, cap);
  rounds = 1;
  if (rc == FA_OK) rc = fa_graph_begin(ctx);
  if (rc == FA_OK) {
    rc = tdt_round(ctx, d, s, proj, W, T, cap);
    fa_graph *g = nullptr;
    const int rc2 = fa_graph_end(ctx, &g);
    if (rc == FA_OK) rc = rc2;
    graph = g;
  }
  int done_host = 0;
  const int max_rounds = T * (MAX_SYMBOLS + 1) + 2, check_every = 16;
  while (rc == FA_OK && done_host < W && rounds < max_rounds) {
    for (int i = 0; i < check_every && rc == FA_OK; i++, rounds++) rc = fa_graph_launch(ctx, graph);
    if (rc == FA_OK) {
      cudaError_t e = cudaMemcpyAsync(&done_host, done, 4, cudaMemcpyDeviceToHost, ctx->stream);
      if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
      if (e != cudaSuccess) rc = fa_fail(ctx, FA_ERR_CUDA, "tdtDecodeProj: %s", cudaGetErrorString(e));
    }
  }
  if (rc == FA_OK && done_host < W) rc = fa_fail(ctx, FA_ERR_INVALID, "tdtDecodeProj: %d of %d windows unfinished after %d rounds", W - done_host, W, rounds);
  if (rc == FA_OK) {
    int *counts = t + 3 * W, *ids = done + 4, *frames = ids + (size_t)W * cap;
    cudaError_t e = cudaMemcpyAsync(counts_host, counts, (size_t)W * 4, cudaMemcpyDeviceToHost, ctx->stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(ids_host, ids, (size_t)W * cap * 4, cudaMemcpyDeviceToHost, ctx->stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(frames_host, frames, (size_t)W * cap * 4, cudaMemcpyDeviceToHost, ctx->stream);
    if (e != cudaSuccess) rc = fa_fail(ctx, FA_ERR_CUDA, "tdtDecodeProj readback: %s", cudaGetErrorString(e));
    if (rc == FA_OK) rc = fa_sync(ctx);
  }
  const std::string msg = ctx->err;
  if (graph) fa_graph_free(ctx, graph);
  if (s.ints) fa_block_release(ctx, s.ints);
  ctx->int8_limbs = saved_limbs;
  fa_pop_arena(ctx, arena);
  if (rc != FA_OK) ctx->err = msg;
  if (rounds_out) *rounds_out = rounds;
  return rc;
}
