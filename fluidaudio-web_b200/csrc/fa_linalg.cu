// The hot path's entry points: matmul / matmulInt8 / matmulNBits, routed by shape and storage only
// (the reference's routers: src/gpu/compute.js:401-436, 593-611, 306-316).
//
//   tiny or ragged problems            -> any-shape f32 CUDA-core kernels (fa_gemm_simt.cu)
//   f16-storage B, int8 B, int4 B      -> tcgen05 kernels (fa_gemm_tc.cu) for every other size,
//                                         decode sizes (M <= 16) included: at 6.5 TB/s of HBM a CUDA
//                                         core has fewer than 3 lane-operations per int4 weight, so
//                                         only the tensor pipe keeps a decode product memory-bound.
//   f32-storage B                      -> f32 CUDA-core kernel (the reference computes those in f32)
#include "fa_internal.cuh"

namespace {

// A tensor-core launch pays for two prepasses and TMA descriptor set-up; below this many
// multiply-adds the any-shape kernel is faster and it is exact f32.
constexpr long long kTcMinMacs = 1ll << 21;

bool tc_shape_ok(fa_ctx *ctx, int M, int N, int K) {
  // big enough to amortise the packing of the row operand, or a weight matrix big enough that the
  // product is a stream over it whatever M is (token-by-token decoding, M = 1)
  return fa_tc_available(ctx) && N >= 64 && K >= 64 && M >= 1 &&
         ((long long)M * N * K >= kTcMinMacs || (long long)N * K >= (1ll << 18));
}

// Few activation rows against a weight matrix worth streaming: the CUDA-core GEMV kernels (no packing,
// f32 or exact-integer activations).  "gemv_rows" = 0 sends these shapes to the tensor-core kernel instead.
bool gemv_shape_ok(fa_ctx *ctx, int M, int N, int K) {
  return M >= 1 && M <= ctx->gemv_rows && (long long)N * K >= (1ll << 14);
}

int check_vec(fa_ctx *ctx, const fa_tensor *t, int n, const char *what) {
  FA_REQUIRE(ctx, fa_valid(ctx, t), "%s: unknown tensor handle", what);
  FA_REQUIRE(ctx, t->storage == FA_F32, "%s must be f32 storage", what);
  FA_REQUIRE(ctx, (long long)t->rows * t->cols >= n, "%s has %d elements, need %d", what, t->rows * t->cols, n);
  return fa_touch_f32(ctx, t);
}

// A handle made before the open recording.  Work that such a handle caches on itself (packed weight copies,
// operand shadows, the f32 fill of a lazy result) must not be started while recording: the kernels would only be
// captured, the handle would look ready, and an eager use before the first replay would read unwritten memory.
bool foreign_to_recording(fa_ctx *ctx, const void *dptr) {
  if (!ctx->capturing) return false;
  auto it = ctx->block_owner.find(const_cast<void *>(dptr));
  return it == ctx->block_owner.end() || it->second != ctx->capturing;
}
#define FA_NO_FIRST_USE_IN_RECORDING(ctx, dptr, what)                                                              \
  FA_REQUIRE(ctx, !foreign_to_recording(ctx, dptr),                                                                \
             "%s: the packed copy of these weights is built on their first use, which must not happen inside a "   \
             "recording; run the sequence once eagerly before fa_graph_begin", what)

// Packed f16 copy of a [K][N] weight tensor, built once per handle.
int ensure_bt_f16(fa_ctx *ctx, fa_tensor *b) {
  if (b->view) return fa_fail(ctx, FA_ERR_INVALID, "matmul: a rowsView cannot be the weight operand of a large product");
  if (b->bt_f16 && !b->bt_stale) return FA_OK;
  FA_NO_FIRST_USE_IN_RECORDING(ctx, b->dptr, "matmul");
  if (b->bt_stale && b->bt_tf32) {  // both copies are out of date: drop the one not being rebuilt
    fa_block_release(ctx, b->bt_tf32);
    b->bt_tf32 = nullptr;
  }
  b->bt_stale = false;
  if (!b->bt_f16) FA_TRY(fa_block_acquire(ctx, fa_tc_weight_bytes(b->cols, b->rows, 2), &b->bt_f16, &b->bt_bytes));
  return fa_pack_w_f16(ctx, b->dptr, b->storage, b->rows, b->cols, (__half *)b->bt_f16);
}

// Value + residue f32 planes of a [K][N] f32 weight tensor (kind::tf32 route), built once per handle.
int ensure_bt_tf32(fa_ctx *ctx, fa_tensor *b) {
  if (b->bt_tf32 && !b->bt_stale) return FA_OK;
  FA_NO_FIRST_USE_IN_RECORDING(ctx, b->dptr, "matmul");
  FA_TRY(fa_touch_f32(ctx, b));
  if (b->bt_stale && b->bt_f16) {
    fa_block_release(ctx, b->bt_f16);
    b->bt_f16 = nullptr;
  }
  b->bt_stale = false;
  if (!b->bt_tf32) FA_TRY(fa_block_acquire(ctx, fa_tc_tf32_weight_bytes(b->cols, b->rows), &b->bt_tf32, &b->bt_tf32_bytes));
  return fa_pack_w_tf32(ctx, (const float *)b->dptr, b->rows, b->cols, (float *)b->bt_tf32);
}

// f32-storage B at the sizes the reference hands to its fastest f32 kernel (M, N, K >= 256, src/gpu/compute.js:426)
// runs on the tensor cores in f32-grade arithmetic (kind::tf32 with value + residue planes), and so do products
// with fewer rows against a weight matrix of that size when there is enough work to pay for packing the row operand
// (the lock-step LSTM and joint products of the batched TDT decoder); smaller or ragged products stay on the
// any-shape CUDA-core kernel.
bool tf32_shape_ok(fa_ctx *ctx, int M, int N, int K) {
  return fa_tc_available(ctx) && N >= 256 && K >= 256 && (M >= 256 || (M >= 8 && (long long)M * N * K >= kTcMinMacs));
}

// Packed int8 copy of a [K][N] int8 payload, built once per handle and (N,K).
int ensure_nk_i8(fa_ctx *ctx, fa_bytes *wq, int N, int K) {
  if (wq->nk_i8 && wq->nk_N == N && wq->nk_K == K) return FA_OK;
  FA_NO_FIRST_USE_IN_RECORDING(ctx, wq->dptr, "matmulInt8");
  if (wq->nk_i8) fa_block_release(ctx, wq->nk_i8);
  wq->nk_i8 = nullptr;
  FA_TRY(fa_block_acquire(ctx, fa_tc_weight_bytes(N, K, 1), &wq->nk_i8, &wq->nk_bytes));
  wq->nk_N = N;
  wq->nk_K = K;
  return fa_pack_w_i8(ctx, (const int8_t *)wq->dptr, K, N, (int8_t *)wq->nk_i8);
}

// Tile-contiguous int8 copy of a [K][N] int8 payload for the f16-activation route, built once per handle and (N,K).
int ensure_nk_i8w(fa_ctx *ctx, fa_bytes *wq, int N, int K) {
  if (wq->nk_i8w && wq->i8w_N == N && wq->i8w_K == K) return FA_OK;
  FA_NO_FIRST_USE_IN_RECORDING(ctx, wq->dptr, "matmulInt8Operand");
  if (wq->nk_i8w) fa_block_release(ctx, wq->nk_i8w);
  wq->nk_i8w = nullptr;
  FA_TRY(fa_block_acquire(ctx, fa_tc_i8w_weight_bytes(N, K), &wq->nk_i8w, &wq->nk_i8w_bytes));
  wq->i8w_N = N;
  wq->i8w_K = K;
  return fa_pack_w_i8_k64(ctx, (const int8_t *)wq->dptr, K, N, (int8_t *)wq->nk_i8w);
}

// Per-call scratch: a pool block that goes back to the pool as soon as the consuming kernel is
// enqueued (reuse is stream-ordered).
struct Scratch {
  fa_ctx *ctx;
  void *p = nullptr;
  size_t bytes = 0;
  explicit Scratch(fa_ctx *c) : ctx(c) {}
  int get(size_t need) { return fa_block_acquire(ctx, need, &p, &bytes); }
  ~Scratch() {
    if (p) fa_block_release(ctx, p);
  }
};

}  // namespace

// Single-plane f16 shadow block of a tensor, for producers that write it alongside their f32 result.
// Tensors in the value+residue regime (few rows) carry a two-plane shadow instead, which only
// fa_shadow_hilo_ensure fills: producers get nullptr for them and write no shadow.
__half *fa_shadow_block(fa_ctx *ctx, fa_tensor *t) {
  if (!t || t->view || t->storage != FA_F32 || t->rows <= 0 || t->cols <= 0) return nullptr;
  if (t->rows <= ctx->f16_hilo_rows) return nullptr;
  if (t->a16 && t->a16_hilo) {
    fa_block_release(ctx, t->a16);
    t->a16 = nullptr;
  }
  if (!t->a16) {
    if (fa_block_acquire(ctx, fa_tc_act_bytes(t->rows, t->cols, 2, 1), &t->a16, &t->a16_bytes) != FA_OK) return nullptr;
    t->a16_valid = false;
    t->a16_hilo = false;
  }
  return (__half *)t->a16;
}

int fa_shadow_ensure(fa_ctx *ctx, fa_tensor *t, const __half **out) {
  __half *blk = fa_shadow_block(ctx, t);
  if (!blk) return fa_fail(ctx, FA_ERR_OOM, "no block for the f16 shadow of a %dx%d tensor", t->rows, t->cols);
  if (!t->a16_valid) {
    FA_TRY(fa_touch_f32(ctx, t));
    FA_TRY(fa_prep_a_f16(ctx, (const float *)t->dptr, t->rows, t->cols, blk));
    t->a16_valid = true;
  }
  *out = blk;
  return FA_OK;
}

// Two-plane (value, residue) shadow block of a few-row tensor, for a producer that fills both planes.
__half *fa_shadow_hilo_block(fa_ctx *ctx, fa_tensor *t) {
  if (!t || t->view || t->storage != FA_F32 || t->rows <= 0 || t->cols <= 0) return nullptr;
  if (fa_touch_f32(ctx, t) != FA_OK) return nullptr;  // a lazy result lives only in the shadow released below
  if (t->a16 && !t->a16_hilo) {
    fa_block_release(ctx, t->a16);
    t->a16 = nullptr;
  }
  if (!t->a16) {
    if (fa_block_acquire(ctx, fa_tc_act_bytes(t->rows, t->cols, 2, 2), &t->a16, &t->a16_bytes) != FA_OK) return nullptr;
    t->a16_valid = false;
    t->a16_hilo = true;
  }
  return (__half *)t->a16;
}

static int fa_shadow_hilo_ensure(fa_ctx *ctx, fa_tensor *t, const __half **out) {
  if (!fa_shadow_hilo_block(ctx, t))
    return fa_fail(ctx, FA_ERR_OOM, "no block for the f16 shadow of a %dx%d tensor", t->rows, t->cols);
  if (!t->a16_valid) {
    FA_TRY(fa_prep_a_f16_hilo(ctx, (const float *)t->dptr, t->rows, t->cols, (__half *)t->a16));
    t->a16_valid = true;
  }
  *out = (const __half *)t->a16;
  return FA_OK;
}

// Packed f16 row operand for `a`: its cached shadow when it can carry one, else a per-call scratch block.
// Products with few rows (token-by-token decoding) are bound by the weight stream, so their row operand is
// packed as two planes, value and rounding residue, which the kernel accumulates together: the result then
// matches an f32-activation product to a few ulps and greedy token choices follow the f32 path.
static int row_operand_f16(fa_ctx *ctx, const fa_tensor *a, const float *ap, Scratch &sa, const __half **out,
                           bool *hilo) {
  *hilo = a->rows <= ctx->f16_hilo_rows;
  // (a tensor from before the open recording that has no current shadow of the right kind is packed into per-call
  // scratch instead: a shadow started here would be marked valid while its kernel is only captured)
  const bool have = a->a16 && a->a16_valid && a->a16_hilo == *hilo;
  const bool can_shadow = a->storage == FA_F32 && !a->view && (have || !foreign_to_recording(ctx, a->dptr));
  if (*hilo) {
    if (can_shadow) return fa_shadow_hilo_ensure(ctx, const_cast<fa_tensor *>(a), out);
    FA_TRY(sa.get(fa_tc_act_bytes(a->rows, a->cols, 2, 2)));
    FA_TRY(fa_prep_a_f16_hilo(ctx, ap, a->rows, a->cols, (__half *)sa.p));
    *out = (const __half *)sa.p;
    return FA_OK;
  }
  if (can_shadow) return fa_shadow_ensure(ctx, const_cast<fa_tensor *>(a), out);
  FA_TRY(sa.get(fa_tc_act_bytes(a->rows, a->cols, 2, 1)));
  FA_TRY(fa_prep_a_f16(ctx, ap, a->rows, a->cols, (__half *)sa.p));
  *out = (const __half *)sa.p;
  return FA_OK;
}

// operand_hint: the caller states that the result is only read as a packed f16 operand (by another product or by
// attnFusedQKV), so it may be written as that alone even without a fused activation.
static int matmul_impl(fa_ctx *ctx, const fa_tensor *a, fa_tensor *b, const fa_tensor *bias, int act, const fa_tensor *add,
                       bool operand_hint, fa_tensor **out) {
  if (!ctx || !out) return fa_fail(ctx, FA_ERR_INVALID, "matmul: NULL argument");
  FA_REQUIRE(ctx, fa_valid(ctx, a) && fa_valid(ctx, b), "matmul: unknown tensor handle");
  const int M = a->rows, K = a->cols, N = b->cols;
  FA_REQUIRE(ctx, b->rows == K, "matmul: A is [%d,%d] but B is [%d,%d]", M, K, b->rows, N);
  FA_REQUIRE(ctx, act >= 0 && act <= 5, "matmul: unknown activation code %d", act);
  if (bias) FA_TRY(check_vec(ctx, bias, N, "matmul: bias"));
  if (add) {
    FA_TRY(check_vec(ctx, add, M * N, "matmul: add"));
    FA_REQUIRE(ctx, add->rows == M && add->cols == N, "matmul: add is [%d,%d], expected [%d,%d]", add->rows, add->cols, M, N);
  }
  FA_CHECK_CUDA(ctx, cudaSetDevice(ctx->device));
  const float *ap = nullptr;
  fa_tensor *atmp = nullptr;
  // A row operand that already carries a valid packed shadow and is headed for the tensor cores is not read as
  // f32 at all (and, if it is a lazy hidden-layer result, must not be: that would fill its f32 storage for nothing).
  const bool tc_route = b->storage == FA_F16 && !b->view && tc_shape_ok(ctx, M, N, K) &&
                        !(gemv_shape_ok(ctx, M, N, K) && fa_gemv_kn_ok(M, N, K, false));
  const bool shadow_only = tc_route && a->storage == FA_F32 && !a->view && a->a16_valid && !a->a16_hilo &&
                           a->rows > ctx->f16_hilo_rows;
  if (!shadow_only) FA_TRY(fa_as_f32(ctx, a, &ap, &atmp));
  fa_tensor *c = nullptr;
  FA_TRY(fa_tensor_new(ctx, M, N, FA_F32, true, &c));
  int rc;
  const float *biasp = bias ? (const float *)bias->dptr : nullptr;
  const float *addp = add ? (const float *)add->dptr : nullptr;
  if (b->storage == FA_F16 && gemv_shape_ok(ctx, M, N, K) && fa_gemv_kn_ok(M, N, K, false)) {
    rc = fa_gemv_kn(ctx, ap, b->dptr, false, nullptr, biasp, act, addp, (float *)c->dptr, M, N, K);
  } else if (b->storage == FA_F16 && !b->view && tc_shape_ok(ctx, M, N, K)) {
    Scratch sa(ctx);
    const __half *a16 = nullptr;
    rc = ensure_bt_f16(ctx, b);
    bool hilo = false;
    if (rc == FA_OK) rc = row_operand_f16(ctx, a, ap, sa, &a16, &hilo);
    if (rc == FA_OK) {
      TcEpilogue ep;
      ep.a_hilo = hilo;
      ep.bias = biasp;
      ep.add = addp;
      ep.act = act;
      // A product with a fused activation is a hidden layer: its result goes straight into the next
      // product, so the epilogue also emits it as that product's packed f16 row operand.
      const bool hinted = operand_hint && !add && fa_operand_only_ok(ctx, M, N);
      if ((act != FA_ACT_NONE || hinted) && (N & 63) == 0 && (ep.out16 = fa_shadow_block(ctx, c)) != nullptr) {
        c->a16_valid = true;
        if (ctx->lazy_f32 && !add && fa_operand_only_ok(ctx, M, N)) {  // ... and only as that: the f32 copy is made if and when something else reads it
          ep.skip_f32 = true;
          c->f32_lazy = true;
          c->lazy_sticky = ctx->capturing != nullptr;
        }
      }
      rc = fa_tc_gemm_f16(ctx, a16, (const __half *)b->bt_f16, (float *)c->dptr, M, N, K, ep);
    }
  } else if (b->storage == FA_F32 && !b->view && tf32_shape_ok(ctx, M, N, K)) {
    Scratch sa(ctx);
    rc = ensure_bt_tf32(ctx, b);
    if (rc == FA_OK) rc = sa.get(fa_tc_tf32_act_bytes(M, K));
    if (rc == FA_OK) rc = fa_prep_a_tf32(ctx, ap, M, K, (float *)sa.p);
    if (rc == FA_OK) {
      TcEpilogue ep;
      ep.bias = biasp;
      ep.add = addp;
      ep.act = act;
      rc = fa_tc_gemm_tf32(ctx, (const float *)sa.p, (const float *)b->bt_tf32, (float *)c->dptr, M, N, K, ep);
    }
  } else {
    rc = fa_simt_gemm(ctx, ap, b->dptr, b->storage == FA_F16 ? 1 : 0, nullptr, biasp, act, addp, (float *)c->dptr, M,
                      N, K);
  }
  if (atmp) fa_free_tensor(ctx, atmp);
  if (rc != FA_OK) {
    fa_free_tensor(ctx, c);
    return rc;
  }
  *out = c;
  return FA_OK;
}

extern "C" int fa_matmul(fa_ctx *ctx, const fa_tensor *a, fa_tensor *b, const fa_tensor *bias, int act,
                         const fa_tensor *add, fa_tensor **out) {
  return matmul_impl(ctx, a, b, bias, act, add, false, out);
}
extern "C" int fa_matmul_operand(fa_ctx *ctx, const fa_tensor *a, fa_tensor *b, const fa_tensor *bias, int act,
                                 fa_tensor **out) {
  return matmul_impl(ctx, a, b, bias, act, nullptr, true, out);
}

// N-sharded product with the all-gather fused into the epilogue: this rank's block of output columns
// C[:, col0 : col0 + Ns] = act(A @ B_shard + bias_shard) is written at its place in EVERY buffer of `outs`
// (n_outs <= 8 device pointers to [M][ldc] f32 results: this GPU's own and, through IPC mappings, the other
// ranks'), tile by tile as the accumulators finish.  The caller orders the ranks afterwards (a stream-ordered
// barrier) before anyone reads a result.
extern "C" int fa_matmul_scatter(fa_ctx *ctx, const fa_tensor *a, fa_tensor *b, const fa_tensor *bias, int act,
                                 void *const *outs, int n_outs, int ldc, int col0) {
  if (!ctx || !outs) return fa_fail(ctx, FA_ERR_INVALID, "matmulScatter: NULL argument");
  FA_REQUIRE(ctx, fa_valid(ctx, a) && fa_valid(ctx, b), "matmulScatter: unknown tensor handle");
  const int M = a->rows, K = a->cols, N = b->cols;
  FA_REQUIRE(ctx, b->rows == K, "matmulScatter: A is [%d,%d] but B is [%d,%d]", M, K, b->rows, N);
  FA_REQUIRE(ctx, n_outs >= 1 && n_outs <= 8, "matmulScatter: %d result buffers (1..8)", n_outs);
  FA_REQUIRE(ctx, col0 >= 0 && col0 + N <= ldc, "matmulScatter: columns [%d,%d) do not fit a row of %d", col0, col0 + N, ldc);
  FA_REQUIRE(ctx, act >= 0 && act <= 5, "matmulScatter: unknown activation code %d", act);
  FA_REQUIRE(ctx, b->storage == FA_F16 && !b->view && tc_shape_ok(ctx, M, N, K) && M > ctx->f16_hilo_rows,
             "matmulScatter: needs f16-storage weights and a tensor-core sized product with more than %d rows",
             ctx->f16_hilo_rows);
  for (int i = 0; i < n_outs; i++) FA_REQUIRE(ctx, outs[i] != nullptr, "matmulScatter: result buffer %d is NULL", i);
  if (bias) FA_TRY(check_vec(ctx, bias, N, "matmulScatter: bias"));
  FA_CHECK_CUDA(ctx, cudaSetDevice(ctx->device));
  const float *ap = nullptr;
  fa_tensor *atmp = nullptr;
  FA_TRY(fa_as_f32(ctx, a, &ap, &atmp));
  Scratch sa(ctx);
  const __half *a16 = nullptr;
  bool hilo = false;
  int rc = ensure_bt_f16(ctx, b);
  if (rc == FA_OK) rc = row_operand_f16(ctx, a, ap, sa, &a16, &hilo);
  if (rc == FA_OK) {
    TcEpilogue ep;
    ep.bias = bias ? (const float *)bias->dptr : nullptr;
    ep.act = act;
    ep.ldc = ldc;
    ep.n_peers = n_outs - 1;
    for (int i = 1; i < n_outs; i++) ep.peer_out[i - 1] = (float *)outs[i] + col0;
    rc = fa_tc_gemm_f16(ctx, a16, (const __half *)b->bt_f16, (float *)outs[0] + col0, M, N, K, ep);
  }
  if (atmp) fa_free_tensor(ctx, atmp);
  return rc;
}

extern "C" int fa_matmul_int8(fa_ctx *ctx, const fa_tensor *a, fa_bytes *wq, const fa_tensor *scale, int N, int K,
                              const fa_tensor *bias, int act, fa_tensor **out) {
  if (!ctx || !out) return fa_fail(ctx, FA_ERR_INVALID, "matmulInt8: NULL argument");
  FA_REQUIRE(ctx, fa_valid(ctx, a) && fa_valid_bytes(ctx, wq), "matmulInt8: unknown handle");
  FA_REQUIRE(ctx, N > 0 && K > 0, "matmulInt8: N=%d K=%d", N, K);
  const int M = a->rows;
  FA_REQUIRE(ctx, a->cols == K, "matmulInt8: A is [%d,%d] but K=%d", M, a->cols, K);
  FA_REQUIRE(ctx, wq->nbytes >= (size_t)N * K, "matmulInt8: packed weights hold %zu bytes, need %zu", wq->nbytes,
             (size_t)N * K);
  FA_REQUIRE(ctx, act >= 0 && act <= 5, "matmulInt8: unknown activation code %d", act);
  FA_TRY(check_vec(ctx, scale, N, "matmulInt8: scale"));
  if (bias) FA_TRY(check_vec(ctx, bias, N, "matmulInt8: bias"));
  FA_CHECK_CUDA(ctx, cudaSetDevice(ctx->device));
  const float *ap = nullptr;
  fa_tensor *atmp = nullptr;
  FA_TRY(fa_as_f32(ctx, a, &ap, &atmp));
  fa_tensor *c = nullptr;
  FA_TRY(fa_tensor_new(ctx, M, N, FA_F32, true, &c));
  int rc = FA_OK;
  const float *biasp = bias ? (const float *)bias->dptr : nullptr;
  if (gemv_shape_ok(ctx, M, N, K) && fa_gemv_kn_ok(M, N, K, true)) {
    rc = fa_gemv_kn(ctx, ap, wq->dptr, true, (const float *)scale->dptr, biasp, act, nullptr, (float *)c->dptr, M, N, K);
  } else if (tc_shape_ok(ctx, M, N, K)) {
    const int limbs = ctx->int8_limbs;
    Scratch sa(ctx), ss(ctx);
    rc = ensure_nk_i8(ctx, wq, N, K);  // one-time repack per handle
    if (rc == FA_OK) rc = sa.get(fa_tc_act_bytes(M, K, 1, limbs));
    if (rc == FA_OK) rc = ss.get((size_t)M * 4);
    if (rc == FA_OK) rc = fa_prep_a_i8(ctx, ap, M, K, limbs, (int8_t *)sa.p, (float *)ss.p);
    if (rc == FA_OK) {
      TcEpilogue ep;
      ep.rowscale = (const float *)ss.p;
      ep.colscale = (const float *)scale->dptr;
      ep.bias = biasp;
      ep.act = act;
      rc = fa_tc_gemm_i8(ctx, (const int8_t *)sa.p, limbs, (const int8_t *)wq->nk_i8, c->dptr, false, M, N, K, ep);
    }
  } else {
    rc = fa_simt_gemm(ctx, ap, wq->dptr, 2, (const float *)scale->dptr, biasp, act, nullptr, (float *)c->dptr, M, N, K);
  }
  if (atmp) fa_free_tensor(ctx, atmp);
  if (rc != FA_OK) {
    fa_free_tensor(ctx, c);
    return rc;
  }
  *out = c;
  return FA_OK;
}

// fa_matmul_int8's tensor-core route for a caller that has written the activation digit planes and the row scales
// itself (the batched TDT joint): same product, same epilogue, no pass over the activations.
bool fa_matmul_int8_planes_ok(fa_ctx *ctx, int M, int N, int K) {
  return !(gemv_shape_ok(ctx, M, N, K) && fa_gemv_kn_ok(M, N, K, true)) && tc_shape_ok(ctx, M, N, K);
}
int fa_matmul_int8_planes(fa_ctx *ctx, const int8_t *a_planes, const float *rowscale, int limbs, int M, fa_bytes *wq,
                          const float *colscale, int N, int K, const float *bias, float *c) {
  FA_REQUIRE(ctx, fa_valid_bytes(ctx, wq) && wq->nbytes >= (size_t)N * K, "matmulInt8: bad weight handle");
  FA_TRY(ensure_nk_i8(ctx, wq, N, K));
  TcEpilogue ep;
  ep.rowscale = rowscale;
  ep.colscale = colscale;
  ep.bias = bias;
  ep.act = FA_ACT_NONE;
  return fa_tc_gemm_i8(ctx, a_planes, limbs, (const int8_t *)wq->nk_i8, c, false, M, N, K, ep);
}

extern "C" int fa_matmul_nbits(fa_ctx *ctx, const fa_tensor *a, fa_bytes *bq, const fa_tensor *scales, fa_bytes *zp,
                               int N, int block_size, fa_tensor **out) {
  if (!ctx || !out) return fa_fail(ctx, FA_ERR_INVALID, "matmulNBits: NULL argument");
  FA_REQUIRE(ctx, fa_valid(ctx, a) && fa_valid_bytes(ctx, bq) && fa_valid_bytes(ctx, zp), "matmulNBits: unknown handle");
  // the reference hard-codes a 16-byte block stride, so 32 is the only block size its layout can hold
  FA_REQUIRE(ctx, block_size == 32, "matmulNBits: block size %d unsupported (the packed layout fixes it at 32)", block_size);
  const int M = a->rows, K = a->cols;
  FA_REQUIRE(ctx, N > 0 && K > 0, "matmulNBits: N=%d K=%d", N, K);
  const int nblk = ceil_div(K, 32), zpb = ceil_div(nblk, 2);
  FA_REQUIRE(ctx, bq->nbytes >= (size_t)N * nblk * 16, "matmulNBits: packed weights hold %zu bytes, need %zu", bq->nbytes,
             (size_t)N * nblk * 16);
  FA_REQUIRE(ctx, zp->nbytes >= (size_t)N * zpb, "matmulNBits: zero-points hold %zu bytes, need %zu", zp->nbytes,
             (size_t)N * zpb);
  FA_TRY(check_vec(ctx, scales, N * nblk, "matmulNBits: scales"));
  FA_CHECK_CUDA(ctx, cudaSetDevice(ctx->device));
  const float *ap = nullptr;
  fa_tensor *atmp = nullptr;
  FA_TRY(fa_as_f32(ctx, a, &ap, &atmp));
  fa_tensor *c = nullptr;
  FA_TRY(fa_tensor_new(ctx, M, N, FA_F32, true, &c));
  int rc = FA_OK;
  if (gemv_shape_ok(ctx, M, N, K) && fa_gemv_nbits_ok(M, N, K, block_size)) {
    rc = fa_gemv_nbits(ctx, ap, (const uint8_t *)bq->dptr, (const float *)scales->dptr, (const uint8_t *)zp->dptr,
                       (float *)c->dptr, M, N, K, nblk, zpb);
  } else if (tc_shape_ok(ctx, M, N, K) && ctx->nbits_fused && (K & 31) == 0) {
    const bool cached = bq->nb_side && bq->side_N == N && bq->side_K == K && bq->side_scales == scales->dptr &&
                        bq->side_zp == zp->dptr;
    const size_t tb = fa_nbits_tiles_bytes(N, K), sb = (size_t)N * nblk * 4;
    if (!cached) {  // one-time tensor-core form of this handle: nibble tiles, block-major scales and zero-points
      FA_NO_FIRST_USE_IN_RECORDING(ctx, bq->dptr, "matmulNBits");
      if (bq->nb_side) fa_block_release(ctx, bq->nb_side);
      bq->nb_side = nullptr;
      rc = fa_block_acquire(ctx, tb + sb + (size_t)N * nblk, &bq->nb_side, &bq->nb_side_bytes);
      if (rc == FA_OK) {
        bq->side_N = N;
        bq->side_K = K;
        bq->side_scales = scales->dptr;
        bq->side_zp = zp->dptr;
        uint8_t *side = (uint8_t *)bq->nb_side;
        rc = fa_nbits_side(ctx, (const uint8_t *)bq->dptr, (const float *)scales->dptr, (const uint8_t *)zp->dptr, N, K, nblk,
                           zpb, side, (float *)(side + tb), side + tb + sb);
      }
    }
    Scratch sa(ctx);
    if (rc == FA_OK) rc = sa.get(fa_tc_act_bytes(M, K, 2, 1));
    if (rc == FA_OK) rc = fa_prep_a_f16_perm8(ctx, ap, M, K, (__half *)sa.p);
    if (rc == FA_OK) {
      const uint8_t *side = (const uint8_t *)bq->nb_side;
      rc = fa_tc_gemm_nbits(ctx, (const __half *)sa.p, side, (const float *)(side + tb), side + tb + sb, (float *)c->dptr, M,
                            N, K, nblk);
    }
  } else if (tc_shape_ok(ctx, M, N, K) && M <= ctx->nbits_mma_rows && fa_nbits_mma_ok(M, N, K, block_size, M <= ctx->f16_hilo_rows) &&
             (fa_nbits_mma_worth(ctx, N) || ctx->nbits_mma_rows > 16)) {
    rc = fa_nbits_mma(ctx, ap, (const uint8_t *)bq->dptr, (const float *)scales->dptr, (const uint8_t *)zp->dptr, (float *)c->dptr,
                      M, N, K, nblk, zpb, M <= ctx->f16_hilo_rows);
  } else if (tc_shape_ok(ctx, M, N, K)) {
    const bool cached = bq->nk_f16 && bq->f16_N == N && bq->f16_K == K && bq->f16_scales == scales->dptr &&
                        bq->f16_zp == zp->dptr;
    if (!cached) {
      FA_NO_FIRST_USE_IN_RECORDING(ctx, bq->dptr, "matmulNBits");
      if (bq->nk_f16) fa_block_release(ctx, bq->nk_f16);
      bq->nk_f16 = nullptr;
      rc = fa_block_acquire(ctx, fa_tc_weight_bytes(N, K, 2), &bq->nk_f16, &bq->nk_f16_bytes);
      if (rc == FA_OK) {
        bq->f16_N = N;
        bq->f16_K = K;
        bq->f16_scales = scales->dptr;
        bq->f16_zp = zp->dptr;
        rc = fa_pack_w_nbits_f16(ctx, (const uint8_t *)bq->dptr, (const float *)scales->dptr,
                                 (const uint8_t *)zp->dptr, N, K, nblk, zpb, (__half *)bq->nk_f16);
      }
    }
    Scratch sa(ctx);
    const __half *a16 = nullptr;
    bool hilo = false;
    if (rc == FA_OK) rc = row_operand_f16(ctx, a, ap, sa, &a16, &hilo);
    if (rc == FA_OK) {
      TcEpilogue ep;
      ep.a_hilo = hilo;
      rc = fa_tc_gemm_f16(ctx, a16, (const __half *)bq->nk_f16, (float *)c->dptr, M, N, K, ep);
    }
  } else {
    rc = fa_simt_nbits(ctx, ap, (const uint8_t *)bq->dptr, (const float *)scales->dptr, (const uint8_t *)zp->dptr,
                       (float *)c->dptr, M, N, K, nblk, zpb);
  }
  if (atmp) fa_free_tensor(ctx, atmp);
  if (rc != FA_OK) {
    fa_free_tensor(ctx, c);
    return rc;
  }
  *out = c;
  return FA_OK;
}

extern "C" int fa_int8_gemm_i32(fa_ctx *ctx, const int8_t *aq_host, int M, fa_bytes *wq, int N, int K,
                                int32_t *acc_out_host) {
  if (!ctx || !aq_host || !acc_out_host) return fa_fail(ctx, FA_ERR_INVALID, "int8GemmI32: NULL argument");
  FA_REQUIRE(ctx, fa_valid_bytes(ctx, wq), "int8GemmI32: unknown handle");
  FA_REQUIRE(ctx, M > 0 && N > 0 && K > 0, "int8GemmI32: M=%d N=%d K=%d", M, N, K);
  FA_REQUIRE(ctx, wq->nbytes >= (size_t)N * K, "int8GemmI32: packed weights hold %zu bytes, need %zu", wq->nbytes,
             (size_t)N * K);
  FA_REQUIRE(ctx, fa_tc_available(ctx), "int8GemmI32: tensor-map encoder unavailable");
  FA_CHECK_CUDA(ctx, cudaSetDevice(ctx->device));
  int rc = FA_OK;
  FA_TRY(ensure_nk_i8(ctx, wq, N, K));
  // stage the caller's int8 activations row-major, then pack them into the chunk-major operand layout
  Scratch raw(ctx), sa(ctx), acc_s(ctx);
  FA_TRY(raw.get((size_t)M * K));
  FA_CHECK_CUDA(ctx, cudaMemcpyAsync(raw.p, aq_host, (size_t)M * K, cudaMemcpyHostToDevice, ctx->stream));
  FA_TRY(sa.get(fa_tc_act_bytes(M, K, 1, 1)));
  FA_TRY(fa_pack_a_i8_raw(ctx, (const int8_t *)raw.p, M, K, (int8_t *)sa.p));
  FA_TRY(acc_s.get((size_t)M * N * 4));
  void *acc = acc_s.p;
  TcEpilogue ep;
  rc = fa_tc_gemm_i8(ctx, (const int8_t *)sa.p, 1, (const int8_t *)wq->nk_i8, acc, true, M, N, K, ep);
  if (rc == FA_OK) {
    cudaError_t e = cudaMemcpyAsync(acc_out_host, acc, (size_t)M * N * 4, cudaMemcpyDeviceToHost, ctx->stream);
    if (e != cudaSuccess) rc = fa_fail(ctx, FA_ERR_CUDA, "int8GemmI32 readback: %s", cudaGetErrorString(e));
  }
  if (rc == FA_OK) rc = fa_sync(ctx);
  return rc;
}


// Optional member matmulInt8Operand: y = act(scale[n] * sum_k f16(a[m,k]) * q[k,n] + bias[n]) + add[m,n] with the
// activations rounded to f16, as on the f16-B route of matmul (the reference's tolerance for that route is 2e-2), while
// the weights STAY int8 in device memory: the tensor-core kernel widens each int8 tile to f16 in shared memory and
// applies the per-column scale to the f32 accumulator.  This is what lets an encoder whose artifact stores int8 per
// output channel keep half the weight bytes resident, with the same producers (layernorm, attention, GLU + depthwise,
// a previous product) handing over packed f16 operands.  Shapes outside the tensor-core route go through matmulInt8.
extern "C" int fa_matmul_int8_operand(fa_ctx *ctx, const fa_tensor *a, fa_bytes *wq, const fa_tensor *scale, int N, int K,
                                      const fa_tensor *bias, int act, const fa_tensor *add, int operand_only, fa_tensor **out) {
  if (!ctx || !out) return fa_fail(ctx, FA_ERR_INVALID, "matmulInt8Operand: NULL argument");
  FA_REQUIRE(ctx, fa_valid(ctx, a) && fa_valid_bytes(ctx, wq), "matmulInt8Operand: unknown handle");
  FA_REQUIRE(ctx, N > 0 && K > 0, "matmulInt8Operand: N=%d K=%d", N, K);
  const int M = a->rows;
  FA_REQUIRE(ctx, a->cols == K, "matmulInt8Operand: A is [%d,%d] but K=%d", M, a->cols, K);
  FA_REQUIRE(ctx, wq->nbytes >= (size_t)N * K, "matmulInt8Operand: packed weights hold %zu bytes, need %zu", wq->nbytes, (size_t)N * K);
  FA_REQUIRE(ctx, act >= 0 && act <= 5, "matmulInt8Operand: unknown activation code %d", act);
  FA_TRY(check_vec(ctx, scale, N, "matmulInt8Operand: scale"));
  if (bias) FA_TRY(check_vec(ctx, bias, N, "matmulInt8Operand: bias"));
  if (add) {
    FA_TRY(check_vec(ctx, add, M * N, "matmulInt8Operand: add"));
    FA_REQUIRE(ctx, add->rows == M && add->cols == N, "matmulInt8Operand: add is [%d,%d], expected [%d,%d]", add->rows, add->cols, M, N);
  }
  if (!(tc_shape_ok(ctx, M, N, K) && M > ctx->f16_hilo_rows)) {  // decode sizes and tiny shapes: exact-activation routes
    fa_tensor *y = nullptr;
    FA_TRY(fa_matmul_int8(ctx, a, wq, scale, N, K, bias, act, &y));
    if (!add) {
      *out = y;
      return FA_OK;
    }
    const int rc = fa_ewise(ctx, y, add, 0, out);
    fa_free_tensor(ctx, y);
    return rc;
  }
  FA_CHECK_CUDA(ctx, cudaSetDevice(ctx->device));
  const float *ap = nullptr;
  fa_tensor *atmp = nullptr;
  const bool shadow_only = a->storage == FA_F32 && !a->view && a->a16_valid && !a->a16_hilo;
  if (!shadow_only) FA_TRY(fa_as_f32(ctx, a, &ap, &atmp));
  fa_tensor *c = nullptr;
  FA_TRY(fa_tensor_new(ctx, M, N, FA_F32, true, &c));
  Scratch sa(ctx);
  const __half *a16 = nullptr;
  bool hilo = false;
  int rc = ensure_nk_i8w(ctx, wq, N, K);
  if (rc == FA_OK) rc = row_operand_f16(ctx, a, ap, sa, &a16, &hilo);
  if (rc == FA_OK) {
    TcEpilogue ep;
    ep.a_hilo = hilo;
    ep.colscale = (const float *)scale->dptr;
    ep.bias = bias ? (const float *)bias->dptr : nullptr;
    ep.add = add ? (const float *)add->dptr : nullptr;
    ep.act = act;
    const bool hinted = operand_only && !add && fa_operand_only_ok(ctx, M, N);
    if ((act != FA_ACT_NONE || hinted) && (N & 63) == 0 && (ep.out16 = fa_shadow_block(ctx, c)) != nullptr) {
      c->a16_valid = true;
      if (ctx->lazy_f32 && !add && fa_operand_only_ok(ctx, M, N)) {
        ep.skip_f32 = true;
        c->f32_lazy = true;
        c->lazy_sticky = ctx->capturing != nullptr;
      }
    }
    rc = fa_tc_gemm_i8w_f16a(ctx, a16, (const int8_t *)wq->nk_i8w, (float *)c->dptr, M, N, K, ep);
  }
  if (atmp) fa_free_tensor(ctx, atmp);
  if (rc != FA_OK) {
    fa_free_tensor(ctx, c);
    return rc;
  }
  *out = c;
  return FA_OK;
}
