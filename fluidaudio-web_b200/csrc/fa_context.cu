// Context, memory pool, arenas, uploads, readback, batching, profiling.
//
// Mirrors the reference's WebGPU plumbing semantics on one CUDA stream:
//   - exact-size buffer pool and arena scopes: src/gpu/buffer-pool.js:49-135
//   - batch = queue order: src/gpu/scheduler.js:17-60 (a CUDA stream already orders work)
//   - staged single-use readback: src/gpu/compute.js:1101-1128
//   - timestamp profiler: src/gpu/scheduler.js:139-180 (here: cudaEvent pairs per launch)
#include "fa_internal.cuh"

static std::string g_err;  // failures that have no context yet

int fa_fail(fa_ctx *ctx, int code, const char *fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  (ctx ? ctx->err : g_err) = buf;
  return code;
}

extern "C" const char *fa_last_error(fa_ctx *ctx) { return (ctx ? ctx->err : g_err).c_str(); }

// ---- small conversion kernels -------------------------------------------------------------

__global__ void k_f32_to_f16(const float *__restrict__ in, __half *__restrict__ out, size_t n) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) out[i] = __float2half_rn(in[i]);
}
__global__ void k_f16_to_f32(const __half *__restrict__ in, float *__restrict__ out, size_t n) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) out[i] = __half2float(in[i]);
}
static int grid_for(fa_ctx *ctx, size_t n, int block) {
  size_t g = (n + block - 1) / block;
  size_t cap = (size_t)ctx->sm_count * 8;
  return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}

// ---- context ---------------------------------------------------------------------------

extern "C" int fa_ctx_create(int device, fa_ctx **out) {
  if (!out) return fa_fail(nullptr, FA_ERR_INVALID, "fa_ctx_create: out is NULL");
  *out = nullptr;
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (e != cudaSuccess || n == 0)
    return fa_fail(nullptr, FA_ERR_NO_DEVICE, "fa_ctx_create: no CUDA device (%s); this backend has no CPU fallback",
                   e != cudaSuccess ? cudaGetErrorString(e) : "count=0");
  if (device < 0 || device >= n) return fa_fail(nullptr, FA_ERR_INVALID, "fa_ctx_create: device %d of %d", device, n);
  cudaDeviceProp prop;
  FA_CHECK_CUDA(nullptr, cudaGetDeviceProperties(&prop, device));
  if (prop.major != 10)
    return fa_fail(nullptr, FA_ERR_NO_DEVICE, "fa_ctx_create: device %d is sm_%d%d; kernels are built for sm_100a only",
                   device, prop.major, prop.minor);
  FA_CHECK_CUDA(nullptr, cudaSetDevice(device));
  fa_ctx *ctx = new fa_ctx();
  ctx->device = device;
  ctx->sm_count = prop.multiProcessorCount;
  cudaError_t se = cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking);
  if (se != cudaSuccess) {
    delete ctx;
    return fa_fail(nullptr, FA_ERR_CUDA, "cudaStreamCreate: %s", cudaGetErrorString(se));
  }
  if (cudaMalloc(&ctx->dev_status, sizeof(int) * 4) != cudaSuccess ||
      cudaMemsetAsync(ctx->dev_status, 0, sizeof(int) * 4, ctx->stream) != cudaSuccess) {
    cudaStreamDestroy(ctx->stream);
    delete ctx;
    return fa_fail(nullptr, FA_ERR_CUDA, "fa_ctx_create: status word allocation failed");
  }
  ctx->gemv_ticket_count = 8192;
  if (cudaMalloc(&ctx->gemv_tickets, sizeof(int) * ctx->gemv_ticket_count) != cudaSuccess ||
      cudaMemsetAsync(ctx->gemv_tickets, 0, sizeof(int) * ctx->gemv_ticket_count, ctx->stream) != cudaSuccess) {
    cudaFree(ctx->dev_status);
    cudaStreamDestroy(ctx->stream);
    delete ctx;
    return fa_fail(nullptr, FA_ERR_CUDA, "fa_ctx_create: ticket array allocation failed");
  }
  *out = ctx;
  return FA_OK;
}

extern "C" int fa_ctx_destroy(fa_ctx *ctx) {
  if (!ctx) return FA_OK;
  cudaSetDevice(ctx->device);
  cudaStreamSynchronize(ctx->stream);
  for (auto &r : ctx->prof) {
    cudaEventDestroy(r.e0);
    cudaEventDestroy(r.e1);
  }
  for (fa_staged *s : ctx->staged) {
    if (s->host) cudaFreeHost(s->host);
    if (s->done) cudaEventDestroy(s->done);
    delete s;
  }
  for (auto &b : ctx->staged_free) cudaFreeHost(b.first);
  for (fa_graph *g : ctx->graphs) {
    if (g->exec) cudaGraphExecDestroy(g->exec);
    if (g->graph) cudaGraphDestroy(g->graph);
    delete g;
  }
  for (fa_tensor *t : ctx->tensors) delete t;
  for (fa_bytes *b : ctx->byte_handles) delete b;
  for (auto &kv : ctx->blocks) cudaFree(kv.first);
  cudaFree(ctx->dev_status);
  cudaFree(ctx->gemv_tickets);
  if (ctx->mark) cudaEventDestroy(ctx->mark);
  cudaStreamDestroy(ctx->stream);
  delete ctx;
  return FA_OK;
}

extern "C" int fa_ctx_set_option(fa_ctx *ctx, const char *key, long long value) {
  if (!ctx || !key) return fa_fail(ctx, FA_ERR_INVALID, "fa_ctx_set_option: NULL argument");
  if (!strcmp(key, "f16_hilo_rows")) {
    FA_REQUIRE(ctx, value >= 0, "f16_hilo_rows must be >= 0 (got %lld)", value);
    ctx->f16_hilo_rows = value > 0x7fffffffLL ? 0x7fffffff : (int)value;
    return FA_OK;
  }
  if (!strcmp(key, "lazy_f32")) {
    FA_REQUIRE(ctx, value == 0 || value == 1, "lazy_f32 must be 0 or 1 (got %lld)", value);
    ctx->lazy_f32 = (int)value;
    return FA_OK;
  }
  if (!strcmp(key, "attn_one_kernel")) {
    FA_REQUIRE(ctx, value == 0 || value == 1, "attn_one_kernel must be 0 or 1 (got %lld)", value);
    ctx->attn_one_kernel = (int)value;
    return FA_OK;
  }
  if (!strcmp(key, "pdl")) {
    FA_REQUIRE(ctx, value == 0 || value == 1, "pdl must be 0 or 1 (got %lld)", value);
    ctx->pdl = (int)value;
    return FA_OK;
  }
  if (!strcmp(key, "nbits_fused")) {
    FA_REQUIRE(ctx, value == 0 || value == 1, "nbits_fused must be 0 or 1 (got %lld)", value);
    ctx->nbits_fused = (int)value;
    return FA_OK;
  }
  if (!strcmp(key, "gemv_rows")) {
    FA_REQUIRE(ctx, value >= 0 && value <= kGemvMaxRows, "gemv_rows must be 0..%d (got %lld)", kGemvMaxRows, value);
    ctx->gemv_rows = (int)value;
    return FA_OK;
  }
  if (!strcmp(key, "int8_limbs")) {
    FA_REQUIRE(ctx, value >= 1 && value <= 3, "int8_limbs must be 1..3 (got %lld)", value);
    ctx->int8_limbs = (int)value;
    return FA_OK;
  }
  if (!strcmp(key, "gemv_ctas_per_sm")) {
    FA_REQUIRE(ctx, value >= 1 && value <= 4, "gemv_ctas_per_sm must be 1..4");
    ctx->gemv_ctas_per_sm = (int)value;
    return FA_OK;
  }
  if (!strcmp(key, "nbits_mma_rows")) {
    if (value < 0 || value > 17) return fa_fail(ctx, FA_ERR_INVALID, "option nbits_mma_rows: %lld (0..16, 17 = up to 16 rows whatever N)", value);
    ctx->nbits_mma_rows = (int)value;
    return FA_OK;
  }
  if (!strcmp(key, "tc_pair")) {
    ctx->tc_pair = value != 0;
    return FA_OK;
  }
  if (!strcmp(key, "tc_tma_store")) {
    ctx->tc_tma_store = value != 0;
    return FA_OK;
  }
  if (!strcmp(key, "tc_tile_rows")) {
    FA_REQUIRE(ctx, value >= 0 && value <= 256, "tc_tile_rows must be 0 (automatic) or 16..256");
    ctx->tc_tile_rows = (int)value;
    return FA_OK;
  }
  if (!strcmp(key, "tc_split_k")) {
    FA_REQUIRE(ctx, value >= 0 && value <= 8, "tc_split_k must be 0 (automatic) or 1..8");
    ctx->tc_split_k = (int)value;
    return FA_OK;
  }
  if (!strcmp(key, "wait_limit")) {
    FA_REQUIRE(ctx, value >= 4096 && value <= (1ll << 28), "wait_limit must be in 4096..2^28 polls");
    ctx->wait_limit = (unsigned)value;
    return FA_OK;
  }
  if (!strcmp(key, "tc_tma_add")) {
    FA_REQUIRE(ctx, value == 0 || value == 1, "tc_tma_add must be 0 or 1");
    ctx->tc_tma_add = (int)value;
    return FA_OK;
  }
  if (!strcmp(key, "tc_test_withhold_chunk")) {
    FA_REQUIRE(ctx, value >= -1 && value < 4096, "tc_test_withhold_chunk must be -1 or a K-chunk index");
    ctx->tc_withhold_chunk = (int)value;
    return FA_OK;
  }
  if (!strcmp(key, "pool_cap_bytes")) {
    FA_REQUIRE(ctx, value >= 0, "pool_cap_bytes must be >= 0");
    ctx->pool_cap = (size_t)value;
    return FA_OK;
  }
  return fa_fail(ctx, FA_ERR_INVALID, "fa_ctx_set_option: unknown option '%s'", key);
}

extern "C" int fa_ctx_stream(fa_ctx *ctx, void **stream_out) {
  if (!ctx || !stream_out) return fa_fail(ctx, FA_ERR_INVALID, "fa_ctx_stream: NULL argument");
  *stream_out = (void *)ctx->stream;
  return FA_OK;
}

// A context is one stream; two contexts on one GPU run concurrently.  fa_ctx_mark records a point in ctx's stream
// (everything enqueued so far), fa_ctx_wait_mark makes everything ctx enqueues from now on wait, on the device, for
// the point `other` marked last (no host wait; a context that never marked is not waited for).  This is how a pipeline
// of contexts keeps its copies concurrent while its forwards run one after the other (engines/fastconformer.py).
extern "C" int fa_ctx_mark(fa_ctx *ctx) {
  if (!ctx) return fa_fail(ctx, FA_ERR_INVALID, "fa_ctx_mark: NULL context");
  FA_REQUIRE(ctx, !ctx->capturing, "fa_ctx_mark: not allowed while a graph is being recorded");
  FA_CHECK_CUDA(ctx, cudaSetDevice(ctx->device));
  if (!ctx->mark) FA_CHECK_CUDA(ctx, cudaEventCreateWithFlags(&ctx->mark, cudaEventDisableTiming));
  FA_CHECK_CUDA(ctx, cudaEventRecord(ctx->mark, ctx->stream));
  return FA_OK;
}

extern "C" int fa_ctx_wait_mark(fa_ctx *ctx, fa_ctx *other) {
  if (!ctx || !other) return fa_fail(ctx, FA_ERR_INVALID, "fa_ctx_wait_mark: NULL context");
  FA_REQUIRE(ctx, !ctx->capturing, "fa_ctx_wait_mark: not allowed while a graph is being recorded");
  FA_REQUIRE(ctx, ctx->device == other->device, "fa_ctx_wait_mark: contexts on different devices (%d, %d)", ctx->device, other->device);
  if (!other->mark || other == ctx) return FA_OK;
  FA_CHECK_CUDA(ctx, cudaSetDevice(ctx->device));
  FA_CHECK_CUDA(ctx, cudaStreamWaitEvent(ctx->stream, other->mark, 0));
  return FA_OK;
}

extern "C" int fa_sync(fa_ctx *ctx) {
  if (!ctx) return fa_fail(ctx, FA_ERR_INVALID, "fa_sync: NULL context");
  FA_REQUIRE(ctx, !ctx->capturing, "sync/download/read is not allowed while a graph is being recorded");
  FA_CHECK_CUDA(ctx, cudaSetDevice(ctx->device));
  int st[4] = {0, 0, 0, 0};
  FA_CHECK_CUDA(ctx, cudaMemcpyAsync(st, ctx->dev_status, sizeof st, cudaMemcpyDeviceToHost, ctx->stream));
  FA_CHECK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  if (st[0] != 0) {
    cudaMemsetAsync(ctx->dev_status, 0, sizeof st, ctx->stream);
    return fa_fail(ctx, FA_ERR_TIMEOUT, "device-side bounded wait ran out (code %d, block %d, detail %d)", st[0], st[1],
                   st[2]);
  }
  if (st[3] != 0) {
    cudaMemsetAsync(ctx->dev_status, 0, sizeof st, ctx->stream);
    return fa_fail(ctx, FA_ERR_INVALID, "embedRows: a token id was outside the embedding table");
  }
  return FA_OK;
}

extern "C" int fa_launch_count(fa_ctx *ctx, unsigned long long *out) {
  if (!ctx || !out) return fa_fail(ctx, FA_ERR_INVALID, "fa_launch_count: NULL argument");
  *out = ctx->launches;
  return FA_OK;
}

// ---- blocks / pool ---------------------------------------------------------------------------

int fa_block_acquire(fa_ctx *ctx, size_t bytes, void **out, size_t *block_bytes) {
  size_t sz = round_up(bytes < 256 ? 256 : bytes, 256);
  if (ctx->capturing) {  // blocks already reserved for the graph being recorded come first
    auto g = ctx->capturing->free_list.find(sz);
    if (g != ctx->capturing->free_list.end() && !g->second.empty()) {
      *out = g->second.back();
      g->second.pop_back();
      ctx->reused++;
      *block_bytes = sz;
      return FA_OK;
    }
  }
  int rc = fa_block_acquire_global(ctx, sz, out);
  if (rc != FA_OK) return rc;
  *block_bytes = sz;
  if (ctx->capturing) {
    ctx->capturing->blocks.push_back(*out);
    ctx->block_owner[*out] = ctx->capturing;
  }
  return FA_OK;
}

int fa_block_acquire_global(fa_ctx *ctx, size_t sz, void **out) {
  auto it = ctx->pool.find(sz);
  if (it != ctx->pool.end() && !it->second.empty()) {
    *out = it->second.back();
    it->second.pop_back();
    ctx->pool_bytes -= sz;
    ctx->reused++;
    return FA_OK;
  }
  if (ctx->pool_cap && ctx->live_bytes + sz > ctx->pool_cap)
    return fa_fail(ctx, FA_ERR_OOM, "allocation of %zu bytes exceeds pool_cap_bytes (%zu live, cap %zu)", sz,
                   ctx->live_bytes, ctx->pool_cap);
  void *p = nullptr;
  cudaError_t e = cudaMalloc(&p, sz);
  if (e == cudaErrorMemoryAllocation && ctx->pool_bytes) {
    // give idle pool blocks back to the driver and retry once
    cudaGetLastError();
    if (!ctx->capturing) cudaStreamSynchronize(ctx->stream);
    for (auto &kv : ctx->pool) {
      for (void *q : kv.second) {
        cudaFree(q);
        ctx->blocks.erase(q);
        ctx->live_bytes -= kv.first;
      }
      kv.second.clear();
    }
    ctx->pool_bytes = 0;
    e = cudaMalloc(&p, sz);
  }
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fa_fail(ctx, e == cudaErrorMemoryAllocation ? FA_ERR_OOM : FA_ERR_CUDA, "cudaMalloc(%zu): %s", sz,
                   cudaGetErrorString(e));
  }
  ctx->blocks[p] = sz;
  ctx->live_bytes += sz;
  ctx->created++;
  ctx->created_bytes += sz;
  *out = p;
  return FA_OK;
}

void fa_block_release(fa_ctx *ctx, void *p) {
  auto it = ctx->blocks.find(p);
  if (it == ctx->blocks.end()) return;
  auto ow = ctx->block_owner.find(p);
  if (ow != ctx->block_owner.end()) {  // reserved for a graph: stays with it
    ow->second->free_list[it->second].push_back(p);
    return;
  }
  ctx->pool[it->second].push_back(p);
  ctx->pool_bytes += it->second;
}

void fa_block_free(fa_ctx *ctx, void *p) {
  auto it = ctx->blocks.find(p);
  if (it == ctx->blocks.end()) return;
  // The stream may still be reading the block: free after the queued work.
  cudaStreamSynchronize(ctx->stream);
  cudaFree(p);
  ctx->live_bytes -= it->second;
  ctx->blocks.erase(it);
}

bool fa_valid(fa_ctx *ctx, const fa_tensor *t) { return t && ctx->tensors.count(const_cast<fa_tensor *>(t)); }
int fa_touch_f32(fa_ctx *ctx, const fa_tensor *t) {
  fa_tensor *m = const_cast<fa_tensor *>(t);
  if (!m || !m->f32_lazy) return FA_OK;
  if (ctx->capturing && !m->lazy_sticky) {
    // a result from before the open recording: the fill below would only be captured, yet the tensor would look
    // current to an eager reader before the first replay
    auto ow = ctx->block_owner.find(m->dptr);
    if (ow == ctx->block_owner.end() || ow->second != ctx->capturing)
      return fa_fail(ctx, FA_ERR_INVALID,
                     "a hidden-layer result made before fa_graph_begin is first read as f32 inside the recording; read it "
                     "once (or run the sequence once eagerly) before recording");
  }
  if (!m->lazy_sticky) m->f32_lazy = false;
  return fa_unpack_a_f16(ctx, (const __half *)m->a16, m->rows, m->cols, (float *)m->dptr);
}

bool fa_valid_bytes(fa_ctx *ctx, const fa_bytes *b) { return b && ctx->byte_handles.count(const_cast<fa_bytes *>(b)); }

int fa_tensor_new(fa_ctx *ctx, int rows, int cols, int storage, bool pooled, fa_tensor **out) {
  FA_REQUIRE(ctx, rows >= 0 && cols >= 0, "tensor shape %dx%d is negative", rows, cols);
  FA_CHECK_CUDA(ctx, cudaSetDevice(ctx->device));
  size_t elt = storage == FA_F16 ? 2 : 4;
  void *p = nullptr;
  size_t blk = 0;
  FA_TRY(fa_block_acquire(ctx, (size_t)rows * cols * elt, &p, &blk));
  fa_tensor *t = new fa_tensor();
  t->rows = rows;
  t->cols = cols;
  t->storage = storage;
  t->dptr = p;
  t->bytes = blk;
  t->pooled = pooled;
  if (pooled && !ctx->arena_stack.empty()) {
    t->arena = ctx->arena_stack.back();
    ctx->arena_members[t->arena].push_back(t);
  }
  ctx->tensors.insert(t);
  *out = t;
  return FA_OK;
}

static void tensor_drop_storage(fa_ctx *ctx, fa_tensor *t) {
  if (t->view) return;
  if (t->bt_f16) fa_block_release(ctx, t->bt_f16);
  if (t->bt_tf32) fa_block_release(ctx, t->bt_tf32);
  t->bt_tf32 = nullptr;
  if (t->a16) fa_block_release(ctx, t->a16);
  if (t->hk16) fa_block_release(ctx, t->hk16);
  t->hk16 = nullptr;
  t->hk16_valid = false;
  if (t->dptr) fa_block_release(ctx, t->dptr);
  t->dptr = t->bt_f16 = t->a16 = nullptr;
  t->a16_valid = false;
}

// ---- uploads ----------------------------------------------------------------------------

static int upload_common(fa_ctx *ctx, const float *host, int rows, int cols, int storage, fa_tensor **out) {
  if (!ctx || !out) return fa_fail(ctx, FA_ERR_INVALID, "upload: NULL argument");
  FA_REQUIRE(ctx, host || (size_t)rows * cols == 0, "upload: host pointer is NULL");
  fa_tensor *t = nullptr;
  FA_TRY(fa_tensor_new(ctx, rows, cols, storage, /*pooled=*/false, &t));  // uploads are pool-exempt
  size_t n = (size_t)rows * cols;
  int rc = FA_OK;
  if (n) {
    if (storage == FA_F32) {
      cudaError_t e = cudaMemcpyAsync(t->dptr, host, n * 4, cudaMemcpyHostToDevice, ctx->stream);
      if (e != cudaSuccess) rc = fa_fail(ctx, FA_ERR_CUDA, "upload: %s", cudaGetErrorString(e));
    } else {
      void *tmp = nullptr;
      size_t blk = 0;
      rc = fa_block_acquire(ctx, n * 4, &tmp, &blk);
      if (rc == FA_OK) {
        cudaError_t e = cudaMemcpyAsync(tmp, host, n * 4, cudaMemcpyHostToDevice, ctx->stream);
        if (e != cudaSuccess) {
          rc = fa_fail(ctx, FA_ERR_CUDA, "uploadF16: %s", cudaGetErrorString(e));
        } else {
          {
            LaunchScope ls(ctx, "cvt_f32_f16");
            k_f32_to_f16<<<grid_for(ctx, n, 256), 256, 0, ctx->stream>>>((const float *)tmp, (__half *)t->dptr, n);
          }
          e = cudaGetLastError();
          if (e != cudaSuccess) rc = fa_fail(ctx, FA_ERR_CUDA, "launch cvt_f32_f16: %s", cudaGetErrorString(e));
        }
        fa_block_release(ctx, tmp);  // stream-ordered: the next user is queued after the convert
      }
    }
  }
  if (rc != FA_OK) {  // no half-made handle stays registered
    fa_free_tensor(ctx, t);
    return rc;
  }
  *out = t;
  return FA_OK;
}
extern "C" int fa_upload_f32(fa_ctx *ctx, const float *host, int rows, int cols, fa_tensor **out) {
  return upload_common(ctx, host, rows, cols, FA_F32, out);
}
extern "C" int fa_upload_f16(fa_ctx *ctx, const float *host, int rows, int cols, fa_tensor **out) {
  return upload_common(ctx, host, rows, cols, FA_F16, out);
}
extern "C" int fa_alloc(fa_ctx *ctx, int rows, int cols, fa_tensor **out) {
  if (!ctx || !out) return fa_fail(ctx, FA_ERR_INVALID, "alloc: NULL argument");
  return fa_tensor_new(ctx, rows, cols, FA_F32, true, out);
}
extern "C" int fa_alloc_f16(fa_ctx *ctx, int rows, int cols, fa_tensor **out) {
  if (!ctx || !out) return fa_fail(ctx, FA_ERR_INVALID, "allocF16: NULL argument");
  return fa_tensor_new(ctx, rows, cols, FA_F16, true, out);
}

extern "C" int fa_upload_bytes(fa_ctx *ctx, const void *host, size_t nbytes, fa_bytes **out) {
  if (!ctx || !out) return fa_fail(ctx, FA_ERR_INVALID, "uploadBytes: NULL argument");
  FA_REQUIRE(ctx, host || nbytes == 0, "uploadBytes: host pointer is NULL");
  FA_CHECK_CUDA(ctx, cudaSetDevice(ctx->device));
  fa_bytes *b = new fa_bytes();
  // 16 spare bytes so vector loads of the last partial group stay inside the block
  int rc = fa_block_acquire(ctx, nbytes + 16, &b->dptr, &b->block);
  if (rc != FA_OK) {
    delete b;
    return rc;
  }
  b->nbytes = nbytes;
  if (nbytes) FA_CHECK_CUDA(ctx, cudaMemcpyAsync(b->dptr, host, nbytes, cudaMemcpyHostToDevice, ctx->stream));
  ctx->byte_handles.insert(b);
  *out = b;
  return FA_OK;
}

extern "C" int fa_free_tensor(fa_ctx *ctx, fa_tensor *t) {
  if (!ctx) return fa_fail(ctx, FA_ERR_INVALID, "freeTensor: NULL context");
  if (!t) return FA_OK;
  FA_REQUIRE(ctx, fa_valid(ctx, t), "freeTensor: unknown or already freed tensor handle");
  if (t->arena >= 0) {
    auto &v = ctx->arena_members[t->arena];
    for (size_t i = 0; i < v.size(); i++)
      if (v[i] == t) {
        v[i] = v.back();
        v.pop_back();
        break;
      }
  }
  tensor_drop_storage(ctx, t);
  ctx->tensors.erase(t);
  delete t;
  return FA_OK;
}

extern "C" int fa_free_bytes(fa_ctx *ctx, fa_bytes *b) {
  if (!ctx) return fa_fail(ctx, FA_ERR_INVALID, "freeBytes: NULL context");
  if (!b) return FA_OK;
  FA_REQUIRE(ctx, fa_valid_bytes(ctx, b), "freeBytes: unknown or already freed handle");
  if (b->nk_i8) fa_block_release(ctx, b->nk_i8);
  if (b->nk_i8w) fa_block_release(ctx, b->nk_i8w);
  if (b->nk_f16) fa_block_release(ctx, b->nk_f16);
  if (b->nb_side) fa_block_release(ctx, b->nb_side);
  fa_block_release(ctx, b->dptr);
  ctx->byte_handles.erase(b);
  delete b;
  return FA_OK;
}

extern "C" int fa_pin(fa_ctx *ctx, fa_tensor *t, int to_parent) {
  if (!ctx) return fa_fail(ctx, FA_ERR_INVALID, "pin: NULL context");
  FA_REQUIRE(ctx, fa_valid(ctx, t), "pin: unknown tensor handle");
  if (t->arena < 0 || t->view) return FA_OK;
  auto &v = ctx->arena_members[t->arena];
  for (size_t i = 0; i < v.size(); i++)
    if (v[i] == t) {
      v[i] = v.back();
      v.pop_back();
      break;
    }
  int target = -1;
  if (to_parent) {
    // the arena opened just before t's arena, if it is still open (buffer-pool.js:103-126)
    for (size_t i = 0; i < ctx->arena_stack.size(); i++)
      if (ctx->arena_stack[i] == t->arena && i > 0) target = ctx->arena_stack[i - 1];
  }
  t->arena = target;
  if (target >= 0) ctx->arena_members[target].push_back(t);
  return FA_OK;
}

extern "C" int fa_push_arena(fa_ctx *ctx, int *handle_out) {
  if (!ctx || !handle_out) return fa_fail(ctx, FA_ERR_INVALID, "pushArena: NULL argument");
  int id = ctx->next_arena++;
  ctx->arena_stack.push_back(id);
  ctx->arena_members[id];
  *handle_out = id;
  return FA_OK;
}

extern "C" int fa_pop_arena(fa_ctx *ctx, int handle) {
  if (!ctx) return fa_fail(ctx, FA_ERR_INVALID, "popArena: NULL context");
  if (ctx->arena_stack.empty()) return FA_OK;  // the reference tolerates an unmatched pop
  int id = handle < 0 ? ctx->arena_stack.back() : handle;
  size_t pos = ctx->arena_stack.size();
  for (size_t i = 0; i < ctx->arena_stack.size(); i++)
    if (ctx->arena_stack[i] == id) pos = i;
  FA_REQUIRE(ctx, pos < ctx->arena_stack.size(), "popArena: arena %d is not open", id);
  ctx->arena_stack.erase(ctx->arena_stack.begin() + pos);  // scopes may close out of order
  auto it = ctx->arena_members.find(id);
  if (it != ctx->arena_members.end()) {
    for (fa_tensor *t : it->second) {
      tensor_drop_storage(ctx, t);
      ctx->tensors.erase(t);
      delete t;
    }
    ctx->arena_members.erase(it);
  }
  return FA_OK;
}

extern "C" int fa_trim_pool(fa_ctx *ctx, size_t budget_bytes) {
  if (!ctx) return fa_fail(ctx, FA_ERR_INVALID, "trimPool: NULL context");
  if (ctx->pool_bytes <= budget_bytes) return FA_OK;
  FA_CHECK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  for (auto &kv : ctx->pool) {
    while (!kv.second.empty() && ctx->pool_bytes > budget_bytes) {
      void *p = kv.second.back();
      kv.second.pop_back();
      cudaFree(p);
      ctx->blocks.erase(p);
      ctx->pool_bytes -= kv.first;
      ctx->live_bytes -= kv.first;
    }
  }
  return FA_OK;
}

extern "C" int fa_tensor_ptr(fa_ctx *ctx, const fa_tensor *t, void **device_ptr) {
  if (!ctx || !device_ptr) return fa_fail(ctx, FA_ERR_INVALID, "tensorPtr: NULL argument");
  FA_REQUIRE(ctx, fa_valid(ctx, t), "tensorPtr: unknown tensor handle");
  FA_CHECK_CUDA(ctx, cudaSetDevice(ctx->device));
  FA_TRY(fa_touch_f32(ctx, t));
  *device_ptr = t->dptr;
  return FA_OK;
}

extern "C" int fa_tensor_info(const fa_tensor *t, int *rows, int *cols, int *storage, void **device_ptr) {
  if (!t) return FA_ERR_INVALID;
  if (rows) *rows = t->rows;
  if (cols) *cols = t->cols;
  if (storage) *storage = t->storage;
  if (device_ptr) *device_ptr = t->dptr;
  return FA_OK;
}

extern "C" int fa_mem_stats(fa_ctx *ctx, unsigned long long *created, unsigned long long *created_bytes,
                            unsigned long long *reused, unsigned long long *pool_bytes) {
  if (!ctx) return fa_fail(ctx, FA_ERR_INVALID, "memStats: NULL context");
  if (created) *created = ctx->created;
  if (created_bytes) *created_bytes = ctx->created_bytes;
  if (reused) *reused = ctx->reused;
  if (pool_bytes) *pool_bytes = ctx->pool_bytes;
  return FA_OK;
}

extern "C" int fa_host_alloc(size_t nbytes, void **out) {
  if (!out) return FA_ERR_INVALID;
  cudaError_t e = cudaMallocHost(out, nbytes ? nbytes : 1);
  if (e != cudaSuccess) return fa_fail(nullptr, FA_ERR_OOM, "cudaMallocHost(%zu): %s", nbytes, cudaGetErrorString(e));
  return FA_OK;
}
extern "C" int fa_host_free(void *p) {
  if (p) cudaFreeHost(p);
  return FA_OK;
}

// ---- readback -----------------------------------------------------------------------------

int fa_as_f32(fa_ctx *ctx, const fa_tensor *t, const float **ptr, fa_tensor **tmp) {
  *tmp = nullptr;
  FA_TRY(fa_touch_f32(ctx, t));
  if (t->storage == FA_F32) {
    *ptr = (const float *)t->dptr;
    return FA_OK;
  }
  fa_tensor *c = nullptr;
  FA_TRY(fa_tensor_new(ctx, t->rows, t->cols, FA_F32, true, &c));
  size_t n = (size_t)t->rows * t->cols;
  if (n) {
    {
      LaunchScope ls(ctx, "cvt_f16_f32");
      k_f16_to_f32<<<grid_for(ctx, n, 256), 256, 0, ctx->stream>>>((const __half *)t->dptr, (float *)c->dptr, n);
    }
    FA_LAUNCH_CHECK(ctx, "cvt_f16_f32");
  }
  *ptr = (const float *)c->dptr;
  *tmp = c;
  return FA_OK;
}

extern "C" int fa_download(fa_ctx *ctx, const fa_tensor *t, float *host_out) {
  if (!ctx) return fa_fail(ctx, FA_ERR_INVALID, "download: NULL context");
  FA_REQUIRE(ctx, fa_valid(ctx, t), "download: unknown tensor handle");
  size_t n = (size_t)t->rows * t->cols;
  FA_REQUIRE(ctx, host_out || n == 0, "download: host pointer is NULL");
  FA_CHECK_CUDA(ctx, cudaSetDevice(ctx->device));
  if (n) {
    const float *src = nullptr;
    fa_tensor *tmp = nullptr;
    FA_TRY(fa_as_f32(ctx, t, &src, &tmp));
    FA_CHECK_CUDA(ctx, cudaMemcpyAsync(host_out, src, n * 4, cudaMemcpyDeviceToHost, ctx->stream));
    int rc = fa_sync(ctx);
    if (tmp) fa_free_tensor(ctx, tmp);
    return rc;
  }
  return fa_sync(ctx);
}

// The copy only, enqueued on the context's stream (recordable): host_out must be page-locked memory (fa_host_alloc)
// and is valid after the next fa_sync - or, inside a recorded batch, after a sync that follows each launch.
extern "C" int fa_download_async(fa_ctx *ctx, const fa_tensor *t, float *host_out) {
  if (!ctx) return fa_fail(ctx, FA_ERR_INVALID, "downloadAsync: NULL context");
  FA_REQUIRE(ctx, fa_valid(ctx, t), "downloadAsync: unknown tensor handle");
  FA_REQUIRE(ctx, t->storage == FA_F32, "downloadAsync: f32-storage tensors only");
  const size_t n = (size_t)t->rows * t->cols;
  FA_REQUIRE(ctx, host_out || n == 0, "downloadAsync: host pointer is NULL");
  FA_CHECK_CUDA(ctx, cudaSetDevice(ctx->device));
  if (!n) return FA_OK;
  FA_TRY(fa_touch_f32(ctx, t));
  FA_CHECK_CUDA(ctx, cudaMemcpyAsync(host_out, t->dptr, n * 4, cudaMemcpyDeviceToHost, ctx->stream));
  return FA_OK;
}

extern "C" int fa_stage_download(fa_ctx *ctx, const fa_tensor *t, fa_staged **out) {
  if (!ctx || !out) return fa_fail(ctx, FA_ERR_INVALID, "stageDownload: NULL argument");
  FA_REQUIRE(ctx, fa_valid(ctx, t), "stageDownload: unknown tensor handle");
  FA_CHECK_CUDA(ctx, cudaSetDevice(ctx->device));
  fa_staged *s = new fa_staged();
  s->count = (size_t)t->rows * t->cols;
  const size_t need = s->count ? s->count * 4 : 4;
  for (size_t i = 0; i < ctx->staged_free.size(); i++) {  // smallest free buffer that fits
    if (ctx->staged_free[i].second >= need && (!s->host || ctx->staged_free[i].second < s->host_bytes)) {
      s->host = ctx->staged_free[i].first;
      s->host_bytes = ctx->staged_free[i].second;
    }
  }
  if (s->host) {
    for (size_t i = 0; i < ctx->staged_free.size(); i++)
      if (ctx->staged_free[i].first == s->host) {
        ctx->staged_free.erase(ctx->staged_free.begin() + i);
        break;
      }
  } else {
    cudaError_t e = cudaMallocHost((void **)&s->host, need);
    if (e != cudaSuccess) {
      delete s;
      return fa_fail(ctx, FA_ERR_OOM, "stageDownload: cudaMallocHost: %s", cudaGetErrorString(e));
    }
    s->host_bytes = need;
  }
  ctx->staged.insert(s);
  int rc = FA_OK;
  if (s->count) {
    const float *src = nullptr;
    fa_tensor *tmp = nullptr;
    rc = fa_as_f32(ctx, t, &src, &tmp);
    if (rc == FA_OK) {
      // The copy is ordered now, at stage time: later ops on the stream cannot change what is read.
      cudaError_t e = cudaMemcpyAsync(s->host, src, s->count * 4, cudaMemcpyDeviceToHost, ctx->stream);
      if (e != cudaSuccess) rc = fa_fail(ctx, FA_ERR_CUDA, "stageDownload: %s", cudaGetErrorString(e));
    }
    if (tmp) fa_free_tensor(ctx, tmp);
  }
  if (rc == FA_OK) {
    cudaError_t e = cudaEventCreateWithFlags(&s->done, cudaEventDisableTiming);
    if (e == cudaSuccess) e = cudaEventRecord(s->done, ctx->stream);
    if (e != cudaSuccess) rc = fa_fail(ctx, FA_ERR_CUDA, "stageDownload: %s", cudaGetErrorString(e));
  }
  if (rc != FA_OK) {  // the caller gets no handle: give the staging buffer back and forget the read
    const std::string msg = ctx->err;
    fa_staged_free(ctx, s);
    ctx->err = msg;
    return rc;
  }
  *out = s;
  return FA_OK;
}

extern "C" int fa_staged_read(fa_ctx *ctx, fa_staged *s, float *host_out) {
  if (!ctx) return fa_fail(ctx, FA_ERR_INVALID, "StagedRead.read(): NULL context");
  FA_REQUIRE(ctx, s && ctx->staged.count(s), "StagedRead.read(): unknown handle");
  FA_REQUIRE(ctx, !s->consumed, "StagedRead.read(): already consumed (single-use)");
  FA_CHECK_CUDA(ctx, cudaEventSynchronize(s->done));
  if (s->count) memcpy(host_out, s->host, s->count * 4);
  s->consumed = true;
  // staging storage is released on first read (compute.d.ts:39-42): back to the context's free list (at most four
  // buffers are kept), and the event with it
  if (ctx->staged_free.size() < 4)
    ctx->staged_free.emplace_back(s->host, s->host_bytes);
  else
    cudaFreeHost(s->host);
  s->host = nullptr;
  cudaEventDestroy(s->done);
  s->done = nullptr;
  return FA_OK;
}

extern "C" int fa_staged_free(fa_ctx *ctx, fa_staged *s) {
  if (!ctx || !s) return FA_OK;
  if (!ctx->staged.count(s)) return fa_fail(ctx, FA_ERR_INVALID, "stagedFree: unknown handle");
  if (s->done) cudaEventSynchronize(s->done);
  if (s->host) cudaFreeHost(s->host);
  if (s->done) cudaEventDestroy(s->done);
  ctx->staged.erase(s);
  delete s;
  return FA_OK;
}

extern "C" int fa_rows_view(fa_ctx *ctx, fa_tensor *t, int rows, fa_tensor **out) {
  if (!ctx || !out) return fa_fail(ctx, FA_ERR_INVALID, "rowsView: NULL argument");
  FA_REQUIRE(ctx, fa_valid(ctx, t), "rowsView: unknown tensor handle");
  FA_TRY(fa_touch_f32(ctx, t));
  FA_REQUIRE(ctx, rows >= 0 && rows <= t->rows, "rowsView: %d rows of a %d-row tensor", rows, t->rows);
  fa_tensor *v = new fa_tensor();
  v->rows = rows;
  v->cols = t->cols;
  v->storage = t->storage;  // routing metadata is preserved (compute.d.ts:142-145)
  v->dptr = t->dptr;
  v->view = true;
  ctx->tensors.insert(v);
  *out = v;
  return FA_OK;
}

extern "C" int fa_reshape_view(fa_ctx *ctx, fa_tensor *t, int rows, int cols, fa_tensor **out) {
  if (!ctx || !out) return fa_fail(ctx, FA_ERR_INVALID, "reshapeView: NULL argument");
  FA_REQUIRE(ctx, fa_valid(ctx, t), "reshapeView: unknown tensor handle");
  FA_TRY(fa_touch_f32(ctx, t));
  FA_REQUIRE(ctx, rows >= 0 && cols >= 0 && (long long)rows * cols <= (long long)t->rows * t->cols,
             "reshapeView: [%d,%d] does not fit a [%d,%d] tensor", rows, cols, t->rows, t->cols);
  fa_tensor *v = new fa_tensor();
  v->rows = rows;
  v->cols = cols;
  v->storage = t->storage;
  v->dptr = t->dptr;
  v->view = true;
  ctx->tensors.insert(v);
  *out = v;
  return FA_OK;
}

// ---- peer mappings (one process per GPU) --------------------------------------------------------
// Every pool block is its own device allocation, so a tensor's storage can be exported as a CUDA IPC handle.

extern "C" int fa_ipc_export(fa_ctx *ctx, const fa_tensor *t, unsigned char handle_out[64]) {
  if (!ctx || !handle_out) return fa_fail(ctx, FA_ERR_INVALID, "ipcExport: NULL argument");
  FA_REQUIRE(ctx, fa_valid(ctx, t) && !t->view, "ipcExport: unknown tensor handle or a view");
  FA_TRY(fa_touch_f32(ctx, t));
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  FA_CHECK_CUDA(ctx, cudaSetDevice(ctx->device));
  cudaIpcMemHandle_t h;
  FA_CHECK_CUDA(ctx, cudaIpcGetMemHandle(&h, t->dptr));
  memcpy(handle_out, &h, 64);
  return FA_OK;
}

extern "C" int fa_ipc_open(fa_ctx *ctx, const unsigned char handle[64], void **dev_ptr_out) {
  if (!ctx || !handle || !dev_ptr_out) return fa_fail(ctx, FA_ERR_INVALID, "ipcOpen: NULL argument");
  FA_CHECK_CUDA(ctx, cudaSetDevice(ctx->device));
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, 64);
  FA_CHECK_CUDA(ctx, cudaIpcOpenMemHandle(dev_ptr_out, h, cudaIpcMemLazyEnablePeerAccess));
  return FA_OK;
}

extern "C" int fa_ipc_close(fa_ctx *ctx, void *dev_ptr) {
  if (!ctx) return fa_fail(ctx, FA_ERR_INVALID, "ipcClose: NULL context");
  FA_CHECK_CUDA(ctx, cudaSetDevice(ctx->device));
  FA_CHECK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  FA_CHECK_CUDA(ctx, cudaIpcCloseMemHandle(dev_ptr));
  return FA_OK;
}

// ---- batching -------------------------------------------------------------------------------

extern "C" int fa_begin_batch(fa_ctx *ctx) {
  if (!ctx) return fa_fail(ctx, FA_ERR_INVALID, "beginBatch: NULL context");
  FA_REQUIRE(ctx, !ctx->in_batch, "beginBatch: batch already open (not re-entrant)");
  ctx->in_batch = true;
  return FA_OK;
}
extern "C" int fa_end_batch(fa_ctx *ctx) {
  if (!ctx) return fa_fail(ctx, FA_ERR_INVALID, "endBatch: NULL context");
  FA_REQUIRE(ctx, ctx->in_batch, "endBatch: no open batch");
  ctx->in_batch = false;
  return FA_OK;
}

// ---- profiling ------------------------------------------------------------------------------

extern "C" int fa_profile_start(fa_ctx *ctx, int max_ops) {
  if (!ctx) return fa_fail(ctx, FA_ERR_INVALID, "startProfile: NULL context");
  for (auto &r : ctx->prof) {
    cudaEventDestroy(r.e0);
    cudaEventDestroy(r.e1);
  }
  ctx->prof.clear();
  ctx->profile_cap = max_ops > 0 ? max_ops : 4096;
  ctx->profiling = true;
  return FA_OK;
}

extern "C" int fa_profile_end(fa_ctx *ctx, fa_profile_entry *out, int capacity, int *n_out) {
  if (!ctx || !n_out) return fa_fail(ctx, FA_ERR_INVALID, "endProfile: NULL argument");
  ctx->profiling = false;
  FA_CHECK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  std::map<std::string, std::pair<float, int>> agg;
  std::vector<std::string> order;
  for (auto &r : ctx->prof) {
    float ms = 0.f;
    cudaEventElapsedTime(&ms, r.e0, r.e1);
    auto it = agg.find(r.label);
    if (it == agg.end()) {
      agg[r.label] = {ms, 1};
      order.push_back(r.label);
    } else {
      it->second.first += ms;
      it->second.second++;
    }
    cudaEventDestroy(r.e0);
    cudaEventDestroy(r.e1);
  }
  ctx->prof.clear();
  int n = 0;
  for (auto &name : order) {
    if (out && n < capacity) {
      memset(&out[n], 0, sizeof out[n]);
      strncpy(out[n].label, name.c_str(), sizeof(out[n].label) - 1);
      out[n].ms = agg[name].first;
      out[n].count = agg[name].second;
    }
    n++;
  }
  *n_out = n;
  return FA_OK;
}

// ---- recorded batches (CUDA graphs) ---------------------------------------------------------------

extern "C" int fa_graph_begin(fa_ctx *ctx) {
  if (!ctx) return fa_fail(ctx, FA_ERR_INVALID, "graphBegin: NULL context");
  FA_REQUIRE(ctx, !ctx->capturing, "graphBegin: a recording is already open");
  FA_CHECK_CUDA(ctx, cudaSetDevice(ctx->device));
  fa_graph *g = new fa_graph();
  // relaxed mode: a pool miss inside the recording may still call cudaMalloc
  cudaError_t e = cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeRelaxed);
  if (e != cudaSuccess) {
    delete g;
    return fa_fail(ctx, FA_ERR_CUDA, "cudaStreamBeginCapture: %s", cudaGetErrorString(e));
  }
  ctx->capturing = g;
  return FA_OK;
}

extern "C" int fa_graph_end(fa_ctx *ctx, fa_graph **out) {
  if (!ctx || !out) return fa_fail(ctx, FA_ERR_INVALID, "graphEnd: NULL argument");
  FA_REQUIRE(ctx, ctx->capturing, "graphEnd: no recording is open");
  fa_graph *g = ctx->capturing;
  ctx->capturing = nullptr;
  cudaError_t e = cudaStreamEndCapture(ctx->stream, &g->graph);
  if (e == cudaSuccess) e = cudaGraphInstantiate(&g->exec, g->graph, 0);
  ctx->graphs.insert(g);
  if (e != cudaSuccess) {
    fa_graph_free(ctx, g);
    return fa_fail(ctx, FA_ERR_CUDA, "graph capture/instantiate: %s", cudaGetErrorString(e));
  }
  *out = g;
  return FA_OK;
}

extern "C" int fa_graph_launch(fa_ctx *ctx, fa_graph *g) {
  if (!ctx) return fa_fail(ctx, FA_ERR_INVALID, "graphLaunch: NULL context");
  FA_REQUIRE(ctx, g && ctx->graphs.count(g) && g->exec, "graphLaunch: unknown graph handle");
  FA_REQUIRE(ctx, !ctx->capturing, "graphLaunch: not allowed while recording");
  FA_CHECK_CUDA(ctx, cudaGraphLaunch(g->exec, ctx->stream));
  return FA_OK;
}

extern "C" int fa_graph_free(fa_ctx *ctx, fa_graph *g) {
  if (!ctx) return fa_fail(ctx, FA_ERR_INVALID, "graphFree: NULL context");
  if (!g) return FA_OK;
  FA_REQUIRE(ctx, ctx->graphs.count(g), "graphFree: unknown graph handle");
  cudaStreamSynchronize(ctx->stream);
  if (g->exec) cudaGraphExecDestroy(g->exec);
  if (g->graph) cudaGraphDestroy(g->graph);
  // reserved blocks that are idle go back to the shared pool; blocks still held by live tensors just
  // lose their reservation and return to the pool when those tensors are freed
  for (void *p : g->blocks) ctx->block_owner.erase(p);
  for (auto &kv : g->free_list)
    for (void *p : kv.second) fa_block_release(ctx, p);
  ctx->graphs.erase(g);
  delete g;
  return FA_OK;
}
