// Internal declarations shared by the translation units of libfa_cuda.so.
// Nothing here crosses the C ABI (include/fa_cuda.h).
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <map>
#include <string>
#include <unordered_map>
#include <unordered_set>
#include <vector>

#include "../../include/fa_cuda.h"

// ---- handles ---------------------------------------------------------------

struct fa_tensor {
  int rows = 0, cols = 0;
  int storage = FA_F32;      // FA_F32 or FA_F16 element storage, row-major [rows][cols]
  void *dptr = nullptr;      // device pointer of element (0,0)
  size_t bytes = 0;          // size of the pool block behind dptr (0 for views)
  bool view = false;         // rowsView alias: owns nothing
  bool pooled = false;       // block returns to the pool (alloc) vs. plain free (upload)
  int arena = -1;            // id of the arena that releases it, -1 = persistent
  // Lazily built packed f16 copy used when this tensor is the weight side of a tensor-core GEMM.
  void *bt_f16 = nullptr;
  size_t bt_bytes = 0;
  // Lazily built value + residue f32 planes used when this f32-storage tensor is the weight side of a large product.
  void *bt_tf32 = nullptr;
  size_t bt_tf32_bytes = 0;
  bool bt_stale = false;  // the tensor was written in place after a packed weight copy was made: repack on next use
  // Packed f16 shadow Ap[k/64][row][k%64] used when this tensor is the row (activation) side of a
  // tensor-core GEMM.  Written by the producing kernel (layernorm, GEMM epilogue) or on first use;
  // dropped whenever the tensor is written in place.  Storage stays opaque to callers (compute.d.ts:10-15).
  void *a16 = nullptr;
  size_t a16_bytes = 0;
  bool a16_valid = false;
  bool a16_hilo = false;  // the shadow holds two planes (value, rounding residue)
  // Hidden-layer results (a product with a fused activation) are consumed by the next product through their
  // packed f16 shadow only, so their f32 storage is left unwritten until somebody else asks for it
  // (fa_touch_f32 then fills it from the shadow: the f16-rounded values the next product sees anyway).
  bool f32_lazy = false;
  bool lazy_sticky = false;  // produced inside a recording: every replay rewrites the shadow only, so the f32
                             // copy is refreshed on EVERY outside read, not just the first
  // Packed per-head f16 copy of this tensor as the shared KEYS of a batched attention product (the projected
  // positional table of a conformer layer is the same every step): built on first use, dropped with the shadow.
  void *hk16 = nullptr;
  size_t hk16_bytes = 0;
  bool hk16_valid = false;
  int hk_Tb = 0, hk_H = 0, hk_HD = 0;
  int hk_kind = 0;  // 0: per-head packed keys of the batched GEMM form; 1: plain row-major f16 copy (one-kernel attention)
};

struct fa_bytes {
  void *dptr = nullptr;
  size_t nbytes = 0;
  size_t block = 0;
  // Lazily built packed int8 copy of a [K][N] int8 payload.
  void *nk_i8 = nullptr;
  size_t nk_bytes = 0;
  int nk_N = 0, nk_K = 0;
  // Lazily built tile-contiguous int8 copy Wp8[n/128][k/64][n%128][64] for the f16-activation route (still one
  // byte per weight).
  void *nk_i8w = nullptr;
  size_t nk_i8w_bytes = 0;
  int i8w_N = 0, i8w_K = 0;
  // Lazily built packed f16 dequantised copy of an int4 payload (with the scales/zp it was built from).
  void *nk_f16 = nullptr;
  size_t nk_f16_bytes = 0;
  int f16_N = 0, f16_K = 0;
  const void *f16_scales = nullptr, *f16_zp = nullptr;
  // Lazily built tensor-core form of an int4 payload, still 4 bits per weight: nibble tiles
  // [n/128][k/64][n%128][32 B], then block-major scales sT f32 [nblk][N], then zero-points zT u8 [nblk][N] (one
  // unpacked nibble per byte) - what the in-kernel unpack reads, a contiguous 4 KB per tile and 32 rows per request.
  void *nb_side = nullptr;
  size_t nb_side_bytes = 0;
  int side_N = 0, side_K = 0;
  const void *side_scales = nullptr, *side_zp = nullptr;
};

struct fa_staged {
  float *host = nullptr;     // page-locked snapshot target (f32)
  void *dev_tmp = nullptr;   // device f32 temp when the source is f16 storage
  size_t dev_tmp_bytes = 0;
  size_t host_bytes = 0;     // capacity of `host` (it may come from the context's free list, larger than needed)
  size_t count = 0;
  cudaEvent_t done = nullptr;
  bool consumed = false;
};

struct fa_graph {
  cudaGraph_t graph = nullptr;
  cudaGraphExec_t exec = nullptr;
  std::vector<void *> blocks;                                 // device blocks reserved for this graph
  std::unordered_map<size_t, std::vector<void *>> free_list;  // reserved blocks not in use right now
};

struct ProfileRec {
  const char *label;
  cudaEvent_t e0, e1;
};

struct fa_ctx {
  int device = 0;
  int sm_count = 0;
  cudaStream_t stream = nullptr;
  cudaEvent_t mark = nullptr;      // fa_ctx_mark / fa_ctx_wait_mark: a point in this context's stream other contexts can wait for
  std::string err;
  bool in_batch = false;
  unsigned long long launches = 0;
  // options
  int int8_limbs = 2;
  int attn_one_kernel = 1; // attnFused as the single mma kernel (fa_attn_rel.cu) when the shape allows, else the GEMM form
  int lazy_f32 = 1;        // hidden-layer products leave their f32 result unwritten until it is asked for
  int pdl = 1;             // programmatic dependent launch between the library's kernels (see fa_launch_dep)
  int nbits_mma_rows = 16; // int4 products with more rows than the GEMV takes and at most this many stream the 4-bit
                           // weights once and multiply with mma.sync (0 = off: tensor-core GEMM on the f16 copy)
  int nbits_fused = 0;     // 1: int4 products on the tensor cores unpack nibbles in shared memory (0: f16 copy, faster today)
  int gemv_rows = 4;       // products with at most this many rows run on the CUDA-core GEMV kernels (0 = never)
  int gemv_ctas_per_sm = 2;  // resident CTAs per SM the int4 GEMV sizes its grid for
  int f16_hilo_rows = 64;  // f16-weight products with at most this many rows use value+residue row planes
  unsigned wait_limit = 1u << 24;  // polls before a device-side barrier wait gives up (about a second)
  int tc_withhold_chunk = -1;      // test hook, one launch: see TcParams::withhold_kb
  int tc_tma_add = 1;              // residual operand of the large f16 products through the copy engine (TcParams::tma_add)
  int tc_pair = 1;       // f16 products with more tiles than SMs run on CTA pairs sharing one 256-lane MMA
  int tc_tma_store = 1;  // results of plain tensor-core products leave through shared-memory slabs and TMA stores (0: per-lane stores)
  int tc_tile_rows = 0, tc_split_k = 0;  // tuning overrides for sub-wave tensor-core products (0 = chosen by the cost model)
  size_t pool_cap = 0;
  // exact-size pool (the reference pools by exact byte size, buffer-pool.js:49-84)
  std::unordered_map<size_t, std::vector<void *>> pool;
  size_t pool_bytes = 0;       // idle bytes in the pool
  size_t live_bytes = 0;       // bytes handed out by cudaMalloc and not yet cudaFree'd
  unsigned long long created = 0, created_bytes = 0, reused = 0;
  std::unordered_map<void *, size_t> blocks;   // every device block we own -> size
  // arenas: id -> tensors allocated while it was the newest open scope
  int next_arena = 1;
  std::vector<int> arena_stack;
  std::unordered_map<int, std::vector<fa_tensor *>> arena_members;
  std::unordered_set<fa_tensor *> tensors;     // every live handle
  std::unordered_set<fa_bytes *> byte_handles;
  std::unordered_set<fa_staged *> staged;
  // Page-locked staging buffers handed back by consumed reads, for the next stageDownload: allocating and freeing
  // page-locked memory costs milliseconds and synchronises the device, which a read-back per step cannot afford.
  std::vector<std::pair<float *, size_t>> staged_free;
  // profiling
  bool profiling = false;
  int profile_cap = 0;
  std::vector<ProfileRec> prof;
  // log-mel front end: device tables (filterbank, window, twiddles) per mel count, built on first use
  std::unordered_map<int, void *> mel_tables;
  std::unordered_map<int, int> mel_spans;  // widest filter of each mel count's filterbank, in bins
  // device-side status word written by kernels whose bounded waits ran out
  int *dev_status = nullptr;
  int *gemv_tickets = nullptr;  // zeroed arrival counters of the split-K GEMV (self-resetting)
  int gemv_ticket_count = 0;
  // graph recording: blocks acquired while `capturing` is set belong to that graph
  fa_graph *capturing = nullptr;
  std::unordered_map<void *, fa_graph *> block_owner;
  std::unordered_set<fa_graph *> graphs;
};

// ---- errors ----------------------------------------------------------------

int fa_fail(fa_ctx *ctx, int code, const char *fmt, ...);
#define FA_CHECK_CUDA(ctx, expr)                                                                      \
  do {                                                                                                \
    cudaError_t e__ = (expr);                                                                         \
    if (e__ != cudaSuccess)                                                                           \
      return fa_fail(ctx, e__ == cudaErrorMemoryAllocation ? FA_ERR_OOM : FA_ERR_CUDA, "%s: %s", #expr, \
                     cudaGetErrorString(e__));                                                        \
  } while (0)
#define FA_REQUIRE(ctx, cond, ...)                            \
  do {                                                        \
    if (!(cond)) return fa_fail(ctx, FA_ERR_INVALID, __VA_ARGS__); \
  } while (0)
#define FA_TRY(expr)            \
  do {                          \
    int rc__ = (expr);          \
    if (rc__ != FA_OK) return rc__; \
  } while (0)

// ---- memory (fa_context.cu) -----------------------------------------------------

int fa_block_acquire(fa_ctx *ctx, size_t bytes, void **out, size_t *block_bytes);
int fa_block_acquire_global(fa_ctx *ctx, size_t rounded_bytes, void **out);
void fa_block_release(fa_ctx *ctx, void *p);            // back to the pool
void fa_block_free(fa_ctx *ctx, void *p);               // cudaFree now
int fa_tensor_new(fa_ctx *ctx, int rows, int cols, int storage, bool pooled, fa_tensor **out);
bool fa_valid(fa_ctx *ctx, const fa_tensor *t);
bool fa_valid_bytes(fa_ctx *ctx, const fa_bytes *b);
// Makes the f32 storage of `t` current (see fa_tensor::f32_lazy); a no-op for every other tensor.  Every path
// that reads or aliases a tensor's f32 storage calls it first.
int fa_touch_f32(fa_ctx *ctx, const fa_tensor *t);
int fa_unpack_a_f16(fa_ctx *ctx, const __half *packed, int M, int K, float *out);
// f32 device pointer for `t`: the tensor itself when it is f32 storage, else a converted
// temporary (arena-scoped like any alloc) returned through *tmp.
int fa_as_f32(fa_ctx *ctx, const fa_tensor *t, const float **ptr, fa_tensor **tmp);

// ---- launch bookkeeping ------------------------------------------------------------

// Wraps one kernel launch: counts it and, while profiling, brackets it with CUDA events on the
// context stream (the reference profiler puts each dispatch in its own timestamped pass,
// scheduler.js:139-180).
struct LaunchScope {
  fa_ctx *ctx;
  bool rec = false;
  cudaEvent_t e0 = nullptr, e1 = nullptr;
  const char *label;
  LaunchScope(fa_ctx *c, const char *lbl) : ctx(c), label(lbl) {
    ctx->launches++;
    if (ctx->profiling && !ctx->capturing && (int)ctx->prof.size() < ctx->profile_cap) {
      if (cudaEventCreate(&e0) == cudaSuccess && cudaEventCreate(&e1) == cudaSuccess) {
        rec = true;
        cudaEventRecord(e0, ctx->stream);
      }
    }
  }
  ~LaunchScope() {
    if (rec) {
      cudaEventRecord(e1, ctx->stream);
      ctx->prof.push_back({label, e0, e1});
    }
  }
};
#define FA_LAUNCH_CHECK(ctx, label)                                                          \
  do {                                                                                       \
    cudaError_t e__ = cudaGetLastError();                                                    \
    if (e__ != cudaSuccess) return fa_fail(ctx, FA_ERR_CUDA, "launch %s: %s", label, cudaGetErrorString(e__)); \
  } while (0)

// ---- programmatic dependent launch -----------------------------------------------------
// Chains of short kernels (a decode step is ~120 of them) lose 1.5-2.5 us per boundary to launch latency and
// kernel prologues.  Kernels launched through fa_launch_dep carry the programmatic-stream-serialization
// attribute: the grid may be scheduled while its predecessor is still running.  Such a kernel MUST execute
// fa_grid_dep_sync() before it reads or writes anything its predecessors touch: the call first lets the NEXT
// grid in the stream be scheduled early in turn, then waits until every earlier grid has completed and its
// writes are visible.  Without the attribute (option "pdl" = 0, or a plain <<<>>> launch) the call is a no-op.
__device__ __forceinline__ void fa_grid_dep_sync() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

template <typename... KArgs, typename... Args>
inline cudaError_t fa_launch_dep(fa_ctx *ctx, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, Args &&...args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = ctx->stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = ctx->pdl ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// ---- device helpers ----------------------------------------------------------------

// Activation table of src/gpu/kernels/actf.js:5-22 (same clamps), f32.
// SiLU and the logistic gate through ONE special-function instruction per element: x*sigmoid(x) = h + h*tanh(h)
// with h = x/2, tanh.approx.f32 (error ~2^-11 of full scale, under the f16 rounding the results get as product
// operands).  The exp + reciprocal form needs two, and the special-function unit (16 results per clock per SM)
// is what the epilogue warps of a product with a fused SiLU wait on.
__device__ __forceinline__ float fa_tanh_approx(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float fa_silu_fast(float x) {
  const float h = 0.5f * x;
  return fmaf(h, fa_tanh_approx(h), h);
}
__device__ __forceinline__ float fa_sigmoid_fast(float x) { return fmaf(0.5f, fa_tanh_approx(0.5f * x), 0.5f); }

__device__ __forceinline__ float fa_actf(float x, int a) {
  switch (a) {
    case FA_ACT_GELU: {
      float t = fminf(fmaxf(0.7978845608028654f * (x + 0.044715f * x * x * x), -20.0f), 20.0f);
      return 0.5f * x * (1.0f + tanhf(t));
    }
    case FA_ACT_TANH: return tanhf(fminf(fmaxf(x, -20.0f), 20.0f));
    case FA_ACT_RELU: return fmaxf(x, 0.0f);
    case FA_ACT_SILU: return x / (1.0f + expf(-fminf(fmaxf(x, -30.0f), 30.0f)));
    case FA_ACT_GELU_ERF: {
      float z = x * 0.70710678118654752f;
      float t = 1.0f / (1.0f + 0.3275911f * fabsf(z));
      float y = 1.0f - (((((1.061405429f * t - 1.453152027f) * t) + 1.421413741f) * t - 0.284496736f) * t +
                        0.254829592f) * t * expf(-z * z);
      return 0.5f * x * (1.0f + (z >= 0.0f ? y : -y));
    }
    default: return x;
  }
}

static inline int ceil_div(int a, int b) { return (a + b - 1) / b; }
static inline size_t round_up(size_t a, size_t b) { return (a + b - 1) / b * b; }

// ---- kernel entry points implemented in other translation units -------------------------

// fa_gemm_simt.cu: any-shape f32-accumulate kernels (B given as f32/f16 [K][N] or int8 [K][N]).
int fa_simt_gemm(fa_ctx *ctx, const float *a, const void *b, int b_kind /*0 f32,1 f16,2 int8*/, const float *colscale,
                 const float *bias, int act, const float *add, float *c, int M, int N, int K);
int fa_simt_nbits(fa_ctx *ctx, const float *a, const uint8_t *bq, const float *scales, const uint8_t *zp, float *y,
                  int M, int N, int K, int nblk, int zpb);
// fa_gemv.cu: decode-size (M <= 16) bandwidth kernels.
int fa_gemv_nbits(fa_ctx *ctx, const float *a, const uint8_t *bq, const float *scales, const uint8_t *zp, float *y,
                  int M, int N, int K, int nblk, int zpb);
int fa_gemv_kn(fa_ctx *ctx, const float *a, const void *b, int b_kind, const float *colscale, const float *bias,
               int act, const float *add, float *c, int M, int N, int K);
// fa_gemm_tc.cu: tcgen05 kernels and their prepasses.
struct TcEpilogue {
  const float *rowscale = nullptr;  // [M] multiplies the accumulator (int8 activation scales)
  const float *colscale = nullptr;  // [N]
  const float *bias = nullptr;      // [N]
  const float *add = nullptr;       // [M][N]
  const float *rowbias = nullptr;   // [M] added before the activation
  int act = 0;
  bool a_hilo = false;
  bool a_shared = false;            // batched mode: all batches share the row operand
  bool skip_f32 = false;            // write only the packed f16 shadow (out16); the f32 result stays lazy
  float *peer_out[7] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};  // see TcParams::peer_out
  int n_peers = 0;
  const float *nb_scales = nullptr;  // int4 variant: per-block scales, packed zero-points, blocks per row
  const uint8_t *nb_zp = nullptr;
  int nblk = 0;              // f16 kind: the row operand is two planes (value, rounding residue)
  // optional second output: the epilogue result as a packed f16 activation shadow of a tensor with
  // o16_rows rows; this launch's rows/cols sit at (+o16_row_hi per batch/o_div, +o16_col_lo per batch%o_div)
  __half *out16 = nullptr;
  int o16_rows = 0, o16_row_hi = 0, o16_col_lo = 0;
  // batched launch: `batches` independent [M][N] products (see TcParams in fa_gemm_tc.cu)
  int batches = 1, w_batch_mod = 0, o_div = 1, ldc = 0;
  long long o_hi = 0, o_lo = 0;
};
// Packed ("box-contiguous") operand sizes: K is cut in chunks of 128 bytes.
static inline int fa_tc_chunks(int K, int elem_bytes) { return ceil_div(K, 128 / elem_bytes); }
static inline size_t fa_tc_weight_bytes(int N, int K, int elem_bytes) {
  return (size_t)ceil_div(N, 128) * fa_tc_chunks(K, elem_bytes) * 128 * 128;
}
static inline size_t fa_tc_act_bytes(int M, int K, int elem_bytes, int limbs) {
  return (size_t)limbs * fa_tc_chunks(K, elem_bytes) * M * 128;
}
int fa_tc_gemm_f16(fa_ctx *ctx, const __half *a_packed, const __half *w_packed, float *c, int M, int N, int K,
                   const TcEpilogue &ep);
int fa_tc_gemm_i8(fa_ctx *ctx, const int8_t *a_packed, int limbs, const int8_t *w_packed, void *c, bool raw_i32, int M,
                  int N, int K, const TcEpilogue &ep);
// CUDA-core products for M <= kGemvMaxRows activation rows, on the weights as uploaded (fa_gemv.cu)
constexpr int kGemvMaxRows = 4;
bool fa_gemv_nbits_ok(int M, int N, int K, int block_size);
bool fa_nbits_mma_ok(int M, int N, int K, int block_size, bool hilo);
bool fa_nbits_mma_worth(fa_ctx *ctx, int N);
int fa_nbits_mma(fa_ctx *ctx, const float *a, const uint8_t *bq, const float *scales, const uint8_t *zp, float *y, int M, int N,
                 int K, int nblk, int zpb, bool hilo);
int fa_gemv_nbits(fa_ctx *ctx, const float *a, const uint8_t *bq, const float *scales, const uint8_t *zp, float *y, int M,
                  int N, int K, int nblk, int zpb);
bool fa_gemv_kn_ok(int M, int N, int K, bool i8);
int fa_gemv_kn(fa_ctx *ctx, const float *a, const void *w, bool i8, const float *colscale, const float *bias, int act,
               const float *add, float *y, int M, int N, int K);
int fa_prep_a_f16(fa_ctx *ctx, const float *a, int M, int K, __half *out);
int fa_prep_a_f16_hilo(fa_ctx *ctx, const float *a, int M, int K, __half *out);
int fa_prep_a_f16_perm8(fa_ctx *ctx, const float *a, int M, int K, __half *out);
int fa_tc_gemm_nbits(fa_ctx *ctx, const __half *a_packed, const uint8_t *bq, const float *scales_t, const uint8_t *zp_t,
                     float *c, int M, int N, int K, int nblk);
size_t fa_nbits_tiles_bytes(int N, int K);
int fa_nbits_side(fa_ctx *ctx, const uint8_t *bq, const float *scales, const uint8_t *zp, int N, int K, int nblk, int zpb,
                  uint8_t *tiles, float *scales_t, uint8_t *zp_t);
int fa_prep_a_i8(fa_ctx *ctx, const float *a, int M, int K, int limbs, int8_t *out, float *rowscale);
// fa_matmul_int8 on digit planes and row scales written by the caller in fa_prep_a_i8's layout (fa_linalg.cu)
bool fa_matmul_int8_planes_ok(fa_ctx *ctx, int M, int N, int K);
int fa_matmul_int8_planes(fa_ctx *ctx, const int8_t *a_planes, const float *rowscale, int limbs, int M, fa_bytes *wq,
                          const float *colscale, int N, int K, const float *bias, float *c);
int fa_pack_a_i8_raw(fa_ctx *ctx, const int8_t *aq, int M, int K, int8_t *out);
int fa_pack_w_i8(fa_ctx *ctx, const int8_t *w_kn, int K, int N, int8_t *out);
int fa_pack_w_f16(fa_ctx *ctx, const void *w_kn, int src_storage, int K, int N, __half *out);
int fa_pack_w_f16_batched(fa_ctx *ctx, const void *w_kn, int K, int N, int batch, size_t src_stride, __half *out);
int fa_pack_w_nbits_f16(fa_ctx *ctx, const uint8_t *bq, const float *scales, const uint8_t *zp, int N, int K, int nblk,
                        int zpb, __half *out);
size_t fa_tc_i8w_weight_bytes(int N, int K);
int fa_pack_w_i8_k64(fa_ctx *ctx, const int8_t *w_kn, int K, int N, int8_t *out);
int fa_tc_gemm_i8w_f16a(fa_ctx *ctx, const __half *a_packed, const int8_t *w_packed, float *c, int M, int N, int K,
                        const TcEpilogue &ep);
size_t fa_tc_tf32_weight_bytes(int N, int K);
size_t fa_tc_tf32_act_bytes(int M, int K);
int fa_pack_w_tf32(fa_ctx *ctx, const float *w_kn, int K, int N, float *out);
int fa_prep_a_tf32(fa_ctx *ctx, const float *a, int M, int K, float *out);
int fa_tc_gemm_tf32(fa_ctx *ctx, const float *a_planes, const float *w_planes, float *c, int M, int N, int K,
                    const TcEpilogue &ep);
bool fa_tc_available(fa_ctx *ctx);
// Batched attention products on the tensor cores (fa_attn_tc.cu); return FA_OK and *done=false when the
// shape does not fit the packed layouts (the caller then uses the any-shape kernels).
int fa_tc_bmm_qk(fa_ctx *ctx, const float *q, const float *b, fa_tensor *b_cache, const float *qb, float *out, int T, int Tb, int H, int HD,
                 int W, int b_shared, bool *done);
int fa_tc_bmm_pv(fa_ctx *ctx, const float *p, const float *v, float *out, __half *out16, int Tq, int Tk, int H, int HD,
                 int W, bool *done);
// A producer whose result only feeds products may leave the f32 storage unwritten (fa_tensor::f32_lazy) when every
// such product is sure to take the tensor-core route and read the packed f16 operand: more rows than the hi/lo
// limit and rows x cols large enough that even a 64-column weight matrix passes the size rule of the router.
static inline bool fa_operand_only_ok(const fa_ctx *ctx, int rows, int cols) {
  return ctx->lazy_f32 && rows > ctx->f16_hilo_rows && cols >= 64 && (long long)rows * cols * 64 >= (1ll << 21);
}
bool fa_attn_rel_shape_ok(int T, int H, int HD, int W);
int fa_attn_rel(fa_ctx *ctx, const float *q, const float *k, const float *v, const float *pos, fa_tensor *pos_cache,
                const float *pbu, const float *pbv, float *out, __half *out16, int T, int H, int HD, int W, int ldq);
int fa_tc_attn_fused(fa_ctx *ctx, const float *q, const float *k, const float *v, const float *pos, fa_tensor *pos_cache, const float *pbu,
                     const float *pbv, float *out, __half *out16, int T, int H, int HD, int W, bool *done);
// Shadow management (fa_linalg.cu): block for t's packed f16 shadow (nullptr when t cannot carry one),
// and the shadow itself, built by the prepass when no producer wrote it.
__half *fa_shadow_block(fa_ctx *ctx, fa_tensor *t);
__half *fa_shadow_hilo_block(fa_ctx *ctx, fa_tensor *t);
int fa_shadow_ensure(fa_ctx *ctx, fa_tensor *t, const __half **out);
// Called by in-place writers AFTER they made the f32 storage current (need_f32): from here on the f32 storage
// is the truth again.
static inline void fa_shadow_drop(fa_tensor *t) {
  t->bt_stale = t->bt_f16 != nullptr || t->bt_tf32 != nullptr;
  t->a16_valid = false;
  t->hk16_valid = false;
  t->f32_lazy = false;
  t->lazy_sticky = false;
}
