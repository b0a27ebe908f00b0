/*
 * fa_cuda.h — C ABI of the CUDA (sm_100a) compute backend for fluidaudio-web's
 * quantized matrix-product path.
 *
 * Each entry point is what an N-API addon binds to implement one member of the
 * reference's ComputeContext interface (src/gpu/compute.d.ts:106-255); the member
 * it replaces is cited beside it.  Plain C types only: opaque handles, pointers,
 * sizes, ints.  Every function returns 0 on success and a non-zero FA_ERR_* code on
 * failure; fa_last_error() then holds a message of the same class the reference
 * throws as a JS Error.  All calls for one fa_ctx come from one host thread
 * (the reference's contexts are single-threaded, compute.d.ts / README.md:135-138).
 *
 * Ops are enqueue-only on the context's CUDA stream (program order = execution
 * order, which is what the reference's batch/submit model guarantees); only
 * fa_download, fa_staged_read and fa_sync block.
 *
 * There is no CPU fallback: without a CUDA device fa_ctx_create fails.
 */
#ifndef FA_CUDA_H
#define FA_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif
#if defined(__GNUC__)
#pragma GCC visibility push(default) /* the library is built with hidden visibility; these are its exports */
#endif

typedef struct fa_ctx fa_ctx;       /* one ComputeContext (compute.d.ts:106) */
typedef struct fa_tensor fa_tensor; /* Tensor {rows, cols}, storage opaque (compute.d.ts:12-15) */
typedef struct fa_bytes fa_bytes;   /* PackedBytes from uploadBytes (compute.d.ts:34) */
typedef struct fa_staged fa_staged; /* StagedRead, single use (compute.d.ts:39-45) */
typedef struct fa_graph fa_graph;   /* a recorded batch that can be submitted repeatedly */

enum {
  FA_OK = 0,
  FA_ERR_INVALID = 1,   /* contract violation: bad handle, shape mismatch, nested batch, second read() */
  FA_ERR_CUDA = 2,      /* a CUDA runtime/driver call failed */
  FA_ERR_OOM = 3,       /* device allocation failed or the configured cap was exceeded */
  FA_ERR_NO_DEVICE = 4, /* no CUDA device / unsupported architecture */
  FA_ERR_TIMEOUT = 5    /* a bounded device-side wait ran out (kernel reported it and returned) */
};

/* Activation codes: src/gpu/kernels/actf.js:24 */
enum { FA_ACT_NONE = 0, FA_ACT_GELU = 1, FA_ACT_TANH = 2, FA_ACT_RELU = 3, FA_ACT_SILU = 4, FA_ACT_GELU_ERF = 5 };

/* Tensor storage kinds reported by fa_tensor_info. */
enum { FA_F32 = 0, FA_F16 = 1 };

/* ---- context ----------------------------------------------------------- */
/* createContext({backend:"cuda"}) branch of src/gpu/context.js:23-37. */
int fa_ctx_create(int device, fa_ctx **out);
/* ComputeContext.destroy (compute.d.ts:133): frees every device allocation of the context. */
int fa_ctx_destroy(fa_ctx *ctx);
/* Message of the most recent failure on ctx (ctx may be NULL for fa_ctx_create failures). */
const char *fa_last_error(fa_ctx *ctx);
/* Integer options: "int8_limbs" (1..3, see fa_matmul_int8), "pool_cap_bytes" (0 = none; allocation
 * beyond it fails with FA_ERR_OOM — the reference's poolBudgetBytes, compute.js:128-137),
 * "f16_hilo_rows" (>= 0, default 64: tensor-core products against f16 weights whose row operand has
 * at most this many rows feed it as two f16 planes, value and rounding residue, summed in the f32
 * accumulator, so token-by-token decoding keeps f32-grade activations at twice the MMA work; 0 turns
 * it off, a huge value applies it to every product), "gemv_rows" (0..4, default 4: products with at
 * most this many activation rows stream the weights through the CUDA-core GEMV kernels - no packing,
 * f32 / exact-integer activations; 0 sends them to the tensor-core kernel), "nbits_fused" (0/1, default 0:
 * 1 = int4 products on the tensor cores stream 4-bit tiles and unpack them in shared memory inside the
 * kernel; 0 = through a one-time dequantised f16 copy of the weights, which is the faster of the two
 * today), "pdl" (0/1, default 1: the library's kernels are chained with programmatic dependent launch, so a
 * kernel's scheduling and prologue overlap its predecessor's tail; every such kernel waits for its
 * predecessors before touching their data; 0 = plain stream order), "lazy_f32" (0/1, default 1: the result of
 * a tensor-core product with a fused activation is written only as the packed f16 operand of the next product;
 * its f32 storage is filled from that, f16-rounded, the first time anything else reads it; the same holds for
 * the results of layernormOperand, gluDwConvTimeMajor and attnFused), "attn_one_kernel" (0/1, default 1:
 * attnFused runs as one kernel per call when head width is 128 and T <= 192; 0 = the batched-GEMM form),
 * "nbits_mma_rows" (0..17, default 16: int4 products with more activation rows than the GEMV takes and at most this
 * many - at most 16 - stream the 4-bit weights once as uploaded, widen them to f16 in registers and multiply with
 * mma.sync, when the matrix is narrow enough for that to beat the tensor-core GEMM on the dequantised copy; 17 = for
 * every width; 0 = never), "tc_pair" (0/1, default 1: f16-weight products with more tiles than SMs run on pairs of thread blocks that
 * share one 256-lane tcgen05 MMA, each loading half of the activation rows of the pair's tile; results are
 * bit-identical to the one-block kernel, 0 selects that kernel), "tc_tma_store" (0/1, default 1: results of plain
 * tensor-core products leave through shared-memory slabs and copy-engine stores; 0 = per-lane stores, same values),
 * "tc_tma_add" (0/1, default 1: the residual operand of an f16-weight product with K <= 2048 and an f32 result reaches
 * the epilogue through copy-engine loads into shared memory, two blocks ahead; 0 = plain loads, same values),
 * "tc_tile_rows" / "tc_split_k" (0 = automatic, the default; otherwise rows per tile - 128..256 for a pair's tile -
 * and CTAs per K-split cluster of tensor-core products with less than one wave of tiles) and "gemv_ctas_per_sm"
 * (1..4, default 2: resident thread blocks per SM the int4 GEMV sizes its grid for) are tuning overrides of choices
 * the library makes by shape, "wait_limit" (4096..2^28, default 2^24, about a second: polls after which a device-side barrier wait gives
 * up; the kernel then records a status word, unwinds and returns, and the next fa_sync fails with
 * FA_ERR_TIMEOUT while the context stays usable), "tc_test_withhold_chunk" (-1 = off; k >= 0: test hook for that
 * path - in the NEXT tensor-core product only, one thread block never loads K chunk k of its first tile, so
 * the waits behind it run out; the product's result is then undefined.  fa_tdt_decode_proj consumes it the same
 * way: one warp of its first prediction-network launch never loads stage k of its operand ring). */
int fa_ctx_set_option(fa_ctx *ctx, const char *key, long long value);
/* cudaStream_t of the context, for callers that order their own work after it. */
int fa_ctx_stream(fa_ctx *ctx, void **stream_out);
/* Ordering between two contexts (streams) of one GPU, on the device, with no host wait: fa_ctx_mark records a point
 * in ctx's stream (all that was enqueued so far); fa_ctx_wait_mark makes what ctx enqueues from now on wait for the
 * point `other` marked last (a no-op when other never marked).  Not part of the reference interface, whose one
 * queue orders everything (src/gpu/scheduler.js:17-60); here it lets a pipeline of contexts overlap the copies of
 * one batch with the forward of another while the forwards themselves run one after the other. */
int fa_ctx_mark(fa_ctx *ctx);
int fa_ctx_wait_mark(fa_ctx *ctx, fa_ctx *other);
/* Block until every enqueued op has finished; surfaces asynchronous kernel errors. */
int fa_sync(fa_ctx *ctx);
/* Number of kernels this library has launched on ctx since creation. */
int fa_launch_count(fa_ctx *ctx, unsigned long long *out);

/* ---- tensors & memory (compute.d.ts:109-133) ----------------------------- */
int fa_upload_f32(fa_ctx *ctx, const float *host, int rows, int cols, fa_tensor **out);  /* upload :110 */
int fa_upload_f16(fa_ctx *ctx, const float *host, int rows, int cols, fa_tensor **out);  /* uploadF16 :112 */
int fa_alloc(fa_ctx *ctx, int rows, int cols, fa_tensor **out);                          /* alloc :113 */
int fa_alloc_f16(fa_ctx *ctx, int rows, int cols, fa_tensor **out);                      /* allocF16 :114 */
int fa_upload_bytes(fa_ctx *ctx, const void *host, size_t nbytes, fa_bytes **out);       /* uploadBytes :119 */
int fa_free_tensor(fa_ctx *ctx, fa_tensor *t);                                           /* freeTensor :122 */
int fa_free_bytes(fa_ctx *ctx, fa_bytes *b);
int fa_pin(fa_ctx *ctx, fa_tensor *t, int to_parent);                                    /* pin :125 */
int fa_push_arena(fa_ctx *ctx, int *handle_out);                                         /* pushArena :128 */
int fa_pop_arena(fa_ctx *ctx, int handle); /* popArena :129; handle < 0 closes the newest open arena */
int fa_trim_pool(fa_ctx *ctx, size_t budget_bytes);                                      /* trimPool :131 */
int fa_tensor_info(const fa_tensor *t, int *rows, int *cols, int *storage, void **device_ptr);
/* Device pointer of a tensor's storage for callers that hand it to other libraries (NCCL, their own kernels).
 * Use this rather than fa_tensor_info's device_ptr: a hidden-layer result (a product with a fused activation)
 * keeps its f32 storage unwritten until something asks for it, and this call is such an ask. */
int fa_tensor_ptr(fa_ctx *ctx, const fa_tensor *t, void **device_ptr);
/* memStats / poolInfo (compute.d.ts:252-254): allocations made, bytes made, pool hits, bytes idle in the pool. */
int fa_mem_stats(fa_ctx *ctx, unsigned long long *created, unsigned long long *created_bytes,
                 unsigned long long *reused, unsigned long long *pool_bytes);
/* Page-locked host memory for callers that want uploads/downloads to be truly asynchronous. */
int fa_host_alloc(size_t nbytes, void **out);
int fa_host_free(void *p);

/* ---- readback (compute.d.ts:135-145) -------------------------------------- */
int fa_download(fa_ctx *ctx, const fa_tensor *t, float *host_out);          /* download / downloadF16 :137-138 */
/* The device-to-host copy of an f32 tensor alone, enqueued on the context's stream (and recorded, inside
 * fa_graph_begin/end): host_out must be page-locked (fa_host_alloc); its contents are valid after the next fa_sync.
 * Lets a recorded batch end with its own read-back, so a replay needs no per-step staging or host-side copy. */
int fa_download_async(fa_ctx *ctx, const fa_tensor *t, float *host_out);
int fa_stage_download(fa_ctx *ctx, const fa_tensor *t, fa_staged **out);    /* stageDownload :141 */
int fa_staged_read(fa_ctx *ctx, fa_staged *s, float *host_out); /* StagedRead.read :44; 2nd call: FA_ERR_INVALID */
int fa_staged_free(fa_ctx *ctx, fa_staged *s);
int fa_rows_view(fa_ctx *ctx, fa_tensor *t, int rows, fa_tensor **out);     /* rowsView :145 */
/* The same storage seen as [rows, cols] with rows*cols <= the tensor's element count (row-major order
 * unchanged).  No counterpart in compute.d.ts, where a JS engine re-labels {rows, cols} on the tensor
 * object itself; the batched multi-stream decoder uses it to see [streams, D] as [1, streams*D]. */
int fa_reshape_view(fa_ctx *ctx, fa_tensor *t, int rows, int cols, fa_tensor **out);

/* ---- batching (compute.d.ts:147-151) --------------------------------------- */
int fa_begin_batch(fa_ctx *ctx); /* beginBatch :148; nested call fails like scheduler.js:20 */
int fa_end_batch(fa_ctx *ctx);   /* endBatch :149 */

/* Recorded batches.  The reference records a whole forward into ONE command buffer and submits it once
 * (withBatchSync, src/gpu/scheduler.js:17-60; src/engines/asr-parakeet/raw-encoder.js:288-291).  The CUDA
 * form is a graph: ops enqueued between fa_graph_begin and fa_graph_end are captured instead of run, and
 * fa_graph_launch replays them with one submission.  Rules: no download/sync/staged read while recording;
 * uploads inside a recording must come from fa_host_alloc memory (replays re-read that memory);
 * device blocks touched by the recording stay reserved for the graph until fa_graph_free, so tensors made
 * inside it (its outputs) stay valid across replays.
 * Run the sequence once eagerly before recording it: handles cache work on their first use (the packed
 * tensor-core copy of a weight matrix, the f32 fill of a hidden-layer result), and a first use inside a
 * recording would only be captured while the handle already looked ready.  Such a first use of a handle
 * made before fa_graph_begin fails with FA_ERR_INVALID; row operands from before the recording that carry
 * no packed copy yet are packed into per-call scratch on every replay instead. */
int fa_graph_begin(fa_ctx *ctx);
int fa_graph_end(fa_ctx *ctx, fa_graph **out);
int fa_graph_launch(fa_ctx *ctx, fa_graph *g);
int fa_graph_free(fa_ctx *ctx, fa_graph *g);

/* ---- linear algebra: the hot path (compute.d.ts:153-168) ------------------- */
/* matmul :155, and matmulV2/V3/V4/F16 :158-162 (one shape-routed implementation):
 * C = act(A[M,K] @ B[K,N] + bias[1,N]) + add[M,N].  bias/add may be NULL.  B may be f32 or
 * f16 storage (uploadF16); routing is by shape and storage only.
 * Precision: f32-storage B and small or ragged shapes are computed in f32.  Against f16-storage B a
 * tensor-core sized product rounds A to f16 (to f16 value + f16 residue, ~22 bits, for at most
 * "f16_hilo_rows" rows) and accumulates in f32 - the reference's f16-B route (tolerance 2e-2 in its gate).
 * With option "lazy_f32" (default) a result with a fused activation and no residual, large enough that every
 * product consuming it takes the tensor-core route (more than "f16_hilo_rows" rows, rows*cols*64 >= 2^21), is
 * kept as its packed f16 operand; read any other way it comes back rounded to f16 (relative 5e-4). */
int fa_matmul(fa_ctx *ctx, const fa_tensor *a, fa_tensor *b, const fa_tensor *bias, int act, const fa_tensor *add,
              fa_tensor **out);
/* Optional member matmul(..., {operandOnly: true}): the caller states that the result is only read as a packed f16
 * operand - by another matmul or by attnFusedQKV.  A tensor-core sized result is then written as that operand alone
 * (f32 storage filled from it, f16-rounded, if anything else reads the tensor).  No residual input. */
int fa_matmul_operand(fa_ctx *ctx, const fa_tensor *a, fa_tensor *b, const fa_tensor *bias, int act, fa_tensor **out);
/* matmulInt8 :164.  wq: int8 weights, byte index k*N+n (rust/wasm-kernels/src/lib.rs:141-142);
 * scale [1,N] per output column; y = act(scale[n]*sum_k a[m,k]*q[k,n] + bias[n]).
 * Large shapes run on int8 tensor cores: each activation row is split into `int8_limbs` int8
 * digits of its own row maximum (1 = plain W8A8 quantisation, 2 = default, 3 = f32-grade), the
 * digit products are exact int32 sums, recombined in the epilogue. */
int fa_matmul_int8(fa_ctx *ctx, const fa_tensor *a, fa_bytes *wq, const fa_tensor *scale, int N, int K,
                   const fa_tensor *bias, int act, fa_tensor **out);
/* Optional member matmulInt8Operand (no counterpart in compute.d.ts; the reference dequantises an int8 artifact to
 * f32 / f16 on the host when it loads it, src/engines/asr-parakeet/raw-encoder.js:55-76,92-95):
 * y = act(scale[n] * sum_k a[m,k] * q[k,n] + bias[n]) + add[m,n], wq and scale as for matmulInt8.  The int8 weights
 * STAY int8 in device memory (tile-contiguous, one byte per weight) and are widened to f16 inside the tensor-core
 * kernel, the per-column scale multiplies the f32 accumulator; the activations are rounded to f16 as on matmul's
 * f16-B route (tolerance 2e-2 in the reference's gate), so the producers that hand over packed f16 operands feed it
 * directly.  operand_only != 0: the caller states the result is only read as a packed f16 operand (see
 * fa_matmul_operand).  Shapes outside the tensor-core route (few rows, tiny products) go through fa_matmul_int8. */
int fa_matmul_int8_operand(fa_ctx *ctx, const fa_tensor *a, fa_bytes *wq, const fa_tensor *scale, int N, int K,
                           const fa_tensor *bias, int act, const fa_tensor *add, int operand_only, fa_tensor **out);
/* matmulNBits :166 (ONNX MatMulNBits, bits=4).  bq [N][nblk][16] bytes, low nibble = even k;
 * scales f32 [N*nblk]; zp packed nibbles [N][ceil(nblk/2)] (lib.rs:164-203).  block_size must be 32. */
int fa_matmul_nbits(fa_ctx *ctx, const fa_tensor *a, fa_bytes *bq, const fa_tensor *scales, fa_bytes *zp, int N,
                    int block_size, fa_tensor **out);
/* Integer mode of the int8 tensor-core kernel, exposed so its accumulators can be checked bit
 * for bit: aq int8 [M,K] row-major (host), wq as above; acc_out int32 [M,N] (host). */
int fa_int8_gemm_i32(fa_ctx *ctx, const int8_t *aq_host, int M, fa_bytes *wq, int N, int K, int32_t *acc_out_host);

/* Allocation-free variant of fa_matmul_int8 on raw device pointers.  It has no counterpart in the
 * reference; it exists for hosts that may not allocate device memory at call time (a process whose own
 * pool already owns the rest of the GPU, a real-time audio thread that must not wait on the driver's
 * allocator).  All scratch (packed weights, activation digit planes, row scales) lives in a fixed array
 * inside the library image, about 11 MiB held by every GPU that loads the library.
 * a_dev f32 [M,K], wq_kn_dev int8 bytes in k*N+n order, scale_dev f32 [N], bias_dev f32 [N] or NULL,
 * y_dev f32 [M,N]; all device pointers, work is enqueued on the context's stream.
 * Limits: M <= 512, 64 <= K <= 2048, N >= 64, ceil(N/128)*ceil(K/128)*16384 <= 8 MiB; otherwise
 * FA_ERR_INVALID.  The first call on a device resolves the array's device address: make that call
 * before any stream capture.  Calls share the array and must not overlap on the GPU (same stream). */
int fa_matmul_int8_static(fa_ctx *ctx, const float *a_dev, const void *wq_kn_dev, const float *scale_dev,
                          const float *bias_dev, int act, float *y_dev, int M, int N, int K);

/* ---- glue ops the encoder/decoder forwards call between GEMMs --------------- */
int fa_layernorm(fa_ctx *ctx, const fa_tensor *x, const fa_tensor *gamma, const fa_tensor *beta, float eps,
                 fa_tensor **out);                                                        /* layernorm :167 */
/* Optional member layernormOperand: same arithmetic; the caller states that the result is only read as the row
 * operand of matmul.  Above the f16_hilo_rows limit the result is then kept as the packed f16 operand alone and
 * its f32 storage is filled from that (values rounded to f16) only if something else reads the tensor. */
int fa_layernorm_operand(fa_ctx *ctx, const fa_tensor *x, const fa_tensor *gamma, const fa_tensor *beta, float eps,
                         fa_tensor **out);
/* Optional member layernormChain: y = layernorm(x, g1, b1) and z = layernormOperand(y, g2, b2) in one pass over the
 * rows (the last layernorm of a conformer block and the first of the next); same values as the two calls. */
int fa_layernorm_chain(fa_ctx *ctx, const fa_tensor *x, const fa_tensor *g1, const fa_tensor *b1, const fa_tensor *g2,
                       const fa_tensor *b2, float eps, fa_tensor **out_y, fa_tensor **out_z);
int fa_softmax(fa_ctx *ctx, const fa_tensor *x, fa_tensor **out);                         /* softmax :168 */
/* conv1d :172 — grouped/depthwise direct form (lib.rs:99-138); w = Cout*(Cin/groups)*K. */
int fa_conv1d(fa_ctx *ctx, const fa_tensor *x, const fa_tensor *w, const fa_tensor *bias, int cout, int k, int stride,
              int pad_left, int pad_right, int dilation, int groups, int act, fa_tensor **out);
/* The per-window loop around conv1d in the conformer conv module (sliceCols -> conv1d -> setCols per
 * window, src/engines/asr-parakeet/raw-encoder.js:343-351) as one call: the columns of x are `windows`
 * independent windows of equal length; stride 1 and same-length output only.  Optional fast path; the
 * per-window op sequence gives the same result. */
int fa_conv1d_windows(fa_ctx *ctx, const fa_tensor *x, const fa_tensor *w, const fa_tensor *bias, int cout, int k,
                      int pad_left, int pad_right, int dilation, int groups, int act, int windows, fa_tensor **out);
/* The conv module's middle (transpose -> glu -> per-window depthwise conv1d + act -> transpose,
 * raw-encoder.js:340-362) as one call in time-major layout: x [W*T, 2D] -> [W*T, D]; w = D*k depthwise
 * taps, same-length output (pad_left + pad_right == k-1, k <= 16).  Optional fast path. */
int fa_glu_dwconv_tm(fa_ctx *ctx, const fa_tensor *x, const fa_tensor *w, const fa_tensor *bias, int k, int pad_left,
                     int pad_right, int act, int windows, fa_tensor **out);
/* conv2d :179 (batch 1). x [Cin, H*W] -> [Cout, Ho*Wo]. */
int fa_conv2d(fa_ctx *ctx, const fa_tensor *x, const fa_tensor *w, const fa_tensor *bias, int cout, int cin, int h,
              int w_, int kh, int kw, int stride_h, int stride_w, int pad_top, int pad_bottom, int pad_left,
              int pad_right, int groups, int act, fa_tensor **out);
int fa_bmm_qk(fa_ctx *ctx, const fa_tensor *q, const fa_tensor *b, const fa_tensor *qb, int H, int HD, int W,
              int b_shared, fa_tensor **out);                                             /* bmmQK :191 */
int fa_bmm_pv(fa_ctx *ctx, const fa_tensor *p, const fa_tensor *v, int H, int HD, int W, fa_tensor **out); /* bmmPV :193 */
/* attnFused :247-248 (optional member; may yield no tensor, the caller then uses the separate ops):
 * rel-pos self-attention for W windows of T = q.rows/W frames; pos [2T-1, H*HD] is the projected
 * positional table, pbu/pbv [1, H*HD].  *out == NULL with status 0 means "not this shape". */
int fa_attn_fused(fa_ctx *ctx, const fa_tensor *q, const fa_tensor *k, const fa_tensor *v, const fa_tensor *pos,
                  const fa_tensor *pbu, const fa_tensor *pbv, int H, int HD, int W, fa_tensor **out);
/* Optional member attnFusedQKV: attnFused over the columns of one fused projection qkv [W*T, 3*H*HD] (q | k | v
 * side by side, the three weight matrices concatenated at load time so that the projections are one product).
 * *out is NULL (and the call succeeds) when the shape is outside the one-kernel form (HD == 128, 16 <= T <= 192). */
int fa_attn_fused_qkv(fa_ctx *ctx, const fa_tensor *qkv, const fa_tensor *pos, const fa_tensor *pbu, const fa_tensor *pbv,
                      int H, int HD, int W, fa_tensor **out);
int fa_rel_shift_b(fa_ctx *ctx, const fa_tensor *x, int H, fa_tensor **out);              /* relShift/relShiftB :195-197 */
int fa_ewise(fa_ctx *ctx, const fa_tensor *a, const fa_tensor *b, int op_mul, fa_tensor **out); /* ewise/add/mul :202-204 */
int fa_scale(fa_ctx *ctx, const fa_tensor *x, float s, fa_tensor **out);                  /* scale :205 */
int fa_unary(fa_ctx *ctx, const fa_tensor *x, int act, fa_tensor **out);                  /* silu :206, relu :207 */
int fa_glu(fa_ctx *ctx, const fa_tensor *x, fa_tensor **out);                             /* glu :212 */
int fa_transpose(fa_ctx *ctx, const fa_tensor *x, fa_tensor **out);                       /* transpose :215 */
int fa_slice_cols(fa_ctx *ctx, const fa_tensor *x, int col0, int width, fa_tensor **out); /* sliceCols :216 */
int fa_set_cols(fa_ctx *ctx, fa_tensor *dst, const fa_tensor *src, int col0);             /* setCols :218 */
int fa_slice_rows(fa_ctx *ctx, const fa_tensor *x, int row0, int count, fa_tensor **out); /* sliceRows :219 */
int fa_copy_rows(fa_ctx *ctx, fa_tensor *dst, const fa_tensor *src, int row_offset);      /* copyRows :221 */
int fa_concat_rows(fa_ctx *ctx, const fa_tensor *const *tensors, int count, fa_tensor **out); /* concatRows :222 */
int fa_sub_reshape(fa_ctx *ctx, const fa_tensor *x, int C, int Tsub, int F, fa_tensor **out); /* subReshape :228 */
/* Window-batched forms of conv2d and subReshape (optional members conv2dWindows / subReshapeWindows): x is
 * [windows, cin*h*w], one image per row; conv2d_windows returns [windows, cout*Ho*Wo], sub_reshape_windows
 * returns [windows*Tsub, C*F] (window b in rows [b*Tsub, (b+1)*Tsub)).  Same arithmetic per window as the
 * single-image members; one launch for all windows instead of the reference's per-window preEncode loop
 * (src/engines/asr-parakeet/raw-encoder.js:177-222, 246-252). */
int fa_conv2d_windows(fa_ctx *ctx, const fa_tensor *x, const fa_tensor *w, const fa_tensor *bias, int cout, int cin, int h,
                      int w_, int kh, int kw, int stride_h, int stride_w, int pad_top, int pad_bottom, int pad_left,
                      int pad_right, int groups, int act, int windows, fa_tensor **out);
int fa_sub_reshape_windows(fa_ctx *ctx, const fa_tensor *x, int C, int Tsub, int F, int windows, fa_tensor **out);
/* Optional member convStemWindows: the first three layers of the subsampling stem (raw-encoder.js:177-222) as one
 * call: conv(1->C, 3x3, stride 2, pad 1, relu) -> depthwise(3x3, stride 2, pad 1) -> pointwise(C->C, relu) over
 * x [windows, h*w]; returns [windows, C*H2*W2] with H2 = ceil(ceil(h/2)/2), W2 = w/4, bit-identical to the three
 * conv2d_windows calls.  Biases may be NULL.  *out is NULL (and the call succeeds) when the geometry is outside
 * the fused kernel's range (w == 128, C a multiple of 64): run the three members instead. */
int fa_conv_stem_windows(fa_ctx *ctx, const fa_tensor *x, const fa_tensor *w0, const fa_tensor *b0, const fa_tensor *w1,
                         const fa_tensor *b1, const fa_tensor *w2, const fa_tensor *b2, int C, int h, int w_, int windows,
                         fa_tensor **out);
/* Optional member convDwPwWindows: the stem's fourth and fifth layers as one call: depthwise(3x3, stride 2, pad 1)
 * -> pointwise(C->C, relu) over x [windows, C*h*w]; returns [windows, C*H2*W2], bit-identical to the two
 * conv2d_windows calls; *out is NULL outside the fused kernel's range (w == 32, C a multiple of 64). */
int fa_conv_dw_pw_windows(fa_ctx *ctx, const fa_tensor *x, const fa_tensor *w1, const fa_tensor *b1, const fa_tensor *w2,
                          const fa_tensor *b2, int C, int h, int w_, int windows, fa_tensor **out);
/* argmax over each row (host picks tokens from it; the reference does this on the host,
 * src/engines/asr-whisper/index.ts:80-97): out [rows,2] = {index, value}.  Only the first `ncols`
 * columns of each row take part (ncols <= 0: all of them) - the tied vocabulary projection is padded
 * with zero columns that must never win (raw-whisper-decoder.js:62-66). */
int fa_argmax_rows(fa_ctx *ctx, const fa_tensor *x, int ncols, fa_tensor **out);
/* N-sharded products (one process per GPU, each holding a block of output columns): `gathered`
 * [world*M, Ns] is what an all-gather of the ranks' [M, Ns] results leaves; out [M, world*Ns] is the
 * row-major product, out[m, r*Ns + j] = gathered[r*M + m, j].  Ns must be a multiple of 4.  The
 * reference has no multi-device path (one GPUDevice, src/gpu/device.js). */
int fa_unshard_cols(fa_ctx *ctx, const fa_tensor *gathered, int world, fa_tensor **out);
/* The same exchange fused into the product (one process per GPU, buffers shared through CUDA IPC): fa_ipc_export
 * gives a 64-byte handle of a tensor's storage, fa_ipc_open maps a peer's handle into this process (a device
 * pointer usable by kernels of this GPU over NVLink), fa_ipc_close unmaps it.  fa_matmul_scatter computes this
 * rank's block of output columns, act(A @ B_shard + bias_shard), and its epilogue stores every finished tile at
 * columns [col0, col0 + Ns) of ALL `n_outs` result buffers ([M][ldc] f32 each: outs[0] this GPU's own, the rest
 * peers'), so no separate all-gather or re-layout pass runs.  The caller must order the ranks (a stream-ordered
 * barrier) between this call and any read of a result, and again before the buffers are overwritten. */
int fa_ipc_export(fa_ctx *ctx, const fa_tensor *t, unsigned char handle_out[64]);
int fa_ipc_open(fa_ctx *ctx, const unsigned char handle[64], void **dev_ptr_out);
int fa_ipc_close(fa_ctx *ctx, void *dev_ptr);
int fa_matmul_scatter(fa_ctx *ctx, const fa_tensor *a, fa_tensor *b_shard, const fa_tensor *bias_shard, int act,
                      void *const *outs, int n_outs, int ldc, int col0);
/* Token embedding + position on the device (the reference gathers on the host and uploads,
 * src/engines/asr-whisper/raw-whisper-decoder.js:106-108): out[s,:] = table[id_s,:] + pos[n,:], where id_s
 * is column 0 of row s of idx (token ids as floats: an fa_argmax_rows result or a [S,1] tensor).  With it
 * a greedy decode never leaves the device between tokens.  An id outside the table reads row 0 and makes
 * the next fa_sync fail with FA_ERR_INVALID. */
int fa_embed_rows(fa_ctx *ctx, const fa_tensor *table, const fa_tensor *pos, const fa_tensor *idx, int n,
                  fa_tensor **out);

/* ---- callers either side of the path ------------------------------------------ */
/* Optional member logMelWindows.  The reference computes log-mel features on the host, one window per worker
 * thread: ParakeetMel.process (src/engines/asr-parakeet/parakeet-mel.js:16-21) = JsPreprocessor.computeRawMel +
 * normalizeFeatures (src/engines/asr-nemotron/nemotron-mel.js:451-573, 586-620).  Here: audio [W, N] f32, W windows
 * of N samples at 16 kHz -> [W, T * n_mels], window b in row b, TIME-major (frame t at columns [t*n_mels,
 * (t+1)*n_mels)), which is the image the encoder's subsampling front end reads.  Pipeline and arithmetic types as in
 * the reference: pre-emphasis 0.97, 512-point frames every 160 samples under a Hann(400) window, FFT in doubles,
 * power as f32, slaney filterbank, log(mel + log_guard).  normalize = 1: per-feature mean / variance normalisation
 * over T = floor(N/160) frames (Parakeet, log_guard 2^-24); normalize = 0: raw log-mel over T = N/160 + 1 frames
 * (Nemotron, log_guard 1e-10). */
int fa_log_mel_windows(fa_ctx *ctx, const fa_tensor *audio, int n_mels, double log_guard, int normalize, fa_tensor **out);

/* Batched greedy TDT decoding: the prediction network + joint of rust/parakeet-decoder/src/lib.rs (set_weights :99-110,
 * set_out_q :93-96, decode_proj :288-319; JS host src/engines/asr-parakeet/raw-decoder-wasm.js:12-70; the reference's
 * own GPU form is src/engines/asr-parakeet/gpu-decoder.js) for W independent windows in lock-step.
 * fa_tdt_create takes HOST pointers in the reference manifest's shapes: embed [8193,640], lNw / lNr [2560,640]
 * (ONNX iofc gate order), lNb [5120], pred_w [640,640], pred_b [640], out_b [8198], and the joint's out matrix either
 * as int8 rows + per-row scales (out_q [640,8198], out_scale [640]; the reference's default, quantised by its loader)
 * or as f32 out_w [640,8198] (pass NULL for the form not used).
 * fa_tdt_decode_proj: proj [W*T, 640] = pre-projected encoder frames (projection bias included), window w in rows
 * [w*T, (w+1)*T).  Writes, per window, counts[w] token ids and their emission frames into ids / frames at offset
 * w*cap (cap >= 10*T holds the worst case, as the reference sizes its buffers); rounds_out (may be NULL) receives the
 * number of lock-step rounds run.  Blocks until the results are on the host. */
typedef struct fa_tdt fa_tdt;
int fa_tdt_create(fa_ctx *ctx, const float *embed, const float *l0w, const float *l0r, const float *l0b, const float *l1w,
                  const float *l1r, const float *l1b, const float *pred_w, const float *pred_b, const float *out_w,
                  const float *out_b, const int8_t *out_q, const float *out_scale, fa_tdt **out);
int fa_tdt_decode_proj(fa_ctx *ctx, fa_tdt *dec, const fa_tensor *proj, int W, int T, int cap, int32_t *ids_host,
                       int32_t *frames_host, int32_t *counts_host, int *rounds_out);
int fa_tdt_free(fa_ctx *ctx, fa_tdt *dec);

/* ---- profiling (compute.d.ts:250-251; scheduler.js:139-180) ----------------- */
typedef struct fa_profile_entry {
  char label[48];     /* kernel label (the reference keys by pipeline label) */
  float ms;           /* summed device time of its launches, CUDA events on the context stream */
  int count;          /* launches */
} fa_profile_entry;
int fa_profile_start(fa_ctx *ctx, int max_ops); /* startProfile */
int fa_profile_end(fa_ctx *ctx, fa_profile_entry *out, int capacity, int *n_out); /* endProfile */

#if defined(__GNUC__)
#pragma GCC visibility pop
#endif
#ifdef __cplusplus
}
#endif
#endif /* FA_CUDA_H */
