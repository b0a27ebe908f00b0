// Batched greedy TDT decoding (prediction network + joint) for many encoder windows at once.
//
// The reference decodes one window at a time on a CPU core, in Rust compiled to wasm
// (rust/parakeet-decoder/src/lib.rs: predict :150-156, compute_predproj :159-175, joint_tail :179-227,
// decode_proj :288-319), and names that stage as the cost right after the encoder
// (src/engines/asr-parakeet/pipeline.js:38-40).  Its own GPU form runs the whole loop of a window in one workgroup
// (src/engines/asr-parakeet/gpu-decoder.js).  Windows are independent, so here they advance in LOCK-STEP, one joint
// evaluation per window per round, and every product of a round is a matrix product over all windows:
//
//   joint in   J[w]   = relu(proj[w, t_w] + predproj[w]) * out_scale      (gather at each window's own frame t_w),
//                                              written directly as the int8 product's digit planes and row scales
//   logits     OUT    = J @ out_q + out_b      int8 out-matrix [640][8198], three int8 digits per activation row on
//                                              kind::i8 (exact integer sums, f32-grade result)
//   pick       argmax over the 8193 tokens and the 5 durations; emit / commit the candidate state / advance t_w
//   predict    G0 = [embed[tok] | H0] @ [W0;R0]^T + b  -> cell -> (NH0, NC0);  G1 = [NH0 | H1] @ [W1;R1]^T + b -> cell
//              (embed[tok] @ W0^T + b is a table over the vocabulary made at creation: layer 0 sums over H0 only)
//   predproj   = NH1 @ pred_w + pred_b         f32 weights, exact f32 multiply-adds (k_tdt_rows: one launch per LSTM
//                                              layer with the cell in its epilogue, one for the projection)
//
// Six launches per round, each scheduled under its predecessor's tail (programmatic dependent launch).
// The prediction network is evaluated for every window in every round: for a window that did not emit, its inputs
// (committed state, last token) are unchanged, so the result is the same as the cached one the reference keeps.
// A round is recorded once and replayed; the host looks at a device counter of finished windows every few rounds.
// Gate nonlinearities are the crate's own exp / tanh approximations (lib.rs:49-68), evaluated with separate
// multiplies and adds, so that the only difference from the reference is the summation order inside the products.
#include "fa_internal.cuh"
#include "fa_tc_common.cuh"

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

// State vectors of the prediction network live in "chunk-transposed" form: windows in chunks of 32, element n of
// window w at ((w / 32) * HID + n) * 32 + w % 32, so that the 32 windows' values of one n are one 128-byte line (what
// k_tdt_rows streams).  Rows past W in the last chunk stay zero.
__device__ __forceinline__ size_t t_idx(int w, int n) { return ((size_t)(w >> 5) * HID + n) * 32 + (w & 31); }

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

// The same joint input, written directly as the int8 product's row operand: per window the row scale max|J|/127 and
// `limbs` int8 digit planes Ap[limb][k/128][w][k%128], with fa_prep_a_i8's arithmetic digit for digit (that kernel
// documents the split), so that the lock-step round needs no separate pass over J.
__global__ void __launch_bounds__(256) k_tdt_joint_digits(const float *__restrict__ proj, const int *__restrict__ t, int T,
                                                          const float *__restrict__ predproj, const float *__restrict__ scale,
                                                          int W, int limbs, int8_t *__restrict__ out, float *__restrict__ rowscale) {
  static_assert(HID % 128 == 0 && HID <= 3 * 256, "three values per thread, whole 128-wide K chunks");
  __shared__ float red[8];
  fa_grid_dep_sync();
  const int w = blockIdx.x, tw = t[w];
  float v[3];
  float mx = 0.0f;
#pragma unroll
  for (int i = 0; i < 3; i++) {
    const int n = threadIdx.x + i * 256;
    float x = 0.0f;
    if (n < HID && tw < T) {
      x = __fadd_rn(proj[((size_t)w * T + tw) * HID + n], predproj[(size_t)w * HID + n]);
      x = x > 0.0f ? x : 0.0f;
      if (scale) x = __fmul_rn(x, scale[n]);
    }
    v[i] = x;
    mx = fmaxf(mx, fabsf(x));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = mx;
  __syncthreads();
  mx = red[0];
#pragma unroll
  for (int k = 1; k < 8; k++) mx = fmaxf(mx, red[k]);
  const float s = mx > 0.0f ? mx / 127.0f : 1.0f;
  if (threadIdx.x == 0) rowscale[w] = s;
  const size_t plane = (size_t)(HID / 128) * W * 128;
#pragma unroll
  for (int i = 0; i < 3; i++) {
    const int k = threadIdx.x + i * 256;
    if (k >= HID) break;
    const size_t o = ((size_t)(k >> 7) * W + w) * 128 + (k & 127);
    const float r = v[i] / s;
    const float q1 = fminf(fmaxf(rintf(r), -127.0f), 127.0f);
    out[o] = (int8_t)q1;
    if (limbs > 1) {
      const float r1 = (r - q1) * 128.0f;
      const float q2 = rintf(r1);
      out[plane + o] = (int8_t)q2;
      if (limbs > 2) out[2 * plane + o] = (int8_t)rintf((r1 - q2) * 128.0f);
    }
  }
}

// One block per window: first-maximum over tokens and durations (the reference scans upwards with a strict >),
// then the TDT bookkeeping of decode_proj (lib.rs:300-316) and, on an emission, the commit of the candidate state.
// Every global read whose address does not depend on the picked token is issued before the first comparison (a
// thread's eight logits, the durations, the bookkeeping words, the candidate state), so that the block pays one
// memory latency for them, not one per loop trip.
constexpr int kPickThreads = 1024;
__global__ void __launch_bounds__(kPickThreads) k_tdt_pick(const float *__restrict__ logits, int ld, int T, int cap, int *__restrict__ t,
                                                           int *__restrict__ emitted, int *__restrict__ last_tok, int *__restrict__ counts,
                                                           int *__restrict__ ids, int *__restrict__ frames,
                                                           float *__restrict__ h0t, const float *__restrict__ nh0t,
                                                           float *__restrict__ h1t, const float *__restrict__ nh1t, float *__restrict__ c0,
                                                           float *__restrict__ c1, const float *__restrict__ nc0, const float *__restrict__ nc1,
                                                           int *__restrict__ done_count) {
  static_assert(VOCAB == 8 * kPickThreads + 1 && HID <= kPickThreads, "eight logits per thread and one more for thread 0");
  __shared__ float sv[32];
  __shared__ int si[32];
  __shared__ int s_tok;
  fa_grid_dep_sync();
  const int w = blockIdx.x, tid = threadIdx.x, tw = t[w];
  if (tw >= T) return;  // this window finished in an earlier round (block-uniform)
  const float *row = logits + (size_t)w * ld;
  float v[8];
#pragma unroll
  for (int j = 0; j < 8; j++) v[j] = row[tid + j * kPickThreads];
  float last = -INFINITY, dur[LOGITS - VOCAB];
  int em = 0, n_out = 0;
  if (tid == 0) {
    last = row[VOCAB - 1];
#pragma unroll
    for (int i = 0; i < LOGITS - VOCAB; i++) dur[i] = row[VOCAB + i];
    em = emitted[w];
    n_out = counts[w];
  }
  float p_h0 = 0.0f, p_h1 = 0.0f, p_c0 = 0.0f, p_c1 = 0.0f;
  if (tid < HID) {
    p_h0 = nh0t[t_idx(w, tid)], p_h1 = nh1t[t_idx(w, tid)];
    p_c0 = nc0[(size_t)w * HID + tid], p_c1 = nc1[(size_t)w * HID + tid];
  }
  float bv = -INFINITY;
  int bi = 0x7fffffff;
#pragma unroll
  for (int j = 0; j < 8; j++)
    if (v[j] > bv) { bv = v[j]; bi = tid + j * kPickThreads; }  // ascending index per thread: keeps the first maximum
  if (tid == 0 && last > bv) { bv = last; bi = VOCAB - 1; }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
  }
  if ((tid & 31) == 0) { sv[tid >> 5] = bv; si[tid >> 5] = bi; }
  __syncthreads();
  if (tid < 32) {
    bv = sv[tid], bi = si[tid];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
  }
  if (tid == 0) {
    const int tok = bi == 0x7fffffff ? 0 : bi;  // every logit NaN or -inf: the reference's scan leaves index 0
    int step = 0;
    float dv = -INFINITY;
#pragma unroll
    for (int i = 0; i < LOGITS - VOCAB; i++)
      if (dur[i] > dv) { dv = dur[i]; step = i; }
    int tn = tw;
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
  if (s_tok != BLANK && tid < HID) {  // commit_state: H = NH, C = NC (layer 0 finds the new token through last_tok)
    const size_t i = t_idx(w, tid);
    h0t[i] = p_h0;
    h1t[i] = p_h1;
    c0[(size_t)w * HID + tid] = p_c0;
    c1[(size_t)w * HID + tid] = p_c1;
  }
}

// ---- k_tdt_rows: the prediction network's products, exact f32 ------------------------------------------------
//
// out[w][n] = sum_k x[w][k] * Wt[k][n] (+ bias) for up to a few hundred windows and f32 weights, K = 1280 (LSTM layer 1:
// [input | committed hidden state] against [W;R]^T, followed in the same kernel by the cell) or K = 640 (layer 0,
// whose input half is a table row per token, and the prediction projection).  With 32 rows a tensor-core tile is
// mostly padding and the f32 weights would need the three-product tf32 scheme; plain FFMA does the 105 MFLOP of a
// layer in a few microseconds and is exact f32.
//
// One block owns 20 output columns (for an LSTM layer: the 4 gates of 5 hidden units, so that the cell can follow
// without a grid-wide step) and one chunk of 32 windows.  Its 16 warps split K; a warp streams its slice of the
// activations (chunk-transposed: 128 bytes per k) and of the block's weights (packed [block][k][20] at upload: 80
// bytes per k) through a private ring of shared-memory stages filled by bulk copies (cp.async.bulk, one elected
// lane, one mbarrier per stage), so that no thread waits on a global load.  A lane holds an 8-row x 10-column
// accumulator tile for every fourth k of the slice (see the loop); the four k-quarters of a warp meet by shuffles
// and the 16 warps in shared memory, both in a fixed order.
constexpr int kRowsWarps = 16, kRowsThreads = kRowsWarps * 32, kRowsCols = 20, kRowsKS = 8, kRowsNS = 3, kRowsAhead = 2;
constexpr int kRowsStageBytes = kRowsKS * (128 + kRowsCols * 4);                       // 1664
constexpr int kRowsRingBytes = kRowsWarps * kRowsNS * kRowsStageBytes;                 // 79872
constexpr int kRowsRedBytes = kRowsWarps * 32 * kRowsCols * 4;                         // 40960
constexpr int kRowsZBytes = (32 + 1) * kRowsCols * 4;  // the block's sums, then one row for the projection's bias
constexpr int kRowsSmem = kRowsRingBytes + kRowsRedBytes + kRowsZBytes + kRowsWarps * kRowsNS * 8;

struct RowsParams {
  const float *xa, *xb;  // activations for k < 640 and k >= 640, chunk-transposed
  const float *wt;       // [blocks][K][20]: per k the columns (g, u < 4) as g*4+u, then (g, u = 4) as 16+g
  const float *bias;     // LSTM: [4*HID] in gate order i, o, f, c; projection: [HID]
  const float *tab;      // MODE 2: [VOCAB][4*HID], W0 . embed[token] + bias in gate order
  const int *last_tok;   // MODE 2: [W]
  const float *c;        // LSTM: committed cell state [W][HID]
  float *nc, *nht;       // LSTM: candidate cell state [W][HID] and hidden state (chunk-transposed)
  float *out;            // projection: [W][HID]
  int W;
  int *status;
  uint32_t wait_limit;
  int withhold;          // >= 0: warp 0 of block 0 never loads this stage (test hook for the bounded wait)
};

__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src),
               "r"(bytes), "r"(bar)
               : "memory");
}

// Packed pair of f32 multiply-adds (sm_100): d.lo = a.lo * b.lo + c.lo, d.hi = a.hi * b.hi + c.hi, each fused and
// rounded to nearest like fmaf.
__device__ __forceinline__ uint64_t ffma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t dup_f32x2(float x) {
  uint64_t d;
  asm("mov.b64 %0, {%1, %1};" : "=l"(d) : "f"(x));
  return d;
}
__device__ __forceinline__ void unpack_f32x2(uint64_t v, float &lo, float &hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}

// MODE 0: the projection (K = 640, bias, row-major result).  MODE 1: an LSTM layer over [input | hidden] (K = 1280).
// MODE 2: an LSTM layer whose input is an embedding row: K = 640 over the hidden state only, the input half of the
// gates (and the bias) comes from a table indexed by each window's last token.
template <int MODE>
__global__ void __launch_bounds__(kRowsThreads, 1) k_tdt_rows(const RowsParams p) {
  constexpr bool LSTM = MODE != 0;
  constexpr int K = MODE == 1 ? 2 * HID : HID, KPER = K / kRowsWarps, NLOAD = KPER / kRowsKS;
  static_assert(KPER % kRowsKS == 0 && HID % KPER == 0, "a warp's K slice is whole stages inside one operand");
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t *ring = smem;
  float *red = reinterpret_cast<float *>(smem + kRowsRingBytes);
  float *z = reinterpret_cast<float *>(smem + kRowsRingBytes + kRowsRedBytes);
  const uint32_t bars = tc::smem_u32(smem + kRowsRingBytes + kRowsRedBytes + kRowsZBytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, blk = blockIdx.x, chunk = blockIdx.y;
  const int ch = lane & 1, rq = (lane >> 1) & 3, kq = lane >> 3;  // gate pair, row octet, k quarter
  const int k0 = warp * KPER;
  const float *xsrc = (k0 < HID ? p.xa + ((size_t)chunk * HID + k0) * 32 : p.xb + ((size_t)chunk * HID + (k0 - HID)) * 32);
  const float *wsrc = p.wt + ((size_t)blk * K + k0) * kRowsCols;
  uint8_t *my = ring + (size_t)warp * kRowsNS * kRowsStageBytes;
  const uint32_t my_u = tc::smem_u32(my), my_bar = bars + warp * kRowsNS * 8;
  const int wh = (blk == 0 && chunk == 0 && warp == 0) ? p.withhold : -1;

  // one lane; what = 1: weights, 2: activations, 3: both.  The barrier expects the whole stage with the weights.
  auto load_stage = [&](int it, int what) {
    const int s = it % kRowsNS;
    const uint32_t bar = my_bar + s * 8, dst = my_u + s * kRowsStageBytes;
    if (what & 1) tc::mbar_expect_tx(bar, kRowsStageBytes);
    if (it == wh) return;
    if (what & 1) bulk_g2s(dst + kRowsKS * 128, wsrc + (size_t)it * kRowsKS * kRowsCols, kRowsKS * kRowsCols * 4, bar);
    if (what & 2) bulk_g2s(dst, xsrc + (size_t)it * kRowsKS * 32, kRowsKS * 128, bar);
  };
  constexpr int kFirst = NLOAD < kRowsAhead ? NLOAD : kRowsAhead;
  if (lane == 0) {
    for (int s = 0; s < kRowsNS; s++) tc::mbar_init(my_bar + s * 8, 1);
    tc::fence_barrier_init();
    tc::fence_proxy_async_smem();
    for (int it = 0; it < kFirst; it++) load_stage(it, 1);  // the weights do not depend on the launch before
  }
  fa_grid_dep_sync();  // the activations do
  if (lane == 0)
    for (int it = 0; it < kFirst; it++) load_stage(it, 2);
  __syncwarp();

  // what the epilogue needs from global memory, fetched under the K loop
  float e_c = 0.0f, e_b[4] = {0.0f, 0.0f, 0.0f, 0.0f};
  if (LSTM) {
    if (threadIdx.x < 32 * 5) {
      const int unit = blk * 5 + (threadIdx.x >> 5), w = chunk * 32 + (threadIdx.x & 31);
      if (w < p.W) e_c = p.c[(size_t)w * HID + unit];
      if (MODE == 2) {
        if (w < p.W) {
          const float *row = p.tab + (size_t)p.last_tok[w] * 4 * HID;
#pragma unroll
          for (int q = 0; q < 4; q++) e_b[q] = row[q * HID + unit];
        }
      } else {
#pragma unroll
        for (int q = 0; q < 4; q++) e_b[q] = p.bias[q * HID + unit];
      }
    }
  } else if (threadIdx.x < kRowsCols) {
    e_b[0] = p.bias[blk * kRowsCols + threadIdx.x];
  }
  // A lane's accumulators: 8 rows x 10 columns (two gates x 5 units) over every fourth k of the warp's slice.
  // Shared memory hands a warp 128 bytes per clock whether or not lanes share an address, so the operand bytes per
  // FFMA decide the pace: this tile reads 18 values for 80 multiply-adds (4.5 clocks of shared-memory time per k and
  // warp, under the 5 clocks the FFMA pipe needs), where a 4 x 5 tile on every k read 9 for 20 (9 clocks).
  // The multiply-adds are packed pairs (fma.rn.f32x2) over two adjacent columns: the weight pairs are the 64-bit
  // halves of the loads as they come, an activation is duplicated into both halves by one move; half the issue
  // slots for the same arithmetic, each lane of a pair rounded exactly like a scalar FFMA.
  // Column pairs: (A0,A1) (A2,A3) (B0,B1) (B2,B3) (A4,B4) for the lane's two gates A, B and units 0..4.
  uint64_t acc2[8][5];
#pragma unroll
  for (int r = 0; r < 8; r++)
#pragma unroll
    for (int c = 0; c < 5; c++) acc2[r][c] = 0ull;
  bool ok = true;
  int s = 0;
  uint32_t ph = 0;
#pragma unroll 1
  for (int it = 0; it < NLOAD; it++) {
    if (it + kRowsAhead < NLOAD) {  // the stage read in the iteration before this one takes the load two ahead
      __syncwarp();
      if (lane == 0) load_stage(it + kRowsAhead, 3);
    }
    if (!__all_sync(0xffffffffu, tc::mbar_wait(my_bar + s * 8, ph, p.wait_limit))) {
      ok = false;
      break;
    }
    const float4 *xs = reinterpret_cast<const float4 *>(my + s * kRowsStageBytes) + rq * 2;
    const float *ws = reinterpret_cast<const float *>(my + s * kRowsStageBytes + kRowsKS * 128);
#pragma unroll
    for (int j = 0; j < kRowsKS / 4; j++) {
      const int kk = kq + 4 * j;
      const float4 xa = xs[kk * 8], xb = xs[kk * 8 + 1];
      const ulonglong2 wa = *reinterpret_cast<const ulonglong2 *>(ws + kk * kRowsCols + ch * 8);
      const ulonglong2 wb = *reinterpret_cast<const ulonglong2 *>(ws + kk * kRowsCols + ch * 8 + 4);
      const uint64_t wc = *reinterpret_cast<const uint64_t *>(ws + kk * kRowsCols + 16 + ch * 2);
      const float xr[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
      const uint64_t wp[5] = {wa.x, wa.y, wb.x, wb.y, wc};
#pragma unroll
      for (int r = 0; r < 8; r++) {
        const uint64_t xx = dup_f32x2(xr[r]);
#pragma unroll
        for (int c = 0; c < 5; c++) acc2[r][c] = ffma2(xx, wp[c], acc2[r][c]);
      }
    }
    if (++s == kRowsNS) { s = 0; ph ^= 1u; }
  }
  float acc[8][10];
#pragma unroll
  for (int r = 0; r < 8; r++) {
    unpack_f32x2(acc2[r][0], acc[r][0], acc[r][1]);
    unpack_f32x2(acc2[r][1], acc[r][2], acc[r][3]);
    unpack_f32x2(acc2[r][2], acc[r][5], acc[r][6]);
    unpack_f32x2(acc2[r][3], acc[r][7], acc[r][8]);
    unpack_f32x2(acc2[r][4], acc[r][4], acc[r][9]);
  }
  if (!ok && lane == 0 && atomicCAS(p.status, 0, 7) == 0) {
    p.status[1] = (int)blockIdx.x;
    p.status[2] = warp;
  }
  // The four k-quarters of a warp meet by two exchange steps that halve what a lane holds: lanes 16 apart split the
  // rows (the lower lane keeps rows 0..3 of its eight), lanes 8 apart split the two gates.  A lane ends with 4 rows x
  // 5 units of one gate, summed over the warp's whole K slice.
  const bool b4 = (lane & 16) != 0, b3 = (lane & 8) != 0;
  float a1[4][10];
#pragma unroll
  for (int r = 0; r < 4; r++)
#pragma unroll
    for (int c = 0; c < 10; c++) {
      const float lo = acc[r][c], hi = acc[r + 4][c];
      a1[r][c] = __fadd_rn(b4 ? hi : lo, __shfl_xor_sync(0xffffffffu, b4 ? lo : hi, 16));
    }
  float a2[4][5];
#pragma unroll
  for (int r = 0; r < 4; r++)
#pragma unroll
    for (int u = 0; u < 5; u++) {
      const float lo = a1[r][u], hi = a1[r][u + 5];
      a2[r][u] = __fadd_rn(b3 ? hi : lo, __shfl_xor_sync(0xffffffffu, b3 ? lo : hi, 8));
    }
  // partial sums: red[warp][r*5+u][lane]
#pragma unroll
  for (int r = 0; r < 4; r++)
#pragma unroll
    for (int u = 0; u < 5; u++) red[(warp * 20 + r * 5 + u) * 32 + lane] = a2[r][u];
  __syncthreads();
  for (int i = threadIdx.x; i < 32 * kRowsCols; i += kRowsThreads) {
    float sum = red[i];
#pragma unroll
    for (int w = 1; w < kRowsWarps; w++) sum = __fadd_rn(sum, red[w * 32 * kRowsCols + i]);
    const int j = i >> 5, l = i & 31;  // j = r*5+u; l = lane: bit 0 gate pair, bits 1-2 row octet, bit 3 gate, bit 4 row half
    const int row = ((l >> 1) & 3) * 8 + (l >> 4) * 4 + j / 5, col = ((l & 1) * 2 + ((l >> 3) & 1)) * 5 + j % 5;
    z[row * kRowsCols + col] = sum;
  }
  __syncthreads();
  if (LSTM) {
    if (threadIdx.x < 32 * 5) {
      const int row = threadIdx.x & 31, u = threadIdx.x >> 5, unit = blk * 5 + u, w = chunk * 32 + row;
      if (w < p.W) {
        const float *zr = z + row * kRowsCols;
        const float zi = __fadd_rn(zr[u], e_b[0]), zo = __fadd_rn(zr[5 + u], e_b[1]);
        const float zf = __fadd_rn(zr[10 + u], e_b[2]), zc = __fadd_rn(zr[15 + u], e_b[3]);
        const size_t i = (size_t)w * HID + unit;
        const float cc = __fadd_rn(__fmul_rn(t_sigmoid(zf), e_c), __fmul_rn(t_sigmoid(zi), t_tanhf(zc)));
        p.nc[i] = cc;
        p.nht[t_idx(w, unit)] = __fmul_rn(t_sigmoid(zo), t_tanhf(cc));
      }
    }
  } else {
    if (threadIdx.x < kRowsCols) z[32 * kRowsCols + threadIdx.x] = e_b[0];
    __syncthreads();
    for (int i = threadIdx.x; i < 32 * kRowsCols; i += kRowsThreads) {
      const int row = i / kRowsCols, col = i - row * kRowsCols, w = chunk * 32 + row, n = blk * kRowsCols + col;
      if (w < p.W) p.out[(size_t)w * HID + n] = __fadd_rn(z[i], z[32 * kRowsCols + col]);
    }
  }
}

__global__ void k_fill_int(int *p, int n, int v) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) p[i] = v;
}

}  // namespace

struct fa_tdt {
  fa_tensor *gate_tab = nullptr, *wr[2] = {nullptr, nullptr}, *bsum1 = nullptr, *pred_w = nullptr, *pred_b = nullptr;
  fa_tensor *out_b = nullptr, *out_scale = nullptr, *ones = nullptr, *out_w = nullptr;
  fa_bytes *out_q = nullptr;
};

static void tdt_release(fa_ctx *ctx, fa_tdt *d) {
  fa_tensor *ts[] = {d->gate_tab, d->wr[0], d->wr[1], d->bsum1, d->pred_w, d->pred_b, d->out_b, d->out_scale, d->ones, d->out_w};
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
  // k_tdt_rows' weight packing: block b owns hidden units 5b..5b+4 (their four gates, ONNX order i, o, f, c).
  // Layer 1 runs over K = 1280: rows 0..639 multiply the layer input, rows 640..1279 the committed hidden state.
  // Layer 0's input is an embedding row, so the input half of its gates is a table over the vocabulary, made here
  // once: gate_tab[token] = embed[token] . W0^T + (b[g] + b[4*HID + g]) (lib.rs:139 adds the two biases first), on the
  // CUDA-core f32 kernel; the layer itself then runs over the hidden state only (K = 640).
  auto pos = [](int g, int u) { return u < 4 ? g * 4 + u : 16 + g; };
  const float *lw[2] = {l0w, l1w}, *lr[2] = {l0r, l1r}, *lb[2] = {l0b, l1b};
  std::vector<float> tmp((size_t)2 * HID * 4 * HID), bs(4 * HID);
  int rc = FA_OK;
  for (int l = 0; l < 2 && rc == FA_OK; l++) {
    const int K = l == 0 ? HID : 2 * HID;
    for (int blk = 0; blk < HID / 5; blk++)
      for (int k = 0; k < K; k++) {
        float *dst = &tmp[((size_t)blk * K + k) * kRowsCols];
        for (int g = 0; g < 4; g++)
          for (int u = 0; u < 5; u++) {
            const size_t row = (size_t)g * HID + blk * 5 + u;
            dst[pos(g, u)] = l == 0 ? lr[l][row * HID + k] : (k < HID ? lw[l][row * HID + k] : lr[l][row * HID + (k - HID)]);
          }
      }
    rc = fa_upload_f32(ctx, tmp.data(), (HID / 5) * K, kRowsCols, &d->wr[l]);
  }
  for (int g = 0; g < 4 * HID; g++) bs[g] = lb[1][g] + lb[1][4 * HID + g];
  if (rc == FA_OK) rc = fa_upload_f32(ctx, bs.data(), 1, 4 * HID, &d->bsum1);
  if (rc == FA_OK) {
    fa_tensor *emb = nullptr, *w0t = nullptr, *b0 = nullptr;
    for (int g = 0; g < 4 * HID; g++) {
      bs[g] = lb[0][g] + lb[0][4 * HID + g];
      for (int k = 0; k < HID; k++) tmp[(size_t)k * 4 * HID + g] = l0w[(size_t)g * HID + k];
    }
    rc = fa_upload_f32(ctx, embed, VOCAB, HID, &emb);
    if (rc == FA_OK) rc = fa_upload_f32(ctx, tmp.data(), HID, 4 * HID, &w0t);
    if (rc == FA_OK) rc = fa_upload_f32(ctx, bs.data(), 1, 4 * HID, &b0);
    if (rc == FA_OK) rc = fa_alloc(ctx, VOCAB, 4 * HID, &d->gate_tab);
    if (rc == FA_OK)
      rc = fa_simt_gemm(ctx, (const float *)emb->dptr, w0t->dptr, 0, nullptr, (const float *)b0->dptr, FA_ACT_NONE, nullptr,
                        (float *)d->gate_tab->dptr, VOCAB, 4 * HID, HID);
    const std::string msg = ctx->err;
    fa_tensor *ts[] = {emb, w0t, b0};
    for (fa_tensor *t : ts)
      if (t) fa_free_tensor(ctx, t);
    if (rc != FA_OK) ctx->err = msg;
  }
  if (rc == FA_OK) {  // the projection [k][n]: block b owns columns 20b..20b+19
    for (int blk = 0; blk < HID / kRowsCols; blk++)
      for (int k = 0; k < HID; k++)
        for (int g = 0; g < 4; g++)
          for (int u = 0; u < 5; u++) tmp[((size_t)blk * HID + k) * kRowsCols + pos(g, u)] = pred_w[(size_t)k * HID + blk * kRowsCols + g * 5 + u];
    rc = fa_upload_f32(ctx, tmp.data(), (HID / kRowsCols) * HID, kRowsCols, &d->pred_w);
  }
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
  // chunk-transposed [ceil(W/32)][HID][32]: committed and candidate hidden states
  fa_tensor *h0t = nullptr, *nh0t = nullptr, *h1t = nullptr, *nh1t = nullptr;
  fa_tensor *c0 = nullptr, *c1 = nullptr, *nc0 = nullptr, *nc1 = nullptr, *predproj = nullptr, *J = nullptr;  // [W][HID]
  fa_tensor *logits = nullptr;                   // [W][LOGITS] when the joint's digit planes are written here
  void *planes = nullptr, *rowscale = nullptr;   // the int8 product's row operand (see k_tdt_joint_digits)
  size_t planes_bytes = 0, rowscale_bytes = 0;
  void *ints = nullptr;  // t, emitted, last_tok, counts [W each], done_count, then ids and frames [W*cap each]
  size_t ints_bytes = 0;
};

template <int MODE>
int tdt_rows(fa_ctx *ctx, const RowsParams &p, int blocks, int W, int withhold) {
  static bool attr_set[3] = {false, false, false};
  if (!attr_set[MODE]) {
    FA_CHECK_CUDA(ctx, cudaFuncSetAttribute(k_tdt_rows<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, kRowsSmem));
    attr_set[MODE] = true;
  }
  RowsParams q = p;
  q.W = W;
  q.status = ctx->dev_status;
  q.wait_limit = ctx->wait_limit;
  q.withhold = withhold;
  LaunchScope ls(ctx, MODE ? "tdt_lstm" : "tdt_pred");
  FA_CHECK_CUDA(ctx, fa_launch_dep(ctx, k_tdt_rows<MODE>, dim3(blocks, ceil_div(W, 32)), dim3(kRowsThreads), kRowsSmem, q));
  return FA_OK;
}

// predict + compute_predproj for every window, from the committed state and the last token's embedding
int tdt_predict(fa_ctx *ctx, fa_tdt *d, TdtState &s, int W, const int *last_tok) {
  const int withhold = ctx->tc_withhold_chunk;
  ctx->tc_withhold_chunk = -1;  // one launch only
  RowsParams p{};
  p.xa = (const float *)s.h0t->dptr, p.xb = p.xa, p.wt = (const float *)d->wr[0]->dptr;
  p.tab = (const float *)d->gate_tab->dptr, p.last_tok = last_tok;
  p.c = (const float *)s.c0->dptr, p.nc = (float *)s.nc0->dptr, p.nht = (float *)s.nh0t->dptr;
  FA_TRY(tdt_rows<2>(ctx, p, HID / 5, W, withhold));
  p.xa = (const float *)s.nh0t->dptr, p.xb = (const float *)s.h1t->dptr, p.wt = (const float *)d->wr[1]->dptr;
  p.bias = (const float *)d->bsum1->dptr, p.c = (const float *)s.c1->dptr, p.nc = (float *)s.nc1->dptr, p.nht = (float *)s.nh1t->dptr;
  FA_TRY(tdt_rows<1>(ctx, p, HID / 5, W, -1));
  RowsParams q{};
  q.xa = (const float *)s.nh1t->dptr, q.xb = q.xa, q.wt = (const float *)d->pred_w->dptr, q.bias = (const float *)d->pred_b->dptr;
  q.out = (float *)s.predproj->dptr;
  FA_TRY(tdt_rows<0>(ctx, q, HID / kRowsCols, W, -1));
  FA_LAUNCH_CHECK(ctx, "tdt_predict");
  return FA_OK;
}

int tdt_round(fa_ctx *ctx, fa_tdt *d, TdtState &s, const fa_tensor *proj, int W, int T, int cap) {
  int *t = (int *)s.ints, *emitted = t + W, *last_tok = t + 2 * W, *counts = t + 3 * W, *done = t + 4 * W;
  int *ids = done + 4, *frames = ids + (size_t)W * cap;
  fa_tensor *logits = nullptr;
  if (s.planes) {
    {
      LaunchScope ls(ctx, "tdt_joint_digits");
      FA_CHECK_CUDA(ctx, fa_launch_dep(ctx, k_tdt_joint_digits, dim3(W), dim3(256), 0, (const float *)proj->dptr, (const int *)t, T,
                                       (const float *)s.predproj->dptr, (const float *)d->out_scale->dptr, W, ctx->int8_limbs,
                                       (int8_t *)s.planes, (float *)s.rowscale));
    }
    FA_TRY(fa_matmul_int8_planes(ctx, (const int8_t *)s.planes, (const float *)s.rowscale, ctx->int8_limbs, W, d->out_q,
                                 (const float *)d->ones->dptr, LOGITS, HID, (const float *)d->out_b->dptr, (float *)s.logits->dptr));
  } else {
    {
      LaunchScope ls(ctx, "tdt_joint_in");
      k_tdt_joint_in<<<W, 256, 0, ctx->stream>>>((const float *)proj->dptr, t, T, (const float *)s.predproj->dptr,
                                                 d->out_scale ? (const float *)d->out_scale->dptr : nullptr, (float *)s.J->dptr);
    }
    if (d->out_q)
      FA_TRY(fa_matmul_int8(ctx, s.J, d->out_q, d->ones, LOGITS, HID, d->out_b, FA_ACT_NONE, &logits));
    else
      FA_TRY(fa_matmul(ctx, s.J, d->out_w, d->out_b, FA_ACT_NONE, nullptr, &logits));
  }
  const float *lg = (const float *)(logits ? logits->dptr : s.logits->dptr);
  {
    LaunchScope ls(ctx, "tdt_pick");
    FA_CHECK_CUDA(ctx, fa_launch_dep(ctx, k_tdt_pick, dim3(W), dim3(kPickThreads), 0, lg, LOGITS, T, cap, t, emitted, last_tok, counts,
                                     ids, frames, (float *)s.h0t->dptr,
                                     (const float *)s.nh0t->dptr, (float *)s.h1t->dptr, (const float *)s.nh1t->dptr,
                                     (float *)s.c0->dptr, (float *)s.c1->dptr, (const float *)s.nc0->dptr,
                                     (const float *)s.nc1->dptr, done));
  }
  if (logits) FA_TRY(fa_free_tensor(ctx, logits));
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
  const int wpad = ceil_div(W, 32) * 32;
  alloc(wpad, HID, &s.h0t), alloc(wpad, HID, &s.nh0t), alloc(wpad, HID, &s.h1t), alloc(wpad, HID, &s.nh1t),
      alloc(W, HID, &s.c0), alloc(W, HID, &s.c1), alloc(W, HID, &s.nc0), alloc(W, HID, &s.nc1), alloc(W, HID, &s.predproj),
      alloc(W, HID, &s.J);
  const size_t n_int = (size_t)4 * W + 4 + (size_t)2 * W * cap;
  if (rc == FA_OK) rc = fa_block_acquire(ctx, n_int * 4, &s.ints, &s.ints_bytes);
  if (rc == FA_OK && d->out_q && fa_matmul_int8_planes_ok(ctx, W, LOGITS, HID)) {
    alloc(W, LOGITS, &s.logits);
    if (rc == FA_OK) rc = fa_block_acquire(ctx, fa_tc_act_bytes(W, HID, 1, ctx->int8_limbs), &s.planes, &s.planes_bytes);
    if (rc == FA_OK) rc = fa_block_acquire(ctx, (size_t)W * 4, &s.rowscale, &s.rowscale_bytes);
  }
  int *t = (int *)s.ints, *last_tok = t + 2 * W, *done = t + 4 * W;
  if (rc == FA_OK) {
    // decode_proj :290-294: zero state, last token = blank, predict + predproj once
    fa_tensor *z[] = {s.h0t, s.nh0t, s.h1t, s.nh1t, s.c0, s.c1, s.nc0, s.nc1};
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
  if (s.planes) fa_block_release(ctx, s.planes);
  if (s.rowscale) fa_block_release(ctx, s.rowscale);
  ctx->int8_limbs = saved_limbs;
  fa_pop_arena(ctx, arena);
  if (rc != FA_OK) ctx->err = msg;
  if (rounds_out) *rounds_out = rounds;
  return rc;
}
