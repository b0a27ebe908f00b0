// Decode-size products (M <= 4 activation rows) on the CUDA cores: pure streams over the weights in the
// layouts the reference uploads them in (no repack, no packing prepass, no TMEM or cluster set-up), with
// 128-bit coalesced loads, in-register dequantisation and f32 / exact-integer accumulation.
//
//   k_gemv_nbits  matmulNBits (rust/wasm-kernels/src/lib.rs:169-203): bq [N][nblk][16] nibbles, K-contiguous.
//                 One warp per output column; a lane takes whole 32-weight blocks (one 16-byte load each).
//                 The activation row is split, inside the kernel, into two int8 digits of its own maximum,
//                 stored in the even/odd order the nibbles unpack to, so a block is 16 dp4a per digit pair
//                 and its sum is an exact integer; zero-point and scale are applied once per block:
//                 y = s_m * sum_blk scale[n,blk] * ((S1 - zp*A1) + (S2 - zp*A2) / 128).
//                 Arithmetic budget: ~1 lane-op per weight at M = 1 (an f32 unpack-and-FMA needs 4).
//   k_gemv_kn     matmul with f16-storage B [K][N] (lib.rs:59-94) and matmulInt8 with wq [K][N]
//                 (lib.rs:143-162): N-contiguous rows.  A warp owns 32*VEC consecutive columns, the 8 warps of
//                 a CTA take rows k round-robin, K is split over gridDim.y; activations stay f32 (exact).
//                 Partial sums meet in a scratch buffer and the last CTA to arrive (an atomic ticket, no
//                 waiting) adds them in slice order, so the result does not depend on scheduling.
#include <cuda_fp16.h>

#include <type_traits>

#include "fa_internal.cuh"

namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ float warp_sum_f(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max_f(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// ---- int4 ---------------------------------------------------------------------------------------

// One 32-weight block of R weight rows against the digits of every activation row.
template <int M, int R>
__device__ __forceinline__ void nbits_block(const uint4 (&wv)[R], const float (&sc)[R], const int (&z)[R], int b, int K, int nblk,
                                            const int8_t *dig, const int *SA, float (&acc)[R][M]) {
  int lo[R][4], hi[R][4];
#pragma unroll
  for (int r = 0; r < R; r++) {
    lo[r][0] = (int)(wv[r].x & 0x0F0F0F0Fu), hi[r][0] = (int)((wv[r].x >> 4) & 0x0F0F0F0Fu);
    lo[r][1] = (int)(wv[r].y & 0x0F0F0F0Fu), hi[r][1] = (int)((wv[r].y >> 4) & 0x0F0F0F0Fu);
    lo[r][2] = (int)(wv[r].z & 0x0F0F0F0Fu), hi[r][2] = (int)((wv[r].z >> 4) & 0x0F0F0F0Fu);
    lo[r][3] = (int)(wv[r].w & 0x0F0F0F0Fu), hi[r][3] = (int)((wv[r].w >> 4) & 0x0F0F0F0Fu);
  }
#pragma unroll
  for (int m = 0; m < M; m++) {
    const int4 e1 = *(const int4 *)(dig + (size_t)(m * 2 + 0) * K + b * 16);
    const int4 o1 = *(const int4 *)(dig + (size_t)(m * 2 + 0) * K + (K >> 1) + b * 16);
    const int4 e2 = *(const int4 *)(dig + (size_t)(m * 2 + 1) * K + b * 16);
    const int4 o2 = *(const int4 *)(dig + (size_t)(m * 2 + 1) * K + (K >> 1) + b * 16);
    const int a1 = SA[(m * 2 + 0) * nblk + b], a2 = SA[(m * 2 + 1) * nblk + b];
#pragma unroll
    for (int r = 0; r < R; r++) {
      int s1 = 0, s2 = 0;
      s1 = __dp4a(lo[r][0], e1.x, s1), s1 = __dp4a(hi[r][0], o1.x, s1);
      s1 = __dp4a(lo[r][1], e1.y, s1), s1 = __dp4a(hi[r][1], o1.y, s1);
      s1 = __dp4a(lo[r][2], e1.z, s1), s1 = __dp4a(hi[r][2], o1.z, s1);
      s1 = __dp4a(lo[r][3], e1.w, s1), s1 = __dp4a(hi[r][3], o1.w, s1);
      s2 = __dp4a(lo[r][0], e2.x, s2), s2 = __dp4a(hi[r][0], o2.x, s2);
      s2 = __dp4a(lo[r][1], e2.y, s2), s2 = __dp4a(hi[r][1], o2.y, s2);
      s2 = __dp4a(lo[r][2], e2.z, s2), s2 = __dp4a(hi[r][2], o2.z, s2);
      s2 = __dp4a(lo[r][3], e2.w, s2), s2 = __dp4a(hi[r][3], o2.w, s2);
      const float f = fmaf((float)(s2 - z[r] * a2), 1.0f / 128.0f, (float)(s1 - z[r] * a1));
      acc[r][m] = fmaf(sc[r], f, acc[r][m]);
    }
  }
}

// The kernel is one pass: a warp's first (for the benchmark shapes: only) group of R weight rows is requested
// from HBM BEFORE the activation digits are made - before the kernel even waits for its predecessor in the stream:
// the packed weights of a PackedBytes handle are only ever written by an upload, never by a kernel, so reading them
// early is safe, while scales, zero-points and activations (tensors a kernel may have produced) are read after the
// wait.  The stream over the weights - the whole cost of the product - thus runs under the predecessor's tail and
// the prologue instead of after them (measured before the change: ~4 us of a 5.5 us launch had no weight byte in
// flight, against 1.6 us of streaming).  PRE blocks per lane are requested early (64 blocks per row at K = 2048 =
// 2 per lane); longer rows load the rest in the loop.
// Prologue: a thread owns 8 consecutive k of one row, which is exactly one 32-bit word of the even-k digit plane and
// one of the odd-k plane, so digits go to shared memory as whole words and the per-block digit sums are two shuffles.
template <int M, int R>
__global__ void __launch_bounds__(kThreads, 2) k_gemv_nbits(const float *__restrict__ a, const uint8_t *__restrict__ bq,
                                                            const float *__restrict__ scales, const uint8_t *__restrict__ zp,
                                                            float *__restrict__ y, int N, int K, int nblk, int zpb) {
  constexpr int PRE = 2;
  extern __shared__ __align__(16) unsigned char smem[];
  int8_t *dig = (int8_t *)smem;                     // [M][2] planes of K bytes: even-k words of every block (16 B
                                                    // each, so 8 lanes read 128 consecutive bytes), then odd-k words
  int *SA = (int *)(smem + (size_t)M * 2 * K);      // [M][2][nblk] digit sums per block
  float *red = (float *)(SA + M * 2 * nblk);        // [8][M] per-warp row maxima
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint4 *bq4 = (const uint4 *)bq;
  const int n_first = (blockIdx.x * 8 + warp) * R, n_stride = gridDim.x * 8 * R;

  // ---- early requests: the first group's weights --------------------------------------------------------------
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  uint4 pw[PRE][R];
#pragma unroll
  for (int i = 0; i < PRE; i++) {
    const int b = lane + 32 * i;
#pragma unroll
    for (int r = 0; r < R; r++) {
      const int n = n_first + r < N ? n_first + r : N - 1;
      pw[i][r] = (b < nblk && n_first < N) ? __ldcs(bq4 + (size_t)n * nblk + b) : make_uint4(0u, 0u, 0u, 0u);
    }
  }
  asm volatile("griddepcontrol.wait;" ::: "memory");
  float psc[PRE][R];
  unsigned pzb[PRE][R];
#pragma unroll
  for (int i = 0; i < PRE; i++) {
    const int b = lane + 32 * i;
#pragma unroll
    for (int r = 0; r < R; r++) {
      const int n = n_first + r < N ? n_first + r : N - 1;
      const bool ok = b < nblk && n_first < N;
      psc[i][r] = ok ? __ldg(scales + (size_t)n * nblk + b) : 0.f;
      pzb[i][r] = ok ? (unsigned)__ldg(zp + (size_t)n * zpb + (b >> 1)) : 0u;
    }
  }

  // ---- activation digits: q1 = rint(a/s), q2 = rint((a/s - q1) * 128) with s = max|row| / 127 --------------------
  // The warps split the rows between them (8 / M warps per row), so the code below handles ONE row per thread and
  // its register need does not grow with M; the second sweep re-reads the row (a few KB, L1-resident).
  constexpr int WPR = 8 / M;                       // warps per row (M = 3: two warps idle here)
  const int row = warp % M, wr = warp / M;
  const bool prow = wr < WPR;
  const float *arow = a + (size_t)row * K;
  float mx = 0.f;
  if (prow)
    for (int k0 = (wr * 32 + lane) * 8; k0 < K; k0 += WPR * 256) {
      const float4 x0 = __ldg((const float4 *)(arow + k0)), x1 = __ldg((const float4 *)(arow + k0 + 4));
      mx = fmaxf(mx, fmaxf(fmaxf(fabsf(x0.x), fabsf(x0.y)), fmaxf(fabsf(x0.z), fabsf(x0.w))));
      mx = fmaxf(mx, fmaxf(fmaxf(fabsf(x1.x), fabsf(x1.y)), fmaxf(fabsf(x1.z), fabsf(x1.w))));
    }
  mx = warp_max_f(mx);
  if (lane == 0) red[warp] = mx;
  __syncthreads();
  float rs[M];
#pragma unroll
  for (int m = 0; m < M; m++) {
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < WPR; w++) t = fmaxf(t, red[w * M + m]);
    rs[m] = t > 0.f ? t / 127.0f : 1.0f;
  }
  if (prow) {
    float inv = 1.0f;
#pragma unroll
    for (int m = 0; m < M; m++)
      if (m == row) inv = 1.0f / rs[m];
    const int kend = ((K + WPR * 256 - 1) / (WPR * 256)) * (WPR * 256);  // whole warps stay together for the shuffles
    for (int k0 = (wr * 32 + lane) * 8; k0 < kend; k0 += WPR * 256) {
      const bool in = k0 < K;
      const int b = k0 >> 5, wi = (k0 & 31) >> 3;
      float x[8];
      if (in) {
        const float4 x0 = __ldg((const float4 *)(arow + k0)), x1 = __ldg((const float4 *)(arow + k0 + 4));
        x[0] = x0.x, x[1] = x0.y, x[2] = x0.z, x[3] = x0.w, x[4] = x1.x, x[5] = x1.y, x[6] = x1.z, x[7] = x1.w;
      } else {
#pragma unroll
        for (int i = 0; i < 8; i++) x[i] = 0.f;
      }
      int q1[8], q2[8], s1 = 0, s2 = 0;
#pragma unroll
      for (int i = 0; i < 8; i++) {
        const float t = x[i] * inv;
        const float f1 = rintf(t);
        q1[i] = (int)f1;
        q2[i] = (int)rintf((t - f1) * 128.0f);
        s1 += q1[i];
        s2 += q2[i];
      }
      // digit words: bytes = k 0,2,4,6 (even plane) and 1,3,5,7 (odd plane) of this thread's 8
      auto pack = [](int b0, int b1, int b2, int b3) {
        return (unsigned)(b0 & 0xFF) | ((unsigned)(b1 & 0xFF) << 8) | ((unsigned)(b2 & 0xFF) << 16) | ((unsigned)(b3 & 0xFF) << 24);
      };
      if (in) {
        *(unsigned *)(dig + (size_t)(row * 2 + 0) * K + b * 16 + wi * 4) = pack(q1[0], q1[2], q1[4], q1[6]);
        *(unsigned *)(dig + (size_t)(row * 2 + 0) * K + (K >> 1) + b * 16 + wi * 4) = pack(q1[1], q1[3], q1[5], q1[7]);
        *(unsigned *)(dig + (size_t)(row * 2 + 1) * K + b * 16 + wi * 4) = pack(q2[0], q2[2], q2[4], q2[6]);
        *(unsigned *)(dig + (size_t)(row * 2 + 1) * K + (K >> 1) + b * 16 + wi * 4) = pack(q2[1], q2[3], q2[5], q2[7]);
      }
      // the 4 lanes of a 32-weight block
      s1 += __shfl_xor_sync(0xffffffffu, s1, 1), s1 += __shfl_xor_sync(0xffffffffu, s1, 2);
      s2 += __shfl_xor_sync(0xffffffffu, s2, 1), s2 += __shfl_xor_sync(0xffffffffu, s2, 2);
      if (in && (lane & 3) == 0) {
        SA[(row * 2 + 0) * nblk + b] = s1;
        SA[(row * 2 + 1) * nblk + b] = s2;
      }
    }
  }
  __syncthreads();

  for (int n0 = n_first; n0 < N; n0 += n_stride) {
    float acc[R][M];
#pragma unroll
    for (int r = 0; r < R; r++)
#pragma unroll
      for (int m = 0; m < M; m++) acc[r][m] = 0.f;
    const bool early = n0 == n_first;
#pragma unroll
    for (int i = 0; i < PRE; i++) {
      const int b = lane + 32 * i;
      if (b >= nblk) break;
      uint4 wv[R];
      float sc[R];
      int z[R];
#pragma unroll
      for (int r = 0; r < R; r++) {
        unsigned zb;
        if (early) {
          wv[r] = pw[i][r], sc[r] = psc[i][r], zb = pzb[i][r];
        } else {
          const int n = n0 + r < N ? n0 + r : N - 1;
          wv[r] = __ldcs(bq4 + (size_t)n * nblk + b);
          sc[r] = scales[(size_t)n * nblk + b];
          zb = zp[(size_t)n * zpb + (b >> 1)];
        }
        z[r] = (b & 1) ? (int)(zb >> 4) : (int)(zb & 15u);
      }
      nbits_block<M, R>(wv, sc, z, b, K, nblk, dig, SA, acc);
    }
    for (int b = lane + 32 * PRE; b < nblk; b += 32) {
      uint4 wv[R];
      float sc[R];
      int z[R];
#pragma unroll
      for (int r = 0; r < R; r++) {
        const int n = n0 + r < N ? n0 + r : N - 1;
        wv[r] = __ldcs(bq4 + (size_t)n * nblk + b);
        sc[r] = scales[(size_t)n * nblk + b];
        const unsigned zb = zp[(size_t)n * zpb + (b >> 1)];
        z[r] = (b & 1) ? (int)(zb >> 4) : (int)(zb & 15u);
      }
      nbits_block<M, R>(wv, sc, z, b, K, nblk, dig, SA, acc);
    }
#pragma unroll
    for (int r = 0; r < R; r++)
#pragma unroll
      for (int m = 0; m < M; m++) {
        const float t = warp_sum_f(acc[r][m]);
        if (lane == 0 && n0 + r < N) y[(size_t)m * N + n0 + r] = t * rs[m];
      }
  }
}

// ---- f16 / int8 weights, N-contiguous ---------------------------------------------------------------

struct GemvEp {
  const float *colscale, *bias, *add;
  int act;
};

__device__ __forceinline__ float gemv_finish(float acc, int m, int n, int N, const GemvEp &ep) {
  float v = acc;
  if (ep.colscale) v *= ep.colscale[n];
  if (ep.bias) v += ep.bias[n];
  v = fa_actf(v, ep.act);
  if (ep.add) v += ep.add[(size_t)m * N + n];
  return v;
}

// VEC weights per lane and row: 8 (f16, 16-byte loads) or 4 (f16, 8-byte loads, for N % 8 != 0) or 16 (int8).
template <int VEC, bool I8>
__device__ __forceinline__ void load_row(const void *w, size_t off, float (&f)[VEC]) {
  if constexpr (I8) {
    static_assert(VEC == 16, "int8 rows are read 16 bytes at a time");
    const uint4 v = __ldcs((const uint4 *)((const int8_t *)w + off));
    const unsigned wd[4] = {v.x ^ 0x80808080u, v.y ^ 0x80808080u, v.z ^ 0x80808080u, v.w ^ 0x80808080u};
#pragma unroll
    for (int i = 0; i < 4; i++) {
      // byte b of (q + 128) into the mantissa of 2^23: the float 8388608 + q + 128, then back to q
      f[i * 4 + 0] = __uint_as_float(__byte_perm(wd[i], 0x4B000000u, 0x7650)) - 8388736.0f;
      f[i * 4 + 1] = __uint_as_float(__byte_perm(wd[i], 0x4B000000u, 0x7651)) - 8388736.0f;
      f[i * 4 + 2] = __uint_as_float(__byte_perm(wd[i], 0x4B000000u, 0x7652)) - 8388736.0f;
      f[i * 4 + 3] = __uint_as_float(__byte_perm(wd[i], 0x4B000000u, 0x7653)) - 8388736.0f;
    }
  } else if constexpr (VEC == 8) {
    const uint4 v = __ldcs((const uint4 *)((const __half *)w + off));
    const __half2 *h = (const __half2 *)&v;
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const float2 t = __half22float2(h[i]);
      f[2 * i] = t.x, f[2 * i + 1] = t.y;
    }
  } else {
    static_assert(VEC == 4, "f16 rows are read 16 or 8 bytes at a time");
    const uint2 v = __ldcs((const uint2 *)((const __half *)w + off));
    const __half2 *h = (const __half2 *)&v;
    const float2 t0 = __half22float2(h[0]), t1 = __half22float2(h[1]);
    f[0] = t0.x, f[1] = t0.y, f[2] = t1.x, f[3] = t1.y;
  }
}

template <int M, int VEC, bool I8>
__global__ void __launch_bounds__(kThreads) k_gemv_kn(const float *__restrict__ a, const void *__restrict__ w,
                                                      float *__restrict__ y, float *__restrict__ partials,
                                                      int *__restrict__ tickets, int K, int N, int kslice, GemvEp ep) {
  extern __shared__ __align__(16) unsigned char smem[];
  float *as = (float *)smem;                 // [M][kslice] activations of this K slice
  float *red = as + (size_t)M * kslice;      // [8][32*VEC]
  __shared__ int last_flag;
  constexpr int U = I8 ? 2 : 4;              // rows in flight per warp
  constexpr int CW = 32 * VEC;               // columns per CTA
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int k0 = blockIdx.y * kslice, k1 = min(K, k0 + kslice), ks = gridDim.y;
  const int c0 = blockIdx.x * CW + lane * VEC;
  const bool live = c0 < N;  // N % VEC == 0, so a live lane owns VEC whole columns
  fa_grid_dep_sync();
  for (int i = tid; i < M * kslice; i += kThreads) {
    const int m = i / kslice, kk = i - m * kslice;
    as[i] = k0 + kk < k1 ? a[(size_t)m * K + k0 + kk] : 0.f;
  }
  __syncthreads();
  float acc[M][VEC];
#pragma unroll
  for (int m = 0; m < M; m++)
#pragma unroll
    for (int v = 0; v < VEC; v++) acc[m][v] = 0.f;
  if (live) {
    for (int kk = k0 + warp * U; kk < k1; kk += 8 * U) {
      float f[U][VEC];
#pragma unroll
      for (int u = 0; u < U; u++) {
        const int k = kk + u < k1 ? kk + u : k1 - 1;
        load_row<VEC, I8>(w, (size_t)k * N + c0, f[u]);
      }
#pragma unroll
      for (int u = 0; u < U; u++) {
        if (kk + u < k1) {
#pragma unroll
          for (int m = 0; m < M; m++) {
            const float av = as[m * kslice + (kk + u - k0)];
#pragma unroll
            for (int v = 0; v < VEC; v++) acc[m][v] = fmaf(av, f[u][v], acc[m][v]);
          }
        }
      }
    }
  }
  // the 8 warps' partial sums, one activation row at a time, added in warp order
  for (int m = 0; m < M; m++) {
#pragma unroll
    for (int v = 0; v < VEC; v++) red[warp * CW + lane * VEC + v] = acc[m][v];
    __syncthreads();
    for (int c = tid; c < CW; c += kThreads) {
      const int n = blockIdx.x * CW + c;
      if (n < N) {
        float s = red[c];
#pragma unroll
        for (int wv = 1; wv < 8; wv++) s += red[wv * CW + c];
        if (ks == 1)
          y[(size_t)m * N + n] = gemv_finish(s, m, n, N, ep);
        else
          partials[((size_t)blockIdx.y * M + m) * N + n] = s;
      }
    }
    __syncthreads();
  }
  if (ks == 1) return;
  __threadfence();
  if (tid == 0) {
    const int old = atomicAdd(&tickets[blockIdx.x], 1);
    last_flag = old == ks - 1;
    if (last_flag) tickets[blockIdx.x] = 0;  // ready for the next launch on this stream
  }
  __syncthreads();
  if (!last_flag) return;
  __threadfence();
  for (int i = tid; i < M * CW; i += kThreads) {
    const int m = i / CW, n = blockIdx.x * CW + (i - m * CW);
    if (n < N) {
      float s = 0.f;
#pragma unroll 8
      for (int q = 0; q < ks; q++) s += __ldcg(&partials[((size_t)q * M + m) * N + n]);
      y[(size_t)m * N + n] = gemv_finish(s, m, n, N, ep);
    }
  }
}

template <int M, int VEC, bool I8>
int launch_kn(fa_ctx *ctx, const float *a, const void *w, float *y, float *partials, int K, int N, int kslice, int ksplit,
              const GemvEp &ep) {
  const size_t smem = ((size_t)M * kslice + 8 * 32 * VEC) * sizeof(float);
  auto kern = k_gemv_kn<M, VEC, I8>;
  if (smem > 48 * 1024) FA_CHECK_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  {
    LaunchScope ls(ctx, I8 ? "gemv_i8" : "gemv_f16");
    fa_launch_dep(ctx, kern, dim3(ceil_div(N, 32 * VEC), ksplit), dim3(kThreads), smem, a, w, y, partials, ctx->gemv_tickets, K,
                  N, kslice, ep);
  }
  FA_LAUNCH_CHECK(ctx, "gemv_kn");
  return FA_OK;
}

template <int VEC, bool I8>
int dispatch_kn(fa_ctx *ctx, int M, const float *a, const void *w, float *y, float *partials, int K, int N, int kslice,
                int ksplit, const GemvEp &ep) {
  switch (M) {
    case 1: return launch_kn<1, VEC, I8>(ctx, a, w, y, partials, K, N, kslice, ksplit, ep);
    case 2: return launch_kn<2, VEC, I8>(ctx, a, w, y, partials, K, N, kslice, ksplit, ep);
    case 3: return launch_kn<3, VEC, I8>(ctx, a, w, y, partials, K, N, kslice, ksplit, ep);
    default: return launch_kn<4, VEC, I8>(ctx, a, w, y, partials, K, N, kslice, ksplit, ep);
  }
}

template <int M>
int launch_nbits(fa_ctx *ctx, const float *a, const uint8_t *bq, const float *scales, const uint8_t *zp, float *y, int N,
                 int K, int nblk, int zpb) {
  const size_t smem = (size_t)M * 2 * K + (size_t)M * 2 * nblk * 4 + 8 * M * 4;
  // output columns per warp pass (each digit load is shared between R rows of weights): 4 for one activation row -
  // with two resident CTAs per SM (register cap 128) one wave then covers 148 * 2 * 8 * 4 = 9472 columns - and 2 for
  // more rows, where 4 would not fit the registers next to the early-requested weights
  constexpr int R = M == 1 ? 4 : 2;
  auto kern = k_gemv_nbits<M, R>;
  if (smem > 48 * 1024) FA_CHECK_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  // one resident wave: every CTA pays the digit prologue once and a second wave would pay it twice
  int per_sm = 0;
  FA_CHECK_CUDA(ctx, cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, kThreads, smem));
  if (per_sm < 1) per_sm = 1;
  if (per_sm > ctx->gemv_ctas_per_sm) per_sm = ctx->gemv_ctas_per_sm;
  int grid = ceil_div(N, 8 * R);
  if (grid > ctx->sm_count * per_sm) grid = ctx->sm_count * per_sm;
  {
    LaunchScope ls(ctx, "gemv_nbits");
    fa_launch_dep(ctx, kern, dim3(grid), dim3(kThreads), smem, a, bq, scales, zp, y, N, K, nblk, zpb);
  }
  FA_LAUNCH_CHECK(ctx, "gemv_nbits");
  return FA_OK;
}

}  // namespace

bool fa_gemv_nbits_ok(int M, int N, int K, int block_size) {
  return M >= 1 && M <= kGemvMaxRows && block_size == 32 && (K & 31) == 0 && K >= 32 && N >= 1 &&
         (size_t)M * 2 * K + (size_t)M * (K / 32) * 8 + 64 <= 96 * 1024;
}

int fa_gemv_nbits(fa_ctx *ctx, const float *a, const uint8_t *bq, const float *scales, const uint8_t *zp, float *y, int M,
                  int N, int K, int nblk, int zpb) {
  switch (M) {
    case 1: return launch_nbits<1>(ctx, a, bq, scales, zp, y, N, K, nblk, zpb);
    case 2: return launch_nbits<2>(ctx, a, bq, scales, zp, y, N, K, nblk, zpb);
    case 3: return launch_nbits<3>(ctx, a, bq, scales, zp, y, N, K, nblk, zpb);
    default: return launch_nbits<4>(ctx, a, bq, scales, zp, y, N, K, nblk, zpb);
  }
}

// ---- int4, 5..16 activation rows: weights streamed once as uploaded, dequantised in registers, mma.sync -------------
// The tensor-core GEMM serves these shapes from a dequantised f16 copy of the weights (4x the bytes of the 4-bit
// matrix) and pays cluster set-up, a packing prepass and a split-K hand-off for ~0.5 GFLOP of work.  Here a CTA owns
// groups of 8 output columns; its 16 warps split the K blocks of a group between them (a warp takes 4 consecutive
// 32-weight blocks, one per lane of a column's 4-lane group, as ONE 16-byte load per lane, so the 4 lanes of a column
// read 64 consecutive bytes), widens its nibbles to f16 with (q - zp) * scale, and multiplies them as the B fragment
// of mma.sync.m16n8k16 against all (up to 16) activation rows at once; partial sums of the 16 warps meet in shared
// memory.  Which K index sits in which of the instruction's 16 k-slots does not matter for a sum, so a lane uses the
// nibbles in the order one mask extracts them (k, k+4 of every group of 8), and the activation rows are stored in
// shared memory in that same order (f16 value plane and, optionally, the rounding-residue plane that keeps f32-grade
// activations) with a row pitch and block pitch that make the A-fragment loads conflict-free.
constexpr int kMmaWarps = 16;
constexpr int kMmaBatch = 4;   // column groups whose partial tiles are reduced together (one pair of block barriers)
constexpr int kMmaSeg = 80;    // bytes per 32-k block of an activation row in shared memory (64 + 16: the 4 lanes of a
                               // column group read blocks b..b+3 of a row at 16-byte bank groups 0, 5, 2, 7)
__host__ __device__ constexpr int mma_row_pitch(int nblk) { return nblk * kMmaSeg + (((nblk * kMmaSeg / 16) % 8) == 4 ? 0 : ((4 - (nblk * kMmaSeg / 16) % 8 + 8) % 8) * 16); }

__device__ __forceinline__ void mma16816_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <bool HILO>
__global__ void __launch_bounds__(kMmaWarps * 32, 1) k_nbits_mma(const float *__restrict__ a, const uint8_t *__restrict__ bq,
                                                                  const float *__restrict__ scales, const uint8_t *__restrict__ zp,
                                                                  float *__restrict__ y, int M, int N, int K, int nblk, int zpb) {
  extern __shared__ __align__(16) unsigned char smem[];
  const int pitch = mma_row_pitch(nblk);
  unsigned char *planes = smem;                                         // [HILO ? 2 : 1][16][pitch]
  float *red = (float *)(smem + (size_t)(HILO ? 2 : 1) * 16 * pitch);   // [kMmaBatch][kMmaWarps][32][4]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
  const int groups = N >> 3, quads = (nblk + 3) >> 2;
  const uint4 *bq4 = (const uint4 *)bq;
  constexpr int D = kMmaBatch;  // column groups whose weights are requested ahead: slot gi of the registers below always
                                // serves the gi-th group of a batch, so a value still in flight is never moved

  // requests of this warp's first quad of the first D column groups (weights do not depend on earlier kernels)
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  uint4 pw[D];
  float psc[D];
  unsigned pzb[D];
#pragma unroll
  for (int d = 0; d < D; d++) {
    const int cg = blockIdx.x + d * gridDim.x, b = 4 * warp + t;
    const bool ok = cg < groups && b < nblk;
    const size_t n = (size_t)(cg * 8 + g);
    pw[d] = ok ? __ldcs(bq4 + n * nblk + b) : make_uint4(0u, 0u, 0u, 0u);
    psc[d] = ok ? __ldg(scales + n * nblk + b) : 0.f;
    pzb[d] = ok ? (unsigned)__ldg(zp + n * zpb + (b >> 1)) : 0u;
  }
  asm volatile("griddepcontrol.wait;" ::: "memory");

  // ---- activation rows -> f16 planes, 8 consecutive k per thread, stored k0,k4,k1,k5,k2,k6,k3,k7 ----
  const int words = nblk * 4;
  unsigned any_residue = 0u;
  const bool avec = (K & 7) == 0 && ((uintptr_t)a & 15) == 0;  // rows start 16-byte aligned: two float4 per word
  for (int e = tid; e < 16 * words; e += kMmaWarps * 32) {
    const int m = e / words, w = e - m * words, k0 = w * 8;
    float x[8];
    if (avec && m < M && k0 + 8 <= K) {
      const float4 x0 = __ldg((const float4 *)(a + (size_t)m * K + k0)), x1 = __ldg((const float4 *)(a + (size_t)m * K + k0 + 4));
      x[0] = x0.x, x[1] = x0.y, x[2] = x0.z, x[3] = x0.w, x[4] = x1.x, x[5] = x1.y, x[6] = x1.z, x[7] = x1.w;
    } else {
#pragma unroll
      for (int i = 0; i < 8; i++) x[i] = (m < M && k0 + i < K) ? __ldg(a + (size_t)m * K + k0 + i) : 0.f;
    }
    __half2 h[4], l[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
      h[i] = __floats2half2_rn(x[i], x[i + 4]);
      const float2 f = __half22float2(h[i]);
      l[i] = __floats2half2_rn(x[i] - f.x, x[i + 4] - f.y);
    }
    unsigned char *dst = planes + (size_t)m * pitch + (w >> 2) * kMmaSeg + (w & 3) * 16;
    *(uint4 *)dst = make_uint4(*(uint32_t *)&h[0], *(uint32_t *)&h[1], *(uint32_t *)&h[2], *(uint32_t *)&h[3]);
    if (HILO) {
      const uint4 lv = make_uint4(*(uint32_t *)&l[0], *(uint32_t *)&l[1], *(uint32_t *)&l[2], *(uint32_t *)&l[3]);
      *(uint4 *)(dst + (size_t)16 * pitch) = lv;
      any_residue |= (lv.x | lv.y | lv.z | lv.w) & 0x7FFF7FFFu;
    }
  }
  // rows that are exactly representable in f16 (activations that arrive as f16 values) have an all-zero residue
  // plane: its products are skipped for the whole launch
  const bool use_residue = HILO && __syncthreads_or(any_residue != 0u);
  if (!HILO) __syncthreads();

  // (the walk over the column groups exists twice, with and without the residue products: as a test inside the loop
  // the compiler predicates the instructions instead of branching around them, and they keep their issue slots)
  auto walk = [&](auto res_tag) {
  constexpr bool kRes = decltype(res_tag)::value;
  for (int cg0 = blockIdx.x; cg0 < groups; cg0 += kMmaBatch * gridDim.x) {
    float c[kMmaBatch][4];
#pragma unroll
    for (int gi = 0; gi < kMmaBatch; gi++) {
      c[gi][0] = c[gi][1] = c[gi][2] = c[gi][3] = 0.f;
      const int cg = cg0 + gi * gridDim.x;
      if (cg >= groups) continue;  // (block-uniform)
      const int n = cg * 8 + g;
      for (int q = warp; q < quads; q += kMmaWarps) {
        const int b = 4 * q + t;
        const bool in = b < nblk;
        uint4 wv;
        float sc;
        unsigned zb;
        if (q == warp) {
          wv = pw[gi], sc = psc[gi], zb = pzb[gi];
        } else {
          wv = in ? __ldcs(bq4 + (size_t)n * nblk + b) : make_uint4(0u, 0u, 0u, 0u);
          sc = in ? __ldg(scales + (size_t)n * nblk + b) : 0.f;
          zb = in ? (unsigned)__ldg(zp + (size_t)n * zpb + (b >> 1)) : 0u;
        }
        const int z = (b & 1) ? (int)(zb >> 4) : (int)(zb & 15u);
        const __half2 s2 = __float2half2_rn(sc);
        const uint32_t s2_u = *(const uint32_t *)&s2, zsub_u = 0x64006400u + (uint32_t)z * 0x00010001u;  // 1024 + zp, both halves
        const unsigned char *arow = planes + (size_t)g * pitch + (size_t)(in ? b : 0) * kMmaSeg;
        const uint32_t wd[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
        for (int wi = 0; wi < 4; wi++) {
          // word wi = k 8wi..8wi+7 of the block: pairs (k0,k4) (k1,k5) (k2,k6) (k3,k7)
          uint32_t bp[4];
#pragma unroll
          for (int pi = 0; pi < 4; pi++) {
            const uint32_t hx = ((wd[wi] >> (4 * pi)) & 0x000F000Fu) | 0x64006400u;  // 1024 + q in both halves
            uint32_t d;
            asm("{\n\t.reg .b32 t;\n\tsub.f16x2 t, %1, %2;\n\tmul.f16x2 %0, t, %3;\n\t}" : "=r"(d) : "r"(hx), "r"(zsub_u), "r"(s2_u));
            bp[pi] = d;
          }
          const uint4 a_lo8 = *(const uint4 *)(arow + wi * 16);                        // row g:     (k0,k4)(k1,k5)(k2,k6)(k3,k7)
          const uint4 a_hi8 = *(const uint4 *)(arow + (size_t)8 * pitch + wi * 16);    // row g + 8
          mma16816_f16(c[gi], a_lo8.x, a_hi8.x, a_lo8.y, a_hi8.y, bp[0], bp[1]);
          mma16816_f16(c[gi], a_lo8.z, a_hi8.z, a_lo8.w, a_hi8.w, bp[2], bp[3]);
          if (kRes) {
            const uint4 r_lo8 = *(const uint4 *)(arow + (size_t)16 * pitch + wi * 16);
            const uint4 r_hi8 = *(const uint4 *)(arow + (size_t)24 * pitch + wi * 16);
            mma16816_f16(c[gi], r_lo8.x, r_hi8.x, r_lo8.y, r_hi8.y, bp[0], bp[1]);
            mma16816_f16(c[gi], r_lo8.z, r_hi8.z, r_lo8.w, r_hi8.w, bp[2], bp[3]);
          }
        }
      }
      // request this warp's first quad of the same slot's group in the next batch
      {
        const int cgn = cg + D * gridDim.x, b = 4 * warp + t;
        const bool ok = cgn < groups && b < nblk;
        const size_t nn = (size_t)(cgn * 8 + g);
        pw[gi] = ok ? __ldcs(bq4 + nn * nblk + b) : make_uint4(0u, 0u, 0u, 0u);
        psc[gi] = ok ? __ldg(scales + nn * nblk + b) : 0.f;
        pzb[gi] = ok ? (unsigned)__ldg(zp + nn * zpb + (b >> 1)) : 0u;
      }
    }
    // the 16 warps' partial tiles of the batch meet in shared memory; every thread adds one (group, element) in warp
    // order and stores it
#pragma unroll
    for (int gi = 0; gi < kMmaBatch; gi++)
      *(float4 *)(red + (((size_t)gi * kMmaWarps + warp) * 32 + lane) * 4) = make_float4(c[gi][0], c[gi][1], c[gi][2], c[gi][3]);
    __syncthreads();
    {
      const int gi = tid >> 7, ln = (tid >> 2) & 31, ci = tid & 3;  // 512 threads = 4 groups x 32 lanes x 4 elements
      const int cg = cg0 + gi * gridDim.x;
      if (cg < groups) {
        float sum = 0.f;
#pragma unroll
        for (int w = 0; w < kMmaWarps; w++) sum += red[(((size_t)gi * kMmaWarps + w) * 32 + ln) * 4 + ci];
        const int gg = ln >> 2, tt = ln & 3;
        const int m = gg + ((ci & 2) ? 8 : 0), col = cg * 8 + 2 * tt + (ci & 1);
        if (m < M) y[(size_t)m * N + col] = sum;
      }
    }
    __syncthreads();
  }
  };
  if (use_residue) walk(std::true_type{}); else walk(std::false_type{});
}

// int4 products with up to 16 activation rows on k_nbits_mma.  hilo: the rows enter as value + residue f16 planes.
bool fa_nbits_mma_ok(int M, int N, int K, int block_size, bool hilo) {
  if (!(M >= 1 && M <= 16 && block_size == 32 && K >= 32 && N >= 8 && (N & 7) == 0)) return false;
  const int nblk = (K + 31) / 32;
  const size_t smem = (size_t)(hilo ? 2 : 1) * 16 * mma_row_pitch(nblk) + (size_t)kMmaBatch * kMmaWarps * 32 * 16;
  return smem <= 224 * 1024;
}

// Measured at K = 2048 (recorded replays): 3.8 us + 1.15 us (1.37 with the residue plane) per column group a thread block
// walks, against 10.5-13 us for the tensor-core GEMM on the dequantised copy whatever N is - this kernel is the faster
// one while a block has at most five groups.
bool fa_nbits_mma_worth(fa_ctx *ctx, int N) { return (long long)(N / 8) <= 5ll * ctx->sm_count; }

int fa_nbits_mma(fa_ctx *ctx, const float *a, const uint8_t *bq, const float *scales, const uint8_t *zp, float *y, int M, int N,
                 int K, int nblk, int zpb, bool hilo) {
  const size_t smem = (size_t)(hilo ? 2 : 1) * 16 * mma_row_pitch(nblk) + (size_t)kMmaBatch * kMmaWarps * 32 * 16;
  const int groups = N / 8;
  const dim3 grid((unsigned)(groups < ctx->sm_count ? groups : ctx->sm_count)), block(kMmaWarps * 32);
  cudaError_t e;
  {
    LaunchScope ls(ctx, "nbits_mma");
    if (hilo) {
      FA_CHECK_CUDA(ctx, cudaFuncSetAttribute(k_nbits_mma<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
      e = fa_launch_dep(ctx, k_nbits_mma<true>, grid, block, smem, a, bq, scales, zp, y, M, N, K, nblk, zpb);
    } else {
      FA_CHECK_CUDA(ctx, cudaFuncSetAttribute(k_nbits_mma<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
      e = fa_launch_dep(ctx, k_nbits_mma<false>, grid, block, smem, a, bq, scales, zp, y, M, N, K, nblk, zpb);
    }
  }
  if (e != cudaSuccess) return fa_fail(ctx, FA_ERR_CUDA, "launch nbits_mma: %s", cudaGetErrorString(e));
  FA_LAUNCH_CHECK(ctx, "nbits_mma");
  return FA_OK;
}

// N-contiguous weights: one activation row only.  From two rows on, the tensor-core kernel (which shares each
// weight tile between all rows for free) is at least as fast as this one; measured on 1280 x 1280 f16 at
// M = 4: 10.6 us here against 7.3 us there.
bool fa_gemv_kn_ok(int M, int N, int K, bool i8) { return M == 1 && K >= 1 && N >= 1 && (N % (i8 ? 16 : 4)) == 0; }

// w: f16 [K][N] (i8 = false) or int8 [K][N]; y = act(acc * colscale[n] + bias[n]) + add[m][n].
int fa_gemv_kn(fa_ctx *ctx, const float *a, const void *w, bool i8, const float *colscale, const float *bias, int act,
               const float *add, float *y, int M, int N, int K) {
  const int vec = i8 ? 16 : ((N & 7) == 0 ? 8 : 4);
  const int strips = ceil_div(N, 32 * vec);
  // enough CTAs to put ~4 on every SM; a K slice of at most 2048 rows so its activations fit shared memory
  const int target = 2, cap = 40;
  int ksplit = ceil_div(ctx->sm_count * target, strips);
  int max_split = ceil_div(K, 32);
  if (max_split > cap) max_split = cap;
  if (ksplit > max_split) ksplit = max_split;
  if (ksplit < ceil_div(K, 2048)) ksplit = ceil_div(K, 2048);
  if (ksplit < 1) ksplit = 1;
  int kslice = ceil_div(K, ksplit);
  kslice = (kslice + 7) / 8 * 8;
  ksplit = ceil_div(K, kslice);
  FA_REQUIRE(ctx, strips <= ctx->gemv_ticket_count, "gemv: %d column strips exceed the ticket array", strips);
  void *partials = nullptr;
  size_t pbytes = 0;
  if (ksplit > 1) FA_TRY(fa_block_acquire(ctx, (size_t)ksplit * M * N * sizeof(float), &partials, &pbytes));
  GemvEp ep{colscale, bias, add, act};
  int rc;
  if (i8)
    rc = dispatch_kn<16, true>(ctx, M, a, w, y, (float *)partials, K, N, kslice, ksplit, ep);
  else if (vec == 8)
    rc = dispatch_kn<8, false>(ctx, M, a, w, y, (float *)partials, K, N, kslice, ksplit, ep);
  else
    rc = dispatch_kn<4, false>(ctx, M, a, w, y, (float *)partials, K, N, kslice, ksplit, ep);
  if (partials) fa_block_release(ctx, partials);
  return rc;
}
