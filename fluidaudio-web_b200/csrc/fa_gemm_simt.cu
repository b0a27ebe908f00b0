// Any-shape f32 kernels on CUDA cores: the route for shapes too small or too ragged for
// the TMA-fed tensor-core kernels (odd M/N/K such as the 37x53x41 conformance case), and for
// f32-storage B where the reference computes in f32 (src/gpu/kernels/gemm.js:10-70).
//
// Same math as the reference kernels: f32 accumulate over k ascending, epilogue order
// acc(*scale[n]) + bias[n] -> act -> + add (gemm.js:401-405, 877-879).
#include "fa_internal.cuh"

namespace {

constexpr int TM = 64, TN = 64, TK = 16;

template <int BKIND>
__device__ __forceinline__ float load_b(const void *b, size_t idx) {
  if (BKIND == 0) return ((const float *)b)[idx];
  if (BKIND == 1) return __half2float(((const __half *)b)[idx]);
  return (float)((const int8_t *)b)[idx];
}

// C[M,N] = epi(A[M,K] @ B[K,N]); 256 threads, 64x64 tile, 4x4 outputs per thread.
template <int BKIND>
__global__ void __launch_bounds__(256) k_gemm_simt(const float *__restrict__ a, const void *__restrict__ b,
                                                   const float *__restrict__ colscale, const float *__restrict__ bias,
                                                   int act, const float *__restrict__ add, float *__restrict__ c, int M,
                                                   int N, int K) {
  __shared__ float As[TK][TM + 4];
  __shared__ float Bs[TK][TN + 4];
  const int tid = threadIdx.x;
  const int tx = tid % 16, ty = tid / 16;
  const int m0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < K; k0 += TK) {
    // A tile: 64 rows x 16 k, 1024 elements, 4 per thread (k fastest for coalescing)
#pragma unroll
    for (int i = 0; i < 4; i++) {
      int e = tid + i * 256;
      int r = e / TK, kk = e % TK;
      int gm = m0 + r, gk = k0 + kk;
      As[kk][r] = (gm < M && gk < K) ? a[(size_t)gm * K + gk] : 0.0f;
    }
    // B tile: 16 k x 64 cols (n fastest)
#pragma unroll
    for (int i = 0; i < 4; i++) {
      int e = tid + i * 256;
      int kk = e / TN, cn = e % TN;
      int gk = k0 + kk, gn = n0 + cn;
      Bs[kk][cn] = (gk < K && gn < N) ? load_b<BKIND>(b, (size_t)gk * N + gn) : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < TK; kk++) {
      float av[4], bv[4];
#pragma unroll
      for (int i = 0; i < 4; i++) av[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; j++) bv[j] = Bs[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; i++) {
    int gm = m0 + ty * 4 + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      int gn = n0 + tx * 4 + j;
      if (gn >= N) continue;
      float v = acc[i][j];
      if (colscale) v *= colscale[gn];
      if (bias) v += bias[gn];
      v = fa_actf(v, act);
      if (add) v += add[(size_t)gm * N + gn];
      c[(size_t)gm * N + gn] = v;
    }
  }
}

// int4 MatMulNBits, one thread per output, the reference's own formulation
// (src/gpu/kernels/gemm.js:893-919): per block w=(q-zp)*s, acc += a*w, k ascending.
// Only used for shapes too small to matter; decode sizes go to fa_gemv_nbits.
__global__ void k_nbits_simt(const float *__restrict__ a, const uint8_t *__restrict__ bq,
                             const float *__restrict__ scales, const uint8_t *__restrict__ zp, float *__restrict__ y,
                             int M, int N, int K, int nblk, int zpb) {
  int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= M * N) return;
  int m = idx / N, n = idx % N;
  const float *arow = a + (size_t)m * K;
  const uint8_t *brow = bq + (size_t)n * nblk * 16;
  float acc = 0.0f;
  for (int blk = 0; blk < nblk; blk++) {
    float s = scales[(size_t)n * nblk + blk];
    uint8_t zb = zp[(size_t)n * zpb + (blk >> 1)];
    float z = (float)((blk & 1) ? (zb >> 4) : (zb & 15));
    int kend = min(32, K - blk * 32);
    for (int t = 0; t < kend; t++) {
      uint8_t byte = brow[blk * 16 + (t >> 1)];
      float q = (float)((t & 1) ? (byte >> 4) : (byte & 15));
      acc = fmaf(arow[blk * 32 + t], (q - z) * s, acc);
    }
  }
  y[idx] = acc;
}

}  // namespace

int fa_simt_gemm(fa_ctx *ctx, const float *a, const void *b, int b_kind, const float *colscale, const float *bias,
                 int act, const float *add, float *c, int M, int N, int K) {
  if (M == 0 || N == 0) return FA_OK;
  dim3 grid(ceil_div(N, TN), ceil_div(M, TM));
  FA_REQUIRE(ctx, grid.y <= 65535, "matmul: M=%d too large for the small-shape kernel", M);
  {
    LaunchScope ls(ctx, b_kind == 0 ? "gemm_simt_f32" : (b_kind == 1 ? "gemm_simt_f16b" : "gemm_simt_i8b"));
    if (b_kind == 0)
      k_gemm_simt<0><<<grid, 256, 0, ctx->stream>>>(a, b, colscale, bias, act, add, c, M, N, K);
    else if (b_kind == 1)
      k_gemm_simt<1><<<grid, 256, 0, ctx->stream>>>(a, b, colscale, bias, act, add, c, M, N, K);
    else
      k_gemm_simt<2><<<grid, 256, 0, ctx->stream>>>(a, b, colscale, bias, act, add, c, M, N, K);
  }
  FA_LAUNCH_CHECK(ctx, "gemm_simt");
  return FA_OK;
}

int fa_simt_nbits(fa_ctx *ctx, const float *a, const uint8_t *bq, const float *scales, const uint8_t *zp, float *y,
                  int M, int N, int K, int nblk, int zpb) {
  if (M == 0 || N == 0) return FA_OK;
  {
    LaunchScope ls(ctx, "nbits_simt");
    k_nbits_simt<<<ceil_div(M * N, 128), 128, 0, ctx->stream>>>(a, bq, scales, zp, y, M, N, K, nblk, zpb);
  }
  FA_LAUNCH_CHECK(ctx, "nbits_simt");
  return FA_OK;
}
