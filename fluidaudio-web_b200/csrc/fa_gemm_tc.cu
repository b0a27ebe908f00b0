// tcgen05 GEMM for the f16-weight and int8-weight products (sm_100a).
//
// Replaces the reference's WGSL GEMM family for large shapes: f16-storage B
// (src/gpu/kernels/gemm.js:336-419, 420-503) and int8 B (gemm.js:679-885).
//
// One orientation for every shape: the WEIGHTS are the MMA M-side operand (128 output columns
// n per CTA, one TMEM lane each), the ACTIVATIONS are the MMA N-side operand (MT rows m per CTA,
// one TMEM column each).  Both operands are K-major in global memory ([rows][K], K contiguous),
// brought in by TMA (128-byte swizzle, no multicast) through a multi-stage mbarrier ring, multiplied
// by tcgen05.mma (kind::f16 -> f32, kind::i8 -> s32) into TMEM, and read back with tcgen05.ld by four
// epilogue warps that apply  acc (*rowscale[m]) (*colscale[n]) + bias[n] -> act -> + add[m,n]  and
// store out[m][n] so that the 32 lanes of a warp write 32 consecutive n (coalesced 128-byte rows).
// Decode sizes (M <= 16) use MT = 16: the kernel then is a pure weight-streaming loop with a deep
// ring, which is what bounds it (HBM), while padding M to 16 costs nothing on the tensor pipe.
//
// int8 activations arrive as `limbs` int8 digit planes [limbs][M][K] (see fa_prep_a_i8): plane l is
// stacked as MT extra MMA-N rows, so ONE instruction stream produces all digit products, each an exact
// int32 sum in its own TMEM column range; the epilogue recombines them as sum_l acc_l * 2^(-7 l).
//
// Warp roles (192 threads): warp 0 = TMA producer, warp 1 = TMEM owner + MMA issuer,
// warps 2..5 = epilogue (TMEM lane quadrant = warp_id % 4).
#include "fa_tc_common.cuh"

namespace {

using namespace tc;

constexpr int kThreads = 192;
constexpr int kRowBytes = 128;             // one swizzle atom of K per stage
constexpr int kPTileBytes = 128 * kRowBytes;  // weights tile: 128 rows

struct TcParams {
  int M, N, K;        // logical sizes; K in elements
  int MT;             // activation rows per CTA (multiple of 16, MT*limbs <= 256)
  int limbs;          // activation digit planes (1 for f16)
  int stages;
  int num_kb;         // K blocks of 128 bytes
  int raw_i32;        // store the limb-0 int32 accumulators instead of the float epilogue
  float *out;         // [M][N] f32 (or int32 when raw_i32)
  const float *rowscale, *colscale, *bias, *add;
  int act;
  int *status;
};

__device__ __forceinline__ void report_timeout(int *status, int code, int detail) {
  if (atomicCAS(status, 0, code) == 0) {
    status[1] = (int)(blockIdx.x + blockIdx.y * gridDim.x);
    status[2] = detail;
  }
}

template <int KIND>
__global__ void __launch_bounds__(kThreads, 1)
k_tc_gemm(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_a, const TcParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // carve: [stages] x (P tile 16 KB | Q tile limbs*MT*128 B), then barriers
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const int q_rows = p.MT * p.limbs;
  const uint32_t q_bytes = (uint32_t)q_rows * kRowBytes;
  const uint32_t stage_bytes = kPTileBytes + q_bytes;
  const uint32_t bars = smem_base + (uint32_t)p.stages * stage_bytes;  // 8-byte aligned (stage_bytes % 1024 == 0)
  auto full_bar = [&](int s) { return bars + (uint32_t)s * 8u; };
  auto empty_bar = [&](int s) { return bars + (uint32_t)(p.stages + s) * 8u; };
  const uint32_t acc_bar = bars + (uint32_t)(2 * p.stages) * 8u;
  const uint32_t tmem_slot = acc_bar + 8u;
  const uint32_t abort_flag = tmem_slot + 4u;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * 128, m0 = blockIdx.y * p.MT;
  uint32_t tmem_cols = 32;
  while ((int)tmem_cols < q_rows) tmem_cols <<= 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; s++) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    mbar_init(acc_bar, 1);
    asm volatile("st.shared.u32 [%0], %1;" ::"r"(abort_flag), "r"(0u) : "memory");
    fence_barrier_init();
    fence_proxy_async_smem();
    tma_prefetch_desc(&map_w);
    tma_prefetch_desc(&map_a);
  }
  if (warp == 1) tmem_alloc(tmem_slot, tmem_cols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  uint32_t tmem_base;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem_base) : "r"(tmem_slot) : "memory");

  auto aborted = [&]() {
    uint32_t v;
    asm volatile("ld.volatile.shared.u32 %0, [%1];" : "=r"(v) : "r"(abort_flag) : "memory");
    return v != 0;
  };
  auto set_abort = [&](int code, int detail) {
    asm volatile("st.volatile.shared.u32 [%0], %1;" ::"r"(abort_flag), "r"(1u) : "memory");
    report_timeout(p.status, code, detail);
  };

  if (warp == 0) {
    // ---- TMA producer -----------------------------------------------------------------
    if (lane == 0) {
      const int k_per_kb = KIND == 0 ? 64 : 128;
      for (int kb = 0; kb < p.num_kb; kb++) {
        const int s = kb % p.stages;
        const uint32_t round = (uint32_t)(kb / p.stages);
        if (kb >= p.stages) {
          if (!mbar_wait(empty_bar(s), (round - 1) & 1)) { set_abort(1, kb); break; }
        }
        if (aborted()) break;
        mbar_expect_tx(full_bar(s), stage_bytes);
        const uint32_t dst = smem_base + (uint32_t)s * stage_bytes;
        tma_load_2d(dst, &map_w, kb * k_per_kb, n0, full_bar(s));
        for (int l = 0; l < p.limbs; l++)
          tma_load_3d(dst + kPTileBytes + (uint32_t)(l * p.MT) * kRowBytes, &map_a, kb * k_per_kb, m0, l, full_bar(s));
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer -------------------------------------------------------------------
    if (lane == 0) {
      const uint32_t idesc = make_idesc(KIND, 128, q_rows);
      bool ok = true;
      for (int kb = 0; kb < p.num_kb; kb++) {
        const int s = kb % p.stages;
        const uint32_t round = (uint32_t)(kb / p.stages);
        if (!mbar_wait(full_bar(s), round & 1)) { set_abort(2, kb); ok = false; break; }
        tc_fence_after();
        const uint32_t pa = smem_base + (uint32_t)s * stage_bytes;
        const uint32_t qa = pa + kPTileBytes;
#pragma unroll
        for (int j = 0; j < 4; j++) {  // 4 x 32 bytes of K per stage
          umma<KIND>(tmem_base, smem_desc_sw128(pa + j * 32), smem_desc_sw128(qa + j * 32), idesc,
                     (kb > 0 || j > 0) ? 1u : 0u);
        }
        umma_commit(empty_bar(s));  // frees the stage when these MMAs have read it
      }
      if (ok) umma_commit(acc_bar);  // accumulators complete
    }
  } else {
    // ---- epilogue: TMEM -> registers -> global ------------------------------------------
    const int quad = warp & 3;
    const int n = n0 + quad * 32 + lane;
    bool ok = mbar_wait(acc_bar, 0);
    if (!ok && lane == 0) set_abort(3, quad);
    ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
    if (ok && !aborted()) {
      tc_fence_after();
      const uint32_t lane_addr = tmem_base + ((uint32_t)(quad * 32) << 16);
      const bool n_ok = n < p.N;
      const float cs = (p.colscale && n_ok) ? p.colscale[n] : 1.0f;
      const float bs = (p.bias && n_ok) ? p.bias[n] : 0.0f;
      for (int c = 0; c < p.MT; c += 16) {
        if (m0 + c >= p.M) break;  // warp-uniform: no rows left in this tile
        uint32_t v0[16], v1[16], v2[16];
        tmem_ld16(lane_addr + (uint32_t)c, v0);
        if (p.limbs > 1) tmem_ld16(lane_addr + (uint32_t)(p.MT + c), v1);
        if (p.limbs > 2) tmem_ld16(lane_addr + (uint32_t)(2 * p.MT + c), v2);
        tmem_ld_wait();
        if (!n_ok) continue;
#pragma unroll
        for (int j = 0; j < 16; j++) {
          const int m = m0 + c + j;
          if (m >= p.M) break;
          const size_t o = (size_t)m * p.N + n;
          if (KIND == 1 && p.raw_i32) {
            ((int32_t *)p.out)[o] = (int32_t)v0[j];
            continue;
          }
          float v;
          if (KIND == 0) {
            v = __uint_as_float(v0[j]);
          } else {
            v = (float)(int32_t)v0[j];
            if (p.limbs > 1) v += (float)(int32_t)v1[j] * (1.0f / 128.0f);
            if (p.limbs > 2) v += (float)(int32_t)v2[j] * (1.0f / 16384.0f);
          }
          if (p.rowscale) v *= p.rowscale[m];
          v *= cs;
          v += bs;
          v = fa_actf(v, p.act);
          if (p.add) v += p.add[o];
          p.out[o] = v;
        }
      }
    }
  }

  // ---- teardown --------------------------------------------------------------------------------
  tc_fence_before();
  __syncthreads();
  if (aborted()) {
    // A wait ran out: give copies still in flight time to land before the CTA's shared memory goes away.
    for (int i = 0; i < 1000; i++) __nanosleep(1000);
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, tmem_cols);
  }
}

// ---- prepasses ------------------------------------------------------------------------------------

// f32 [M][K] -> f16 [M][kpad], zero padded.
__global__ void k_prep_a_f16(const float *__restrict__ a, int M, int K, int kpad, __half *__restrict__ out) {
  const size_t total = (size_t)M * (kpad / 2);
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int m = (int)(i / (kpad / 2)), k = (int)(i % (kpad / 2)) * 2;
    const float *row = a + (size_t)m * K;
    float x = k < K ? row[k] : 0.0f, y = k + 1 < K ? row[k + 1] : 0.0f;
    ((__half2 *)out)[i] = __floats2half2_rn(x, y);
  }
}

// One CTA per activation row: s = max|a|/127 (1 when the row is all zero), r = a/s,
// q1 = rint(r), q2 = rint((r-q1)*128), q3 = rint(((r-q1)*128-q2)*128); planes [limbs][M][kpad], zero padded.
// With one limb this is the usual symmetric per-row int8 quantiser; each further limb adds 7 bits.
__global__ void __launch_bounds__(256) k_prep_a_i8(const float *__restrict__ a, int M, int K, int kpad, int limbs,
                                                   int8_t *__restrict__ out, float *__restrict__ rowscale) {
  __shared__ float red[8];
  const int m = blockIdx.x;
  const float *row = a + (size_t)m * K;
  float mx = 0.0f;
  for (int k = threadIdx.x; k < K; k += blockDim.x) mx = fmaxf(mx, fabsf(row[k]));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = mx;
  __syncthreads();
  mx = red[0];
#pragma unroll
  for (int w = 1; w < 8; w++) mx = fmaxf(mx, red[w]);
  const float s = mx > 0.0f ? mx / 127.0f : 1.0f;
  if (threadIdx.x == 0) rowscale[m] = s;
  const size_t plane = (size_t)M * kpad;
  for (int k = threadIdx.x; k < kpad; k += blockDim.x) {
    float r = k < K ? row[k] / s : 0.0f;
    float q1 = rintf(r);
    q1 = fminf(fmaxf(q1, -127.0f), 127.0f);
    out[(size_t)m * kpad + k] = (int8_t)q1;
    if (limbs > 1) {
      float r1 = (r - q1) * 128.0f;  // exact: |r-q1| <= 0.5, scaling by 2^7
      float q2 = rintf(r1);
      out[plane + (size_t)m * kpad + k] = (int8_t)q2;
      if (limbs > 2) {
        float q3 = rintf((r1 - q2) * 128.0f);
        out[2 * plane + (size_t)m * kpad + k] = (int8_t)q3;
      }
    }
  }
}

// int8 [K][N] (reference byte order k*N+n) -> int8 [N][kpad], zero padded.  32x32 tiles through smem.
__global__ void k_repack_i8(const int8_t *__restrict__ w, int K, int N, int kpad, int8_t *__restrict__ out) {
  __shared__ int8_t t[32][33];
  const int k0 = blockIdx.x * 32, n0 = blockIdx.y * 32;
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    int k = k0 + r, n = n0 + threadIdx.x;
    t[r][threadIdx.x] = (k < K && n < N) ? w[(size_t)k * N + n] : (int8_t)0;
  }
  __syncthreads();
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    int n = n0 + r, k = k0 + threadIdx.x;
    if (n < N && k < kpad) out[(size_t)n * kpad + k] = t[threadIdx.x][r];
  }
}

// f32 or f16 [K][N] -> f16 [N][kpad], zero padded.
template <typename SRC>
__global__ void k_repack_f16(const SRC *__restrict__ w, int K, int N, int kpad, __half *__restrict__ out) {
  __shared__ __half t[32][33];
  const int k0 = blockIdx.x * 32, n0 = blockIdx.y * 32;
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    int k = k0 + r, n = n0 + threadIdx.x;
    float v = 0.0f;
    if (k < K && n < N) v = (float)w[(size_t)k * N + n];
    t[r][threadIdx.x] = __float2half_rn(v);
  }
  __syncthreads();
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    int n = n0 + r, k = k0 + threadIdx.x;
    if (n < N && k < kpad) out[(size_t)n * kpad + k] = t[threadIdx.x][r];
  }
}

// int4 MatMulNBits payload -> f16 [N][kpad]: w = (q - zp) * scale rounded to f16 once.
// One thread per 16-byte block (32 weights).
__global__ void k_dequant_nbits(const uint8_t *__restrict__ bq, const float *__restrict__ scales,
                                const uint8_t *__restrict__ zp, int N, int K, int nblk, int zpb, int kpad,
                                __half *__restrict__ out) {
  const int blocks_per_row = kpad / 32;
  const size_t total = (size_t)N * blocks_per_row;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int n = (int)(i / blocks_per_row), blk = (int)(i % blocks_per_row);
    __half2 vals[16];
    if (blk < nblk) {
      const uint4 raw = *(const uint4 *)(bq + ((size_t)n * nblk + blk) * 16);
      const float s = scales[(size_t)n * nblk + blk];
      const uint8_t zb = zp[(size_t)n * zpb + (blk >> 1)];
      const float z = (float)((blk & 1) ? (zb >> 4) : (zb & 15));
      const uint32_t wds[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
      for (int wv = 0; wv < 4; wv++)
#pragma unroll
        for (int b = 0; b < 4; b++) {
          const uint32_t byte = (wds[wv] >> (8 * b)) & 0xffu;
          const int k = blk * 32 + wv * 8 + b * 2;
          float lo = k < K ? ((float)(byte & 15u) - z) * s : 0.0f;
          float hi = k + 1 < K ? ((float)(byte >> 4) - z) * s : 0.0f;
          vals[wv * 4 + b] = __floats2half2_rn(lo, hi);
        }
    } else {
#pragma unroll
      for (int j = 0; j < 16; j++) vals[j] = __floats2half2_rn(0.0f, 0.0f);
    }
    uint4 *dst = (uint4 *)(out + (size_t)n * kpad + (size_t)blk * 32);
#pragma unroll
    for (int j = 0; j < 4; j++) dst[j] = *(const uint4 *)&vals[j * 4];
  }
}

// ---- host -----------------------------------------------------------------------------------------

typedef CUresult (*PFN_encodeTiled)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                    const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

PFN_encodeTiled get_encode() {
  static PFN_encodeTiled fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void *p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = (PFN_encodeTiled)p;
  }
  return fn;
}

template <int KIND>
int launch_tc(fa_ctx *ctx, const void *w_nk, int ldw, const void *a_lmk, int lda, int limbs, void *out, bool raw_i32,
              int M, int N, int K, const TcEpilogue &ep) {
  const int elem = KIND == 0 ? 2 : 1;
  const int k_per_kb = kRowBytes / elem;
  TcParams p{};
  p.M = M;
  p.N = N;
  p.K = K;
  p.limbs = limbs;
  p.num_kb = ceil_div(K, k_per_kb);
  // activation rows per CTA: as many as fit 256 MMA-N columns, rounded to 16, no more than needed
  int mt_max = (256 / limbs) / 16 * 16;
  int mt = ((M + 15) / 16) * 16;
  p.MT = mt < mt_max ? mt : mt_max;
  const size_t stage_bytes = (size_t)kPTileBytes + (size_t)p.MT * limbs * kRowBytes;
  int stages = (int)((200 * 1024) / stage_bytes);
  if (stages > 12) stages = 12;
  if (stages > p.num_kb) stages = p.num_kb;
  if (stages < 1) stages = 1;
  p.stages = stages;
  p.raw_i32 = raw_i32 ? 1 : 0;
  p.out = (float *)out;
  p.rowscale = ep.rowscale;
  p.colscale = ep.colscale;
  p.bias = ep.bias;
  p.add = ep.add;
  p.act = ep.act;
  p.status = ctx->dev_status;
  const size_t smem = stage_bytes * stages + (size_t)(2 * stages + 1) * 8 + 16 + 1024;

  CUtensorMap map_w, map_a;
  FA_TRY(tc::make_tmap_k128(ctx, &map_w, w_nk, elem, (uint64_t)K, (uint64_t)N, (uint64_t)ldw, 0, 0, 128));
  FA_TRY(tc::make_tmap_k128(ctx, &map_a, a_lmk, elem, (uint64_t)K, (uint64_t)M, (uint64_t)lda, (uint64_t)limbs,
                            (uint64_t)M * lda, (uint32_t)p.MT));
  FA_CHECK_CUDA(ctx, cudaFuncSetAttribute(k_tc_gemm<KIND>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
  dim3 grid(ceil_div(N, 128), ceil_div(M, p.MT));
  {
    LaunchScope ls(ctx, KIND == 0 ? "tc_gemm_f16" : "tc_gemm_i8");
    k_tc_gemm<KIND><<<grid, kThreads, smem, ctx->stream>>>(map_w, map_a, p);
  }
  FA_LAUNCH_CHECK(ctx, "tc_gemm");
  return FA_OK;
}

}  // namespace

int tc::make_tmap_k128(fa_ctx *ctx, CUtensorMap *out, const void *base, int elem_bytes, uint64_t k_elems, uint64_t rows,
                       uint64_t ld_elems, uint64_t planes, uint64_t plane_stride_elems, uint32_t box_rows) {
  PFN_encodeTiled enc = get_encode();
  if (!enc) return fa_fail(ctx, FA_ERR_CUDA, "cuTensorMapEncodeTiled is unavailable in this driver");
  FA_REQUIRE(ctx, ((uintptr_t)base & 15) == 0 && (ld_elems * elem_bytes) % 16 == 0,
             "tensor-core operand is not 16-byte aligned (base %p, row pitch %llu bytes)", base,
             (unsigned long long)(ld_elems * elem_bytes));
  // planes == 0: 2-d map [rows][k]; planes >= 1: 3-d map [planes][rows][k]
  const cuuint32_t rank = planes == 0 ? 2 : 3;
  cuuint64_t dims[3] = {k_elems, rows, planes ? planes : 1};
  cuuint64_t strides[2] = {ld_elems * elem_bytes, plane_stride_elems * elem_bytes};
  cuuint32_t box[3] = {(cuuint32_t)(kRowBytes / elem_bytes), box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(out, elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8, rank,
                   const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fa_fail(ctx, FA_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return FA_OK;
}

bool fa_tc_available(fa_ctx *) { return get_encode() != nullptr; }

int fa_tc_gemm_f16(fa_ctx *ctx, const __half *a_mk, int lda, const __half *b_nk, int ldb, float *c, int M, int N,
                   int K, const TcEpilogue &ep) {
  return launch_tc<0>(ctx, b_nk, ldb, a_mk, lda, 1, c, false, M, N, K, ep);
}

int fa_tc_gemm_i8(fa_ctx *ctx, const int8_t *a_lmk, int lda, int limbs, const int8_t *b_nk, int ldb, void *c,
                  bool raw_i32, int M, int N, int K, const TcEpilogue &ep) {
  return launch_tc<1>(ctx, b_nk, ldb, a_lmk, lda, limbs, c, raw_i32, M, N, K, ep);
}

int fa_prep_a_f16(fa_ctx *ctx, const float *a, int M, int K, int kpad, __half *out) {
  if (M == 0) return FA_OK;
  size_t total = (size_t)M * (kpad / 2);
  int grid = (int)((total + 255) / 256);
  int cap = ctx->sm_count * 8;
  if (grid > cap) grid = cap;
  {
    LaunchScope ls(ctx, "prep_a_f16");
    k_prep_a_f16<<<grid, 256, 0, ctx->stream>>>(a, M, K, kpad, out);
  }
  FA_LAUNCH_CHECK(ctx, "prep_a_f16");
  return FA_OK;
}

int fa_prep_a_i8(fa_ctx *ctx, const float *a, int M, int K, int kpad, int limbs, int8_t *out, float *rowscale) {
  if (M == 0) return FA_OK;
  {
    LaunchScope ls(ctx, "prep_a_i8");
    k_prep_a_i8<<<M, 256, 0, ctx->stream>>>(a, M, K, kpad, limbs, out, rowscale);
  }
  FA_LAUNCH_CHECK(ctx, "prep_a_i8");
  return FA_OK;
}

int fa_repack_i8_kn_to_nk(fa_ctx *ctx, const int8_t *w_kn, int K, int N, int kpad, int8_t *out_nk) {
  dim3 grid(ceil_div(kpad, 32), ceil_div(N, 32)), block(32, 8);
  {
    LaunchScope ls(ctx, "repack_i8");
    k_repack_i8<<<grid, block, 0, ctx->stream>>>(w_kn, K, N, kpad, out_nk);
  }
  FA_LAUNCH_CHECK(ctx, "repack_i8");
  return FA_OK;
}

int fa_repack_f_kn_to_nk_f16(fa_ctx *ctx, const void *w_kn, int src_storage, int K, int N, int kpad, __half *out_nk) {
  dim3 grid(ceil_div(kpad, 32), ceil_div(N, 32)), block(32, 8);
  {
    LaunchScope ls(ctx, "repack_f16");
    if (src_storage == FA_F16)
      k_repack_f16<__half><<<grid, block, 0, ctx->stream>>>((const __half *)w_kn, K, N, kpad, out_nk);
    else
      k_repack_f16<float><<<grid, block, 0, ctx->stream>>>((const float *)w_kn, K, N, kpad, out_nk);
  }
  FA_LAUNCH_CHECK(ctx, "repack_f16");
  return FA_OK;
}

int fa_dequant_nbits_f16(fa_ctx *ctx, const uint8_t *bq, const float *scales, const uint8_t *zp, int N, int K,
                         int nblk, int zpb, int kpad, __half *out_nk) {
  size_t total = (size_t)N * (kpad / 32);
  int grid = (int)((total + 127) / 128);
  int cap = ctx->sm_count * 16;
  if (grid > cap) grid = cap;
  {
    LaunchScope ls(ctx, "dequant_nbits_f16");
    k_dequant_nbits<<<grid, 128, 0, ctx->stream>>>(bq, scales, zp, N, K, nblk, zpb, kpad, out_nk);
  }
  FA_LAUNCH_CHECK(ctx, "dequant_nbits_f16");
  return FA_OK;
}
