// Relative-position self-attention of one conformer block in ONE kernel (the optional attnFused member,
// src/gpu/compute.d.ts:247-248; op sequence of src/engines/asr-parakeet/raw-encoder.js:335-341):
//   ac[i][j] = (q[i] + u) . k[j]          bd[i][p] = (q[i] + v) . pos[p]
//   prob[i]  = softmax_j( ac[i][j] + bd[i][T-1-i+j] )          out[i] = sum_j prob[i][j] * v[j]
// per (window, head), T <= 192 frames, head width 128.  The separate-op form stores ac and bd (36 + 72 MB per
// block for 32 windows), reads them back for the shifted softmax and packs q, k, v and the probabilities into
// GEMM operand layouts with four more kernels: seven launches that are all memory traffic for 9 GFLOP of arithmetic.
// Here one CTA owns one (window, head): keys and the head's slice of the positional projection are converted to
// f16 into shared memory once, each of the 12 warps owns 16 query rows and keeps their whole score row block
// (16 x 192, f32) in registers, the positional scores of a 64-key block are computed for the 80 positions those
// rows can reach, shifted through a per-warp staging tile (row r of the tile is read 15 - r columns to the
// right) and added, the softmax runs on the registers, and the probabilities - rounded to f16 exactly as the
// packed operand of the separate-op form is - multiply V from the same shared memory.  Operands f16,
// accumulation f32 (mma.sync m16n8k16: the problem is 0.04 GFLOP per CTA and latency bound, a tcgen05 pipeline
// with TMEM accumulators cannot shift rows by a per-row amount without the same round trip through shared memory).
#include "fa_internal.cuh"

namespace {

constexpr int kAT = 192;          // keys / queries per (window, head), padded
constexpr int kAHD = 128;         // head width
constexpr int kALd = 136;         // shared-memory row pitch in halves: 272 B, conflict-free for ldmatrix
constexpr int kAPosPad = 16;      // zero rows in front of positional row 0
constexpr int kAPosRows = 400;    // 16 + (2*192 - 1) rounded up to whole 8-row matrices past the last read
constexpr int kAStLd = 88;        // staging tile pitch in floats (rows 0..3 / 4..7 of a 64-bit store land in distinct banks)
constexpr int kAWarps = 12;
constexpr size_t kAKBytes = (size_t)kAT * kALd * 2, kAPBytes = (size_t)kAPosRows * kALd * 2,
                 kAStBytes = (size_t)kAWarps * 16 * kAStLd * 4, kASmem = kAKBytes + kAPBytes + kAStBytes;

__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldsm4(uint32_t (&r)[4], const __half *p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldsm4t(uint32_t (&r)[4], const __half *p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(a));
}
__device__ __forceinline__ uint32_t pack_h2(float x, float y) {
  const __half2 h = __floats2half2_rn(x, y);
  return *(const uint32_t *)&h;
}

// rows [0, nvalid) of src (row stride S floats, 128 columns) -> f16 rows of dst, rows [nvalid, nrows) zero.
// Eight 16-byte loads are in flight per thread before the first conversion: the fill is latency, not bandwidth.
__device__ __forceinline__ void fill_rows_f16(__half *dst, const float *__restrict__ src, int S, int nvalid, int nrows) {
  constexpr int U = 8, NT = kAWarps * 32;
  const int total = nrows * 32;
  for (int base = threadIdx.x; base < total; base += NT * U) {
    float4 v[U];
#pragma unroll
    for (int u = 0; u < U; u++) {
      const int e = base + u * NT, r = e >> 5, c = (e & 31) * 4;
      v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (e < total && r < nvalid) v[u] = __ldg((const float4 *)(src + (size_t)r * S + c));
    }
#pragma unroll
    for (int u = 0; u < U; u++) {
      const int e = base + u * NT, r = e >> 5, c = (e & 31) * 4;
      if (e < total) {
        uint2 o;
        o.x = pack_h2(v[u].x, v[u].y);
        o.y = pack_h2(v[u].z, v[u].w);
        *(uint2 *)(dst + (size_t)r * kALd + c) = o;
      }
    }
  }
}

// The warp's 16 query rows plus a per-head bias vector as an f16 tile [16][kALd] (warp-private): a lane owns four
// columns, eight rows are in flight at a time, every load instruction reads one 512-byte row.
__device__ __forceinline__ void q_tile_f16(__half *dst, const float *__restrict__ qrows, const float *__restrict__ bias,
                                           int S, int nvalid, int lane) {
  const float4 bb = *(const float4 *)(bias + lane * 4);
#pragma unroll
  for (int half = 0; half < 2; half++) {
    float4 x[8];
#pragma unroll
    for (int r = 0; r < 8; r++) {
      x[r] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (half * 8 + r < nvalid) x[r] = __ldg((const float4 *)(qrows + (size_t)(half * 8 + r) * S) + lane);
    }
#pragma unroll
    for (int r = 0; r < 8; r++) {
      uint2 o;
      o.x = pack_h2(x[r].x + bb.x, x[r].y + bb.y);
      o.y = pack_h2(x[r].z + bb.z, x[r].w + bb.w);
      *(uint2 *)(dst + (size_t)(half * 8 + r) * kALd + lane * 4) = o;
    }
  }
}

// The same two moves when the projection arrives as the packed f16 row operand of a product, Xp[col/64][m][col%64]
// (m = row of the [Mrows, *] projection): a row's 128 head columns are two 128-byte runs, so keys and values go to
// shared memory as sixteen asynchronous 16-byte copies per row and the query tile needs one 8-byte load per lane.
__device__ __forceinline__ void fill_rows_packed(__half *dst, const __half *__restrict__ src, int col0, size_t m0, int Mrows,
                                                 int nvalid, int nrows) {
  for (int e = threadIdx.x; e < nrows * 16; e += kAWarps * 32) {
    const int r = e >> 4, ch = e & 15, col = col0 + ch * 8;
    __half *d = dst + (size_t)r * kALd + ch * 8;
    if (r < nvalid) {
      const uint32_t da = (uint32_t)__cvta_generic_to_shared(d);
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(da),
                   "l"(src + ((size_t)(col >> 6) * Mrows + m0 + r) * 64 + (col & 63))
                   : "memory");
    } else {
      *(uint4 *)d = make_uint4(0u, 0u, 0u, 0u);
    }
  }
}
__device__ __forceinline__ void q_tile_packed(__half *dst, const __half *__restrict__ src, int col0, size_t m0, int Mrows,
                                              const float *__restrict__ bias, int nvalid, int lane) {
  const float4 bb = *(const float4 *)(bias + lane * 4);
  const int col = col0 + lane * 4;
  const __half *base = src + ((size_t)(col >> 6) * Mrows + m0) * 64 + (col & 63);
  uint2 x[16];
#pragma unroll
  for (int r = 0; r < 16; r++) x[r] = r < nvalid ? __ldg((const uint2 *)(base + (size_t)r * 64)) : make_uint2(0u, 0u);
#pragma unroll
  for (int r = 0; r < 16; r++) {
    const float2 a = __half22float2(*(const __half2 *)&x[r].x), b = __half22float2(*(const __half2 *)&x[r].y);
    uint2 o;
    o.x = r < nvalid ? pack_h2(a.x + bb.x, a.y + bb.y) : 0u;
    o.y = r < nvalid ? pack_h2(b.x + bb.z, b.y + bb.w) : 0u;
    *(uint2 *)(dst + (size_t)r * kALd + lane * 4) = o;
  }
}

// PACKED: q, k, v are column ranges [0,S), [S,2S), [2S,3S) of ONE projection stored as its packed f16 operand
// (q points at it, k and v are unused, ldq is ignored); otherwise f32 rows ldq floats apart.
template <bool PACKED>
__global__ void __launch_bounds__(kAWarps * 32, 1)
    k_attn_rel(const float *__restrict__ q, const float *__restrict__ k, const float *__restrict__ v,
               const __half *__restrict__ pos16, const float *__restrict__ pbu, const float *__restrict__ pbv,
               float *__restrict__ out, __half *__restrict__ out16, int T, int H, int Mrows, int ldq) {
  fa_grid_dep_sync();
  extern __shared__ __align__(16) unsigned char attn_smem[];
  __half *Ks = (__half *)attn_smem;                              // [192][136]; V after the scores are done
  __half *Ps = (__half *)(attn_smem + kAKBytes);                 // [400][136], positional row p at row p + 16
  float *stage = (float *)(attn_smem + kAKBytes + kAPBytes);     // [12][16][84]
  const int S = H * kAHD, w = blockIdx.x / H, h = blockIdx.x - w * H;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
  const int NP = 2 * T - 1;

  const int i0 = warp * 16, r0 = i0 + g, r1 = r0 + 8;
  const bool ok0 = r0 < T, ok1 = r1 < T;
  const bool active = i0 < T;  // warps whose 16 rows all lie past T only help with the fills and the barriers
  const float *qrows = q + ((size_t)w * T + (active ? i0 : 0)) * ldq + h * kAHD;  // q, k, v rows are ldq floats apart
  const int qvalid = active ? min(16, T - i0) : 0;
  float *st = stage + (size_t)warp * 16 * kAStLd;
  __half *qu_tile = (__half *)st;                               // the staging tile is idle until the positional scores
  __half *qv_tile = Ks + (size_t)warp * 16 * kALd;              // the key rows are idle after the content scores

  const __half *qkv16 = (const __half *)q;
  const size_t mw = (size_t)w * T;
  if (PACKED) {  // the keys first: their copy group is the one the content scores wait for
    fill_rows_packed(Ks, qkv16, S + h * kAHD, mw, Mrows, T, kAT);
    asm volatile("cp.async.commit_group;" ::: "memory");
  }
  // the head's positional rows (already f16) go to shared memory as asynchronous 16-byte copies that nobody waits
  // for until the content scores are done; the zero rows around them are plain stores
  for (int e = threadIdx.x; e < NP * 16; e += kAWarps * 32) {
    const int r = e >> 4, ch = e & 15;
    const uint32_t dst = (uint32_t)__cvta_generic_to_shared(Ps + (size_t)(kAPosPad + r) * kALd + ch * 8);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(pos16 + (size_t)r * S + h * kAHD + ch * 8) : "memory");
  }
  asm volatile("cp.async.commit_group;" ::: "memory");
  for (int e = threadIdx.x; e < (kAPosRows - NP) * 16; e += kAWarps * 32) {
    const int r = e >> 4, ch = e & 15, row = r < kAPosPad ? r : NP + r;
    *(uint4 *)(Ps + (size_t)row * kALd + ch * 8) = make_uint4(0u, 0u, 0u, 0u);
  }
  if (PACKED) {
    if (active) q_tile_packed(qu_tile, qkv16, h * kAHD, mw + i0, Mrows, pbu + h * kAHD, qvalid, lane);
    asm volatile("cp.async.wait_group 1;" ::: "memory");  // the keys have landed, the positional rows may still fly
  } else {
    fill_rows_f16(Ks, k + (size_t)w * T * ldq + h * kAHD, ldq, T, kAT);
    if (active) q_tile_f16(qu_tile, qrows, pbu + h * kAHD, ldq, qvalid, lane);
  }
  __syncthreads();

  // ldmatrix row addresses: lane l names row l%8 of matrix l/8.  B operands: matrices = (n tile 0|1) x (k half 0|1);
  // A operand: matrices = (k half 0|1) x (row half 0|1)
  const int lm_row = (lane & 7) + ((lane >> 4) << 3), lm_col = ((lane >> 3) & 1) << 3;
  const int la_off = ((lane & 7) + (((lane >> 3) & 1) << 3)) * kALd + ((lane >> 4) << 3);

  float s[24][4];
#pragma unroll
  for (int n = 0; n < 24; n++) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;

  // content scores: S = (q + u) K^T, 16 x 192 per warp
  if (active) {
#pragma unroll 2
    for (int ks = 0; ks < 8; ks++) {
      uint32_t a[4];
      ldsm4(a, qu_tile + la_off + ks * 16);
      const __half *kb = Ks + (size_t)lm_row * kALd + ks * 16 + lm_col;
#pragma unroll
      for (int np = 0; np < 12; np++) {
        uint32_t b[4];
        ldsm4(b, kb + (size_t)np * 16 * kALd);
        mma16816(s[2 * np], a, b[0], b[1]);
        mma16816(s[2 * np + 1], a, b[2], b[3]);
      }
    }
  }
  asm volatile("cp.async.wait_all;" ::: "memory");
  __syncthreads();  // every warp is done with the keys (their rows hold the q + v tiles next, V after that) and
                    // everybody's share of the positional rows has landed
  if (active) {
    if (PACKED)
      q_tile_packed(qv_tile, qkv16, h * kAHD, mw + i0, Mrows, pbv + h * kAHD, qvalid, lane);
    else
      q_tile_f16(qv_tile, qrows, pbv + h * kAHD, ldq, qvalid, lane);
    __syncwarp();
  }

  // positional scores, one 64-key block at a time: the 80 positions p_lo .. p_lo+79 with
  // p_lo = T - 16 - i0 + j0 cover bd[i][T-1-i+j] for the warp's 16 rows and the block's 64 keys
  if (active) {
#pragma unroll  // (unrolled so that s[] is indexed statically and stays in registers)
    for (int jb = 0; jb < 3; jb++) {
      float c[10][4];
#pragma unroll
      for (int n = 0; n < 10; n++) c[n][0] = c[n][1] = c[n][2] = c[n][3] = 0.f;
      const __half *pb = Ps + (size_t)(T - i0 + jb * 64 + lm_row) * kALd + lm_col;  // row (p_lo + 16) + ...
#pragma unroll 2
      for (int ks = 0; ks < 8; ks++) {
        uint32_t a[4];
        ldsm4(a, qv_tile + la_off + ks * 16);
#pragma unroll
        for (int np = 0; np < 5; np++) {
          uint32_t b[4];
          ldsm4(b, pb + (size_t)np * 16 * kALd + ks * 16);
          mma16816(c[2 * np], a, b[0], b[1]);
          mma16816(c[2 * np + 1], a, b[2], b[3]);
        }
      }
#pragma unroll
      for (int n = 0; n < 10; n++) {
        *(float2 *)(st + g * kAStLd + 8 * n + 2 * t) = make_float2(c[n][0], c[n][1]);
        *(float2 *)(st + (g + 8) * kAStLd + 8 * n + 2 * t) = make_float2(c[n][2], c[n][3]);
      }
      __syncwarp();
      const float *s0 = st + g * kAStLd + 15 - g + 2 * t, *s1 = st + (g + 8) * kAStLd + 7 - g + 2 * t;
#pragma unroll
      for (int n = 0; n < 8; n++) {
        float(&d)[4] = s[jb * 8 + n];
        d[0] += s0[8 * n];
        d[1] += s0[8 * n + 1];
        d[2] += s1[8 * n];
        d[3] += s1[8 * n + 1];
      }
      __syncwarp();
    }
  }

  // softmax over the keys (columns j >= T masked), rows r0 and r1 of this thread's quad
  uint32_t pf[12][4];
  if (active) {
    float m0 = -INFINITY, m1 = -INFINITY;
#pragma unroll
    for (int n = 0; n < 24; n++) {
      const int j = 8 * n + 2 * t;
      if (j >= T) s[n][0] = s[n][2] = -INFINITY;
      if (j + 1 >= T) s[n][1] = s[n][3] = -INFINITY;
      m0 = fmaxf(m0, fmaxf(s[n][0], s[n][1]));
      m1 = fmaxf(m1, fmaxf(s[n][2], s[n][3]));
    }
    m0 = fmaxf(m0, __shfl_xor_sync(0xffffffffu, m0, 1));
    m0 = fmaxf(m0, __shfl_xor_sync(0xffffffffu, m0, 2));
    m1 = fmaxf(m1, __shfl_xor_sync(0xffffffffu, m1, 1));
    m1 = fmaxf(m1, __shfl_xor_sync(0xffffffffu, m1, 2));
    float z0 = 0.f, z1 = 0.f;
#pragma unroll
    for (int n = 0; n < 24; n++) {
      s[n][0] = __expf(s[n][0] - m0);
      s[n][1] = __expf(s[n][1] - m0);
      s[n][2] = __expf(s[n][2] - m1);
      s[n][3] = __expf(s[n][3] - m1);
      z0 += s[n][0] + s[n][1];
      z1 += s[n][2] + s[n][3];
    }
    z0 += __shfl_xor_sync(0xffffffffu, z0, 1);
    z0 += __shfl_xor_sync(0xffffffffu, z0, 2);
    z1 += __shfl_xor_sync(0xffffffffu, z1, 1);
    z1 += __shfl_xor_sync(0xffffffffu, z1, 2);
    const float inv0 = 1.0f / z0, inv1 = 1.0f / z1;
#pragma unroll
    for (int kk = 0; kk < 12; kk++) {
      pf[kk][0] = pack_h2(s[2 * kk][0] * inv0, s[2 * kk][1] * inv0);
      pf[kk][1] = pack_h2(s[2 * kk][2] * inv1, s[2 * kk][3] * inv1);
      pf[kk][2] = pack_h2(s[2 * kk + 1][0] * inv0, s[2 * kk + 1][1] * inv0);
      pf[kk][3] = pack_h2(s[2 * kk + 1][2] * inv1, s[2 * kk + 1][3] * inv1);
    }
  }
  __syncthreads();  // every warp is done with its q + v tile
  if (PACKED) {
    fill_rows_packed(Ks, qkv16, 2 * S + h * kAHD, mw, Mrows, T, kAT);
    asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_all;" ::: "memory");
  } else {
    fill_rows_f16(Ks, v + (size_t)w * T * ldq + h * kAHD, ldq, T, kAT);
  }
  __syncthreads();  // V is in place
  if (!active) return;

  // out = P V: 16 x 128 per warp
  float o[16][4];
#pragma unroll
  for (int n = 0; n < 16; n++) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
  {
    // transposed loads: matrices = (key half 0|1) x (n tile 0|1)
    const __half *vb = Ks + (size_t)((lane & 7) + (((lane >> 3) & 1) << 3)) * kALd + ((lane >> 4) << 3);
#pragma unroll
    for (int kk = 0; kk < 12; kk++) {
#pragma unroll
      for (int np = 0; np < 8; np++) {
        uint32_t b[4];
        ldsm4t(b, vb + (size_t)kk * 16 * kALd + np * 16);
        mma16816(o[2 * np], pf[kk], b[0], b[1]);
        mma16816(o[2 * np + 1], pf[kk], b[2], b[3]);
      }
    }
  }
  const size_t m0 = (size_t)w * T + r0, m1 = (size_t)w * T + r1;
#pragma unroll
  for (int n = 0; n < 16; n++) {
    const int col = h * kAHD + 8 * n + 2 * t;
    if (out) {
      if (ok0) *(float2 *)(out + m0 * S + col) = make_float2(o[n][0], o[n][1]);
      if (ok1) *(float2 *)(out + m1 * S + col) = make_float2(o[n][2], o[n][3]);
    }
    if (out16) {
      __half *d = out16 + (size_t)(col >> 6) * Mrows * 64 + (col & 63);
      if (ok0) *(__half2 *)(d + m0 * 64) = __floats2half2_rn(o[n][0], o[n][1]);
      if (ok1) *(__half2 *)(d + m1 * 64) = __floats2half2_rn(o[n][2], o[n][3]);
    }
  }
}

struct Block {  // pool block released at scope exit
  fa_ctx *ctx;
  void *p = nullptr;
  size_t bytes = 0;
  explicit Block(fa_ctx *c) : ctx(c) {}
  int get(size_t need) { return fa_block_acquire(ctx, need, &p, &bytes); }
  ~Block() {
    if (p) fa_block_release(ctx, p);
  }
};

__global__ void k_f32_to_f16(const float *__restrict__ x, __half *__restrict__ y, size_t n4) {
  fa_grid_dep_sync();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x) {
    const float4 v = ((const float4 *)x)[i];
    uint2 o;
    o.x = pack_h2(v.x, v.y);
    o.y = pack_h2(v.z, v.w);
    ((uint2 *)y)[i] = o;
  }
}

}  // namespace

bool fa_attn_rel_shape_ok(int T, int H, int HD, int W) {
  return HD == kAHD && T >= 16 && T <= kAT && H >= 1 && W >= 1 && (long long)W * H <= 0x7fffffffll;
}

// out (f32 [W*T, H*HD]) may be NULL when out16 (the packed f16 row operand of the projection that follows) is given.
// q, k, v: rows ldq floats apart (H*HD for separate projections, 3*H*HD for the columns of one fused projection);
// ldq == 0: q is the packed f16 row operand Xp[col/64][m][col%64] of the fused [W*T, 3*H*HD] projection (k, v unused).
// pos_cache (may be NULL): the tensor behind `pos`; its f16 copy is kept on it across calls (the projected positional
// table of a layer is the same every step) unless the call is being recorded.
int fa_attn_rel(fa_ctx *ctx, const float *q, const float *k, const float *v, const float *pos, fa_tensor *pos_cache,
                const float *pbu, const float *pbv, float *out, __half *out16, int T, int H, int HD, int W, int ldq) {
  FA_REQUIRE(ctx, fa_attn_rel_shape_ok(T, H, HD, W) && (out || out16), "attnFused: shape outside the one-kernel form");
  FA_REQUIRE(ctx, ldq == 0 || (ldq >= H * HD && (ldq & 3) == 0 && ((((uintptr_t)q | (uintptr_t)k | (uintptr_t)v)) & 15) == 0),
             "attnFused: q/k/v rows must be 16-byte aligned");
  static bool attr_set[64] = {false};
  if (!attr_set[ctx->device & 63]) {
    FA_CHECK_CUDA(ctx, cudaFuncSetAttribute(k_attn_rel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kASmem));
    FA_CHECK_CUDA(ctx, cudaFuncSetAttribute(k_attn_rel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kASmem));
    attr_set[ctx->device & 63] = true;
  }
  const int NP = 2 * T - 1, S = H * HD;
  const size_t halves = (size_t)NP * S;
  Block tmp(ctx);
  const __half *pos16 = nullptr;
  const bool cacheable = pos_cache && !pos_cache->view;
  if (cacheable && pos_cache->hk16_valid && pos_cache->hk_kind == 1 && pos_cache->hk_Tb == NP && pos_cache->hk_H == H &&
      pos_cache->hk_HD == HD) {
    pos16 = (const __half *)pos_cache->hk16;
  } else {
    __half *dst = nullptr;
    if (cacheable && !ctx->capturing) {  // (a block taken while recording belongs to the recording)
      if (pos_cache->hk16 && pos_cache->hk16_bytes < halves * 2) {
        fa_block_release(ctx, pos_cache->hk16);
        pos_cache->hk16 = nullptr;
      }
      if (!pos_cache->hk16) FA_TRY(fa_block_acquire(ctx, halves * 2, &pos_cache->hk16, &pos_cache->hk16_bytes));
      pos_cache->hk_kind = 1, pos_cache->hk_Tb = NP, pos_cache->hk_H = H, pos_cache->hk_HD = HD;
      pos_cache->hk16_valid = true;
      dst = (__half *)pos_cache->hk16;
    } else {
      FA_TRY(tmp.get(halves * 2));
      dst = (__half *)tmp.p;
    }
    {
      LaunchScope ls(ctx, "attn_pos_f16");
      const size_t n4 = halves / 4;
      size_t gsz = (n4 + 255) / 256, cap = (size_t)ctx->sm_count * 8;
      fa_launch_dep(ctx, k_f32_to_f16, dim3((unsigned)(gsz < cap ? gsz : cap)), dim3(256), 0, pos, dst, n4);
    }
    FA_LAUNCH_CHECK(ctx, "attn_pos_f16");
    pos16 = dst;
  }
  {
    LaunchScope ls(ctx, "attn_rel");
    if (ldq == 0)  // q is the packed f16 operand of the fused q|k|v projection
      fa_launch_dep(ctx, k_attn_rel<true>, dim3((unsigned)(W * H)), dim3(kAWarps * 32), kASmem, q, k, v, pos16, pbu, pbv, out,
                    out16, T, H, W * T, ldq);
    else
      fa_launch_dep(ctx, k_attn_rel<false>, dim3((unsigned)(W * H)), dim3(kAWarps * 32), kASmem, q, k, v, pos16, pbu, pbv, out,
                    out16, T, H, W * T, ldq);
  }
  FA_LAUNCH_CHECK(ctx, "attn_rel");
  return FA_OK;
}
