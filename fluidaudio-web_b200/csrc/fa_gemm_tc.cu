// tcgen05 GEMM for the f16-weight, int8-weight and int4-weight products (sm_100a).
//
// Replaces the reference's WGSL GEMM family for large shapes: f16-storage B
// (src/gpu/kernels/gemm.js:336-419, 420-503), int8 B (gemm.js:679-885) and int4 B (gemm.js:893-919).
//
// One orientation for every shape: the WEIGHTS are the MMA M-side operand (128 output columns
// n per CTA, one TMEM lane each), the ACTIVATIONS are the MMA N-side operand (MT rows m per CTA,
// one TMEM column each).  Operands are brought in by TMA (128-byte swizzle, no multicast) through
// a multi-stage mbarrier ring, multiplied by tcgen05.mma (kind::f16 -> f32, kind::i8 -> s32) into
// TMEM, and read back with tcgen05.ld by eight epilogue warps that apply
//   acc (*rowscale[m]) (*colscale[n]) + bias[n] -> act -> + add[m,n]
// and store out[m][n] so that the 32 lanes of a warp write 32 consecutive n (coalesced rows).
// The kernel is persistent (one CTA per SM walks the tiles) with two TMEM accumulator buffers, so a
// tile's epilogue overlaps the next tile's main loop.  Products with fewer tiles than SMs and at most
// 128 rows split K over a cluster of up to 8 CTAs and reduce over distributed shared memory.
//
// Operand layout in HBM ("box-contiguous"): every TMA box is one contiguous run of memory, so a
// CTA streams its weights as a single linear region instead of 128-byte pieces a row pitch apart
// (which opens a new DRAM page per piece).  With ck = elements per 128 bytes of K:
//   weights     Wp[n/128][k/ck][n%128][k%ck]            (one-time repack, cached on the handle)
//   activations Ap[plane][k/ck][m][k%ck]                 (prepass, or written by the producing kernel)
// The reference itself prepacks weights tile-major for its fastest GEMM (compute.js:224-243).
//
// int8 activations arrive as `limbs` int8 digit planes (see fa_prep_a_i8): plane l is stacked as
// MT extra MMA-N rows, so ONE instruction stream produces all digit products, each an exact int32
// sum in its own TMEM column range; the epilogue recombines them as sum_l acc_l * 2^(-7 l).
// f16 activations of few-row products arrive as two planes, value and rounding residue, accumulated
// into the SAME TMEM columns (f32-grade activations where the weight stream is the cost anyway).
//
// Warp roles (352 threads): warp 0 = TMA producer of the weight tiles, warp 1 = TMEM owner + MMA issuer,
// warps 2..9 = epilogue (TMEM lane quadrant = warp_id % 4, two warps per quadrant), warp 10 = TMA producer of the
// activation tiles.  Shapes with more tiles than SMs run as k_tc_gemm_pair: two CTAs of a cluster share one
// 256-lane MMA (cta_group::2) and each loads half of the activation rows of the pair's tile.
#include <type_traits>

#include "fa_tc_common.cuh"

namespace {

using namespace tc;

constexpr int kEpiWarps = 8;                   // two per TMEM lane quadrant (one per quadrant leaves the MMA and
                                               // producer warps more issue slots - later tiles ran ~15 % faster - but
                                               // doubles the epilogue's own time, and the encoder step got 20 % slower)
constexpr int kThreads = 96 + 32 * kEpiWarps;  // warp 0 weights producer, warp 1 MMA, warps 2..9 epilogue, warp 10
                                               // activations producer.  ONE thread sustains a tile load only every
                                               // ~300-400 clocks whatever the tile's size (measured: 407 clocks per
                                               // load per issuing thread for 4 KB..16 KB tiles, four threads four times
                                               // the loads), so a K chunk's two loads from one thread paced the whole
                                               // pipeline at ~650 clocks per chunk against 448-512 for its MMAs
constexpr int kRowBytes = 128;                 // one swizzle atom of K per stage
constexpr int kPTileBytes = 128 * kRowBytes;   // weights tile: 128 rows
// int4 variant: 8 more warps unpack nibbles into the f16 weights tile.  They sit on the warp ids above the epilogue
// warps whose id has bit 1 set (10,11,14,15,18,19,22,23; the ids between have no role and park at the closing barrier): with warps dealt to the four schedulers round-robin, that keeps the busy
// unpack warps off the schedulers of warp 0 (TMA producer) and warp 1 (MMA issuer), whose single-lane loops
// otherwise get every third issue slot and set the pace of the whole pipeline (measured: ~550 ns per K chunk).
constexpr int kDeqWarps = 8;
constexpr int kThreadsNbits = 32 * (2 + kEpiWarps + 2 * kDeqWarps - 2);
constexpr int kRawTileBytes = 128 * 32;        // int4 variant: 128 rows x 64 nibbles of one K chunk, as uploaded
// int8-weight variant with f16 activations (KIND 5): 128 rows x 64 int8 of one K chunk; two groups of four warps (the
// warp ids of the int4 variant's unpack warps) take alternate chunks and turn them into the f16 weights tile
constexpr int kRaw8TileBytes = 128 * 64;
constexpr int kThreadsI8W = kThreadsNbits;
template <int KIND>
__host__ __device__ constexpr int tc_threads() { return KIND == 2 ? kThreadsNbits : (KIND == 5 ? kThreadsI8W : kThreads); }
template <int KIND>
__host__ __device__ constexpr int tc_raw_bytes() { return KIND == 2 ? kRawTileBytes : 0; }  // (KIND 5 lands its raw tile inside the weights tile)
constexpr int kSlabsMax = 4;                    // store slabs per epilogue warp and result kind (TcParams::nslab = 2 or 4): a
                                                // slab is refilled only when the copy engine has read it, and the engine takes
                                                // the stores in turn with the tile loads queued ahead of them; four are used
                                                // when they do not cost the ring a stage (+1-2 %)
constexpr int kSplitMaxMT = 128;               // split-K mode keeps a [MT][128] f32 partial tile in smem

struct TcParams {
  int M, N, K;        // logical sizes; K in elements
  int MT;             // activation rows per tile (multiple of 16, MT*limbs <= 256)
  int limbs;          // activation digit planes (1 for f16)
  int limb_sum;       // f16 kind, limbs == 2: plane 1 holds the f16 rounding residue of plane 0 and both are
                      // accumulated into the SAME TMEM columns (f32-grade activations for decode-size products)
  int stages;
  int num_kb;         // K chunks of 128 bytes
  int tiles_n, tiles_m;
  int splitk;         // > 1: cluster of `splitk` CTAs along z shares one tile, each taking kb_per_split chunks
  int kb_per_split;
  int split_rb;       // split-K: 16-row blocks of a tile each CTA of the cluster owns, ceil(MT / 16 / splitk)
  int raw_i32;        // 1: store the limb-0 int32 accumulators instead of the float epilogue
  // batched mode (attention products): `batches` independent [M][N] problems share one launch.  Batch b
  // reads weight slab (w_batch_mod ? b % w_batch_mod : b) and activation slabs of batch b, and writes at
  // out + (b / o_div) * o_hi + (b % o_div) * o_lo with row pitch ldc.
  int batches, w_batch_mod, o_div, ldc;
  int a_shared;       // batched mode: every batch multiplies the same activation slabs
  long long o_hi, o_lo;
  __half *out16;      // optional packed f16 shadow of the result (see TcEpilogue), or nullptr
  int skip_f32;       // with out16: the f32 result is not stored at all (fa_tensor::f32_lazy)
  int o16_rows, o16_row_hi, o16_col_lo;
  float *out;         // [M][N] f32 (or int32 when raw_i32)
  // N-sharded products: besides `out`, every finished tile is also stored at the same [row][column] of up to 7
  // more result buffers - the other GPUs' copies of the full product, reached by plain stores over NVLink
  // (peer pointers), so the all-gather of output columns happens inside the epilogue, tile by tile.
  float *peer_out[7];
  int n_peers;
  const float *rowscale, *colscale, *bias, *add, *rowbias;
  int act;
  // int4 variant (KIND 2): block-major scales [nblk][N] and zero-points [nblk][N] (one per byte)
  const float *nb_scales;
  const uint8_t *nb_zp;
  int nblk;
  int w_lo_rows;        // KIND 4: row offset of the weights' residue plane in the weight map
  int *status;
  int tma_out;          // 1: results leave through shared-memory slabs and TMA stores (see epilogue_tile)
  uint32_t slab_f16_off;  // byte offset of the f16 slabs behind the f32 slabs (0 when no f32 result is stored)
  int nslab;              // store slabs per epilogue warp and result kind: 2 or 4
  int tma_add;            // 1: the residual operand comes in through the copy engine, block by block, into residual slabs
                          // behind the store slabs (see epilogue_tile_resadd); needs tma_out and an f32 result
  uint32_t slab_res_off;  // byte offset of the residual slabs from the first store slab
  uint32_t wait_limit;  // polls before a barrier wait gives up (fa_ctx::wait_limit)
  int withhold_kb;      // >= 0: CTA 0 never loads this K chunk of its first tile, so the waits downstream of it run
                        // out (the way the bounded-wait path is tested without faulting the GPU); -1 in normal use
};

__device__ __forceinline__ void report_timeout(int *status, int code, int detail) {
  if (atomicCAS(status, 0, code) == 0) {
    status[1] = (int)blockIdx.x;
    status[2] = detail;
  }
}

__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_arrive_all() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait_all() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }

// Activation applied to 16 values at once with the selector outside the loop, so the 16 chains stay
// independent (one warp per scheduler has no other work to hide a per-element branch behind).
__device__ __forceinline__ void act16(float (&v)[16], int act) {
  switch (act) {
    case FA_ACT_NONE: break;
    case FA_ACT_RELU:
#pragma unroll
      for (int j = 0; j < 16; j++) v[j] = fmaxf(v[j], 0.0f);
      break;
    case FA_ACT_SILU:
#pragma unroll
      // one tanh.approx per element (fa_silu_fast).  The IEEE-division form made the SiLU products epilogue-bound
      // (84 us against 53 us for the same product without activation); ex2.approx + rcp.approx still cost 8 us of
      // special-function time per product.
      for (int j = 0; j < 16; j++) v[j] = fa_silu_fast(v[j]);
      break;
    default:
#pragma unroll
      for (int j = 0; j < 16; j++) v[j] = fa_actf(v[j], act);
  }
}

// One tile's epilogue for one warp: TMEM lanes [32*quad, 32*quad+32) = output columns n0 + 32*quad + lane,
// column chunks c = 16*half, 16*half + 32, ... = output rows m0 + c .. m0 + c + 15.
//
// Where results go.  Plain products (one batch, no peer buffers, no K split) stage every 16-row x 32-column block
// in a slab of shared memory owned by the warp - lane = column, so the 32 lanes of a store instruction fill one
// 128-byte row and no bank is hit twice - and one lane hands the slab to the copy engine (cp.async.bulk.tensor
// store: rows and columns past the edge of the tensor are clipped by the engine).  The epilogue warps then never
// wait on the global store path: with per-lane st.global a 128 x 224 tile spent 1.7 us of its 8.6 us there,
// next to a 6 us main loop.  Two slabs per warp and per result kind alternate; before a slab is refilled the
// issuing lane waits until the store that last used it has finished reading it.  The other modes (batched
// attention products, peer stores, raw int32, ragged row pitches) keep the direct stores.
template <int KIND, bool PEERS = false>
__device__ __forceinline__ void epilogue_tile(const TcParams &p, uint32_t lane_addr, int n0, int m0, int quad, int lane,
                                              int half, float *outb, int r16, int c16, uint32_t partial,
                                              const CUtensorMap *map_o, const CUtensorMap *map_o16, uint32_t slab_f32,
                                              uint32_t slab_f16, uint32_t &slab_turn, uint32_t cl_rank) {
  const int n = n0 + quad * 32 + lane;
  const bool n_ok = n < p.N;
  const float cs = (p.colscale && n_ok) ? p.colscale[n] : 1.0f;
  const float bs = (p.bias && n_ok) ? p.bias[n] : 0.0f;
  for (int c = half * 16; c < p.MT; c += 4 * kEpiWarps) {
    if (m0 + c >= p.M) break;  // warp-uniform: no rows left in this tile
    uint32_t v0[16], v1[16], v2[16];
    tmem_ld16(lane_addr + (uint32_t)c, v0);
    if (KIND == 1 && p.limbs > 1) tmem_ld16(lane_addr + (uint32_t)(p.MT + c), v1);
    if (KIND == 1 && p.limbs > 2) tmem_ld16(lane_addr + (uint32_t)(2 * p.MT + c), v2);
    const bool full_rows = m0 + c + 16 <= p.M;
    // independent loads issued together while the TMEM read is in flight
    float rs[16], ad[16];
    if (p.rowscale) {
      if (full_rows) {
        const float4 *r4 = (const float4 *)(p.rowscale + m0 + c);
#pragma unroll
        for (int j = 0; j < 4; j++) {
          float4 t = __ldg(r4 + j);
          rs[4 * j] = t.x; rs[4 * j + 1] = t.y; rs[4 * j + 2] = t.z; rs[4 * j + 3] = t.w;
        }
      } else {
#pragma unroll
        for (int j = 0; j < 16; j++) rs[j] = __ldg(p.rowscale + min(m0 + c + j, p.M - 1));
      }
    } else {
#pragma unroll
      for (int j = 0; j < 16; j++) rs[j] = 1.0f;
    }
    if (p.add && n_ok && p.splitk <= 1) {
      const float *arow = p.add + (size_t)(m0 + c) * p.N + n;
      if (full_rows) {  // one base address, constant row stride: no per-row clamp and 64-bit multiply
#pragma unroll
        for (int j = 0; j < 16; j++) ad[j] = __ldg(arow + (size_t)j * p.N);
      } else {
#pragma unroll
        for (int j = 0; j < 16; j++) ad[j] = m0 + c + j < p.M ? __ldg(arow + (size_t)j * p.N) : 0.0f;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 16; j++) ad[j] = 0.0f;
    }
    float rb[16];  // per-row bias (the output-channel bias of a pointwise convolution run as a GEMM)
    if (p.rowbias) {
#pragma unroll
      for (int j = 0; j < 16; j++) rb[j] = __ldg(p.rowbias + min(m0 + c + j, p.M - 1));
    } else {
#pragma unroll
      for (int j = 0; j < 16; j++) rb[j] = 0.0f;
    }
    tmem_ld_wait();
    if (KIND == 1 && p.raw_i32 == 1) {
      if (n_ok) {
#pragma unroll
        for (int j = 0; j < 16; j++)
          if (m0 + c + j < p.M) ((int32_t *)outb)[(size_t)(m0 + c + j) * p.ldc + n] = (int32_t)v0[j];
      }
      continue;
    }
    float v[16];
#pragma unroll
    for (int j = 0; j < 16; j++) {
      if (KIND != 1) {
        v[j] = __uint_as_float(v0[j]);
      } else {
        v[j] = (float)(int32_t)v0[j];
        if (p.limbs > 1) v[j] = fmaf((float)(int32_t)v1[j], 1.0f / 128.0f, v[j]);
        if (p.limbs > 2) v[j] = fmaf((float)(int32_t)v2[j], 1.0f / 16384.0f, v[j]);
      }
    }
    if (p.splitk > 1) {
      // K split over a cluster: 16-row blocks of the tile are dealt to the CTAs of the cluster in turn; this CTA's
      // partial sums of a block go straight into the OWNER's shared memory (remote stores, nothing waits on them),
      // slot [source rank][owned block][row][column]: lanes write consecutive addresses.
      const uint32_t blk = (uint32_t)c >> 4, owner = blk % (uint32_t)p.splitk, ob = blk / (uint32_t)p.splitk;
      const uint32_t local = partial + ((((cl_rank * (uint32_t)p.split_rb + ob) * 16u) * 128u + (uint32_t)(quad * 32 + lane)) * 4u);
      uint32_t remote;
      asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(owner));
#pragma unroll
      for (int j = 0; j < 16; j++)
        asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote + (uint32_t)(j * 128 * 4)), "f"(v[j]) : "memory");
      continue;
    }
#pragma unroll
    for (int j = 0; j < 16; j++) v[j] = fmaf(v[j] * rs[j], cs, bs) + rb[j];
    act16(v, p.act);
    if (!PEERS && p.tma_out) {
      const uint32_t b = slab_turn & (uint32_t)(p.nslab - 1);
      slab_turn++;
      if (p.nslab == 4) tma_store_wait_read<3>(); else tma_store_wait_read<1>();  // lane 0: the group that last used slab b has read it (the other lanes own no groups)
      __syncwarp();
      if (p.out16) {
        const uint32_t dst = slab_f16 + b * 1024u + (uint32_t)lane * 2u;
#pragma unroll
        for (int j = 0; j < 16; j++)
          asm volatile("st.shared.b16 [%0], %1;" ::"r"(dst + (uint32_t)j * 64u), "h"(__half_as_ushort(__float2half_rn(v[j] + ad[j])))
                       : "memory");
      }
      if (!p.skip_f32) {
        const uint32_t dst = slab_f32 + b * 2048u + (uint32_t)lane * 4u;
#pragma unroll
        for (int j = 0; j < 16; j++)
          asm volatile("st.shared.f32 [%0], %1;" ::"r"(dst + (uint32_t)j * 128u), "f"(v[j] + ad[j]) : "memory");
      }
      fence_proxy_async_smem();  // the copy engine reads the slab through the async proxy
      __syncwarp();
      {
        const uint32_t lead = lane == 0 ? 1u : 0u;
        const int gn = n0 + quad * 32 + c16;
        if (p.out16) tma_store_3d_w(lead, map_o16, slab_f16 + b * 1024u, gn & 63, r16 + m0 + c, gn >> 6);
        if (!p.skip_f32) tma_store_2d_w(lead, map_o, slab_f32 + b * 2048u, n0 + quad * 32, m0 + c);
        tma_store_commit();
      }
      continue;
    }
    if (n_ok) {
      if (p.out16) {  // shadow: Ap[k/64][row][k%64] of the output tensor, 32 lanes = 64 contiguous bytes
        const int gn = n + c16;
        __half *h16 = p.out16 + ((size_t)(gn >> 6) * p.o16_rows + (r16 + m0 + c)) * 64 + (gn & 63);
#pragma unroll
        for (int j = 0; j < 16; j++)
          if (full_rows || m0 + c + j < p.M) h16[(size_t)j * 64] = __float2half_rn(v[j] + ad[j]);
      }
      float *orow = outb + (size_t)(m0 + c) * p.ldc + n;
      if (p.skip_f32) {
        // hidden-layer result: the shadow above is all the next product reads
      } else if (full_rows) {
#pragma unroll
        for (int j = 0; j < 16; j++) orow[(size_t)j * p.ldc] = v[j] + ad[j];
      } else {
#pragma unroll
        for (int j = 0; j < 16; j++)
          if (m0 + c + j < p.M) orow[(size_t)j * p.ldc] = v[j] + ad[j];
      }
      if (PEERS)
      for (int pi = 0; pi < p.n_peers; pi++) {  // the same tile into the peers' result buffers (batches == 1)
        float *prow = p.peer_out[pi] + (size_t)(m0 + c) * p.ldc + n;
#pragma unroll
        for (int j = 0; j < 16; j++)
          if (full_rows || m0 + c + j < p.M) prow[(size_t)j * p.ldc] = v[j] + ad[j];
      }
    }
  }
}

// The fast epilogue below for a launch with a residual operand, with the residual brought in by the copy engine: the
// [16][32] f32 block a warp is going to add is loaded (TMA, one mbarrier per slab) two blocks ahead into one of three
// residual slabs of the warp, and read from shared memory when its turn comes.  As plain loads the residual cost a
// product with K = 1024 four microseconds of nineteen: sixteen global loads of dependent latency per block in warps
// that are paced by their own instruction count, where a block now costs sixteen shared-memory reads (19.1 -> 17.4 us
// at M = 6016, N = K = 1024; 60.4 -> 57.0 at N = 4096).  The loads share the copy engine's ingest with the operand
// tiles, which is what paces the main loop: a residual tile is 20 % of a tile's operand bytes at K = 1024 and 5 % at
// K = 4096, where the exchange no longer pays (43.9 -> 44.2 us) - the launch uses this path up to K = 2048.  One block
// of look-ahead (two slabs) gave 18.4 us: the look-ahead is latency cover, not the ring's depth.
constexpr int kResSlabs = 3;
__device__ __forceinline__ void epilogue_tile_resadd(const TcParams &p, uint32_t lane_addr, int n0, int m0, int quad, int lane,
                                                     int half, int r16, int c16, const CUtensorMap *map_o,
                                                     const CUtensorMap *map_o16, const CUtensorMap *map_add, uint32_t slab_f32,
                                                     uint32_t slab_f16, uint32_t slab_res, uint32_t res_bar0, uint32_t &slab_turn,
                                                     uint32_t &res_turn) {
  const int n = n0 + quad * 32 + lane;
  const bool n_ok = n < p.N;
  const float cs = (p.colscale && n_ok) ? p.colscale[n] : 1.0f;
  const float bs = (p.bias && n_ok) ? p.bias[n] : 0.0f;
  constexpr int kStep = 4 * kEpiWarps;  // rows between a warp's consecutive blocks
  int c = half * 16;
  if (c >= p.MT || m0 + c >= p.M) return;
  auto has = [&](int cc) { return cc < p.MT && m0 + cc < p.M; };

  // residual rows m0+cc .. +15 of this warp's 32 columns into the residual slab of turn t (its last reader was turn
  // t - 3, whose reads ended before that turn's stores were issued)
  auto res_issue = [&](int cc, uint32_t t) {
    if (lane == 0) {
      const uint32_t b = t % kResSlabs, bar = res_bar0 + b * 8u;
      mbar_expect_tx(bar, 2048u);
      tma_load_2d(slab_res + b * 2048u, map_add, n0 + quad * 32, m0 + cc, bar);
    }
  };
  auto finish = [&](int cc, const uint32_t (&vr)[16], uint32_t t) {
    float v[16];
#pragma unroll
    for (int j = 0; j < 16; j++) v[j] = fmaf(__uint_as_float(vr[j]), cs, bs);
    act16(v, p.act);
    const uint32_t rb = t % kResSlabs;
    if (!mbar_wait(res_bar0 + rb * 8u, (t / kResSlabs) & 1u, p.wait_limit) && lane == 0) report_timeout(p.status, 9, cc);
    {
      const uint32_t src = slab_res + rb * 2048u + (uint32_t)lane * 4u;
#pragma unroll
      for (int j = 0; j < 16; j++) {
        float r;
        asm volatile("ld.shared.f32 %0, [%1];" : "=f"(r) : "r"(src + (uint32_t)j * 128u) : "memory");
        v[j] += r;
      }
    }
    const uint32_t b = slab_turn & (uint32_t)(p.nslab - 1);
    slab_turn++;
    if (p.nslab == 4) tma_store_wait_read<3>(); else tma_store_wait_read<1>();  // lane 0 owns the groups
    __syncwarp();
    if (p.out16) {
      const uint32_t d16 = slab_f16 + b * 1024u + (uint32_t)lane * 2u;
#pragma unroll
      for (int j = 0; j < 16; j++)
        asm volatile("st.shared.b16 [%0], %1;" ::"r"(d16 + (uint32_t)j * 64u), "h"(__half_as_ushort(__float2half_rn(v[j]))) : "memory");
    }
    {
      const uint32_t dst = slab_f32 + b * 2048u + (uint32_t)lane * 4u;
#pragma unroll
      for (int j = 0; j < 16; j++) asm volatile("st.shared.f32 [%0], %1;" ::"r"(dst + (uint32_t)j * 128u), "f"(v[j]) : "memory");
    }
    fence_proxy_async_smem();
    __syncwarp();
    {
      const uint32_t lead = lane == 0 ? 1u : 0u;
      const int gn = n0 + quad * 32 + c16;
      if (p.out16) tma_store_3d_w(lead, map_o16, slab_f16 + b * 1024u, gn & 63, r16 + m0 + cc, gn >> 6);
      tma_store_2d_w(lead, map_o, slab_f32 + b * 2048u, n0 + quad * 32, m0 + cc);
      tma_store_commit();
    }
  };

  uint32_t va[16], vb[16];
  uint32_t turn = res_turn;
  constexpr int kAhead = kResSlabs - 1;  // blocks a residual load is issued ahead of its use
#pragma unroll
  for (int i = 0; i < kAhead; i++)
    if (has(c + i * kStep)) res_issue(c + i * kStep, turn + (uint32_t)i);
  tmem_ld16(lane_addr + (uint32_t)c, va);
  for (;;) {
    tmem_ld_wait();
    int cn = c + kStep;
    bool more = has(cn);
    if (more) tmem_ld16(lane_addr + (uint32_t)cn, vb);
    if (has(c + kAhead * kStep)) res_issue(c + kAhead * kStep, turn + kAhead);
    finish(c, va, turn);
    turn++;
    if (!more) break;
    c = cn;
    tmem_ld_wait();
    cn = c + kStep;
    more = has(cn);
    if (more) tmem_ld16(lane_addr + (uint32_t)cn, va);
    if (has(c + kAhead * kStep)) res_issue(c + kAhead * kStep, turn + kAhead);
    finish(c, vb, turn);
    turn++;
    if (!more) break;
    c = cn;
  }
  res_turn = turn;
}

// The same epilogue for the common case (float accumulators, one output per accumulator, no row scale / row bias, no
// K split), software-pipelined: the TMEM read and the residual loads of a warp's NEXT 16-row block are issued before
// the current block is finished, so their latencies (a few hundred cycles for the TMEM read, an L2 round trip for the
// residual) overlap the arithmetic and stores of the current block instead of adding up block after block.  With
// K = 1024 a tile's epilogue (28 blocks of 16 x 32 values per warp pair) was longer than its main loop: the warps
// spent most of it waiting on one load at a time.
// ADD: the launch has a residual operand.  The epilogue is paced by its own instruction count (two warps per
// scheduler, dependent chains), so the variant without a residual carries no registers, loads or adds for one:
// +2..5 % on the products without residual.  (Fixing the result kinds and the activation at compile time as well
// made the register allocator of the whole kernel spill and cost more than it saved.)
template <bool PEERS, bool ADD>
__device__ __forceinline__ void epilogue_tile_fast(const TcParams &p, uint32_t lane_addr, int n0, int m0, int quad, int lane,
                                                   int half, float *outb, int r16, int c16, const CUtensorMap *map_o,
                                                   const CUtensorMap *map_o16, uint32_t slab_f32, uint32_t slab_f16,
                                                   uint32_t &slab_turn) {
  const int n = n0 + quad * 32 + lane;
  const bool n_ok = n < p.N;
  const float cs = (p.colscale && n_ok) ? p.colscale[n] : 1.0f;
  const float bs = (p.bias && n_ok) ? p.bias[n] : 0.0f;
  const bool has_add = ADD && n_ok;
  int c = half * 16;
  if (c >= p.MT || m0 + c >= p.M) return;

  auto issue = [&](int cc, uint32_t (&v)[16], float (&ad)[ADD ? 16 : 1]) {
    tmem_ld16(lane_addr + (uint32_t)cc, v);
    if (!ADD) return;
    if (has_add) {
      const float *arow = p.add + (size_t)(m0 + cc) * p.N + n;
      if (m0 + cc + 16 <= p.M) {
#pragma unroll
        for (int j = 0; j < (ADD ? 16 : 1); j++) ad[j] = __ldg(arow + (size_t)j * p.N);
      } else {
#pragma unroll
        for (int j = 0; j < (ADD ? 16 : 1); j++) ad[j] = m0 + cc + j < p.M ? __ldg(arow + (size_t)j * p.N) : 0.0f;
      }
    } else {
#pragma unroll
      for (int j = 0; j < (ADD ? 16 : 1); j++) ad[j] = 0.0f;
    }
  };
  auto finish = [&](int cc, const uint32_t (&vr)[16], const float (&ad)[ADD ? 16 : 1]) {
    const bool full_rows = m0 + cc + 16 <= p.M;
    float v[16];
#pragma unroll
    for (int j = 0; j < 16; j++) v[j] = fmaf(__uint_as_float(vr[j]), cs, bs);
    act16(v, p.act);
    if (ADD) {
#pragma unroll
      for (int j = 0; j < 16; j++) v[j] += ad[ADD ? j : 0];
    }
    if (!PEERS && p.tma_out) {
      const uint32_t b = slab_turn & (uint32_t)(p.nslab - 1);
      slab_turn++;
      if (p.nslab == 4) tma_store_wait_read<3>(); else tma_store_wait_read<1>();  // lane 0: the group that last used slab b has read it (the other lanes own no groups)
      __syncwarp();
      if (p.out16) {
        const uint32_t dst = slab_f16 + b * 1024u + (uint32_t)lane * 2u;
#pragma unroll
        for (int j = 0; j < 16; j++)
          asm volatile("st.shared.b16 [%0], %1;" ::"r"(dst + (uint32_t)j * 64u), "h"(__half_as_ushort(__float2half_rn(v[j]))) : "memory");
      }
      if (!p.skip_f32) {
        const uint32_t dst = slab_f32 + b * 2048u + (uint32_t)lane * 4u;
#pragma unroll
        for (int j = 0; j < 16; j++) asm volatile("st.shared.f32 [%0], %1;" ::"r"(dst + (uint32_t)j * 128u), "f"(v[j]) : "memory");
      }
      fence_proxy_async_smem();
      __syncwarp();
      {
        const uint32_t lead = lane == 0 ? 1u : 0u;
        const int gn = n0 + quad * 32 + c16;
        if (p.out16) tma_store_3d_w(lead, map_o16, slab_f16 + b * 1024u, gn & 63, r16 + m0 + cc, gn >> 6);
        if (!p.skip_f32) tma_store_2d_w(lead, map_o, slab_f32 + b * 2048u, n0 + quad * 32, m0 + cc);
        tma_store_commit();
      }
      return;
    }
    if (!n_ok) return;
    if (p.out16) {
      const int gn = n + c16;
      __half *h16 = p.out16 + ((size_t)(gn >> 6) * p.o16_rows + (r16 + m0 + cc)) * 64 + (gn & 63);
#pragma unroll
      for (int j = 0; j < 16; j++)
        if (full_rows || m0 + cc + j < p.M) h16[(size_t)j * 64] = __float2half_rn(v[j]);
    }
    if (!p.skip_f32) {
      float *orow = outb + (size_t)(m0 + cc) * p.ldc + n;
#pragma unroll
      for (int j = 0; j < 16; j++)
        if (full_rows || m0 + cc + j < p.M) orow[(size_t)j * p.ldc] = v[j];
    }
    if (PEERS)
      for (int pi = 0; pi < p.n_peers; pi++) {
        float *prow = p.peer_out[pi] + (size_t)(m0 + cc) * p.ldc + n;
#pragma unroll
        for (int j = 0; j < 16; j++)
          if (full_rows || m0 + cc + j < p.M) prow[(size_t)j * p.ldc] = v[j];
      }
  };

  uint32_t va[16], vb[16];
  float aa[ADD ? 16 : 1], ab[ADD ? 16 : 1];
  issue(c, va, aa);
  for (;;) {
    tmem_ld_wait();
    int cn = c + 4 * kEpiWarps;
    bool more = cn < p.MT && m0 + cn < p.M;
    if (more) issue(cn, vb, ab);
    finish(c, va, aa);
    if (!more) break;
    c = cn;
    tmem_ld_wait();
    cn = c + 4 * kEpiWarps;
    more = cn < p.MT && m0 + cn < p.M;
    if (more) issue(cn, va, aa);
    finish(c, vb, ab);
    if (!more) break;
    c = cn;
  }
}

// KIND 4: f32 weights AND f32 activations on the tensor cores (kind::tf32), each operand as two planes - the f32 value,
// of which the MMA reads the top 19 bits, and what that truncation drops, computed by the prepass - with three products
// per K step (value x value, residue x value, value x residue) accumulated into the same TMEM columns: f32 range,
// relative error ~2^-20 per term, which is how f32-storage B keeps the reference's f32 arithmetic (1e-3 gate with three
// orders of magnitude to spare) at tensor-core speed.  A stage holds both weight planes and both activation planes.
// KIND 0: f16 weights, 1: int8 weights, 2: int4 (MatMulNBits) weights, 3: f16 weights with the epilogue also storing
// into peer GPUs' result buffers (TcParams::peer_out; a separate instantiation so the common epilogue stays lean -
// as a run-time loop it cost the plain f16 product 5 %).  KIND 2 is the f16 pipeline with one more
// stage in front of the MMA: TMA brings the RAW nibbles of a K chunk (128 rows x 32 bytes, the reference's
// layout as uploaded) next to the activation tile, eight extra warps unpack them in shared memory into the
// swizzled f16 weights tile - (q - zp) * scale per 32-weight block, two f16 lanes per instruction - and hand the
// slot to the MMA warp through a third barrier.  HBM sees 0.5 byte per weight instead of a 2-byte f16 copy.
// Within every group of 8 weights the unpack leaves k in the order 0,4,1,5,2,6,3,7 (the pairs one mask
// extracts); the activation tile is packed in the same order, and a sum over k does not care.
template <int KIND>
__global__ void __launch_bounds__(tc_threads<KIND>(), 1)
k_tc_gemm(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_a,
          const __grid_constant__ CUtensorMap map_o, const __grid_constant__ CUtensorMap map_o16,
          const __grid_constant__ CUtensorMap map_add, const TcParams p) {
  constexpr int MK = KIND == 4 ? 2 : (KIND >= 2 ? 0 : KIND);  // MMA kind and epilogue arithmetic (KIND 3: f16 with peer stores)
  constexpr bool kDeq = KIND == 2 || KIND == 5;               // a weights tile is made in shared memory from a raw tile
  constexpr uint32_t kWTiles = KIND == 4 ? 2u : 1u;  // weight tiles per stage (KIND 4: value and residue planes)
  constexpr bool kTwoProd = !kDeq;  // a second producer thread (warp 2 + kEpiWarps) loads the activation tiles
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // carve: [stages] x (P tile 16 KB | Q tile limbs*MT*128 B | raw nibble tile 4 KB for KIND 2), barriers,
  // split-K partial tile
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const int q_rows = p.MT * p.limbs;
  const uint32_t q_bytes = (uint32_t)q_rows * kRowBytes;
  const uint32_t stage_bytes = kWTiles * kPTileBytes + q_bytes + (uint32_t)tc_raw_bytes<KIND>();
  const uint32_t bars = smem_base + (uint32_t)p.stages * stage_bytes;  // 8-byte aligned (stage_bytes % 1024 == 0)
  auto full_bar = [&](int s) { return bars + (uint32_t)s * 8u; };
  auto empty_bar = [&](int s) { return bars + (uint32_t)(p.stages + s) * 8u; };
  auto acc_full = [&](int b) { return bars + (uint32_t)(2 * p.stages + b) * 8u; };
  auto acc_empty = [&](int b) { return bars + (uint32_t)(2 * p.stages + 2 + b) * 8u; };
  auto deq_bar = [&](int s) { return bars + (uint32_t)(2 * p.stages + 4 + s) * 8u; };  // KIND 2 only
  const uint32_t tmem_slot = bars + (uint32_t)(2 * p.stages + 4 + (kDeq ? p.stages : 0)) * 8u;
  const uint32_t abort_flag = tmem_slot + 4u;
  const uint32_t partial = (tmem_slot + 16u + 15u) & ~15u;  // [MT][128] f32, split-K mode only; 16-byte aligned for
                                                            // the vector loads of the reduction (3*stages+4 may be odd)
  // store slabs of the epilogue warps (tma_out mode only, never together with the split-K tile): per warp two
  // [16][32] f32 slabs, then per warp two [16][32] f16 slabs
  const uint32_t res_bars = (tmem_slot + 16u + 7u) & ~7u;  // tma_add: one barrier per epilogue warp and residual slab
  const uint32_t slabs = (tmem_slot + 16u + (p.tma_add ? (uint32_t)(kEpiWarps * kResSlabs) * 8u : 0u) + 127u) & ~127u;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int acc_cols = p.limb_sum ? p.MT : q_rows;
  uint32_t acc_stride = 32;  // TMEM columns per accumulator buffer
  while ((int)acc_stride < acc_cols) acc_stride <<= 1;
  const uint32_t tmem_cols = 2 * acc_stride;
  const int num_tiles = p.tiles_n * p.tiles_m * p.batches;
  const int kb0 = p.splitk > 1 ? (int)blockIdx.z * p.kb_per_split : 0;
  const int kb1 = p.splitk > 1 ? min(p.num_kb, kb0 + p.kb_per_split) : p.num_kb;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; s++) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
      if (kDeq) mbar_init(deq_bar(s), 4);  // KIND 2: the four warps of the group that owns the chunk; KIND 5: its four warps
    }
    for (int b = 0; b < 2; b++) {
      mbar_init(acc_full(b), 1);
      mbar_init(acc_empty(b), kEpiWarps);
    }
    if (p.tma_add)
      for (int i = 0; i < kEpiWarps * kResSlabs; i++) mbar_init(res_bars + (uint32_t)i * 8u, 1);
    asm volatile("st.shared.u32 [%0], %1;" ::"r"(abort_flag), "r"(0u) : "memory");
    fence_barrier_init();
    fence_proxy_async_smem();
    tma_prefetch_desc(&map_w);
    tma_prefetch_desc(&map_a);
    if (p.tma_out) {
      if (!p.skip_f32) tma_prefetch_desc(&map_o);
      if (p.out16) tma_prefetch_desc(&map_o16);
    }
    if (p.tma_add) tma_prefetch_desc(&map_add);
  }
  if (warp == 1) tmem_alloc(tmem_slot, tmem_cols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  uint32_t tmem_base;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem_base) : "r"(tmem_slot) : "memory");
  // K split over a cluster: a CTA's shared memory may be written by its peers only once it is known to be running.
  // Everyone arrives here; the epilogue warps complete the barrier before their first remote store, the other
  // warps after their role.
  if (p.splitk > 1) cluster_arrive_all();
  fa_grid_dep_sync();  // barriers, TMEM and descriptors were set up while the previous kernel drained

  auto aborted = [&]() {
    uint32_t v;
    asm volatile("ld.volatile.shared.u32 %0, [%1];" : "=r"(v) : "r"(abort_flag) : "memory");
    return v != 0;
  };
  auto set_abort = [&](int code, int detail) {
    asm volatile("st.volatile.shared.u32 [%0], %1;" ::"r"(abort_flag), "r"(1u) : "memory");
    report_timeout(p.status, code, detail);
  };

  // The role loops below are latency-critical: one warp issues every weight load, one every activation load, one
  // every MMA of the CTA, and with little else on its scheduler to hide behind, each extra instruction or taken
  // branch costs its full latency per K chunk (measured: the loops, not bandwidth or the tensor pipe, set the pace
  // of the ring).  So: whole warps execute them with warp-uniform operands and ONE elected lane issues the
  // tcgen05 / TMA instructions (the operands then stay in the uniform datapath those instructions read); no
  // division, ring position and barrier addresses kept as running values that wrap by select, one inline poll
  // per barrier.  The __syncwarp that closes a role reconverges the warp before the block-wide barriers.
  if (warp == 0) {
    // ---- TMA producer: runs ahead across tiles, bounded only by the ring ----------------------
    // Ring position as running values (barrier address, slot address, parity) advanced without a branch; the wait on
    // a slot's empty barrier uses the opposite parity of its full barrier, which a freshly initialised barrier
    // passes at once, so the first trip round the ring needs no special case.
    {
      const uint32_t lead = elect_lead();
      const uint32_t fb_end = bars + (uint32_t)p.stages * 8u, eoff = (uint32_t)p.stages * 8u;
      uint32_t fb = bars, dst = smem_base, ph = 0;
      bool stop = false;
      for (int tile = blockIdx.x; tile < num_tiles && !stop; tile += gridDim.x) {
        const int tpb = p.tiles_n * p.tiles_m, batch = tile / tpb, tin = tile - batch * tpb;
        const int tn = tin % p.tiles_n, tm = tin / p.tiles_n;
        const int wb = p.w_batch_mod ? batch % p.w_batch_mod : batch;
        int wrow = ((wb * p.tiles_n + tn) * p.num_kb + kb0) * 128;
        int aslab = (p.a_shared ? 0 : batch) * p.limbs * p.num_kb + kb0;
        const int m0 = tm * p.MT;
        const int wh = tile == 0 ? p.withhold_kb : -1;  // test hook: this chunk never arrives
        for (int kb = kb0; kb < kb1; kb++, wrow += 128, aslab++) {
          if (!__all_sync(0xffffffffu, mbar_wait(fb + eoff, ph ^ 1u, p.wait_limit))) {  // empty barrier of the slot, previous use
            if (lane == 0) set_abort(1, kb);
            stop = true;
            break;
          }
          if (kb != wh) {
            if (KIND == 5) {
              mbar_expect_tx_w(lead, fb, q_bytes + kRaw8TileBytes);
              tma_load_2d_w(lead, dst + kPTileBytes - kRaw8TileBytes, &map_w, 0, (tn * p.num_kb + kb) * 32, fb);  // 8 KB int8 tile, in
                                                                                                        // the upper half of the f16 tile
            } else if (KIND == 2) {
              mbar_expect_tx_w(lead, fb, q_bytes + kRawTileBytes);
              tma_load_2d_w(lead, dst + kPTileBytes + q_bytes, &map_w, 0, (tn * p.num_kb + kb) * 16, fb);  // 4 KB nibble tile
            } else {
              mbar_expect_tx_w(lead, fb, stage_bytes);
              tma_load_2d_w(lead, dst, &map_w, 0, wrow, fb);
              if (KIND == 4) tma_load_2d_w(lead, dst + kPTileBytes, &map_w, 0, wrow + p.w_lo_rows, fb);  // residue plane
            }
            if (!kTwoProd) {
              tma_load_3d_w(lead, dst + kWTiles * kPTileBytes, &map_a, 0, m0, aslab, fb);
              for (int l = 1; l < p.limbs; l++)
                tma_load_3d_w(lead, dst + kWTiles * kPTileBytes + (uint32_t)(l * p.MT) * kRowBytes, &map_a, 0, m0, aslab + l * p.num_kb, fb);
            }
          }
          fb += 8u;
          dst += stage_bytes;
          const bool wrap = fb == fb_end;
          fb = wrap ? bars : fb;
          dst = wrap ? smem_base : dst;
          ph ^= wrap ? 1u : 0u;
        }
      }
    }
    __syncwarp();
  } else if (kTwoProd && warp == 2 + kEpiWarps) {
    // ---- second producer: the activation tiles of every chunk.  It walks the ring exactly like warp 0 and lands its
    // bytes on the same full barrier; warp 0's expect_tx announces the whole stage, and bytes that arrive before that
    // announcement are simply counted early (the phase cannot complete before warp 0's arrival). ----
    {
      const uint32_t lead = elect_lead();
      const uint32_t fb_end = bars + (uint32_t)p.stages * 8u, eoff = (uint32_t)p.stages * 8u;
      uint32_t fb = bars, dst = smem_base + kWTiles * kPTileBytes, ph = 0;
      const uint32_t dst0 = dst;
      bool stop = false;
      for (int tile = blockIdx.x; tile < num_tiles && !stop; tile += gridDim.x) {
        const int tpb = p.tiles_n * p.tiles_m, batch = tile / tpb, tin = tile - batch * tpb;
        const int tm = tin / p.tiles_n;
        int aslab = (p.a_shared ? 0 : batch) * p.limbs * p.num_kb + kb0;
        const int m0 = tm * p.MT;
        const int wh = tile == 0 ? p.withhold_kb : -1;
        for (int kb = kb0; kb < kb1; kb++, aslab++) {
          if (!__all_sync(0xffffffffu, mbar_wait(fb + eoff, ph ^ 1u, p.wait_limit))) {
            if (lane == 0) set_abort(7, kb);
            stop = true;
            break;
          }
          if (kb != wh) {
            tma_load_3d_w(lead, dst, &map_a, 0, m0, aslab, fb);
            for (int l = 1; l < p.limbs; l++)
              tma_load_3d_w(lead, dst + (uint32_t)(l * p.MT) * kRowBytes, &map_a, 0, m0, aslab + l * p.num_kb, fb);
          }
          fb += 8u;
          dst += stage_bytes;
          const bool wrap = fb == fb_end;
          fb = wrap ? bars : fb;
          dst = wrap ? dst0 : dst;
          ph ^= wrap ? 1u : 0u;
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---- MMA issuer: alternates between the two TMEM accumulator buffers -----------------------
    // Per K chunk: one poll of the slot's full barrier, four MMAs (eight with a second plane), one commit, and a
    // branch-free step round the ring.  The loop exists twice (with and without the residue plane of the
    // activations) so that choice is not a branch per chunk.
    {
      const uint32_t lead = elect_lead();
      const uint32_t idesc = make_idesc(MK, 128, acc_cols);
      const uint64_t desc0 = smem_desc_sw128(smem_base);  // slot 0 weights tile; other tiles are address offsets
      const uint32_t d_hi = (uint32_t)(desc0 >> 32), da0 = (uint32_t)desc0;
      const uint32_t q_off = (kWTiles * kPTileBytes) >> 4, st_off = stage_bytes >> 4;
      const uint32_t wlo_off = kPTileBytes >> 4;                    // KIND 4: residue plane of the weights
      const uint32_t lo_off = (uint32_t)(p.MT * kRowBytes) >> 4;    // residue plane of the activations
      const uint32_t fb_end = bars + (uint32_t)p.stages * 8u, eoff = (uint32_t)p.stages * 8u;
      const uint32_t doff = (2u * (uint32_t)p.stages + 4u) * 8u;    // full barrier -> unpack barrier of the slot
      uint32_t fb = bars, da = da0, ph = 0, lt = 0;
      bool ok = true;
      auto run = [&](auto ls_tag) {
        constexpr bool kLimbSum = decltype(ls_tag)::value;
        for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, lt++) {
          const uint32_t buf = lt & 1, use = lt >> 1;
          if (use > 0 && !__all_sync(0xffffffffu, mbar_wait(acc_empty(buf), (use - 1) & 1, p.wait_limit))) {
            if (lane == 0) set_abort(4, tile);
            break;
          }
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + buf * acc_stride;
          uint32_t acc = 0;
          for (int kb = kb0; kb < kb1; kb++) {
            if (!__all_sync(0xffffffffu, mbar_wait(fb, ph, p.wait_limit))) {
              if (lane == 0) set_abort(2, kb);
              ok = false;
              break;
            }
            if (kDeq) {
              if (!__all_sync(0xffffffffu, mbar_wait(fb + doff, ph, p.wait_limit))) {  // weights tile unpacked
                if (lane == 0) set_abort(6, kb);
                ok = false;
                break;
              }
              tc_fence_after();
            }
            const uint32_t db = da + q_off;
            umma_lo_w<MK>(lead, d_tmem, da, db, d_hi, idesc, acc);  // 4 x 32 bytes of K per slot
            acc = 1u;
            umma_lo_w<MK>(lead, d_tmem, da + 2, db + 2, d_hi, idesc, 1u);
            umma_lo_w<MK>(lead, d_tmem, da + 4, db + 4, d_hi, idesc, 1u);
            umma_lo_w<MK>(lead, d_tmem, da + 6, db + 6, d_hi, idesc, 1u);
            if (kLimbSum) {
              umma_lo_w<MK>(lead, d_tmem, da, db + lo_off, d_hi, idesc, 1u);
              umma_lo_w<MK>(lead, d_tmem, da + 2, db + lo_off + 2, d_hi, idesc, 1u);
              umma_lo_w<MK>(lead, d_tmem, da + 4, db + lo_off + 4, d_hi, idesc, 1u);
              umma_lo_w<MK>(lead, d_tmem, da + 6, db + lo_off + 6, d_hi, idesc, 1u);
            }
            if (KIND == 4) {  // weights' residue x activations' value
              umma_lo_w<MK>(lead, d_tmem, da + wlo_off, db, d_hi, idesc, 1u);
              umma_lo_w<MK>(lead, d_tmem, da + wlo_off + 2, db + 2, d_hi, idesc, 1u);
              umma_lo_w<MK>(lead, d_tmem, da + wlo_off + 4, db + 4, d_hi, idesc, 1u);
              umma_lo_w<MK>(lead, d_tmem, da + wlo_off + 6, db + 6, d_hi, idesc, 1u);
            }
            umma_commit_w(lead, fb + eoff);  // frees the slot when these MMAs have read it
            fb += 8u;
            da += st_off;
            const bool wrap = fb == fb_end;
            fb = wrap ? bars : fb;
            da = wrap ? da0 : da;
            ph ^= wrap ? 1u : 0u;
          }
          if (ok) umma_commit_w(lead, acc_full(buf));  // this tile's accumulators are complete
        }
      };
      if (p.limb_sum) run(std::true_type{}); else run(std::false_type{});
    }
    __syncwarp();
  } else if (KIND == 5 && warp >= 2 + kEpiWarps && (warp & 2) == 0) {
    // spare warp ids (see kDeqWarps): no role
  } else if (KIND == 5 && warp >= 2 + kEpiWarps) {
    // ---- int8 weights -> f16 weights tile: two groups of four warps take alternate K chunks; thread r of a group
    // owns weight row r of the tile.  A byte q becomes the f16 value q exactly: (q ^ 0x80) placed under the exponent
    // byte 0x64 is the f16 number 1024 + q + 128, minus 1152.  The per-column scale of the weights is applied to the
    // f32 accumulator in the epilogue. ----
    const int dw = ((warp - (2 + kEpiWarps)) >> 2) * 2 + (warp & 1);
    const int dq = dw * 32 + lane, r = dq & 127, grp = dq >> 7;
    const uint32_t nst = (uint32_t)p.stages;
    const int chunks = kb1 - kb0;
    const __half2 off = __float2half2_rn(1152.0f);
    uint32_t it = 0;  // ring index of the next chunk (all chunks, both groups)
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      for (int c = 0; c < chunks && ok; c++, it++) {
        if ((int)(it & 1u) != grp) continue;
        const uint32_t slot_i = it % nst, ph = (it / nst) & 1u;
        int okw = 1;
        if (lane == 0 && !mbar_wait(full_bar((int)slot_i), ph, p.wait_limit)) {
          set_abort(5, c);
          okw = 0;
        }
        ok = __shfl_sync(0xffffffffu, okw, 0) != 0 && !aborted();
        if (!ok) break;
        const uint32_t slot = smem_base + slot_i * stage_bytes;
        // The int8 tile sits in the upper half of the f16 tile it becomes (no shared memory of its own, so the ring is
        // as deep as the f16 kernel's): every thread of the group first takes its 64 bytes into registers, the group
        // meets at its own named barrier, and only then are the f16 rows written over them.
        const uint32_t src = slot + (uint32_t)(kPTileBytes - kRaw8TileBytes) + (uint32_t)(r * 64);
        uint32_t wd[16];
#pragma unroll
        for (int j = 0; j < 4; j++)
          asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(wd[4 * j]), "=r"(wd[4 * j + 1]), "=r"(wd[4 * j + 2]), "=r"(wd[4 * j + 3]) : "r"(src + (uint32_t)(j * 16)) : "memory");
        asm volatile("bar.sync %0, 128;" ::"r"(1 + grp) : "memory");
#pragma unroll
        for (int j = 0; j < 4; j++) {  // 16 weights per step -> two 16-byte pieces of the 128-byte f16 row
          uint32_t h[8];
#pragma unroll
          for (int q = 0; q < 4; q++) {
            const uint32_t x = wd[4 * j + q] ^ 0x80808080u;
            uint32_t a0 = __byte_perm(x, 0x64646464u, 0x5140), a1 = __byte_perm(x, 0x64646464u, 0x5342);
            __half2 h0 = __hsub2(*(__half2 *)&a0, off), h1 = __hsub2(*(__half2 *)&a1, off);
            h[2 * q] = *(uint32_t *)&h0;
            h[2 * q + 1] = *(uint32_t *)&h1;
          }
#pragma unroll
          for (int e = 0; e < 2; e++) {
            const uint32_t cc = (uint32_t)(2 * j + e);
            asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(slot + (uint32_t)(r * 128) + ((cc ^ (uint32_t)(r & 7)) << 4)),
                         "r"(h[4 * e]), "r"(h[4 * e + 1]), "r"(h[4 * e + 2]), "r"(h[4 * e + 3])
                         : "memory");
          }
        }
        fence_proxy_async_smem();  // the tile is read by the tensor core through the async proxy
        __syncwarp();
        if (lane == 0) mbar_arrive(deq_bar((int)slot_i));
      }
    }
    __syncwarp();
  } else if (KIND == 2 && warp >= 2 + kEpiWarps && (warp & 2) == 0) {
    // spare warp ids (see kDeqWarps): no role; they wait at the barriers below with everyone else
  } else if (KIND == 2 && warp >= 2 + kEpiWarps) {
    // ---- int4 unpack: two groups of four warps take alternate K chunks, so one group's load-unpack-store
    // chain overlaps the other's; a thread owns weight row r of the tile for both 32-weight blocks of a chunk
    // the first four unpack warps (by id) form group 0, the last four group 1
    const int dw = ((warp - (2 + kEpiWarps)) >> 2) * 2 + (warp & 1);
    const int dq = dw * 32 + lane, r = dq & 127, grp = dq >> 7;
    const uint32_t nst = (uint32_t)p.stages;
    const int chunks = kb1 - kb0;
    uint32_t tiles_done = 0;
    bool ok = true;
    const __half2 sixteenth = __float2half2_rn(0.0625f);
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, tiles_done++) {
      const int tn = (tile % (p.tiles_n * p.tiles_m)) % p.tiles_n;
      const int n = min(tn * 128 + r, p.N - 1);
      // Scale and zero-point of (block, row) from the block-major side copy: a warp's 32 rows are one
      // 128-byte (scales) and one 32-byte (zero-points) request.  (Read in the uploaded [N][nblk] order, every
      // lane touched its own sector and the load/store unit, not DRAM, set the pace of the unpack.)  Fetched
      // for 4 of this group's chunks at a time, one batch ahead.
      const float *srow = p.nb_scales + n;
      const uint8_t *zrow = p.nb_zp + n;
      constexpr int G = 4;
      float scg[2 * G], scn[2 * G];
      unsigned long long zbg = 0, zbn = 0;  // (chunk i, block hb) in bits [8(2i+hb), 8(2i+hb)+8)
      const uint32_t it_base = tiles_done * (uint32_t)chunks;   // ring index of this tile's first chunk
      const int first = (int)((grp - (it_base & 1u)) & 1u);     // this group's first chunk within the tile
      auto fetch = [&](int c0, float *sc, unsigned long long &zb) {
        zb = 0;
#pragma unroll
        for (int i = 0; i < G; i++)
#pragma unroll
          for (int hb = 0; hb < 2; hb++) {
            const size_t blk = (size_t)min(2 * (kb0 + c0 + 2 * i) + hb, p.nblk - 1);
            sc[2 * i + hb] = __ldg(srow + blk * p.N);
            zb |= (unsigned long long)__ldg(zrow + blk * p.N) << (8 * (2 * i + hb));
          }
      };
      fetch(first, scg, zbg);
      for (int cg = first; cg < chunks && ok; cg += 2 * G) {
        if (cg + 2 * G < chunks) fetch(cg + 2 * G, scn, zbn);
#pragma unroll
        for (int i = 0; i < G; i++) {
          const int c = cg + 2 * i;
          if (c >= chunks) break;
          const uint32_t it = it_base + (uint32_t)c, slot_i = it % nst, ph = (it / nst) & 1u;
          int okw = 1;
          if (lane == 0 && !mbar_wait(full_bar((int)slot_i), ph, p.wait_limit)) {
            set_abort(5, c);
            okw = 0;
          }
          ok = __shfl_sync(0xffffffffu, okw, 0) != 0 && !aborted();
          if (!ok) break;
          const uint32_t slot = smem_base + slot_i * stage_bytes;
#pragma unroll
          for (int hb = 0; hb < 2; hb++) {
            uint32_t wd[4];
            asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(wd[0]), "=r"(wd[1]), "=r"(wd[2]), "=r"(wd[3])
                         : "r"(slot + kPTileBytes + q_bytes + (uint32_t)(r * 32 + hb * 16))
                         : "memory");
            const int z = (int)((unsigned)(zbg >> (8 * (2 * i + hb))) & 0xFFu);
            const __half2 s2 = __float2half2_rn(scg[2 * i + hb]);
            const __half2 zsub = __half2half2(__int2half_rn(1024 + z));   // (1024 + q) - (1024 + zp)
            const __half2 zneg = __half2half2(__int2half_rn(-(64 + z)));  // (1024 + 16 q) / 16 - (64 + zp)
#pragma unroll
            for (int j = 0; j < 4; j++) {
              const uint32_t w0 = wd[j], w8 = wd[j] >> 8;
              uint32_t a0 = (w0 & 0x000F000Fu) | 0x64006400u;  // nibbles 0,4 as 1024 + q
              uint32_t a1 = (w0 & 0x00F000F0u) | 0x64006400u;  // nibbles 1,5 as 1024 + 16 q
              uint32_t a2 = (w8 & 0x000F000Fu) | 0x64006400u;  // nibbles 2,6
              uint32_t a3 = (w8 & 0x00F000F0u) | 0x64006400u;  // nibbles 3,7
              __half2 h0 = __hmul2(__hsub2(*(__half2 *)&a0, zsub), s2);
              __half2 h1 = __hmul2(__hfma2(*(__half2 *)&a1, sixteenth, zneg), s2);
              __half2 h2 = __hmul2(__hsub2(*(__half2 *)&a2, zsub), s2);
              __half2 h3 = __hmul2(__hfma2(*(__half2 *)&a3, sixteenth, zneg), s2);
              const uint32_t cc = (uint32_t)(hb * 4 + j);
              asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(slot + (uint32_t)(r * 128) + ((cc ^ (uint32_t)(r & 7)) << 4)),
                           "r"(*(uint32_t *)&h0), "r"(*(uint32_t *)&h1), "r"(*(uint32_t *)&h2), "r"(*(uint32_t *)&h3)
                           : "memory");
            }
          }
          fence_proxy_async_smem();  // the tile is read by the tensor core through the async proxy
          __syncwarp();
          if (lane == 0) mbar_arrive(deq_bar((int)slot_i));
        }
#pragma unroll
        for (int i = 0; i < 2 * G; i++) scg[i] = scn[i];
        zbg = zbn;
      }
    }
    __syncwarp();
  } else {
    // ---- epilogue: TMEM -> registers -> global (or -> smem partial in split-K mode) -------------
    const int ew = warp - 2, quad = warp & 3, half = ew >> 2;
    uint32_t lt = 0, slab_turn = 0, cl_rank = 0, res_turn = 0;
    if (p.splitk > 1) {
      asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(cl_rank));
      cluster_wait_all();
    }
    const uint32_t slab_f32 = slabs + (uint32_t)(ew * p.nslab) * 2048u, slab_f16 = slabs + p.slab_f16_off + (uint32_t)(ew * p.nslab) * 1024u;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, lt++) {
      const int tpb = p.tiles_n * p.tiles_m, batch = tile / tpb, tin = tile - batch * tpb;
      const int tn = tin % p.tiles_n, tm = tin / p.tiles_n;
      const int n0 = tn * 128, m0 = tm * p.MT;
      float *const outb = p.out + (size_t)(batch / p.o_div) * p.o_hi + (size_t)(batch % p.o_div) * p.o_lo;
      const int r16 = (batch / p.o_div) * p.o16_row_hi, c16 = (batch % p.o_div) * p.o16_col_lo;
      const uint32_t buf = lt & 1, use = lt >> 1;
      if (kDeq) {  // leave the issue slots to the unpack warps while the tile is being accumulated
        ok = false;
        for (uint32_t i = 0; i < (p.wait_limit >> 4) && !ok; i++) {
          ok = mbar_try_wait(acc_full(buf), use & 1) != 0;
          if (!ok) __nanosleep(256);
        }
      } else {
        ok = mbar_wait(acc_full(buf), use & 1, p.wait_limit);
      }
      if (!ok && lane == 0) set_abort(3, tile);
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0 && !aborted();
      if (!ok) break;
      tc_fence_after();
      const uint32_t lane_addr = tmem_base + buf * acc_stride + ((uint32_t)(quad * 32) << 16);
      if (!kDeq && MK != 1 && p.splitk == 1 && !p.rowscale && !p.rowbias)
      {
        if (KIND == 0 && p.tma_add)
          epilogue_tile_resadd(p, lane_addr, n0, m0, quad, lane, half, r16, c16, &map_o, &map_o16, &map_add, slab_f32, slab_f16,
                               slabs + p.slab_res_off + (uint32_t)(ew * kResSlabs) * 2048u, res_bars + (uint32_t)(ew * kResSlabs) * 8u,
                               slab_turn, res_turn);
        else if (p.add)
          epilogue_tile_fast<KIND == 3, true>(p, lane_addr, n0, m0, quad, lane, half, outb, r16, c16, &map_o, &map_o16, slab_f32,
                                              slab_f16, slab_turn);
        else
          epilogue_tile_fast<KIND == 3, false>(p, lane_addr, n0, m0, quad, lane, half, outb, r16, c16, &map_o, &map_o16, slab_f32,
                                               slab_f16, slab_turn);
      }
      else
        epilogue_tile<MK, KIND == 3>(p, lane_addr, n0, m0, quad, lane, half, outb, r16, c16, partial, &map_o, &map_o16,
                                     slab_f32, slab_f16, slab_turn, cl_rank);
      // hand the accumulator buffer back to the MMA warp
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty(buf));
    }
    if (p.tma_out && lane == 0) tma_store_wait_all();  // the slabs must outlive the stores that read them
    __syncwarp();
  }

  if (p.splitk > 1 && !(warp >= 2 && warp < 2 + kEpiWarps)) {
    __syncwarp();
    cluster_wait_all();
  }
  if (p.splitk > 1) {
    // ---- split-K finish: after the cluster barrier every CTA holds, for the 16-row blocks it owns, one partial
    // block from each CTA of the cluster in its OWN shared memory; it adds them in rank order (deterministic),
    // applies the epilogue and stores.  No remote access happens after the barrier. ----
    __syncwarp();
    cluster_sync_all();
    uint32_t rank;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
    if (warp >= 2 && warp < 2 + kEpiWarps && !aborted()) {
      const int tile = blockIdx.x, tn = tile % p.tiles_n, tm = tile / p.tiles_n;
      const int n0 = tn * 128, m0 = tm * p.MT;
      const int t = threadIdx.x - 64;  // the epilogue threads, each owns groups of 4 consecutive columns
      const bool vec_ok = (p.N & 3) == 0;
      constexpr int ET = 32 * kEpiWarps;
      for (int g = t; g < p.split_rb * 16 * 32; g += ET) {
        const int lrow = g >> 5, nl = (g & 31) * 4;         // row within this CTA's owned blocks, first column
        const int ml = ((lrow >> 4) * p.splitk + (int)rank) * 16 + (lrow & 15);  // row within the tile
        const int m = m0 + ml, n = n0 + nl;
        if (ml >= p.MT || m >= p.M || n >= p.N) continue;
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        for (int r = 0; r < p.splitk; r++) {
          float4 v;
          asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
                       : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                       : "r"(partial + (uint32_t)((((r * p.split_rb * 16) + lrow) * 128 + nl) * 4))
                       : "memory");
          acc[0] += v.x; acc[1] += v.y; acc[2] += v.z; acc[3] += v.w;
        }
        const float rs = p.rowscale ? p.rowscale[m] : 1.0f;
        float o[4];
#pragma unroll
        for (int q = 0; q < 4; q++) {
          const int nn = min(n + q, p.N - 1);
          float v = fmaf(acc[q] * rs, p.colscale ? p.colscale[nn] : 1.0f, p.bias ? p.bias[nn] : 0.0f);
          if (p.rowbias) v += p.rowbias[m];
          v = fa_actf(v, p.act);
          if (p.add) v += p.add[(size_t)m * p.N + nn];
          o[q] = v;
        }
        float *dst = p.out + (size_t)m * p.N + n;
        if (vec_ok && n + 3 < p.N) {
          *(float4 *)dst = make_float4(o[0], o[1], o[2], o[3]);
        } else {
          for (int q = 0; q < 4 && n + q < p.N; q++) dst[q] = o[q];
        }
      }
    }
    __syncwarp();
  }

  // ---- teardown --------------------------------------------------------------------------------
  __syncwarp();
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

// ---- CTA pairs: the f16 product for shapes with many tiles -----------------------------------------------------
// What bounds the one-CTA kernel above at large M is the SM's shared-memory bandwidth: every operand byte is written
// once by the copy engine and read once by the tensor core, and a 128 x 256 tile moves 2 x 48 KB per K chunk
// through a ~128 B/clk port while its four MMAs need 512 clocks (measured: 650 clocks per chunk with nothing else
// running, 770-840 with the epilogue's slab traffic beside it, the same on 16 busy SMs as on 148).  Here two CTAs of a
// cluster share one 256-lane MMA (cta_group::2): the pair's tile is 256 output columns x MT rows, each CTA loads its
// own 128 weight rows and HALF of the activation rows (2 x 32 KB per chunk), the hardware feeds both tensor cores
// from the two halves, and each CTA finds its 128 columns x all MT rows in its own TMEM - so its epilogue is the
// one-CTA epilogue unchanged.  Barriers: `full` lives in the leader (even) CTA and counts the bytes of both CTAs'
// loads; `empty` and `acc_full` exist in both CTAs and are signalled together by the leader's tcgen05.commit;
// `acc_empty` lives in the leader and collects the epilogue warps of both CTAs.  No load is delivered to more than
// one CTA.
__global__ void __launch_bounds__(kThreads, 1)
k_tc_gemm_pair(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_a,
               const __grid_constant__ CUtensorMap map_o, const __grid_constant__ CUtensorMap map_o16,
               const __grid_constant__ CUtensorMap map_add, const TcParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const int half_rows = p.MT / 2;  // activation rows this CTA stages
  const uint32_t stage_bytes = kPTileBytes + (uint32_t)half_rows * kRowBytes;
  const uint32_t bars = smem_base + (uint32_t)p.stages * stage_bytes;
  auto acc_full = [&](int b) { return bars + (uint32_t)(2 * p.stages + b) * 8u; };
  auto acc_empty = [&](int b) { return bars + (uint32_t)(2 * p.stages + 2 + b) * 8u; };
  const uint32_t tmem_slot = bars + (uint32_t)(2 * p.stages + 4) * 8u;
  const uint32_t abort_flag = tmem_slot + 4u;
  const uint32_t res_bars = (tmem_slot + 16u + 7u) & ~7u;  // tma_add: one barrier per epilogue warp and residual slab
  const uint32_t slabs = (tmem_slot + 16u + (p.tma_add ? (uint32_t)(kEpiWarps * kResSlabs) * 8u : 0u) + 127u) & ~127u;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();
  uint32_t acc_stride = 32;
  while ((int)acc_stride < p.MT) acc_stride <<= 1;
  const uint32_t tmem_cols = 2 * acc_stride;
  const int tiles_n2 = p.tiles_n / 2;  // tiles_n is even in this mode
  const int num_tiles = tiles_n2 * p.tiles_m;
  const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; s++) {
      mbar_init(bars + (uint32_t)s * 8u, 1);               // full (used in the leader)
      mbar_init(bars + (uint32_t)(p.stages + s) * 8u, 1);  // empty
    }
    for (int b = 0; b < 2; b++) {
      mbar_init(acc_full(b), 1);
      mbar_init(acc_empty(b), 2 * kEpiWarps);  // both CTAs' epilogue warps arrive on the leader's barrier
    }
    if (p.tma_add)
      for (int i = 0; i < kEpiWarps * kResSlabs; i++) mbar_init(res_bars + (uint32_t)i * 8u, 1);
    asm volatile("st.shared.u32 [%0], %1;" ::"r"(abort_flag), "r"(0u) : "memory");
    fence_barrier_init();
    fence_proxy_async_smem();
    tma_prefetch_desc(&map_w);
    tma_prefetch_desc(&map_a);
    if (p.tma_out) {
      if (!p.skip_f32) tma_prefetch_desc(&map_o);
      if (p.out16) tma_prefetch_desc(&map_o16);
    }
    if (p.tma_add) tma_prefetch_desc(&map_add);
  }
  if (warp == 1) tmem_alloc2(tmem_slot, tmem_cols);
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer's barriers exist before anything signals them
  tc_fence_after();
  uint32_t tmem_base;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem_base) : "r"(tmem_slot) : "memory");
  fa_grid_dep_sync();

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
    // ---- TMA producer (both CTAs): own weights tile; the leader announces the bytes of the whole pair ----
    {
      const uint32_t lead = elect_lead();
      const uint32_t fb_end = bars + (uint32_t)p.stages * 8u, eoff = (uint32_t)p.stages * 8u;
      uint32_t fb = bars, dst = smem_base, ph = 0;
      bool stop = false;
      for (int tile = pair; tile < num_tiles && !stop; tile += npairs) {
        const int tn2 = tile % tiles_n2;
        int wrow = (tn2 * 2 + (int)rank) * p.num_kb * 128;
        const int wh = (tile == pair && blockIdx.x == 0) ? p.withhold_kb : -1;  // test hook: the leader of pair 0 never
                                                                                // announces this chunk of its first tile
        for (int kb = 0; kb < p.num_kb; kb++, wrow += 128) {
          if (!__all_sync(0xffffffffu, mbar_wait(fb + eoff, ph ^ 1u, p.wait_limit))) {
            if (lane == 0) set_abort(11, kb);
            stop = true;
            break;
          }
          const uint32_t go = kb != wh ? lead : 0u;
          mbar_expect_tx_w(rank == 0 ? go : 0u, fb, 2 * stage_bytes);  // the bytes of both CTAs land on this barrier
          tma_load_2d_pair_w(go, dst, &map_w, 0, wrow, fb);
          fb += 8u;
          dst += stage_bytes;
          const bool wrap = fb == fb_end;
          fb = wrap ? bars : fb;
          dst = wrap ? smem_base : dst;
          ph ^= wrap ? 1u : 0u;
        }
      }
    }
    __syncwarp();
  } else if (warp == 2 + kEpiWarps) {
    // ---- second producer (both CTAs): own half of the activation rows (one thread sustains only one tile load per
    // ~300-400 clocks, see kThreads) ----
    {
      const uint32_t lead = elect_lead();
      const uint32_t fb_end = bars + (uint32_t)p.stages * 8u, eoff = (uint32_t)p.stages * 8u;
      uint32_t fb = bars, dst = smem_base + kPTileBytes, ph = 0;
      bool stop = false;
      for (int tile = pair; tile < num_tiles && !stop; tile += npairs) {
        const int tm = tile / tiles_n2;
        const int arow = tm * p.MT + (int)rank * half_rows;
        for (int kb = 0; kb < p.num_kb; kb++) {
          if (!__all_sync(0xffffffffu, mbar_wait(fb + eoff, ph ^ 1u, p.wait_limit))) {
            if (lane == 0) set_abort(15, kb);
            stop = true;
            break;
          }
          tma_load_3d_pair_w(lead, dst, &map_a, 0, arow, kb, fb);
          fb += 8u;
          dst += stage_bytes;
          const bool wrap = fb == fb_end;
          fb = wrap ? bars : fb;
          dst = wrap ? smem_base + kPTileBytes : dst;
          ph ^= wrap ? 1u : 0u;
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---- MMA issuer (leader CTA only): the whole warp walks the ring, one elected lane issues ----
    if (rank == 0) {
      const uint32_t lead = elect_lead();
      const uint32_t idesc = make_idesc(0, 256, p.MT);
      const uint64_t desc0 = smem_desc_sw128(smem_base);
      const uint32_t d_hi = (uint32_t)(desc0 >> 32), da0 = (uint32_t)desc0;
      const uint32_t q_off = kPTileBytes >> 4, st_off = stage_bytes >> 4;
      const uint32_t fb_end = bars + (uint32_t)p.stages * 8u, eoff = (uint32_t)p.stages * 8u;
      uint32_t fb = bars, da = da0, ph = 0, lt = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += npairs, lt++) {
        const uint32_t buf = lt & 1, use = lt >> 1;
        if (use > 0 && !__all_sync(0xffffffffu, mbar_wait(acc_empty(buf), (use - 1) & 1, p.wait_limit))) {
          if (lane == 0) set_abort(14, tile);
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * acc_stride;
        uint32_t acc = 0;
        for (int kb = 0; kb < p.num_kb; kb++) {
          if (!__all_sync(0xffffffffu, mbar_wait(fb, ph, p.wait_limit))) {
            if (lane == 0) set_abort(12, kb);
            ok = false;
            break;
          }
          const uint32_t db = da + q_off;
          umma2_f16_lo_w(lead, d_tmem, da, db, d_hi, idesc, acc);
          acc = 1u;
          umma2_f16_lo_w(lead, d_tmem, da + 2, db + 2, d_hi, idesc, 1u);
          umma2_f16_lo_w(lead, d_tmem, da + 4, db + 4, d_hi, idesc, 1u);
          umma2_f16_lo_w(lead, d_tmem, da + 6, db + 6, d_hi, idesc, 1u);
          umma_commit_pair_w(lead, fb + eoff);
          fb += 8u;
          da += st_off;
          const bool wrap = fb == fb_end;
          fb = wrap ? bars : fb;
          da = wrap ? da0 : da;
          ph ^= wrap ? 1u : 0u;
        }
        if (ok) umma_commit_pair_w(lead, acc_full(buf));
      }
    }
    __syncwarp();
  } else {
    // ---- epilogue (both CTAs): this CTA's 128 output columns x all MT rows of the pair's tile ----
    const int ew = warp - 2, quad = warp & 3, half = ew >> 2;
    uint32_t lt = 0, slab_turn = 0, res_turn = 0;
    const uint32_t slab_f32 = slabs + (uint32_t)(ew * p.nslab) * 2048u, slab_f16 = slabs + p.slab_f16_off + (uint32_t)(ew * p.nslab) * 1024u;
    bool ok = true;
    for (int tile = pair; tile < num_tiles && ok; tile += npairs, lt++) {
      const int tn2 = tile % tiles_n2, tm = tile / tiles_n2;
      const int n0 = (tn2 * 2 + (int)rank) * 128, m0 = tm * p.MT;
      const uint32_t buf = lt & 1, use = lt >> 1;
      ok = mbar_wait(acc_full(buf), use & 1, p.wait_limit);
      if (!ok && lane == 0) set_abort(13, tile);
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0 && !aborted();
      if (!ok) break;
      tc_fence_after();
      const uint32_t lane_addr = tmem_base + buf * acc_stride + ((uint32_t)(quad * 32) << 16);
      if (p.tma_add)
        epilogue_tile_resadd(p, lane_addr, n0, m0, quad, lane, half, 0, 0, &map_o, &map_o16, &map_add, slab_f32, slab_f16,
                             slabs + p.slab_res_off + (uint32_t)(ew * kResSlabs) * 2048u, res_bars + (uint32_t)(ew * kResSlabs) * 8u,
                             slab_turn, res_turn);
      else if (!p.rowscale && !p.rowbias && p.add)
        epilogue_tile_fast<false, true>(p, lane_addr, n0, m0, quad, lane, half, p.out, 0, 0, &map_o, &map_o16, slab_f32, slab_f16,
                                        slab_turn);
      else if (!p.rowscale && !p.rowbias)
        epilogue_tile_fast<false, false>(p, lane_addr, n0, m0, quad, lane, half, p.out, 0, 0, &map_o, &map_o16, slab_f32, slab_f16,
                                         slab_turn);
      else
        epilogue_tile<0, false>(p, lane_addr, n0, m0, quad, lane, half, p.out, 0, 0, 0u, &map_o, &map_o16, slab_f32,
                                slab_f16, slab_turn, 0u);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_remote(acc_empty(buf), 0);
    }
    if (p.tma_out && lane == 0) tma_store_wait_all();
    __syncwarp();
  }

  // ---- teardown: neither CTA leaves while the other may still read its shared memory or TMEM ----
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (aborted()) {
    for (int i = 0; i < 1000; i++) __nanosleep(1000);
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc2(tmem_base, tmem_cols);
  }
}

// ---- prepasses (write the box-contiguous layouts described at the top) --------------------------

// f32 [M][K] -> f16 Ap[k/64][m][k%64], K tail zero padded.
__global__ void k_prep_a_f16(const float *__restrict__ a, int M, int K, int nch, __half *__restrict__ out) {
  fa_grid_dep_sync();
  const size_t total = (size_t)nch * M * 32;  // half2 pairs
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int pr = (int)(i % 32), m = (int)((i / 32) % M), c = (int)(i / ((size_t)32 * M));
    const int k = c * 64 + pr * 2;
    const float *row = a + (size_t)m * K;
    float x = k < K ? row[k] : 0.0f, y = k + 1 < K ? row[k + 1] : 0.0f;
    ((__half2 *)out)[i] = __floats2half2_rn(x, y);
  }
}

// bq [N][nblk][16] -> nibble tiles [n/128][k/64][n%128][32 B] (same 4-bit payload, tile-contiguous: a K chunk of
// a 128-row tile read from the uploaded layout is 128 separate 32-byte pieces, one DRAM access each).
__global__ void k_nbits_tiles(const uint4 *__restrict__ bq, int N, int nblk, int tiles_n, int num_kb, uint4 *__restrict__ out) {
  const size_t total = (size_t)tiles_n * num_kb * 128 * 2;  // 16-byte pieces = one 32-weight block each
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int hb = (int)(i & 1), r = (int)((i >> 1) & 127);
    const size_t tk = i >> 8;
    const int kb = (int)(tk % num_kb), tn = (int)(tk / num_kb);
    const int n = tn * 128 + r, blk = kb * 2 + hb;
    out[i] = (n < N && blk < nblk) ? bq[(size_t)n * nblk + blk] : make_uint4(0u, 0u, 0u, 0u);
  }
}

__global__ void k_nbits_side(const float *__restrict__ scales, const uint8_t *__restrict__ zp, int N, int nblk, int zpb,
                             float *__restrict__ scales_t, uint8_t *__restrict__ zp_t) {
  const size_t total = (size_t)N * nblk;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int n = (int)(i % N), blk = (int)(i / N);
    scales_t[i] = scales[(size_t)n * nblk + blk];
    const unsigned zb = zp[(size_t)n * zpb + (blk >> 1)];
    zp_t[i] = (uint8_t)((blk & 1) ? (zb >> 4) : (zb & 15u));
  }
}

// The reverse of k_prep_a_f16: packed f16 Ap[k/64][m][k%64] -> f32 [M][K] (fills a lazy tensor's f32 storage).
__global__ void k_unpack_a_f16(const __half *__restrict__ packed, int M, int K, int nch, float *__restrict__ out) {
  fa_grid_dep_sync();
  const size_t total = (size_t)nch * M * 32;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int pr = (int)(i % 32), m = (int)((i / 32) % M), c = (int)(i / ((size_t)32 * M));
    const int k = c * 64 + pr * 2;
    const float2 v = __half22float2(((const __half2 *)packed)[i]);
    float *row = out + (size_t)m * K;
    if (k < K) row[k] = v.x;
    if (k + 1 < K) row[k + 1] = v.y;
  }
}

// f32 [M][K] -> f16 Ap[k/64][m][64] for the int4 variant: inside every group of 8 the order of k is
// 0,4,1,5,2,6,3,7, the order its in-kernel nibble unpack produces.
__global__ void k_prep_a_f16_perm8(const float *__restrict__ a, int M, int K, int nch, __half *__restrict__ out) {
  fa_grid_dep_sync();
  const size_t total = (size_t)nch * M * 32;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int pr = (int)(i % 32), m = (int)((i / 32) % M), c = (int)(i / ((size_t)32 * M));
    const int k = c * 64 + (pr >> 2) * 8 + (pr & 3);  // pair j of group g holds k = 8g + j and 8g + j + 4
    const float *row = a + (size_t)m * K;
    const float x = k < K ? row[k] : 0.0f, y = k + 4 < K ? row[k + 4] : 0.0f;
    ((__half2 *)out)[i] = __floats2half2_rn(x, y);
  }
}

// f32 [M][K] -> two f16 planes Ap[2][k/64][m][k%64]: hi = f16(a), lo = f16(a - hi).  hi + lo carries about
// 22 bits of a, so a product that accumulates both planes in f32 is as accurate as an f32-activation one.
__global__ void k_prep_a_f16_hilo(const float *__restrict__ a, int M, int K, int nch, __half *__restrict__ out) {
  fa_grid_dep_sync();
  const size_t total = (size_t)nch * M * 32;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int pr = (int)(i % 32), m = (int)((i / 32) % M), c = (int)(i / ((size_t)32 * M));
    const int k = c * 64 + pr * 2;
    const float *row = a + (size_t)m * K;
    const float x = k < K ? row[k] : 0.0f, y = k + 1 < K ? row[k + 1] : 0.0f;
    const __half2 hi = __floats2half2_rn(x, y);
    const float2 hf = __half22float2(hi);
    ((__half2 *)out)[i] = hi;
    ((__half2 *)out)[total + i] = __floats2half2_rn(x - hf.x, y - hf.y);
  }
}

// f32 [M][K] -> two f32 planes Ap[2][k/32][m][k%32] for the kind::tf32 product: the value as is (the MMA reads its top
// 19 bits) and what that truncation drops, a - trunc19(a), exact in f32.
__global__ void k_prep_a_tf32(const float *__restrict__ a, int M, int K, int nch, float *__restrict__ out) {
  fa_grid_dep_sync();
  const size_t total = (size_t)nch * M * 32;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int kk = (int)(i % 32), m = (int)((i / 32) % M), c = (int)(i / ((size_t)32 * M));
    const int k = c * 32 + kk;
    const float x = k < K ? a[(size_t)m * K + k] : 0.0f;
    out[i] = x;
    out[total + i] = x - __uint_as_float(__float_as_uint(x) & 0xFFFFE000u);
  }
}

// f32 [K][N] -> Wp[2][n/128][k/32][n%128][k%32] (value plane, residue plane), 32x32 tiles through shared memory;
// the destination was zero-filled.
__global__ void k_pack_w_tf32(const float *__restrict__ w, int K, int N, int nch, size_t plane, float *__restrict__ out) {
  __shared__ float t[32][33];
  const int k0 = blockIdx.x * 32, n0 = blockIdx.y * 32;
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    int k = k0 + r, n = n0 + threadIdx.x;
    t[r][threadIdx.x] = (k < K && n < N) ? w[(size_t)k * N + n] : 0.0f;
  }
  __syncthreads();
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    int n = n0 + r, k = k0 + threadIdx.x;
    if (n < N && k < K) {
      const float x = t[threadIdx.x][r];
      const size_t o = (((size_t)(n >> 7) * nch + (k >> 5)) * 128 + (n & 127)) * 32 + (k & 31);
      out[o] = x;
      out[plane + o] = x - __uint_as_float(__float_as_uint(x) & 0xFFFFE000u);
    }
  }
}

// One CTA per activation row: s = max|a|/127 (1 when the row is all zero), r = a/s,
// q1 = rint(r), q2 = rint((r-q1)*128), q3 = rint(((r-q1)*128-q2)*128); planes Ap[limb][k/128][m][k%128].
// With one limb this is the usual symmetric per-row int8 quantiser; each further limb adds 7 bits.
__global__ void __launch_bounds__(256) k_prep_a_i8(const float *__restrict__ a, int M, int K, int nch, int limbs,
                                                   int8_t *__restrict__ out, float *__restrict__ rowscale) {
  __shared__ float red[8];
  fa_grid_dep_sync();
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
  const size_t plane = (size_t)nch * M * 128;
  for (int k = threadIdx.x; k < nch * 128; k += blockDim.x) {
    const size_t o = ((size_t)(k >> 7) * M + m) * 128 + (k & 127);
    float r = k < K ? row[k] / s : 0.0f;
    float q1 = fminf(fmaxf(rintf(r), -127.0f), 127.0f);
    out[o] = (int8_t)q1;
    if (limbs > 1) {
      float r1 = (r - q1) * 128.0f;  // exact: |r-q1| <= 0.5, scaling by 2^7
      float q2 = rintf(r1);
      out[plane + o] = (int8_t)q2;
      if (limbs > 2) out[2 * plane + o] = (int8_t)rintf((r1 - q2) * 128.0f);
    }
  }
}

// int8 [M][K] (already quantised by the caller) -> Ap[0][k/128][m][k%128].
__global__ void k_pack_a_i8_raw(const int8_t *__restrict__ aq, int M, int K, int nch, int8_t *__restrict__ out) {
  const size_t total = (size_t)nch * M * 128;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int kk = (int)(i & 127), m = (int)((i >> 7) % M), c = (int)((i >> 7) / M);
    const int k = c * 128 + kk;
    out[i] = k < K ? aq[(size_t)m * K + k] : (int8_t)0;
  }
}

// int8 [K][N] (reference byte order k*N+n) -> Wp[n/128][k/128][n%128][k%128].  32x32 tiles through smem;
// the destination was zero-filled, so padding rows/columns stay zero.
__global__ void k_pack_w_i8(const int8_t *__restrict__ w, int K, int N, int nch, int8_t *__restrict__ out) {
  __shared__ int8_t t[32][33];
  const int k0 = blockIdx.x * 32, n0 = blockIdx.y * 32;
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    int k = k0 + r, n = n0 + threadIdx.x;
    t[r][threadIdx.x] = (k < K && n < N) ? w[(size_t)k * N + n] : (int8_t)0;
  }
  __syncthreads();
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    int n = n0 + r, k = k0 + threadIdx.x;
    if (n < N && k < K) out[(((size_t)(n >> 7) * nch + (k >> 7)) * 128 + (n & 127)) * 128 + (k & 127)] = t[threadIdx.x][r];
  }
}

// int8 [K][N] (reference byte order k*N+n) -> Wp8[n/128][k/64][n%128][k%64] for the f16-activation route (KIND 5): the K
// chunks of the f16 kernels, one byte per weight.  The destination was zero-filled.
__global__ void k_pack_w_i8_k64(const int8_t *__restrict__ w, int K, int N, int nch, int8_t *__restrict__ out) {
  __shared__ int8_t t[32][33];
  const int k0 = blockIdx.x * 32, n0 = blockIdx.y * 32;
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    int k = k0 + r, n = n0 + threadIdx.x;
    t[r][threadIdx.x] = (k < K && n < N) ? w[(size_t)k * N + n] : (int8_t)0;
  }
  __syncthreads();
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    int n = n0 + r, k = k0 + threadIdx.x;
    if (n < N && k < K) out[(((size_t)(n >> 7) * nch + (k >> 6)) * 128 + (n & 127)) * 64 + (k & 63)] = t[threadIdx.x][r];
  }
}

// f32 or f16 [K][N] -> f16 Wp[n/128][k/64][n%128][k%64].
template <typename SRC>
__global__ void k_pack_w_f16(const SRC *__restrict__ w, int K, int N, int nch, __half *__restrict__ out,
                             size_t src_stride = 0, size_t dst_stride = 0) {
  __shared__ __half t[32][33];
  const int k0 = blockIdx.x * 32, n0 = blockIdx.y * 32;
  w += (size_t)blockIdx.z * src_stride;  // blockIdx.z = matrix of a batch
  out += (size_t)blockIdx.z * dst_stride;
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    int k = k0 + r, n = n0 + threadIdx.x;
    float v = 0.0f;
    if (k < K && n < N) v = (float)w[(size_t)k * N + n];
    t[r][threadIdx.x] = __float2half_rn(v);
  }
  __syncthreads();
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    int n = n0 + r, k = k0 + threadIdx.x;
    if (n < N && k < K) out[(((size_t)(n >> 7) * nch + (k >> 6)) * 128 + (n & 127)) * 64 + (k & 63)] = t[threadIdx.x][r];
  }
}

// int4 MatMulNBits payload -> f16 Wp: w = (q - zp) * scale rounded to f16 once.
// One thread per 16-byte block (32 weights = half a 128-byte row of the packed layout).
__global__ void k_pack_w_nbits(const uint8_t *__restrict__ bq, const float *__restrict__ scales,
                               const uint8_t *__restrict__ zp, int N, int K, int nblk, int zpb, int nch,
                               __half *__restrict__ out) {
  const size_t total = (size_t)N * nblk;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int n = (int)(i / nblk), blk = (int)(i % nblk);
    __half2 vals[16];
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
    uint4 *dst = (uint4 *)(out + (((size_t)(n >> 7) * nch + (blk >> 1)) * 128 + (n & 127)) * 64 + (blk & 1) * 32);
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

int grid_for(fa_ctx *ctx, size_t n, int block, int per_sm) {
  size_t g = (n + block - 1) / block, cap = (size_t)ctx->sm_count * per_sm;
  return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}

template <int KIND>
int launch_tc(fa_ctx *ctx, const void *w_packed, const void *a_packed, int limbs, void *out, bool raw_i32, int M, int N,
              int K, const TcEpilogue &ep) {
  const int elem = KIND == 1 ? 1 : (KIND == 4 ? 4 : 2);
  TcParams p{};
  p.M = M;
  p.N = N;
  p.K = K;
  p.limbs = limbs;
  p.limb_sum = (KIND != 1 && limbs == 2) ? 1 : 0;
  p.nb_scales = ep.nb_scales;
  p.nb_zp = ep.nb_zp;
  p.nblk = ep.nblk;
  p.num_kb = fa_tc_chunks(K, elem);
  // activation rows per tile: as many as fit 256 MMA-N columns, rounded to 16, no more than needed
  int mt_max = (256 / limbs) / 16 * 16;
  int mt = ((M + 15) / 16) * 16;
  p.MT = mt < mt_max ? mt : mt_max;
  p.tiles_n = ceil_div(N, 128);
  if (M > mt_max) {
    // Several row tiles: pick the tile height that minimises (rounds over the SMs) x (bytes a tile pulls per
    // K chunk, 128 weight rows + MT activation rows) - a full last wave matters more than the tallest tile.
    const long long batches = ep.batches > 0 ? ep.batches : 1;
    long long best = -1;
    for (int cand = mt_max; cand >= 64; cand -= 16) {
      const long long tiles = (long long)p.tiles_n * ceil_div(M, cand) * batches;
      const long long cost = ((tiles + ctx->sm_count - 1) / ctx->sm_count) * (128 + cand * limbs);
      if (best < 0 || cost < best) {
        best = cost;
        p.MT = cand;
      }
    }
  }
  p.tiles_m = ceil_div(M, p.MT);
  p.batches = ep.batches;
  p.w_batch_mod = ep.w_batch_mod;
  p.a_shared = ep.a_shared ? 1 : 0;
  p.n_peers = ep.n_peers;
  for (int i = 0; i < 7; i++) p.peer_out[i] = i < ep.n_peers ? ep.peer_out[i] : nullptr;
  p.o_div = ep.o_div > 0 ? ep.o_div : 1;
  p.ldc = ep.ldc > 0 ? ep.ldc : N;
  p.o_hi = ep.o_hi;
  p.o_lo = ep.o_lo;
  p.out16 = ep.out16;
  p.skip_f32 = (ep.skip_f32 && ep.out16) ? 1 : 0;
  p.o16_rows = ep.o16_rows > 0 ? ep.o16_rows : M;
  p.o16_row_hi = ep.o16_row_hi;
  p.o16_col_lo = ep.o16_col_lo;
  int num_tiles = p.tiles_n * p.tiles_m * p.batches;
  // Products whose tiles fit one wave of the SMs (decode sizes, thin encoder shapes) are bound by what ONE thread
  // block can pull from L2 / HBM (measured ~120 GB/s per SM) on top of a fixed launch-and-ramp cost, so the aim is
  // as many busy SMs as possible without a second wave: first shorter row tiles (no reduction needed), then K split
  // over a cluster of 2, 4 or 8 CTAs whose partial tiles meet in shared memory.  Measured on 24 thin shapes: a
  // second wave costs more than any split saves; clusters of 3, 5, 6, 7 place badly on the GPCs (2x slower);
  // fewer than 4 K chunks per CTA no longer pays for the reduction.
  // (the split-K finish stores rows at pitch N: a caller-chosen pitch keeps the one-CTA-per-tile form)
  p.splitk = 1;
  p.kb_per_split = p.num_kb;
  const bool split_ok = !raw_i32 && !ep.out16 && ep.n_peers == 0 && (ep.ldc == 0 || ep.ldc == N) && p.batches == 1;
  if (split_ok && num_tiles <= ctx->sm_count) {
    const int mt_hi = p.MT;
    int best_mt = p.MT, best_s = 1;
    // shortest row tile of at least 64 rows (or the whole of a shorter M) whose tiles still fit one wave
    for (int cand = mt_hi; cand >= (mt_hi < 64 ? mt_hi : 64); cand -= 16) {
      if ((long long)p.tiles_n * ceil_div(M, cand) > ctx->sm_count) break;
      best_mt = cand;
    }
    while (best_mt > 16 && ceil_div(M, best_mt - 16) == ceil_div(M, best_mt)) best_mt -= 16;  // same tiling, less padding
    // K split (tiles of at most 64 rows: the reduction of taller tiles costs more than the split saves): the widest
    // power-of-two cluster that keeps one wave and at least 4 K chunks per CTA
    if (best_mt <= 64) {
      const long long tiles = (long long)p.tiles_n * ceil_div(M, best_mt);
      for (int sp = 2; sp <= 8; sp *= 2) {
        if (tiles * sp > ctx->sm_count || p.num_kb / sp < 4) break;
        best_s = sp;
      }
    }
    if (ctx->tc_tile_rows > 0 || ctx->tc_split_k > 0) {  // tuning overrides (options "tc_tile_rows", "tc_split_k")
      if (ctx->tc_tile_rows > 0) best_mt = ((ctx->tc_tile_rows + 15) / 16) * 16 < mt_hi ? ((ctx->tc_tile_rows + 15) / 16) * 16 : mt_hi;
      best_s = ctx->tc_split_k > 0 ? ctx->tc_split_k : 1;
      if (best_mt > kSplitMaxMT) best_s = 1;
      while (best_s > 1 && p.num_kb / best_s < 2) best_s--;
      if (best_s > 1) best_s = ceil_div(p.num_kb, ceil_div(p.num_kb, best_s));
    }
    p.MT = best_mt;
    p.tiles_m = ceil_div(M, p.MT);
    if (best_s > 1) {
      p.kb_per_split = ceil_div(p.num_kb, best_s);
      p.splitk = best_s;
    }
    num_tiles = p.tiles_n * p.tiles_m * p.batches;
  }
  // Many tiles: CTA pairs (see k_tc_gemm_pair).  Row tile by the same rule as above over half as many workers,
  // with a per-tile constant for the ramp of a tile's first loads.
  bool pair = false;
  if (KIND == 0 && ctx->tc_pair && limbs == 1 && p.batches == 1 && p.splitk == 1 && ep.n_peers == 0 && !raw_i32 && (N & 255) == 0 &&
      M >= 512 && num_tiles > ctx->sm_count && ctx->sm_count >= 2) {
    pair = true;
    const int npairs = ctx->sm_count / 2;
    long long best = -1;
    for (int cand = 256; cand >= 128; cand -= 16) {
      const long long tiles = (long long)(p.tiles_n / 2) * ceil_div(M, cand);
      const long long cost = ((tiles + npairs - 1) / npairs) * (cand + 24);
      if (best < 0 || cost < best) {
        best = cost;
        p.MT = cand;
      }
    }
    if (ctx->tc_tile_rows >= 128 && ctx->tc_tile_rows <= 256) p.MT = ctx->tc_tile_rows / 16 * 16;
    p.tiles_m = ceil_div(M, p.MT);
    num_tiles = (p.tiles_n / 2) * p.tiles_m;  // pair tiles
  }
  const size_t stage_bytes = pair ? (size_t)kPTileBytes + (size_t)(p.MT / 2) * kRowBytes :
      (size_t)(KIND == 4 ? 2 : 1) * kPTileBytes + (size_t)p.MT * limbs * kRowBytes + (size_t)tc_raw_bytes<KIND>();
  p.w_lo_rows = KIND == 4 ? p.tiles_n * p.num_kb * 128 : 0;
  // Results through shared-memory slabs and TMA stores: plain products only (see epilogue_tile), and only where the
  // copy engine's alignment rules hold (16-byte row pitch and base address).
  p.split_rb = p.splitk > 1 ? ceil_div(ceil_div(p.MT, 16), p.splitk) : 0;
  p.tma_out = (ctx->tc_tma_store && (KIND <= 1 || KIND == 4 || KIND == 5) && !raw_i32 && p.splitk == 1 && p.batches == 1 && ep.n_peers == 0 && (p.ldc & 3) == 0 &&
               ((uintptr_t)out & 15) == 0 && (!ep.out16 || ((uintptr_t)ep.out16 & 127) == 0) && M >= 16)
                  ? 1
                  : 0;
  // the residual through the copy engine (epilogue_tile_resadd): the plain f16 product with an f32 result and TMA stores
  const bool want_add = KIND == 0 && p.tma_out && ep.add && !p.skip_f32 && !ep.rowscale && !ep.rowbias && (N & 3) == 0 && K <= 2048 &&
                        ((uintptr_t)ep.add & 15) == 0 && ctx->tc_tma_add;
  // two store slabs per warp and result kind, four when that leaves the ring as deep
  auto slab_bytes_for = [&](int nslab) {
    const size_t f16_off = p.skip_f32 ? 0 : (size_t)kEpiWarps * nslab * 2048;
    return p.tma_out ? f16_off + (p.out16 ? (size_t)kEpiWarps * nslab * 1024 : 0) + 128 : (size_t)0;
  };
  const size_t res_bytes = want_add ? (size_t)kEpiWarps * kResSlabs * 2048 : 0;
  const size_t tail_fixed = (size_t)(3 * 12 + 4) * 8 + 16 + (p.splitk > 1 ? (size_t)p.splitk * p.split_rb * 16 * 128 * 4 : 0) + 1024 +
                            (want_add ? (size_t)kEpiWarps * kResSlabs * 8 : 0) + res_bytes;
  const int st2 = (int)((227 * 1024 - tail_fixed - slab_bytes_for(2)) / stage_bytes), st4 = (int)((227 * 1024 - tail_fixed - slab_bytes_for(kSlabsMax)) / stage_bytes);
  p.nslab = (p.tma_out && (st4 == st2 || st4 >= 12)) ? kSlabsMax : 2;
  p.tma_add = want_add ? 1 : 0;
  p.slab_res_off = (uint32_t)(slab_bytes_for(p.nslab) - 128);
  p.slab_f16_off = p.skip_f32 ? 0u : (uint32_t)(kEpiWarps * p.nslab) * 2048u;
  const size_t slab_bytes = slab_bytes_for(p.nslab);
  const size_t tail_bytes = tail_fixed + slab_bytes;
  int stages = (int)((227 * 1024 - tail_bytes) / stage_bytes);
  if (stages > 12) stages = 12;
  const int kb_per_cta = p.kb_per_split * ceil_div(num_tiles, p.splitk > 1 ? num_tiles : (pair ? ctx->sm_count / 2 : ctx->sm_count));
  if (stages > kb_per_cta) stages = kb_per_cta;
  if (stages < 1) stages = 1;
  p.stages = stages;
  p.raw_i32 = raw_i32 ? 1 : 0;
  p.out = (float *)out;
  p.rowscale = ep.rowscale;
  p.colscale = ep.colscale;
  p.bias = ep.bias;
  p.add = ep.add;
  p.rowbias = ep.rowbias;
  p.act = ep.act;
  p.status = ctx->dev_status;
  p.wait_limit = ctx->wait_limit;
  p.withhold_kb = ctx->tc_withhold_chunk;
  ctx->tc_withhold_chunk = -1;  // one launch only
  const size_t smem = stage_bytes * stages + tail_bytes;

  CUtensorMap map_w, map_a;
  // weights: rows of 128 bytes, (tiles_n * num_kb * 128) of them, boxes of 128 rows
  const uint64_t w_batches = p.w_batch_mod ? p.w_batch_mod : p.batches;
  if (KIND == 5)  // int8 tiles [n/128][k/64][n%128][64 B]: one contiguous 8 KB run each, as 32 rows of 256 bytes
    FA_TRY(tc::make_tmap_bytes2d(ctx, &map_w, w_packed, 256, (uint64_t)p.tiles_n * p.num_kb * 32, 256, 32));
  else if (KIND == 2)  // nibble tiles [n/128][k/64][n%128][32 B]: a tile is one contiguous 4 KB run, described to the copy
                  // engine as 16 rows of 256 bytes (as 128 rows of 32 bytes it cost the engine ~0.5 us per tile)
    FA_TRY(tc::make_tmap_bytes2d(ctx, &map_w, w_packed, 256, (uint64_t)p.tiles_n * p.num_kb * 16, 256, 16));
  else
    FA_TRY(tc::make_tmap_rows128(ctx, &map_w, w_packed, elem, (KIND == 4 ? 2 : 1) * w_batches * p.tiles_n * p.num_kb * 128, 0, 128));
  // activations: [limbs * num_kb] slabs of M rows of 128 bytes, boxes of MT rows (rows >= M read as zero)
  FA_TRY(tc::make_tmap_rows128(ctx, &map_a, a_packed, elem, (uint64_t)M,
                               (uint64_t)(p.a_shared ? 1 : p.batches) * limbs * p.num_kb, (uint32_t)(pair ? p.MT / 2 : p.MT)));
  CUtensorMap map_o = map_w, map_o16 = map_w;  // placeholders when unused (never dereferenced then)
  if (p.tma_out) {
    if (!p.skip_f32) FA_TRY(tc::make_tmap_out_f32(ctx, &map_o, (const float *)out, (uint64_t)M, (uint64_t)N, (uint64_t)p.ldc));
    if (p.out16) FA_TRY(tc::make_tmap_out_f16_packed(ctx, &map_o16, p.out16, (uint64_t)p.o16_rows, (uint64_t)(N >> 6)));
  }
  CUtensorMap map_add = map_w;
  if (p.tma_add) FA_TRY(tc::make_tmap_out_f32(ctx, &map_add, ep.add, (uint64_t)M, (uint64_t)N, (uint64_t)N));
  cudaLaunchConfig_t cfg{};
  cudaLaunchAttribute attr[2];
  cfg.blockDim = dim3(tc_threads<KIND>());
  cfg.dynamicSmemBytes = smem;
  cfg.stream = ctx->stream;
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;  // see fa_launch_dep
  attr[0].val.programmaticStreamSerializationAllowed = ctx->pdl ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (pair) {
    FA_CHECK_CUDA(ctx, cudaFuncSetAttribute(k_tc_gemm_pair, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    const int npairs = ctx->sm_count / 2;
    cfg.gridDim = dim3(2 * (num_tiles < npairs ? num_tiles : npairs));
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = 2;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    cfg.numAttrs = 2;
    {
      LaunchScope ls(ctx, "tc_gemm_f16_pair");
      cudaError_t e = cudaLaunchKernelEx(&cfg, k_tc_gemm_pair, map_w, map_a, map_o, map_o16, map_add, p);
      if (e != cudaSuccess) return fa_fail(ctx, FA_ERR_CUDA, "launch tc_gemm_pair: %s", cudaGetErrorString(e));
    }
    FA_LAUNCH_CHECK(ctx, "tc_gemm_pair");
    return FA_OK;
  }
  FA_CHECK_CUDA(ctx, cudaFuncSetAttribute(k_tc_gemm<KIND>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
  if (p.splitk > 1) {
    cfg.gridDim = dim3(num_tiles, 1, p.splitk);
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = 1;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = p.splitk;
    cfg.numAttrs = 2;
  } else {
    cfg.gridDim = dim3(num_tiles < ctx->sm_count ? num_tiles : ctx->sm_count);  // persistent: one CTA per SM
  }
  {
    LaunchScope ls(ctx, KIND == 0 ? "tc_gemm_f16" : (KIND == 1 ? "tc_gemm_i8" : (KIND == 2 ? "tc_gemm_nbits" : (KIND == 4 ? "tc_gemm_tf32x3" : (KIND == 5 ? "tc_gemm_i8w_f16a" : "tc_gemm_f16_scatter")))));
    cudaError_t e = cudaLaunchKernelEx(&cfg, k_tc_gemm<KIND>, map_w, map_a, map_o, map_o16, map_add, p);
    if (e != cudaSuccess) return fa_fail(ctx, FA_ERR_CUDA, "launch tc_gemm: %s", cudaGetErrorString(e));
  }
  FA_LAUNCH_CHECK(ctx, "tc_gemm");
  return FA_OK;
}

}  // namespace

// Tensor of 128-byte rows: `slabs` == 0 gives a 2-d map [rows][128 B]; otherwise a 3-d map
// [slabs][rows][128 B] with slabs stored back to back.  Boxes are box_rows x 128 bytes, swizzled.
int tc::make_tmap_rows128(fa_ctx *ctx, CUtensorMap *out, const void *base, int elem_bytes, uint64_t rows, uint64_t slabs,
                          uint32_t box_rows) {
  PFN_encodeTiled enc = get_encode();
  if (!enc) return fa_fail(ctx, FA_ERR_CUDA, "cuTensorMapEncodeTiled is unavailable in this driver");
  FA_REQUIRE(ctx, ((uintptr_t)base & 127) == 0, "tensor-core operand %p is not 128-byte aligned", base);
  const cuuint32_t rank = slabs == 0 ? 2 : 3;
  const cuuint32_t inner = (cuuint32_t)(kRowBytes / elem_bytes);
  cuuint64_t dims[3] = {inner, rows, slabs ? slabs : 1};
  cuuint64_t strides[2] = {(cuuint64_t)kRowBytes, rows * (cuuint64_t)kRowBytes};
  cuuint32_t box[3] = {inner, box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(out, elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : (elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_UINT8), rank,
                   const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fa_fail(ctx, FA_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return FA_OK;
}

// Plain byte matrix [rows][row_bytes] (row_bytes a multiple of 16), boxes of box_rows x box_bytes, no swizzle;
// bytes past either end read as zero.
int tc::make_tmap_bytes2d(fa_ctx *ctx, CUtensorMap *out, const void *base, uint64_t row_bytes, uint64_t rows,
                          uint32_t box_bytes, uint32_t box_rows) {
  PFN_encodeTiled enc = get_encode();
  if (!enc) return fa_fail(ctx, FA_ERR_CUDA, "cuTensorMapEncodeTiled is unavailable in this driver");
  FA_REQUIRE(ctx, ((uintptr_t)base & 15) == 0 && (row_bytes & 15) == 0 && (box_bytes & 15) == 0,
             "byte tensor %p with rows of %llu bytes is not 16-byte aligned", base, (unsigned long long)row_bytes);
  cuuint64_t dims[2] = {row_bytes, rows};
  cuuint64_t strides[1] = {row_bytes};
  cuuint32_t box[2] = {box_bytes, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fa_fail(ctx, FA_ERR_CUDA, "cuTensorMapEncodeTiled (bytes) failed with CUresult %d", (int)r);
  return FA_OK;
}

int tc::make_tmap_out_f32(fa_ctx *ctx, CUtensorMap *out, const float *base, uint64_t rows, uint64_t cols, uint64_t ld) {
  PFN_encodeTiled enc = get_encode();
  if (!enc) return fa_fail(ctx, FA_ERR_CUDA, "cuTensorMapEncodeTiled is unavailable in this driver");
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * 4};
  cuuint32_t box[2] = {32, 16};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float *>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fa_fail(ctx, FA_ERR_CUDA, "cuTensorMapEncodeTiled (f32 result) failed with CUresult %d", (int)r);
  return FA_OK;
}

int tc::make_tmap_out_f16_packed(fa_ctx *ctx, CUtensorMap *out, const __half *base, uint64_t rows, uint64_t chunks) {
  PFN_encodeTiled enc = get_encode();
  if (!enc) return fa_fail(ctx, FA_ERR_CUDA, "cuTensorMapEncodeTiled is unavailable in this driver");
  cuuint64_t dims[3] = {64, rows, chunks};
  cuuint64_t strides[2] = {128, rows * 128};
  cuuint32_t box[3] = {32, 16, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<__half *>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fa_fail(ctx, FA_ERR_CUDA, "cuTensorMapEncodeTiled (f16 operand result) failed with CUresult %d", (int)r);
  return FA_OK;
}

bool fa_tc_available(fa_ctx *) { return get_encode() != nullptr; }

// int4 weights as tile-contiguous nibbles with block-major scales and zero-points (fa_nbits_side) against
// activations packed by fa_prep_a_f16_perm8: the nibbles are unpacked in shared memory inside the kernel.
int fa_tc_gemm_nbits(fa_ctx *ctx, const __half *a_packed, const uint8_t *bq, const float *scales_t, const uint8_t *zp_t,
                     float *c, int M, int N, int K, int nblk) {
  TcEpilogue ep;
  ep.nb_scales = scales_t;
  ep.nb_zp = zp_t;
  ep.nblk = nblk;
  return launch_tc<2>(ctx, bq, a_packed, 1, c, false, M, N, K, ep);
}

size_t fa_nbits_tiles_bytes(int N, int K) { return (size_t)ceil_div(N, 128) * fa_tc_chunks(K, 2) * kRawTileBytes; }

// scales [N][nblk], zp nibbles [N][zpb] (even block = low nibble) -> scales_t [nblk][N], zp_t [nblk][N] bytes;
// bq -> tile-contiguous nibbles (see k_nbits_tiles).
int fa_nbits_side(fa_ctx *ctx, const uint8_t *bq, const float *scales, const uint8_t *zp, int N, int K, int nblk, int zpb,
                  uint8_t *tiles, float *scales_t, uint8_t *zp_t) {
  {
    LaunchScope ls(ctx, "nbits_tiles");
    const int tiles_n = ceil_div(N, 128), num_kb = fa_tc_chunks(K, 2);
    k_nbits_tiles<<<grid_for(ctx, (size_t)tiles_n * num_kb * 256, 256, 8), 256, 0, ctx->stream>>>(
        (const uint4 *)bq, N, nblk, tiles_n, num_kb, (uint4 *)tiles);
  }
  FA_LAUNCH_CHECK(ctx, "nbits_tiles");
  {
    LaunchScope ls(ctx, "nbits_side");
    k_nbits_side<<<grid_for(ctx, (size_t)N * nblk, 256, 8), 256, 0, ctx->stream>>>(scales, zp, N, nblk, zpb, scales_t, zp_t);
  }
  FA_LAUNCH_CHECK(ctx, "nbits_side");
  return FA_OK;
}

int fa_prep_a_f16_perm8(fa_ctx *ctx, const float *a, int M, int K, __half *out) {
  if (M == 0) return FA_OK;
  const int nch = fa_tc_chunks(K, 2);
  {
    LaunchScope ls(ctx, "prep_a_f16_perm8");
    fa_launch_dep(ctx, k_prep_a_f16_perm8, dim3(grid_for(ctx, (size_t)nch * M * 32, 256, 8)), dim3(256), 0, a, M, K, nch, out);
  }
  FA_LAUNCH_CHECK(ctx, "prep_a_f16_perm8");
  return FA_OK;
}

int fa_tc_gemm_f16(fa_ctx *ctx, const __half *a_packed, const __half *w_packed, float *c, int M, int N, int K,
                   const TcEpilogue &ep) {
  if (ep.n_peers > 0) return launch_tc<3>(ctx, w_packed, a_packed, ep.a_hilo ? 2 : 1, c, false, M, N, K, ep);
  return launch_tc<0>(ctx, w_packed, a_packed, ep.a_hilo ? 2 : 1, c, false, M, N, K, ep);
}

int fa_tc_gemm_i8(fa_ctx *ctx, const int8_t *a_packed, int limbs, const int8_t *w_packed, void *c, bool raw_i32, int M,
                  int N, int K, const TcEpilogue &ep) {
  return launch_tc<1>(ctx, w_packed, a_packed, limbs, c, raw_i32, M, N, K, ep);
}

// int8 weights x f16 activations (KIND 5): weights stay int8 in HBM, are widened to f16 in shared memory.
size_t fa_tc_i8w_weight_bytes(int N, int K) { return (size_t)ceil_div(N, 128) * fa_tc_chunks(K, 2) * kRaw8TileBytes; }
int fa_pack_w_i8_k64(fa_ctx *ctx, const int8_t *w_kn, int K, int N, int8_t *out) {
  FA_CHECK_CUDA(ctx, cudaMemsetAsync(out, 0, fa_tc_i8w_weight_bytes(N, K), ctx->stream));
  dim3 grid(ceil_div(K, 32), ceil_div(N, 32)), block(32, 8);
  {
    LaunchScope ls(ctx, "pack_w_i8_k64");
    k_pack_w_i8_k64<<<grid, block, 0, ctx->stream>>>(w_kn, K, N, fa_tc_chunks(K, 2), out);
  }
  FA_LAUNCH_CHECK(ctx, "pack_w_i8_k64");
  return FA_OK;
}
int fa_tc_gemm_i8w_f16a(fa_ctx *ctx, const __half *a_packed, const int8_t *w_packed, float *c, int M, int N, int K,
                        const TcEpilogue &ep) {
  return launch_tc<5>(ctx, w_packed, a_packed, ep.a_hilo ? 2 : 1, c, false, M, N, K, ep);
}

// f32 x f32 on the tensor cores (kind::tf32, value + residue planes on both sides; see KIND 4).
size_t fa_tc_tf32_weight_bytes(int N, int K) { return 2 * fa_tc_weight_bytes(N, K, 4); }
size_t fa_tc_tf32_act_bytes(int M, int K) { return fa_tc_act_bytes(M, K, 4, 2); }
int fa_pack_w_tf32(fa_ctx *ctx, const float *w_kn, int K, int N, float *out) {
  FA_CHECK_CUDA(ctx, cudaMemsetAsync(out, 0, fa_tc_tf32_weight_bytes(N, K), ctx->stream));
  dim3 grid(ceil_div(K, 32), ceil_div(N, 32)), block(32, 8);
  {
    LaunchScope ls(ctx, "pack_w_tf32");
    k_pack_w_tf32<<<grid, block, 0, ctx->stream>>>(w_kn, K, N, fa_tc_chunks(K, 4), fa_tc_weight_bytes(N, K, 4) / 4, out);
  }
  FA_LAUNCH_CHECK(ctx, "pack_w_tf32");
  return FA_OK;
}
int fa_prep_a_tf32(fa_ctx *ctx, const float *a, int M, int K, float *out) {
  if (M == 0) return FA_OK;
  const int nch = fa_tc_chunks(K, 4);
  {
    LaunchScope ls(ctx, "prep_a_tf32");
    fa_launch_dep(ctx, k_prep_a_tf32, dim3(grid_for(ctx, (size_t)nch * M * 32, 256, 8)), dim3(256), 0, a, M, K, nch, out);
  }
  FA_LAUNCH_CHECK(ctx, "prep_a_tf32");
  return FA_OK;
}
int fa_tc_gemm_tf32(fa_ctx *ctx, const float *a_planes, const float *w_planes, float *c, int M, int N, int K, const TcEpilogue &ep) {
  return launch_tc<4>(ctx, w_planes, a_planes, 2, c, false, M, N, K, ep);
}

int fa_prep_a_f16(fa_ctx *ctx, const float *a, int M, int K, __half *out) {
  if (M == 0) return FA_OK;
  const int nch = fa_tc_chunks(K, 2);
  {
    LaunchScope ls(ctx, "prep_a_f16");
    fa_launch_dep(ctx, k_prep_a_f16, dim3(grid_for(ctx, (size_t)nch * M * 32, 256, 8)), dim3(256), 0, a, M, K, nch, out);
  }
  FA_LAUNCH_CHECK(ctx, "prep_a_f16");
  return FA_OK;
}

int fa_unpack_a_f16(fa_ctx *ctx, const __half *packed, int M, int K, float *out) {
  if (M == 0 || K == 0) return FA_OK;
  const int nch = fa_tc_chunks(K, 2);
  {
    LaunchScope ls(ctx, "unpack_a_f16");
    fa_launch_dep(ctx, k_unpack_a_f16, dim3(grid_for(ctx, (size_t)nch * M * 32, 256, 8)), dim3(256), 0, packed, M, K, nch, out);
  }
  FA_LAUNCH_CHECK(ctx, "unpack_a_f16");
  return FA_OK;
}

int fa_prep_a_f16_hilo(fa_ctx *ctx, const float *a, int M, int K, __half *out) {
  if (M == 0) return FA_OK;
  const int nch = fa_tc_chunks(K, 2);
  {
    LaunchScope ls(ctx, "prep_a_f16_hilo");
    fa_launch_dep(ctx, k_prep_a_f16_hilo, dim3(grid_for(ctx, (size_t)nch * M * 32, 256, 8)), dim3(256), 0, a, M, K, nch, out);
  }
  FA_LAUNCH_CHECK(ctx, "prep_a_f16_hilo");
  return FA_OK;
}

int fa_prep_a_i8(fa_ctx *ctx, const float *a, int M, int K, int limbs, int8_t *out, float *rowscale) {
  if (M == 0) return FA_OK;
  {
    LaunchScope ls(ctx, "prep_a_i8");
    fa_launch_dep(ctx, k_prep_a_i8, dim3(M), dim3(256), 0, a, M, K, fa_tc_chunks(K, 1), limbs, out, rowscale);
  }
  FA_LAUNCH_CHECK(ctx, "prep_a_i8");
  return FA_OK;
}

int fa_pack_a_i8_raw(fa_ctx *ctx, const int8_t *aq, int M, int K, int8_t *out) {
  const int nch = fa_tc_chunks(K, 1);
  {
    LaunchScope ls(ctx, "pack_a_i8_raw");
    k_pack_a_i8_raw<<<grid_for(ctx, (size_t)nch * M * 128, 256, 8), 256, 0, ctx->stream>>>(aq, M, K, nch, out);
  }
  FA_LAUNCH_CHECK(ctx, "pack_a_i8_raw");
  return FA_OK;
}

int fa_pack_w_i8(fa_ctx *ctx, const int8_t *w_kn, int K, int N, int8_t *out) {
  FA_CHECK_CUDA(ctx, cudaMemsetAsync(out, 0, fa_tc_weight_bytes(N, K, 1), ctx->stream));
  dim3 grid(ceil_div(K, 32), ceil_div(N, 32)), block(32, 8);
  {
    LaunchScope ls(ctx, "pack_w_i8");
    k_pack_w_i8<<<grid, block, 0, ctx->stream>>>(w_kn, K, N, fa_tc_chunks(K, 1), out);
  }
  FA_LAUNCH_CHECK(ctx, "pack_w_i8");
  return FA_OK;
}

int fa_pack_w_f16(fa_ctx *ctx, const void *w_kn, int src_storage, int K, int N, __half *out) {
  FA_CHECK_CUDA(ctx, cudaMemsetAsync(out, 0, fa_tc_weight_bytes(N, K, 2), ctx->stream));
  dim3 grid(ceil_div(K, 32), ceil_div(N, 32)), block(32, 8);
  const int nch = fa_tc_chunks(K, 2);
  {
    LaunchScope ls(ctx, "pack_w_f16");
    if (src_storage == FA_F16)
      k_pack_w_f16<__half><<<grid, block, 0, ctx->stream>>>((const __half *)w_kn, K, N, nch, out);
    else
      k_pack_w_f16<float><<<grid, block, 0, ctx->stream>>>((const float *)w_kn, K, N, nch, out);
  }
  FA_LAUNCH_CHECK(ctx, "pack_w_f16");
  return FA_OK;
}

// `batch` f32 matrices [K][N], matrix b at w + b*src_stride -> packed slabs back to back.
int fa_pack_w_f16_batched(fa_ctx *ctx, const void *w_kn, int K, int N, int batch, size_t src_stride, __half *out) {
  const size_t slab = fa_tc_weight_bytes(N, K, 2);
  FA_CHECK_CUDA(ctx, cudaMemsetAsync(out, 0, slab * batch, ctx->stream));
  dim3 grid(ceil_div(K, 32), ceil_div(N, 32), batch), block(32, 8);
  FA_REQUIRE(ctx, batch <= 65535 && grid.y <= 65535, "pack_w_f16: batch or N too large");
  {
    LaunchScope ls(ctx, "pack_w_f16");
    k_pack_w_f16<float><<<grid, block, 0, ctx->stream>>>((const float *)w_kn, K, N, fa_tc_chunks(K, 2), out, src_stride,
                                                         slab / sizeof(__half));
  }
  FA_LAUNCH_CHECK(ctx, "pack_w_f16");
  return FA_OK;
}

int fa_pack_w_nbits_f16(fa_ctx *ctx, const uint8_t *bq, const float *scales, const uint8_t *zp, int N, int K, int nblk,
                        int zpb, __half *out) {
  FA_CHECK_CUDA(ctx, cudaMemsetAsync(out, 0, fa_tc_weight_bytes(N, K, 2), ctx->stream));
  {
    LaunchScope ls(ctx, "pack_w_nbits_f16");
    k_pack_w_nbits<<<grid_for(ctx, (size_t)N * nblk, 128, 16), 128, 0, ctx->stream>>>(bq, scales, zp, N, K, nblk, zpb,
                                                                                     fa_tc_chunks(K, 2), out);
  }
  FA_LAUNCH_CHECK(ctx, "pack_w_nbits_f16");
  return FA_OK;
}

// ---- allocation-free int8 product -------------------------------------------------------------------
//
// Some hosts of this library may not allocate device memory when they call it: a serving process that
// has already handed every remaining byte of the GPU to its own pool (so cudaMalloc can fail at any
// moment), or a real-time audio thread that must never wait on the driver's allocation lock.  For them
// fa_matmul_int8_static runs the int8 tensor-core product with all of its scratch - the packed copy of
// the weights, the int8 digit planes of the activations and the per-row scales - inside one fixed array
// that is part of the library image.  Every GPU that loads the library holds these bytes until exit.
//
// Limits (checked, FA_ERR_INVALID beyond them): M <= 512, 64 <= K <= 2048, N >= 64 and the packed weights
// (N rounded up to 128 times K rounded up to 128 bytes) <= 8 MiB.
//
// All calls share the array and it keeps the previous call's contents: this entry point rewrites every
// byte it later reads (zero padding included), and calls that overlap on the GPU - two streams, two
// contexts on one device - race on it.  Issue them on one stream.
constexpr int kStaticMaxM = 512, kStaticMaxK = 2048;
constexpr size_t kStaticWBytes = 8u << 20;
constexpr size_t kStaticABytes = (size_t)3 * kStaticMaxM * kStaticMaxK;
constexpr size_t kStaticSBytes = 4096;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticWBytes + kStaticABytes + kStaticSBytes];

// In host code `g_static_scratch` is only a handle for the runtime, not an address a kernel can use:
// the device address is looked up once per device, with that device current.
static unsigned char *g_static_scratch_dev[64] = {nullptr};

extern "C" int fa_matmul_int8_static(fa_ctx *ctx, const float *a_dev, const void *wq_kn_dev, const float *scale_dev,
                                     const float *bias_dev, int act, float *y_dev, int M, int N, int K) {
  if (!ctx) return fa_fail(ctx, FA_ERR_INVALID, "matmulInt8Static: NULL context");
  FA_REQUIRE(ctx, a_dev && wq_kn_dev && scale_dev && y_dev, "matmulInt8Static: NULL device pointer");
  FA_REQUIRE(ctx, act >= 0 && act <= 5, "matmulInt8Static: unknown activation code %d", act);
  FA_REQUIRE(ctx, M >= 1 && M <= kStaticMaxM, "matmulInt8Static: M=%d is outside 1..%d", M, kStaticMaxM);
  FA_REQUIRE(ctx, K >= 64 && K <= kStaticMaxK, "matmulInt8Static: K=%d is outside 64..%d", K, kStaticMaxK);
  FA_REQUIRE(ctx, N >= 64, "matmulInt8Static: N=%d is below 64", N);
  FA_REQUIRE(ctx, fa_tc_weight_bytes(N, K, 1) <= kStaticWBytes,
             "matmulInt8Static: packed weights need %zu bytes, the static scratch holds %zu", fa_tc_weight_bytes(N, K, 1),
             kStaticWBytes);
  FA_REQUIRE(ctx, ctx->device >= 0 && ctx->device < 64, "matmulInt8Static: device ordinal %d unsupported", ctx->device);
  FA_REQUIRE(ctx, get_encode() != nullptr, "matmulInt8Static: tensor-map encoder unavailable");
  FA_CHECK_CUDA(ctx, cudaSetDevice(ctx->device));
  if (!g_static_scratch_dev[ctx->device]) {
    // first call on this device: resolve the array's device address (do this before any stream capture)
    void *ptr = nullptr;
    FA_CHECK_CUDA(ctx, cudaGetSymbolAddress(&ptr, g_static_scratch));
    g_static_scratch_dev[ctx->device] = (unsigned char *)ptr;
  }
  unsigned char *base = g_static_scratch_dev[ctx->device];
  int8_t *w_packed = (int8_t *)base;
  int8_t *a_planes = (int8_t *)(base + kStaticWBytes);
  float *rowscale = (float *)(base + kStaticWBytes + kStaticABytes);
  const int limbs = ctx->int8_limbs;
  const bool was_profiling = ctx->profiling;  // per-launch event pairs would create events: keep them off here
  ctx->profiling = false;
  int rc = fa_pack_w_i8(ctx, (const int8_t *)wq_kn_dev, K, N, w_packed);  // zero-fills the packed region first
  if (rc == FA_OK) rc = fa_prep_a_i8(ctx, a_dev, M, K, limbs, a_planes, rowscale);
  if (rc == FA_OK) {
    TcEpilogue ep;
    ep.rowscale = rowscale;
    ep.colscale = scale_dev;
    ep.bias = bias_dev;
    ep.act = act;
    rc = launch_tc<1>(ctx, w_packed, a_planes, limbs, y_dev, false, M, N, K, ep);
  }
  ctx->profiling = was_profiling;
  return rc;
}
