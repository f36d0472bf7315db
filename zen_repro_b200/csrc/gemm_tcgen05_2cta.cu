// bf16 GEMM on tcgen05 with CTA pairs (cta_group::2): two CTAs of a cluster share one 256 x 256 output tile.
//
//   C[M, N] (+)= A[M, K] * B[N, K]^T (+ bias[N])
//
// Each CTA of the pair holds 128 rows of A and 128 of the 256 rows of the B tile; one thread of the leader CTA
// issues tcgen05.mma.cta_group::2 (M 256 x N 256 x K 16), the hardware reads both CTAs' shared memory and each
// CTA's tensor memory receives its 128 accumulator rows.  Per SM that halves the shared-memory traffic of B, which
// is what bounds the single-CTA kernel.  Roles per CTA: warp 0 TMA producer (both CTAs' loads complete on the
// leader's "full" barrier), warp 1 MMA issuer (leader only; commits are multicast to both CTAs' barriers),
// warps 2..5 epilogue.  Bounded waits everywhere; a CTA that gives up still joins the final cluster barrier.
// Operands may be K-major or MN-major as in gemm_tcgen05.cu.
#include "tc_common.cuh"
#include "tmap_util.cuh"

namespace {

using namespace tc;

constexpr int BM2 = 128;          // rows per CTA (256 per pair)
// N extent of the pair tile: 256 (default) or 128 (for outputs whose 256-wide tiles quantise badly over the 74 CTA
// pairs, e.g. 96 tiles = 1.3 waves); each CTA holds BN / 2 rows of the B tile.
constexpr int BK2 = 64;
template <int BN> struct PairCfg {
  static constexpr int BNH = BN / 2;
  static constexpr int STAGES = (BN >= 192) ? 6 : 8;
  static constexpr int TMEM_COLS = (2 * BN <= 256) ? 256 : 512;        // two accumulators; the allocation is a power of two
  static constexpr int STAGE_BYTES = 128 * 64 * 2 + BNH * 64 * 2;      // A rows of this CTA + its half of B
};
constexpr int MAX_SPLITS = 3;      // K slices per output tile at most (the last slice to arrive holds the others' partials in registers)
constexpr int EPI_STAGE_BYTES = 4 * 2 * 4096;   // per epilogue warp two [32 rows][64 bf16] boxes for the TMA store
template <int BN> constexpr int pair_smem_bytes() { return PairCfg<BN>::STAGES * PairCfg<BN>::STAGE_BYTES + EPI_STAGE_BYTES + 1024 + 256; }

__device__ int g_gemm2_error = 0;

// One GEMM of a launch.  A launch runs up to MAX_GROUP of them (same operand layouts) as ONE list of output tiles over
// the persistent clusters: small products that each fill the clusters badly (the four weight gradients of a
// transformer layer: 27 + 9 + 36 + 36 tiles on 74 clusters) then share rounds, and the fixed cost of a launch
// (pipeline fill, last epilogue) is paid once.
constexpr int MAX_GROUP = 6;
struct GemmProblem {
  CUtensorMap ta, tb, tc;
  void* C;
  const void* bias;
  int M, N, K, ldc;
  int out_fp32, accumulate;
  int tma_store;                    // bf16 output written through shared memory and TMA stores (full lines, async)
  int num_m_pairs, num_n_tiles;
  int tile_start;                   // index of this product's first tile in the launch's list
};
struct GemmGroup {
  GemmProblem pr[MAX_GROUP];
  int n, num_tiles;                 // products, tiles of all of them
  // split-K (one product only): a work unit is (output tile, K slice).  Every unit stores its fp32 partial tile in
  // `ws`; per 32-row group a counter tells the last unit to arrive, which sums the slices in slice order and writes
  // the output; with two slices and a TMA-stored output the slices exchange half an accumulator each instead.
  int splits, kb_per_split;
  // tail split (splits == 1): the last `tail` tiles of the list, the ones of the launch's final, partly filled wave
  // of clusters, are cut into two K halves that run side by side in that wave and exchange half an accumulator
  // each (the two-slice TMA-store path); 0 = every tile is one unit
  int tail;
  float* ws;                        // [slices * tiles][2 CTAs][8 column chunks][8 float4 of a row][128 rows] float4:
                                    // consecutive lanes (rows) are consecutive in memory, so a warp's store covers whole lines
  int* counters;                    // [tiles][2 CTAs][4 row groups][2], zero between launches
};

// One unit of work of a cluster: an output tile, or one K slice of it.
struct Unit {
  int pi, tile, lt, ks, kb0, kb1;   // product, tile in the launch's list, tile within the product, K slice and its blocks
  int wtile, wtiles;                // index of the tile among the split ones and their number (workspace / flag addressing)
  bool split;
};
__device__ __forceinline__ Unit decode_unit(const GemmGroup& g, int unit) {
  Unit u;
  const int T = g.num_tiles;
  if (g.tail == 0) {
    u.tile = unit % T;
    u.ks = unit / T;
    u.split = g.splits > 1;
    u.wtile = u.tile;
    u.wtiles = T;
  } else {
    const int whole = T - g.tail;
    u.wtiles = g.tail;
    if (unit < whole) {
      u.tile = unit; u.ks = 0; u.split = false; u.wtile = 0;
    } else {
      const int j = unit - whole;
      u.ks = j >= g.tail ? 1 : 0;
      u.wtile = j - u.ks * g.tail;
      u.tile = whole + u.wtile;
      u.split = true;
    }
  }
  u.pi = 0;
#pragma unroll
  for (int i = 1; i < MAX_GROUP; ++i)
    if (i < g.n && u.tile >= g.pr[i].tile_start) u.pi = i;
  u.lt = u.tile - g.pr[u.pi].tile_start;
  const int nkb = (g.pr[u.pi].K + BK2 - 1) / BK2;
  if (g.tail == 0) {
    u.kb0 = u.ks * g.kb_per_split;
    u.kb1 = min(nkb, u.kb0 + g.kb_per_split);
  } else if (!u.split) {
    u.kb0 = 0; u.kb1 = nkb;
  } else {
    const int half = (nkb + 1) / 2;
    u.kb0 = u.ks ? half : 0;
    u.kb1 = u.ks ? nkb : half;
  }
  return u;
}

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// TMA load whose completion is signalled on the pair leader's barrier (same offset, CTA-rank bit cleared).
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1) {
  const uint32_t bar_leader = smem_u32(bar) & 0xFEFFFFFFu;
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(bar_leader), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(ncols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on the barrier at this offset in BOTH CTAs of the pair once all previously issued MMAs have completed.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  const uint16_t mask = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(smem_u32(bar)), "h"(mask) : "memory");
}
// Arrive on the leader CTA's copy of a barrier from either CTA of the pair.
__device__ __forceinline__ void mbar_arrive_leader(uint64_t* bar) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, 0;" : "=r"(remote) : "r"(smem_u32(bar)));
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(remote) : "memory");
}

__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* src, int c0, int c1) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(map), "r"(smem_u32(src)), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

template <bool A_MN, bool B_MN, int BN2>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(192, 1)
gemm_bf16_2cta_kernel(const __grid_constant__ GemmGroup gg) {
  constexpr int BNH = PairCfg<BN2>::BNH, STAGES2 = PairCfg<BN2>::STAGES, STAGE_BYTES2 = PairCfg<BN2>::STAGE_BYTES;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* epi_stage = smem + STAGES2 * STAGE_BYTES2;              // 1024-byte aligned
  uint64_t* bars = reinterpret_cast<uint64_t*>(epi_stage + EPI_STAGE_BYTES);
  uint64_t* full = bars;                       // [STAGES2]   used on the leader
  uint64_t* empty = bars + STAGES2;            // [STAGES2]   one copy per CTA
  uint64_t* tfull = bars + 2 * STAGES2;        // [2]         one copy per CTA
  uint64_t* tempty = bars + 2 * STAGES2 + 2;   // [2]         used on the leader, 8 arrivals
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES2 + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  constexpr uint32_t IDESC = make_idesc(256, BN2, A_MN, B_MN);
  constexpr int A_BYTES = BM2 * BK2 * 2;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t cta = cluster_ctarank();
  const int cluster_id = blockIdx.x >> 1, num_clusters = gridDim.x >> 1;
  const int num_tiles = gg.num_tiles;
  const int num_units = gg.tail ? num_tiles + gg.tail : num_tiles * gg.splits;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES2; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&tfull[a], 1); mbar_init(&tempty[a], 8); }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) tmem_alloc_pair(tmem_slot, PairCfg<BN2>::TMEM_COLS);
  fence_before();
  __syncthreads();
  cluster_sync_all();                            // both CTAs' barriers exist before anyone signals them
  fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      // ---------------------------------------------------------------- TMA producer (both CTAs)
      uint32_t it = 0;
      bool ok = true;
      for (int unit = cluster_id; unit < num_units && ok; unit += num_clusters) {
        const Unit u = decode_unit(gg, unit);
        const GemmProblem& p = gg.pr[u.pi];
        const int m0 = (u.lt % p.num_m_pairs) * 256 + (int)cta * BM2;
        const int n0 = (u.lt / p.num_m_pairs) * BN2 + (int)cta * BNH;
        for (int kb = u.kb0; kb < u.kb1; ++kb, ++it) {
          const int s = it % STAGES2;
          const uint32_t ph = (it / STAGES2) & 1;
          if (!mbar_wait(&empty[s], ph ^ 1, abort_flag, 1, &g_gemm2_error)) { ok = false; break; }
          unsigned char* sa = smem + s * STAGE_BYTES2;
          unsigned char* sb = sa + A_BYTES;
          if (cta == 0) mbar_expect_tx(&full[s], 2 * STAGE_BYTES2);
          const int k0 = kb * BK2;
          if (!A_MN) {
            tma_load_2d_pair(sa, &p.ta, &full[s], k0, m0);
          } else {
#pragma unroll
            for (int j = 0; j < BM2 / 64; ++j) tma_load_2d_pair(sa + j * 8192, &p.ta, &full[s], m0 + 64 * j, k0);
          }
          if (!B_MN) {
            tma_load_2d_pair(sb, &p.tb, &full[s], k0, n0);
          } else {
#pragma unroll
            for (int j = 0; j < BNH / 64; ++j) tma_load_2d_pair(sb + j * 8192, &p.tb, &full[s], n0 + 64 * j, k0);
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && cta == 0) {
      // ---------------------------------------------------------------- MMA issuer (leader CTA only)
      uint32_t it = 0, tcount = 0;
      bool ok = true;
      for (int unit = cluster_id; unit < num_units && ok; unit += num_clusters, ++tcount) {
        const uint32_t acc = tcount & 1, aph = (tcount >> 1) & 1;
        if (!mbar_wait(&tempty[acc], aph ^ 1, abort_flag, 2, &g_gemm2_error)) { ok = false; break; }
        fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN2;
        const Unit u = decode_unit(gg, unit);
        const int kb0 = u.kb0, kb1 = u.kb1;
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % STAGES2;
          const uint32_t ph = (it / STAGES2) & 1;
          if (!mbar_wait(&full[s], ph, abort_flag, 3, &g_gemm2_error)) { ok = false; break; }
          fence_after();
          const uint32_t sa = smem_u32(smem + s * STAGE_BYTES2);
          const uint32_t sb = sa + A_BYTES;
          const uint64_t adesc = A_MN ? make_desc(sa, 8192, 1024) : make_desc(sa, 16, 1024);
          const uint64_t bdesc = B_MN ? make_desc(sb, 8192, 1024) : make_desc(sb, 16, 1024);
#pragma unroll
          for (int j = 0; j < BK2 / 16; ++j) {
            const uint64_t astep = (uint64_t)((A_MN ? j * 2048 : j * 32) >> 4);
            const uint64_t bstep = (uint64_t)((B_MN ? j * 2048 : j * 32) >> 4);
            umma_bf16_pair(d_tmem, adesc + astep, bdesc + bstep, IDESC, (kb != kb0 || j != 0) ? 1u : 0u);
          }
          umma_commit_pair(&empty[s]);
        }
        if (ok) umma_commit_pair(&tfull[acc]);
      }
    }
  } else {
    // -------------------------------------------------------------------- epilogue (warps 2..5, both CTAs)
    const int grp = warp & 3;
    uint32_t tcount = 0;
    bool ok = true;
    for (int unit = cluster_id; unit < num_units && ok; unit += num_clusters, ++tcount) {
      const Unit u = decode_unit(gg, unit);
      const GemmProblem& p = gg.pr[u.pi];
      const int tile = u.tile, ks = u.ks;
      const int m0 = (u.lt % p.num_m_pairs) * 256 + (int)cta * BM2, n0 = (u.lt / p.num_m_pairs) * BN2;
      const uint32_t acc = tcount & 1, aph = (tcount >> 1) & 1;
      if (!mbar_wait(&tfull[acc], aph, abort_flag, 4, &g_gemm2_error)) { ok = false; break; }
      fence_after();
      const int row = m0 + grp * 32 + lane;
      const uint32_t taddr0 = tmem_base + ((uint32_t)(grp * 32) << 16) + acc * BN2;
      const bool split = u.split;
      if (split && !p.tma_store) {
        // store this K slice's partial tile and count in.  Every slice but the last to arrive for these 32 rows is
        // done then; the last one adds the others' partials to its own accumulator, in slice order, below.
        float4* wp = reinterpret_cast<float4*>(gg.ws + ((size_t)(ks * num_tiles + tile) * 2 + cta) * (BM2 * BN2)) + (grp * 32 + lane);
#pragma unroll 1
        for (int ch = 0; ch < BN2 / 32; ch += 2) {
          uint32_t r[32], r2[32];
          tmem_ld32_nowait(taddr0 + ch * 32, r);
          tmem_ld32_nowait(taddr0 + ch * 32 + 32, r2);
          tmem_wait_ld();
          float4* dst = wp + (size_t)ch * (8 * BM2);
          float4* dst2 = wp + (size_t)(ch + 1) * (8 * BM2);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            dst[i * BM2] = make_float4(__uint_as_float(r[4 * i]), __uint_as_float(r[4 * i + 1]), __uint_as_float(r[4 * i + 2]), __uint_as_float(r[4 * i + 3]));
            dst2[i * BM2] = make_float4(__uint_as_float(r2[4 * i]), __uint_as_float(r2[4 * i + 1]), __uint_as_float(r2[4 * i + 2]), __uint_as_float(r2[4 * i + 3]));
          }
        }
        __threadfence();
        __syncwarp();
        int* cnt = gg.counters + (tile * 2 + (int)cta) * 4 + grp;
        int old = 0;
        if (lane == 0) {
          old = atomicAdd(cnt, 1);
          if (old == gg.splits - 1) *cnt = 0;           // every slice has arrived: ready for the next launch
        }
        old = __shfl_sync(0xffffffffu, old, 0);
        if (old != gg.splits - 1) {
          fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive_leader(&tempty[acc]);
          continue;
        }
        __threadfence();
      }
      if (p.tma_store) {
        // bf16 output: each warp turns its 32 rows into [32][64] boxes in shared memory (the swizzled layout of the
        // tensor map) and one lane stores each box with TMA: whole lines, clipped at the matrix edge, no waiting.
        // With two K slices each slice finishes half of the columns: it hands the other half of its accumulator to
        // the peer through the workspace, waits (bounded) for the peer's half and adds it to its own.
        unsigned char* stg = epi_stage + grp * 8192;
        int cb_lo = 0, cb_hi = BN2 / 64;
        const float4* peer = nullptr;
        if (split) {
          const int other = 1 - ks;
          float4* wp = reinterpret_cast<float4*>(gg.ws + ((size_t)(ks * u.wtiles + u.wtile) * 2 + cta) * (BM2 * BN2)) + (grp * 32 + lane);
#pragma unroll 1
          for (int ch = other * (BN2 / 64); ch < (other + 1) * (BN2 / 64); ch += 2) {
            uint32_t r[32], r2[32];
            tmem_ld32_nowait(taddr0 + ch * 32, r);
            tmem_ld32_nowait(taddr0 + ch * 32 + 32, r2);
            tmem_wait_ld();
            float4* dst = wp + (size_t)ch * (8 * BM2);
            float4* dst2 = wp + (size_t)(ch + 1) * (8 * BM2);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              dst[i * BM2] = make_float4(__uint_as_float(r[4 * i]), __uint_as_float(r[4 * i + 1]), __uint_as_float(r[4 * i + 2]), __uint_as_float(r[4 * i + 3]));
              dst2[i * BM2] = make_float4(__uint_as_float(r2[4 * i]), __uint_as_float(r2[4 * i + 1]), __uint_as_float(r2[4 * i + 2]), __uint_as_float(r2[4 * i + 3]));
            }
          }
          __threadfence();
          __syncwarp();
          // flags[..][ks] = 1: "slice ks has published its half"; the consumer clears it for the next launch
          int* flags = gg.counters + ((u.wtile * 2 + (int)cta) * 4 + grp) * 2;
          int got = 1;
          if (lane == 0) {
            atomicExch(flags + ks, 1);
            const uint64_t t0 = gtimer();
            while (atomicAdd(flags + other, 0) == 0) {
              if (*abort_flag || gtimer() - t0 > WAIT_NS) { got = 0; break; }
            }
            if (got) atomicExch(flags + other, 0);
            else { *abort_flag = 5; atomicCAS(&g_gemm2_error, 0, 5); }
          }
          got = __shfl_sync(0xffffffffu, got, 0);
          if (!got) { ok = false; break; }
          __threadfence();
          peer = reinterpret_cast<const float4*>(gg.ws + ((size_t)(other * u.wtiles + u.wtile) * 2 + cta) * (BM2 * BN2)) + (grp * 32 + lane);
          cb_lo = ks * (BN2 / 128);
          cb_hi = cb_lo + BN2 / 128;
        }
#pragma unroll 1
        for (int cb = cb_lo; cb < cb_hi; ++cb) {
          unsigned char* st = stg + (cb & 1) * 4096;
          uint32_t ra[32], rb[32];
          tmem_ld32_nowait(taddr0 + cb * 64, ra);
          tmem_ld32_nowait(taddr0 + cb * 64 + 32, rb);
          float4 oa[8], ob[8];
          if (split) {
            const float4* qa = peer + (size_t)(2 * cb) * (8 * BM2);
            const float4* qb = peer + (size_t)(2 * cb + 1) * (8 * BM2);
#pragma unroll
            for (int i = 0; i < 8; ++i) { oa[i] = __ldcg(qa + i * BM2); ob[i] = __ldcg(qb + i * BM2); }
          }
          if (lane == 0) bulk_wait_read<1>();          // the store that read this buffer two boxes ago is done
          __syncwarp();
          tmem_wait_ld();
          if (split) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              ra[4 * i] = __float_as_uint(__uint_as_float(ra[4 * i]) + oa[i].x);
              ra[4 * i + 1] = __float_as_uint(__uint_as_float(ra[4 * i + 1]) + oa[i].y);
              ra[4 * i + 2] = __float_as_uint(__uint_as_float(ra[4 * i + 2]) + oa[i].z);
              ra[4 * i + 3] = __float_as_uint(__uint_as_float(ra[4 * i + 3]) + oa[i].w);
              rb[4 * i] = __float_as_uint(__uint_as_float(rb[4 * i]) + ob[i].x);
              rb[4 * i + 1] = __float_as_uint(__uint_as_float(rb[4 * i + 1]) + ob[i].y);
              rb[4 * i + 2] = __float_as_uint(__uint_as_float(rb[4 * i + 2]) + ob[i].z);
              rb[4 * i + 3] = __float_as_uint(__uint_as_float(rb[4 * i + 3]) + ob[i].w);
            }
          }
          const int col0 = n0 + cb * 64;
          if (p.bias) {
            const __nv_bfloat16* bp = reinterpret_cast<const __nv_bfloat16*>(p.bias) + col0;
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              if (col0 + i < p.N) ra[i] = __float_as_uint(__uint_as_float(ra[i]) + __bfloat162float(bp[i]));
              if (col0 + 32 + i < p.N) rb[i] = __float_as_uint(__uint_as_float(rb[i]) + __bfloat162float(bp[32 + i]));
            }
          }
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            *reinterpret_cast<uint4*>(st + swz128(lane, q * 8)) =
                make_uint4(pack_bf16(__uint_as_float(ra[8 * q]), __uint_as_float(ra[8 * q + 1])),
                           pack_bf16(__uint_as_float(ra[8 * q + 2]), __uint_as_float(ra[8 * q + 3])),
                           pack_bf16(__uint_as_float(ra[8 * q + 4]), __uint_as_float(ra[8 * q + 5])),
                           pack_bf16(__uint_as_float(ra[8 * q + 6]), __uint_as_float(ra[8 * q + 7])));
            *reinterpret_cast<uint4*>(st + swz128(lane, 32 + q * 8)) =
                make_uint4(pack_bf16(__uint_as_float(rb[8 * q]), __uint_as_float(rb[8 * q + 1])),
                           pack_bf16(__uint_as_float(rb[8 * q + 2]), __uint_as_float(rb[8 * q + 3])),
                           pack_bf16(__uint_as_float(rb[8 * q + 4]), __uint_as_float(rb[8 * q + 5])),
                           pack_bf16(__uint_as_float(rb[8 * q + 6]), __uint_as_float(rb[8 * q + 7])));
          }
          fence_async_smem();
          __syncwarp();
          if (lane == 0) {
            if (col0 < p.N && m0 + grp * 32 < p.M) tma_store_2d(&p.tc, st, col0, m0 + grp * 32);
            bulk_commit();
          }
        }
        fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_leader(&tempty[acc]);
        continue;
      }
#pragma unroll 1
      for (int ch = 0; ch < BN2 / 32; ++ch) {
        uint32_t r[32];
        if (split) {
          // the other slices' partials of this chunk first (independent loads, all in flight together), then the
          // own accumulator; the sum runs over slice indices whichever slice arrived last
          float4 buf[MAX_SPLITS][8];
          const float4* src = reinterpret_cast<const float4*>(gg.ws + ((size_t)tile * 2 + cta) * (BM2 * BN2)) + (size_t)ch * (8 * BM2) + (grp * 32 + lane);
#pragma unroll
          for (int sidx = 0; sidx < MAX_SPLITS; ++sidx) {
            if (sidx < gg.splits && sidx != ks) {
              const float4* q = src + (size_t)sidx * num_tiles * 2 * (BM2 * BN2 / 4);
#pragma unroll
              for (int i = 0; i < 8; ++i) buf[sidx][i] = __ldcg(q + i * BM2);
            }
          }
          tmem_ld32(taddr0 + ch * 32, r);
          float a[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) a[i] = 0.f;
#pragma unroll
          for (int sidx = 0; sidx < MAX_SPLITS; ++sidx) {
            if (sidx < gg.splits) {
              const bool own = (sidx == ks);
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                a[4 * i] += own ? __uint_as_float(r[4 * i]) : buf[sidx][i].x;
                a[4 * i + 1] += own ? __uint_as_float(r[4 * i + 1]) : buf[sidx][i].y;
                a[4 * i + 2] += own ? __uint_as_float(r[4 * i + 2]) : buf[sidx][i].z;
                a[4 * i + 3] += own ? __uint_as_float(r[4 * i + 3]) : buf[sidx][i].w;
              }
            }
          }
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(a[i]);
        } else {
          tmem_ld32(taddr0 + ch * 32, r);
        }
        const int col0 = n0 + ch * 32;
        if (row < p.M && col0 < p.N) {
          float v[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
          const bool fullw = (col0 + 32 <= p.N);
          if (p.bias) {
            const __nv_bfloat16* bp = reinterpret_cast<const __nv_bfloat16*>(p.bias) + col0;
#pragma unroll
            for (int i = 0; i < 32; ++i) if (fullw || col0 + i < p.N) v[i] += __bfloat162float(bp[i]);
          }
          if (p.out_fp32) {
            float* cp = reinterpret_cast<float*>(p.C) + (size_t)row * p.ldc + col0;
            if (fullw && (p.ldc % 4 == 0)) {
#pragma unroll
              for (int i = 0; i < 32; i += 4) {
                float4 o = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
                if (p.accumulate) { const float4 c = *reinterpret_cast<const float4*>(cp + i); o.x += c.x; o.y += c.y; o.z += c.z; o.w += c.w; }
                *reinterpret_cast<float4*>(cp + i) = o;
              }
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (col0 + i < p.N) cp[i] = p.accumulate ? cp[i] + v[i] : v[i];
            }
          } else {
            __nv_bfloat16* cp = reinterpret_cast<__nv_bfloat16*>(p.C) + (size_t)row * p.ldc + col0;
            if (fullw && (p.ldc % 8 == 0)) {
#pragma unroll
              for (int i = 0; i < 32; i += 8) {
                if (p.accumulate) {
                  const uint4 c = *reinterpret_cast<const uint4*>(cp + i);
                  const uint32_t w[4] = {c.x, c.y, c.z, c.w};
#pragma unroll
                  for (int q = 0; q < 4; ++q) { v[i + 2 * q] += __uint_as_float(w[q] << 16); v[i + 2 * q + 1] += __uint_as_float(w[q] & 0xffff0000u); }
                }
                *reinterpret_cast<uint4*>(cp + i) = make_uint4(pack_bf16(v[i], v[i + 1]), pack_bf16(v[i + 2], v[i + 3]),
                                                               pack_bf16(v[i + 4], v[i + 5]), pack_bf16(v[i + 6], v[i + 7]));
              }
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i) {
                if (col0 + i < p.N) {
                  const float o = p.accumulate ? __bfloat162float(cp[i]) + v[i] : v[i];
                  cp[i] = __float2bfloat16_rn(o);
                }
              }
            }
          }
        }
      }
      fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_leader(&tempty[acc]);
    }
    if (lane == 0) bulk_wait_all();                    // shared memory stays valid until the last store has read it
  }

  // ---------------------------------------------------------------------- teardown
  fence_before();
  __syncthreads();
  if (*abort_flag) {
    const uint64_t t0 = gtimer();
    while (gtimer() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  cluster_sync_all();                            // the peer may still be reading this CTA's shared memory / barriers
  if (warp == 1) {
    fence_after();
    tmem_dealloc_pair(tmem_base, PairCfg<BN2>::TMEM_COLS);
  }
}

template <bool A_MN, bool B_MN, int BN2>
int launch2(const GemmGroup& g, cudaStream_t st) {
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(gemm_bf16_2cta_kernel<A_MN, B_MN, BN2>, cudaFuncAttributeMaxDynamicSharedMemorySize, pair_smem_bytes<BN2>());
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  const int units = g.tail ? g.num_tiles + g.tail : g.num_tiles * g.splits;
  int clusters = zen_tmap::sm_count() / 2;
  if (units < clusters) clusters = units;
  gemm_bf16_2cta_kernel<A_MN, B_MN, BN2><<<clusters * 2, 192, pair_smem_bytes<BN2>(), st>>>(g);
  return (int)cudaGetLastError();
}

int launch2_layout(const GemmGroup& g, int a_mn, int b_mn, int bn, cudaStream_t st) {
#define LAUNCH2(BN_)                                                   \
  do {                                                                 \
    if (!a_mn && !b_mn) return launch2<false, false, BN_>(g, st);      \
    if (!a_mn && b_mn) return launch2<false, true, BN_>(g, st);        \
    if (a_mn && !b_mn) return launch2<true, false, BN_>(g, st);        \
    return launch2<true, true, BN_>(g, st);                            \
  } while (0)
  if (bn == 128) LAUNCH2(128);
  if (bn == 192) {                                             // K-major B only (see pick_pair_bn)
    if (!a_mn) return launch2<false, false, 192>(g, st);
    return launch2<true, false, 192>(g, st);
  }
  LAUNCH2(256);
#undef LAUNCH2
}

// Tensor maps, tile counts and the output path of one product.  n_store: 0, or a width in [N, ldc] that the kernel may
// write (columns N.. receive zeros); max_slices: K slices that will write this output (the TMA-store path sums at most two).
int fill_problem(GemmProblem& q, const void* A, const void* B, void* C, const void* bias, int M, int N, int K, int lda,
                 int ldb, int ldc, int a_mn, int b_mn, int out_fp32, int accumulate, int n_store, int bn, int max_slices) {
  if (M <= 0 || N <= 0 || K <= 0) return -1;
  if ((lda % 8) || (ldb % 8) || (reinterpret_cast<uintptr_t>(A) % 16) || (reinterpret_cast<uintptr_t>(B) % 16)) return -2;
  int rc;
  if (!a_mn) rc = zen_tmap::get(A, (uint64_t)K, (uint64_t)M, (uint64_t)lda, 64, 128, &q.ta);
  else rc = zen_tmap::get(A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, 64, 64, &q.ta);
  if (rc) return rc;
  if (!b_mn) rc = zen_tmap::get(B, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, 64, (uint32_t)(bn / 2), &q.tb);
  else rc = zen_tmap::get(B, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, 64, 64, &q.tb);
  if (rc) return rc;
  // Plain bf16 output with a TMA-compatible layout: store through shared memory.  The stored width must be a
  // multiple of 8 columns (16 bytes); a caller whose buffer has spare columns after N may allow them to be written
  // (with zeros) by passing n_store = N rounded up.
  if (n_store < N || n_store > ldc) n_store = N;
  q.tma_store = (!out_fp32 && !accumulate && max_slices <= 2 && (ldc % 8) == 0 && (n_store % 8) == 0 &&
                 (reinterpret_cast<uintptr_t>(C) % 16) == 0) ? 1 : 0;
  q.tc = q.ta;
  if (q.tma_store) {
    rc = zen_tmap::get(C, (uint64_t)n_store, (uint64_t)M, (uint64_t)ldc, 64, 32, &q.tc);
    if (rc) return rc;
  }
  q.C = C; q.bias = bias; q.M = M; q.N = N; q.K = K; q.ldc = ldc; q.out_fp32 = out_fp32; q.accumulate = accumulate;
  q.num_m_pairs = (M + 255) / 256;
  q.num_n_tiles = (N + bn - 1) / bn;
  q.tile_start = 0;
  return 0;
}

}  // namespace

int g_force_bn = 0;
int g_tail_min_kb = 16;            // fewest 64-wide K blocks for which the tiles of the last wave are cut in two; 0 = never

// 256-wide pair tiles.  The 128-wide variant exists for outputs whose 256-wide tiles fill the 74 CTA pairs unevenly
// (96 tiles = 1.3 waves), but measured on 8192 x 768 outputs it lost (662 vs 858 TFLOP/s at K = 3072, 410 vs 472 at
// K = 768): with half the columns per tile the A rows are fetched twice as often and the kernel is bound by that
// traffic, not by the idle third of the second wave.  It is therefore only taken when forced.
// 192-wide tiles (K-major B only: its half of 96 rows is one TMA box; an MN-major half would need one and a half
// 64-column boxes) exist for the same 1.3-wave outputs: 8192 x 768 is 96 tiles of 256 = two waves of full tiles, but 128
// tiles of 192 = two waves of three-quarter tiles.  Measured, they gain nothing either (857.9 TFLOP/s both at
// 8192 x 768 x 3072): a 256 x 256 x 64 step takes 0.47 us here against 0.28 us of tensor-core time, i.e. the main loop
// is bound by the operand traffic from L2, which per FLOP is higher for the narrower tile.  Taken only when forced.
int pick_pair_bn(int M, int N, int b_mn, int splits) {
  (void)M; (void)N;
  if (g_force_bn == 192) return (!b_mn && splits == 1) ? 192 : 256;
  return g_force_bn ? g_force_bn : 256;
}

extern "C" {

// Same contract as zen_gemm_bf16 (without the tile choice): C[M,N] (+)= A * B^T (+ bias), CTA-pair kernel.
// splits > 1 cuts K into that many slices per output tile (for outputs with too few tiles to fill the GPU and a
// long K, the weight-gradient shape): `ws` must hold splits * tiles * 2 * 128 * 256 floats and `counters`
// tiles * 16 ints that are zero on entry (the kernel leaves them zero); both are caller-owned and used in stream
// order.  The slices are summed in slice order, so the result does not depend on timing.
// With splits == 1 a caller may still pass `ws` and `counters` (same sizes as for two slices of one wave of clusters):
// the launcher then cuts the tiles of the last, partly filled wave in two (see zen_gemm2_tail_split).
// n_store: 0, or a width in [N, ldc] that the kernel may write (columns N.. receive zeros).
int zen_gemm_bf16_2cta_splitk(const void* A, const void* B, void* C, const void* bias, int M, int N, int K, int lda,
                              int ldb, int ldc, int a_mn, int b_mn, int out_fp32, int accumulate, int splits, float* ws,
                              uint64_t ws_floats, int* counters, int n_counters, int n_store, void* stream);

int zen_gemm_bf16_2cta(const void* A, const void* B, void* C, const void* bias, int M, int N, int K, int lda, int ldb,
                       int ldc, int a_mn, int b_mn, int out_fp32, int accumulate, void* stream) {
  return zen_gemm_bf16_2cta_splitk(A, B, C, bias, M, N, K, lda, ldb, ldc, a_mn, b_mn, out_fp32, accumulate, 1, nullptr, 0,
                                   nullptr, 0, 0, stream);
}

int zen_gemm_bf16_2cta_splitk(const void* A, const void* B, void* C, const void* bias, int M, int N, int K, int lda,
                              int ldb, int ldc, int a_mn, int b_mn, int out_fp32, int accumulate, int splits, float* ws,
                              uint64_t ws_floats, int* counters, int n_counters, int n_store, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0) return -1;
  const int nkb = (K + BK2 - 1) / BK2;
  if (splits < 1) splits = 1;
  if (splits > MAX_SPLITS) splits = MAX_SPLITS;
  if (splits > nkb) splits = nkb;
  int kb_per = (nkb + splits - 1) / splits;
  splits = (nkb + kb_per - 1) / kb_per;                     // no empty slice
  if (splits > 1) {
    // The two slices of a tile hand each other half of the columns and wait for it: both must be resident at the
    // same time, i.e. every (tile, slice) unit needs its own cluster in the one wave that the launch has.
    const uint64_t units = (uint64_t)((M + 255) / 256) * ((N + 255) / 256) * (uint64_t)splits;
    if (units > (uint64_t)(zen_tmap::sm_count() / 2)) { splits = 1; kb_per = nkb; }
  }
  const int bn = (splits > 1) ? 256 : pick_pair_bn(M, N, b_mn, splits);
  if (splits > 1) {
    const uint64_t tiles = (uint64_t)((M + 255) / 256) * ((N + 255) / 256);
    if (!ws || !counters || ws_floats < tiles * splits * 2 * BM2 * 256 || (uint64_t)n_counters < tiles * 16) return -4;
    if (reinterpret_cast<uintptr_t>(ws) % 16) return -2;
  }
  GemmGroup g;
  int rc = fill_problem(g.pr[0], A, B, C, bias, M, N, K, lda, ldb, ldc, a_mn, b_mn, out_fp32, accumulate, n_store, bn, splits);
  if (rc) return rc;
  g.n = 1;
  g.num_tiles = g.pr[0].num_m_pairs * g.pr[0].num_n_tiles;
  g.splits = splits;
  g.kb_per_split = kb_per;
  g.ws = ws;
  g.counters = counters;
  // Tail split: the tiles of the last, partly filled wave of clusters run as two K slices each when both slices of
  // all of them fit in that wave (so that the slices that wait for each other are resident together, as above) and K
  // is long enough for half a tile to outweigh the exchange of half an accumulator.
  g.tail = 0;
  if (splits == 1 && bn == 256 && g.pr[0].tma_store && g_tail_min_kb > 0 && nkb >= g_tail_min_kb && ws && counters &&
      (reinterpret_cast<uintptr_t>(ws) % 16) == 0) {
    const int clusters = zen_tmap::sm_count() / 2;
    const int rem = g.num_tiles % clusters;
    if (g.num_tiles > clusters && rem > 0 && 2 * rem <= clusters && ws_floats >= (uint64_t)rem * 2 * 2 * BM2 * 256 &&
        n_counters >= rem * 16)
      g.tail = rem;
  }
  return launch2_layout(g, a_mn, b_mn, bn, (cudaStream_t)stream);
}

// Several products with the same operand layouts in ONE launch (see GemmProblem): the tiles of all of them form one
// list that the persistent clusters walk, and the tiles of the last, partly filled wave are cut into two K halves when
// their outputs take the TMA-store path.  `descs`: n records of ZenGemmDesc; every product follows the contract of
// zen_gemm_bf16_2cta (no bias).  ws / counters as for zen_gemm_bf16_2cta_splitk (may be null: no tail split).
struct ZenGemmDesc {
  const void* A;
  const void* B;
  void* C;
  int32_t M, N, K, lda, ldb, ldc;
  int32_t out_fp32, accumulate;
};
int zen_gemm_desc_size() { return (int)sizeof(ZenGemmDesc); }
int zen_gemm_group_max() { return MAX_GROUP; }

int zen_gemm_bf16_2cta_group(const ZenGemmDesc* descs, int n, int a_mn, int b_mn, float* ws, uint64_t ws_floats,
                             int* counters, int n_counters, void* stream) {
  if (!descs || n < 1 || n > MAX_GROUP) return -1;
  GemmGroup g;
  int tiles = 0, min_kb = 1 << 30;
  for (int i = 0; i < n; ++i) {
    const ZenGemmDesc& d = descs[i];
    int rc = fill_problem(g.pr[i], d.A, d.B, d.C, nullptr, d.M, d.N, d.K, d.lda, d.ldb, d.ldc, a_mn, b_mn, d.out_fp32,
                          d.accumulate, 0, 256, 2);
    if (rc) return rc;
    g.pr[i].tile_start = tiles;
    tiles += g.pr[i].num_m_pairs * g.pr[i].num_n_tiles;
    const int nkb = (d.K + BK2 - 1) / BK2;
    if (nkb < min_kb) min_kb = nkb;
  }
  g.n = n;
  g.num_tiles = tiles;
  g.splits = 1;
  g.kb_per_split = 1 << 30;
  g.ws = ws;
  g.counters = counters;
  g.tail = 0;
  const int clusters = zen_tmap::sm_count() / 2;
  const int rem = tiles % clusters;
  if (g_tail_min_kb > 0 && min_kb >= g_tail_min_kb && ws && counters && (reinterpret_cast<uintptr_t>(ws) % 16) == 0 &&
      rem > 0 && 2 * rem <= clusters && ws_floats >= (uint64_t)rem * 2 * 2 * BM2 * 256 && n_counters >= rem * 16) {
    bool ok = true;                                           // every tile of the tail must take the two-slice store path
    for (int i = 0; i < n; ++i) {
      const int end = g.pr[i].tile_start + g.pr[i].num_m_pairs * g.pr[i].num_n_tiles;
      if (end > tiles - rem && !g.pr[i].tma_store) ok = false;
    }
    if (ok) g.tail = rem;
  }
  return launch2_layout(g, a_mn, b_mn, 256, (cudaStream_t)stream);
}

// 0 = choose the N tile per call, 128 / 256 = force it (tests, measurements); returns the previous setting.
int zen_gemm2_force_bn(int bn) {
  const int old = g_force_bn;
  if (bn == 0 || bn == 128 || bn == 192 || bn == 256) g_force_bn = bn;
  return old;
}

// Fewest K blocks (of 64) from which the tiles of a launch's last, partly filled wave run as two K slices; 0 switches
// the tail split off.  Returns the previous setting.
int zen_gemm2_tail_split(int min_kb) {
  const int old = g_tail_min_kb;
  if (min_kb >= 0) g_tail_min_kb = (min_kb > 0 && min_kb < 2) ? 2 : min_kb;
  return old;
}

int zen_gemm2_error() {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_gemm2_error, sizeof(int)) != cudaSuccess) return -1;
  if (v) cudaMemcpyToSymbol(g_gemm2_error, &zero, sizeof(int));
  return v;
}

}  // extern "C"
