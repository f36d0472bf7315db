// bf16 GEMM on the 5th-generation tensor cores (tcgen05) for sm_100a.
//
//   C[M, N] (+)= A[M, K] * B[N, K]^T (+ bias[N])        fp32 accumulation in tensor memory
//
// Each operand may be stored K-major (rows of K contiguous) or MN-major (its transpose), which
// covers forward (x W^T), input-gradient (dy W) and weight-gradient (dy^T x) products of a linear
// layer without materialising a transpose.
//
// Structure: persistent CTAs, one per SM, 192 threads in three roles.
//   warp 0      TMA producer: cp.async.bulk.tensor tiles (128-byte swizzle) into a 4..6 stage ring.
//   warp 1      MMA issuer: one thread issues tcgen05.mma (M128 x N{128,256} x K16) from shared-memory
//               descriptors into one of two TMEM accumulators, tcgen05.commit signals stage release
//               and accumulator completion.
//   warps 2..5  epilogue: tcgen05.ld the accumulator (each warp its 32 TMEM lanes), add bias /
//               previous C, convert, store.  Overlaps with the next tile's main loop.
// All waits on mbarriers are bounded; on a timeout the kernel records an error code, leaves its
// loops, frees its tensor memory and returns.
//
// The reference gets its GEMMs from cuBLAS through PyTorch / HuggingFace modules (train.py:149).
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>
#include <unordered_map>

namespace {

constexpr int BM = 128;
constexpr int BK = 64;                 // 64 bf16 = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr int NUM_THREADS = 192;
constexpr uint64_t WAIT_NS = 2000000000ull;   // 2 s per wait, then give up

__device__ int g_gemm_error = 0;

struct GemmParams {
  void* C;
  const void* bias;     // bf16 [N] or null
  int M, N, K;
  int ldc;
  int out_fp32;         // C is float instead of bf16
  int accumulate;       // C += result
  int num_m_tiles, num_n_tiles;
  // ---- fused all-reduce over tensor-parallel peers (npeers == 0: plain GEMM) ----
  int npeers;                 // other ranks of the TP group
  int rank;                   // this rank's index in the group
  uint32_t epoch;             // call counter, same on every rank; parity selects the exchange buffer
  uint32_t max_tiles;         // capacity of one flag row
  const uint32_t* epoch_dev;  // optional step counter on the device: the call counter is *epoch_dev * epoch_stride + epoch
  uint32_t epoch_stride;      // (same parity as the number of calls per step, so that consecutive calls alternate buffers)
  uint64_t wait_ns;
  __nv_bfloat16* my_recv;     // this rank's exchange region: [2 parities][npeers slots][M * recv_ld] bf16
  uint32_t* my_flags;         // this rank's flags: [2 parities][npeers slots][max_tiles] epochs
  __nv_bfloat16* peer_recv[7];// peers' exchange regions (same layout), indexed by peer slot
  uint32_t* peer_flags[7];
  int peer_slot_of_me[7];     // which slot this rank writes in peer i's region
  int peer_rank[7];           // group rank of peer slot i (for the fixed summation order)
  uint64_t slot_elems;        // elements per (parity, slot)
  int recv_ld;                // row stride of exchanged partial tiles
  uint32_t* status;           // device word: bit 2 set when a peer wait timed out
  // ---- collective flavour of the fused kernel ----
  // 0: all-reduce of C (every rank gets the sum).
  // 1: reduce-scatter of C over rows: A is [M, K], rank r ends up with rows [r * rows_per_rank, ...) of the sum in
  //    C[rows_per_rank, N]; partial tiles of rows owned by a peer are pushed to that peer only, and those tiles run
  //    first so that they are on their way while this rank computes its own rows.
  // 2: all-gather of A over rows: this rank holds rows [rank * rows_per_rank, ...) of A (a_local); the epilogue warps
  //    of the first CTAs push it chunk by chunk (128 rows) into the peer's gather region at kernel start, tiles of local
  //    rows run first, and the producer waits (bounded) for a chunk's flag before it loads a tile of gathered rows
  //    through a tensor map over this rank's own region, never over peer memory.
  int coll_mode;
  int rows_per_rank;
  const __nv_bfloat16* a_local;
  int lda_local;
};

// The call counter as the kernels compare it: by value, or derived from a device-resident step counter so that a
// captured launch sees a new value at every replay.
__device__ __forceinline__ uint32_t cur_epoch(const GemmParams& p) {
  return p.epoch_dev ? (*p.epoch_dev) * p.epoch_stride + p.epoch : p.epoch;
}

constexpr int COLL_AR = 0, COLL_RS = 1, COLL_AG = 2;

// Tile index -> coordinates.  owner: rank whose rows the tile covers; m0: first row in the full row space; mloc:
// first row relative to the owner's block; fidx: index of the tile among the owner's tiles (flag slot).
struct TileCoord { int m0, n0, owner, mloc, fidx; };
template <int BN>
__device__ __forceinline__ TileCoord decode_tile(const GemmParams& p, int tile) {
  TileCoord t;
  if (p.npeers == 0 || p.coll_mode == COLL_AR) {
    t.m0 = (tile % p.num_m_tiles) * BM;
    t.n0 = (tile / p.num_m_tiles) * BN;
    t.owner = p.rank; t.mloc = t.m0; t.fidx = tile;
    return t;
  }
  const int tpr = p.rows_per_rank / BM, per_owner = tpr * p.num_n_tiles, nranks = p.npeers + 1;
  const int rel = tile / per_owner, within = tile % per_owner;
  t.owner = (p.rank + rel + (p.coll_mode == COLL_RS ? 1 : 0)) % nranks;   // RS: peers' rows first; AG: own rows first
  t.mloc = (within % tpr) * BM;
  t.n0 = (within / tpr) * BN;
  t.m0 = t.owner * p.rows_per_rank + t.mloc;
  t.fidx = within;
  return t;
}

// ------------------------------------------------------------------------------------ PTX helpers
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_test(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ uint64_t gtimer() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
// Bounded wait.  Returns false (and raises the abort flag) when the budget runs out or when another
// role has already aborted.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int code) {
  if (mbar_test(bar, parity)) return true;
  const uint64_t t0 = gtimer();
  for (;;) {
    for (int i = 0; i < 256; ++i)
      if (mbar_test(bar, parity)) return true;
    if (*abort_flag) return false;
    if (gtimer() - t0 > WAIT_NS) {
      *abort_flag = code;
      atomicCAS(&g_gemm_error, 0, code);
      return false;
    }
  }
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
      : "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(ncols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_ld32_nowait(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ void st_release_sys_u32(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_cg_v4(const void* p) {   // L2-coherent load: peers write this memory
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ void epilogue_barrier() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// Shared-memory matrix descriptor (128-byte swizzle).  K-major: rows of 128 bytes, 8-row groups
// 1024 bytes apart (SBO).  MN-major: 64-element groups along M/N `lbo_bytes` apart, 8-row groups
// along K 1024 bytes apart.
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= (uint64_t)1 << 46;       // descriptor version for sm_100
  d |= (uint64_t)2 << 61;       // SWIZZLE_128B
  return d;
}

// Second half of a deferred tile (all 128 epilogue threads): bounded wait for the peers' partials of tile `tile`,
// then C = bias + sum over ranks, in rank order, of the bf16 partials (own partial already in C).  Rows are walked
// with consecutive threads on consecutive 16-byte vectors, four rows in flight per thread.
template <int BN>
__device__ __forceinline__ bool finish_tile(const GemmParams& p, int tile, uint32_t par, volatile int* abort_flag) {
  const TileCoord tc = decode_tile<BN>(p, tile);
  const int et = threadIdx.x - 64;
  const bool rs = p.coll_mode == COLL_RS;
  if (et < p.npeers) {
    const uint32_t* f = p.my_flags + ((size_t)par * p.npeers + et) * p.max_tiles + tc.fidx;
    const uint64_t t0 = gtimer();
    bool got = ld_acquire_sys_u32(f) == cur_epoch(p);
    while (!got) {
      for (int i = 0; i < 64 && !got; ++i) got = ld_acquire_sys_u32(f) == cur_epoch(p);
      if (!got && (gtimer() - t0 > p.wait_ns || *abort_flag)) break;
    }
    if (!got) { atomicOr(p.status, 4u); *abort_flag = 5; atomicCAS(&g_gemm_error, 0, 5); }
  }
  epilogue_barrier();
  if (*abort_flag) return false;
  constexpr int VPR = BN / 8, RPP = 128 / VPR;       // vectors per row, rows per pass of the 128 threads
  const int cv = et % VPR, col = tc.n0 + cv * 8;
  const bool vec_ok = (p.ldc % 8) == 0 && col + 8 <= p.N;
  __nv_bfloat16* C = reinterpret_cast<__nv_bfloat16*>(p.C);
  const __nv_bfloat16* bias = reinterpret_cast<const __nv_bfloat16*>(p.bias);
  for (int r0 = et / VPR; r0 < BM; r0 += 4 * RPP) {
    float v[4][8];
    uint4 own[4];
    bool live[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int r = r0 + u * RPP;
      live[u] = r < BM && tc.m0 + r < p.M && col < p.N;
      if (live[u] && vec_ok) own[u] = *reinterpret_cast<const uint4*>(C + (size_t)((rs ? tc.mloc : tc.m0) + r) * p.ldc + col);
#pragma unroll
      for (int i = 0; i < 8; ++i) v[u][i] = 0.f;
    }
    bool own_added = false;
    for (int pe = 0; pe <= p.npeers; ++pe) {
      if (!own_added && (pe == p.npeers || p.peer_rank[pe] > p.rank)) {
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          if (!live[u]) continue;
          const int xr = (rs ? tc.mloc : tc.m0) + r0 + u * RPP;
          if (vec_ok) {
            const uint32_t w[4] = {own[u].x, own[u].y, own[u].z, own[u].w};
#pragma unroll
            for (int k2 = 0; k2 < 4; ++k2) { v[u][2 * k2] += __uint_as_float(w[k2] << 16); v[u][2 * k2 + 1] += __uint_as_float(w[k2] & 0xffff0000u); }
          } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) if (col + i < p.N) v[u][i] += __bfloat162float(C[(size_t)xr * p.ldc + col + i]);
          }
        }
        own_added = true;
      }
      if (pe == p.npeers) break;
      uint4 pv[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int xr = (rs ? tc.mloc : tc.m0) + r0 + u * RPP;
        const __nv_bfloat16* src = p.my_recv + ((size_t)par * p.npeers + pe) * p.slot_elems + (size_t)xr * p.recv_ld + col;
        if (live[u] && vec_ok) pv[u] = ld_cg_v4(src);
        else if (live[u]) {
#pragma unroll
          for (int i = 0; i < 8; ++i) if (col + i < p.N) v[u][i] += __bfloat162float(*reinterpret_cast<const volatile __nv_bfloat16*>(src + i));
        }
      }
      if (vec_ok) {
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          if (!live[u]) continue;
          const uint32_t w[4] = {pv[u].x, pv[u].y, pv[u].z, pv[u].w};
#pragma unroll
          for (int k2 = 0; k2 < 4; ++k2) { v[u][2 * k2] += __uint_as_float(w[k2] << 16); v[u][2 * k2 + 1] += __uint_as_float(w[k2] & 0xffff0000u); }
        }
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      if (!live[u]) continue;
      const int xr = (rs ? tc.mloc : tc.m0) + r0 + u * RPP;
      if (bias) {
#pragma unroll
        for (int i = 0; i < 8; ++i) if (col + i < p.N) v[u][i] += __bfloat162float(bias[col + i]);
      }
      __nv_bfloat16* cp = C + (size_t)xr * p.ldc + col;
      if (vec_ok) {
        uint32_t o[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          __nv_bfloat162 h = __floats2bfloat162_rn(v[u][2 * q], v[u][2 * q + 1]);
          o[q] = *reinterpret_cast<uint32_t*>(&h);
        }
        *reinterpret_cast<uint4*>(cp) = make_uint4(o[0], o[1], o[2], o[3]);
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) if (col + i < p.N) cp[i] = __float2bfloat16_rn(v[u][i]);
      }
    }
  }
  return true;
}

// Column slices per 128-row chunk of the all-gather push: as many as the grid can work on at once (same value on
// every rank: same shapes, same grid), within the flag capacity.
__device__ __forceinline__ int ag_slices(int grid, int nchunks, uint32_t max_tiles) {
  int n = grid / nchunks;
  if (n < 1) n = 1;
  if (n > 16) n = 16;
  while (n > 1 && (uint32_t)(nchunks * n) > max_tiles) --n;
  return n;
}

template <int BN, bool A_MN, bool B_MN>
struct Cfg {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (BN == 256) ? 4 : 6;
  static constexpr int XCHG_BYTES = 4 * 4096;          // per epilogue warp a [32 rows][64 bf16] staging box (peer pushes)
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/ + XCHG_BYTES;
  static constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((A_MN ? 1u : 0u) << 15) |
                                    ((B_MN ? 1u : 0u) << 16) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
};

template <int BN, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                 const __grid_constant__ CUtensorMap tma_g, const GemmParams p) {
  using C = Cfg<BN, A_MN, B_MN>;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::STAGES * C::STAGE_BYTES);
  uint64_t* full = bars;                         // [STAGES]
  uint64_t* empty = bars + C::STAGES;            // [STAGES]
  uint64_t* tfull = bars + 2 * C::STAGES;        // [2]
  uint64_t* tempty = bars + 2 * C::STAGES + 2;   // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * C::STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_tiles = p.num_m_tiles * p.num_n_tiles;
  const int nkb = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&tfull[a], 1); mbar_init(&tempty[a], 4); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(tmem_slot, 2 * BN);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      // ------------------------------------------------------------------ TMA producer
      uint32_t it = 0;
      bool ok = true;
      const bool ag = p.npeers > 0 && p.coll_mode == COLL_AG;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const TileCoord tc = decode_tile<BN>(p, tile);
        const int n0 = tc.n0;
        int m0 = tc.m0;
        const CUtensorMap* amap = &tma_a;
        if (ag) {
          m0 = tc.mloc;                             // row inside the local shard or inside the gathered copy
          if (tc.owner != p.rank) {
            // rows of a peer: its epilogue warps push them into this rank's gather region; wait for the chunk
            amap = &tma_g;
            const int nslices = ag_slices(gridDim.x, p.rows_per_rank / BM, p.max_tiles);
            const uint32_t* f = p.my_flags + (size_t)(cur_epoch(p) & 1u) * p.npeers * p.max_tiles + (tc.mloc / BM) * nslices;
            const uint64_t t0 = gtimer();
            bool got = true;
            for (int sl = 0; sl < nslices && got; ++sl) {               // every column slice of the chunk
              got = ld_acquire_sys_u32(f + sl) == cur_epoch(p);
              while (!got) {
                for (int i = 0; i < 64 && !got; ++i) got = ld_acquire_sys_u32(f + sl) == cur_epoch(p);
                if (!got && (gtimer() - t0 > p.wait_ns || *abort_flag)) break;
              }
            }
            if (!got) { atomicOr(p.status, 4u); *abort_flag = 6; atomicCAS(&g_gemm_error, 0, 6); ok = false; break; }
            asm volatile("fence.proxy.async;" ::: "memory");      // the peer's stores, then this rank's TMA reads
          }
        }
        for (int kb = 0; kb < nkb; ++kb, ++it) {
          const int s = it % C::STAGES;
          const uint32_t ph = (it / C::STAGES) & 1;
          if (!mbar_wait(&empty[s], ph ^ 1, abort_flag, 1)) { ok = false; break; }
          unsigned char* sa = smem + s * C::STAGE_BYTES;
          unsigned char* sb = sa + C::A_BYTES;
          mbar_expect_tx(&full[s], C::STAGE_BYTES);
          const int k0 = kb * BK;
          if (!A_MN) {
            tma_load_2d(sa, amap, &full[s], k0, m0);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_2d(sa + j * 8192, &tma_a, &full[s], m0 + 64 * j, k0);
          }
          if (!B_MN) {
            tma_load_2d(sb, &tma_b, &full[s], k0, n0);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j) tma_load_2d(sb + j * 8192, &tma_b, &full[s], n0 + 64 * j, k0);
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ------------------------------------------------------------------ MMA issuer
      uint32_t it = 0, tcount = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++tcount) {
        const uint32_t acc = tcount & 1, aph = (tcount >> 1) & 1;
        if (!mbar_wait(&tempty[acc], aph ^ 1, abort_flag, 2)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < nkb; ++kb, ++it) {
          const int s = it % C::STAGES;
          const uint32_t ph = (it / C::STAGES) & 1;
          if (!mbar_wait(&full[s], ph, abort_flag, 3)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * C::STAGE_BYTES);
          const uint32_t sb = sa + C::A_BYTES;
          const uint64_t adesc = A_MN ? make_desc(sa, 8192, 1024) : make_desc(sa, 16, 1024);
          const uint64_t bdesc = B_MN ? make_desc(sb, 8192, 1024) : make_desc(sb, 16, 1024);
#pragma unroll
          for (int j = 0; j < BK / UMMA_K; ++j) {
            const uint64_t astep = (uint64_t)((A_MN ? j * 2048 : j * 32) >> 4);
            const uint64_t bstep = (uint64_t)((B_MN ? j * 2048 : j * 32) >> 4);
            umma_bf16(d_tmem, adesc + astep, bdesc + bstep, C::IDESC, (kb | j) != 0 ? 1u : 0u);
          }
          umma_commit(&empty[s]);               // frees the stage once these MMAs have read it
        }
        if (ok) umma_commit(&tfull[acc]);       // accumulator complete
      }
    }
  } else {
    // -------------------------------------------------------------------- epilogue (warps 2..5)
    const int grp = warp & 3;                   // TMEM lane quarter this warp may read
    uint32_t tcount = 0;
    bool ok = true;
    const uint32_t par = cur_epoch(p) & 1u;
    const bool rs = p.npeers > 0 && p.coll_mode == COLL_RS, ag = p.npeers > 0 && p.coll_mode == COLL_AG;
    if (ag) {
      // ---- all-gather: push this rank's rows to the peer, one 128-row chunk per CTA, while the first tiles
      // (local rows) are in their main loops.  The gathered copy is dense [rows_per_rank, K].
      const int et = threadIdx.x - 64;
      const int nchunks = p.rows_per_rank / BM, vec_per_row = p.K / 8;
      const int nslices = ag_slices(gridDim.x, nchunks, p.max_tiles);
      const int vps = (vec_per_row + nslices - 1) / nslices;          // 16-byte vectors per row and slice
      // work item = (128-row chunk, column slice); every CTA takes the items b, b + grid, ...
      for (int item = blockIdx.x; item < nchunks * nslices; item += gridDim.x) {
        const int c = item % nchunks, sl = item / nchunks;
        const int v0 = sl * vps, v1 = min(vec_per_row, v0 + vps), w = v1 - v0;
        for (int pe = 0; pe < p.npeers; ++pe) {
          __nv_bfloat16* dst = p.peer_recv[pe] + ((size_t)par * p.npeers + p.peer_slot_of_me[pe]) * p.slot_elems + (size_t)c * BM * p.K;
          const __nv_bfloat16* src = p.a_local + (size_t)c * BM * p.lda_local;
          for (int v = et; v < BM * w; v += 4 * 128) {
            uint4 x[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const int vv = v + u * 128;
              if (vv < BM * w) x[u] = *reinterpret_cast<const uint4*>(src + (size_t)(vv / w) * p.lda_local + (v0 + vv % w) * 8);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const int vv = v + u * 128;
              if (vv < BM * w) *reinterpret_cast<uint4*>(dst + (size_t)(vv / w) * p.K + (v0 + vv % w) * 8) = x[u];
            }
          }
        }
        __threadfence_system();
        epilogue_barrier();
        if (et < p.npeers)
          st_release_sys_u32(p.peer_flags[et] + ((size_t)par * p.npeers + p.peer_slot_of_me[et]) * p.max_tiles + c * nslices + sl, cur_epoch(p));
      }
    }
    // Deferred reduction (bf16 output, no accumulation): a tile's epilogue pushes the partial to the peers, stores
    // the own partial in C and moves on; the sum over ranks for that tile is taken one tile later (after the next
    // tile's push), when the peers' partials have normally arrived, so that no epilogue stalls on NVLink latency.
    const bool deferred = p.npeers > 0 && !ag && !p.out_fp32 && !p.accumulate;
    int pending = -1;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++tcount) {
      const TileCoord tc = decode_tile<BN>(p, tile);
      const int m0 = tc.m0, n0 = tc.n0;
      const uint32_t acc = tcount & 1, aph = (tcount >> 1) & 1;
      if (!mbar_wait(&tfull[acc], aph, abort_flag, 4)) { ok = false; break; }
      tc_fence_after();
      const int row = m0 + grp * 32 + lane;     // row in the full row space (bounds)
      const int xrow = rs ? tc.mloc + grp * 32 + lane : row;    // row inside an exchange slot / inside C
      const int ftile = tc.fidx;
      const bool mine = tc.owner == p.rank;
      const uint32_t taddr0 = tmem_base + ((uint32_t)(grp * 32) << 16) + acc * BN;
      if (p.npeers > 0 && !ag) {
        // ---- step 1: push this rank's partial tile (bf16) into the exchange region of every peer (all-reduce) or of
        // the rank that owns these rows (reduce-scatter; nothing to push for own rows)
        // Whole-line version (deferred mode, 16-byte-aligned rows, N a multiple of 8): a thread's 64 columns go
        // through a swizzled [32][64] box in shared memory and come back transposed, so that every store instruction
        // of the warp writes four complete 128-byte lines instead of 32 pieces of 16 bytes in 32 different rows,
        // which is what NVLink packets and the L2 want.
        const bool staged = deferred && (p.ldc % 8) == 0 && (p.N % 8) == 0;
        if (staged) {
          unsigned char* stg = smem + C::STAGES * C::STAGE_BYTES + 256 + grp * 4096;
          const bool keep = !rs || mine;
          __nv_bfloat16* Cb = reinterpret_cast<__nv_bfloat16*>(p.C);
#pragma unroll 1
          for (int cb = 0; cb < BN / 64; ++cb) {
            uint32_t ra[32], rb[32];
            tmem_ld32_nowait(taddr0 + cb * 64, ra);
            tmem_ld32_nowait(taddr0 + cb * 64 + 32, rb);
            tmem_wait_ld();
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              uint32_t o[4], o2[4];
#pragma unroll
              for (int k2 = 0; k2 < 4; ++k2) {
                __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(ra[8 * q + 2 * k2]), __uint_as_float(ra[8 * q + 2 * k2 + 1]));
                __nv_bfloat162 h2 = __floats2bfloat162_rn(__uint_as_float(rb[8 * q + 2 * k2]), __uint_as_float(rb[8 * q + 2 * k2 + 1]));
                o[k2] = *reinterpret_cast<uint32_t*>(&h);
                o2[k2] = *reinterpret_cast<uint32_t*>(&h2);
              }
              *reinterpret_cast<uint4*>(stg + lane * 128 + ((q ^ (lane & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
              *reinterpret_cast<uint4*>(stg + lane * 128 + (((4 + q) ^ (lane & 7)) << 4)) = make_uint4(o2[0], o2[1], o2[2], o2[3]);
            }
            __syncwarp();
#pragma unroll
            for (int it = 0; it < 8; ++it) {
              const int r = it * 4 + (lane >> 3), c = lane & 7;
              const uint4 v = *reinterpret_cast<const uint4*>(stg + r * 128 + ((c ^ (r & 7)) << 4));
              const int grow = m0 + grp * 32 + r, col = n0 + cb * 64 + c * 8;
              if (grow < p.M && col < p.N) {
                const size_t xr = (size_t)((rs ? tc.mloc : m0) + grp * 32 + r);
                if (keep) *reinterpret_cast<uint4*>(Cb + xr * p.ldc + col) = v;
                for (int pe = 0; pe < p.npeers; ++pe) {
                  if (rs && p.peer_rank[pe] != tc.owner) continue;
                  *reinterpret_cast<uint4*>(p.peer_recv[pe] + ((size_t)par * p.npeers + p.peer_slot_of_me[pe]) * p.slot_elems + xr * p.recv_ld + col) = v;
                }
              }
            }
            __syncwarp();
          }
        }
#pragma unroll 1
        for (int ch = 0; ch < ((staged || (rs && mine && !deferred)) ? 0 : BN / 32); ++ch) {
          uint32_t r[32];
          tmem_ld32(taddr0 + ch * 32, r);
          const int col0 = n0 + ch * 32;
          if (row < p.M && col0 < p.N) {
            uint32_t o[16];
#pragma unroll
            for (int q = 0; q < 16; ++q) {
              __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(r[2 * q]), __uint_as_float(r[2 * q + 1]));
              o[q] = *reinterpret_cast<uint32_t*>(&h);
            }
            if (deferred && (!rs || mine)) {      // own partial waits in C for the peers' (summed by finish_tile)
              __nv_bfloat16* cp = reinterpret_cast<__nv_bfloat16*>(p.C) + (size_t)xrow * p.ldc + col0;
              if (col0 + 32 <= p.N && (p.ldc % 8) == 0) {
#pragma unroll
                for (int q = 0; q < 4; ++q) *reinterpret_cast<uint4*>(cp + 8 * q) = make_uint4(o[4 * q], o[4 * q + 1], o[4 * q + 2], o[4 * q + 3]);
              } else {
#pragma unroll
                for (int i = 0; i < 32; ++i)
                  if (col0 + i < p.N) cp[i] = __ushort_as_bfloat16((unsigned short)((o[i >> 1] >> ((i & 1) * 16)) & 0xffffu));
              }
            }
            for (int pe = 0; pe < p.npeers; ++pe) {
              if (rs && p.peer_rank[pe] != tc.owner) continue;
              __nv_bfloat16* dst = p.peer_recv[pe] + ((size_t)par * p.npeers + p.peer_slot_of_me[pe]) * p.slot_elems +
                                   (size_t)xrow * p.recv_ld + col0;
              if (col0 + 32 <= p.N) {
#pragma unroll
                for (int q = 0; q < 4; ++q) *reinterpret_cast<uint4*>(dst + 8 * q) = make_uint4(o[4 * q], o[4 * q + 1], o[4 * q + 2], o[4 * q + 3]);
              } else {
#pragma unroll
                for (int i = 0; i < 32; ++i)
                  if (col0 + i < p.N) dst[i] = __ushort_as_bfloat16((unsigned short)((o[i >> 1] >> ((i & 1) * 16)) & 0xffffu));
              }
            }
          }
        }
        __threadfence_system();
        epilogue_barrier();
        const int et = threadIdx.x - 64;                                   // 0..127 among the epilogue threads
        if (et < p.npeers && !(rs && (mine || p.peer_rank[et] != tc.owner)))
          st_release_sys_u32(p.peer_flags[et] + ((size_t)par * p.npeers + p.peer_slot_of_me[et]) * p.max_tiles + ftile, cur_epoch(p));
        if (deferred) {
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&tempty[acc]);
          if (pending >= 0 && !finish_tile<BN>(p, pending, par, abort_flag)) { ok = false; break; }
          pending = (!rs || mine) ? tile : -1;
          continue;
        }
        if (rs && !mine) {                       // a peer's rows: pushed, nothing to write here
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&tempty[acc]);
          continue;
        }
        // ---- step 2: bounded wait for every peer's partial of this tile
        if (et < p.npeers) {
          const uint32_t* f = p.my_flags + ((size_t)par * p.npeers + et) * p.max_tiles + ftile;
          const uint64_t t0 = gtimer();
          bool got = ld_acquire_sys_u32(f) == cur_epoch(p);
          while (!got) {
            for (int i = 0; i < 64 && !got; ++i) got = ld_acquire_sys_u32(f) == cur_epoch(p);
            if (!got && (gtimer() - t0 > p.wait_ns || *abort_flag)) break;
          }
          if (!got) { atomicOr(p.status, 4u); *abort_flag = 5; atomicCAS(&g_gemm_error, 0, 5); }
        }
        epilogue_barrier();
      }
#pragma unroll 1
      for (int ch = 0; ch < BN / 32; ++ch) {
        uint32_t r[32];
        tmem_ld32(taddr0 + ch * 32, r);         // warp-wide, must not be skipped by single lanes
        const int col0 = n0 + ch * 32;
        if (row < p.M && col0 < p.N) {
          float v[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
          if (p.npeers > 0 && !ag) {
            // step 3: sum the bf16-rounded partials of all ranks in rank order, so every rank gets the same bits
            float own[32];
#pragma unroll
            for (int q = 0; q < 16; ++q) {
              __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * q], v[2 * q + 1]);
              own[2 * q] = __bfloat162float(h.x); own[2 * q + 1] = __bfloat162float(h.y);
            }
            bool own_added = false;
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = 0.f;
            for (int pe = 0; pe <= p.npeers; ++pe) {
              if (!own_added && (pe == p.npeers || p.peer_rank[pe] > p.rank)) {
#pragma unroll
                for (int i = 0; i < 32; ++i) v[i] += own[i];
                own_added = true;
              }
              if (pe == p.npeers) break;
              const __nv_bfloat16* src = p.my_recv + ((size_t)par * p.npeers + pe) * p.slot_elems + (size_t)xrow * p.recv_ld + col0;
              if (col0 + 32 <= p.N) {
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                  const uint4 w4 = ld_cg_v4(src + 8 * q);
                  const uint32_t w[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
                  for (int k2 = 0; k2 < 4; ++k2) { v[8 * q + 2 * k2] += __uint_as_float(w[k2] << 16); v[8 * q + 2 * k2 + 1] += __uint_as_float(w[k2] & 0xffff0000u); }
                }
              } else {
#pragma unroll
                for (int i = 0; i < 32; ++i)
                  if (col0 + i < p.N) v[i] += __bfloat162float(*reinterpret_cast<const volatile __nv_bfloat16*>(src + i));
              }
            }
          }
          const bool fullw = (col0 + 32 <= p.N);
          if (p.bias) {
            const __nv_bfloat16* bp = reinterpret_cast<const __nv_bfloat16*>(p.bias) + col0;
#pragma unroll
            for (int i = 0; i < 32; ++i) if (fullw || col0 + i < p.N) v[i] += __bfloat162float(bp[i]);
          }
          if (p.out_fp32) {
            float* cp = reinterpret_cast<float*>(p.C) + (size_t)xrow * p.ldc + col0;
            if (fullw && (p.ldc % 4 == 0)) {
#pragma unroll
              for (int i = 0; i < 32; i += 4) {
                float4 o = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
                if (p.accumulate) { const float4 c = *reinterpret_cast<const float4*>(cp + i); o.x += c.x; o.y += c.y; o.z += c.z; o.w += c.w; }
                *reinterpret_cast<float4*>(cp + i) = o;
              }
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i)        // fully unrolled: v[] must stay in registers
                if (col0 + i < p.N) cp[i] = p.accumulate ? cp[i] + v[i] : v[i];
            }
          } else {
            __nv_bfloat16* cp = reinterpret_cast<__nv_bfloat16*>(p.C) + (size_t)xrow * p.ldc + col0;
            if (fullw && (p.ldc % 8 == 0)) {
#pragma unroll
              for (int i = 0; i < 32; i += 8) {
                if (p.accumulate) {
                  const uint4 c = *reinterpret_cast<const uint4*>(cp + i);
                  const uint32_t w[4] = {c.x, c.y, c.z, c.w};
#pragma unroll
                  for (int q = 0; q < 4; ++q) { v[i + 2 * q] += __uint_as_float(w[q] << 16); v[i + 2 * q + 1] += __uint_as_float(w[q] & 0xffff0000u); }
                }
                uint32_t o[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                  __nv_bfloat162 h = __floats2bfloat162_rn(v[i + 2 * q], v[i + 2 * q + 1]);
                  o[q] = *reinterpret_cast<uint32_t*>(&h);
                }
                *reinterpret_cast<uint4*>(cp + i) = make_uint4(o[0], o[1], o[2], o[3]);
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
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[acc]);
    }
    if (ok && pending >= 0) finish_tile<BN>(p, pending, par, abort_flag);
  }

  // ---------------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    // let any bulk copy still in flight land before the CTA's shared memory goes away
    const uint64_t t0 = gtimer();
    while (gtimer() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * BN);
  }
}

// ------------------------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(f);
  });
  return fn;
}

struct MapKey {
  const void* ptr; uint64_t d0, d1, ld; uint32_t b0, b1;
  bool operator==(const MapKey& o) const { return ptr == o.ptr && d0 == o.d0 && d1 == o.d1 && ld == o.ld && b0 == o.b0 && b1 == o.b1; }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    size_t h = reinterpret_cast<size_t>(k.ptr);
    for (uint64_t v : {k.d0, k.d1, k.ld, (uint64_t)k.b0, (uint64_t)k.b1}) h = h * 1000003u ^ v;
    return h;
  }
};
std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_maps;
std::mutex g_maps_mu;

// 2-D bf16 tensor map: dims {d0 (contiguous), d1}, row stride ld elements, box {b0, b1}, 128-byte swizzle.
int get_map(const void* ptr, uint64_t d0, uint64_t d1, uint64_t ld, uint32_t b0, uint32_t b1, CUtensorMap* out) {
  MapKey key{ptr, d0, d1, ld, b0, b1};
  {
    std::lock_guard<std::mutex> g(g_maps_mu);
    auto it = g_maps.find(key);
    if (it != g_maps.end()) { *out = it->second; return 0; }
  }
  EncodeTiledFn enc = get_encode();
  if (!enc) return -10;
  cuuint64_t dims[2] = {d0, d1};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {b0, b1};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return -11;
  std::lock_guard<std::mutex> g(g_maps_mu);
  if (g_maps.size() > 4096) g_maps.clear();
  g_maps[key] = *out;
  return 0;
}

int sm_count_g() {
  static int n = 0;
  if (!n) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

template <int BN, bool A_MN, bool B_MN>
int launch(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tg, GemmParams p, cudaStream_t st) {
  using C = Cfg<BN, A_MN, B_MN>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(gemm_bf16_kernel<BN, A_MN, B_MN>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  p.num_m_tiles = (p.M + BM - 1) / BM;
  p.num_n_tiles = (p.N + BN - 1) / BN;
  const int tiles = p.num_m_tiles * p.num_n_tiles;
  const int grid = tiles < sm_count_g() ? tiles : sm_count_g();
  gemm_bf16_kernel<BN, A_MN, B_MN><<<grid, NUM_THREADS, C::SMEM_BYTES, st>>>(ta, tb, tg, p);
  return (int)cudaGetLastError();
}

}  // namespace

// Exchange set-up handed in by zen_gemm_bf16_ar for the launch that follows on the same thread.
struct ZenGemmArCtx {
  int32_t nranks;
  int32_t rank;
  uint32_t epoch;
  uint32_t max_tiles;
  uint64_t wait_ns;
  uint64_t slot_elems;        // capacity (elements) of one (parity, slot) exchange buffer
  void* recv[8];              // exchange region of every rank (this rank's own address included)
  void* flags[8];             // flag region of every rank
  uint32_t* status;
  const uint32_t* epoch_dev;  // optional device step counter (see GemmParams::epoch_dev); `epoch` is then the call's index in the step
  uint32_t epoch_stride;
  uint32_t pad;
};
namespace {
thread_local const ZenGemmArCtx* g_ar_next = nullptr;
thread_local int g_coll_next = 0;                // COLL_* of the launch that follows on this thread
void fill_ar(GemmParams& p, const ZenGemmArCtx& c) {
  p.npeers = c.nranks - 1;
  p.rank = c.rank;
  p.epoch = c.epoch;
  p.epoch_dev = c.epoch_dev;
  p.epoch_stride = c.epoch_stride;
  p.max_tiles = c.max_tiles;
  p.wait_ns = c.wait_ns;
  p.slot_elems = c.slot_elems;
  p.recv_ld = (p.N + 7) / 8 * 8;
  p.status = c.status;
  p.my_recv = reinterpret_cast<__nv_bfloat16*>(c.recv[c.rank]);
  p.my_flags = reinterpret_cast<uint32_t*>(c.flags[c.rank]);
  int s = 0;
  for (int r = 0; r < c.nranks; ++r) {
    if (r == c.rank) continue;
    p.peer_recv[s] = reinterpret_cast<__nv_bfloat16*>(c.recv[r]);
    p.peer_flags[s] = reinterpret_cast<uint32_t*>(c.flags[r]);
    p.peer_rank[s] = r;
    p.peer_slot_of_me[s] = c.rank < r ? c.rank : c.rank - 1;   // this rank's slot among r's peers (rank order)
    ++s;
  }
}
}  // namespace

extern "C" {

// C[M,N] (+)= A * B^T (+ bias).  a_mn / b_mn: operand stored MN-major ([K, M] resp. [K, N] row-major)
// instead of K-major ([M, K] resp. [N, K]).  lda / ldb / ldc are row strides in elements.
// Requirements: bf16 operands, 16-byte aligned base pointers, lda and ldb multiples of 8.
// bn: 0 = choose, 128 or 256 = force the N tile.
int zen_gemm_bf16(const void* A, const void* B, void* C, const void* bias, int M, int N, int K, int lda, int ldb,
                  int ldc, int a_mn, int b_mn, int out_fp32, int accumulate, int bn, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0) return -1;
  if ((lda % 8) || (ldb % 8) || (reinterpret_cast<uintptr_t>(A) % 16) || (reinterpret_cast<uintptr_t>(B) % 16)) return -2;
  if (bn == 0) {
    const int sms = sm_count_g();
    const long t256 = (long)((M + 127) / 128) * ((N + 255) / 256), t128 = (long)((M + 127) / 128) * ((N + 127) / 128);
    const long c256 = ((t256 + sms - 1) / sms) * 2, c128 = (t128 + sms - 1) / sms;
    bn = (N <= 128 || c128 < c256) ? 128 : 256;
  }
  GemmParams p{};
  p.C = C; p.bias = bias; p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.out_fp32 = out_fp32; p.accumulate = accumulate;
  if (g_ar_next) {
    fill_ar(p, *g_ar_next);
    p.coll_mode = g_coll_next;
    g_ar_next = nullptr;
    g_coll_next = 0;
  }
  const bool ag = p.npeers > 0 && p.coll_mode == COLL_AG, rs = p.npeers > 0 && p.coll_mode == COLL_RS;
  int a_rows = M;
  if (ag || rs) {
    const int nranks = p.npeers + 1;
    if (M % nranks || (M / nranks) % BM) return -6;
    p.rows_per_rank = M / nranks;
    if (rs) p.recv_ld = (N + 7) / 8 * 8;
    if (ag) {
      // A is this rank's row block; the peer's block arrives in this rank's own region
      // the gathered rows are read through a tensor map that is chosen here, on the host, by the parity of `epoch`:
      // with a device step counter that equals the parity of the full counter only for an even stride
      if (p.epoch_dev && (p.epoch_stride & 1u)) return -8;
      if (a_mn || nranks != 2 || (K % 8) || (uint64_t)p.rows_per_rank * K > p.slot_elems ||
          (uint32_t)(p.rows_per_rank / BM) > p.max_tiles) return -7;
      p.a_local = reinterpret_cast<const __nv_bfloat16*>(A);
      p.lda_local = lda;
      a_rows = p.rows_per_rank;
    }
  }
  CUtensorMap ta, tb, tg;
  int rc;
  if (!a_mn) rc = get_map(A, (uint64_t)K, (uint64_t)a_rows, (uint64_t)lda, 64, 128, &ta);
  else rc = get_map(A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, 64, 64, &ta);
  if (rc) return rc;
  if (!b_mn) rc = get_map(B, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, 64, (uint32_t)bn, &tb);
  else rc = get_map(B, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, 64, 64, &tb);
  if (rc) return rc;
  tg = ta;
  if (ag) {
    const __nv_bfloat16* gsrc = p.my_recv + (size_t)(p.epoch & 1u) * p.npeers * p.slot_elems;
    rc = get_map(gsrc, (uint64_t)K, (uint64_t)p.rows_per_rank, (uint64_t)K, 64, 128, &tg);
    if (rc) return rc;
  }
  cudaStream_t st = (cudaStream_t)stream;
#define LAUNCH(BN_)                                                            \
  do {                                                                         \
    if (!a_mn && !b_mn) return launch<BN_, false, false>(ta, tb, tg, p, st);   \
    if (!a_mn && b_mn) return launch<BN_, false, true>(ta, tb, tg, p, st);     \
    if (a_mn && !b_mn) return launch<BN_, true, false>(ta, tb, tg, p, st);     \
    return launch<BN_, true, true>(ta, tb, tg, p, st);                         \
  } while (0)
  if (bn == 256) LAUNCH(256);
  LAUNCH(128);
#undef LAUNCH
}

int zen_gemm_ar_ctx_size() { return (int)sizeof(ZenGemmArCtx); }

// GEMM fused with an all-reduce (SUM) over a tensor-parallel group: every rank computes its partial product and
// the epilogue exchanges bf16 partial tiles through peer memory (P2P stores into the peers' exchange regions, one
// flag per tile, bounded waits), so the reduction overlaps the main loop of the following tiles.  All ranks end up
// with identical results.  Requirements on top of zen_gemm_bf16: the same M, N, K on every rank,
// M * round_up(N, 8) <= ctx->slot_elems, number of tiles <= ctx->max_tiles, out_fp32 == 0 or 1 as wanted.
int zen_gemm_bf16_ar(const void* A, const void* B, void* C, const void* bias, int M, int N, int K, int lda, int ldb,
                     int ldc, int a_mn, int b_mn, int out_fp32, int accumulate, int bn, const ZenGemmArCtx* ctx,
                     void* stream) {
  if (!ctx || ctx->nranks < 1 || ctx->nranks > 8) return -3;
  if ((uint64_t)M * (uint64_t)((N + 7) / 8 * 8) > ctx->slot_elems) return -4;
  if (bn == 0) bn = (N >= 1024 && N % 256 == 0) ? 256 : 128;
  const uint64_t tiles = (uint64_t)((M + 127) / 128) * ((N + bn - 1) / bn);
  if (tiles > ctx->max_tiles) return -5;
  if (ctx->nranks > 1) g_ar_next = ctx;
  const int rc = zen_gemm_bf16(A, B, C, bias, M, N, K, lda, ldb, ldc, a_mn, b_mn, out_fp32, accumulate, bn, stream);
  g_ar_next = nullptr;
  return rc;
}

// The same kernel with the collective chosen by `mode`: 0 = all-reduce (as zen_gemm_bf16_ar), 1 = reduce-scatter of
// the output over rows (A [M, K], C [M / nranks, N] = this rank's rows of the sum), 2 = all-gather of A over rows
// (A is this rank's [M / nranks, K] block, C [M, N]; two ranks).  M / nranks must be a multiple of 128.  Capacity:
// mode 1 needs (M / nranks) * round_up(N, 8) <= slot_elems, mode 2 needs (M / nranks) * K <= slot_elems.
int zen_gemm_bf16_coll(const void* A, const void* B, void* C, const void* bias, int M, int N, int K, int lda, int ldb,
                       int ldc, int a_mn, int b_mn, int out_fp32, int accumulate, int bn, const ZenGemmArCtx* ctx,
                       int mode, void* stream) {
  if (mode == COLL_AR) return zen_gemm_bf16_ar(A, B, C, bias, M, N, K, lda, ldb, ldc, a_mn, b_mn, out_fp32, accumulate, bn, ctx, stream);
  if (!ctx || ctx->nranks < 2 || ctx->nranks > 8 || (mode != COLL_RS && mode != COLL_AG)) return -3;
  if (bn == 0) bn = (N >= 1024 && N % 256 == 0) ? 256 : 128;
  const int rpr = M / ctx->nranks;
  if (mode == COLL_RS && (uint64_t)rpr * (uint64_t)((N + 7) / 8 * 8) > ctx->slot_elems) return -4;
  const uint64_t tiles = (uint64_t)((rpr + 127) / 128) * ((N + bn - 1) / bn);
  if (tiles > ctx->max_tiles) return -5;
  g_ar_next = ctx;
  g_coll_next = mode;
  const int rc = zen_gemm_bf16(A, B, C, bias, M, N, K, lda, ldb, ldc, a_mn, b_mn, out_fp32, accumulate, bn, stream);
  g_ar_next = nullptr;
  g_coll_next = 0;
  return rc;
}

// Last error code recorded by a kernel that gave up a wait (0 = none); clears it.
int zen_gemm_error() {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_gemm_error, sizeof(int)) != cudaSuccess) return -1;
  if (v) cudaMemcpyToSymbol(g_gemm_error, &zero, sizeof(int));
  return v;
}

}  // extern "C"
