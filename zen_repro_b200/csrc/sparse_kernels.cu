// Sparse all-reduce kernels (element granule) for sm_100a.
//
// Pipeline per bucket, one launch each, all on one stream, no host sync:
//   zen_partition_push  : stream the flat bucket through a shared-memory ring filled by bulk
//                         asynchronous copies (cp.async.bulk + mbarrier), hash 64-element blocks to
//                         owners, stage (slot, value) records per owner in shared memory and push
//                         them in large contiguous runs straight into the owner's receive region
//                         over NVLink (P2P stores).
//   zen_owner_reduce    : bounded wait on every source's mailbox at once, red.add the records
//                         into this owner's fp32 slots, red.or the occupancy bitmap.
//   zen_gather_push     : walk the occupancy bitmap, compact the touched slots chunk by chunk,
//                         reserve room in the payload with one atomic per CTA step and push
//                         bitmap|COO + values to every peer (P2P stores, or one multimem store
//                         through the NVSwitch when a multicast alias of the region exists).
//   zen_densify         : bounded wait on each owner's mailbox, one pass over the output that
//                         writes zeros and values together.
//
// Record slots and their mailboxes exist twice and alternate with the parity of the call number, so a
// rank that is one call ahead never writes into records that a slower peer is still reading.
//
// Replaces, in the reference: the three sparse_balance kernels and the
// boolean-mask compaction after them (functions_cuda_kernel.cu:97-167,
// tensor_load_balance.py:24-51), both all_to_all calls and the scatter_add /
// nonzero between them (comm.py:117-127), encode_bitmap / decode_bitmap and the
// padded all_gathers (comm.py:59-99, 128-145).
#include "tc_common.cuh"
#include "zen_common.cuh"

struct ZenSparseCtx {
  int32_t rank;
  int32_t nranks;
  uint32_t epoch;
  uint32_t fmt_mode;        // 0 auto, ZEN_FMT_COO, ZEN_FMT_BITMAP
  uint64_t wait_ns;
  char* sym[ZEN_MAX_RANKS]; // base of every rank's symmetric region
  uint64_t off_rec_mail;    // ZenMail[2][ZEN_MAX_RANKS], indexed by call parity and source
  uint64_t off_g_mail;      // ZenMail[ZEN_MAX_RANKS], indexed by owner
  uint64_t off_rec;         // uint2[2][P][cap_rec], indexed by call parity and source
  uint64_t off_g_idx;       // uint32[P][g_idx_words]: bitmap words or COO slots
  uint64_t off_g_off;       // uint32[P][nchunks + 1]: value offset of every 1024-slot chunk
  uint64_t off_g_val;       // T[P][cap_g] (stride in bytes: cap_g * 4)
  uint32_t cap_rec;
  uint32_t cap_g;
  uint32_t g_idx_words;
  uint32_t nchunks;
  float* acc;               // [S] local
  uint32_t* bitmap;         // [nwords] local
  uint32_t* chunk_off;      // unused by the kernels (kept for layout stability of the binding)
  uint32_t* cursors;        // [P] record cursors, [MAX] done counter K1, [MAX+1] done counter K3, [MAX+2] payload cursor
  uint32_t* status;         // status word
  uint64_t numel;           // N
  uint32_t nslots;          // S = sb * G
  uint32_t nwords;          // ceil(S / 32)
  ZenPerm perm;
  const uint32_t* epoch_dev;  // optional: call counter on the device (zen_sparse_epoch_bump); overrides `epoch`
  char* mc;                   // optional: multicast alias of the symmetric region (stores reach every rank)
  uint32_t k1_density_ppm;    // nonzeros per million elements that the plan was sized for (0 = unknown)
  uint32_t pad0;
};

__device__ __forceinline__ uint32_t zen_epoch(const ZenSparseCtx& c) { return c.epoch_dev ? *c.epoch_dev : c.epoch; }
__device__ __forceinline__ uint2* zen_rec_slots(const ZenSparseCtx& c, int at_rank, int src, uint32_t epoch) {
  return reinterpret_cast<uint2*>(c.sym[at_rank] + c.off_rec) + ((uint64_t)(epoch & 1u) * c.nranks + src) * c.cap_rec;
}
__device__ __forceinline__ ZenMail* zen_rec_mail(const ZenSparseCtx& c, int at_rank, int src, uint32_t epoch) {
  return reinterpret_cast<ZenMail*>(c.sym[at_rank] + c.off_rec_mail) + (epoch & 1u) * ZEN_MAX_RANKS + src;
}

#define K1_THREADS 288                                  // eight consumer warps and the producer warp
#define K1_WARPS 8
#define K1_QCAP 256
#define K1_FLUSH_MIN 128
#define K1_STAGE_BYTES 8192
#define K1_NS 3

// Eight consecutive elements as raw bits: one 16-byte vector for 16-bit types, two for fp32.
template <typename T> struct Raw8;
template <> struct Raw8<float> {
  uint32_t w[8];
  __device__ __forceinline__ void load(const float* g, uint64_t e0, uint64_t n, bool aligned) {
    if (aligned && e0 + 8 <= n) {
      const uint4 a = __ldg(reinterpret_cast<const uint4*>(g + e0)), b = __ldg(reinterpret_cast<const uint4*>(g + e0 + 4));
      w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w; w[4] = b.x; w[5] = b.y; w[6] = b.z; w[7] = b.w;
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) w[i] = (e0 + i < n) ? __float_as_uint(g[e0 + i]) : 0u;
    }
  }
  __device__ __forceinline__ void zero() {
#pragma unroll
    for (int i = 0; i < 8; ++i) w[i] = 0u;
  }
  __device__ __forceinline__ bool any() const { return ((w[0] | w[1] | w[2] | w[3] | w[4] | w[5] | w[6] | w[7]) & 0x7fffffffu) != 0u; }
  // cheap test "some element reaches the threshold" (tbits as in keep_mask; hint unused for fp32)
  __device__ __forceinline__ bool hit(uint32_t tbits, uint32_t) const {
    if (tbits <= 1u) return any();
    bool r = false;
#pragma unroll
    for (int i = 0; i < 8; ++i) r |= (w[i] & 0x7fffffffu) >= tbits;
    return r;
  }
  // select chains instead of dynamic indexing keep the vector in registers
  __device__ __forceinline__ uint32_t bits(int i) const {
    const uint32_t a = (i & 1) ? w[1] : w[0], b = (i & 1) ? w[3] : w[2], c = (i & 1) ? w[5] : w[4], d = (i & 1) ? w[7] : w[6];
    const uint32_t ab = (i & 2) ? b : a, cd = (i & 2) ? d : c;
    return (i & 4) ? cd : ab;
  }
  __device__ __forceinline__ float value(int i) const { return __uint_as_float(bits(i)); }
  __device__ __forceinline__ bool nonzero(int i) const { return (bits(i) & 0x7fffffffu) != 0u; }
  // bit i set when element i is kept: |x| >= threshold, as an integer compare of the magnitude bits (monotonic for
  // non-negative floats); tbits = 1 keeps every nonzero; NaNs are dropped when a real threshold is in force
  __device__ __forceinline__ uint32_t keep_mask(uint32_t tbits, bool use_thr, float) const {
    uint32_t m = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint32_t a = w[i] & 0x7fffffffu;
      m |= (a >= tbits && (!use_thr || a <= 0x7f800000u)) ? (1u << i) : 0u;
    }
    return m;
  }
};
template <typename T16> struct Raw8Half {
  uint32_t w[4];
  __device__ __forceinline__ void load(const T16* g, uint64_t e0, uint64_t n, bool aligned) {
    if (aligned && e0 + 8 <= n) {
      const uint4 a = __ldg(reinterpret_cast<const uint4*>(g + e0));
      w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w;
    } else {
      const unsigned short* gs = reinterpret_cast<const unsigned short*>(g);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint32_t lo = (e0 + 2 * i < n) ? gs[e0 + 2 * i] : 0u, hi = (e0 + 2 * i + 1 < n) ? gs[e0 + 2 * i + 1] : 0u;
        w[i] = lo | (hi << 16);
      }
    }
  }
  __device__ __forceinline__ void zero() { w[0] = w[1] = w[2] = w[3] = 0u; }
  __device__ __forceinline__ bool any() const { return ((w[0] | w[1] | w[2] | w[3]) & 0x7fff7fffu) != 0u; }
  __device__ __forceinline__ uint32_t bits(int i) const {
    const uint32_t a = (i & 2) ? w[1] : w[0], b = (i & 2) ? w[3] : w[2];
    return (((i & 4) ? b : a) >> ((i & 1) * 16)) & 0xffffu;
  }
  __device__ __forceinline__ bool nonzero(int i) const { return (bits(i) & 0x7fffu) != 0u; }
};
template <> struct Raw8<__nv_bfloat16> : Raw8Half<__nv_bfloat16> {
  __device__ __forceinline__ float value(int i) const { return __uint_as_float(bits(i) << 16); }
  // cheap test "some element reaches the threshold": both halves of a word at once.  addc = (0x8000 - t16) in each
  // half, t16 the threshold's magnitude bits rounded up to bf16: a half's bit 15 comes out set exactly when its
  // 15-bit magnitude is >= t16 (no carry crosses the halves, the sums stay below 0x10000).
  __device__ __forceinline__ bool hit(uint32_t, uint32_t addc) const {
    uint32_t acc = 0;
#pragma unroll
    for (int k = 0; k < 4; ++k) acc |= ((w[k] & 0x7fff7fffu) + addc) & 0x80008000u;
    return acc != 0u;
  }
  __device__ __forceinline__ uint32_t keep_mask(uint32_t tbits, bool use_thr, float) const {
    uint32_t m = 0;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const uint32_t lo = (w[k] & 0x7fffu) << 16, hi = w[k] & 0x7fff0000u;     // magnitudes as fp32 bit patterns
      m |= (lo >= tbits && (!use_thr || lo <= 0x7f800000u)) ? (1u << (2 * k)) : 0u;
      m |= (hi >= tbits && (!use_thr || hi <= 0x7f800000u)) ? (2u << (2 * k)) : 0u;
    }
    return m;
  }
};
template <> struct Raw8<__half> : Raw8Half<__half> {
  __device__ __forceinline__ float value(int i) const { return __half2float(__ushort_as_half((unsigned short)bits(i))); }
  __device__ __forceinline__ bool hit(uint32_t, uint32_t) const { return any(); }     // the threshold is applied in keep_mask
  __device__ __forceinline__ uint32_t keep_mask(uint32_t, bool use_thr, float thr) const {
    uint32_t m = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      bool keep = nonzero(i);
      if (use_thr) keep = keep && (fabsf(value(i)) >= thr);
      m |= keep ? (1u << i) : 0u;
    }
    return m;
  }
};

// ---------------------------------------------------------------------------------------------
// K1: partition + compact + push.  The bucket streams through a ring of K1_NS shared-memory stages:
// a producer warp keeps them filled with bulk asynchronous copies (full / empty mbarriers per stage),
// eight consumer warps scan them.  Every lane owns 8 consecutive elements at a time (all in one
// 64-element block, hence one owner); vectors that hold a nonzero are first compacted into a per-warp
// list, and the expensive part -- owner lookup, queue reservation, record writes -- runs on 32 listed
// vectors at a time with every lane busy.  Records go to per-owner queues in shared memory; every
// `batch` stages the consumer warps meet at a named barrier and warp w drains queue w to the owner's
// receive region in runs of at least K1_FLUSH_MIN records (a queue that fills up earlier spills
// straight to the destination).  kBroadcast = true is the method-1 variant: one queue of
// (global index, value) records pushed to every peer.  kRing = false reads the bucket with plain
// loads instead (a base pointer that is not 16-byte aligned).
#define K1_CONSUMERS 256
__device__ __forceinline__ void k1_consumer_sync() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

template <typename T> struct K1Entry { uint32_t w[sizeof(Raw8<T>) / 4]; };

template <typename T, bool kBroadcast, bool kRing>
__global__ void __launch_bounds__(K1_THREADS, 4)
zen_partition_push_kernel(const ZenSparseCtx c, const T* __restrict__ g, const float* __restrict__ thr_ptr, int batch) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  constexpr uint32_t VB = 8 * sizeof(T);                              // bytes of one 8-element vector
  constexpr uint32_t EPS = K1_STAGE_BYTES / sizeof(T);                // elements per stage
  constexpr int VPL = K1_STAGE_BYTES / VB / K1_CONSUMERS;             // vectors per lane per stage
  static_assert(VPL >= 1, "stage too small");
  constexpr int RAWW = sizeof(Raw8<T>) / 4;                           // words per vector (4 or 8)
  const int nq = kBroadcast ? 1 : c.nranks;
  unsigned char* ring = smem_raw;                                     // [K1_NS][K1_STAGE_BYTES] (kRing)
  uint2* q = reinterpret_cast<uint2*>(smem_raw + (kRing ? K1_NS * K1_STAGE_BYTES : 0));   // [nq][K1_QCAP]
  __shared__ uint64_t full[K1_NS], empty[K1_NS];
  __shared__ uint32_t qn[ZEN_MAX_RANKS];
  __shared__ uint32_t qvalid[ZEN_MAX_RANKS];
  __shared__ uint32_t s_last;
  __shared__ int s_abort;
  __shared__ __align__(16) K1Entry<T> wdat[K1_WARPS][64];             // per-warp list of vectors with a nonzero (a ring)
  __shared__ uint32_t wel[K1_WARPS][64];                              // ... and their first element index

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const bool use_thr = thr_ptr != nullptr;
  const float thr = use_thr ? fmaxf(*thr_ptr, 0.f) : 0.f;
  const uint32_t tbits = use_thr ? max(__float_as_uint(thr), 1u) : 1u; // magnitude bits an element must reach to be kept
  // the same threshold for the cheap per-vector test of 16-bit types: rounded up to 16 bits, as an addend per half
  const uint32_t t16 = min((tbits + 0xffffu) >> 16, 0x8000u) == 0u ? 1u : min((tbits + 0xffffu) >> 16, 0x8000u);
  const uint32_t addc = (0x8000u - t16) * 0x00010001u;
  const uint64_t N = c.numel;
  const uint32_t nst = (uint32_t)((N + EPS - 1) / EPS);               // stages of the whole bucket
  const uint64_t copy_end = (N * sizeof(T)) & ~15ull;                 // bytes that bulk copies may fetch
  const uint32_t full_stages = (uint32_t)(copy_end / K1_STAGE_BYTES);
  const uint32_t epoch = zen_epoch(c);
  const uint64_t rec_base = ((uint64_t)(epoch & 1u) * c.nranks + c.rank) * c.cap_rec;
  uint32_t local_status = 0;
  if (batch < 1) batch = 1;

  if (tid < ZEN_MAX_RANKS) { qn[tid] = 0; qvalid[tid] = 0; }
  if (tid == 0) {
    s_abort = 0;
    if (kRing) {
      for (int s = 0; s < K1_NS; ++s) { tc::mbar_init(&full[s], 1); tc::mbar_init(&empty[s], K1_WARPS); }
      tc::fence_barrier_init();
    }
  }
  __syncthreads();

  auto stage_bytes = [&](uint32_t it) -> uint32_t {
    if (it < full_stages) return K1_STAGE_BYTES;
    const uint64_t b0 = (uint64_t)it * K1_STAGE_BYTES;
    return b0 >= copy_end ? 0u : (uint32_t)(copy_end - b0);
  };
  // bounded wait on an mbarrier phase; gives up at once when the CTA has already aborted
  auto wait_phase = [&](uint64_t* bar, uint32_t parity) -> bool {
    if (tc::mbar_test(bar, parity)) return true;
    const uint64_t t0 = zen_globaltimer();
    for (;;) {
      for (int i = 0; i < 128; ++i)
        if (tc::mbar_test(bar, parity)) return true;
      if (*(volatile int*)&s_abort || zen_globaltimer() - t0 > c.wait_ns) { s_abort = 1; return false; }
    }
  };

  if (warp == K1_WARPS) {
    // ---- producer warp: one lane keeps the ring full
    if (kRing && lane == 0) {
      uint32_t issued[K1_NS] = {};
      uint32_t k = 0;
      for (uint32_t it = blockIdx.x; it < nst; it += gridDim.x, ++k) {
        const int s = k % K1_NS;
        if (k >= K1_NS && !wait_phase(&empty[s], ((k / K1_NS) - 1u) & 1u)) break;
        const uint32_t b = stage_bytes(it);
        tc::mbar_expect_tx(&full[s], b);
        if (b) tc::bulk_load_1d(ring + s * K1_STAGE_BYTES, reinterpret_cast<const unsigned char*>(g) + (uint64_t)it * K1_STAGE_BYTES, b, &full[s]);
        ++issued[s];
      }
      if (*(volatile int*)&s_abort) {
        // give the copies that are still in flight a bounded chance to land before the CTA (and its shared memory) goes
        const uint64_t t0 = zen_globaltimer();
        for (int s = 0; s < K1_NS; ++s) {
          if (!issued[s]) continue;
          while (!tc::mbar_test(&full[s], (issued[s] - 1u) & 1u) && zen_globaltimer() - t0 < c.wait_ns) {}
        }
      }
    }
  } else {
    // ---- consumer warps
    uint32_t wtail = 0, whead = 0;                                    // list entries appended / consumed (warp-uniform)

    // Records of one 8-element vector starting at element e32: choose the owner, reserve queue space, write them.
    auto emit = [&](uint32_t e32, const Raw8<T>& vec) {
      uint32_t m = vec.keep_mask(tbits, use_thr, thr);
      if (!m) return;
      uint32_t owner = 0, slot0 = e32;
      if (!kBroadcast) {
        const uint32_t pb = zen_perm_fwd(c.perm, e32 >> c.perm.lg);
        owner = zen_owner_of(c.perm, pb, c.nranks);
        slot0 = ((pb - owner * c.perm.sb) << c.perm.lg) + (e32 & (c.perm.block - 1u));
      }
      const uint32_t cnt = __popc(m);
      uint32_t k = atomicAdd(&qn[owner], cnt);
      bool direct = false;
      if (k + cnt > K1_QCAP) {
        if (k <= K1_QCAP) qvalid[owner] = k;                          // exactly one lane per overflow sees this
        direct = true;
        k = atomicAdd(&c.cursors[owner], cnt);                        // reserve directly in the destination
      }
      while (m) {
        const int i = __ffs(m) - 1;
        m &= m - 1;
        const uint2 rec = make_uint2(slot0 + i, vec.bits(i));
        if (!direct) {
          q[owner * K1_QCAP + k] = rec;
        } else if (k < c.cap_rec) {
          if (kBroadcast) {
            for (int p = 0; p < c.nranks; ++p)
              (reinterpret_cast<uint2*>(c.sym[p] + c.off_rec) + rec_base)[k] = rec;
          } else {
            (reinterpret_cast<uint2*>(c.sym[owner] + c.off_rec) + rec_base)[k] = rec;
          }
        } else {
          local_status |= ZEN_REC_OVERFLOW;
        }
        ++k;
      }
    };
    auto emit_entry = [&](uint32_t idx) {
      Raw8<T> r;
      const uint4* p4 = reinterpret_cast<const uint4*>(&wdat[warp][idx & 63u]);
#pragma unroll
      for (int k = 0; k < RAWW / 4; ++k) {
        const uint4 a = p4[k];
        r.w[4 * k] = a.x; r.w[4 * k + 1] = a.y; r.w[4 * k + 2] = a.z; r.w[4 * k + 3] = a.w;
      }
      emit(wel[warp][idx & 63u], r);
    };
    // warp w drains queue w when it holds a worthwhile run (or at the end)
    auto flush = [&](bool final_flush) {
      if (warp < nq) {
        uint32_t n = qn[warp];
        const bool overflowed = n > K1_QCAP;
        if (overflowed) n = qvalid[warp];
        if (n > 0 && (n >= K1_FLUSH_MIN || final_flush || overflowed)) {
          uint32_t gbase = 0;
          if (lane == 0) gbase = atomicAdd(&c.cursors[warp], n);
          gbase = __shfl_sync(0xffffffffu, gbase, 0);
          const uint32_t fit = (gbase >= c.cap_rec) ? 0u : min(n, c.cap_rec - gbase);
          if (fit < n) local_status |= ZEN_REC_OVERFLOW;
          const uint2* src = q + warp * K1_QCAP;
          if (kBroadcast) {
            for (int p = 0; p < c.nranks; ++p) {
              uint2* dst = reinterpret_cast<uint2*>(c.sym[p] + c.off_rec) + rec_base + gbase;
              for (uint32_t i = lane; i < fit; i += 32) dst[i] = src[i];
            }
          } else {
            uint2* dst = reinterpret_cast<uint2*>(c.sym[warp] + c.off_rec) + rec_base + gbase;
            for (uint32_t i = lane; i < fit; i += 32) dst[i] = src[i];
          }
          __syncwarp();
          if (lane == 0) { qn[warp] = 0; qvalid[warp] = 0; }
        } else if (overflowed && lane == 0) {
          qn[warp] = 0; qvalid[warp] = 0;
        }
      }
    };

    uint32_t kk = 0;
    int since = 0;
    const uint32_t lt_mask = (1u << lane) - 1u;
    for (uint32_t it = blockIdx.x; it < nst; it += gridDim.x, ++kk) {
      const int s = kk % K1_NS;
      Raw8<T> v[VPL];
      const uint32_t ebase = it * EPS + tid * 8u;                      // first element of this lane's first vector
      if (kRing) {
        const bool ok = wait_phase(&full[s], (kk / K1_NS) & 1u);
        const unsigned char* st = ring + s * K1_STAGE_BYTES + tid * VB;
        if (ok && it < full_stages) {                                  // a whole stage: no bounds to look at
#pragma unroll
          for (int u = 0; u < VPL; ++u) {
            const uint4* p4 = reinterpret_cast<const uint4*>(st + u * K1_CONSUMERS * VB);
#pragma unroll
            for (int k = 0; k < RAWW / 4; ++k) {
              const uint4 a = p4[k];
              v[u].w[4 * k] = a.x; v[u].w[4 * k + 1] = a.y; v[u].w[4 * k + 2] = a.z; v[u].w[4 * k + 3] = a.w;
            }
          }
        } else {
          const uint32_t sb = ok ? stage_bytes(it) : 0u;
#pragma unroll
          for (int u = 0; u < VPL; ++u) {
            const uint32_t vi = u * K1_CONSUMERS + tid;
            const uint64_t e0 = (uint64_t)it * EPS + (uint64_t)vi * 8;
            if ((vi + 1) * VB <= sb) {
              const uint4* p4 = reinterpret_cast<const uint4*>(st + u * K1_CONSUMERS * VB);
#pragma unroll
              for (int k = 0; k < RAWW / 4; ++k) {
                const uint4 a = p4[k];
                v[u].w[4 * k] = a.x; v[u].w[4 * k + 1] = a.y; v[u].w[4 * k + 2] = a.z; v[u].w[4 * k + 3] = a.w;
              }
            } else if (ok && e0 < N) {
              v[u].load(g, e0, N, false);                              // ragged end of the bucket: guarded plain loads
            } else {
              v[u].zero();
            }
          }
        }
        __syncwarp();
        if (lane == 0) tc::mbar_arrive(&empty[s]);                     // this warp is done with the stage
      } else {
#pragma unroll
        for (int u = 0; u < VPL; ++u) {
          const uint64_t e0 = (uint64_t)it * EPS + (uint64_t)(u * K1_CONSUMERS + tid) * 8;
          if (e0 < N) v[u].load(g, e0, N, false); else v[u].zero();
        }
      }
      const bool last_it = (it + gridDim.x >= nst);
#pragma unroll
      for (int u = 0; u < VPL; ++u) {
        const bool has = v[u].hit(tbits, addc);            // with a threshold most vectors of a dense bucket stop here
        const uint32_t bal = __ballot_sync(0xffffffffu, has);
        if (!bal) continue;
        if (has) {
          const uint32_t idx = (wtail + __popc(bal & lt_mask)) & 63u;
          wel[warp][idx] = ebase + (uint32_t)u * (K1_CONSUMERS * 8u);
          uint4* p4 = reinterpret_cast<uint4*>(&wdat[warp][idx]);
#pragma unroll
          for (int k = 0; k < RAWW / 4; ++k) p4[k] = make_uint4(v[u].w[4 * k], v[u].w[4 * k + 1], v[u].w[4 * k + 2], v[u].w[4 * k + 3]);
        }
        wtail += __popc(bal);
        if (wtail - whead >= 32) {
          __syncwarp();
          emit_entry(whead + lane);
          whead += 32;
          __syncwarp();
        }
      }
      if (last_it && wtail != whead) {                     // leftovers of this warp: drain with the lanes that have one
        __syncwarp();
        if ((uint32_t)lane < wtail - whead) emit_entry(whead + lane);
        whead = wtail;
      }
      if (++since >= batch || last_it) {
        since = 0;
        k1_consumer_sync();                                // every consumer's records are in the queues
        flush(last_it);
        k1_consumer_sync();                                // queues drained before the next records arrive
      }
    }
  }

  if (s_abort) local_status |= ZEN_TIMEOUT;
  if (local_status) atomicOr(c.status, local_status);
  // completion: the last CTA to arrive publishes counts and epochs to the consumers.  Every thread's stores are
  // ordered before thread 0's system-scope fence by the barrier (the fence is cumulative).
  __syncthreads();
  if (tid == 0) {
    __threadfence_system();
    const uint32_t prev = atomicAdd(&c.cursors[ZEN_MAX_RANKS], 1u);
    s_last = (prev == gridDim.x - 1) ? 1u : 0u;
  }
  __syncthreads();
  if (s_last) {
    __threadfence_system();
    if (tid < c.nranks) {
      const int p = tid;
      const uint32_t raw = atomicAdd(&c.cursors[kBroadcast ? 0 : p], 0u);
      const uint32_t st = atomicOr(c.status, 0u);
      ZenMail* mail = zen_rec_mail(c, p, c.rank, epoch);
      mail->count = min(raw, c.cap_rec);
      mail->info = ((raw > c.cap_rec) || (st & ZEN_REC_OVERFLOW)) ? 1u : 0u;
      mail->aux = 0;
      __threadfence_system();
      zen_st_release_sys(&mail->epoch, epoch);
    }
    __syncthreads();
    if (tid < ZEN_MAX_RANKS + 1) c.cursors[tid] = 0;                  // ready for the next call
  }
}

// ---------------------------------------------------------------------------------------------
// K2: owner-side reduce of sources [src_begin, src_end).  One launch over all sources is the fast
// mode; one launch per source gives a fixed accumulation order.  The waits on the sources' mailboxes
// run side by side (one thread each); records are read two per 16-byte load, four loads in flight.
template <typename T>
__global__ void __launch_bounds__(256)
zen_owner_reduce_kernel(const ZenSparseCtx c, int src_begin, int src_end, int allow_dense) {
  __shared__ uint32_t s_n[ZEN_MAX_RANKS];
  __shared__ uint32_t s_flag[ZEN_MAX_RANKS];
  const uint32_t epoch = zen_epoch(c);
  const int ns = src_end - src_begin;
  if ((int)threadIdx.x < ns) {
    const int s = src_begin + threadIdx.x;
    const ZenMail* mail = zen_rec_mail(c, c.rank, s, epoch);
    uint32_t n = 0, fl = 0;
    if (zen_wait_epoch(&mail->epoch, epoch, c.wait_ns)) {
      // count and info were written before the epoch's release store: plain loads after the acquire above see them
      const uint32_t cnt = *reinterpret_cast<const volatile uint32_t*>(&mail->count);
      const uint32_t info = *reinterpret_cast<const volatile uint32_t*>(&mail->info);
      n = min(cnt, c.cap_rec);
      if (info & 1u) fl = ZEN_PEER_OVERFLOW;
    } else {
      fl = ZEN_TIMEOUT;
    }
    s_n[threadIdx.x] = n;
    s_flag[threadIdx.x] = fl;
  }
  __syncthreads();
  uint32_t local_status = 0;
  // With many records (more than one per eight slots) the occupancy bitmap is not kept: the gather then reads every
  // slot anyway and takes "touched" to mean "sum is not zero" (a slot whose sum is exactly zero need not travel), which
  // halves the number of atomics here.  The choice is published for the gather kernel of this call.
  uint64_t total = 0;
  for (int k = 0; k < ns; ++k) total += s_n[k];
  const bool dense_mode = allow_dense && total * 8ull > (uint64_t)c.nslots;
  if (blockIdx.x == 0 && threadIdx.x == 0) c.cursors[ZEN_MAX_RANKS + 3] = dense_mode ? 1u : 0u;
  auto apply = [&](uint32_t slot, uint32_t bits) {
    if (slot < c.nslots) {
      atomicAdd(&c.acc[slot], ZenVal<T>::unbits(bits));
      if (!dense_mode) atomicOr(&c.bitmap[slot >> 5], 1u << (slot & 31));
    } else {
      local_status |= ZEN_BAD_ARG;
    }
  };
  const uint32_t gtid = blockIdx.x * blockDim.x + threadIdx.x, gstride = gridDim.x * blockDim.x;
  for (int k = 0; k < ns; ++k) {
    if (threadIdx.x == 0 && blockIdx.x == 0) local_status |= s_flag[k];
    const uint32_t n = s_n[k];
    const uint2* rec = zen_rec_slots(c, c.rank, src_begin + k, epoch);
    const uint4* rec4 = reinterpret_cast<const uint4*>(rec);
    const uint32_t npair = n >> 1;
    for (uint32_t i = gtid; i < npair; i += 4 * gstride) {
      uint4 r[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const uint32_t j = i + u * gstride;
        r[u] = (j < npair) ? rec4[j] : make_uint4(0xffffffffu, 0u, 0xffffffffu, 0u);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (i + u * gstride < npair) { apply(r[u].x, r[u].y); apply(r[u].z, r[u].w); }
      }
    }
    if ((n & 1u) && gtid == 0) { const uint2 r = rec[n - 1]; apply(r.x, r.y); }
  }
  if (local_status) atomicOr(c.status, local_status);
}

// ---------------------------------------------------------------------------------------------
// K3: one warp per 1024-slot chunk: compact the chunk's touched slots into the warp's shared-memory
// staging area and push the run -- values, and COO slots or bitmap words + the chunk's value offset --
// to every peer.  Room in this owner's payload is reserved per CTA step (8 to 32 chunks) with one atomic;
// runs start on 8-value boundaries, so every push is a 16-byte vector store.  Chunks may land in the
// payload in any order: the consumer finds a chunk's values through its offset (bitmap) or does not
// care (COO).
#define K3_WARPS 8
#define K3_RUN_ALIGN 8u

__device__ __forceinline__ void zen_multimem_st16(void* mc_addr, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr), "f"(__uint_as_float(v.x)),
               "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)), "f"(__uint_as_float(v.w)) : "memory");
}
__device__ __forceinline__ void zen_multimem_st4(void* mc_addr, uint32_t v) {
  asm volatile("multimem.st.relaxed.sys.global.b32 [%0], %1;" ::"l"(mc_addr), "r"(v) : "memory");
}

#define K3_CPW 4                                          // chunks per warp and step
#define K3_CPS (K3_WARPS * K3_CPW)                        // chunks per CTA step: one reservation in the payload for all of them

template <typename T>
__global__ void __launch_bounds__(K3_WARPS * 32)
zen_gather_push_kernel(const ZenSparseCtx c, int cpw) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // cpw = chunks per warp and step (1 .. K3_CPW), chosen by the launcher so that the steps fill one wave of CTAs
  // per-warp staging of one chunk: up to 1024 slot ids and values (plus padding to a whole 16-byte vector)
  uint32_t* s_idx = reinterpret_cast<uint32_t*>(smem_raw) + warp * 1032;
  T* s_val = reinterpret_cast<T*>(smem_raw + K3_WARPS * 1032 * 4) + warp * 1032;
  __shared__ uint32_t s_last, s_fmt, s_gbase, s_tot[K3_CPS];
  const uint32_t epoch = zen_epoch(c);
  if (tid == 0) {
    // index format: bitmap when more than one slot in 32 is expected to be touched.  The estimate is the number of
    // records received (an upper bound of the union), which every CTA reads from the same mails.
    uint32_t fmt = c.fmt_mode;
    uint64_t recs = 0;
    for (int s = 0; s < c.nranks; ++s) recs += min(zen_rec_mail(c, c.rank, s, epoch)->count, c.cap_rec);
    if (fmt == 0) fmt = (recs * 32ull > (uint64_t)c.nslots) ? ZEN_FMT_BITMAP : ZEN_FMT_COO;
    // a COO list (touched slots plus the padding between runs) must fit the index region
    if (fmt == ZEN_FMT_COO && min(recs, (uint64_t)c.nslots) + K3_RUN_ALIGN * (uint64_t)c.nchunks > (uint64_t)c.g_idx_words) fmt = ZEN_FMT_BITMAP;
    s_fmt = fmt;
  }
  __syncthreads();
  const uint32_t fmt = s_fmt;
  constexpr uint32_t VPV = 16 / sizeof(T);                               // values per 16-byte vector
  uint32_t local_status = 0;
  char* mc = c.mc;
  const bool no_bitmap = c.cursors[ZEN_MAX_RANKS + 3] != 0u;            // the reduce kept no bitmap: touched = nonzero sum
  const uint32_t cps = K3_WARPS * (uint32_t)cpw;                        // chunks per CTA step
  const uint32_t nsteps = (c.nchunks + cps - 1) / cps;

  // One step = K3_CPS consecutive chunks, K3_CPW per warp.  The warps count their chunks' touched slots, the CTA
  // reserves room for all of them with ONE atomic on the payload cursor (atomics on one address are served one after
  // the other, so there must be few), then every warp compacts and pushes its chunks on its own.
  for (uint32_t step = blockIdx.x; step < nsteps; step += gridDim.x) {
    const uint32_t ch_first = step * cps + warp * cpw;
    uint32_t word[K3_CPW], incl[K3_CPW];
#pragma unroll
    for (int j = 0; j < K3_CPW; ++j) {
      const uint32_t ch = ch_first + j, wi = ch * 32 + lane;
      word[j] = 0;
      if (j < cpw && ch < c.nchunks && wi < c.nwords) {
        if (no_bitmap) {
          const float4* ap4 = reinterpret_cast<const float4*>(c.acc + (size_t)wi * 32);
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const float4 v = ap4[k];
            word[j] |= ((__float_as_uint(v.x) & 0x7fffffffu) ? 1u : 0u) << (4 * k) | ((__float_as_uint(v.y) & 0x7fffffffu) ? 2u : 0u) << (4 * k) |
                       ((__float_as_uint(v.z) & 0x7fffffffu) ? 4u : 0u) << (4 * k) | ((__float_as_uint(v.w) & 0x7fffffffu) ? 8u : 0u) << (4 * k);
          }
        } else {
          word[j] = c.bitmap[wi];
          if (word[j]) c.bitmap[wi] = 0;                                 // leave the bitmap clean for the next call
        }
      }
    }
#pragma unroll
    for (int j = 0; j < K3_CPW; ++j) {
      uint32_t v = __popc(word[j]);
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        uint32_t t = __shfl_up_sync(0xffffffffu, v, d);
        if (lane >= d) v += t;
      }
      incl[j] = v;
      if (lane == 31 && j < cpw) s_tot[warp * cpw + j] = (v + K3_RUN_ALIGN - 1) & ~(K3_RUN_ALIGN - 1u);   // run length, padded
    }
    __syncthreads();
    // offsets of this warp's chunks inside the CTA's reservation: prefix over the padded run lengths (one per lane)
    uint32_t pre = ((uint32_t)lane < cps) ? s_tot[lane] : 0u;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      uint32_t t = __shfl_up_sync(0xffffffffu, pre, d);
      if (lane >= d) pre += t;
    }
    const uint32_t cta_total = __shfl_sync(0xffffffffu, pre, 31);
    pre -= ((uint32_t)lane < cps) ? s_tot[lane] : 0u;                    // exclusive
    if (tid == 0) s_gbase = cta_total ? atomicAdd(&c.cursors[ZEN_MAX_RANKS + 2], cta_total) : 0u;
    __syncthreads();
    const uint32_t cta_base = s_gbase;
    const bool fits = cta_base + cta_total <= c.cap_g && (fmt != ZEN_FMT_COO || cta_base + cta_total <= c.g_idx_words);
    if (cta_total && !fits) local_status |= ZEN_GATHER_OVERFLOW;
#pragma unroll
    for (int j = 0; j < K3_CPW; ++j) {
      const uint32_t ch = ch_first + j, wi = ch * 32 + lane;
      if (j >= cpw || ch >= c.nchunks) continue;
      const uint32_t w0 = word[j], pc = __popc(w0);
      const uint32_t n = __shfl_sync(0xffffffffu, incl[j], 31);
      const uint32_t nres = (n + K3_RUN_ALIGN - 1) & ~(K3_RUN_ALIGN - 1u);
      const uint32_t gbase = cta_base + __shfl_sync(0xffffffffu, pre, warp * cpw + j);
      {
        // A lane whose word is non-empty appends its touched slots (in slot order) to the staging run and clears
        // them.  Sparse words are walked bit by bit (only the touched 32-byte sectors move); a warp with dense words
        // streams all 32 slots of each word as eight 16-byte vectors instead.
        uint32_t r = incl[j] - pc;
        float* ap = c.acc + (size_t)ch * 1024 + (size_t)lane * 32;
        const uint32_t slot0 = ch * 1024 + lane * 32;
        const bool dense = no_bitmap || __any_sync(0xffffffffu, pc > 10);
        if (dense) {
          if (w0) {
            float f[32];
            float4* ap4 = reinterpret_cast<float4*>(ap);
#pragma unroll
            for (int k = 0; k < 8; ++k) *reinterpret_cast<float4*>(&f[4 * k]) = ap4[k];
#pragma unroll
            for (int k = 0; k < 8; ++k) ap4[k] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              if ((w0 >> i) & 1u) {
                s_val[r] = ZenVal<T>::from_f(f[i]);
                if (fmt == ZEN_FMT_COO) s_idx[r] = slot0 + i;
                ++r;
              }
            }
          }
        } else {
          uint32_t w = w0;
          while (w) {
            int i[4];
            float fv[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) { i[u] = w ? (__ffs(w) - 1) : -1; w &= w - 1; }
#pragma unroll
            for (int u = 0; u < 4; ++u) fv[u] = (i[u] >= 0) ? ap[i[u]] : 0.f;
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              if (i[u] >= 0) {
                ap[i[u]] = 0.f;
                s_val[r] = ZenVal<T>::from_f(fv[u]);
                if (fmt == ZEN_FMT_COO) s_idx[r] = slot0 + i[u];
                ++r;
              }
            }
          }
        }
      }
      if (fmt == ZEN_FMT_COO && (uint32_t)lane < nres - n) s_idx[n + lane] = 0xffffffffu;   // padding entries are skipped by the consumer
      __syncwarp();
      if (fits) {
        const uint32_t nvec = nres / VPV, nvi = nres / 4;
        const uint64_t val_off = c.off_g_val + (uint64_t)c.rank * c.cap_g * 4ull + (uint64_t)gbase * sizeof(T);
        const uint64_t idx_off = c.off_g_idx + ((uint64_t)c.rank * c.g_idx_words + gbase) * 4ull;
        const uint64_t bm_off = c.off_g_idx + ((uint64_t)c.rank * c.g_idx_words + wi) * 4ull;
        const uint64_t off_off = c.off_g_off + ((uint64_t)c.rank * (c.nchunks + 1) + ch) * 4ull;
        const uint4* sv4 = reinterpret_cast<const uint4*>(s_val);
        const uint4* si4 = reinterpret_cast<const uint4*>(s_idx);
        if (mc) {                                                        // one store, replicated by the switch
          for (uint32_t i = lane; i < nvec; i += 32) zen_multimem_st16(mc + val_off + (uint64_t)i * 16, sv4[i]);
          if (fmt == ZEN_FMT_COO) {
            for (uint32_t i = lane; i < nvi; i += 32) zen_multimem_st16(mc + idx_off + (uint64_t)i * 16, si4[i]);
          } else {
            if (wi < c.nwords) zen_multimem_st4(mc + bm_off, w0);
            if (lane == 0) zen_multimem_st4(mc + off_off, gbase);
          }
        } else {
          for (int p = 0; p < c.nranks; ++p) {
            char* base = c.sym[p];
            uint4* dv = reinterpret_cast<uint4*>(base + val_off);
            for (uint32_t i = lane; i < nvec; i += 32) dv[i] = sv4[i];
            if (fmt == ZEN_FMT_COO) {
              uint4* di = reinterpret_cast<uint4*>(base + idx_off);
              for (uint32_t i = lane; i < nvi; i += 32) di[i] = si4[i];
            } else {
              if (wi < c.nwords) *reinterpret_cast<uint32_t*>(base + bm_off) = w0;
              if (lane == 0) *reinterpret_cast<uint32_t*>(base + off_off) = gbase;
            }
          }
        }
      }
      __syncwarp();                                                      // the staging area is free again
    }
  }

  if (local_status) atomicOr(c.status, local_status);
  __syncthreads();
  if (tid == 0) {
    __threadfence_system();
    const uint32_t prev = atomicAdd(&c.cursors[ZEN_MAX_RANKS + 1], 1u);
    s_last = (prev == gridDim.x - 1) ? 1u : 0u;
  }
  __syncthreads();
  if (s_last) {
    __threadfence_system();
    if (tid < c.nranks) {
      const uint32_t total = atomicAdd(&c.cursors[ZEN_MAX_RANKS + 2], 0u);
      const uint32_t st = atomicOr(c.status, 0u);
      const bool overflow = total > c.cap_g || (st & ZEN_GATHER_OVERFLOW);
      ZenMail* mail = reinterpret_cast<ZenMail*>(c.sym[tid] + c.off_g_mail) + c.rank;
      mail->count = overflow ? 0u : total;
      mail->info = ((overflow || (st & (ZEN_REC_OVERFLOW | ZEN_PEER_OVERFLOW | ZEN_TIMEOUT))) ? 1u : 0u) | (fmt << 8);
      mail->aux = 0;
      __threadfence_system();
      zen_st_release_sys(&mail->epoch, epoch);
    }
    __syncthreads();
    if (tid == 0) { c.cursors[ZEN_MAX_RANKS + 1] = 0; c.cursors[ZEN_MAX_RANKS + 2] = 0; }
  }
}

// ---------------------------------------------------------------------------------------------
// K4: densify.  Walks every owner's slot space chunk by chunk; every output element is written once
// (zeros included), so the output needs no memset.  Owners that chose COO get their blocks
// zero-filled here and their values scattered by zen_densify_coo_kernel afterwards.  The bitmap word
// and value offset of a warp's next chunk are fetched while it works on the current one.
template <typename T>
__global__ void __launch_bounds__(256)
zen_densify_kernel(const ZenSparseCtx c, T* __restrict__ out) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ uint32_t s_fmt[ZEN_MAX_RANKS];
  const int tid = threadIdx.x, lane = tid & 31;
  T* tile = reinterpret_cast<T*>(smem_raw) + (tid >> 5) * 1024;       // this warp's 1024-element staging tile
  const uint32_t epoch = zen_epoch(c);
  uint32_t local_status = 0;
  if (tid < c.nranks) {
    const ZenMail* mail = reinterpret_cast<const ZenMail*>(c.sym[c.rank] + c.off_g_mail) + tid;
    uint32_t f = 0;
    if (zen_wait_epoch(&mail->epoch, epoch, c.wait_ns)) {
      const uint32_t info = zen_ld_acquire_sys(&mail->info);
      f = (info >> 8) & 0xffu;
      if (info & 1u) { local_status |= ZEN_PEER_OVERFLOW; f = 0; }
    } else {
      local_status |= ZEN_TIMEOUT;
    }
    s_fmt[tid] = f;
  }
  __syncthreads();
  const uint32_t G = c.perm.block;
  const uint64_t N = c.numel;
  const uint32_t gw = (blockIdx.x * blockDim.x + tid) >> 5;
  const uint32_t nw = (gridDim.x * blockDim.x) >> 5;
  const uint32_t nunits = (uint32_t)c.nranks * c.nchunks;
  const char* base = c.sym[c.rank];
  const uint32_t* gidx = reinterpret_cast<const uint32_t*>(base + c.off_g_idx);
  const uint32_t* goff = reinterpret_cast<const uint32_t*>(base + c.off_g_off);
  // units are (owner, chunk) pairs walked with a fixed stride; the pair is advanced without divisions
  const uint32_t stride_o = nw / c.nchunks, stride_ch = nw % c.nchunks;
  auto advance = [&](uint32_t& o, uint32_t& ch) {
    o += stride_o; ch += stride_ch;
    if (ch >= c.nchunks) { ch -= c.nchunks; ++o; }
  };
  auto fetch = [&](uint32_t o, uint32_t ch, uint32_t& word, uint32_t& coff) {
    word = 0; coff = 0;
    if (o >= (uint32_t)c.nranks || s_fmt[o] != ZEN_FMT_BITMAP) return;
    const uint32_t wi = ch * 32 + lane;
    if (wi < c.nwords) word = gidx[(size_t)o * c.g_idx_words + wi];
    coff = goff[(size_t)o * (c.nchunks + 1) + ch];
  };
  uint32_t o = gw / c.nchunks, ch = gw % c.nchunks;
  uint32_t word, coff;
  fetch(o, ch, word, coff);
  for (uint32_t unit = gw; unit < nunits; unit += nw) {
    uint32_t no = o, nch = ch, nword, ncoff;
    advance(no, nch);
    fetch(no, nch, nword, ncoff);
    const T* gval = reinterpret_cast<const T*>(base + c.off_g_val + (uint64_t)o * c.cap_g * 4ull);
    uint32_t incl = __popc(word);
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      uint32_t t = __shfl_up_sync(0xffffffffu, incl, d);
      if (lane >= d) incl += t;
    }
    const uint32_t woff = coff + incl - __popc(word);
    const uint32_t n_chunk = __shfl_sync(0xffffffffu, incl, 31);
    (void)n_chunk;
    if (G == 64u) {
      // Assemble the chunk's sixteen 64-element blocks in this warp's shared-memory tile (zeros, then the values at
      // their slots) and write each block out with full 16-byte vectors: the memory system sees whole lines, however
      // few or many values the chunk holds.  Lane j < 16 finds where block j lives in the output.
      constexpr int NV = 1024 * sizeof(T) / 16 / 32;      // 16-byte vectors per lane in the tile (4 or 8)
      constexpr int VPB = 64 * sizeof(T) / 16;            // vectors per block (8 or 16)
      constexpr int EPV = 16 / sizeof(T);                 // elements per vector
      uint64_t eb = ~0ull;
      {
        const uint32_t slotb = ch * 1024 + (lane & 15) * 64;
        if (slotb < c.nslots) {
          const uint64_t e = (uint64_t)zen_perm_inv(c.perm, o * c.perm.sb + (slotb >> 6)) << 6;
          if (e < N) eb = e;
        }
      }
      uint4* tv = reinterpret_cast<uint4*>(tile);
#pragma unroll
      for (int k = 0; k < NV; ++k) tv[k * 32 + lane] = make_uint4(0u, 0u, 0u, 0u);
      __syncwarp();
      {
        uint32_t w = word, at = woff;
        T* mine = tile + lane * 32;
        while (w) {
          const int i = __ffs(w) - 1;
          w &= w - 1;
          if (at < c.cap_g) mine[i] = gval[at];
          ++at;
        }
      }
      __syncwarp();
#pragma unroll
      for (int k = 0; k < NV; ++k) {
        const int v = k * 32 + lane;
        const uint64_t e0 = __shfl_sync(0xffffffffu, eb, v / VPB);
        if (e0 == ~0ull) continue;
        const uint64_t e = e0 + (uint64_t)(v % VPB) * EPV;
        if (e + EPV <= N) {
          *reinterpret_cast<uint4*>(out + e) = tv[v];
        } else {
#pragma unroll
          for (int i = 0; i < EPV; ++i)
            if (e + i < N) out[e + i] = tile[v * EPV + i];
        }
      }
      __syncwarp();                                        // the tile is free for the next chunk
      word = nword; coff = ncoff; o = no; ch = nch;
      continue;
    }
    // four passes of 256 slots: every lane produces 8 consecutive output elements (one or two 16-byte stores)
#pragma unroll
    for (int it = 0; it < 4; ++it) {
      const int wsel = it * 8 + (lane >> 2);
      const uint32_t w = __shfl_sync(0xffffffffu, word, wsel);
      const uint32_t wo = __shfl_sync(0xffffffffu, woff, wsel);
      const uint32_t slot0 = ch * 1024 + it * 256 + lane * 8;
      if (slot0 >= c.nslots) continue;
      const uint32_t blk = zen_perm_inv(c.perm, o * c.perm.sb + (slot0 >> c.perm.lg));
      const uint64_t e = ((uint64_t)blk << c.perm.lg) + (slot0 & (G - 1u));
      if (e >= N) continue;
      const uint32_t sh = (lane & 3) * 8;
      const uint32_t byte = (w >> sh) & 0xffu;
      const uint32_t off0 = wo + __popc(w & ((1u << sh) - 1u));
      // walk the set bits of this lane's byte only (most bytes are empty or hold one or two values) and drop each value
      // into its place in the 16-byte (32-byte for fp32) output vector
      constexpr int NW = sizeof(T) == 2 ? 4 : 8;
      uint32_t pk[NW];
#pragma unroll
      for (int k = 0; k < NW; ++k) pk[k] = 0u;
      uint32_t b = byte, at = off0;
      while (b) {
        const int i = __ffs(b) - 1;
        b &= b - 1;
        uint32_t bits = 0u;
        if (at < c.cap_g) bits = ZenVal<T>::bits(gval[at]);
        ++at;
        if (sizeof(T) == 2) {
          const uint32_t v = bits << ((i & 1) * 16);
#pragma unroll
          for (int k = 0; k < 4; ++k) pk[k] |= ((i >> 1) == k) ? v : 0u;
        } else {
#pragma unroll
          for (int k = 0; k < NW; ++k) pk[k] |= (i == k) ? bits : 0u;
        }
      }
      if (e + 8 <= N) {
        reinterpret_cast<uint4*>(out + e)[0] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
        if (sizeof(T) == 4) reinterpret_cast<uint4*>(out + e)[1] = make_uint4(pk[NW - 4], pk[NW - 3], pk[NW - 2], pk[NW - 1]);
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          if (e + i < N) {
            const uint32_t bits = (sizeof(T) == 2) ? ((pk[(i >> 1) % NW] >> ((i & 1) * 16)) & 0xffffu) : pk[i % NW];
            out[e + i] = ZenVal<T>::from_bits(bits);
          }
        }
      }
    }
    word = nword; coff = ncoff; o = no; ch = nch;
  }
  if (local_status) atomicOr(c.status, local_status);
}

template <typename T>
__global__ void __launch_bounds__(256)
zen_densify_coo_kernel(const ZenSparseCtx c, T* __restrict__ out) {
  __shared__ uint32_t s_n[ZEN_MAX_RANKS];
  const uint32_t G = c.perm.block;
  const uint32_t epoch = zen_epoch(c);
  if (threadIdx.x < c.nranks) {
    const ZenMail* mail = reinterpret_cast<const ZenMail*>(c.sym[c.rank] + c.off_g_mail) + threadIdx.x;
    uint32_t n = 0;
    // the bitmap pass of this call already waited for this epoch
    if (zen_ld_acquire_sys(&mail->epoch) == epoch) {
      const uint32_t info = zen_ld_acquire_sys(&mail->info);
      if (((info >> 8) & 0xffu) == ZEN_FMT_COO && !(info & 1u))
        n = min(zen_ld_acquire_sys(&mail->count), min(c.cap_g, c.g_idx_words));
    }
    s_n[threadIdx.x] = n;
  }
  __syncthreads();
  for (int o = 0; o < c.nranks; ++o) {
    const uint32_t n = s_n[o];
    if (n == 0) continue;
    const char* base = c.sym[c.rank];
    const uint32_t* gi = reinterpret_cast<const uint32_t*>(base + c.off_g_idx) + (uint64_t)o * c.g_idx_words;
    const T* gv = reinterpret_cast<const T*>(base + c.off_g_val + (uint64_t)o * c.cap_g * 4ull);
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
      const uint32_t slot = gi[i];
      if (slot >= c.nslots) continue;                                  // padding between runs
      const uint32_t blk = zen_perm_inv(c.perm, o * c.perm.sb + (slot >> c.perm.lg));
      const uint64_t e = ((uint64_t)blk << c.perm.lg) + (slot & (G - 1u));
      if (e < c.numel) out[e] = gv[i];
    }
  }
}

// Method 1 consumer: out[idx] += val for one source, read-modify-write in T (indices are unique
// within a source, and sources are applied by separate launches in rank order).
template <typename T>
__global__ void __launch_bounds__(256)
zen_scatter_source_kernel(const ZenSparseCtx c, T* __restrict__ out, int src) {
  __shared__ uint32_t s_ok;
  const uint32_t epoch = zen_epoch(c);
  const ZenMail* mail = zen_rec_mail(c, c.rank, src, epoch);
  if (threadIdx.x == 0) s_ok = zen_wait_epoch(&mail->epoch, epoch, c.wait_ns) ? 1u : 0u;
  __syncthreads();
  if (!s_ok) { if (threadIdx.x == 0) atomicOr(c.status, ZEN_TIMEOUT); return; }
  if ((mail->info & 1u) && threadIdx.x == 0) atomicOr(c.status, ZEN_PEER_OVERFLOW);
  const uint32_t n = min(mail->count, c.cap_rec);
  const uint2* rec = zen_rec_slots(c, c.rank, src, epoch);
  for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    const uint2 r = rec[i];
    if (r.x < c.numel) out[r.x] = ZenVal<T>::from_f(ZenVal<T>::to_f(out[r.x]) + ZenVal<T>::unbits(r.y));
  }
}

__global__ void zen_sparse_epoch_bump_kernel(uint32_t* e) { *e += 1u; }

// ---------------------------------------------------------------------------------------------
// Owner map (API parity with hash_index, functions_cuda_kernel.cu:169-177): out[i] = owner(i).
// mode 0: block permutation; mode 1: the reference's cubic polynomial, owner = (h % M) / (M / P).
__device__ __forceinline__ uint32_t zen_poly3(uint32_t k, uint32_t seed) {
  return 573729859u * k * k * k + 0xcc9e2d51u * k * k + 0x1b873593u * k + seed;
}

__global__ void __launch_bounds__(256)
zen_owner_map_kernel(int32_t* __restrict__ out, uint64_t n, ZenPerm perm, int mode, uint32_t table, int parts) {
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
    if (mode == 0) {
      out[i] = (int32_t)zen_owner_of(perm, zen_perm_fwd(perm, (uint32_t)(i >> perm.lg)), parts);
    } else {
      const uint32_t per = table / parts;
      out[i] = (int32_t)((zen_poly3((uint32_t)i, 10001861u) % table) / per);
    }
  }
}

// Reference-compatible balancer (sparse_balance, functions_cuda_kernel.cu:97-167): open-addressing
// table of element indices with up to `rehash` probes inside the partition chosen by the first
// probe, overflow appended per partition.  Differences: slots are claimed with atomicCAS (no lost
// indices), indices are stored +1 so that element 0 is representable, the overflow cursor is bounded.
template <typename T>
__global__ void __launch_bounds__(256)
zen_sparse_balance_kernel(const T* __restrict__ in, uint64_t n, int32_t* __restrict__ table, uint32_t table_size,
                          int32_t* __restrict__ serial, uint32_t serial_per_part, uint32_t* __restrict__ cursors,
                          int parts, int rehash, uint32_t* __restrict__ status) {
  const uint32_t per = table_size / parts;
  const uint32_t seeds[3] = {10001861u, 100703u, 5002639u};
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
    if (ZenVal<T>::to_f(in[i]) == 0.f) continue;
    const uint32_t first = zen_poly3((uint32_t)i, seeds[0]) % table_size;
    const uint32_t part = first / per, start = part * per;
    bool placed = atomicCAS(&table[first], 0, (int32_t)i + 1) == 0;
    for (int r = 1; r < rehash && r < 3 && !placed; ++r) {
      const uint32_t s = start + zen_poly3((uint32_t)i, seeds[r]) % per;
      placed = atomicCAS(&table[s], 0, (int32_t)i + 1) == 0;
    }
    if (!placed) {
      const uint32_t k = atomicAdd(&cursors[part], 1u);
      if (k < serial_per_part) serial[(uint64_t)part * serial_per_part + k] = (int32_t)i + 1;
      else atomicOr(status, ZEN_REC_OVERFLOW);
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Host launchers (C ABI, called through ctypes with raw pointers and the caller's stream).
static inline int grid_for(uint64_t work_items, int per_cta, int max_ctas) {
  uint64_t g = (work_items + per_cta - 1) / per_cta;
  if (g < 1) g = 1;
  if (g > (uint64_t)max_ctas) g = max_ctas;
  return (int)g;
}

static int g_sm_count = 0;
static int sm_count() {
  if (!g_sm_count) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_sm_count, cudaDevAttrMultiProcessorCount, dev);
    if (g_sm_count <= 0) g_sm_count = 148;
  }
  return g_sm_count;
}

template <typename T, bool kBroadcast, bool kRing>
static int launch_partition_as(const ZenSparseCtx& c, const void* g, const float* thr, cudaStream_t st) {
  constexpr uint32_t EPS = K1_STAGE_BYTES / sizeof(T);
  const uint64_t nst = (c.numel + EPS - 1) / EPS;
  const int nq = kBroadcast ? 1 : c.nranks;
  const size_t smem = (size_t)nq * K1_QCAP * sizeof(uint2) + (kRing ? (size_t)K1_NS * K1_STAGE_BYTES : 0);
  ZEN_CUDA_CHECK_RET(cudaFuncSetAttribute(zen_partition_push_kernel<T, kBroadcast, kRing>,
                                          cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  // every CTA takes a fixed share of the stages, so the grid is exactly what is resident at once
  int per_sm = 0;
  ZEN_CUDA_CHECK_RET(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, zen_partition_push_kernel<T, kBroadcast, kRing>,
                                                                   K1_THREADS, smem));
  if (per_sm < 1) per_sm = 1;
  const int grid = grid_for(nst, 1, sm_count() * per_sm);
  // stages between two drains of the queues: as many as keep a queue below half of its capacity at the density the
  // plan was sized for (c.k1_density_ppm nonzeros per million elements; 0 = unknown)
  int batch = 4;
  if (c.k1_density_ppm) {
    const double per_stage = (double)EPS * c.k1_density_ppm * 1e-6 / nq;
    batch = per_stage > 0 ? (int)((K1_QCAP / 2) / per_stage) : 8;
    if (batch < 1) batch = 1;
    if (batch > 8) batch = 8;
  }
  zen_partition_push_kernel<T, kBroadcast, kRing><<<grid, K1_THREADS, smem, st>>>(c, (const T*)g, thr, batch);
  return (int)cudaGetLastError();
}

template <typename T>
static int launch_partition(const ZenSparseCtx& c, const void* g, const float* thr, int broadcast, cudaStream_t st) {
  const bool ring = reinterpret_cast<uintptr_t>(g) % 16 == 0;       // bulk copies need a 16-byte aligned source
  if (broadcast) return ring ? launch_partition_as<T, true, true>(c, g, thr, st) : launch_partition_as<T, true, false>(c, g, thr, st);
  return ring ? launch_partition_as<T, false, true>(c, g, thr, st) : launch_partition_as<T, false, false>(c, g, thr, st);
}

#define DISPATCH_DTYPE(dtype, ...)                                       \
  switch (dtype) {                                                       \
    case ZEN_DTYPE_F32: { using T = float; __VA_ARGS__; } break;         \
    case ZEN_DTYPE_BF16: { using T = __nv_bfloat16; __VA_ARGS__; } break; \
    case ZEN_DTYPE_F16: { using T = __half; __VA_ARGS__; } break;        \
    default: return -1;                                                  \
  }

extern "C" {

int zen_sparse_ctx_size() { return (int)sizeof(ZenSparseCtx); }

// Advance a device-resident call counter by one (first launch of a call whose kernels read `epoch_dev`).
int zen_sparse_epoch_bump(uint32_t* epoch_dev, void* stream) {
  zen_sparse_epoch_bump_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(epoch_dev);
  return (int)cudaGetLastError();
}

// K1.  `thr` may be null (keep every nonzero) or point at a device float threshold on |g|.
int zen_partition_push(const ZenSparseCtx* c, const void* g, const float* thr, int dtype, int broadcast, void* stream) {
  int rc = 0;
  DISPATCH_DTYPE(dtype, rc = launch_partition<T>(*c, g, thr, broadcast, (cudaStream_t)stream));
  return rc;
}

// K2.  deterministic != 0: one launch per source, in rank order.
int zen_owner_reduce(const ZenSparseCtx* c, int dtype, int deterministic, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  const int grid = sm_count() * 4;
  if (deterministic) {
    for (int s = 0; s < c->nranks; ++s) {
      DISPATCH_DTYPE(dtype, zen_owner_reduce_kernel<T><<<grid, 256, 0, st>>>(*c, s, s + 1, 0));
    }
  } else {
    DISPATCH_DTYPE(dtype, zen_owner_reduce_kernel<T><<<grid, 256, 0, st>>>(*c, 0, c->nranks, 1));
  }
  return (int)cudaGetLastError();
}

// K3 (compact + push in one launch).
int zen_gather_push(const ZenSparseCtx* c, int dtype, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  // chunks per warp and step: as few as still let all steps run in one wave of CTAs (three per SM)
  const int wave = sm_count() * 3;
  int cpw = (int)((c->nchunks + (uint32_t)(K3_WARPS * wave) - 1) / (uint32_t)(K3_WARPS * wave));
  if (cpw < 1) cpw = 1;
  if (cpw > K3_CPW) cpw = K3_CPW;
  const int g3 = grid_for(c->nchunks, K3_WARPS * cpw, wave);
  DISPATCH_DTYPE(dtype, {
    const size_t smem = (size_t)K3_WARPS * 1032 * (4 + sizeof(T));
    ZEN_CUDA_CHECK_RET(cudaFuncSetAttribute(zen_gather_push_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    zen_gather_push_kernel<T><<<g3, K3_WARPS * 32, smem, st>>>(*c, cpw);
  });
  return (int)cudaGetLastError();
}

// K4 (bitmap walk with zero fill, then COO scatter for owners that chose COO).
int zen_densify(const ZenSparseCtx* c, void* out, int dtype, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  const uint64_t units = (uint64_t)c->nranks * c->nchunks;
  const int g1 = grid_for(units, 8, sm_count() * 8);
  DISPATCH_DTYPE(dtype, {
    const size_t smem = 8 * 1024 * sizeof(T);                        // one staging tile per warp
    ZEN_CUDA_CHECK_RET(cudaFuncSetAttribute(zen_densify_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    zen_densify_kernel<T><<<g1, 256, smem, st>>>(*c, (T*)out);
  });
  if (c->fmt_mode != ZEN_FMT_BITMAP) {
    DISPATCH_DTYPE(dtype, zen_densify_coo_kernel<T><<<sm_count() * 4, 256, 0, st>>>(*c, (T*)out));
  }
  return (int)cudaGetLastError();
}

// Method 1 consumer: zero `out`, then add every source in rank order.
int zen_scatter_sources(const ZenSparseCtx* c, void* out, int dtype, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  const size_t es = (dtype == ZEN_DTYPE_F32) ? 4 : 2;
  ZEN_CUDA_CHECK_RET(cudaMemsetAsync(out, 0, c->numel * es, st));
  for (int s = 0; s < c->nranks; ++s) {
    DISPATCH_DTYPE(dtype, zen_scatter_source_kernel<T><<<sm_count() * 4, 256, 0, st>>>(*c, (T*)out, s));
  }
  return (int)cudaGetLastError();
}

// One whole call from a single entry (one crossing from the host language instead of five): optional bump of the
// device call counter, partition + push, then scatter (method 1) or reduce + gather + densify (methods 2 / 3 / auto;
// `c->fmt_mode` carries the format).  `out` may be `x`: the scan of `x` ends before the first write.
int zen_sparse_allreduce(const ZenSparseCtx* c, const void* x, const float* thr, void* out, int dtype, int method1,
                         int deterministic, void* stream) {
  int rc = 0;
  if (c->epoch_dev && (rc = zen_sparse_epoch_bump(const_cast<uint32_t*>(c->epoch_dev), stream))) return rc;
  if ((rc = zen_partition_push(c, x, thr, dtype, method1 ? 1 : 0, stream))) return rc;
  if (method1) return zen_scatter_sources(c, out, dtype, stream);
  if ((rc = zen_owner_reduce(c, dtype, deterministic, stream))) return rc;
  if ((rc = zen_gather_push(c, dtype, stream))) return rc;
  return zen_densify(c, out, dtype, stream);
}

int zen_owner_map(int32_t* out, uint64_t n, const ZenPerm* perm, int mode, uint32_t table, int parts, void* stream) {
  ZenPerm p = *perm;
  zen_owner_map_kernel<<<grid_for(n, 256 * 8, sm_count() * 8), 256, 0, (cudaStream_t)stream>>>(out, n, p, mode, table, parts);
  return (int)cudaGetLastError();
}

int zen_sparse_balance(const void* in, uint64_t n, int dtype, int32_t* table, uint32_t table_size, int32_t* serial,
                       uint32_t serial_per_part, uint32_t* cursors, int parts, int rehash, uint32_t* status,
                       void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  const int grid = grid_for(n, 256 * 4, sm_count() * 8);
  DISPATCH_DTYPE(dtype, zen_sparse_balance_kernel<T><<<grid, 256, 0, st>>>((const T*)in, n, table, table_size, serial,
                                                                           serial_per_part, cursors, parts, rehash,
                                                                           status));
  return (int)cudaGetLastError();
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------
// Sampled top-k threshold (the sparsifier of train.py:56-73 without a sort and without leaving the device):
//   zen_sample_abs       |x| at `nsamples` pseudo-random positions (counter-based hash, with replacement)
//   zen_select_kth       k-th largest of the (gathered) samples by a three-pass radix select on the float bits
// The result is one device float that zen_partition_push consumes as its threshold.
__device__ __forceinline__ uint32_t zen_mix32(uint32_t x) {
  x ^= x >> 16; x *= 0x7feb352du; x ^= x >> 15; x *= 0x846ca68bu; x ^= x >> 16;
  return x;
}

template <typename T>
__global__ void __launch_bounds__(256)
zen_sample_abs_kernel(const T* __restrict__ x, uint64_t n, float* __restrict__ out, uint32_t nsamples, uint32_t seed) {
  for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < nsamples; i += gridDim.x * blockDim.x) {
    const uint64_t r = ((uint64_t)zen_mix32(i * 2u + seed) << 32) | zen_mix32(i * 2u + 1u + seed * 0x9e3779b9u);
    out[i] = fabsf(ZenVal<T>::to_f(x[r % n]));
  }
}

// Histogram of bits [shift, shift + nbits) of the samples whose higher bits equal `prefix` (prefix_bits of them).
__global__ void __launch_bounds__(256)
zen_select_hist_kernel(const float* __restrict__ v, uint32_t n, uint32_t* __restrict__ hist, const uint32_t* __restrict__ state,
                       int pass) {
  __shared__ uint32_t sh[2048];
  for (int i = threadIdx.x; i < 2048; i += blockDim.x) sh[i] = 0;
  __syncthreads();
  // state[0] = prefix found so far (high bits), state[1] = remaining rank k (1-based among the candidates)
  const uint32_t prefix = state[0];
  const int shift = pass == 0 ? 21 : (pass == 1 ? 10 : 0);
  const int nbits = pass == 2 ? 10 : 11;
  const int hi_shift = shift + nbits;                                  // bits above the current digit
  for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    const uint32_t b = __float_as_uint(v[i]) & 0x7fffffffu;
    if (pass == 0 || (b >> hi_shift) == prefix) atomicAdd(&sh[(b >> shift) & ((1u << nbits) - 1u)], 1u);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < 2048; i += blockDim.x)
    if (sh[i]) atomicAdd(&hist[i], sh[i]);
}

// One CTA: walk the histogram from the top bin down to the bin holding the k-th largest; update state; clear hist.
__global__ void __launch_bounds__(1024)
zen_select_pick_kernel(uint32_t* __restrict__ hist, uint32_t* __restrict__ state, float* __restrict__ out, int pass) {
  __shared__ uint32_t cnt[2048];
  const int nbins = pass == 2 ? 1024 : 2048;
  for (int i = threadIdx.x; i < 2048; i += blockDim.x) { cnt[i] = i < nbins ? hist[i] : 0u; hist[i] = 0u; }
  __syncthreads();
  if (threadIdx.x == 0) {
    uint32_t k = state[1], acc = 0;
    int bin = 0;
    for (int i = nbins - 1; i >= 0; --i) {
      if (acc + cnt[i] >= k) { bin = i; break; }
      acc += cnt[i];
    }
    const int nbits = pass == 2 ? 10 : 11;
    state[0] = (state[0] << nbits) | (uint32_t)bin;
    state[1] = k - acc;
    if (pass == 2) *out = __uint_as_float(state[0]);
  }
}

__global__ void zen_select_init_kernel(uint32_t* state, uint32_t k) { state[0] = 0u; state[1] = k; }

extern "C" {

int zen_sample_abs(const void* x, uint64_t n, float* out, uint32_t nsamples, uint32_t seed, int dtype, void* stream) {
  if (n == 0 || nsamples == 0) return -1;
  const int grid = grid_for(nsamples, 256, sm_count() * 4);
  DISPATCH_DTYPE(dtype, zen_sample_abs_kernel<T><<<grid, 256, 0, (cudaStream_t)stream>>>((const T*)x, n, out, nsamples, seed));
  return (int)cudaGetLastError();
}

// k-th largest (1-based) of v[0..n) (non-negative floats) -> *out.  hist: 2048 zeroed uint32 (left zeroed),
// state: 2 uint32 scratch.  Seven small launches, no host synchronisation.
int zen_select_kth(const float* v, uint32_t n, uint32_t k, uint32_t* hist, uint32_t* state, float* out, void* stream) {
  if (n == 0 || k == 0 || k > n) return -1;
  cudaStream_t st = (cudaStream_t)stream;
  zen_select_init_kernel<<<1, 1, 0, st>>>(state, k);
  const int grid = grid_for(n, 256 * 8, sm_count() * 2);
  for (int pass = 0; pass < 3; ++pass) {
    zen_select_hist_kernel<<<grid, 256, 0, st>>>(v, n, hist, state, pass);
    zen_select_pick_kernel<<<1, 1024, 0, st>>>(hist, state, out, pass);
  }
  return (int)cudaGetLastError();
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------
// Exchange of the threshold samples among the ranks of a tensor-parallel group (every shard of a replica must use one
// threshold: train.py:62-63 all-gathers the samples with NCCL).  Every rank stores its `ns` samples into slot `rank` of
// every peer's buffer with P2P stores, the last CTA publishes a flag per peer and then waits (bounded) for the flags of
// all peers: when the kernel ends, this rank's buffer holds the samples of the whole group.  Buffers and flags exist
// twice and alternate with the call parity, so a rank that is one call ahead writes where nobody reads.
struct ZenSampleXchg {
  int32_t rank;
  int32_t nranks;
  uint32_t epoch;
  uint32_t ns;                       // samples per rank
  uint64_t wait_ns;
  float* buf[ZEN_MAX_RANKS];         // per rank: float [2][nranks][ns]
  uint32_t* flags[ZEN_MAX_RANKS];    // per rank: uint32 [2][ZEN_MAX_RANKS]
  uint32_t* status;
  uint32_t* done;                    // CTA arrival counter (left at zero)
  const uint32_t* epoch_dev;         // optional device-resident call counter
};

__global__ void __launch_bounds__(256)
zen_sample_exchange_kernel(const ZenSampleXchg c, const float* __restrict__ mine) {
  __shared__ uint32_t s_last;
  const uint32_t epoch = c.epoch_dev ? *c.epoch_dev : c.epoch;
  const uint32_t par = epoch & 1u;
  const size_t slot = ((size_t)par * c.nranks + c.rank) * c.ns;
  for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < c.ns; i += gridDim.x * blockDim.x) {
    const float v = mine[i];
    for (int p = 0; p < c.nranks; ++p) c.buf[p][slot + i] = v;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    s_last = (atomicAdd(c.done, 1u) == gridDim.x - 1) ? 1u : 0u;
  }
  __syncthreads();
  if (s_last) {
    __threadfence_system();
    if ((int)threadIdx.x < c.nranks) {
      zen_st_release_sys(c.flags[threadIdx.x] + par * ZEN_MAX_RANKS + c.rank, epoch);
      if (!zen_wait_epoch(c.flags[c.rank] + par * ZEN_MAX_RANKS + threadIdx.x, epoch, c.wait_ns)) atomicOr(c.status, ZEN_TIMEOUT);
    }
    if (threadIdx.x == 0) *c.done = 0u;
  }
}

// The gathered samples of this call (the half of the buffer that its parity selects) copied to a fixed place, so that
// a captured consumer reads the same address at every replay.
__global__ void __launch_bounds__(256)
zen_sample_collect_kernel(const ZenSampleXchg c, float* __restrict__ out) {
  const uint32_t epoch = c.epoch_dev ? *c.epoch_dev : c.epoch;
  const size_t n = (size_t)c.nranks * c.ns;
  const float* src = c.buf[c.rank] + (size_t)(epoch & 1u) * n;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) out[i] = src[i];
}

extern "C" {

int zen_sample_xchg_size() { return (int)sizeof(ZenSampleXchg); }

// out: nranks * ns floats (slot r = rank r's samples), valid when the two kernels have run.
int zen_sample_exchange(const ZenSampleXchg* c, const float* mine, float* out, void* stream) {
  if (!c || c->nranks < 1 || c->nranks > ZEN_MAX_RANKS || c->ns == 0) return -1;
  const int grid = grid_for(c->ns, 256 * 8, 16);
  zen_sample_exchange_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(*c, mine);
  zen_sample_collect_kernel<<<grid_for((uint64_t)c->nranks * c->ns, 256 * 4, sm_count()), 256, 0, (cudaStream_t)stream>>>(*c, out);
  return (int)cudaGetLastError();
}

}  // extern "C"
