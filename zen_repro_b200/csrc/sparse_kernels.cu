// Sparse all-reduce kernels (element granule) for sm_100a.
//
// Pipeline per bucket, one launch each, all on one stream, no host sync:
//   zen_partition_push  : scan the flat bucket once, hash 64-element blocks to
//                         owners, stage (slot, value) records per owner in shared
//                         memory and push them in large contiguous runs straight
//                         into the owner's receive region over NVLink (P2P stores).
//   zen_owner_reduce    : bounded wait on each source's mailbox, red.add the
//                         records into this owner's fp32 slots, red.or the
//                         occupancy bitmap.
//   zen_gather_push     : count / scan the bitmap, compact the touched slots in
//                         slot order and push bitmap|COO + values to every peer.
//   zen_densify         : bounded wait on each owner's mailbox, one pass over
//                         the output that writes zeros and values together.
//
// Replaces, in the reference: the three sparse_balance kernels and the
// boolean-mask compaction after them (functions_cuda_kernel.cu:97-167,
// tensor_load_balance.py:24-51), both all_to_all calls and the scatter_add /
// nonzero between them (comm.py:117-127), encode_bitmap / decode_bitmap and the
// padded all_gathers (comm.py:59-99, 128-145).
#include "zen_common.cuh"

struct ZenSparseCtx {
  int32_t rank;
  int32_t nranks;
  uint32_t epoch;
  uint32_t fmt_mode;        // 0 auto, ZEN_FMT_COO, ZEN_FMT_BITMAP
  uint64_t wait_ns;
  char* sym[ZEN_MAX_RANKS]; // base of every rank's symmetric region
  uint64_t off_rec_mail;    // ZenMail[P], indexed by source
  uint64_t off_g_mail;      // ZenMail[P], indexed by owner
  uint64_t off_rec;         // uint2[P][cap_rec], indexed by source
  uint64_t off_g_idx;       // uint32[P][g_idx_words]: bitmap words or COO slots
  uint64_t off_g_off;       // uint32[P][nchunks + 1]: value offset of every 1024-slot chunk
  uint64_t off_g_val;       // T[P][cap_g] (stride in bytes: cap_g * 4)
  uint32_t cap_rec;
  uint32_t cap_g;
  uint32_t g_idx_words;
  uint32_t nchunks;
  float* acc;               // [S] local
  uint32_t* bitmap;         // [nwords] local
  uint32_t* chunk_off;      // [nchunks + 1] local: counts, then exclusive offsets
  uint32_t* cursors;        // [P] record cursors, [P] = done counter K1, [P+1] = done counter K3
  uint32_t* status;         // status word
  uint64_t numel;           // N
  uint32_t nslots;          // S = sb * G
  uint32_t nwords;          // ceil(S / 32)
  ZenPerm perm;
};

#define K1_THREADS 256
#define K1_WARPS 8
#define K1_U 4
#define K1_QCAP 1024
#define K1_FLUSH_MIN 256

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
  // select chains instead of dynamic indexing keep the vector in registers
  __device__ __forceinline__ uint32_t bits(int i) const {
    const uint32_t a = (i & 1) ? w[1] : w[0], b = (i & 1) ? w[3] : w[2], c = (i & 1) ? w[5] : w[4], d = (i & 1) ? w[7] : w[6];
    const uint32_t ab = (i & 2) ? b : a, cd = (i & 2) ? d : c;
    return (i & 4) ? cd : ab;
  }
  __device__ __forceinline__ float value(int i) const { return __uint_as_float(bits(i)); }
  __device__ __forceinline__ bool nonzero(int i) const { return (bits(i) & 0x7fffffffu) != 0u; }
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
};
template <> struct Raw8<__half> : Raw8Half<__half> {
  __device__ __forceinline__ float value(int i) const { return __half2float(__ushort_as_half((unsigned short)bits(i))); }
};

// ---------------------------------------------------------------------------------------------
// K1: partition + compact + push.  Every lane owns 8 consecutive elements (all in one 64-element
// block, hence one owner); a lane with nonzeros reserves room in its owner's shared-memory queue
// with one atomic and writes its records there.  Warp w drains queue w to the owner's receive
// region in runs of at least K1_FLUSH_MIN records.  kBroadcast = true is the method-1 variant: one
// queue of (global index, value) records pushed to every peer.
template <typename T, bool kBroadcast>
__global__ void __launch_bounds__(K1_THREADS, 2)
zen_partition_push_kernel(const ZenSparseCtx c, const T* __restrict__ g, const float* __restrict__ thr_ptr,
                          int aligned) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int nq = kBroadcast ? 1 : c.nranks;
  uint2* q = reinterpret_cast<uint2*>(smem_raw);                    // [nq][K1_QCAP]
  __shared__ uint32_t qn[ZEN_MAX_RANKS];
  __shared__ uint32_t qvalid[ZEN_MAX_RANKS];
  __shared__ uint32_t s_last;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const bool use_thr = thr_ptr != nullptr;
  const float thr = use_thr ? *thr_ptr : 0.f;
  const uint64_t N = c.numel;
  const uint64_t nwi = (N + 255) / 256;                               // warp-iterations of 256 elements
  const uint64_t ncta_it = (nwi + K1_WARPS * K1_U - 1) / (K1_WARPS * K1_U);
  uint32_t local_status = 0;

  if (tid < ZEN_MAX_RANKS) { qn[tid] = 0; qvalid[tid] = 0; }
  __syncthreads();

  constexpr int RAWW = sizeof(Raw8<T>) / 4;                           // words per staged vector (4 or 8)
  __shared__ uint32_t wbuf[K1_WARPS][64][RAWW + 1];                   // per-warp staging: {first element, raw vector}
  uint32_t wcnt = 0;                                                  // staged vectors of this warp (warp-uniform)

  // Records of one 8-element vector starting at element e32: choose the owner, reserve queue space, write them.
  auto emit = [&](uint32_t e32, const Raw8<T>& vec) {
    uint32_t m = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      bool keep = vec.nonzero(i);
      if (use_thr) keep = keep && (fabsf(vec.value(i)) >= thr);
      m |= keep ? (1u << i) : 0u;
    }
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
      if (k <= K1_QCAP) qvalid[owner] = k;                            // exactly one lane per overflow sees this
      direct = true;
      k = atomicAdd(&c.cursors[owner], cnt);                          // reserve directly in the destination
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
            reinterpret_cast<uint2*>(c.sym[p] + c.off_rec)[(uint64_t)c.rank * c.cap_rec + k] = rec;
        } else {
          reinterpret_cast<uint2*>(c.sym[owner] + c.off_rec)[(uint64_t)c.rank * c.cap_rec + k] = rec;
        }
      } else {
        local_status |= ZEN_REC_OVERFLOW;
      }
      ++k;
    }
  };

  for (uint64_t it = blockIdx.x; it < ncta_it; it += gridDim.x) {
    Raw8<T> v[K1_U];
#pragma unroll
    for (int u = 0; u < K1_U; ++u) {
      const uint64_t e0 = (it * (K1_WARPS * K1_U) + (uint64_t)u * K1_WARPS + warp) * 256 + (uint64_t)lane * 8;
      if (e0 < N) v[u].load(g, e0, N, aligned != 0); else v[u].zero();
    }
    const bool last_it = (it + gridDim.x >= ncta_it);
    // Vectors that hold a nonzero are first compacted into this warp's staging list (a ballot and one shared-memory
    // store), and the expensive part -- owner lookup, queue reservation, record writes -- runs on 32 staged vectors
    // at a time with every lane busy, instead of once per warp-load for the two or three lanes that have work.
#pragma unroll
    for (int u = 0; u < K1_U; ++u) {
      const bool has = v[u].any();
      const uint32_t bal = __ballot_sync(0xffffffffu, has);
      if (!bal) continue;
      if (has) {
        uint32_t* ent = wbuf[warp][wcnt + __popc(bal & ((1u << lane) - 1u))];
        ent[0] = (uint32_t)((it * (K1_WARPS * K1_U) + (uint64_t)u * K1_WARPS + warp) * 256) + lane * 8;
#pragma unroll
        for (int k = 0; k < RAWW; ++k) ent[1 + k] = v[u].w[k];
      }
      wcnt += __popc(bal);
      if (wcnt >= 32) {
        __syncwarp();
        {
          Raw8<T> r;
          const uint32_t* ent = wbuf[warp][lane];
#pragma unroll
          for (int k = 0; k < RAWW; ++k) r.w[k] = ent[1 + k];
          emit(ent[0], r);
        }
        const uint32_t rest = wcnt - 32;
        uint32_t tmp[RAWW + 1];
        if (lane < rest) {
#pragma unroll
          for (int k = 0; k <= RAWW; ++k) tmp[k] = wbuf[warp][32 + lane][k];
        }
        __syncwarp();
        if (lane < rest) {
#pragma unroll
          for (int k = 0; k <= RAWW; ++k) wbuf[warp][lane][k] = tmp[k];
        }
        __syncwarp();
        wcnt = rest;
      }
    }
    if (last_it && wcnt) {                               // leftovers of this warp: drain with the lanes that have one
      __syncwarp();
      if (lane < wcnt) {
        Raw8<T> r;
        const uint32_t* ent = wbuf[warp][lane];
#pragma unroll
        for (int k = 0; k < RAWW; ++k) r.w[k] = ent[1 + k];
        emit(ent[0], r);
      }
      wcnt = 0;
    }
    __syncthreads();
    // flush phase: warp w drains queue w when it holds a worthwhile run (or on the last iteration)
    if (warp < nq) {
      uint32_t n = qn[warp];
      const bool overflowed = n > K1_QCAP;
      if (overflowed) n = qvalid[warp];
      if (n > 0 && (n >= K1_FLUSH_MIN || last_it || overflowed)) {
        uint32_t gbase = 0;
        if (lane == 0) gbase = atomicAdd(&c.cursors[warp], n);
        gbase = __shfl_sync(0xffffffffu, gbase, 0);
        const uint32_t fit = (gbase >= c.cap_rec) ? 0u : min(n, c.cap_rec - gbase);
        if (fit < n) local_status |= ZEN_REC_OVERFLOW;
        const uint2* src = q + warp * K1_QCAP;
        if (kBroadcast) {
          for (int p = 0; p < c.nranks; ++p) {
            uint2* dst = reinterpret_cast<uint2*>(c.sym[p] + c.off_rec) + (uint64_t)c.rank * c.cap_rec + gbase;
            for (uint32_t i = lane; i < fit; i += 32) dst[i] = src[i];
          }
        } else {
          uint2* dst = reinterpret_cast<uint2*>(c.sym[warp] + c.off_rec) + (uint64_t)c.rank * c.cap_rec + gbase;
          for (uint32_t i = lane; i < fit; i += 32) dst[i] = src[i];
        }
        __syncwarp();
        if (lane == 0) { qn[warp] = 0; qvalid[warp] = 0; }
      } else if (overflowed && lane == 0) {
        qn[warp] = 0; qvalid[warp] = 0;
      }
    }
    __syncthreads();
  }

  if (local_status) atomicOr(c.status, local_status);
  // completion: the last CTA to arrive publishes counts and epochs to the consumers
  __threadfence_system();
  __syncthreads();
  if (tid == 0) {
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
      ZenMail* mail = reinterpret_cast<ZenMail*>(c.sym[p] + c.off_rec_mail) + c.rank;
      mail->count = min(raw, c.cap_rec);
      mail->info = ((raw > c.cap_rec) || (st & ZEN_REC_OVERFLOW)) ? 1u : 0u;
      mail->aux = 0;
      __threadfence_system();
      zen_st_release_sys(&mail->epoch, c.epoch);
    }
    __syncthreads();
    if (tid < ZEN_MAX_RANKS + 1) c.cursors[tid] = 0;                  // ready for the next call
  }
}

// ---------------------------------------------------------------------------------------------
// K2: owner-side reduce of sources [src_begin, src_end).  One launch over all sources is the fast
// mode; one launch per source gives a fixed accumulation order.
template <typename T>
__global__ void __launch_bounds__(256)
zen_owner_reduce_kernel(const ZenSparseCtx c, int src_begin, int src_end) {
  __shared__ uint32_t s_ok;
  uint32_t local_status = 0;
  for (int s = src_begin; s < src_end; ++s) {
    const ZenMail* mail = reinterpret_cast<const ZenMail*>(c.sym[c.rank] + c.off_rec_mail) + s;
    if (threadIdx.x == 0) s_ok = zen_wait_epoch(&mail->epoch, c.epoch, c.wait_ns) ? 1u : 0u;
    __syncthreads();
    const bool ok = s_ok != 0;
    __syncthreads();
    if (!ok) { local_status |= ZEN_TIMEOUT; continue; }
    const uint32_t n = min(zen_ld_acquire_sys(&mail->count), c.cap_rec);
    if (zen_ld_acquire_sys(&mail->info) & 1u) local_status |= ZEN_PEER_OVERFLOW;
    const uint2* rec = reinterpret_cast<const uint2*>(c.sym[c.rank] + c.off_rec) + (uint64_t)s * c.cap_rec;
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
      const uint2 r = rec[i];
      if (r.x < c.nslots) {
        atomicAdd(&c.acc[r.x], ZenVal<T>::unbits(r.y));
        atomicOr(&c.bitmap[r.x >> 5], 1u << (r.x & 31));
      } else {
        local_status |= ZEN_BAD_ARG;
      }
    }
  }
  if (local_status) atomicOr(c.status, local_status);
}

// ---------------------------------------------------------------------------------------------
// K3a: touched slots per 1024-slot chunk.
__global__ void __launch_bounds__(256) zen_chunk_count_kernel(const ZenSparseCtx c) {
  const int lane = threadIdx.x & 31;
  const uint32_t gw = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const uint32_t nw = (gridDim.x * blockDim.x) >> 5;
  for (uint32_t ch = gw; ch < c.nchunks; ch += nw) {
    const uint32_t wi = ch * 32 + lane;
    uint32_t n = (wi < c.nwords) ? __popc(c.bitmap[wi]) : 0u;
#pragma unroll
    for (int d = 16; d; d >>= 1) n += __shfl_xor_sync(0xffffffffu, n, d);
    if (lane == 0) c.chunk_off[ch] = n;
  }
}

// K3b: exclusive scan of the chunk counts in place; total at [nchunks].  One CTA.
__global__ void __launch_bounds__(1024) zen_chunk_scan_kernel(const ZenSparseCtx c) {
  __shared__ uint32_t part[1024];
  const uint32_t n = c.nchunks;
  const uint32_t per = (n + 1023) / 1024;
  const uint32_t b = threadIdx.x * per, e = min(n, b + per);
  uint32_t s = 0;
  for (uint32_t i = b; i < e; ++i) s += c.chunk_off[i];
  part[threadIdx.x] = s;
  __syncthreads();
  for (int d = 1; d < 1024; d <<= 1) {
    uint32_t t = (threadIdx.x >= (unsigned)d) ? part[threadIdx.x - d] : 0u;
    __syncthreads();
    part[threadIdx.x] += t;
    __syncthreads();
  }
  uint32_t run = part[threadIdx.x] - s;
  for (uint32_t i = b; i < e; ++i) {
    const uint32_t t = c.chunk_off[i];
    c.chunk_off[i] = run;
    run += t;
  }
  if (threadIdx.x == 1023) c.chunk_off[n] = part[1023];
}

// K3c: compact the touched slots of 8 consecutive chunks per CTA into shared memory, then push the
// contiguous run (values, and COO slots or bitmap words + chunk offsets) to every peer.
#define K3_WARPS 8
template <typename T>
__global__ void __launch_bounds__(K3_WARPS * 32)
zen_gather_push_kernel(const ZenSparseCtx c) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  uint32_t* s_idx = reinterpret_cast<uint32_t*>(smem_raw);                       // [K3_WARPS * 1024 + 16]
  T* s_val = reinterpret_cast<T*>(smem_raw + (K3_WARPS * 1024 + 16) * 4);        // [K3_WARPS * 1024 + 16]
  __shared__ uint32_t s_last;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint32_t total = c.chunk_off[c.nchunks];
  const bool overflow = total > c.cap_g;
  uint32_t fmt = c.fmt_mode;
  if (fmt == 0) fmt = ((uint64_t)total * 32ull > (uint64_t)c.nslots) ? ZEN_FMT_BITMAP : ZEN_FMT_COO;
  if (fmt == ZEN_FMT_COO && total > c.g_idx_words) fmt = ZEN_FMT_BITMAP;   // COO list would not fit
  const uint32_t ngroups = (c.nchunks + K3_WARPS - 1) / K3_WARPS;
  constexpr uint32_t VPV = 16 / sizeof(T);                               // values per 16-byte vector

  for (uint32_t grp = blockIdx.x; grp < ngroups; grp += gridDim.x) {
    const uint32_t ch0 = grp * K3_WARPS;
    const uint32_t ch = ch0 + warp;
    const uint32_t gbase = c.chunk_off[ch0];                             // first value of this CTA's run
    const uint32_t gend = c.chunk_off[min(ch0 + K3_WARPS, c.nchunks)];
    const uint32_t mis_v = gbase % VPV, mis_i = gbase % 4;
    uint32_t word = 0, coff = 0;
    if (ch < c.nchunks) {
      const uint32_t wi = ch * 32 + lane;
      word = (wi < c.nwords) ? c.bitmap[wi] : 0u;
      coff = c.chunk_off[ch];
      if (wi < c.nwords && word) c.bitmap[wi] = 0;                       // leave the bitmap clean for the next call
    }
    uint32_t incl = __popc(word);
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      uint32_t t = __shfl_up_sync(0xffffffffu, incl, d);
      if (lane >= d) incl += t;
    }
    const uint32_t woff = incl - __popc(word);
    {
      // Stream the accumulator: a lane whose bitmap word is non-empty loads its 32 slots as eight independent
      // 16-byte vectors, clears them, and appends the touched ones (in slot order) to the CTA's staging run.
      uint32_t r = (coff - gbase) + woff;
      if (word) {
        float f[32];
        float4* ap = reinterpret_cast<float4*>(c.acc + (size_t)ch * 1024 + (size_t)lane * 32);
#pragma unroll
        for (int k = 0; k < 8; ++k) *reinterpret_cast<float4*>(&f[4 * k]) = ap[k];
#pragma unroll
        for (int k = 0; k < 8; ++k) ap[k] = make_float4(0.f, 0.f, 0.f, 0.f);
        const uint32_t slot0 = ch * 1024 + lane * 32;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          if ((word >> i) & 1u) {
            s_val[mis_v + r] = ZenVal<T>::from_f(f[i]);
            if (fmt == ZEN_FMT_COO) s_idx[mis_i + r] = slot0 + i;
            ++r;
          }
        }
      }
    }
    __syncthreads();
    if (!overflow) {
      const uint32_t n = gend - gbase;
      for (int p = 0; p < c.nranks; ++p) {
        char* base = c.sym[p];
        // values: scalar head up to a 16-byte boundary, vector body, scalar tail
        T* dv = reinterpret_cast<T*>(base + c.off_g_val + (uint64_t)c.rank * c.cap_g * 4ull) + gbase;
        const uint32_t head = min(n, (VPV - mis_v) % VPV);
        for (uint32_t i = tid; i < head; i += blockDim.x) dv[i] = s_val[mis_v + i];
        const uint32_t nvec = (n - head) / VPV;
        {
          uint4* d4 = reinterpret_cast<uint4*>(dv + head);
          const uint4* s4 = reinterpret_cast<const uint4*>(s_val + mis_v + head);
          for (uint32_t i = tid; i < nvec; i += blockDim.x) d4[i] = s4[i];
        }
        for (uint32_t i = head + nvec * VPV + tid; i < n; i += blockDim.x) dv[i] = s_val[mis_v + i];
        if (fmt == ZEN_FMT_COO) {
          uint32_t* di = reinterpret_cast<uint32_t*>(base + c.off_g_idx) + (uint64_t)c.rank * c.g_idx_words + gbase;
          const uint32_t hi = min(n, (4u - mis_i) % 4u);
          for (uint32_t i = tid; i < hi; i += blockDim.x) di[i] = s_idx[mis_i + i];
          const uint32_t nv = (n - hi) / 4;
          uint4* d4 = reinterpret_cast<uint4*>(di + hi);
          const uint4* s4 = reinterpret_cast<const uint4*>(s_idx + mis_i + hi);
          for (uint32_t i = tid; i < nv; i += blockDim.x) d4[i] = s4[i];
          for (uint32_t i = hi + nv * 4 + tid; i < n; i += blockDim.x) di[i] = s_idx[mis_i + i];
        } else if (ch < c.nchunks) {
          uint32_t* db = reinterpret_cast<uint32_t*>(base + c.off_g_idx) + (uint64_t)c.rank * c.g_idx_words;
          const uint32_t wi = ch * 32 + lane;
          if (wi < c.nwords) db[wi] = word;
          if (lane == 0)
            reinterpret_cast<uint32_t*>(base + c.off_g_off)[(uint64_t)c.rank * (c.nchunks + 1) + ch] = coff;
        }
      }
    }
    __syncthreads();
  }

  __threadfence_system();
  __syncthreads();
  if (tid == 0) {
    const uint32_t prev = atomicAdd(&c.cursors[ZEN_MAX_RANKS + 1], 1u);
    s_last = (prev == gridDim.x - 1) ? 1u : 0u;
  }
  __syncthreads();
  if (s_last) {
    __threadfence_system();
    if (overflow && tid == 0) atomicOr(c.status, ZEN_GATHER_OVERFLOW);
    if (tid < c.nranks) {
      const uint32_t st = atomicOr(c.status, 0u);
      ZenMail* mail = reinterpret_cast<ZenMail*>(c.sym[tid] + c.off_g_mail) + c.rank;
      mail->count = overflow ? 0u : total;
      mail->info = ((overflow || (st & (ZEN_REC_OVERFLOW | ZEN_PEER_OVERFLOW | ZEN_TIMEOUT))) ? 1u : 0u) | (fmt << 8);
      mail->aux = 0;
      __threadfence_system();
      zen_st_release_sys(&mail->epoch, c.epoch);
    }
    if (tid == 0) c.cursors[ZEN_MAX_RANKS + 1] = 0;
  }
}

// ---------------------------------------------------------------------------------------------
// K4: densify.  Walks every owner's slot space chunk by chunk; every output element is written once
// (zeros included), so the output needs no memset.  Owners that chose COO get their blocks
// zero-filled here and their values scattered by zen_densify_coo_kernel afterwards.
template <typename T>
__global__ void __launch_bounds__(256)
zen_densify_kernel(const ZenSparseCtx c, T* __restrict__ out) {
  __shared__ uint32_t s_fmt[ZEN_MAX_RANKS];
  const int tid = threadIdx.x, lane = tid & 31;
  uint32_t local_status = 0;
  if (tid < c.nranks) {
    const ZenMail* mail = reinterpret_cast<const ZenMail*>(c.sym[c.rank] + c.off_g_mail) + tid;
    uint32_t f = 0;
    if (zen_wait_epoch(&mail->epoch, c.epoch, c.wait_ns)) {
      f = (mail->info >> 8) & 0xffu;
      if (mail->info & 1u) { local_status |= ZEN_PEER_OVERFLOW; f = 0; }
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
  const uint64_t nunits = (uint64_t)c.nranks * c.nchunks;
  for (uint64_t unit = gw; unit < nunits; unit += nw) {
    const uint32_t o = (uint32_t)(unit / c.nchunks), ch = (uint32_t)(unit % c.nchunks);
    const bool bm = s_fmt[o] == ZEN_FMT_BITMAP;
    const char* base = c.sym[c.rank];
    const uint32_t* gbm = reinterpret_cast<const uint32_t*>(base + c.off_g_idx) + (uint64_t)o * c.g_idx_words;
    const T* gval = reinterpret_cast<const T*>(base + c.off_g_val + (uint64_t)o * c.cap_g * 4ull);
    const uint32_t wi = ch * 32 + lane;
    uint32_t word = (bm && wi < c.nwords) ? gbm[wi] : 0u;
    uint32_t incl = __popc(word);
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      uint32_t t = __shfl_up_sync(0xffffffffu, incl, d);
      if (lane >= d) incl += t;
    }
    const uint32_t coff = bm ? reinterpret_cast<const uint32_t*>(base + c.off_g_off)[(uint64_t)o * (c.nchunks + 1) + ch] : 0u;
    const uint32_t woff = coff + incl - __popc(word);
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
      T v[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        v[i] = ZenVal<T>::from_f(0.f);
        if ((byte >> i) & 1u) v[i] = gval[off0 + __popc(byte & ((1u << i) - 1u))];
      }
      if (e + 8 <= N) {
        if (sizeof(T) == 2) {
          uint4 pk;
          pk.x = ZenVal<T>::bits(v[0]) | (ZenVal<T>::bits(v[1]) << 16);
          pk.y = ZenVal<T>::bits(v[2]) | (ZenVal<T>::bits(v[3]) << 16);
          pk.z = ZenVal<T>::bits(v[4]) | (ZenVal<T>::bits(v[5]) << 16);
          pk.w = ZenVal<T>::bits(v[6]) | (ZenVal<T>::bits(v[7]) << 16);
          *reinterpret_cast<uint4*>(out + e) = pk;
        } else {
          uint4 lo, hi;
          lo.x = ZenVal<T>::bits(v[0]); lo.y = ZenVal<T>::bits(v[1]); lo.z = ZenVal<T>::bits(v[2]); lo.w = ZenVal<T>::bits(v[3]);
          hi.x = ZenVal<T>::bits(v[4]); hi.y = ZenVal<T>::bits(v[5]); hi.z = ZenVal<T>::bits(v[6]); hi.w = ZenVal<T>::bits(v[7]);
          reinterpret_cast<uint4*>(out + e)[0] = lo;
          reinterpret_cast<uint4*>(out + e)[1] = hi;
        }
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i)
          if (e + i < N) out[e + i] = v[i];
      }
    }
  }
  if (local_status) atomicOr(c.status, local_status);
}

template <typename T>
__global__ void __launch_bounds__(256)
zen_densify_coo_kernel(const ZenSparseCtx c, T* __restrict__ out) {
  __shared__ uint32_t s_n[ZEN_MAX_RANKS];
  const uint32_t G = c.perm.block;
  if (threadIdx.x < c.nranks) {
    const ZenMail* mail = reinterpret_cast<const ZenMail*>(c.sym[c.rank] + c.off_g_mail) + threadIdx.x;
    uint32_t n = 0;
    // the bitmap pass of this call already waited for this epoch
    if (zen_ld_acquire_sys(&mail->epoch) == c.epoch) {
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
      if (slot >= c.nslots) continue;
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
  const ZenMail* mail = reinterpret_cast<const ZenMail*>(c.sym[c.rank] + c.off_rec_mail) + src;
  if (threadIdx.x == 0) s_ok = zen_wait_epoch(&mail->epoch, c.epoch, c.wait_ns) ? 1u : 0u;
  __syncthreads();
  if (!s_ok) { if (threadIdx.x == 0) atomicOr(c.status, ZEN_TIMEOUT); return; }
  if ((mail->info & 1u) && threadIdx.x == 0) atomicOr(c.status, ZEN_PEER_OVERFLOW);
  const uint32_t n = min(mail->count, c.cap_rec);
  const uint2* rec = reinterpret_cast<const uint2*>(c.sym[c.rank] + c.off_rec) + (uint64_t)src * c.cap_rec;
  for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    const uint2 r = rec[i];
    if (r.x < c.numel) out[r.x] = ZenVal<T>::from_f(ZenVal<T>::to_f(out[r.x]) + ZenVal<T>::unbits(r.y));
  }
}

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

template <typename T>
static int launch_partition(const ZenSparseCtx& c, const void* g, const float* thr, int broadcast, cudaStream_t st) {
  const uint64_t nwi = (c.numel + 255) / 256;
  const uint64_t nit = (nwi + K1_WARPS * K1_U - 1) / (K1_WARPS * K1_U);
  const int grid = grid_for(nit, 1, sm_count() * 3);
  const int nq = broadcast ? 1 : c.nranks;
  const size_t smem = (size_t)nq * K1_QCAP * sizeof(uint2);
  const int aligned = (reinterpret_cast<uintptr_t>(g) % 16 == 0) ? 1 : 0;
  if (broadcast) {
    ZEN_CUDA_CHECK_RET(cudaFuncSetAttribute(zen_partition_push_kernel<T, true>,
                                            cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    zen_partition_push_kernel<T, true><<<grid, K1_THREADS, smem, st>>>(c, (const T*)g, thr, aligned);
  } else {
    ZEN_CUDA_CHECK_RET(cudaFuncSetAttribute(zen_partition_push_kernel<T, false>,
                                            cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    zen_partition_push_kernel<T, false><<<grid, K1_THREADS, smem, st>>>(c, (const T*)g, thr, aligned);
  }
  return (int)cudaGetLastError();
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
      DISPATCH_DTYPE(dtype, zen_owner_reduce_kernel<T><<<grid, 256, 0, st>>>(*c, s, s + 1));
    }
  } else {
    DISPATCH_DTYPE(dtype, zen_owner_reduce_kernel<T><<<grid, 256, 0, st>>>(*c, 0, c->nranks));
  }
  return (int)cudaGetLastError();
}

// K3 (count, scan, compact + push).
int zen_gather_push(const ZenSparseCtx* c, int dtype, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  const int g1 = grid_for(c->nchunks, 8, sm_count() * 8);
  zen_chunk_count_kernel<<<g1, 256, 0, st>>>(*c);
  zen_chunk_scan_kernel<<<1, 1024, 0, st>>>(*c);
  const int g3 = grid_for(c->nchunks, K3_WARPS, sm_count() * 3);
  DISPATCH_DTYPE(dtype, {
    const size_t smem = (K3_WARPS * 1024 + 16) * (4 + sizeof(T));
    ZEN_CUDA_CHECK_RET(cudaFuncSetAttribute(zen_gather_push_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    zen_gather_push_kernel<T><<<g3, K3_WARPS * 32, smem, st>>>(*c);
  });
  return (int)cudaGetLastError();
}

// K4 (bitmap walk with zero fill, then COO scatter for owners that chose COO).
int zen_densify(const ZenSparseCtx* c, void* out, int dtype, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  const uint64_t units = (uint64_t)c->nranks * c->nchunks;
  const int g1 = grid_for(units, 8, sm_count() * 8);
  DISPATCH_DTYPE(dtype, zen_densify_kernel<T><<<g1, 256, 0, st>>>(*c, (T*)out));
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
