// Row-granule sparse all-reduce for embedding gradients (sm_100a).
//
// Input on every rank: `count` unique row ids and their d-wide gradient rows, as produced by the
// row-sparse embedding backward.  Rows are hashed to owners with the same invertible permutation
// as the element path (block = 1 row), pushed with 16-byte P2P stores into the owner's receive
// slots, reduced there in fp32, and the reduced rows are pushed to every rank, which adds them
// into its dense gradient.  Traffic and work are O(touched rows * d); the dense [V, d] gradient is
// never scanned.  The reference has no row mode: it top-k sparsifies whole DDP buckets
// (train.py:167-183).
#include "zen_common.cuh"

struct ZenRowCtx {
  int32_t rank;
  int32_t nranks;
  uint32_t epoch;
  uint32_t d;                // row width in elements (multiple of 8)
  uint64_t wait_ns;
  char* sym[ZEN_MAX_RANKS];
  uint64_t off_rec_mail;     // ZenMail[P] by source
  uint64_t off_g_mail;       // ZenMail[P] by owner
  uint64_t off_rec_slot;     // uint32[P][cap_rec]
  uint64_t off_rec_val;      // T[P][cap_rec][d]
  uint64_t off_g_row;        // uint32[P][cap_g]   global row ids
  uint64_t off_g_val;        // T[P][cap_g][d]
  uint32_t cap_rec;
  uint32_t cap_g;
  uint32_t nslots;           // rows owned per rank (sb)
  uint32_t nwords;
  float* acc;                // [nslots][d]
  uint32_t* bitmap;          // [nwords]
  uint32_t* list;            // [nslots] compacted touched slots
  uint32_t* cursors;         // [P] + done counters + list count
  uint32_t* status;
  uint32_t vocab;
  uint32_t pad;
  const uint32_t* epoch_dev;  // optional: call counter on the device (bumped by zen_row_epoch_bump); overrides `epoch`
  ZenPerm perm;
};

__device__ __forceinline__ uint32_t row_epoch(const ZenRowCtx& c) { return c.epoch_dev ? *c.epoch_dev : c.epoch; }

namespace {

template <typename T> __device__ __forceinline__ void ld8(const T* p, float (&v)[8]);
template <> __device__ __forceinline__ void ld8<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 r = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) { v[2 * i] = __uint_as_float(w[i] << 16); v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u); }
}
template <> __device__ __forceinline__ void ld8<float>(const float* p, float (&v)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
template <> __device__ __forceinline__ void ld8<__half>(const __half* p, float (&v)[8]) {
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = __half2float(p[i]);
}
template <typename T> __device__ __forceinline__ void st8(T* p, const float (&v)[8]);
template <> __device__ __forceinline__ void st8<__nv_bfloat16>(__nv_bfloat16* p, const float (&v)[8]) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) { __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]); w[i] = *reinterpret_cast<uint32_t*>(&h); }
  *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
}
template <> __device__ __forceinline__ void st8<float>(float* p, const float (&v)[8]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
template <> __device__ __forceinline__ void st8<__half>(__half* p, const float (&v)[8]) {
#pragma unroll
  for (int i = 0; i < 8; ++i) p[i] = __float2half_rn(v[i]);
}

// Publish mails from the last CTA to finish.  which = 0: record mails (count per destination from
// cursors[p]); which = 1: gather mails (same count to everyone).
__device__ __forceinline__ void publish(const ZenRowCtx& c, int which, uint32_t same_count, uint32_t overflow) {
  __shared__ uint32_t s_last;
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint32_t prev = atomicAdd(&c.cursors[ZEN_MAX_RANKS + which], 1u);
    s_last = (prev == gridDim.x - 1) ? 1u : 0u;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence_system();
  if ((int)threadIdx.x < c.nranks) {
    const int p = threadIdx.x;
    const uint32_t st = atomicOr(c.status, 0u);
    ZenMail* mail = reinterpret_cast<ZenMail*>(c.sym[p] + (which ? c.off_g_mail : c.off_rec_mail)) + c.rank;
    uint32_t cnt = same_count, ovf = overflow;
    if (!which) {
      const uint32_t raw = atomicAdd(&c.cursors[p], 0u);
      cnt = min(raw, c.cap_rec);
      ovf = raw > c.cap_rec;
    }
    mail->count = cnt;
    mail->info = (ovf || (st & (ZEN_REC_OVERFLOW | ZEN_PEER_OVERFLOW | ZEN_GATHER_OVERFLOW | ZEN_TIMEOUT))) ? 1u : 0u;
    mail->aux = 0;
    __threadfence_system();
    zen_st_release_sys(&mail->epoch, row_epoch(c));
  }
  __syncthreads();
  if (!which) { if (threadIdx.x < ZEN_MAX_RANKS) c.cursors[threadIdx.x] = 0; }
  if (threadIdx.x == 0) c.cursors[ZEN_MAX_RANKS + which] = 0;
}

// R1: one warp per input row: pick the owner, reserve a record, copy the row into the owner's memory.
template <typename T>
__global__ void __launch_bounds__(256)
row_push_kernel(const ZenRowCtx c, const int32_t* __restrict__ rows, const int32_t* __restrict__ count,
                const T* __restrict__ vals, int max_rows) {
  const int lane = threadIdx.x & 31;
  const int gw = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, nw = (gridDim.x * blockDim.x) >> 5;
  const int n = min(*count, max_rows);
  uint32_t local_status = 0;
  for (int u = gw; u < n; u += nw) {
    const uint32_t row = (uint32_t)rows[u];
    if (row >= c.vocab) { local_status |= ZEN_BAD_ARG; continue; }
    const uint32_t pb = zen_perm_fwd(c.perm, row);
    const uint32_t owner = zen_owner_of(c.perm, pb, c.nranks);
    const uint32_t slot = pb - owner * c.perm.sb;
    uint32_t pos = 0;
    if (lane == 0) pos = atomicAdd(&c.cursors[owner], 1u);
    pos = __shfl_sync(0xffffffffu, pos, 0);
    if (pos >= c.cap_rec) { local_status |= ZEN_REC_OVERFLOW; continue; }
    char* base = c.sym[owner];
    if (lane == 0) reinterpret_cast<uint32_t*>(base + c.off_rec_slot)[(uint64_t)c.rank * c.cap_rec + pos] = slot;
    uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<T*>(base + c.off_rec_val) + ((uint64_t)c.rank * c.cap_rec + pos) * c.d);
    const uint4* src = reinterpret_cast<const uint4*>(vals + (uint64_t)u * c.d);
    const int nv = c.d * sizeof(T) / 16;
    for (int i = lane; i < nv; i += 32) dst[i] = src[i];
  }
  if (local_status) atomicOr(c.status, local_status);
  publish(c, 0, 0, 0);
}

// R2: add the records of sources [src_begin, src_end) into the fp32 row accumulator.
template <typename T>
__global__ void __launch_bounds__(256)
row_reduce_kernel(const ZenRowCtx c, int src_begin, int src_end) {
  __shared__ uint32_t s_ok;
  const int lane = threadIdx.x & 31;
  const int gw = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, nw = (gridDim.x * blockDim.x) >> 5;
  uint32_t local_status = 0;
  for (int s = src_begin; s < src_end; ++s) {
    const ZenMail* mail = reinterpret_cast<const ZenMail*>(c.sym[c.rank] + c.off_rec_mail) + s;
    if (threadIdx.x == 0) s_ok = zen_wait_epoch(&mail->epoch, row_epoch(c), c.wait_ns) ? 1u : 0u;
    __syncthreads();
    const bool ok = s_ok != 0;
    __syncthreads();
    if (!ok) { local_status |= ZEN_TIMEOUT; continue; }
    const uint32_t n = min(zen_ld_acquire_sys(&mail->count), c.cap_rec);
    if (zen_ld_acquire_sys(&mail->info) & 1u) local_status |= ZEN_PEER_OVERFLOW;
    const char* base = c.sym[c.rank];
    const uint32_t* rslot = reinterpret_cast<const uint32_t*>(base + c.off_rec_slot) + (uint64_t)s * c.cap_rec;
    const T* rval = reinterpret_cast<const T*>(base + c.off_rec_val) + (uint64_t)s * c.cap_rec * c.d;
    for (uint32_t i = gw; i < n; i += nw) {
      const uint32_t slot = rslot[i];
      if (slot >= c.nslots) { local_status |= ZEN_BAD_ARG; continue; }
      if (lane == 0) atomicOr(&c.bitmap[slot >> 5], 1u << (slot & 31));
      float* a = c.acc + (uint64_t)slot * c.d;
      const T* v = rval + (uint64_t)i * c.d;
      for (uint32_t col = lane * 8; col < c.d; col += 256) {
        float x[8];
        ld8<T>(v + col, x);
        atomicAdd(reinterpret_cast<float4*>(a + col), make_float4(x[0], x[1], x[2], x[3]));
        atomicAdd(reinterpret_cast<float4*>(a + col + 4), make_float4(x[4], x[5], x[6], x[7]));
      }
    }
  }
  if (local_status) atomicOr(c.status, local_status);
}

// R3a: one CTA lists the touched slots in ascending order (nslots is at most a few hundred thousand).
__global__ void __launch_bounds__(1024) row_list_kernel(const ZenRowCtx c) {
  __shared__ uint32_t part[1024];
  const uint32_t per = (c.nwords + 1023) / 1024;
  const uint32_t b = threadIdx.x * per, e = min(c.nwords, b + per);
  uint32_t s = 0;
  for (uint32_t i = b; i < e; ++i) s += __popc(c.bitmap[i]);
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
    uint32_t w = c.bitmap[i];
    if (w) c.bitmap[i] = 0;
    while (w) {
      c.list[run++] = i * 32 + (uint32_t)(__ffs(w) - 1);
      w &= w - 1;
    }
  }
  if (threadIdx.x == 1023) c.cursors[ZEN_MAX_RANKS + 2] = part[1023];
}

// R3b: one warp per touched slot: convert, push (global row id, row) to every rank, clear the accumulator.
template <typename T>
__global__ void __launch_bounds__(256)
row_gather_push_kernel(const ZenRowCtx c) {
  const int lane = threadIdx.x & 31;
  const int gw = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, nw = (gridDim.x * blockDim.x) >> 5;
  const uint32_t total = c.cursors[ZEN_MAX_RANKS + 2];
  const bool overflow = total > c.cap_g;
  for (uint32_t k = gw; k < total; k += nw) {
    const uint32_t slot = c.list[k];
    const uint32_t row = zen_perm_inv(c.perm, c.rank * c.perm.sb + slot);
    float* a = c.acc + (uint64_t)slot * c.d;
    for (uint32_t col = lane * 8; col < c.d; col += 256) {
      float x[8];
      ld8<float>(a + col, x);
      const float z[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      st8<float>(a + col, z);
      if (!overflow) {
        for (int p = 0; p < c.nranks; ++p)
          st8<T>(reinterpret_cast<T*>(c.sym[p] + c.off_g_val) + ((uint64_t)c.rank * c.cap_g + k) * c.d + col, x);
      }
    }
    if (lane == 0 && !overflow) {
      for (int p = 0; p < c.nranks; ++p)
        reinterpret_cast<uint32_t*>(c.sym[p] + c.off_g_row)[(uint64_t)c.rank * c.cap_g + k] = row;
    }
  }
  if (overflow && blockIdx.x == 0 && threadIdx.x == 0) atomicOr(c.status, ZEN_GATHER_OVERFLOW);
  publish(c, 1, overflow ? 0u : total, overflow ? 1u : 0u);
}

// R4: grad[row] += reduced row, for every owner's payload.  Rows are unique across owners.
// With `scale` the received sum is multiplied first (1 / P turns the sum into DDP's mean).
template <typename T>
__global__ void __launch_bounds__(256)
row_apply_kernel(const ZenRowCtx c, T* __restrict__ grad, float scale, int overwrite) {
  __shared__ uint32_t s_n[ZEN_MAX_RANKS];
  const int lane = threadIdx.x & 31;
  const int gw = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, nw = (gridDim.x * blockDim.x) >> 5;
  uint32_t local_status = 0;
  if ((int)threadIdx.x < c.nranks) {
    const ZenMail* mail = reinterpret_cast<const ZenMail*>(c.sym[c.rank] + c.off_g_mail) + threadIdx.x;
    uint32_t n = 0;
    if (zen_wait_epoch(&mail->epoch, row_epoch(c), c.wait_ns)) {
      if (zen_ld_acquire_sys(&mail->info) & 1u) local_status |= ZEN_PEER_OVERFLOW;
      else n = min(zen_ld_acquire_sys(&mail->count), c.cap_g);
    } else {
      local_status |= ZEN_TIMEOUT;
    }
    s_n[threadIdx.x] = n;
  }
  __syncthreads();
  for (int o = 0; o < c.nranks; ++o) {
    const uint32_t n = s_n[o];
    const char* base = c.sym[c.rank];
    const uint32_t* grow = reinterpret_cast<const uint32_t*>(base + c.off_g_row) + (uint64_t)o * c.cap_g;
    const T* gval = reinterpret_cast<const T*>(base + c.off_g_val) + (uint64_t)o * c.cap_g * c.d;
    for (uint32_t k = gw; k < n; k += nw) {
      const uint32_t row = grow[k];
      if (row >= c.vocab) continue;
      for (uint32_t col = lane * 8; col < c.d; col += 256) {
        float x[8], y[8];
        ld8<T>(gval + (uint64_t)k * c.d + col, x);
        if (!overwrite) ld8<T>(grad + (uint64_t)row * c.d + col, y);
#pragma unroll
        for (int i = 0; i < 8; ++i) x[i] = overwrite ? x[i] * scale : y[i] + x[i] * scale;
        st8<T>(grad + (uint64_t)row * c.d + col, x);
      }
    }
  }
  if (local_status) atomicOr(c.status, local_status);
}

int sm_count_r() {
  static int n = 0;
  if (!n) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

}  // namespace

#define DISPATCH_R(dtype, ...)                                             \
  switch (dtype) {                                                         \
    case ZEN_DTYPE_F32: { using T = float; __VA_ARGS__; } break;           \
    case ZEN_DTYPE_BF16: { using T = __nv_bfloat16; __VA_ARGS__; } break;  \
    case ZEN_DTYPE_F16: { using T = __half; __VA_ARGS__; } break;          \
    default: return -1;                                                    \
  }

__global__ void row_epoch_bump_kernel(uint32_t* e) { *e += 1; }

extern "C" {

// Advance the device-side call counter (first launch of every call when the counter lives on the device).
int zen_row_epoch_bump(uint32_t* epoch_dev, void* stream) {
  row_epoch_bump_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(epoch_dev);
  return (int)cudaGetLastError();
}

int zen_row_ctx_size() { return (int)sizeof(ZenRowCtx); }

int zen_row_push(const ZenRowCtx* c, const int32_t* rows, const int32_t* count, const void* vals, int max_rows,
                 int dtype, void* stream) {
  if (c->d % 8) return -2;
  DISPATCH_R(dtype, row_push_kernel<T><<<sm_count_r() * 2, 256, 0, (cudaStream_t)stream>>>(*c, rows, count, (const T*)vals, max_rows));
  return (int)cudaGetLastError();
}

int zen_row_reduce(const ZenRowCtx* c, int dtype, int deterministic, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  if (deterministic) {
    for (int s = 0; s < c->nranks; ++s) { DISPATCH_R(dtype, row_reduce_kernel<T><<<sm_count_r() * 2, 256, 0, st>>>(*c, s, s + 1)); }
  } else {
    DISPATCH_R(dtype, row_reduce_kernel<T><<<sm_count_r() * 2, 256, 0, st>>>(*c, 0, c->nranks));
  }
  return (int)cudaGetLastError();
}

int zen_row_gather_push(const ZenRowCtx* c, int dtype, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  row_list_kernel<<<1, 1024, 0, st>>>(*c);
  DISPATCH_R(dtype, row_gather_push_kernel<T><<<sm_count_r() * 2, 256, 0, st>>>(*c));
  return (int)cudaGetLastError();
}

int zen_row_apply(const ZenRowCtx* c, void* grad, float scale, int overwrite, int dtype, void* stream) {
  DISPATCH_R(dtype, row_apply_kernel<T><<<sm_count_r() * 2, 256, 0, (cudaStream_t)stream>>>(*c, (T*)grad, scale, overwrite));
  return (int)cudaGetLastError();
}

}  // extern "C"
