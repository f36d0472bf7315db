// All-reduce of a dense gradient bucket through the NVSwitch (NVLS): every rank owns 1/P of the bucket,
// pulls the sum of that slice from all ranks with ONE `multimem.ld_reduce` per 16 bytes (the switch adds
// the P copies in fp32), scales it, and pushes the result to all ranks with ONE `multimem.st`.  The
// reduction itself costs no SM arithmetic and each byte crosses this GPU's links once in each
// direction, so a handful of CTAs saturates the links and the rest of the GPU keeps running backward.
// (The library ring all-reduce that this replaces on the data-parallel path occupied 32 SMs at two
// GPUs.)  Two flag exchanges bracket the data movement: "my bucket is complete" before anybody pulls, "my
// stores have landed and I have finished pulling from you" before anybody's kernel ends.  Every wait
// is bounded and reports through a status word.
//
// The bucket must live in a multicast-mapped symmetric region (torch symmetric memory): `mc` is the
// multicast alias of the region's base, `flags[r]` the flag block inside rank r's copy.
// Reference counterpart: the dense bucket all-reduce of torch DDP (train.py:184-185, NCCL).
#include "zen_common.cuh"

struct ZenMcArCtx {
  int32_t rank;
  int32_t nranks;
  uint32_t epoch;              // call counter by value (ignored when epoch_dev is set)
  uint32_t pad;
  uint64_t wait_ns;
  char* mc;                    // multicast alias of the region
  uint32_t* flags[ZEN_MAX_RANKS];   // per rank: uint32 [2 exchanges][ZEN_MAX_RANKS sources]
  const uint32_t* epoch_dev;   // optional device-resident call counter (bumped by zen_sparse_epoch_bump before the call)
  uint32_t* status;            // device word, ZEN_TIMEOUT is OR-ed in when a wait runs out
  uint32_t* done;              // device word, CTA arrival counter (left at zero)
};

namespace {

__device__ __forceinline__ void mm_ld_reduce_bf16(const void* mc_addr, uint32_t (&v)[4]) {
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]) : "l"(mc_addr) : "memory");
}
__device__ __forceinline__ void mm_ld_reduce_f32(const void* mc_addr, uint32_t (&v)[4]) {
  float a, b, c, d;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(a), "=f"(b), "=f"(c), "=f"(d) : "l"(mc_addr) : "memory");
  v[0] = __float_as_uint(a); v[1] = __float_as_uint(b); v[2] = __float_as_uint(c); v[3] = __float_as_uint(d);
}
__device__ __forceinline__ void mm_st16(void* mc_addr, const uint32_t (&v)[4]) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr), "f"(__uint_as_float(v[0])),
               "f"(__uint_as_float(v[1])), "f"(__uint_as_float(v[2])), "f"(__uint_as_float(v[3])) : "memory");
}
__device__ __forceinline__ uint32_t scale_bf16x2(uint32_t w, float s) {
  const float lo = __uint_as_float(w << 16) * s, hi = __uint_as_float(w & 0xffff0000u) * s;
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

// is_bf16: 16-byte vectors of eight bf16, else of four fp32.  nvec 16-byte vectors starting at byte_off of the region.
#define MCAR_THREADS 512
#define MCAR_UNROLL 8
template <bool is_bf16>
__global__ void __launch_bounds__(MCAR_THREADS)
zen_multimem_allreduce_kernel(const ZenMcArCtx c, uint64_t byte_off, uint64_t nvec, float scale) {
  __shared__ uint32_t s_ok, s_last;
  const uint32_t epoch = c.epoch_dev ? *c.epoch_dev : c.epoch;
  const int tid = threadIdx.x;
  // first flag exchange: tell every rank that this rank's bucket is complete (the kernels that wrote it ran earlier on this
  // stream), then wait until every rank has said so
  if (blockIdx.x == 0 && tid < c.nranks) zen_st_release_sys(c.flags[tid] + c.rank, epoch);
  if (tid == 0) s_ok = 1u;
  __syncthreads();
  if (tid < c.nranks && !zen_wait_epoch(c.flags[c.rank] + tid, epoch, c.wait_ns)) s_ok = 0u;
  __syncthreads();
  const bool ok = s_ok != 0u;
  if (ok) {
    const uint64_t per = (nvec + c.nranks - 1) / c.nranks;
    const uint64_t lo = min(nvec, per * (uint64_t)c.rank), hi = min(nvec, lo + per);
    char* base = c.mc + byte_off;
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    // MCAR_UNROLL pulls in flight per thread: the round trip through the switch is a few microseconds, so a CTA needs
    // on the order of 100 KB outstanding to move tens of GB/s
    for (uint64_t i = lo + (uint64_t)blockIdx.x * blockDim.x + tid; i < hi; i += MCAR_UNROLL * stride) {
      uint32_t v[MCAR_UNROLL][4];
#pragma unroll
      for (int u = 0; u < MCAR_UNROLL; ++u) {
        const uint64_t j = i + u * stride;
        if (j < hi) { if (is_bf16) mm_ld_reduce_bf16(base + j * 16, v[u]); else mm_ld_reduce_f32(base + j * 16, v[u]); }
      }
#pragma unroll
      for (int u = 0; u < MCAR_UNROLL; ++u) {
        const uint64_t j = i + u * stride;
        if (j >= hi) continue;
        if (scale != 1.f) {
#pragma unroll
          for (int k = 0; k < 4; ++k)
            v[u][k] = is_bf16 ? scale_bf16x2(v[u][k], scale) : __float_as_uint(__uint_as_float(v[u][k]) * scale);
        }
        mm_st16(base + j * 16, v[u]);
      }
    }
  }
  // second flag exchange: when every CTA of this rank has stored its part, tell every rank; the last CTA stays until every rank
  // has said the same, so that this kernel's end means "the whole bucket is reduced here, and nobody still reads mine"
  __syncthreads();
  if (tid == 0) {
    __threadfence_system();
    const uint32_t prev = atomicAdd(c.done, 1u);
    s_last = (prev == gridDim.x - 1) ? 1u : 0u;
  }
  __syncthreads();
  if (!ok && tid == 0) atomicOr(c.status, ZEN_TIMEOUT);
  if (s_last) {
    __threadfence_system();
    if (tid < c.nranks) {
      zen_st_release_sys(c.flags[tid] + ZEN_MAX_RANKS + c.rank, epoch);
      if (!zen_wait_epoch(c.flags[c.rank] + ZEN_MAX_RANKS + tid, epoch, c.wait_ns)) atomicOr(c.status, ZEN_TIMEOUT);
    }
    if (tid == 0) *c.done = 0u;
  }
}

}  // namespace

extern "C" {

int zen_mc_ar_ctx_size() { return (int)sizeof(ZenMcArCtx); }

// In-place all-reduce (sum, times `scale`) of `nbytes` at `byte_off` of the multicast-mapped region.  byte_off and nbytes
// are multiples of 16.  dtype: ZEN_DTYPE_BF16 or ZEN_DTYPE_F32.  ctas: CTAs to use (0 = 8).
int zen_multimem_allreduce(const ZenMcArCtx* c, uint64_t byte_off, uint64_t nbytes, int dtype, float scale, int ctas,
                           void* stream) {
  if (!c || !c->mc || c->nranks < 2 || c->nranks > ZEN_MAX_RANKS) return -3;
  if ((byte_off % 16) || (nbytes % 16) || (dtype != ZEN_DTYPE_BF16 && dtype != ZEN_DTYPE_F32)) return -2;
  if (nbytes == 0) return 0;
  if (ctas <= 0) ctas = 8;
  if (ctas > 148) ctas = 148;
  if (dtype == ZEN_DTYPE_BF16) zen_multimem_allreduce_kernel<true><<<ctas, MCAR_THREADS, 0, (cudaStream_t)stream>>>(*c, byte_off, nbytes / 16, scale);
  else zen_multimem_allreduce_kernel<false><<<ctas, MCAR_THREADS, 0, (cudaStream_t)stream>>>(*c, byte_off, nbytes / 16, scale);
  return (int)cudaGetLastError();
}

}  // extern "C"
