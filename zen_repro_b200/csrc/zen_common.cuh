// Shared device-side helpers for the sm_100a kernels of this library.
//
// Everything that waits on another GPU waits with a bound and reports through
// a status word instead of trapping, so that a missing peer costs a timeout,
// never a hung context.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define ZEN_MAX_RANKS 8

// Bits of the per-launch status word (OR-ed by kernels, read by the host).
enum ZenStatus : uint32_t {
  ZEN_OK = 0u,
  ZEN_REC_OVERFLOW = 1u,     // a (source, owner) record slot was too small
  ZEN_GATHER_OVERFLOW = 2u,  // an owner's gather payload was too small
  ZEN_TIMEOUT = 4u,          // a bounded wait on a peer's mailbox ran out
  ZEN_PEER_OVERFLOW = 8u,    // a peer reported an overflow in its mail
  ZEN_BAD_ARG = 16u,
};

// Mailbox written by a producer into the consumer's memory: payload first,
// then the epoch with release semantics at system scope.
struct __align__(16) ZenMail {
  uint32_t count;
  uint32_t info;   // bit0: overflow seen by the sender; bits 8..15: index format
  uint32_t aux;
  uint32_t epoch;
};

#define ZEN_FMT_COO 1u
#define ZEN_FMT_BITMAP 2u

// Block permutation parameters; see sparse/hashing.py for the maths.
struct ZenPerm {
  uint32_t block;      // G
  uint32_t nblocks;    // nb' = P * sb
  uint32_t sb;         // blocks per owner
  uint32_t mask;       // 2^k - 1, 2^k >= nb'
  uint32_t mult;       // a (odd)
  uint32_t mult_inv;   // a^-1 mod 2^k
  uint32_t add;        // c
  uint32_t lg;         // log2(G); G is a power of two
};

// Affine bijection of [0, 2^k) restricted to [0, nb') by cycle walking.  The walk always ends (the
// orbit of an in-range value returns in range); the cap only guards against bad parameters.
__device__ __forceinline__ uint32_t zen_perm_fwd(const ZenPerm& p, uint32_t blk) {
  uint32_t y = (p.mult * blk + p.add) & p.mask;
  for (int i = 0; i < 64 && y >= p.nblocks; ++i) y = (p.mult * y + p.add) & p.mask;
  return y;
}
__device__ __forceinline__ uint32_t zen_perm_inv(const ZenPerm& p, uint32_t pb) {
  uint32_t y = (p.mult_inv * ((pb - p.add) & p.mask)) & p.mask;
  for (int i = 0; i < 64 && y >= p.nblocks; ++i) y = (p.mult_inv * ((y - p.add) & p.mask)) & p.mask;
  return y;
}
// owner = y / sb for y < P * sb with P <= 8, without a division.
__device__ __forceinline__ uint32_t zen_owner_of(const ZenPerm& p, uint32_t y, int nranks) {
  uint32_t o = 0, t = p.sb;
#pragma unroll
  for (int i = 1; i < ZEN_MAX_RANKS; ++i) { o += (i < nranks && y >= t) ? 1u : 0u; t += p.sb; }
  return o;
}

__device__ __forceinline__ void zen_st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t zen_ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint64_t zen_globaltimer() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// Spin until *flag == epoch or `budget_ns` has passed. Returns true on success.
__device__ __forceinline__ bool zen_wait_epoch(const uint32_t* flag, uint32_t epoch, uint64_t budget_ns) {
  if (zen_ld_acquire_sys(flag) == epoch) return true;
  const uint64_t t0 = zen_globaltimer();
  for (;;) {
    for (int i = 0; i < 64; ++i) {
      if (zen_ld_acquire_sys(flag) == epoch) return true;
      __nanosleep(64);
    }
    if (zen_globaltimer() - t0 > budget_ns) return false;
  }
}

template <typename T> struct ZenVal;
template <> struct ZenVal<float> {
  static __device__ __forceinline__ float to_f(float v) { return v; }
  static __device__ __forceinline__ float from_f(float v) { return v; }
  static __device__ __forceinline__ uint32_t bits(float v) { return __float_as_uint(v); }
  static __device__ __forceinline__ float unbits(uint32_t b) { return __uint_as_float(b); }
  static __device__ __forceinline__ float from_bits(uint32_t b) { return __uint_as_float(b); }
};
template <> struct ZenVal<__nv_bfloat16> {
  static __device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 from_f(float v) { return __float2bfloat16_rn(v); }
  static __device__ __forceinline__ uint32_t bits(__nv_bfloat16 v) { return (uint32_t)__bfloat16_as_ushort(v); }
  static __device__ __forceinline__ float unbits(uint32_t b) { return __uint_as_float(b << 16); }
  static __device__ __forceinline__ __nv_bfloat16 from_bits(uint32_t b) { return __ushort_as_bfloat16((unsigned short)b); }
};
template <> struct ZenVal<__half> {
  static __device__ __forceinline__ float to_f(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half from_f(float v) { return __float2half_rn(v); }
  static __device__ __forceinline__ uint32_t bits(__half v) { return (uint32_t)__half_as_ushort(v); }
  static __device__ __forceinline__ float unbits(uint32_t b) { return __half2float(__ushort_as_half((unsigned short)b)); }
  static __device__ __forceinline__ __half from_bits(uint32_t b) { return __ushort_as_half((unsigned short)b); }
};

#define ZEN_DTYPE_F32 0
#define ZEN_DTYPE_BF16 1
#define ZEN_DTYPE_F16 2

#define ZEN_CUDA_CHECK_RET(expr)                 \
  do {                                           \
    cudaError_t _e = (expr);                     \
    if (_e != cudaSuccess) return (int)_e;       \
  } while (0)
