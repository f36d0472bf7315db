// Causal self-attention forward on tcgen05 tensor cores (sm_100a), flash style: the score matrix never leaves
// the SM.  Input is the fused projection qkv[B*S, (Hq + 2*Hkv) * hd] (bf16); output out[B*S, Hq * hd] and the
// per-row log-sum-exp (base 2, of scores scaled by scale * log2 e) that the backward kernels reuse.
//
// One CTA per (128-query tile, head, batch); 192 threads:
//   warps 0..3  softmax: thread t owns query row t.  Reads S from tensor memory (tcgen05.ld), online softmax in
//               the exp2 domain, writes P (bf16) into shared memory in the 128-byte-swizzled operand layout,
//               rescales the O accumulator in tensor memory (tcgen05.ld / tcgen05.st) when a row maximum moved.
//   warp 4      TMA producer: Q once, then K and V tiles of 128 keys through a ring of stages.
//   warp 5      MMA issuer: S = Q K^T (both operands K-major) and O += P V (V as MN-major operand, so no
//               transpose of V is ever made), tcgen05.commit to mbarriers.
// Tensor memory: S in columns [0, 128), O in [128, 128 + hd).  All mbarrier waits are bounded.
//
// The reference runs HuggingFace "eager" attention (matmul + softmax + matmul, train.py:155), which
// materialises the [B, H, S, S] scores.
#include "tc_common.cuh"

#include <mutex>
#include <unordered_map>

namespace {

using namespace tc;

__device__ int g_attn_error = 0;

struct AttnParams {
  __nv_bfloat16* out;     // [B*S, Hq*hd]
  float* lse2;            // [B, Hq, S]
  int B, S, Hq, Hkv;
  int ld_out;
  float scale_log2;       // softmax scale * log2(e)
};

template <int HD>
struct FwdCfg {
  static constexpr int ATOMS = HD / 64;
  static constexpr int TILE_BYTES = 128 * HD * 2;
  static constexpr int KV_STAGES = (HD <= 128) ? 2 : 1;
  static constexpr int P_BYTES = 128 * 128 * 2;
  static constexpr int SMEM_BYTES = TILE_BYTES + KV_STAGES * 2 * TILE_BYTES + P_BYTES + 1024 + 256;
  static constexpr int TMEM_COLS = (HD <= 128) ? 256 : 512;
  static constexpr uint32_t IDESC_S = make_idesc(128, 128, false, false);
  static constexpr uint32_t IDESC_PV = make_idesc(128, HD, false, true);
};

template <int HD>
__global__ void __launch_bounds__(192)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmap, const AttnParams p) {
  using C = FwdCfg<HD>;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* q_s = smem;
  unsigned char* kv_s = q_s + C::TILE_BYTES;                       // [stage][K | V]
  unsigned char* p_s = kv_s + C::KV_STAGES * 2 * C::TILE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(p_s + C::P_BYTES);
  uint64_t* q_full = bars;
  uint64_t* kv_full = bars + 1;                                    // [2]
  uint64_t* kv_empty = bars + 3;                                   // [2]
  uint64_t* s_full = bars + 5;
  uint64_t* p_ready = bars + 6;
  uint64_t* o_full = bars + 7;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qi = gridDim.x - 1 - blockIdx.x;                       // heavy (late) query tiles first
  const int h = blockIdx.y, b = blockIdx.z;
  const int g = h / (p.Hq / p.Hkv);
  const int row0 = b * p.S + qi * 128;                             // first query row in the [B*S] dimension
  const int ntiles = qi + 1;                                       // causal: key tiles 0..qi

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) { mbar_init(&kv_full[i], 1); mbar_init(&kv_empty[i], 1); }
    mbar_init(s_full, 1);
    mbar_init(p_ready, 4);
    mbar_init(o_full, 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 5) tmem_alloc(tmem_slot, C::TMEM_COLS);
  fence_before();
  __syncthreads();
  fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS = tmem_base, tO = tmem_base + 128;

  if (warp == 4) {
    if (lane == 0) {
      // ---------------------------------------------------------------- TMA producer
      mbar_expect_tx(q_full, C::TILE_BYTES);
#pragma unroll
      for (int a = 0; a < C::ATOMS; ++a) tma_load_2d(q_s + a * 16384, &tmap, q_full, h * HD + a * 64, row0);
      for (int j = 0; j < ntiles; ++j) {
        const int st = j % C::KV_STAGES;
        const uint32_t ph = (j / C::KV_STAGES) & 1;
        if (!mbar_wait(&kv_empty[st], ph ^ 1, abort_flag, 1, &g_attn_error)) break;
        unsigned char* k_s = kv_s + st * 2 * C::TILE_BYTES;
        unsigned char* v_s = k_s + C::TILE_BYTES;
        mbar_expect_tx(&kv_full[st], 2 * C::TILE_BYTES);
        const int krow = b * p.S + j * 128;
#pragma unroll
        for (int a = 0; a < C::ATOMS; ++a) {
          tma_load_2d(k_s + a * 16384, &tmap, &kv_full[st], (p.Hq + g) * HD + a * 64, krow);
          tma_load_2d(v_s + a * 16384, &tmap, &kv_full[st], (p.Hq + p.Hkv + g) * HD + a * 64, krow);
        }
      }
    }
  } else if (warp == 5) {
    if (lane == 0) {
      // ---------------------------------------------------------------- MMA issuer
      bool ok = mbar_wait(q_full, 0, abort_flag, 2, &g_attn_error);
      const uint32_t qa = smem_u32(q_s), pa = smem_u32(p_s);
      for (int j = 0; j < ntiles && ok; ++j) {
        const int st = j % C::KV_STAGES;
        const uint32_t ph = (j / C::KV_STAGES) & 1;
        if (!mbar_wait(&kv_full[st], ph, abort_flag, 3, &g_attn_error)) { ok = false; break; }
        fence_after();
        const uint32_t ka = smem_u32(kv_s + st * 2 * C::TILE_BYTES), va = ka + C::TILE_BYTES;
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;
          umma_bf16(tS, make_desc(qa + off, 16, 1024), make_desc(ka + off, 16, 1024), C::IDESC_S, kk > 0 ? 1u : 0u);
        }
        umma_commit(s_full);
        if (!mbar_wait(p_ready, j & 1, abort_flag, 4, &g_attn_error)) { ok = false; break; }
        fence_after();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t aoff = (kk >> 2) * 16384 + (kk & 3) * 32;
          umma_bf16(tO, make_desc(pa + aoff, 16, 1024), make_desc(va + kk * 2048, 16384, 1024), C::IDESC_PV,
                    (j > 0 || kk > 0) ? 1u : 0u);
        }
        umma_commit(o_full);
        umma_commit(&kv_empty[st]);
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax / correction / epilogue
    const int row = threadIdx.x;                                    // 0..127, also the TMEM lane
    const uint32_t lane_addr = (uint32_t)(warp * 32) << 16;
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < ntiles && ok; ++j) {
      if (!mbar_wait(s_full, j & 1, abort_flag, 5, &g_attn_error)) { ok = false; break; }
      if (j > 0 && !mbar_wait(o_full, (j - 1) & 1, abort_flag, 6, &g_attn_error)) { ok = false; break; }
      fence_after();
      const bool diag = (j == qi);
      float mx = -INFINITY;
#pragma unroll 1
      for (int c4 = 0; c4 < 4; ++c4) {
        uint32_t r[32];
        tmem_ld32(tS + lane_addr + c4 * 32, r);
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float v = __uint_as_float(r[i]) * p.scale_log2;
          if (diag && (c4 * 32 + i) > row) v = -INFINITY;
          mx = fmaxf(mx, v);
        }
      }
      const float m_new = fmaxf(m, mx);
      const float alpha = exp2f(m - m_new);
      float rowsum = 0.f;
#pragma unroll 1
      for (int c4 = 0; c4 < 4; ++c4) {
        uint32_t r[32];
        tmem_ld32(tS + lane_addr + c4 * 32, r);
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float v0 = __uint_as_float(r[i]) * p.scale_log2, v1 = __uint_as_float(r[i + 1]) * p.scale_log2;
          float e0 = exp2f(v0 - m_new), e1 = exp2f(v1 - m_new);
          if (diag && (c4 * 32 + i) > row) e0 = 0.f;
          if (diag && (c4 * 32 + i + 1) > row) e1 = 0.f;
          rowsum += e0 + e1;
          __nv_bfloat162 hh = __floats2bfloat162_rn(e0, e1);
          pk[i >> 1] = *reinterpret_cast<uint32_t*>(&hh);
        }
        unsigned char* atom = p_s + (c4 >> 1) * 16384;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const uint32_t col = (c4 & 1) * 32 + q * 8;
          *reinterpret_cast<uint4*>(atom + swz128(row, col)) = make_uint4(pk[4 * q], pk[4 * q + 1], pk[4 * q + 2], pk[4 * q + 3]);
        }
      }
      l = l * alpha + rowsum;
      m = m_new;
      if (j > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll 1
        for (int c = 0; c < HD / 32; ++c) {
          uint32_t r[32];
          tmem_ld32(tO + lane_addr + c * 32, r);
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
          tmem_st32(tO + lane_addr + c * 32, r);
        }
      }
      fence_before();
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_ready);
    }
    if (ok && mbar_wait(o_full, (ntiles - 1) & 1, abort_flag, 7, &g_attn_error)) {
      fence_after();
      const float inv = 1.f / l;
      __nv_bfloat16* op = p.out + (size_t)(row0 + row) * p.ld_out + h * HD;
#pragma unroll 1
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(tO + lane_addr + c * 32, r);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          uint32_t o[4];
#pragma unroll
          for (int k2 = 0; k2 < 4; ++k2) {
            __nv_bfloat162 hh = __floats2bfloat162_rn(__uint_as_float(r[8 * q + 2 * k2]) * inv, __uint_as_float(r[8 * q + 2 * k2 + 1]) * inv);
            o[k2] = *reinterpret_cast<uint32_t*>(&hh);
          }
          *reinterpret_cast<uint4*>(op + c * 32 + q * 8) = make_uint4(o[0], o[1], o[2], o[3]);
        }
      }
      p.lse2[((size_t)b * p.Hq + h) * p.S + qi * 128 + row] = m + log2f(l);
    }
  }

  fence_before();
  __syncthreads();
  if (*abort_flag) {
    const uint64_t t0 = gtimer();
    while (gtimer() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 5) {
    fence_after();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

// ------------------------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn attn_get_encode() {
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

// bf16 [rows, cols] row-major (row stride ld elements) with a {64, 128} box and 128-byte swizzle.
int attn_make_map(const void* ptr, uint64_t cols, uint64_t rows, uint64_t ld, CUtensorMap* out) {
  EncodeTiledFn enc = attn_get_encode();
  if (!enc) return -10;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {64, 128};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -11;
}

template <int HD>
int launch_fwd(const CUtensorMap& tm, const AttnParams& p, cudaStream_t st) {
  using C = FwdCfg<HD>;
  static bool attr = false;
  if (!attr) {
    cudaError_t e = cudaFuncSetAttribute(attn_fwd_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    attr = true;
  }
  dim3 grid(p.S / 128, p.Hq, p.B);
  attn_fwd_kernel<HD><<<grid, 192, C::SMEM_BYTES, st>>>(tm, p);
  return (int)cudaGetLastError();
}

}  // namespace

extern "C" {

// Causal attention forward.  qkv: bf16 [B*S, (Hq + 2*Hkv) * hd] with row stride ld_qkv (elements, multiple of 8,
// base 16-byte aligned); out: bf16 [B*S, Hq*hd] (row stride ld_out); lse2: fp32 [B, Hq, S].
// Supported: hd in {64, 128, 256}, S a multiple of 128, Hq a multiple of Hkv.
int zen_attn_fwd(const void* qkv, void* out, float* lse2, int B, int S, int Hq, int Hkv, int hd, int ld_qkv, int ld_out,
                 float scale, void* stream) {
  if (S % 128 || Hq % Hkv || (hd != 64 && hd != 128 && hd != 256)) return -2;
  if ((ld_qkv % 8) || (ld_out % 8) || (reinterpret_cast<uintptr_t>(qkv) % 16) || (reinterpret_cast<uintptr_t>(out) % 16)) return -3;
  CUtensorMap tm;
  int rc = attn_make_map(qkv, (uint64_t)(Hq + 2 * Hkv) * hd, (uint64_t)B * S, (uint64_t)ld_qkv, &tm);
  if (rc) return rc;
  AttnParams p{(__nv_bfloat16*)out, lse2, B, S, Hq, Hkv, ld_out, scale * 1.4426950408889634f};
  cudaStream_t st = (cudaStream_t)stream;
  if (hd == 64) return launch_fwd<64>(tm, p, st);
  if (hd == 128) return launch_fwd<128>(tm, p, st);
  return launch_fwd<256>(tm, p, st);
}

int zen_attn_error() {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_attn_error, sizeof(int)) != cudaSuccess) return -1;
  if (v) cudaMemcpyToSymbol(g_attn_error, &zero, sizeof(int));
  return v;
}

}  // extern "C"
