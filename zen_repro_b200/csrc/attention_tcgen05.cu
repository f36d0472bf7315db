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
  float cap_a;            // soft-capping of the scaled scores, cap * tanh(s * scale / cap): scale / cap, or 0 for none
};

// Soft-capped raw score: the value x' with x' * scale = cap * tanh(x * scale / cap), so that everything after it
// (maximum, exponentials, the saved log-sum-exp) goes on as for plain scores.  a = scale / cap.
__device__ __forceinline__ float tanh_fast(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t softcap_bits(uint32_t raw, float a, float inv_a) {
  return __float_as_uint(tanh_fast(__uint_as_float(raw) * a) * inv_a);
}

template <int HD>
struct FwdCfg {
  static constexpr int ATOMS = HD / 64;
  static constexpr int TILE_BYTES = 128 * HD * 2;
  static constexpr int KV_STAGES = (HD <= 128) ? 2 : 1;
  // With two K / V stages S = Q K^T of tile j + 1 is issued as soon as the softmax warps have read the scores of tile j
  // out of tensor memory, ahead of P V of tile j, so that it leaves the per-tile chain softmax -> P V -> next softmax.
  static constexpr bool EARLY_SCORES = KV_STAGES >= 2;
  static constexpr int P_BYTES = 128 * 128 * 2;
  // No slack for re-aligning the base: the kernel has no static shared memory, so its dynamic window starts at the
  // CTA's shared-memory base, which is 1024-byte aligned; the kernel checks this and gives up cleanly otherwise.
  // (With the slack, two hd = 64 CTAs would miss the per-SM capacity by 512 bytes.)
  static constexpr int SMEM_BYTES = TILE_BYTES + KV_STAGES * 2 * TILE_BYTES + P_BYTES + 256;
  static constexpr int TMEM_COLS = (HD <= 128) ? 256 : 512;
  static constexpr uint32_t IDESC_S = make_idesc(128, 128, false, false);
  static constexpr uint32_t IDESC_PV = make_idesc(128, HD, false, true);
};

template <int HD>
__global__ void __launch_bounds__(192, (HD <= 64) ? 2 : 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmap, const AttnParams p) {
  using C = FwdCfg<HD>;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* smem = smem_raw;
  if ((smem_u32(smem_raw) & 1023u) != 0u) {          // uniform over the CTA: nothing has been allocated yet
    if (threadIdx.x == 0) atomicCAS(&g_attn_error, 0, 99);
    return;
  }
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
  uint64_t* s_free = bars + 8;                                     // the softmax warps hold the scores in registers
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 9);
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
    mbar_init(s_free, 4);
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
      auto issue_scores = [&](int t) -> bool {
        const int st = t % C::KV_STAGES;
        const uint32_t ph = (t / C::KV_STAGES) & 1;
        if (!mbar_wait(&kv_full[st], ph, abort_flag, 3, &g_attn_error)) return false;
        fence_after();
        const uint32_t ka = smem_u32(kv_s + st * 2 * C::TILE_BYTES);
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;
          umma_bf16(tS, make_desc(qa + off, 16, 1024), make_desc(ka + off, 16, 1024), C::IDESC_S, kk > 0 ? 1u : 0u);
        }
        umma_commit(s_full);
        return true;
      };
      if (C::EARLY_SCORES && ok && ntiles > 0) ok = issue_scores(0);
      for (int j = 0; j < ntiles && ok; ++j) {
        const int st = j % C::KV_STAGES;
        if (!C::EARLY_SCORES) {
          if (!issue_scores(j)) { ok = false; break; }
        } else if (j + 1 < ntiles) {
          if (!mbar_wait(s_free, j & 1, abort_flag, 8, &g_attn_error)) { ok = false; break; }
          fence_after();
          if (!issue_scores(j + 1)) { ok = false; break; }
        }
        const uint32_t va = smem_u32(kv_s + st * 2 * C::TILE_BYTES) + C::TILE_BYTES;
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
      fence_after();
      const bool diag = (j == qi);
      // the whole score row of this thread (128 values) in registers: one tensor-memory round trip
      uint32_t r0[32], r1[32], r2[32], r3[32];
      tmem_ld32_nowait(tS + lane_addr, r0);
      tmem_ld32_nowait(tS + lane_addr + 32, r1);
      tmem_ld32_nowait(tS + lane_addr + 64, r2);
      tmem_ld32_nowait(tS + lane_addr + 96, r3);
      // P of the previous tile is still being read by its P V product (and O is not final): wait while the loads fly
      if (j > 0 && !mbar_wait(o_full, (j - 1) & 1, abort_flag, 6, &g_attn_error)) { tmem_wait_ld(); ok = false; break; }
      tmem_wait_ld();
      if (C::EARLY_SCORES) {
        fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(s_free);
      }
      if (p.cap_a != 0.f) {
        const float a = p.cap_a, ia = 1.f / p.cap_a;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          r0[i] = softcap_bits(r0[i], a, ia); r1[i] = softcap_bits(r1[i], a, ia);
          r2[i] = softcap_bits(r2[i], a, ia); r3[i] = softcap_bits(r3[i], a, ia);
        }
      }
      if (diag) {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          if (i > row) r0[i] = 0xff800000u;
          if (32 + i > row) r1[i] = 0xff800000u;
          if (64 + i > row) r2[i] = 0xff800000u;
          if (96 + i > row) r3[i] = 0xff800000u;
        }
      }
      float x0 = -INFINITY, x1 = -INFINITY, x2 = -INFINITY, x3 = -INFINITY;
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        x0 = fmaxf(x0, __uint_as_float(r0[i])); x1 = fmaxf(x1, __uint_as_float(r1[i]));
        x2 = fmaxf(x2, __uint_as_float(r2[i])); x3 = fmaxf(x3, __uint_as_float(r3[i]));
      }
      const float mx = fmaxf(fmaxf(x0, x1), fmaxf(x2, x3)) * p.scale_log2;
      // lazy maximum: keep the old reference unless the row maximum grew by more than 2^8; P stays below 256,
      // the final normalisation is exact either way, and O is rescaled only on such jumps
      const bool need = mx > m + 8.f;
      const float m_new = need ? mx : m;
      const float alpha = need ? ex2f(m - m_new) : 1.f;
      const float cs = p.scale_log2, nm = -m_new;
      float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
#define ZEN_SOFTMAX_CHUNK(RR, C4, SUM)                                                                  \
      {                                                                                                 \
        uint32_t pk[16];                                                                                \
        _Pragma("unroll") for (int i = 0; i < 32; i += 2) {                                             \
          const float e0 = ex2f(fmaf(__uint_as_float(RR[i]), cs, nm));                                  \
          const float e1 = ex2f(fmaf(__uint_as_float(RR[i + 1]), cs, nm));                              \
          SUM += e0 + e1;                                                                               \
          pk[i >> 1] = pack_bf16(e0, e1);                                                               \
        }                                                                                               \
        unsigned char* atom = p_s + ((C4) >> 1) * 16384;                                                \
        _Pragma("unroll") for (int q = 0; q < 4; ++q)                                                   \
          *reinterpret_cast<uint4*>(atom + swz128(row, ((C4) & 1) * 32 + q * 8)) =                      \
              make_uint4(pk[4 * q], pk[4 * q + 1], pk[4 * q + 2], pk[4 * q + 3]);                       \
      }
      ZEN_SOFTMAX_CHUNK(r0, 0, s0)
      ZEN_SOFTMAX_CHUNK(r1, 1, s1)
      ZEN_SOFTMAX_CHUNK(r2, 2, s2)
      ZEN_SOFTMAX_CHUNK(r3, 3, s3)
#undef ZEN_SOFTMAX_CHUNK
      l = l * alpha + ((s0 + s1) + (s2 + s3));
      m = m_new;
      if (j > 0 && __any_sync(0xffffffffu, need)) {
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

// ====================================================================================== backward
// D[b, h, s] = sum_c dO[row, h*hd + c] * O[row, h*hd + c]   (one warp per (row, head))
__global__ void __launch_bounds__(256)
attn_bwd_prep_kernel(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ out, float* __restrict__ D,
                     int B, int S, int Hq, int hd, int ld) {
  const int lane = threadIdx.x & 31;
  const long gw = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 5, nw = ((long)gridDim.x * blockDim.x) >> 5;
  const long total = (long)B * S * Hq;
  for (long u = gw; u < total; u += nw) {
    const int h = (int)(u % Hq);
    const long row = u / Hq;
    const __nv_bfloat16* a = dout + row * ld + h * hd;
    const __nv_bfloat16* o = out + row * ld + h * hd;
    float acc = 0.f;
    for (int c = lane * 8; c < hd; c += 256) {
      const uint4 x = *reinterpret_cast<const uint4*>(a + c), y = *reinterpret_cast<const uint4*>(o + c);
      const uint32_t xw[4] = {x.x, x.y, x.z, x.w}, yw[4] = {y.x, y.y, y.z, y.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        acc += __uint_as_float(xw[i] << 16) * __uint_as_float(yw[i] << 16);
        acc += __uint_as_float(xw[i] & 0xffff0000u) * __uint_as_float(yw[i] & 0xffff0000u);
      }
    }
#pragma unroll
    for (int d = 16; d; d >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, d);
    if (lane == 0) {
      const int b = (int)(row / S), sidx = (int)(row % S);
      D[((size_t)b * Hq + h) * S + sidx] = acc;
    }
  }
}

struct AttnBwdParams {
  __nv_bfloat16* dqkv;    // [B*S, (Hq + 2*Hkv) * hd]
  const float* lse2;      // [B, Hq, S]
  const float* D;         // [B, Hq, S]
  int B, S, Hq, Hkv;
  int ld_dqkv;
  float scale_log2;
  float scale;
  float* part;            // hd 256, hsplit > 1: fp32 partial dK | dV, each [hsplit][B*S][Hkv * 256]
  int hsplit;             // CTAs that share one KV head (each takes Hq / Hkv / hsplit query heads)
  float cap_a;            // soft-capping (head_dim 256 kernels): scale / cap, or 0 for none
};

// ---- dQ: one CTA per (query tile, head, batch).  Per key tile: S = Q K^T and dP = dO V^T into tensor memory,
// dS = P * (dP - D) written to shared memory as an operand, dQ += dS K (K as MN-major operand).
template <int HD>
struct DqCfg {
  static constexpr int ATOMS = HD / 64;
  static constexpr int TILE_BYTES = 128 * HD * 2;
  static constexpr int KV_STAGES = (HD <= 128) ? 2 : 1;     // hd 128: 64 + 128 + 32 KB = 224 KB, still one CTA's worth
  // with two K / V stages the scores of tile j + 1 are issued ahead of dQ += dS K of tile j (see FwdCfg)
  static constexpr bool EARLY_SCORES = KV_STAGES >= 2;
  static constexpr int DS_BYTES = 128 * 128 * 2;
  static constexpr int SMEM_BYTES = 2 * TILE_BYTES + KV_STAGES * 2 * TILE_BYTES + DS_BYTES + 1024 + 256;
  static constexpr int TMEM_COLS = 512;
  static constexpr uint32_t IDESC_S = make_idesc(128, 128, false, false);
  static constexpr uint32_t IDESC_DQ = make_idesc(128, HD, false, true);
};

template <int HD>
__global__ void __launch_bounds__(320)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmap_qkv, const __grid_constant__ CUtensorMap tmap_do,
                   const AttnBwdParams p) {
  using C = DqCfg<HD>;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* q_s = smem;
  unsigned char* do_s = q_s + C::TILE_BYTES;
  unsigned char* kv_s = do_s + C::TILE_BYTES;
  unsigned char* ds_s = kv_s + C::KV_STAGES * 2 * C::TILE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(ds_s + C::DS_BYTES);
  uint64_t* q_full = bars;
  uint64_t* kv_full = bars + 1;
  uint64_t* kv_empty = bars + 3;
  uint64_t* sdp_full = bars + 5;
  uint64_t* ds_ready = bars + 6;
  uint64_t* dq_done = bars + 7;
  uint64_t* s_free = bars + 8;                                     // the softmax warps hold S and dP in registers
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 9);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qi = gridDim.x - 1 - blockIdx.x;
  const int h = blockIdx.y, b = blockIdx.z;
  const int g = h / (p.Hq / p.Hkv);
  const int row0 = b * p.S + qi * 128;
  const int ntiles = qi + 1;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) { mbar_init(&kv_full[i], 1); mbar_init(&kv_empty[i], 1); }
    mbar_init(sdp_full, 1);
    mbar_init(ds_ready, 8);
    mbar_init(dq_done, 1);
    mbar_init(s_free, 8);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 9) tmem_alloc(tmem_slot, C::TMEM_COLS);
  fence_before();
  __syncthreads();
  fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS = tmem_base, tDP = tmem_base + 128, tDQ = tmem_base + 256;

  if (warp == 8) {
    if (lane == 0) {
      mbar_expect_tx(q_full, 2 * C::TILE_BYTES);
#pragma unroll
      for (int a = 0; a < C::ATOMS; ++a) {
        tma_load_2d(q_s + a * 16384, &tmap_qkv, q_full, h * HD + a * 64, row0);
        tma_load_2d(do_s + a * 16384, &tmap_do, q_full, h * HD + a * 64, row0);
      }
      for (int j = 0; j < ntiles; ++j) {
        const int st = j % C::KV_STAGES;
        const uint32_t ph = (j / C::KV_STAGES) & 1;
        if (!mbar_wait(&kv_empty[st], ph ^ 1, abort_flag, 11, &g_attn_error)) break;
        unsigned char* k_s = kv_s + st * 2 * C::TILE_BYTES;
        unsigned char* v_s = k_s + C::TILE_BYTES;
        mbar_expect_tx(&kv_full[st], 2 * C::TILE_BYTES);
        const int krow = b * p.S + j * 128;
#pragma unroll
        for (int a = 0; a < C::ATOMS; ++a) {
          tma_load_2d(k_s + a * 16384, &tmap_qkv, &kv_full[st], (p.Hq + g) * HD + a * 64, krow);
          tma_load_2d(v_s + a * 16384, &tmap_qkv, &kv_full[st], (p.Hq + p.Hkv + g) * HD + a * 64, krow);
        }
      }
    }
  } else if (warp == 9) {
    if (lane == 0) {
      bool ok = mbar_wait(q_full, 0, abort_flag, 12, &g_attn_error);
      const uint32_t qa = smem_u32(q_s), doa = smem_u32(do_s), dsa = smem_u32(ds_s);
      auto issue_scores = [&](int t) -> bool {
        const int st = t % C::KV_STAGES;
        const uint32_t ph = (t / C::KV_STAGES) & 1;
        if (!mbar_wait(&kv_full[st], ph, abort_flag, 13, &g_attn_error)) return false;
        fence_after();
        const uint32_t ka = smem_u32(kv_s + st * 2 * C::TILE_BYTES), va = ka + C::TILE_BYTES;
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;
          umma_bf16(tS, make_desc(qa + off, 16, 1024), make_desc(ka + off, 16, 1024), C::IDESC_S, kk > 0 ? 1u : 0u);
        }
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;
          umma_bf16(tDP, make_desc(doa + off, 16, 1024), make_desc(va + off, 16, 1024), C::IDESC_S, kk > 0 ? 1u : 0u);
        }
        umma_commit(sdp_full);
        return true;
      };
      if (C::EARLY_SCORES && ok && ntiles > 0) ok = issue_scores(0);
      for (int j = 0; j < ntiles && ok; ++j) {
        const int st = j % C::KV_STAGES;
        if (!C::EARLY_SCORES) {
          if (!issue_scores(j)) { ok = false; break; }
        } else if (j + 1 < ntiles) {
          if (!mbar_wait(s_free, j & 1, abort_flag, 17, &g_attn_error)) { ok = false; break; }
          fence_after();
          if (!issue_scores(j + 1)) { ok = false; break; }
        }
        const uint32_t ka = smem_u32(kv_s + st * 2 * C::TILE_BYTES);
        if (!mbar_wait(ds_ready, j & 1, abort_flag, 14, &g_attn_error)) { ok = false; break; }
        fence_after();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t aoff = (kk >> 2) * 16384 + (kk & 3) * 32;
          umma_bf16(tDQ, make_desc(dsa + aoff, 16, 1024), make_desc(ka + kk * 2048, 16384, 1024), C::IDESC_DQ,
                    (j > 0 || kk > 0) ? 1u : 0u);
        }
        umma_commit(dq_done);
        umma_commit(&kv_empty[st]);
      }
    }
  } else {
    // warps w and w + 4 share the rows of TMEM lane group w & 3 and split the 128 key columns in two halves
    const int row = (warp & 3) * 32 + lane;
    const int hf = warp >> 2;
    const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
    const size_t vec = ((size_t)b * p.Hq + h) * p.S + qi * 128 + row;
    const float lse = p.lse2[vec], Dr = p.D[vec];
    bool ok = true;
    for (int j = 0; j < ntiles && ok; ++j) {
      if (!mbar_wait(sdp_full, j & 1, abort_flag, 15, &g_attn_error)) { ok = false; break; }
      fence_after();
      const bool diag = (j == qi);
      const float cs = p.scale_log2, nl = -lse;
      {
        uint32_t sa[32], sb[32], da[32], db[32];
        tmem_ld32_nowait(tS + lane_addr + hf * 64, sa);
        tmem_ld32_nowait(tS + lane_addr + hf * 64 + 32, sb);
        tmem_ld32_nowait(tDP + lane_addr + hf * 64, da);
        tmem_ld32_nowait(tDP + lane_addr + hf * 64 + 32, db);
        tmem_wait_ld();
        if (C::EARLY_SCORES) {                                     // S and dP are in registers: the next tile's may be issued
          fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(s_free);
        }
        if (diag) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            if (hf * 64 + i > row) sa[i] = 0xff800000u;
            if (hf * 64 + 32 + i > row) sb[i] = 0xff800000u;
          }
        }
        // dS of this tile in registers first: the previous tile's copy in shared memory is still being read by its
        // dQ product, which finishes meanwhile
        uint32_t pk0[16], pk1[16];
#define ZEN_DS_CHUNK(SS, DD, PK)                                                                        \
        _Pragma("unroll") for (int i = 0; i < 32; i += 2) {                                             \
          const float p0 = ex2f(fmaf(__uint_as_float(SS[i]), cs, nl));                                  \
          const float p1 = ex2f(fmaf(__uint_as_float(SS[i + 1]), cs, nl));                              \
          PK[i >> 1] = pack_bf16(p0 * (__uint_as_float(DD[i]) - Dr), p1 * (__uint_as_float(DD[i + 1]) - Dr)); \
        }
        ZEN_DS_CHUNK(sa, da, pk0)
        ZEN_DS_CHUNK(sb, db, pk1)
#undef ZEN_DS_CHUNK
        if (j > 0 && !mbar_wait(dq_done, (j - 1) & 1, abort_flag, 16, &g_attn_error)) { ok = false; break; }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          *reinterpret_cast<uint4*>(ds_s + hf * 16384 + swz128(row, q * 8)) =
              make_uint4(pk0[4 * q], pk0[4 * q + 1], pk0[4 * q + 2], pk0[4 * q + 3]);
          *reinterpret_cast<uint4*>(ds_s + hf * 16384 + swz128(row, 32 + q * 8)) =
              make_uint4(pk1[4 * q], pk1[4 * q + 1], pk1[4 * q + 2], pk1[4 * q + 3]);
        }
      }
      fence_before();
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(ds_ready);
    }
    if (ok && mbar_wait(dq_done, (ntiles - 1) & 1, abort_flag, 17, &g_attn_error)) {
      fence_after();
      __nv_bfloat16* op = p.dqkv + (size_t)(row0 + row) * p.ld_dqkv + h * HD;
#pragma unroll 1
      for (int c = hf * (HD / 64); c < (hf + 1) * (HD / 64); ++c) {
        uint32_t r[32];
        tmem_ld32(tDQ + lane_addr + c * 32, r);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          uint32_t o[4];
#pragma unroll
          for (int k2 = 0; k2 < 4; ++k2) {
            __nv_bfloat162 hh = __floats2bfloat162_rn(__uint_as_float(r[8 * q + 2 * k2]) * p.scale, __uint_as_float(r[8 * q + 2 * k2 + 1]) * p.scale);
            o[k2] = *reinterpret_cast<uint32_t*>(&hh);
          }
          *reinterpret_cast<uint4*>(op + c * 32 + q * 8) = make_uint4(o[0], o[1], o[2], o[3]);
        }
      }
    }
  }

  fence_before();
  __syncthreads();
  if (*abort_flag) {
    const uint64_t t0 = gtimer();
    while (gtimer() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 9) {
    fence_after();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

// ---- dK, dV: one CTA per (key tile, KV head, batch); loops over the query heads of the group and the query
// tiles at or after the key tile.  S = Q K^T and dP = dO V^T are computed as in the dQ kernel (a thread owns a
// query row, so its log-sum-exp and D are scalars); P and dS are stored [query][key] and the products
// dV += P^T dO, dK += dS^T Q read them transposed as MN-major A operands, with dO and Q as MN-major B operands.
template <int HD>
struct DkvCfg {
  static constexpr int ATOMS = HD / 64;
  static constexpr int TILE_BYTES = 128 * HD * 2;
  static constexpr int Q_STAGES = (HD <= 64) ? 3 : 1;
  // With more than one Q / dO stage the scores of tile i + 1 are issued as soon as the softmax warps have read those of
  // tile i out of tensor memory, so the two score products leave the per-tile dependency chain.
  static constexpr bool EARLY_SCORES = Q_STAGES >= 2;
  static constexpr int PT_BYTES = 128 * 128 * 2;
  static constexpr int SMEM_BYTES = 2 * TILE_BYTES + Q_STAGES * 2 * TILE_BYTES + 2 * PT_BYTES + 2 * 2 * 128 * 4 + 1024 + 256;
  static constexpr int TMEM_COLS = 512;
  static constexpr uint32_t IDESC_S = make_idesc(128, 128, false, false);
  static constexpr uint32_t IDESC_DKV = make_idesc(128, HD, true, true);   // A = P / dS read transposed (MN-major)
};

template <int HD>
__global__ void __launch_bounds__(320)
attn_bwd_dkv_kernel(const __grid_constant__ CUtensorMap tmap_qkv, const __grid_constant__ CUtensorMap tmap_do,
                    const AttnBwdParams p) {
  using C = DkvCfg<HD>;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* k_s = smem;
  unsigned char* v_s = k_s + C::TILE_BYTES;
  unsigned char* qdo_s = v_s + C::TILE_BYTES;                       // [stage][Q | dO]
  unsigned char* pt_s = qdo_s + C::Q_STAGES * 2 * C::TILE_BYTES;
  unsigned char* dst_s = pt_s + C::PT_BYTES;
  float* vec_s = reinterpret_cast<float*>(dst_s + C::PT_BYTES);     // [2 parities][lse | D][128]
  uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<unsigned char*>(vec_s) + 2 * 2 * 128 * 4);
  uint64_t* kv_full = bars;
  uint64_t* qdo_full = bars + 1;                                    // [3]
  uint64_t* qdo_empty = bars + 4;                                   // [3]
  uint64_t* st_full = bars + 7;
  uint64_t* pt_ready = bars + 8;
  uint64_t* dkv_done = bars + 9;
  uint64_t* st_free = bars + 10;                                    // the softmax warps hold S and dP in registers
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 11);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kj = blockIdx.x;                                        // key tile (small index = most work, runs first)
  const int g = blockIdx.y, b = blockIdx.z;
  const int rep = p.Hq / p.Hkv;
  const int nq = p.S / 128;
  const int per_head = nq - kj;                                     // query tiles kj..nq-1
  const int niter = rep * per_head;
  const int krow0 = b * p.S + kj * 128;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int i = 0; i < 3; ++i) { mbar_init(&qdo_full[i], 1); mbar_init(&qdo_empty[i], 1); }
    mbar_init(st_full, 1);
    mbar_init(pt_ready, 8);
    mbar_init(dkv_done, 1);
    mbar_init(st_free, 8);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 9) tmem_alloc(tmem_slot, C::TMEM_COLS);
  fence_before();
  __syncthreads();
  fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tST = tmem_base, tDPT = tmem_base + 128, tDV = tmem_base + 256, tDK = tmem_base + 256 + HD;

  if (warp == 8) {
    if (lane == 0) {
      mbar_expect_tx(kv_full, 2 * C::TILE_BYTES);
#pragma unroll
      for (int a = 0; a < C::ATOMS; ++a) {
        tma_load_2d(k_s + a * 16384, &tmap_qkv, kv_full, (p.Hq + g) * HD + a * 64, krow0);
        tma_load_2d(v_s + a * 16384, &tmap_qkv, kv_full, (p.Hq + p.Hkv + g) * HD + a * 64, krow0);
      }
      for (int it = 0; it < niter; ++it) {
        const int h = g * rep + it / per_head, qi = kj + it % per_head;
        const int st = it % C::Q_STAGES;
        const uint32_t ph = (it / C::Q_STAGES) & 1;
        if (!mbar_wait(&qdo_empty[st], ph ^ 1, abort_flag, 21, &g_attn_error)) break;
        unsigned char* q_s = qdo_s + st * 2 * C::TILE_BYTES;
        unsigned char* do_s = q_s + C::TILE_BYTES;
        mbar_expect_tx(&qdo_full[st], 2 * C::TILE_BYTES);
        const int qrow = b * p.S + qi * 128;
#pragma unroll
        for (int a = 0; a < C::ATOMS; ++a) {
          tma_load_2d(q_s + a * 16384, &tmap_qkv, &qdo_full[st], h * HD + a * 64, qrow);
          tma_load_2d(do_s + a * 16384, &tmap_do, &qdo_full[st], h * HD + a * 64, qrow);
        }
      }
    }
  } else if (warp == 9) {
    if (lane == 0) {
      bool ok = mbar_wait(kv_full, 0, abort_flag, 22, &g_attn_error);
      const uint32_t ka = smem_u32(k_s), va = smem_u32(v_s), pta = smem_u32(pt_s), dsta = smem_u32(dst_s);
      // S = Q K^T and dP = dO V^T of tile `t` into tensor memory
      auto issue_scores = [&](int t) -> bool {
        const int st = t % C::Q_STAGES;
        const uint32_t ph = (t / C::Q_STAGES) & 1;
        if (!mbar_wait(&qdo_full[st], ph, abort_flag, 23, &g_attn_error)) return false;
        fence_after();
        const uint32_t qa = smem_u32(qdo_s + st * 2 * C::TILE_BYTES), doa = qa + C::TILE_BYTES;
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;
          umma_bf16(tST, make_desc(qa + off, 16, 1024), make_desc(ka + off, 16, 1024), C::IDESC_S, kk > 0 ? 1u : 0u);
        }
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;
          umma_bf16(tDPT, make_desc(doa + off, 16, 1024), make_desc(va + off, 16, 1024), C::IDESC_S, kk > 0 ? 1u : 0u);
        }
        umma_commit(st_full);
        return true;
      };
      if (C::EARLY_SCORES && ok && niter > 0) ok = issue_scores(0);
      for (int it = 0; it < niter && ok; ++it) {
        const int st = it % C::Q_STAGES;
        if (!C::EARLY_SCORES) {
          if (!issue_scores(it)) { ok = false; break; }
        } else if (it + 1 < niter) {
          // the scores of the next tile, as soon as the softmax warps have taken this tile's out of tensor memory
          if (!mbar_wait(st_free, it & 1, abort_flag, 28, &g_attn_error)) { ok = false; break; }
          fence_after();
          if (!issue_scores(it + 1)) { ok = false; break; }
        }
        const uint32_t qa = smem_u32(qdo_s + st * 2 * C::TILE_BYTES), doa = qa + C::TILE_BYTES;
        if (!mbar_wait(pt_ready, it & 1, abort_flag, 24, &g_attn_error)) { ok = false; break; }
        fence_after();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          // P is stored [query row][key] (as the dQ kernel stores dS); read as an MN-major A operand it is P^T:
          // M = keys (two 64-key groups 16 KB apart), K = queries (16 rows of 128 bytes per step)
          umma_bf16(tDV, make_desc(pta + kk * 2048, 16384, 1024), make_desc(doa + kk * 2048, 16384, 1024), C::IDESC_DKV,
                    (it > 0 || kk > 0) ? 1u : 0u);
        }
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          umma_bf16(tDK, make_desc(dsta + kk * 2048, 16384, 1024), make_desc(qa + kk * 2048, 16384, 1024), C::IDESC_DKV,
                    (it > 0 || kk > 0) ? 1u : 0u);
        }
        umma_commit(dkv_done);
        umma_commit(&qdo_empty[st]);
      }
    }
  } else {
    const int row = (warp & 3) * 32 + lane;                         // query row in the loop, key row in the epilogue
    const int hf = warp >> 2;                                       // which 64-key half of the score columns
    const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
    bool ok = true;
    for (int it = 0; it < niter && ok; ++it) {
      const int h = g * rep + it / per_head, qi = kj + it % per_head;
      // inside the loop a thread owns QUERY row `row` of tile qi (scores are computed as in the dQ kernel), so its
      // softmax statistics are two scalars
      const size_t vec = ((size_t)b * p.Hq + h) * p.S + qi * 128 + row;
      const float nl = -p.lse2[vec], Dr = p.D[vec];
      if (!mbar_wait(st_full, it & 1, abort_flag, 25, &g_attn_error)) { ok = false; break; }
      fence_after();
      const bool diag = (qi == kj);
      const float cs = p.scale_log2;
      {
        uint32_t sa[32], sb[32], da[32], db[32];
        tmem_ld32_nowait(tST + lane_addr + hf * 64, sa);
        tmem_ld32_nowait(tST + lane_addr + hf * 64 + 32, sb);
        tmem_ld32_nowait(tDPT + lane_addr + hf * 64, da);
        tmem_ld32_nowait(tDPT + lane_addr + hf * 64 + 32, db);
        tmem_wait_ld();
        if (C::EARLY_SCORES) {                                     // S and dP are in registers: the next tile's may be issued
          fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(st_free);
        }
        if (diag) {                                                // causal: key column beyond the query row
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            if (hf * 64 + i > row) sa[i] = 0xff800000u;
            if (hf * 64 + 32 + i > row) sb[i] = 0xff800000u;
          }
        }
        // P and dS of this tile in registers first: the shared-memory copies of the previous tile are still being read
        // by its dV / dK products, which finish meanwhile
        uint32_t pk0[16], dk0[16], pk1[16], dk1[16];
#define ZEN_DKV_CHUNK(SS, DD, PK, DK)                                                                   \
        _Pragma("unroll") for (int i = 0; i < 32; i += 2) {                                             \
          const float p0 = ex2f(fmaf(__uint_as_float(SS[i]), cs, nl));                                  \
          const float p1 = ex2f(fmaf(__uint_as_float(SS[i + 1]), cs, nl));                              \
          PK[i >> 1] = pack_bf16(p0, p1);                                                               \
          DK[i >> 1] = pack_bf16(p0 * (__uint_as_float(DD[i]) - Dr), p1 * (__uint_as_float(DD[i + 1]) - Dr)); \
        }
        ZEN_DKV_CHUNK(sa, da, pk0, dk0)
        ZEN_DKV_CHUNK(sb, db, pk1, dk1)
#undef ZEN_DKV_CHUNK
        if (it > 0 && !mbar_wait(dkv_done, (it - 1) & 1, abort_flag, 26, &g_attn_error)) { ok = false; break; }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const uint32_t off0 = hf * 16384 + swz128(row, q * 8), off1 = hf * 16384 + swz128(row, 32 + q * 8);
          *reinterpret_cast<uint4*>(pt_s + off0) = make_uint4(pk0[4 * q], pk0[4 * q + 1], pk0[4 * q + 2], pk0[4 * q + 3]);
          *reinterpret_cast<uint4*>(dst_s + off0) = make_uint4(dk0[4 * q], dk0[4 * q + 1], dk0[4 * q + 2], dk0[4 * q + 3]);
          *reinterpret_cast<uint4*>(pt_s + off1) = make_uint4(pk1[4 * q], pk1[4 * q + 1], pk1[4 * q + 2], pk1[4 * q + 3]);
          *reinterpret_cast<uint4*>(dst_s + off1) = make_uint4(dk1[4 * q], dk1[4 * q + 1], dk1[4 * q + 2], dk1[4 * q + 3]);
        }
      }
      fence_before();
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(pt_ready);
    }
    if (ok && mbar_wait(dkv_done, (niter - 1) & 1, abort_flag, 27, &g_attn_error)) {
      fence_after();
      __nv_bfloat16* dvp = p.dqkv + (size_t)(krow0 + row) * p.ld_dqkv + (p.Hq + p.Hkv + g) * HD;
      __nv_bfloat16* dkp = p.dqkv + (size_t)(krow0 + row) * p.ld_dqkv + (p.Hq + g) * HD;
#pragma unroll 1
      for (int c = hf * (HD / 64); c < (hf + 1) * (HD / 64); ++c) {
        uint32_t r[32], r2[32];
        tmem_ld32(tDV + lane_addr + c * 32, r);
        tmem_ld32(tDK + lane_addr + c * 32, r2);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          uint32_t o[4], o2[4];
#pragma unroll
          for (int k2 = 0; k2 < 4; ++k2) {
            __nv_bfloat162 hv = __floats2bfloat162_rn(__uint_as_float(r[8 * q + 2 * k2]), __uint_as_float(r[8 * q + 2 * k2 + 1]));
            __nv_bfloat162 hk = __floats2bfloat162_rn(__uint_as_float(r2[8 * q + 2 * k2]) * p.scale, __uint_as_float(r2[8 * q + 2 * k2 + 1]) * p.scale);
            o[k2] = *reinterpret_cast<uint32_t*>(&hv);
            o2[k2] = *reinterpret_cast<uint32_t*>(&hk);
          }
          *reinterpret_cast<uint4*>(dvp + c * 32 + q * 8) = make_uint4(o[0], o[1], o[2], o[3]);
          *reinterpret_cast<uint4*>(dkp + c * 32 + q * 8) = make_uint4(o2[0], o2[1], o2[2], o2[3]);
        }
      }
    }
  }

  fence_before();
  __syncthreads();
  if (*abort_flag) {
    const uint64_t t0 = gtimer();
    while (gtimer() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 9) {
    fence_after();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

// ---- head_dim 256 backward.  The accumulators of dK and dV alone would fill tensor memory (2 x 256 columns) and a
// 128-row tile of each of Q, K, V, dO would overflow shared memory, so the work is cut differently: one kernel
// template, run in three modes, always with a RESIDENT 128-row operand pair and a STREAMED side in 64-row tiles:
//
//   mode     resident (128 rows)   streamed (64 rows)   S' [128 x 64]        weights W'        accumulator [128 x 256]
//   BWD_DQ   Q, dO  (query tile)   K, V  (key tiles)     Q K^T, dP = dO V^T   dS  (row stats)   dQ += dS K
//   BWD_DK   K, V   (key tile)     Q, dO (query tiles)   K Q^T, dP' = V dO^T  dS^T (col stats)  dK += dS^T Q
//   BWD_DV   K      (key tile)     Q, dO (query tiles)   K Q^T                P^T (col stats)   dV += P^T dO
//
// A softmax thread owns one resident row; W' is written to shared memory as a K-major [128][64] operand and the
// streamed tile serves as the MN-major B operand of the accumulating product.  Tensor memory: S' 64 + dP' 64 +
// accumulator 256 columns.  The scores are computed in each of the three launches (3 x the exponentials of a fused
// kernel), which is the price of fitting hd = 256 on chip.
enum { BWD_DQ = 0, BWD_DK = 1, BWD_DV = 2 };

struct Bwd256Cfg {
  static constexpr int HD = 256;
  static constexpr int RES_BYTES = 128 * HD * 2;        // 64 KB: four [128][64] atoms
  static constexpr int STR_BYTES = 64 * HD * 2;         // 32 KB: four [64][64] atoms
  static constexpr int W_BYTES = 128 * 64 * 2;
  static constexpr int SMEM_BYTES = 2 * RES_BYTES + 2 * STR_BYTES + W_BYTES + 512 + 1024 + 256;
  static constexpr int TMEM_COLS = 512;
  static constexpr uint32_t IDESC_S = make_idesc(128, 64, false, false);
  static constexpr uint32_t IDESC_ACC = make_idesc(128, 256, false, true);
};

template <int MODE>
__global__ void __launch_bounds__(320)
attn_bwd256_kernel(const __grid_constant__ CUtensorMap tmap_qkv128, const __grid_constant__ CUtensorMap tmap_do128,
                   const __grid_constant__ CUtensorMap tmap_qkv64, const __grid_constant__ CUtensorMap tmap_do64,
                   const AttnBwdParams p) {
  using C = Bwd256Cfg;
  constexpr int HD = C::HD;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* r1_s = smem;
  unsigned char* r2_s = r1_s + C::RES_BYTES;
  unsigned char* t1_s = r2_s + C::RES_BYTES;
  unsigned char* t2_s = t1_s + C::STR_BYTES;
  unsigned char* w_s = t2_s + C::STR_BYTES;
  float* stats_s = reinterpret_cast<float*>(w_s + C::W_BYTES);      // [lse | D][64] of the streamed queries (dK / dV)
  uint64_t* bars = reinterpret_cast<uint64_t*>(w_s + C::W_BYTES + 512);
  uint64_t* r_full = bars;
  uint64_t* t_full = bars + 1;
  uint64_t* t_empty = bars + 2;
  uint64_t* sdp_full = bars + 3;
  uint64_t* w_ready = bars + 4;
  uint64_t* acc_done = bars + 5;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 6);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.z;
  const int rep = p.Hq / p.Hkv;
  // resident tile index (heavy tiles first), head of the resident operand, and the iteration space
  const int ri = (MODE == BWD_DQ) ? (int)(gridDim.x - 1 - blockIdx.x) : (int)blockIdx.x;
  const int hs = (MODE == BWD_DQ) ? 1 : p.hsplit;
  const int hres = (MODE == BWD_DQ) ? (int)blockIdx.y : (int)blockIdx.y / hs;   // query head (dQ) or KV head (dK / dV)
  const int hpart = (MODE == BWD_DQ) ? 0 : (int)blockIdx.y % hs;
  const int g = (MODE == BWD_DQ) ? hres / rep : hres;
  const int reph = rep / hs;                                 // query heads this CTA walks (dK / dV)
  const int h0 = g * rep + hpart * reph;
  const int nq64 = p.S / 64;
  const int per_head = (MODE == BWD_DQ) ? 2 * ri + 2 : nq64 - 2 * ri;   // streamed tiles per head
  const int niter = (MODE == BWD_DQ) ? per_head : reph * per_head;
  const int rrow0 = b * p.S + ri * 128;

  if (threadIdx.x == 0) {
    mbar_init(r_full, 1);
    mbar_init(t_full, 1);
    mbar_init(t_empty, 1);
    mbar_init(sdp_full, 1);
    mbar_init(w_ready, 8);
    mbar_init(acc_done, 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 9) tmem_alloc(tmem_slot, C::TMEM_COLS);
  fence_before();
  __syncthreads();
  fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS = tmem_base, tDP = tmem_base + 64, tACC = tmem_base + 128;

  if (warp == 8) {
    if (lane == 0) {
      // ---------------------------------------------------------------- TMA producer
      mbar_expect_tx(r_full, (MODE == BWD_DV ? 1 : 2) * C::RES_BYTES);
#pragma unroll
      for (int a = 0; a < 4; ++a) {
        if (MODE == BWD_DQ) {
          tma_load_2d(r1_s + a * 16384, &tmap_qkv128, r_full, hres * HD + a * 64, rrow0);
          tma_load_2d(r2_s + a * 16384, &tmap_do128, r_full, hres * HD + a * 64, rrow0);
        } else {
          tma_load_2d(r1_s + a * 16384, &tmap_qkv128, r_full, (p.Hq + g) * HD + a * 64, rrow0);
          if (MODE == BWD_DK) tma_load_2d(r2_s + a * 16384, &tmap_qkv128, r_full, (p.Hq + p.Hkv + g) * HD + a * 64, rrow0);
        }
      }
      for (int it = 0; it < niter; ++it) {
        if (!mbar_wait(t_empty, (it & 1) ^ 1, abort_flag, 31, &g_attn_error)) break;
        mbar_expect_tx(t_full, 2 * C::STR_BYTES + (MODE == BWD_DQ ? 0 : 512));
        if (MODE == BWD_DQ) {
          const int krow = b * p.S + it * 64;
#pragma unroll
          for (int a = 0; a < 4; ++a) {
            tma_load_2d(t1_s + a * 8192, &tmap_qkv64, t_full, (p.Hq + g) * HD + a * 64, krow);
            tma_load_2d(t2_s + a * 8192, &tmap_qkv64, t_full, (p.Hq + p.Hkv + g) * HD + a * 64, krow);
          }
        } else {
          const int h = h0 + it / per_head, t = 2 * ri + it % per_head;
          const int qrow = b * p.S + t * 64;
#pragma unroll
          for (int a = 0; a < 4; ++a) {
            tma_load_2d(t1_s + a * 8192, &tmap_qkv64, t_full, h * HD + a * 64, qrow);
            tma_load_2d(t2_s + a * 8192, &tmap_do64, t_full, h * HD + a * 64, qrow);
          }
          // log-sum-exp and D of these 64 queries ride on the same barrier (256 bytes each)
          const size_t sv = ((size_t)b * p.Hq + h) * p.S + t * 64;
          bulk_load_1d(stats_s, p.lse2 + sv, 256, t_full);
          bulk_load_1d(stats_s + 64, p.D + sv, 256, t_full);
        }
      }
    }
  } else if (warp == 9) {
    if (lane == 0) {
      // ---------------------------------------------------------------- MMA issuer
      bool ok = mbar_wait(r_full, 0, abort_flag, 32, &g_attn_error);
      const uint32_t r1a = smem_u32(r1_s), r2a = smem_u32(r2_s), t1a = smem_u32(t1_s), t2a = smem_u32(t2_s), wa = smem_u32(w_s);
      for (int it = 0; it < niter && ok; ++it) {
        if (!mbar_wait(t_full, it & 1, abort_flag, 33, &g_attn_error)) { ok = false; break; }
        fence_after();
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t roff = (kk >> 2) * 16384 + (kk & 3) * 32, toff = (kk >> 2) * 8192 + (kk & 3) * 32;
          umma_bf16(tS, make_desc(r1a + roff, 16, 1024), make_desc(t1a + toff, 16, 1024), C::IDESC_S, kk > 0 ? 1u : 0u);
        }
        if (MODE != BWD_DV) {
#pragma unroll
          for (int kk = 0; kk < HD / 16; ++kk) {
            const uint32_t roff = (kk >> 2) * 16384 + (kk & 3) * 32, toff = (kk >> 2) * 8192 + (kk & 3) * 32;
            umma_bf16(tDP, make_desc(r2a + roff, 16, 1024), make_desc(t2a + toff, 16, 1024), C::IDESC_S, kk > 0 ? 1u : 0u);
          }
        }
        umma_commit(sdp_full);
        if (!mbar_wait(w_ready, it & 1, abort_flag, 34, &g_attn_error)) { ok = false; break; }
        fence_after();
        const uint32_t tba = (MODE == BWD_DV) ? t2a : t1a;    // streamed tile as the MN-major B operand
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          umma_bf16(tACC, make_desc(wa + kk * 32, 16, 1024), make_desc(tba + kk * 2048, 8192, 1024), C::IDESC_ACC,
                    (it > 0 || kk > 0) ? 1u : 0u);
        umma_commit(acc_done);
        umma_commit(t_empty);
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax warps: thread = resident row,
    // warps w and w + 4 split the 64 streamed columns in halves of 32
    const int row = (warp & 3) * 32 + lane;
    const int hf = warp >> 2;
    const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
    const float cs = p.scale_log2;
    float nl_row = 0.f, d_row = 0.f;
    if (MODE == BWD_DQ) {
      const size_t vec = ((size_t)b * p.Hq + hres) * p.S + ri * 128 + row;
      nl_row = -p.lse2[vec];
      d_row = p.D[vec];
    }
    bool ok = true;
    for (int it = 0; it < niter && ok; ++it) {
      const int h = (MODE == BWD_DQ) ? hres : h0 + it / per_head;
      const int t = (MODE == BWD_DQ) ? it : 2 * ri + it % per_head;         // streamed 64-row tile index
      if (!mbar_wait(sdp_full, it & 1, abort_flag, 35, &g_attn_error)) { ok = false; break; }
      if (it > 0 && !mbar_wait(acc_done, (it - 1) & 1, abort_flag, 36, &g_attn_error)) { ok = false; break; }
      fence_after();
      uint32_t sa[32], da[32];
      tmem_ld32_nowait(tS + lane_addr + hf * 32, sa);
      if (MODE != BWD_DV) tmem_ld32_nowait(tDP + lane_addr + hf * 32, da);
      tmem_wait_ld();
      const bool capped = p.cap_a != 0.f;
      if (capped) {
        const float a = p.cap_a, ia = 1.f / p.cap_a;
#pragma unroll
        for (int i = 0; i < 32; ++i) sa[i] = softcap_bits(sa[i], a, ia);
      }
      // causal mask: key index against query index (resident row is the query in dQ, the key otherwise)
      const int res_idx = ri * 128 + row, str0 = t * 64 + hf * 32;
      const bool need_mask = (MODE == BWD_DQ) ? (str0 + 31 > ri * 128) : (str0 < ri * 128 + 128);
      if (need_mask) {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const bool dead = (MODE == BWD_DQ) ? (str0 + i > res_idx) : (res_idx > str0 + i);
          if (dead) sa[i] = 0xff800000u;
        }
      }
      if (MODE != BWD_DQ) {               // the statistics arrived with the tile; this wait is over already (acquire)
        if (!mbar_wait(t_full, it & 1, abort_flag, 38, &g_attn_error)) { ok = false; break; }
      }
      const float* lse_c = stats_s + hf * 32;                               // per-column statistics (dK / dV)
      const float* d_c = lse_c + 64;
      (void)h;
      uint32_t pk[16];
#pragma unroll
      for (int i = 0; i < 32; i += 2) {
        float w0, w1;
        if (MODE == BWD_DQ) {
          const float p0 = ex2f(fmaf(__uint_as_float(sa[i]), cs, nl_row));
          const float p1 = ex2f(fmaf(__uint_as_float(sa[i + 1]), cs, nl_row));
          w0 = p0 * (__uint_as_float(da[i]) - d_row);
          w1 = p1 * (__uint_as_float(da[i + 1]) - d_row);
        } else {
          const float p0 = ex2f(fmaf(__uint_as_float(sa[i]), cs, -lse_c[i]));
          const float p1 = ex2f(fmaf(__uint_as_float(sa[i + 1]), cs, -lse_c[i + 1]));
          if (MODE == BWD_DK) {
            w0 = p0 * (__uint_as_float(da[i]) - d_c[i]);
            w1 = p1 * (__uint_as_float(da[i + 1]) - d_c[i + 1]);
          } else {
            w0 = p0;
            w1 = p1;
          }
        }
        if (capped && MODE != BWD_DV) {
          // chain rule through cap * tanh(.): 1 - tanh^2, with tanh = capped score * a (masked entries: factor 0)
          const float t0 = fminf(fabsf(__uint_as_float(sa[i]) * p.cap_a), 1.f), t1 = fminf(fabsf(__uint_as_float(sa[i + 1]) * p.cap_a), 1.f);
          w0 *= 1.f - t0 * t0;
          w1 *= 1.f - t1 * t1;
        }
        pk[i >> 1] = pack_bf16(w0, w1);
      }
#pragma unroll
      for (int q = 0; q < 4; ++q)
        *reinterpret_cast<uint4*>(w_s + swz128(row, hf * 32 + q * 8)) = make_uint4(pk[4 * q], pk[4 * q + 1], pk[4 * q + 2], pk[4 * q + 3]);
      fence_before();
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(w_ready);
    }
    if (ok && mbar_wait(acc_done, (niter - 1) & 1, abort_flag, 37, &g_attn_error)) {
      fence_after();
      const int col_base = (MODE == BWD_DQ) ? hres * HD : (MODE == BWD_DK ? (p.Hq + g) * HD : (p.Hq + p.Hkv + g) * HD);
      const float osc = (MODE == BWD_DV) ? 1.f : p.scale;
      __nv_bfloat16* op = p.dqkv + (size_t)(rrow0 + row) * p.ld_dqkv + col_base;
      float* pp = nullptr;
      if (MODE != BWD_DQ && hs > 1) {
        const size_t rows_all = (size_t)p.B * p.S, wid = (size_t)p.Hkv * HD;
        pp = p.part + (MODE == BWD_DV ? (size_t)hs * rows_all * wid : 0) + ((size_t)hpart * rows_all + rrow0 + row) * wid + (size_t)g * HD;
      }
#pragma unroll 1
      for (int c = hf * 4; c < hf * 4 + 4; ++c) {
        uint32_t r[32];
        tmem_ld32(tACC + lane_addr + c * 32, r);
        if (pp) {                                            // several CTAs share this KV head: fp32 partials, summed later
#pragma unroll
          for (int q = 0; q < 8; ++q)
            *reinterpret_cast<float4*>(pp + c * 32 + q * 4) = make_float4(__uint_as_float(r[4 * q]) * osc, __uint_as_float(r[4 * q + 1]) * osc,
                                                                        __uint_as_float(r[4 * q + 2]) * osc, __uint_as_float(r[4 * q + 3]) * osc);
          continue;
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          uint32_t o[4];
#pragma unroll
          for (int k2 = 0; k2 < 4; ++k2)
            o[k2] = pack_bf16(__uint_as_float(r[8 * q + 2 * k2]) * osc, __uint_as_float(r[8 * q + 2 * k2 + 1]) * osc);
          *reinterpret_cast<uint4*>(op + c * 32 + q * 8) = make_uint4(o[0], o[1], o[2], o[3]);
        }
      }
    }
  }

  fence_before();
  __syncthreads();
  if (*abort_flag) {
    const uint64_t t0 = gtimer();
    while (gtimer() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 9) {
    fence_after();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

// ---- head_dim 64 backward, same resident / streamed scheme as the hd = 256 kernel but small enough for TWO CTAs per
// SM (96 KB of shared memory, 256 tensor-memory columns each), so that one CTA's softmax pass overlaps the other's MMAs
// and prologue, with a two-stage ring for the streamed tiles.  Modes: RS_DQ (resident Q, dO; streamed K, V; dQ += dS K)
// and RS_DKV (resident K, V; streamed Q, dO; dK += dS^T Q and dV += P^T dO from one pass over the scores:
// S' 64 + dP' 64 + dK 64 + dV 64 columns).
enum { RS_DQ = 0, RS_DKV = 1 };

struct Rs64Cfg {
  static constexpr int HD = 64;
  static constexpr int STAGES = 2;
  static constexpr int RES_BYTES = 128 * HD * 2;        // one [128][64] atom
  static constexpr int STR_BYTES = 64 * HD * 2;         // one [64][64] atom
  static constexpr int W_BYTES = 128 * 64 * 2;
  static constexpr int SMEM_BYTES = 2 * RES_BYTES + STAGES * 2 * STR_BYTES + 2 * W_BYTES + STAGES * 512 + 1024 + 256;
  static constexpr int TMEM_COLS = 256;
  // Issuing the next tile's scores ahead of this tile's accumulating products (as the 128 x 128 kernels do) measured
  // 3 % slower here: the second CTA of the SM already fills the gaps, and the two-stage ring leaves no tile to run ahead on.
  static constexpr bool EARLY_SCORES = false;
  static constexpr uint32_t IDESC_S = make_idesc(128, 64, false, false);
  static constexpr uint32_t IDESC_ACC = make_idesc(128, 64, false, true);
};

template <int MODE>
__global__ void __launch_bounds__(320, 2)
attn_bwd64_kernel(const __grid_constant__ CUtensorMap tmap_qkv128, const __grid_constant__ CUtensorMap tmap_do128,
                  const __grid_constant__ CUtensorMap tmap_qkv64, const __grid_constant__ CUtensorMap tmap_do64,
                  const __grid_constant__ CUtensorMap tmap_o128, const AttnBwdParams p) {
  using C = Rs64Cfg;
  constexpr int HD = C::HD;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* r1_s = smem;
  unsigned char* r2_s = r1_s + C::RES_BYTES;
  unsigned char* t_s = r2_s + C::RES_BYTES;                       // [stage][T1 | T2]
  unsigned char* w1_s = t_s + C::STAGES * 2 * C::STR_BYTES;       // dS (dQ mode) or dS^T
  unsigned char* w2_s = w1_s + C::W_BYTES;                        // P^T (dK/dV mode)
  float* stats_s = reinterpret_cast<float*>(w2_s + C::W_BYTES);   // [stage][lse | D][64]: statistics of the streamed queries
  uint64_t* bars = reinterpret_cast<uint64_t*>(w2_s + C::W_BYTES + C::STAGES * 512);
  uint64_t* r_full = bars;
  uint64_t* t_full = bars + 1;                                    // [2]
  uint64_t* t_empty = bars + 3;                                   // [2]
  uint64_t* sdp_full = bars + 5;
  uint64_t* w_ready = bars + 6;
  uint64_t* acc_done = bars + 7;
  uint64_t* s_free = bars + 8;                                    // the softmax warps hold S' and dP' in registers
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 9);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.z;
  const int rep = p.Hq / p.Hkv;
  const int ri = (MODE == RS_DQ) ? (int)(gridDim.x - 1 - blockIdx.x) : (int)blockIdx.x;
  const int hres = blockIdx.y;
  const int g = (MODE == RS_DQ) ? hres / rep : hres;
  const int nq64 = p.S / 64;
  const int per_head = (MODE == RS_DQ) ? 2 * ri + 2 : nq64 - 2 * ri;
  const int niter = (MODE == RS_DQ) ? per_head : rep * per_head;
  const int rrow0 = b * p.S + ri * 128;

  if (threadIdx.x == 0) {
    mbar_init(r_full, 1);
    for (int i = 0; i < 2; ++i) { mbar_init(&t_full[i], 1); mbar_init(&t_empty[i], 1); }
    mbar_init(sdp_full, 1);
    mbar_init(w_ready, 8);
    mbar_init(acc_done, 1);
    mbar_init(s_free, 8);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 9) tmem_alloc(tmem_slot, C::TMEM_COLS);
  fence_before();
  __syncthreads();
  fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS = tmem_base, tDP = tmem_base + 64, tA1 = tmem_base + 128, tA2 = tmem_base + 192;

  if (warp == 8) {
    if (lane == 0) {
      mbar_expect_tx(r_full, (MODE == RS_DQ ? 3 : 2) * C::RES_BYTES);
      if (MODE == RS_DQ) {
        tma_load_2d(r1_s, &tmap_qkv128, r_full, hres * HD, rrow0);
        tma_load_2d(r2_s, &tmap_do128, r_full, hres * HD, rrow0);
        tma_load_2d(w2_s, &tmap_o128, r_full, hres * HD, rrow0);     // O tile: D = rowsum(dO * O) is computed here
      } else {
        tma_load_2d(r1_s, &tmap_qkv128, r_full, (p.Hq + g) * HD, rrow0);
        tma_load_2d(r2_s, &tmap_qkv128, r_full, (p.Hq + p.Hkv + g) * HD, rrow0);
      }
      for (int it = 0; it < niter; ++it) {
        const int st = it % C::STAGES;
        const uint32_t ph = (it / C::STAGES) & 1;
        if (!mbar_wait(&t_empty[st], ph ^ 1, abort_flag, 41, &g_attn_error)) break;
        unsigned char* t1 = t_s + st * 2 * C::STR_BYTES;
        unsigned char* t2 = t1 + C::STR_BYTES;
        mbar_expect_tx(&t_full[st], 2 * C::STR_BYTES + (MODE == RS_DKV ? 512 : 0));
        if (MODE == RS_DQ) {
          const int krow = b * p.S + it * 64;
          tma_load_2d(t1, &tmap_qkv64, &t_full[st], (p.Hq + g) * HD, krow);
          tma_load_2d(t2, &tmap_qkv64, &t_full[st], (p.Hq + p.Hkv + g) * HD, krow);
        } else {
          const int h = g * rep + it / per_head, t = 2 * ri + it % per_head;
          const int qrow = b * p.S + t * 64;
          tma_load_2d(t1, &tmap_qkv64, &t_full[st], h * HD, qrow);
          tma_load_2d(t2, &tmap_do64, &t_full[st], h * HD, qrow);
          // log-sum-exp and D of these 64 queries ride on the same barrier (256 bytes each)
          const size_t sv = ((size_t)b * p.Hq + h) * p.S + t * 64;
          bulk_load_1d(stats_s + st * 128, p.lse2 + sv, 256, &t_full[st]);
          bulk_load_1d(stats_s + st * 128 + 64, p.D + sv, 256, &t_full[st]);
        }
      }
    }
  } else if (warp == 9) {
    if (lane == 0) {
      bool ok = mbar_wait(r_full, 0, abort_flag, 42, &g_attn_error);
      const uint32_t r1a = smem_u32(r1_s), r2a = smem_u32(r2_s), w1a = smem_u32(w1_s), w2a = smem_u32(w2_s);
      // S' and dP' of streamed tile `t`
      auto issue_scores = [&](int t) -> bool {
        const int st = t % C::STAGES;
        const uint32_t ph = (t / C::STAGES) & 1;
        if (!mbar_wait(&t_full[st], ph, abort_flag, 43, &g_attn_error)) return false;
        fence_after();
        const uint32_t t1a = smem_u32(t_s + st * 2 * C::STR_BYTES), t2a = t1a + C::STR_BYTES;
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk)
          umma_bf16(tS, make_desc(r1a + kk * 32, 16, 1024), make_desc(t1a + kk * 32, 16, 1024), C::IDESC_S, kk > 0 ? 1u : 0u);
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk)
          umma_bf16(tDP, make_desc(r2a + kk * 32, 16, 1024), make_desc(t2a + kk * 32, 16, 1024), C::IDESC_S, kk > 0 ? 1u : 0u);
        umma_commit(sdp_full);
        return true;
      };
      if (C::EARLY_SCORES && ok && niter > 0) ok = issue_scores(0);
      for (int it = 0; it < niter && ok; ++it) {
        const int st = it % C::STAGES;
        if (!C::EARLY_SCORES) {
          if (!issue_scores(it)) { ok = false; break; }
        } else if (it + 1 < niter) {
          if (!mbar_wait(s_free, it & 1, abort_flag, 50, &g_attn_error)) { ok = false; break; }
          fence_after();
          if (!issue_scores(it + 1)) { ok = false; break; }
        }
        const uint32_t t1a = smem_u32(t_s + st * 2 * C::STR_BYTES), t2a = t1a + C::STR_BYTES;
        if (!mbar_wait(w_ready, it & 1, abort_flag, 44, &g_attn_error)) { ok = false; break; }
        fence_after();
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)           // dQ += dS K   or   dK += dS^T Q   (streamed tile 1 as MN-major B)
          umma_bf16(tA1, make_desc(w1a + kk * 32, 16, 1024), make_desc(t1a + kk * 2048, 8192, 1024), C::IDESC_ACC,
                    (it > 0 || kk > 0) ? 1u : 0u);
        if (MODE == RS_DKV) {
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)         // dV += P^T dO
            umma_bf16(tA2, make_desc(w2a + kk * 32, 16, 1024), make_desc(t2a + kk * 2048, 8192, 1024), C::IDESC_ACC,
                      (it > 0 || kk > 0) ? 1u : 0u);
        }
        umma_commit(acc_done);
        umma_commit(&t_empty[st]);
      }
    }
  } else {
    const int row = (warp & 3) * 32 + lane;
    const int hf = warp >> 2;
    const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
    const float cs = p.scale_log2;
    float nl_row = 0.f, d_row = 0.f;
    bool ok = true;
    if (MODE == RS_DQ) {
      const size_t vec = ((size_t)b * p.Hq + hres) * p.S + ri * 128 + row;
      nl_row = -p.lse2[vec];
      // D of this query row from the dO and O tiles in shared memory (both warps of the lane group compute it, one
      // stores it for the dK / dV kernel that runs after this one)
      ok = mbar_wait(r_full, 0, abort_flag, 48, &g_attn_error);
      if (ok) {
#pragma unroll
        for (int c8 = 0; c8 < 8; ++c8) {
          const uint4 x = *reinterpret_cast<const uint4*>(r2_s + swz128(row, c8 * 8));
          const uint4 y = *reinterpret_cast<const uint4*>(w2_s + swz128(row, c8 * 8));
          const uint32_t xw[4] = {x.x, x.y, x.z, x.w}, yw[4] = {y.x, y.y, y.z, y.w};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            d_row += __uint_as_float(xw[i] << 16) * __uint_as_float(yw[i] << 16);
            d_row += __uint_as_float(xw[i] & 0xffff0000u) * __uint_as_float(yw[i] & 0xffff0000u);
          }
        }
        if (hf == 0) const_cast<float*>(p.D)[vec] = d_row;
      }
    }
    for (int it = 0; it < niter && ok; ++it) {
      const int h = (MODE == RS_DQ) ? hres : g * rep + it / per_head;
      const int t = (MODE == RS_DQ) ? it : 2 * ri + it % per_head;
      if (!mbar_wait(sdp_full, it & 1, abort_flag, 45, &g_attn_error)) { ok = false; break; }
      fence_after();
      uint32_t sa[32], da[32];
      tmem_ld32_nowait(tS + lane_addr + hf * 32, sa);
      tmem_ld32_nowait(tDP + lane_addr + hf * 32, da);
      // the weights of the previous tile are still being read by its accumulating products: wait while the loads fly
      if (it > 0 && !mbar_wait(acc_done, (it - 1) & 1, abort_flag, 46, &g_attn_error)) { tmem_wait_ld(); ok = false; break; }
      tmem_wait_ld();
      if (C::EARLY_SCORES) {                                      // S' and dP' are in registers: the next tile's may be issued
        fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(s_free);
      }
      const int res_idx = ri * 128 + row, str0 = t * 64 + hf * 32;
      const bool need_mask = (MODE == RS_DQ) ? (str0 + 31 > ri * 128) : (str0 < ri * 128 + 128);
      if (need_mask) {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const bool dead = (MODE == RS_DQ) ? (str0 + i > res_idx) : (res_idx > str0 + i);
          if (dead) sa[i] = 0xff800000u;
        }
      }
      const int sst = it % C::STAGES;
      if (MODE != RS_DQ) {                // the statistics arrived with the tile; this wait is over already (acquire)
        if (!mbar_wait(&t_full[sst], (it / C::STAGES) & 1, abort_flag, 49, &g_attn_error)) { ok = false; break; }
      }
      const float* lse_c = stats_s + sst * 128 + hf * 32;
      const float* d_c = lse_c + 64;
      (void)h;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        uint32_t pk[4], dk[4];
        float lv[8], dv[8];
        if (MODE != RS_DQ) {              // statistics of the 8 streamed queries of this vector (same for every thread)
          const float4 l0 = *reinterpret_cast<const float4*>(lse_c + 8 * q), l1 = *reinterpret_cast<const float4*>(lse_c + 8 * q + 4);
          const float4 e0 = *reinterpret_cast<const float4*>(d_c + 8 * q), e1 = *reinterpret_cast<const float4*>(d_c + 8 * q + 4);
          lv[0] = l0.x; lv[1] = l0.y; lv[2] = l0.z; lv[3] = l0.w; lv[4] = l1.x; lv[5] = l1.y; lv[6] = l1.z; lv[7] = l1.w;
          dv[0] = e0.x; dv[1] = e0.y; dv[2] = e0.z; dv[3] = e0.w; dv[4] = e1.x; dv[5] = e1.y; dv[6] = e1.z; dv[7] = e1.w;
        }
#pragma unroll
        for (int k2 = 0; k2 < 4; ++k2) {
          const int i = 8 * q + 2 * k2;
          float p0, p1, w0, w1;
          if (MODE == RS_DQ) {
            p0 = ex2f(fmaf(__uint_as_float(sa[i]), cs, nl_row));
            p1 = ex2f(fmaf(__uint_as_float(sa[i + 1]), cs, nl_row));
            w0 = p0 * (__uint_as_float(da[i]) - d_row);
            w1 = p1 * (__uint_as_float(da[i + 1]) - d_row);
          } else {
            p0 = ex2f(fmaf(__uint_as_float(sa[i]), cs, -lv[2 * k2]));
            p1 = ex2f(fmaf(__uint_as_float(sa[i + 1]), cs, -lv[2 * k2 + 1]));
            w0 = p0 * (__uint_as_float(da[i]) - dv[2 * k2]);
            w1 = p1 * (__uint_as_float(da[i + 1]) - dv[2 * k2 + 1]);
          }
          dk[k2] = pack_bf16(w0, w1);
          pk[k2] = pack_bf16(p0, p1);
        }
        const uint32_t off = swz128(row, hf * 32 + q * 8);
        *reinterpret_cast<uint4*>(w1_s + off) = make_uint4(dk[0], dk[1], dk[2], dk[3]);
        if (MODE == RS_DKV) *reinterpret_cast<uint4*>(w2_s + off) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
      }
      fence_before();
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(w_ready);
    }
    if (ok && mbar_wait(acc_done, (niter - 1) & 1, abort_flag, 47, &g_attn_error)) {
      fence_after();
      // 64 accumulator columns = two chunks of 32: the two warps of a lane group take one chunk each
      uint32_t r[32], r2[32];
      tmem_ld32_nowait(tA1 + lane_addr + hf * 32, r);
      if (MODE == RS_DKV) tmem_ld32_nowait(tA2 + lane_addr + hf * 32, r2);
      tmem_wait_ld();
      const int col1 = (MODE == RS_DQ) ? hres * HD : (p.Hq + g) * HD;
      __nv_bfloat16* o1 = p.dqkv + (size_t)(rrow0 + row) * p.ld_dqkv + col1 + hf * 32;
      __nv_bfloat16* o2 = p.dqkv + (size_t)(rrow0 + row) * p.ld_dqkv + (p.Hq + p.Hkv + g) * HD + hf * 32;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        uint32_t a[4], c[4];
#pragma unroll
        for (int k2 = 0; k2 < 4; ++k2) {
          a[k2] = pack_bf16(__uint_as_float(r[8 * q + 2 * k2]) * p.scale, __uint_as_float(r[8 * q + 2 * k2 + 1]) * p.scale);
          if (MODE == RS_DKV) c[k2] = pack_bf16(__uint_as_float(r2[8 * q + 2 * k2]), __uint_as_float(r2[8 * q + 2 * k2 + 1]));
        }
        *reinterpret_cast<uint4*>(o1 + q * 8) = make_uint4(a[0], a[1], a[2], a[3]);
        if (MODE == RS_DKV) *reinterpret_cast<uint4*>(o2 + q * 8) = make_uint4(c[0], c[1], c[2], c[3]);
      }
    }
  }

  fence_before();
  __syncthreads();
  if (*abort_flag) {
    const uint64_t t0 = gtimer();
    while (gtimer() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 9) {
    fence_after();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

// dK and dV of the head-split hd = 256 backward: sum the hsplit fp32 partials in order, write bf16 into dqkv.
__global__ void __launch_bounds__(256)
attn_bwd256_reduce_kernel(const float* __restrict__ part, __nv_bfloat16* __restrict__ dqkv, int rows, int Hq, int Hkv,
                          int hsplit, int ld) {
  const size_t wid = (size_t)Hkv * 256, per = (size_t)rows * wid;
  const size_t nvec = 2 * per / 8;
  for (size_t v = (size_t)blockIdx.x * blockDim.x + threadIdx.x; v < nvec; v += (size_t)gridDim.x * blockDim.x) {
    const size_t e = v * 8;
    const int which = (int)(e / per);                      // 0 = dK, 1 = dV
    const size_t off = e % per;
    const size_t row = off / wid;
    const int col = (int)(off % wid);
    float a[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int sidx = 0; sidx < hsplit; ++sidx) {
      const float4* q = reinterpret_cast<const float4*>(part + ((size_t)which * hsplit + sidx) * per + off);
      const float4 x = __ldcs(q), y = __ldcs(q + 1);
      a[0] += x.x; a[1] += x.y; a[2] += x.z; a[3] += x.w; a[4] += y.x; a[5] += y.y; a[6] += y.z; a[7] += y.w;
    }
    __nv_bfloat16* dst = dqkv + row * ld + (size_t)(Hq + which * Hkv) * 256 + col;
    *reinterpret_cast<uint4*>(dst) = make_uint4(pack_bf16(a[0], a[1]), pack_bf16(a[2], a[3]), pack_bf16(a[4], a[5]), pack_bf16(a[6], a[7]));
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

// bf16 [rows, cols] row-major (row stride ld elements) with a {64, box_rows} box and 128-byte swizzle.
int attn_make_map(const void* ptr, uint64_t cols, uint64_t rows, uint64_t ld, CUtensorMap* out, uint32_t box_rows = 128) {
  EncodeTiledFn enc = attn_get_encode();
  if (!enc) return -10;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {64, box_rows};
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

int g_bwd64_variant = 2;       // 0: the 128 x 128 tile kernels; 1: two-CTAs-per-SM kernels with 64-row streamed tiles;
                               // 2: that dQ kernel with the 128 x 128 tile dK/dV kernel

extern "C" {

// Which head_dim 64 backward runs (see g_bwd64_variant); returns the previous choice.
int zen_attn_bwd64_variant(int v) {
  const int old = g_bwd64_variant;
  if (v >= 0 && v <= 2) g_bwd64_variant = v;
  return old;
}

// Causal attention forward.  qkv: bf16 [B*S, (Hq + 2*Hkv) * hd] with row stride ld_qkv (elements, multiple of 8,
// base 16-byte aligned); out: bf16 [B*S, Hq*hd] (row stride ld_out); lse2: fp32 [B, Hq, S].
// Supported: hd in {64, 128, 256}, S a multiple of 128, Hq a multiple of Hkv.
// softcap > 0: scores are soft-capped, cap * tanh(s * scale / cap), before the softmax (0 = none).
int zen_attn_fwd(const void* qkv, void* out, float* lse2, int B, int S, int Hq, int Hkv, int hd, int ld_qkv, int ld_out,
                 float scale, float softcap, void* stream) {
  if (S % 128 || Hq % Hkv || (hd != 64 && hd != 128 && hd != 256)) return -2;
  if ((ld_qkv % 8) || (ld_out % 8) || (reinterpret_cast<uintptr_t>(qkv) % 16) || (reinterpret_cast<uintptr_t>(out) % 16)) return -3;
  CUtensorMap tm;
  int rc = attn_make_map(qkv, (uint64_t)(Hq + 2 * Hkv) * hd, (uint64_t)B * S, (uint64_t)ld_qkv, &tm);
  if (rc) return rc;
  AttnParams p{(__nv_bfloat16*)out, lse2, B, S, Hq, Hkv, ld_out, scale * 1.4426950408889634f, softcap > 0.f ? scale / softcap : 0.f};
  cudaStream_t st = (cudaStream_t)stream;
  if (hd == 64) return launch_fwd<64>(tm, p, st);
  if (hd == 128) return launch_fwd<128>(tm, p, st);
  return launch_fwd<256>(tm, p, st);
}

// Causal attention backward.  dout / out: bf16 [B*S, Hq*hd] (row stride ld_o); lse2 from the forward; Dbuf: fp32
// scratch [B, Hq, S]; dqkv: bf16 [B*S, (Hq + 2*Hkv)*hd] (row stride ld_qkv), fully overwritten.  hd in {64, 128, 256}.
// part / hsplit (hd 256 only): with hsplit > 1 the query heads of a KV head are spread over hsplit CTAs whose fp32
// partial dK / dV go to `part` (2 * hsplit * B*S * Hkv*256 floats) and are summed by a last kernel; hsplit divides
// Hq / Hkv.  Pass hsplit <= 1 (part unused) to let one CTA walk all heads of its group.
// softcap > 0 (as in the forward) is taken by the head_dim 256 kernels only.
int zen_attn_bwd(const void* qkv, const void* out, const void* dout, const float* lse2, float* Dbuf, void* dqkv, int B,
                 int S, int Hq, int Hkv, int hd, int ld_qkv, int ld_o, float scale, float softcap, float* part, int hsplit,
                 void* stream) {
  if (S % 128 || Hq % Hkv || (hd != 64 && hd != 128 && hd != 256)) return -2;
  if (softcap > 0.f && hd != 256) return -9;
  if ((ld_qkv % 8) || (ld_o % 8) || (reinterpret_cast<uintptr_t>(qkv) % 16) || (reinterpret_cast<uintptr_t>(dout) % 16) ||
      (reinterpret_cast<uintptr_t>(dqkv) % 16) || (reinterpret_cast<uintptr_t>(out) % 16)) return -3;
  cudaStream_t st = (cudaStream_t)stream;
  CUtensorMap tq, tdo;
  int rc = attn_make_map(qkv, (uint64_t)(Hq + 2 * Hkv) * hd, (uint64_t)B * S, (uint64_t)ld_qkv, &tq);
  if (rc) return rc;
  rc = attn_make_map(dout, (uint64_t)Hq * hd, (uint64_t)B * S, (uint64_t)ld_o, &tdo);
  if (rc) return rc;
  if (!(hd == 64 && g_bwd64_variant >= 1)) {       // the hd 64 dQ kernel of variants 1 and 2 computes D itself
    const long warps = (long)B * S * Hq;
    long blocks = (warps + 7) / 8;
    if (blocks > 148 * 16) blocks = 148 * 16;
    attn_bwd_prep_kernel<<<(int)blocks, 256, 0, st>>>((const __nv_bfloat16*)dout, (const __nv_bfloat16*)out, Dbuf, B, S, Hq, hd, ld_o);
  }
  if (hsplit < 1 || hd != 256 || !part) hsplit = 1;
  if ((Hq / Hkv) % hsplit) return -2;
  AttnBwdParams p{(__nv_bfloat16*)dqkv, lse2, Dbuf, B, S, Hq, Hkv, ld_qkv, scale * 1.4426950408889634f, scale, part, hsplit,
                  softcap > 0.f ? scale / softcap : 0.f};
  dim3 gq(S / 128, Hq, B), gk(S / 128, Hkv, B);
  if (hd == 64 && g_bwd64_variant >= 1) {
    CUtensorMap tq64, tdo64, to128;
    rc = attn_make_map(out, (uint64_t)Hq * hd, (uint64_t)B * S, (uint64_t)ld_o, &to128);
    if (rc) return rc;
    rc = attn_make_map(qkv, (uint64_t)(Hq + 2 * Hkv) * hd, (uint64_t)B * S, (uint64_t)ld_qkv, &tq64, 64);
    if (rc) return rc;
    rc = attn_make_map(dout, (uint64_t)Hq * hd, (uint64_t)B * S, (uint64_t)ld_o, &tdo64, 64);
    if (rc) return rc;
    static bool attr64 = false;
    if (!attr64) {
      cudaError_t e = cudaFuncSetAttribute(attn_bwd64_kernel<RS_DQ>, cudaFuncAttributeMaxDynamicSharedMemorySize, Rs64Cfg::SMEM_BYTES);
      if (e == cudaSuccess) e = cudaFuncSetAttribute(attn_bwd64_kernel<RS_DKV>, cudaFuncAttributeMaxDynamicSharedMemorySize, Rs64Cfg::SMEM_BYTES);
      if (e != cudaSuccess) return (int)e;
      attr64 = true;
    }
    attn_bwd64_kernel<RS_DQ><<<gq, 320, Rs64Cfg::SMEM_BYTES, st>>>(tq, tdo, tq64, tdo64, to128, p);
    if (g_bwd64_variant == 1) {
      attn_bwd64_kernel<RS_DKV><<<gk, 320, Rs64Cfg::SMEM_BYTES, st>>>(tq, tdo, tq64, tdo64, to128, p);
    } else {
      static bool attr_old = false;
      if (!attr_old) {
        cudaError_t e = cudaFuncSetAttribute(attn_bwd_dkv_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, DkvCfg<64>::SMEM_BYTES);
        if (e != cudaSuccess) return (int)e;
        attr_old = true;
      }
      attn_bwd_dkv_kernel<64><<<gk, 320, DkvCfg<64>::SMEM_BYTES, st>>>(tq, tdo, p);
    }
    return (int)cudaGetLastError();
  }
  if (hd == 256) {
    CUtensorMap tq64, tdo64;
    rc = attn_make_map(qkv, (uint64_t)(Hq + 2 * Hkv) * hd, (uint64_t)B * S, (uint64_t)ld_qkv, &tq64, 64);
    if (rc) return rc;
    rc = attn_make_map(dout, (uint64_t)Hq * hd, (uint64_t)B * S, (uint64_t)ld_o, &tdo64, 64);
    if (rc) return rc;
    static bool attr256 = false;
    if (!attr256) {
      cudaError_t e = cudaFuncSetAttribute(attn_bwd256_kernel<BWD_DQ>, cudaFuncAttributeMaxDynamicSharedMemorySize, Bwd256Cfg::SMEM_BYTES);
      if (e == cudaSuccess) e = cudaFuncSetAttribute(attn_bwd256_kernel<BWD_DK>, cudaFuncAttributeMaxDynamicSharedMemorySize, Bwd256Cfg::SMEM_BYTES);
      if (e == cudaSuccess) e = cudaFuncSetAttribute(attn_bwd256_kernel<BWD_DV>, cudaFuncAttributeMaxDynamicSharedMemorySize, Bwd256Cfg::SMEM_BYTES);
      if (e != cudaSuccess) return (int)e;
      attr256 = true;
    }
    attn_bwd256_kernel<BWD_DQ><<<gq, 320, Bwd256Cfg::SMEM_BYTES, st>>>(tq, tdo, tq64, tdo64, p);
    dim3 gks(S / 128, Hkv * hsplit, B);
    attn_bwd256_kernel<BWD_DK><<<gks, 320, Bwd256Cfg::SMEM_BYTES, st>>>(tq, tdo, tq64, tdo64, p);
    attn_bwd256_kernel<BWD_DV><<<gks, 320, Bwd256Cfg::SMEM_BYTES, st>>>(tq, tdo, tq64, tdo64, p);
    if (hsplit > 1) {
      const size_t nvec = (size_t)2 * B * S * Hkv * 256 / 8;
      size_t blocks = (nvec + 255) / 256;
      if (blocks > 148 * 8) blocks = 148 * 8;
      attn_bwd256_reduce_kernel<<<(int)blocks, 256, 0, st>>>(part, (__nv_bfloat16*)dqkv, B * S, Hq, Hkv, hsplit, ld_qkv);
    }
    return (int)cudaGetLastError();
  }
#define LAUNCH_BWD(HD_)                                                                                              \
  do {                                                                                                               \
    static bool attr = false;                                                                                        \
    if (!attr) {                                                                                                     \
      cudaError_t e = cudaFuncSetAttribute(attn_bwd_dq_kernel<HD_>, cudaFuncAttributeMaxDynamicSharedMemorySize, DqCfg<HD_>::SMEM_BYTES); \
      if (e != cudaSuccess) return (int)e;                                                                           \
      e = cudaFuncSetAttribute(attn_bwd_dkv_kernel<HD_>, cudaFuncAttributeMaxDynamicSharedMemorySize, DkvCfg<HD_>::SMEM_BYTES); \
      if (e != cudaSuccess) return (int)e;                                                                           \
      attr = true;                                                                                                   \
    }                                                                                                                \
    attn_bwd_dq_kernel<HD_><<<gq, 320, DqCfg<HD_>::SMEM_BYTES, st>>>(tq, tdo, p);                                    \
    attn_bwd_dkv_kernel<HD_><<<gk, 320, DkvCfg<HD_>::SMEM_BYTES, st>>>(tq, tdo, p);                                  \
  } while (0)
  if (hd == 64) LAUNCH_BWD(64); else LAUNCH_BWD(128);
#undef LAUNCH_BWD
  return (int)cudaGetLastError();
}

int zen_attn_error() {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_attn_error, sizeof(int)) != cudaSuccess) return -1;
  if (v) cudaMemcpyToSymbol(g_attn_error, &zero, sizeof(int));
  return v;
}

}  // extern "C"
