// Memory-bound model ops for sm_100a: norms (with the residual add fused in), gated activations,
// RoPE, embedding forward / row-sparse backward, cross-entropy (loss and dlogits in one kernel),
// column sums, and a multi-tensor AdamW.  All are bandwidth kernels: 16-byte accesses, one pass over
// each operand, fp32 math, bf16 / fp32 / fp16 storage.
//
// The reference takes these from HuggingFace modules and ColossalAI's HybridAdam
// (train.py:149-157); nothing of them is in its tree.
#include "zen_common.cuh"

namespace {

template <typename T> struct Vec8;   // 8 elements of T <-> 8 floats
template <> struct Vec8<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[8]) {
    uint4 r = *reinterpret_cast<const uint4*>(p);
    uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) { v[2 * i] = __uint_as_float(w[i] << 16); v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u); }
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&v)[8]) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
      w[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
  }
};
template <> struct Vec8<__half> {
  static __device__ __forceinline__ void load(const __half* p, float (&v)[8]) {
    uint4 r = *reinterpret_cast<const uint4*>(p);
    const __half2* h = reinterpret_cast<const __half2*>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) { float2 f = __half22float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
  }
  static __device__ __forceinline__ void store(__half* p, const float (&v)[8]) {
    uint4 r;
    __half2* h = reinterpret_cast<__half2*>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = r;
  }
};
template <> struct Vec8<float> {
  static __device__ __forceinline__ void load(const float* p, float (&v)[8]) {
    float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  }
  static __device__ __forceinline__ void store(float* p, const float (&v)[8]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
  }
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int d = 16; d; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int d = 16; d; d >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, d));
  return v;
}
// Sum over the CTA (blockDim.x a multiple of 32, at most 1024); every thread gets the result.
__device__ __forceinline__ float block_sum(float v, float* sh) {
  v = warp_sum(v);
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
  __syncthreads();
  if (lane == 0) sh[w] = v;
  __syncthreads();
  float t = (lane < nw) ? sh[lane] : 0.f;
  return warp_sum(t);
}
__device__ __forceinline__ float block_max(float v, float* sh) {
  v = warp_max(v);
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
  __syncthreads();
  if (lane == 0) sh[w] = v;
  __syncthreads();
  float t = (lane < nw) ? sh[lane] : -INFINITY;
  return warp_max(t);
}

#define NORM_THREADS 128
#define NORM_MAXV 8   // up to 128 * 8 * 8 = 8192 columns held in registers; kernels are instantiated for 1, 2, 4, 8

// --------------------------------------------------------------------------------------------
// Norm forward.  h = x (+ res); y = (h - mean) * rstd * wgt + bias   (LayerNorm, kLayer)
//                                y = h * rstd * (wgt or 1 + wgt)     (RMSNorm)
// `hout` (optional) receives h, the new residual stream.  stats: rstd[rows] (+ mean[rows]).
template <typename T, bool kLayer, int NV>
__global__ void __launch_bounds__(NORM_THREADS)
norm_fwd_kernel(const T* __restrict__ x, const T* __restrict__ res, const T* __restrict__ wgt,
                const T* __restrict__ bias, T* __restrict__ y, T* __restrict__ hout, float* __restrict__ rstd_out,
                float* __restrict__ mean_out, int rows, int cols, float eps, int unit_offset) {
  __shared__ float sh[32];
  const int nv = cols / 8;                         // cols % 8 == 0 checked on the host
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const size_t base = (size_t)row * cols;
    float h[NV][8];
    float s = 0.f, ss = 0.f;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int v = threadIdx.x + j * NORM_THREADS;
      if (v < nv) {
        Vec8<T>::load(x + base + (size_t)v * 8, h[j]);
        if (res) {
          float r[8];
          Vec8<T>::load(res + base + (size_t)v * 8, r);
#pragma unroll
          for (int i = 0; i < 8; ++i) h[j][i] += r[i];
        }
        if (hout) {
          Vec8<T>::store(hout + base + (size_t)v * 8, h[j]);
          // keep exactly what was stored so that forward and backward see the same h
          Vec8<T>::load(hout + base + (size_t)v * 8, h[j]);
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) { s += h[j][i]; ss += h[j][i] * h[j][i]; }
      }
    }
    float mean = 0.f, var;
    if (kLayer) {
      mean = block_sum(s, sh) / cols;
      float d2 = 0.f;
#pragma unroll
      for (int j = 0; j < NV; ++j) {
        const int v = threadIdx.x + j * NORM_THREADS;
        if (v < nv) {
#pragma unroll
          for (int i = 0; i < 8; ++i) { const float d = h[j][i] - mean; d2 += d * d; }
        }
      }
      var = block_sum(d2, sh) / cols;
    } else {
      var = block_sum(ss, sh) / cols;
    }
    const float rstd = rsqrtf(var + eps);
    if (threadIdx.x == 0) { rstd_out[row] = rstd; if (kLayer) mean_out[row] = mean; }
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int v = threadIdx.x + j * NORM_THREADS;
      if (v < nv) {
        float w[8], o[8];
        Vec8<T>::load(wgt + (size_t)v * 8, w);
        if (kLayer) {
          float b[8];
          if (bias) Vec8<T>::load(bias + (size_t)v * 8, b);
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] = (h[j][i] - mean) * rstd * w[i] + (bias ? b[i] : 0.f);
        } else {
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] = h[j][i] * rstd * (unit_offset ? 1.f + w[i] : w[i]);
        }
        Vec8<T>::store(y + base + (size_t)v * 8, o);
      }
    }
  }
}

// Rows kept as raw 16-byte vectors (8 registers per vector for fp32, 4 for 16-bit types) and unpacked on use.
template <typename T> struct Pack;
template <> struct Pack<float> {
  struct raw_t { float4 a, b; };
  static __device__ __forceinline__ raw_t load(const float* p) { raw_t r; r.a = *reinterpret_cast<const float4*>(p); r.b = *reinterpret_cast<const float4*>(p + 4); return r; }
  static __device__ __forceinline__ void unpack(const raw_t& r, float (&v)[8]) { v[0] = r.a.x; v[1] = r.a.y; v[2] = r.a.z; v[3] = r.a.w; v[4] = r.b.x; v[5] = r.b.y; v[6] = r.b.z; v[7] = r.b.w; }
};
template <> struct Pack<__nv_bfloat16> {
  typedef uint4 raw_t;
  static __device__ __forceinline__ raw_t load(const __nv_bfloat16* p) { return *reinterpret_cast<const uint4*>(p); }
  static __device__ __forceinline__ void unpack(const raw_t& r, float (&v)[8]) {
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) { v[2 * i] = __uint_as_float(w[i] << 16); v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u); }
  }
};
template <> struct Pack<__half> {
  typedef uint4 raw_t;
  static __device__ __forceinline__ raw_t load(const __half* p) { return *reinterpret_cast<const uint4*>(p); }
  static __device__ __forceinline__ void unpack(const raw_t& r, float (&v)[8]) {
    const __half2* h = reinterpret_cast<const __half2*>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) { float2 f = __half22float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
  }
};

// Norm backward.  dh = grad through the norm (+ dres, the gradient arriving on the residual stream).
// Per-CTA partial sums of dw (and db) go to part_dw/part_db [gridDim.x][cols] (fp32 scratch) and are
// folded by colreduce_kernel.
template <typename T, bool kLayer, int NV, bool kParams>
__global__ void __launch_bounds__(NORM_THREADS)
norm_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ h, const T* __restrict__ wgt,
                const float* __restrict__ rstd_in, const float* __restrict__ mean_in, const T* __restrict__ dres,
                T* __restrict__ dh, float* __restrict__ part_dw, float* __restrict__ part_db, int rows, int cols,
                int unit_offset) {
  __shared__ float sh[32];
  const int nv = cols / 8;
  // kParams = false: only dh here (the parameter gradients come from norm_dwdb_partial_kernel), which frees the
  // 16 * NV accumulator registers and lets several CTAs share an SM
  float aw[kParams ? NV : 1][8], ab[kParams ? NV : 1][8];
  if (kParams) {
#pragma unroll
    for (int j = 0; j < NV; ++j)
#pragma unroll
      for (int i = 0; i < 8; ++i) { aw[j][i] = 0.f; ab[j][i] = 0.f; }
  }
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const size_t base = (size_t)row * cols;
    const float rstd = rstd_in[row];
    const float mean = kLayer ? mean_in[row] : 0.f;
    float g[NV][8], xh[NV][8];
    typename Pack<T>::raw_t rres[NV];               // residual-stream gradient, fetched with the first loads
    float s1 = 0.f, s2 = 0.f;                       // sum(g), sum(g * xhat)
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int v = threadIdx.x + j * NORM_THREADS;
      if (v < nv && dres) rres[j] = Pack<T>::load(dres + base + (size_t)v * 8);
    }
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int v = threadIdx.x + j * NORM_THREADS;
      if (v < nv) {
        float d[8], w[8];
        Vec8<T>::load(dy + base + (size_t)v * 8, d);
        Vec8<T>::load(h + base + (size_t)v * 8, xh[j]);
        Vec8<T>::load(wgt + (size_t)v * 8, w);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          xh[j][i] = (xh[j][i] - mean) * rstd;
          if (kParams) { aw[j][i] += d[i] * xh[j][i]; ab[j][i] += d[i]; }
          g[j][i] = d[i] * (kLayer ? w[i] : (unit_offset ? 1.f + w[i] : w[i]));
          s1 += g[j][i];
          s2 += g[j][i] * xh[j][i];
        }
      }
    }
    s2 = block_sum(s2, sh) / cols;
    if (kLayer) s1 = block_sum(s1, sh) / cols; else s1 = 0.f;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int v = threadIdx.x + j * NORM_THREADS;
      if (v < nv) {
        float o[8];
        if (dres) Pack<T>::unpack(rres[j], o);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float t = rstd * (g[j][i] - s1 - xh[j][i] * s2);
          o[i] = dres ? o[i] + t : t;
        }
        Vec8<T>::store(dh + base + (size_t)v * 8, o);
      }
    }
  }
  if (!kParams) return;
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    const int v = threadIdx.x + j * NORM_THREADS;
    if (v < nv) {
      Vec8<float>::store(part_dw + (size_t)blockIdx.x * cols + (size_t)v * 8, aw[j]);
      if (kLayer && part_db) Vec8<float>::store(part_db + (size_t)blockIdx.x * cols + (size_t)v * 8, ab[j]);
    }
  }
}

// ---- warp-per-row variants for narrow rows (cols <= 256 * NV): no block barriers, many rows in flight per SM.
// Rows are kept as raw 16-byte vectors (8 registers per vector for fp32, 4 for 16-bit types) and unpacked on use.
#define NORMW_WARPS 8

template <typename T, bool kLayer, int NV>
__global__ void __launch_bounds__(NORMW_WARPS * 32, 4)      // 64 registers: four CTAs (32 warps, a row each) per SM
norm_fwd_warp_kernel(const T* __restrict__ x, const T* __restrict__ res, const T* __restrict__ wgt,
                     const T* __restrict__ bias, T* __restrict__ y, T* __restrict__ hout, float* __restrict__ rstd_out,
                     float* __restrict__ mean_out, int rows, int cols, float eps, int unit_offset) {
  const int lane = threadIdx.x & 31;
  const int gw = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, nw = (gridDim.x * blockDim.x) >> 5;
  const int nv = cols / 8;
  for (int row = gw; row < rows; row += nw) {
    const size_t base = (size_t)row * cols;
    float h[NV][8];
    float s = 0.f, ss = 0.f;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int v = lane + 32 * j;
      if (v < nv) {
        Vec8<T>::load(x + base + (size_t)v * 8, h[j]);
        if (res) {
          float r[8];
          Vec8<T>::load(res + base + (size_t)v * 8, r);
#pragma unroll
          for (int i = 0; i < 8; ++i) h[j][i] += r[i];
        }
        if (hout) {
          Vec8<T>::store(hout + base + (size_t)v * 8, h[j]);
          if (sizeof(T) == 2) {   // continue with exactly what was stored
#pragma unroll
            for (int i = 0; i < 8; ++i) h[j][i] = ZenVal<T>::to_f(ZenVal<T>::from_f(h[j][i]));
          }
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) { s += h[j][i]; ss += h[j][i] * h[j][i]; }
      }
    }
    float mean = 0.f, var;
    if (kLayer) {
      mean = warp_sum(s) / cols;
      float d2 = 0.f;
#pragma unroll
      for (int j = 0; j < NV; ++j) {
        if (lane + 32 * j < nv) {
#pragma unroll
          for (int i = 0; i < 8; ++i) { const float d = h[j][i] - mean; d2 += d * d; }
        }
      }
      var = warp_sum(d2) / cols;
    } else {
      var = warp_sum(ss) / cols;
    }
    const float rstd = rsqrtf(var + eps);
    if (lane == 0) { rstd_out[row] = rstd; if (kLayer) mean_out[row] = mean; }
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int v = lane + 32 * j;
      if (v < nv) {
        float w[8], o[8];
        Vec8<T>::load(wgt + (size_t)v * 8, w);
        if (kLayer) {
          float b[8];
          if (bias) Vec8<T>::load(bias + (size_t)v * 8, b);
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] = (h[j][i] - mean) * rstd * w[i] + (bias ? b[i] : 0.f);
        } else {
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] = h[j][i] * rstd * (unit_offset ? 1.f + w[i] : w[i]);
        }
        Vec8<T>::store(y + base + (size_t)v * 8, o);
      }
    }
  }
}

template <typename T, bool kLayer, int NV, bool kParams>
__global__ void __launch_bounds__(NORMW_WARPS * 32, (NV <= 3 && !kParams) ? 4 : 2)   // up to 768 columns: four CTAs per SM
norm_bwd_warp_kernel(const T* __restrict__ dy, const T* __restrict__ h, const T* __restrict__ wgt,
                     const float* __restrict__ rstd_in, const float* __restrict__ mean_in, const T* __restrict__ dres,
                     T* __restrict__ dh, float* __restrict__ part_dw, float* __restrict__ part_db, int rows, int cols,
                     int unit_offset) {
  extern __shared__ float sm_acc[];                 // [2][cols]: dw and db sums of this CTA
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int gw = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, nw = (gridDim.x * blockDim.x) >> 5;
  const int nv = cols / 8;
  float aw[kParams ? NV : 1][8], ab[(kLayer && kParams) ? NV : 1][8];
  // the weights stay packed (a warp usually handles one or two rows: half the registers of an unpacked copy, and with
  // them a fourth CTA per SM)
  typename Pack<T>::raw_t rw[NV];
  const float woff = (!kLayer && unit_offset) ? 1.f : 0.f;
#pragma unroll
  for (int j = 0; j < NV; ++j) {
#pragma unroll
    for (int i = 0; i < 8; ++i) { if (kParams) { aw[j][i] = 0.f; if (kLayer) ab[j][i] = 0.f; } }
    if (lane + 32 * j < nv) rw[j] = Pack<T>::load(wgt + (size_t)(lane + 32 * j) * 8);
  }
  for (int row = gw; row < rows; row += nw) {
    const size_t base = (size_t)row * cols;
    const float rstd = rstd_in[row];
    const float mean = kLayer ? mean_in[row] : 0.f;
    typename Pack<T>::raw_t rd[NV], rh[NV];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      if (lane + 32 * j < nv) {
        rd[j] = Pack<T>::load(dy + base + (size_t)(lane + 32 * j) * 8);
        rh[j] = Pack<T>::load(h + base + (size_t)(lane + 32 * j) * 8);
      }
    }
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      if (lane + 32 * j < nv) {
        float d[8], xh[8], wv[8];
        Pack<T>::unpack(rd[j], d);
        Pack<T>::unpack(rh[j], xh);
        Pack<T>::unpack(rw[j], wv);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          xh[i] = (xh[i] - mean) * rstd;
          if (kParams) { aw[j][i] += d[i] * xh[i]; if (kLayer) ab[j][i] += d[i]; }
          const float g = d[i] * (wv[i] + woff);
          s1 += g;
          s2 += g * xh[i];
        }
      }
    }
    s2 = warp_sum(s2) / cols;
    s1 = kLayer ? warp_sum(s1) / cols : 0.f;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int v = lane + 32 * j;
      if (v < nv) {
        float d[8], xh[8], o[8], wv[8];
        Pack<T>::unpack(rd[j], d);
        Pack<T>::unpack(rh[j], xh);
        Pack<T>::unpack(rw[j], wv);
        if (dres) Vec8<T>::load(dres + base + (size_t)v * 8, o);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float xhat = (xh[i] - mean) * rstd;
          const float t = rstd * (d[i] * (wv[i] + woff) - s1 - xhat * s2);
          o[i] = dres ? o[i] + t : t;
        }
        Vec8<T>::store(dh + base + (size_t)v * 8, o);
      }
    }
  }
  if (!kParams) return;
  // fold the warps' partial dw / db through shared memory, one warp at a time (fixed order)
  float* sdw = sm_acc;
  float* sdb = sm_acc + cols;
  for (int wsel = 0; wsel < NORMW_WARPS; ++wsel) {
    if (warp == wsel) {
#pragma unroll
      for (int j = 0; j < NV; ++j) {
        const int v = lane + 32 * j;
        if (v < nv) {
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            sdw[v * 8 + i] = (wsel == 0 ? 0.f : sdw[v * 8 + i]) + aw[j][i];
            if (kLayer) sdb[v * 8 + i] = (wsel == 0 ? 0.f : sdb[v * 8 + i]) + ab[j][i];
          }
        }
      }
    }
    __syncthreads();
  }
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    part_dw[(size_t)blockIdx.x * cols + c] = sdw[c];
    if (kLayer && part_db) part_db[(size_t)blockIdx.x * cols + c] = sdb[c];
  }
}

// Parameter gradients of a norm, column-sum style: CTA b covers rows [32 b, 32 b + 32) and every column (a thread
// owns 8 columns, loads are coalesced along the row): part_dw[b][c] = sum_r dy * xhat, part_db[b][c] = sum_r dy.
template <typename T, bool kLayer>
__global__ void __launch_bounds__(256)
norm_dwdb_partial_kernel(const T* __restrict__ dy, const T* __restrict__ h, const float* __restrict__ rstd_in,
                         const float* __restrict__ mean_in, float* __restrict__ part_dw, float* __restrict__ part_db,
                         int rows, int cols, int rows_per_cta) {
  // Wide matrices: blockIdx.y selects a 2048-column slice (one vector per thread), blockIdx.x a group of rows.
  // Narrow matrices (fewer 8-column vectors than threads): the threads form `groups` row groups that walk
  // interleaved rows of the CTA's 32 and meet in shared memory, group by group, so that no thread idles.
  __shared__ float red_w[2048], red_b[2048];
  const int r0 = blockIdx.x * rows_per_cta, r1 = min(rows, r0 + rows_per_cta);
  const int vpr = cols / 8;
  const int groups = vpr <= 128 ? 256 / vpr : 1;
  const int g = groups > 1 ? threadIdx.x / vpr : 0;
  const int first = groups > 1 ? (threadIdx.x % vpr) * 8 : (blockIdx.y * 256 + threadIdx.x) * 8;
  const int stride = cols;                                   // every thread owns exactly one vector
  if (g >= groups) {                                         // leftover threads (256 not a multiple of vpr)
    for (int k = 1; k < groups; ++k) { __syncthreads(); __syncthreads(); }
    return;
  }
  for (int c8 = first; c8 < cols; c8 += stride) {
    float aw[8] = {0, 0, 0, 0, 0, 0, 0, 0}, ab[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll 4
    for (int r = r0 + g; r < r1; r += groups) {
      float d[8], x[8];
      Vec8<T>::load(dy + (size_t)r * cols + c8, d);
      Vec8<T>::load(h + (size_t)r * cols + c8, x);
      const float rs = rstd_in[r], mu = kLayer ? mean_in[r] : 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) { aw[i] += d[i] * (x[i] - mu) * rs; ab[i] += d[i]; }
    }
    for (int k = 1; k < groups; ++k) {                       // fold group k into group 0, in group order
      if (g == k) {
#pragma unroll
        for (int i = 0; i < 8; ++i) { red_w[c8 + i] = aw[i]; red_b[c8 + i] = ab[i]; }
      }
      __syncthreads();
      if (g == 0) {
#pragma unroll
        for (int i = 0; i < 8; ++i) { aw[i] += red_w[c8 + i]; ab[i] += red_b[c8 + i]; }
      }
      __syncthreads();
    }
    if (g == 0) {
      Vec8<float>::store(part_dw + (size_t)blockIdx.x * cols + c8, aw);
      if (kLayer && part_db) Vec8<float>::store(part_db + (size_t)blockIdx.x * cols + c8, ab);
    }
  }
}

// out[c] (+)= sum_p part[p][c], cast to T.  CTA = 32 columns x 32 part-lanes; fixed summation order.
// blockIdx.y == 1 reduces a second (part, out) pair of the same shape in the same launch (dw and db of a LayerNorm).
template <typename T>
__global__ void __launch_bounds__(1024)
colreduce_kernel(const float* __restrict__ part, T* __restrict__ out, int nparts, int cols, int accumulate,
                 const float* __restrict__ part2 = nullptr, T* __restrict__ out2 = nullptr) {
  if (blockIdx.y == 1) { part = part2; out = out2; }
  __shared__ float sh[32][33];
  const int x = threadIdx.x & 31, y = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + x;
  float s = 0.f;
  if (c < cols)
    for (int p = y; p < nparts; p += 32) s += part[(size_t)p * cols + c];
  sh[y][x] = s;
  __syncthreads();
  if (y == 0 && c < cols) {
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < 32; ++i) t += sh[i][x];
    if (accumulate) t += ZenVal<T>::to_f(out[c]);
    out[c] = ZenVal<T>::from_f(t);
  }
}

// Several reductions of that kind in one launch (the bias and norm-parameter gradients of a layer): blockIdx.y = 2 * job
// (+ 1 for the job's second pair, if it has one), blockIdx.x = 32-column block of that job.
#define COLREDUCE_MAX_JOBS 8
struct ColReduceJob {
  const float* part;
  void* out;
  const float* part2;             // optional second (part, out) pair of the same shape (dw and db of a LayerNorm)
  void* out2;
  int nparts, cols, accumulate, pad;
};
struct ColReduceJobs {
  ColReduceJob j[COLREDUCE_MAX_JOBS];
  int n;
};
template <typename T>
__global__ void __launch_bounds__(1024)
colreduce_multi_kernel(const ColReduceJobs jobs) {
  const ColReduceJob& jb = jobs.j[blockIdx.y >> 1];
  const float* part = (blockIdx.y & 1) ? jb.part2 : jb.part;
  T* out = reinterpret_cast<T*>((blockIdx.y & 1) ? jb.out2 : jb.out);
  if (!part || !out || (int)blockIdx.x * 32 >= jb.cols) return;                // uniform over the CTA
  __shared__ float sh[32][33];
  const int x = threadIdx.x & 31, y = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + x;
  float s = 0.f;
  if (c < jb.cols)
    for (int p = y; p < jb.nparts; p += 32) s += part[(size_t)p * jb.cols + c];
  sh[y][x] = s;
  __syncthreads();
  if (y == 0 && c < jb.cols) {
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < 32; ++i) t += sh[i][x];
    if (jb.accumulate) t += ZenVal<T>::to_f(out[c]);
    out[c] = ZenVal<T>::from_f(t);
  }
}

// Column sums of a [rows, cols] matrix: CTA b sums rows [b * COLSUM_ROWS, ...) for every column (thread = one
// 8-column vector, coalesced along the row) into part[b][cols] (bias gradients).
#define COLSUM_ROWS 32
template <typename T>
__global__ void __launch_bounds__(256) colsum_partial_kernel(const T* __restrict__ a, float* __restrict__ part, int rows, int cols) {
  __shared__ float red[2048];                                // see norm_dwdb_partial_kernel: row groups for narrow matrices
  const int r0 = blockIdx.x * COLSUM_ROWS, r1 = min(rows, r0 + COLSUM_ROWS);
  const int vpr = cols / 8;
  const int groups = vpr <= 128 ? 256 / vpr : 1;
  if (groups == 1) {                                          // wide matrix: every thread has columns of its own
    for (int c8 = threadIdx.x * 8; c8 < cols; c8 += blockDim.x * 8) {
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll 8
      for (int r = r0; r < r1; ++r) {
        float v[8];
        Vec8<T>::load(a + (size_t)r * cols + c8, v);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] += v[i];
      }
      Vec8<float>::store(part + (size_t)blockIdx.x * cols + c8, acc);
    }
    return;
  }
  const int g = threadIdx.x / vpr;
  const int first = (threadIdx.x % vpr) * 8;
  const int stride = cols;
  if (g >= groups) {
    for (int k = 1; k < groups; ++k) { __syncthreads(); __syncthreads(); }
    return;
  }
  for (int c8 = first; c8 < cols; c8 += stride) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll 8
    for (int r = r0 + g; r < r1; r += groups) {
      float v[8];
      Vec8<T>::load(a + (size_t)r * cols + c8, v);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += v[i];
    }
    for (int k = 1; k < groups; ++k) {
      if (g == k) {
#pragma unroll
        for (int i = 0; i < 8; ++i) red[c8 + i] = acc[i];
      }
      __syncthreads();
      if (g == 0) {
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] += red[c8 + i];
      }
      __syncthreads();
    }
    if (g == 0) Vec8<float>::store(part + (size_t)blockIdx.x * cols + c8, acc);
  }
}

// --------------------------------------------------------------------------------------------
// Activations.  mode: 0 gelu(tanh) 1 relu 2 silu(a)*b 3 gelu_tanh(a)*b
__device__ __forceinline__ float tanh_fast(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));   // max relative error about 2^-11, below bf16 resolution
  return y;
}
__device__ __forceinline__ float gelu_tanh(float x) {
  const float k = 0.7978845608028654f;
  return 0.5f * x * (1.f + tanh_fast(k * (x + 0.044715f * x * x * x)));
}
__device__ __forceinline__ float gelu_tanh_grad(float x) {
  const float k = 0.7978845608028654f;
  const float t = tanh_fast(k * (x + 0.044715f * x * x * x));
  return 0.5f * (1.f + t) + 0.5f * x * (1.f - t * t) * k * (1.f + 3.f * 0.044715f * x * x);
}
__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + __expf(-x)); }

// a and b may be the two halves of one [rows, 2 * inner] matrix (strided) or separate tensors.
template <typename T>
__global__ void __launch_bounds__(256)
act_fwd_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ out, int rows, int inner, int lda,
               int ldb, int mode) {
  const size_t nvec = (size_t)rows * (inner / 8);
  for (size_t v = (size_t)blockIdx.x * blockDim.x + threadIdx.x; v < nvec; v += (size_t)gridDim.x * blockDim.x) {
    const int r = (int)(v / (inner / 8)), c = (int)(v % (inner / 8)) * 8;
    float x[8], y[8], o[8];
    Vec8<T>::load(a + (size_t)r * lda + c, x);
    if (mode >= 2) Vec8<T>::load(b + (size_t)r * ldb + c, y);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (mode == 0) o[i] = gelu_tanh(x[i]);
      else if (mode == 1) o[i] = fmaxf(x[i], 0.f);
      else if (mode == 2) o[i] = x[i] * sigmoidf_(x[i]) * y[i];
      else o[i] = gelu_tanh(x[i]) * y[i];
    }
    Vec8<T>::store(out + (size_t)r * inner + c, o);
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
act_bwd_kernel(const T* __restrict__ a, const T* __restrict__ b, const T* __restrict__ dout, T* __restrict__ da,
               T* __restrict__ db, int rows, int inner, int lda, int ldb, int mode) {
  const size_t nvec = (size_t)rows * (inner / 8);
  for (size_t v = (size_t)blockIdx.x * blockDim.x + threadIdx.x; v < nvec; v += (size_t)gridDim.x * blockDim.x) {
    const int r = (int)(v / (inner / 8)), c = (int)(v % (inner / 8)) * 8;
    float x[8], y[8], g[8], ga[8], gb[8];
    Vec8<T>::load(a + (size_t)r * lda + c, x);
    Vec8<T>::load(dout + (size_t)r * inner + c, g);
    if (mode >= 2) Vec8<T>::load(b + (size_t)r * ldb + c, y);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (mode == 0) ga[i] = g[i] * gelu_tanh_grad(x[i]);
      else if (mode == 1) ga[i] = x[i] > 0.f ? g[i] : 0.f;
      else if (mode == 2) {
        const float s = sigmoidf_(x[i]);
        ga[i] = g[i] * y[i] * s * (1.f + x[i] * (1.f - s));
        gb[i] = g[i] * x[i] * s;
      } else {
        ga[i] = g[i] * y[i] * gelu_tanh_grad(x[i]);
        gb[i] = g[i] * gelu_tanh(x[i]);
      }
    }
    Vec8<T>::store(da + (size_t)r * lda + c, ga);
    if (mode >= 2) Vec8<T>::store(db + (size_t)r * ldb + c, gb);
  }
}

// Backward of an ungated activation (mode 0 / 1) that also leaves the column sums of its result, the bias gradient of
// the linear layer that produced the activation's input: CTA b handles rows [b * rows_per_cta, ...) of every column and
// writes part[b][inner], the layout that colreduce_kernel sums.  The separate column-sum kernel would read da again.
template <typename T>
__global__ void __launch_bounds__(512)
act_bwd_colsum_kernel(const T* __restrict__ a, const T* __restrict__ dout, T* __restrict__ da, float* __restrict__ part,
                      int rows, int inner, int mode, int rows_per_cta) {
  const int r0 = blockIdx.x * rows_per_cta, r1 = min(rows, r0 + rows_per_cta);
  for (int c8 = threadIdx.x * 8; c8 < inner; c8 += blockDim.x * 8) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll 4
    for (int r = r0; r < r1; ++r) {
      float x[8], g[8], ga[8];
      Vec8<T>::load(a + (size_t)r * inner + c8, x);
      Vec8<T>::load(dout + (size_t)r * inner + c8, g);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float v = (mode == 0) ? g[i] * gelu_tanh_grad(x[i]) : (x[i] > 0.f ? g[i] : 0.f);
        ga[i] = ZenVal<T>::to_f(ZenVal<T>::from_f(v));       // the sum is that of the stored values
        acc[i] += ga[i];
      }
      Vec8<T>::store(da + (size_t)r * inner + c8, ga);
    }
    Vec8<float>::store(part + (size_t)blockIdx.x * inner + c8, acc);
  }
}

// --------------------------------------------------------------------------------------------
// RoPE (rotate-half convention): x is [tokens, heads, hd] with row stride `ld` elements between
// tokens; token t sits at position pos0 + t % seq.  sign = -1 applies the inverse rotation
// (the backward pass).  In place.
template <typename T>
__global__ void __launch_bounds__(256)
rope_kernel(T* __restrict__ x, int tokens, int heads, int hd, int ld, int seq, int pos0, float log2_theta, float sign) {
  const int half = hd / 2;
  const size_t n = (size_t)tokens * heads * half;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const int j = (int)(i % half);
    const int hh = (int)((i / half) % heads);
    const int t = (int)(i / ((size_t)half * heads));
    const float inv_freq = exp2f(-log2_theta * (2.f * j / hd));
    float s, c;
    sincosf((float)(pos0 + t % seq) * inv_freq, &s, &c);
    s *= sign;
    T* p = x + (size_t)t * ld + (size_t)hh * hd;
    const float a = ZenVal<T>::to_f(p[j]), b = ZenVal<T>::to_f(p[j + half]);
    p[j] = ZenVal<T>::from_f(a * c - b * s);
    p[j + half] = ZenVal<T>::from_f(b * c + a * s);
  }
}

// Vectorised form for hd / 2 a multiple of 8: a thread owns 8 consecutive frequencies of one token, computes their
// sines and cosines once and walks all heads with 16-byte loads and stores (the scalar kernel above recomputes the
// trigonometry for every head and moves two bytes per access).
template <typename T>
__global__ void __launch_bounds__(256)
rope_vec_kernel(T* __restrict__ x, int tokens, int heads, int hd, int ld, int seq, int pos0, float log2_theta, float sign) {
  const int half = hd / 2, vph = half / 8;
  const size_t n = (size_t)tokens * vph;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += (size_t)gridDim.x * blockDim.x) {
    const int jv = (int)(idx % vph);
    const int t = (int)(idx / vph);
    const float pos = (float)(pos0 + t % seq);
    float c[8], sn[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float inv_freq = exp2f(-log2_theta * (2.f * (jv * 8 + i) / hd));
      sincosf(pos * inv_freq, &sn[i], &c[i]);
      sn[i] *= sign;
    }
    T* p = x + (size_t)t * ld + jv * 8;
#pragma unroll 4
    for (int hh = 0; hh < heads; ++hh) {
      float a[8], b[8], oa[8], ob[8];
      Vec8<T>::load(p + (size_t)hh * hd, a);
      Vec8<T>::load(p + (size_t)hh * hd + half, b);
#pragma unroll
      for (int i = 0; i < 8; ++i) { oa[i] = a[i] * c[i] - b[i] * sn[i]; ob[i] = b[i] * c[i] + a[i] * sn[i]; }
      Vec8<T>::store(p + (size_t)hh * hd, oa);
      Vec8<T>::store(p + (size_t)hh * hd + half, ob);
    }
  }
}

// --------------------------------------------------------------------------------------------
// Embedding forward: out[t] = wte[ids[t]] * scale (+ wpe[pos_offset + t % seq]).
template <typename T>
__global__ void __launch_bounds__(128)
embedding_fwd_kernel(const int64_t* __restrict__ ids, const T* __restrict__ wte, const T* __restrict__ wpe,
                     T* __restrict__ out, int tokens, int d, int seq, int pos_offset, float scale, int vocab) {
  for (int t = blockIdx.x; t < tokens; t += gridDim.x) {
    int64_t id = ids[t];
    if (id < 0 || id >= vocab) id = 0;
    for (int c = threadIdx.x * 8; c < d; c += blockDim.x * 8) {
      float v[8];
      Vec8<T>::load(wte + (size_t)id * d + c, v);
      if (scale != 1.f) {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = ZenVal<T>::to_f(ZenVal<T>::from_f(v[i] * scale));
      }
      if (wpe) {
        float p[8];
        Vec8<T>::load(wpe + (size_t)(pos_offset + t % seq) * d + c, p);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] += p[i];
      }
      Vec8<T>::store(out + (size_t)t * d + c, v);
    }
  }
}

// Row-sparse embedding backward, three kernels:
//   mark    : flag[id] = 1 for every token id
//   compact : single-CTA scan over flag[V]: cid[row] = rank among touched rows, rows[] ascending, *count
//   accum   : acc[cid[id]][:] += dy[t][:] * scale   (fp32 atomics into a [U, d] scratch)
__global__ void embed_mark_kernel(const int64_t* __restrict__ ids, int32_t* __restrict__ flag, int tokens, int vocab) {
  for (int t = blockIdx.x * blockDim.x + threadIdx.x; t < tokens; t += gridDim.x * blockDim.x) {
    const int64_t id = ids[t];
    if (id >= 0 && id < vocab) flag[id] = 1;
  }
}

// One CTA; warp w owns the contiguous range [w * per, (w + 1) * per) of the vocabulary and walks it 32 flags at a
// time (coalesced), first counting with ballots, then, after a scan over the 32 warp totals, handing out compact ids
// in ascending row order.
__global__ void __launch_bounds__(1024)
embed_compact_kernel(int32_t* __restrict__ flag_cid, int32_t* __restrict__ rows, int32_t* __restrict__ count, int vocab) {
  __shared__ uint32_t wtot[32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int per = ((vocab + 31) / 32 + 31) / 32 * 32;                 // per-warp range, a multiple of 32
  const int b = warp * per, e = min(vocab, b + per);
  uint32_t s = 0;
  for (int i = b + lane; i < b + per; i += 32) {
    const bool f = i < e && flag_cid[i] != 0;
    s += __popc(__ballot_sync(0xffffffffu, f));
  }
  if (lane == 0) wtot[warp] = s;
  __syncthreads();
  uint32_t pre = wtot[lane];                                          // every warp scans the 32 totals
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const uint32_t t = __shfl_up_sync(0xffffffffu, pre, d);
    if (lane >= d) pre += t;
  }
  const uint32_t total = __shfl_sync(0xffffffffu, pre, 31);
  uint32_t run = __shfl_sync(0xffffffffu, pre, warp) - wtot[warp];    // exclusive offset of this warp
  for (int i = b + lane; i < b + per; i += 32) {
    const bool in = i < e;
    const bool f = in && flag_cid[i] != 0;
    const uint32_t bal = __ballot_sync(0xffffffffu, f);
    if (f) {
      const uint32_t u = run + __popc(bal & ((1u << lane) - 1u));
      flag_cid[i] = (int32_t)u;
      rows[u] = i;
    } else if (in) {
      flag_cid[i] = -1;
    }
    run += __popc(bal);
  }
  if (threadIdx.x == 0) *count = (int32_t)total;
}

template <typename T>
__global__ void __launch_bounds__(128)
embed_accum_kernel(const int64_t* __restrict__ ids, const int32_t* __restrict__ cid, const T* __restrict__ dy,
                   float* __restrict__ acc, int tokens, int d, int vocab, float scale) {
  for (int t = blockIdx.x; t < tokens; t += gridDim.x) {
    const int64_t id = ids[t];
    if (id < 0 || id >= vocab) continue;
    const int u = cid[id];
    if (u < 0) continue;
    for (int c = threadIdx.x * 8; c < d; c += blockDim.x * 8) {
      float v[8];
      Vec8<T>::load(dy + (size_t)t * d + c, v);
      float* a = acc + (size_t)u * d + c;
      atomicAdd(reinterpret_cast<float4*>(a), make_float4(v[0] * scale, v[1] * scale, v[2] * scale, v[3] * scale));
      atomicAdd(reinterpret_cast<float4*>(a + 4), make_float4(v[4] * scale, v[5] * scale, v[6] * scale, v[7] * scale));
    }
  }
}

// vals[u][:] = T(acc[u][:]) for u < *count, and reset acc, cid (through rows) for the next call.
template <typename T>
__global__ void __launch_bounds__(128)
embed_finish_kernel(float* __restrict__ acc, int32_t* __restrict__ flag_cid, const int32_t* __restrict__ rows,
                    const int32_t* __restrict__ count, T* __restrict__ vals, int d) {
  const int n = *count;
  for (int u = blockIdx.x; u < n; u += gridDim.x) {
    for (int c = threadIdx.x * 8; c < d; c += blockDim.x * 8) {
      float v[8];
      Vec8<float>::load(acc + (size_t)u * d + c, v);
      Vec8<T>::store(vals + (size_t)u * d + c, v);
      const float z[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      Vec8<float>::store(acc + (size_t)u * d + c, z);
    }
  }
}
__global__ void embed_clear_flags_kernel(int32_t* __restrict__ flag_cid, int vocab) {
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < vocab; i += gridDim.x * blockDim.x) flag_cid[i] = 0;
}

// grad[rows[u]][:] += vals[u][:] for u < *count (rows unique): applies a row-sparse gradient to a dense one.
template <typename T>
__global__ void __launch_bounds__(128)
rows_add_kernel(T* __restrict__ grad, const int32_t* __restrict__ rows, const int32_t* __restrict__ count,
                const T* __restrict__ vals, int d, int vocab, int max_rows) {
  const int n = min(*count, max_rows);
  for (int u = blockIdx.x; u < n; u += gridDim.x) {
    const int r = rows[u];
    if (r < 0 || r >= vocab) continue;
    for (int c = threadIdx.x * 8; c < d; c += blockDim.x * 8) {
      float a[8], b[8];
      Vec8<T>::load(grad + (size_t)r * d + c, a);
      Vec8<T>::load(vals + (size_t)u * d + c, b);
#pragma unroll
      for (int i = 0; i < 8; ++i) a[i] += b[i];
      Vec8<T>::store(grad + (size_t)r * d + c, a);
    }
  }
}

// --------------------------------------------------------------------------------------------
// Cross-entropy over [rows, vocab] logits.  One CTA per row, two passes: online max / sum-exp, then
// dlogits = (softmax - onehot) * gscale written in place (or to `dlogits`).  loss[row] = lse - logit[label];
// rows with label == ignore give loss 0 and zero gradient.  `ld` = row stride in elements.
template <typename T>
__global__ void __launch_bounds__(512)
xent_kernel(const T* __restrict__ logits, const int64_t* __restrict__ labels, float* __restrict__ loss,
            T* __restrict__ dlogits, int rows, int vocab, int ld, float gscale_host, const float* __restrict__ gscale_dev,
            int64_t ignore_index) {
  __shared__ float sh[32];
  const float gscale = gscale_dev ? gscale_host * (*gscale_dev) : gscale_host;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* lp = logits + (size_t)row * ld;
    T* dp = dlogits ? dlogits + (size_t)row * ld : nullptr;
    const int64_t label = labels[row];
    const bool valid = label != ignore_index && label >= 0 && label < vocab;
    float m = -INFINITY, s = 0.f;
    const int nv = vocab / 8;                       // vector body; tail handled scalar
    const bool vec_ok = (ld % 8 == 0);
    if (vec_ok) {
      for (int v = threadIdx.x; v < nv; v += blockDim.x) {
        float x[8];
        Vec8<T>::load(lp + (size_t)v * 8, x);
        float mx = x[0];
#pragma unroll
        for (int i = 1; i < 8; ++i) mx = fmaxf(mx, x[i]);
        const float nm = fmaxf(m, mx);
        float add = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) add += __expf(x[i] - nm);
        s = s * __expf(m - nm) + add;
        m = nm;
      }
    }
    for (int c = (vec_ok ? nv * 8 : 0) + threadIdx.x; c < vocab; c += blockDim.x) {
      const float x = ZenVal<T>::to_f(lp[c]);
      const float nm = fmaxf(m, x);
      s = s * __expf(m - nm) + __expf(x - nm);
      m = nm;
    }
    const float gm = block_max(m, sh);
    s = (m == -INFINITY) ? 0.f : s * __expf(m - gm);
    const float gs = block_sum(s, sh);
    const float lse = gm + logf(gs);
    if (threadIdx.x == 0) loss[row] = valid ? lse - ZenVal<T>::to_f(lp[label]) : 0.f;
    if (dp) {
      const float sc = valid ? gscale : 0.f;
      if (vec_ok) {
        for (int v = threadIdx.x; v < nv; v += blockDim.x) {
          float x[8];
          Vec8<T>::load(lp + (size_t)v * 8, x);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            float p = __expf(x[i] - lse);
            if (v * 8 + i == label) p -= 1.f;
            x[i] = p * sc;
          }
          Vec8<T>::store(dp + (size_t)v * 8, x);
        }
      }
      for (int c = (vec_ok ? nv * 8 : 0) + threadIdx.x; c < vocab; c += blockDim.x) {
        float p = __expf(ZenVal<T>::to_f(lp[c]) - lse);
        if (c == label) p -= 1.f;
        dp[c] = ZenVal<T>::from_f(p * sc);
      }
    }
  }
}

// Vocabulary-parallel cross-entropy, two kernels around the small cross-rank reductions:
//   xent_partial_kernel : per row, max and sum-exp over this rank's vocabulary shard (columns >= valid_cols are
//                         padding and ignored), plus the target logit when the label falls in the shard
//   xent_apply_kernel   : dlogits = (exp(x - lse) - onehot) * scale in place, with the global lse of each row
template <typename T>
__global__ void __launch_bounds__(512)
xent_partial_kernel(const T* __restrict__ logits, const int64_t* __restrict__ labels, float* __restrict__ rowmax,
                    float* __restrict__ sumexp, float* __restrict__ target, int rows, int valid_cols, int ld,
                    int64_t vocab_start, int64_t ignore_index) {
  __shared__ float sh[32];
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* lp = logits + (size_t)row * ld;
    float m = -INFINITY, s = 0.f;
    for (int c = threadIdx.x; c < valid_cols; c += blockDim.x) {
      const float x = ZenVal<T>::to_f(lp[c]);
      const float nm = fmaxf(m, x);
      s = s * __expf(m - nm) + __expf(x - nm);
      m = nm;
    }
    const float gm = block_max(m, sh);
    s = (m == -INFINITY) ? 0.f : s * __expf(m - gm);
    const float gs = block_sum(s, sh);
    if (threadIdx.x == 0) {
      rowmax[row] = gm;
      sumexp[row] = gs;
      const int64_t lab = labels[row] - vocab_start;
      target[row] = (labels[row] != ignore_index && lab >= 0 && lab < valid_cols) ? ZenVal<T>::to_f(lp[lab]) : 0.f;
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(512)
xent_apply_kernel(T* __restrict__ logits, const int64_t* __restrict__ labels, const float* __restrict__ lse,
                  int rows, int cols, int valid_cols, int ld, float gscale_host, const float* __restrict__ gscale_dev,
                  int64_t vocab_start, int64_t ignore_index) {
  const float gscale = gscale_dev ? gscale_host * (*gscale_dev) : gscale_host;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    T* lp = logits + (size_t)row * ld;
    const bool valid = labels[row] != ignore_index;
    const int64_t lab = labels[row] - vocab_start;
    const float l = lse[row], sc = valid ? gscale : 0.f;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) {
      float pr = (c < valid_cols) ? __expf(ZenVal<T>::to_f(lp[c]) - l) : 0.f;
      if (c == lab) pr -= 1.f;
      lp[c] = ZenVal<T>::from_f(pr * sc);
    }
  }
}

// --------------------------------------------------------------------------------------------
// Multi-tensor AdamW.  One table entry per tensor; CTAs walk a flat list of 64K-element chunks.
struct AdamTensor {
  void* param;       // T (bf16 / fp32) weights used by the model
  float* master;     // optional fp32 master copy (null when param is fp32)
  const void* grad;  // T gradient
  float* m;
  float* v;
  uint64_t numel;
  uint64_t chunk0;   // index of this tensor's first chunk
  float wd;          // weight decay for this tensor
  float pad;
};
#define ADAM_CHUNK 65536

// One AdamW element update.  The square root and the quotient use the approximate units (about 2 ulp): the update is
// rounded to bf16 (or added to an fp32 master) right after, and the exact sequences cost several times the
// instructions, enough to show against the 22 bytes per element this kernel moves.
__device__ __forceinline__ void adam_update(float& p, float& m, float& v, float g, float b1, float b2, float eps,
                                            float ibc1, float isb2, float decay, float lr) {
  m = b1 * m + (1.f - b1) * g;
  v = b2 * v + (1.f - b2) * g * g;
  float sq;
  asm("sqrt.approx.f32 %0, %1;" : "=f"(sq) : "f"(v));
  const float den = fmaf(sq, isb2, eps);
  p = fmaf(-lr, __fdividef(m * ibc1, den), p * decay);
}

template <typename T>
__global__ void __launch_bounds__(256)
adamw_kernel(const AdamTensor* __restrict__ tab, int ntensors, const int32_t* __restrict__ chunk_tensor,
             uint64_t nchunks, float lr, float b1, float b2, float eps, float bc1, float bc2, float gscale,
             const int32_t* __restrict__ step_dev) {
  if (step_dev) {                        // step count kept on the device (CUDA-graph replay): derive the bias corrections here
    const float t = (float)(*step_dev);
    bc1 = 1.f - powf(b1, t);
    bc2 = 1.f - powf(b2, t);
  }
  const float ibc1 = 1.f / bc1, isb2 = rsqrtf(bc2);
  for (uint64_t ch = blockIdx.x; ch < nchunks; ch += gridDim.x) {
    const AdamTensor t = tab[chunk_tensor[ch]];
    const uint64_t start = (ch - t.chunk0) * ADAM_CHUNK;
    const uint64_t end = min(t.numel, start + ADAM_CHUNK);
    T* p = reinterpret_cast<T*>(t.param);
    const T* g = reinterpret_cast<const T*>(t.grad);
    const float decay = 1.f - lr * t.wd;
    // two 8-element vectors per thread and trip, all loads issued before the arithmetic
    for (uint64_t i0 = start + (uint64_t)threadIdx.x * 8; i0 < end; i0 += 2 * 256 * 8) {
      const uint64_t i1 = i0 + 256 * 8;
      if (i1 + 8 <= end) {
        float pv[2][8], gv[2][8], mv[2][8], vv[2][8];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const uint64_t i = u ? i1 : i0;
          if (t.master) Vec8<float>::load(t.master + i, pv[u]); else Vec8<T>::load(p + i, pv[u]);
          Vec8<T>::load(g + i, gv[u]);
          Vec8<float>::load(t.m + i, mv[u]);
          Vec8<float>::load(t.v + i, vv[u]);
        }
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const uint64_t i = u ? i1 : i0;
#pragma unroll
          for (int k = 0; k < 8; ++k) adam_update(pv[u][k], mv[u][k], vv[u][k], gv[u][k] * gscale, b1, b2, eps, ibc1, isb2, decay, lr);
          Vec8<float>::store(t.m + i, mv[u]);
          Vec8<float>::store(t.v + i, vv[u]);
          if (t.master) Vec8<float>::store(t.master + i, pv[u]);
          Vec8<T>::store(p + i, pv[u]);
        }
        continue;
      }
      for (int u = 0; u < 2; ++u) {
        const uint64_t i = u ? i1 : i0;
        if (i >= end) break;
        if (i + 8 <= end) {
          float pv[8], gv[8], mv[8], vv[8];
          if (t.master) Vec8<float>::load(t.master + i, pv); else Vec8<T>::load(p + i, pv);
          Vec8<T>::load(g + i, gv);
          Vec8<float>::load(t.m + i, mv);
          Vec8<float>::load(t.v + i, vv);
#pragma unroll
          for (int k = 0; k < 8; ++k) adam_update(pv[k], mv[k], vv[k], gv[k] * gscale, b1, b2, eps, ibc1, isb2, decay, lr);
          Vec8<float>::store(t.m + i, mv);
          Vec8<float>::store(t.v + i, vv);
          if (t.master) Vec8<float>::store(t.master + i, pv);
          Vec8<T>::store(p + i, pv);
        } else {
          for (uint64_t k = i; k < end; ++k) {
            float pv = t.master ? t.master[k] : ZenVal<T>::to_f(p[k]);
            float mm = t.m[k], vv = t.v[k];
            adam_update(pv, mm, vv, ZenVal<T>::to_f(g[k]) * gscale, b1, b2, eps, ibc1, isb2, decay, lr);
            t.m[k] = mm; t.v[k] = vv;
            if (t.master) t.master[k] = pv;
            p[k] = ZenVal<T>::from_f(pv);
          }
        }
      }
    }
  }
}

int sm_count_e() {
  static int n = 0;
  if (!n) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}
inline int cap_grid(size_t want, int mult) {
  size_t mx = (size_t)sm_count_e() * mult;
  return (int)(want < 1 ? 1 : (want > mx ? mx : want));
}

}  // namespace

#define DISPATCH_T(dtype, ...)                                             \
  switch (dtype) {                                                         \
    case ZEN_DTYPE_F32: { using T = float; __VA_ARGS__; } break;           \
    case ZEN_DTYPE_BF16: { using T = __nv_bfloat16; __VA_ARGS__; } break;  \
    case ZEN_DTYPE_F16: { using T = __half; __VA_ARGS__; } break;          \
    default: return -1;                                                    \
  }

extern "C" {

// Rows of at most NORMW_MAXCOLS columns use the warp-per-row kernels, wider rows the CTA-per-row kernels.

#define NORMW_MAXCOLS 1024
static inline bool norm_warp_path(int cols, int dtype) { (void)dtype; return cols <= NORMW_MAXCOLS; }

// Number of per-CTA partial rows the norm backward writes (the caller sizes its scratch with this).
int zen_norm_bwd_parts(int rows) { const int a = cap_grid((size_t)rows, 2), b = (rows + 7) / 8; return a > b ? a : b; }

#define NORM_NV_DISPATCH(cols, ...)                                   \
  if (cols <= NORM_THREADS * 8) { constexpr int NV = 1; __VA_ARGS__; } \
  else if (cols <= NORM_THREADS * 16) { constexpr int NV = 2; __VA_ARGS__; } \
  else if (cols <= NORM_THREADS * 32) { constexpr int NV = 4; __VA_ARGS__; } \
  else { constexpr int NV = 8; __VA_ARGS__; }
#define NORMW_NV_DISPATCH(cols, ...)                        \
  if (cols <= 256) { constexpr int NV = 1; __VA_ARGS__; }   \
  else if (cols <= 512) { constexpr int NV = 2; __VA_ARGS__; } \
  else if (cols <= 768) { constexpr int NV = 3; __VA_ARGS__; } \
  else { constexpr int NV = 4; __VA_ARGS__; }

int zen_norm_fwd(const void* x, const void* res, const void* w, const void* b, void* y, void* hout, float* rstd,
                 float* mean, int rows, int cols, float eps, int layer, int unit_offset, int dtype, void* stream) {
  if (cols % 8 || cols > NORM_THREADS * NORM_MAXV * 8) return -2;
  cudaStream_t st = (cudaStream_t)stream;
  if (norm_warp_path(cols, dtype)) {
    const int grid = cap_grid((size_t)(rows + NORMW_WARPS - 1) / NORMW_WARPS, 8);
    DISPATCH_T(dtype, {
      NORMW_NV_DISPATCH(cols, {
        if (layer) norm_fwd_warp_kernel<T, true, NV><<<grid, NORMW_WARPS * 32, 0, st>>>((const T*)x, (const T*)res, (const T*)w, (const T*)b, (T*)y, (T*)hout, rstd, mean, rows, cols, eps, unit_offset);
        else norm_fwd_warp_kernel<T, false, NV><<<grid, NORMW_WARPS * 32, 0, st>>>((const T*)x, (const T*)res, (const T*)w, (const T*)b, (T*)y, (T*)hout, rstd, mean, rows, cols, eps, unit_offset);
      });
    });
    return (int)cudaGetLastError();
  }
  const int grid = cap_grid((size_t)rows, 16);
  DISPATCH_T(dtype, {
    NORM_NV_DISPATCH(cols, {
      if (layer) norm_fwd_kernel<T, true, NV><<<grid, NORM_THREADS, 0, st>>>((const T*)x, (const T*)res, (const T*)w, (const T*)b, (T*)y, (T*)hout, rstd, mean, rows, cols, eps, unit_offset);
      else norm_fwd_kernel<T, false, NV><<<grid, NORM_THREADS, 0, st>>>((const T*)x, (const T*)res, (const T*)w, (const T*)b, (T*)y, (T*)hout, rstd, mean, rows, cols, eps, unit_offset);
    });
  });
  return (int)cudaGetLastError();
}

// part_dw / part_db: fp32 scratch of zen_norm_bwd_parts(rows) * cols each.  dw / db are written (or
// accumulated into when accumulate != 0) in dtype.
int zen_norm_bwd_ex(const void* dy, const void* h, const void* w, const float* rstd, const float* mean, const void* dres,
                    void* dh, float* part_dw, float* part_db, void* dw, void* db, int rows, int cols, int layer,
                    int unit_offset, int accumulate, int dtype, int skip_reduce, void* stream);

int zen_norm_bwd(const void* dy, const void* h, const void* w, const float* rstd, const float* mean, const void* dres,
                 void* dh, float* part_dw, float* part_db, void* dw, void* db, int rows, int cols, int layer,
                 int unit_offset, int accumulate, int dtype, void* stream) {
  return zen_norm_bwd_ex(dy, h, w, rstd, mean, dres, dh, part_dw, part_db, dw, db, rows, cols, layer, unit_offset, accumulate,
                         dtype, 0, stream);
}

// Rows per CTA of the column-sum pass of the wide-row norm backward: 32, fewer when that would leave SMs idle.
static int norm_wide_rpc(int rows) {
  int rpc = 32;
  while (rpc > 8 && (rows + rpc - 1) / rpc < 4 * sm_count_e() && (rows + rpc / 2 - 1) / (rpc / 2) <= zen_norm_bwd_parts(rows)) rpc /= 2;
  return rpc;
}
// Partial rows that zen_norm_bwd_ex leaves in part_dw / part_db for a matrix of this shape.
int zen_norm_bwd_parts_used(int rows, int cols) {
  if (norm_warp_path(cols, 0)) return (rows + 31) / 32;
  const int rpc = norm_wide_rpc(rows);
  return (rows + rpc - 1) / rpc;
}

// skip_reduce != 0: leave the partial sums in part_dw / part_db (zen_norm_bwd_parts_used(rows, cols) rows of cols floats)
// for a later zen_colreduce_multi; dw / db are not touched.
int zen_norm_bwd_ex(const void* dy, const void* h, const void* w, const float* rstd, const float* mean, const void* dres,
                    void* dh, float* part_dw, float* part_db, void* dw, void* db, int rows, int cols, int layer,
                    int unit_offset, int accumulate, int dtype, int skip_reduce, void* stream) {
  if (cols % 8 || cols > NORM_THREADS * NORM_MAXV * 8) return -2;
  cudaStream_t st = (cudaStream_t)stream;
  const int grid = cap_grid((size_t)rows, 2);
  if (norm_warp_path(cols, dtype)) {
    // dh by warp-per-row (light on registers, many rows in flight), then dw / db by a column-sum pass
    const int g1 = cap_grid((size_t)(rows + NORMW_WARPS - 1) / NORMW_WARPS, 8);
    const int parts = (rows + 31) / 32;
    DISPATCH_T(dtype, {
      NORMW_NV_DISPATCH(cols, {
        if (layer) norm_bwd_warp_kernel<T, true, NV, false><<<g1, NORMW_WARPS * 32, 0, st>>>((const T*)dy, (const T*)h, (const T*)w, rstd, mean, (const T*)dres, (T*)dh, part_dw, part_db, rows, cols, unit_offset);
        else norm_bwd_warp_kernel<T, false, NV, false><<<g1, NORMW_WARPS * 32, 0, st>>>((const T*)dy, (const T*)h, (const T*)w, rstd, mean, (const T*)dres, (T*)dh, part_dw, part_db, rows, cols, unit_offset);
      });
      if (layer) norm_dwdb_partial_kernel<T, true><<<dim3(parts, (cols + 2047) / 2048), 256, 0, st>>>((const T*)dy, (const T*)h, rstd, mean, part_dw, part_db, rows, cols, 32);
      else norm_dwdb_partial_kernel<T, false><<<dim3(parts, (cols + 2047) / 2048), 256, 0, st>>>((const T*)dy, (const T*)h, rstd, mean, part_dw, part_db, rows, cols, 32);
      if (skip_reduce) {}
      else if (layer && db) colreduce_kernel<T><<<dim3((cols + 31) / 32, 2), 1024, 0, st>>>(part_dw, (T*)dw, parts, cols, accumulate, part_db, (T*)db);
      else colreduce_kernel<T><<<(cols + 31) / 32, 1024, 0, st>>>(part_dw, (T*)dw, parts, cols, accumulate);
    });
    return (int)cudaGetLastError();
  }
  (void)grid;
  // wide rows: dh by one CTA per row (no parameter accumulators, so several CTAs fit an SM), then dw / db by the
  // column-sum pass, as on the warp path
  const int g2 = cap_grid((size_t)rows, 6);
  // rows per CTA of the column-sum pass: 32, fewer when that would leave SMs idle (the partial buffer holds
  // zen_norm_bwd_parts(rows) rows)
  const int rpc = norm_wide_rpc(rows);
  const int parts = (rows + rpc - 1) / rpc;
  DISPATCH_T(dtype, {
    NORM_NV_DISPATCH(cols, {
      if (layer) norm_bwd_kernel<T, true, NV, false><<<g2, NORM_THREADS, 0, st>>>((const T*)dy, (const T*)h, (const T*)w, rstd, mean, (const T*)dres, (T*)dh, part_dw, part_db, rows, cols, unit_offset);
      else norm_bwd_kernel<T, false, NV, false><<<g2, NORM_THREADS, 0, st>>>((const T*)dy, (const T*)h, (const T*)w, rstd, mean, (const T*)dres, (T*)dh, part_dw, part_db, rows, cols, unit_offset);
    });
    if (layer) norm_dwdb_partial_kernel<T, true><<<dim3(parts, (cols + 2047) / 2048), 256, 0, st>>>((const T*)dy, (const T*)h, rstd, mean, part_dw, part_db, rows, cols, rpc);
    else norm_dwdb_partial_kernel<T, false><<<dim3(parts, (cols + 2047) / 2048), 256, 0, st>>>((const T*)dy, (const T*)h, rstd, mean, part_dw, part_db, rows, cols, rpc);
    if (skip_reduce) {}
    else if (layer && db) colreduce_kernel<T><<<dim3((cols + 31) / 32, 2), 1024, 0, st>>>(part_dw, (T*)dw, parts, cols, accumulate, part_db, (T*)db);
    else colreduce_kernel<T><<<(cols + 31) / 32, 1024, 0, st>>>(part_dw, (T*)dw, parts, cols, accumulate);
  });
  return (int)cudaGetLastError();
}

int zen_colsum_parts(int rows) { return (rows + COLSUM_ROWS - 1) / COLSUM_ROWS; }

// out[c] (+)= sum_r a[r][c]; part: fp32 scratch zen_colsum_parts(rows) * cols.
int zen_colsum(const void* a, float* part, void* out, int rows, int cols, int accumulate, int dtype, void* stream) {
  if (cols % 8) return -2;
  cudaStream_t st = (cudaStream_t)stream;
  const int parts = zen_colsum_parts(rows);
  DISPATCH_T(dtype, {
    colsum_partial_kernel<T><<<parts, 256, 0, st>>>((const T*)a, part, rows, cols);
    colreduce_kernel<T><<<(cols + 31) / 32, 1024, 0, st>>>(part, (T*)out, parts, cols, accumulate);
  });
  return (int)cudaGetLastError();
}

int zen_act_fwd(const void* a, const void* b, void* out, int rows, int inner, int lda, int ldb, int mode, int dtype,
                void* stream) {
  if (inner % 8 || lda % 8 || ldb % 8) return -2;
  const int grid = cap_grid(((size_t)rows * (inner / 8) + 255) / 256, 16);
  DISPATCH_T(dtype, act_fwd_kernel<T><<<grid, 256, 0, (cudaStream_t)stream>>>((const T*)a, (const T*)b, (T*)out, rows, inner, lda, ldb, mode));
  return (int)cudaGetLastError();
}

int zen_act_bwd(const void* a, const void* b, const void* dout, void* da, void* db, int rows, int inner, int lda,
                int ldb, int mode, int dtype, void* stream) {
  if (inner % 8 || lda % 8 || ldb % 8) return -2;
  const int grid = cap_grid(((size_t)rows * (inner / 8) + 255) / 256, 16);
  DISPATCH_T(dtype, act_bwd_kernel<T><<<grid, 256, 0, (cudaStream_t)stream>>>((const T*)a, (const T*)b, (const T*)dout, (T*)da, (T*)db, rows, inner, lda, ldb, mode));
  return (int)cudaGetLastError();
}

// Rows per CTA of zen_act_bwd_colsum: three CTAs per SM, all resident at once and evenly loaded, at least 8 rows each.
static int act_colsum_rows_per_cta(int rows) {
  const int target = sm_count_e() * 3;
  const int rpc = (rows + target - 1) / target;
  return rpc < 8 ? 8 : rpc;
}
int zen_act_colsum_parts(int rows) { const int rpc = act_colsum_rows_per_cta(rows); return (rows + rpc - 1) / rpc; }

// Ungated activation backward (mode 0 gelu_tanh, 1 relu) on dense [rows, inner] tensors that also writes the partial
// column sums of da: part[zen_act_colsum_parts(rows)][inner] floats, to be summed by zen_colsum_reduce.
int zen_act_bwd_colsum(const void* a, const void* dout, void* da, float* part, int rows, int inner, int mode, int dtype,
                       void* stream) {
  if (inner % 8 || mode < 0 || mode > 1) return -2;
  if (rows <= 0) return 0;
  int threads = ((inner / 8 + 31) / 32) * 32;
  if (threads > 512) threads = 512;
  const int rpc = act_colsum_rows_per_cta(rows);
  DISPATCH_T(dtype, act_bwd_colsum_kernel<T><<<(rows + rpc - 1) / rpc, threads, 0, (cudaStream_t)stream>>>((const T*)a, (const T*)dout, (T*)da, part, rows, inner, mode, rpc));
  return (int)cudaGetLastError();
}

// First half of zen_colsum only: part[zen_colsum_parts(rows)][cols] partial column sums of a.
int zen_colsum_partial(const void* a, float* part, int rows, int cols, int dtype, void* stream) {
  if (cols % 8) return -2;
  DISPATCH_T(dtype, colsum_partial_kernel<T><<<zen_colsum_parts(rows), 256, 0, (cudaStream_t)stream>>>((const T*)a, part, rows, cols));
  return (int)cudaGetLastError();
}

// Up to COLREDUCE_MAX_JOBS reductions out[c] (+)= sum_p part[p][c] in ONE launch; a job may carry a second (part2, out2)
// pair of the same shape.  All outputs have type `dtype`.
int zen_colreduce_job_size() { return (int)sizeof(ColReduceJob); }
int zen_colreduce_max_jobs() { return COLREDUCE_MAX_JOBS; }
int zen_colreduce_multi(const void* jobs_, int n, int dtype, void* stream) {
  const ColReduceJob* jobs = static_cast<const ColReduceJob*>(jobs_);      // records of zen_colreduce_job_size() bytes
  if (!jobs || n < 1 || n > COLREDUCE_MAX_JOBS) return -2;
  ColReduceJobs t;
  int max_cols = 0;
  for (int i = 0; i < n; ++i) {
    t.j[i] = jobs[i];
    if (jobs[i].nparts <= 0 || jobs[i].cols <= 0 || !jobs[i].part || !jobs[i].out) return -2;
    if (jobs[i].cols > max_cols) max_cols = jobs[i].cols;
  }
  for (int i = n; i < COLREDUCE_MAX_JOBS; ++i) t.j[i] = ColReduceJob{nullptr, nullptr, nullptr, nullptr, 0, 0, 0, 0};
  t.n = n;
  DISPATCH_T(dtype, colreduce_multi_kernel<T><<<dim3((max_cols + 31) / 32, 2 * n), 1024, 0, (cudaStream_t)stream>>>(t));
  return (int)cudaGetLastError();
}

// out[c] (+)= sum over p of part[p][c]: the second half of zen_colsum for partial sums that another kernel produced.
int zen_colsum_reduce(const float* part, void* out, int parts, int cols, int accumulate, int dtype, void* stream) {
  if (parts <= 0 || cols <= 0) return -2;
  DISPATCH_T(dtype, colreduce_kernel<T><<<(cols + 31) / 32, 1024, 0, (cudaStream_t)stream>>>(part, (T*)out, parts, cols, accumulate));
  return (int)cudaGetLastError();
}

int zen_rope(void* x, int tokens, int heads, int hd, int ld, int seq, int pos0, float theta, int inverse, int dtype,
             void* stream) {
  if (hd % 2) return -2;
  const size_t n = (size_t)tokens * heads * (hd / 2);
  const int grid = cap_grid((n + 255) / 256, 16);
  if ((hd / 2) % 8 == 0 && (ld % 8) == 0 && (reinterpret_cast<uintptr_t>(x) % 16) == 0) {
    const size_t nvec = (size_t)tokens * (hd / 16);
    const int gv = cap_grid((nvec + 255) / 256, 16);
    DISPATCH_T(dtype, rope_vec_kernel<T><<<gv, 256, 0, (cudaStream_t)stream>>>((T*)x, tokens, heads, hd, ld, seq, pos0, log2f(theta), inverse ? -1.f : 1.f));
    return (int)cudaGetLastError();
  }
  DISPATCH_T(dtype, rope_kernel<T><<<grid, 256, 0, (cudaStream_t)stream>>>((T*)x, tokens, heads, hd, ld, seq, pos0, log2f(theta), inverse ? -1.f : 1.f));
  return (int)cudaGetLastError();
}

int zen_embedding_fwd(const int64_t* ids, const void* wte, const void* wpe, void* out, int tokens, int d, int seq,
                      int pos_offset, float scale, int vocab, int dtype, void* stream) {
  if (d % 8) return -2;
  DISPATCH_T(dtype, embedding_fwd_kernel<T><<<cap_grid((size_t)tokens, 32), 128, 0, (cudaStream_t)stream>>>(ids, (const T*)wte, (const T*)wpe, (T*)out, tokens, d, seq, pos_offset, scale, vocab));
  return (int)cudaGetLastError();
}

// Row-sparse embedding backward.  Scratch owned by the caller and zero on entry (this call leaves it
// zero again): flag_cid int32[vocab], acc fp32[max_rows][d].  Outputs: rows int32[max_rows] (ascending
// unique ids), count int32[1], vals T[max_rows][d].  max_rows >= min(tokens, vocab).
int zen_embedding_bwd_rows(const int64_t* ids, const void* dy, int32_t* flag_cid, float* acc, int32_t* rows,
                           int32_t* count, void* vals, int tokens, int d, int vocab, float scale, int dtype,
                           void* stream) {
  if (d % 8) return -2;
  cudaStream_t st = (cudaStream_t)stream;
  embed_mark_kernel<<<cap_grid(((size_t)tokens + 255) / 256, 8), 256, 0, st>>>(ids, flag_cid, tokens, vocab);
  embed_compact_kernel<<<1, 1024, 0, st>>>(flag_cid, rows, count, vocab);
  DISPATCH_T(dtype, {
    embed_accum_kernel<T><<<cap_grid((size_t)tokens, 32), 128, 0, st>>>(ids, flag_cid, (const T*)dy, acc, tokens, d, vocab, scale);
    embed_finish_kernel<T><<<cap_grid((size_t)(tokens < vocab ? tokens : vocab), 32), 128, 0, st>>>(acc, flag_cid, rows, count, (T*)vals, d);
  });
  embed_clear_flags_kernel<<<cap_grid(((size_t)vocab + 255) / 256, 8), 256, 0, st>>>(flag_cid, vocab);
  return (int)cudaGetLastError();
}

int zen_rows_add(void* grad, const int32_t* rows, const int32_t* count, const void* vals, int d, int vocab,
                 int max_rows, int dtype, void* stream) {
  if (d % 8) return -2;
  DISPATCH_T(dtype, rows_add_kernel<T><<<cap_grid((size_t)max_rows, 32), 128, 0, (cudaStream_t)stream>>>((T*)grad, rows, count, (const T*)vals, d, vocab, max_rows));
  return (int)cudaGetLastError();
}

// gscale_dev (optional device float) multiplies gscale; lets the caller scale by 1 / (valid tokens) without a host sync.
int zen_xent(const void* logits, const int64_t* labels, float* loss, void* dlogits, int rows, int vocab, int ld,
             float gscale, const float* gscale_dev, int64_t ignore_index, int dtype, void* stream) {
  DISPATCH_T(dtype, xent_kernel<T><<<cap_grid((size_t)rows, 8), 512, 0, (cudaStream_t)stream>>>((const T*)logits, labels, loss, (T*)dlogits, rows, vocab, ld, gscale, gscale_dev, ignore_index));
  return (int)cudaGetLastError();
}

int zen_xent_partial(const void* logits, const int64_t* labels, float* rowmax, float* sumexp, float* target, int rows,
                     int valid_cols, int ld, int64_t vocab_start, int64_t ignore_index, int dtype, void* stream) {
  DISPATCH_T(dtype, xent_partial_kernel<T><<<cap_grid((size_t)rows, 8), 512, 0, (cudaStream_t)stream>>>((const T*)logits, labels, rowmax, sumexp, target, rows, valid_cols, ld, vocab_start, ignore_index));
  return (int)cudaGetLastError();
}

int zen_xent_apply(void* logits, const int64_t* labels, const float* lse, int rows, int cols, int valid_cols, int ld,
                   float gscale, const float* gscale_dev, int64_t vocab_start, int64_t ignore_index, int dtype, void* stream) {
  DISPATCH_T(dtype, xent_apply_kernel<T><<<cap_grid((size_t)rows, 8), 512, 0, (cudaStream_t)stream>>>((T*)logits, labels, lse, rows, cols, valid_cols, ld, gscale, gscale_dev, vocab_start, ignore_index));
  return (int)cudaGetLastError();
}

int zen_adam_tensor_size() { return (int)sizeof(AdamTensor); }

// step_dev (optional): device int32 holding the 1-based step count; when given, bc1 / bc2 are ignored and computed
// from it inside the kernel, so that a captured launch stays correct across replays.
int zen_adamw(const void* table, int ntensors, const int32_t* chunk_tensor, uint64_t nchunks, float lr, float b1,
              float b2, float eps, float bc1, float bc2, float gscale, const int32_t* step_dev, int dtype, void* stream) {
  const int grid = cap_grid((size_t)nchunks, 8);
  DISPATCH_T(dtype, adamw_kernel<T><<<grid, 256, 0, (cudaStream_t)stream>>>((const AdamTensor*)table, ntensors, chunk_tensor, nchunks, lr, b1, b2, eps, bc1, bc2, gscale, step_dev));
  return (int)cudaGetLastError();
}

}  // extern "C"

// ------------------------------------------------------------------------------------------------
// Allocation-free column sum (declared in zen_noalloc.h, which says who needs it and why).
#include "zen_noalloc.h"

#include <mutex>
#include <stdio.h>

// Scratch of the allocation-free entry point: per-CTA partial sums, [ceil(rows / 32)][cols] floats.
// In host code this name is only a handle for cudaGetSymbolAddress, never a pointer to hand to a kernel.
static __device__ __align__(256) float g_colsum_noalloc_scratch[ZEN_COLSUM_NOALLOC_MAX_FLOATS];

namespace {
constexpr int kMaxDevices = 64;
float* g_noalloc_ptr[kMaxDevices] = {nullptr};   // device address of the scratch, per device
std::mutex g_noalloc_mu;
thread_local char g_noalloc_err[256] = "";

int noalloc_fail(int code, const char* what) {
  snprintf(g_noalloc_err, sizeof(g_noalloc_err), "%s", what);
  return code;
}

// Device address of the scratch array on the current device; looked up once per device.
int noalloc_scratch(float** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return noalloc_fail((int)e, cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices) return noalloc_fail(ZEN_NOALLOC_BAD_ARG, "device index out of range");
  std::lock_guard<std::mutex> g(g_noalloc_mu);
  if (!g_noalloc_ptr[dev]) {
    float* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_colsum_noalloc_scratch);
    if (e != cudaSuccess) return noalloc_fail((int)e, cudaGetErrorString(e));
    g_noalloc_ptr[dev] = p;
  }
  *out = g_noalloc_ptr[dev];
  return 0;
}
}  // namespace

extern "C" {

const char* zen_noalloc_last_error(void) { return g_noalloc_err; }

int zen_colsum_noalloc(const void* a, void* out, int rows, int cols, int accumulate, int dtype, void* stream) {
  if (!a || !out || rows <= 0 || cols <= 0) return noalloc_fail(ZEN_NOALLOC_BAD_ARG, "null pointer or empty matrix");
  if (cols % 8) return noalloc_fail(ZEN_NOALLOC_BAD_ARG, "cols must be a multiple of 8");
  if (reinterpret_cast<uintptr_t>(a) % 16) return noalloc_fail(ZEN_NOALLOC_BAD_ARG, "input must be 16-byte aligned");
  if (dtype < 0 || dtype > 2) return noalloc_fail(ZEN_NOALLOC_BAD_ARG, "dtype must be 0 (fp32), 1 (bf16) or 2 (fp16)");
  const int parts = (rows + COLSUM_ROWS - 1) / COLSUM_ROWS;
  if ((uint64_t)parts * (uint64_t)cols > (uint64_t)ZEN_COLSUM_NOALLOC_MAX_FLOATS) {
    snprintf(g_noalloc_err, sizeof(g_noalloc_err),
             "scratch of %llu floats needed for %d x %d, the built-in array holds %u: use zen_colsum with caller scratch",
             (unsigned long long)parts * cols, rows, cols, (unsigned)ZEN_COLSUM_NOALLOC_MAX_FLOATS);
    return ZEN_NOALLOC_TOO_LARGE;
  }
  float* part = nullptr;
  int rc = noalloc_scratch(&part);
  if (rc) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  DISPATCH_T(dtype, {
    colsum_partial_kernel<T><<<parts, 256, 0, st>>>((const T*)a, part, rows, cols);
    colreduce_kernel<T><<<(cols + 31) / 32, 1024, 0, st>>>(part, (T*)out, parts, cols, accumulate);
  });
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return noalloc_fail((int)e, cudaGetErrorString(e));
  return 0;
}

}  // extern "C"
