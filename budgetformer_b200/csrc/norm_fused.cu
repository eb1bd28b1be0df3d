// Bandwidth-bound row kernels: LayerNorm forward / backward (one warp per row, fp32 statistics,
// 16-bit or fp32 activations) and counter-based dropout whose keep mask is a pure function of
// (seed, row, col) - the same function the GEMM epilogue applies - so that backward regenerates
// the mask instead of storing it.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "bf_kernels.h"

namespace {

template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_f<__half>(__half v) { return __half2float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half from_f<__half>(float v) { return __float2half_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

constexpr int LN_MAX_PER_LANE = 16;   // h <= 512

// Column owned by (lane, i): contiguous chunks of `per` elements per lane when h == 32*per (vector-friendly,
// the common case h = 64/128/256/512), otherwise lane-strided.
__device__ __forceinline__ int ln_col(int lane, int i, int per, bool packed) { return packed ? lane * per + i : lane + 32 * i; }

template <typename T, int PER>
__device__ __forceinline__ void ln_load_row(const T* __restrict__ p, int lane, float* v) {
  // PER contiguous elements starting at p + lane*PER, loaded as one or more 16/8/4-byte vectors
  constexpr int BYTES = PER * (int)sizeof(T);
  const T* q = p + lane * PER;
  if constexpr (BYTES % 16 == 0) {
    __align__(16) T tmp[PER];
#pragma unroll
    for (int j = 0; j < BYTES / 16; ++j) reinterpret_cast<uint4*>(tmp)[j] = reinterpret_cast<const uint4*>(q)[j];
#pragma unroll
    for (int i = 0; i < PER; ++i) v[i] = to_f<T>(tmp[i]);
  } else if constexpr (BYTES % 8 == 0) {
    __align__(16) T tmp[PER];
#pragma unroll
    for (int j = 0; j < BYTES / 8; ++j) reinterpret_cast<uint2*>(tmp)[j] = reinterpret_cast<const uint2*>(q)[j];
#pragma unroll
    for (int i = 0; i < PER; ++i) v[i] = to_f<T>(tmp[i]);
  } else {
    __align__(16) T tmp[PER];
#pragma unroll
    for (int j = 0; j < BYTES / 4; ++j) reinterpret_cast<uint32_t*>(tmp)[j] = reinterpret_cast<const uint32_t*>(q)[j];
#pragma unroll
    for (int i = 0; i < PER; ++i) v[i] = to_f<T>(tmp[i]);
  }
}
template <typename T, int PER>
__device__ __forceinline__ void ln_store_row(T* __restrict__ p, int lane, const float* v) {
  constexpr int BYTES = PER * (int)sizeof(T);
  __align__(16) T tmp[PER];
#pragma unroll
  for (int i = 0; i < PER; ++i) tmp[i] = from_f<T>(v[i]);
  T* q = p + lane * PER;
  if constexpr (BYTES % 16 == 0) {
#pragma unroll
    for (int j = 0; j < BYTES / 16; ++j) reinterpret_cast<uint4*>(q)[j] = reinterpret_cast<const uint4*>(tmp)[j];
  } else if constexpr (BYTES % 8 == 0) {
#pragma unroll
    for (int j = 0; j < BYTES / 8; ++j) reinterpret_cast<uint2*>(q)[j] = reinterpret_cast<const uint2*>(tmp)[j];
  } else {
#pragma unroll
    for (int j = 0; j < BYTES / 4; ++j) reinterpret_cast<uint32_t*>(q)[j] = reinterpret_cast<const uint32_t*>(tmp)[j];
  }
}

// PER > 0: packed layout with h == 32*PER (rows must be 16-byte aligned); PER == 0: generic lane-strided layout.
template <typename T, int PER>
__global__ void __launch_bounds__(256) ln_fwd_kernel(const T* __restrict__ x, long long ldx, const float* __restrict__ gamma,
                                                     const float* __restrict__ beta, T* __restrict__ y, long long ldy,
                                                     float* __restrict__ stats, long long rows, int h, float eps) {
  constexpr int NV = PER > 0 ? PER : LN_MAX_PER_LANE;
  const int lane = threadIdx.x & 31;
  const long long warps = ((long long)gridDim.x * blockDim.x) >> 5;
  const int per = PER > 0 ? PER : (h + 31) / 32;
  for (long long row = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5; row < rows; row += warps) {
    const T* xr = x + row * ldx;
    float v[NV];
    if constexpr (PER > 0) {
      ln_load_row<T, PER>(xr, lane, v);
    } else {
#pragma unroll
      for (int i = 0; i < NV; ++i) { const int c = lane + 32 * i; v[i] = (i < per && c < h) ? to_f<T>(xr[c]) : 0.f; }
    }
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) s += v[i];
    const float mean = warp_sum(s) / h;
    float q = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = ln_col(lane, i, per, PER > 0);
      const float d = (i < per && c < h) ? v[i] - mean : 0.f;
      q += d * d;
    }
    const float rstd = rsqrtf(warp_sum(q) / h + eps);
    T* yr = y + row * ldy;
    if constexpr (PER > 0) {
      float o[NV];
#pragma unroll
      for (int i = 0; i < NV; ++i) { const int c = lane * PER + i; o[i] = (v[i] - mean) * rstd * gamma[c] + beta[c]; }
      ln_store_row<T, PER>(yr, lane, o);
    } else {
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const int c = lane + 32 * i;
        if (i < per && c < h) yr[c] = from_f<T>((v[i] - mean) * rstd * gamma[c] + beta[c]);
      }
    }
    if (lane == 0 && stats) { stats[2 * row] = mean; stats[2 * row + 1] = rstd; }
  }
}

// dx = rstd * (g*dy - mean(g*dy) - xhat * mean(g*dy*xhat)); dgamma += dy*xhat; dbeta += dy.
// Persistent grid: every warp walks many rows and keeps its dgamma/dbeta partials in registers, so the global
// atomics at the end number (blocks * h), not (rows * h / 128).
template <typename T, int PER>
__global__ void __launch_bounds__(256) ln_bwd_kernel(const T* __restrict__ dy, long long lddy, const T* __restrict__ x,
                                                     long long ldx, const float* __restrict__ stats,
                                                     const float* __restrict__ gamma, T* __restrict__ dx, long long lddx,
                                                     float* __restrict__ dgamma, float* __restrict__ dbeta,
                                                     long long rows, int h) {
  constexpr int NV = PER > 0 ? PER : LN_MAX_PER_LANE;
  extern __shared__ float s_acc[];      // [2, h]
  for (int i = threadIdx.x; i < 2 * h; i += blockDim.x) s_acc[i] = 0.f;
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const long long warps = ((long long)gridDim.x * blockDim.x) >> 5;
  const int per = PER > 0 ? PER : (h + 31) / 32;
  float dg[NV], db[NV], gam[NV];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    dg[i] = 0.f; db[i] = 0.f;
    const int c = ln_col(lane, i, per, PER > 0);
    gam[i] = (i < per && c < h) ? gamma[c] : 0.f;
  }
  for (long long row = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5; row < rows; row += warps) {
    const float mean = stats[2 * row], rstd = stats[2 * row + 1];
    float xv[NV], dv[NV];
    if constexpr (PER > 0) {
      ln_load_row<T, PER>(x + row * ldx, lane, xv);
      ln_load_row<T, PER>(dy + row * lddy, lane, dv);
    } else {
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const int c = lane + 32 * i;
        const bool ok = i < per && c < h;
        xv[i] = ok ? to_f<T>(x[row * ldx + c]) : mean;
        dv[i] = ok ? to_f<T>(dy[row * lddy + c]) : 0.f;
      }
    }
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      xv[i] = (xv[i] - mean) * rstd;            // xhat
      dg[i] += dv[i] * xv[i];
      db[i] += dv[i];
      dv[i] *= gam[i];                          // g * dy
      s1 += dv[i];
      s2 += dv[i] * xv[i];
    }
    s1 = warp_sum(s1) / h;
    s2 = warp_sum(s2) / h;
    if constexpr (PER > 0) {
      float o[NV];
#pragma unroll
      for (int i = 0; i < NV; ++i) o[i] = rstd * (dv[i] - s1 - xv[i] * s2);
      ln_store_row<T, PER>(dx + row * lddx, lane, o);
    } else {
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const int c = lane + 32 * i;
        if (i < per && c < h) dx[row * lddx + c] = from_f<T>(rstd * (dv[i] - s1 - xv[i] * s2));
      }
    }
  }
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = ln_col(lane, i, per, PER > 0);
    if (i < per && c < h) { atomicAdd(&s_acc[c], dg[i]); atomicAdd(&s_acc[h + c], db[i]); }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < h; i += blockDim.x) {
    atomicAdd(dgamma + i, s_acc[i]);
    atomicAdd(dbeta + i, s_acc[h + i]);
  }
}

// ---------------------------------------------------------------------------------------------------
// Wide variants for 16-bit rows of 64 / 128 / 256 columns: LPR = h / 8 lanes share a row (one 16-byte vector per
// lane), so a warp covers 32 / LPR rows per pass and U passes are loaded before any arithmetic.  A warp therefore
// keeps U * 32 independent 16-byte loads in flight instead of one row's worth, which is what a bandwidth-bound
// row kernel needs on 8 TB/s memory; gamma / beta live in registers for the whole kernel.
// ---------------------------------------------------------------------------------------------------
template <int LPR> __device__ __forceinline__ float row_sum(float v) {
#pragma unroll
  for (int o = LPR / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
template <typename T> __device__ __forceinline__ void unpack8(const uint4& u, float* f) {
  const T* t = reinterpret_cast<const T*>(&u);
#pragma unroll
  for (int i = 0; i < 8; ++i) f[i] = to_f<T>(t[i]);
}
template <typename T> __device__ __forceinline__ uint4 pack8(const float* f) {
  uint4 u;
  T* t = reinterpret_cast<T*>(&u);
#pragma unroll
  for (int i = 0; i < 8; ++i) t[i] = from_f<T>(f[i]);
  return u;
}

template <typename T, int LPR>
__global__ void __launch_bounds__(256, 3) ln_fwd_wide_kernel(const T* __restrict__ x, long long ldx, const float* __restrict__ gamma,
                                                          const float* __restrict__ beta, T* __restrict__ y, long long ldy,
                                                          float* __restrict__ stats, long long rows, float eps) {
  constexpr int RPW = 32 / LPR, U = 4, H = LPR * 8;
  const int lane = threadIdx.x & 31;
  const int sub = lane / LPR, c0 = (lane % LPR) * 8;
  float gam[8], bet[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) { gam[i] = gamma[c0 + i]; bet[i] = beta[c0 + i]; }
  const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long warps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long r0 = warp * (U * RPW); r0 < rows; r0 += warps * (U * RPW)) {
    uint4 raw[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long row = r0 + u * RPW + sub;
      raw[u] = row < rows ? *reinterpret_cast<const uint4*>(x + row * ldx + c0) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long row = r0 + u * RPW + sub;
      float v[8];
      unpack8<T>(raw[u], v);
      float s = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) s += v[i];
      const float mean = row_sum<LPR>(s) * (1.f / H);
      float q = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) { v[i] -= mean; q += v[i] * v[i]; }
      const float rstd = rsqrtf(row_sum<LPR>(q) * (1.f / H) + eps);
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = v[i] * rstd * gam[i] + bet[i];
      if (row < rows) {
        *reinterpret_cast<uint4*>(y + row * ldy + c0) = pack8<T>(v);
        if (stats && (lane % LPR) == 0) *reinterpret_cast<float2*>(stats + 2 * row) = make_float2(mean, rstd);
      }
    }
  }
}

// dxsum (optional) receives the column sums of dx: the bias gradient of the linear layer that produced the
// normalised row, for free.
template <typename T, int LPR>
__global__ void __launch_bounds__(256, 2) ln_bwd_wide_kernel(const T* __restrict__ dy, long long lddy, const T* __restrict__ x,
                                                          long long ldx, const float* __restrict__ stats,
                                                          const float* __restrict__ gamma, T* __restrict__ dx, long long lddx,
                                                          float* __restrict__ dgamma, float* __restrict__ dbeta,
                                                          float* __restrict__ dxsum, long long rows) {
  constexpr int RPW = 32 / LPR, U = 2, H = LPR * 8;
  extern __shared__ float s_acc[];      // [3, H]
  for (int i = threadIdx.x; i < 3 * H; i += blockDim.x) s_acc[i] = 0.f;
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int sub = lane / LPR, c0 = (lane % LPR) * 8;
  float gam[8], dg[8], db[8], dxs[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) { gam[i] = gamma[c0 + i]; dg[i] = 0.f; db[i] = 0.f; dxs[i] = 0.f; }
  const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long warps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long r0 = warp * (U * RPW); r0 < rows; r0 += warps * (U * RPW)) {
    uint4 rx[U], rd[U];
    float2 st[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long row = r0 + u * RPW + sub;
      const bool ok = row < rows;
      rx[u] = ok ? *reinterpret_cast<const uint4*>(x + row * ldx + c0) : make_uint4(0, 0, 0, 0);
      rd[u] = ok ? *reinterpret_cast<const uint4*>(dy + row * lddy + c0) : make_uint4(0, 0, 0, 0);
      st[u] = ok ? *reinterpret_cast<const float2*>(stats + 2 * row) : make_float2(0.f, 0.f);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long row = r0 + u * RPW + sub;
      const float mean = st[u].x, rstd = st[u].y;
      float xv[8], dv[8];
      unpack8<T>(rx[u], xv);
      unpack8<T>(rd[u], dv);
      float s1 = 0.f, s2 = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        xv[i] = (xv[i] - mean) * rstd;            // xhat (0 for rows past the end: rstd = 0)
        dg[i] += dv[i] * xv[i];
        db[i] += dv[i];
        dv[i] *= gam[i];                          // g * dy
        s1 += dv[i];
        s2 += dv[i] * xv[i];
      }
      s1 = row_sum<LPR>(s1) * (1.f / H);
      s2 = row_sum<LPR>(s2) * (1.f / H);
      uint4 o;
      {
        float ov[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) ov[i] = rstd * (dv[i] - s1 - xv[i] * s2);
        o = pack8<T>(ov);
        if (dxsum) {
          // sum what is stored (the rounded value), like a column sum of the stored tensor would
          float rv[8];
          unpack8<T>(o, rv);
#pragma unroll
          for (int i = 0; i < 8; ++i) dxs[i] += rv[i];
        }
      }
      if (row < rows) *reinterpret_cast<uint4*>(dx + row * lddx + c0) = o;
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    atomicAdd(&s_acc[c0 + i], dg[i]);
    atomicAdd(&s_acc[H + c0 + i], db[i]);
    if (dxsum) atomicAdd(&s_acc[2 * H + c0 + i], dxs[i]);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    atomicAdd(dgamma + i, s_acc[i]);
    atomicAdd(dbeta + i, s_acc[H + i]);
    if (dxsum) atomicAdd(dxsum + i, s_acc[2 * H + i]);
  }
}

__device__ __forceinline__ uint32_t mix32(uint32_t x) {
  x = (x ^ (x >> 16)) * 0x7FEB352Du;
  x = (x ^ (x >> 15)) * 0x846CA68Bu;
  return x ^ (x >> 16);
}

__device__ __forceinline__ float gelu_erf_f(float x) { return 0.5f * x * (1.f + erff(x * 0.70710678118654752f)); }

// y = dropout(GELU ? gelu(x) : x): the keep mask is the GEMM epilogue's hash of (seed, row, column)
template <typename T, bool GELU>
__global__ void __launch_bounds__(256) hash_dropout_kernel(const T* __restrict__ x, long long ldx, T* __restrict__ y,
                                                           long long ldy, long long rows, int cols, uint32_t seed,
                                                           uint32_t thresh, float scale) {
  // one thread per 8 consecutive columns of a row (2-D indexing: no 64-bit division per element)
  const int chunks = (cols + 7) / 8;
  const long long total = rows * chunks;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const long long r = i / chunks;
    const int c0 = (int)(i - r * chunks) * 8;
    const uint32_t rh = (uint32_t)r * 0x9E3779B1u + seed;
    const T* xp = x + r * ldx + c0;
    T* yp = y + r * ldy + c0;
    const bool full = c0 + 8 <= cols && sizeof(T) == 2 && ((reinterpret_cast<uintptr_t>(xp) | reinterpret_cast<uintptr_t>(yp)) & 15) == 0;
    if (full) {
      __align__(16) T tmp[8];
      *reinterpret_cast<uint4*>(tmp) = *reinterpret_cast<const uint4*>(xp);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const bool keep = mix32(rh + (uint32_t)(c0 + k) * 0x85EBCA77u) >= thresh;
        const float val = GELU ? gelu_erf_f(to_f<T>(tmp[k])) : to_f<T>(tmp[k]);
        tmp[k] = from_f<T>(keep ? val * scale : 0.f);
      }
      *reinterpret_cast<uint4*>(yp) = *reinterpret_cast<const uint4*>(tmp);
    } else {
      for (int k = 0; k < 8 && c0 + k < cols; ++k) {
        const bool keep = mix32(rh + (uint32_t)(c0 + k) * 0x85EBCA77u) >= thresh;
        const float val = GELU ? gelu_erf_f(to_f<T>(xp[k])) : to_f<T>(xp[k]);
        yp[k] = from_f<T>(keep ? val * scale : 0.f);
      }
    }
  }
}

// out[c] += sum_r x[r, c] (fp32 accumulation): bias gradients without an fp32 copy of the activation gradient.
// Each thread owns 8 consecutive columns and strides over rows; partials meet in shared memory, then one atomic
// per column and block.
template <typename T>
__global__ void __launch_bounds__(256) colsum_kernel(const T* __restrict__ x, long long ldx, long long rows, int cols,
                                                     float* __restrict__ out) {
  extern __shared__ float s_sum[];            // [cols]
  for (int i = threadIdx.x; i < cols; i += blockDim.x) s_sum[i] = 0.f;
  __syncthreads();
  const int chunks = cols / 8;
  const int row_lanes = blockDim.x / chunks;  // threads that share one column chunk
  const int chunk = threadIdx.x % chunks;
  const int rl = threadIdx.x / chunks;
  float acc[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) acc[k] = 0.f;
  if (rl < row_lanes) {
    const long long rstride = (long long)gridDim.x * row_lanes;
    for (long long r = (long long)blockIdx.x * row_lanes + rl; r < rows; r += rstride) {
      __align__(16) T tmp[8];
      if (sizeof(T) == 2) {
        *reinterpret_cast<uint4*>(tmp) = *reinterpret_cast<const uint4*>(x + r * ldx + chunk * 8);
      } else {
        reinterpret_cast<uint4*>(tmp)[0] = reinterpret_cast<const uint4*>(x + r * ldx + chunk * 8)[0];
        reinterpret_cast<uint4*>(tmp)[1] = reinterpret_cast<const uint4*>(x + r * ldx + chunk * 8)[1];
      }
#pragma unroll
      for (int k = 0; k < 8; ++k) acc[k] += to_f<T>(tmp[k]);
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) atomicAdd(&s_sum[chunk * 8 + k], acc[k]);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < cols; i += blockDim.x) atomicAdd(out + i, s_sum[i]);
}


// ---------------------------------------------------------------------------------------------------
// BatchNorm over the rows of a [rows, cols] activation (16-bit or fp32), statistics in fp32.
//   colstats<MODE 1>:  s1[c] += sum_r (x - shift[c]),  s2[c] += sum_r (x - shift[c])^2     (forward statistics;
//                      the shift - the running mean - keeps the one-pass variance well conditioned)
//   colstats<MODE 2>:  s1[c] += sum_r dy,              s2[c] += sum_r dy * (x - mean[c]) * rstd[c]   (dbeta, dgamma)
//   affine1:           y  = x * a[c] + b[c]                        (normalise + scale + shift in one multiply-add)
//   affine2:           dx = dy * a[c] + x * b[c] + c0[c]           (the whole BatchNorm input gradient)
// Each thread owns 8 consecutive columns and strides over rows; partials meet in shared memory, then one atomic per
// column and block.
// ---------------------------------------------------------------------------------------------------
template <typename T> __device__ __forceinline__ void load8(const T* p, float* f) {
  if (sizeof(T) == 2) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    const T* t = reinterpret_cast<const T*>(&u);
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = to_f<T>(t[i]);
  } else {
    const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
  }
}
template <typename T> __device__ __forceinline__ void store8(T* p, const float* f) {
  if (sizeof(T) == 2) {
    uint4 u;
    T* t = reinterpret_cast<T*>(&u);
#pragma unroll
    for (int i = 0; i < 8; ++i) t[i] = from_f<T>(f[i]);
    *reinterpret_cast<uint4*>(p) = u;
  } else {
    reinterpret_cast<float4*>(p)[0] = make_float4(f[0], f[1], f[2], f[3]);
    reinterpret_cast<float4*>(p)[1] = make_float4(f[4], f[5], f[6], f[7]);
  }
}

template <typename T, int MODE>
__global__ void __launch_bounds__(256) colstats_kernel(const T* __restrict__ x, long long ldx, const T* __restrict__ dy,
                                                       long long lddy, const float* __restrict__ p0,
                                                       const float* __restrict__ p1, long long rows, int cols,
                                                       float* __restrict__ s1, float* __restrict__ s2) {
  extern __shared__ float s_sum[];            // [2, cols]
  for (int i = threadIdx.x; i < 2 * cols; i += blockDim.x) s_sum[i] = 0.f;
  __syncthreads();
  const int chunks = cols / 8;
  const int row_lanes = blockDim.x / chunks;  // threads that share one column chunk
  const int chunk = threadIdx.x % chunks;
  const int rl = threadIdx.x / chunks;
  if (rl < row_lanes) {
    float a1[8], a2[8], q0[8], q1[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      a1[k] = 0.f; a2[k] = 0.f;
      q0[k] = p0 ? p0[chunk * 8 + k] : 0.f;    // MODE 1: shift; MODE 2: mean
      q1[k] = p1 ? p1[chunk * 8 + k] : 1.f;    // MODE 2: rstd
    }
    const long long rstride = (long long)gridDim.x * row_lanes;
    long long r = (long long)blockIdx.x * row_lanes + rl;
    // two rows per iteration: both loads are issued before either is used
    for (; r + rstride < rows; r += 2 * rstride) {
      float u[8], v[8], du[8], dv[8];
      load8<T>(x + r * ldx + chunk * 8, u);
      load8<T>(x + (r + rstride) * ldx + chunk * 8, v);
      if (MODE == 2) {
        load8<T>(dy + r * lddy + chunk * 8, du);
        load8<T>(dy + (r + rstride) * lddy + chunk * 8, dv);
      }
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        if (MODE == 1) {
          const float d0 = u[k] - q0[k], d1 = v[k] - q0[k];
          a1[k] += d0 + d1;
          a2[k] += d0 * d0 + d1 * d1;
        } else {
          a1[k] += du[k] + dv[k];
          a2[k] += (du[k] * (u[k] - q0[k]) + dv[k] * (v[k] - q0[k])) * q1[k];
        }
      }
    }
    for (; r < rows; r += rstride) {
      float u[8], du[8];
      load8<T>(x + r * ldx + chunk * 8, u);
      if (MODE == 2) load8<T>(dy + r * lddy + chunk * 8, du);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        if (MODE == 1) { const float d0 = u[k] - q0[k]; a1[k] += d0; a2[k] += d0 * d0; }
        else { a1[k] += du[k]; a2[k] += du[k] * (u[k] - q0[k]) * q1[k]; }
      }
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      atomicAdd(&s_sum[chunk * 8 + k], a1[k]);
      atomicAdd(&s_sum[cols + chunk * 8 + k], a2[k]);
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < cols; i += blockDim.x) {
    atomicAdd(s1 + i, s_sum[i]);
    atomicAdd(s2 + i, s_sum[cols + i]);
  }
}

// TWO = false: y = x*a + b;  TWO = true: y = in2*a + x*b + c0
template <typename T, bool TWO>
__global__ void __launch_bounds__(256) col_affine_kernel(const T* __restrict__ x, long long ldx, const T* __restrict__ in2,
                                                         long long ld2, const float* __restrict__ a,
                                                         const float* __restrict__ b, const float* __restrict__ c0,
                                                         T* __restrict__ y, long long ldy, long long rows, int cols) {
  const int chunks = cols / 8;
  const long long total = rows * chunks;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const long long r = i / chunks;
    const int c = (int)(i - r * chunks) * 8;
    float u[8], w[8], o[8];
    load8<T>(x + r * ldx + c, u);
    if (TWO) load8<T>(in2 + r * ld2 + c, w);
#pragma unroll
    for (int k = 0; k < 8; ++k) o[k] = TWO ? w[k] * a[c + k] + u[k] * b[c + k] + c0[c + k] : u[k] * a[c + k] + b[c + k];
    store8<T>(y + r * ldy + c, o);
  }
}

}  // namespace

#define BF_DT_SWITCH(DT, CALL)                                          \
  if (DT == BF_BF16) { CALL(__nv_bfloat16); }                           \
  else if (DT == BF_FP16) { CALL(__half); }                             \
  else if (DT == BF_FP32) { CALL(float); }                              \
  else return (int)cudaErrorInvalidValue;

static bool ln_packed_ok(int h, int dtype, const void* a, long long lda, const void* b2, long long ldb) {
  const int esz = dtype == BF_FP32 ? 4 : 2;
  if (h % 32 != 0) return false;
  const int per = h / 32;
  if (!(per == 2 || per == 4 || per == 8 || per == 16)) return false;
  if ((per * esz) % 4 != 0) return false;
  return ((uintptr_t)a % 16 == 0) && ((uintptr_t)b2 % 16 == 0) && ((lda * esz) % 16 == 0) && ((ldb * esz) % 16 == 0);
}

static bool ln_wide_ok(int h, int dtype, const void* a, long long lda, const void* b2, long long ldb) {
  if (dtype == BF_FP32 || !(h == 64 || h == 128 || h == 256)) return false;
  return ((uintptr_t)a % 16 == 0) && ((uintptr_t)b2 % 16 == 0) && ((lda * 2) % 16 == 0) && ((ldb * 2) % 16 == 0);
}

#define BF_LN_WIDE_SWITCH(DT, LPRV, CALL)                                                      \
  if (DT == BF_BF16) {                                                                         \
    if (LPRV == 8) { CALL(__nv_bfloat16, 8); } else if (LPRV == 16) { CALL(__nv_bfloat16, 16); } \
    else { CALL(__nv_bfloat16, 32); }                                                          \
  } else {                                                                                     \
    if (LPRV == 8) { CALL(__half, 8); } else if (LPRV == 16) { CALL(__half, 16); }             \
    else { CALL(__half, 32); }                                                                 \
  }

#define BF_LN_PER_SWITCH(T, PERV, KERNEL_CALL)              \
  switch (PERV) {                                            \
    case 2: { constexpr int P_ = 2; KERNEL_CALL; break; }    \
    case 4: { constexpr int P_ = 4; KERNEL_CALL; break; }    \
    case 8: { constexpr int P_ = 8; KERNEL_CALL; break; }    \
    case 16: { constexpr int P_ = 16; KERNEL_CALL; break; }  \
    default: { constexpr int P_ = 0; KERNEL_CALL; break; }   \
  }

extern "C" int bf_layernorm_fwd(const void* x, long long ldx, const float* gamma, const float* beta, void* y,
                                long long ldy, float* stats, long long rows, int h, float eps, int dtype,
                                cudaStream_t st) {
  if (h > 32 * LN_MAX_PER_LANE || h < 1) return (int)cudaErrorInvalidValue;
  if (rows == 0) return 0;
  if (ln_wide_ok(h, dtype, x, ldx, y, ldy)) {
    const int lpr = h / 8;
    long long wb = (rows + 8 * 4 * (32 / lpr) - 1) / (8 * 4 * (32 / lpr));
    if (wb > 148 * 16) wb = 148 * 16;
#define WIDE(T, L) ln_fwd_wide_kernel<T, L><<<(unsigned)wb, 256, 0, st>>>((const T*)x, ldx, gamma, beta, (T*)y, ldy, stats, rows, eps)
    BF_LN_WIDE_SWITCH(dtype, lpr, WIDE)
#undef WIDE
    return (int)cudaGetLastError();
  }
  long long blocks = (rows * 32 + 255) / 256;
  if (blocks > 148 * 64) blocks = 148 * 64;      // many short-lived warps hide the row-load latency better than a few long ones
  const int per = ln_packed_ok(h, dtype, x, ldx, y, ldy) ? h / 32 : 0;
#define CALL(T) BF_LN_PER_SWITCH(T, per, (ln_fwd_kernel<T, P_><<<(unsigned)blocks, 256, 0, st>>>((const T*)x, ldx, gamma, beta, (T*)y, ldy, stats, rows, h, eps)))
  BF_DT_SWITCH(dtype, CALL)
#undef CALL
  return (int)cudaGetLastError();
}

extern "C" int bf_layernorm_bwd(const void* dy, long long lddy, const void* x, long long ldx, const float* stats,
                                const float* gamma, void* dx, long long lddx, float* dgamma, float* dbeta,
                                float* dxsum, long long rows, int h, int dtype, cudaStream_t st) {
  if (h > 32 * LN_MAX_PER_LANE || h < 1) return (int)cudaErrorInvalidValue;
  if (rows == 0) return 0;
  if (ln_wide_ok(h, dtype, x, ldx, dy, lddy) && ln_wide_ok(h, dtype, dx, lddx, dx, lddx)) {
    const int lpr = h / 8;
    long long wb = (rows + 8 * 2 * (32 / lpr) - 1) / (8 * 2 * (32 / lpr));
    if (wb > 148 * 8) wb = 148 * 8;
    const size_t wsm = sizeof(float) * 3 * h;
#define WIDE(T, L) ln_bwd_wide_kernel<T, L><<<(unsigned)wb, 256, wsm, st>>>((const T*)dy, lddy, (const T*)x, ldx, stats, gamma, (T*)dx, lddx, dgamma, dbeta, dxsum, rows)
    BF_LN_WIDE_SWITCH(dtype, lpr, WIDE)
#undef WIDE
    return (int)cudaGetLastError();
  }
  if (dxsum) return (int)cudaErrorNotSupported;   // only the wide kernels produce the extra column sums
  long long blocks = (rows * 32 + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  const size_t smem = sizeof(float) * 2 * h;
  const int per = (ln_packed_ok(h, dtype, x, ldx, dy, lddy) && ln_packed_ok(h, dtype, dx, lddx, dx, lddx)) ? h / 32 : 0;
#define CALL(T) BF_LN_PER_SWITCH(T, per, (ln_bwd_kernel<T, P_><<<(unsigned)blocks, 256, smem, st>>>((const T*)dy, lddy, (const T*)x, ldx, stats, gamma, (T*)dx, lddx, dgamma, dbeta, rows, h)))
  BF_DT_SWITCH(dtype, CALL)
#undef CALL
  return (int)cudaGetLastError();
}

extern "C" int bf_hash_dropout(const void* x, long long ldx, void* y, long long ldy, long long rows, int cols,
                               uint32_t seed, float p, int dtype, cudaStream_t st) {
  if (rows * cols == 0) return 0;
  const uint32_t thresh = (uint32_t)(p * 4294967296.0);
  const float scale = 1.f / (1.f - p);
  long long blocks = (rows * ((cols + 7) / 8) + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
#define CALL(T) hash_dropout_kernel<T, false><<<(unsigned)blocks, 256, 0, st>>>((const T*)x, ldx, (T*)y, ldy, rows, cols, seed, thresh, scale)
  BF_DT_SWITCH(dtype, CALL)
#undef CALL
  return (int)cudaGetLastError();
}

// y = dropout(gelu(x), p) in one pass (p = 0: plain GELU); same keep mask as bf_hash_dropout
extern "C" int bf_gelu_dropout(const void* x, long long ldx, void* y, long long ldy, long long rows, int cols,
                               uint32_t seed, float p, int dtype, cudaStream_t st) {
  if (rows * cols == 0) return 0;
  if (p < 0.f || p >= 1.f) return (int)cudaErrorInvalidValue;
  const uint32_t thresh = (uint32_t)(p * 4294967296.0);
  const float scale = 1.f / (1.f - p);
  long long blocks = (rows * ((cols + 7) / 8) + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
#define CALL(T) hash_dropout_kernel<T, true><<<(unsigned)blocks, 256, 0, st>>>((const T*)x, ldx, (T*)y, ldy, rows, cols, seed, thresh, scale)
  BF_DT_SWITCH(dtype, CALL)
#undef CALL
  return (int)cudaGetLastError();
}

extern "C" int bf_colsum(const void* x, long long ldx, long long rows, int cols, float* out, int dtype, cudaStream_t st) {
  const int esz = dtype == BF_FP32 ? 4 : 2;
  if (cols % 8 != 0 || cols > 2048 || cols < 8 || ((uintptr_t)x) % 16 != 0 || (ldx * esz) % 16 != 0)
    return (int)cudaErrorInvalidValue;
  if (rows == 0) return 0;
  const int chunks = cols / 8;
  if (chunks > 256) return (int)cudaErrorInvalidValue;
  const int row_lanes = 256 / chunks;
  long long blocks = (rows + row_lanes * 16 - 1) / (row_lanes * 16);
  if (blocks > 148 * 4) blocks = 148 * 4;
  if (blocks < 1) blocks = 1;
  const size_t smem = sizeof(float) * cols;
#define CALL(T) colsum_kernel<T><<<(unsigned)blocks, 256, smem, st>>>((const T*)x, ldx, rows, cols, out)
  BF_DT_SWITCH(dtype, CALL)
#undef CALL
  return (int)cudaGetLastError();
}

static bool cols8_ok(int cols, int dtype, const void* p, long long ld) {
  const int esz = dtype == BF_FP32 ? 4 : 2;
  return cols % 8 == 0 && cols >= 8 && cols <= 2048 && ((uintptr_t)p) % 16 == 0 && (ld * esz) % 16 == 0;
}

extern "C" int bf_bn_stats(const void* x, long long ldx, const float* shift, long long rows, int cols, float* s1,
                           float* s2, int dtype, cudaStream_t st) {
  if (!cols8_ok(cols, dtype, x, ldx)) return (int)cudaErrorInvalidValue;
  if (rows == 0) return 0;
  const int row_lanes = 256 / (cols / 8);
  if (row_lanes < 1) return (int)cudaErrorInvalidValue;
  long long blocks = (rows + row_lanes * 16 - 1) / (row_lanes * 16);
  if (blocks > 148 * 6) blocks = 148 * 6;
  const size_t smem = sizeof(float) * 2 * cols;
#define CALL(T) colstats_kernel<T, 1><<<(unsigned)blocks, 256, smem, st>>>((const T*)x, ldx, nullptr, 0, shift, nullptr, rows, cols, s1, s2)
  BF_DT_SWITCH(dtype, CALL)
#undef CALL
  return (int)cudaGetLastError();
}

extern "C" int bf_bn_bwd_reduce(const void* dy, long long lddy, const void* x, long long ldx, const float* mean,
                                const float* rstd, long long rows, int cols, float* dbeta, float* dgamma, int dtype,
                                cudaStream_t st) {
  if (!cols8_ok(cols, dtype, x, ldx) || !cols8_ok(cols, dtype, dy, lddy)) return (int)cudaErrorInvalidValue;
  if (rows == 0) return 0;
  const int row_lanes = 256 / (cols / 8);
  if (row_lanes < 1) return (int)cudaErrorInvalidValue;
  long long blocks = (rows + row_lanes * 16 - 1) / (row_lanes * 16);
  if (blocks > 148 * 6) blocks = 148 * 6;
  const size_t smem = sizeof(float) * 2 * cols;
#define CALL(T) colstats_kernel<T, 2><<<(unsigned)blocks, 256, smem, st>>>((const T*)x, ldx, (const T*)dy, lddy, mean, rstd, rows, cols, dbeta, dgamma)
  BF_DT_SWITCH(dtype, CALL)
#undef CALL
  return (int)cudaGetLastError();
}

extern "C" int bf_col_affine(const void* x, long long ldx, const void* in2, long long ld2, const float* a, const float* b,
                             const float* c0, void* y, long long ldy, long long rows, int cols, int dtype,
                             cudaStream_t st) {
  if (!cols8_ok(cols, dtype, x, ldx) || !cols8_ok(cols, dtype, y, ldy) || (in2 && !cols8_ok(cols, dtype, in2, ld2)))
    return (int)cudaErrorInvalidValue;
  if (rows == 0) return 0;
  long long blocks = (rows * (cols / 8) + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (in2) {
#define CALL(T) col_affine_kernel<T, true><<<(unsigned)blocks, 256, 0, st>>>((const T*)x, ldx, (const T*)in2, ld2, a, b, c0, (T*)y, ldy, rows, cols)
    BF_DT_SWITCH(dtype, CALL)
#undef CALL
  } else {
#define CALL(T) col_affine_kernel<T, false><<<(unsigned)blocks, 256, 0, st>>>((const T*)x, ldx, nullptr, 0, a, b, nullptr, (T*)y, ldy, rows, cols)
    BF_DT_SWITCH(dtype, CALL)
#undef CALL
  }
  return (int)cudaGetLastError();
}
