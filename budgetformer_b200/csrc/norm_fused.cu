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

template <typename T>
__global__ void __launch_bounds__(256) ln_fwd_kernel(const T* __restrict__ x, long long ldx, const float* __restrict__ gamma,
                                                     const float* __restrict__ beta, T* __restrict__ y, long long ldy,
                                                     float* __restrict__ stats, long long rows, int h, float eps) {
  const long long row = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const T* xr = x + row * ldx;
  float v[LN_MAX_PER_LANE];
  float s = 0.f;
  const int per = (h + 31) / 32;
#pragma unroll
  for (int i = 0; i < LN_MAX_PER_LANE; ++i) {
    const int c = lane + 32 * i;
    v[i] = (i < per && c < h) ? to_f<T>(xr[c]) : 0.f;
    s += v[i];
  }
  const float mean = warp_sum(s) / h;
  float q = 0.f;
#pragma unroll
  for (int i = 0; i < LN_MAX_PER_LANE; ++i) {
    const int c = lane + 32 * i;
    const float d = (i < per && c < h) ? v[i] - mean : 0.f;
    q += d * d;
  }
  const float rstd = rsqrtf(warp_sum(q) / h + eps);
  T* yr = y + row * ldy;
#pragma unroll
  for (int i = 0; i < LN_MAX_PER_LANE; ++i) {
    const int c = lane + 32 * i;
    if (i < per && c < h) yr[c] = from_f<T>((v[i] - mean) * rstd * gamma[c] + beta[c]);
  }
  if (lane == 0 && stats) { stats[2 * row] = mean; stats[2 * row + 1] = rstd; }
}

// dx = rstd * (g*dy - mean(g*dy) - xhat * mean(g*dy*xhat)); dgamma += dy*xhat; dbeta += dy
template <typename T>
__global__ void __launch_bounds__(256) ln_bwd_kernel(const T* __restrict__ dy, long long lddy, const T* __restrict__ x,
                                                     long long ldx, const float* __restrict__ stats,
                                                     const float* __restrict__ gamma, T* __restrict__ dx, long long lddx,
                                                     float* __restrict__ dgamma, float* __restrict__ dbeta,
                                                     long long rows, int h, int rows_per_warp) {
  extern __shared__ float s_acc[];      // [2, h]
  for (int i = threadIdx.x; i < 2 * h; i += blockDim.x) s_acc[i] = 0.f;
  __syncthreads();
  const long long warp_id = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const int per = (h + 31) / 32;
  float dg[LN_MAX_PER_LANE], db[LN_MAX_PER_LANE];
#pragma unroll
  for (int i = 0; i < LN_MAX_PER_LANE; ++i) { dg[i] = 0.f; db[i] = 0.f; }
  for (int rr = 0; rr < rows_per_warp; ++rr) {
    const long long row = warp_id * rows_per_warp + rr;
    if (row >= rows) break;
    const float mean = stats[2 * row], rstd = stats[2 * row + 1];
    float xh[LN_MAX_PER_LANE], gdy[LN_MAX_PER_LANE];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < LN_MAX_PER_LANE; ++i) {
      const int c = lane + 32 * i;
      if (i < per && c < h) {
        const float d = to_f<T>(dy[row * lddy + c]);
        xh[i] = (to_f<T>(x[row * ldx + c]) - mean) * rstd;
        gdy[i] = d * gamma[c];
        dg[i] += d * xh[i];
        db[i] += d;
        s1 += gdy[i];
        s2 += gdy[i] * xh[i];
      } else { xh[i] = 0.f; gdy[i] = 0.f; }
    }
    s1 = warp_sum(s1) / h;
    s2 = warp_sum(s2) / h;
#pragma unroll
    for (int i = 0; i < LN_MAX_PER_LANE; ++i) {
      const int c = lane + 32 * i;
      if (i < per && c < h) dx[row * lddx + c] = from_f<T>(rstd * (gdy[i] - s1 - xh[i] * s2));
    }
  }
#pragma unroll
  for (int i = 0; i < LN_MAX_PER_LANE; ++i) {
    const int c = lane + 32 * i;
    if (i < per && c < h) { atomicAdd(&s_acc[c], dg[i]); atomicAdd(&s_acc[h + c], db[i]); }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < h; i += blockDim.x) {
    atomicAdd(dgamma + i, s_acc[i]);
    atomicAdd(dbeta + i, s_acc[h + i]);
  }
}

__device__ __forceinline__ uint32_t mix32(uint32_t x) {
  x = (x ^ (x >> 16)) * 0x7FEB352Du;
  x = (x ^ (x >> 15)) * 0x846CA68Bu;
  return x ^ (x >> 16);
}

template <typename T>
__global__ void __launch_bounds__(256) hash_dropout_kernel(const T* __restrict__ x, long long ldx, T* __restrict__ y,
                                                           long long ldy, long long rows, int cols, uint32_t seed,
                                                           uint32_t thresh, float scale) {
  const long long total = rows * cols;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const long long r = i / cols;
    const int c = (int)(i - r * cols);
    const bool keep = mix32((uint32_t)r * 0x9E3779B1u + (uint32_t)c * 0x85EBCA77u + seed) >= thresh;
    y[r * ldy + c] = from_f<T>(keep ? to_f<T>(x[r * ldx + c]) * scale : 0.f);
  }
}

}  // namespace

#define BF_DT_SWITCH(DT, CALL)                                          \
  if (DT == BF_BF16) { CALL(__nv_bfloat16); }                           \
  else if (DT == BF_FP16) { CALL(__half); }                             \
  else if (DT == BF_FP32) { CALL(float); }                              \
  else return (int)cudaErrorInvalidValue;

extern "C" int bf_layernorm_fwd(const void* x, long long ldx, const float* gamma, const float* beta, void* y,
                                long long ldy, float* stats, long long rows, int h, float eps, int dtype,
                                cudaStream_t st) {
  if (h > 32 * LN_MAX_PER_LANE || h < 1) return (int)cudaErrorInvalidValue;
  if (rows == 0) return 0;
  const long long blocks = (rows * 32 + 255) / 256;
#define CALL(T) ln_fwd_kernel<T><<<(unsigned)blocks, 256, 0, st>>>((const T*)x, ldx, gamma, beta, (T*)y, ldy, stats, rows, h, eps)
  BF_DT_SWITCH(dtype, CALL)
#undef CALL
  return (int)cudaGetLastError();
}

extern "C" int bf_layernorm_bwd(const void* dy, long long lddy, const void* x, long long ldx, const float* stats,
                                const float* gamma, void* dx, long long lddx, float* dgamma, float* dbeta,
                                long long rows, int h, int dtype, cudaStream_t st) {
  if (h > 32 * LN_MAX_PER_LANE || h < 1) return (int)cudaErrorInvalidValue;
  if (rows == 0) return 0;
  const int rows_per_warp = 16;
  const long long warps = (rows + rows_per_warp - 1) / rows_per_warp;
  const long long blocks = (warps * 32 + 255) / 256;
  const size_t smem = sizeof(float) * 2 * h;
#define CALL(T) ln_bwd_kernel<T><<<(unsigned)blocks, 256, smem, st>>>((const T*)dy, lddy, (const T*)x, ldx, stats, gamma, (T*)dx, lddx, dgamma, dbeta, rows, h, rows_per_warp)
  BF_DT_SWITCH(dtype, CALL)
#undef CALL
  return (int)cudaGetLastError();
}

extern "C" int bf_hash_dropout(const void* x, long long ldx, void* y, long long ldy, long long rows, int cols,
                               uint32_t seed, float p, int dtype, cudaStream_t st) {
  if (rows * cols == 0) return 0;
  const uint32_t thresh = (uint32_t)(p * 4294967296.0);
  const float scale = 1.f / (1.f - p);
  long long blocks = (rows * cols + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
#define CALL(T) hash_dropout_kernel<T><<<(unsigned)blocks, 256, 0, st>>>((const T*)x, ldx, (T*)y, ldy, rows, cols, seed, thresh, scale)
  BF_DT_SWITCH(dtype, CALL)
#undef CALL
  return (int)cudaGetLastError();
}
