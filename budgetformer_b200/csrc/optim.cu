// Optimizer step on flat fp32 buckets: global gradient-norm clipping and AdamW in two launches per bucket,
// with the clip coefficient computed on the device (no host round trip).  Replaces clip_grad_norm_ + the
// per-tensor AdamW loop of the reference step (main_node_fullgraph_sp.py:1284-1293).
#include <cuda_runtime.h>
#include <stdint.h>

#include "bf_kernels.h"

namespace {

__global__ void __launch_bounds__(512) sumsq_kernel(const float* __restrict__ g, long long n, float* __restrict__ out) {
  float acc = 0.f;
  const long long stride = (long long)gridDim.x * blockDim.x;
  const long long n4 = n / 4;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
    const float4 v = reinterpret_cast<const float4*>(g)[i];
    acc += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  for (long long i = n4 * 4 + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) acc += g[i] * g[i];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  __shared__ float s[16];
  if ((threadIdx.x & 31) == 0) s[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = threadIdx.x < (blockDim.x >> 5) ? s[threadIdx.x] : 0.f;
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (threadIdx.x == 0) atomicAdd(out, v);
  }
}

// Squared gradient norm from its parts, added in index order by every thread alike (a handful of floats).
__device__ __forceinline__ float total_sumsq(const float* __restrict__ parts, int n) {
  float t = 0.f;
  for (int i = 0; i < n; ++i) t += parts[i];
  return t;
}

__global__ void __launch_bounds__(512) adamw_flat_kernel(float* __restrict__ p, const float* __restrict__ g,
                                                         float* __restrict__ m, float* __restrict__ v, long long n,
                                                         float lr, float beta1, float beta2, float eps, float wd,
                                                         float bc1, float bc2_sqrt, const float* __restrict__ sumsq,
                                                         int n_sumsq, float max_norm) {
  float clip = 1.f;
  if (sumsq != nullptr && max_norm > 0.f) clip = fminf(1.f, max_norm / (sqrtf(total_sumsq(sumsq, n_sumsq)) + 1e-6f));
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const float gi = g[i] * clip;
    float pi = p[i] * (1.f - lr * wd);
    const float mi = beta1 * m[i] + (1.f - beta1) * gi;
    const float vi = beta2 * v[i] + (1.f - beta2) * gi * gi;
    m[i] = mi;
    v[i] = vi;
    pi -= (lr / bc1) * mi / (sqrtf(vi) / bc2_sqrt + eps);
    p[i] = pi;
  }
}

// Same update with the step-dependent scalars (lr, 1 - beta1^t, sqrt(1 - beta2^t)) read from device memory, so that the
// launch can sit in a CUDA graph that is replayed every step.
__global__ void __launch_bounds__(512) adamw_flat_dev_kernel(float* __restrict__ p, const float* __restrict__ g,
                                                             float* __restrict__ m, float* __restrict__ v, long long n,
                                                             float beta1, float beta2, float eps, float wd,
                                                             const float* __restrict__ hyper,
                                                             const float* __restrict__ sumsq, int n_sumsq, float max_norm) {
  const float lr = hyper[0], bc1 = hyper[1], bc2_sqrt = hyper[2];
  float clip = 1.f;
  if (sumsq != nullptr && max_norm > 0.f) clip = fminf(1.f, max_norm / (sqrtf(total_sumsq(sumsq, n_sumsq)) + 1e-6f));
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const float gi = g[i] * clip;
    float pi = p[i] * (1.f - lr * wd);
    const float mi = beta1 * m[i] + (1.f - beta1) * gi;
    const float vi = beta2 * v[i] + (1.f - beta2) * gi * gi;
    m[i] = mi;
    v[i] = vi;
    pi -= (lr / bc1) * mi / (sqrtf(vi) / bc2_sqrt + eps);
    p[i] = pi;
  }
}

int grid_for(long long n) {
  long long b = (n + 511) / 512;
  if (b < 1) b = 1;
  if (b > 148 * 4) b = 148 * 4;
  return (int)b;
}

}  // namespace

extern "C" int bf_grad_sumsq(const float* g, long long n, float* out, cudaStream_t st) {
  if (n <= 0) return 0;
  sumsq_kernel<<<grid_for(n / 4 + 1), 512, 0, st>>>(g, n, out);
  return (int)cudaGetLastError();
}

extern "C" int bf_adamw_flat(float* p, const float* g, float* m, float* v, long long n, float lr, float beta1,
                             float beta2, float eps, float weight_decay, int step, const float* sumsq, int n_sumsq,
                             float max_norm, cudaStream_t st) {
  if (n <= 0) return 0;
  const float bc1 = 1.f - powf(beta1, (float)step);
  const float bc2_sqrt = sqrtf(1.f - powf(beta2, (float)step));
  adamw_flat_kernel<<<grid_for(n), 512, 0, st>>>(p, g, m, v, n, lr, beta1, beta2, eps, weight_decay, bc1, bc2_sqrt, sumsq,
                                                 n_sumsq, max_norm);
  return (int)cudaGetLastError();
}

extern "C" int bf_adamw_flat_dev(float* p, const float* g, float* m, float* v, long long n, float beta1, float beta2,
                                 float eps, float weight_decay, const float* hyper, const float* sumsq, int n_sumsq,
                                 float max_norm, cudaStream_t st) {
  if (n <= 0) return 0;
  adamw_flat_dev_kernel<<<grid_for(n), 512, 0, st>>>(p, g, m, v, n, beta1, beta2, eps, weight_decay, hyper, sumsq,
                                                     n_sumsq, max_norm);
  return (int)cudaGetLastError();
}
