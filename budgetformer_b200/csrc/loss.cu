// Fused readout loss: log-softmax + negative log-likelihood over the rank's training rows, mean-reduced, and its
// gradient for all rows in one pass (zeros for rows that are not training rows).  Replaces log_softmax -> index ->
// nll_loss of the reference step (main_node_fullgraph_sp.py:1234-1237) and their three backward kernels.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "bf_kernels.h"

namespace {

template <typename T> __device__ __forceinline__ float ldf(const T* p);
template <> __device__ __forceinline__ float ldf<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <> __device__ __forceinline__ float ldf<__half>(const __half* p) { return __half2float(*p); }
template <typename T> __device__ __forceinline__ T stf(float v);
template <> __device__ __forceinline__ float stf<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 stf<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half stf<__half>(float v) { return __float2half_rn(v); }

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_add(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// One warp per row.  mask[row] != 0 marks training rows.  loss_sum += sum over training rows of (lse - logit[y]).
// dlogits (optional) = mask ? (softmax - onehot) * grad_scale : 0.
template <typename T>
__global__ void __launch_bounds__(256) nll_fwd_bwd_kernel(const T* __restrict__ logits, long long ld, const long long* __restrict__ y,
                                                          const uint8_t* __restrict__ mask, long long rows, int classes,
                                                          float* __restrict__ loss_sum, T* __restrict__ dlogits,
                                                          float grad_scale) {
  const int lane = threadIdx.x & 31;
  const long long warps = ((long long)gridDim.x * blockDim.x) >> 5;
  float local = 0.f;
  for (long long row = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5; row < rows; row += warps) {
    const bool train = mask[row] != 0;
    if (!train) {
      if (dlogits) for (int c = lane; c < classes; c += 32) dlogits[row * classes + c] = stf<T>(0.f);
      continue;
    }
    const T* lr = logits + row * ld;
    float mx = -3.0e38f;
    for (int c = lane; c < classes; c += 32) mx = fmaxf(mx, ldf<T>(lr + c));
    mx = warp_max(mx);
    float se = 0.f;
    for (int c = lane; c < classes; c += 32) se += __expf(ldf<T>(lr + c) - mx);
    se = warp_add(se);
    const float lse = mx + __logf(se);
    const int label = (int)y[row];
    if (lane == 0) local += lse - ldf<T>(lr + label);
    if (dlogits) {
      for (int c = lane; c < classes; c += 32) {
        const float p = __expf(ldf<T>(lr + c) - lse);
        dlogits[row * classes + c] = stf<T>((p - (c == label ? 1.f : 0.f)) * grad_scale);
      }
    }
  }
  local = warp_add(local);
  if (lane == 0 && local != 0.f) atomicAdd(loss_sum, local);
}

}  // namespace

extern "C" int bf_nll_fwd_bwd(const void* logits, long long ld, const long long* y, const uint8_t* mask, long long rows,
                              int classes, float* loss_sum, void* dlogits, float grad_scale, int dtype, cudaStream_t st) {
  if (rows == 0) return 0;
  long long blocks = (rows * 32 + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (dtype == BF_BF16)
    nll_fwd_bwd_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, st>>>((const __nv_bfloat16*)logits, ld, y, mask, rows, classes, loss_sum, (__nv_bfloat16*)dlogits, grad_scale);
  else if (dtype == BF_FP16)
    nll_fwd_bwd_kernel<__half><<<(unsigned)blocks, 256, 0, st>>>((const __half*)logits, ld, y, mask, rows, classes, loss_sum, (__half*)dlogits, grad_scale);
  else if (dtype == BF_FP32)
    nll_fwd_bwd_kernel<float><<<(unsigned)blocks, 256, 0, st>>>((const float*)logits, ld, y, mask, rows, classes, loss_sum, (float*)dlogits, grad_scale);
  else
    return (int)cudaErrorInvalidValue;
  return (int)cudaGetLastError();
}
