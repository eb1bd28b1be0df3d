// In-kernel collectives over NVLink / NVSwitch peer memory (symmetric buffers mapped into every rank).
//
//  * bf_peer_barrier     - every rank raises a monotonically increasing epoch in each peer's flag
//                          page (st.release.sys after a system fence) and waits until all peers have
//                          raised theirs (ld.acquire.sys, bounded spin -> status word on expiry);
//  * bf_allreduce_mean   - gradient bucket all-reduce fused with the 1/P scale, in place:
//                          rank r sums slice r of every peer's bucket with 16-byte peer loads and
//                          stores the scaled result into slice r of every peer's bucket (two-shot,
//                          bandwidth optimal: each byte crosses NVLink once in and once out).
//                          With an NVSwitch multicast mapping the same slice is reduced inside the
//                          switch (multimem.ld_reduce) and broadcast with multimem.st.  The same kernel
//                          leaves the sum of squares of the reduced slice with every rank, so that global-norm
//                          clipping needs no further pass over the gradients;
//  * bf_peer_gather_cols - heads->nodes all-to-all as a pull: this rank's rows of every peer's
//                          [N, h/P] context buffer are copied into a local [N/P, h] matrix.
// Replaces the reference's NCCL all_reduce with three elementwise passes (gt_sp/reducer.py:120-146)
// and its list all_to_all (gt_sp/layer.py:35-41).
#include <cuda_runtime.h>
#include <stdint.h>

#include "bf_kernels.h"

namespace {

constexpr uint32_t SPIN_LIMIT = 1u << 21;   // x (128 ns sleep + one system-scope load): a few seconds

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

struct PeerPtrs {
  void* p[BF_MAX_PEERS];
};

// flags layout on every rank: uint32 flags[n_channels][BF_MAX_PEERS]; writer rank w owns column w.
__global__ void peer_barrier_kernel(PeerPtrs flag_pages, int rank, int world, int channel, uint32_t epoch, int* status) {
  const int t = threadIdx.x;
  if (t < world) {
    __threadfence_system();
    uint32_t* remote = static_cast<uint32_t*>(flag_pages.p[t]) + channel * BF_MAX_PEERS + rank;
    st_release_sys(remote, epoch);
    const uint32_t* mine = static_cast<const uint32_t*>(flag_pages.p[rank]) + channel * BF_MAX_PEERS + t;
    // an earlier wait of this process already gave up: the host will discard everything queued behind it, so raise
    // the flag for the peers and return without spending another bound here
    if (*reinterpret_cast<volatile int*>(status) != 0) return;
    bool ok = false;
    for (uint32_t it = 0; it < SPIN_LIMIT; ++it) {
      // epochs only grow; signed distance handles wrap-around
      if ((int32_t)(ld_acquire_sys(mine) - epoch) >= 0) { ok = true; break; }
      __nanosleep(128);
    }
    if (!ok) { atomicExch(status, 16 + t); atomicExch(status + 1, (int)epoch); }
  }
}

// Sum of squares of the values this rank reduced, finished by the last block to arrive: block partials go to
// `scratch[0 .. gridDim.x)`, the counter behind them elects the last block, which adds the partials in a fixed order
// and stores the slice total into slot `rank` of every rank's `parts` array (gradient-norm clipping needs the norm of
// the whole reduced bucket: the optimizer adds the P slice totals).  Resets the counter for the next launch.
__device__ void finish_sumsq(float sq, float* scratch, PeerPtrs parts, int rank, int world) {
  __shared__ float s_warp[16];
  __shared__ int s_last;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
  if ((threadIdx.x & 31) == 0) s_warp[threadIdx.x >> 5] = sq;
  __syncthreads();
  if (threadIdx.x == 0) {
    float v = 0.f;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) v += s_warp[w];
    scratch[blockIdx.x] = v;
    __threadfence();
    unsigned* counter = reinterpret_cast<unsigned*>(scratch + gridDim.x);
    s_last = (atomicAdd(counter, 1u) == gridDim.x - 1) ? 1 : 0;
  }
  __syncthreads();
  if (s_last && threadIdx.x < 32) {
    __threadfence();
    float v = 0.f;
    for (int b = threadIdx.x; b < (int)gridDim.x; b += 32) v += *reinterpret_cast<volatile float*>(scratch + b);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (threadIdx.x == 0) {
      for (int r = 0; r < world; ++r) static_cast<float*>(parts.p[r])[rank] = v;
      *reinterpret_cast<unsigned*>(scratch + gridDim.x) = 0u;
    }
  }
}

__global__ void __launch_bounds__(512) allreduce_mean_kernel(PeerPtrs bufs, int rank, int world, long long n_vec4,
                                                             float scale, float* norm_scratch, PeerPtrs norm_parts) {
  // slice of 16-byte vectors owned by this rank
  const long long per = (n_vec4 + world - 1) / world;
  const long long beg = per * rank;
  const long long end = beg + per < n_vec4 ? beg + per : n_vec4;
  const long long stride = (long long)gridDim.x * blockDim.x;
  float sq = 0.f;
  for (long long i = beg + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < end; i += stride) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int r = 0; r < BF_MAX_PEERS; ++r) {
      if (r < world) {
        const float4 v = static_cast<const float4*>(bufs.p[(rank + r) % world])[i];
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
      }
    }
    acc.x *= scale; acc.y *= scale; acc.z *= scale; acc.w *= scale;
    sq += acc.x * acc.x + acc.y * acc.y + acc.z * acc.z + acc.w * acc.w;
#pragma unroll
    for (int r = 0; r < BF_MAX_PEERS; ++r)
      if (r < world) static_cast<float4*>(bufs.p[(rank + r) % world])[i] = acc;
  }
  if (norm_scratch != nullptr) finish_sumsq(sq, norm_scratch, norm_parts, rank, world);
}

__global__ void __launch_bounds__(512) allreduce_mean_multimem_kernel(float* mc_ptr, int rank, int world,
                                                                      long long n_vec4, float scale, float* norm_scratch,
                                                                      PeerPtrs norm_parts) {
  const long long per = (n_vec4 + world - 1) / world;
  const long long beg = per * rank;
  const long long end = beg + per < n_vec4 ? beg + per : n_vec4;
  const long long stride = (long long)gridDim.x * blockDim.x;
  float sq = 0.f;
  for (long long i = beg + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < end; i += stride) {
    float* addr = mc_ptr + 4 * i;
    float x, y, z, w;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(x), "=f"(y), "=f"(z), "=f"(w)
                 : "l"(addr)
                 : "memory");
    x *= scale; y *= scale; z *= scale; w *= scale;
    sq += x * x + y * y + z * z + w * w;
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(x), "f"(y), "f"(z),
                 "f"(w)
                 : "memory");
  }
  if (norm_scratch != nullptr) finish_sumsq(sq, norm_scratch, norm_parts, rank, world);
}

// dst[row, r*cols + c] = peer_r[(row0 + row), c]   (16-byte vectors; cols*elem_size % 16 == 0)
__global__ void __launch_bounds__(256) peer_gather_cols_kernel(PeerPtrs src, int world, long long row0, long long rows,
                                                               int vec_per_row_src, long long src_ld_vec, uint4* dst,
                                                               long long dst_ld_vec) {
  const long long total = rows * world * vec_per_row_src;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int v = (int)(i % vec_per_row_src);
    const long long t = i / vec_per_row_src;
    const int r = (int)(t % world);
    const long long row = t / world;
    const uint4 x = static_cast<const uint4*>(src.p[r])[(row0 + row) * src_ld_vec + v];
    dst[row * dst_ld_vec + (long long)r * vec_per_row_src + v] = x;
  }
}

// peer_r[(row0 + row), c] = src[row, r*cols + c]  (nodes->heads push of an already computed matrix)
__global__ void __launch_bounds__(256) peer_scatter_cols_kernel(PeerPtrs dst, int world, long long row0, long long rows,
                                                                int vec_per_row_dst, long long dst_ld_vec,
                                                                const uint4* src, long long src_ld_vec) {
  const long long total = rows * world * vec_per_row_dst;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int v = (int)(i % vec_per_row_dst);
    const long long t = i / vec_per_row_dst;
    const int r = (int)(t % world);
    const long long row = t / world;
    static_cast<uint4*>(dst.p[r])[(row0 + row) * dst_ld_vec + v] = src[row * src_ld_vec + (long long)r * vec_per_row_dst + v];
  }
}

// dst[r * n + i] = src_r[i]: the ranks' shards laid end to end (element-wise, so that shards of any length line up)
template <typename T>
__global__ void __launch_bounds__(256) peer_concat_kernel(PeerPtrs src, int world, long long n, T* dst) {
  const long long total = n * world;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int r = (int)(i / n);
    dst[i] = static_cast<const T*>(src.p[r])[i - (long long)r * n];
  }
}

PeerPtrs to_ptrs(void* const* p, int world) {
  PeerPtrs o;
  for (int i = 0; i < BF_MAX_PEERS; ++i) o.p[i] = i < world ? p[i] : nullptr;
  return o;
}

int grid_for(long long work, int threads) {
  long long b = (work + threads - 1) / threads;
  if (b < 1) b = 1;
  if (b > 148 * 8) b = 148 * 8;
  return (int)b;
}

}  // namespace

extern "C" int bf_peer_barrier(void* const* flag_pages, int rank, int world, int channel, uint32_t epoch, int* status,
                               cudaStream_t st) {
  if (world < 1 || world > BF_MAX_PEERS || channel < 0 || channel >= BF_FLAG_CHANNELS) return (int)cudaErrorInvalidValue;
  peer_barrier_kernel<<<1, 32, 0, st>>>(to_ptrs(flag_pages, world), rank, world, channel, epoch, status);
  return (int)cudaGetLastError();
}

extern "C" int bf_allreduce_mean_grid(long long n_floats, int world) {
  if (world < 1 || n_floats <= 0) return 1;
  const long long per = (n_floats / 4 + world - 1) / world;
  return grid_for(per, 512);
}

extern "C" int bf_allreduce_mean(void* const* bufs, float* multicast_ptr, int rank, int world, long long n_floats,
                                 float* norm_scratch, void* const* norm_parts, cudaStream_t st) {
  if (world < 1 || world > BF_MAX_PEERS || n_floats % 4 != 0) return (int)cudaErrorInvalidValue;
  if ((norm_scratch == nullptr) != (norm_parts == nullptr)) return (int)cudaErrorInvalidValue;
  const long long n_vec4 = n_floats / 4;
  const int grid = bf_allreduce_mean_grid(n_floats, world);
  const float scale = 1.0f / (float)world;
  PeerPtrs parts = norm_parts ? to_ptrs(norm_parts, world) : PeerPtrs{};
  if (multicast_ptr)
    allreduce_mean_multimem_kernel<<<grid, 512, 0, st>>>(multicast_ptr, rank, world, n_vec4, scale, norm_scratch, parts);
  else
    allreduce_mean_kernel<<<grid, 512, 0, st>>>(to_ptrs(bufs, world), rank, world, n_vec4, scale, norm_scratch, parts);
  return (int)cudaGetLastError();
}

extern "C" int bf_peer_gather_cols(void* const* src, int world, long long row0, long long rows, int cols_bytes,
                                   long long src_ld_bytes, void* dst, long long dst_ld_bytes, cudaStream_t st) {
  if (cols_bytes % 16 || src_ld_bytes % 16 || dst_ld_bytes % 16 || world < 1 || world > BF_MAX_PEERS)
    return (int)cudaErrorInvalidValue;
  const int vpr = cols_bytes / 16;
  const long long total = rows * world * vpr;
  if (total == 0) return 0;
  peer_gather_cols_kernel<<<grid_for(total, 256), 256, 0, st>>>(to_ptrs(src, world), world, row0, rows, vpr,
                                                                src_ld_bytes / 16, static_cast<uint4*>(dst),
                                                                dst_ld_bytes / 16);
  return (int)cudaGetLastError();
}

extern "C" int bf_peer_scatter_cols(void* const* dst, int world, long long row0, long long rows, int cols_bytes,
                                    long long dst_ld_bytes, const void* src, long long src_ld_bytes, cudaStream_t st) {
  if (cols_bytes % 16 || src_ld_bytes % 16 || dst_ld_bytes % 16 || world < 1 || world > BF_MAX_PEERS)
    return (int)cudaErrorInvalidValue;
  const int vpr = cols_bytes / 16;
  const long long total = rows * world * vpr;
  if (total == 0) return 0;
  peer_scatter_cols_kernel<<<grid_for(total, 256), 256, 0, st>>>(to_ptrs(dst, world), world, row0, rows, vpr,
                                                                 dst_ld_bytes / 16, static_cast<const uint4*>(src),
                                                                 src_ld_bytes / 16);
  return (int)cudaGetLastError();
}

extern "C" int bf_peer_concat(void* const* src, int world, long long n_elem, int elem_bytes, void* dst, cudaStream_t st) {
  if (world < 1 || world > BF_MAX_PEERS || n_elem < 0 || (elem_bytes != 1 && elem_bytes != 4 && elem_bytes != 8))
    return (int)cudaErrorInvalidValue;
  if (n_elem == 0) return 0;
  const int grid = grid_for(n_elem * world, 256);
  if (elem_bytes == 4) peer_concat_kernel<uint32_t><<<grid, 256, 0, st>>>(to_ptrs(src, world), world, n_elem, static_cast<uint32_t*>(dst));
  else if (elem_bytes == 8) peer_concat_kernel<uint64_t><<<grid, 256, 0, st>>>(to_ptrs(src, world), world, n_elem, static_cast<uint64_t*>(dst));
  else peer_concat_kernel<uint8_t><<<grid, 256, 0, st>>>(to_ptrs(src, world), world, n_elem, static_cast<uint8_t*>(dst));
  return (int)cudaGetLastError();
}
