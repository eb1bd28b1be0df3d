// Weight-gradient GEMM for sm_100a:  dW[N, K] = dY[M, N]^T * X[M, K]  (+ the column sums of dY = bias gradient).
//
// The reduction runs over the rows (millions of them), the output is a small matrix: each CTA owns one 128-row
// tile of dW (128 columns of dY) and one slice of the rows, streams both operands through a TMA ring and leaves
// a fp32 partial tile; a second kernel adds the partials of all row slices in slice order (bit-reproducible) and
// writes - or accumulates into - the gradient.
//
// * both operands are row-major [rows, features], i.e. the reduction dimension is the *strided* one: the TMA boxes
//   (64 features x 64 rows, 128-byte swizzle) land as MN-major operand tiles and the instruction descriptor marks A
//   and B as MN-major; one tcgen05.mma covers 16 rows (M = 128 features of dY, N <= 256 features of X);
// * the bias gradient comes from the same instruction stream: one more 16-column group of the B tile is a constant
//   matrix whose first column is ones, so accumulator column K holds sum_r dY[r, :] (no second pass over dY);
// * rows beyond M and features beyond N / K are zero-filled by TMA, so ragged shapes need no special code;
// * every mbarrier wait is bounded (status word + early return, tensor memory freed).
// Replaces the autograd of the reference's nn.Linear layers (e.g. models/gt_dist_node_level.py:558-560,651,655-660),
// which runs as library GEMMs there.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include "bf_kernels.h"
#include "sm100_ptx.cuh"

namespace {

constexpr int DW_TILE_M = 128;       // features of dY per CTA (accumulator lanes)
constexpr int DW_ROWS = 64;          // rows per ring stage
// Features of X per work item.  128 (not the 256 one instruction could take): a 256-wide item measured 0.72 of the copy
// bandwidth against 0.92-1.0 for 128-wide ones, and two 128-wide items of one row slice run side by side and share
// their dY tiles through L2 (as the feature tiles of a wide dY share X); the accumulator always has 16 columns to
// spare for the bias gradient.
constexpr int DW_CHUNK_K = 128;
constexpr int DW_STAGES = 4;
constexpr int DW_THREADS = 192;      // warp 0: TMA, warp 1: MMA + TMEM owner, warps 2-5: epilogue (one lane quarter each)
constexpr int DW_GROUP_BYTES = DW_ROWS * 128;   // one 64-feature group of a stage: 64 rows x 128 bytes

struct DwArgs {
  int M, N, K;                       // rows, features of dY, features of X
  int n_tiles;                       // ceil(N / 128)
  int k_chunks;                      // column chunks of X (<= DW_CHUNK_K features each)
  int splits;                        // row slices
  long long rows_per_split;          // multiple of DW_ROWS
  int bias_chunk;                    // column chunk whose B tile carries the ones group (-1: no bias gradient)
  int is_fp16;
  float* partial;                    // [splits, N, K] fp32
  float* bias_partial;               // [splits, N] fp32 (with_bias)
  int* status;
};

// MN-major operand tile, 128-byte swizzle: 64 features contiguous (128 bytes) per row, rows 128 bytes apart, 8-row
// groups 1024 bytes apart (stride offset), 64-feature groups `group_bytes` apart (leading offset).
__device__ __forceinline__ uint64_t make_smem_desc_mn(uint32_t smem_addr, uint32_t group_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)((group_bytes >> 4) & 0x3FFFu) << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;                               // SWIZZLE_128B
  return d;
}

__device__ __forceinline__ uint32_t make_instr_desc_mn(int n, int is_fp16) {
  uint32_t d = 0;
  d |= 1u << 4;                                  // accumulator fp32
  d |= (is_fp16 ? 0u : 1u) << 7;                 // A format
  d |= (is_fp16 ? 0u : 1u) << 10;                // B format
  d |= 1u << 15;                                 // A is MN-major
  d |= 1u << 16;                                 // B is MN-major
  d |= (uint32_t)(n >> 3) << 17;
  d |= (uint32_t)(DW_TILE_M >> 4) << 24;
  return d;
}

struct DwControl {
  uint64_t full[DW_STAGES];
  uint64_t empty[DW_STAGES];
  uint64_t done;
  uint32_t tmem_base;
  int abort_flag;
};

__global__ void __launch_bounds__(DW_THREADS, 1)
gemm_dw_tcgen05_kernel(const __grid_constant__ CUtensorMap map_y, const __grid_constant__ CUtensorMap map_x, const DwArgs g) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  // work item: (row slice, feature tile of dY, column chunk of X); items of one slice are adjacent so that they
  // stream the same rows at the same time and share them through L2
  const int per_split = g.n_tiles * g.k_chunks;
  const int split = blockIdx.x / per_split;
  const int tile = (blockIdx.x % per_split) / g.k_chunks;
  const int chunk = blockIdx.x % g.k_chunks;
  const int k0 = chunk * DW_CHUNK_K;
  const int kw = min(DW_CHUNK_K, g.K - k0);              // features of X in this chunk
  const bool bias_here = chunk == g.bias_chunk;
  const int x_groups = (kw + 63) / 64;
  // the ones columns live in a 64-feature group of their own, which no TMA box ever overwrites
  const int b_groups = x_groups + (bias_here ? 1 : 0);
  const int bias_col = x_groups * 64;                                     // accumulator column of the bias gradient
  const int n_mma = bias_here ? bias_col + 16 : ((kw + 15) & ~15);        // N of the instruction (<= 256 by construction)
  const uint32_t a_bytes = 2 * DW_GROUP_BYTES;
  const uint32_t stage_bytes = a_bytes + (uint32_t)b_groups * DW_GROUP_BYTES;
  DwControl* ctl = reinterpret_cast<DwControl*>(smem + DW_STAGES * stage_bytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long row_begin = (long long)split * g.rows_per_split;
  const long long row_end = min((long long)g.M, row_begin + g.rows_per_split);
  const int n_iter = row_end > row_begin ? (int)((row_end - row_begin + DW_ROWS - 1) / DW_ROWS) : 0;
  const uint32_t tmem_cols = n_mma <= 32 ? 32 : n_mma <= 64 ? 64 : n_mma <= 128 ? 128 : 256;

  if (threadIdx.x == 0) {
    for (int s = 0; s < DW_STAGES; ++s) { mbar_init(&ctl->full[s], 1); mbar_init(&ctl->empty[s], 1); }
    mbar_init(&ctl->done, 1);
    ctl->abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (bias_here) {
    // constant part of every stage's B tile: feature 0 of the extra group is 1 in every row, features 1..15 are 0, so
    // accumulator column `bias_col` sums dY over the rows.  Chunks are placed like the TMA places them (chunk ^ (row & 7)).
    for (int s = 0; s < DW_STAGES; ++s) {
      uint8_t* gbase = smem + s * stage_bytes + a_bytes + x_groups * DW_GROUP_BYTES;
      for (int i = threadIdx.x; i < DW_ROWS * 2; i += blockDim.x) {
        const int r = i >> 1, c = i & 1;                                     // the 16 features used: two 16-byte chunks
        uint4 v = make_uint4(0, 0, 0, 0);
        if (c == 0) v.x = g.is_fp16 ? 0x00003C00u : 0x00003F80u;            // 1.0 in the low half-word
        *reinterpret_cast<uint4*>(gbase + r * 128 + ((c ^ (r & 7)) << 4)) = v;
      }
    }
    fence_async_smem();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&ctl->tmem_base)),
                 "r"(tmem_cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ctl->tmem_base;
  volatile int* abort_flag = &ctl->abort_flag;

  if (warp == 0) {
    if (lane == 0) {
      bool ok = true;
      for (int it = 0; it < n_iter && ok; ++it) {
        const int stage = it % DW_STAGES;
        const uint32_t phase = (uint32_t)((it / DW_STAGES) & 1);
        if (!mbar_wait(&ctl->empty[stage], phase ^ 1u, abort_flag)) { ok = false; break; }
        uint8_t* sa = smem + stage * stage_bytes;
        uint8_t* sb = sa + a_bytes;
        mbar_expect_tx(&ctl->full[stage], a_bytes + (uint32_t)x_groups * DW_GROUP_BYTES);
        const int y = (int)(row_begin + (long long)it * DW_ROWS);     // rows past M read zeros
        tma_load_2d(sa, &map_y, &ctl->full[stage], tile * DW_TILE_M, y);
        tma_load_2d(sa + DW_GROUP_BYTES, &map_y, &ctl->full[stage], tile * DW_TILE_M + 64, y);
        for (int gi = 0; gi < x_groups; ++gi)
          tma_load_2d(sb + gi * DW_GROUP_BYTES, &map_x, &ctl->full[stage], k0 + gi * 64, y);
      }
      if (!ok) { *abort_flag = 1; atomicExch(g.status, 6); }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = make_instr_desc_mn(n_mma, g.is_fp16);
      bool ok = true;
      for (int it = 0; it < n_iter && ok; ++it) {
        const int stage = it % DW_STAGES;
        const uint32_t phase = (uint32_t)((it / DW_STAGES) & 1);
        if (!mbar_wait(&ctl->full[stage], phase, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t sa = smem_u32(smem + stage * stage_bytes);
        const uint32_t sb = sa + a_bytes;
#pragma unroll
        for (int kk = 0; kk < DW_ROWS / 16; ++kk) {
          // 16 rows further along the reduction: two 8-row groups = 2048 bytes
          umma_f16(tmem_base, make_smem_desc_mn(sa + kk * 2048, DW_GROUP_BYTES), make_smem_desc_mn(sb + kk * 2048, DW_GROUP_BYTES),
                   idesc, (it > 0 || kk > 0) ? 1u : 0u);
        }
        umma_commit(&ctl->empty[stage]);
      }
      if (ok) umma_commit(&ctl->done);
      else { *abort_flag = 1; atomicExch(g.status, 7); }
    }
  } else {
    // ------------------------------------------------------------------ epilogue: accumulator -> fp32 partial tile
    const int quarter = warp & 3;                        // TMEM lane quarter this warp may read
    const int m_local = quarter * 32 + lane;
    const int n_row = tile * DW_TILE_M + m_local;        // row of dW
    bool ok = true;
    if (n_iter > 0) ok = mbar_wait(&ctl->done, 0, abort_flag);
    if (ok) {
      tc_fence_after();
      float* prow = g.partial + ((long long)split * g.N + n_row) * g.K + k0;
      for (int c0 = 0; c0 < n_mma; c0 += 16) {
        uint32_t r[16];
        if (n_iter > 0) {
          tmem_ld_32x32b_x16(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c0, r);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i) r[i] = 0u;        // an empty row slice contributes zeros
        }
        if (n_row >= g.N) continue;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int c = c0 + 4 * q;
          if (c + 4 <= kw) {
            *reinterpret_cast<float4*>(prow + c) = make_float4(__uint_as_float(r[4 * q]), __uint_as_float(r[4 * q + 1]),
                                                               __uint_as_float(r[4 * q + 2]), __uint_as_float(r[4 * q + 3]));
          } else {
#pragma unroll
            for (int i = 0; i < 4; ++i)
              if (c + i < kw) prow[c + i] = __uint_as_float(r[4 * q + i]);
          }
        }
        if (bias_here && c0 == bias_col) g.bias_partial[(long long)split * g.N + n_row] = __uint_as_float(r[0]);
      }
    } else if (lane == 0) {
      *abort_flag = 1;
      atomicExch(g.status, 8);
    }
  }

  __syncwarp();
  if (*abort_flag) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);    // copies still in flight land before shared memory is released
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
  }
}

// out[i] (= or +=) sum over slices of partial[s][i], slices added in order.
__global__ void __launch_bounds__(256) dw_reduce_kernel(const float* __restrict__ partial, long long n_elem, int splits,
                                                        float* __restrict__ out, int accumulate, float scale) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_elem) return;
  float acc = 0.f;
  for (int s = 0; s < splits; ++s) acc += partial[(long long)s * n_elem + i];
  acc *= scale;
  out[i] = accumulate ? out[i] + acc : acc;
}

}  // namespace

extern "C" int bf_gemm_dw_supported(long long M, int N, int K) {
  return (M > 0 && N >= 8 && N % 8 == 0 && K >= 8 && K % 8 == 0) ? 1 : 0;
}

extern "C" long long bf_gemm_dw_splits(long long M, int N, int K) {
  if (!bf_gemm_dw_supported(M, N, K)) return 0;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int items = ((N + DW_TILE_M - 1) / DW_TILE_M) * ((K + DW_CHUNK_K - 1) / DW_CHUNK_K);
  long long splits = sms / items;
  if (splits < 1) splits = 1;
  const long long max_splits = (M + DW_ROWS - 1) / DW_ROWS;
  return splits < max_splits ? splits : max_splits;
}

extern "C" int bf_gemm_dw_bias_supported(int K) {
  const int kw_last = K - DW_CHUNK_K * ((K + DW_CHUNK_K - 1) / DW_CHUNK_K - 1);
  return (kw_last + 63) / 64 * 64 + 16 <= 256 ? 1 : 0;      // always true for chunks of at most 128 features
}

extern "C" size_t bf_gemm_dw_scratch_bytes(long long M, int N, int K) {
  const long long s = bf_gemm_dw_splits(M, N, K);
  return (size_t)s * (size_t)N * ((size_t)K + 1) * sizeof(float);
}

extern "C" int bf_gemm_dw(const bf_gemm_dw_params* p, cudaStream_t st) {
  if (!bf_gemm_dw_supported(p->M, p->N, p->K)) return (int)cudaErrorInvalidValue;
  if (((uintptr_t)p->dY) % 16 || ((uintptr_t)p->X) % 16 || (p->ldy * 2) % 16 || (p->ldx * 2) % 16 || !p->dW || !p->scratch)
    return (int)cudaErrorInvalidValue;
  DwArgs g;
  g.M = (int)p->M; g.N = p->N; g.K = p->K;
  g.n_tiles = (p->N + DW_TILE_M - 1) / DW_TILE_M;
  g.k_chunks = (p->K + DW_CHUNK_K - 1) / DW_CHUNK_K;
  g.splits = (int)bf_gemm_dw_splits(p->M, p->N, p->K);
  const long long per = (p->M + g.splits - 1) / g.splits;
  g.rows_per_split = (per + DW_ROWS - 1) / DW_ROWS * DW_ROWS;
  // the ones group rides with the last column chunk when that chunk leaves 16 accumulator columns free
  const int kw_last = p->K - DW_CHUNK_K * (g.k_chunks - 1);
  const bool bias_fits = (kw_last + 63) / 64 * 64 + 16 <= 256;
  if (p->dbias != nullptr && !bias_fits) return (int)cudaErrorNotSupported;
  g.bias_chunk = p->dbias != nullptr ? g.k_chunks - 1 : -1;
  g.is_fp16 = p->dtype == BF_FP16 ? 1 : 0;
  g.partial = static_cast<float*>(p->scratch);
  g.bias_partial = g.partial + (size_t)g.splits * p->N * p->K;
  g.status = p->status;
  CUtensorMap map_y, map_x;
  if (make_map(&map_y, p->dY, p->M, p->N, p->ldy, DW_ROWS, g.is_fp16) != 0) return (int)cudaErrorNotSupported;
  if (make_map(&map_x, p->X, p->M, p->K, p->ldx, DW_ROWS, g.is_fp16) != 0) return (int)cudaErrorNotSupported;
  // shared memory: the widest work item decides
  int groups0 = 0;
  for (int c = 0; c < g.k_chunks; ++c) {
    const int kw = (p->K - DW_CHUNK_K * c) < DW_CHUNK_K ? (p->K - DW_CHUNK_K * c) : DW_CHUNK_K;
    const int gr = (kw + 63) / 64 + (c == g.bias_chunk ? 1 : 0);
    groups0 = gr > groups0 ? gr : groups0;
  }
  const size_t smem = 1024 + (size_t)DW_STAGES * (2 + groups0) * DW_GROUP_BYTES + sizeof(DwControl) + 64;
  if (smem > 227 * 1024) return (int)cudaErrorNotSupported;
  int dev = 0;
  cudaGetDevice(&dev);
  {
    constexpr int MAX_DEV = 64;
    static bool attr_set[MAX_DEV] = {};
    if (dev < 0 || dev >= MAX_DEV || !attr_set[dev]) {
      cudaError_t e = cudaFuncSetAttribute(gemm_dw_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
      if (e != cudaSuccess) return (int)e;
      if (dev >= 0 && dev < MAX_DEV) attr_set[dev] = true;
    }
  }
  const int grid = g.splits * g.n_tiles * g.k_chunks;
  gemm_dw_tcgen05_kernel<<<grid, DW_THREADS, smem, st>>>(map_y, map_x, g);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  const long long n_elem = (long long)p->N * p->K;
  dw_reduce_kernel<<<(unsigned)((n_elem + 255) / 256), 256, 0, st>>>(g.partial, n_elem, g.splits, p->dW, p->accumulate,
                                                                    p->scale == 0.f ? 1.f : p->scale);
  if (g.bias_chunk >= 0)
    dw_reduce_kernel<<<(unsigned)((p->N + 255) / 256), 256, 0, st>>>(g.bias_partial, p->N, g.splits, p->dbias, p->accumulate,
                                                                    p->scale == 0.f ? 1.f : p->scale);
  return (int)cudaGetLastError();
}
