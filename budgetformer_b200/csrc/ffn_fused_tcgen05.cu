// Feed-forward block with the hidden tile kept on chip, for sm_100a:
//
//     Y[M, 128] = [X +] drop2( act( drop1-free hidden ) ... ) precisely:
//     H = drop1(act(X W1^T + b1))   [128 rows x 256 hidden]   never leaves the SM
//     Y = [X +] drop2(H W2^T + b2)
//
// for the layer shape of the GT / Graphormer configurations (model width 128, hidden width 256), where both weight
// matrices (2 x 64 KB in 16-bit) stay resident in shared memory for the whole persistent kernel.  Per 128-row tile:
//
//   producer warp   TMA-loads the X tile (two 64-column panels, 128-byte swizzle) into one of two buffers
//   MMA warp        GEMM1 for the two 128-column halves of the hidden tile into two TMEM accumulators (tcgen05.mma,
//                   K = 128), then for each half - once the epilogue warps have turned it into a 16-bit A operand in
//                   shared memory - GEMM2 (K = 128 per half) accumulating the 128 output columns in a third accumulator
//   16 epilogue     tcgen05.ld of a hidden half -> bias, ReLU / GELU, dropout -> 16-bit, written in the K-major
//   warps           128-byte-swizzled layout the tensor core reads (the same layout a TMA load would have produced);
//                   finally the output accumulator -> bias, dropout, residual (read from the X tile in shared memory,
//                   result written over it) -> one TMA store per 64-column panel
//
// The [M, 256] hidden matrix is neither written to nor read from HBM: the kernel moves X in and Y out (256 bytes per
// row each) where the two-GEMM form moves 4 x that.  Used where no backward pass needs the hidden matrix (evaluation,
// budget probes, the first forward of recomputed layers).  A training forward that retains activations can ask for the
// hidden matrix as a side output: a further warp bulk-stores each half from the operand buffer the second GEMM reads
// (and the epilogue leaves one bit per element, value > 0, for the backward's mask), so the matrix is written once and
// never read back by the forward pass.  Dropout masks are the hash masks of the GEMM epilogues, so a
// recomputation on the two-GEMM path reproduces them.  Every mbarrier wait is bounded (status word, early return,
// tensor memory freed).  Replaces Linear -> act -> Dropout -> Linear -> Dropout -> add of the reference layers
// (models/gt_dist_node_level.py:655-660, models/graphormer_dist_node_level.py:48-60).
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include "bf_kernels.h"
#include "sm100_ptx.cuh"

namespace {

constexpr int FF_H = 128;            // model width
constexpr int FF_F = 256;            // hidden width
constexpr int FF_M = 128;            // rows per tile
constexpr int FF_HC = 128;           // hidden columns per half
constexpr int FF_NHC = FF_F / FF_HC; // 2
constexpr int FF_PANEL = FF_M * 128; // bytes of one 64-column panel of 128 rows
constexpr int FF_EPI_WARPS = 16;
constexpr int FF_STORE_WARP = 2 + FF_EPI_WARPS;       // writes the hidden halves out when the caller keeps them
constexpr int FF_THREADS = 32 * (3 + FF_EPI_WARPS);
constexpr int FF_UMMA_K = 16;

struct FfnArgs {
  int M, m_tiles;
  const float* b1;               // [256] or null
  const float* b2;               // [128] or null
  int act;                       // 1 relu, 2 gelu (erf)
  uint32_t thresh1, seed1;       // dropout on the hidden tile (thresh 0 = off)
  float scale1;
  uint32_t thresh2, seed2;       // dropout on the output before the residual
  float scale2;
  int residual;                  // 1: Y += X
  int is_fp16;
  int* status;
  // training forward: the hidden matrix is also written out (the backward pass needs it for the weight gradient),
  // from the same shared-memory operand the second GEMM reads, together with one bit per element (value > 0)
  int store_h;
  unsigned short* bits_out;      // [256 / 16, ldmb >= M] or null
  long long ldmb;
};

struct FfnControl {
  uint64_t w_full;
  uint64_t x_full[2], x_empty[2];
  uint64_t acc1_full[2], acc1_empty[2];
  uint64_t hs_full, hs_empty, hs_stored;
  uint64_t acc2_full, acc2_empty;
  uint32_t tmem_base;
  int abort_flag;
};

__device__ __forceinline__ uint32_t ff_mix32(uint32_t x) {
  x = (x ^ (x >> 16)) * 0x7FEB352Du;
  x = (x ^ (x >> 15)) * 0x846CA68Bu;
  return x ^ (x >> 16);
}
// keep decision of ops.gemm.hash_keep_mask for element (row, col)
__device__ __forceinline__ bool ff_keep(uint32_t seed, uint32_t row, uint32_t col, uint32_t thresh) {
  return ff_mix32(row * 0x9E3779B1u + col * 0x85EBCA77u + seed) >= thresh;
}
__device__ __forceinline__ float ff_gelu(float x) { return 0.5f * x * (1.f + erff(x * 0.70710678118654752f)); }
__device__ __forceinline__ uint32_t ff_pack2(float a, float b, bool is_fp16) {
  if (is_fp16) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ float ff_lo(uint32_t w, bool is_fp16) {
  if (is_fp16) return __half2float(__ushort_as_half((unsigned short)(w & 0xFFFFu)));
  return __uint_as_float(w << 16);
}
__device__ __forceinline__ float ff_hi(uint32_t w, bool is_fp16) {
  if (is_fp16) return __half2float(__ushort_as_half((unsigned short)(w >> 16)));
  return __uint_as_float(w & 0xFFFF0000u);
}
__device__ __forceinline__ uint32_t ff_instr_desc(int n, int is_fp16) {
  uint32_t d = 0;
  d |= 1u << 4;                                  // accumulator fp32
  d |= (is_fp16 ? 0u : 1u) << 7;                 // A format: 0 fp16, 1 bf16
  d |= (is_fp16 ? 0u : 1u) << 10;                // B format
  d |= (uint32_t)(n >> 3) << 17;                 // N / 8
  d |= (uint32_t)(FF_M >> 4) << 24;              // M / 16
  return d;
}
__device__ __forceinline__ void ff_bar_sync(int threads) { asm volatile("bar.sync 2, %0;" ::"r"(threads) : "memory"); }

// 16-byte chunk holding columns [col, col + 8) of row r in a two-panel (128-column) K-major tile with the 128-byte swizzle
__device__ __forceinline__ uint8_t* ff_chunk(uint8_t* tile, int r, int col) {
  return tile + (size_t)(col >> 6) * FF_PANEL + (size_t)r * 128 + ((((col & 63) >> 3) ^ (r & 7)) << 4);
}

__global__ void __launch_bounds__(FF_THREADS, 1)
ffn_fused_tcgen05_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w1,
                         const __grid_constant__ CUtensorMap map_w2, const __grid_constant__ CUtensorMap map_y,
                         const __grid_constant__ CUtensorMap map_h, const FfnArgs g) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* s_x = smem;                                    // [2 buffers][2 panels][128 rows][128 B]
  uint8_t* s_w1 = s_x + 2 * 2 * FF_PANEL;                 // [2 halves][2 K panels][128 hidden rows][128 B]
  uint8_t* s_w2 = s_w1 + 2 * 2 * FF_PANEL;                // [4 K panels of the hidden width][128 output rows][128 B]
  uint8_t* s_h = s_w2 + 4 * FF_PANEL;                     // [2 panels][128 rows][128 B]: one hidden half as A operand
  FfnControl* ctl = reinterpret_cast<FfnControl*>(s_h + 2 * FF_PANEL);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool is_fp16 = g.is_fp16 != 0;

  if (threadIdx.x == 0) {
    mbar_init(&ctl->w_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&ctl->x_full[i], 1);
      mbar_init(&ctl->x_empty[i], 1);
      mbar_init(&ctl->acc1_full[i], 1);
      mbar_init(&ctl->acc1_empty[i], FF_EPI_WARPS);
    }
    mbar_init(&ctl->hs_full, FF_EPI_WARPS);
    mbar_init(&ctl->hs_empty, 1);
    mbar_init(&ctl->hs_stored, 1);
    mbar_init(&ctl->acc2_full, 1);
    mbar_init(&ctl->acc2_empty, FF_EPI_WARPS);
    ctl->abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    // two hidden-half accumulators (columns 0-127, 128-255) and the output accumulator (256-383): 512 columns
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&ctl->tmem_base)), "r"(512)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ctl->tmem_base;
  volatile int* abort_flag = &ctl->abort_flag;

  if (warp == 0) {
    // ------------------------------------------------------------------ producer: weights once, then X tiles
    if (lane == 0) {
      mbar_expect_tx(&ctl->w_full, 8u * FF_PANEL);
      for (int c = 0; c < FF_NHC; ++c)
        for (int p = 0; p < 2; ++p) tma_load_2d(s_w1 + (c * 2 + p) * FF_PANEL, &map_w1, &ctl->w_full, p * 64, c * FF_HC);
      for (int kp = 0; kp < 4; ++kp) tma_load_2d(s_w2 + kp * FF_PANEL, &map_w2, &ctl->w_full, kp * 64, 0);
      bool ok = true;
      int i = 0;
      for (int t = blockIdx.x; t < g.m_tiles && ok; t += gridDim.x, ++i) {
        const int b = i & 1;
        if (!mbar_wait(&ctl->x_empty[b], (uint32_t)(((i >> 1) & 1) ^ 1), abort_flag)) { ok = false; break; }
        mbar_expect_tx(&ctl->x_full[b], 2u * FF_PANEL);
        for (int p = 0; p < 2; ++p) tma_load_2d(s_x + (b * 2 + p) * FF_PANEL, &map_x, &ctl->x_full[b], p * 64, t * FF_M);
      }
      if (!ok) { *abort_flag = 1; atomicExch(g.status, 9); }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = ff_instr_desc(128, g.is_fp16);
      bool ok = mbar_wait(&ctl->w_full, 0, abort_flag);
      tc_fence_after();
      int i = 0;
      for (int t = blockIdx.x; t < g.m_tiles && ok; t += gridDim.x, ++i) {
        const int b = i & 1;
        const uint32_t par = (uint32_t)(i & 1);
        if (!mbar_wait(&ctl->x_full[b], (uint32_t)((i >> 1) & 1), abort_flag)) { ok = false; break; }
        tc_fence_after();
        // GEMM1: both hidden halves, each into its own accumulator
        for (int c = 0; c < FF_NHC && ok; ++c) {
          if (!mbar_wait(&ctl->acc1_empty[c], par ^ 1u, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t d = tmem_base + (uint32_t)(c * FF_HC);
          for (int p = 0; p < 2; ++p) {
            const uint64_t adesc = make_smem_desc(smem_u32(s_x + (b * 2 + p) * FF_PANEL));
            const uint64_t bdesc = make_smem_desc(smem_u32(s_w1 + (c * 2 + p) * FF_PANEL));
#pragma unroll
            for (int kk = 0; kk < 64 / FF_UMMA_K; ++kk)
              umma_f16(d, adesc + 2 * kk, bdesc + 2 * kk, idesc, (p > 0 || kk > 0) ? 1u : 0u);
          }
          umma_commit(&ctl->acc1_full[c]);
        }
        if (!ok) break;
        // GEMM2: as each half arrives as a 16-bit operand, accumulate its K = 128 slice of the output
        for (int c = 0; c < FF_NHC && ok; ++c) {
          if (!mbar_wait(&ctl->hs_full, (uint32_t)(c & 1), abort_flag)) { ok = false; break; }   // use index 2 i + c
          if (c == 0 && !mbar_wait(&ctl->acc2_empty, par ^ 1u, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t d = tmem_base + 2u * FF_HC;
          for (int p = 0; p < 2; ++p) {
            const uint64_t adesc = make_smem_desc(smem_u32(s_h + p * FF_PANEL));
            const uint64_t bdesc = make_smem_desc(smem_u32(s_w2 + (c * 2 + p) * FF_PANEL));
#pragma unroll
            for (int kk = 0; kk < 64 / FF_UMMA_K; ++kk)
              umma_f16(d, adesc + 2 * kk, bdesc + 2 * kk, idesc, (c > 0 || p > 0 || kk > 0) ? 1u : 0u);
          }
          umma_commit(&ctl->hs_empty);
        }
        if (!ok) break;
        umma_commit(&ctl->acc2_full);
      }
      if (!ok) { *abort_flag = 1; atomicExch(g.status, 10); }
    }
  } else if (warp == FF_STORE_WARP) {
    // ------------------------------------------------------------------ hidden halves -> HBM (training forward only)
    if (lane == 0 && g.store_h) {
      bool ok = true;
      int i = 0;
      for (int t = blockIdx.x; t < g.m_tiles && ok; t += gridDim.x, ++i) {
        for (int c = 0; c < FF_NHC && ok; ++c) {
          if (!mbar_wait(&ctl->hs_full, (uint32_t)(c & 1), abort_flag)) { ok = false; break; }   // every warp has written its part
          for (int p = 0; p < 2; ++p) tma_store_2d(&map_h, s_h + p * FF_PANEL, c * FF_HC + p * 64, t * FF_M);
          tma_store_commit();
          tma_store_wait_read<0>();
          mbar_arrive(&ctl->hs_stored);                     // the operand buffer may be overwritten as far as this copy goes
        }
      }
      tma_store_wait_all();
      if (!ok) { *abort_flag = 1; atomicExch(g.status, 12); }
    }
  } else {
    // ------------------------------------------------------------------ epilogue warps (2..17)
    const int quarter = warp & 3;                          // TMEM lane quarter this warp may read
    const int group = (warp - 2) >> 2;                     // 32 columns of every 128-column accumulator
    const int r = quarter * 32 + lane;                     // row inside the tile
    const bool leader = (warp == 2 && lane == 0);
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    bool ok = true;
    int i = 0;
    for (int t = blockIdx.x; t < g.m_tiles && ok; t += gridDim.x, ++i) {
      const int b = i & 1;
      const uint32_t par = (uint32_t)(i & 1);
      const long long row = (long long)t * FF_M + r;
      // ---- hidden halves: accumulator -> activation -> A operand in shared memory
      for (int c = 0; c < FF_NHC && ok; ++c) {
        if (!mbar_wait(&ctl->acc1_full[c], par, abort_flag)) { ok = false; break; }
        tc_fence_after();
        uint32_t acc[2][16];
        tmem_ld_32x32b_x16(tmem_base + lane_addr + (uint32_t)(c * FF_HC + group * 32), acc[0]);
        tmem_ld_32x32b_x16(tmem_base + lane_addr + (uint32_t)(c * FF_HC + group * 32 + 16), acc[1]);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&ctl->acc1_empty[c]);
        uint4 packed[2][2];
#pragma unroll
        for (int it = 0; it < 2; ++it) {
          const int hcol = c * FF_HC + group * 32 + it * 16;           // hidden column of element 0
          float v[16];
#pragma unroll
          for (int e = 0; e < 16; ++e) v[e] = __uint_as_float(acc[it][e]);
          if (g.b1 != nullptr) {
            const float4* bp = reinterpret_cast<const float4*>(g.b1 + hcol);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const float4 b4 = __ldg(bp + q);
              v[4 * q] += b4.x; v[4 * q + 1] += b4.y; v[4 * q + 2] += b4.z; v[4 * q + 3] += b4.w;
            }
          }
          if (g.act == 1) {
#pragma unroll
            for (int e = 0; e < 16; ++e) v[e] = fmaxf(v[e], 0.f);
          } else if (g.act == 2) {
#pragma unroll
            for (int e = 0; e < 16; ++e) v[e] = ff_gelu(v[e]);
          }
          if (g.thresh1) {
#pragma unroll
            for (int e = 0; e < 16; ++e)
              v[e] = ff_keep(g.seed1, (uint32_t)row, (uint32_t)(hcol + e), g.thresh1) ? v[e] * g.scale1 : 0.f;
          }
          if (g.bits_out != nullptr && row < g.M) {
            unsigned bits = 0;
#pragma unroll
            for (int e = 0; e < 16; ++e) bits |= (v[e] > 0.f ? 1u : 0u) << e;
            g.bits_out[(long long)(hcol >> 4) * g.ldmb + row] = (unsigned short)bits;
          }
          packed[it][0] = make_uint4(ff_pack2(v[0], v[1], is_fp16), ff_pack2(v[2], v[3], is_fp16),
                                     ff_pack2(v[4], v[5], is_fp16), ff_pack2(v[6], v[7], is_fp16));
          packed[it][1] = make_uint4(ff_pack2(v[8], v[9], is_fp16), ff_pack2(v[10], v[11], is_fp16),
                                     ff_pack2(v[12], v[13], is_fp16), ff_pack2(v[14], v[15], is_fp16));
        }
        // the operand buffer is free once the GEMM2 of the previous half (use index 2 i + c - 1) has retired
        if (!mbar_wait(&ctl->hs_empty, (uint32_t)((c & 1) ^ 1), abort_flag)) { ok = false; break; }
        // ... and, when the halves are kept, once the bulk store of the previous half has read it
        if (g.store_h && !mbar_wait(&ctl->hs_stored, (uint32_t)((c & 1) ^ 1), abort_flag)) { ok = false; break; }
#pragma unroll
        for (int it = 0; it < 2; ++it) {
          const int kcol = group * 32 + it * 16;                        // column inside the half = K index of GEMM2
          *reinterpret_cast<uint4*>(ff_chunk(s_h, r, kcol)) = packed[it][0];
          *reinterpret_cast<uint4*>(ff_chunk(s_h, r, kcol + 8)) = packed[it][1];
        }
        fence_async_smem();                                             // generic-proxy writes -> visible to the tensor core
        __syncwarp();
        if (lane == 0) mbar_arrive(&ctl->hs_full);
      }
      if (!ok) break;
      // ---- output: accumulator -> bias, dropout, residual -> over the X tile -> TMA store
      if (!mbar_wait(&ctl->acc2_full, par, abort_flag)) { ok = false; break; }
      tc_fence_after();
      uint32_t acc[2][16];
      tmem_ld_32x32b_x16(tmem_base + lane_addr + (uint32_t)(2 * FF_HC + group * 32), acc[0]);
      tmem_ld_32x32b_x16(tmem_base + lane_addr + (uint32_t)(2 * FF_HC + group * 32 + 16), acc[1]);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ctl->acc2_empty);
      uint8_t* xt = s_x + (size_t)b * 2 * FF_PANEL;
#pragma unroll
      for (int it = 0; it < 2; ++it) {
        const int col = group * 32 + it * 16;
        float v[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) v[e] = __uint_as_float(acc[it][e]);
        if (g.b2 != nullptr) {
          const float4* bp = reinterpret_cast<const float4*>(g.b2 + col);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const float4 b4 = __ldg(bp + q);
            v[4 * q] += b4.x; v[4 * q + 1] += b4.y; v[4 * q + 2] += b4.z; v[4 * q + 3] += b4.w;
          }
        }
        if (g.thresh2) {
#pragma unroll
          for (int e = 0; e < 16; ++e)
            v[e] = ff_keep(g.seed2, (uint32_t)row, (uint32_t)(col + e), g.thresh2) ? v[e] * g.scale2 : 0.f;
        }
        uint4* s0 = reinterpret_cast<uint4*>(ff_chunk(xt, r, col));
        uint4* s1 = reinterpret_cast<uint4*>(ff_chunk(xt, r, col + 8));
        if (g.residual) {
          const uint4 x0 = *s0, x1 = *s1;
          const uint32_t w0[4] = {x0.x, x0.y, x0.z, x0.w}, w1[4] = {x1.x, x1.y, x1.z, x1.w};
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            v[2 * q] += ff_lo(w0[q], is_fp16);     v[2 * q + 1] += ff_hi(w0[q], is_fp16);
            v[8 + 2 * q] += ff_lo(w1[q], is_fp16); v[8 + 2 * q + 1] += ff_hi(w1[q], is_fp16);
          }
        }
        *s0 = make_uint4(ff_pack2(v[0], v[1], is_fp16), ff_pack2(v[2], v[3], is_fp16),
                         ff_pack2(v[4], v[5], is_fp16), ff_pack2(v[6], v[7], is_fp16));
        *s1 = make_uint4(ff_pack2(v[8], v[9], is_fp16), ff_pack2(v[10], v[11], is_fp16),
                         ff_pack2(v[12], v[13], is_fp16), ff_pack2(v[14], v[15], is_fp16));
      }
      fence_async_smem();
      ff_bar_sync(FF_EPI_WARPS * 32);                       // the whole tile is in place
      if (leader) {
        for (int p = 0; p < 2; ++p) tma_store_2d(&map_y, xt + p * FF_PANEL, p * 64, t * FF_M);   // rows past M are clipped
        tma_store_commit();
        tma_store_wait_read<0>();                           // the buffer may be refilled once the store has read it
        mbar_arrive(&ctl->x_empty[b]);
      }
    }
    if (leader) tma_store_wait_all();
    if (!ok && lane == 0) { *abort_flag = 1; atomicExch(g.status, 11); }
  }

  // ------------------------------------------------------------------ teardown
  __syncwarp();
  if (*abort_flag) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);        // copies still in flight land before shared memory is released
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
  }
}

}  // namespace

extern "C" int bf_ffn_fused_supported(long long M, int hidden, int ffn) {
  return (M > 0 && M < (1ll << 31) - FF_M && hidden == FF_H && ffn == FF_F) ? 1 : 0;
}

extern "C" int bf_ffn_fused_fwd(const bf_ffn_params* p, cudaStream_t st) {
  if (!bf_ffn_fused_supported(p->M, p->hidden, p->ffn)) return (int)cudaErrorInvalidValue;
  if (p->act != 1 && p->act != 2) return (int)cudaErrorInvalidValue;
  if (p->dropout1 < 0.f || p->dropout1 >= 1.f || p->dropout2 < 0.f || p->dropout2 >= 1.f) return (int)cudaErrorInvalidValue;
  const uintptr_t align = (uintptr_t)p->X | (uintptr_t)p->Y | (uintptr_t)p->W1 | (uintptr_t)p->W2 | (uintptr_t)p->b1 | (uintptr_t)p->b2;
  if (!p->X || !p->Y || !p->W1 || !p->W2 || !p->status || align % 16 != 0 || (p->ldx * 2) % 16 != 0 || (p->ldy * 2) % 16 != 0 ||
      p->ldx < FF_H || p->ldy < FF_H)
    return (int)cudaErrorInvalidValue;
  FfnArgs g;
  g.M = (int)p->M; g.m_tiles = (int)((p->M + FF_M - 1) / FF_M);
  g.b1 = p->b1; g.b2 = p->b2; g.act = p->act;
  g.thresh1 = p->dropout1 > 0.f ? (uint32_t)(p->dropout1 * 4294967296.0) : 0u;
  g.scale1 = p->dropout1 > 0.f ? 1.f / (1.f - p->dropout1) : 1.f;
  g.seed1 = p->seed1;
  g.thresh2 = p->dropout2 > 0.f ? (uint32_t)(p->dropout2 * 4294967296.0) : 0u;
  g.scale2 = p->dropout2 > 0.f ? 1.f / (1.f - p->dropout2) : 1.f;
  g.seed2 = p->seed2;
  g.residual = p->residual ? 1 : 0;
  g.is_fp16 = p->dtype == BF_FP16 ? 1 : 0;
  g.status = p->status;
  g.store_h = p->H_out != nullptr ? 1 : 0;
  g.bits_out = static_cast<unsigned short*>(p->relu_bits_out);
  g.ldmb = p->ldmb;
  if (g.store_h && (((uintptr_t)p->H_out) % 16 != 0 || (p->ldh * 2) % 16 != 0 || p->ldh < FF_F)) return (int)cudaErrorInvalidValue;
  if (g.bits_out != nullptr && p->ldmb < p->M) return (int)cudaErrorInvalidValue;
  CUtensorMap map_x, map_w1, map_w2, map_y, map_h;
  memset(&map_h, 0, sizeof(map_h));
  if (g.store_h && make_map(&map_h, p->H_out, p->M, FF_F, p->ldh, FF_M, g.is_fp16) != 0) return (int)cudaErrorNotSupported;
  if (make_map(&map_x, p->X, p->M, FF_H, p->ldx, FF_M, g.is_fp16) != 0) return (int)cudaErrorNotSupported;
  if (make_map(&map_w1, p->W1, FF_F, FF_H, FF_H, FF_HC, g.is_fp16) != 0) return (int)cudaErrorNotSupported;
  if (make_map(&map_w2, p->W2, FF_H, FF_F, FF_F, FF_H, g.is_fp16) != 0) return (int)cudaErrorNotSupported;
  if (make_map(&map_y, p->Y, p->M, FF_H, p->ldy, FF_M, g.is_fp16) != 0) return (int)cudaErrorNotSupported;
  const size_t smem = 1024 + (size_t)14 * FF_PANEL + sizeof(FfnControl) + 64;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  {
    constexpr int MAX_DEV = 64;
    static bool attr_set[MAX_DEV] = {};
    if (dev < 0 || dev >= MAX_DEV || !attr_set[dev]) {
      cudaError_t e = cudaFuncSetAttribute(ffn_fused_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return (int)e;
      if (dev >= 0 && dev < MAX_DEV) attr_set[dev] = true;
    }
  }
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int grid = g.m_tiles < sms ? g.m_tiles : sms;
  ffn_fused_tcgen05_kernel<<<grid, FF_THREADS, smem, st>>>(map_x, map_w1, map_w2, map_y, map_h, g);
  return (int)cudaGetLastError();
}
