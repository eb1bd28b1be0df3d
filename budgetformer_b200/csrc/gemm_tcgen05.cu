// Persistent tcgen05 GEMM for sm_100a with fused epilogues and a fused nodes->heads all-to-all.
//
//   C[M, N] = A[M, K] * B[N, K]^T      bf16 / fp16 operands, fp32 accumulation in tensor memory
//
// * operands are staged by TMA (cp.async.bulk.tensor, 128-byte swizzle, one 64-element K panel per
//   stage; a ragged last panel is zero-filled) into a 3- or 4-deep shared-memory ring; one elected thread
//   issues tcgen05.mma (M = 128, N = BLOCK_N <= 256, K = 16 per instruction) and releases ring stages with
//   tcgen05.commit;
// * two accumulators of BLOCK_N columns alternate in tensor memory, so the sixteen epilogue warps drain
//   tile i (tcgen05.ld) while tile i+1 is being multiplied;
// * epilogue (per thread = one output row, four column groups): + bias, ReLU / GELU, counter-based dropout,
//   + residual, ReLU-gradient mask (residual / mask tiles are fetched with cp.async one tile ahead), results
//   staged in shared memory and written with bulk TMA stores.  With `n_dest > 1` the columns of a tile are
//   routed to the owning rank's buffer through peer pointers: this is the sequence-parallel nodes->heads
//   all-to-all (3 projections + 3 all-to-alls + 6 copies in the reference: gt_sp/layer.py:35-41,264-266)
//   executed by the GEMM itself, tile by tile, over NVLink - one bulk store per destination slice of a row
//   tile (plain 32-byte st.global only when a slice is not a multiple of 16 columns);
// * the epilogue feature set is a template parameter for the combinations the layers use (bf16), a generic
//   instance covers everything else;
// * with `n_src > 1` the A operand itself is gathered over NVLink: columns [s*K/n_src, (s+1)*K/n_src) of a row
//   tile are this rank's rows of source s's buffer (the heads->nodes all-to-all of gt_sp/layer.py:280 and its
//   backward twin).  One loader warp per ring stage fetches them with 16-byte asynchronous copies (cp.async from the
//   peers' memory, lanes running along each source's contiguous rows so that a request covers whole 128-byte lines)
//   straight to their place in the 128-byte-swizzled operand stage, so the transfer of tile i+1 overlaps the
//   multiplication of tile i and no gathered [M, K] matrix exists unless the caller asks for it: `a_copy` makes one
//   more warp write every landed operand stage to a local row-major matrix with bulk stores (what the
//   weight-gradient GEMM of the backward pass reads);
// * every mbarrier wait is bounded: on expiry the kernel records a status word, stops issuing work,
//   lets copies in flight land, frees its tensor memory and returns.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>
#include <stdlib.h>

#include "bf_kernels.h"
#include "sm100_ptx.cuh"

namespace {

constexpr int BLOCK_M = 128;
constexpr int BLOCK_K = 64;          // one 128-byte swizzle panel of 16-bit elements
constexpr int UMMA_K = 16;
constexpr int MAX_STAGES = 4;
constexpr int NUM_THREADS = 576;     // warp 0: TMA, warp 1: MMA + TMEM owner, warps 2-17: epilogue (four column groups)
// gathered operand: + warp 18 (writes landed A stages to the local copy) + warps 19-22 (one loader per ring stage)
constexpr int COPY_WARP = 18;
constexpr int FIRST_LOADER_WARP = 19;
constexpr int NUM_THREADS_PULL = (FIRST_LOADER_WARP + MAX_STAGES) * 32;

struct GemmArgs {
  int M, N, K;
  int block_n, n_chunks, m_tiles;
  int is_fp16;
  // epilogue
  const float* bias;             // [N] or null
  int act;                       // 0 none, 1 relu, 2 gelu
  float dropout_p;               // applied after activation
  uint32_t dropout_seed;
  const void* residual;          // [M, ldr] 16-bit or null
  long long ldr;
  const void* relu_mask;         // [M, ldm] 16-bit: out = mask > 0 ? acc : 0
  long long ldm;
  int mask_mode;                 // 1: out = acc * gelu'(mask) instead (mask holds the pre-activation)
  unsigned short* bits_out;      // [N/16, ldmb >= M] one bit per element, word (c, r) = columns 16c..16c+15 of row r: bit = result > 0
  const unsigned short* bits_in; // same layout: out = bit ? acc : 0
  long long ldmb;
  float out_scale;
  int out_fp32;
  // output routing
  int n_dest;                    // 1 = plain row-major output
  int cols_per_dest;             // N / n_dest
  long long dst_row_offset;      // row offset inside every destination buffer
  long long ldc;                 // destination row stride (elements)
  void* dst[BF_MAX_PEERS];
  int* status;                   // [4] device status words (0 = ok)
  // shared-memory plan (host decides what fits in 227 KB)
  int stages;                    // operand ring depth (3 or 4)
  int tma_store;                 // 1: epilogue stages 64-column panels in shared memory and writes them with TMA
  int out_bufs;                  // staging buffers (1 to 3) when tma_store
  int bias_in_smem;              // bias copied to shared memory once per CTA (N <= 1024)
  int n_groups;                  // epilogue column groups in use (4, 2 or 1)
  int panel_w;                   // columns per staged output panel: 64 (128-byte swizzle) or a destination's slice (unswizzled)
  // gathered A operand
  int n_src;                     // 1 = A is one local matrix
  int cols_per_src;              // K / n_src, a multiple of 8
  long long src_row_offset;      // first row of this rank's block inside every source buffer
  long long src_ld;              // row stride of the source buffers (elements)
  const void* src[BF_MAX_PEERS];
  int a_copy;                    // 1: the copy warp stores every landed A stage to the local copy
};

struct OutMaps {
  CUtensorMap m[BF_MAX_PEERS];   // one per destination; row extent = dst_row_offset + M so that tail rows are clipped
};



__device__ __forceinline__ uint32_t make_instr_desc(int block_n, int is_fp16) {
  uint32_t d = 0;
  d |= 1u << 4;                                  // accumulator fp32
  d |= (is_fp16 ? 0u : 1u) << 7;                 // A format: 0 fp16, 1 bf16
  d |= (is_fp16 ? 0u : 1u) << 10;                // B format
  d |= (uint32_t)(block_n >> 3) << 17;           // N / 8
  d |= (uint32_t)(BLOCK_M >> 4) << 24;           // M / 16
  return d;
}


__device__ __forceinline__ uint32_t mix32(uint32_t x) {
  x = (x ^ (x >> 16)) * 0x7FEB352Du;
  x = (x ^ (x >> 15)) * 0x846CA68Bu;
  return x ^ (x >> 16);
}
// keep decision for element (row, col) — identical to ops/dropout.py::hash_keep_mask
__device__ __forceinline__ bool keep_elem(uint32_t seed, uint32_t row, uint32_t col, uint32_t thresh) {
  return mix32(row * 0x9E3779B1u + col * 0x85EBCA77u + seed) >= thresh;
}

__device__ __forceinline__ float gelu_erf(float x) { return 0.5f * x * (1.f + erff(x * 0.70710678118654752f)); }
// d/dx of the above: Phi(x) + x * phi(x)
__device__ __forceinline__ float gelu_erf_grad(float x) {
  return 0.5f * (1.f + erff(x * 0.70710678118654752f)) + x * 0.3989422804014327f * __expf(-0.5f * x * x);
}

// the two 16-bit floats packed in one 32-bit word, widened
__device__ __forceinline__ float lo16_as_float(uint32_t w, bool is_fp16) {
  if (is_fp16) return __half2float(__ushort_as_half((unsigned short)(w & 0xFFFFu)));
  return __uint_as_float(w << 16);
}
__device__ __forceinline__ float hi16_as_float(uint32_t w, bool is_fp16) {
  if (is_fp16) return __half2float(__ushort_as_half((unsigned short)(w >> 16)));
  return __uint_as_float(w & 0xFFFF0000u);
}
__device__ __forceinline__ uint32_t pack2(float a, float b, bool is_fp16) {
  if (is_fp16) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

__device__ __forceinline__ void epilogue_bar_sync(int threads) { asm volatile("bar.sync 1, %0;" ::"r"(threads) : "memory"); }

struct __align__(1024) SmemLayout {
  // operand ring follows at offset 0 of the dynamic buffer (A stages then B stages), then this control block
};

struct Control {
  uint64_t full[MAX_STAGES];
  uint64_t empty[MAX_STAGES];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

// Epilogue features fixed at compile time in the specialised instantiations (bf16 only); EPI < 0 reads all of
// them from the arguments at run time (any dtype, any combination).
constexpr int EPI_BIAS = 1, EPI_RELU = 2, EPI_GELU = 4, EPI_DROP = 8, EPI_RES = 16, EPI_MASK = 32, EPI_SCALE = 64;

template <int EPI, bool PULL>
__global__ void __launch_bounds__(PULL ? NUM_THREADS_PULL : NUM_THREADS, 1)
gemm_tn_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                       const __grid_constant__ OutMaps omaps, const __grid_constant__ CUtensorMap map_copy, const GemmArgs g) {
  constexpr bool GEN = EPI < 0;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // 1024-byte alignment is required by the 128-byte swizzle atoms
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t a_stage_bytes = BLOCK_M * BLOCK_K * 2;
  const uint32_t b_stage_bytes = (uint32_t)g.block_n * BLOCK_K * 2;
  const int STAGES = g.stages;
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem + STAGES * a_stage_bytes;
  uint8_t* smem_out = smem_b + STAGES * b_stage_bytes;              // [out_bufs][block_n/64][128 rows][128 B], swizzled
  const uint32_t out_buf_bytes = g.tma_store ? (uint32_t)(g.block_n / 64) * BLOCK_M * 128u : 0u;
  Control* ctl = reinterpret_cast<Control*>(smem_out + (size_t)g.out_bufs * out_buf_bytes);
  float* s_bias = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(ctl) + ((sizeof(Control) + 15) & ~size_t(15)));  // [N]

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int k_panels = (g.K + BLOCK_K - 1) / BLOCK_K;   // a ragged last panel is zero-filled by TMA (both operands)
  const int total_tiles = g.m_tiles * g.n_chunks;
  const uint32_t tmem_cols = (2 * g.block_n <= 32) ? 32 : (2 * g.block_n <= 64) ? 64 : (2 * g.block_n <= 128) ? 128
                            : (2 * g.block_n <= 256) ? 256 : 512;

  if (threadIdx.x == 0) {
    // gathered operand: a stage is full when the TMA bytes of B have landed and its loader warp has arrived; it is
    // free again when its MMAs have retired and, with a local copy, when the copy warp has read it
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&ctl->full[s], PULL ? 2 : 1);
      mbar_init(&ctl->empty[s], 1 + ((PULL && g.a_copy) ? 1 : 0));
    }
    for (int a = 0; a < 2; ++a) { mbar_init(&ctl->tmem_full[a], 1); mbar_init(&ctl->tmem_empty[a], 4 * g.n_groups); }
    ctl->abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (g.bias != nullptr && g.bias_in_smem) {
    for (int i = threadIdx.x; i < g.N; i += blockDim.x) s_bias[i] = g.bias[i];
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
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        const int m_tile = t / g.n_chunks, n_chunk = t % g.n_chunks;
        for (int kp = 0; kp < k_panels; ++kp) {
          if (!mbar_wait(&ctl->empty[stage], phase ^ 1u, abort_flag)) { ok = false; break; }
          if (PULL) {
            mbar_expect_tx(&ctl->full[stage], b_stage_bytes);            // A arrives through the loader warps
          } else {
            mbar_expect_tx(&ctl->full[stage], a_stage_bytes + b_stage_bytes);
            tma_load_2d(smem_a + stage * a_stage_bytes, &map_a, &ctl->full[stage], kp * BLOCK_K, m_tile * BLOCK_M);
          }
          tma_load_2d(smem_b + stage * b_stage_bytes, &map_b, &ctl->full[stage], kp * BLOCK_K, n_chunk * g.block_n);
          if (++stage == (uint32_t)STAGES) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) { *abort_flag = 1; atomicExch(g.status, 1); }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = make_instr_desc(g.block_n, g.is_fp16);
      uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        if (!mbar_wait(&ctl->tmem_empty[acc], acc_phase ^ 1u, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * (uint32_t)g.block_n;
        for (int kp = 0; kp < k_panels; ++kp) {
          if (!mbar_wait(&ctl->full[stage], phase, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint64_t bdesc = make_smem_desc(smem_u32(smem_b + stage * b_stage_bytes));
          const uint64_t adesc = make_smem_desc(smem_u32(smem_a + stage * a_stage_bytes));
          // a gathered operand has no zero-filled tail: a short last stage issues fewer K steps
          const int k_steps = PULL ? min(BLOCK_K, g.K - kp * BLOCK_K) / UMMA_K : BLOCK_K / UMMA_K;
#pragma unroll
          for (int kk = 0; kk < BLOCK_K / UMMA_K; ++kk) {
            // advance 32 bytes (16 elements) along K inside the swizzle atom: +2 in 16-byte units
            if (kk < k_steps) umma_f16(tmem_d, adesc + 2 * kk, bdesc + 2 * kk, idesc, (kp > 0 || kk > 0) ? 1u : 0u);
          }
          umma_commit(&ctl->empty[stage]);
          if (++stage == (uint32_t)STAGES) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        umma_commit(&ctl->tmem_full[acc]);
        if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
      }
      if (!ok) { *abort_flag = 1; atomicExch(g.status, 2); }
    }
  } else if (PULL && warp == COPY_WARP) {
    // ------------------------------------------------------------------ local copy of the gathered A operand
    if (lane == 0 && g.a_copy) {
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        const int m_tile = t / g.n_chunks, n_chunk = t % g.n_chunks;
        for (int kp = 0; kp < k_panels; ++kp) {
          if (!mbar_wait(&ctl->full[stage], phase, abort_flag)) { ok = false; break; }
          // a row tile is fetched once per column chunk of the output: only the first visit is written out; columns
          // past K and rows past M are outside the map and are clipped
          if (n_chunk == 0) {
            tma_store_2d(&map_copy, smem_a + stage * a_stage_bytes, kp * BLOCK_K, m_tile * BLOCK_M);
            tma_store_commit();
            tma_store_wait_read<0>();
          }
          mbar_arrive(&ctl->empty[stage]);
          if (++stage == (uint32_t)STAGES) { stage = 0; phase ^= 1u; }
        }
      }
      tma_store_wait_all();
      if (!ok) { *abort_flag = 1; atomicExch(g.status, 4); }
    }
  } else if (PULL && warp >= FIRST_LOADER_WARP) {
    // ------------------------------------------------------------------ loaders of the gathered A operand
    // Loader j owns ring stage j (a waiter on a phase parity may never be more than one phase behind, so a stage is
    // not shared between loaders).  Within a stage the 64 columns fall into segments that belong to one source each;
    // the lanes run along a segment's rows, which are contiguous in the source when the segment is a whole row.
    const int lw = warp - FIRST_LOADER_WARP;
    if (lw < STAGES) {
      bool ok = true;
      long long it = 0;                                      // stage counter of this CTA
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        const int m_tile = t / g.n_chunks;
        const long long row_base = g.src_row_offset + (long long)m_tile * BLOCK_M;
        const int rows_valid = min(BLOCK_M, g.M - m_tile * BLOCK_M);
        for (int kp = 0; kp < k_panels; ++kp, ++it) {
          if ((int)(it % STAGES) != lw) continue;
          const uint32_t phase = (uint32_t)((it / STAGES) & 1);
          if (!mbar_wait(&ctl->empty[lw], phase ^ 1u, abort_flag)) { ok = false; break; }
          uint8_t* dst = smem_a + lw * a_stage_bytes;
          const int k0 = kp * BLOCK_K;
          const int k_end = min(g.K, k0 + BLOCK_K);
          for (int col = k0; col < k_end;) {
            const int src = col / g.cols_per_src;
            const int seg_end = min(k_end, (src + 1) * g.cols_per_src);
            const int wch = (seg_end - col) >> 3;            // 16-byte chunks per row of this segment
            const int c0 = (col - k0) >> 3;                  // its first chunk inside the stage row
            const unsigned short* base = static_cast<const unsigned short*>(g.src[src]) + (col - src * g.cols_per_src);
            const int n = BLOCK_M * wch;
            for (int q = lane; q < n; q += 32) {
              const int r = q / wch, cc = q - r * wch;
              // rows past M (tail tile) repeat the last valid row: their products are clipped by the epilogue
              const int rr = r < rows_valid ? r : rows_valid - 1;
              const int c = c0 + cc;
              cp_async_16(dst + r * 128 + ((c ^ (r & 7)) << 4), base + (row_base + rr) * g.src_ld + cc * 8);
            }
            col = seg_end;
          }
          cp_async_wait_all();
          fence_async_smem();                                // generic-proxy writes -> visible to the MMA and the bulk store
          __syncwarp();
          if (lane == 0) mbar_arrive(&ctl->full[lw]);
        }
      }
      if (!ok && lane == 0) { *abort_flag = 1; atomicExch(g.status, 5); }
    }
  } else {
    // ------------------------------------------------------------------ epilogue warps (2..17)
    // Sixteen warps in four column groups: a warp may only touch the TMEM lane quarter given by warp % 4, so four
    // consecutive warps cover the 128 rows of a tile and every group of four drains block_n / n_groups columns.
    // Four warps per scheduler hide the latency of tcgen05.ld and of the conversion chain; tiles whose width is
    // not a multiple of 64 use fewer groups.
    const int quarter = warp & 3;
    const int group = (warp - 2) >> 2;
    const int n_groups = g.n_groups;
    const int cpg = g.block_n / n_groups;                  // columns per group, a multiple of 16, at most 64
    const int col_begin = group * cpg;
    const bool group_active = group < n_groups;
    const int row_in_tile = quarter * 32 + lane;
    const int epi_threads = n_groups * 128;
    const bool leader = (warp == 2 && lane == 0);
    const bool is_fp16 = GEN ? (g.is_fp16 != 0) : false;
    const bool has_bias = GEN ? (g.bias != nullptr) : ((EPI & EPI_BIAS) != 0);
    const int act = GEN ? g.act : ((EPI & EPI_RELU) ? 1 : (EPI & EPI_GELU) ? 2 : 0);
    const bool has_res = GEN ? (g.residual != nullptr) : ((EPI & EPI_RES) != 0);
    const bool has_mask = GEN ? (g.relu_mask != nullptr) : ((EPI & EPI_MASK) != 0);
    const bool has_scale = GEN ? (g.out_scale != 1.f) : ((EPI & EPI_SCALE) != 0);
    const bool may_drop = GEN ? true : ((EPI & EPI_DROP) != 0);
    const uint32_t thresh = (may_drop && g.dropout_p > 0.f) ? (uint32_t)(g.dropout_p * 4294967296.0) : 0u;
    const float keep_scale = thresh ? 1.f / (1.f - g.dropout_p) : 1.f;
    // operand fetched ahead of the arithmetic: the residual, else the ReLU mask
    const bool pre_is_res = has_res;
    const bool pre_any = has_res || has_mask;
    const unsigned short* pre_base = static_cast<const unsigned short*>(pre_is_res ? g.residual : g.relu_mask);
    const long long pre_ld = pre_is_res ? g.ldr : g.ldm;
    // With TMA stores the warp's block of the residual (else: mask) tile goes global -> staging buffer with 16-byte
    // asynchronous copies, lanes running along rows so that a request covers whole lines, and lands at the swizzled
    // place where the result will be written; only this warp reads or writes that block.  The copy is issued before
    // the wait for the accumulator (one whole tile earlier when there are three buffers).
    const bool staged = pre_any && g.tma_store;
    const bool ahead = staged && g.out_bufs == 3;
    // address of the 16-byte chunk holding columns [ct, ct + 8) of tile row `r` in a staging buffer.  64-column panels
    // use the 128-byte swizzle of the TMA store (chunk c of row r at c ^ (r & 7)); panels as wide as one destination's
    // column slice (fused all-to-all with slices that are not multiples of 64) are plain row-major.
    const int pw = g.panel_w;
    auto chunk_ptr = [&](uint8_t* buf, int r, int ct) -> uint8_t* {
      if (pw == 64) return buf + (size_t)(ct >> 6) * (BLOCK_M * 128) + (size_t)r * 128 + ((((ct & 63) >> 3) ^ (r & 7)) << 4);
      const int pn = ct / pw;
      return buf + (size_t)pn * (BLOCK_M * pw * 2) + (size_t)r * (pw * 2) + (size_t)(ct - pn * pw) * 2;
    };
    auto stage_operand = [&](int tile, uint8_t* buf) {
      const int mt = tile / g.n_chunks, nc = tile % g.n_chunks;
      const int L = cpg >> 3;                                     // 16-byte chunks per row of the block
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (j < L) {
          const int q = j * 32 + lane;
          const int rr = quarter * 32 + q / L, cc = q % L;
          const long long grow = (long long)mt * BLOCK_M + rr;
          if (grow < g.M) {
            const int ct = col_begin + cc * 8;
            cp_async_16(chunk_ptr(buf, rr, ct), pre_base + grow * pre_ld + nc * g.block_n + ct);
          }
        }
      }
    };
    // this thread's four possible 16-column slots inside a staging buffer (fixed for the whole kernel)
    uint32_t soff0[4], soff1[4];
#pragma unroll
    for (int it = 0; it < 4; ++it) {
      const int ct = col_begin + it * 16;
      const bool in_tile = group_active && it * 16 < cpg && g.tma_store;
      soff0[it] = in_tile ? (uint32_t)(chunk_ptr(smem_out, row_in_tile, ct) - smem_out) : 0u;
      soff1[it] = in_tile ? (uint32_t)(chunk_ptr(smem_out, row_in_tile, ct + 8) - smem_out) : 0u;
    }
    uint32_t acc = 0, acc_phase = 0;
    int out_sel = 0;
    bool ok = true;
    if (ahead && group_active && (int)blockIdx.x < total_tiles) {
      stage_operand(blockIdx.x, smem_out);
      cp_async_commit();
    }
    for (int t = blockIdx.x; t < total_tiles && ok && group_active; t += gridDim.x) {
      const int m_tile = t / g.n_chunks, n_chunk = t % g.n_chunks;
      const long long row = (long long)m_tile * BLOCK_M + row_in_tile;
      const bool row_ok = row < g.M;
      const int gcol_begin = n_chunk * g.block_n + col_begin;   // first global column of this thread's slice
      if (g.tma_store && g.out_bufs == 1) {
        // single staging buffer: its previous bulk store must have been read before it is overwritten
        if (leader) tma_store_wait_read<0>();
        epilogue_bar_sync(epi_threads);
      }
      uint8_t* stage_out = smem_out + (size_t)out_sel * out_buf_bytes;
      if (ahead) {
        // three staging buffers: the next tile's operand is fetched now (its buffer's last store drained before the
        // barrier that ended the previous tile), this tile's was fetched one tile ago
        const int tn = t + gridDim.x;
        if (tn < total_tiles) stage_operand(tn, smem_out + (size_t)((out_sel + 1) % 3) * out_buf_bytes);
        cp_async_commit();
      } else if (staged) {
        stage_operand(t, stage_out);
        cp_async_commit();
      }
      // mask words of this thread's (row, 16-column chunks): fetched before the wait for the accumulator
      unsigned bits_pre[4] = {0u, 0u, 0u, 0u};
      if (g.bits_in != nullptr && row_ok) {
#pragma unroll
        for (int it = 0; it < 4; ++it)
          if (it * 16 < cpg) bits_pre[it] = __ldg(g.bits_in + (long long)((gcol_begin >> 4) + it) * g.ldmb + row);
      }
      if (!mbar_wait(&ctl->tmem_full[acc], acc_phase, abort_flag)) { ok = false; break; }
      tc_fence_after();
      if (staged) {
        if (ahead) cp_async_wait_group<1>(); else cp_async_wait_group<0>();
        __syncwarp();
      }
      const uint32_t taddr = tmem_base + acc * (uint32_t)g.block_n + ((uint32_t)(quarter * 32) << 16) + (uint32_t)col_begin;
#pragma unroll
      for (int it = 0; it < 4; ++it) {
        const int c0 = it * 16;                                 // column inside the group's slice
        if (c0 >= cpg) break;
        uint32_t r[16];
        tmem_ld_32x32b_x16(taddr + (uint32_t)c0, r);
        const int col0 = gcol_begin + c0;
        // where this thread's 16 results go in the staging buffer (and where a staged residual / mask waits)
        uint4* slot0 = reinterpret_cast<uint4*>(stage_out + soff0[it]);
        uint4* slot1 = reinterpret_cast<uint4*>(stage_out + soff1[it]);
        uint4 pre0 = make_uint4(0, 0, 0, 0), pre1 = pre0;
        if (pre_any && row_ok) {
          if (staged) { pre0 = *slot0; pre1 = *slot1; }
          else {
            const uint4* pp = reinterpret_cast<const uint4*>(pre_base + row * pre_ld + col0);
            pre0 = __ldg(pp); pre1 = __ldg(pp + 1);
          }
        }
        tmem_ld_wait();
        if (it * 16 + 16 >= cpg) {
          // last read of this accumulator by the warp: hand it back to the MMA issuer before the arithmetic
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&ctl->tmem_empty[acc]);
        }
        if (!row_ok && !g.tma_store) continue;
        float v[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
        if (has_scale) {
#pragma unroll
          for (int i = 0; i < 16; ++i) v[i] *= g.out_scale;
        }
        if (has_bias) {
          const float4* bp = reinterpret_cast<const float4*>((g.bias_in_smem ? s_bias : g.bias) + col0);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float4 b4 = g.bias_in_smem ? bp[i] : __ldg(bp + i);
            v[4 * i] += b4.x; v[4 * i + 1] += b4.y; v[4 * i + 2] += b4.z; v[4 * i + 3] += b4.w;
          }
        }
        if (act == 1) {
#pragma unroll
          for (int i = 0; i < 16; ++i) v[i] = fmaxf(v[i], 0.f);
        } else if (act == 2) {
#pragma unroll
          for (int i = 0; i < 16; ++i) v[i] = gelu_erf(v[i]);
        }
        if (thresh) {
#pragma unroll
          for (int i = 0; i < 16; ++i)
            v[i] = keep_elem(g.dropout_seed, (uint32_t)row, (uint32_t)(col0 + i), thresh) ? v[i] * keep_scale : 0.f;
        }
        if (g.bits_in != nullptr && row_ok) {
          const unsigned bits = bits_pre[it];          // [N/16, M] layout: a warp's 32 rows read adjacent words
#pragma unroll
          for (int i = 0; i < 16; ++i) v[i] = ((bits >> i) & 1u) ? v[i] : 0.f;
        }
        if (g.bits_out != nullptr && row_ok) {
          unsigned bits = 0;
#pragma unroll
          for (int i = 0; i < 16; ++i) bits |= (v[i] > 0.f ? 1u : 0u) << i;
          g.bits_out[(long long)(col0 >> 4) * g.ldmb + row] = (unsigned short)bits;
        }
        if (has_mask && row_ok) {
          uint4 m0, m1;
          if (!pre_is_res) { m0 = pre0; m1 = pre1; }
          else {
            const uint4* mp = reinterpret_cast<const uint4*>(static_cast<const unsigned short*>(g.relu_mask) + row * g.ldm + col0);
            m0 = __ldg(mp); m1 = __ldg(mp + 1);
          }
          const unsigned short* ms0 = reinterpret_cast<const unsigned short*>(&m0);
          const unsigned short* ms1 = reinterpret_cast<const unsigned short*>(&m1);
          if (GEN && g.mask_mode == 1) {
            // GELU backward: the mask operand is the pre-activation z, the result is scaled by gelu'(z)
            const uint32_t z0[4] = {m0.x, m0.y, m0.z, m0.w}, z1[4] = {m1.x, m1.y, m1.z, m1.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              v[2 * i] *= gelu_erf_grad(lo16_as_float(z0[i], is_fp16));
              v[2 * i + 1] *= gelu_erf_grad(hi16_as_float(z0[i], is_fp16));
              v[8 + 2 * i] *= gelu_erf_grad(lo16_as_float(z1[i], is_fp16));
              v[8 + 2 * i + 1] *= gelu_erf_grad(hi16_as_float(z1[i], is_fp16));
            }
          } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              // positive in either 16-bit float format: sign bit clear and magnitude non-zero
              if (!((ms0[i] & 0x8000u) == 0 && (ms0[i] & 0x7FFFu) != 0)) v[i] = 0.f;
              if (!((ms1[i] & 0x8000u) == 0 && (ms1[i] & 0x7FFFu) != 0)) v[8 + i] = 0.f;
            }
          }
        }
        if (has_res && row_ok) {
          const uint4 q0 = pre0, q1 = pre1;
          const uint32_t w0[4] = {q0.x, q0.y, q0.z, q0.w}, w1[4] = {q1.x, q1.y, q1.z, q1.w};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            v[2 * i] += lo16_as_float(w0[i], is_fp16);     v[2 * i + 1] += hi16_as_float(w0[i], is_fp16);
            v[8 + 2 * i] += lo16_as_float(w1[i], is_fp16); v[8 + 2 * i + 1] += hi16_as_float(w1[i], is_fp16);
          }
        }
        if (g.out_fp32) {
          const int dest = g.n_dest > 1 ? col0 / g.cols_per_dest : 0;
          const int dcol = g.n_dest > 1 ? col0 - dest * g.cols_per_dest : col0;
          float4* op = reinterpret_cast<float4*>(static_cast<float*>(g.dst[dest]) + (g.dst_row_offset + row) * g.ldc + dcol);
#pragma unroll
          for (int i = 0; i < 4; ++i) op[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
          continue;
        }
        uint4 o0, o1;
        o0.x = pack2(v[0], v[1], is_fp16); o0.y = pack2(v[2], v[3], is_fp16);
        o0.z = pack2(v[4], v[5], is_fp16); o0.w = pack2(v[6], v[7], is_fp16);
        o1.x = pack2(v[8], v[9], is_fp16); o1.y = pack2(v[10], v[11], is_fp16);
        o1.z = pack2(v[12], v[13], is_fp16); o1.w = pack2(v[14], v[15], is_fp16);
        if (g.tma_store) {
                *slot0 = o0;
          *slot1 = o1;
        } else {
          // route the 16 columns: they never straddle a destination because cols_per_dest % 16 == 0
          const int dest = g.n_dest > 1 ? col0 / g.cols_per_dest : 0;
          const int dcol = g.n_dest > 1 ? col0 - dest * g.cols_per_dest : col0;
          uint4* op = reinterpret_cast<uint4*>(static_cast<unsigned short*>(g.dst[dest]) + (g.dst_row_offset + row) * g.ldc + dcol);
          op[0] = o0;
          op[1] = o1;
        }
      }
      if (g.tma_store) {
        fence_async_smem();                                  // generic-proxy writes -> visible to the bulk copy engine
        // with several staging buffers the store issued one tile ago must have drained before the barrier lets a
        // later tile write (or prefetch) there; it was issued a whole tile earlier, so this rarely waits
        if (leader && g.out_bufs >= 2) tma_store_wait_read<0>();
        epilogue_bar_sync(epi_threads);
        if (leader) {
          const int tile_col0 = n_chunk * g.block_n;
          const int y = (int)(g.dst_row_offset + (long long)m_tile * BLOCK_M);
          for (int pnl = 0; pnl < g.block_n / pw; ++pnl) {
            const int gc = tile_col0 + pnl * pw;
            const int dest = g.n_dest > 1 ? gc / g.cols_per_dest : 0;
            const int dcol = g.n_dest > 1 ? gc - dest * g.cols_per_dest : gc;
            tma_store_2d(&omaps.m[dest], stage_out + (size_t)pnl * (BLOCK_M * pw * 2), dcol, y);
          }
          tma_store_commit();
        }
        if (g.out_bufs >= 2) out_sel = (out_sel + 1 == g.out_bufs) ? 0 : out_sel + 1;
      }
      if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
    }
    if (!ok) cp_async_wait_all();                            // staged copies of the abandoned tile
    if (g.tma_store && leader) tma_store_wait_all();
    if (!ok && lane == 0) { *abort_flag = 1; atomicExch(g.status, 3); }
  }

  // ------------------------------------------------------------------ teardown
  __syncwarp();
  if (*abort_flag) {
    // give copies that are still in flight time to land before shared memory is released
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
  }
}

// ---------------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------------

int pick_block_n(int n, int cap) {
  const int cands[] = {256, 192, 128, 96, 64, 48, 32, 16};
  for (int c : cands)
    if (c <= cap && n % c == 0) return c;
  return 0;
}

}  // namespace

extern "C" int bf_gemm_supported(int M, int N, int K) {
  // K only has to keep rows 16-byte aligned: the tensor maps zero-fill the tail of the last 64-element panel, and a
  // matrix narrower than one panel (K = 16 or 32: the small output layers and their input gradients) is a single
  // panel that is mostly zero-fill
  return (M > 0 && K >= 16 && K % 8 == 0 && N >= 16 && pick_block_n(N, 256) > 0) ? 1 : 0;
}

extern "C" int bf_gemm_tn(const bf_gemm_params* p, cudaStream_t st) {
  const bool gathered = p->n_src > 1;
  if (gathered) {
    if (p->n_src > BF_MAX_PEERS || p->cols_per_src <= 0 || p->cols_per_src % 8 != 0 || p->K % UMMA_K != 0 ||
        p->K != p->n_src * p->cols_per_src || (p->src_ld * 2) % 16 != 0 || p->src_row_offset < 0)
      return (int)cudaErrorInvalidValue;
    for (int i = 0; i < p->n_src; ++i)
      if (p->src[i] == nullptr || ((uintptr_t)p->src[i]) % 16 != 0) return (int)cudaErrorInvalidValue;
    if (p->a_copy && (((uintptr_t)p->a_copy) % 16 != 0 || (p->ld_copy * 2) % 16 != 0 || p->ld_copy < p->K))
      return (int)cudaErrorInvalidValue;
  } else if (p->a_copy) {
    return (int)cudaErrorInvalidValue;
  }
  if (!bf_gemm_supported(p->M, p->N, p->K)) return (int)cudaErrorInvalidValue;
  if (p->n_dest < 1 || p->n_dest > BF_MAX_PEERS || p->N % p->n_dest != 0) return (int)cudaErrorInvalidValue;
  const int cols_per_dest = p->N / p->n_dest;
  if (p->n_dest > 1 && cols_per_dest % 16 != 0) return (int)cudaErrorInvalidValue;
  if ((p->ldb * 2) % 16 != 0 || ((uintptr_t)p->B) % 16 != 0) return (int)cudaErrorInvalidValue;
  if (!gathered && ((p->lda * 2) % 16 != 0 || ((uintptr_t)p->A) % 16 != 0)) return (int)cudaErrorInvalidValue;
  GemmArgs g;
  g.M = p->M; g.N = p->N; g.K = p->K;
  // a residual / mask tile is staged in the output buffers: 128-wide tiles leave room for three of them
  const bool wants_staging = (p->residual != nullptr || p->relu_mask != nullptr) && !p->out_fp32;
  g.block_n = pick_block_n(p->N, 256);
  // 256-wide tiles leave room for a single output staging buffer (the epilogue then waits for every bulk store to
  // drain).  With short K, two 128-wide chunks per row tile (two buffers, four-deep operand ring) are faster
  // (0.47 -> 0.40 ms at M = 2.9 M, K = 128); with K = 256 re-reading the A tile per chunk costs more than it saves.
  if (g.block_n == 256 && p->K <= 128 && !p->out_fp32) g.block_n = 128;
  if (wants_staging) {
    const int capped = pick_block_n(p->N, 128);
    if (capped > 0 && capped % 64 == 0) g.block_n = capped;
  }
  // a gathered operand crosses NVLink: one column chunk per row tile whenever the output is at most 256 wide, so that
  // no A tile is fetched twice
  if (gathered) g.block_n = pick_block_n(p->N, 256);
  g.n_chunks = p->N / g.block_n;
  g.m_tiles = (p->M + BLOCK_M - 1) / BLOCK_M;
  g.is_fp16 = p->dtype == BF_FP16 ? 1 : 0;
  g.bias = p->bias; g.act = p->act; g.dropout_p = p->dropout_p; g.dropout_seed = p->dropout_seed;
  g.residual = p->residual; g.ldr = p->ldr; g.relu_mask = p->relu_mask; g.ldm = p->ldm;
  g.mask_mode = (p->relu_mask != nullptr && p->mask_mode == 1) ? 1 : 0;
  g.bits_out = static_cast<unsigned short*>(p->relu_bits_out); g.bits_in = static_cast<const unsigned short*>(p->relu_bits_in);
  g.ldmb = p->ldmb;
  if ((g.bits_out || g.bits_in) && p->N % 16 != 0) return (int)cudaErrorInvalidValue;
  g.out_scale = p->out_scale == 0.f ? 1.f : p->out_scale;
  g.out_fp32 = p->out_fp32;
  g.n_dest = p->n_dest; g.cols_per_dest = cols_per_dest; g.dst_row_offset = p->dst_row_offset; g.ldc = p->ldc;
  for (int i = 0; i < BF_MAX_PEERS; ++i) g.dst[i] = i < p->n_dest ? p->dst[i] : nullptr;
  g.status = p->status;
  g.n_src = gathered ? p->n_src : 1;
  g.cols_per_src = gathered ? p->cols_per_src : p->K;
  g.src_row_offset = gathered ? p->src_row_offset : 0;
  g.a_copy = (gathered && p->a_copy) ? 1 : 0;
  CUtensorMap map_a, map_b;
  CUtensorMap map_copy;
  memset(&map_copy, 0, sizeof(map_copy));
  memset(&map_a, 0, sizeof(map_a));
  g.src_ld = gathered ? p->src_ld : 0;
  for (int i = 0; i < BF_MAX_PEERS; ++i) g.src[i] = (gathered && i < p->n_src) ? p->src[i] : nullptr;
  if (gathered) {
    // 64-column boxes with the 128-byte swizzle of the operand stage; rows past M and columns past K are clipped
    if (g.a_copy && make_map(&map_copy, p->a_copy, p->M, p->K, p->ld_copy, BLOCK_M, g.is_fp16) != 0)
      return (int)cudaErrorNotSupported;
  } else if (make_map(&map_a, p->A, p->M, p->K, p->lda, BLOCK_M, g.is_fp16) != 0) {
    return (int)cudaErrorNotSupported;
  }
  if (make_map(&map_b, p->B, p->N, p->K, p->ldb, g.block_n, g.is_fp16) != 0) return (int)cudaErrorNotSupported;
  // ---- shared-memory plan -------------------------------------------------------------------------
  const size_t stage_bytes = (size_t)BLOCK_M * BLOCK_K * 2 + (size_t)g.block_n * BLOCK_K * 2;
  const size_t out_bytes = (size_t)g.block_n * 256;                       // block_n/64 panels of 128 rows x 128 bytes
  g.bias_in_smem = (p->bias != nullptr && p->N <= 1024) ? 1 : 0;
  const size_t bias_bytes = g.bias_in_smem ? (size_t)p->N * 4 + 16 : 0;
  const size_t budget = 227 * 1024 - 1024 /*alignment slack*/ - sizeof(Control) - 64 - bias_bytes;
  // staged output panels: 64 columns (swizzled) when every destination's slice is a multiple of 64 columns, else one
  // panel per destination slice (e.g. 48 columns of q|k|v per rank with 8 ranks): a slice of a row tile is then one
  // contiguous bulk store into the peer's buffer instead of 128 separate 32-byte stores
  g.panel_w = 64;
  bool slice_panels = false;
  if (p->n_dest > 1 && cols_per_dest % 64 != 0) {
    slice_panels = cols_per_dest % 16 == 0 && cols_per_dest <= 256 && g.block_n % cols_per_dest == 0;
    if (slice_panels) g.panel_w = cols_per_dest;
  }
  bool tma_ok = !p->out_fp32 && g.block_n % 64 == 0 && (p->n_dest == 1 || cols_per_dest % 64 == 0 || slice_panels) &&
                (p->ldc * 2) % 16 == 0;
  for (int i = 0; i < p->n_dest && tma_ok; ++i) tma_ok = ((uintptr_t)p->dst[i]) % 16 == 0;
  g.tma_store = 0; g.out_bufs = 0; g.stages = MAX_STAGES;
  if (tma_ok) {
    const int plans[6][2] = {{4, 3}, {3, 3}, {4, 2}, {3, 2}, {4, 1}, {3, 1}};
    for (const auto& pl : plans) {
      if (pl[1] == 3 && !wants_staging) continue;
      if (pl[0] * stage_bytes + pl[1] * out_bytes <= budget) { g.stages = pl[0]; g.out_bufs = pl[1]; g.tma_store = 1; break; }
    }
  }
  OutMaps omaps;
  memset(&omaps, 0, sizeof(omaps));
  if (g.tma_store) {
    for (int d = 0; d < p->n_dest; ++d) {
      // rows beyond this call's region are out of range for the map, so the tail of the last row tile is clipped
      if (make_map(&omaps.m[d], p->dst[d], p->dst_row_offset + p->M, cols_per_dest, p->ldc, BLOCK_M, g.is_fp16, g.panel_w) != 0) {
        g.tma_store = 0; g.out_bufs = 0; g.stages = MAX_STAGES;
        break;
      }
    }
  }
  const size_t smem = 1024 + g.stages * stage_bytes + (size_t)g.out_bufs * out_bytes + sizeof(Control) + 64 + bias_bytes;
  g.n_groups = (g.block_n % 64 == 0) ? 4 : (g.block_n % 32 == 0) ? 2 : 1;
  // epilogue specialisation: the combinations the model layers use on bf16; everything else takes the generic kernel
  int epi = -1;
  if (!g.is_fp16 && !p->out_fp32) {
    int f = 0;
    if (p->bias) f |= EPI_BIAS;
    if (p->act == 1) f |= EPI_RELU;
    if (p->act == 2) f |= EPI_GELU;
    if (p->dropout_p > 0.f) f |= EPI_DROP;
    if (p->residual) f |= EPI_RES;
    if (p->relu_mask) f |= EPI_MASK;
    if (g.out_scale != 1.f) f |= EPI_SCALE;
    if (f == 0 || f == EPI_BIAS) epi = f;
    else if ((f | EPI_DROP) == (EPI_BIAS | EPI_DROP | EPI_RES)) epi = EPI_BIAS | EPI_DROP | EPI_RES;
    else if ((f | EPI_DROP) == (EPI_BIAS | EPI_RELU | EPI_DROP)) epi = EPI_BIAS | EPI_RELU | EPI_DROP;
    else if ((f | EPI_SCALE) == (EPI_MASK | EPI_SCALE)) epi = EPI_MASK | EPI_SCALE;
    else if (f == EPI_SCALE) epi = EPI_SCALE;
    if (g.mask_mode == 1) epi = -1;                 // the GELU-gradient mask lives in the generic kernel only
  }
  using Kern = void (*)(const CUtensorMap, const CUtensorMap, const OutMaps, const CUtensorMap, const GemmArgs);
  Kern kern = gemm_tn_tcgen05_kernel<-1, false>;
  if (gathered) {
    // gathered operand: the output projection's epilogue is specialised, the input-gradient GEMM takes the generic one
    if (epi != (EPI_BIAS | EPI_DROP | EPI_RES)) epi = -1;
    kern = epi < 0 ? (Kern)gemm_tn_tcgen05_kernel<-1, true> : (Kern)gemm_tn_tcgen05_kernel<EPI_BIAS | EPI_DROP | EPI_RES, true>;
  } else {
    switch (epi) {
      case 0: kern = gemm_tn_tcgen05_kernel<0, false>; break;
      case EPI_BIAS: kern = gemm_tn_tcgen05_kernel<EPI_BIAS, false>; break;
      case EPI_BIAS | EPI_DROP | EPI_RES: kern = gemm_tn_tcgen05_kernel<EPI_BIAS | EPI_DROP | EPI_RES, false>; break;
      case EPI_BIAS | EPI_RELU | EPI_DROP: kern = gemm_tn_tcgen05_kernel<EPI_BIAS | EPI_RELU | EPI_DROP, false>; break;
      case EPI_MASK | EPI_SCALE: kern = gemm_tn_tcgen05_kernel<EPI_MASK | EPI_SCALE, false>; break;
      case EPI_SCALE: kern = gemm_tn_tcgen05_kernel<EPI_SCALE, false>; break;
      default: break;
    }
  }
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  {
    // the attribute belongs to (function, device): remember it per device, not per process
    constexpr int MAX_DEV = 64;
    static bool attr_set[MAX_DEV][10] = {};
    const int slot = gathered ? (epi < 0 ? 8 : 9)
                     : epi < 0 ? 0 : epi == 0 ? 1 : epi == EPI_BIAS ? 2 : epi == (EPI_BIAS | EPI_DROP | EPI_RES) ? 3
                     : epi == (EPI_BIAS | EPI_RELU | EPI_DROP) ? 4 : epi == EPI_SCALE ? 6 : 5;
    if (dev < 0 || dev >= MAX_DEV || !attr_set[dev][slot]) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
      if (e != cudaSuccess) return (int)e;
      if (dev >= 0 && dev < MAX_DEV) attr_set[dev][slot] = true;
    }
  }
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int total = g.m_tiles * g.n_chunks;
  const int grid = total < sms ? total : sms;
  kern<<<grid, gathered ? NUM_THREADS_PULL : NUM_THREADS, smem, st>>>(map_a, map_b, omaps, map_copy, g);
  return (int)cudaGetLastError();
}
