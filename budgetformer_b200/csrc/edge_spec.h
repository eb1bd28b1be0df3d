// Bit-exact specification shared by the CUDA builder (edge_build.cu) and the C++/OpenMP builder
// (cpu/edge_builder.cpp): the Philox-4x32-10 walk generator and the per-edge ranking hash.
// The numpy restatement used as the test oracle lives in graph/rng.py.
#pragma once
#include <stdint.h>

#if defined(__CUDACC__)
#define BF_HD __host__ __device__ __forceinline__
#else
#define BF_HD inline
#endif

#define BF_PHILOX_TAG 0x42554447u
#define BF_REAL_SEED_OFFSET 17
#define BF_RW_SEED_OFFSET 37
#define BF_MAX_SIDE_BUDGET 32   // per-side (real / random-walk) budget handled by the warp kernels
#define BF_MAX_WALK_LEN 16

BF_HD uint32_t bf_mulhi32(uint32_t a, uint32_t b) { return (uint32_t)(((uint64_t)a * (uint64_t)b) >> 32); }

// First output word of Philox-4x32-10 with counter (walk_lo, walk_hi, step, TAG), key (seed_lo, seed_hi).
BF_HD uint32_t bf_walk_uniform32(uint64_t walk_id, uint32_t step, uint64_t seed) {
  uint32_t c0 = (uint32_t)walk_id, c1 = (uint32_t)(walk_id >> 32), c2 = step, c3 = BF_PHILOX_TAG;
  uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint64_t p0 = (uint64_t)0xD2511F53u * c0;
    const uint64_t p1 = (uint64_t)0xCD9E8D57u * c2;
    const uint32_t hi0 = (uint32_t)(p0 >> 32), lo0 = (uint32_t)p0;
    const uint32_t hi1 = (uint32_t)(p1 >> 32), lo1 = (uint32_t)p1;
    const uint32_t n0 = hi1 ^ c1 ^ k0, n2 = hi0 ^ c3 ^ k1;
    c0 = n0; c1 = lo1; c2 = n2; c3 = lo0;
    k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
  }
  return c0;
}

// Ranking composite: (31-bit hash << 32) | src.  Hash as in the reference's per-query sampler
// (utils/fullgraph_sp_support.py:982-989), evaluated modulo 2^64 which is equivalent modulo 2^31.
BF_HD uint64_t bf_edge_composite(uint32_t src, uint32_t dst, int64_t seed) {
  const uint64_t c = (uint64_t)seed * 2654435761ull + 12345ull;
  const uint64_t k = (uint64_t)src * 1103515245ull + (uint64_t)dst * 214013ull + c;
  return ((k & 0x7FFFFFFFull) << 32) | (uint64_t)src;
}
