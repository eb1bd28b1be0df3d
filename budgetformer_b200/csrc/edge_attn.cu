// Budgeted sparse edge attention for sm_100a: forward, dQ pass (over queries) and dK/dV pass
// (over the transposed graph).  Gather-only on regular rows: every query owns <= B sampled
// in-edges, so one lane group streams them with 16-byte loads and keeps the running
// numerator / normaliser in registers.  Rows longer than BF_HUB_DEGREE (the Graphormer virtual
// node, popular keys in the transposed graph) are split into chunks whose partial sums meet in
// an fp32 scratch buffer through atomics and are finalised by a second small kernel.
//
// Math (reference: models/graphormer_dist_node_level.py:231-263, models/gt_dist_node_level.py:
// 224-262, models/graphgps_dist_node_level.py:151-177, models/exphormer_dist_node_level.py:92-121):
//   s = clamp(<q_i,k_j>/sqrt(hn) [*E_type], -5, 5);  w = exp(s);  Z_i = sum w
//   plain/exphormer: out_i = sum w v_j / (Z_i + 1e-6)
//   gps:             out_i = sum (w/(Z_i+1e-6)) * keep/(1-p) * v_j
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include "bf_kernels.h"

namespace {

constexpr float kEps = 1e-6f;
constexpr float kClamp = 5.0f;

template <typename T> struct Vec;
template <> struct Vec<__nv_bfloat16> { static constexpr int N = 8; };
template <> struct Vec<__half> { static constexpr int N = 8; };
template <> struct Vec<float> { static constexpr int N = 4; };

template <typename T> __device__ __forceinline__ void load_vec(const T* p, float* f);
template <> __device__ __forceinline__ void load_vec<__nv_bfloat16>(const __nv_bfloat16* p, float* f) {
  uint4 u = __ldg(reinterpret_cast<const uint4*>(p));
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) { float2 t = __bfloat1622float2(h[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
}
template <> __device__ __forceinline__ void load_vec<__half>(const __half* p, float* f) {
  uint4 u = __ldg(reinterpret_cast<const uint4*>(p));
  const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) { float2 t = __half22float2(h[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
}
template <> __device__ __forceinline__ void load_vec<float>(const float* p, float* f) {
  float4 u = __ldg(reinterpret_cast<const float4*>(p));
  f[0] = u.x; f[1] = u.y; f[2] = u.z; f[3] = u.w;
}
template <typename T> __device__ __forceinline__ void store_vec(T* p, const float* f);
template <> __device__ __forceinline__ void store_vec<__nv_bfloat16>(__nv_bfloat16* p, const float* f) {
  uint4 u; __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  *reinterpret_cast<uint4*>(p) = u;
}
template <> __device__ __forceinline__ void store_vec<__half>(__half* p, const float* f) {
  uint4 u; __half2* h = reinterpret_cast<__half2*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
  *reinterpret_cast<uint4*>(p) = u;
}
template <> __device__ __forceinline__ void store_vec<float>(float* p, const float* f) {
  *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
}

// A gathered row slice kept packed (one 16-byte register quad) and widened element by element where it is used:
// the dQ pass holds several gathered slices at once, and packed they cost half the registers (four resident
// blocks per SM instead of three).
template <typename T> struct Raw;
template <> struct Raw<__nv_bfloat16> {
  uint4 u;
  __device__ __forceinline__ void load(const __nv_bfloat16* p) { u = *reinterpret_cast<const uint4*>(p); }
  __device__ __forceinline__ float get(int i) const {
    const uint32_t w = (i >> 1) == 0 ? u.x : (i >> 1) == 1 ? u.y : (i >> 1) == 2 ? u.z : u.w;
    return (i & 1) ? __uint_as_float(w & 0xFFFF0000u) : __uint_as_float(w << 16);
  }
};
template <> struct Raw<__half> {
  uint4 u;
  __device__ __forceinline__ void load(const __half* p) { u = *reinterpret_cast<const uint4*>(p); }
  __device__ __forceinline__ float get(int i) const {
    const uint32_t w = (i >> 1) == 0 ? u.x : (i >> 1) == 1 ? u.y : (i >> 1) == 2 ? u.z : u.w;
    return __half2float(__ushort_as_half((unsigned short)((i & 1) ? (w >> 16) : (w & 0xFFFFu))));
  }
};
template <> struct Raw<float> {
  float4 f;
  __device__ __forceinline__ void load(const float* p) { f = *reinterpret_cast<const float4*>(p); }
  __device__ __forceinline__ float get(int i) const { return i == 0 ? f.x : i == 1 ? f.y : i == 2 ? f.z : f.w; }
};

template <typename T> __device__ __forceinline__ T from_float(float x);
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }
template <> __device__ __forceinline__ __half from_float<__half>(float x) { return __float2half_rn(x); }
template <> __device__ __forceinline__ float from_float<float>(float x) { return x; }

__device__ __forceinline__ bool keep_edge(uint32_t seed, uint32_t eid, uint32_t head, uint32_t thresh) {
  uint32_t x = eid * 0x9E3779B1u + head * 0x85EBCA77u + seed;
  x = (x ^ (x >> 16)) * 0x7FEB352Du;
  x = (x ^ (x >> 15)) * 0x846CA68Bu;
  x ^= x >> 16;
  return x >= thresh;
}

template <int HN> __host__ __device__ constexpr float inv_sqrt_hn() {
  return HN == 8 ? 0.35355339059327373f : HN == 16 ? 0.25f : HN == 32 ? 0.17677669529663687f
       : HN == 64 ? 0.125f : 0.08838834764831845f;
}

// Lane-group geometry: LPH lanes cover one head (HN elements, 16 bytes per lane); a task is one
// (row, head chunk) handled by TL = LPH*HPT lanes, 32/TL tasks per warp.
struct Geo {
  int lph, hpt, tl, n_hc;
};
template <typename T, int HN> __host__ __device__ inline Geo make_geo(int hl) {
  Geo g;
  g.lph = HN / Vec<T>::N;
  int cap = 32 / g.lph;
  int hpt = 1;
  while (hpt * 2 <= cap && hpt * 2 <= hl) hpt *= 2;
  g.hpt = hpt;
  g.tl = g.lph * hpt;
  g.n_hc = (hl + hpt - 1) / hpt;
  return g;
}

// Sum over the LPH lanes of one head.  The mask names only those lanes: they always share
// control flow (same row, same head), so no wider convergence is needed.
template <int LPH> __device__ __forceinline__ unsigned head_mask() {
  const unsigned lane = threadIdx.x & 31u;
  return LPH >= 32 ? 0xffffffffu : (((1u << LPH) - 1u) << (lane & ~(unsigned)(LPH - 1)));
}
template <int LPH> __device__ __forceinline__ float head_sum(float x, unsigned m) {
#pragma unroll
  for (int o = LPH / 2; o > 0; o >>= 1) x += __shfl_xor_sync(m, x, o);
  return x;
}

// Routed rows: the result row of query / key `row` belongs to the rank that owns that node (row / rows_per) and is
// stored straight into that rank's buffer - the heads->nodes all-to-all of sequence parallelism done by the stores of
// the kernel that produces the rows.  Every destination holds one slab of `rows_per` rows per source rank
// ([n_dest * rows_per, ld] elements); `slab_row0` = this rank's slab.  n_dest == 0: off.
struct Route {
  unsigned long long base[BF_MAX_PEERS];   // buffer base address on every destination (peer mappings)
  int n_dest;
  int rows_per;
  long long ld;                            // row stride of the destination buffers (elements)
  long long slab_row0;                     // source rank * rows_per
};

template <typename T>
__device__ __forceinline__ T* routed(const Route& r, long long row, int col) {
  const int d = (int)(row / r.rows_per);
  const long long lr = row - (long long)d * r.rows_per + r.slab_row0;
  return reinterpret_cast<T*>(r.base[d]) + lr * r.ld + col;
}

struct AttnArgs {
  const void *q, *k, *v;       // [n, Hl, HN] with row strides ldq/ldk/ldv (elements)
  long long ldq, ldk, ldv;
  void* out;                   // [n, Hl, HN] contiguous
  float* z;                    // [n, Hl]
  const int* rowptr;           // [n+1]
  const int* col;              // [E]
  const uint8_t* etype;        // [E] or null
  const float* etab;           // [T, Hl, HN] fp32 or null
  int n, hl;
  int variant;                 // 0 plain, 1 gps, 2 exphormer
  float inv_keep;              // 1/(1-p)
  uint32_t thresh, seed;
  // hub path
  const int* hub_rows;         // [n_hub]
  int n_hub, hub_chunk;
  float* hub_scratch;          // forward: [n_hub, Hl*HN + Hl]
  // fused dropout on the stored output (out_thresh == 0: off)
  uint32_t out_thresh, out_seed;
  float out_inv_keep, out_keep;
  int out_rows_local, out_col0;
  Route route_out;             // second copy of every output row, delivered to the row's owner (n_dest == 0: none)
};

// keep decision of ops.gemm.hash_keep_mask / bf_hash_dropout for element (row, col)
__device__ __forceinline__ bool keep_out(const AttnArgs& a, int row, int c) {
  const uint32_t r = (uint32_t)(a.out_rows_local > 0 ? row % a.out_rows_local : row);
  uint32_t x = r * 0x9E3779B1u + (uint32_t)(a.out_col0 + c) * 0x85EBCA77u + a.out_seed;
  x = (x ^ (x >> 16)) * 0x7FEB352Du;
  x = (x ^ (x >> 15)) * 0x846CA68Bu;
  x ^= x >> 16;
  return x >= a.out_thresh;
}

// Two edges of one query for one task lane (second one optional).
template <typename T, int HN>
__device__ __forceinline__ void fwd_pair(const AttnArgs& a, int head, int off, int e0, int e1, bool has1, unsigned hm,
                                         const float* qs0, const float* qs1, float* acc, float& zsum) {
  constexpr int VN = Vec<T>::N;
  constexpr int LPH = HN / VN;
  const T* kp = static_cast<const T*>(a.k);
  const T* vp = static_cast<const T*>(a.v);
  const int j0 = __ldg(a.col + e0);
  const int j1 = has1 ? __ldg(a.col + e1) : j0;
  float k0[VN], v0[VN], k1[VN], v1[VN];
  load_vec<T>(kp + (long long)j0 * a.ldk + off, k0);
  load_vec<T>(kp + (long long)j1 * a.ldk + off, k1);
  load_vec<T>(vp + (long long)j0 * a.ldv + off, v0);
  load_vec<T>(vp + (long long)j1 * a.ldv + off, v1);
  int t0 = 0, t1 = 0;
  if (a.variant == 2) { t0 = a.etype[e0]; t1 = has1 ? a.etype[e1] : 0; }
  float d0 = 0.f, d1 = 0.f;
#pragma unroll
  for (int i = 0; i < VN; ++i) { d0 += (t0 ? qs1[i] : qs0[i]) * k0[i]; d1 += (t1 ? qs1[i] : qs0[i]) * k1[i]; }
  d0 = head_sum<LPH>(d0, hm);
  d1 = head_sum<LPH>(d1, hm);
  float w0 = __expf(fminf(fmaxf(d0, -kClamp), kClamp));
  float w1 = has1 ? __expf(fminf(fmaxf(d1, -kClamp), kClamp)) : 0.f;
  zsum += w0 + w1;
  if (a.variant == 1 && a.thresh) {
    if (!keep_edge(a.seed, (uint32_t)e0, (uint32_t)head, a.thresh)) w0 = 0.f;
    if (has1 && !keep_edge(a.seed, (uint32_t)e1, (uint32_t)head, a.thresh)) w1 = 0.f;
  }
#pragma unroll
  for (int i = 0; i < VN; ++i) acc[i] += w0 * v0[i] + w1 * v1[i];
}

template <typename T, int HN>
__device__ __forceinline__ void load_q_scaled(const AttnArgs& a, int row, int head, int off, float* qs0, float* qs1) {
  constexpr int VN = Vec<T>::N;
  const float scale = inv_sqrt_hn<HN>();
  float qf[VN];
  load_vec<T>(static_cast<const T*>(a.q) + (long long)row * a.ldq + off, qf);
#pragma unroll
  for (int i = 0; i < VN; ++i) { qs0[i] = qf[i] * scale; qs1[i] = qs0[i]; }
  if (a.variant == 2) {
    const int hlhn = a.hl * HN;
#pragma unroll
    for (int i = 0; i < VN; ++i) {
      qs0[i] = qf[i] * scale * a.etab[off + i];
      qs1[i] = qf[i] * scale * a.etab[hlhn + off + i];
    }
  }
}

template <typename T, int HN>
__global__ void __launch_bounds__(256) edge_attn_fwd_kernel(AttnArgs a) {
  constexpr int VN = Vec<T>::N;
  constexpr int LPH = HN / VN;
  const Geo g = make_geo<T, HN>(a.hl);
  const int lane = threadIdx.x & 31;
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int tpw = 32 / g.tl;
  const long long task = (long long)warp * tpw + lane / g.tl;
  const int lt = lane % g.tl;
  const long long n_task = (long long)a.n * g.n_hc;
  const bool live = task < n_task;
  const int row = live ? (int)(task / g.n_hc) : 0;
  const int hc = live ? (int)(task % g.n_hc) : 0;
  const int head = hc * g.hpt + lt / LPH;
  const bool head_ok = live && head < a.hl;
  const int hsafe = head_ok ? head : 0;
  const int off = hsafe * HN + (lt % LPH) * VN;
  int beg = 0, end = 0;
  if (head_ok) { beg = a.rowptr[row]; end = a.rowptr[row + 1]; }
  // long rows go to the hub kernels when the caller listed them; without a list they are walked here (slow, complete)
  const bool hub = a.n_hub > 0 && (end - beg) > BF_HUB_DEGREE;
  if (hub) end = beg;
  float qs0[VN], qs1[VN], acc[VN];
  float zsum = 0.f;
#pragma unroll
  for (int i = 0; i < VN; ++i) acc[i] = 0.f;
  load_q_scaled<T, HN>(a, row, hsafe, off, qs0, qs1);
  const unsigned hm = head_mask<LPH>();
  for (int e = beg; e < end; e += 2) fwd_pair<T, HN>(a, hsafe, off, e, e + 1, e + 1 < end, hm, qs0, qs1, acc, zsum);
  if (head_ok && !hub) {
    float inv = 1.f / (zsum + kEps);
    if (a.variant == 1) inv *= a.inv_keep;
    float o[VN];
#pragma unroll
    for (int i = 0; i < VN; ++i) o[i] = acc[i] * inv;
    if (a.out_thresh) {
#pragma unroll
      for (int i = 0; i < VN; ++i) o[i] = keep_out(a, row, off + i) ? o[i] * a.out_inv_keep : 0.f;
    }
    store_vec<T>(static_cast<T*>(a.out) + (long long)row * a.hl * HN + off, o);
    if (a.route_out.n_dest) store_vec<T>(routed<T>(a.route_out, row, off), o);
    if ((lt % LPH) == 0) a.z[(long long)row * a.hl + head] = zsum;
  }
}

// Hub rows: grid = (n_hub * chunks_per_hub) blocks; each warp strides over its block's chunk.
template <typename T, int HN>
__global__ void __launch_bounds__(256) edge_attn_fwd_hub_kernel(AttnArgs a, int chunks_per_hub) {
  constexpr int VN = Vec<T>::N;
  constexpr int LPH = HN / VN;
  const Geo g = make_geo<T, HN>(a.hl);
  const int hub_i = blockIdx.x / chunks_per_hub;
  const int row = a.hub_rows[hub_i];
  const int rbeg = a.rowptr[row], rend = a.rowptr[row + 1];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  const int tpw = 32 / g.tl;
  const int lt = lane % g.tl;
  const int sub_task = lane / g.tl;            // parallel edge streams inside the warp
  const int streams = nwarp * tpw;
  const int stream = warp * tpw + sub_task;
  float* scratch = a.hub_scratch + (long long)hub_i * (a.hl * HN + a.hl);
  // a block walks the row's chunks with stride chunks_per_hub: a row longer than the caller's bound costs parallelism,
  // never edges
  for (int chunk = blockIdx.x % chunks_per_hub; (long long)chunk * a.hub_chunk < rend - rbeg; chunk += chunks_per_hub) {
  const int cbeg = rbeg + chunk * a.hub_chunk;
  const int cend = min(rend, cbeg + a.hub_chunk);
  for (int hc = 0; hc < g.n_hc; ++hc) {
    const int head = hc * g.hpt + lt / LPH;
    const bool head_ok = head < a.hl;
    const int hsafe = head_ok ? head : 0;
    const int off = hsafe * HN + (lt % LPH) * VN;
    float qs0[VN], qs1[VN], acc[VN];
    float zsum = 0.f;
#pragma unroll
    for (int i = 0; i < VN; ++i) acc[i] = 0.f;
    load_q_scaled<T, HN>(a, row, hsafe, off, qs0, qs1);
    const unsigned hm = head_mask<LPH>();
    if (head_ok)
      for (int e = cbeg + stream; e < cend; e += 2 * streams)
        fwd_pair<T, HN>(a, hsafe, off, e, e + streams, e + streams < cend, hm, qs0, qs1, acc, zsum);
    if (head_ok) {
#pragma unroll
      for (int i = 0; i < VN; ++i) atomicAdd(scratch + off + i, acc[i]);
      if ((lt % LPH) == 0) atomicAdd(scratch + a.hl * HN + head, zsum);
    }
  }
  }
}

template <typename T, int HN>
__global__ void edge_attn_fwd_hub_finalize(AttnArgs a) {
  const int hub_i = blockIdx.x;
  const int row = a.hub_rows[hub_i];
  const int w = a.hl * HN;
  const float* scratch = a.hub_scratch + (long long)hub_i * (w + a.hl);
  for (int c = threadIdx.x; c < w; c += blockDim.x) {
    const int head = c / HN;
    const float zs = scratch[w + head];
    float inv = 1.f / (zs + kEps);
    if (a.variant == 1) inv *= a.inv_keep;
    float ov = scratch[c] * inv;
    if (a.out_thresh) ov = keep_out(a, row, c) ? ov * a.out_inv_keep : 0.f;
    static_cast<T*>(a.out)[(long long)row * w + c] = from_float<T>(ov);
    if (a.route_out.n_dest) *routed<T>(a.route_out, row, c) = from_float<T>(ov);
    if ((c % HN) == 0) a.z[(long long)row * a.hl + head] = zs;
  }
}

// ---------------------------------------------------------------------------------------------
// Backward
// ---------------------------------------------------------------------------------------------
struct BwdArgs {
  AttnArgs f;
  const void* dout;            // [n, Hl, HN] contiguous
  void *dq, *dk, *dv;          // [n, Hl, HN], row stride ldg (elements)
  long long ldg;
  float2* zd;                  // [n, Hl]: (1/(Z+eps), D = <dout,out>)
  const int *t_rowptr, *t_row, *t_eid;
  float* detab;                // [T, Hl, HN] fp32 or null
  const int* t_hub_rows;
  int n_t_hub;
  float* hub_scratch_q;        // [n_hub, Hl*HN]
  float* hub_scratch_kv;       // [n_t_hub, 2*Hl*HN]
  // balanced dK/dV work list
  const int4* kv_task;         // [n_kv_task]: key row, first edge, end edge, partial slot (-1 = direct store)
  int n_kv_task;
  const int* kv_split;         // [n_kv_split, 3]: key row, first slot, number of slots
  int n_kv_split;
  float* kv_partial;           // [slots, 2*Hl*HN] fp32
  // Packed query records for narrow rows (optional): the dQ pass writes, per (row, head), [q | dout / (Z + eps)] next to
  // each other plus one float D / (Z + eps); the dK/dV pass then gathers one contiguous record per edge instead of
  // three separate short rows (q, dout, (1/Z, D)), which matters when a row of q is only 32 or 64 bytes.
  void* qg;                    // [n, Hl, 2, HN] in the operand dtype, or null
  float* cz;                   // [n, Hl]
  // Routed gradients (route.n_dest > 0): dq / dk / dv rows go to the owner of the row instead of the local buffers, at
  // column offsets cq / ck / cv of the destination's packed row
  Route route;
  int cq, ck, cv;
};

// first element of gradient row `row`: in the local buffer, or in the row owner's slab when the gradients are routed
template <typename T>
__device__ __forceinline__ T* grad_row(const BwdArgs& b, void* local, int col0, long long row) {
  if (b.route.n_dest == 0) return static_cast<T*>(local) + row * b.ldg;
  return routed<T>(b.route, row, col0);
}

// One edge of the dQ pass for one task lane.
template <typename T, int HN>
__device__ __forceinline__ void dq_edge(const BwdArgs& b, int e, int head, int off, const float* qs0, const float* qs1,
                                        const float* qraw, const float* dof, float invz, float dterm, float* dq,
                                        float* de0, float* de1, unsigned hm) {
  constexpr int VN = Vec<T>::N;
  constexpr int LPH = HN / VN;
  const AttnArgs& a = b.f;
  const float scale = inv_sqrt_hn<HN>();
  const int j = __ldg(a.col + e);
  float kf[VN], vf[VN];
  load_vec<T>(static_cast<const T*>(a.k) + (long long)j * a.ldk + off, kf);
  load_vec<T>(static_cast<const T*>(a.v) + (long long)j * a.ldv + off, vf);
  const int t = (a.variant == 2) ? a.etype[e] : 0;
  float d = 0.f, dv = 0.f;
#pragma unroll
  for (int i = 0; i < VN; ++i) { d += (t ? qs1[i] : qs0[i]) * kf[i]; dv += dof[i] * vf[i]; }
  d = head_sum<LPH>(d, hm);
  dv = head_sum<LPH>(dv, hm);
  const bool inr = (d > -kClamp) && (d < kClamp);
  const float w = __expf(fminf(fmaxf(d, -kClamp), kClamp));
  float mf = 1.f;
  if (a.variant == 1 && a.thresh) mf = keep_edge(a.seed, (uint32_t)e, (uint32_t)head, a.thresh) ? a.inv_keep : 0.f;
  else if (a.variant == 1) mf = a.inv_keep;
  const float ds = inr ? (dv * mf - dterm) * invz * w : 0.f;
  if (a.variant == 2) {
    const float* et = a.etab + (t ? a.hl * HN : 0) + off;
#pragma unroll
    for (int i = 0; i < VN; ++i) {
      dq[i] += ds * scale * kf[i] * et[i];
      const float g = ds * scale * qraw[i] * kf[i];
      de0[i] += t ? 0.f : g;
      de1[i] += t ? g : 0.f;
    }
  } else {
#pragma unroll
    for (int i = 0; i < VN; ++i) dq[i] += ds * scale * kf[i];
  }
}

// Four edges of one query at a time (see dkv_edge4).
template <typename T, int HN, bool EXPH, int NB>
__device__ __forceinline__ void dq_edge4(const BwdArgs& b, int e, int end, int head, int off, const float* qs0,
                                         const float* qs1, const float* qraw, const float* dof, float invz, float dterm,
                                         float* dq, float* de0, float* de1, unsigned hm) {
  constexpr int VN = Vec<T>::N;
  constexpr int LPH = HN / VN;
  const AttnArgs& a = b.f;
  const float scale = inv_sqrt_hn<HN>();
  int j[NB], ty[NB];
  bool ok[NB];
#pragma unroll
  for (int u = 0; u < NB; ++u) {
    ok[u] = e + u < end;
    j[u] = ok[u] ? __ldg(a.col + e + u) : 0;
    ty[u] = (EXPH && ok[u]) ? a.etype[e + u] : 0;
  }
  if constexpr (!EXPH) {
    // gathered k | v slices stay packed until used (64 registers: four resident blocks per SM)
    Raw<T> kr[NB], vr[NB];
#pragma unroll
    for (int u = 0; u < NB; ++u) {
      kr[u].load(static_cast<const T*>(a.k) + (long long)j[u] * a.ldk + off);
      vr[u].load(static_cast<const T*>(a.v) + (long long)j[u] * a.ldv + off);
    }
#pragma unroll
    for (int u = 0; u < NB; ++u) {
      float d = 0.f, dv = 0.f;
#pragma unroll
      for (int i = 0; i < VN; ++i) { d += qs0[i] * kr[u].get(i); dv += dof[i] * vr[u].get(i); }
      d = head_sum<LPH>(d, hm);
      dv = head_sum<LPH>(dv, hm);
      const bool inr = (d > -kClamp) && (d < kClamp);
      const float w = ok[u] ? __expf(fminf(fmaxf(d, -kClamp), kClamp)) : 0.f;
      float mf = 1.f;
      if (a.variant == 1 && a.thresh) mf = keep_edge(a.seed, (uint32_t)(e + u), (uint32_t)head, a.thresh) ? a.inv_keep : 0.f;
      else if (a.variant == 1) mf = a.inv_keep;
      const float dss = inr ? (dv * mf - dterm) * invz * w * scale : 0.f;
#pragma unroll
      for (int i = 0; i < VN; ++i) dq[i] += dss * kr[u].get(i);
    }
  } else {
    float kf[NB][VN], vf[NB][VN];
#pragma unroll
    for (int u = 0; u < NB; ++u) {
      load_vec<T>(static_cast<const T*>(a.k) + (long long)j[u] * a.ldk + off, kf[u]);
      load_vec<T>(static_cast<const T*>(a.v) + (long long)j[u] * a.ldv + off, vf[u]);
    }
#pragma unroll
    for (int u = 0; u < NB; ++u) {
      float d = 0.f, dv = 0.f;
#pragma unroll
      for (int i = 0; i < VN; ++i) { d += (ty[u] ? qs1[i] : qs0[i]) * kf[u][i]; dv += dof[i] * vf[u][i]; }
      d = head_sum<LPH>(d, hm);
      dv = head_sum<LPH>(dv, hm);
      const bool inr = (d > -kClamp) && (d < kClamp);
      const float w = ok[u] ? __expf(fminf(fmaxf(d, -kClamp), kClamp)) : 0.f;
      float mf = 1.f;
      if (a.variant == 1 && a.thresh) mf = keep_edge(a.seed, (uint32_t)(e + u), (uint32_t)head, a.thresh) ? a.inv_keep : 0.f;
      else if (a.variant == 1) mf = a.inv_keep;
      const float ds = inr ? (dv * mf - dterm) * invz * w : 0.f;
      const float* et = a.etab + (ty[u] ? a.hl * HN : 0) + off;
#pragma unroll
      for (int i = 0; i < VN; ++i) {
        dq[i] += ds * scale * kf[u][i] * et[i];
        const float gg = ds * scale * qraw[i] * kf[u][i];
        de0[i] += ty[u] ? 0.f : gg;
        de1[i] += ty[u] ? gg : 0.f;
      }
    }
  }
}

template <typename T, int HN, bool EXPH>
__global__ void __launch_bounds__(256, EXPH ? 3 : 4) edge_attn_bwd_q_kernel(BwdArgs b) {
  constexpr int VN = Vec<T>::N;
  constexpr int LPH = HN / VN;
  const AttnArgs& a = b.f;
  extern __shared__ float s_detab[];   // [2, Hl*HN] when exphormer
  const int w_row = a.hl * HN;
  if (EXPH) {
    for (int i = threadIdx.x; i < 2 * w_row; i += blockDim.x) s_detab[i] = 0.f;
    __syncthreads();
  }
  const Geo g = make_geo<T, HN>(a.hl);
  const int lane = threadIdx.x & 31;
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int tpw = 32 / g.tl;
  const long long task = (long long)warp * tpw + lane / g.tl;
  const int lt = lane % g.tl;
  const long long n_task = (long long)a.n * g.n_hc;
  const bool live = task < n_task;
  const int row = live ? (int)(task / g.n_hc) : 0;
  const int hc = live ? (int)(task % g.n_hc) : 0;
  const int head = hc * g.hpt + lt / LPH;
  const bool head_ok = live && head < a.hl;
  const int hsafe = head_ok ? head : 0;
  const int off = hsafe * HN + (lt % LPH) * VN;
  int beg = 0, end = 0;
  if (head_ok) { beg = a.rowptr[row]; end = a.rowptr[row + 1]; }
  const bool hub = a.n_hub > 0 && (end - beg) > BF_HUB_DEGREE;
  float qs0[VN], qs1[VN], qraw[VN], dof[VN], of[VN], dq[VN], de0[VN], de1[VN];
  load_q_scaled<T, HN>(a, row, hsafe, off, qs0, qs1);
  load_vec<T>(static_cast<const T*>(a.q) + (long long)row * a.ldq + off, qraw);
  load_vec<T>(static_cast<const T*>(b.dout) + (long long)row * w_row + off, dof);
  load_vec<T>(static_cast<const T*>(a.out) + (long long)row * w_row + off, of);
  float dterm = 0.f;
#pragma unroll
  for (int i = 0; i < VN; ++i) { dterm += dof[i] * of[i]; dq[i] = 0.f; de0[i] = 0.f; de1[i] = 0.f; }
  const unsigned hm = head_mask<LPH>();
  dterm = head_sum<LPH>(dterm, hm);
  if (a.out_thresh) dterm *= a.out_keep;        // the stored output is the dropped one, rescaled by 1 / (1 - p)
  float zsum = head_ok ? a.z[(long long)row * a.hl + hsafe] : 1.f;
  const float invz = 1.f / (zsum + kEps);
  if (head_ok && (lt % LPH) == 0) b.zd[(long long)row * a.hl + head] = make_float2(invz, dterm);
  if (b.qg != nullptr && head_ok) {
    T* rec = static_cast<T*>(b.qg) + ((long long)row * a.hl + head) * 2 * HN + (lt % LPH) * VN;
    float gz[VN];
#pragma unroll
    for (int i = 0; i < VN; ++i) gz[i] = dof[i] * invz;
    store_vec<T>(rec, qraw);
    store_vec<T>(rec + HN, gz);
    if ((lt % LPH) == 0) b.cz[(long long)row * a.hl + head] = dterm * invz;
  }
  if (hub) end = beg;
  for (int e = beg; e < end; e += 2)
    dq_edge4<T, HN, EXPH, 2>(b, e, end, hsafe, off, qs0, qs1, qraw, dof, invz, dterm, dq, de0, de1, hm);
  if (head_ok && !hub) store_vec<T>(grad_row<T>(b, b.dq, b.cq, row) + off, dq);
  if (EXPH) {
    if (head_ok) {
#pragma unroll
      for (int i = 0; i < VN; ++i) {
        atomicAdd(&s_detab[off + i], de0[i]);
        atomicAdd(&s_detab[w_row + off + i], de1[i]);
      }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < 2 * w_row; i += blockDim.x)
      if (s_detab[i] != 0.f) atomicAdd(b.detab + i, s_detab[i]);
  }
}

template <typename T, int HN>
__global__ void __launch_bounds__(256) edge_attn_bwd_q_hub_kernel(BwdArgs b, int chunks_per_hub) {
  constexpr int VN = Vec<T>::N;
  constexpr int LPH = HN / VN;
  const AttnArgs& a = b.f;
  const Geo g = make_geo<T, HN>(a.hl);
  const int w_row = a.hl * HN;
  const int hub_i = blockIdx.x / chunks_per_hub;
  const int row = a.hub_rows[hub_i];
  const int rbeg = a.rowptr[row], rend = a.rowptr[row + 1];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  const int tpw = 32 / g.tl;
  const int lt = lane % g.tl;
  const int streams = nwarp * tpw;
  const int stream = warp * tpw + lane / g.tl;
  float* scratch = b.hub_scratch_q + (long long)hub_i * w_row;
  for (int chunk = blockIdx.x % chunks_per_hub; (long long)chunk * a.hub_chunk < rend - rbeg; chunk += chunks_per_hub) {
  const int cbeg = rbeg + chunk * a.hub_chunk;
  const int cend = min(rend, cbeg + a.hub_chunk);
  for (int hc = 0; hc < g.n_hc; ++hc) {
    const int head = hc * g.hpt + lt / LPH;
    const bool head_ok = head < a.hl;
    const int hsafe = head_ok ? head : 0;
    const int off = hsafe * HN + (lt % LPH) * VN;
    float qs0[VN], qs1[VN], qraw[VN], dof[VN], of[VN], dq[VN], de0[VN], de1[VN];
    load_q_scaled<T, HN>(a, row, hsafe, off, qs0, qs1);
    load_vec<T>(static_cast<const T*>(a.q) + (long long)row * a.ldq + off, qraw);
    load_vec<T>(static_cast<const T*>(b.dout) + (long long)row * w_row + off, dof);
    load_vec<T>(static_cast<const T*>(a.out) + (long long)row * w_row + off, of);
    float dterm = 0.f;
#pragma unroll
    for (int i = 0; i < VN; ++i) { dterm += dof[i] * of[i]; dq[i] = 0.f; de0[i] = 0.f; de1[i] = 0.f; }
    const unsigned hm = head_mask<LPH>();
    dterm = head_sum<LPH>(dterm, hm);
    if (a.out_thresh) dterm *= a.out_keep;
    const float invz = 1.f / (a.z[(long long)row * a.hl + hsafe] + kEps);
    if (head_ok)
      for (int e = cbeg + stream; e < cend; e += streams)
        dq_edge<T, HN>(b, e, hsafe, off, qs0, qs1, qraw, dof, invz, dterm, dq, de0, de1, hm);
    if (head_ok) {
#pragma unroll
      for (int i = 0; i < VN; ++i) atomicAdd(scratch + off + i, dq[i]);
      if (a.variant == 2) {
#pragma unroll
        for (int i = 0; i < VN; ++i) {
          atomicAdd(b.detab + off + i, de0[i]);
          atomicAdd(b.detab + w_row + off + i, de1[i]);
        }
      }
    }
  }
  }
}

// One transposed edge (key j fixed, query i varies) for one task lane.
template <typename T, int HN>
__device__ __forceinline__ void dkv_edge(const BwdArgs& b, int te, int head, int off, const float* kf, const float* vf,
                                         float* dk, float* dv, unsigned hm) {
  constexpr int VN = Vec<T>::N;
  constexpr int LPH = HN / VN;
  const AttnArgs& a = b.f;
  const float scale = inv_sqrt_hn<HN>();
  const int w_row = a.hl * HN;
  const int i_row = __ldg(b.t_row + te);
  const int eid = __ldg(b.t_eid + te);
  float qf[VN], dof[VN];
  load_vec<T>(static_cast<const T*>(a.q) + (long long)i_row * a.ldq + off, qf);
  load_vec<T>(static_cast<const T*>(b.dout) + (long long)i_row * w_row + off, dof);
  const float2 zd = __ldg(b.zd + (long long)i_row * a.hl + head);
  const int t = (a.variant == 2) ? a.etype[eid] : 0;
  float et[VN];
  if (a.variant == 2) {
#pragma unroll
    for (int i = 0; i < VN; ++i) et[i] = a.etab[(t ? w_row : 0) + off + i];
  } else {
#pragma unroll
    for (int i = 0; i < VN; ++i) et[i] = 1.f;
  }
  float d = 0.f, dotv = 0.f;
#pragma unroll
  for (int i = 0; i < VN; ++i) { d += qf[i] * kf[i] * et[i]; dotv += dof[i] * vf[i]; }
  d = head_sum<LPH>(d, hm) * scale;
  dotv = head_sum<LPH>(dotv, hm);
  const bool inr = (d > -kClamp) && (d < kClamp);
  const float w = __expf(fminf(fmaxf(d, -kClamp), kClamp));
  float mf = 1.f;
  if (a.variant == 1 && a.thresh) mf = keep_edge(a.seed, (uint32_t)eid, (uint32_t)head, a.thresh) ? a.inv_keep : 0.f;
  else if (a.variant == 1) mf = a.inv_keep;
  const float ds = inr ? (dotv * mf - zd.y) * zd.x * w : 0.f;
  const float wn = w * mf * zd.x;
#pragma unroll
  for (int i = 0; i < VN; ++i) {
    dk[i] += ds * scale * qf[i] * et[i];
    dv[i] += wn * dof[i];
  }
}

// Four transposed edges at a time: all index and row loads are issued before any arithmetic so that a lane group
// keeps 8 independent 16-byte gathers in flight (the pass is bound by gather latency, not by math).
template <typename T, int HN, bool EXPH, int NB, bool PACKED>
__device__ __forceinline__ void dkv_edge4(const BwdArgs& b, int te, int end, int head, int off, const Raw<T>& kf,
                                          const Raw<T>& vf, float* dk, float* dv, unsigned hm) {
  constexpr int VN = Vec<T>::N;
  constexpr int LPH = HN / VN;
  const AttnArgs& a = b.f;
  const float scale = inv_sqrt_hn<HN>();
  const int w_row = a.hl * HN;
  int i_row[NB], eid[NB];
  bool ok[NB];
#pragma unroll
  for (int u = 0; u < NB; ++u) {
    ok[u] = te + u < end;
    i_row[u] = ok[u] ? __ldg(b.t_row + te + u) : 0;
    eid[u] = ok[u] ? __ldg(b.t_eid + te + u) : 0;
  }
  Raw<T> qr[NB], dr[NB];                      // gathered slices stay packed until used
  float2 zd[NB];
  int ty[NB];
#pragma unroll
  for (int u = 0; u < NB; ++u) {
    if constexpr (PACKED) {
      // one contiguous record per (query, head): q, then dout already divided by the normaliser; zd = (1, D / (Z + eps))
      const T* rec = static_cast<const T*>(b.qg) + ((long long)i_row[u] * a.hl + head) * 2 * HN + (off - head * HN);
      qr[u].load(rec);
      dr[u].load(rec + HN);
      zd[u] = make_float2(1.f, __ldg(b.cz + (long long)i_row[u] * a.hl + head));
    } else {
      qr[u].load(static_cast<const T*>(a.q) + (long long)i_row[u] * a.ldq + off);
      dr[u].load(static_cast<const T*>(b.dout) + (long long)i_row[u] * w_row + off);
      zd[u] = __ldg(b.zd + (long long)i_row[u] * a.hl + head);
    }
    ty[u] = (EXPH && ok[u]) ? a.etype[eid[u]] : 0;
  }
#pragma unroll
  for (int u = 0; u < NB; ++u) {
    float et[VN];
#pragma unroll
    for (int i = 0; i < VN; ++i) et[i] = EXPH ? a.etab[(ty[u] ? w_row : 0) + off + i] : 1.f;
    float d = 0.f, dotv = 0.f;
#pragma unroll
    for (int i = 0; i < VN; ++i) { d += qr[u].get(i) * kf.get(i) * et[i]; dotv += dr[u].get(i) * vf.get(i); }
    d = head_sum<LPH>(d, hm) * scale;
    dotv = head_sum<LPH>(dotv, hm);
    const bool inr = (d > -kClamp) && (d < kClamp);
    const float w = ok[u] ? __expf(fminf(fmaxf(d, -kClamp), kClamp)) : 0.f;
    float mf = 1.f;
    if (a.variant == 1 && a.thresh) mf = keep_edge(a.seed, (uint32_t)eid[u], (uint32_t)head, a.thresh) ? a.inv_keep : 0.f;
    else if (a.variant == 1) mf = a.inv_keep;
    const float ds = inr ? (dotv * mf - zd[u].y) * zd[u].x * w : 0.f;
    const float wn = w * mf * zd[u].x;
#pragma unroll
    const float dss = ds * scale;
#pragma unroll
    for (int i = 0; i < VN; ++i) {
      dk[i] += dss * qr[u].get(i) * et[i];
      dv[i] += wn * dr[u].get(i);
    }
  }
}

// dK/dV over the balanced work list: one lane group per (work item, head chunk).  (Letting two lane groups share an
// item and split its edges was measured slower: most items are short, and the shared form halves the items in flight.)
template <typename T, int HN, bool EXPH, int MINB, bool PACKED>
__global__ void __launch_bounds__(256, MINB) edge_attn_bwd_kv_task_kernel(BwdArgs b) {
  constexpr int VN = Vec<T>::N;
  constexpr int LPH = HN / VN;
  const AttnArgs& a = b.f;
  const Geo g = make_geo<T, HN>(a.hl);
  const int w_row = a.hl * HN;
  const int lane = threadIdx.x & 31;
  const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int tpw = 32 / g.tl;
  const long long task = warp * tpw + lane / g.tl;
  const int lt = lane % g.tl;
  const long long n_task = (long long)b.n_kv_task * g.n_hc;
  const bool live = task < n_task;
  const int item = live ? (int)(task / g.n_hc) : 0;
  const int hc = live ? (int)(task % g.n_hc) : 0;
  const int head = hc * g.hpt + lt / LPH;
  const bool head_ok = live && head < a.hl;
  if (!head_ok) return;                       // whole head groups leave together; shuffles use head masks
  const int off = head * HN + (lt % LPH) * VN;
  const int4 it = __ldg(b.kv_task + item);
  const int row = it.x, beg = it.y, end = it.z, slot = it.w;
  Raw<T> kf, vf;                              // this key's k | v slice stays packed for the whole task
  float dk[VN], dv[VN];
  kf.load(static_cast<const T*>(a.k) + (long long)row * a.ldk + off);
  vf.load(static_cast<const T*>(a.v) + (long long)row * a.ldv + off);
#pragma unroll
  for (int i = 0; i < VN; ++i) { dk[i] = 0.f; dv[i] = 0.f; }
  const unsigned hm = head_mask<LPH>();
  for (int e = beg; e < end; e += 2) dkv_edge4<T, HN, EXPH, 2, PACKED>(b, e, end, head, off, kf, vf, dk, dv, hm);
  if (slot < 0) {
    store_vec<T>(grad_row<T>(b, b.dk, b.ck, row) + off, dk);
    store_vec<T>(grad_row<T>(b, b.dv, b.cv, row) + off, dv);
  } else {
    float* pp = b.kv_partial + (long long)slot * 2 * w_row;
#pragma unroll
    for (int i = 0; i < VN; ++i) { pp[off + i] = dk[i]; pp[w_row + off + i] = dv[i]; }
  }
}

// Adds the partials of every split key row (fixed association => bit-reproducible).  A hub key owns thousands of
// slots, so a block spreads them over G thread groups (slot j goes to group j % G), every thread keeps 16 independent
// sums in flight, and the groups' results meet in shared memory in group order.
constexpr int KV_REDUCE_THREADS = 1024;
template <typename T>
__global__ void __launch_bounds__(KV_REDUCE_THREADS) edge_attn_bwd_kv_reduce_kernel(BwdArgs b, int w_row) {
  extern __shared__ float s_part[];           // [G, 2 * w_row]
  const int s = blockIdx.x;
  const int row = b.kv_split[3 * s], first = b.kv_split[3 * s + 1], n = b.kv_split[3 * s + 2];
  const int ncol = 2 * w_row;
  const int G = ncol <= KV_REDUCE_THREADS ? KV_REDUCE_THREADS / ncol : 1;
  const int grp = ncol <= KV_REDUCE_THREADS ? (int)threadIdx.x / ncol : 0;
  for (int c0 = 0; c0 < ncol; c0 += KV_REDUCE_THREADS) {
    const int c = c0 + (ncol <= KV_REDUCE_THREADS ? (int)threadIdx.x % ncol : (int)threadIdx.x);
    const bool act = c < ncol && grp < G;
    float acc = 0.f;
    if (act) {
      float a16[16];
#pragma unroll
      for (int u = 0; u < 16; ++u) a16[u] = 0.f;
      const float* pp = b.kv_partial + (long long)first * ncol + c;
      int j = grp;
      for (; j + 15 * G < n; j += 16 * G) {
#pragma unroll
        for (int u = 0; u < 16; ++u) a16[u] += pp[(long long)(j + u * G) * ncol];
      }
      for (; j < n; j += G) a16[0] += pp[(long long)j * ncol];
#pragma unroll
      for (int w = 8; w > 0; w >>= 1) {
#pragma unroll
        for (int u = 0; u < w; ++u) a16[u] += a16[u + w];
      }
      acc = a16[0];
    }
    if (G > 1) {
      if (act) s_part[grp * ncol + c] = acc;
      __syncthreads();
      if (act && grp == 0) {
        for (int q = 1; q < G; ++q) acc += s_part[q * ncol + c];
      }
    }
    if (act && grp == 0) {
      T* dst = c < w_row ? grad_row<T>(b, b.dk, b.ck, row) : grad_row<T>(b, b.dv, b.cv, row);
      dst[c < w_row ? c : c - w_row] = from_float<T>(acc);
    }
    if (G > 1) __syncthreads();
  }
}

template <typename T, int HN>
__global__ void __launch_bounds__(256) edge_attn_bwd_kv_kernel(BwdArgs b) {
  constexpr int VN = Vec<T>::N;
  constexpr int LPH = HN / VN;
  const AttnArgs& a = b.f;
  const Geo g = make_geo<T, HN>(a.hl);
  const int w_row = a.hl * HN;
  const int lane = threadIdx.x & 31;
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int tpw = 32 / g.tl;
  const long long task = (long long)warp * tpw + lane / g.tl;
  const int lt = lane % g.tl;
  const long long n_task = (long long)a.n * g.n_hc;
  const bool live = task < n_task;
  const int row = live ? (int)(task / g.n_hc) : 0;
  const int hc = live ? (int)(task % g.n_hc) : 0;
  const int head = hc * g.hpt + lt / LPH;
  const bool head_ok = live && head < a.hl;
  const int hsafe = head_ok ? head : 0;
  const int off = hsafe * HN + (lt % LPH) * VN;
  int beg = 0, end = 0;
  if (head_ok) { beg = b.t_rowptr[row]; end = b.t_rowptr[row + 1]; }
  const bool hub = b.n_t_hub > 0 && (end - beg) > BF_HUB_DEGREE;
  if (hub) end = beg;
  float kf[VN], vf[VN], dk[VN], dv[VN];
  load_vec<T>(static_cast<const T*>(a.k) + (long long)row * a.ldk + off, kf);
  load_vec<T>(static_cast<const T*>(a.v) + (long long)row * a.ldv + off, vf);
#pragma unroll
  for (int i = 0; i < VN; ++i) { dk[i] = 0.f; dv[i] = 0.f; }
  const unsigned hm = head_mask<LPH>();
  for (int e = beg; e < end; ++e) dkv_edge<T, HN>(b, e, hsafe, off, kf, vf, dk, dv, hm);
  if (head_ok && !hub) {
    store_vec<T>(grad_row<T>(b, b.dk, b.ck, row) + off, dk);
    store_vec<T>(grad_row<T>(b, b.dv, b.cv, row) + off, dv);
  }
}

template <typename T, int HN>
__global__ void __launch_bounds__(256) edge_attn_bwd_kv_hub_kernel(BwdArgs b, int chunks_per_hub) {
  constexpr int VN = Vec<T>::N;
  constexpr int LPH = HN / VN;
  const AttnArgs& a = b.f;
  const Geo g = make_geo<T, HN>(a.hl);
  const int w_row = a.hl * HN;
  const int hub_i = blockIdx.x / chunks_per_hub;
  const int row = b.t_hub_rows[hub_i];
  const int rbeg = b.t_rowptr[row], rend = b.t_rowptr[row + 1];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  const int tpw = 32 / g.tl;
  const int lt = lane % g.tl;
  const int streams = nwarp * tpw;
  const int stream = warp * tpw + lane / g.tl;
  float* scratch = b.hub_scratch_kv + (long long)hub_i * 2 * w_row;
  for (int chunk = blockIdx.x % chunks_per_hub; (long long)chunk * a.hub_chunk < rend - rbeg; chunk += chunks_per_hub) {
  const int cbeg = rbeg + chunk * a.hub_chunk;
  const int cend = min(rend, cbeg + a.hub_chunk);
  for (int hc = 0; hc < g.n_hc; ++hc) {
    const int head = hc * g.hpt + lt / LPH;
    const bool head_ok = head < a.hl;
    const int hsafe = head_ok ? head : 0;
    const int off = hsafe * HN + (lt % LPH) * VN;
    float kf[VN], vf[VN], dk[VN], dv[VN];
    load_vec<T>(static_cast<const T*>(a.k) + (long long)row * a.ldk + off, kf);
    load_vec<T>(static_cast<const T*>(a.v) + (long long)row * a.ldv + off, vf);
#pragma unroll
    for (int i = 0; i < VN; ++i) { dk[i] = 0.f; dv[i] = 0.f; }
    const unsigned hm = head_mask<LPH>();
    if (head_ok)
      for (int e = cbeg + stream; e < cend; e += streams) dkv_edge<T, HN>(b, e, hsafe, off, kf, vf, dk, dv, hm);
    if (head_ok) {
#pragma unroll
      for (int i = 0; i < VN; ++i) {
        atomicAdd(scratch + off + i, dk[i]);
        atomicAdd(scratch + w_row + off + i, dv[i]);
      }
    }
  }
  }
}

template <typename T>
__global__ void hub_scatter_rows(const float* scratch, int scratch_ld, int scratch_off, const int* rows, BwdArgs b, void* local,
                                 int col0, int width) {
  const int hub_i = blockIdx.x;
  const int row = rows[hub_i];
  T* dst = grad_row<T>(b, local, col0, row);
  for (int c = threadIdx.x; c < width; c += blockDim.x)
    dst[c] = from_float<T>(scratch[(long long)hub_i * scratch_ld + scratch_off + c]);
}

template <typename T, int HN>
cudaError_t launch_fwd_t(const AttnArgs& a, int chunks_per_hub, cudaStream_t st) {
  const Geo g = make_geo<T, HN>(a.hl);
  const long long n_task = (long long)a.n * g.n_hc;
  const int tpw = 32 / g.tl;
  const long long warps = (n_task + tpw - 1) / tpw;
  const long long blocks = (warps + 7) / 8;
  if (blocks > 0) edge_attn_fwd_kernel<T, HN><<<(unsigned)blocks, 256, 0, st>>>(a);
  if (a.n_hub > 0) {
    edge_attn_fwd_hub_kernel<T, HN><<<a.n_hub * chunks_per_hub, 256, 0, st>>>(a, chunks_per_hub);
    edge_attn_fwd_hub_finalize<T, HN><<<a.n_hub, 256, 0, st>>>(a);
  }
  return cudaGetLastError();
}

template <typename T, int HN>
cudaError_t launch_bwd_t(const BwdArgs& b, int chunks_q, int chunks_kv, cudaStream_t st) {
  const AttnArgs& a = b.f;
  const Geo g = make_geo<T, HN>(a.hl);
  const long long n_task = (long long)a.n * g.n_hc;
  const int tpw = 32 / g.tl;
  const long long warps = (n_task + tpw - 1) / tpw;
  const long long blocks = (warps + 7) / 8;
  const int w_row = a.hl * HN;
  const size_t smem = a.variant == 2 ? sizeof(float) * 2 * w_row : 0;
  if (blocks > 0) {
    if (a.variant == 2) edge_attn_bwd_q_kernel<T, HN, true><<<(unsigned)blocks, 256, smem, st>>>(b);
    else edge_attn_bwd_q_kernel<T, HN, false><<<(unsigned)blocks, 256, smem, st>>>(b);
  }
  if (a.n_hub > 0) {
    edge_attn_bwd_q_hub_kernel<T, HN><<<a.n_hub * chunks_q, 256, 0, st>>>(b, chunks_q);
    hub_scatter_rows<T><<<a.n_hub, 256, 0, st>>>(b.hub_scratch_q, w_row, 0, a.hub_rows, b, b.dq, b.cq, w_row);
  }
  if (b.kv_task) {
    const long long kv_tasks = (long long)b.n_kv_task * g.n_hc;
    const long long kv_warps = (kv_tasks + tpw - 1) / tpw;
    const long long kv_blocks = (kv_warps + 7) / 8;
    if (kv_blocks > 0) {
      if (a.variant == 2) {
        if (b.qg) edge_attn_bwd_kv_task_kernel<T, HN, true, 3, true><<<(unsigned)kv_blocks, 256, 0, st>>>(b);
        else edge_attn_bwd_kv_task_kernel<T, HN, true, 3, false><<<(unsigned)kv_blocks, 256, 0, st>>>(b);
      } else {
        if (b.qg) edge_attn_bwd_kv_task_kernel<T, HN, false, 4, true><<<(unsigned)kv_blocks, 256, 0, st>>>(b);
        else edge_attn_bwd_kv_task_kernel<T, HN, false, 4, false><<<(unsigned)kv_blocks, 256, 0, st>>>(b);
      }
    }
    if (b.n_kv_split > 0) {
      const int ncol = 2 * w_row;
      const int G = ncol <= KV_REDUCE_THREADS ? KV_REDUCE_THREADS / ncol : 1;
      edge_attn_bwd_kv_reduce_kernel<T><<<b.n_kv_split, KV_REDUCE_THREADS, (size_t)G * ncol * sizeof(float), st>>>(b, w_row);
    }
    return cudaGetLastError();
  }
  if (blocks > 0) edge_attn_bwd_kv_kernel<T, HN><<<(unsigned)blocks, 256, 0, st>>>(b);
  if (b.n_t_hub > 0) {
    edge_attn_bwd_kv_hub_kernel<T, HN><<<b.n_t_hub * chunks_kv, 256, 0, st>>>(b, chunks_kv);
    hub_scatter_rows<T><<<b.n_t_hub, 256, 0, st>>>(b.hub_scratch_kv, 2 * w_row, 0, b.t_hub_rows, b, b.dk, b.ck, w_row);
    hub_scatter_rows<T><<<b.n_t_hub, 256, 0, st>>>(b.hub_scratch_kv, 2 * w_row, w_row, b.t_hub_rows, b, b.dv, b.cv, w_row);
  }
  return cudaGetLastError();
}

AttnArgs to_args(const bf_attn_params& p) {
  AttnArgs a;
  a.q = p.q; a.k = p.k; a.v = p.v; a.ldq = p.ldq; a.ldk = p.ldk; a.ldv = p.ldv;
  a.out = p.out; a.z = p.z; a.rowptr = p.rowptr; a.col = p.col; a.etype = p.etype; a.etab = p.etab;
  a.n = p.n; a.hl = p.hl; a.variant = p.variant;
  a.inv_keep = p.dropout_p > 0.f ? 1.f / (1.f - p.dropout_p) : 1.f;
  a.thresh = p.dropout_p > 0.f ? (uint32_t)(p.dropout_p * 4294967296.0) : 0u;
  a.seed = p.dropout_seed;
  a.out_thresh = p.out_dropout_p > 0.f ? (uint32_t)(p.out_dropout_p * 4294967296.0) : 0u;
  a.out_seed = p.out_dropout_seed;
  a.out_keep = 1.f - p.out_dropout_p;
  a.out_inv_keep = p.out_dropout_p > 0.f ? 1.f / (1.f - p.out_dropout_p) : 1.f;
  a.out_rows_local = p.out_rows_local; a.out_col0 = p.out_col0;
  a.hub_rows = p.hub_rows; a.n_hub = p.n_hub; a.hub_chunk = BF_HUB_CHUNK; a.hub_scratch = p.hub_scratch;
  memset(&a.route_out, 0, sizeof(a.route_out));
  return a;
}

// Validated copy of a caller's route for `n` rows of `width` elements each; false = reject the call.
bool to_route(const bf_attn_route* r, int n, long long width, Route* out) {
  memset(out, 0, sizeof(*out));
  if (r == nullptr || r->n_dest <= 0) return true;
  if (r->n_dest > BF_MAX_PEERS || r->rows_per <= 0 || (long long)r->rows_per * r->n_dest != n || r->ld < width || r->ld % 8 != 0 ||
      r->slab_row0 < 0 || r->slab_row0 + r->rows_per > (long long)r->rows_per * r->n_dest)
    return false;
  for (int i = 0; i < r->n_dest; ++i) {
    if (r->base[i] == nullptr || ((uintptr_t)r->base[i]) % 16 != 0) return false;
    out->base[i] = (unsigned long long)(uintptr_t)r->base[i];
  }
  out->n_dest = r->n_dest; out->rows_per = r->rows_per; out->ld = r->ld; out->slab_row0 = r->slab_row0;
  return true;
}

}  // namespace

#define BF_DISPATCH(DT, HN, CALL)                                                           \
  do {                                                                                      \
    if (DT == BF_BF16) {                                                                    \
      if (HN == 16) return CALL(__nv_bfloat16, 16); if (HN == 32) return CALL(__nv_bfloat16, 32); \
      if (HN == 64) return CALL(__nv_bfloat16, 64); if (HN == 8) return CALL(__nv_bfloat16, 8);   \
      if (HN == 128) return CALL(__nv_bfloat16, 128);                                       \
    } else if (DT == BF_FP16) {                                                             \
      if (HN == 16) return CALL(__half, 16); if (HN == 32) return CALL(__half, 32);         \
      if (HN == 64) return CALL(__half, 64); if (HN == 8) return CALL(__half, 8);           \
      if (HN == 128) return CALL(__half, 128);                                              \
    } else if (DT == BF_FP32) {                                                             \
      if (HN == 16) return CALL(float, 16); if (HN == 32) return CALL(float, 32);           \
      if (HN == 64) return CALL(float, 64); if (HN == 8) return CALL(float, 8);             \
      if (HN == 128) return CALL(float, 128);                                               \
    }                                                                                       \
  } while (0)

extern "C" int bf_edge_attn_fwd_routed(const bf_attn_params* p, const bf_attn_route* route, cudaStream_t st) {
  AttnArgs a = to_args(*p);
  if (!to_route(route, p->n, (long long)p->hl * p->hn, &a.route_out)) return (int)cudaErrorInvalidValue;
  const int chunks = p->max_hub_degree > 0 ? (p->max_hub_degree + BF_HUB_CHUNK - 1) / BF_HUB_CHUNK : 1;
#define CALL_FWD(T, H) (int)launch_fwd_t<T, H>(a, chunks, st)
  BF_DISPATCH(p->dtype, p->hn, CALL_FWD);
#undef CALL_FWD
  return (int)cudaErrorInvalidValue;
}

extern "C" int bf_edge_attn_fwd(const bf_attn_params* p, cudaStream_t st) {
  AttnArgs a = to_args(*p);
  const int chunks = p->max_hub_degree > 0 ? (p->max_hub_degree + BF_HUB_CHUNK - 1) / BF_HUB_CHUNK : 1;
#define CALL_FWD(T, H) (int)launch_fwd_t<T, H>(a, chunks, st)
  BF_DISPATCH(p->dtype, p->hn, CALL_FWD);
#undef CALL_FWD
  return (int)cudaErrorInvalidValue;
}

extern "C" int bf_edge_attn_bwd(const bf_attn_params* p, const bf_attn_bwd_params* q, cudaStream_t st) {
  BwdArgs b;
  b.f = to_args(*p);
  b.dout = q->dout; b.dq = q->dq; b.dk = q->dk; b.dv = q->dv;
  b.ldg = q->ldg > 0 ? q->ldg : (long long)p->hl * p->hn;
  b.zd = reinterpret_cast<float2*>(q->zd);
  b.t_rowptr = q->t_rowptr; b.t_row = q->t_row; b.t_eid = q->t_eid; b.detab = q->detab;
  b.t_hub_rows = q->t_hub_rows; b.n_t_hub = q->n_t_hub;
  b.hub_scratch_q = q->hub_scratch_q; b.hub_scratch_kv = q->hub_scratch_kv;
  b.kv_task = reinterpret_cast<const int4*>(q->kv_task); b.n_kv_task = q->n_kv_task;
  b.kv_split = q->kv_split; b.n_kv_split = q->n_kv_split; b.kv_partial = q->kv_partial;
  // the packed records serve the work-list form of the dK/dV pass only
  b.qg = (q->kv_task != nullptr && q->qg != nullptr && q->cz != nullptr) ? q->qg : nullptr;
  b.cz = b.qg ? q->cz : nullptr;
  b.cq = q->route_cq; b.ck = q->route_ck; b.cv = q->route_cv;
  {
    // a routed row is [.. ck: dk .. cv: dv .. cq: dq ..]: every part must fit the destination's row stride
    const long long w = (long long)p->hl * p->hn;
    const long long hi = (long long)(b.cq > b.ck ? (b.cq > b.cv ? b.cq : b.cv) : (b.ck > b.cv ? b.ck : b.cv)) + w;
    if (!to_route(&q->route, p->n, q->route.n_dest > 0 ? hi : w, &b.route)) return (int)cudaErrorInvalidValue;
    if (b.route.n_dest > 0 && (b.cq < 0 || b.ck < 0 || b.cv < 0 || ((b.cq | b.ck | b.cv) % 8) != 0))
      return (int)cudaErrorInvalidValue;
  }
  const int cq = p->max_hub_degree > 0 ? (p->max_hub_degree + BF_HUB_CHUNK - 1) / BF_HUB_CHUNK : 1;
  const int ckv = q->max_t_hub_degree > 0 ? (q->max_t_hub_degree + BF_HUB_CHUNK - 1) / BF_HUB_CHUNK : 1;
#define CALL_BWD(T, H) (int)launch_bwd_t<T, H>(b, cq, ckv, st)
  BF_DISPATCH(p->dtype, p->hn, CALL_BWD);
#undef CALL_BWD
  return (int)cudaErrorInvalidValue;
}

// ---------------------------------------------------------------------------------------------------
// Allocation-free variant of the forward entry point (declared and documented in bf_noalloc.h).
// ---------------------------------------------------------------------------------------------------
#include "bf_noalloc.h"

#include <mutex>

// Scratch of the long-row kernels for callers that cannot allocate.  In host code this name is only a handle for
// the runtime (it is not a device address); the address is resolved per device below.
static __device__ __align__(256) float g_bf_noalloc_scratch[BF_NOALLOC_SCRATCH_FLOATS];

namespace {
constexpr int kMaxDevices = 64;
float* g_noalloc_ptr[kMaxDevices] = {nullptr};
std::mutex g_noalloc_mutex;

// Device address of the scratch array on the current device (looked up once per device).
int noalloc_scratch_ptr(float** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) return BF_NOALLOC_ERR_SETUP;
  std::lock_guard<std::mutex> lock(g_noalloc_mutex);
  if (g_noalloc_ptr[dev] == nullptr) {
    float* ptr = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_bf_noalloc_scratch);
    if (e != cudaSuccess || ptr == nullptr) return BF_NOALLOC_ERR_SETUP;
    g_noalloc_ptr[dev] = ptr;
  }
  *out = g_noalloc_ptr[dev];
  return 0;
}
}  // namespace

extern "C" int bf_edge_attn_fwd_noalloc(const bf_attn_params* p, cudaStream_t stream) {
  if (p == nullptr) return (int)cudaErrorInvalidValue;
  const long long width = (long long)p->hl * p->hn;
  if (p->n_hub < 0 || p->n_hub > BF_NOALLOC_MAX_HUBS || width > BF_NOALLOC_MAX_WIDTH || p->hl > BF_NOALLOC_MAX_HEADS)
    return BF_NOALLOC_ERR_TOO_LARGE;
  // everything the launcher would reject is rejected here, before anything is queued on the stream
  const bool hn_ok = p->hn == 8 || p->hn == 16 || p->hn == 32 || p->hn == 64 || p->hn == 128;
  const bool dtype_ok = p->dtype == BF_BF16 || p->dtype == BF_FP16 || p->dtype == BF_FP32;
  if (!hn_ok || !dtype_ok || p->n <= 0 || p->hl <= 0) return (int)cudaErrorInvalidValue;
  if (p->n_hub > 0 && (p->hub_rows == nullptr || p->max_hub_degree <= 0)) return (int)cudaErrorInvalidValue;
  bf_attn_params q = *p;
  q.hub_scratch = nullptr;
  if (p->n_hub > 0) {
    float* scratch = nullptr;
    const int rc = noalloc_scratch_ptr(&scratch);
    if (rc != 0) return rc;
    // the array keeps the previous call's sums: clear the part this call accumulates into
    const size_t bytes = sizeof(float) * (size_t)p->n_hub * (size_t)(width + p->hl);
    const cudaError_t e = cudaMemsetAsync(scratch, 0, bytes, stream);
    if (e != cudaSuccess) return (int)e;
    q.hub_scratch = scratch;
  }
  return bf_edge_attn_fwd(&q, stream);
}

extern "C" size_t bf_attn_params_size(void) { return sizeof(bf_attn_params); }

extern "C" const char* bf_noalloc_strerror(int code) {
  switch (code) {
    case 0: return "success";
    case BF_NOALLOC_ERR_TOO_LARGE:
      return "bf_edge_attn_fwd_noalloc: problem exceeds the built-in scratch (n_hub <= 64, hl*hn <= 1024, hl <= 64)";
    case BF_NOALLOC_ERR_SETUP:
      return "bf_edge_attn_fwd_noalloc: could not resolve the device address of the built-in scratch array";
    default: return code > 0 ? cudaGetErrorString((cudaError_t)code) : "unknown error";
  }
}
