// Per-epoch attention-graph construction on the GPU: one warp per query node.
//   1. real edges: stream the query's in-edge row, keep the b_real smallest (hash, src) in a
//      lane-distributed sorted list (ballot + shuffle insertion; no global sort);
//   2. random walks: lane w runs walk w (Philox counter RNG, dead ends stay), the W*L candidates are
//      ranked into a second lane-distributed list of size b_rw;
//   3. merge: sorted unique union by key id (Exphormer: typed concatenation + self loop) written to a
//      fixed-width row [cap] plus a count; ell_to_csr compacts rows after a prefix sum.
// Replaces the reference's argsort / scatter_reduce rounds / coalesce pipeline
// (utils/fullgraph_sp_support.py:975-1192, gt_sp/utils.py:1198-1248, :877-887) and is bit-identical
// to cpu/edge_builder.cpp and graph/builder_spec.py.
#include <cuda_runtime.h>
#include <stdint.h>

#include "bf_kernels.h"
#include "edge_spec.h"

namespace {

constexpr uint64_t kInf = ~0ull;

// Lane groups: WIDTH lanes (8 or 32) cooperate on one query.  Every *_sync primitive names only the group's lanes,
// so groups of one warp may diverge from each other (different degrees, different insertion counts).
template <int WIDTH> __device__ __forceinline__ unsigned group_mask(int lane) {
  return WIDTH == 32 ? 0xffffffffu : (((1u << WIDTH) - 1u) << (lane & ~(WIDTH - 1)));
}
template <int WIDTH> __device__ __forceinline__ unsigned group_ballot(unsigned gm, int lane, bool pred) {
  const unsigned b = __ballot_sync(gm, pred);
  return WIDTH == 32 ? b : ((b >> (lane & ~(WIDTH - 1))) & ((1u << WIDTH) - 1u));
}

// Insert every candidate (valid, comp) held by the group's lanes into the sorted lane-distributed list
// (lane i of the group holds the i-th smallest composite; K <= WIDTH).
template <int WIDTH>
__device__ __forceinline__ void group_insert(uint64_t& list, int K, bool valid, uint64_t comp, int gl, unsigned gm, int lane) {
  const unsigned kmask = K >= 32 ? 0xffffffffu : ((1u << K) - 1u);
  for (int guard = 0; guard <= WIDTH; ++guard) {
    const uint64_t kth = __shfl_sync(gm, list, K - 1, WIDTH);
    const unsigned ball = group_ballot<WIDTH>(gm, lane, valid && comp < kth);
    if (ball == 0) break;
    const int src_lane = __ffs(ball) - 1;
    const uint64_t c = __shfl_sync(gm, comp, src_lane, WIDTH);
    const unsigned le = group_ballot<WIDTH>(gm, lane, list <= c) & kmask;
    const int p = __popc(le);
    const uint64_t up = __shfl_up_sync(gm, list, 1, WIDTH);
    if (gl == p) list = c;
    else if (gl > p && gl < K) list = up;
    if (gl == src_lane) valid = false;
  }
}

struct BuildArgs {
  const int *in_rowptr, *in_src, *out_rowptr, *out_col;
  int n;
  int row_begin;       // first query of this launch; rows are stored at index (query - row_begin)
  int b_real, b_rw, walks, walk_len, exphormer;
  long long seed;
  int cap;
  int* ell_col;        // [n, cap]
  uint8_t* ell_type;   // [n, cap] or null
  int* ell_cnt;        // [n]
  unsigned long long* totals;  // [2] selected real / rw edges (with multiplicity)
  const int* hub_rows;         // ascending ids of queries with more than BF_BUILD_HUB_DEGREE in-edges, or null
  int n_hub;
  unsigned long long* hub_top; // [n_hub, 32] ranked real candidates of those queries
};

// Real-edge ranking of the long rows: one block per listed query.  Each warp keeps the b_real smallest composites of
// its share of the row (chunks of 32 edges, strided by the block), warp 0 merges the eight lists.  The b_real smallest
// of a multiset do not depend on the order of insertion, so the result equals the single stream of the main kernel.
__global__ void __launch_bounds__(256) budget_hub_topk_kernel(BuildArgs a) {
  __shared__ uint64_t s_list[8][32];
  const int row = a.hub_rows[blockIdx.x];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const bool mine = row >= a.row_begin && (long long)row < (long long)a.row_begin + a.n;   // uniform over the block
  uint64_t list = kInf;
  if (mine) {
    const int beg = a.in_rowptr[row], end = a.in_rowptr[row + 1];
    const int64_t rs = a.seed + BF_REAL_SEED_OFFSET;
    for (long long base = (long long)beg + warp * 32; base < end; base += 256) {
      const long long e = base + lane;
      const bool valid = e < end;
      const uint32_t s = valid ? (uint32_t)__ldg(a.in_src + e) : 0u;
      group_insert<32>(list, a.b_real, valid, valid ? bf_edge_composite(s, (uint32_t)row, rs) : kInf, lane, 0xffffffffu, lane);
    }
  }
  s_list[warp][lane] = list;
  __syncthreads();
  if (warp == 0 && mine) {
    for (int w = 1; w < 8; ++w) {
      const uint64_t c = s_list[w][lane];
      group_insert<32>(list, a.b_real, c != kInf, c, lane, 0xffffffffu, lane);
    }
    a.hub_top[(long long)blockIdx.x * 32 + lane] = list;
  }
}

template <int WIDTH>
__global__ void __launch_bounds__(256) budget_select_kernel(BuildArgs a) {
  __shared__ unsigned s_tot[2];
  if (threadIdx.x < 2) s_tot[threadIdx.x] = 0;
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int gl = lane & (WIDTH - 1);                       // lane inside the group
  const unsigned gm = group_mask<WIDTH>(lane);
  const long long slot = ((long long)blockIdx.x * blockDim.x + threadIdx.x) / WIDTH;   // row of the output
  const long long v = slot + a.row_begin;                                              // query node
  if (slot < a.n) {
    const uint32_t q = (uint32_t)v;
    // ---- real edges ----
    uint64_t rlist = kInf;
    int r_cnt = 0;
    if (a.b_real > 0) {
      const int beg = a.in_rowptr[v], end = a.in_rowptr[v + 1];
      const int64_t rs = a.seed + BF_REAL_SEED_OFFSET;
      int hub = -1;
      if (a.n_hub > 0 && end - beg > BF_BUILD_HUB_DEGREE) {   // ranked by budget_hub_topk_kernel if the caller listed it
        int lo = 0, hi = a.n_hub - 1;
        while (lo < hi) {
          const int mid = (lo + hi) >> 1;
          if (a.hub_rows[mid] < (int)v) lo = mid + 1; else hi = mid;
        }
        if (a.hub_rows[lo] == (int)v) hub = lo;
      }
      if (hub >= 0) {
        rlist = gl < a.b_real ? (uint64_t)a.hub_top[(long long)hub * 32 + gl] : kInf;
      } else {
        for (int base = beg; base < end; base += WIDTH) {
          const int e = base + gl;
          const bool valid = e < end;
          const uint32_t s = valid ? (uint32_t)__ldg(a.in_src + e) : 0u;
          group_insert<WIDTH>(rlist, a.b_real, valid, valid ? bf_edge_composite(s, q, rs) : kInf, gl, gm, lane);
        }
      }
      r_cnt = min(end - beg, a.b_real);
    }
    // ---- random walks ----
    uint64_t wlist = kInf;
    int w_cnt = 0;
    if (a.b_rw > 0 && a.walks > 0 && a.walk_len > 0) {
      const int64_t ws = a.seed + BF_RW_SEED_OFFSET;
      int n_cand = 0;
      for (int wbase = 0; wbase < a.walks; wbase += WIDTH) {
        const int w = wbase + gl;
        const bool active = w < a.walks;
        const uint64_t walk_id = (uint64_t)v * (uint64_t)a.walks + (uint64_t)w;
        int cur = (int)v, prev = (int)v;
        for (int d = 1; d <= a.walk_len; ++d) {
          bool emit = false;
          if (active) {
            const int ob = a.out_rowptr[cur], oe = a.out_rowptr[cur + 1];
            const uint32_t deg = (uint32_t)(oe - ob);
            prev = cur;
            if (deg > 0) {
              const uint32_t r = bf_walk_uniform32(walk_id, (uint32_t)d, (uint64_t)a.seed);
              cur = __ldg(a.out_col + ob + (int)bf_mulhi32(r, deg));
            }
            emit = (d == 1) || (cur != prev);
          }
          n_cand += __popc(group_ballot<WIDTH>(gm, lane, emit));
          group_insert<WIDTH>(wlist, a.b_rw, emit, emit ? bf_edge_composite((uint32_t)cur, q, ws) : kInf, gl, gm, lane);
        }
      }
      w_cnt = min(n_cand, a.b_rw);
    }
    // ---- merge ----
    const bool has_r = gl < r_cnt, has_w = gl < w_cnt;
    const uint32_t sr = (uint32_t)rlist, sw = (uint32_t)wlist;
    int* row = a.ell_col + slot * a.cap;
    if (a.exphormer) {
      int rank_r = 0, rank_w = 0;
      for (int t = 0; t < WIDTH; ++t) {
        const uint32_t yr = __shfl_sync(gm, sr, t, WIDTH);
        const uint32_t yw = __shfl_sync(gm, sw, t, WIDTH);
        if (t < r_cnt && (yr < sr || (yr == sr && t < gl))) ++rank_r;
        if (t < w_cnt && (yw < sw || (yw == sw && t < gl))) ++rank_w;
      }
      uint8_t* trow = a.ell_type + slot * a.cap;
      if (has_r) { row[rank_r] = (int)sr; trow[rank_r] = 0; }
      if (has_w) { row[r_cnt + rank_w] = (int)sw; trow[r_cnt + rank_w] = 1; }
      if (gl == 0) { row[r_cnt + w_cnt] = (int)v; trow[r_cnt + w_cnt] = 0; a.ell_cnt[slot] = r_cnt + w_cnt + 1; }
    } else {
      bool dup_r = false, dup_w = false;
      for (int t = 0; t < WIDTH; ++t) {
        const uint32_t yr = __shfl_sync(gm, sr, t, WIDTH);
        const uint32_t yw = __shfl_sync(gm, sw, t, WIDTH);
        if (t < r_cnt && t < gl && yr == sr) dup_r = true;
        if (t < r_cnt && yr == sw) dup_w = true;
        if (t < w_cnt && t < gl && yw == sw) dup_w = true;
      }
      const bool keep_r = has_r && !dup_r, keep_w = has_w && !dup_w;
      int rank_r = 0, rank_w = 0;
      for (int t = 0; t < WIDTH; ++t) {
        const uint32_t yr = __shfl_sync(gm, sr, t, WIDTH);
        const uint32_t yw = __shfl_sync(gm, sw, t, WIDTH);
        const bool kr = __shfl_sync(gm, (int)keep_r, t, WIDTH) != 0;
        const bool kw = __shfl_sync(gm, (int)keep_w, t, WIDTH) != 0;
        if (kr && yr < sr) ++rank_r;
        if (kw && yw < sr) ++rank_r;
        if (kr && yr < sw) ++rank_w;
        if (kw && yw < sw) ++rank_w;
      }
      if (keep_r) row[rank_r] = (int)sr;
      if (keep_w) row[rank_w] = (int)sw;
      const int total = __popc(group_ballot<WIDTH>(gm, lane, keep_r)) + __popc(group_ballot<WIDTH>(gm, lane, keep_w));
      if (gl == 0) a.ell_cnt[slot] = total;
    }
    if (gl == 0) { atomicAdd(&s_tot[0], (unsigned)r_cnt); atomicAdd(&s_tot[1], (unsigned)w_cnt); }
  }
  __syncthreads();
  if (threadIdx.x < 2 && s_tot[threadIdx.x]) atomicAdd(a.totals + threadIdx.x, (unsigned long long)s_tot[threadIdx.x]);
}

__global__ void ell_to_csr_kernel(const int* ell_col, const uint8_t* ell_type, const int* rowptr, int n, int cap,
                                  int* col, uint8_t* etype) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)n * cap) return;
  const int row = (int)(i / cap), slot = (int)(i % cap);
  const int beg = rowptr[row], cnt = rowptr[row + 1] - beg;
  if (slot < cnt) {
    col[beg + slot] = ell_col[i];
    if (etype) etype[beg + slot] = ell_type[i];
  }
}

}  // namespace

extern "C" int bf_budget_select(const bf_build_params* p, cudaStream_t st) {
  if (p->b_real > BF_MAX_SIDE_BUDGET || p->b_rw > BF_MAX_SIDE_BUDGET || p->walk_len > BF_MAX_WALK_LEN)
    return (int)cudaErrorInvalidValue;
  BuildArgs a;
  a.in_rowptr = p->in_rowptr; a.in_src = p->in_src; a.out_rowptr = p->out_rowptr; a.out_col = p->out_col;
  a.n = p->row_count > 0 ? p->row_count : p->n; a.row_begin = p->row_count > 0 ? p->row_begin : 0;
  if (a.row_begin < 0 || (long long)a.row_begin + a.n > p->n) return (int)cudaErrorInvalidValue;
  a.b_real = p->b_real; a.b_rw = p->b_rw; a.walks = p->walks; a.walk_len = p->walk_len;
  a.exphormer = p->exphormer; a.seed = p->seed; a.cap = p->cap;
  a.ell_col = p->ell_col; a.ell_type = p->ell_type; a.ell_cnt = p->ell_cnt;
  a.totals = reinterpret_cast<unsigned long long*>(p->totals);
  // eight lanes per query when both budgets and the walk count fit in eight slots, else a full warp
  const bool narrow = p->b_real <= 8 && p->b_rw <= 8 && p->walks <= 8;
  const int width = narrow ? 8 : 32;
  const long long blocks = ((long long)a.n * width + 255) / 256;
  const bool hubs = p->hub_rows != nullptr && p->hub_top != nullptr && p->n_hub > 0 && p->b_real > 0;
  a.hub_rows = hubs ? p->hub_rows : nullptr; a.n_hub = hubs ? p->n_hub : 0; a.hub_top = hubs ? p->hub_top : nullptr;
  if (blocks > 0 && hubs) budget_hub_topk_kernel<<<(unsigned)p->n_hub, 256, 0, st>>>(a);
  if (blocks > 0) {
    if (narrow) budget_select_kernel<8><<<(unsigned)blocks, 256, 0, st>>>(a);
    else budget_select_kernel<32><<<(unsigned)blocks, 256, 0, st>>>(a);
  }
  return (int)cudaGetLastError();
}

extern "C" int bf_ell_to_csr(const int* ell_col, const uint8_t* ell_type, const int* rowptr, int n, int cap, int* col,
                             uint8_t* etype, cudaStream_t st) {
  const long long total = (long long)n * cap;
  const long long blocks = (total + 255) / 256;
  if (blocks > 0) ell_to_csr_kernel<<<(unsigned)blocks, 256, 0, st>>>(ell_col, ell_type, rowptr, n, cap, col, etype);
  return (int)cudaGetLastError();
}
