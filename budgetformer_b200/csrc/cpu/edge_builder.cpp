// C++/OpenMP twin of edge_build.cu: the same per-query selection, walk and merge rules evaluated
// with std::sort per query.  Used by the CPU edge policies of the execution planner (the raw
// topology stays in host memory and only the compact per-query rows are uploaded) and as the
// integer oracle for the CUDA builder — outputs are bit-identical.
// Reference behaviour restated: utils/fullgraph_sp_support.py:1119-1192 (CPU per-query sampler),
// gt_sp/utils.py:1198-1248 (walk edge emission), gt_sp/utils.py:1396-1442 (CPU walker).
#include <algorithm>
#include <cstdint>
#include <vector>

#ifdef _OPENMP
#include <omp.h>
#endif

#include "../edge_spec.h"

namespace {

// Keep the k smallest composites (hash << 32 | source id) of one side.
inline void keep_smallest(std::vector<uint64_t>& c, int k) {
  if ((int)c.size() > k) {
    std::nth_element(c.begin(), c.begin() + k, c.end());
    c.resize(k);
  }
}

// Merge the selected real and walk sources of query v into its fixed-width row.  Plain models: union, ascending,
// duplicates removed.  Exphormer: real sources (type 0), walk sources (type 1), then the self loop (type 0), each
// part ascending and nothing removed.
inline int write_row(int v, const std::vector<uint64_t>& rc, const std::vector<uint64_t>& wc, bool exphormer,
                     std::vector<uint32_t>& tmp, int* row, uint8_t* trow) {
  int c = 0;
  if (exphormer) {
    tmp.clear();
    for (uint64_t x : rc) tmp.push_back((uint32_t)x);
    std::sort(tmp.begin(), tmp.end());
    for (uint32_t s : tmp) { row[c] = (int)s; trow[c++] = 0; }
    tmp.clear();
    for (uint64_t x : wc) tmp.push_back((uint32_t)x);
    std::sort(tmp.begin(), tmp.end());
    for (uint32_t s : tmp) { row[c] = (int)s; trow[c++] = 1; }
    row[c] = v; trow[c++] = 0;
    return c;
  }
  tmp.clear();
  for (uint64_t x : rc) tmp.push_back((uint32_t)x);
  for (uint64_t x : wc) tmp.push_back((uint32_t)x);
  std::sort(tmp.begin(), tmp.end());
  tmp.erase(std::unique(tmp.begin(), tmp.end()), tmp.end());
  for (uint32_t s : tmp) row[c++] = (int)s;
  return c;
}

}  // namespace

extern "C" int bf_budget_select_cpu(const int* in_rowptr, const int* in_src, const int* out_rowptr,
                                    const int* out_col, int n, int b_real, int b_rw, int walks, int walk_len,
                                    int exphormer, long long seed, int cap, int* ell_col, uint8_t* ell_type,
                                    int* ell_cnt, unsigned long long* totals, int num_threads) {
  unsigned long long tot_r = 0, tot_w = 0;
#ifdef _OPENMP
  if (num_threads > 0) omp_set_num_threads(num_threads);
#endif
#pragma omp parallel reduction(+ : tot_r, tot_w)
  {
    std::vector<uint64_t> rc, wc;
    std::vector<uint32_t> merged;
#pragma omp for schedule(dynamic, 1024)
    for (int v = 0; v < n; ++v) {
      rc.clear();
      wc.clear();
      if (b_real > 0) {
        const int beg = in_rowptr[v], end = in_rowptr[v + 1];
        for (int e = beg; e < end; ++e)
          rc.push_back(bf_edge_composite((uint32_t)in_src[e], (uint32_t)v, seed + BF_REAL_SEED_OFFSET));
        keep_smallest(rc, b_real);
      }
      if (b_rw > 0 && walks > 0 && walk_len > 0) {
        for (int w = 0; w < walks; ++w) {
          const uint64_t walk_id = (uint64_t)v * (uint64_t)walks + (uint64_t)w;
          int cur = v;
          for (int d = 1; d <= walk_len; ++d) {
            const int prev = cur;
            const int ob = out_rowptr[cur], oe = out_rowptr[cur + 1];
            const uint32_t deg = (uint32_t)(oe - ob);
            if (deg > 0) cur = out_col[ob + (int)bf_mulhi32(bf_walk_uniform32(walk_id, (uint32_t)d, (uint64_t)seed), deg)];
            if (d == 1 || cur != prev) wc.push_back(bf_edge_composite((uint32_t)cur, (uint32_t)v, seed + BF_RW_SEED_OFFSET));
          }
        }
        keep_smallest(wc, b_rw);
      }
      tot_r += rc.size();
      tot_w += wc.size();
      ell_cnt[v] = write_row(v, rc, wc, exphormer != 0, merged, ell_col + (long long)v * cap,
                             exphormer ? ell_type + (long long)v * cap : nullptr);
    }
  }
  totals[0] = tot_r;
  totals[1] = tot_w;
  return 0;
}

extern "C" int bf_ell_to_csr_cpu(const int* ell_col, const uint8_t* ell_type, const int* rowptr, int n, int cap,
                                 int* col, uint8_t* etype) {
#pragma omp parallel for schedule(static)
  for (int v = 0; v < n; ++v) {
    const int beg = rowptr[v], cnt = rowptr[v + 1] - beg;
    for (int s = 0; s < cnt; ++s) {
      col[beg + s] = ell_col[(long long)v * cap + s];
      if (etype) etype[beg + s] = ell_type[(long long)v * cap + s];
    }
  }
  return 0;
}

// -----------------------------------------------------------------------------------------------------
// Fan-out k-hop expansion with origin tracking (`--rw_edge_mode dgl_neighbor`; the reference delegates it
// to DGL's neighbour sampler, gt_sp/utils.py:1281-1384).  From every origin node, hop h keeps at most
// fanout[h] out-neighbours of each frontier node (negative = all), ranked by a seeded hash so that the
// choice is reproducible on every rank, and emits (reached node -> origin).  The next frontier is the set
// of distinct reached nodes.  Origins are independent, so the expansion runs one origin per OpenMP task
// in two passes (count, then fill at prefix-sum offsets); rows come out origin-major, hop-minor, node ids
// ascending inside a hop.  Same candidate multiset as graph/builder_spec.py::khop_neighbor_candidates.
// -----------------------------------------------------------------------------------------------------
namespace {

struct KhopScratch {
  std::vector<int> frontier, next;
  std::vector<std::pair<uint64_t, int>> ranked;   // (key, position in the CSR row) of one frontier node's neighbours
};

// Runs the expansion of one origin; `emit` receives every reached node of every hop.
template <typename Emit>
inline void khop_expand(const int* rowptr, const int* col, int origin, const int* fanout, int n_hops, long long seed,
                        KhopScratch& s, Emit emit) {
  s.frontier.assign(1, origin);
  const uint64_t omix = ((uint64_t)origin * 2654435761ull) & 0x7FFFFFFFull;
  for (int h = 0; h < n_hops && !s.frontier.empty(); ++h) {
    s.next.clear();
    const int f = fanout[h];
    const long long hseed = seed + 101ll * (h + 1);
    for (int node : s.frontier) {
      const int beg = rowptr[node], deg = rowptr[node + 1] - beg;
      if (f < 0 || deg <= f) {
        s.next.insert(s.next.end(), col + beg, col + beg + deg);
        continue;
      }
      s.ranked.clear();
      for (int i = 0; i < deg; ++i) {
        const uint64_t hash31 = bf_edge_composite((uint32_t)col[beg + i], (uint32_t)node, hseed) >> 32;
        s.ranked.emplace_back(hash31 ^ omix, i);           // ties keep CSR order (pair comparison)
      }
      std::partial_sort(s.ranked.begin(), s.ranked.begin() + f, s.ranked.end());
      for (int i = 0; i < f; ++i) s.next.push_back(col[beg + s.ranked[i].second]);
    }
    std::sort(s.next.begin(), s.next.end());
    s.next.erase(std::unique(s.next.begin(), s.next.end()), s.next.end());
    for (int v : s.next) emit(v);
    s.frontier.swap(s.next);
  }
}

}  // namespace

// Pass 1: counts[origin] = number of candidates of that origin.
extern "C" int bf_khop_count_cpu(const int* out_rowptr, const int* out_col, int n, const int* fanout, int n_hops,
                                 long long seed, long long* counts, int num_threads) {
#ifdef _OPENMP
  if (num_threads > 0) omp_set_num_threads(num_threads);
#endif
#pragma omp parallel
  {
    KhopScratch s;
#pragma omp for schedule(dynamic, 256)
    for (int o = 0; o < n; ++o) {
      long long c = 0;
      khop_expand(out_rowptr, out_col, o, fanout, n_hops, seed, s, [&](int) { ++c; });
      counts[o] = c;
    }
  }
  return 0;
}

// Pass 2: offsets = exclusive prefix sums of the counts; src[offsets[o] + i] = i-th reached node, dst = origin.
extern "C" int bf_khop_fill_cpu(const int* out_rowptr, const int* out_col, int n, const int* fanout, int n_hops,
                                long long seed, const long long* offsets, long long* src, long long* dst,
                                int num_threads) {
#ifdef _OPENMP
  if (num_threads > 0) omp_set_num_threads(num_threads);
#endif
#pragma omp parallel
  {
    KhopScratch s;
#pragma omp for schedule(dynamic, 256)
    for (int o = 0; o < n; ++o) {
      long long w = offsets[o];
      khop_expand(out_rowptr, out_col, o, fanout, n_hops, seed, s, [&](int v) { src[w] = v; dst[w] = o; ++w; });
    }
  }
  return 0;
}

// -----------------------------------------------------------------------------------------------------
// General CPU build with rows of any length: budgets above the fixed-width limit of the CUDA builder and
// "no budget" (b < 0: keep every candidate - the reference's default without budget flags, all real edges and
// the whole walk pool).  Two passes over the queries [row_begin, row_end) - a rank may build only its own rows, they
// do not depend on one another: `offsets == nullptr` counts the row lengths, otherwise the rows are written at
// their prefix-sum offsets (counts and offsets are indexed from row_begin).  Walk candidates come from Philox walks (n_hops == 0) or from
// the fan-out expansion (n_hops > 0).  Same selection and merge rules as the fixed-width builders above.
// -----------------------------------------------------------------------------------------------------
extern "C" int bf_build_rows_cpu(const int* in_rowptr, const int* in_src, const int* out_rowptr, const int* out_col,
                                 int row_begin, int row_end, int b_real, int b_rw, int use_real, int use_rw, int walks,
                                 int walk_len,
                                 const int* fanout, int n_hops, int exphormer, long long seed,
                                 const long long* offsets, long long* counts, int* col, uint8_t* etype,
                                 unsigned long long* totals, int num_threads) {
  unsigned long long tot_r = 0, tot_w = 0;
#ifdef _OPENMP
  if (num_threads > 0) omp_set_num_threads(num_threads);
#endif
#pragma omp parallel reduction(+ : tot_r, tot_w)
  {
    std::vector<uint64_t> rc, wc;
    std::vector<uint32_t> merged;
    std::vector<int> row;
    std::vector<uint8_t> trow;
    KhopScratch scratch;
#pragma omp for schedule(dynamic, 256)
    for (int v = row_begin; v < row_end; ++v) {
      rc.clear();
      wc.clear();
      if (use_real && b_real != 0) {
        for (int e = in_rowptr[v]; e < in_rowptr[v + 1]; ++e)
          rc.push_back(bf_edge_composite((uint32_t)in_src[e], (uint32_t)v, seed + BF_REAL_SEED_OFFSET));
        if (b_real > 0) keep_smallest(rc, b_real);
      }
      if (use_rw && b_rw != 0) {
        auto add = [&](int u) { wc.push_back(bf_edge_composite((uint32_t)u, (uint32_t)v, seed + BF_RW_SEED_OFFSET)); };
        if (n_hops > 0) {
          khop_expand(out_rowptr, out_col, v, fanout, n_hops, seed, scratch, add);
        } else {
          for (int w = 0; w < walks; ++w) {
            const uint64_t walk_id = (uint64_t)v * (uint64_t)walks + (uint64_t)w;
            int cur = v;
            for (int d = 1; d <= walk_len; ++d) {
              const int prev = cur;
              const int ob = out_rowptr[cur];
              const uint32_t deg = (uint32_t)(out_rowptr[cur + 1] - ob);
              if (deg > 0) cur = out_col[ob + (int)bf_mulhi32(bf_walk_uniform32(walk_id, (uint32_t)d, (uint64_t)seed), deg)];
              if (d == 1 || cur != prev) add(cur);
            }
          }
        }
        if (b_rw > 0) keep_smallest(wc, b_rw);
      }
      tot_r += rc.size();
      tot_w += wc.size();
      const size_t width = rc.size() + wc.size() + 1;
      row.resize(width);
      trow.resize(width);
      const int c = write_row(v, rc, wc, exphormer != 0, merged, row.data(), trow.data());
      if (offsets == nullptr) {
        counts[v - row_begin] = c;
      } else {
        const long long o = offsets[v - row_begin];
        std::copy(row.begin(), row.begin() + c, col + o);
        if (exphormer) std::copy(trow.begin(), trow.begin() + c, etype + o);
      }
    }
  }
  totals[0] = tot_r;
  totals[1] = tot_w;
  return 0;
}
