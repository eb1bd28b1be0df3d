// Balanced k-way node partition for locality reordering of the legacy mini-batch path.
//
// The reference relabels nodes so that each METIS part owns a contiguous id range (gt_sp/utils.py:787-819, through
// dgl.metis_partition_assignment).  Neither DGL nor METIS is a dependency here; the partition is made by
//   1. a breadth-first ordering of every connected component from a pseudo-peripheral node (two sweeps: the node
//      farthest from an arbitrary start becomes the root), which lays neighbours next to one another,
//   2. cutting that ordering into k equal ranges, and
//   3. sweeps of balance-constrained boundary refinement: a node moves to the part that holds most of its neighbours
//      when that lowers the edge cut and keeps both parts inside [floor((1-eps) n/k), ceil((1+eps) n/k)].
// Deterministic (single thread, fixed visiting order).  Input is a symmetric CSR without self loops.
#include <algorithm>
#include <cstdint>
#include <vector>

namespace {

// BFS from `root` over unvisited nodes; appends to `order`, returns the last node reached (a farthest one).
int bfs_component(const int* rowptr, const int* col, int root, std::vector<uint8_t>& seen, std::vector<int>& order) {
  size_t head = order.size();
  order.push_back(root);
  seen[root] = 1;
  int last = root;
  while (head < order.size()) {
    const int v = order[head++];
    last = v;
    for (int e = rowptr[v]; e < rowptr[v + 1]; ++e) {
      const int u = col[e];
      if (!seen[u]) {
        seen[u] = 1;
        order.push_back(u);
      }
    }
  }
  return last;
}

}  // namespace

// part[v] in [0, k).  Returns the number of nodes moved by the refinement sweeps (>= 0) or -1 on bad arguments.
extern "C" long long bf_partition_cpu(const int* rowptr, const int* col, int n, int k, float imbalance, int refine_passes,
                                      int* part) {
  if (n < 0 || k <= 0) return -1;
  if (n == 0) return 0;
  if (k > n) k = n;

  // 1. component-wise BFS ordering from pseudo-peripheral roots
  std::vector<int> order;
  order.reserve(n);
  {
    std::vector<uint8_t> probe(n, 0), seen(n, 0);
    std::vector<int> scratch;
    scratch.reserve(n);
    for (int s = 0; s < n; ++s) {
      if (seen[s]) continue;
      scratch.clear();
      const int far = bfs_component(rowptr, col, s, probe, scratch);   // marks the component in `probe`
      bfs_component(rowptr, col, far, seen, order);                    // the ordering proper
    }
  }

  // 2. equal ranges of the ordering
  std::vector<long long> size(k, 0);
  for (int i = 0; i < n; ++i) {
    const int p = (int)(((long long)i * k) / n);
    part[order[i]] = p;
    ++size[p];
  }

  // 3. boundary refinement under the balance constraint
  const double ideal = (double)n / (double)k;
  const double eps = imbalance > 0.f ? (double)imbalance : 0.0;
  const long long max_size = (long long)((1.0 + eps) * ideal) + 1;
  long long min_size = (long long)((1.0 - eps) * ideal);
  if (min_size < 1) min_size = 1;
  std::vector<int> cnt(k, 0), touched;
  touched.reserve(64);
  long long moved_total = 0;
  for (int pass = 0; pass < refine_passes; ++pass) {
    long long moved = 0;
    for (int i = 0; i < n; ++i) {
      const int v = order[i];
      const int beg = rowptr[v], end = rowptr[v + 1];
      if (beg == end) continue;
      const int cur = part[v];
      touched.clear();
      for (int e = beg; e < end; ++e) {
        const int p = part[col[e]];
        if (cnt[p]++ == 0) touched.push_back(p);
      }
      int best = cur, best_cnt = cnt[cur];
      for (int p : touched) {
        // strict gain; ties go to the lower part id so that the result does not depend on neighbour order
        if (p != cur && (cnt[p] > best_cnt || (cnt[p] == best_cnt && best != cur && p < best)) &&
            size[p] + 1 <= max_size)
          best = p, best_cnt = cnt[p];
      }
      for (int p : touched) cnt[p] = 0;
      if (best != cur && size[cur] - 1 >= min_size) {
        part[v] = best;
        --size[cur];
        ++size[best];
        ++moved;
      }
    }
    moved_total += moved;
    if (moved == 0) break;
  }
  return moved_total;
}
