// Balanced k-way node partition for locality reordering of the legacy mini-batch path.
//
// The reference relabels nodes so that each METIS part owns a contiguous id range (gt_sp/utils.py:787-819, through
// dgl.metis_partition_assignment).  Neither DGL nor METIS is a dependency here; this file is a small multilevel
// partitioner of the same family:
//   1. coarsening by heavy-edge matching (a node is merged with the unmatched neighbour it shares the heaviest
//      edge with, under a cap on the merged weight) until the graph is small or stops shrinking;
//   2. initial partition of the coarsest graph: breadth-first ordering of every component from a pseudo-peripheral
//      node, cut into k ranges of equal node weight;
//   3. projection back level by level, each followed by sweeps of balance-constrained boundary refinement: a node
//      moves to the part it is most strongly connected to when that lowers the cut (or keeps it and improves the
//      balance) and both parts stay inside [(1 - eps), (1 + eps)] x (total weight / k).
// Deterministic (single thread, fixed visiting orders).  Input is a symmetric CSR without self loops.
#include <algorithm>
#include <cstdint>
#include <numeric>
#include <vector>

namespace {

struct Graph {
  int n = 0;
  std::vector<int> xadj, adj, ew, vw;   // CSR, edge weights, node weights
  long long total_vw = 0;
};

inline uint32_t mix(uint32_t x) {
  x ^= x >> 16; x *= 0x7feb352dU; x ^= x >> 15; x *= 0x846ca68bU; x ^= x >> 16;
  return x;
}

// Fixed pseudo-random visiting order of the matching (one sort per level; the matching is sensitive to structure
// in the order, the refinement sweeps are not and walk the nodes in memory order).
std::vector<int> shuffled_order(int n, uint32_t salt) {
  std::vector<int> order(n);
  std::iota(order.begin(), order.end(), 0);
  std::sort(order.begin(), order.end(), [salt](int a, int b) {
    const uint32_t ha = mix((uint32_t)a ^ salt), hb = mix((uint32_t)b ^ salt);
    return ha != hb ? ha < hb : a < b;
  });
  return order;
}

// Heavy-edge matching; returns the number of coarse nodes and fills cmap (fine node -> coarse node).
int match_nodes(const Graph& g, int max_vw, std::vector<int>& cmap, uint32_t salt) {
  std::vector<int> mate(g.n, -1);
  const std::vector<int> order = shuffled_order(g.n, salt);
  for (int v : order) {
    if (mate[v] >= 0) continue;
    int best = -1, best_w = 0;
    for (int e = g.xadj[v]; e < g.xadj[v + 1]; ++e) {
      const int u = g.adj[e];
      if (mate[u] >= 0 || u == v || g.vw[v] + g.vw[u] > max_vw) continue;
      if (g.ew[e] > best_w || (g.ew[e] == best_w && best >= 0 && g.vw[u] < g.vw[best])) best = u, best_w = g.ew[e];
    }
    mate[v] = best >= 0 ? best : v;
    if (best >= 0) mate[best] = v;
  }
  int nc = 0;
  cmap.assign(g.n, -1);
  for (int v = 0; v < g.n; ++v) {
    if (cmap[v] >= 0) continue;
    cmap[v] = nc;
    if (mate[v] != v) cmap[mate[v]] = nc;
    ++nc;
  }
  return nc;
}

Graph contract(const Graph& g, const std::vector<int>& cmap, int nc) {
  Graph c;
  c.n = nc;
  c.vw.assign(nc, 0);
  c.total_vw = g.total_vw;
  std::vector<int> first(nc + 1, 0), members(g.n);           // fine nodes grouped by coarse node (counting sort)
  for (int v = 0; v < g.n; ++v) {
    c.vw[cmap[v]] += g.vw[v];
    ++first[cmap[v] + 1];
  }
  for (int cv = 0; cv < nc; ++cv) first[cv + 1] += first[cv];
  {
    std::vector<int> fill(first.begin(), first.end() - 1);
    for (int v = 0; v < g.n; ++v) members[fill[cmap[v]]++] = v;
  }
  c.adj.reserve(g.adj.size());
  c.ew.reserve(g.adj.size());
  c.xadj.assign(nc + 1, 0);
  std::vector<int> slot(nc, -1);             // position of a coarse neighbour in the row being built
  for (int cv = 0; cv < nc; ++cv) {
    const int row_begin = (int)c.adj.size();
    for (int m = first[cv]; m < first[cv + 1]; ++m) {
      const int v = members[m];
      for (int e = g.xadj[v]; e < g.xadj[v + 1]; ++e) {
        const int cu = cmap[g.adj[e]];
        if (cu == cv) continue;
        if (slot[cu] < row_begin) {           // first time in this row (older rows left smaller positions behind)
          slot[cu] = (int)c.adj.size();
          c.adj.push_back(cu);
          c.ew.push_back(g.ew[e]);
        } else {
          c.ew[slot[cu]] += g.ew[e];
        }
      }
    }
    c.xadj[cv + 1] = (int)c.adj.size();
  }
  return c;
}

// BFS from `root` over unvisited nodes; appends to `order`, returns the last node reached (a farthest one).
int bfs_component(const Graph& g, int root, std::vector<uint8_t>& seen, std::vector<int>& order) {
  size_t head = order.size();
  order.push_back(root);
  seen[root] = 1;
  int last = root;
  while (head < order.size()) {
    const int v = order[head++];
    last = v;
    for (int e = g.xadj[v]; e < g.xadj[v + 1]; ++e) {
      const int u = g.adj[e];
      if (!seen[u]) {
        seen[u] = 1;
        order.push_back(u);
      }
    }
  }
  return last;
}

void initial_partition(const Graph& g, int k, std::vector<int>& part) {
  std::vector<int> order, scratch;
  order.reserve(g.n);
  std::vector<uint8_t> probe(g.n, 0), seen(g.n, 0);
  for (int s = 0; s < g.n; ++s) {
    if (seen[s]) continue;
    scratch.clear();
    const int far = bfs_component(g, s, probe, scratch);
    bfs_component(g, far, seen, order);
  }
  part.assign(g.n, 0);
  long long acc = 0;
  for (int v : order) {                                       // ranges of equal node weight along the ordering
    const long long mid = acc + g.vw[v] / 2;
    part[v] = (int)std::min<long long>(k - 1, (mid * k) / std::max<long long>(g.total_vw, 1));
    acc += g.vw[v];
  }
}

long long refine(const Graph& g, int k, double eps, int passes, std::vector<int>& part, uint32_t salt) {
  std::vector<long long> size(k, 0);
  for (int v = 0; v < g.n; ++v) size[part[v]] += g.vw[v];
  const double ideal = (double)g.total_vw / (double)k;
  int heaviest = 0;
  for (int w : g.vw) heaviest = std::max(heaviest, w);
  // a coarse node can be heavier than the slack: allow one such node on top of the bound
  const long long max_size = (long long)((1.0 + eps) * ideal) + (heaviest > 1 ? heaviest : 1);
  const long long min_size = std::max<long long>((long long)((1.0 - eps) * ideal) - (heaviest > 1 ? heaviest : 0), 1);
  std::vector<long long> conn(k, 0);
  std::vector<int> touched;
  long long moved_total = 0;
  for (int pass = 0; pass < passes; ++pass) {
    long long moved = 0;
    const bool forward = ((pass + salt) & 1u) == 0;          // alternate the sweep direction
    for (int i = 0; i < g.n; ++i) {
      const int v = forward ? i : g.n - 1 - i;
      if (g.xadj[v] == g.xadj[v + 1]) continue;
      const int cur = part[v];
      touched.clear();
      for (int e = g.xadj[v]; e < g.xadj[v + 1]; ++e) {
        const int p = part[g.adj[e]];
        if (conn[p] == 0) touched.push_back(p);
        conn[p] += g.ew[e];
      }
      int best = cur;
      long long best_conn = conn[cur];
      for (int p : touched) {
        if (p == cur || size[p] + g.vw[v] > max_size) continue;
        const bool better = conn[p] > best_conn ||
                            (conn[p] == best_conn && (best == cur ? size[p] + g.vw[v] < size[cur]
                                                                  : (size[p] < size[best] || (size[p] == size[best] && p < best))));
        if (better) best = p, best_conn = conn[p];
      }
      for (int p : touched) conn[p] = 0;
      if (best != cur && size[cur] - g.vw[v] >= min_size) {
        part[v] = best;
        size[cur] -= g.vw[v];
        size[best] += g.vw[v];
        ++moved;
      }
    }
    moved_total += moved;
    if (moved * 2000 < g.n) break;                            // converged: under 0.05 % of the nodes moved
  }
  return moved_total;
}

// Final pass on the original graph: bring every part inside the requested bounds by moving, out of an overweight
// part, the nodes that lose the least connectivity (all node weights are 1 here).
void rebalance(const Graph& g, int k, double eps, std::vector<int>& part) {
  std::vector<long long> size(k, 0);
  for (int v = 0; v < g.n; ++v) size[part[v]] += g.vw[v];
  const long long max_size = (long long)((1.0 + eps) * (double)g.total_vw / k) + 1;
  std::vector<long long> conn(k, 0);
  for (int sweep = 0; sweep < 4; ++sweep) {
    bool over = false;
    for (int p = 0; p < k; ++p) over |= size[p] > max_size;
    if (!over) return;
    for (int v = 0; v < g.n; ++v) {
      const int cur = part[v];
      if (size[cur] <= max_size) continue;
      std::fill(conn.begin(), conn.end(), 0);
      for (int e = g.xadj[v]; e < g.xadj[v + 1]; ++e) conn[part[g.adj[e]]] += g.ew[e];
      int best = -1;
      for (int p = 0; p < k; ++p) {
        if (p == cur || size[p] + g.vw[v] > max_size) continue;
        if (best < 0 || conn[p] > conn[best] || (conn[p] == conn[best] && size[p] < size[best])) best = p;
      }
      if (best < 0) continue;
      part[v] = best;
      size[cur] -= g.vw[v];
      size[best] += g.vw[v];
    }
  }
}

}  // namespace

// part[v] in [0, k).  Returns the number of moves made by the refinement sweeps of all levels (>= 0), -1 on bad
// arguments.  `refine_passes` sweeps are made per level.
extern "C" long long bf_partition_cpu(const int* rowptr, const int* col, int n, int k, float imbalance, int refine_passes,
                                      int* part_out) {
  if (n < 0 || k <= 0) return -1;
  if (n == 0) return 0;
  if (k >= n) {                                               // one node per part
    for (int v = 0; v < n; ++v) part_out[v] = v;
    return 0;
  }
  const double eps = imbalance > 0.f ? (double)imbalance : 0.0;

  std::vector<Graph> levels(1);
  Graph& g0 = levels[0];
  g0.n = n;
  g0.xadj.assign(rowptr, rowptr + n + 1);
  g0.adj.assign(col, col + rowptr[n]);
  g0.ew.assign(g0.adj.size(), 1);
  g0.vw.assign(n, 1);
  g0.total_vw = n;

  // 1. coarsen
  std::vector<std::vector<int>> cmaps;
  const int target = std::max(128, 24 * k);
  const int max_vw = std::max<long long>(1, (long long)n / (long long)(4 * (long long)k) );   // merged weight stays well below a part
  while (levels.back().n > target && cmaps.size() < 40) {
    std::vector<int> cmap;
    const Graph& fine = levels.back();
    const int nc = match_nodes(fine, max_vw, cmap, 0x51ed27u + (uint32_t)cmaps.size());
    if (nc > 0.95 * fine.n) break;                            // stopped shrinking
    Graph coarse = contract(fine, cmap, nc);
    cmaps.push_back(std::move(cmap));
    levels.push_back(std::move(coarse));
  }

  // 2. initial partition of the coarsest graph, 3. refine and project back
  std::vector<int> part;
  initial_partition(levels.back(), k, part);
  long long moved = 0;
  for (int lvl = (int)levels.size() - 1; lvl >= 0; --lvl) {
    const int passes = lvl == (int)levels.size() - 1 ? std::max(refine_passes, 4) * 2 : refine_passes;
    moved += refine(levels[lvl], k, eps, passes, part, 0xa511e9b3u + (uint32_t)lvl);
    if (lvl > 0) {
      const std::vector<int>& cmap = cmaps[lvl - 1];
      std::vector<int> fine_part(levels[lvl - 1].n);
      for (int v = 0; v < levels[lvl - 1].n; ++v) fine_part[v] = part[cmap[v]];
      part.swap(fine_part);
    }
  }
  rebalance(levels[0], k, eps, part);
  std::copy(part.begin(), part.end(), part_out);
  return moved;
}
