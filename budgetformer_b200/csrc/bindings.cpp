// PyTorch bindings: tensor checks, allocation of workspaces and stream plumbing around the C
// launchers declared in bf_kernels.h.  No kernel code lives here.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "bf_kernels.h"

extern "C" int bf_budget_select_cpu(const int*, const int*, const int*, const int*, int, int, int, int, int, int,
                                    long long, int, int*, uint8_t*, int*, unsigned long long*, int);
extern "C" int bf_ell_to_csr_cpu(const int*, const uint8_t*, const int*, int, int, int*, uint8_t*);
extern "C" int bf_build_rows_cpu(const int*, const int*, const int*, const int*, int, int, int, int, int, int, int, int,
                                 const int*, int, int, long long, const long long*, long long*, int*, uint8_t*,
                                 unsigned long long*, int);

namespace {

using torch::Tensor;
using OptTensor = c10::optional<Tensor>;

void check_cuda(int err, const char* what) {
  TORCH_CHECK(err == 0, what, " failed: ", cudaGetErrorString((cudaError_t)err));
}

int dtype_code(const Tensor& t) {
  if (t.scalar_type() == torch::kBFloat16) return BF_BF16;
  if (t.scalar_type() == torch::kHalf) return BF_FP16;
  if (t.scalar_type() == torch::kFloat) return BF_FP32;
  TORCH_CHECK(false, "unsupported dtype ", t.scalar_type());
}

void check_qkv(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.dim() == 3, name, " must be a CUDA [n, heads, head_dim] tensor");
  TORCH_CHECK(t.stride(2) == 1 && t.stride(1) == t.size(2), name, " must be contiguous in its last two dims");
  TORCH_CHECK((t.stride(0) * t.element_size()) % 16 == 0 && ((uintptr_t)t.data_ptr()) % 16 == 0, name,
              " rows must be 16-byte aligned");
}

const int* iptr(const Tensor& t) { return t.data_ptr<int>(); }

struct HubInfo {
  Tensor rows;
  int n = 0;
  int max_deg = 0;
};

// Rows of a CSR longer than BF_HUB_DEGREE.  `known_max` >= 0 skips the device query.
HubInfo find_hubs(const Tensor& rowptr, int64_t known_max) {
  HubInfo h;
  if (known_max >= 0 && known_max <= BF_HUB_DEGREE) return h;
  auto deg = rowptr.slice(0, 1) - rowptr.slice(0, 0, rowptr.size(0) - 1);
  auto rows = torch::nonzero(deg > BF_HUB_DEGREE).flatten().to(torch::kInt);
  h.n = (int)rows.size(0);
  if (h.n > 0) {
    h.rows = rows;
    h.max_deg = deg.max().item<int>();
  }
  return h;
}

// out_drop = {p, seed, rows per owning rank, column offset} or empty: dropout fused into the attention output
void fill_common(bf_attn_params& p, const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& out,
                 const Tensor& z, const Tensor& rowptr, const Tensor& col, const OptTensor& etype,
                 const OptTensor& etab, int64_t variant, double dropout_p, int64_t seed,
                 const std::vector<double>& out_drop) {
  if (!out_drop.empty()) {
    TORCH_CHECK(out_drop.size() == 4 && out_drop[0] >= 0.0 && out_drop[0] < 1.0, "out_drop = [p, seed, rows_local, col0]");
    p.out_dropout_p = (float)out_drop[0]; p.out_dropout_seed = (uint32_t)(int64_t)out_drop[1];
    p.out_rows_local = (int)out_drop[2]; p.out_col0 = (int)out_drop[3];
  }
  check_qkv(q, "q"); check_qkv(k, "k"); check_qkv(v, "v");
  TORCH_CHECK(out.is_contiguous() && z.is_contiguous());
  TORCH_CHECK(rowptr.scalar_type() == torch::kInt && col.scalar_type() == torch::kInt, "graph indices must be int32");
  p.q = q.data_ptr(); p.k = k.data_ptr(); p.v = v.data_ptr();
  p.ldq = q.stride(0); p.ldk = k.stride(0); p.ldv = v.stride(0);
  p.out = out.data_ptr(); p.z = z.data_ptr<float>();
  p.rowptr = iptr(rowptr); p.col = iptr(col);
  p.etype = etype.has_value() ? etype->data_ptr<uint8_t>() : nullptr;
  p.etab = etab.has_value() ? etab->data_ptr<float>() : nullptr;
  p.n = (int)q.size(0); p.hl = (int)q.size(1); p.hn = (int)q.size(2);
  p.dtype = dtype_code(q); p.variant = (int)variant;
  p.dropout_p = (float)dropout_p; p.dropout_seed = (uint32_t)seed;
  TORCH_CHECK(variant != 2 || (p.etype && p.etab), "exphormer variant needs edge types and a type table");
}

// route = {} or {rows per destination, first row of this rank's slab, destination row stride (elements),
// base pointer of destination 0, 1, ...}: see bf_attn_route
bf_attn_route parse_route(const std::vector<int64_t>& route, size_t header) {
  bf_attn_route r{};
  if (route.empty()) return r;
  TORCH_CHECK(route.size() > header && route.size() - header <= BF_MAX_PEERS, "route: header + 1..", BF_MAX_PEERS, " destinations");
  r.rows_per = (int)route[0]; r.slab_row0 = route[1]; r.ld = route[2];
  r.n_dest = (int)(route.size() - header);
  for (int i = 0; i < r.n_dest; ++i) r.base[i] = reinterpret_cast<void*>(route[header + i]);
  return r;
}

void edge_attn_fwd(Tensor q, Tensor k, Tensor v, Tensor out, Tensor z, Tensor rowptr, Tensor col, OptTensor etype,
                   OptTensor etab, int64_t variant, double dropout_p, int64_t seed, int64_t known_max_degree,
                   std::vector<double> out_drop, std::vector<int64_t> route) {
  c10::cuda::CUDAGuard guard(q.device());
  bf_attn_params p{};
  fill_common(p, q, k, v, out, z, rowptr, col, etype, etab, variant, dropout_p, seed, out_drop);
  HubInfo hub = find_hubs(rowptr, known_max_degree);
  Tensor scratch;
  if (hub.n > 0) {
    scratch = torch::zeros({hub.n, (int64_t)p.hl * p.hn + p.hl}, q.options().dtype(torch::kFloat));
    p.hub_rows = iptr(hub.rows); p.n_hub = hub.n; p.max_hub_degree = hub.max_deg;
    p.hub_scratch = scratch.data_ptr<float>();
  }
  const bf_attn_route r = parse_route(route, 3);
  check_cuda(bf_edge_attn_fwd_routed(&p, &r, at::cuda::getCurrentCUDAStream()), "edge_attn_fwd");
}

void edge_attn_bwd(Tensor q, Tensor k, Tensor v, Tensor out, Tensor z, Tensor dout, Tensor dq, Tensor dk, Tensor dv,
                   Tensor zd, Tensor rowptr, Tensor col, OptTensor etype, Tensor t_rowptr, Tensor t_row, Tensor t_eid,
                   OptTensor etab, OptTensor detab, int64_t variant, double dropout_p, int64_t seed,
                   int64_t known_max_degree, OptTensor kv_task, OptTensor kv_split, int64_t kv_slots,
                   std::vector<double> out_drop, std::vector<int64_t> route) {
  c10::cuda::CUDAGuard guard(q.device());
  bf_attn_params p{};
  fill_common(p, q, k, v, out, z, rowptr, col, etype, etab, variant, dropout_p, seed, out_drop);
  TORCH_CHECK(dout.is_contiguous());
  check_qkv(dq, "dq"); check_qkv(dk, "dk"); check_qkv(dv, "dv");
  TORCH_CHECK(dq.stride(0) == dk.stride(0) && dq.stride(0) == dv.stride(0), "dq/dk/dv must share one row stride");
  TORCH_CHECK(zd.is_contiguous() && zd.numel() == 2 * z.numel());
  bf_attn_bwd_params b{};
  b.dout = dout.data_ptr(); b.dq = dq.data_ptr(); b.dk = dk.data_ptr(); b.dv = dv.data_ptr();
  b.ldg = dq.stride(0);
  b.zd = zd.data_ptr<float>();
  b.t_rowptr = iptr(t_rowptr); b.t_row = iptr(t_row); b.t_eid = iptr(t_eid);
  b.detab = detab.has_value() ? detab->data_ptr<float>() : nullptr;
  HubInfo hub = find_hubs(rowptr, known_max_degree);
  const bool use_tasks = kv_task.has_value() && kv_task->numel() > 0;
  HubInfo thub = use_tasks ? HubInfo() : find_hubs(t_rowptr, -1);
  Tensor sq, skv, partial, qg, cz;
  if (use_tasks && (int64_t)p.hl * p.hn * q.element_size() <= 64) {
    // narrow rows: one packed record per (query, head) for the dK/dV pass (see bf_attn_bwd_params)
    qg = torch::empty({q.size(0), (int64_t)p.hl, 2, (int64_t)p.hn}, q.options());
    cz = torch::empty({q.size(0), (int64_t)p.hl}, q.options().dtype(torch::kFloat));
    b.qg = qg.data_ptr(); b.cz = cz.data_ptr<float>();
  }
  if (use_tasks) {
    TORCH_CHECK(kv_task->scalar_type() == torch::kInt && kv_task->is_contiguous() && kv_task->size(1) == 4 &&
                ((uintptr_t)kv_task->data_ptr()) % 16 == 0, "kv_task must be contiguous int32 [T, 4]");
    b.kv_task = kv_task->data_ptr<int>(); b.n_kv_task = (int)kv_task->size(0);
    if (kv_split.has_value() && kv_split->numel() > 0 && kv_slots > 0) {
      b.kv_split = kv_split->data_ptr<int>(); b.n_kv_split = (int)kv_split->size(0);
      partial = torch::empty({kv_slots, 2 * (int64_t)p.hl * p.hn}, q.options().dtype(torch::kFloat));
      b.kv_partial = partial.data_ptr<float>();
    }
  }
  const int64_t w = (int64_t)p.hl * p.hn;
  if (hub.n > 0) {
    sq = torch::zeros({hub.n, w}, q.options().dtype(torch::kFloat));
    p.hub_rows = iptr(hub.rows); p.n_hub = hub.n; p.max_hub_degree = hub.max_deg;
    b.hub_scratch_q = sq.data_ptr<float>();
  }
  if (thub.n > 0) {
    skv = torch::zeros({thub.n, 2 * w}, q.options().dtype(torch::kFloat));
    b.t_hub_rows = iptr(thub.rows); b.n_t_hub = thub.n; b.max_t_hub_degree = thub.max_deg;
    b.hub_scratch_kv = skv.data_ptr<float>();
  }
  if (!route.empty()) {
    // {rows per destination, slab row, row stride, column of dq, of dk, of dv, destination pointers...}
    TORCH_CHECK(route.size() > 6, "route: six header fields + destinations");
    b.route = parse_route(route, 6);
    b.route_cq = (int)route[3]; b.route_ck = (int)route[4]; b.route_cv = (int)route[5];
  }
  check_cuda(bf_edge_attn_bwd(&p, &b, at::cuda::getCurrentCUDAStream()), "edge_attn_bwd");
}

// Returns (rowptr int32 [n+1], col int32 [E], etype uint8 [E] or empty, totals int64 [2]).
// The caller's list of long in-edge rows (ascending int32 ids on the topology's device) and the scratch their ranked
// candidates go to; the returned tensor owns the scratch until the launch is queued (the caching allocator keeps it
// valid for work already in the stream).
Tensor attach_hub_rows(bf_build_params& p, const OptTensor& hub_rows, const Tensor& like) {
  if (!hub_rows.has_value() || hub_rows->numel() == 0) return Tensor();
  TORCH_CHECK(hub_rows->is_cuda() && hub_rows->scalar_type() == torch::kInt && hub_rows->is_contiguous() &&
              hub_rows->device() == like.device(), "hub_rows: contiguous int32 on the topology's device");
  Tensor top = torch::empty({hub_rows->numel() * 32}, like.options().dtype(torch::kLong));
  p.hub_rows = hub_rows->data_ptr<int>();
  p.n_hub = (int)hub_rows->numel();
  p.hub_top = reinterpret_cast<unsigned long long*>(top.data_ptr<int64_t>());
  return top;
}

std::vector<Tensor> build_attn_graph(Tensor in_rowptr, Tensor in_src, Tensor out_rowptr, Tensor out_col, int64_t n,
                                     int64_t b_real, int64_t b_rw, int64_t walks, int64_t walk_len, bool exphormer,
                                     int64_t seed, int64_t num_threads, OptTensor hub_rows) {
  TORCH_CHECK(b_real >= 0 && b_rw >= 0 && b_real <= 32 && b_rw <= 32, "per-side budgets must be in [0, 32]");
  TORCH_CHECK(walk_len <= 16, "walk_length must be <= 16");
  for (const Tensor* t : {&in_rowptr, &in_src, &out_rowptr, &out_col})
    TORCH_CHECK(t->scalar_type() == torch::kInt && t->is_contiguous(), "topology must be contiguous int32");
  const int cap = (int)(b_real + b_rw + (exphormer ? 1 : 0));
  auto iopt = in_src.options();
  Tensor ell_col = torch::empty({n, std::max(cap, 1)}, iopt);
  Tensor ell_type = exphormer ? torch::empty({n, std::max(cap, 1)}, iopt.dtype(torch::kUInt8)) : Tensor();
  Tensor ell_cnt = torch::zeros({n}, iopt);
  Tensor totals = torch::zeros({2}, iopt.dtype(torch::kLong));
  const bool cuda = in_src.is_cuda();
  if (cuda) {
    c10::cuda::CUDAGuard guard(in_src.device());
    bf_build_params p{};
    p.in_rowptr = iptr(in_rowptr); p.in_src = iptr(in_src); p.out_rowptr = iptr(out_rowptr); p.out_col = iptr(out_col);
    p.n = (int)n; p.b_real = (int)b_real; p.b_rw = (int)b_rw; p.walks = (int)walks; p.walk_len = (int)walk_len;
    p.exphormer = exphormer ? 1 : 0; p.seed = seed; p.cap = std::max(cap, 1);
    p.ell_col = ell_col.data_ptr<int>(); p.ell_type = exphormer ? ell_type.data_ptr<uint8_t>() : nullptr;
    p.ell_cnt = ell_cnt.data_ptr<int>();
    p.totals = reinterpret_cast<unsigned long long*>(totals.data_ptr<int64_t>());
    Tensor hub_top = attach_hub_rows(p, hub_rows, in_src);
    check_cuda(bf_budget_select(&p, at::cuda::getCurrentCUDAStream()), "budget_select");
  } else {
    bf_budget_select_cpu(iptr(in_rowptr), iptr(in_src), iptr(out_rowptr), iptr(out_col), (int)n, (int)b_real,
                         (int)b_rw, (int)walks, (int)walk_len, exphormer ? 1 : 0, seed, std::max(cap, 1),
                         ell_col.data_ptr<int>(), exphormer ? ell_type.data_ptr<uint8_t>() : nullptr,
                         ell_cnt.data_ptr<int>(), reinterpret_cast<unsigned long long*>(totals.data_ptr<int64_t>()),
                         (int)num_threads);
  }
  Tensor rowptr = torch::zeros({n + 1}, iopt);
  rowptr.slice(0, 1).copy_(torch::cumsum(ell_cnt, 0, torch::kInt));
  // The edge count sizes the output; this is the one host read of the build.
  const int64_t n_edges = n > 0 ? rowptr[n].item<int64_t>() : 0;
  Tensor col = torch::empty({n_edges}, iopt);
  Tensor etype = exphormer ? torch::empty({n_edges}, iopt.dtype(torch::kUInt8)) : Tensor();
  if (cuda) {
    check_cuda(bf_ell_to_csr(ell_col.data_ptr<int>(), exphormer ? ell_type.data_ptr<uint8_t>() : nullptr,
                             rowptr.data_ptr<int>(), (int)n, std::max(cap, 1), col.data_ptr<int>(),
                             exphormer ? etype.data_ptr<uint8_t>() : nullptr, at::cuda::getCurrentCUDAStream()),
               "ell_to_csr");
  } else {
    bf_ell_to_csr_cpu(ell_col.data_ptr<int>(), exphormer ? ell_type.data_ptr<uint8_t>() : nullptr,
                      rowptr.data_ptr<int>(), (int)n, std::max(cap, 1), col.data_ptr<int>(),
                      exphormer ? etype.data_ptr<uint8_t>() : nullptr);
  }
  return {rowptr, col, exphormer ? etype : torch::empty({0}, iopt.dtype(torch::kUInt8)), totals};
}

// One rank's shard of a device build: fixed-width rows of the queries [row_begin, row_begin + row_count) written into
// caller-provided buffers (symmetric memory, so that the peers can fetch them): ell_col [row_count, cap] int32,
// ell_cnt [row_count] int32, ell_type [row_count, cap] uint8 (typed rows only), totals [2] int64 (zeroed here).
void budget_select_rows(Tensor in_rowptr, Tensor in_src, Tensor out_rowptr, Tensor out_col, int64_t n, int64_t b_real,
                        int64_t b_rw, int64_t walks, int64_t walk_len, bool exphormer, int64_t seed, int64_t row_begin,
                        int64_t row_count, Tensor ell_col, Tensor ell_cnt, OptTensor ell_type, Tensor totals,
                        OptTensor hub_rows) {
  TORCH_CHECK(b_real >= 0 && b_rw >= 0 && b_real <= 32 && b_rw <= 32, "per-side budgets must be in [0, 32]");
  TORCH_CHECK(walk_len <= 16, "walk_length must be <= 16");
  for (const Tensor* t : {&in_rowptr, &in_src, &out_rowptr, &out_col})
    TORCH_CHECK(t->is_cuda() && t->scalar_type() == torch::kInt && t->is_contiguous(), "topology must be contiguous int32 on CUDA");
  const int cap = std::max((int)(b_real + b_rw + (exphormer ? 1 : 0)), 1);
  TORCH_CHECK(ell_col.is_cuda() && ell_col.scalar_type() == torch::kInt && ell_col.is_contiguous() &&
              ell_col.numel() >= row_count * cap && ell_cnt.scalar_type() == torch::kInt && ell_cnt.numel() >= row_count);
  TORCH_CHECK(!exphormer || (ell_type.has_value() && ell_type->scalar_type() == torch::kUInt8 && ell_type->numel() >= row_count * cap));
  TORCH_CHECK(totals.scalar_type() == torch::kLong && totals.numel() >= 2);
  c10::cuda::CUDAGuard guard(in_src.device());
  totals.zero_();
  bf_build_params p{};
  p.in_rowptr = iptr(in_rowptr); p.in_src = iptr(in_src); p.out_rowptr = iptr(out_rowptr); p.out_col = iptr(out_col);
  p.n = (int)n; p.b_real = (int)b_real; p.b_rw = (int)b_rw; p.walks = (int)walks; p.walk_len = (int)walk_len;
  p.exphormer = exphormer ? 1 : 0; p.seed = seed; p.cap = cap;
  p.ell_col = ell_col.data_ptr<int>(); p.ell_type = exphormer ? ell_type->data_ptr<uint8_t>() : nullptr;
  p.ell_cnt = ell_cnt.data_ptr<int>();
  p.totals = reinterpret_cast<unsigned long long*>(totals.data_ptr<int64_t>());
  p.row_begin = (int)row_begin; p.row_count = (int)row_count;
  Tensor hub_top = attach_hub_rows(p, hub_rows, in_src);
  check_cuda(bf_budget_select(&p, at::cuda::getCurrentCUDAStream()), "budget_select_rows");
}

// Fixed-width rows of all n queries -> CSR (rowptr, col, etype or empty): prefix sum of the counts, one host read of
// the edge count, compaction.
std::vector<Tensor> ell_rows_to_csr(Tensor ell_col, Tensor ell_cnt, OptTensor ell_type, int64_t n, int64_t cap) {
  TORCH_CHECK(ell_col.is_cuda() && ell_col.scalar_type() == torch::kInt && ell_col.is_contiguous() && ell_col.numel() >= n * cap);
  TORCH_CHECK(ell_cnt.scalar_type() == torch::kInt && ell_cnt.is_contiguous() && ell_cnt.numel() >= n);
  c10::cuda::CUDAGuard guard(ell_col.device());
  auto iopt = ell_col.options();
  const bool typed = ell_type.has_value();
  Tensor rowptr = torch::zeros({n + 1}, iopt);
  rowptr.slice(0, 1).copy_(torch::cumsum(ell_cnt.slice(0, 0, n), 0, torch::kInt));
  const int64_t n_edges = n > 0 ? rowptr[n].item<int64_t>() : 0;
  Tensor col = torch::empty({n_edges}, iopt);
  Tensor etype = typed ? torch::empty({n_edges}, iopt.dtype(torch::kUInt8)) : torch::empty({0}, iopt.dtype(torch::kUInt8));
  check_cuda(bf_ell_to_csr(ell_col.data_ptr<int>(), typed ? ell_type->data_ptr<uint8_t>() : nullptr, rowptr.data_ptr<int>(),
                           (int)n, (int)cap, col.data_ptr<int>(), typed ? etype.data_ptr<uint8_t>() : nullptr,
                           at::cuda::getCurrentCUDAStream()), "ell_to_csr");
  return {rowptr, col, etype};
}

// dst[r * n + i] = src_r[i]: the shards of all ranks (n elements of dst's dtype each), fetched with peer loads and laid
// end to end.
void peer_concat(std::vector<int64_t> src, int64_t n_elem, Tensor dst) {
  c10::cuda::CUDAGuard guard(dst.device());
  TORCH_CHECK(dst.is_contiguous() && dst.numel() >= (int64_t)src.size() * n_elem && src.size() <= BF_MAX_PEERS, "peer_concat: bad sizes");
  std::vector<void*> p(BF_MAX_PEERS, nullptr);
  for (size_t i = 0; i < src.size(); ++i) p[i] = reinterpret_cast<void*>(src[i]);
  check_cuda(bf_peer_concat(p.data(), (int)src.size(), n_elem, (int)dst.element_size(), dst.data_ptr(),
                            at::cuda::getCurrentCUDAStream()), "peer_concat");
}

// General CPU build (rows of any length; a negative budget keeps every candidate of that side; an empty fan-out
// list selects Philox walks).  Same outputs as build_attn_graph.
std::vector<Tensor> build_attn_graph_rows_cpu(Tensor in_rowptr, Tensor in_src, Tensor out_rowptr, Tensor out_col,
                                              int64_t n, int64_t b_real, int64_t b_rw, bool use_real, bool use_rw,
                                              int64_t walks, int64_t walk_len, std::vector<int64_t> fanout,
                                              bool exphormer, int64_t seed, int64_t num_threads, int64_t row_begin,
                                              int64_t row_end) {
  for (const Tensor* t : {&in_rowptr, &in_src, &out_rowptr, &out_col})
    TORCH_CHECK(!t->is_cuda() && t->scalar_type() == torch::kInt && t->is_contiguous(), "int32 contiguous CPU CSR expected");
  std::vector<int> fo(fanout.begin(), fanout.end());
  if (row_end < 0) row_end = n;                       // default: every query
  TORCH_CHECK(0 <= row_begin && row_begin <= row_end && row_end <= n, "bad row range");
  const int64_t rows = row_end - row_begin;
  Tensor counts = torch::zeros({rows}, torch::kLong);
  Tensor totals = torch::zeros({2}, torch::kLong);
  auto run = [&](const long long* offsets, int* col, uint8_t* etype) {
    bf_build_rows_cpu(iptr(in_rowptr), iptr(in_src), iptr(out_rowptr), iptr(out_col), (int)row_begin, (int)row_end,
                      (int)b_real, (int)b_rw,
                      use_real ? 1 : 0, use_rw ? 1 : 0, (int)walks, (int)walk_len, fo.data(), (int)fo.size(),
                      exphormer ? 1 : 0, seed, offsets, reinterpret_cast<long long*>(counts.data_ptr<int64_t>()), col, etype,
                      reinterpret_cast<unsigned long long*>(totals.data_ptr<int64_t>()), (int)num_threads);
  };
  run(nullptr, nullptr, nullptr);
  Tensor incl = torch::cumsum(counts, 0);
  const int64_t n_edges = rows > 0 ? incl[rows - 1].item<int64_t>() : 0;
  TORCH_CHECK(n_edges < (int64_t)INT32_MAX, "attention graph too large for int32 offsets: ", n_edges, " edges");
  Tensor offsets = (incl - counts).contiguous();
  auto iopt = torch::TensorOptions().dtype(torch::kInt);
  Tensor col = torch::empty({n_edges}, iopt);
  Tensor etype = exphormer ? torch::empty({n_edges}, iopt.dtype(torch::kUInt8)) : torch::empty({0}, iopt.dtype(torch::kUInt8));
  run(reinterpret_cast<const long long*>(offsets.data_ptr<int64_t>()), col.data_ptr<int>(),
      exphormer ? etype.data_ptr<uint8_t>() : nullptr);
  Tensor rowptr = torch::zeros({rows + 1}, iopt);
  rowptr.slice(0, 1).copy_(incl.to(torch::kInt));
  return {rowptr, col, etype, totals};
}

// Part id per node of a symmetric int32 CPU CSR; second tensor = number of nodes the refinement moved.
std::vector<Tensor> partition_cpu(Tensor rowptr, Tensor col, int64_t n, int64_t k, double imbalance, int64_t passes) {
  TORCH_CHECK(!rowptr.is_cuda() && !col.is_cuda() && rowptr.scalar_type() == torch::kInt &&
              col.scalar_type() == torch::kInt && rowptr.is_contiguous() && col.is_contiguous());
  TORCH_CHECK(rowptr.numel() == n + 1 && k >= 1);
  Tensor part = torch::zeros({n}, torch::kInt);
  const long long moved = bf_partition_cpu(iptr(rowptr), iptr(col), (int)n, (int)k, (float)imbalance, (int)passes,
                                           part.data_ptr<int>());
  TORCH_CHECK(moved >= 0, "bf_partition_cpu: bad arguments");
  return {part, torch::tensor((int64_t)moved, torch::kLong)};
}

// (src, dst) int64 candidates of the fan-out k-hop expansion over a CPU out-edge CSR.
std::vector<Tensor> khop_candidates_cpu(Tensor out_rowptr, Tensor out_col, int64_t n, std::vector<int64_t> fanout,
                                        int64_t seed, int64_t num_threads) {
  TORCH_CHECK(!out_rowptr.is_cuda() && !out_col.is_cuda() && out_rowptr.scalar_type() == torch::kInt &&
              out_col.scalar_type() == torch::kInt && out_rowptr.is_contiguous() && out_col.is_contiguous());
  std::vector<int> fo(fanout.begin(), fanout.end());
  Tensor counts = torch::zeros({n}, torch::kLong);
  bf_khop_count_cpu(iptr(out_rowptr), iptr(out_col), (int)n, fo.data(), (int)fo.size(), seed,
                    reinterpret_cast<long long*>(counts.data_ptr<int64_t>()), (int)num_threads);
  Tensor incl = torch::cumsum(counts, 0);
  const int64_t total = n > 0 ? incl[n - 1].item<int64_t>() : 0;
  Tensor offsets = incl - counts;
  Tensor src = torch::empty({total}, torch::kLong), dst = torch::empty({total}, torch::kLong);
  bf_khop_fill_cpu(iptr(out_rowptr), iptr(out_col), (int)n, fo.data(), (int)fo.size(), seed,
                   reinterpret_cast<const long long*>(offsets.data_ptr<int64_t>()),
                   reinterpret_cast<long long*>(src.data_ptr<int64_t>()),
                   reinterpret_cast<long long*>(dst.data_ptr<int64_t>()), (int)num_threads);
  return {src, dst};
}

// By-key view + balanced dK/dV work list of a device-resident attention graph.
// Returns (t_rowptr [n+1], t_row [E], t_eid [E], tasks [T, 4], splits [S, 3], sizes int64 [3] = T, slots, S on the host).
std::vector<Tensor> graph_transpose(Tensor rowptr, Tensor col, int64_t n, int64_t chunk) {
  TORCH_CHECK(rowptr.is_cuda() && col.is_cuda() && rowptr.scalar_type() == torch::kInt && col.scalar_type() == torch::kInt);
  TORCH_CHECK(rowptr.is_contiguous() && col.is_contiguous() && rowptr.numel() == n + 1 && chunk >= 1);
  c10::cuda::CUDAGuard guard(col.device());
  auto st = at::cuda::getCurrentCUDAStream();
  auto iopt = col.options();
  const int64_t n_edges = col.numel();
  Tensor t_rowptr = torch::empty({n + 1}, iopt), t_row = torch::empty({n_edges}, iopt), t_eid = torch::empty({n_edges}, iopt);
  {
    const size_t bytes = bf_graph_transpose_scratch((int)n, n_edges);
    Tensor scratch = torch::empty({(int64_t)bytes}, iopt.dtype(torch::kUInt8));
    check_cuda(bf_graph_transpose(rowptr.data_ptr<int>(), col.data_ptr<int>(), (int)n, n_edges, t_rowptr.data_ptr<int>(),
                                  t_row.data_ptr<int>(), t_eid.data_ptr<int>(), scratch.data_ptr(), bytes, st),
               "graph_transpose");
  }
  Tensor firsts = torch::empty({3, n + 1}, iopt);
  {
    const size_t bytes = bf_kv_task_scratch((int)n);
    Tensor scratch = torch::empty({(int64_t)bytes}, iopt.dtype(torch::kUInt8));
    check_cuda(bf_kv_task_counts(t_rowptr.data_ptr<int>(), (int)n, (int)chunk, firsts[0].data_ptr<int>(),
                                 firsts[1].data_ptr<int>(), firsts[2].data_ptr<int>(), scratch.data_ptr(), bytes, st),
               "kv_task_counts");
  }
  // the three totals size the outputs: the one host read of this build
  Tensor sizes = firsts.select(1, n).to(torch::kCPU).to(torch::kLong);
  const int64_t n_tasks = sizes[0].item<int64_t>(), n_splits = sizes[2].item<int64_t>();
  Tensor tasks = torch::empty({n_tasks, 4}, iopt), splits = torch::empty({n_splits, 3}, iopt);
  check_cuda(bf_kv_task_fill(t_rowptr.data_ptr<int>(), firsts[0].data_ptr<int>(), firsts[1].data_ptr<int>(),
                             firsts[2].data_ptr<int>(), (int)n, (int)chunk, tasks.data_ptr<int>(),
                             splits.data_ptr<int>(), st),
             "kv_task_fill");
  return {t_rowptr, t_row, t_eid, tasks, splits, sizes};
}

// C = A * W^T with fused epilogue.  `dst_ptrs` holds one device pointer per destination (1 = plain output).
void gemm_tn(Tensor A, Tensor W, OptTensor bias, int64_t act, double dropout_p, int64_t seed, OptTensor residual,
             OptTensor relu_mask, double out_scale, bool out_fp32, std::vector<int64_t> dst_ptrs, int64_t dst_row_offset,
             int64_t ldc, Tensor status, OptTensor relu_bits_out, OptTensor relu_bits_in, int64_t mask_mode) {
  TORCH_CHECK(A.is_cuda() && W.is_cuda() && A.dim() == 2 && W.dim() == 2, "gemm_tn: A [M,K], W [N,K] on CUDA");
  TORCH_CHECK(A.scalar_type() == W.scalar_type() && (A.scalar_type() == torch::kBFloat16 || A.scalar_type() == torch::kHalf),
              "gemm_tn: bf16/fp16 operands");
  TORCH_CHECK(A.stride(1) == 1 && W.stride(1) == 1 && A.size(1) == W.size(1), "gemm_tn: K-contiguous operands");
  TORCH_CHECK(status.is_cuda() && status.scalar_type() == torch::kInt && status.numel() >= 4);
  TORCH_CHECK(!dst_ptrs.empty() && (int)dst_ptrs.size() <= BF_MAX_PEERS);
  c10::cuda::CUDAGuard guard(A.device());
  bf_gemm_params p{};
  p.A = A.data_ptr(); p.B = W.data_ptr(); p.lda = A.stride(0); p.ldb = W.stride(0);
  p.M = (int)A.size(0); p.N = (int)W.size(0); p.K = (int)A.size(1);
  p.dtype = dtype_code(A);
  if (bias.has_value()) {
    TORCH_CHECK(bias->scalar_type() == torch::kFloat && bias->is_contiguous() && bias->numel() == p.N &&
                ((uintptr_t)bias->data_ptr()) % 16 == 0, "gemm_tn: bias must be contiguous fp32 [N], 16-byte aligned");
    p.bias = bias->data_ptr<float>();
  }
  p.act = (int)act; p.dropout_p = (float)dropout_p; p.dropout_seed = (uint32_t)seed;
  if (residual.has_value()) {
    TORCH_CHECK(residual->scalar_type() == A.scalar_type() && residual->stride(1) == 1 && residual->size(0) == p.M &&
                residual->size(1) == p.N && dst_ptrs.size() == 1);
    TORCH_CHECK(((uintptr_t)residual->data_ptr()) % 16 == 0 && (residual->stride(0) * 2) % 16 == 0,
                "gemm_tn: residual rows must be 16-byte aligned");
    p.residual = residual->data_ptr(); p.ldr = residual->stride(0);
  }
  for (const OptTensor* bt : {&relu_bits_out, &relu_bits_in}) {
    if (!bt->has_value()) continue;
    const Tensor& t = **bt;
    TORCH_CHECK(t.is_cuda() && t.scalar_type() == torch::kShort && t.dim() == 2 && t.stride(1) == 1 && t.size(1) == p.M &&
                t.size(0) * 16 == p.N, "gemm_tn: ReLU bit mask must be int16 [N / 16, M]");
    p.ldmb = t.stride(0);
  }
  if (relu_bits_out.has_value()) p.relu_bits_out = relu_bits_out->data_ptr();
  if (relu_bits_in.has_value()) p.relu_bits_in = relu_bits_in->data_ptr();
  if (relu_mask.has_value()) {
    TORCH_CHECK(relu_mask->scalar_type() == A.scalar_type() && relu_mask->stride(1) == 1 && relu_mask->size(0) == p.M &&
                relu_mask->size(1) == p.N && (relu_mask->stride(0) * 2) % 16 == 0 && ((uintptr_t)relu_mask->data_ptr()) % 16 == 0);
    p.relu_mask = relu_mask->data_ptr(); p.ldm = relu_mask->stride(0);
    TORCH_CHECK(mask_mode == 0 || mask_mode == 1, "gemm_tn: mask_mode 0 (ReLU gradient) or 1 (GELU gradient)");
    p.mask_mode = (int)mask_mode;
  }
  p.out_scale = (float)out_scale; p.out_fp32 = out_fp32 ? 1 : 0;
  p.n_dest = (int)dst_ptrs.size(); p.dst_row_offset = dst_row_offset; p.ldc = ldc;
  TORCH_CHECK((ldc * (out_fp32 ? 4 : 2)) % 16 == 0, "gemm_tn: destination rows must be 16-byte aligned");
  for (size_t i = 0; i < dst_ptrs.size(); ++i) {
    TORCH_CHECK(((uintptr_t)dst_ptrs[i]) % 16 == 0);
    p.dst[i] = reinterpret_cast<void*>(dst_ptrs[i]);
  }
  p.status = status.data_ptr<int>();
  TORCH_CHECK(bf_gemm_supported(p.M, p.N, p.K), "gemm_tn: unsupported shape M=", p.M, " N=", p.N, " K=", p.K);
  check_cuda(bf_gemm_tn(&p, at::cuda::getCurrentCUDAStream()), "gemm_tn");
}

// C = gathered(A) @ W^T with the A operand pulled from `src_ptrs` (peer mappings) inside the GEMM; see bf_gemm_params.
void gemm_tn_pull(std::vector<int64_t> src_ptrs, int64_t src_row_offset, int64_t src_ld, int64_t cols_per_src, int64_t M,
                  Tensor W, OptTensor a_copy, OptTensor bias, double dropout_p, int64_t seed, OptTensor residual,
                  double out_scale, Tensor out, Tensor status) {
  TORCH_CHECK(W.is_cuda() && W.dim() == 2 && W.stride(1) == 1 &&
              (W.scalar_type() == torch::kBFloat16 || W.scalar_type() == torch::kHalf), "gemm_tn_pull: W [N,K] 16-bit on CUDA");
  TORCH_CHECK(src_ptrs.size() >= 2 && (int)src_ptrs.size() <= BF_MAX_PEERS, "gemm_tn_pull: 2..", BF_MAX_PEERS, " sources");
  TORCH_CHECK((int64_t)src_ptrs.size() * cols_per_src == W.size(1), "gemm_tn_pull: sources x columns must equal K");
  TORCH_CHECK(out.is_cuda() && out.dim() == 2 && out.stride(1) == 1 && out.size(0) == M && out.size(1) == W.size(0) &&
              out.scalar_type() == W.scalar_type(), "gemm_tn_pull: out [M,N] in the operand dtype");
  TORCH_CHECK(status.is_cuda() && status.scalar_type() == torch::kInt && status.numel() >= 4);
  c10::cuda::CUDAGuard guard(W.device());
  bf_gemm_params p{};
  p.B = W.data_ptr(); p.ldb = W.stride(0);
  p.M = (int)M; p.N = (int)W.size(0); p.K = (int)W.size(1);
  p.dtype = dtype_code(W);
  p.n_src = (int)src_ptrs.size(); p.cols_per_src = (int)cols_per_src; p.src_row_offset = src_row_offset; p.src_ld = src_ld;
  for (size_t i = 0; i < src_ptrs.size(); ++i) p.src[i] = reinterpret_cast<const void*>(src_ptrs[i]);
  if (a_copy.has_value()) {
    TORCH_CHECK(a_copy->is_cuda() && a_copy->dim() == 2 && a_copy->stride(1) == 1 && a_copy->size(0) == M &&
                a_copy->size(1) == W.size(1) && a_copy->scalar_type() == W.scalar_type(), "gemm_tn_pull: a_copy [M,K]");
    p.a_copy = a_copy->data_ptr(); p.ld_copy = a_copy->stride(0);
  }
  if (bias.has_value()) {
    TORCH_CHECK(bias->scalar_type() == torch::kFloat && bias->is_contiguous() && bias->numel() == p.N &&
                ((uintptr_t)bias->data_ptr()) % 16 == 0, "gemm_tn_pull: bias must be contiguous fp32 [N], 16-byte aligned");
    p.bias = bias->data_ptr<float>();
  }
  p.dropout_p = (float)dropout_p; p.dropout_seed = (uint32_t)seed;
  if (residual.has_value()) {
    TORCH_CHECK(residual->scalar_type() == W.scalar_type() && residual->stride(1) == 1 && residual->size(0) == M &&
                residual->size(1) == p.N && ((uintptr_t)residual->data_ptr()) % 16 == 0 && (residual->stride(0) * 2) % 16 == 0,
                "gemm_tn_pull: residual [M,N], 16-byte aligned rows");
    p.residual = residual->data_ptr(); p.ldr = residual->stride(0);
  }
  p.out_scale = (float)out_scale;
  p.n_dest = 1; p.ldc = out.stride(0); p.dst[0] = out.data_ptr();
  TORCH_CHECK((p.ldc * 2) % 16 == 0 && ((uintptr_t)p.dst[0]) % 16 == 0, "gemm_tn_pull: output rows must be 16-byte aligned");
  p.status = status.data_ptr<int>();
  check_cuda(bf_gemm_tn(&p, at::cuda::getCurrentCUDAStream()), "gemm_tn_pull");
}

// y = [x +] drop2(act(x W1^T + b1) W2^T + b2) with the hidden tile kept on chip (no autograd: forward-only uses)
Tensor ffn_fused_fwd(Tensor x, Tensor w1, OptTensor b1, Tensor w2, OptTensor b2, int64_t act, bool residual, double p1,
                     int64_t seed1, double p2, int64_t seed2, Tensor status, OptTensor h_out, OptTensor relu_bits_out) {
  TORCH_CHECK(x.is_cuda() && x.dim() == 2 && x.stride(1) == 1 &&
              (x.scalar_type() == torch::kBFloat16 || x.scalar_type() == torch::kHalf), "ffn_fused_fwd: x [M, h] 16-bit on CUDA");
  TORCH_CHECK(w1.is_cuda() && w2.is_cuda() && w1.is_contiguous() && w2.is_contiguous() && w1.scalar_type() == x.scalar_type() &&
              w2.scalar_type() == x.scalar_type() && w1.dim() == 2 && w2.dim() == 2 && w1.size(1) == x.size(1) &&
              w2.size(0) == x.size(1) && w2.size(1) == w1.size(0), "ffn_fused_fwd: W1 [f, h], W2 [h, f] contiguous in the dtype of x");
  TORCH_CHECK(bf_ffn_fused_supported(x.size(0), (int)x.size(1), (int)w1.size(0)), "ffn_fused_fwd: unsupported shape");
  TORCH_CHECK(status.is_cuda() && status.scalar_type() == torch::kInt && status.numel() >= 4);
  c10::cuda::CUDAGuard guard(x.device());
  Tensor y = torch::empty({x.size(0), x.size(1)}, x.options());
  bf_ffn_params p{};
  p.X = x.data_ptr(); p.Y = y.data_ptr(); p.ldx = x.stride(0); p.ldy = y.stride(0);
  p.W1 = w1.data_ptr(); p.W2 = w2.data_ptr();
  for (const OptTensor* bt : {&b1, &b2}) {
    if (!bt->has_value()) continue;
    TORCH_CHECK((*bt)->scalar_type() == torch::kFloat && (*bt)->is_contiguous() && ((uintptr_t)(*bt)->data_ptr()) % 16 == 0,
                "ffn_fused_fwd: biases must be contiguous fp32, 16-byte aligned");
  }
  TORCH_CHECK(!b1.has_value() || b1->numel() == w1.size(0));
  TORCH_CHECK(!b2.has_value() || b2->numel() == w2.size(0));
  p.b1 = b1.has_value() ? b1->data_ptr<float>() : nullptr;
  p.b2 = b2.has_value() ? b2->data_ptr<float>() : nullptr;
  p.M = x.size(0); p.hidden = (int)x.size(1); p.ffn = (int)w1.size(0);
  p.dtype = dtype_code(x); p.act = (int)act;
  p.dropout1 = (float)p1; p.dropout2 = (float)p2; p.seed1 = (uint32_t)seed1; p.seed2 = (uint32_t)seed2;
  p.residual = residual ? 1 : 0;
  p.status = status.data_ptr<int>();
  if (h_out.has_value()) {
    TORCH_CHECK(h_out->is_cuda() && h_out->dim() == 2 && h_out->stride(1) == 1 && h_out->size(0) == x.size(0) &&
                h_out->size(1) == w1.size(0) && h_out->scalar_type() == x.scalar_type(), "ffn_fused_fwd: h_out [M, f] in the dtype of x");
    p.H_out = h_out->data_ptr(); p.ldh = h_out->stride(0);
  }
  if (relu_bits_out.has_value()) {
    const Tensor& t = *relu_bits_out;
    TORCH_CHECK(t.is_cuda() && t.scalar_type() == torch::kShort && t.dim() == 2 && t.stride(1) == 1 && t.size(1) == x.size(0) &&
                t.size(0) * 16 == w1.size(0), "ffn_fused_fwd: ReLU bit mask must be int16 [f / 16, M]");
    p.relu_bits_out = t.data_ptr(); p.ldmb = t.stride(0);
  }
  check_cuda(bf_ffn_fused_fwd(&p, at::cuda::getCurrentCUDAStream()), "ffn_fused_fwd");
  return y;
}

// dW = dY^T X (fp32 [N, K]) and, with `want_bias`, the column sums of dY (fp32 [N]) from the same kernel.
std::vector<Tensor> gemm_dw(Tensor dY, Tensor X, bool want_bias, Tensor status) {
  TORCH_CHECK(dY.is_cuda() && X.is_cuda() && dY.dim() == 2 && X.dim() == 2 && dY.size(0) == X.size(0), "gemm_dw: dY [M,N], X [M,K]");
  TORCH_CHECK(dY.scalar_type() == X.scalar_type() && (dY.scalar_type() == torch::kBFloat16 || dY.scalar_type() == torch::kHalf),
              "gemm_dw: bf16/fp16 operands");
  TORCH_CHECK(dY.stride(1) == 1 && X.stride(1) == 1, "gemm_dw: feature-contiguous operands");
  c10::cuda::CUDAGuard guard(dY.device());
  bf_gemm_dw_params p{};
  p.dY = dY.data_ptr(); p.X = X.data_ptr(); p.ldy = dY.stride(0); p.ldx = X.stride(0);
  p.M = dY.size(0); p.N = (int)dY.size(1); p.K = (int)X.size(1);
  p.dtype = dtype_code(dY);
  TORCH_CHECK(bf_gemm_dw_supported(p.M, p.N, p.K), "gemm_dw: unsupported shape");
  TORCH_CHECK(!want_bias || bf_gemm_dw_bias_supported(p.K), "gemm_dw: bias gradient not available for K = ", p.K);
  auto f32 = torch::TensorOptions().dtype(torch::kFloat).device(dY.device());
  Tensor dW = torch::empty({p.N, p.K}, f32);
  Tensor db = want_bias ? torch::empty({p.N}, f32) : Tensor();
  Tensor scratch = torch::empty({(int64_t)(bf_gemm_dw_scratch_bytes(p.M, p.N, p.K) / 4)}, f32);
  p.dW = dW.data_ptr<float>();
  p.dbias = want_bias ? db.data_ptr<float>() : nullptr;
  p.scratch = scratch.data_ptr();
  p.status = status.data_ptr<int>();
  check_cuda(bf_gemm_dw(&p, at::cuda::getCurrentCUDAStream()), "gemm_dw");
  if (want_bias) return {dW, db};
  return {dW};
}

bool gemm_dw_supported(int64_t M, int64_t N, int64_t K, bool want_bias) {
  return bf_gemm_dw_supported(M, (int)N, (int)K) != 0 && (!want_bias || bf_gemm_dw_bias_supported((int)K) != 0);
}

std::vector<void*> as_ptrs(const std::vector<int64_t>& v) {
  std::vector<void*> o(BF_MAX_PEERS, nullptr);
  TORCH_CHECK(v.size() <= BF_MAX_PEERS, "at most ", BF_MAX_PEERS, " peers");
  for (size_t i = 0; i < v.size(); ++i) o[i] = reinterpret_cast<void*>(v[i]);
  return o;
}

void peer_barrier(std::vector<int64_t> flag_pages, int64_t rank, int64_t channel, int64_t epoch, Tensor status) {
  c10::cuda::CUDAGuard guard(status.device());
  auto p = as_ptrs(flag_pages);
  check_cuda(bf_peer_barrier(p.data(), (int)rank, (int)flag_pages.size(), (int)channel, (uint32_t)epoch,
                             status.data_ptr<int>(), at::cuda::getCurrentCUDAStream()), "peer_barrier");
}

// norm_scratch / norm_parts: optional by-product, see bf_allreduce_mean (pass an empty list and None to skip it).
void allreduce_mean(std::vector<int64_t> bufs, int64_t multicast_ptr, int64_t rank, int64_t n_floats, Tensor anchor,
                    OptTensor norm_scratch, std::vector<int64_t> norm_parts) {
  c10::cuda::CUDAGuard guard(anchor.device());
  auto p = as_ptrs(bufs);
  const bool with_norm = norm_scratch.has_value() && !norm_parts.empty();
  std::vector<void*> parts;
  if (with_norm) {
    TORCH_CHECK(norm_parts.size() == bufs.size() && norm_scratch->scalar_type() == torch::kFloat && norm_scratch->is_contiguous() &&
                norm_scratch->numel() >= bf_allreduce_mean_grid(n_floats, (int)bufs.size()) + 1, "allreduce_mean: norm scratch too small");
    parts = as_ptrs(norm_parts);
  }
  check_cuda(bf_allreduce_mean(p.data(), reinterpret_cast<float*>(multicast_ptr), (int)rank, (int)bufs.size(), n_floats,
                               with_norm ? norm_scratch->data_ptr<float>() : nullptr, with_norm ? parts.data() : nullptr,
                               at::cuda::getCurrentCUDAStream()), "allreduce_mean");
}

void peer_gather_cols(std::vector<int64_t> src, int64_t row0, int64_t rows, int64_t cols_bytes, int64_t src_ld_bytes,
                      Tensor dst) {
  c10::cuda::CUDAGuard guard(dst.device());
  TORCH_CHECK(dst.dim() == 2 && dst.stride(1) == 1 && dst.size(0) >= rows);
  auto p = as_ptrs(src);
  check_cuda(bf_peer_gather_cols(p.data(), (int)src.size(), row0, rows, (int)cols_bytes, src_ld_bytes, dst.data_ptr(),
                                 dst.stride(0) * dst.element_size(), at::cuda::getCurrentCUDAStream()), "peer_gather_cols");
}

void peer_scatter_cols(std::vector<int64_t> dstp, int64_t row0, int64_t rows, int64_t cols_bytes, int64_t dst_ld_bytes,
                       Tensor src) {
  c10::cuda::CUDAGuard guard(src.device());
  TORCH_CHECK(src.dim() == 2 && src.stride(1) == 1 && src.size(0) >= rows);
  auto p = as_ptrs(dstp);
  check_cuda(bf_peer_scatter_cols(p.data(), (int)dstp.size(), row0, rows, (int)cols_bytes, dst_ld_bytes, src.data_ptr(),
                                  src.stride(0) * src.element_size(), at::cuda::getCurrentCUDAStream()), "peer_scatter_cols");
}

std::vector<Tensor> layernorm_fwd(Tensor x, Tensor gamma, Tensor beta, double eps) {
  TORCH_CHECK(x.is_cuda() && x.dim() == 2 && x.stride(1) == 1);
  c10::cuda::CUDAGuard guard(x.device());
  Tensor y = torch::empty({x.size(0), x.size(1)}, x.options());
  Tensor stats = torch::empty({x.size(0), 2}, x.options().dtype(torch::kFloat));
  check_cuda(bf_layernorm_fwd(x.data_ptr(), x.stride(0), gamma.data_ptr<float>(), beta.data_ptr<float>(), y.data_ptr(),
                              y.stride(0), stats.data_ptr<float>(), x.size(0), (int)x.size(1), (float)eps, dtype_code(x),
                              at::cuda::getCurrentCUDAStream()), "layernorm_fwd");
  return {y, stats};
}

std::vector<Tensor> layernorm_bwd(Tensor dy, Tensor x, Tensor stats, Tensor gamma, bool want_dxsum) {
  TORCH_CHECK(dy.is_cuda() && dy.dim() == 2 && dy.stride(1) == 1 && x.stride(1) == 1 && dy.scalar_type() == x.scalar_type());
  c10::cuda::CUDAGuard guard(x.device());
  Tensor dx = torch::empty({x.size(0), x.size(1)}, x.options());
  Tensor dgamma = torch::zeros({x.size(1)}, x.options().dtype(torch::kFloat));
  Tensor dbeta = torch::zeros({x.size(1)}, x.options().dtype(torch::kFloat));
  const int64_t h = x.size(1);
  const bool wide = x.scalar_type() != torch::kFloat && (h == 64 || h == 128 || h == 256) &&
                    (dy.stride(0) * 2) % 16 == 0 && (x.stride(0) * 2) % 16 == 0 &&
                    ((uintptr_t)dy.data_ptr()) % 16 == 0 && ((uintptr_t)x.data_ptr()) % 16 == 0;
  Tensor dxsum;
  if (want_dxsum && wide) dxsum = torch::zeros({h}, x.options().dtype(torch::kFloat));
  check_cuda(bf_layernorm_bwd(dy.data_ptr(), dy.stride(0), x.data_ptr(), x.stride(0), stats.data_ptr<float>(),
                              gamma.data_ptr<float>(), dx.data_ptr(), dx.stride(0), dgamma.data_ptr<float>(),
                              dbeta.data_ptr<float>(), dxsum.defined() ? dxsum.data_ptr<float>() : nullptr,
                              x.size(0), (int)h, dtype_code(x), at::cuda::getCurrentCUDAStream()), "layernorm_bwd");
  if (want_dxsum && !wide) dxsum = dx.sum(0, /*keepdim=*/false, torch::kFloat);
  if (want_dxsum) return {dx, dgamma, dbeta, dxsum};
  return {dx, dgamma, dbeta};
}

Tensor colsum(Tensor x) {
  TORCH_CHECK(x.is_cuda() && x.dim() == 2 && x.stride(1) == 1);
  c10::cuda::CUDAGuard guard(x.device());
  Tensor out = torch::zeros({x.size(1)}, x.options().dtype(torch::kFloat));
  check_cuda(bf_colsum(x.data_ptr(), x.stride(0), x.size(0), (int)x.size(1), out.data_ptr<float>(), dtype_code(x),
                       at::cuda::getCurrentCUDAStream()), "colsum");
  return out;
}

// (sum (x - shift), sum (x - shift)^2) per column, fp32
std::vector<Tensor> bn_stats(Tensor x, OptTensor shift) {
  TORCH_CHECK(x.is_cuda() && x.dim() == 2 && x.stride(1) == 1);
  c10::cuda::CUDAGuard guard(x.device());
  auto fopt = x.options().dtype(torch::kFloat);
  Tensor s1 = torch::zeros({x.size(1)}, fopt), s2 = torch::zeros({x.size(1)}, fopt);
  check_cuda(bf_bn_stats(x.data_ptr(), x.stride(0), shift.has_value() ? shift->data_ptr<float>() : nullptr, x.size(0),
                         (int)x.size(1), s1.data_ptr<float>(), s2.data_ptr<float>(), dtype_code(x),
                         at::cuda::getCurrentCUDAStream()), "bn_stats");
  return {s1, s2};
}

// (sum dy, sum dy * (x - mean) * rstd) per column, fp32
std::vector<Tensor> bn_bwd_reduce(Tensor dy, Tensor x, Tensor mean, Tensor rstd) {
  TORCH_CHECK(x.is_cuda() && x.dim() == 2 && x.stride(1) == 1 && dy.stride(1) == 1 && dy.scalar_type() == x.scalar_type());
  c10::cuda::CUDAGuard guard(x.device());
  auto fopt = x.options().dtype(torch::kFloat);
  Tensor dbeta = torch::zeros({x.size(1)}, fopt), dgamma = torch::zeros({x.size(1)}, fopt);
  check_cuda(bf_bn_bwd_reduce(dy.data_ptr(), dy.stride(0), x.data_ptr(), x.stride(0), mean.data_ptr<float>(),
                              rstd.data_ptr<float>(), x.size(0), (int)x.size(1), dbeta.data_ptr<float>(),
                              dgamma.data_ptr<float>(), dtype_code(x), at::cuda::getCurrentCUDAStream()), "bn_bwd_reduce");
  return {dbeta, dgamma};
}

// y = x*a + b, or y = in2*a + x*b + c0 when in2 is given (per-column fp32 coefficients)
Tensor col_affine(Tensor x, OptTensor in2, Tensor a, Tensor b, OptTensor c0) {
  TORCH_CHECK(x.is_cuda() && x.dim() == 2 && x.stride(1) == 1);
  TORCH_CHECK(in2.has_value() == c0.has_value());
  c10::cuda::CUDAGuard guard(x.device());
  Tensor y = torch::empty({x.size(0), x.size(1)}, x.options());
  check_cuda(bf_col_affine(x.data_ptr(), x.stride(0), in2.has_value() ? in2->data_ptr() : nullptr,
                           in2.has_value() ? in2->stride(0) : 0, a.data_ptr<float>(), b.data_ptr<float>(),
                           c0.has_value() ? c0->data_ptr<float>() : nullptr, y.data_ptr(), y.stride(0), x.size(0),
                           (int)x.size(1), dtype_code(x), at::cuda::getCurrentCUDAStream()), "col_affine");
  return y;
}

Tensor hash_dropout(Tensor x, int64_t seed, double p) {
  TORCH_CHECK(x.is_cuda() && x.dim() == 2 && x.stride(1) == 1);
  c10::cuda::CUDAGuard guard(x.device());
  Tensor y = torch::empty({x.size(0), x.size(1)}, x.options());
  check_cuda(bf_hash_dropout(x.data_ptr(), x.stride(0), y.data_ptr(), y.stride(0), x.size(0), (int)x.size(1),
                             (uint32_t)seed, (float)p, dtype_code(x), at::cuda::getCurrentCUDAStream()), "hash_dropout");
  return y;
}

// dropout(gelu(x), p) in one pass (the FFN's GELU path); p = 0 gives plain GELU
Tensor gelu_dropout(Tensor x, int64_t seed, double p) {
  TORCH_CHECK(x.is_cuda() && x.dim() == 2 && x.stride(1) == 1 && p >= 0.0 && p < 1.0);
  c10::cuda::CUDAGuard guard(x.device());
  Tensor y = torch::empty({x.size(0), x.size(1)}, x.options());
  check_cuda(bf_gelu_dropout(x.data_ptr(), x.stride(0), y.data_ptr(), y.stride(0), x.size(0), (int)x.size(1),
                             (uint32_t)seed, (float)p, dtype_code(x), at::cuda::getCurrentCUDAStream()), "gelu_dropout");
  return y;
}

void grad_sumsq(Tensor g, Tensor out) {
  TORCH_CHECK(g.is_cuda() && g.scalar_type() == torch::kFloat && g.is_contiguous() && out.scalar_type() == torch::kFloat);
  c10::cuda::CUDAGuard guard(g.device());
  check_cuda(bf_grad_sumsq(g.data_ptr<float>(), g.numel(), out.data_ptr<float>(), at::cuda::getCurrentCUDAStream()), "grad_sumsq");
}

void adamw_flat(Tensor p, Tensor g, Tensor m, Tensor v, int64_t n, double lr, double beta1, double beta2, double eps,
                double wd, int64_t step, OptTensor sumsq, double max_norm) {
  for (const Tensor* t : {&p, &g, &m, &v})
    TORCH_CHECK(t->is_cuda() && t->scalar_type() == torch::kFloat && t->is_contiguous() && t->numel() >= n);
  c10::cuda::CUDAGuard guard(p.device());
  check_cuda(bf_adamw_flat(p.data_ptr<float>(), g.data_ptr<float>(), m.data_ptr<float>(), v.data_ptr<float>(), n, (float)lr,
                           (float)beta1, (float)beta2, (float)eps, (float)wd, (int)step,
                           sumsq.has_value() ? sumsq->data_ptr<float>() : nullptr, sumsq.has_value() ? (int)sumsq->numel() : 0,
                           (float)max_norm, at::cuda::getCurrentCUDAStream()), "adamw_flat");
}

void adamw_flat_dev(Tensor p, Tensor g, Tensor m, Tensor v, int64_t n, double beta1, double beta2, double eps, double wd,
                    Tensor hyper, OptTensor sumsq, double max_norm) {
  for (const Tensor* t : {&p, &g, &m, &v, &hyper})
    TORCH_CHECK(t->is_cuda() && t->scalar_type() == torch::kFloat && t->is_contiguous());
  TORCH_CHECK(p.numel() >= n && g.numel() >= n && m.numel() >= n && v.numel() >= n && hyper.numel() >= 3);
  c10::cuda::CUDAGuard guard(p.device());
  check_cuda(bf_adamw_flat_dev(p.data_ptr<float>(), g.data_ptr<float>(), m.data_ptr<float>(), v.data_ptr<float>(), n,
                               (float)beta1, (float)beta2, (float)eps, (float)wd, hyper.data_ptr<float>(),
                               sumsq.has_value() ? sumsq->data_ptr<float>() : nullptr,
                               sumsq.has_value() ? (int)sumsq->numel() : 0, (float)max_norm,
                               at::cuda::getCurrentCUDAStream()), "adamw_flat_dev");
}

// Returns (loss_sum [1] fp32, dlogits or empty).
std::vector<Tensor> nll_fwd_bwd(Tensor logits, Tensor y, Tensor mask, bool want_grad, double grad_scale) {
  TORCH_CHECK(logits.is_cuda() && logits.dim() == 2 && logits.stride(1) == 1);
  TORCH_CHECK(y.scalar_type() == torch::kLong && y.is_contiguous() && mask.scalar_type() == torch::kUInt8 && mask.is_contiguous());
  TORCH_CHECK(y.numel() == logits.size(0) && mask.numel() == logits.size(0));
  c10::cuda::CUDAGuard guard(logits.device());
  Tensor loss = torch::zeros({1}, logits.options().dtype(torch::kFloat));
  Tensor d = want_grad ? torch::empty({logits.size(0), logits.size(1)}, logits.options()) : Tensor();
  check_cuda(bf_nll_fwd_bwd(logits.data_ptr(), logits.stride(0), reinterpret_cast<const long long*>(y.data_ptr<int64_t>()), mask.data_ptr<uint8_t>(), logits.size(0),
                            (int)logits.size(1), loss.data_ptr<float>(), want_grad ? d.data_ptr() : nullptr, (float)grad_scale,
                            dtype_code(logits), at::cuda::getCurrentCUDAStream()), "nll_fwd_bwd");
  return {loss, want_grad ? d : torch::empty({0}, logits.options())};
}

bool gemm_supported(int64_t M, int64_t N, int64_t K) { return bf_gemm_supported((int)M, (int)N, (int)K) != 0; }

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("edge_attn_fwd", &edge_attn_fwd);
  m.def("edge_attn_bwd", &edge_attn_bwd);
  m.attr("BUILD_HUB_DEGREE") = (int64_t)BF_BUILD_HUB_DEGREE;
  m.def("build_attn_graph", &build_attn_graph);
  m.def("budget_select_rows", &budget_select_rows);
  m.def("ell_rows_to_csr", &ell_rows_to_csr);
  m.def("peer_concat", &peer_concat);
  m.def("khop_candidates_cpu", &khop_candidates_cpu);
  m.def("partition_cpu", &partition_cpu);
  m.def("build_attn_graph_rows_cpu", &build_attn_graph_rows_cpu);
  m.def("graph_transpose", &graph_transpose);
  m.def("gemm_tn", &gemm_tn);
  m.def("gemm_tn_pull", &gemm_tn_pull);
  m.def("gemm_dw", &gemm_dw);
  m.def("ffn_fused_fwd", &ffn_fused_fwd);
  m.def("ffn_fused_supported", [](int64_t M, int64_t h, int64_t f) { return bf_ffn_fused_supported(M, (int)h, (int)f) != 0; });
  m.def("gemm_dw_supported", &gemm_dw_supported);
  m.def("gemm_supported", &gemm_supported);
  m.def("layernorm_fwd", &layernorm_fwd);
  m.def("layernorm_bwd", &layernorm_bwd);
  m.def("hash_dropout", &hash_dropout);
  m.def("gelu_dropout", &gelu_dropout);
  m.def("bn_stats", &bn_stats);
  m.def("bn_bwd_reduce", &bn_bwd_reduce);
  m.def("col_affine", &col_affine);
  m.def("colsum", &colsum);
  m.def("nll_fwd_bwd", &nll_fwd_bwd);
  m.def("grad_sumsq", &grad_sumsq);
  m.def("adamw_flat", &adamw_flat);
  m.def("adamw_flat_dev", &adamw_flat_dev);
  m.def("peer_barrier", &peer_barrier);
  m.def("allreduce_mean", &allreduce_mean);
  m.def("allreduce_mean_grid", [](int64_t n_floats, int64_t world) { return (int64_t)bf_allreduce_mean_grid(n_floats, (int)world); });
  m.def("peer_gather_cols", &peer_gather_cols);
  m.def("peer_scatter_cols", &peer_scatter_cols);
}
