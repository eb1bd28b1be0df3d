// C interface of the sm_100a kernels.  Every launcher takes raw device pointers and a stream,
// allocates nothing and returns a cudaError_t value (0 = success) unless stated otherwise, so the
// same entry points serve the PyTorch bindings (bindings.cpp) and callers that own their memory.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define BF_BF16 0
#define BF_FP16 1
#define BF_FP32 2

#define BF_MAX_PEERS 8
#define BF_FLAG_CHANNELS 64      // barrier channels per flag page (uint32[BF_FLAG_CHANNELS][BF_MAX_PEERS])

#define BF_HUB_DEGREE 1024   // rows longer than this use the chunked hub kernels
#define BF_HUB_CHUNK 8192    // edges per hub chunk (one thread block)

// ---- edge attention (edge_attn.cu) ----------------------------------------------------------
typedef struct {
  const void *q, *k, *v;            // [n, hl, hn], inner two dims contiguous, row strides in elements
  long long ldq, ldk, ldv;
  void* out;                        // [n, hl, hn] contiguous
  float* z;                         // [n, hl] softmax normaliser
  const int* rowptr;                // [n+1] CSR over queries
  const int* col;                   // [E] key ids
  const uint8_t* etype;             // [E] or NULL
  const float* etab;                // [2, hl, hn] fp32 or NULL (Exphormer edge-type table)
  int n, hl, hn, dtype, variant;    // variant: 0 plain, 1 gps, 2 exphormer
  float dropout_p;
  uint32_t dropout_seed;
  const int* hub_rows;              // rows with degree > BF_HUB_DEGREE (may be NULL when n_hub == 0)
  int n_hub, max_hub_degree;
  float* hub_scratch;               // zero-filled [n_hub, hl*hn + hl] fp32
  // Optional dropout on the attention output, fused into the store (0 = off).  The keep decision of element
  // (row, c) is that of bf_hash_dropout / the GEMM epilogue for (row % out_rows_local, out_col0 + c): the context
  // rows a rank computes are consumed by the rank owning them, at this rank's column offset.  The backward pass
  // reads the stored (dropped, rescaled) output and rescales <dout, out> by (1 - p).
  float out_dropout_p;
  uint32_t out_dropout_seed;
  int out_rows_local;               // rows per owning rank (0 = n)
  int out_col0;                     // column offset of this rank's head slice in the owner's row
} bf_attn_params;

// Result rows delivered to the rank that owns the node (sequence parallelism: the heads->nodes all-to-all done by the
// stores of the attention kernels).  Destination d = row / rows_per holds one slab of rows_per rows per source rank:
// row lands at base[d] + ((slab_row0 + row - d * rows_per) * ld + column) elements.  n_dest == 0: off.
typedef struct {
  void* base[BF_MAX_PEERS];         // 16-byte aligned buffer base per destination (peer mappings)
  int n_dest;                       // n_dest * rows_per must equal the row count of the call
  int rows_per;
  long long ld;                     // destination row stride in elements, a multiple of 8
  long long slab_row0;              // this (source) rank's slab: source index * rows_per
} bf_attn_route;

typedef struct {
  const void* dout;                 // [n, hl, hn] contiguous
  void *dq, *dk, *dv;               // [n, hl, hn], common row stride ldg (elements; 0 = hl*hn)
  long long ldg;
  float* zd;                        // [n, hl, 2] fp32 workspace (written by the dQ pass)
  const int *t_rowptr, *t_row, *t_eid;  // transposed CSR over keys
  float* detab;                     // zero-filled [2, hl, hn] fp32 or NULL
  const int* t_hub_rows;
  int n_t_hub, max_t_hub_degree;
  float* hub_scratch_q;             // zero-filled [n_hub, hl*hn]
  float* hub_scratch_kv;            // zero-filled [n_t_hub, 2*hl*hn]
  // Optional balanced dK/dV work list (replaces the t_hub_* path when kv_task != NULL)
  const int* kv_task;               // [n_kv_task, 4] int32, 16-byte aligned: key row, first edge, end edge, slot (-1 direct)
  int n_kv_task;
  const int* kv_split;              // [n_kv_split, 3] int32: key row, first slot, slot count
  int n_kv_split;
  float* kv_partial;                // [total slots, 2*hl*hn] fp32 scratch
  // Optional workspace for narrow rows (hl*hn elements of 64 bytes or less), used with kv_task: the dQ pass leaves one
  // contiguous record [q | dout / (Z + eps)] per (row, head) in qg and D / (Z + eps) in cz, and the dK/dV pass gathers
  // those instead of q, dout and zd separately.
  void* qg;                         // [n, hl, 2, hn] in the operand dtype, or NULL
  float* cz;                        // [n, hl] fp32, or NULL
  // Optional: dq / dk / dv rows go to the owner of each row (route.n_dest > 0) at column offsets route_cq / _ck / _cv
  // (multiples of 8) of the destination's row, instead of into dq / dk / dv
  bf_attn_route route;
  int route_cq, route_ck, route_cv;
} bf_attn_bwd_params;

int bf_edge_attn_fwd(const bf_attn_params* p, cudaStream_t st);
// as above; additionally every output row is stored into its owner's buffer (route may be NULL)
int bf_edge_attn_fwd_routed(const bf_attn_params* p, const bf_attn_route* route, cudaStream_t st);
int bf_edge_attn_bwd(const bf_attn_params* p, const bf_attn_bwd_params* q, cudaStream_t st);

// ---- attention-graph construction (edge_build.cu) -------------------------------------------
typedef struct {
  const int *in_rowptr, *in_src;    // CSR over destinations (multiplicity kept)
  const int *out_rowptr, *out_col;  // coalesced CSR over sources (random walks)
  int n;
  int b_real, b_rw;                 // per-query budgets, each in [0, 32]
  int walks, walk_len;              // W walks of length L (L <= 16) from every node
  int exphormer;                    // 1: typed rows (real 0 | walk 1 | self 0) without dedup
  long long seed;                   // epoch seed; +17 ranks real edges, +37 ranks walk edges
  int cap;                          // row capacity >= b_real + b_rw (+1 for exphormer)
  int* ell_col;                     // [n, cap]
  uint8_t* ell_type;                // [n, cap] (exphormer) or NULL
  int* ell_cnt;                     // [n]
  unsigned long long* totals;       // zero-filled [2]: selected real / walk edges
  // Optional row range (row_count > 0): only the queries [row_begin, row_begin + row_count) are built and their rows are
  // stored at index (query - row_begin) of ell_col / ell_type / ell_cnt - one rank's shard of a build that the
  // sequence-parallel ranks split between them.  row_count == 0 builds all n queries.
  int row_begin, row_count;
  // Optional list of the queries whose in-edge row is longer than BF_BUILD_HUB_DEGREE (ascending ids, n_hub of them) and
  // scratch of 32 * n_hub 64-bit words: those rows are ranked by one thread block each before the row-per-lane-group
  // kernel runs, which then reads the ranked list instead of streaming the row.  Same rows out either way; queries
  // missing from the list are streamed as before.
  const int* hub_rows;
  int n_hub;
  unsigned long long* hub_top;
} bf_build_params;

#define BF_BUILD_HUB_DEGREE 4096

int bf_budget_select(const bf_build_params* p, cudaStream_t st);
int bf_ell_to_csr(const int* ell_col, const uint8_t* ell_type, const int* rowptr, int n, int cap, int* col,
                  uint8_t* etype, cudaStream_t st);

// ---- feed-forward block with the hidden tile kept on chip (ffn_fused_tcgen05.cu) ----------------
typedef struct {
  const void* X;                    // [M, hidden] 16-bit, row stride ldx (elements)
  void* Y;                          // [M, hidden] 16-bit, row stride ldy
  long long ldx, ldy;
  const void* W1;                   // [ffn, hidden] contiguous (nn.Linear layout)
  const void* W2;                   // [hidden, ffn] contiguous
  const float* b1;                  // [ffn] fp32 or NULL
  const float* b2;                  // [hidden] fp32 or NULL
  long long M;
  int hidden, ffn;                  // supported: 128 / 256 (bf_ffn_fused_supported)
  int dtype;                        // BF_BF16 or BF_FP16
  int act;                          // 1 ReLU, 2 GELU (erf)
  float dropout1, dropout2;         // on the hidden tile / on the output before the residual; masks = hash(seed, row, col)
  uint32_t seed1, seed2;
  int residual;                     // 1: Y = X + ...
  int* status;                      // [4] device status words (0 = ok)
  // Optional (training forward): the hidden matrix after activation and dropout, written from the on-chip operand, and
  // one bit per hidden element (value > 0) in the layout of bf_gemm_params.relu_bits_out
  void* H_out;                      // [M, ffn] 16-bit, row stride ldh (elements), or NULL
  long long ldh;
  void* relu_bits_out;              // uint16 [ffn / 16, ldmb >= M] or NULL
  long long ldmb;
} bf_ffn_params;

int bf_ffn_fused_supported(long long M, int hidden, int ffn);
int bf_ffn_fused_fwd(const bf_ffn_params* p, cudaStream_t st);

// ---- tcgen05 GEMM with fused epilogue / fused nodes->heads all-to-all (gemm_tcgen05.cu) ---------
typedef struct {
  const void* A;                    // [M, K] 16-bit, row stride lda (elements)
  const void* B;                    // [N, K] 16-bit (nn.Linear weight layout), row stride ldb
  long long lda, ldb;
  int M, N, K;                      // K % 64 == 0, N % 16 == 0
  int dtype;                        // BF_BF16 or BF_FP16
  const float* bias;                // [N] fp32 or NULL
  int act;                          // 0 none, 1 ReLU, 2 GELU (erf)
  float dropout_p;                  // after the activation; mask = hash(seed, row, col)
  uint32_t dropout_seed;
  const void* residual;             // [M, ldr] 16-bit added last, or NULL
  long long ldr;
  const void* relu_mask;            // [M, ldm] 16-bit: result zeroed where mask <= 0, or NULL
  long long ldm;
  int mask_mode;                    // 0: as above (ReLU gradient); 1: result *= gelu'(mask), mask = the pre-activation
  // The same mask as one bit per element, 16 columns per uint16 word, stored column-block major ([N/16, ldmb >= M]
  // words, so that the 32 rows of a warp touch adjacent words; N % 16 == 0): written by a
  // forward GEMM (bit = result > 0 after activation and dropout), consumed by the backward GEMM instead of re-reading
  // the 16-bit activation.
  void* relu_bits_out;
  const void* relu_bits_in;
  long long ldmb;
  float out_scale;                  // multiplies the accumulator (0 means 1)
  int out_fp32;                     // 1: fp32 output
  int n_dest;                       // >1: columns [d*N/n_dest, (d+1)*N/n_dest) go to dst[d] (peer buffers)
  long long dst_row_offset;         // added to the row index in every destination
  long long ldc;                    // destination row stride (elements)
  void* dst[BF_MAX_PEERS];
  int* status;                      // device int[4]; non-zero after a bounded wait expired
  // Gathered A operand (n_src > 1; A / lda are then ignored and K = n_src * cols_per_src): columns
  // [s * cols_per_src, (s + 1) * cols_per_src) of row r are row (src_row_offset + r) of src[s], a 16-bit matrix with
  // row stride src_ld (elements) that may live in another GPU's memory (peer mapping).  cols_per_src % 16 == 0.
  int n_src;
  int cols_per_src;
  const void* src[BF_MAX_PEERS];
  long long src_row_offset;
  long long src_ld;
  void* a_copy;                     // optional local [M, K] matrix (row stride ld_copy) that receives the gathered operand
  long long ld_copy;
} bf_gemm_params;

int bf_gemm_supported(int M, int N, int K);
int bf_gemm_tn(const bf_gemm_params* p, cudaStream_t st);

// ---- tcgen05 weight-gradient GEMM (gemm_dw_tcgen05.cu) ----------------------------------------------
// dW[N, K] (= or +=) scale * dY[M, N]^T X[M, K]; dbias[N] (= or +=) scale * column sums of dY (optional).
typedef struct {
  const void* dY;                   // [M, N] 16-bit, row stride ldy (elements), 16-byte aligned rows
  const void* X;                    // [M, K] 16-bit, row stride ldx
  long long ldy, ldx;
  long long M;
  int N, K;                         // both multiples of 8
  int dtype;                        // BF_BF16 or BF_FP16
  float* dW;                        // [N, K] fp32 contiguous
  float* dbias;                     // [N] fp32 or NULL; needs bf_gemm_dw_bias_supported(K)
  int accumulate;                   // 0: overwrite, 1: add to what dW / dbias hold
  float scale;                      // 0 means 1
  void* scratch;                    // bf_gemm_dw_scratch_bytes(M, N, K) bytes of device memory
  int* status;                      // device int[4]; non-zero after a bounded wait expired
} bf_gemm_dw_params;

int bf_gemm_dw_supported(long long M, int N, int K);
int bf_gemm_dw_bias_supported(int K);
size_t bf_gemm_dw_scratch_bytes(long long M, int N, int K);
int bf_gemm_dw(const bf_gemm_dw_params* p, cudaStream_t st);

// ---- peer-memory collectives (symm_comm.cu) ----------------------------------------------------
// `flag_pages[r]` / `bufs[r]` are this process's mappings of rank r's symmetric allocation.
int bf_peer_barrier(void* const* flag_pages, int rank, int world, int channel, uint32_t epoch, int* status,
                    cudaStream_t st);
// In-place mean over ranks of a symmetric fp32 buffer.  Optional gradient-norm by-product (both NULL = off):
// norm_scratch = local float[bf_allreduce_mean_grid(n_floats, world) + 1], zero before the first use;
// norm_parts[r] = rank r's float[world] array (symmetric): slot `rank` of every array receives the sum of squares of the
// slice this rank reduced, so after the collective every rank holds the `world` slice totals of the averaged buffer.
int bf_allreduce_mean_grid(long long n_floats, int world);
int bf_allreduce_mean(void* const* bufs, float* multicast_ptr, int rank, int world, long long n_floats,
                      float* norm_scratch, void* const* norm_parts, cudaStream_t st);
int bf_peer_gather_cols(void* const* src, int world, long long row0, long long rows, int cols_bytes,
                        long long src_ld_bytes, void* dst, long long dst_ld_bytes, cudaStream_t st);
int bf_peer_scatter_cols(void* const* dst, int world, long long row0, long long rows, int cols_bytes,
                         long long dst_ld_bytes, const void* src, long long src_ld_bytes, cudaStream_t st);
// dst[r * n_elem + i] = src[r][i] for every rank r: equal-length shards fetched with peer loads and laid end to end.
int bf_peer_concat(void* const* src, int world, long long n_elem, int elem_bytes /* 1, 4 or 8 */, void* dst, cudaStream_t st);

// Balanced k-way partition of a symmetric CSR (cpu/partition.cpp: BFS ordering + boundary refinement); returns the
// number of nodes the refinement moved, or -1 on bad arguments.
long long bf_partition_cpu(const int* rowptr, const int* col, int n, int k, float imbalance, int refine_passes, int* part);
// Fan-out k-hop candidate expansion on the CPU (cpu/edge_builder.cpp): two passes, count then fill.
int bf_khop_count_cpu(const int* out_rowptr, const int* out_col, int n, const int* fanout, int n_hops, long long seed,
                      long long* counts /* [n] */, int num_threads);
int bf_khop_fill_cpu(const int* out_rowptr, const int* out_col, int n, const int* fanout, int n_hops, long long seed,
                     const long long* offsets /* [n] exclusive prefix sums */, long long* src, long long* dst,
                     int num_threads);

// ---- by-key view of the attention graph + dK/dV work list (graph_transpose.cu) --------------------------
size_t bf_graph_transpose_scratch(int n, long long n_edges);
int bf_graph_transpose(const int* rowptr, const int* col, int n, long long n_edges, int* t_rowptr /* [n+1] */,
                       int* t_row /* [E] */, int* t_eid /* [E] */, void* scratch, size_t scratch_bytes, cudaStream_t st);
size_t bf_kv_task_scratch(int n);
int bf_kv_task_counts(const int* t_rowptr, int n, int chunk, int* item_first /* [n+1] */, int* slot_first /* [n+1] */,
                      int* split_first /* [n+1] */, void* scratch, size_t scratch_bytes, cudaStream_t st);
int bf_kv_task_fill(const int* t_rowptr, const int* item_first, const int* slot_first, const int* split_first, int n,
                    int chunk, int* tasks /* [T, 4] */, int* splits /* [S, 3] */, cudaStream_t st);

// ---- row kernels (norm_fused.cu) -----------------------------------------------------------------
int bf_layernorm_fwd(const void* x, long long ldx, const float* gamma, const float* beta, void* y, long long ldy,
                     float* stats /* [rows, 2] mean, rstd or NULL */, long long rows, int h, float eps, int dtype,
                     cudaStream_t st);
int bf_layernorm_bwd(const void* dy, long long lddy, const void* x, long long ldx, const float* stats,
                     const float* gamma, void* dx, long long lddx, float* dgamma /* += */, float* dbeta /* += */,
                     float* dxsum /* += column sums of dx, or NULL; 16-bit rows of 64/128/256 columns only */,
                     long long rows, int h, int dtype, cudaStream_t st);
int bf_colsum(const void* x, long long ldx, long long rows, int cols /* % 8 == 0 */, float* out /* += */, int dtype,
              cudaStream_t st);
int bf_hash_dropout(const void* x, long long ldx, void* y, long long ldy, long long rows, int cols, uint32_t seed,
                    float p, int dtype, cudaStream_t st);
int bf_gelu_dropout(const void* x, long long ldx, void* y, long long ldy, long long rows, int cols, uint32_t seed,
                    float p, int dtype, cudaStream_t st);

// BatchNorm building blocks (cols % 8 == 0, 16-byte aligned rows): shifted one-pass statistics, the backward
// reductions, and per-column affine maps y = x*a + b / y = in2*a + x*b + c0 (in2 == NULL selects the first form).
int bf_bn_stats(const void* x, long long ldx, const float* shift /* [cols] or NULL */, long long rows, int cols,
                float* s1 /* += sum (x - shift) */, float* s2 /* += sum (x - shift)^2 */, int dtype, cudaStream_t st);
int bf_bn_bwd_reduce(const void* dy, long long lddy, const void* x, long long ldx, const float* mean, const float* rstd,
                     long long rows, int cols, float* dbeta /* += */, float* dgamma /* += */, int dtype, cudaStream_t st);
int bf_col_affine(const void* x, long long ldx, const void* in2, long long ld2, const float* a, const float* b,
                  const float* c0, void* y, long long ldy, long long rows, int cols, int dtype, cudaStream_t st);

// ---- optimizer on flat fp32 buckets (optim.cu) -----------------------------------------------------
int bf_grad_sumsq(const float* g, long long n, float* out /* += sum g^2 */, cudaStream_t st);
// sumsq: n_sumsq floats whose sum is the squared global gradient norm (one float from bf_grad_sumsq, or the per-rank
// slice totals left by bf_allreduce_mean), or NULL for no clipping.
int bf_adamw_flat(float* p, const float* g, float* m, float* v, long long n, float lr, float beta1, float beta2,
                  float eps, float weight_decay, int step, const float* sumsq /* or NULL */, int n_sumsq, float max_norm,
                  cudaStream_t st);
// Graph-capturable form: hyper = device float[3] {lr, 1 - beta1^t, sqrt(1 - beta2^t)} refreshed by the host each step.
int bf_adamw_flat_dev(float* p, const float* g, float* m, float* v, long long n, float beta1, float beta2, float eps,
                      float weight_decay, const float* hyper, const float* sumsq, int n_sumsq, float max_norm,
                      cudaStream_t st);

// ---- readout loss (loss.cu) ---------------------------------------------------------------------------
// loss_sum += sum over rows with mask != 0 of -log softmax(logits[row])[y[row]]; when dlogits != NULL it receives
// (softmax - onehot) * grad_scale on those rows and zeros elsewhere (contiguous [rows, classes]).
int bf_nll_fwd_bwd(const void* logits, long long ld, const long long* y, const uint8_t* mask, long long rows, int classes,
                   float* loss_sum, void* dlogits, float grad_scale, int dtype, cudaStream_t st);

#ifdef __cplusplus
}
#endif
