/*
 * matris_b200 — C ABI of the B200 (sm_100a) evaluation path for MatRIS.
 *
 * Plain C: raw device pointers and sizes, int status returns, no C++/torch types.
 * Every entry point launches on the CUDA stream passed as its last argument
 * (a cudaStream_t passed as void*; NULL = default stream) on the CURRENT device.
 * The library owns no device memory: every buffer is allocated by the caller.
 * Unless stated otherwise calls are asynchronous and return MB_OK as soon as the
 * launches are queued.
 *
 * Each declaration cites the reference code it replaces (paths are relative to
 * the reference project root).
 */
#ifndef MATRIS_B200_H
#define MATRIS_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MB_VERSION 1

/* status codes */
#define MB_OK 0
#define MB_ERR_INVALID 1   /* bad argument (null pointer, negative size, unsupported shape) */
#define MB_ERR_CUDA 2      /* a CUDA runtime call failed; see mb_last_cuda_error() */
#define MB_ERR_OVERFLOW 3  /* a count exceeds int32 or an image index exceeds +-127 */
#define MB_ERR_UNPAIRED 4  /* a directed edge has no reverse edge (bond exactly on the cutoff) */
#define MB_ERR_ISOLATED 5  /* an atom has no neighbour inside the cutoff */
#define MB_ERR_TOO_LARGE 6 /* problem exceeds the fixed capacity of an allocation-free entry point */
#define MB_ERR_CAPACITY 7  /* a caller-supplied capacity buffer is too small; the needed sizes are in counts[] */

int mb_version(void);
const char* mb_status_string(int status);
const char* mb_last_cuda_error(void);

/* ------------------------------------------------------------------ graph build
 * Replaces, for a whole batch of structures at once,
 *   Structure.get_neighbor_list call        matris/graph/converter.py:85-87
 *   create_graph (C) / Graph.add_edge       matris/graph/fast_converter_libraries/create_graph.c:100-219,
 *                                           matris/graph/radiusgraph.py:298-386
 *   adjacency_list / undirected2directed    matris/graph/radiusgraph.py:388-410, 489-496
 *   line_graph_adjacency_list               matris/graph/radiusgraph.py:412-487
 *   index offsetting of process_graphs      matris/model/processgraph.py:93-166
 *
 * All indices are global over the batch (atom, directed-edge, bond and triplet
 * numbering runs through all structures in order).  Directed edges come out
 * sorted by (centre, neighbour, image); bonds are numbered by their first
 * directed edge; triplets are grouped by target bond.  This is exactly what the
 * reference's Graph produces when fed a neighbour list in that order.
 *
 * One asynchronous call: mb_graph_build queues ONE cooperative kernel and returns; it never synchronises.  The
 * caller supplies capacity buffers (cap_edges directed edges, cap_triplets triplets) and a device status block
 * `counts`; after the stream has reached the call it holds
 *   counts[0] directed edges, [1] bonds, [2] triplets (the sizes actually needed, also when a capacity was too
 *   small), [3] isolated atoms, [4] image index outside +-127, [5] unpaired edges, [6] edge capacity too small,
 *   [7] triplet capacity too small, [8] triplets counted by source bond (must equal [2]), [9] candidate list
 *   unusable (Verlet-skin reuse, below).
 * Copy the 16 ints to the host together with whatever else the caller reads back and pass them to mb_graph_status,
 * which maps them to a status code; on MB_ERR_CAPACITY enlarge the buffers to counts[0] / counts[2] and call again
 * (in a molecular-dynamics loop the previous step's counts plus a margin make that rare).
 *
 * Neighbour-list reuse with a Verlet skin (the reference rebuilds from scratch at every step,
 * matris/applications/base.py:96-97; the graphs here are identical to a rebuild, only cheaper to get):
 *   1. a CANDIDATE build: the same call with cutoff + skin, flags = MB_GRAPH_EDGES_ONLY (it stops after the sorted
 *      directed-edge list; the pairing / line-graph scratch and outputs may be NULL) and its own status block;
 *      with run_if set it runs only when *run_if != 0, so it can be queued at every step;
 *   2. every step: mb_graph_skin_check sets a flag when an atom is half the skin or more away from where it was at
 *      the last candidate build; the candidate build is queued with run_if = flag; mb_graph_skin_commit then
 *      records the positions (and clears the flag) if it ran; the step's graph is a build with cand_ptr / cand_nbr /
 *      cand_img = edge_ptr / neighbor / image of the candidate build and cand_counts = its status block: the cell
 *      search is replaced by a distance test of the candidates (same expression, same order: bit-identical edges).
 *      If the candidate build did not succeed, counts[9] is set and nothing else is written (status
 *      MB_ERR_CAPACITY: enlarge the candidate buffers, set the flag, repeat).
 *   Nothing in this sequence synchronises with the host; lattices must not change between candidate builds.
 */
#define MB_GRAPH_EDGES_ONLY 1
typedef struct mb_graph {
  /* sizes and parameters (host) */
  int32_t n_atoms, n_struct, n_cells;
  int32_t cap_edges, cap_triplets, flags;      /* capacities of the edge / triplet buffers below; MB_GRAPH_* bits */
  double cutoff, line_cutoff, tol;             /* tol < d <= cutoff ; line graph: target d <= lc, source d < lc */
  /* inputs (device) */
  const double* cart;         /* [n_atoms,3] Cartesian, not wrapped */
  const double* lattice;      /* [n_struct,3,3] rows = cell vectors */
  const double* inv_lattice;  /* [n_struct,3,3] inverse of the above (frac = cart @ inv) */
  const int32_t* atom_struct; /* [n_atoms] structure index of each atom (non-decreasing) */
  const int32_t* grid;        /* [n_struct,8]: cells per axis g0,g1,g2; search half-width in cells s0,s1,s2;
                                 first global cell index; unused */
  /* scratch (device) */
  int32_t* cell_ptr;          /* [n_cells+1] */
  int32_t* cell_fill;         /* [n_cells] */
  int32_t* cell_atoms;        /* [n_atoms] */
  int32_t* atom_cell;         /* [n_atoms,4] */
  int32_t* atom_wrap;         /* [n_atoms,4] */
  int32_t* scan_tmp;          /* [mb_graph_scan_tmp_len(max(n_atoms, n_cells, cap_edges))] */
  int32_t* counts;            /* [16] device status block, see above */
  uint64_t* key_unsorted;     /* [cap_edges] */
  double* dist_unsorted;      /* [cap_edges] */
  uint64_t* key;              /* [cap_edges] */
  int32_t* atom_counts;       /* [n_atoms,2] source- / target-eligible out-edge counts */
  int32_t* edge_rank;         /* [2*cap_edges+2] */
  int32_t* bond_counts;       /* [cap_edges+4] */
  uint8_t* edge_flag;         /* [cap_edges] bit0: may be a triplet target, bit1: may be a triplet source */
  /* outputs (device) */
  int32_t* edge_ptr;          /* [n_atoms+1] CSR of directed edges by centre atom */
  int32_t* center;            /* [cap_edges] */
  int32_t* neighbor;          /* [cap_edges] */
  int32_t* image;             /* [cap_edges,3] */
  double* dist;               /* [cap_edges] float64 bond lengths used for the membership tests */
  int32_t* rev;               /* [cap_edges] index of the reverse directed edge */
  int32_t* d2u;               /* [cap_edges] directed -> bond */
  int32_t* u2d;               /* [cap_edges/2] bond -> its first directed edge */
  int32_t* trip_ptr;          /* [cap_edges/2+1] CSR of triplets by target bond */
  int32_t* trip_src_ptr;      /* [cap_edges/2+1] CSR of triplets by source bond */
  int32_t* line_graph;        /* [cap_triplets,5] rows (centre atom, target bond, target DE, source bond, source DE) */
  int32_t* trip_src_perm;     /* [cap_triplets] triplet ids grouped by source bond (see trip_src_ptr) */
  /* Verlet-skin reuse (device; all NULL for a plain build) */
  const int32_t* run_if;      /* [1] when non-NULL and zero at launch time the call does nothing */
  const int32_t* cand_ptr;    /* [n_atoms+1] candidate CSR by centre atom ... */
  const int32_t* cand_nbr;    /* [candidates] ... neighbour atom ... */
  const int32_t* cand_img;    /* [candidates,3] ... and image; sorted by (neighbour, image) within an atom */
  const int32_t* cand_counts; /* [16] status block of the build that produced the candidates */
} mb_graph;

size_t mb_graph_scan_tmp_len(int64_t n);
int mb_graph_build(const mb_graph* g, void* stream);
/* status code of a build from the host copy of counts[16]: MB_OK, MB_ERR_ISOLATED, MB_ERR_OVERFLOW (image index or
 * a count beyond int32), MB_ERR_CAPACITY, MB_ERR_UNPAIRED */
int mb_graph_status(const int32_t* counts_host);
/* flag[0] |= 1 if any atom is >= half_skin away from cart_ref (flag is int32[2]; flag[1] counts candidate rebuilds) */
int mb_graph_skin_check(int32_t n_atoms, const double* cart, const double* cart_ref, double half_skin, int32_t* flag,
                        void* stream);
/* if flag[0]: cart_ref = cart, flag[0] = 0, flag[1] += 1.  Queue it after the conditional candidate build. */
int mb_graph_skin_commit(int32_t n_atoms, const double* cart, double* cart_ref, int32_t* flag, void* stream);

/* ------------------------------------------------------------------ dense row GEMM
 * out[r, 128*j + n] = epilogue( sum_k A_j[r, k] * W_j[n, k] )        j = 0..n_blocks-1
 *
 * The one contraction kernel behind every 128-wide linear layer of the model
 * (nn.Linear calls in matris/model/functions.py:112-126,157 via MLP / GatedMLP,
 * matris/model/interaction_block.py:96-137, 232-273, matris/model/feature_embed.py,
 * matris/model/readout.py) and behind their data-gradient products in the backward
 * pass (the reference gets those from torch.autograd).  A_j is the concatenation
 * of up to four 128-wide row segments, each optionally gathered through an index
 * (this is the torch.cat([... index_select ...]) of interaction_block.py:96-108,
 * 232-250 without materialising it) and optionally passed through SiLU on load.
 * Epilogue, in order: + bias, * silu'(gate), SiLU, + res_w * res, * out_scale,
 * then store / accumulate / atomic scatter-add through out_idx.
 */
typedef struct mb_src {
  const float* ptr;      /* rows of >= 128 floats starting at column `col` */
  const int32_t* idx;    /* optional gather index per output row (NULL: row r) */
  int64_t ld;            /* row stride in floats */
  int32_t col;           /* first column (multiple of 4) */
  int32_t act;           /* 0: as is, 1: SiLU applied on load */
} mb_src;

#define MB_OUT_STORE 0
#define MB_OUT_ADD 1      /* non-atomic read-modify-write (each destination row written once) */
#define MB_OUT_ATOMIC 2   /* atomic add (destination rows may repeat) */

typedef struct mb_colblock {
  int32_t n_src;               /* 1..4 ; K = 128 * n_src */
  int32_t out_act;             /* 0 none, 1 SiLU */
  mb_src src[4];
  const float* W;              /* [128, K] row-major: weight rows of this column block */
  const float* W_hi;           /* tf32(W), same layout (3xTF32 modes 2, 3; NULL allowed otherwise) */
  const float* W_lo;           /* W - tf32(W), same layout */
  const uint16_t* W_hi16;      /* bf16(W), same layout in 16-bit elements (3xBF16, mode 0; NULL allowed otherwise) */
  const uint16_t* W_lo16;      /* bf16(W - bf16(W)) */
  int64_t ldw;                 /* row stride of W and of every split, in elements (>= K; a multiple of 8 in mode 0) */
  const float* bias;           /* [128] or NULL */
  const float* gate;           /* optional pre-activation z: multiply by d/dz SiLU(z) */
  int64_t ld_gate; int32_t col_gate; int32_t pad0;
  const float* res;            /* optional residual rows */
  const float* res_w;          /* [128] per-channel residual weight (NULL: 1) */
  int64_t ld_res; int32_t col_res; int32_t mode;
  float* out; const int32_t* out_idx;
  int64_t ld_out; int32_t col_out; float out_scale;
} mb_colblock;

typedef struct mb_gemm_desc {
  int64_t n_rows;
  int32_t n_blocks;            /* 1..4 column blocks of 128 outputs */
  int32_t pad;
  mb_colblock blk[4];
} mb_gemm_desc;

int mb_gemm(const mb_gemm_desc* desc, void* stream);
/* Contraction core used by mb_gemm and mb_gated_mlp_fwd.  Every tensor-core core splits both operands into hi + lo
 * and accumulates lo*hi + hi*lo + hi*hi in fp32 tensor memory:
 *   0 (default) persistent kernels, one CTA per SM, 3xBF16: hi = bf16(x), lo = bf16(x - hi), kind::f16 MMAs at twice
 *               the tf32 rate; an operand pair carries 16 mantissa bits;
 *   3           the persistent GEMM kernel with 3xTF32: hi = x cut to tf32, lo = x - hi, kind::tf32 MMAs; 22 mantissa bits;
 *   2           3xTF32 in a one-tile-per-CTA kernel;
 *   1           fp32 SIMT FMA (bit-faithful fp32, the cross-check).
 * A test knob: it is process-wide and not meant to be switched while other host threads launch.
 * MB_OUT_ADD is performed as one memory-side fp32 addition per element in mode 0 (read-add-write in modes 1, 2):
 * identical results as long as no other kernel writes the output rows concurrently. */
int mb_set_gemm_mode(int mode);
/* Status word of the tensor-core kernels on the CURRENT device (bit 0: a bounded mbarrier wait expired and the
 * affected tiles were not written; bit 1: misaligned dynamic shared memory).  No counterpart in the reference (its
 * kernels have no bounded waits).
 *   mb_gemm_status        synchronises the stream, returns the word and clears it;
 *   mb_gemm_status_async  copies the word to `host_status` (pinned host memory) in stream order, without
 *                         synchronising and without clearing it: a caller that launches evaluation after
 *                         evaluation reads the word of the previous one when it starts the next, at no cost;
 *   mb_gemm_status_clear  zeroes the word in stream order (after an expiry has been reported). */
int mb_gemm_status(int* status, void* stream);
int mb_gemm_status_async(int* host_status, void* stream);
int mb_gemm_status_clear(void* stream);
/* Self-test of the failure path above: launches one CTA that waits, with a limit of a few polls, on an mbarrier
 * that nothing ever arrives at.  The wait runs out, the kernel sets bit 0 of the status word and returns through
 * its normal exit; nothing faults, traps or hangs.  The next mb_gemm_status* call sees bit 0. */
int mb_selftest_wait_expiry(void* stream);
/* Timed issue rate of the tensor-core instruction the kernels above are built on: every SM runs `iters` batches of
 * four M128 x N128 tcgen05.mma (kind 0: tf32, K = 8; kind 1: bf16, K = 16) on operands resident in tensor / shared
 * memory; returns the elapsed time of the launch (CUDA events on `stream`, which is synchronised) and the number
 * of SMs used, from which the caller derives TFLOP/s = 2 * 128 * 128 * K * 4 * iters * sms / ms.  This is the
 * denominator the 3-pass tf32 GEMMs are judged against. */
int mb_bench_mma_rate(int kind, int iters, float* elapsed_ms, int* n_sms, void* stream);

/* ------------------------------------------------------------------ fused gated MLP (forward)
 * GatedMLP.forward (matris/model/functions.py:245-311) as ONE kernel per call:
 *   z1 = X W1^T + b1            X = up to four gathered 128-wide row segments (as in mb_gemm), W1 [256, K]:
 *                               rows 0..127 the core branch's first layer, 128..255 the gate branch's
 *   z2 = SiLU(z1) (.) W2^T + b2 W2 [256, 128]: rows 0..127 act on z1[:, :128] (core), 128..255 on z1[:, 128:] (gate)
 *   h  = SiLU(RMSNorm(z2[:, :128]) * norm_core) * sigmoid(RMSNorm(z2[:, 128:]) * norm_gate)
 *   out2 = h + res_w * res      (optional)
 * Layer 1's accumulator never leaves tensor memory: it is read back, biased, passed through SiLU, split into
 * bf16 hi / lo and stored as the A operand of layer 2 on chip; RMSNorm and the gate run in the epilogue of
 * layer 2.  z1 / z2 are written only when the pointers are given (the backward pass wants them).  The fused kernel
 * exists for the default GEMM mode (0, 3xBF16); in modes 1, 2 and 3 (see mb_set_gemm_mode) the same result is
 * composed from mb_gemm and mb_gate_fwd, which needs z1 and z2 as scratch: they are required there.
 *
 * kind = MB_MLP_PLAIN runs the same pipeline for a plain two-layer perceptron (node_FFN / edge_FFN,
 * matris/model/interaction_block.py:197-210):
 *   z1 = X W1^T + b1            W1 [128, K], b1 [128]
 *   h  = SiLU(z1) W2^T + b2     W2 [128, 128], b2 [128];   out2 = h + res_w * res (optional)
 * z1 is then [R, 128] (optional in mode 0, required as scratch in the other modes); z2, norm_core and norm_gate are
 * not read. */
#define MB_MLP_GATED 0
#define MB_MLP_PLAIN 1
typedef struct mb_gated_mlp {
  int64_t n_rows;
  int32_t n_src;               /* 1..4 ; K = 128 * n_src */
  int32_t kind;                /* MB_MLP_GATED or MB_MLP_PLAIN */
  mb_src src[4];               /* src[].act is honoured (SiLU on load) */
  const float* W1;             /* [256, K] row-major (SIMT mode) */
  const float* W1_hi;          /* tf32(W1) */
  const float* W1_lo;          /* W1 - tf32(W1) */
  const uint16_t* W1_hi16;     /* bf16(W1) */
  const uint16_t* W1_lo16;     /* bf16(W1 - bf16(W1)) */
  int64_t ldw1;                /* row stride of W1* in floats (>= K) */
  const float* b1;             /* [256] or NULL */
  const float* W2;             /* [256, 128] */
  const float* W2_hi;
  const float* W2_lo;
  const uint16_t* W2_hi16;
  const uint16_t* W2_lo16;
  int64_t ldw2;                /* row stride of W2* in floats (>= 128) */
  const float* b2;             /* [256] or NULL */
  const float* norm_core;      /* [128] RMSNorm weights */
  const float* norm_gate;      /* [128] */
  float* z1; int64_t ld_z1;    /* optional [R, 256] */
  float* z2; int64_t ld_z2;    /* optional [R, 256] */
  float* h; int64_t ld_h;      /* optional [R, 128] (h or out2 must be given) */
  const float* res;            /* [R, 128] rows, required with out2 */
  const float* res_w;          /* [128] or NULL (= 1) */
  int64_t ld_res;
  float* out2; int64_t ld_out2;
} mb_gated_mlp;
int mb_gated_mlp_fwd(const mb_gated_mlp* desc, void* stream);

/* ------------------------------------------------------------------ row-wise model kernels
 * All feature tensors are float32 row-major with 128 channels unless noted.
 */

/* GatedMLP tail (matris/model/functions.py:300-311): z [R,256] = (core | gate) pre-norm;
 * h = SiLU(RMSNorm(z_core)*w_core) * sigmoid(RMSNorm(z_gate)*w_gate); optional out2 = h + res_w*res. */
int mb_gate_fwd(int64_t n_rows, const float* z, const float* w_core, const float* w_gate, float* h,
                const float* res, const float* res_w, float* out2, void* stream);
/* data gradient of the above: dz [R,256] from dh [R,128] (recomputes the norms from z) */
int mb_gate_bwd(int64_t n_rows, const float* z, const float* w_core, const float* w_gate, const float* dh,
                float* dz, void* stream);

/* Per-channel segment softmax + weighted segment sums of the attention layer
 * (Dimwise_softmax + aggregate, matris/model/functions.py:97-160, as used in
 * matris/model/interaction_block.py:116-137).  Rows are grouped by target node
 * (tgt_ptr CSR, contiguous) and by source node (src_ptr CSR over src_perm).
 * logits [*,256]: columns 0..127 source logits, 128..255 target logits, row
 * emap[r] (NULL: r).  stats [n_nodes,4,128] = (max_t, 1/sum_t, max_s, 1/sum_s). */
int mb_seg_attn_fwd(int32_t n_nodes, const int32_t* tgt_ptr, const int32_t* src_ptr, const int32_t* src_perm,
                    const int32_t* emap, const float* logits, const float* h, float* agg_t, float* agg_s,
                    float* stats, void* stream);
/* per row: dh = a_t*dagg_t[tgt] + a_s*dagg_s[src] + dh_scale*dh_in[dh_map ? dh_map[r] : r];
 * dlogits[r] = (a_s*dagg_s*(h-agg_s) | a_t*dagg_t*(h-agg_t)).
 * With gate_dz != NULL the row's dh is not written: it goes on, in registers, through the adjoint of the gated MLP's
 * tail (what mb_gate_bwd computes from gate_z = z2 [rows,256] and the two norm weights) and gate_dz [rows,256]
 * receives the result; dh may then be NULL. */
int mb_seg_attn_bwd(int64_t n_rows, const int32_t* tgt, const int32_t* src, int32_t idx_stride,
                    const int32_t* emap, const float* logits, const float* h, const float* agg_t,
                    const float* agg_s, const float* stats, const float* dagg_t, const float* dagg_s,
                    const float* dh_in, const int32_t* dh_map, float dh_scale, float* dh, float* dlogits,
                    const float* gate_z, const float* gate_wc, const float* gate_wg, float* gate_dz, void* stream);

/* Refinement aggregation (matris/model/interaction_block.py:246-262):
 * agg[n] = sum_{r in target segment n} h[r] * s[r]; s[r] = env[emap[r]] (atom graph, src == NULL)
 * or env[src[r]] * env[n] (line graph). */
int mb_seg_smooth_sum_fwd(int32_t n_nodes, const int32_t* tgt_ptr, const int32_t* emap, const int32_t* src,
                          int32_t idx_stride, const float* env, const float* h, float* agg, void* stream);
/* per row: dh[r] (+)= dagg[tgt[r]] * s[r]   (accumulate != 0: add to existing dh).  gate_z / gate_wc / gate_wg /
 * gate_dz as in mb_seg_attn_bwd: the finished dh row goes through the gated MLP's tail adjoint instead of to memory. */
int mb_seg_smooth_sum_bwd_rows(int64_t n_rows, const int32_t* tgt, const int32_t* src, int32_t idx_stride,
                               const int32_t* emap, const float* env, const float* dagg, float* dh,
                               int32_t accumulate, const float* gate_z, const float* gate_wc, const float* gate_wg,
                               float* gate_dz, void* stream);
/* gradient w.r.t. env.  Atom graph (src_ptr == NULL): denv[u] = sum over the two directed rows e of
 * bond u of (dagg[tgt[e]] + drow[e])*h[e]  (u2d / rev give the rows; drow, optional, is a gradient that reached
 * the smoothed rows h*s directly: use_smoothed_for_delta_edge, matris/model/interaction_block.py:262-266).
 * Line graph (drow must be NULL): denv[n] = sum_{r in tgt segment n} dagg[n]*h[r]*env[src[r]]
 * + sum_{r in src segment n} dagg[tgt[r]]*h[r]*env[tgt[r]]. */
int mb_seg_smooth_sum_bwd_env(int32_t n_nodes, const int32_t* tgt_ptr, const int32_t* src_ptr,
                              const int32_t* src_perm, const int32_t* tgt, const int32_t* src, int32_t idx_stride,
                              const int32_t* u2d, const int32_t* rev, const float* env, const float* h,
                              const float* dagg, const float* drow, float* denv, void* stream);
/* y[r] = x[r] * s[idx ? idx[r] : r] channel-wise: the smoothed rows h * envelope of the refinement layer
 * (matris/model/interaction_block.py:253) where they are needed as a tensor, and their adjoint w.r.t. x. */
int mb_mul_rows_gather(int64_t n_rows, const float* x, const float* s, const int32_t* idx, float* y, void* stream);

/* directed -> bond mean with residual (aggregate(..., average=True) over directed2undirected,
 * matris/model/interaction_block.py:123, 270-273): out[u] = 0.5*(y[u2d[u]] + y[rev[u2d[u]]]) + res_w*res[u] */
int mb_pair_mean_res(int32_t n_bonds, const int32_t* u2d, const int32_t* rev, const float* y, const float* res,
                     const float* res_w, float* out, void* stream);
/* y = a*x (elementwise per channel weight a[128]) ; accumulate != 0: y += a*x */
int mb_scale_rows(int64_t n_rows, const float* x, const float* a, float* y, int32_t accumulate, void* stream);

/* K <= 16 linear layers (edge_linear1 / learnable_envelope: K=7, angle_embedding: K=16;
 * matris/model/feature_embed.py:105-106,176, matris/model/interaction_block.py:213-215):
 * y[R,128] = x[R,K] @ W[128,K]^T and dx[R,K] (+)= dy[R,128] @ W */
int mb_small_linear_fwd(int64_t n_rows, int32_t k, const float* x, const float* w, float* y, void* stream);
int mb_small_linear_bwd(int64_t n_rows, int32_t k, const float* dy, const float* w, float* dx, int32_t accumulate,
                        void* stream);

/* LayerNorm(128, eps=1e-5, affine) of the bond embedding (matris/model/feature_embed.py:113,140) */
int mb_layernorm_fwd(int64_t n_rows, const float* x, const float* w, const float* b, float* y, void* stream);
int mb_layernorm_bwd(int64_t n_rows, const float* x, const float* w, const float* dy, float* dx, void* stream);
/* RMSNorm(128, eps = float32 epsilon, affine) (readout_norm, matris/model/model.py:167,216) */
int mb_rmsnorm_fwd(int64_t n_rows, const float* x, const float* w, float* y, void* stream);
int mb_rmsnorm_bwd(int64_t n_rows, const float* x, const float* w, const float* dy, float* dx, void* stream);

/* embedding lookup: y[r] = table[idx[r] + offset] (nn.Embedding, matris/model/feature_embed.py:37) */
int mb_embedding(int64_t n_rows, const int32_t* idx, int32_t offset, const float* table, float* y, void* stream);

/* Final projection of the heads: out[r] = SiLU(z[r, 0:k]) . w + b ; optional |.| (magmom,
 * matris/model/readout.py:131) ; energy head: summed per structure through atom_ptr in mb_energy_sum. */
int mb_head_dot_fwd(int64_t n_rows, int32_t k, const float* z, const float* w, const float* b, int32_t take_abs,
                    float* out, void* stream);
/* dz[r, c] = seed[seed_map[r]] * w[c] * silu'(z[r, c])   (seed: upstream gradient per structure) */
int mb_head_dot_bwd(int64_t n_rows, int32_t k, const float* z, const float* w, const float* seed,
                    const int32_t* seed_map, float* dz, void* stream);
/* dz = dy * d/dz SiLU(z), element-wise on [n_rows,128]: the reference's fused SiLU backward
 * (matris/model/op/fused_silu_op.py:5-13,32-43; matris/model/op/src/kernel/fused_silu_bwd.cu:5-25) */
int mb_silu_bwd(int64_t n_rows, const float* dy, const float* z, float* dz, void* stream);
/* per-structure sum of per-atom energies (GraphPooling, matris/model/functions.py:340-365) */
int mb_segment_sum_scalar(int32_t n_seg, const int32_t* seg_ptr, const float* x, float* out, void* stream);

/* ------------------------------------------------------------------ geometry and bases
 * Edge vectors of process_graphs (matris/model/processgraph.py:87, 192-199), float32:
 * v = r_c - (r_n + image @ L), d = |v|, u = v/d; cart = frac32 @ lattice32 is computed by the caller. */
int mb_edge_geometry_fwd(int64_t n_edges, const float* cart, const float* lattice, const int32_t* atom_struct,
                         const int32_t* center, const int32_t* neighbor, const int32_t* image, float* vec,
                         float* len, float* unit, void* stream);
/* Backward of the above plus the conservative head (matris/model/readout.py:202-224): from dE/dlen [E] and
 * dE/dunit [E,3] form g_e = dE/dv_e, then dE/dr_i = sum_{e:c=i} g_e - sum_{e:c=i} g_rev(e) (no atomics) and
 * per-atom virial partials, reduced per structure into dE/dstrain = sym(sum_e v_e (x) g_e) [B,3,3]. */
int mb_edge_geometry_bwd(int32_t n_atoms, int32_t n_struct, int64_t n_edges, const int32_t* edge_ptr,
                         const int32_t* atom_ptr,
                         const int32_t* rev, const float* vec, const float* len, const float* unit,
                         const float* dlen, const float* dunit, float* g_edge, float* dcart, float* virial_atom,
                         float* dstrain, void* stream);

/* Allocation-free twin of mb_edge_geometry_bwd.  No counterpart in the reference: the reference reaches forces and
 * stress through torch.autograd, which allocates freely.
 *
 * Who needs it: programs that bind this C ABI directly and own the whole device-memory budget themselves - a
 * molecular-dynamics engine written in C, C++ or Fortran that carves all of its device memory up at start-up and
 * then calls the force / virial reduction once per time step from its own integrator.  Such a caller has no
 * caching allocator behind it; a cudaMalloc / cudaFree pair per step would synchronise the whole device each time
 * (and can simply fail once the engine has handed out the rest of the memory), and inside its per-step callback it
 * is often not allowed to allocate at all.  mb_edge_geometry_bwd needs two scratch arrays from the caller (the
 * per-edge gradient and the per-atom virial partials); this entry takes them from a fixed array inside the library
 * instead, so the caller passes inputs and outputs only.
 *
 * Limits and rules:
 *  - at most MB_STATIC_MAX_EDGES directed edges and MB_STATIC_MAX_ATOMS atoms per call; larger problems are
 *    rejected with MB_ERR_TOO_LARGE before anything is launched (use mb_edge_geometry_bwd for those);
 *  - the array (3*MB_STATIC_MAX_EDGES + 9*MB_STATIC_MAX_ATOMS floats = 7,471,104 bytes: 7.5 MB, 7.1 MiB) is part of
 *    the library image: every GPU that loads the library holds it until the process exits;
 *  - the first call on a device looks the array's device address up (with that device current) and remembers it;
 *    where the CUDA runtime loads modules lazily, that first call is also what loads the module, and the driver
 *    allocates the module's device memory (the array included) then.  Make that first call during set-up, from one
 *    thread, before any stream capture is started;
 *  - after that first call it calls no cudaMalloc, cudaFree or other allocating routine;
 *  - all calls share the one array and it keeps whatever the previous call left there.  Nothing has to start at
 *    zero: each call overwrites every element it later reads.  Two calls that overlap on the GPU (different
 *    streams, or different host threads without ordering) race on the array: serialise them.
 * Same results as mb_edge_geometry_bwd (same kernels, same summation order). */
#define MB_STATIC_MAX_EDGES (1 << 19)
#define MB_STATIC_MAX_ATOMS (1 << 15)
int mb_edge_geometry_bwd_static(int32_t n_atoms, int32_t n_struct, int64_t n_edges, const int32_t* edge_ptr,
                                const int32_t* atom_ptr, const int32_t* rev, const float* vec, const float* len,
                                const float* unit, const float* dlen, const float* dunit, float* dcart,
                                float* dstrain, void* stream);

/* Bessel * polynomial envelope, both cutoffs at once (matris/model/basis_function.py:8-50, 162-186):
 * per bond u with d = len[u2d[u]]: rbf_a[u,7] (cutoff ca, frequencies fa) and rbf_b[u,7] (cb, fb). */
int mb_bessel_fwd(int32_t n_bonds, const int32_t* u2d, const float* len, const float* freq_a, float cut_a,
                  const float* freq_b, float cut_b, int32_t p, float* rbf_a, float* rbf_b, void* stream);
/* dlen[u2d[u]] += d(rbf_a)/dd . drbf_a + d(rbf_b)/dd . drbf_b */
int mb_bessel_bwd(int32_t n_bonds, const int32_t* u2d, const float* len, const float* freq_a, float cut_a,
                  const float* freq_b, float cut_b, int32_t p, const float* drbf_a, const float* drbf_b,
                  float* dlen, void* stream);

/* GaussianExpansion (distance_expansion = "gaussian"; matris/model/basis_function.py:189-216, built in
 * matris/model/feature_embed.py:86-99): rbf[u,k] = exp(coeff (d_u - offset[k])^2), seven offsets per set (the module's
 * `offset` buffer), coeff = -0.5 / (2 (offset[1] - offset[0]))^2; no envelope.  Same layout as mb_bessel_*. */
int mb_gaussian_fwd(int32_t n_bonds, const int32_t* u2d, const float* len, const float* off_a, float coeff_a,
                    const float* off_b, float coeff_b, float* rbf_a, float* rbf_b, void* stream);
int mb_gaussian_bwd(int32_t n_bonds, const int32_t* u2d, const float* len, const float* off_a, float coeff_a,
                    const float* off_b, float coeff_b, const float* drbf_a, const float* drbf_b, float* dlen,
                    void* stream);

/* Angle basis of ThreebodyEmbedding + SphericalExpansion (matris/model/feature_embed.py:183-197,
 * matris/model/basis_function.py:222-338): x = (u_a . u_b)(1-1e-6), theta = acos x, 16 = 4 radial orders x 4
 * roots of spherical Bessel functions at |u_b|/cutoff times real m=0 harmonics of cos(theta). */
int mb_angle_basis_fwd(int64_t n_trip, const int32_t* line_graph, const float* unit, float factor, float cutoff,
                       float* basis, void* stream);
/* dunit[tDE] += ..., dunit[sDE] += ... (atomic) from dbasis [T,16] */
int mb_angle_basis_bwd(int64_t n_trip, const int32_t* line_graph, const float* unit, float factor, float cutoff,
                       const float* dbasis, float* dunit, void* stream);

/* Angle basis of ThreebodyEmbedding + FourierExpansion (three_body_expansion = "fourier";
 * matris/model/basis_function.py:79-113 with num_angular = 7): basis[t] = [1/sqrt 2, sin(f_k theta), cos(f_k theta)]
 * / sqrt(pi), k = 0..2, theta as above, f = the module's `frequencies` [3].  basis / dbasis are [T,7]. */
int mb_fourier_basis_fwd(int64_t n_trip, const int32_t* line_graph, const float* unit, const float* freq,
                         float* basis, void* stream);
int mb_fourier_basis_bwd(int64_t n_trip, const int32_t* line_graph, const float* unit, const float* freq,
                         const float* dbasis, float* dunit, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* MATRIS_B200_H */
