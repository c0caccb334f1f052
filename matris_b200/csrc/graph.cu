// Periodic radius graph, bond graph and line graph (angle triplets) on the GPU.
//
// Integer / indexing work, HBM-bound.  The inclusion tests run in float64 with
// explicit round-to-nearest intrinsics (no FMA contraction) in a fixed operation
// order, so membership is decided by exactly the same numbers as a NumPy
// evaluation of the same formula.
//
// Pipeline (see include/matris_b200.h for what each phase returns):
//   bin atoms into cells -> per-atom neighbour count (warp per atom, ballot
//   compaction) -> scan -> fill -> per-atom rank sort by (neighbour, image) ->
//   reverse-edge search (binary search inside the neighbour's own segment) ->
//   bond numbering (scan of "first of its pair" flags) -> per-bond triplet counts
//   -> scan -> triplet fill grouped by target bond + permutation grouped by
//   source bond.
#include "common.cuh"

namespace mb {

// ---------------------------------------------------------------- exclusive scan
constexpr int SCAN_THREADS = 256;
constexpr int SCAN_ITEMS = 8;  // per thread
constexpr int SCAN_CHUNK = SCAN_THREADS * SCAN_ITEMS;

__device__ __forceinline__ int block_exclusive_scan(int v, int* total) {
  __shared__ int warp_sums[SCAN_THREADS / 32];
  __shared__ int block_total;
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  int x = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    int y = __shfl_up_sync(0xffffffffu, x, o);
    if (lane >= o) x += y;
  }
  if (lane == 31) warp_sums[w] = x;
  __syncthreads();
  if (w == 0) {
    int s = lane < SCAN_THREADS / 32 ? warp_sums[lane] : 0;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      int y = __shfl_up_sync(0xffffffffu, s, o);
      if (lane >= o) s += y;
    }
    if (lane < SCAN_THREADS / 32) warp_sums[lane] = s;  // inclusive over warps
    if (lane == SCAN_THREADS / 32 - 1) block_total = s;
  }
  __syncthreads();
  int prefix = (w > 0 ? warp_sums[w - 1] : 0) + x - v;
  *total = block_total;
  __syncthreads();
  return prefix;
}

__global__ void k_scan_reduce(const int32_t* __restrict__ in, int64_t n, int32_t* __restrict__ block_sums) {
  int64_t base = (int64_t)blockIdx.x * SCAN_CHUNK;
  int s = 0;
#pragma unroll
  for (int k = 0; k < SCAN_ITEMS; ++k) {
    int64_t i = base + (int64_t)threadIdx.x * SCAN_ITEMS + k;
    if (i < n) s += in[i];
  }
  int total;
  block_exclusive_scan(s, &total);
  if (threadIdx.x == 0) block_sums[blockIdx.x] = total;
}

// single block: exclusive scan of the block sums in place, sequentially over chunks
__global__ void k_scan_block_sums(int32_t* __restrict__ block_sums, int n_blocks) {
  __shared__ int carry;
  if (threadIdx.x == 0) carry = 0;
  __syncthreads();
  for (int base = 0; base < n_blocks; base += SCAN_THREADS) {
    int i = base + threadIdx.x;
    int v = i < n_blocks ? block_sums[i] : 0;
    int total;
    int p = block_exclusive_scan(v, &total);
    if (i < n_blocks) block_sums[i] = carry + p;
    __syncthreads();
    if (threadIdx.x == 0) carry += total;
    __syncthreads();
  }
  if (threadIdx.x == 0) block_sums[n_blocks] = carry;
}

__global__ void k_scan_apply(const int32_t* in, int64_t n, const int32_t* __restrict__ block_sums, int32_t* out,
                             int n_blocks) {
  int64_t base = (int64_t)blockIdx.x * SCAN_CHUNK;
  int v[SCAN_ITEMS];
  int s = 0;
#pragma unroll
  for (int k = 0; k < SCAN_ITEMS; ++k) {
    int64_t i = base + (int64_t)threadIdx.x * SCAN_ITEMS + k;
    v[k] = i < n ? in[i] : 0;
    s += v[k];
  }
  int total;
  int p = block_exclusive_scan(s, &total) + block_sums[blockIdx.x];
#pragma unroll
  for (int k = 0; k < SCAN_ITEMS; ++k) {
    int64_t i = base + (int64_t)threadIdx.x * SCAN_ITEMS + k;
    if (i < n) out[i] = p;
    p += v[k];
  }
  if (blockIdx.x == n_blocks - 1 && threadIdx.x == 0) out[n] = block_sums[n_blocks];
}

int scan_exclusive(const int32_t* in, int32_t* out, int64_t n, int32_t* tmp, cudaStream_t s) {
  if (n <= 0) {
    MB_CUDA_CHECK(cudaMemsetAsync(out, 0, sizeof(int32_t), s));
    return MB_OK;
  }
  int n_blocks = cdiv(n, SCAN_CHUNK);
  k_scan_reduce<<<n_blocks, SCAN_THREADS, 0, s>>>(in, n, tmp);
  k_scan_block_sums<<<1, SCAN_THREADS, 0, s>>>(tmp, n_blocks);
  k_scan_apply<<<n_blocks, SCAN_THREADS, 0, s>>>(in, n, tmp, out, n_blocks);
  MB_LAUNCH_CHECK("scan_exclusive");
  return MB_OK;
}

// ---------------------------------------------------------------- status words
enum { ST_ISOLATED = 0, ST_IMAGE_OVERFLOW = 1, ST_UNPAIRED = 2 };

// ---------------------------------------------------------------- binning
__global__ void k_bin_count(int n_atoms, const double* __restrict__ cart, const double* __restrict__ inv_lattice,
                            const int32_t* __restrict__ atom_struct, const int32_t* __restrict__ grid,
                            int32_t* __restrict__ atom_cell, int32_t* __restrict__ atom_wrap,
                            int32_t* __restrict__ cell_count) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_atoms) return;
  int b = atom_struct[i];
  const double* inv = inv_lattice + 9 * b;
  const int32_t* g = grid + 8 * b;
  double x = cart[3 * i], y = cart[3 * i + 1], z = cart[3 * i + 2];
  int c[3], w[3];
#pragma unroll
  for (int k = 0; k < 3; ++k) {
    double f = x * inv[k] + y * inv[3 + k] + z * inv[6 + k];
    double fl = floor(f);
    double fw = f - fl;
    if (fw >= 1.0) { fw = 0.0; fl += 1.0; }
    w[k] = (int)fl;
    int ck = (int)(fw * (double)g[k]);
    c[k] = ck < g[k] - 1 ? ck : g[k] - 1;
    if (c[k] < 0) c[k] = 0;
  }
  int cell = g[6] + (c[0] * g[1] + c[1]) * g[2] + c[2];
  reinterpret_cast<int4*>(atom_cell)[i] = make_int4(c[0], c[1], c[2], cell);
  reinterpret_cast<int4*>(atom_wrap)[i] = make_int4(w[0], w[1], w[2], 0);
  atomicAdd(&cell_count[cell], 1);
}

__global__ void k_bin_fill(int n_atoms, const int32_t* __restrict__ atom_cell, const int32_t* __restrict__ cell_ptr,
                           int32_t* __restrict__ cell_fill, int32_t* __restrict__ cell_atoms) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_atoms) return;
  int cell = atom_cell[4 * i + 3];
  int pos = cell_ptr[cell] + atomicAdd(&cell_fill[cell], 1);
  cell_atoms[pos] = i;
}

// ---------------------------------------------------------------- neighbour search
__device__ __forceinline__ int floor_div(int a, int b) {
  int q = a / b;
  return (a % b != 0 && ((a < 0) != (b < 0))) ? q - 1 : q;
}

__device__ __forceinline__ uint64_t pack_key(int j, int n0, int n1, int n2) {
  return ((uint64_t)(uint32_t)j << 24) | ((uint64_t)(uint32_t)(n0 + 128) << 16) |
         ((uint64_t)(uint32_t)(n1 + 128) << 8) | (uint64_t)(uint32_t)(n2 + 128);
}

template <bool FILL>
__global__ void k_neighbors(int n_atoms, double cutoff, double tol, const double* __restrict__ cart,
                            const double* __restrict__ lattice, const int32_t* __restrict__ atom_struct,
                            const int32_t* __restrict__ grid, const int32_t* __restrict__ atom_cell,
                            const int32_t* __restrict__ atom_wrap, const int32_t* __restrict__ cell_ptr,
                            const int32_t* __restrict__ cell_atoms, int32_t* __restrict__ edge_ptr,
                            uint64_t* __restrict__ key_out, double* __restrict__ dist_out,
                            int32_t* __restrict__ status) {
  const int lane = threadIdx.x & 31;
  const int i = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (i >= n_atoms) return;
  const int b = atom_struct[i];
  const int32_t* g = grid + 8 * b;
  const int g0 = g[0], g1 = g[1], g2 = g[2], s0 = g[3], s1 = g[4], s2 = g[5], base = g[6];
  double L[9];
#pragma unroll
  for (int k = 0; k < 9; ++k) L[k] = lattice[9 * b + k];
  const double xi = cart[3 * i], yi = cart[3 * i + 1], zi = cart[3 * i + 2];
  const int4 ci = reinterpret_cast<const int4*>(atom_cell)[i];
  const int4 wi = reinterpret_cast<const int4*>(atom_wrap)[i];
  const int out_base = FILL ? edge_ptr[i] : 0;
  int count = 0;
  for (int d0 = -s0; d0 <= s0; ++d0) {
    int c0 = ci.x + d0, h0 = floor_div(c0, g0);
    c0 -= h0 * g0;
    for (int d1 = -s1; d1 <= s1; ++d1) {
      int c1 = ci.y + d1, h1 = floor_div(c1, g1);
      c1 -= h1 * g1;
      for (int d2 = -s2; d2 <= s2; ++d2) {
        int c2 = ci.z + d2, h2 = floor_div(c2, g2);
        c2 -= h2 * g2;
        const int cell = base + (c0 * g1 + c1) * g2 + c2;
        const int p0 = cell_ptr[cell], p1 = cell_ptr[cell + 1];
        for (int pb = p0; pb < p1; pb += 32) {
          const int p = pb + lane;
          bool ok = false;
          int j = 0, n0 = 0, n1 = 0, n2 = 0;
          double d = 0.0;
          if (p < p1) {
            j = cell_atoms[p];
            const int4 wj = reinterpret_cast<const int4*>(atom_wrap)[j];
            n0 = h0 - wj.x + wi.x;
            n1 = h1 - wj.y + wi.y;
            n2 = h2 - wj.z + wi.z;
            const double f0 = (double)n0, f1 = (double)n1, f2 = (double)n2;
            // s = (n0*L0 + n1*L1) + n2*L2 ; dx = (x_j + s) - x_i ; no FMA contraction
            const double sx = __dadd_rn(__dadd_rn(__dmul_rn(f0, L[0]), __dmul_rn(f1, L[3])), __dmul_rn(f2, L[6]));
            const double sy = __dadd_rn(__dadd_rn(__dmul_rn(f0, L[1]), __dmul_rn(f1, L[4])), __dmul_rn(f2, L[7]));
            const double sz = __dadd_rn(__dadd_rn(__dmul_rn(f0, L[2]), __dmul_rn(f1, L[5])), __dmul_rn(f2, L[8]));
            const double dx = __dsub_rn(__dadd_rn(cart[3 * j], sx), xi);
            const double dy = __dsub_rn(__dadd_rn(cart[3 * j + 1], sy), yi);
            const double dz = __dsub_rn(__dadd_rn(cart[3 * j + 2], sz), zi);
            const double q = __dadd_rn(__dadd_rn(__dmul_rn(dx, dx), __dmul_rn(dy, dy)), __dmul_rn(dz, dz));
            d = __dsqrt_rn(q);
            ok = (d > tol) && (d <= cutoff);
          }
          const unsigned mask = __ballot_sync(0xffffffffu, ok);
          if (FILL && ok) {
            const int pos = out_base + count + __popc(mask & ((1u << lane) - 1u));
            key_out[pos] = pack_key(j, n0, n1, n2);
            dist_out[pos] = d;
            if (n0 < -127 || n0 > 127 || n1 < -127 || n1 > 127 || n2 < -127 || n2 > 127)
              atomicOr(&status[ST_IMAGE_OVERFLOW], 1);
          }
          count += __popc(mask);
        }
      }
    }
  }
  if (!FILL && lane == 0) {
    edge_ptr[i] = count;
    if (count == 0) atomicAdd(&status[ST_ISOLATED], 1);
  }
}

// rank sort of each atom's out-edges by key (neighbour, image); warp per atom
__global__ void k_sort_edges(int n_atoms, const int32_t* __restrict__ edge_ptr,
                             const uint64_t* __restrict__ key_in, const double* __restrict__ dist_in,
                             uint64_t* __restrict__ key, double* __restrict__ dist, int32_t* __restrict__ center,
                             int32_t* __restrict__ neighbor, int32_t* __restrict__ image) {
  const int lane = threadIdx.x & 31;
  const int i = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (i >= n_atoms) return;
  const int e0 = edge_ptr[i], n = edge_ptr[i + 1] - e0;
  for (int a = lane; a < n; a += 32) {
    const uint64_t k = key_in[e0 + a];
    int rank = 0;
    for (int m = 0; m < n; ++m) rank += key_in[e0 + m] < k ? 1 : 0;
    const int e = e0 + rank;
    key[e] = k;
    dist[e] = dist_in[e0 + a];
    center[e] = i;
    neighbor[e] = (int)(k >> 24);
    image[3 * e + 0] = (int)((k >> 16) & 0xff) - 128;
    image[3 * e + 1] = (int)((k >> 8) & 0xff) - 128;
    image[3 * e + 2] = (int)(k & 0xff) - 128;
  }
}

// reverse edge of e = (i, j, n): the edge (j, i, -n), found by binary search in j's segment
__global__ void k_pair_edges(int n_edges, const int32_t* __restrict__ edge_ptr, const uint64_t* __restrict__ key,
                             const int32_t* __restrict__ center, int32_t* __restrict__ rev,
                             int32_t* __restrict__ first_flag, int32_t* __restrict__ status) {
  int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= n_edges) return;
  const uint64_t k = key[e];
  const int i = center[e], j = (int)(k >> 24);
  const int n0 = (int)((k >> 16) & 0xff) - 128, n1 = (int)((k >> 8) & 0xff) - 128, n2 = (int)(k & 0xff) - 128;
  const uint64_t want = pack_key(i, -n0, -n1, -n2);
  int lo = edge_ptr[j], hi = edge_ptr[j + 1];
  while (lo < hi) {
    int mid = (lo + hi) >> 1;
    if (key[mid] < want) lo = mid + 1; else hi = mid;
  }
  int r = -1;
  if (lo < edge_ptr[j + 1] && key[lo] == want) r = lo;
  if (r < 0) atomicAdd(&status[ST_UNPAIRED], 1);
  rev[e] = r;
  first_flag[e] = (r < 0 || r > e) ? 1 : 0;
}

__global__ void k_number_bonds(int n_edges, const int32_t* __restrict__ rev, const int32_t* __restrict__ first_rank,
                               int32_t* __restrict__ d2u, int32_t* __restrict__ u2d) {
  int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= n_edges) return;
  const int r = rev[e];
  const int f = (r >= 0 && r < e) ? r : e;
  const int u = first_rank[f];
  d2u[e] = u;
  if (f == e) u2d[u] = e;
}

// bit0: the bond of e may be a triplet target (first directed edge's length <= lc)
// bit1: e may be the source ("other") edge of a triplet (its own length < lc)
__global__ void k_edge_flags(int n_edges, double lc, const double* __restrict__ dist, const int32_t* __restrict__ rev,
                             uint8_t* __restrict__ flag) {
  int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= n_edges) return;
  const int r = rev[e];
  const int f = (r >= 0 && r < e) ? r : e;
  flag[e] = (uint8_t)((dist[f] <= lc ? 1 : 0) | (dist[e] < lc ? 2 : 0));
}

// per atom: exclusive ranks of source-/target-eligible edges inside the atom's segment
__global__ void k_edge_ranks(int n_atoms, const int32_t* __restrict__ edge_ptr, const uint8_t* __restrict__ flag,
                             int32_t* __restrict__ edge_rank, int32_t* __restrict__ atom_counts) {
  const int lane = threadIdx.x & 31;
  const int i = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (i >= n_atoms) return;
  const int e0 = edge_ptr[i], e1 = edge_ptr[i + 1];
  int ns = 0, nt = 0;
  for (int eb = e0; eb < e1; eb += 32) {
    const int e = eb + lane;
    const int f = e < e1 ? flag[e] : 0;
    const unsigned ms = __ballot_sync(0xffffffffu, f & 2), mt = __ballot_sync(0xffffffffu, f & 1);
    const unsigned lt = (1u << lane) - 1u;
    if (e < e1) {
      edge_rank[2 * e] = ns + __popc(ms & lt);
      edge_rank[2 * e + 1] = nt + __popc(mt & lt);
    }
    ns += __popc(ms);
    nt += __popc(mt);
  }
  if (lane == 0) {
    atom_counts[2 * i] = ns;
    atom_counts[2 * i + 1] = nt;
  }
}

__global__ void k_bond_counts(int n_bonds, const int32_t* __restrict__ u2d, const int32_t* __restrict__ rev,
                              const int32_t* __restrict__ center, const uint8_t* __restrict__ flag,
                              const int32_t* __restrict__ atom_counts, int32_t* __restrict__ tgt_count,
                              int32_t* __restrict__ src_count) {
  int u = blockIdx.x * blockDim.x + threadIdx.x;
  if (u >= n_bonds) return;
  const int a0 = u2d[u], a1 = rev[a0];
  int tc = 0, sc = 0;
  const int a[2] = {a0, a1};
#pragma unroll
  for (int s = 0; s < 2; ++s) {
    if (a[s] < 0) continue;
    const int f = flag[a[s]], c = center[a[s]];
    if (f & 1) tc += atom_counts[2 * c] - ((f >> 1) & 1);
    if (f & 2) sc += atom_counts[2 * c + 1] - (f & 1);
  }
  tgt_count[u] = tc;
  src_count[u] = sc;
}

// warp per bond: rows with this bond as target (contiguous), and the ids of the
// rows that have this bond as source
__global__ void k_fill_triplets(int n_bonds, const int32_t* __restrict__ edge_ptr, const int32_t* __restrict__ u2d,
                                const int32_t* __restrict__ rev, const int32_t* __restrict__ center,
                                const int32_t* __restrict__ d2u, const uint8_t* __restrict__ flag,
                                const int32_t* __restrict__ edge_rank, const int32_t* __restrict__ atom_counts,
                                const int32_t* __restrict__ trip_ptr, const int32_t* __restrict__ trip_src_ptr,
                                int32_t* __restrict__ line_graph, int32_t* __restrict__ src_perm) {
  const int lane = threadIdx.x & 31;
  const int u = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (u >= n_bonds) return;
  const unsigned lt = (1u << lane) - 1u;
  const int a0 = u2d[u], a1 = rev[a0];
  int t_out = trip_ptr[u], s_out = trip_src_ptr[u];
  for (int s = 0; s < 2; ++s) {
    const int a = s == 0 ? a0 : a1;
    if (a < 0) continue;
    const int fa = flag[a], c = center[a];
    const int e0 = edge_ptr[c], e1 = edge_ptr[c + 1];
    if (fa & 1) {  // target rows (c, u, a, bond(b), b) for b != a with length < lc
      for (int eb = e0; eb < e1; eb += 32) {
        const int b = eb + lane;
        const bool ok = b < e1 && b != a && (flag[b] & 2);
        const unsigned m = __ballot_sync(0xffffffffu, ok);
        if (ok) {
          int32_t* row = line_graph + 5 * (size_t)(t_out + __popc(m & lt));
          row[0] = c; row[1] = u; row[2] = a; row[3] = d2u[b]; row[4] = b;
        }
        t_out += __popc(m);
      }
    }
    if (fa & 2) {  // rows whose source edge is a: targets t != a at the same centre
      const int rank_a = edge_rank[2 * a];
      for (int eb = e0; eb < e1; eb += 32) {
        const int t = eb + lane;
        const bool ok = t < e1 && t != a && (flag[t] & 1);
        const unsigned m = __ballot_sync(0xffffffffu, ok);
        if (ok) {
          const int ut = d2u[t], tf = u2d[ut];
          int side_off = 0;
          if (t != tf) side_off = atom_counts[2 * center[tf]] - ((flag[tf] >> 1) & 1);
          const int row = trip_ptr[ut] + side_off + rank_a - ((t < a && (flag[t] & 2)) ? 1 : 0);
          src_perm[s_out + __popc(m & lt)] = row;
        }
        s_out += __popc(m);
      }
    }
  }
}

static int check_graph(const mb_graph* g) {
  if (!g || g->n_atoms <= 0 || g->n_struct <= 0 || g->n_cells <= 0) return MB_ERR_INVALID;
  if (!g->cart || !g->lattice || !g->inv_lattice || !g->atom_struct || !g->grid) return MB_ERR_INVALID;
  if (!g->cell_ptr || !g->cell_fill || !g->cell_atoms || !g->atom_cell || !g->atom_wrap || !g->scan_tmp ||
      !g->status || !g->edge_ptr)
    return MB_ERR_INVALID;
  return MB_OK;
}

}  // namespace mb

using namespace mb;

extern "C" size_t mb_graph_scan_tmp_len(int64_t n) { return (size_t)(n / SCAN_CHUNK + 4); }

extern "C" int mb_graph_count_edges(mb_graph* g, void* stream_) {
  cudaStream_t s = (cudaStream_t)stream_;
  int rc = check_graph(g);
  if (rc) return rc;
  const int n = g->n_atoms, tb = 128;
  MB_CUDA_CHECK(cudaMemsetAsync(g->cell_ptr, 0, sizeof(int32_t) * (size_t)(g->n_cells + 1), s));
  MB_CUDA_CHECK(cudaMemsetAsync(g->cell_fill, 0, sizeof(int32_t) * (size_t)g->n_cells, s));
  MB_CUDA_CHECK(cudaMemsetAsync(g->status, 0, sizeof(int32_t) * 8, s));
  k_bin_count<<<cdiv(n, tb), tb, 0, s>>>(n, g->cart, g->inv_lattice, g->atom_struct, g->grid, g->atom_cell,
                                         g->atom_wrap, g->cell_ptr);
  MB_LAUNCH_CHECK("k_bin_count");
  rc = scan_exclusive(g->cell_ptr, g->cell_ptr, g->n_cells, g->scan_tmp, s);
  if (rc) return rc;
  k_bin_fill<<<cdiv(n, tb), tb, 0, s>>>(n, g->atom_cell, g->cell_ptr, g->cell_fill, g->cell_atoms);
  k_neighbors<false><<<cdiv((long long)n * 32, tb), tb, 0, s>>>(
      n, g->cutoff, g->tol, g->cart, g->lattice, g->atom_struct, g->grid, g->atom_cell, g->atom_wrap, g->cell_ptr,
      g->cell_atoms, g->edge_ptr, nullptr, nullptr, g->status);
  MB_LAUNCH_CHECK("k_neighbors<count>");
  rc = scan_exclusive(g->edge_ptr, g->edge_ptr, n, g->scan_tmp, s);
  if (rc) return rc;
  int32_t total = 0, st[8];
  MB_CUDA_CHECK(cudaMemcpyAsync(&total, g->edge_ptr + n, sizeof(int32_t), cudaMemcpyDeviceToHost, s));
  MB_CUDA_CHECK(cudaMemcpyAsync(st, g->status, sizeof(st), cudaMemcpyDeviceToHost, s));
  MB_CUDA_CHECK(cudaStreamSynchronize(s));
  if (total < 0) return MB_ERR_OVERFLOW;
  g->n_edges = total;
  if (st[ST_ISOLATED]) return MB_ERR_ISOLATED;
  return MB_OK;
}

extern "C" int mb_graph_build_edges(mb_graph* g, void* stream_) {
  cudaStream_t s = (cudaStream_t)stream_;
  int rc = check_graph(g);
  if (rc) return rc;
  const int n = g->n_atoms, ne = g->n_edges, tb = 128;
  if (ne <= 0 || (ne & 1)) return ne <= 0 ? MB_ERR_INVALID : MB_ERR_UNPAIRED;
  if (!g->key_unsorted || !g->dist_unsorted || !g->key || !g->atom_counts || !g->edge_rank || !g->bond_counts ||
      !g->edge_flag || !g->center || !g->neighbor || !g->image || !g->dist || !g->rev || !g->d2u || !g->u2d ||
      !g->trip_ptr || !g->trip_src_ptr)
    return MB_ERR_INVALID;
  k_neighbors<true><<<cdiv((long long)n * 32, tb), tb, 0, s>>>(
      n, g->cutoff, g->tol, g->cart, g->lattice, g->atom_struct, g->grid, g->atom_cell, g->atom_wrap, g->cell_ptr,
      g->cell_atoms, g->edge_ptr, g->key_unsorted, g->dist_unsorted, g->status);
  MB_LAUNCH_CHECK("k_neighbors<fill>");
  k_sort_edges<<<cdiv((long long)n * 32, tb), tb, 0, s>>>(n, g->edge_ptr, g->key_unsorted, g->dist_unsorted, g->key,
                                                         g->dist, g->center, g->neighbor, g->image);
  // edge_rank doubles as scratch here: [0, ne) first-of-pair flags, [ne, 2ne+1) their scan
  int32_t* first_flag = g->edge_rank;
  int32_t* first_rank = g->edge_rank + ne;
  k_pair_edges<<<cdiv(ne, tb), tb, 0, s>>>(ne, g->edge_ptr, g->key, g->center, g->rev, first_flag, g->status);
  MB_LAUNCH_CHECK("k_pair_edges");
  rc = scan_exclusive(first_flag, first_rank, ne, g->scan_tmp, s);
  if (rc) return rc;
  int32_t nb = 0, st[8];
  MB_CUDA_CHECK(cudaMemcpyAsync(&nb, first_rank + ne, sizeof(int32_t), cudaMemcpyDeviceToHost, s));
  MB_CUDA_CHECK(cudaMemcpyAsync(st, g->status, sizeof(st), cudaMemcpyDeviceToHost, s));
  MB_CUDA_CHECK(cudaStreamSynchronize(s));
  if (st[ST_IMAGE_OVERFLOW]) return MB_ERR_OVERFLOW;
  if (st[ST_UNPAIRED] || nb * 2 != ne) return MB_ERR_UNPAIRED;
  g->n_bonds = nb;
  k_number_bonds<<<cdiv(ne, tb), tb, 0, s>>>(ne, g->rev, first_rank, g->d2u, g->u2d);
  k_edge_flags<<<cdiv(ne, tb), tb, 0, s>>>(ne, g->line_cutoff, g->dist, g->rev, g->edge_flag);
  MB_LAUNCH_CHECK("k_edge_flags");
  // first_rank is dead from here on: edge_rank takes its final meaning
  k_edge_ranks<<<cdiv((long long)n * 32, tb), tb, 0, s>>>(n, g->edge_ptr, g->edge_flag, g->edge_rank, g->atom_counts);
  int32_t* tgt_count = g->bond_counts;
  int32_t* src_count = g->bond_counts + (nb + 1);
  k_bond_counts<<<cdiv(nb, tb), tb, 0, s>>>(nb, g->u2d, g->rev, g->center, g->edge_flag, g->atom_counts, tgt_count,
                                            src_count);
  MB_LAUNCH_CHECK("k_bond_counts");
  rc = scan_exclusive(tgt_count, g->trip_ptr, nb, g->scan_tmp, s);
  if (rc) return rc;
  rc = scan_exclusive(src_count, g->trip_src_ptr, nb, g->scan_tmp, s);
  if (rc) return rc;
  int32_t nt = 0, nt2 = 0;
  MB_CUDA_CHECK(cudaMemcpyAsync(&nt, g->trip_ptr + nb, sizeof(int32_t), cudaMemcpyDeviceToHost, s));
  MB_CUDA_CHECK(cudaMemcpyAsync(&nt2, g->trip_src_ptr + nb, sizeof(int32_t), cudaMemcpyDeviceToHost, s));
  MB_CUDA_CHECK(cudaStreamSynchronize(s));
  if (nt < 0) return MB_ERR_OVERFLOW;
  if (nt != nt2) return MB_ERR_INVALID;
  g->n_triplets = nt;
  return MB_OK;
}

extern "C" int mb_graph_build_triplets(mb_graph* g, void* stream_) {
  cudaStream_t s = (cudaStream_t)stream_;
  int rc = check_graph(g);
  if (rc) return rc;
  if (g->n_triplets == 0) return MB_OK;
  if (!g->line_graph || !g->trip_src_perm || g->n_bonds <= 0) return MB_ERR_INVALID;
  const int tb = 128;
  k_fill_triplets<<<cdiv((long long)g->n_bonds * 32, tb), tb, 0, s>>>(
      g->n_bonds, g->edge_ptr, g->u2d, g->rev, g->center, g->d2u, g->edge_flag, g->edge_rank, g->atom_counts,
      g->trip_ptr, g->trip_src_ptr, g->line_graph, g->trip_src_perm);
  MB_LAUNCH_CHECK("k_fill_triplets");
  return MB_OK;
}
