// Periodic radius graph, bond graph and line graph (angle triplets) on the GPU: ONE cooperative kernel per batch.
//
// Integer / indexing work, HBM-bound.  The inclusion tests run in float64 with explicit round-to-nearest
// intrinsics (no FMA contraction) in a fixed operation order, so membership is decided by exactly the same numbers
// as a NumPy evaluation of the same formula.
//
// The whole pipeline is a single persistent kernel (cudaLaunchCooperativeKernel, as many CTAs as are co-resident)
// whose phases are separated by grid-wide barriers, so a build is one launch and no host synchronisation: every
// count stays on the device (counts[]), the outputs go into caller-supplied capacity buffers, and a capacity that
// turns out too small is reported in counts[] (the caller enlarges the buffer and calls again).
//
//   bin atoms into cells -> per-atom neighbour count (warp per atom in cell order; the atoms of each visited cell
//   pass through a shared-memory stage, ballot compaction) -> scan -> fill -> per-atom rank sort by
//   (neighbour, image) -> reverse-edge
//   search (binary search inside the neighbour's own segment) -> bond numbering (scan of "first of its pair" flags)
//   -> per-bond triplet counts -> scans -> triplet fill grouped by target bond + permutation grouped by source bond.
#include <cooperative_groups.h>
#include "common.cuh"

namespace cg = cooperative_groups;

namespace mb {

constexpr int GB_THREADS = 1024;  // one CTA per SM: a grid-wide barrier costs less the fewer CTAs take part
constexpr int SCAN_ITEMS = 8;  // per thread
constexpr int SCAN_CHUNK = GB_THREADS * SCAN_ITEMS;

// counts[] layout (device, int32[16]); also the status block the caller reads back
enum {
  CT_EDGES = 0, CT_BONDS = 1, CT_TRIPLETS = 2, CT_ISOLATED = 3, CT_IMAGE_OVERFLOW = 4, CT_UNPAIRED = 5,
  CT_EDGE_CAPACITY = 6, CT_TRIPLET_CAPACITY = 7, CT_TRIPLETS_BY_SOURCE = 8, CT_CANDIDATES_UNUSABLE = 9
};

// ---------------------------------------------------------------- block / grid exclusive scan
__device__ __forceinline__ int block_exclusive_scan(int v, int* total) {
  __shared__ int warp_sums[GB_THREADS / 32];
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
    int s = lane < GB_THREADS / 32 ? warp_sums[lane] : 0;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      int y = __shfl_up_sync(0xffffffffu, s, o);
      if (lane >= o) s += y;
    }
    if (lane < GB_THREADS / 32) warp_sums[lane] = s;  // inclusive over warps
    if (lane == GB_THREADS / 32 - 1) block_total = s;
  }
  __syncthreads();
  int prefix = (w > 0 ? warp_sums[w - 1] : 0) + x - v;
  *total = block_total;
  __syncthreads();
  return prefix;
}

// Exclusive scan of in[0..n) into out[0..n], out[n] = total; in may alias out; n is the same in every thread.
// Two steps separated by a grid barrier: per-chunk sums, then every block adds up the sums of the chunks in front of
// its own (a few thousand values at most) and applies them.  A second array can ride along (in2 / out2, same n).
__device__ void grid_scan(cg::grid_group& grid, const int32_t* in, int32_t* out, int64_t n, int32_t* tmp,
                          const int32_t* in2 = nullptr, int32_t* out2 = nullptr) {
  const int n_chunks = (int)((n + SCAN_CHUNK - 1) / SCAN_CHUNK);
  int32_t* const tmp2 = tmp + n_chunks;
  for (int ch = blockIdx.x; ch < n_chunks; ch += gridDim.x) {
    const int64_t base = (int64_t)ch * SCAN_CHUNK + (int64_t)threadIdx.x * SCAN_ITEMS;
    int s = 0, s2 = 0;
#pragma unroll
    for (int k = 0; k < SCAN_ITEMS; ++k)
      if (base + k < n) {
        s += in[base + k];
        if (in2) s2 += in2[base + k];
      }
    int total;
    block_exclusive_scan(s, &total);
    if (threadIdx.x == 0) tmp[ch] = total;
    if (in2) {
      block_exclusive_scan(s2, &total);
      if (threadIdx.x == 0) tmp2[ch] = total;
    }
  }
  if (n_chunks == 0 && blockIdx.x == 0 && threadIdx.x == 0) {
    out[0] = 0;
    if (out2) out2[0] = 0;
  }
  grid.sync();
  for (int ch = blockIdx.x; ch < n_chunks; ch += gridDim.x) {
    // sum of the chunk totals in front of this chunk
    int part = 0, part2 = 0;
    for (int i = threadIdx.x; i < ch; i += GB_THREADS) {
      part += tmp[i];
      if (in2) part2 += tmp2[i];
    }
    int offset, offset2 = 0, dummy;
    block_exclusive_scan(part, &offset);
    if (in2) block_exclusive_scan(part2, &offset2);
    const int64_t base = (int64_t)ch * SCAN_CHUNK + (int64_t)threadIdx.x * SCAN_ITEMS;
    int v[SCAN_ITEMS], v2[SCAN_ITEMS];
    int s = 0, s2 = 0;
#pragma unroll
    for (int k = 0; k < SCAN_ITEMS; ++k) {
      v[k] = base + k < n ? in[base + k] : 0;
      v2[k] = (in2 && base + k < n) ? in2[base + k] : 0;
      s += v[k];
      s2 += v2[k];
    }
    int total, total2 = 0;
    int p = block_exclusive_scan(s, &total) + offset;
    int p2 = in2 ? block_exclusive_scan(s2, &total2) + offset2 : 0;
    (void)dummy;
#pragma unroll
    for (int k = 0; k < SCAN_ITEMS; ++k) {
      if (base + k < n) {
        out[base + k] = p;
        if (in2) out2[base + k] = p2;
      }
      p += v[k];
      p2 += v2[k];
    }
    if (ch == n_chunks - 1 && threadIdx.x == 0) {
      out[n] = offset + total;
      if (in2) out2[n] = offset2 + total2;
    }
  }
  grid.sync();
}

// ---------------------------------------------------------------- helpers
__device__ __forceinline__ int floor_div(int a, int b) {
  int q = a / b;
  return (a % b != 0 && ((a < 0) != (b < 0))) ? q - 1 : q;
}

__device__ __forceinline__ uint64_t pack_key(int j, int n0, int n1, int n2) {
  return ((uint64_t)(uint32_t)j << 24) | ((uint64_t)(uint32_t)(n0 + 128) << 16) |
         ((uint64_t)(uint32_t)(n1 + 128) << 8) | (uint64_t)(uint32_t)(n2 + 128);
}

// Neighbour search of one atom by one warp.  The atoms of a visited cell pass through a per-warp shared-memory
// stage, 32 at a time (index, wrap count and position: one coalesced fetch per round, then every lane tests one
// staged candidate); atoms are taken in cell order, so the warps of a CTA work on neighbouring atoms and their
// fetches hit the same lines.  FILL = false counts (edge_ptr[i] = number of neighbours of atom i), FILL = true
// writes packed keys and distances from edge_ptr[i] on.  Both passes walk the candidates in the same order.
struct CellStage {
  int j[32];
  int4 wrap[32];
  double x[32], y[32], z[32];
};

template <bool FILL>
__device__ __forceinline__ void neighbors_of_atom(const mb_graph& g, int i, int lane, CellStage& st) {
  const int b = g.atom_struct[i];
  const int32_t* gr = g.grid + 8 * b;
  const int g0 = gr[0], g1 = gr[1], g2 = gr[2], s0 = gr[3], s1 = gr[4], s2 = gr[5], base = gr[6];
  double L[9];
#pragma unroll
  for (int k = 0; k < 9; ++k) L[k] = g.lattice[9 * b + k];
  const double xi = g.cart[3 * i], yi = g.cart[3 * i + 1], zi = g.cart[3 * i + 2];
  const int4 ci = reinterpret_cast<const int4*>(g.atom_cell)[i];
  const int4 wi = reinterpret_cast<const int4*>(g.atom_wrap)[i];
  const int out_base = FILL ? g.edge_ptr[i] : 0;
  const double cutoff = g.cutoff, tol = g.tol;
  int count = 0;
  bool bad_image = false;
  for (int d0 = -s0; d0 <= s0; ++d0) {
    int c0 = ci.x + d0;
    const int h0 = floor_div(c0, g0);
    c0 -= h0 * g0;
    for (int d1 = -s1; d1 <= s1; ++d1) {
      int c1 = ci.y + d1;
      const int h1 = floor_div(c1, g1);
      c1 -= h1 * g1;
      for (int d2 = -s2; d2 <= s2; ++d2) {
        int c2 = ci.z + d2;
        const int h2 = floor_div(c2, g2);
        c2 -= h2 * g2;
        const int cell = base + (c0 * g1 + c1) * g2 + c2;
        const int p0 = g.cell_ptr[cell], p1 = g.cell_ptr[cell + 1];
        // a structure with one cell per axis names the same atoms at every offset: they stay staged
        const bool restage = !(g0 == 1 && g1 == 1 && g2 == 1 && p1 - p0 <= 32 && (d0 != -s0 || d1 != -s1 || d2 != -s2));
        for (int pb = p0; pb < p1; pb += 32) {
          const int p = pb + lane;
          if (restage) {
            __syncwarp();
            if (p < p1) {
              const int jj = g.cell_atoms[p];
              st.j[lane] = jj;
              st.wrap[lane] = reinterpret_cast<const int4*>(g.atom_wrap)[jj];
              st.x[lane] = g.cart[3 * jj];
              st.y[lane] = g.cart[3 * jj + 1];
              st.z[lane] = g.cart[3 * jj + 2];
            }
            __syncwarp();
          }
          bool ok = false;
          int j = 0, n0 = 0, n1 = 0, n2 = 0;
          double d = 0.0;
          if (p < p1) {
            j = st.j[lane];
            const int4 wj = st.wrap[lane];
            n0 = h0 - wj.x + wi.x;
            n1 = h1 - wj.y + wi.y;
            n2 = h2 - wj.z + wi.z;
            const double f0 = (double)n0, f1 = (double)n1, f2 = (double)n2;
            // s = (n0*L0 + n1*L1) + n2*L2 ; dx = (x_j + s) - x_i ; no FMA contraction
            const double sx = __dadd_rn(__dadd_rn(__dmul_rn(f0, L[0]), __dmul_rn(f1, L[3])), __dmul_rn(f2, L[6]));
            const double sy = __dadd_rn(__dadd_rn(__dmul_rn(f0, L[1]), __dmul_rn(f1, L[4])), __dmul_rn(f2, L[7]));
            const double sz = __dadd_rn(__dadd_rn(__dmul_rn(f0, L[2]), __dmul_rn(f1, L[5])), __dmul_rn(f2, L[8]));
            const double dx = __dsub_rn(__dadd_rn(st.x[lane], sx), xi);
            const double dy = __dsub_rn(__dadd_rn(st.y[lane], sy), yi);
            const double dz = __dsub_rn(__dadd_rn(st.z[lane], sz), zi);
            const double q = __dadd_rn(__dadd_rn(__dmul_rn(dx, dx), __dmul_rn(dy, dy)), __dmul_rn(dz, dz));
            d = __dsqrt_rn(q);
            ok = (d > tol) && (d <= cutoff);
          }
          const unsigned mask = __ballot_sync(0xffffffffu, ok);
          if (ok) {
            if (n0 < -127 || n0 > 127 || n1 < -127 || n1 > 127 || n2 < -127 || n2 > 127) bad_image = true;
            if (FILL) {
              const int pos = out_base + count + __popc(mask & ((1u << lane) - 1u));
              if (pos < g.cap_edges) {
                g.key_unsorted[pos] = pack_key(j, n0, n1, n2);
                g.dist_unsorted[pos] = d;
              }
            }
          }
          count += __popc(mask);
        }
      }
    }
  }
  __syncwarp();
  if (!FILL) {
    // the image range is checked in the counting pass: nothing is packed or paired when it fails
    if (__any_sync(0xffffffffu, bad_image) && lane == 0) atomicOr(&g.counts[CT_IMAGE_OVERFLOW], 1);
    if (lane == 0) {
      g.edge_ptr[i] = count;
      if (count == 0) atomicAdd(&g.counts[CT_ISOLATED], 1);
    }
  }
}

// Neighbour search of one atom among its candidates (Verlet-skin reuse): the candidate list is the sorted directed-edge
// list of an earlier build with the cut-off enlarged by the skin, so it names every pair that can be inside the
// cut-off while no atom has moved by half the skin; the distance is recomputed with the same expression as above
// (same atom, same image, same operation order), so the surviving edges and their lengths are the fresh build's.
template <bool FILL>
__device__ __forceinline__ void neighbors_from_candidates(const mb_graph& g, int i, int lane) {
  const int b = g.atom_struct[i];
  double L[9];
#pragma unroll
  for (int k = 0; k < 9; ++k) L[k] = g.lattice[9 * b + k];
  const double xi = g.cart[3 * i], yi = g.cart[3 * i + 1], zi = g.cart[3 * i + 2];
  const int out_base = FILL ? g.edge_ptr[i] : 0;
  const double cutoff = g.cutoff, tol = g.tol;
  const int c0 = g.cand_ptr[i], c1 = g.cand_ptr[i + 1];
  int count = 0;
  for (int cb = c0; cb < c1; cb += 32) {
    const int c = cb + lane;
    bool ok = false;
    int j = 0, n0 = 0, n1 = 0, n2 = 0;
    double d = 0.0;
    if (c < c1) {
      j = g.cand_nbr[c];
      n0 = g.cand_img[3 * c], n1 = g.cand_img[3 * c + 1], n2 = g.cand_img[3 * c + 2];
      const double f0 = (double)n0, f1 = (double)n1, f2 = (double)n2;
      const double sx = __dadd_rn(__dadd_rn(__dmul_rn(f0, L[0]), __dmul_rn(f1, L[3])), __dmul_rn(f2, L[6]));
      const double sy = __dadd_rn(__dadd_rn(__dmul_rn(f0, L[1]), __dmul_rn(f1, L[4])), __dmul_rn(f2, L[7]));
      const double sz = __dadd_rn(__dadd_rn(__dmul_rn(f0, L[2]), __dmul_rn(f1, L[5])), __dmul_rn(f2, L[8]));
      const double dx = __dsub_rn(__dadd_rn(g.cart[3 * j], sx), xi);
      const double dy = __dsub_rn(__dadd_rn(g.cart[3 * j + 1], sy), yi);
      const double dz = __dsub_rn(__dadd_rn(g.cart[3 * j + 2], sz), zi);
      const double q = __dadd_rn(__dadd_rn(__dmul_rn(dx, dx), __dmul_rn(dy, dy)), __dmul_rn(dz, dz));
      d = __dsqrt_rn(q);
      ok = (d > tol) && (d <= cutoff);
    }
    const unsigned mask = __ballot_sync(0xffffffffu, ok);
    if (FILL && ok) {
      const int pos = out_base + count + __popc(mask & ((1u << lane) - 1u));
      if (pos < g.cap_edges) {
        g.key_unsorted[pos] = pack_key(j, n0, n1, n2);
        g.dist_unsorted[pos] = d;
      }
    }
    count += __popc(mask);
  }
  if (!FILL && lane == 0) {
    g.edge_ptr[i] = count;
    if (count == 0) atomicAdd(&g.counts[CT_ISOLATED], 1);
  }
}

// ---------------------------------------------------------------- the kernel
__global__ void __launch_bounds__(GB_THREADS, 1) k_graph_build(const mb_graph g) {
  cg::grid_group grid = cg::this_grid();
  __shared__ CellStage stage[GB_THREADS / 32];
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x, nth = (int64_t)gridDim.x * blockDim.x;
  const int warp_g = (int)(tid >> 5), n_warps = (int)(nth >> 5);
  const int n_atoms = g.n_atoms, n_cells = g.n_cells;
  int32_t* const counts = g.counts;
  // A conditional build (the candidate list of a Verlet-skin loop is rebuilt only when an atom has moved too far):
  // every thread reads the same word, so the whole grid stays or leaves, before any barrier and any write.
  if (g.run_if && *g.run_if == 0) return;
  const bool from_candidates = g.cand_ptr != nullptr;
  if (from_candidates) {
    // the candidate list is usable only if the build that made it ran to its end
    const int32_t* cc = g.cand_counts;
    const bool usable = cc[CT_EDGES] > 0 && !cc[CT_EDGE_CAPACITY] && !cc[CT_IMAGE_OVERFLOW] && !cc[CT_ISOLATED] &&
                        !(cc[CT_EDGES] & 1);
    if (!usable) {
      if (tid < 16) counts[tid] = tid == CT_CANDIDATES_UNUSABLE ? 1 : 0;
      return;
    }
  }

  // ---- clear the cell counters and the status block
  if (!from_candidates) {
    for (int64_t i = tid; i <= n_cells; i += nth) g.cell_ptr[i] = 0;
    for (int64_t i = tid; i < n_cells; i += nth) g.cell_fill[i] = 0;
  }
  if (tid < 16) counts[tid] = 0;
  grid.sync();

  if (from_candidates) {
    for (int i = warp_g; i < n_atoms; i += n_warps) neighbors_from_candidates<false>(g, i, lane);
    grid.sync();
  } else {
  // ---- bin the atoms
  for (int64_t i = tid; i < n_atoms; i += nth) {
    const int b = g.atom_struct[i];
    const double* inv = g.inv_lattice + 9 * b;
    const int32_t* gr = g.grid + 8 * b;
    const double x = g.cart[3 * i], y = g.cart[3 * i + 1], z = g.cart[3 * i + 2];
    int c[3], w[3];
#pragma unroll
    for (int k = 0; k < 3; ++k) {
      const double f = x * inv[k] + y * inv[3 + k] + z * inv[6 + k];
      double fl = floor(f);
      double fw = f - fl;
      if (fw >= 1.0) { fw = 0.0; fl += 1.0; }
      w[k] = (int)fl;
      const int ck = (int)(fw * (double)gr[k]);
      c[k] = ck < gr[k] - 1 ? ck : gr[k] - 1;
      if (c[k] < 0) c[k] = 0;
    }
    const int cell = gr[6] + (c[0] * gr[1] + c[1]) * gr[2] + c[2];
    reinterpret_cast<int4*>(g.atom_cell)[i] = make_int4(c[0], c[1], c[2], cell);
    reinterpret_cast<int4*>(g.atom_wrap)[i] = make_int4(w[0], w[1], w[2], 0);
    atomicAdd(&g.cell_ptr[cell], 1);
  }
  grid.sync();
  grid_scan(grid, g.cell_ptr, g.cell_ptr, n_cells, g.scan_tmp);
  for (int64_t i = tid; i < n_atoms; i += nth) {
    const int cell = g.atom_cell[4 * i + 3];
    g.cell_atoms[g.cell_ptr[cell] + atomicAdd(&g.cell_fill[cell], 1)] = (int)i;
  }
  grid.sync();

  // ---- directed edges: count, scan, fill
  for (int ii = warp_g; ii < n_atoms; ii += n_warps) neighbors_of_atom<false>(g, g.cell_atoms[ii], lane, stage[wib]);
  grid.sync();
  }
  grid_scan(grid, g.edge_ptr, g.edge_ptr, n_atoms, g.scan_tmp);
  const int ne = g.edge_ptr[n_atoms];
  if (tid == 0) counts[CT_EDGES] = ne;
  if (ne > g.cap_edges) {  // the same value in every thread: the whole grid leaves here
    if (tid == 0) counts[CT_EDGE_CAPACITY] = 1;
    return;
  }
  if (counts[CT_IMAGE_OVERFLOW] || counts[CT_ISOLATED] || ne <= 0 || (ne & 1)) {
    if (tid == 0 && (ne & 1)) counts[CT_UNPAIRED] = 1;
    return;
  }
  if (from_candidates) {
    for (int i = warp_g; i < n_atoms; i += n_warps) neighbors_from_candidates<true>(g, i, lane);
  } else {
    for (int ii = warp_g; ii < n_atoms; ii += n_warps) neighbors_of_atom<true>(g, g.cell_atoms[ii], lane, stage[wib]);
  }
  grid.sync();

  // ---- rank sort of each atom's out-edges by key (neighbour, image); warp per atom
  for (int i = warp_g; i < n_atoms; i += n_warps) {
    const int e0 = g.edge_ptr[i], n = g.edge_ptr[i + 1] - e0;
    for (int a = lane; a < n; a += 32) {
      const uint64_t k = g.key_unsorted[e0 + a];
      int rank = 0;
      for (int m = 0; m < n; ++m) rank += g.key_unsorted[e0 + m] < k ? 1 : 0;
      const int e = e0 + rank;
      g.key[e] = k;
      g.dist[e] = g.dist_unsorted[e0 + a];
      g.center[e] = i;
      g.neighbor[e] = (int)(k >> 24);
      g.image[3 * e + 0] = (int)((k >> 16) & 0xff) - 128;
      g.image[3 * e + 1] = (int)((k >> 8) & 0xff) - 128;
      g.image[3 * e + 2] = (int)(k & 0xff) - 128;
    }
  }
  grid.sync();
  if (g.flags & MB_GRAPH_EDGES_ONLY) return;  // a candidate build: the sorted directed-edge list is all that is read

  // ---- reverse edge of e = (i, j, n): the edge (j, i, -n), found by binary search in j's segment
  // edge_rank doubles as scratch here: [0, ne) first-of-pair flags, [ne, 2 ne + 1) their scan
  int32_t* const first_flag = g.edge_rank;
  int32_t* const first_rank = g.edge_rank + ne;
  for (int64_t e = tid; e < ne; e += nth) {
    const uint64_t k = g.key[e];
    const int i = g.center[e], j = (int)(k >> 24);
    const int n0 = (int)((k >> 16) & 0xff) - 128, n1 = (int)((k >> 8) & 0xff) - 128, n2 = (int)(k & 0xff) - 128;
    const uint64_t want = pack_key(i, -n0, -n1, -n2);
    int lo = g.edge_ptr[j], hi = g.edge_ptr[j + 1];
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      if (g.key[mid] < want) lo = mid + 1; else hi = mid;
    }
    int r = -1;
    if (lo < g.edge_ptr[j + 1] && g.key[lo] == want) r = lo;
    if (r < 0) atomicAdd(&counts[CT_UNPAIRED], 1);
    g.rev[e] = r;
    first_flag[e] = (r < 0 || r > e) ? 1 : 0;
  }
  grid.sync();
  grid_scan(grid, first_flag, first_rank, ne, g.scan_tmp);
  const int nb = first_rank[ne];
  if (tid == 0) counts[CT_BONDS] = nb;
  if (counts[CT_UNPAIRED] || nb * 2 != ne) {
    if (tid == 0) counts[CT_UNPAIRED] = counts[CT_UNPAIRED] ? counts[CT_UNPAIRED] : 1;
    return;
  }

  // ---- bond numbering and triplet eligibility of every directed edge
  // flag bit0: the bond of e may be a triplet target (first directed edge's length <= lc)
  //      bit1: e may be the source ("other") edge of a triplet (its own length < lc)
  for (int64_t e = tid; e < ne; e += nth) {
    const int r = g.rev[e];
    const int f = (r >= 0 && r < e) ? r : (int)e;
    const int u = first_rank[f];
    g.d2u[e] = u;
    if (f == e) g.u2d[u] = (int)e;
    g.edge_flag[e] = (uint8_t)((g.dist[f] <= g.line_cutoff ? 1 : 0) | (g.dist[e] < g.line_cutoff ? 2 : 0));
  }
  grid.sync();  // first_rank is dead from here on: edge_rank takes its final meaning

  // ---- per atom: exclusive ranks of source- / target-eligible edges inside the atom's segment
  for (int i = warp_g; i < n_atoms; i += n_warps) {
    const int e0 = g.edge_ptr[i], e1 = g.edge_ptr[i + 1];
    int ns = 0, nt = 0;
    for (int eb = e0; eb < e1; eb += 32) {
      const int e = eb + lane;
      const int f = e < e1 ? g.edge_flag[e] : 0;
      const unsigned ms = __ballot_sync(0xffffffffu, f & 2), mt = __ballot_sync(0xffffffffu, f & 1);
      const unsigned lt = (1u << lane) - 1u;
      if (e < e1) {
        g.edge_rank[2 * e] = ns + __popc(ms & lt);
        g.edge_rank[2 * e + 1] = nt + __popc(mt & lt);
      }
      ns += __popc(ms);
      nt += __popc(mt);
    }
    if (lane == 0) {
      g.atom_counts[2 * i] = ns;
      g.atom_counts[2 * i + 1] = nt;
    }
  }
  grid.sync();

  // ---- triplets per bond, as target and as source
  int32_t* const tgt_count = g.bond_counts;
  int32_t* const src_count = g.bond_counts + (nb + 1);
  for (int64_t u = tid; u < nb; u += nth) {
    const int a0 = g.u2d[u], a1 = g.rev[a0];
    int tc = 0, sc = 0;
    const int a[2] = {a0, a1};
#pragma unroll
    for (int s = 0; s < 2; ++s) {
      if (a[s] < 0) continue;
      const int f = g.edge_flag[a[s]], c = g.center[a[s]];
      if (f & 1) tc += g.atom_counts[2 * c] - ((f >> 1) & 1);
      if (f & 2) sc += g.atom_counts[2 * c + 1] - (f & 1);
    }
    tgt_count[u] = tc;
    src_count[u] = sc;
  }
  grid.sync();
  grid_scan(grid, tgt_count, g.trip_ptr, nb, g.scan_tmp, src_count, g.trip_src_ptr);
  const int ntr = g.trip_ptr[nb];
  if (tid == 0) {
    counts[CT_TRIPLETS] = ntr;
    counts[CT_TRIPLETS_BY_SOURCE] = g.trip_src_ptr[nb];
  }
  if (ntr > g.cap_triplets) {
    if (tid == 0) counts[CT_TRIPLET_CAPACITY] = 1;
    return;
  }
  if (ntr <= 0) return;

  // ---- warp per bond: rows with this bond as target (contiguous), and the ids of the rows that have it as source
  const unsigned lt = (1u << lane) - 1u;
  for (int u = warp_g; u < nb; u += n_warps) {
    const int a0 = g.u2d[u], a1 = g.rev[a0];
    int t_out = g.trip_ptr[u], s_out = g.trip_src_ptr[u];
    for (int s = 0; s < 2; ++s) {
      const int a = s == 0 ? a0 : a1;
      if (a < 0) continue;
      const int fa = g.edge_flag[a], c = g.center[a];
      const int e0 = g.edge_ptr[c], e1 = g.edge_ptr[c + 1];
      if (fa & 1) {  // target rows (c, u, a, bond(b), b) for b != a with length < lc
        for (int eb = e0; eb < e1; eb += 32) {
          const int b = eb + lane;
          const bool ok = b < e1 && b != a && (g.edge_flag[b] & 2);
          const unsigned m = __ballot_sync(0xffffffffu, ok);
          if (ok) {
            int32_t* row = g.line_graph + 5 * (size_t)(t_out + __popc(m & lt));
            row[0] = c; row[1] = u; row[2] = a; row[3] = g.d2u[b]; row[4] = b;
          }
          t_out += __popc(m);
        }
      }
      if (fa & 2) {  // rows whose source edge is a: targets t != a at the same centre
        const int rank_a = g.edge_rank[2 * a];
        for (int eb = e0; eb < e1; eb += 32) {
          const int t = eb + lane;
          const bool ok = t < e1 && t != a && (g.edge_flag[t] & 1);
          const unsigned m = __ballot_sync(0xffffffffu, ok);
          if (ok) {
            const int ut = g.d2u[t], tf = g.u2d[ut];
            int side_off = 0;
            if (t != tf) side_off = g.atom_counts[2 * g.center[tf]] - ((g.edge_flag[tf] >> 1) & 1);
            const int row = g.trip_ptr[ut] + side_off + rank_a - ((t < a && (g.edge_flag[t] & 2)) ? 1 : 0);
            g.trip_src_perm[s_out + __popc(m & lt)] = row;
          }
          s_out += __popc(m);
        }
      }
    }
  }
}

static int check_graph(const mb_graph* g) {
  if (!g || g->n_atoms <= 0 || g->n_struct <= 0 || g->n_cells <= 0 || g->cap_edges < 2 || g->cap_triplets < 0)
    return MB_ERR_INVALID;
  if (!g->cart || !g->lattice || !g->inv_lattice || !g->atom_struct || !g->grid || !g->counts) return MB_ERR_INVALID;
  const bool from_candidates = g->cand_ptr != nullptr, edges_only = (g->flags & MB_GRAPH_EDGES_ONLY) != 0;
  if (from_candidates && (!g->cand_nbr || !g->cand_img || !g->cand_counts)) return MB_ERR_INVALID;
  if (!from_candidates && (!g->cell_ptr || !g->cell_fill || !g->cell_atoms || !g->atom_cell || !g->atom_wrap))
    return MB_ERR_INVALID;
  if (!g->scan_tmp || !g->edge_ptr || !g->key_unsorted || !g->dist_unsorted || !g->key) return MB_ERR_INVALID;
  if (!g->center || !g->neighbor || !g->image || !g->dist) return MB_ERR_INVALID;
  if (edges_only) return MB_OK;
  if (!g->atom_counts || !g->edge_rank || !g->bond_counts || !g->edge_flag) return MB_ERR_INVALID;
  if (!g->rev || !g->d2u || !g->u2d || !g->trip_ptr || !g->trip_src_ptr ||
      (g->cap_triplets > 0 && (!g->line_graph || !g->trip_src_perm)))
    return MB_ERR_INVALID;
  return MB_OK;
}

}  // namespace mb

using namespace mb;

extern "C" size_t mb_graph_scan_tmp_len(int64_t n) { return (size_t)(2 * (n / SCAN_CHUNK + 4)); }

extern "C" int mb_graph_build(const mb_graph* g, void* stream_) {
  int rc = check_graph(g);
  if (rc) return rc;
  // as many CTAs as the device keeps resident at once (a cooperative launch requires it); per device
  static int grid_of_device[64];
  int dev = 0;
  MB_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return MB_ERR_INVALID;
  if (grid_of_device[dev] == 0) {
    int n_sm = 0, per_sm = 0;
    MB_CUDA_CHECK(cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev));
    MB_CUDA_CHECK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, k_graph_build, GB_THREADS, 0));
    if (per_sm < 1) return MB_ERR_CUDA;
    grid_of_device[dev] = n_sm;  // one CTA per SM (per_sm >= 1 was checked above)
  }
  mb_graph arg = *g;
  void* params[] = {&arg};
  MB_CUDA_CHECK(cudaLaunchCooperativeKernel((const void*)k_graph_build, dim3(grid_of_device[dev]), dim3(GB_THREADS),
                                            params, 0, (cudaStream_t)stream_));
  return MB_OK;
}

// ---- Verlet-skin bookkeeping: has any atom moved by half the skin since the candidate list was built?
namespace mb {
__global__ void k_skin_check(int n_atoms, const double* __restrict__ cart, const double* __restrict__ ref, double limit2,
                             int32_t* flag) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  bool far = false;
  if (i < n_atoms) {
    const double dx = cart[3 * i] - ref[3 * i], dy = cart[3 * i + 1] - ref[3 * i + 1], dz = cart[3 * i + 2] - ref[3 * i + 2];
    const double d2 = dx * dx + dy * dy + dz * dz;
    far = !(d2 < limit2);  // also true for a NaN position: the full search then reports what it finds
  }
  if (__syncthreads_or(far) && threadIdx.x == 0) atomicOr(flag, 1);
}

// One CTA: the flag is cleared only after every thread has acted on it.
__global__ void __launch_bounds__(1024) k_skin_commit(int n_atoms, const double* __restrict__ cart, double* __restrict__ ref,
                                                      int32_t* flag) {
  const bool rebuilt = flag[0] != 0;
  if (rebuilt)
    for (int i = threadIdx.x; i < 3 * n_atoms; i += blockDim.x) ref[i] = cart[i];
  __syncthreads();
  if (threadIdx.x == 0 && rebuilt) {
    flag[0] = 0;
    flag[1] += 1;
  }
}
}  // namespace mb

extern "C" int mb_graph_skin_check(int32_t n_atoms, const double* cart, const double* cart_ref, double half_skin,
                                   int32_t* flag, void* stream_) {
  if (n_atoms <= 0 || !cart || !cart_ref || !flag || !(half_skin > 0.0)) return MB_ERR_INVALID;
  k_skin_check<<<(n_atoms + 255) / 256, 256, 0, (cudaStream_t)stream_>>>(n_atoms, cart, cart_ref, half_skin * half_skin, flag);
  MB_LAUNCH_CHECK("k_skin_check");
  return MB_OK;
}

extern "C" int mb_graph_skin_commit(int32_t n_atoms, const double* cart, double* cart_ref, int32_t* flag, void* stream_) {
  if (n_atoms <= 0 || !cart || !cart_ref || !flag) return MB_ERR_INVALID;
  k_skin_commit<<<1, 1024, 0, (cudaStream_t)stream_>>>(n_atoms, cart, cart_ref, flag);
  MB_LAUNCH_CHECK("k_skin_commit");
  return MB_OK;
}

extern "C" int mb_graph_status(const int32_t* counts_host) {
  if (!counts_host) return MB_ERR_INVALID;
  if (counts_host[CT_IMAGE_OVERFLOW]) return MB_ERR_OVERFLOW;
  if (counts_host[CT_ISOLATED]) return MB_ERR_ISOLATED;
  if (counts_host[CT_EDGES] < 0 || counts_host[CT_TRIPLETS] < 0) return MB_ERR_OVERFLOW;
  if (counts_host[CT_EDGE_CAPACITY] || counts_host[CT_TRIPLET_CAPACITY] || counts_host[CT_CANDIDATES_UNUSABLE])
    return MB_ERR_CAPACITY;
  if (counts_host[CT_UNPAIRED]) return MB_ERR_UNPAIRED;
  if (counts_host[CT_TRIPLETS] != counts_host[CT_TRIPLETS_BY_SOURCE]) return MB_ERR_INVALID;
  return MB_OK;
}
