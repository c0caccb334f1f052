// Fused gated MLP, forward (included by gemm.cu inside namespace mb, after gemm_persistent.cuh).
//
//   z1 = X W1^T + b1          [rows, 256] = core | gate pre-activations    (K = 128 n_src, gathered A as in k_gemm_ps)
//   z2 = SiLU(z1) (.) W2^T + b2   per branch: [rows, 128] x [128, 128]
//   h  = SiLU(RMSNorm(z2_core) w_core) * sigmoid(RMSNorm(z2_gate) w_gate)  (+ optional out2 = h + res_w * res)
//
// 3xBF16 arithmetic (see gemm_persistent.cuh).  One persistent CTA per SM.  The unit of work is (128-row tile, branch);
// a CTA takes row tiles blockIdx.x, + gridDim.x, ... and runs the core unit (even k) and then the gate unit (odd k) of
// each.  A unit is two chained contractions on one tensor-memory accumulator (unit k uses accumulator k % 3):
//
//   L1(k)   12 or 16 K chunks (of 32 floats) of X against rows 128 (k & 1).. of W1  ->  D (128 x 128 fp32)
//   mid(k)  four epilogue warps read D back (tcgen05.ld, thread = row), add b1, optionally write z1, apply SiLU,
//           split into bf16 hi / lo and store the result as the A operand of layer 2 into the four A buffers
//           (tcgen05.st): z1 never travels through shared or global memory on its way to layer 2
//   L2(k)   4 K chunks against rows 128 (k & 1).. of W2, written over D (every column of D has been read by then)
//   epi(k)  the same four warps: pass 1 reads D (+ b2, optional z2 store) for the row's sum of squares, pass 2 reads
//           it again, normalises and activates; the core unit parks c = SiLU(.) in the output row, the gate unit
//           reads it back, multiplies by sigmoid(.) and writes h / out2.
//
// kind = MB_MLP_PLAIN runs the same pipeline for a plain two-layer MLP  y = W2 SiLU(W1 x + b1) + b2  (+ out2 = y +
// res_w * res): one unit per row tile (W1 [128, K], W2 [128, 128]), no normalisation, nothing parked; z1 is then the
// [rows, 128] pre-activation of the hidden layer.
//
// The eight epilogue warps form two groups of four (one warp per tensor-memory lane quarter, each owning whole rows):
// group 0 takes the even units, group 1 the odd ones.  While one group waits for DRAM in its epilogue the other
// prepares the next layer-2 operand, so the tensor pipe is not starved by the epilogue's memory traffic; with three
// accumulators an accumulator can stay with its epilogue for a whole extra unit before layer 1 needs it again.
// The tensor pipe executes L1(0) L1(1) L2(0) L1(2) L2(1) ... L1(n-1) L2(n-2) L2(n-1).  All roles walk that one chunk
// sequence (counter g): chunk g uses A buffer g % 4 and W-slot use g / 2, exactly as in k_gemm_ps.
//
// Tensor memory (512 columns): accumulators at 0, 128, 256; four A buffers of 32 columns (hi | lo) from 384.
// Shared memory: W ring 4 x 32 KB | producer patches 64 KB | per-channel constants 3.5 KB | barriers | descriptor.
// Every mbarrier wait is bounded; on expiry the status word is set, the role stops waiting and runs to the common exit.

struct alignas(64) GatedMaps { CUtensorMap w1[2]; CUtensorMap w2[2]; };  // hi, lo of W1 [256, K] and W2 [256, 128]

constexpr int GP_THREADS = PS_THREADS;
constexpr uint32_t GP_NB = 4;        // A buffers
constexpr uint32_t GP_A_BASE = 384;  // their first tensor-memory column
constexpr int GP_CONST_OFF = PS_RING_BYTES + PS_PATCH_BYTES;  // b1[256] b2[256] norm_core[128] norm_gate[128] res_w[128]
constexpr int GP_BAR_OFF = GP_CONST_OFF + 896 * 4;
constexpr int GP_DESC_OFF = GP_BAR_OFF + 448;
constexpr int GP_SMEM_BYTES = GP_DESC_OFF + (int)((sizeof(mb_gated_mlp) + 15) / 16 * 16);
constexpr float GP_RMS_EPS = 1.1920928955078125e-07f;  // nn.RMSNorm(eps=None): float32 machine epsilon
static_assert(GP_SMEM_BYTES <= 227 * 1024, "shared memory of one CTA");
static_assert(sizeof(mb_gated_mlp) % 4 == 0, "descriptor is copied word by word");

template <bool PLAIN>
__global__ void __launch_bounds__(GP_THREADS, 1)
k_gated_fwd(const __grid_constant__ mb_gated_mlp d_param, const __grid_constant__ GatedMaps maps) {
  constexpr uint32_t NB = GP_NB;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + GP_BAR_OFF);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + GP_BAR_OFF + 416);
  if ((smem_u32(smem) & 1023u) != 0) {  // the swizzled tiles need a 1024-byte aligned base
    if (threadIdx.x == 0) atomicOr(&g_gemm_status, 2);
    return;
  }
  // barriers: a_ready[4] (A chunk stored: 4 warps) | a_done[4] (its MMAs retired) | w_ready[4] (W slot landed) |
  //           w_done[4] (slot free) | d1_full[6] | d2_full[6] | d_free[6] (4 epilogue warps) | l2_free[2][4] |
  //           park_ready[4][2]
  // A parity wait can tell apart only the current and the preceding phase of a barrier, so every waiter must see
  // every phase of the barriers it waits on.  The MMA warp sees every chunk and the TMA warp every W-slot use.
  //   * The per-unit barriers d1_full / d2_full / d_free are indexed by k % 6: a barrier then always belongs to the
  //     same accumulator (k % 3) and the same epilogue group (k % 2), and completes once every six units.
  //   * The epilogue warps skip the layer-1 chunks: "the A buffer of layer-2 chunk c may be written" comes on
  //     l2_free[group][c], which completes once per unit of that group; it is committed with an earlier chunk that
  //     used the same buffer.
  //   * The producers skip the layer-2 chunks: they wait for the previous layer-1 phase to be complete (d1_full)
  //     before the first chunk of a phase that follows a layer-2 phase, so that a_done[b] is at most one phase
  //     away from the one they wait for.
  //   * park_ready[q][t & 1]: the core unit's parked values of lane quarter q and row tile t are in memory (group 0 ->
  //     group 1).  Group 0 can be two tiles ahead of group 1's wait (not three: layer 1 of its third tile needs the
  //     accumulator group 1 still holds), so two barriers alternate; each completes once per two tiles.
  const uint32_t a_ready = smem_u32(bars), a_done = smem_u32(bars + 4);
  const uint32_t w_ready = smem_u32(bars + 8), w_done = smem_u32(bars + 12);
  const uint32_t d1_full = smem_u32(bars + 16), d2_full = smem_u32(bars + 22), d_free = smem_u32(bars + 28);
  const uint32_t l2_free = smem_u32(bars + 34), park_ready = smem_u32(bars + 42);
  const uint32_t ring = smem_u32(smem);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const mb_gated_mlp& d = *reinterpret_cast<const mb_gated_mlp*>(smem + GP_DESC_OFF);
  constexpr bool plain = PLAIN;  // MB_MLP_PLAIN: one unit per row tile, branch 0 only
  {
    const uint32_t* src = reinterpret_cast<const uint32_t*>(&d_param);
    uint32_t* dst = reinterpret_cast<uint32_t*>(smem + GP_DESC_OFF);
    for (int i = tid; i < (int)(sizeof(mb_gated_mlp) / 4); i += GP_THREADS) dst[i] = src[i];
  }
  __syncthreads();
  // per-channel constants -> shared memory (missing biases read as 0, a missing residual weight as 1): the epilogue
  // warps fetch them per column group, and from global memory each fetch would be a dependent round trip
  float* const cst = reinterpret_cast<float*>(smem + GP_CONST_OFF);
  for (int i = tid; i < 896; i += GP_THREADS) {
    float v;
    if (i < 256) v = (d.b1 && !(plain && i >= 128)) ? d.b1[i] : 0.f;
    else if (i < 512) v = (d.b2 && !(plain && i >= 384)) ? d.b2[i - 256] : 0.f;
    else if (i < 640) v = plain ? 1.f : d.norm_core[i - 512];
    else if (i < 768) v = plain ? 1.f : d.norm_gate[i - 640];
    else v = d.res_w ? d.res_w[i - 768] : 1.f;
    cst[i] = v;
  }
  const int64_t n_rows = d.n_rows;
  const int n_row_tiles = (int)((n_rows + 127) >> 7);
  const int n_src = d.n_src, nch1 = 4 * n_src;
  const int first_rt = (int)blockIdx.x, step_rt = (int)gridDim.x;
  const int n_tiles_mine = (n_row_tiles - first_rt + step_rt - 1) / step_rt;  // the grid never exceeds the tile count
  const int n_units = plain ? n_tiles_mine : 2 * n_tiles_mine;
  const int unit_shift = plain ? 0 : 1;  // row tile of unit k = k >> unit_shift, branch = plain ? 0 : k & 1
  const int n_phases = 2 * n_units;
  // phase p of the tensor pipe's sequence -> (layer, unit)
  auto decode = [&](int p, bool& is_l2, int& k) {
    if (p == n_phases - 1) { is_l2 = true; k = n_units - 1; }
    else if (p == 0) { is_l2 = false; k = 0; }
    else if (p & 1) { is_l2 = false; k = (p + 1) >> 1; }
    else { is_l2 = true; k = (p >> 1) - 1; }
  };
  // first chunk of L2(k) in the chunk sequence
  auto l2_start = [&](int k) { return (uint32_t)((k + 2 < n_units ? k + 2 : n_units) * nch1 + 4 * k); };

  // ---- producer state (same gather as k_gemm_ps; both units of a row tile read the same rows)
  const int pw = (warp - PS_PROD_WARP0) & 7;
  const int par = pw >> 2, quarter = warp & 3;
  const int lr = lane >> 3, lc = lane & 7;
  const uint32_t patch0 = smem_u32(smem + PS_RING_BYTES + pw * (2 * 32 * 128));
  const uint32_t dst_even = patch0 + lr * 128 + ((lc ^ lr) << 4), dst_odd = patch0 + lr * 128 + ((lc ^ (lr | 4)) << 4);
  const float* a_ptr[8];
  int32_t a_row[8];
  int g_unit = 0, g_seg = 0, g_cnt = 0;
  bool g_second = false;
  auto resolve_rows = [&](int unit, int seg) {
    const int64_t row0 = (int64_t)(first_rt + (unit >> unit_shift) * step_rt) * 128;
    const int32_t* idx = d.src[seg].idx;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      int64_t r = row0 + quarter * 32 + lr + 4 * i;
      r = r < n_rows ? r : n_rows - 1;  // rows past the end repeat the last row; their results are never written
      a_row[i] = idx ? idx[r] : (int32_t)(r - row0);
    }
  };
  auto gather_next = [&]() {
    if (g_unit >= n_units) {
      asm volatile("cp.async.commit_group;" ::: "memory");
      return;
    }
    const uint32_t st = (uint32_t)(g_cnt & 1) * (32 * 128);
    const uint32_t de = dst_even + st, dq = dst_odd + st;
    if (!g_second) {
      const mb_src& s = d.src[g_seg];
      const float* base = s.ptr + s.col + lc * 4 + par * TC_BK;
      const int64_t ld = s.ld;
      const int64_t row0 = s.idx ? 0 : (int64_t)(first_rt + (g_unit >> unit_shift) * step_rt) * 128;
#pragma unroll
      for (int i = 0; i < 8; ++i) a_ptr[i] = base + (row0 + a_row[i]) * ld;
      MB_CP16(de, 0, a_ptr[0], 0);    MB_CP16(dq, 512, a_ptr[1], 0);  MB_CP16(de, 1024, a_ptr[2], 0); MB_CP16(dq, 1536, a_ptr[3], 0);
      MB_CP16(de, 2048, a_ptr[4], 0); MB_CP16(dq, 2560, a_ptr[5], 0); MB_CP16(de, 3072, a_ptr[6], 0); MB_CP16(dq, 3584, a_ptr[7], 0);
    } else {
      MB_CP16(de, 0, a_ptr[0], 256);    MB_CP16(dq, 512, a_ptr[1], 256);  MB_CP16(de, 1024, a_ptr[2], 256); MB_CP16(dq, 1536, a_ptr[3], 256);
      MB_CP16(de, 2048, a_ptr[4], 256); MB_CP16(dq, 2560, a_ptr[5], 256); MB_CP16(de, 3072, a_ptr[6], 256); MB_CP16(dq, 3584, a_ptr[7], 256);
      if (++g_seg == n_src) {
        g_seg = 0;
        ++g_unit;
      }
      if (g_unit < n_units) resolve_rows(g_unit, g_seg);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    ++g_cnt;
    g_second = !g_second;
  };

  if (warp == PS_MMA_WARP) {
    if (lane == 0) {
      for (int b = 0; b < 4; ++b) {
        mbar_init(a_ready + 8 * b, 4); mbar_init(a_done + 8 * b, 1);
        mbar_init(w_ready + 8 * b, 1); mbar_init(w_done + 8 * b, 1);
      }
      for (int b = 0; b < 8; ++b) { mbar_init(l2_free + 8 * b, 1); mbar_init(park_ready + 8 * b, 1); }
      for (int b = 0; b < 6; ++b) {
        mbar_init(d1_full + 8 * b, 1); mbar_init(d2_full + 8 * b, 1); mbar_init(d_free + 8 * b, 4);
      }
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncwarp();
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 :: "r"(smem_u32(tmem_slot)), "r"(PS_TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  } else if (warp >= PS_PROD_WARP0 && warp < PS_EPI_WARP0) {
    resolve_rows(0, 0);
    gather_next();
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  if (warp == PS_MMA_WARP) {
    // ---------------------------------------------------------------- MMA warp (warp-uniform, one elected lane issues)
    uint32_t elected;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(elected));
    const uint32_t tmem_u = __shfl_sync(0xffffffffu, tmem_base, 0);
    const uint32_t ring_u = __shfl_sync(0xffffffffu, ring, 0);
    bool alive = true;
    uint32_t g = 0;
    // Hand-over of the A buffers to the layer-2 writers (the epilogue warps): chunk t of layer-2 phase k_l2 may be
    // written once the chunk NB before it has retired, which is signalled on l2_free[k_l2 & 1][t].  The writers of a
    // group must have seen one completion before the next can happen, so the signal is never given before the same
    // chunk of the preceding layer-2 phase, which needs the other group's operand and comes after this group's
    // previous one: sig_first = max(first chunk of the phase - NB, first chunk of the preceding layer-2 phase).
    int k_l2 = 0;
    uint32_t sig_first = l2_start(0) - NB;  // n_units >= 2 and nch1 >= 4: never negative
    for (int p = 0; p < n_phases; ++p) {
      bool is_l2;
      int k;
      decode(p, is_l2, k);
      const int k6 = k % 6;
      const uint32_t d_tmem = tmem_u + 128u * (uint32_t)(k % 3);
      const int nch = is_l2 ? 4 : nch1;
      const uint32_t full_bar = (is_l2 ? d2_full : d1_full) + 8 * k6;
      for (int c = 0; c < nch; ++c, ++g) {
        const uint32_t ab = g % NB, wu = g >> 1, slot = wu & 3;
        if (c == 0 && is_l2) {
          // Layer 2 overwrites the accumulator that holds z1: its first MMA may issue only when all four operand
          // chunks have been read out of it and stored (each a_ready phase below implies that chunk's tcgen05.ld).
          for (uint32_t b = 0; b < 4; ++b)
            if (alive) alive = mbar_wait(a_ready + 8 * ((g + b) % NB), ((g + b) / NB) & 1);
        } else {
          if (alive) alive = mbar_wait(a_ready + 8 * ab, (g / NB) & 1);
        }
        if ((g & 1) == 0 && alive) alive = mbar_wait(w_ready + 8 * slot, (wu >> 2) & 1);
        // layer 1 of unit k overwrites the accumulator unit k - 3 left: its epilogue must have read it twice
        if (c == 0 && !is_l2 && k >= 3 && alive)
          alive = mbar_wait(d_free + 8 * ((k - 3) % 6), (uint32_t)(((k - 3) / 6) & 1));
        alive = __all_sync(0xffffffffu, alive);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t wb = ring_u + slot * 2 * TC_TILE_BYTES;
        const uint32_t ta = tmem_u + GP_A_BASE + 32u * ab;
        // < 4: this chunk's retirement frees layer-2 chunk t_l2 of unit k_l2
        const uint32_t t_l2 = k_l2 < n_units ? g - sig_first : 4u;
        if (elected) {
          issue_chunk_mmas<true>(d_tmem, ta, wb, g & 1, c == 0);
          asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                       :: "r"(a_done + 8 * ab) : "memory");
          if (g & 1)
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                         :: "r"(w_done + 8 * slot) : "memory");
          if (t_l2 < 4u)
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                         :: "r"(l2_free + 8 * (4 * (k_l2 & 1) + t_l2)) : "memory");
          if (c == nch - 1)
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                         :: "r"(full_bar) : "memory");
        }
        __syncwarp();
        if (t_l2 == 3u) {
          ++k_l2;
          const uint32_t by_buffer = l2_start(k_l2) - NB, by_order = l2_start(k_l2 - 1);
          sig_first = by_buffer > by_order ? by_buffer : by_order;
        }
      }
    }
  } else if (warp == PS_TMA_WARP) {
    // ---------------------------------------------------------------- TMA warp: W1 / W2 tiles (hi, lo), 4 chunks ahead
    uint32_t elected;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(elected));
    const uint32_t ring_u = __shfl_sync(0xffffffffu, ring, 0);
    bool alive = true;
    uint32_t wu = 0;  // W-slot uses issued so far
    for (int p = 0; p < n_phases && alive; ++p) {
      bool is_l2;
      int k;
      decode(p, is_l2, k);
      const int n_w = (is_l2 ? 4 : nch1) / 2;
      const int wrow = plain ? 0 : 128 * (k & 1);  // first weight row of this unit's branch
      const CUtensorMap* const m_hi = is_l2 ? &maps.w2[0] : &maps.w1[0];
      const CUtensorMap* const m_lo = is_l2 ? &maps.w2[1] : &maps.w1[1];
      for (int wi = 0; wi < n_w && alive; ++wi, ++wu) {
        const uint32_t slot = wu & 3;
        if (wu >= 4) alive = mbar_wait(w_done + 8 * slot, ((wu >> 2) - 1) & 1);
        alive = __all_sync(0xffffffffu, alive);
        if (!alive) break;
        const uint32_t bar = w_ready + 8 * slot;
        if (elected) {
          const uint32_t dst = ring_u + slot * 2 * TC_TILE_BYTES;
          asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(bar), "r"(2 * TC_TILE_BYTES) : "memory");
          tma_load_2d(dst, m_hi, bar, wi * 64, wrow);
          tma_load_2d(dst + TC_TILE_BYTES, m_lo, bar, wi * 64, wrow);
        }
        __syncwarp();
      }
    }
    if (!alive) {  // failure path only: no TMA write may still be in flight when the CTA's shared memory is released
      for (uint32_t i = wu >= 4 ? wu - 4 : 0; i < wu; ++i) mbar_wait(w_ready + 8 * (i & 3), (i >> 2) & 1);
    }
  } else if (warp >= PS_EPI_WARP0) {
    // ---------------------------------------------------------------- epilogue warps: mid(k) then epi(k) of every
    // other unit.  Warp (q, grp): rows 32 q.. of the tile (its tensor-memory lane quarter), all 128 columns of the
    // units k = grp, grp + 2, ... (grp 0: core branch, grp 1: gate branch); thread = row.
    const int e = warp - PS_EPI_WARP0, q = warp & 3, grp = e >> 2;
    const int br = plain ? 0 : grp;  // branch of this group's units
    const uint32_t lane_q = tmem_base + ((uint32_t)(q * 32) << 16);
    const float4* const b1s = reinterpret_cast<const float4*>(cst) + 32 * br;
    const float4* const b2s = reinterpret_cast<const float4*>(cst + 256) + 32 * br;
    const float4* const nws = reinterpret_cast<const float4*>(cst + 512 + 128 * br);
    const float4* const rws = reinterpret_cast<const float4*>(cst + 768);
    float* const z1 = d.z1;
    float* const z2 = d.z2;
    float* const hout = d.h;
    float* const out2 = d.out2;
    const float* const res = d.res;
    bool alive = true;
    for (int k = grp; k < n_units; k += 2) {
      const int k6 = k % 6;
      const uint32_t par6 = (uint32_t)((k / 6) & 1), part = (uint32_t)((k >> 1) & 1);
      const uint32_t park_bar = park_ready + 8 * (2 * q + (int)part), park_par = (uint32_t)((k >> 2) & 1);
      const int64_t row = (int64_t)(first_rt + (k >> unit_shift) * step_rt) * 128 + q * 32 + lane;
      const bool valid = row < n_rows;
      const uint32_t d_lane = lane_q + 128u * (uint32_t)(k % 3);
      // ------------------------------------------------ mid(k): z1 -> SiLU -> hi / lo -> A operand of layer 2
      if (alive) alive = mbar_wait(d1_full + 8 * k6, par6);
      alive = __all_sync(0xffffffffu, alive);
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t gl2 = l2_start(k);
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {  // K chunk of layer 2 = columns 32 c.. of this branch's z1
        float x[32];
        {
          uint32_t v[32];
          MB_TMEM_LD32(d_lane + 32u * c, v);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
          for (int i = 0; i < 32; ++i) x[i] = __uint_as_float(v[i]);
        }
#pragma unroll
        for (int jj = 0; jj < 8; ++jj) {  // same address in every lane: a broadcast read
          const float4 bv = b1s[8 * c + jj];
          x[4 * jj] += bv.x; x[4 * jj + 1] += bv.y; x[4 * jj + 2] += bv.z; x[4 * jj + 3] += bv.w;
        }
        if (z1 && valid) {
          float* zp = z1 + row * d.ld_z1 + 128 * br + 32 * c;
#pragma unroll
          for (int jj = 0; jj < 4; ++jj) {
            float o[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) o[i] = x[8 * jj + i];
            st8(zp + 8 * jj, o);
          }
        }
        __syncwarp();
        const uint32_t ab = (gl2 + (uint32_t)c) % NB;
        const uint32_t ta = lane_q + GP_A_BASE + 32u * ab;
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          float sx[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) sx[i] = silu_fast_f(x[16 * hh + i]);
          uint32_t hi[8], lo[8];
          split_bf16(sx, hi, lo);
          if (hh == 0) {
            if (alive) alive = mbar_wait(l2_free + 8 * (4 * grp + c), part);  // the A buffer may take this chunk
            __syncwarp();
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          }
          MB_TMEM_ST8(ta + 8 * hh, hi);
          MB_TMEM_ST8(ta + 16 + 8 * hh, lo);
        }
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(a_ready + 8 * ab);
      }
      // ------------------------------------------------ epi(k), pass 1: + b2, optional z2 store, sum of squares
      if (alive) alive = mbar_wait(d2_full + 8 * k6, par6);
      alive = __all_sync(0xffffffffu, alive);
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      float ss = 0.f;
#pragma unroll 1
      for (int c = 0; c < (plain ? 0 : 4); ++c) {
        float y[32];
        {
          uint32_t v[32];
          MB_TMEM_LD32(d_lane + 32u * c, v);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
          for (int i = 0; i < 32; ++i) y[i] = __uint_as_float(v[i]);
        }
#pragma unroll
        for (int jj = 0; jj < 8; ++jj) {
          const float4 bv = b2s[8 * c + jj];
          y[4 * jj] += bv.x; y[4 * jj + 1] += bv.y; y[4 * jj + 2] += bv.z; y[4 * jj + 3] += bv.w;
#pragma unroll
          for (int i = 0; i < 4; ++i) ss = fmaf(y[4 * jj + i], y[4 * jj + i], ss);
        }
        if (z2 && valid && alive) {
          float* zp = z2 + row * d.ld_z2 + 128 * br + 32 * c;
#pragma unroll
          for (int jj = 0; jj < 4; ++jj) {
            float o[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) o[i] = y[8 * jj + i];
            st8(zp + 8 * jj, o);
          }
        }
        __syncwarp();
      }
      const float rinv = plain ? 1.0f : rsqrtf(ss * (1.0f / 128.0f) + GP_RMS_EPS);
      // the core unit parks c = SiLU(.) in the output row; the gate unit's warp of the same lane quarter reads it back
      float* const park = hout ? hout + row * d.ld_h : out2 + row * d.ld_out2;
      if (grp == 1 && !plain) {
        if (alive) alive = mbar_wait(park_bar, park_par);
        alive = __all_sync(0xffffffffu, alive);
      }
      // ------------------------------------------------ pass 2: normalise, activate, write
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        float y[32];
        {
          uint32_t v[32];
          MB_TMEM_LD32(d_lane + 32u * c, v);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
          for (int i = 0; i < 32; ++i) y[i] = __uint_as_float(v[i]);
        }
        if (c == 3) {  // the accumulator has been read for the last time: layer 1 of unit k + 3 may overwrite it
          asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
          __syncwarp();
          if (lane == 0) mbar_arrive(d_free + 8 * k6);
        }
        if (alive && valid) {  // nothing to write for rows past the end (or after an expired wait)
#pragma unroll
        for (int jj = 0; jj < 8; ++jj) {
          const float4 bv = b2s[8 * c + jj], wv = nws[8 * c + jj];
          y[4 * jj] = (y[4 * jj] + bv.x) * rinv * wv.x;
          y[4 * jj + 1] = (y[4 * jj + 1] + bv.y) * rinv * wv.y;
          y[4 * jj + 2] = (y[4 * jj + 2] + bv.z) * rinv * wv.z;
          y[4 * jj + 3] = (y[4 * jj + 3] + bv.w) * rinv * wv.w;
        }
        if (plain) {
          // y = W2 SiLU(.) + b2 is the result: h and / or out2 = y + res_w * res (16 columns of the residual per round)
          const float* const rrow = out2 ? res + row * d.ld_res + 32 * c : nullptr;
          float* const orow = out2 ? out2 + row * d.ld_out2 + 32 * c : nullptr;
          float* const hrow = hout ? hout + row * d.ld_h + 32 * c : nullptr;
#pragma unroll
          for (int b = 0; b < 2; ++b) {
            float rr[2][8];
            if (out2) {
              ld8(rrow + 16 * b, rr[0]);
              ld8(rrow + 16 * b + 8, rr[1]);
            }
#pragma unroll
            for (int t = 0; t < 2; ++t) {
              const int jj = 2 * b + t;
              float o[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) o[i] = y[8 * jj + i];
              if (hout) st8(hrow + 8 * jj, o);
              if (out2) {
                const float4 ra = rws[8 * c + 2 * jj], rb = rws[8 * c + 2 * jj + 1];
                const float rw[8] = {ra.x, ra.y, ra.z, ra.w, rb.x, rb.y, rb.z, rb.w};
#pragma unroll
                for (int i = 0; i < 8; ++i) o[i] = fmaf(rw[i], rr[t][i], o[i]);
                st8(orow + 8 * jj, o);
              }
            }
          }
        } else if (grp == 0) {
#pragma unroll
          for (int jj = 0; jj < 4; ++jj) {
            float o[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) o[i] = silu_fast_f(y[8 * jj + i]);
            st8(park + 32 * c + 8 * jj, o);
          }
        } else {
          // 16 columns per round: the parked values and the residual row are requested together, so a round costs one
          // memory latency (both were touched by this SM a moment ago and sit in L2)
          const float* const rrow = out2 ? res + row * d.ld_res + 32 * c : nullptr;
          float* const orow = out2 ? out2 + row * d.ld_out2 + 32 * c : nullptr;
#pragma unroll
          for (int b = 0; b < 2; ++b) {
            float cp[2][8], rr[2][8];
            ld8(park + 32 * c + 16 * b, cp[0]);
            ld8(park + 32 * c + 16 * b + 8, cp[1]);
            if (out2) {
              ld8(rrow + 16 * b, rr[0]);
              ld8(rrow + 16 * b + 8, rr[1]);
            }
#pragma unroll
            for (int t = 0; t < 2; ++t) {
              const int jj = 2 * b + t;
              float o[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) o[i] = cp[t][i] * sigmoid_fast_f(y[8 * jj + i]);
              if (hout) st8(park + 32 * c + 8 * jj, o);
              if (out2) {
                const float4 ra = rws[8 * c + 2 * jj], rb = rws[8 * c + 2 * jj + 1];
                const float rw[8] = {ra.x, ra.y, ra.z, ra.w, rb.x, rb.y, rb.z, rb.w};
#pragma unroll
                for (int i = 0; i < 8; ++i) o[i] = fmaf(rw[i], rr[t][i], o[i]);
                st8(orow + 8 * jj, o);
              }
            }
          }
        }
        }
        __syncwarp();  // the lanes meet again before the next (warp-wide) tensor-memory load
      }
      if (grp == 0 && !plain) {  // the parked values of this lane quarter are complete and visible to the CTA
        __threadfence_block();
        __syncwarp();
        if (lane == 0) mbar_arrive(park_bar);
      }
      __syncwarp();
    }
  } else {
    // ---------------------------------------------------------------- producers (layer-1 chunks only)
    const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16);
    bool alive = true;
    uint32_t g = 0;
    int n = 0;
    int act_mask = 0;
#pragma unroll
    for (int s = 0; s < 4; ++s) act_mask |= (s < n_src && d.src[s].act) ? (1 << s) : 0;
    for (int p = 0; p < n_phases; ++p) {
      bool is_l2;
      int k;
      decode(p, is_l2, k);
      if (is_l2) {
        g += 4;
        continue;
      }
      if (k >= 2) {  // this phase follows a layer-2 phase (see the note on the barriers)
        if (alive) alive = mbar_wait(d1_full + 8 * ((k - 1) % 6), (uint32_t)(((k - 1) / 6) & 1));
        alive = __all_sync(0xffffffffu, alive);
      }
      for (int c = par; c < nch1; c += 2, ++n) {
        const uint32_t gi = g + c, ab = gi % NB;
        gather_next();
        asm volatile("cp.async.wait_group 1;" ::: "memory");
        __syncwarp();
        const uint32_t patch = patch0 + (uint32_t)(n & 1) * (32 * 128);
        const bool act = (act_mask >> (c >> 2)) & 1;
        const uint32_t ta = lane_base + GP_A_BASE + 32u * ab;
        convert_chunk<true>(patch, lane, act, ta, [&]() {
          if (gi >= NB && alive) alive = mbar_wait(a_done + 8 * ab, ((gi / NB) - 1) & 1);  // A buffer ab is free again
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        });
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(a_ready + 8 * ab);
      }
      g += (uint32_t)nch1;
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
  }

  // ------------------------------------------------------------------ common exit: release tensor memory
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == PS_MMA_WARP) {
    __syncwarp();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem_base), "r"(PS_TMEM_COLS) : "memory");
  }
}
