// Persistent tcgen05 GEMM (included by gemm.cu inside namespace mb, after the tcgen05 / TMA / mbarrier helpers).
//
// Same contract as k_gemm_tc (gathered, K-concatenated A operand; split-operand products with fp32 accumulation in
// tensor memory; bias / SiLU' gate / SiLU / residual / scale epilogue with store, accumulate or atomic scatter), but
// one CTA per SM walks over many 128x128 output tiles, so that the three stages of a tile run concurrently on
// DIFFERENT tiles instead of one after the other.
//
// Two operand formats (template parameter BF):
//   BF = true   3xBF16: x = hi + lo with hi = bf16(x), lo = bf16(x - hi); kind::f16 MMAs (K = 16) at twice the
//               tf32 rate; an operand pair carries 16 mantissa bits, which end to end stays within a small multiple
//               of the float32 rounding noise of the same evaluation (measured on the golden cases).  Weights
//               arrive as bf16 tiles of 64 K values (one 32 KB ring slot = hi + lo tile serves TWO 32-float A
//               chunks); an A chunk takes 32 tensor-memory columns (two values per column), so there are 8 A buffers.
//   BF = false  3xTF32: hi = x cut to 10 mantissa bits, lo = x - hi (exact), kind::tf32 MMAs (K = 8); 22 mantissa
//               bits per operand pair.  A ring slot serves one chunk, an A chunk takes 64 columns, 4 A buffers.
// Roles:
//
//   warp 0      MMA.  The whole warp walks the chunk sequence with warp-uniform addresses and descriptors; one elected
//               lane issues the tcgen05.mma of every chunk (lo*hi + hi*lo + hi*hi per K step, A from tensor memory)
//               into one of TWO accumulators; tcgen05.commit signals "A buffer free", "W slot free" and, after a
//               tile's last chunk, "accumulator full".
//   warp 1      TMA.  Same structure; the elected lane streams W_hi / W_lo tiles into a 4-slot ring, up to four slots
//               ahead and across tile boundaries; a column block with K = 128 is loaded once and stays.
//   warps 2-9   producers.  A warp owns rows 32 (warp & 3).. of the tile (= its TMEM lane quarter); the first four
//               take the even 32-float K chunks, the other four the odd ones.  A chunk is gathered with cp.async
//               (coalesced 128-byte row reads through the optional index, two stages per warp) into a swizzled
//               shared-memory patch, read back one row per thread, passed through the optional SiLU, split into tf32
//               hi / lo and written with tcgen05.st into one of the A buffers in tensor memory.
//   warps 10-17 epilogue.  Epilogue warp e takes rows 32 (warp & 3).., columns 64 (e >> 2).. of the finished
//               accumulator into registers (tcgen05.ld, thread = row), releases the accumulator, and finishes its
//               rows there with 256-bit global loads / stores (a full 32-byte sector per thread) while the tensor
//               cores already work on the next tile.  Scatter / accumulate modes go through a 4 KB patch per warp
//               instead, so that their memory-side reductions leave as 128-byte row segments.
//
// Shared-A mode (shared_a != 0; the host picks it when every column block reads the SAME A operand and its K chunks
// fit the A buffers, i.e. K <= 256 in bf16 form): a CTA takes whole row tiles and runs their column blocks one after
// the other; chunk c of the tile lives in A buffer c, is gathered and converted ONCE, read by every block's MMAs and
// handed back to the producers by the last block's.  (Otherwise the tiles of one row tile run on neighbouring CTAs
// and each gathers and converts the A rows for itself.)
//
// Tensor memory (512 columns): accumulators at 0 and 128, A buffers from 256 on (hi | lo each).
// Shared memory: W ring 4 x 32 KB | producer patches 64 KB | epilogue patches 32 KB | barriers | descriptor copy.
// Every mbarrier wait is bounded; on expiry a status word is set, the role stops waiting and runs to the common exit,
// where tensor memory is released.

// 256-bit global accesses (one full 32-byte sector per thread)
__device__ __forceinline__ void ld8(const float* p, float (&v)[8]) {
  asm volatile("ld.global.v8.f32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=f"(v[0]), "=f"(v[1]), "=f"(v[2]), "=f"(v[3]), "=f"(v[4]), "=f"(v[5]), "=f"(v[6]), "=f"(v[7]) : "l"(p));
}
__device__ __forceinline__ void st8(float* p, const float (&v)[8]) {
  asm volatile("st.global.v8.f32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
               :: "l"(p), "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3]), "f"(v[4]), "f"(v[5]), "f"(v[6]), "f"(v[7]) : "memory");
}

#define MB_TMEM_ST8(taddr, v)                                                                                    \
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"                   \
               :: "r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]),      \
                  "r"(v[7]) : "memory")

// two floats -> one 32-bit word of two bf16 (round to nearest even): `first` in the low half (the lower K index)
// Two floats -> one word of two bf16 (round to nearest even), the first value in the low half.
__device__ __forceinline__ uint32_t pack_bf16x2(float first, float second) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(second), "f"(first));
  return r;
}

// hi / lo split of 16 consecutive K values into 8 + 8 packed words (BF16): hi = bf16(x), lo = bf16(x - hi) ...
__device__ __forceinline__ void split_bf16(const float (&x)[16], uint32_t (&hi)[8], uint32_t (&lo)[8]) {
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    hi[i] = pack_bf16x2(x[2 * i], x[2 * i + 1]);
    const float r0 = x[2 * i] - __uint_as_float(hi[i] << 16);
    const float r1 = x[2 * i + 1] - __uint_as_float(hi[i] & 0xFFFF0000u);
    lo[i] = pack_bf16x2(r0, r1);
  }
}
// ... or into 16 + 16 words (TF32): hi = x cut to tf32's 10 mantissa bits, lo = the exact remainder
__device__ __forceinline__ void split_tf32(const float (&x)[16], uint32_t (&hi)[16], uint32_t (&lo)[16]) {
#pragma unroll
  for (int q = 0; q < 16; ++q) {
    hi[q] = __float_as_uint(x[q]) & 0xFFFFE000u;
    lo[q] = __float_as_uint(x[q] - __uint_as_float(hi[q]));
  }
}

// D[tmem] (+)= A[tmem] * B[smem]^T, M = 128, N = 128, K = 16 (bf16 operands, fp32 accumulation)
constexpr uint32_t TC_IDESC_BF16 = (1u << 4) | (1u << 7) | (1u << 10) | ((128u >> 3) << 17) | ((128u >> 4) << 24);
__device__ __forceinline__ void umma_bf16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t db, uint32_t accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
               :: "r"(tmem_d), "r"(tmem_a), "l"(db), "r"(TC_IDESC_BF16), "r"(accumulate) : "memory");
}

// per-format constants of the persistent GEMM kernel
template <bool BF> struct PsFormat {
  static constexpr uint32_t A_COLS = BF ? 32 : 64;   // tensor-memory columns of one A chunk (hi | lo)
  static constexpr uint32_t N_ABUF = BF ? 8 : 4;     // A buffers (256 columns in all)
  static constexpr uint32_t CH_PER_W = BF ? 2 : 1;   // A chunks served by one W ring slot
  static constexpr int W_BOX_K = BF ? 64 : 32;       // K values per W tile
};

// One chunk's MMAs: A buffer at tmem column `ta`, W slot at shared address `wb`, `half` = which 32-K half of a bf16
// W tile this chunk reads (always 0 for tf32); `fresh` = this is the first chunk of the accumulation.
template <bool BF>
__device__ __forceinline__ void issue_chunk_mmas(uint32_t d_tmem, uint32_t ta, uint32_t wb, uint32_t half, bool fresh) {
  const uint64_t dbh = umma_desc(wb), dbl = umma_desc(wb + TC_TILE_BYTES);
  if (BF) {
    const uint32_t ta_hi = ta, ta_lo = ta + 16;
#pragma unroll
    for (int kk = 0; kk < 2; ++kk) {  // K steps of 16: 8 TMEM columns of A, 32 bytes (>> 4 = 2) of the W rows
      const uint64_t adv = (uint64_t)(2 * (2 * half + kk));
      umma_bf16_ts(d_tmem, ta_lo + 8 * kk, dbh + adv, (!fresh || kk > 0) ? 1u : 0u);
      umma_bf16_ts(d_tmem, ta_hi + 8 * kk, dbl + adv, 1u);
      umma_bf16_ts(d_tmem, ta_hi + 8 * kk, dbh + adv, 1u);
    }
  } else {
    const uint32_t ta_hi = ta, ta_lo = ta + 32;
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {  // K steps of 8: 8 TMEM columns of A, 32 bytes (>> 4 = 2) of the W rows
      const uint64_t adv = (uint64_t)(2 * kk);
      umma_tf32_ts(d_tmem, ta_lo + 8 * kk, dbh + adv, (!fresh || kk > 0) ? 1u : 0u);
      umma_tf32_ts(d_tmem, ta_hi + 8 * kk, dbl + adv, 1u);
      umma_tf32_ts(d_tmem, ta_hi + 8 * kk, dbh + adv, 1u);
    }
  }
}

// One producer chunk: 32 floats of this thread's row from the swizzled patch -> optional SiLU -> hi / lo -> A buffer.
// `wait_free` is called once, right before the first tcgen05.st (the conversion of the first half overlaps the wait).
template <bool BF, typename WaitFree>
__device__ __forceinline__ void convert_chunk(uint32_t patch, int lane, bool act, uint32_t ta, WaitFree wait_free) {
#pragma unroll
  for (int h = 0; h < 2; ++h) {  // two halves of 16 floats keep the live registers of the split low
    float x[16];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint32_t addr = patch + lane * 128 + (((4 * h + j) ^ (lane & 7)) << 4);
      asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(x[4 * j]), "=f"(x[4 * j + 1]),
                   "=f"(x[4 * j + 2]), "=f"(x[4 * j + 3]) : "r"(addr) : "memory");
    }
    if (act) {
#pragma unroll
      for (int q = 0; q < 16; ++q) x[q] = silu_fast_f(x[q]);
    }
    if (BF) {
      uint32_t hi[8], lo[8];
      split_bf16(x, hi, lo);
      if (h == 0) wait_free();
      MB_TMEM_ST8(ta + 8 * h, hi);
      MB_TMEM_ST8(ta + 16 + 8 * h, lo);
    } else {
      uint32_t hi[16], lo[16];
      split_tf32(x, hi, lo);
      if (h == 0) wait_free();
      MB_TMEM_ST16(ta + 16 * h, hi);
      MB_TMEM_ST16(ta + 32 + 16 * h, lo);
    }
  }
}

constexpr int PS_THREADS = 576;          // 18 warps
constexpr int PS_MMA_WARP = 0, PS_TMA_WARP = 1, PS_PROD_WARP0 = 2, PS_EPI_WARP0 = 10;
// The two issuing warps come first: the warp schedulers favour the oldest (lowest-numbered) eligible warp, and the
// MMA thread's few instructions per chunk must not queue behind the sixteen data-moving warps.
constexpr int PS_W_SLOTS = 4;
constexpr int PS_RING_BYTES = PS_W_SLOTS * 2 * TC_TILE_BYTES;
constexpr int PS_PATCH_BYTES = 8 * 2 * 32 * 128;
constexpr int PS_STAGE_BYTES = 8 * 32 * 128;   // per epilogue warp: 32 rows x 32 columns (scatter / accumulate modes only)
constexpr int PS_BAR_OFF = PS_RING_BYTES + PS_PATCH_BYTES + PS_STAGE_BYTES;
constexpr int PS_DESC_OFF = PS_BAR_OFF + 256;
constexpr int PS_SMEM_BYTES = PS_DESC_OFF + (int)((sizeof(mb_gemm_desc) + 15) / 16 * 16);
constexpr uint32_t PS_TMEM_COLS = 512;
static_assert(PS_SMEM_BYTES <= 227 * 1024, "shared memory of one CTA");

template <bool BF>
__global__ void __launch_bounds__(PS_THREADS, 1)
k_gemm_ps(const __grid_constant__ mb_gemm_desc d_param, const __grid_constant__ TcMaps maps, const int shared_a) {
  using Fmt = PsFormat<BF>;
  constexpr uint32_t NB = Fmt::N_ABUF, CPW = Fmt::CH_PER_W;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + PS_BAR_OFF);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + PS_BAR_OFF + 240);
  if ((smem_u32(smem) & 1023u) != 0) {  // the swizzled tiles need a 1024-byte aligned base
    if (threadIdx.x == 0) atomicOr(&g_gemm_status, 2);
    return;
  }
  // barriers: a_ready[8] (A chunk stored: 4 producer warps) | a_done[8] (its MMAs retired: the A buffer is free) |
  //           w_ready[4] (W slot landed: the TMA thread's expect_tx arrival + bytes) | w_done[4] (slot free) |
  //           d_full[2] | d_free[2] (8 epilogue warps).  Chunk g uses A buffer g % NB; W-slot use u = g / CPW uses
  //           ring slot u % w_period.  Every waiter sees every phase of the barriers it waits on (a parity wait can
  //           tell apart only two consecutive phases).
  const uint32_t a_ready = smem_u32(bars), a_done = smem_u32(bars + 8);
  const uint32_t w_ready = smem_u32(bars + 16), w_done = smem_u32(bars + 20);
  const uint32_t d_full = smem_u32(bars + 24), d_free = smem_u32(bars + 26);
  const uint32_t ring = smem_u32(smem);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // The descriptor is indexed dynamically (column block, K segment) all through the kernel.  From kernel-parameter
  // memory every such read is a round trip through the memory system; from this shared-memory copy it is not.
  const mb_gemm_desc& d = *reinterpret_cast<const mb_gemm_desc*>(smem + PS_DESC_OFF);
  {
    const uint32_t* src = reinterpret_cast<const uint32_t*>(&d_param);
    uint32_t* dst = reinterpret_cast<uint32_t*>(smem + PS_DESC_OFF);
    for (int i = tid; i < (int)(sizeof(mb_gemm_desc) / 4); i += PS_THREADS) dst[i] = src[i];
  }
  __syncthreads();
  const int64_t n_rows = d.n_rows;
  const int n_blocks = d.n_blocks;
  // Tiles are numbered row tile * n_blocks + column block; this CTA takes tiles blockIdx.x, + gridDim.x, ...  Every
  // role walks that sequence as a (row tile, column block) pair advanced by (step_rt, step_jb): no division in loops.
  // Shared-A mode: this CTA takes row tiles blockIdx.x, + gridDim.x, ... and walks the column blocks of each.
  const int n_row_tiles = (int)((n_rows + 127) >> 7);
  const bool sh = shared_a != 0;
  const int first_rt = sh ? (int)blockIdx.x : (int)(blockIdx.x / (unsigned)n_blocks);
  const int first_jb = sh ? 0 : (int)(blockIdx.x % (unsigned)n_blocks);
  const int step_rt = sh ? (int)gridDim.x : (int)(gridDim.x / (unsigned)n_blocks);
  const int step_jb = sh ? 0 : (int)(gridDim.x % (unsigned)n_blocks);
  // When every tile of this CTA belongs to the same column block and that block has a single 128-wide K segment,
  // its W tiles fill w_period ring slots once and stay there for the whole kernel.
  const bool w_resident = !sh && step_jb == 0 && d.blk[first_jb].n_src == 1;
  const uint32_t w_period = w_resident ? 4u / CPW : 4u;
  auto next_tile = [&](int& rt, int& jb) {  // the (row tile, column block) sequence of the MMA, TMA and epilogue warps
    if (sh) {
      if (++jb == n_blocks) { jb = 0; rt += step_rt; }
      return;
    }
    jb += step_jb;
    rt += step_rt;
    if (jb >= n_blocks) { jb -= n_blocks; ++rt; }
  };
  auto next_a_tile = [&](int& rt, int& jb) {  // the sequence of A tiles the producers gather and convert
    if (sh) rt += step_rt;  // once per row tile, from column block 0's sources
    else next_tile(rt, jb);
  };

  // ---- producer state
  const int pw = (warp - PS_PROD_WARP0) & 7;  // producer index 0-7 (meaningful in producer warps only)
  const int par = pw >> 2, quarter = warp & 3;  // chunk parity set; TMEM lane quarter = warp id mod 4
  const int lr = lane >> 3, lc = lane & 7;  // 8 lanes read one row's 128 bytes, 4 rows per instruction
  // row (lr + 4i), 16-byte chunk lc -> patch[row][lc ^ (row & 7)]; (row & 7) is lr for even i and lr + 4 for odd i
  const uint32_t patch0 = smem_u32(smem + PS_RING_BYTES + pw * (2 * 32 * 128));
  const uint32_t dst_even = patch0 + lr * 128 + ((lc ^ lr) << 4), dst_odd = patch0 + lr * 128 + ((lc ^ (lr | 4)) << 4);
  const float* a_ptr[8];  // this lane's 8 row pointers in the current K segment, at this warp's first chunk
  int32_t a_row[8];       // source rows of the NEXT segment (looked up one chunk ahead, so the index loads are hidden)
  int g_rt = first_rt, g_jb = first_jb;  // gather iterator: the next chunk this warp will request
  int g_seg = 0, g_nsrc = d.blk[first_jb].n_src, g_cnt = 0;
  bool g_second = false;
  // Rows past the end of the matrix are clamped to the last row: their products land in accumulator rows that the
  // epilogue never writes, and every copy stays a plain 16-byte one.
  auto resolve_rows = [&](int rt, int jb, int seg) {
    const int64_t row0 = (int64_t)rt * 128;
    const int32_t* idx = d.blk[jb].src[seg].idx;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      int64_t r = row0 + quarter * 32 + lr + 4 * i;
      r = r < n_rows ? r : n_rows - 1;
      a_row[i] = idx ? idx[r] : (int32_t)(r - row0);
    }
  };
#define MB_CP16(dst, off, src, soff)                                                                    \
  asm volatile("cp.async.cg.shared.global [%0 + %1], [%2 + %3], 16;" :: "r"(dst), "n"(off), "l"(src), "n"(soff) : "memory")
  auto gather_next = [&]() {
    if (g_rt >= n_row_tiles) {
      asm volatile("cp.async.commit_group;" ::: "memory");
      return;
    }
    const uint32_t st = (uint32_t)(g_cnt & 1) * (32 * 128);
    const uint32_t de = dst_even + st, dq = dst_odd + st;
    if (!g_second) {  // first of this warp's two chunks in the segment: rows -> pointers (chunk par of the segment)
      const mb_src& s = d.blk[g_jb].src[g_seg];
      const float* base = s.ptr + s.col + lc * 4 + par * TC_BK;
      const int64_t ld = s.ld;
      const int64_t row0 = s.idx ? 0 : (int64_t)g_rt * 128;
#pragma unroll
      for (int i = 0; i < 8; ++i) a_ptr[i] = base + (row0 + a_row[i]) * ld;
      MB_CP16(de, 0, a_ptr[0], 0);    MB_CP16(dq, 512, a_ptr[1], 0);  MB_CP16(de, 1024, a_ptr[2], 0); MB_CP16(dq, 1536, a_ptr[3], 0);
      MB_CP16(de, 2048, a_ptr[4], 0); MB_CP16(dq, 2560, a_ptr[5], 0); MB_CP16(de, 3072, a_ptr[6], 0); MB_CP16(dq, 3584, a_ptr[7], 0);
    } else {          // chunk par + 2 of the segment: 64 floats further along every row
      MB_CP16(de, 0, a_ptr[0], 256);    MB_CP16(dq, 512, a_ptr[1], 256);  MB_CP16(de, 1024, a_ptr[2], 256); MB_CP16(dq, 1536, a_ptr[3], 256);
      MB_CP16(de, 2048, a_ptr[4], 256); MB_CP16(dq, 2560, a_ptr[5], 256); MB_CP16(de, 3072, a_ptr[6], 256); MB_CP16(dq, 3584, a_ptr[7], 256);
      if (++g_seg == g_nsrc) {  // on to the next tile
        g_seg = 0;
        next_a_tile(g_rt, g_jb);
        if (g_rt < n_row_tiles) g_nsrc = d.blk[g_jb].n_src;
      }
      if (g_rt < n_row_tiles) resolve_rows(g_rt, g_jb, g_seg);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    ++g_cnt;
    g_second = !g_second;
  };

  if (warp == PS_MMA_WARP) {
    if (lane == 0) {
      for (int b = 0; b < 8; ++b) { mbar_init(a_ready + 8 * b, 4); mbar_init(a_done + 8 * b, 1); }
      for (int b = 0; b < 4; ++b) { mbar_init(w_ready + 8 * b, 1); mbar_init(w_done + 8 * b, 1); }
      for (int b = 0; b < 2; ++b) { mbar_init(d_full + 8 * b, 1); mbar_init(d_free + 8 * b, 8); }
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncwarp();
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 :: "r"(smem_u32(tmem_slot)), "r"(PS_TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  } else if (warp >= PS_PROD_WARP0 && warp < PS_EPI_WARP0) {
    resolve_rows(first_rt, first_jb, 0);
    gather_next();
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  if (warp == PS_MMA_WARP) {
    // ---------------------------------------------------------------- MMA warp
    // The whole warp runs the loop and computes the (warp-uniform) addresses and descriptors; one elected lane issues
    // the tcgen05 instructions.  Their operands must sit in uniform registers: computed by a single lane inside a
    // divergent branch they would each be moved there one by one in front of every MMA, which costs more than the MMA.
    uint32_t elected;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(elected));
    const uint32_t tmem_u = __shfl_sync(0xffffffffu, tmem_base, 0);
    const uint32_t ring_u = __shfl_sync(0xffffffffu, ring, 0);
    bool alive = true;
    uint32_t nch_of = 0;  // chunks per tile of the (up to four) column blocks, a byte each: no descriptor read per tile
    for (int j = 0; j < n_blocks; ++j) nch_of |= (uint32_t)(d.blk[j].n_src * 4) << (8 * j);
    nch_of = __shfl_sync(0xffffffffu, nch_of, 0);
    uint32_t g = 0;  // chunks issued so far (all tiles); a multiple of 4 at every tile start
    uint32_t t_sh = 0;  // shared-A mode: row tiles finished
    int k = 0;
    for (int rt = first_rt, jb = first_jb; rt < n_row_tiles; next_tile(rt, jb), ++k) {
      const int acc = k & 1;
      const uint32_t d_tmem = tmem_u + 128u * acc;
      const int nch = (int)((nch_of >> (8 * jb)) & 0xffu);
      const bool first_blk = !sh || jb == 0, last_blk = !sh || jb == n_blocks - 1;
      for (int c = 0; c < nch; ++c, ++g) {
        // A buffer, W-slot use and ring slot of chunk g (shared-A mode: chunk c of the row tile sits in buffer c)
        const uint32_t ab = sh ? (uint32_t)c : g % NB, wu = g / CPW, slot = wu % w_period;
        // A rows stored (shared-A mode: seen once per row tile, by its first column block)
        if (first_blk && alive) alive = mbar_wait(a_ready + 8 * ab, (sh ? t_sh : g / NB) & 1);
        if (g % CPW == 0 && alive) alive = mbar_wait(w_ready + 8 * slot, (wu / w_period) & 1);  // W tiles landed
        if (c == 0 && k >= 2 && alive) alive = mbar_wait(d_free + 8 * acc, (uint32_t)(((k >> 1) - 1) & 1));
        alive = __all_sync(0xffffffffu, alive);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t wb = ring_u + slot * 2 * TC_TILE_BYTES;
        const uint32_t ta = tmem_u + 256 + Fmt::A_COLS * ab;
        if (elected) {
          issue_chunk_mmas<BF>(d_tmem, ta, wb, g % CPW, c == 0);
          if (last_blk)  // the A buffer goes back to the producers
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                         :: "r"(a_done + 8 * ab) : "memory");
          if (g % CPW == CPW - 1)
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                         :: "r"(w_done + 8 * slot) : "memory");
          if (c == nch - 1)
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                         :: "r"(d_full + 8 * acc) : "memory");
        }
        __syncwarp();
      }
      if (sh && jb == n_blocks - 1) ++t_sh;
    }
  } else if (warp == PS_TMA_WARP) {
    // ---------------------------------------------------------------- TMA warp: W_hi / W_lo tiles, up to 4 chunks ahead
    // (warp-uniform loop, one elected lane issues: same reason as in the MMA warp)
    uint32_t elected;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(elected));
    const uint32_t ring_u = __shfl_sync(0xffffffffu, ring, 0);
    bool alive = true;
    uint32_t wu = 0;  // W-slot uses issued so far
    for (int rt = first_rt, jb = first_jb; rt < n_row_tiles && alive; next_tile(rt, jb)) {
      const int n_w = __shfl_sync(0xffffffffu, d.blk[jb].n_src * 4 / (int)CPW, 0);
      for (int wi = 0; wi < n_w && alive; ++wi, ++wu) {
        const uint32_t slot = wu % w_period;
        // slot and barrier were last used w_period uses ago
        if (wu >= w_period) alive = mbar_wait(w_done + 8 * slot, ((wu / w_period) - 1) & 1);
        alive = __all_sync(0xffffffffu, alive);
        if (!alive) break;
        const uint32_t bar = w_ready + 8 * slot;
        if (elected) {
          if (w_resident && wu >= w_period) {  // the tiles are in their slot already: only this thread's arrival is due
            mbar_arrive(bar);
          } else {
            const uint32_t dst = ring_u + slot * 2 * TC_TILE_BYTES;
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(bar), "r"(2 * TC_TILE_BYTES) : "memory");
            tma_load_2d(dst, &maps.m[jb][0], bar, wi * Fmt::W_BOX_K, 0);
            tma_load_2d(dst + TC_TILE_BYTES, &maps.m[jb][1], bar, wi * Fmt::W_BOX_K, 0);
          }
        }
        __syncwarp();
      }
    }
    if (!alive) {  // failure path only: no TMA write may still be in flight when the CTA's shared memory is released
      for (uint32_t i = wu >= w_period ? wu - w_period : 0; i < wu; ++i)
        mbar_wait(w_ready + 8 * (i % w_period), (i / w_period) & 1);
    }
  } else if (warp >= PS_EPI_WARP0) {
    // ---------------------------------------------------------------- epilogue warps
    // Epilogue warp e finishes rows 32 (warp & 3).. (its TMEM lane quarter), columns 64 (e >> 2).. of the accumulator
    // straight from the tcgen05.ld layout: thread = row, 32 columns per load, global accesses of 32 bytes (one full
    // sector) per thread with 256-bit loads and stores.  No shared-memory staging: every sector is still written
    // exactly once, and the row's sixteen sectors merge in L2.
    const int e = warp - PS_EPI_WARP0, quarter_e = warp & 3, half = e >> 2;
    const uint32_t lane_base = tmem_base + ((uint32_t)(quarter_e * 32) << 16) + (uint32_t)(half * 64);
    bool alive = true;
    int k = 0;
    for (int rt = first_rt, jb = first_jb; rt < n_row_tiles; next_tile(rt, jb), ++k) {
      const int acc = k & 1;
      const int64_t row = (int64_t)rt * 128 + quarter_e * 32 + lane;  // this thread's row
      const bool valid = row < n_rows;
      const int64_t rowc = valid ? row : n_rows - 1;
      const mb_colblock& cb = d.blk[jb];
      const int c0 = half * 64;
      const float* const gate = cb.gate ? cb.gate + rowc * cb.ld_gate + cb.col_gate + c0 : nullptr;
      const float* const res = cb.res ? cb.res + rowc * cb.ld_res + cb.col_res + c0 : nullptr;
      const float* const bias = cb.bias ? cb.bias + c0 : nullptr;
      const float* const res_w = (cb.res && cb.res_w) ? cb.res_w + c0 : nullptr;
      const int64_t dr = cb.out_idx ? (int64_t)cb.out_idx[rowc] : rowc;
      float* const out = cb.out + dr * cb.ld_out + cb.col_out + c0;
      const int mode = cb.mode, out_act = cb.out_act;
      const float sc = cb.out_scale;
      // the row segments this thread will read are pulled into L2 while the tile is still being multiplied
      if (gate) {
        asm volatile("prefetch.global.L2 [%0];" :: "l"(gate));
        asm volatile("prefetch.global.L2 [%0];" :: "l"(gate + 32));
      }
      if (res) {
        asm volatile("prefetch.global.L2 [%0];" :: "l"(res));
        asm volatile("prefetch.global.L2 [%0];" :: "l"(res + 32));
      }
      if (alive) alive = mbar_wait(d_full + 8 * acc, (uint32_t)((k >> 1) & 1));
      alive = __all_sync(0xffffffffu, alive);
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      auto finish = [&](auto has_gate, auto has_act, auto has_res) {
#pragma unroll 1
        for (int cg = 0; cg < 2; ++cg) {
          uint32_t v[32];
          MB_TMEM_LD32(lane_base + 128u * acc + 32u * cg, v);
          // the gate values of these 32 columns are requested before the accumulator load is waited for, all four
          // 32-byte pieces at once: one memory latency per 32 columns instead of four
          float z[decltype(has_gate)::value ? 4 : 1][8];
          if constexpr (decltype(has_gate)::value) {
#pragma unroll
            for (int j = 0; j < 4; ++j) ld8(gate + cg * 32 + j * 8, z[j]);
          }
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
          if (cg == 1) {  // the accumulator is in registers: the tensor cores may overwrite it
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(d_free + 8 * acc);
          }
          if (!alive) continue;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int c = cg * 32 + j * 8;
            float o[8];
#pragma unroll
            for (int q = 0; q < 8; ++q) o[q] = __uint_as_float(v[8 * j + q]);
            if (bias) {  // same address in every lane: a broadcast load
              float bv[8];
              ld8(bias + c, bv);
#pragma unroll
              for (int q = 0; q < 8; ++q) o[q] += bv[q];
            }
            if constexpr (decltype(has_gate)::value) {
#pragma unroll
              for (int q = 0; q < 8; ++q) o[q] *= silu_grad_fast_f(z[j][q]);
            }
            if constexpr (decltype(has_act)::value) {
#pragma unroll
              for (int q = 0; q < 8; ++q) o[q] = silu_fast_f(o[q]);
            }
            if constexpr (decltype(has_res)::value) {
              float x[8];
              ld8(res + c, x);
              if (res_w) {
                float w[8];
                ld8(res_w + c, w);
#pragma unroll
                for (int q = 0; q < 8; ++q) o[q] = fmaf(w[q], x[q], o[q]);
              } else {
#pragma unroll
                for (int q = 0; q < 8; ++q) o[q] += x[q];
              }
            }
#pragma unroll
            for (int q = 0; q < 8; ++q) o[q] *= sc;
            if (valid) {
              st8(out + c, o);
            }
          }
        }
      };
      // Scatter / accumulate modes go through a 4 KB swizzled patch instead, 32 columns at a time, so that eight lanes
      // cover one row's 128 contiguous bytes: the memory-side reductions then arrive as four 128-byte requests per
      // instruction, not as 32 requests of 16 bytes (which the direct layout would give).
      auto finish_reduce = [&]() {
        uint8_t* const stage = smem + PS_RING_BYTES + PS_PATCH_BYTES + e * (32 * 128);
        const uint32_t stage_u = smem_u32(stage);
        const int sub = lane >> 3, ch = lane & 7;
        const int64_t row0 = (int64_t)rt * 128 + quarter_e * 32;
        const int64_t left = n_rows - row0;
        const int rows_here = left >= 32 ? 32 : (left > 0 ? (int)left : 0);
#pragma unroll 1
        for (int pass = 0; pass < 2; ++pass) {
          {
            uint32_t v[32];
            MB_TMEM_LD32(lane_base + 128u * acc + 32u * pass, v);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
            for (int q = 0; q < 8; ++q) {  // 16-byte chunk q of row r sits at position q ^ (r & 7)
              const uint32_t addr = stage_u + lane * 128 + ((q ^ (lane & 7)) << 4);
              asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};"
                           :: "r"(addr), "r"(v[4 * q]), "r"(v[4 * q + 1]), "r"(v[4 * q + 2]), "r"(v[4 * q + 3]) : "memory");
            }
          }
          if (pass == 1) asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
          __syncwarp();
          if (pass == 1 && lane == 0) mbar_arrive(d_free + 8 * acc);
          if (!alive) continue;
          const int col = c0 + pass * 32 + ch * 4;  // column within the 128-wide block
          float4 bias4 = make_float4(0.f, 0.f, 0.f, 0.f), resw4 = make_float4(1.f, 1.f, 1.f, 1.f);
          if (cb.bias) bias4 = ld4(cb.bias + col);
          if (cb.res && cb.res_w) resw4 = ld4(cb.res_w + col);
#pragma unroll 1
          for (int r0 = 0; r0 < rows_here; r0 += 16) {
            float4 av[4];
            int64_t drow[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const int rq = r0 + 4 * i + sub;
              const int64_t gr = row0 + (rq < rows_here ? rq : r0);
              drow[i] = cb.out_idx ? (int64_t)cb.out_idx[gr] : gr;
              av[i] = *reinterpret_cast<const float4*>(stage + rq * 128 + ((ch ^ (rq & 7)) << 4));
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const int rq = r0 + 4 * i + sub;
              const int64_t gr = row0 + (rq < rows_here ? rq : r0);
              float o[4] = {av[i].x + bias4.x, av[i].y + bias4.y, av[i].z + bias4.z, av[i].w + bias4.w};
              if (cb.gate) {
                const float4 z = ld4(cb.gate + gr * cb.ld_gate + cb.col_gate + col);
                o[0] *= silu_grad_fast_f(z.x); o[1] *= silu_grad_fast_f(z.y); o[2] *= silu_grad_fast_f(z.z); o[3] *= silu_grad_fast_f(z.w);
              }
              if (out_act) { o[0] = silu_fast_f(o[0]); o[1] = silu_fast_f(o[1]); o[2] = silu_fast_f(o[2]); o[3] = silu_fast_f(o[3]); }
              if (cb.res) {
                const float4 x = ld4(cb.res + gr * cb.ld_res + cb.col_res + col);
                o[0] = fmaf(resw4.x, x.x, o[0]); o[1] = fmaf(resw4.y, x.y, o[1]); o[2] = fmaf(resw4.z, x.z, o[2]); o[3] = fmaf(resw4.w, x.w, o[3]);
              }
              // accumulate = one reduction at the memory side: the same single fp32 addition as read-add-write
              // when nobody else touches the row, without the read's round trip
              if (rq < rows_here)
                atomicAdd(reinterpret_cast<float4*>(cb.out + drow[i] * cb.ld_out + cb.col_out + col),
                          make_float4(o[0] * sc, o[1] * sc, o[2] * sc, o[3] * sc));
            }
          }
          __syncwarp();  // the patch is rewritten by the next pass / tile
        }
      };
      using T = std::true_type;
      using F = std::false_type;
      auto pick_res = [&](auto g_, auto a_) { if (res) finish(g_, a_, T{}); else finish(g_, a_, F{}); };
      auto pick_act = [&](auto g_) { if (out_act) pick_res(g_, T{}); else pick_res(g_, F{}); };
      if (mode != MB_OUT_STORE) finish_reduce();
      else if (gate) pick_act(T{});
      else pick_act(F{});
    }
  } else {
    // ---------------------------------------------------------------- producers: thread = row = TMEM lane
    const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16);
    bool alive = true;
    uint32_t g = 0;
    int n = 0;  // chunks this warp has converted
    for (int rt = first_rt, jb = first_jb; rt < n_row_tiles; next_a_tile(rt, jb)) {
      const mb_colblock& cb = d.blk[jb];
      const int nch = cb.n_src * 4;
      int act_mask = 0;
#pragma unroll
      for (int s = 0; s < 4; ++s) act_mask |= (s < cb.n_src && cb.src[s].act) ? (1 << s) : 0;
      for (int c = par; c < nch; c += 2, ++n) {
        const uint32_t gi = g + c, ab = gi % NB;
        gather_next();  // into the stage read one chunk ago; the __syncwarp that closed that chunk orders the reads
        asm volatile("cp.async.wait_group 1;" ::: "memory");  // this chunk's copies of this lane have landed
        __syncwarp();                                          // ... and so have the other lanes'
        const uint32_t patch = patch0 + (uint32_t)(n & 1) * (32 * 128);
        const bool act = (act_mask >> (c >> 2)) & 1;  // branch once per chunk: no SiLU is evaluated on the plain path
        const uint32_t ta = lane_base + 256 + Fmt::A_COLS * ab;
        convert_chunk<BF>(patch, lane, act, ta, [&]() {
          if (gi >= NB && alive) alive = mbar_wait(a_done + 8 * ab, ((gi / NB) - 1) & 1);  // A buffer ab is free again
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        });
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();  // all lanes have read their patch rows and written their A rows
        if (lane == 0) mbar_arrive(a_ready + 8 * ab);
      }
      g += sh ? NB : (uint32_t)nch;  // shared-A mode: chunk c always in buffer c, one barrier phase per row tile
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
