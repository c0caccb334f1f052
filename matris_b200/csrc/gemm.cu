// Row GEMM with gathered, concatenated A operands and a fused epilogue.
// Two cores share one descriptor: a tcgen05/TMEM tensor-core kernel (default, below)
// and this exact-fp32 SIMT kernel (selectable with mb_set_gemm_mode, used as the
// bit-faithful cross-check of the tensor-core path).
//
// SIMT core: one CTA computes a 128-row x 128-column output tile.  A is never materialised:
// each 128-wide K segment is read through its own (pointer, gather index, column)
// triple, optionally through SiLU.  W rows are read straight from global memory
// (the whole weight set of a layer is ~1 MB and stays L2 resident).  Register
// tile 8x8 per thread, K staged through shared memory in chunks of 16 with a
// register-prefetched double buffer.
#include "common.cuh"

namespace mb {

constexpr int BM = 128, BN = 128, BK = 16, GEMM_THREADS = 256, LDS = BM + 4;

__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }

__global__ void __launch_bounds__(GEMM_THREADS, 2) k_gemm(const __grid_constant__ mb_gemm_desc d) {
  const mb_colblock& cb = d.blk[blockIdx.y];
  __shared__ __align__(16) float As[2][BK][LDS];
  __shared__ __align__(16) float Bs[2][BK][LDS];
  const int tid = threadIdx.x;
  const int64_t row0 = (int64_t)blockIdx.x * BM;
  const int lrow = tid >> 2, lk = (tid & 3) * 4;  // loader: 64 rows x 4 float4 per pass, 2 passes
  const int ty = tid >> 4, tx = tid & 15;         // compute: rows {ty*4.., 64+ty*4..}, cols {tx*4.., 64+tx*4..}
  const int n_chunks = cb.n_src * (128 / BK);

  float acc[8][8];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;

  const float* a_ptr[2] = {nullptr, nullptr};
  int a_act = 0;
  const float* b_ptr[2] = {cb.W + (int64_t)lrow * cb.ldw + lk, cb.W + (int64_t)(lrow + 64) * cb.ldw + lk};
  float4 a_reg[2], b_reg[2];

  auto load_chunk = [&](int c) {
    if ((c & 7) == 0) {  // new K segment: resolve the gathered row pointers
      const mb_src& s = cb.src[c >> 3];
      a_act = s.act;
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int64_t r = row0 + lrow + 64 * i;
        if (r < d.n_rows) {
          const int64_t sr = s.idx ? (int64_t)s.idx[r] : r;
          a_ptr[i] = s.ptr + sr * s.ld + s.col + lk;
        } else {
          a_ptr[i] = nullptr;
        }
      }
    }
    const int kofs = (c & 7) * BK;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (a_ptr[i]) {
        v = ld4(a_ptr[i] + kofs);
        if (a_act) { v.x = silu_f(v.x); v.y = silu_f(v.y); v.z = silu_f(v.z); v.w = silu_f(v.w); }
      }
      a_reg[i] = v;
      b_reg[i] = ld4(b_ptr[i] + c * BK);
    }
  };
  auto store_chunk = [&](int buf) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int m = lrow + 64 * i;
      As[buf][lk + 0][m] = a_reg[i].x; As[buf][lk + 1][m] = a_reg[i].y;
      As[buf][lk + 2][m] = a_reg[i].z; As[buf][lk + 3][m] = a_reg[i].w;
      Bs[buf][lk + 0][m] = b_reg[i].x; Bs[buf][lk + 1][m] = b_reg[i].y;
      Bs[buf][lk + 2][m] = b_reg[i].z; Bs[buf][lk + 3][m] = b_reg[i].w;
    }
  };

  load_chunk(0);
  store_chunk(0);
  __syncthreads();
  for (int c = 0; c < n_chunks; ++c) {
    const int buf = c & 1;
    if (c + 1 < n_chunks) load_chunk(c + 1);
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      const float4 a0 = *reinterpret_cast<const float4*>(&As[buf][k][ty * 4]);
      const float4 a1 = *reinterpret_cast<const float4*>(&As[buf][k][64 + ty * 4]);
      const float4 b0 = *reinterpret_cast<const float4*>(&Bs[buf][k][tx * 4]);
      const float4 b1 = *reinterpret_cast<const float4*>(&Bs[buf][k][64 + tx * 4]);
      const float a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
      const float b[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    if (c + 1 < n_chunks) store_chunk(buf ^ 1);
    __syncthreads();
  }

  // ---- epilogue
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int64_t r = row0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4));
    if (r >= d.n_rows) continue;
    const int64_t dr = cb.out_idx ? (int64_t)cb.out_idx[r] : r;
#pragma unroll
    for (int jh = 0; jh < 2; ++jh) {
      const int col = jh * 64 + tx * 4;
      float v[4] = {acc[i][jh * 4 + 0], acc[i][jh * 4 + 1], acc[i][jh * 4 + 2], acc[i][jh * 4 + 3]};
      if (cb.bias) {
        const float4 bb = ld4(cb.bias + col);
        v[0] += bb.x; v[1] += bb.y; v[2] += bb.z; v[3] += bb.w;
      }
      if (cb.gate) {
        const float4 z = ld4(cb.gate + r * cb.ld_gate + cb.col_gate + col);
        v[0] *= silu_grad_f(z.x); v[1] *= silu_grad_f(z.y); v[2] *= silu_grad_f(z.z); v[3] *= silu_grad_f(z.w);
      }
      if (cb.out_act) {
        v[0] = silu_f(v[0]); v[1] = silu_f(v[1]); v[2] = silu_f(v[2]); v[3] = silu_f(v[3]);
      }
      if (cb.res) {
        const float4 x = ld4(cb.res + r * cb.ld_res + cb.col_res + col);
        float4 w = make_float4(1.f, 1.f, 1.f, 1.f);
        if (cb.res_w) w = ld4(cb.res_w + col);
        v[0] = fmaf(w.x, x.x, v[0]); v[1] = fmaf(w.y, x.y, v[1]);
        v[2] = fmaf(w.z, x.z, v[2]); v[3] = fmaf(w.w, x.w, v[3]);
      }
      const float sc = cb.out_scale;
      float4 o = make_float4(v[0] * sc, v[1] * sc, v[2] * sc, v[3] * sc);
      float* dst = cb.out + dr * cb.ld_out + cb.col_out + col;
      if (cb.mode == MB_OUT_STORE) {
        *reinterpret_cast<float4*>(dst) = o;
      } else if (cb.mode == MB_OUT_ADD) {
        float4 p = ld4(dst);
        p.x += o.x; p.y += o.y; p.z += o.z; p.w += o.w;
        *reinterpret_cast<float4*>(dst) = p;
      } else {
        atomicAdd(reinterpret_cast<float4*>(dst), o);
      }
    }
  }
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace mb

static int gemm_validate(const mb_gemm_desc* desc) {
  if (!desc || desc->n_rows < 0 || desc->n_blocks < 1 || desc->n_blocks > 4) return MB_ERR_INVALID;
  for (int j = 0; j < desc->n_blocks; ++j) {
    const mb_colblock& cb = desc->blk[j];
    if (cb.n_src < 1 || cb.n_src > 4 || !cb.W || !cb.out) return MB_ERR_INVALID;
    if (!mb::aligned16(cb.W) || (cb.ldw & 3) || cb.ldw < 128 * cb.n_src) return MB_ERR_INVALID;
    if (!mb::aligned16(cb.out) || (cb.ld_out & 3) || (cb.col_out & 3)) return MB_ERR_INVALID;
    if (cb.mode < MB_OUT_STORE || cb.mode > MB_OUT_ATOMIC) return MB_ERR_INVALID;
    if (cb.bias && !mb::aligned16(cb.bias)) return MB_ERR_INVALID;
    if (cb.gate && (!mb::aligned16(cb.gate) || (cb.ld_gate & 3) || (cb.col_gate & 3))) return MB_ERR_INVALID;
    if (cb.res && (!mb::aligned16(cb.res) || (cb.ld_res & 3) || (cb.col_res & 3))) return MB_ERR_INVALID;
    if (cb.res_w && !mb::aligned16(cb.res_w)) return MB_ERR_INVALID;
    for (int s = 0; s < cb.n_src; ++s) {
      const mb_src& sr = cb.src[s];
      if (!sr.ptr || !mb::aligned16(sr.ptr) || (sr.ld & 3) || (sr.col & 3)) return MB_ERR_INVALID;
    }
  }
  return MB_OK;
}

// =====================================================================================
// tcgen05 / TMEM core: the same GEMM on the 5th-generation tensor cores, fp32-accurate.
//
// kind::tf32 reads 19 of the 32 operand bits, so each operand is split into
// hi = tf32(x) and lo = x - hi and three MMAs per K step accumulate
// lo*hi + hi*lo + hi*hi in the fp32 TMEM accumulator (the dropped lo*lo term is
// ~2^-22 relative): results sit at the fp32 rounding floor.
//
// Shared-memory bandwidth is what bounds a 3-term tf32 product with both operands
// in shared memory (every MMA re-reads a 4 KB A tile and a 4 KB W tile), so the A
// operand lives in TENSOR MEMORY instead:
//   * One CTA = one 128x128 output tile; 4 producer/epilogue warps + 1 control warp;
//     256 TMEM columns per CTA (128 accumulator + 2 x (32 hi + 32 lo) A columns),
//     two CTAs resident per SM.
//   * Producer warp w owns rows 32w..32w+31 of the tile; thread t owns row t (= TMEM
//     lane t).  The warp gathers its rows' 32-float K chunk with cp.async (coalesced
//     128-byte row reads through the optional index, three stages = two chunks in
//     flight, no registers held) into a swizzled shared-memory patch, from which
//     every thread reads its own row, applies the optional SiLU, splits into hi / lo
//     and writes both with tcgen05.st into the A buffer of that chunk.
//   * W tiles: hi / lo parts of the weights (split once by the caller: W_hi, W_lo)
//     arrive by TMA (cp.async.bulk.tensor, 128-byte swizzle, no cluster forms) into
//     a double buffer, completing on mbarrier transaction counts.
//   * The control thread issues 12 tcgen05.mma per chunk (4 K steps x 3 split terms,
//     A from TMEM, W from shared memory) and commits them to mbarriers that free the
//     A buffer and the W slot.
//   * Epilogue: tcgen05.ld (one thread per row) -> shared-memory staging -> coalesced
//     row-wise bias / SiLU' gate / SiLU / residual / scale and store, accumulate or
//     atomic scatter.
// Every mbarrier wait is bounded; on expiry a status word is set and the kernel
// finishes normally (TMEM is always released).
#include <cuda.h>
#include <stdio.h>
#include <type_traits>

namespace mb {

constexpr int TC_THREADS = 160;                 // warps 0-3: producers + epilogue, warp 4: control
constexpr int TC_BK = 32;                       // floats per K chunk = one 128-byte swizzle row
constexpr int TC_TILE_BYTES = 128 * 128;        // 128 rows x 128 bytes
constexpr int TC_W_SLOTS = 2;
constexpr int TC_A_STAGES = 3;                  // cp.async stages of the A gather, per producer warp
constexpr int TC_STAGE_LD = 132;                // floats per staged output row (128 + 4 padding)
constexpr int TC_RING_BYTES = TC_W_SLOTS * 2 * TC_TILE_BYTES;  // 96 KB, reused as the epilogue staging area
constexpr int TC_XPOSE_BYTES = 4 * TC_A_STAGES * 32 * 128;  // per producer warp and stage: 32 rows x 128 bytes, chunk-swizzled
constexpr int TC_SMEM_BYTES = TC_RING_BYTES + TC_XPOSE_BYTES + 128 /*barriers, tmem slot*/;
constexpr uint32_t TC_TMEM_COLS = 256;
constexpr uint32_t TC_IDESC = (1u << 4) | (2u << 7) | (2u << 10) | ((128u >> 3) << 17) | ((128u >> 4) << 24);
constexpr uint32_t TC_WAIT_LIMIT = 1u << 20;     // polls per wait; each may park for up to TC_WAIT_HINT_NS
constexpr uint32_t TC_WAIT_HINT_NS = 4000;
static_assert(128 * TC_STAGE_LD * 4 <= TC_RING_BYTES + TC_XPOSE_BYTES, "staging area must fit in ring + patches");
static_assert(2 * (TC_SMEM_BYTES + 1024) <= 227 * 1024, "two CTAs per SM");

struct alignas(64) TcMaps { CUtensorMap m[4][2]; };  // per column block: W_hi, W_lo

__device__ int g_gemm_status = 0;  // bit 0: an mbarrier wait expired

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// Bounded wait.  The suspend-time hint lets the hardware park the thread until the phase completes (or the hint runs
// out) instead of re-issuing the poll: waiting warps then leave the issue slots to the warps that convert and store.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, uint32_t limit = TC_WAIT_LIMIT) {
  uint32_t ok;
  // fast path: a phase that has already completed is seen by one non-blocking test
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
               : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  if (ok) return true;
  for (uint32_t it = 0; it < limit; ++it) {
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity), "r"(TC_WAIT_HINT_NS) : "memory");
    if (ok) return true;
  }
  atomicOr(&g_gemm_status, 1);
  return false;
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(bar) : "memory");
}

__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr) {
  // K-major, SWIZZLE_128B: start address, LBO = 1 (unused), SBO = 1024 B between 8-row groups, version 1
  return (uint64_t)((saddr & 0x3FFFFu) >> 4) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}

// D[tmem] (+)= A[tmem] * B[smem]^T, M = 128, N = 128, K = 8 (tf32)
__device__ __forceinline__ void umma_tf32_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t db, uint32_t accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
               "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t}"
               :: "r"(tmem_d), "r"(tmem_a), "l"(db), "r"(TC_IDESC), "r"(accumulate) : "memory");
}

__device__ __forceinline__ float to_tf32(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return __uint_as_float(r);
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
               :: "r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y) : "memory");
}

#define MB_TMEM_ST32(taddr, v)                                                                                   \
  asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "                                                   \
               "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "                        \
               "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"                \
               :: "r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]),      \
                  "r"(v[7]), "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]),  \
                  "r"(v[15]), "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]),           \
                  "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]),           \
                  "r"(v[29]), "r"(v[30]), "r"(v[31]) : "memory")

#define MB_TMEM_ST16(taddr, v)                                                                                   \
  asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "                                                   \
               "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"                        \
               :: "r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]),      \
                  "r"(v[7]), "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]),  \
                  "r"(v[15]) : "memory")

#define MB_TMEM_LD32(taddr, v)                                                                                   \
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "                                                         \
               "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "                         \
               "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"         \
               : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), \
                 "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]),        \
                 "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]),      \
                 "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]),      \
                 "=r"(v[29]), "=r"(v[30]), "=r"(v[31]) : "r"(taddr) : "memory")

__global__ void __launch_bounds__(TC_THREADS, 2)
k_gemm_tc(const __grid_constant__ mb_gemm_desc d, const __grid_constant__ TcMaps maps) {
  const int jb = (int)(blockIdx.x % (unsigned)d.n_blocks);  // column block (fastest: the blocks of a row tile share A in L2)
  const int64_t row0 = (int64_t)(blockIdx.x / (unsigned)d.n_blocks) * 128;
  const mb_colblock& cb = d.blk[jb];
  extern __shared__ __align__(1024) uint8_t smem[];  // W ring (1024-byte aligned tiles) | transpose patches | barriers
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + TC_RING_BYTES + TC_XPOSE_BYTES);
  // bars[0..1]: A buffer full (4 producer warps); bars[2..3]: W slot landed (TMA); bars[5..6]: MMAs of a chunk done
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + TC_RING_BYTES + TC_XPOSE_BYTES + 64);
  if ((smem_u32(smem) & 1023u) != 0) {  // the swizzled tiles need a 1024-byte aligned base
    if (threadIdx.x == 0) atomicOr(&g_gemm_status, 2);
    return;
  }
  const uint32_t a_full = smem_u32(bars), w_full = smem_u32(bars + 2), mma_done = smem_u32(bars + 5);
  const uint32_t ring = smem_u32(smem);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // Descriptor fields are read once into registers: the descriptor sits in kernel-parameter memory that is
  // indexed dynamically (column block), and re-reading it inside the loops costs a memory round trip each time.
  const int64_t n_rows = d.n_rows;
  const int n_chunks = cb.n_src * (128 / TC_BK);

  // Producer state: thread = row = TMEM lane; declared before the set-up barrier so that the first two chunks'
  // gathers are already in flight while the control warp initialises barriers and allocates tensor memory.
  const int lr = lane >> 3, lc = lane & 7;  // coalesced loads: 8 lanes read one row's 128 bytes, 4 rows per instruction
  const uint32_t patch0 = smem_u32(smem + TC_RING_BYTES + (warp & 3) * (TC_A_STAGES * 32 * 128));
  const float* a_ptr[8];
  int32_t a_row[8];  // source row of each of this lane's 8 rows in the NEXT K segment (-1: past the end)
  const int n_src = cb.n_src;
  const float* const dummy_src = cb.src[0].ptr;  // valid address for zero-length copies of rows past the end
  auto resolve_rows = [&](int seg) {  // issued well before the segment starts, so the index loads are hidden
    const int32_t* idx = cb.src[seg].idx;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int64_t r = row0 + warp * 32 + lr + 4 * i;
      a_row[i] = r < n_rows ? (idx ? idx[r] : (int32_t)(r - row0)) : -1;
    }
  };
  // Asynchronous gather of chunk c: 8 lanes copy one row's 128 bytes (4 rows per instruction) straight into the
  // chunk-swizzled patch of stage c % 3: row (lr + 4i), 16-byte chunk lc -> patch[row][lc ^ (row & 7)].
  auto gather = [&](int c) {
    if ((c & 3) == 0) {  // new 128-wide K segment: turn the resolved rows into pointers
      const mb_src& s = cb.src[c >> 2];
      const float* base = s.ptr + s.col + lc * 4;
      const int64_t ld = s.ld;
      const bool gathered = s.idx != nullptr;
#pragma unroll
      for (int i = 0; i < 8; ++i)
        a_ptr[i] = a_row[i] < 0 ? nullptr : base + (gathered ? (int64_t)a_row[i] : row0 + a_row[i]) * ld;
    }
    if ((c & 3) == 1 && (c >> 2) + 1 < n_src) resolve_rows((c >> 2) + 1);
    const int kofs = (c & 3) * TC_BK;
    const uint32_t patch = patch0 + (uint32_t)(c % TC_A_STAGES) * (32 * 128);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int row = lr + 4 * i;
      const uint32_t dst = patch + row * 128 + ((lc ^ (row & 7)) << 4);
      const float* src = a_ptr[i] ? a_ptr[i] + kofs : dummy_src;
      const int bytes = a_ptr[i] ? 16 : 0;  // 0: nothing is read, the 16 destination bytes are zero-filled
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" :: "r"(dst), "l"(src), "r"(bytes) : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };

  const CUtensorMap* const map_hi = &maps.m[jb][0];
  const CUtensorMap* const map_lo = &maps.m[jb][1];
  auto load_w = [&](int c) {  // W_hi / W_lo rows 0..127, K columns 32c..32c+31 -> ring slot c & 1
    const int slot = c % TC_W_SLOTS;
    const uint32_t bar = w_full + 8 * slot, dst = ring + (uint32_t)slot * 2 * TC_TILE_BYTES;
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(bar), "r"(2 * TC_TILE_BYTES) : "memory");
    tma_load_2d(dst, map_hi, bar, c * TC_BK, 0);
    tma_load_2d(dst + TC_TILE_BYTES, map_lo, bar, c * TC_BK, 0);
  };

  if (warp == 4) {
    if (lane == 0) {
      mbar_init(a_full, 4); mbar_init(a_full + 8, 4);
      mbar_init(w_full, 1); mbar_init(w_full + 8, 1);
      mbar_init(mma_done, 1); mbar_init(mma_done + 8, 1);
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      load_w(0);  // the first weight tiles travel while tensor memory is being allocated
      if (n_chunks > 1) load_w(1);
    }
    __syncwarp();
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 :: "r"(smem_u32(tmem_slot)), "r"(TC_TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  } else {
    resolve_rows(0);
    gather(0);
    if (n_chunks > 1) gather(1); else asm volatile("cp.async.commit_group;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 4) {
    // ------------------------------------------------------------ control thread: TMA + MMA issue
    if (lane == 0) {
      bool alive = true;
      for (int c = 0; c < n_chunks; ++c) {
        const int ab = c & 1;  // A buffer, W slot and completion barrier of this chunk
        if (alive) alive = mbar_wait(a_full + 8 * ab, (uint32_t)((c >> 1) & 1));
        if (alive) alive = mbar_wait(w_full + 8 * ab, (uint32_t)((c >> 1) & 1));
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t wb = ring + (uint32_t)ab * 2 * TC_TILE_BYTES;
        const uint64_t dbh = umma_desc(wb), dbl = umma_desc(wb + TC_TILE_BYTES);
        const uint32_t ta_hi = tmem_base + 128 + 64 * ab, ta_lo = ta_hi + 32;
#pragma unroll
        for (int k = 0; k < 4; ++k) {  // K steps of 8: 8 TMEM columns of A, 32 bytes (>> 4 = 2) of the W rows
          const uint64_t adv = (uint64_t)(2 * k);
          umma_tf32_ts(tmem_base, ta_lo + 8 * k, dbh + adv, (c > 0 || k > 0) ? 1u : 0u);
          umma_tf32_ts(tmem_base, ta_hi + 8 * k, dbl + adv, 1u);
          umma_tf32_ts(tmem_base, ta_hi + 8 * k, dbh + adv, 1u);
        }
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                     :: "r"(mma_done + 8 * ab) : "memory");
        if (c + 2 < n_chunks) {  // this chunk's W slot is refilled as soon as its MMAs have retired
          if (alive) alive = mbar_wait(mma_done + 8 * ab, (uint32_t)((c >> 1) & 1));
          load_w(c + 2);
        }
      }
    }
    return;
  }

  // -------------------------------------------------------------- producers: thread = row = TMEM lane
  const uint32_t lane_base = tmem_base + ((uint32_t)(warp * 32) << 16);
  int act_of_seg[4];
#pragma unroll
  for (int sgm = 0; sgm < 4; ++sgm) act_of_seg[sgm] = sgm < cb.n_src ? cb.src[sgm].act : 0;

  bool alive = true;
  for (int c = 0; c < n_chunks; ++c) {
    const int ab = c & 1;
    // stage (c+2) % 3 was last read for chunk c-1, and the __syncwarp that closed that chunk orders those reads
    if (c + 2 < n_chunks) gather(c + 2); else asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group 2;" ::: "memory");  // chunk c's copies of this lane have landed
    __syncwarp();                                          // ... and so have the other lanes'
    const uint32_t patch = patch0 + (uint32_t)(c % TC_A_STAGES) * (32 * 128);
    float x[32];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const uint32_t addr = patch + lane * 128 + ((j ^ (lane & 7)) << 4);
      asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(x[4 * j]), "=f"(x[4 * j + 1]), "=f"(x[4 * j + 2]),
                   "=f"(x[4 * j + 3]) : "r"(addr) : "memory");
    }
    uint32_t hi[32], lo[32];
    if (act_of_seg[c >> 2]) {  // branch once per chunk: the SiLU must not be evaluated (and discarded) on the plain path
#pragma unroll
      for (int q = 0; q < 32; ++q) x[q] = silu_fast_f(x[q]);
    }
#pragma unroll
    for (int q = 0; q < 32; ++q) {
      const float h = to_tf32(x[q]);
      hi[q] = __float_as_uint(h);
      lo[q] = __float_as_uint(x[q] - h);
    }
    if (c >= 2 && alive) alive = mbar_wait(mma_done + 8 * ab, (uint32_t)(((c >> 1) - 1) & 1));  // A buffer ab is free again
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t ta = lane_base + 128 + 64 * ab;
    MB_TMEM_ST32(ta, hi);
    MB_TMEM_ST32(ta + 32, lo);
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncwarp();  // all lanes have read their patch rows: the stage may be overwritten two chunks from now
    if (lane == 0) mbar_arrive(a_full + 8 * ab);
  }
  // all MMAs retire in order: the last chunk's commit covers the whole accumulator
  if (alive) alive = mbar_wait(mma_done + 8 * ((n_chunks - 1) & 1), (uint32_t)(((n_chunks - 1) >> 1) & 1));
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");

  // -------------------------------------------------------------- epilogue
  // (1) accumulator row -> staging (the W ring is idle: every TMA landed and every MMA retired)
  float* stage = reinterpret_cast<float*>(smem);
#pragma unroll 1
  for (int cg = 0; cg < 4; ++cg) {
    uint32_t v[32];
    MB_TMEM_LD32(lane_base + (uint32_t)(cg * 32), v);
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int q = 0; q < 8; ++q)
      *reinterpret_cast<uint4*>(stage + tid * TC_STAGE_LD + cg * 32 + 4 * q) = make_uint4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  asm volatile("bar.sync 1, 128;" ::: "memory");  // the four epilogue warps only
  if (warp == 0) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem_base), "r"(TC_TMEM_COLS) : "memory");
  }
  // (2) warp w finishes rows w, w+4, ...: lane l owns columns 4l..4l+3, every global access is a full 512-byte row
  const int col = lane * 4;
  const float* const gate = cb.gate;
  const float* const res = cb.res;
  const int32_t* const out_idx = cb.out_idx;
  float* const out = cb.out;
  const int64_t ld_gate = cb.ld_gate, ld_res = cb.ld_res, ld_out = cb.ld_out;
  const int gcol = cb.col_gate + col, rcol = cb.col_res + col, ocol = cb.col_out + col;
  const int mode = cb.mode, out_act = cb.out_act;
  const float sc = cb.out_scale;
  float4 bias4 = make_float4(0.f, 0.f, 0.f, 0.f), resw4 = make_float4(1.f, 1.f, 1.f, 1.f);
  if (cb.bias) bias4 = ld4(cb.bias + col);
  if (res && cb.res_w) resw4 = ld4(cb.res_w + col);
  if (!alive) return;
  const int rows_here = (int)((n_rows - row0) < 128 ? (n_rows - row0) : 128);
  // Rows are finished eight at a time per warp: all global reads of a batch (gate, residual, scatter index, old
  // value) are issued before the first dependent use, so eight rows' latencies overlap instead of adding up.
  constexpr int RB = 8;
  auto finish_rows = [&](auto has_gate, auto has_act, auto has_res) {
#pragma unroll 1
    for (int r0 = warp; r0 < rows_here; r0 += 4 * RB) {
      float4 z[RB], x[RB];
      int64_t dr[RB];
#pragma unroll
      for (int i = 0; i < RB; ++i) {
        const int rr = r0 + 4 * i;
        const bool valid = rr < rows_here;
        const int64_t gr = row0 + (valid ? rr : r0);
        if constexpr (decltype(has_gate)::value) z[i] = ld4(gate + gr * ld_gate + gcol);
        if constexpr (decltype(has_res)::value) x[i] = ld4(res + gr * ld_res + rcol);
        dr[i] = out_idx ? (int64_t)out_idx[gr] : gr;
      }
#pragma unroll
      for (int i = 0; i < RB; ++i) {
        const int rr = r0 + 4 * i;
        if (rr >= rows_here) break;
        const float4 a = *reinterpret_cast<const float4*>(stage + rr * TC_STAGE_LD + col);
        float o[4] = {a.x + bias4.x, a.y + bias4.y, a.z + bias4.z, a.w + bias4.w};
        if constexpr (decltype(has_gate)::value) {
          o[0] *= silu_grad_fast_f(z[i].x); o[1] *= silu_grad_fast_f(z[i].y);
          o[2] *= silu_grad_fast_f(z[i].z); o[3] *= silu_grad_fast_f(z[i].w);
        }
        if constexpr (decltype(has_act)::value) {
          o[0] = silu_fast_f(o[0]); o[1] = silu_fast_f(o[1]); o[2] = silu_fast_f(o[2]); o[3] = silu_fast_f(o[3]);
        }
        if constexpr (decltype(has_res)::value) {
          o[0] = fmaf(resw4.x, x[i].x, o[0]); o[1] = fmaf(resw4.y, x[i].y, o[1]);
          o[2] = fmaf(resw4.z, x[i].z, o[2]); o[3] = fmaf(resw4.w, x[i].w, o[3]);
        }
        const float4 ov = make_float4(o[0] * sc, o[1] * sc, o[2] * sc, o[3] * sc);
        float* dst = out + dr[i] * ld_out + ocol;
        if (mode == MB_OUT_STORE) {
          *reinterpret_cast<float4*>(dst) = ov;
        } else if (mode == MB_OUT_ADD) {
          float4 p = ld4(dst);
          p.x += ov.x; p.y += ov.y; p.z += ov.z; p.w += ov.w;
          *reinterpret_cast<float4*>(dst) = p;
        } else {
          atomicAdd(reinterpret_cast<float4*>(dst), ov);
        }
      }
    }
  };
  // the transcendental epilogue terms are compiled out of the variants that do not use them
  using T = std::true_type;
  using F = std::false_type;
  auto pick_res = [&](auto g, auto a) { if (res) finish_rows(g, a, T{}); else finish_rows(g, a, F{}); };
  auto pick_act = [&](auto g) { if (out_act) pick_res(g, T{}); else pick_res(g, F{}); };
  if (gate) pick_act(T{}); else pick_act(F{});
}

#include "gemm_persistent.cuh"
#include "gated_persistent.cuh"

// 0: persistent tcgen05 3xBF16 (default), 1: fp32 SIMT, 2: one-tile-per-CTA tcgen05 3xTF32, 3: persistent tcgen05 3xTF32
static int g_gemm_mode = 0;

// TMA descriptor of a [rows, k] float32 weight block (row stride ldw), box 128 rows x 32 columns, 128-byte swizzle.
// Encoding depends only on (address, stride, k, rows), so descriptors are cached per host thread.
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static int weight_map(const void* w, int64_t ldw, int k, CUtensorMap* out, int rows = 128, bool bf16 = false) {
  static EncodeTiledFn encode = nullptr;
  if (!encode) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    MB_CUDA_CHECK(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q));
    if (!fn || q != cudaDriverEntryPointSuccess) return MB_ERR_CUDA;
    encode = (EncodeTiledFn)fn;
  }
  static thread_local bool bound = false;
  if (!bound) {  // the driver call below needs this thread to have the device's context current
    MB_CUDA_CHECK(cudaFree(nullptr));
    bound = true;
  }
  struct Key { const void* w; int64_t ld; int k; int rows; int bf16; };
  struct Entry { Key key; CUtensorMap map; };
  constexpr int SLOTS = 1024;
  static thread_local Entry* cache = nullptr;
  if (!cache) cache = new Entry[SLOTS]();
  const size_t hsh = ((reinterpret_cast<uintptr_t>(w) >> 4) * 0x9E3779B97F4A7C15ull + (uint64_t)(k + rows)) >> 54;  // 10 bits
  Entry& e = cache[hsh % SLOTS];
  if (e.key.w == w && e.key.ld == ldw && e.key.k == k && e.key.rows == rows && e.key.bf16 == (int)bf16) {
    *out = e.map;
    return MB_OK;
  }
  const cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
  // float32 tiles: 128 rows x 32 values; bfloat16 tiles: 128 rows x 64 values (both 128 bytes per row).  The format
  // is part of the cache key: an allocator may hand the address of a freed weight of one format to one of the other.
  const cuuint64_t strides[1] = {(cuuint64_t)ldw * (bf16 ? 2 : 4)};
  const cuuint32_t box[2] = {(cuuint32_t)(bf16 ? 64 : TC_BK), 128};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = encode(out, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2,
                      const_cast<void*>(w), dims, strides, box, estr,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    char where[64];
    snprintf(where, sizeof(where), "cuTensorMapEncodeTiled (CUresult %d)", (int)r);
    set_cuda_error(cudaErrorInvalidValue, where);
    return MB_ERR_CUDA;
  }
  e.key = Key{w, ldw, k, rows, (int)bf16};
  e.map = *out;
  return MB_OK;
}

// Per-device set-up of the tensor-core kernels: the dynamic shared-memory attribute belongs to the (function, device)
// pair and the persistent grids are sized by the device's SM count.  One slot per device ordinal; two host threads
// that race on a device's first call write the same values.
struct DeviceConfig { bool ready; int n_sm; };
static DeviceConfig g_device_config[64];

static int device_config(int* n_sm) {
  int dev = 0;
  MB_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return MB_ERR_INVALID;
  DeviceConfig& c = g_device_config[dev];
  if (!c.ready) {
    MB_CUDA_CHECK(cudaFuncSetAttribute(k_gemm_tc, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM_BYTES));
    MB_CUDA_CHECK(cudaFuncSetAttribute(k_gemm_ps<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, PS_SMEM_BYTES));
    MB_CUDA_CHECK(cudaFuncSetAttribute(k_gemm_ps<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, PS_SMEM_BYTES));
    MB_CUDA_CHECK(cudaFuncSetAttribute(k_gated_fwd<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, GP_SMEM_BYTES));
    MB_CUDA_CHECK(cudaFuncSetAttribute(k_gated_fwd<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, GP_SMEM_BYTES));
    int n = 0;
    MB_CUDA_CHECK(cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev));
    c.n_sm = n;
    c.ready = true;
  }
  *n_sm = c.n_sm;
  return MB_OK;
}

// ---- self-test of the bounded wait: a barrier nothing arrives at, a limit of a few polls
__global__ void k_selftest_wait_expiry() {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bar), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  // same wait, same give-up path as in the GEMM kernels (status bit 0), with 8 polls of at most 4 us instead of 2^20
  if (threadIdx.x == 0) mbar_wait(smem_u32(&bar), 0, 8);
  __syncthreads();
}

// ---- issue rate of tcgen05.mma with resident operands (TS form: A in tensor memory, B in shared memory)
template <int KIND>  // 0: kind::tf32 (K = 8 per instruction), 1: kind::f16 with bf16 operands (K = 16)
__global__ void __launch_bounds__(128, 1) k_mma_rate(int iters) {
  extern __shared__ __align__(1024) uint8_t smem[];
  __shared__ uint64_t bar;
  __shared__ uint32_t slot;
  if ((smem_u32(smem) & 1023u) != 0) return;
  for (int i = threadIdx.x; i < 32 * 1024 / 4; i += blockDim.x) reinterpret_cast<float*>(smem)[i] = 0.f;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bar), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (threadIdx.x < 32) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" :: "r"(smem_u32(&slot)) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tb = slot;
  if (threadIdx.x < 32) {  // warp-uniform loop, one elected lane issues
    uint32_t elected;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(elected));
    const uint32_t fmt = KIND == 0 ? 2u : 1u;  // operand format field: tf32 / bf16
    const uint32_t idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((128u >> 3) << 17) | ((128u >> 4) << 24);
    const uint64_t db = umma_desc(smem_u32(smem));
    const uint32_t ta = tb + 256;
    for (int i = 0; i < iters; ++i) {
      if (elected) {
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          if (KIND == 0)
            asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                         "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t}"
                         :: "r"(tb), "r"(ta + 8 * kk), "l"(db + (uint64_t)(2 * kk)), "r"(idesc), "r"(1u) : "memory");
          else
            asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                         "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
                         :: "r"(tb), "r"(ta + 8 * kk), "l"(db + (uint64_t)(2 * kk)), "r"(idesc), "r"(1u) : "memory");
        }
      }
      __syncwarp();
    }
    if (elected)
      asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                   :: "r"(smem_u32(&bar)) : "memory");
    __syncwarp();
    // every issued instruction has retired when the commit arrives; bounded like every other wait here
    mbar_wait(smem_u32(&bar), 0, 1u << 22);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (threadIdx.x < 32) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" :: "r"(tb) : "memory");
  }
}

}  // namespace mb

extern "C" int mb_set_gemm_mode(int mode) {
  if (mode < 0 || mode > 3) return MB_ERR_INVALID;
  mb::g_gemm_mode = mode;
  return MB_OK;
}

extern "C" int mb_gemm_status(int* status, void* stream_) {
  if (!status) return MB_ERR_INVALID;
  int zero = 0;
  MB_CUDA_CHECK(cudaStreamSynchronize((cudaStream_t)stream_));
  MB_CUDA_CHECK(cudaMemcpyFromSymbol(status, mb::g_gemm_status, sizeof(int)));
  MB_CUDA_CHECK(cudaMemcpyToSymbol(mb::g_gemm_status, &zero, sizeof(int)));
  return MB_OK;
}

extern "C" int mb_gemm_status_async(int* host_status, void* stream_) {
  if (!host_status) return MB_ERR_INVALID;
  MB_CUDA_CHECK(cudaMemcpyFromSymbolAsync(host_status, mb::g_gemm_status, sizeof(int), 0, cudaMemcpyDeviceToHost,
                                          (cudaStream_t)stream_));
  return MB_OK;
}

extern "C" int mb_gemm_status_clear(void* stream_) {
  void* addr = nullptr;
  MB_CUDA_CHECK(cudaGetSymbolAddress(&addr, mb::g_gemm_status));
  MB_CUDA_CHECK(cudaMemsetAsync(addr, 0, sizeof(int), (cudaStream_t)stream_));
  return MB_OK;
}

extern "C" int mb_selftest_wait_expiry(void* stream_) {
  mb::k_selftest_wait_expiry<<<1, 32, 0, (cudaStream_t)stream_>>>();
  MB_LAUNCH_CHECK("k_selftest_wait_expiry");
  return MB_OK;
}

extern "C" int mb_bench_mma_rate(int kind, int iters, float* elapsed_ms, int* n_sms, void* stream_) {
  if ((kind != 0 && kind != 1) || iters < 1 || iters > (1 << 24) || !elapsed_ms || !n_sms) return MB_ERR_INVALID;
  int n_sm = 0;
  int rc = mb::device_config(&n_sm);
  if (rc) return rc;
  cudaStream_t st = (cudaStream_t)stream_;
  const int smem = 33 * 1024;
  cudaEvent_t e0, e1;
  MB_CUDA_CHECK(cudaEventCreate(&e0));
  MB_CUDA_CHECK(cudaEventCreate(&e1));
  cudaError_t err = cudaEventRecord(e0, st);
  if (err == cudaSuccess) {
    if (kind == 0) mb::k_mma_rate<0><<<n_sm, 128, smem, st>>>(iters);
    else mb::k_mma_rate<1><<<n_sm, 128, smem, st>>>(iters);
    err = cudaGetLastError();
  }
  if (err == cudaSuccess) err = cudaEventRecord(e1, st);
  if (err == cudaSuccess) err = cudaEventSynchronize(e1);
  if (err == cudaSuccess) err = cudaEventElapsedTime(elapsed_ms, e0, e1);
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  if (err != cudaSuccess) {
    mb::set_cuda_error(err, "mb_bench_mma_rate");
    return MB_ERR_CUDA;
  }
  *n_sms = n_sm;
  return MB_OK;
}

extern "C" int mb_gemm(const mb_gemm_desc* desc, void* stream_) {
  int rc = gemm_validate(desc);
  if (rc) return rc;
  if (desc->n_rows == 0) return MB_OK;
  const long long gx = (desc->n_rows + 127) / 128;
  if (gx * desc->n_blocks > 0x7fffffffLL) return MB_ERR_OVERFLOW;
  if (mb::g_gemm_mode == 1) {
    dim3 grid((unsigned)gx, (unsigned)desc->n_blocks);
    mb::k_gemm<<<grid, mb::GEMM_THREADS, 0, (cudaStream_t)stream_>>>(*desc);
  } else {
    int n_sm = 0;
    rc = mb::device_config(&n_sm);
    if (rc) return rc;
    // The persistent kernels' epilogue uses 32-byte accesses.  Operands aligned to 16 bytes only (a caller of the C
    // ABI that passes views at odd column offsets; the Python host side never does) take the one-tile kernel.
    bool wide_ok = true;
    for (int j = 0; j < desc->n_blocks; ++j) {
      const mb_colblock& cb = desc->blk[j];
      auto ok32 = [](const void* p, int64_t ld, int col) {
        return (reinterpret_cast<uintptr_t>(p) & 31) == 0 && (ld & 7) == 0 && (col & 7) == 0;
      };
      wide_ok = wide_ok && ok32(cb.out, cb.ld_out, cb.col_out) && (!cb.gate || ok32(cb.gate, cb.ld_gate, cb.col_gate)) &&
                (!cb.res || ok32(cb.res, cb.ld_res, cb.col_res)) && (!cb.bias || ok32(cb.bias, 0, 0)) &&
                (!cb.res_w || ok32(cb.res_w, 0, 0));
    }
    const bool persistent = (mb::g_gemm_mode == 0 || mb::g_gemm_mode == 3) && wide_ok;
    const bool bf16 = persistent && mb::g_gemm_mode == 0;
    mb::TcMaps maps;
    for (int j = 0; j < desc->n_blocks; ++j) {
      const mb_colblock& cb = desc->blk[j];
      const void* hi = bf16 ? (const void*)cb.W_hi16 : (const void*)cb.W_hi;
      const void* lo = bf16 ? (const void*)cb.W_lo16 : (const void*)cb.W_lo;
      if (!hi || !lo || !mb::aligned16(hi) || !mb::aligned16(lo) || (bf16 && (cb.ldw & 7))) return MB_ERR_INVALID;
      rc = mb::weight_map(hi, cb.ldw, 128 * cb.n_src, &maps.m[j][0], 128, bf16);
      if (rc) return rc;
      rc = mb::weight_map(lo, cb.ldw, 128 * cb.n_src, &maps.m[j][1], 128, bf16);
      if (rc) return rc;
    }
    const long long n_tiles = gx * desc->n_blocks;
    if (persistent) {
      // Shared-A mode: all column blocks read the same A operand and its chunks fit the kernel's A buffers (eight
      // 32-float chunks in bf16 form, four in tf32 form): a CTA then converts the A rows of a row tile once for all
      // of its column blocks.
      bool shared_a = desc->n_blocks > 1 && desc->blk[0].n_src * 4 <= (bf16 ? 8 : 4);
      for (int j = 1; j < desc->n_blocks && shared_a; ++j) {
        const mb_colblock& a = desc->blk[0], &b = desc->blk[j];
        shared_a = a.n_src == b.n_src;
        for (int s = 0; s < a.n_src && shared_a; ++s)
          shared_a = a.src[s].ptr == b.src[s].ptr && a.src[s].idx == b.src[s].idx && a.src[s].ld == b.src[s].ld &&
                     a.src[s].col == b.src[s].col && a.src[s].act == b.src[s].act;
      }
      const long long n_items = shared_a ? gx : n_tiles;
      const unsigned grid = (unsigned)(n_items < n_sm ? n_items : n_sm);
      const int sa = shared_a ? 1 : 0;
      if (bf16) mb::k_gemm_ps<true><<<grid, mb::PS_THREADS, mb::PS_SMEM_BYTES, (cudaStream_t)stream_>>>(*desc, maps, sa);
      else mb::k_gemm_ps<false><<<grid, mb::PS_THREADS, mb::PS_SMEM_BYTES, (cudaStream_t)stream_>>>(*desc, maps, sa);
    } else {
      mb::k_gemm_tc<<<(unsigned)n_tiles, mb::TC_THREADS, mb::TC_SMEM_BYTES, (cudaStream_t)stream_>>>(*desc, maps);
    }
  }
  MB_LAUNCH_CHECK("k_gemm");
  return MB_OK;
}

// The same result as the fused kernel from the separate kernels (GEMM modes 1 and 2, or operands that are only
// 16-byte aligned): two mb_gemm launches and the row-wise gate kernel, with z1 / z2 as scratch.
static int gated_mlp_composed(const mb_gated_mlp* g, void* stream_) {
  if (g->kind == MB_MLP_PLAIN) {
    if (!g->z1 || !g->W1 || !g->W2) return MB_ERR_INVALID;
    mb_gemm_desc a = {}, b = {};
    a.n_rows = b.n_rows = g->n_rows;
    a.n_blocks = b.n_blocks = 1;
    mb_colblock& ca = a.blk[0];
    ca.n_src = g->n_src;
    for (int s = 0; s < g->n_src; ++s) ca.src[s] = g->src[s];
    ca.W = g->W1; ca.W_hi = g->W1_hi; ca.W_lo = g->W1_lo; ca.W_hi16 = g->W1_hi16; ca.W_lo16 = g->W1_lo16;
    ca.ldw = g->ldw1; ca.bias = g->b1;
    ca.out = g->z1; ca.ld_out = g->ld_z1; ca.out_scale = 1.f; ca.mode = MB_OUT_STORE;
    int rc = mb_gemm(&a, stream_);
    if (rc) return rc;
    mb_colblock& cb = b.blk[0];
    cb.n_src = 1;
    cb.src[0].ptr = g->z1; cb.src[0].ld = g->ld_z1; cb.src[0].act = 1;
    cb.W = g->W2; cb.W_hi = g->W2_hi; cb.W_lo = g->W2_lo; cb.W_hi16 = g->W2_hi16; cb.W_lo16 = g->W2_lo16;
    cb.ldw = g->ldw2; cb.bias = g->b2; cb.out_scale = 1.f; cb.mode = MB_OUT_STORE;
    if (g->h) {  // h = y; out2, when also wanted, by a second pass of the (cheap) second layer
      cb.out = g->h; cb.ld_out = g->ld_h;
      if ((rc = mb_gemm(&b, stream_))) return rc;
    }
    if (g->out2) {
      cb.out = g->out2; cb.ld_out = g->ld_out2;
      cb.res = g->res; cb.res_w = g->res_w; cb.ld_res = g->ld_res;
      if ((rc = mb_gemm(&b, stream_))) return rc;
    }
    return MB_OK;
  }
  if (!g->z1 || !g->z2 || g->ld_z2 != 256 || !g->W1 || !g->W2) return MB_ERR_INVALID;
  if ((g->h && g->ld_h != 128) || (g->out2 && (g->ld_out2 != 128 || g->ld_res != 128))) return MB_ERR_INVALID;
  mb_gemm_desc a = {}, b = {};
  a.n_rows = b.n_rows = g->n_rows;
  a.n_blocks = b.n_blocks = 2;
  for (int j = 0; j < 2; ++j) {
    mb_colblock& ca = a.blk[j];
    ca.n_src = g->n_src;
    for (int s = 0; s < g->n_src; ++s) ca.src[s] = g->src[s];
    ca.W = g->W1 + (int64_t)128 * j * g->ldw1;
    ca.W_hi = g->W1_hi ? g->W1_hi + (int64_t)128 * j * g->ldw1 : nullptr;
    ca.W_lo = g->W1_lo ? g->W1_lo + (int64_t)128 * j * g->ldw1 : nullptr;
    ca.W_hi16 = g->W1_hi16 ? g->W1_hi16 + (int64_t)128 * j * g->ldw1 : nullptr;
    ca.W_lo16 = g->W1_lo16 ? g->W1_lo16 + (int64_t)128 * j * g->ldw1 : nullptr;
    ca.ldw = g->ldw1;
    ca.bias = g->b1 ? g->b1 + 128 * j : nullptr;
    ca.out = g->z1; ca.ld_out = g->ld_z1; ca.col_out = 128 * j; ca.out_scale = 1.f; ca.mode = MB_OUT_STORE;
    mb_colblock& cb = b.blk[j];
    cb.n_src = 1;
    cb.src[0].ptr = g->z1; cb.src[0].ld = g->ld_z1; cb.src[0].col = 128 * j; cb.src[0].act = 1;
    cb.W = g->W2 + (int64_t)128 * j * g->ldw2;
    cb.W_hi = g->W2_hi ? g->W2_hi + (int64_t)128 * j * g->ldw2 : nullptr;
    cb.W_lo = g->W2_lo ? g->W2_lo + (int64_t)128 * j * g->ldw2 : nullptr;
    cb.W_hi16 = g->W2_hi16 ? g->W2_hi16 + (int64_t)128 * j * g->ldw2 : nullptr;
    cb.W_lo16 = g->W2_lo16 ? g->W2_lo16 + (int64_t)128 * j * g->ldw2 : nullptr;
    cb.ldw = g->ldw2;
    cb.bias = g->b2 ? g->b2 + 128 * j : nullptr;
    cb.out = g->z2; cb.ld_out = g->ld_z2; cb.col_out = 128 * j; cb.out_scale = 1.f; cb.mode = MB_OUT_STORE;
  }
  int rc = mb_gemm(&a, stream_);
  if (rc) return rc;
  rc = mb_gemm(&b, stream_);
  if (rc) return rc;
  return mb_gate_fwd(g->n_rows, g->z2, g->norm_core, g->norm_gate, g->h, g->res, g->res_w, g->out2, stream_);
}

extern "C" int mb_gated_mlp_fwd(const mb_gated_mlp* g, void* stream_) {
  if (!g || g->n_rows < 0 || g->n_src < 1 || g->n_src > 4) return MB_ERR_INVALID;
  if (g->kind != MB_MLP_GATED && g->kind != MB_MLP_PLAIN) return MB_ERR_INVALID;
  const bool plain = g->kind == MB_MLP_PLAIN;
  if ((!plain && (!g->norm_core || !g->norm_gate)) || (!g->h && !g->out2) || (g->out2 && !g->res)) return MB_ERR_INVALID;
  if (g->ldw1 < 128 * g->n_src || (g->ldw1 & 3) || g->ldw2 < 128 || (g->ldw2 & 3)) return MB_ERR_INVALID;
  for (int s = 0; s < g->n_src; ++s) {
    const mb_src& sr = g->src[s];
    if (!sr.ptr || !mb::aligned16(sr.ptr) || (sr.ld & 3) || (sr.col & 3)) return MB_ERR_INVALID;
  }
  if (g->n_rows == 0) return MB_OK;
  if ((g->n_rows + 127) / 128 > 0x3fffffffLL) return MB_ERR_OVERFLOW;
  auto ok32 = [](const void* p, int64_t ld) { return (reinterpret_cast<uintptr_t>(p) & 31) == 0 && (ld & 7) == 0; };
  const bool wide_ok = (!g->z1 || ok32(g->z1, g->ld_z1)) && (plain || !g->z2 || ok32(g->z2, g->ld_z2)) &&
                       (!g->h || ok32(g->h, g->ld_h)) && (!g->out2 || (ok32(g->out2, g->ld_out2) && ok32(g->res, g->ld_res))) &&
                       (!g->b1 || ok32(g->b1, 0)) && (!g->b2 || ok32(g->b2, 0)) &&
                       (plain || (ok32(g->norm_core, 0) && ok32(g->norm_gate, 0))) && (!g->res_w || ok32(g->res_w, 0));
  // The fused kernel computes with the 3xBF16 split (the default mode); the other modes compose the three launches.
  if (mb::g_gemm_mode != 0 || !wide_ok) return gated_mlp_composed(g, stream_);
  const void* w1h = g->W1_hi16, *w1l = g->W1_lo16, *w2h = g->W2_hi16, *w2l = g->W2_lo16;
  if (!w1h || !w1l || !w2h || !w2l) return MB_ERR_INVALID;
  if (!mb::aligned16(w1h) || !mb::aligned16(w1l) || !mb::aligned16(w2h) || !mb::aligned16(w2l)) return MB_ERR_INVALID;
  if ((g->ldw1 & 7) || (g->ldw2 & 7)) return MB_ERR_INVALID;
  int n_sm = 0;
  int rc = mb::device_config(&n_sm);
  if (rc) return rc;
  mb::GatedMaps maps;
  const int w_rows = plain ? 128 : 256;
  if ((rc = mb::weight_map(w1h, g->ldw1, 128 * g->n_src, &maps.w1[0], w_rows, true))) return rc;
  if ((rc = mb::weight_map(w1l, g->ldw1, 128 * g->n_src, &maps.w1[1], w_rows, true))) return rc;
  if ((rc = mb::weight_map(w2h, g->ldw2, 128, &maps.w2[0], w_rows, true))) return rc;
  if ((rc = mb::weight_map(w2l, g->ldw2, 128, &maps.w2[1], w_rows, true))) return rc;
  const long long n_tiles = (g->n_rows + 127) / 128;
  const unsigned grid = (unsigned)(n_tiles < n_sm ? n_tiles : n_sm);
  if (plain) mb::k_gated_fwd<true><<<grid, mb::GP_THREADS, mb::GP_SMEM_BYTES, (cudaStream_t)stream_>>>(*g, maps);
  else mb::k_gated_fwd<false><<<grid, mb::GP_THREADS, mb::GP_SMEM_BYTES, (cudaStream_t)stream_>>>(*g, maps);
  MB_LAUNCH_CHECK("k_gated_fwd");
  return MB_OK;
}
