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
// hi = tf32(x) and lo = tf32(x - hi) and three MMAs per K step accumulate
// lo*hi + hi*lo + hi*hi in the fp32 TMEM accumulator (the dropped lo*lo term is
// ~2^-22 relative): results sit at the fp32 rounding floor.
//
// One CTA = one 128x128 output tile, 128 threads.  Per K chunk of 32: all threads
// gather/convert the A rows and the W rows into four 128x32 K-major tiles in the
// 128-byte-swizzled canonical layout (hi/lo of A and of W), then one thread issues
// 12 tcgen05.mma (4 K steps x 3 split terms) and commits them to an mbarrier.  The
// next chunk's global loads are already in flight in registers.  Three CTAs are
// resident per SM (64 KB of tiles + 128 TMEM columns each), so one CTA's MMAs
// overlap the other CTAs' tile fills.  Epilogue: tcgen05.ld, one thread per row.
// Every mbarrier wait is bounded; on expiry a status word is set and the kernel
// finishes normally (TMEM is always released).
namespace mb {

constexpr int TC_THREADS = 128;
constexpr int TC_BK = 32;                       // floats per K chunk = one 128-byte swizzle row
constexpr int TC_TILE_BYTES = 128 * 128;        // 128 rows x 128 bytes
constexpr int TC_SMEM_BYTES = 4 * TC_TILE_BYTES + 1024 /*alignment slack*/ + 64 /*barrier, tmem slot*/;
constexpr uint32_t TC_IDESC = (1u << 4) | (2u << 7) | (2u << 10) | ((128u >> 3) << 17) | ((128u >> 4) << 24);
constexpr uint32_t TC_WAIT_LIMIT = 1u << 24;

__device__ int g_gemm_status = 0;  // bit 0: an mbarrier wait expired

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  for (uint32_t it = 0; it < TC_WAIT_LIMIT; ++it) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    if (ok) return true;
  }
  atomicOr(&g_gemm_status, 1);
  return false;
}

__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr) {
  // K-major, SWIZZLE_128B: start address, LBO = 1 (unused), SBO = 1024 B between 8-row groups, version 1
  return (uint64_t)((saddr & 0x3FFFFu) >> 4) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}

__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
               "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
               :: "r"(tmem_d), "l"(da), "l"(db), "r"(TC_IDESC), "r"(accumulate) : "memory");
}

__device__ __forceinline__ float to_tf32(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return __uint_as_float(r);
}

// write a float4 (4 consecutive K values of one row) as hi / lo into the swizzled tiles
__device__ __forceinline__ void store_split(uint8_t* tile_hi, uint8_t* tile_lo, int row, int chunk, float4 v) {
  const int off = (row >> 3) * 1024 + (row & 7) * 128 + ((chunk ^ (row & 7)) << 4);
  float4 h = make_float4(to_tf32(v.x), to_tf32(v.y), to_tf32(v.z), to_tf32(v.w));
  float4 l = make_float4(to_tf32(v.x - h.x), to_tf32(v.y - h.y), to_tf32(v.z - h.z), to_tf32(v.w - h.w));
  *reinterpret_cast<float4*>(tile_hi + off) = h;
  *reinterpret_cast<float4*>(tile_lo + off) = l;
}

__global__ void __launch_bounds__(TC_THREADS, 3) k_gemm_tc(const __grid_constant__ mb_gemm_desc d) {
  const mb_colblock& cb = d.blk[blockIdx.y];
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* a_hi = smem;
  uint8_t* a_lo = smem + TC_TILE_BYTES;
  uint8_t* b_hi = smem + 2 * TC_TILE_BYTES;
  uint8_t* b_lo = smem + 3 * TC_TILE_BYTES;
  uint64_t* bar = reinterpret_cast<uint64_t*>(smem + 4 * TC_TILE_BYTES);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + 4 * TC_TILE_BYTES + 16);

  const int tid = threadIdx.x, warp = tid >> 5;
  const int64_t row0 = (int64_t)blockIdx.x * 128;
  const int lrow = tid >> 3, chunk = tid & 7;   // loader: rows lrow + 16 i (i = 0..7), 16-byte chunk `chunk`
  const int n_chunks = cb.n_src * (128 / TC_BK);
  const uint32_t bar_addr = smem_u32(bar);

  if (tid == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" :: "r"(bar_addr) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 128;" :: "r"(smem_u32(tmem_slot)) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  const float* a_ptr[8];
  int a_act = 0;
  const float* b_ptr = cb.W + (int64_t)lrow * cb.ldw + chunk * 4;
  const int64_t b_step = 16 * cb.ldw;
  float4 a_reg[8], b_reg[8];

  auto prefetch = [&](int c) {
    if ((c & 3) == 0) {  // new 128-wide K segment: resolve the gathered row pointers
      const mb_src& s = cb.src[c >> 2];
      a_act = s.act;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int64_t r = row0 + lrow + 16 * i;
        if (r < d.n_rows) {
          const int64_t sr = s.idx ? (int64_t)s.idx[r] : r;
          a_ptr[i] = s.ptr + sr * s.ld + s.col + chunk * 4;
        } else {
          a_ptr[i] = nullptr;
        }
      }
    }
    const int kofs = (c & 3) * TC_BK;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (a_ptr[i]) v = ld4(a_ptr[i] + kofs);
      a_reg[i] = v;
      b_reg[i] = ld4(b_ptr + i * b_step + c * TC_BK);
    }
  };

  bool alive = true;
  prefetch(0);
  for (int c = 0; c < n_chunks; ++c) {
    if (c > 0 && alive) alive = mbar_wait(bar_addr, (uint32_t)((c - 1) & 1));  // previous chunk's MMAs have read the tiles
    const int act = a_act;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float4 v = a_reg[i];
      if (act) { v.x = silu_f(v.x); v.y = silu_f(v.y); v.z = silu_f(v.z); v.w = silu_f(v.w); }
      store_split(a_hi, a_lo, lrow + 16 * i, chunk, v);
      store_split(b_hi, b_lo, lrow + 16 * i, chunk, b_reg[i]);
    }
    if (c + 1 < n_chunks) prefetch(c + 1);
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy stores -> visible to the MMA's async proxy
    __syncthreads();
    if (tid == 0) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint64_t dah = umma_desc(smem_u32(a_hi)), dal = umma_desc(smem_u32(a_lo));
      const uint64_t dbh = umma_desc(smem_u32(b_hi)), dbl = umma_desc(smem_u32(b_lo));
#pragma unroll
      for (int k = 0; k < 4; ++k) {  // 4 K steps of 8 tf32 = 32 bytes: advance the start address by 32 >> 4
        const uint64_t adv = (uint64_t)(2 * k);
        umma_tf32(tmem_base, dal + adv, dbh + adv, (c > 0 || k > 0) ? 1u : 0u);
        umma_tf32(tmem_base, dah + adv, dbl + adv, 1u);
        umma_tf32(tmem_base, dah + adv, dbh + adv, 1u);
      }
      asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(bar_addr) : "memory");
    }
  }
  if (alive) alive = mbar_wait(bar_addr, (uint32_t)((n_chunks - 1) & 1));
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");

  // ---- epilogue: thread tid owns output row row0 + tid (TMEM lane tid), 32 columns per tcgen05.ld
  const int64_t r = row0 + tid;
  const bool valid = alive && r < d.n_rows;
  const int64_t dr = (valid && cb.out_idx) ? (int64_t)cb.out_idx[r] : r;
#pragma unroll 1
  for (int cg = 0; cg < 4; ++cg) {
    uint32_t v[32];
    const uint32_t taddr = tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)(cg * 32);
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                   "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
                   "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
                   "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                 : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
    if (!valid) continue;
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      const int col = cg * 32 + q * 4;
      float o[4] = {__uint_as_float(v[4 * q]), __uint_as_float(v[4 * q + 1]), __uint_as_float(v[4 * q + 2]),
                    __uint_as_float(v[4 * q + 3])};
      if (cb.bias) {
        const float4 bb = ld4(cb.bias + col);
        o[0] += bb.x; o[1] += bb.y; o[2] += bb.z; o[3] += bb.w;
      }
      if (cb.gate) {
        const float4 z = ld4(cb.gate + r * cb.ld_gate + cb.col_gate + col);
        o[0] *= silu_grad_f(z.x); o[1] *= silu_grad_f(z.y); o[2] *= silu_grad_f(z.z); o[3] *= silu_grad_f(z.w);
      }
      if (cb.out_act) { o[0] = silu_f(o[0]); o[1] = silu_f(o[1]); o[2] = silu_f(o[2]); o[3] = silu_f(o[3]); }
      if (cb.res) {
        const float4 x = ld4(cb.res + r * cb.ld_res + cb.col_res + col);
        float4 w = make_float4(1.f, 1.f, 1.f, 1.f);
        if (cb.res_w) w = ld4(cb.res_w + col);
        o[0] = fmaf(w.x, x.x, o[0]); o[1] = fmaf(w.y, x.y, o[1]); o[2] = fmaf(w.z, x.z, o[2]); o[3] = fmaf(w.w, x.w, o[3]);
      }
      const float sc = cb.out_scale;
      const float4 ov = make_float4(o[0] * sc, o[1] * sc, o[2] * sc, o[3] * sc);
      float* dst = cb.out + dr * cb.ld_out + cb.col_out + col;
      if (cb.mode == MB_OUT_STORE) {
        *reinterpret_cast<float4*>(dst) = ov;
      } else if (cb.mode == MB_OUT_ADD) {
        float4 p = ld4(dst);
        p.x += ov.x; p.y += ov.y; p.z += ov.z; p.w += ov.w;
        *reinterpret_cast<float4*>(dst) = p;
      } else {
        atomicAdd(reinterpret_cast<float4*>(dst), ov);
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 128;" :: "r"(tmem_base) : "memory");
  }
}

static int g_gemm_mode = 0;  // 0: tcgen05 3xTF32, 1: fp32 SIMT

}  // namespace mb

extern "C" int mb_set_gemm_mode(int mode) {
  if (mode != 0 && mode != 1) return MB_ERR_INVALID;
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

extern "C" int mb_gemm(const mb_gemm_desc* desc, void* stream_) {
  int rc = gemm_validate(desc);
  if (rc) return rc;
  if (desc->n_rows == 0) return MB_OK;
  const long long gx = (desc->n_rows + 127) / 128;
  if (gx > 0x7fffffffLL) return MB_ERR_OVERFLOW;
  dim3 grid((unsigned)gx, (unsigned)desc->n_blocks);
  if (mb::g_gemm_mode == 1) {
    mb::k_gemm<<<grid, mb::GEMM_THREADS, 0, (cudaStream_t)stream_>>>(*desc);
  } else {
    static bool configured = false;  // per process; the attribute is per device function and context
    if (!configured) {
      MB_CUDA_CHECK(cudaFuncSetAttribute(mb::k_gemm_tc, cudaFuncAttributeMaxDynamicSharedMemorySize, mb::TC_SMEM_BYTES));
      configured = true;
    }
    mb::k_gemm_tc<<<grid, mb::TC_THREADS, mb::TC_SMEM_BYTES, (cudaStream_t)stream_>>>(*desc);
  }
  MB_LAUNCH_CHECK("k_gemm");
  return MB_OK;
}
