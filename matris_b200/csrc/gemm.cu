// Row GEMM with gathered, concatenated A operands and a fused epilogue (fp32 SIMT core).
//
// One CTA computes a 128-row x 128-column output tile.  A is never materialised:
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

using namespace mb;

extern "C" int mb_gemm(const mb_gemm_desc* desc, void* stream_) {
  if (!desc || desc->n_rows < 0 || desc->n_blocks < 1 || desc->n_blocks > 4) return MB_ERR_INVALID;
  if (desc->n_rows == 0) return MB_OK;
  for (int j = 0; j < desc->n_blocks; ++j) {
    const mb_colblock& cb = desc->blk[j];
    if (cb.n_src < 1 || cb.n_src > 4 || !cb.W || !cb.out) return MB_ERR_INVALID;
    if (!aligned16(cb.W) || (cb.ldw & 3) || cb.ldw < 128 * cb.n_src) return MB_ERR_INVALID;
    if (!aligned16(cb.out) || (cb.ld_out & 3) || (cb.col_out & 3)) return MB_ERR_INVALID;
    if (cb.mode < MB_OUT_STORE || cb.mode > MB_OUT_ATOMIC) return MB_ERR_INVALID;
    if (cb.bias && !aligned16(cb.bias)) return MB_ERR_INVALID;
    if (cb.gate && (!aligned16(cb.gate) || (cb.ld_gate & 3) || (cb.col_gate & 3))) return MB_ERR_INVALID;
    if (cb.res && (!aligned16(cb.res) || (cb.ld_res & 3) || (cb.col_res & 3))) return MB_ERR_INVALID;
    if (cb.res_w && !aligned16(cb.res_w)) return MB_ERR_INVALID;
    for (int s = 0; s < cb.n_src; ++s) {
      const mb_src& sr = cb.src[s];
      if (!sr.ptr || !aligned16(sr.ptr) || (sr.ld & 3) || (sr.col & 3)) return MB_ERR_INVALID;
    }
  }
  const long long gx = (desc->n_rows + BM - 1) / BM;
  if (gx > 0x7fffffffLL) return MB_ERR_OVERFLOW;
  dim3 grid((unsigned)gx, (unsigned)desc->n_blocks);
  k_gemm<<<grid, GEMM_THREADS, 0, (cudaStream_t)stream_>>>(*desc);
  MB_LAUNCH_CHECK("k_gemm");
  return MB_OK;
}
