// Row-wise and segment kernels of the interaction blocks (HBM-bound).
//
// Layout: every feature tensor is float32 row-major with 128 channels.  One warp
// owns one row (or one segment); lane l holds channels 4l..4l+3 as a float4, so a
// row is one coalesced 512-byte access and row reductions are warp shuffles.
// Segment reductions walk CSR ranges (rows are stored grouped by target node;
// the source-side grouping is a permutation), so there are no atomics and the
// summation order is fixed.
#include <float.h>
#include "common.cuh"

namespace mb {

constexpr int RW_THREADS = 256;
constexpr float RMS_EPS = FLT_EPSILON;  // nn.RMSNorm(eps=None) uses the dtype's machine epsilon

__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ void st4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ float dot4(float4 a, float4 b) { return a.x * b.x + a.y * b.y + a.z * b.z + a.w * b.w; }
__device__ __forceinline__ float4 mul4(float4 a, float4 b) { return make_float4(a.x * b.x, a.y * b.y, a.z * b.z, a.w * b.w); }
__device__ __forceinline__ float4 add4(float4 a, float4 b) { return make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w); }
__device__ __forceinline__ float4 sub4(float4 a, float4 b) { return make_float4(a.x - b.x, a.y - b.y, a.z - b.z, a.w - b.w); }
__device__ __forceinline__ float4 scl4(float4 a, float s) { return make_float4(a.x * s, a.y * s, a.z * s, a.w * s); }
__device__ __forceinline__ float4 fma4(float4 a, float4 b, float4 c) {
  return make_float4(fmaf(a.x, b.x, c.x), fmaf(a.y, b.y, c.y), fmaf(a.z, b.z, c.z), fmaf(a.w, b.w, c.w));
}
__device__ __forceinline__ float4 max4(float4 a, float4 b) {
  return make_float4(fmaxf(a.x, b.x), fmaxf(a.y, b.y), fmaxf(a.z, b.z), fmaxf(a.w, b.w));
}
__device__ __forceinline__ float4 exp4(float4 a) { return make_float4(expf(a.x), expf(a.y), expf(a.z), expf(a.w)); }
__device__ __forceinline__ float4 zero4() { return make_float4(0.f, 0.f, 0.f, 0.f); }

#define MB_ROW_PROLOGUE(n_rows)                                                       \
  const int lane = threadIdx.x & 31;                                                  \
  const int64_t row = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;          \
  if (row >= (n_rows)) return;                                                        \
  const int c = lane * 4;                                                             \
  (void)c;

static inline unsigned row_grid(int64_t n_rows) { return (unsigned)((n_rows * 32 + RW_THREADS - 1) / RW_THREADS); }

// ------------------------------------------------------------------ gated MLP tail
__global__ void k_gate_fwd(int64_t n_rows, const float* __restrict__ z, const float* __restrict__ wc,
                           const float* __restrict__ wg, float* __restrict__ h, const float* __restrict__ res,
                           const float* __restrict__ res_w, float* __restrict__ out2) {
  MB_ROW_PROLOGUE(n_rows)
  const float4 xc = ld4(z + row * 256 + c), xg = ld4(z + row * 256 + 128 + c);
  const float rc = rsqrtf(warp_sum(dot4(xc, xc)) * (1.f / 128.f) + RMS_EPS);
  const float rg = rsqrtf(warp_sum(dot4(xg, xg)) * (1.f / 128.f) + RMS_EPS);
  const float4 yc = mul4(scl4(xc, rc), ld4(wc + c)), yg = mul4(scl4(xg, rg), ld4(wg + c));
  const float4 o = make_float4(silu_f(yc.x) * sigmoid_f(yg.x), silu_f(yc.y) * sigmoid_f(yg.y),
                               silu_f(yc.z) * sigmoid_f(yg.z), silu_f(yc.w) * sigmoid_f(yg.w));
  if (h) st4(h + row * 128 + c, o);
  if (out2) {
    float4 w = make_float4(1.f, 1.f, 1.f, 1.f);
    if (res_w) w = ld4(res_w + c);
    st4(out2 + row * 128 + c, fma4(w, ld4(res + row * 128 + c), o));
  }
}

// Adjoint of  h = SiLU(RMSNorm(z_core) w_core) * sigmoid(RMSNorm(z_gate) w_gate)  for one row held by a warp (lane =
// four channels at c): g = dh of the row, result written to dz[row, 0:128 | 128:256].  Shared by k_gate_bwd and by the
// kernels that produce dh and can hand it over in registers.
__device__ __forceinline__ void gate_bwd_row(int64_t row, int c, const float* __restrict__ z,
                                             const float* __restrict__ wc, const float* __restrict__ wg, float4 g,
                                             float* __restrict__ dz) {
  const float4 xc = ld4(z + row * 256 + c), xg = ld4(z + row * 256 + 128 + c);
  const float rc = rsqrtf(warp_sum(dot4(xc, xc)) * (1.f / 128.f) + RMS_EPS);
  const float rg = rsqrtf(warp_sum(dot4(xg, xg)) * (1.f / 128.f) + RMS_EPS);
  const float4 gwc = ld4(wc + c), gwg = ld4(wg + c);
  const float4 nc = scl4(xc, rc), ng = scl4(xg, rg);
  const float4 yc = mul4(nc, gwc), yg = mul4(ng, gwg);
  float dnc[4], dng[4];
  const float ycv[4] = {yc.x, yc.y, yc.z, yc.w}, ygv[4] = {yg.x, yg.y, yg.z, yg.w};
  const float gv[4] = {g.x, g.y, g.z, g.w}, wcv[4] = {gwc.x, gwc.y, gwc.z, gwc.w}, wgv[4] = {gwg.x, gwg.y, gwg.z, gwg.w};
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float core = silu_f(ycv[k]), gate = sigmoid_f(ygv[k]);
    dnc[k] = gv[k] * gate * silu_grad_f(ycv[k]) * wcv[k];
    dng[k] = gv[k] * core * gate * (1.f - gate) * wgv[k];
  }
  const float4 dn_c = make_float4(dnc[0], dnc[1], dnc[2], dnc[3]), dn_g = make_float4(dng[0], dng[1], dng[2], dng[3]);
  const float mc = warp_sum(dot4(dn_c, nc)) * (1.f / 128.f), mg = warp_sum(dot4(dn_g, ng)) * (1.f / 128.f);
  st4(dz + row * 256 + c, scl4(sub4(dn_c, scl4(nc, mc)), rc));
  st4(dz + row * 256 + 128 + c, scl4(sub4(dn_g, scl4(ng, mg)), rg));
}

__global__ void k_gate_bwd(int64_t n_rows, const float* __restrict__ z, const float* __restrict__ wc,
                           const float* __restrict__ wg, const float* __restrict__ dh, float* __restrict__ dz) {
  MB_ROW_PROLOGUE(n_rows)
  gate_bwd_row(row, c, z, wc, wg, ld4(dh + row * 128 + c), dz);
}

// ------------------------------------------------------------------ attention aggregation
// warp per node; side 0: target segment (contiguous rows), side 1: source segment (through perm)
__global__ void k_seg_attn_fwd(int n_nodes, const int32_t* __restrict__ tgt_ptr, const int32_t* __restrict__ src_ptr,
                               const int32_t* __restrict__ src_perm, const int32_t* __restrict__ emap,
                               const float* __restrict__ logits, const float* __restrict__ h,
                               float* __restrict__ agg_t, float* __restrict__ agg_s, float* __restrict__ stats) {
  MB_ROW_PROLOGUE(n_nodes)
  constexpr int NB = 8;  // rows in flight per warp: their index and data loads are issued together
#pragma unroll
  for (int side = 0; side < 2; ++side) {
    const int32_t* ptr = side == 0 ? tgt_ptr : src_ptr;
    const int q0 = ptr[row], q1 = ptr[row + 1];
    const int lcol = side == 0 ? 128 : 0;
    auto rows_of = [&](int q, int64_t (&r)[NB], int64_t (&er)[NB]) {
#pragma unroll
      for (int i = 0; i < NB; ++i) {
        const int qq = q + i < q1 ? q + i : q1 - 1;
        r[i] = side == 0 ? qq : src_perm[qq];
      }
#pragma unroll
      for (int i = 0; i < NB; ++i) er[i] = emap ? emap[r[i]] : r[i];
    };
    float4 mx = make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
    float4 s = zero4(), acc = zero4();
    if (q1 - q0 <= NB) {  // the common case: the whole segment is held in registers, every row is read once
      if (q1 > q0) {
        int64_t r[NB], er[NB];
        rows_of(q0, r, er);
        float4 x[NB], hv[NB];
#pragma unroll
        for (int i = 0; i < NB; ++i) x[i] = ld4(logits + er[i] * 256 + lcol + c);
#pragma unroll
        for (int i = 0; i < NB; ++i) hv[i] = ld4(h + r[i] * 128 + c);
#pragma unroll
        for (int i = 0; i < NB; ++i) mx = max4(mx, x[i]);  // rows past the end repeat the last one
#pragma unroll
        for (int i = 0; i < NB; ++i) {
          if (q0 + i < q1) {
            const float4 e = exp4(sub4(x[i], mx));
            s = add4(s, e);
            acc = fma4(e, hv[i], acc);
          }
        }
      }
    } else {
      for (int q = q0; q < q1; q += NB) {
        int64_t r[NB], er[NB];
        rows_of(q, r, er);
        float4 x[NB];
#pragma unroll
        for (int i = 0; i < NB; ++i) x[i] = ld4(logits + er[i] * 256 + lcol + c);
#pragma unroll
        for (int i = 0; i < NB; ++i) mx = max4(mx, x[i]);
      }
      for (int q = q0; q < q1; q += NB) {
        int64_t r[NB], er[NB];
        rows_of(q, r, er);
        float4 x[NB], hv[NB];
#pragma unroll
        for (int i = 0; i < NB; ++i) x[i] = ld4(logits + er[i] * 256 + lcol + c);
#pragma unroll
        for (int i = 0; i < NB; ++i) hv[i] = ld4(h + r[i] * 128 + c);
#pragma unroll
        for (int i = 0; i < NB; ++i) {
          if (q + i < q1) {
            const float4 e = exp4(sub4(x[i], mx));
            s = add4(s, e);
            acc = fma4(e, hv[i], acc);
          }
        }
      }
    }
    float4 inv = zero4();
    if (q1 > q0) inv = make_float4(1.f / s.x, 1.f / s.y, 1.f / s.z, 1.f / s.w);
    else mx = zero4();
    st4((side == 0 ? agg_t : agg_s) + row * 128 + c, mul4(acc, inv));
    st4(stats + row * 512 + side * 256 + c, mx);
    st4(stats + row * 512 + side * 256 + 128 + c, inv);
  }
}

__global__ void k_seg_attn_bwd(int64_t n_rows, const int32_t* __restrict__ tgt, const int32_t* __restrict__ src,
                               int idx_stride, const int32_t* __restrict__ emap, const float* __restrict__ logits,
                               const float* __restrict__ h, const float* __restrict__ agg_t,
                               const float* __restrict__ agg_s, const float* __restrict__ stats,
                               const float* __restrict__ dagg_t, const float* __restrict__ dagg_s,
                               const float* __restrict__ dh_in, const int32_t* __restrict__ dh_map, float dh_scale,
                               float* __restrict__ dh, float* __restrict__ dlogits, const float* __restrict__ gate_z,
                               const float* __restrict__ gate_wc, const float* __restrict__ gate_wg,
                               float* __restrict__ gate_dz) {
  MB_ROW_PROLOGUE(n_rows)
  const int64_t nt = tgt[row * idx_stride], ns = src[row * idx_stride];
  const int64_t er = emap ? emap[row] : row;
  const float4 xs = ld4(logits + er * 256 + c), xt = ld4(logits + er * 256 + 128 + c);
  const float4 at = mul4(exp4(sub4(xt, ld4(stats + nt * 512 + c))), ld4(stats + nt * 512 + 128 + c));
  const float4 as = mul4(exp4(sub4(xs, ld4(stats + ns * 512 + 256 + c))), ld4(stats + ns * 512 + 384 + c));
  const float4 hv = ld4(h + row * 128 + c);
  const float4 gt = mul4(at, ld4(dagg_t + nt * 128 + c)), gs = mul4(as, ld4(dagg_s + ns * 128 + c));
  float4 o = add4(gt, gs);
  if (dh_in) {
    const int64_t mr = dh_map ? dh_map[row] : row;
    o = add4(o, scl4(ld4(dh_in + mr * 128 + c), dh_scale));
  }
  if (gate_dz) gate_bwd_row(row, c, gate_z, gate_wc, gate_wg, o, gate_dz);  // dh goes on in registers
  else st4(dh + row * 128 + c, o);
  st4(dlogits + row * 256 + c, mul4(gs, sub4(hv, ld4(agg_s + ns * 128 + c))));
  st4(dlogits + row * 256 + 128 + c, mul4(gt, sub4(hv, ld4(agg_t + nt * 128 + c))));
}

// ------------------------------------------------------------------ refinement aggregation
__global__ void k_seg_smooth_sum_fwd(int n_nodes, const int32_t* __restrict__ tgt_ptr,
                                     const int32_t* __restrict__ emap, const int32_t* __restrict__ src,
                                     int idx_stride, const float* __restrict__ env, const float* __restrict__ h,
                                     float* __restrict__ agg) {
  MB_ROW_PROLOGUE(n_nodes)
  const int q0 = tgt_ptr[row], q1 = tgt_ptr[row + 1];
  float4 acc = zero4();
  float4 env_n = zero4();
  if (src && q1 > q0) env_n = ld4(env + row * 128 + c);
  for (int64_t r = q0; r < q1; ++r) {
    float4 s;
    if (src) s = mul4(ld4(env + (int64_t)src[r * idx_stride] * 128 + c), env_n);
    else s = ld4(env + (int64_t)emap[r] * 128 + c);
    acc = add4(acc, mul4(ld4(h + r * 128 + c), s));
  }
  st4(agg + row * 128 + c, acc);
}

__global__ void k_seg_smooth_sum_bwd_rows(int64_t n_rows, const int32_t* __restrict__ tgt,
                                          const int32_t* __restrict__ src, int idx_stride,
                                          const int32_t* __restrict__ emap, const float* __restrict__ env,
                                          const float* __restrict__ dagg, float* __restrict__ dh, int accumulate,
                                          const float* __restrict__ gate_z, const float* __restrict__ gate_wc,
                                          const float* __restrict__ gate_wg, float* __restrict__ gate_dz) {
  MB_ROW_PROLOGUE(n_rows)
  const int64_t nt = tgt[row * idx_stride];
  float4 s;
  if (src) s = mul4(ld4(env + (int64_t)src[row * idx_stride] * 128 + c), ld4(env + nt * 128 + c));
  else s = ld4(env + (int64_t)emap[row] * 128 + c);
  float4 o = mul4(ld4(dagg + nt * 128 + c), s);
  if (accumulate) o = add4(o, ld4(dh + row * 128 + c));
  if (gate_dz) gate_bwd_row(row, c, gate_z, gate_wc, gate_wg, o, gate_dz);  // dh goes on in registers
  else st4(dh + row * 128 + c, o);
}

__global__ void k_smooth_env_bwd_atom(int n_bonds, const int32_t* __restrict__ u2d, const int32_t* __restrict__ rev,
                                      const int32_t* __restrict__ tgt, const float* __restrict__ h,
                                      const float* __restrict__ dagg, const float* __restrict__ drow,
                                      float* __restrict__ denv) {
  MB_ROW_PROLOGUE(n_bonds)
  const int64_t e1 = u2d[row], e2 = rev[e1];
  float4 g1 = ld4(dagg + (int64_t)tgt[e1] * 128 + c), g2 = ld4(dagg + (int64_t)tgt[e2] * 128 + c);
  if (drow) {  // gradient that reached the smoothed rows directly (edge FFN fed with h * s)
    g1 = add4(g1, ld4(drow + e1 * 128 + c));
    g2 = add4(g2, ld4(drow + e2 * 128 + c));
  }
  st4(denv + row * 128 + c, add4(mul4(g1, ld4(h + e1 * 128 + c)), mul4(g2, ld4(h + e2 * 128 + c))));
}

// y[r] = x[r] * s[idx[r]]  (rows scaled channel-wise by a gathered row)
__global__ void k_mul_rows_gather(int64_t n_rows, const float* __restrict__ x, const float* __restrict__ s,
                                  const int32_t* __restrict__ idx, float* __restrict__ y) {
  MB_ROW_PROLOGUE(n_rows)
  const int64_t sr = idx ? idx[row] : row;
  st4(y + row * 128 + c, mul4(ld4(x + row * 128 + c), ld4(s + sr * 128 + c)));
}

__global__ void k_smooth_env_bwd_line(int n_nodes, const int32_t* __restrict__ tgt_ptr,
                                      const int32_t* __restrict__ src_ptr, const int32_t* __restrict__ src_perm,
                                      const int32_t* __restrict__ tgt, const int32_t* __restrict__ src,
                                      int idx_stride, const float* __restrict__ env, const float* __restrict__ h,
                                      const float* __restrict__ dagg, float* __restrict__ denv) {
  MB_ROW_PROLOGUE(n_nodes)
  float4 acc = zero4();
  const int q0 = tgt_ptr[row], q1 = tgt_ptr[row + 1];
  if (q1 > q0) {
    float4 inner = zero4();
    for (int64_t r = q0; r < q1; ++r)
      inner = fma4(ld4(h + r * 128 + c), ld4(env + (int64_t)src[r * idx_stride] * 128 + c), inner);
    acc = mul4(ld4(dagg + row * 128 + c), inner);
  }
  for (int q = src_ptr[row]; q < src_ptr[row + 1]; ++q) {
    const int64_t r = src_perm[q];
    const int64_t nt = tgt[r * idx_stride];
    acc = add4(acc, mul4(mul4(ld4(dagg + nt * 128 + c), ld4(h + r * 128 + c)), ld4(env + nt * 128 + c)));
  }
  st4(denv + row * 128 + c, acc);
}

// ------------------------------------------------------------------ pair mean / scaling
__global__ void k_pair_mean_res(int n_bonds, const int32_t* __restrict__ u2d, const int32_t* __restrict__ rev,
                                const float* __restrict__ y, const float* __restrict__ res,
                                const float* __restrict__ res_w, float* __restrict__ out) {
  MB_ROW_PROLOGUE(n_bonds)
  const int64_t e1 = u2d[row], e2 = rev[e1];
  float4 o = scl4(add4(ld4(y + e1 * 128 + c), ld4(y + e2 * 128 + c)), 0.5f);
  if (res) {
    float4 w = make_float4(1.f, 1.f, 1.f, 1.f);
    if (res_w) w = ld4(res_w + c);
    o = fma4(w, ld4(res + row * 128 + c), o);
  }
  st4(out + row * 128 + c, o);
}

__global__ void k_scale_rows(int64_t n_rows, const float* __restrict__ x, const float* __restrict__ a,
                             float* __restrict__ y, int accumulate) {
  MB_ROW_PROLOGUE(n_rows)
  float4 o = mul4(ld4(a + c), ld4(x + row * 128 + c));
  if (accumulate) o = add4(o, ld4(y + row * 128 + c));
  st4(y + row * 128 + c, o);
}

// ------------------------------------------------------------------ K <= 16 linear layers
__global__ void k_small_linear_fwd(int64_t n_rows, int k, const float* __restrict__ x, const float* __restrict__ w,
                                   float* __restrict__ y) {
  __shared__ float ws[16][128];
  for (int i = threadIdx.x; i < 128 * k; i += blockDim.x) ws[i % k][i / k] = w[i];
  __syncthreads();
  MB_ROW_PROLOGUE(n_rows)
  float4 acc = zero4();
  for (int j = 0; j < k; ++j) {
    const float xv = x[row * k + j];
    acc = fma4(make_float4(xv, xv, xv, xv), ld4(&ws[j][c]), acc);
  }
  st4(y + row * 128 + c, acc);
}

__global__ void k_small_linear_bwd(int64_t n_rows, int k, const float* __restrict__ dy, const float* __restrict__ w,
                                   float* __restrict__ dx, int accumulate) {
  __shared__ float ws[16][128];
  for (int i = threadIdx.x; i < 128 * k; i += blockDim.x) ws[i % k][i / k] = w[i];
  __syncthreads();
  MB_ROW_PROLOGUE(n_rows)
  const float4 g = ld4(dy + row * 128 + c);
  float mine = 0.f;
  for (int j = 0; j < k; ++j) {
    const float s = warp_sum(dot4(g, ld4(&ws[j][c])));
    if (lane == j) mine = s;
  }
  if (lane < k) {
    if (accumulate) mine += dx[row * k + lane];
    dx[row * k + lane] = mine;
  }
}

// ------------------------------------------------------------------ norms
__global__ void k_layernorm_fwd(int64_t n_rows, const float* __restrict__ x, const float* __restrict__ w,
                                const float* __restrict__ b, float* __restrict__ y) {
  MB_ROW_PROLOGUE(n_rows)
  const float4 v = ld4(x + row * 128 + c);
  const float mean = warp_sum(v.x + v.y + v.z + v.w) * (1.f / 128.f);
  const float4 dv = make_float4(v.x - mean, v.y - mean, v.z - mean, v.w - mean);
  const float rstd = rsqrtf(warp_sum(dot4(dv, dv)) * (1.f / 128.f) + 1e-5f);
  st4(y + row * 128 + c, fma4(scl4(dv, rstd), ld4(w + c), ld4(b + c)));
}

__global__ void k_layernorm_bwd(int64_t n_rows, const float* __restrict__ x, const float* __restrict__ w,
                                const float* __restrict__ dy, float* __restrict__ dx) {
  MB_ROW_PROLOGUE(n_rows)
  const float4 v = ld4(x + row * 128 + c);
  const float mean = warp_sum(v.x + v.y + v.z + v.w) * (1.f / 128.f);
  const float4 dv = make_float4(v.x - mean, v.y - mean, v.z - mean, v.w - mean);
  const float rstd = rsqrtf(warp_sum(dot4(dv, dv)) * (1.f / 128.f) + 1e-5f);
  const float4 xh = scl4(dv, rstd);
  const float4 g = mul4(ld4(dy + row * 128 + c), ld4(w + c));
  const float m1 = warp_sum(g.x + g.y + g.z + g.w) * (1.f / 128.f);
  const float m2 = warp_sum(dot4(g, xh)) * (1.f / 128.f);
  st4(dx + row * 128 + c, make_float4(rstd * (g.x - m1 - xh.x * m2), rstd * (g.y - m1 - xh.y * m2),
                                      rstd * (g.z - m1 - xh.z * m2), rstd * (g.w - m1 - xh.w * m2)));
}

__global__ void k_rmsnorm_fwd(int64_t n_rows, const float* __restrict__ x, const float* __restrict__ w,
                              float* __restrict__ y) {
  MB_ROW_PROLOGUE(n_rows)
  const float4 v = ld4(x + row * 128 + c);
  const float r = rsqrtf(warp_sum(dot4(v, v)) * (1.f / 128.f) + RMS_EPS);
  st4(y + row * 128 + c, mul4(scl4(v, r), ld4(w + c)));
}

__global__ void k_rmsnorm_bwd(int64_t n_rows, const float* __restrict__ x, const float* __restrict__ w,
                              const float* __restrict__ dy, float* __restrict__ dx) {
  MB_ROW_PROLOGUE(n_rows)
  const float4 v = ld4(x + row * 128 + c);
  const float r = rsqrtf(warp_sum(dot4(v, v)) * (1.f / 128.f) + RMS_EPS);
  const float4 n = scl4(v, r);
  const float4 g = mul4(ld4(dy + row * 128 + c), ld4(w + c));
  const float m = warp_sum(dot4(g, n)) * (1.f / 128.f);
  st4(dx + row * 128 + c, scl4(sub4(g, scl4(n, m)), r));
}

__global__ void k_embedding(int64_t n_rows, const int32_t* __restrict__ idx, int offset,
                            const float* __restrict__ table, float* __restrict__ y) {
  MB_ROW_PROLOGUE(n_rows)
  st4(y + row * 128 + c, ld4(table + (int64_t)(idx[row] + offset) * 128 + c));
}

// ------------------------------------------------------------------ head projections
__global__ void k_head_dot_fwd(int64_t n_rows, int k, const float* __restrict__ z, const float* __restrict__ w,
                               const float* __restrict__ b, int take_abs, float* __restrict__ out) {
  MB_ROW_PROLOGUE(n_rows)
  float s = 0.f;
  for (int j = c; j < k; j += 128) {
    const float4 v = ld4(z + row * k + j), ww = ld4(w + j);
    s += silu_f(v.x) * ww.x + silu_f(v.y) * ww.y + silu_f(v.z) * ww.z + silu_f(v.w) * ww.w;
  }
  s = warp_sum(s) + b[0];
  if (lane == 0) out[row] = take_abs ? fabsf(s) : s;
}

__global__ void k_head_dot_bwd(int64_t n_rows, int k, const float* __restrict__ z, const float* __restrict__ w,
                               const float* __restrict__ seed, const int32_t* __restrict__ seed_map,
                               float* __restrict__ dz) {
  MB_ROW_PROLOGUE(n_rows)
  const float g = seed ? seed[seed_map ? seed_map[row] : row] : 1.f;
  for (int j = c; j < k; j += 128) {
    const float4 v = ld4(z + row * k + j), ww = ld4(w + j);
    st4(dz + row * k + j, make_float4(g * ww.x * silu_grad_f(v.x), g * ww.y * silu_grad_f(v.y),
                                      g * ww.z * silu_grad_f(v.z), g * ww.w * silu_grad_f(v.w)));
  }
}

__global__ void k_silu_bwd(int64_t n_rows, const float* __restrict__ dy, const float* __restrict__ z,
                           float* __restrict__ dz) {
  MB_ROW_PROLOGUE(n_rows)
  const float4 g = ld4(dy + row * 128 + c), v = ld4(z + row * 128 + c);
  st4(dz + row * 128 + c, make_float4(g.x * silu_grad_f(v.x), g.y * silu_grad_f(v.y), g.z * silu_grad_f(v.z),
                                      g.w * silu_grad_f(v.w)));
}

__global__ void k_segment_sum_scalar(int n_seg, const int32_t* __restrict__ seg_ptr, const float* __restrict__ x,
                                     float* __restrict__ out) {
  MB_ROW_PROLOGUE(n_seg)
  float s = 0.f;
  for (int i = seg_ptr[row] + lane; i < seg_ptr[row + 1]; i += 32) s += x[i];
  s = warp_sum(s);
  if (lane == 0) out[row] = s;
}

}  // namespace mb

using namespace mb;
#define STREAM ((cudaStream_t)stream)
#define MB_REQUIRE(cond) do { if (!(cond)) return MB_ERR_INVALID; } while (0)

extern "C" int mb_gate_fwd(int64_t n_rows, const float* z, const float* w_core, const float* w_gate, float* h,
                           const float* res, const float* res_w, float* out2, void* stream) {
  MB_REQUIRE(n_rows >= 0 && z && w_core && w_gate && (h || out2) && (!out2 || res));
  if (n_rows == 0) return MB_OK;
  k_gate_fwd<<<row_grid(n_rows), RW_THREADS, 0, STREAM>>>(n_rows, z, w_core, w_gate, h, res, res_w, out2);
  MB_LAUNCH_CHECK("k_gate_fwd");
  return MB_OK;
}

extern "C" int mb_gate_bwd(int64_t n_rows, const float* z, const float* w_core, const float* w_gate, const float* dh,
                           float* dz, void* stream) {
  MB_REQUIRE(n_rows >= 0 && z && w_core && w_gate && dh && dz);
  if (n_rows == 0) return MB_OK;
  k_gate_bwd<<<row_grid(n_rows), RW_THREADS, 0, STREAM>>>(n_rows, z, w_core, w_gate, dh, dz);
  MB_LAUNCH_CHECK("k_gate_bwd");
  return MB_OK;
}

extern "C" int mb_seg_attn_fwd(int32_t n_nodes, const int32_t* tgt_ptr, const int32_t* src_ptr,
                               const int32_t* src_perm, const int32_t* emap, const float* logits, const float* h,
                               float* agg_t, float* agg_s, float* stats, void* stream) {
  MB_REQUIRE(n_nodes >= 0 && tgt_ptr && src_ptr && src_perm && logits && h && agg_t && agg_s && stats);
  if (n_nodes == 0) return MB_OK;
  k_seg_attn_fwd<<<row_grid(n_nodes), RW_THREADS, 0, STREAM>>>(n_nodes, tgt_ptr, src_ptr, src_perm, emap, logits, h,
                                                              agg_t, agg_s, stats);
  MB_LAUNCH_CHECK("k_seg_attn_fwd");
  return MB_OK;
}

extern "C" int mb_seg_attn_bwd(int64_t n_rows, const int32_t* tgt, const int32_t* src, int32_t idx_stride,
                               const int32_t* emap, const float* logits, const float* h, const float* agg_t,
                               const float* agg_s, const float* stats, const float* dagg_t, const float* dagg_s,
                               const float* dh_in, const int32_t* dh_map, float dh_scale, float* dh, float* dlogits,
                               const float* gate_z, const float* gate_wc, const float* gate_wg, float* gate_dz,
                               void* stream) {
  MB_REQUIRE(n_rows >= 0 && tgt && src && idx_stride > 0 && logits && h && agg_t && agg_s && stats && dagg_t &&
             dagg_s && dlogits && (gate_dz ? (gate_z && gate_wc && gate_wg) : dh != nullptr));
  if (n_rows == 0) return MB_OK;
  k_seg_attn_bwd<<<row_grid(n_rows), RW_THREADS, 0, STREAM>>>(n_rows, tgt, src, idx_stride, emap, logits, h, agg_t,
                                                             agg_s, stats, dagg_t, dagg_s, dh_in, dh_map, dh_scale,
                                                             dh, dlogits, gate_z, gate_wc, gate_wg, gate_dz);
  MB_LAUNCH_CHECK("k_seg_attn_bwd");
  return MB_OK;
}

extern "C" int mb_seg_smooth_sum_fwd(int32_t n_nodes, const int32_t* tgt_ptr, const int32_t* emap,
                                     const int32_t* src, int32_t idx_stride, const float* env, const float* h,
                                     float* agg, void* stream) {
  MB_REQUIRE(n_nodes >= 0 && tgt_ptr && (emap || src) && env && h && agg && idx_stride > 0);
  if (n_nodes == 0) return MB_OK;
  k_seg_smooth_sum_fwd<<<row_grid(n_nodes), RW_THREADS, 0, STREAM>>>(n_nodes, tgt_ptr, emap, src, idx_stride, env, h,
                                                                    agg);
  MB_LAUNCH_CHECK("k_seg_smooth_sum_fwd");
  return MB_OK;
}

extern "C" int mb_seg_smooth_sum_bwd_rows(int64_t n_rows, const int32_t* tgt, const int32_t* src, int32_t idx_stride,
                                          const int32_t* emap, const float* env, const float* dagg, float* dh,
                                          int32_t accumulate, const float* gate_z, const float* gate_wc,
                                          const float* gate_wg, float* gate_dz, void* stream) {
  MB_REQUIRE(n_rows >= 0 && tgt && (emap || src) && env && dagg && idx_stride > 0 && (dh || (gate_dz && !accumulate)) &&
             (!gate_dz || (gate_z && gate_wc && gate_wg)));
  if (n_rows == 0) return MB_OK;
  k_seg_smooth_sum_bwd_rows<<<row_grid(n_rows), RW_THREADS, 0, STREAM>>>(n_rows, tgt, src, idx_stride, emap, env,
                                                                        dagg, dh, accumulate, gate_z, gate_wc, gate_wg,
                                                                        gate_dz);
  MB_LAUNCH_CHECK("k_seg_smooth_sum_bwd_rows");
  return MB_OK;
}

extern "C" int mb_seg_smooth_sum_bwd_env(int32_t n_nodes, const int32_t* tgt_ptr, const int32_t* src_ptr,
                                         const int32_t* src_perm, const int32_t* tgt, const int32_t* src,
                                         int32_t idx_stride, const int32_t* u2d, const int32_t* rev, const float* env,
                                         const float* h, const float* dagg, const float* drow, float* denv,
                                         void* stream) {
  MB_REQUIRE(n_nodes >= 0 && tgt && h && dagg && denv && idx_stride > 0);
  if (n_nodes == 0) return MB_OK;
  if (!src_ptr) {
    MB_REQUIRE(u2d && rev && idx_stride == 1);
    k_smooth_env_bwd_atom<<<row_grid(n_nodes), RW_THREADS, 0, STREAM>>>(n_nodes, u2d, rev, tgt, h, dagg, drow, denv);
  } else {
    MB_REQUIRE(tgt_ptr && src_perm && src && env && !drow);
    k_smooth_env_bwd_line<<<row_grid(n_nodes), RW_THREADS, 0, STREAM>>>(n_nodes, tgt_ptr, src_ptr, src_perm, tgt, src,
                                                                       idx_stride, env, h, dagg, denv);
  }
  MB_LAUNCH_CHECK("k_smooth_env_bwd");
  return MB_OK;
}

extern "C" int mb_mul_rows_gather(int64_t n_rows, const float* x, const float* s, const int32_t* idx, float* y,
                                  void* stream) {
  MB_REQUIRE(n_rows >= 0 && x && s && y);
  if (n_rows == 0) return MB_OK;
  k_mul_rows_gather<<<row_grid(n_rows), RW_THREADS, 0, STREAM>>>(n_rows, x, s, idx, y);
  MB_LAUNCH_CHECK("k_mul_rows_gather");
  return MB_OK;
}

extern "C" int mb_pair_mean_res(int32_t n_bonds, const int32_t* u2d, const int32_t* rev, const float* y,
                                const float* res, const float* res_w, float* out, void* stream) {
  MB_REQUIRE(n_bonds >= 0 && u2d && rev && y && out);
  if (n_bonds == 0) return MB_OK;
  k_pair_mean_res<<<row_grid(n_bonds), RW_THREADS, 0, STREAM>>>(n_bonds, u2d, rev, y, res, res_w, out);
  MB_LAUNCH_CHECK("k_pair_mean_res");
  return MB_OK;
}

extern "C" int mb_scale_rows(int64_t n_rows, const float* x, const float* a, float* y, int32_t accumulate,
                             void* stream) {
  MB_REQUIRE(n_rows >= 0 && x && a && y);
  if (n_rows == 0) return MB_OK;
  k_scale_rows<<<row_grid(n_rows), RW_THREADS, 0, STREAM>>>(n_rows, x, a, y, accumulate);
  MB_LAUNCH_CHECK("k_scale_rows");
  return MB_OK;
}

extern "C" int mb_small_linear_fwd(int64_t n_rows, int32_t k, const float* x, const float* w, float* y, void* stream) {
  MB_REQUIRE(n_rows >= 0 && k >= 1 && k <= 16 && x && w && y);
  if (n_rows == 0) return MB_OK;
  k_small_linear_fwd<<<row_grid(n_rows), RW_THREADS, 0, STREAM>>>(n_rows, k, x, w, y);
  MB_LAUNCH_CHECK("k_small_linear_fwd");
  return MB_OK;
}

extern "C" int mb_small_linear_bwd(int64_t n_rows, int32_t k, const float* dy, const float* w, float* dx,
                                   int32_t accumulate, void* stream) {
  MB_REQUIRE(n_rows >= 0 && k >= 1 && k <= 16 && dy && w && dx);
  if (n_rows == 0) return MB_OK;
  k_small_linear_bwd<<<row_grid(n_rows), RW_THREADS, 0, STREAM>>>(n_rows, k, dy, w, dx, accumulate);
  MB_LAUNCH_CHECK("k_small_linear_bwd");
  return MB_OK;
}

extern "C" int mb_layernorm_fwd(int64_t n_rows, const float* x, const float* w, const float* b, float* y,
                                void* stream) {
  MB_REQUIRE(n_rows >= 0 && x && w && b && y);
  if (n_rows == 0) return MB_OK;
  k_layernorm_fwd<<<row_grid(n_rows), RW_THREADS, 0, STREAM>>>(n_rows, x, w, b, y);
  MB_LAUNCH_CHECK("k_layernorm_fwd");
  return MB_OK;
}

extern "C" int mb_layernorm_bwd(int64_t n_rows, const float* x, const float* w, const float* dy, float* dx,
                                void* stream) {
  MB_REQUIRE(n_rows >= 0 && x && w && dy && dx);
  if (n_rows == 0) return MB_OK;
  k_layernorm_bwd<<<row_grid(n_rows), RW_THREADS, 0, STREAM>>>(n_rows, x, w, dy, dx);
  MB_LAUNCH_CHECK("k_layernorm_bwd");
  return MB_OK;
}

extern "C" int mb_rmsnorm_fwd(int64_t n_rows, const float* x, const float* w, float* y, void* stream) {
  MB_REQUIRE(n_rows >= 0 && x && w && y);
  if (n_rows == 0) return MB_OK;
  k_rmsnorm_fwd<<<row_grid(n_rows), RW_THREADS, 0, STREAM>>>(n_rows, x, w, y);
  MB_LAUNCH_CHECK("k_rmsnorm_fwd");
  return MB_OK;
}

extern "C" int mb_rmsnorm_bwd(int64_t n_rows, const float* x, const float* w, const float* dy, float* dx,
                              void* stream) {
  MB_REQUIRE(n_rows >= 0 && x && w && dy && dx);
  if (n_rows == 0) return MB_OK;
  k_rmsnorm_bwd<<<row_grid(n_rows), RW_THREADS, 0, STREAM>>>(n_rows, x, w, dy, dx);
  MB_LAUNCH_CHECK("k_rmsnorm_bwd");
  return MB_OK;
}

extern "C" int mb_embedding(int64_t n_rows, const int32_t* idx, int32_t offset, const float* table, float* y,
                            void* stream) {
  MB_REQUIRE(n_rows >= 0 && idx && table && y);
  if (n_rows == 0) return MB_OK;
  k_embedding<<<row_grid(n_rows), RW_THREADS, 0, STREAM>>>(n_rows, idx, offset, table, y);
  MB_LAUNCH_CHECK("k_embedding");
  return MB_OK;
}

extern "C" int mb_head_dot_fwd(int64_t n_rows, int32_t k, const float* z, const float* w, const float* b,
                               int32_t take_abs, float* out, void* stream) {
  MB_REQUIRE(n_rows >= 0 && k > 0 && (k % 128) == 0 && z && w && b && out);
  if (n_rows == 0) return MB_OK;
  k_head_dot_fwd<<<row_grid(n_rows), RW_THREADS, 0, STREAM>>>(n_rows, k, z, w, b, take_abs, out);
  MB_LAUNCH_CHECK("k_head_dot_fwd");
  return MB_OK;
}

extern "C" int mb_head_dot_bwd(int64_t n_rows, int32_t k, const float* z, const float* w, const float* seed,
                               const int32_t* seed_map, float* dz, void* stream) {
  MB_REQUIRE(n_rows >= 0 && k > 0 && (k % 128) == 0 && z && w && dz);
  if (n_rows == 0) return MB_OK;
  k_head_dot_bwd<<<row_grid(n_rows), RW_THREADS, 0, STREAM>>>(n_rows, k, z, w, seed, seed_map, dz);
  MB_LAUNCH_CHECK("k_head_dot_bwd");
  return MB_OK;
}

extern "C" int mb_silu_bwd(int64_t n_rows, const float* dy, const float* z, float* dz, void* stream) {
  MB_REQUIRE(n_rows >= 0 && dy && z && dz);
  if (n_rows == 0) return MB_OK;
  k_silu_bwd<<<row_grid(n_rows), RW_THREADS, 0, STREAM>>>(n_rows, dy, z, dz);
  MB_LAUNCH_CHECK("k_silu_bwd");
  return MB_OK;
}

extern "C" int mb_segment_sum_scalar(int32_t n_seg, const int32_t* seg_ptr, const float* x, float* out,
                                     void* stream) {
  MB_REQUIRE(n_seg >= 0 && seg_ptr && x && out);
  if (n_seg == 0) return MB_OK;
  k_segment_sum_scalar<<<row_grid(n_seg), RW_THREADS, 0, STREAM>>>(n_seg, seg_ptr, x, out);
  MB_LAUNCH_CHECK("k_segment_sum_scalar");
  return MB_OK;
}
