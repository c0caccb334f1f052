// Edge geometry, radial (Bessel x envelope) and angular (spherical Bessel x real
// m=0 harmonics) bases, forward and backward, plus the force / virial reduction.
// Element-wise and HBM-bound; float32 throughout, evaluated in the same operation
// order as the PyTorch expressions they replace so that rounding stays comparable.
#include "common.cuh"

namespace mb {

constexpr int GEO_THREADS = 256;
static inline unsigned grid1(int64_t n) { return (unsigned)((n + GEO_THREADS - 1) / GEO_THREADS); }

// ------------------------------------------------------------------ edge vectors
__global__ void k_edge_geometry_fwd(int64_t n_edges, const float* __restrict__ cart, const float* __restrict__ lattice,
                                    const int32_t* __restrict__ atom_struct, const int32_t* __restrict__ center,
                                    const int32_t* __restrict__ neighbor, const int32_t* __restrict__ image,
                                    float* __restrict__ vec, float* __restrict__ len, float* __restrict__ unit) {
  const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= n_edges) return;
  const int i = center[e], j = neighbor[e];
  const float* L = lattice + 9 * (int64_t)atom_struct[i];
  const float n0 = (float)image[3 * e], n1 = (float)image[3 * e + 1], n2 = (float)image[3 * e + 2];
  float v[3];
#pragma unroll
  for (int k = 0; k < 3; ++k) {
    const float shift = n0 * L[k] + n1 * L[3 + k] + n2 * L[6 + k];
    v[k] = cart[3 * (int64_t)i + k] - (cart[3 * (int64_t)j + k] + shift);
  }
  const float d = sqrtf(v[0] * v[0] + v[1] * v[1] + v[2] * v[2]);
  len[e] = d;
#pragma unroll
  for (int k = 0; k < 3; ++k) {
    vec[3 * e + k] = v[k];
    unit[3 * e + k] = v[k] / d;
  }
}

// g_e = dE/dv_e from dE/dlen and dE/dunit:  d len/dv = u ; d unit/dv = (I - u u^T)/len
__global__ void k_edge_grad(int64_t n_edges, const float* __restrict__ len, const float* __restrict__ unit,
                            const float* __restrict__ dlen, const float* __restrict__ dunit, float* __restrict__ g) {
  const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= n_edges) return;
  const float ux = unit[3 * e], uy = unit[3 * e + 1], uz = unit[3 * e + 2];
  const float dx = dunit[3 * e], dy = dunit[3 * e + 1], dz = dunit[3 * e + 2];
  const float dl = dlen[e], inv = 1.0f / len[e];
  const float p = dx * ux + dy * uy + dz * uz;
  g[3 * e] = dl * ux + (dx - p * ux) * inv;
  g[3 * e + 1] = dl * uy + (dy - p * uy) * inv;
  g[3 * e + 2] = dl * uz + (dz - p * uz) * inv;
}

// warp per atom: dE/dr_i = sum_{e: centre i} (g_e - g_rev(e)); virial partial sum_e v_e (x) g_e
__global__ void k_atom_grad(int n_atoms, const int32_t* __restrict__ edge_ptr, const int32_t* __restrict__ rev,
                            const float* __restrict__ vec, const float* __restrict__ g, float* __restrict__ dcart,
                            float* __restrict__ virial_atom) {
  const int lane = threadIdx.x & 31;
  const int i = (int)(((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5);
  if (i >= n_atoms) return;
  float f[3] = {0.f, 0.f, 0.f}, w[9] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  for (int e = edge_ptr[i] + lane; e < edge_ptr[i + 1]; e += 32) {
    const int r = rev[e];
    float ge[3], ve[3];
#pragma unroll
    for (int k = 0; k < 3; ++k) {
      ge[k] = g[3 * (int64_t)e + k];
      ve[k] = vec[3 * (int64_t)e + k];
      f[k] += ge[k] - g[3 * (int64_t)r + k];
    }
#pragma unroll
    for (int a = 0; a < 3; ++a)
#pragma unroll
      for (int b = 0; b < 3; ++b) w[3 * a + b] += ve[a] * ge[b];
  }
#pragma unroll
  for (int k = 0; k < 3; ++k) f[k] = warp_sum(f[k]);
#pragma unroll
  for (int k = 0; k < 9; ++k) w[k] = warp_sum(w[k]);
  if (lane == 0) {
#pragma unroll
    for (int k = 0; k < 3; ++k) dcart[3 * (int64_t)i + k] = f[k];
#pragma unroll
    for (int k = 0; k < 9; ++k) virial_atom[9 * (int64_t)i + k] = w[k];
  }
}

// warp per structure: dE/dstrain = 0.5 (G + G^T), G = sum over the structure's atoms of the partials
__global__ void k_struct_virial(int n_struct, const int32_t* __restrict__ atom_ptr,
                                const float* __restrict__ virial_atom, float* __restrict__ dstrain) {
  const int lane = threadIdx.x & 31;
  const int b = (int)(((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5);
  if (b >= n_struct) return;
  float w[9] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  for (int i = atom_ptr[b] + lane; i < atom_ptr[b + 1]; i += 32)
#pragma unroll
    for (int k = 0; k < 9; ++k) w[k] += virial_atom[9 * (int64_t)i + k];
#pragma unroll
  for (int k = 0; k < 9; ++k) w[k] = warp_sum(w[k]);
  if (lane == 0)
#pragma unroll
    for (int a = 0; a < 3; ++a)
#pragma unroll
      for (int c = 0; c < 3; ++c) dstrain[9 * (int64_t)b + 3 * a + c] = 0.5f * (w[3 * a + c] + w[3 * c + a]);
}

// ------------------------------------------------------------------ Bessel * envelope
__device__ __forceinline__ float ipow(float x, int p) {
  float r = 1.f;
  for (int k = 0; k < p; ++k) r *= x;
  return r;
}

// value and d/dd of one basis set; outputs 7 values each
__device__ __forceinline__ void bessel_eval(float d, float cut, const float* __restrict__ freq, int p, float* val,
                                            float* der) {
  const float inv_cut = 1.0f / cut;
  const float norm = sqrtf(2.0f * inv_cut);
  const float ds = d * inv_cut;  // argument scaling of the sine
  const float x = d / cut;       // argument of the envelope
  const float fp = (float)p;
  const float a = -(fp + 1.f) * (fp + 2.f) / 2.f, b = fp * (fp + 2.f), c = -fp * (fp + 1.f) / 2.f;
  float env = 0.f, denv = 0.f;
  if (x < 1.f) {
    const float xp1 = ipow(x, p - 1), xp = xp1 * x, xq = xp * x, xr = xq * x;
    env = 1.f + a * xp + b * xq + c * xr;
    denv = (a * fp * xp1 + b * (fp + 1.f) * xp + c * (fp + 2.f) * xq) * inv_cut;
  }
#pragma unroll
  for (int k = 0; k < 7; ++k) {
    const float arg = freq[k] * ds;
    const float s = sinf(arg), co = cosf(arg);
    const float out = norm * s / d;
    const float dout = norm * (freq[k] * inv_cut * co / d - s / (d * d));
    val[k] = env * out;
    if (der) der[k] = denv * out + env * dout;
  }
}

__global__ void k_bessel_fwd(int n_bonds, const int32_t* __restrict__ u2d, const float* __restrict__ len,
                             const float* __restrict__ fa, float ca, const float* __restrict__ fb, float cb, int p,
                             float* __restrict__ ra, float* __restrict__ rb) {
  const int u = blockIdx.x * blockDim.x + threadIdx.x;
  if (u >= n_bonds) return;
  const float d = len[u2d[u]];
  float v[7];
  bessel_eval(d, ca, fa, p, v, nullptr);
#pragma unroll
  for (int k = 0; k < 7; ++k) ra[7 * (int64_t)u + k] = v[k];
  bessel_eval(d, cb, fb, p, v, nullptr);
#pragma unroll
  for (int k = 0; k < 7; ++k) rb[7 * (int64_t)u + k] = v[k];
}

__global__ void k_bessel_bwd(int n_bonds, const int32_t* __restrict__ u2d, const float* __restrict__ len,
                             const float* __restrict__ fa, float ca, const float* __restrict__ fb, float cb, int p,
                             const float* __restrict__ dra, const float* __restrict__ drb, float* __restrict__ dlen) {
  const int u = blockIdx.x * blockDim.x + threadIdx.x;
  if (u >= n_bonds) return;
  const int e = u2d[u];
  const float d = len[e];
  float v[7], dv[7], acc = 0.f;
  bessel_eval(d, ca, fa, p, v, dv);
#pragma unroll
  for (int k = 0; k < 7; ++k) acc += dv[k] * dra[7 * (int64_t)u + k];
  bessel_eval(d, cb, fb, p, v, dv);
#pragma unroll
  for (int k = 0; k < 7; ++k) acc += dv[k] * drb[7 * (int64_t)u + k];
  dlen[e] += acc;  // each bond owns one directed edge: no race
}

// Gaussian distance expansion (distance_expansion = "gaussian"; matris/model/basis_function.py:189-216):
// out[k] = exp(coeff (d - offset[k])^2) for the pairwise and the three-body set of seven offsets; no envelope.
__global__ void k_gaussian_fwd(int n_bonds, const int32_t* __restrict__ u2d, const float* __restrict__ len,
                               const float* __restrict__ off_a, float coeff_a, const float* __restrict__ off_b,
                               float coeff_b, float* __restrict__ ra, float* __restrict__ rb) {
  const int u = blockIdx.x * blockDim.x + threadIdx.x;
  if (u >= n_bonds) return;
  const float d = len[u2d[u]];
#pragma unroll
  for (int k = 0; k < 7; ++k) {
    const float ta = d - off_a[k], tb = d - off_b[k];
    ra[7 * (int64_t)u + k] = expf(coeff_a * (ta * ta));
    rb[7 * (int64_t)u + k] = expf(coeff_b * (tb * tb));
  }
}

__global__ void k_gaussian_bwd(int n_bonds, const int32_t* __restrict__ u2d, const float* __restrict__ len,
                               const float* __restrict__ off_a, float coeff_a, const float* __restrict__ off_b,
                               float coeff_b, const float* __restrict__ dra, const float* __restrict__ drb,
                               float* __restrict__ dlen) {
  const int u = blockIdx.x * blockDim.x + threadIdx.x;
  if (u >= n_bonds) return;
  const int e = u2d[u];
  const float d = len[e];
  float acc = 0.f;
#pragma unroll
  for (int k = 0; k < 7; ++k) {
    const float ta = d - off_a[k], tb = d - off_b[k];
    acc += dra[7 * (int64_t)u + k] * expf(coeff_a * (ta * ta)) * (2.f * coeff_a * ta);
    acc += drb[7 * (int64_t)u + k] * expf(coeff_b * (tb * tb)) * (2.f * coeff_b * tb);
  }
  dlen[e] += acc;  // each bond owns one directed edge: no race
}

// ------------------------------------------------------------------ angle basis
// Coefficients of the closed-form spherical Bessel radial functions j_l(z_{l,n} r)
// for l = 0..3 at their first four roots z_{l,n} (the published MatterSim /
// DimeNet-style tabulation that SphericalExpansion evaluates), as float32.
__constant__ float c_sph[4][8][4] = {
    {{3.14159274101257f, 6.28318548202515f, 9.42477798461914f, 12.5663709640503f}},
    {{-1.02446483277785f, -1.00834335996107f, -1.00419641763893f, -1.00252381898662f},
     {4.49340963363647f, 7.7252516746521f, 10.9041213989258f, 14.0661935806274f},
     {0.22799275301076f, 0.130525632358311f, 0.092093290316619f, 0.0712718627992818f},
     {4.49340963363647f, 7.7252516746521f, 10.9041213989258f, 14.0661935806274f}},
    {{-1.04807944170731f, -1.01861796359391f, -1.01002272174988f, -1.00628955560036f},
     {5.76345920562744f, 9.09501171112061f, 12.322940826416f, 15.5146026611328f},
     {0.545547077361439f, 0.335992298618515f, 0.245888396928293f, 0.194582402961821f},
     {5.76345920562744f, 9.09501171112061f, 12.322940826416f, 15.5146026611328f},
     {0.0946561878721665f, 0.0369424811413594f, 0.0199537107571916f, 0.0125418876146463f},
     {5.76345920562744f, 9.09501171112061f, 12.322940826416f, 15.5146026611328f}},
    {{1.06942831392075f, 1.0292173312802f, 1.01650804843248f, 1.01069656069999f},
     {6.9879322052002f, 10.4171180725098f, 13.6980228424072f, 16.9236221313477f},
     {0.918235852195231f, 0.592803493701152f, 0.445250264272671f, 0.358326327374518f},
     {6.9879322052002f, 10.4171180725098f, 13.6980228424072f, 16.9236221313477f},
     {0.328507713452024f, 0.142266673367543f, 0.0812617757677838f, 0.0529328657590962f},
     {6.9879322052002f, 10.4171180725098f, 13.6980228424072f, 16.9236221313477f},
     {0.0470107184508114f, 0.0136570088173405f, 0.0059323726279831f, 0.00312775039221944f},
     {6.9879322052002f, 10.4171180725098f, 13.6980228424072f, 16.9236221313477f}}};

__device__ __forceinline__ void radial16(float x, float factor, float* r) {
  const float x2 = x * x, x3 = x2 * x, x4 = x2 * x2;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    r[j] = sinf(c_sph[0][0][j] * x) / x * factor;
    r[4 + j] = (c_sph[1][0][j] * x * cosf(c_sph[1][1][j] * x) + c_sph[1][2][j] * sinf(c_sph[1][3][j] * x)) / x2 * factor;
    r[8 + j] = (c_sph[2][0][j] * x2 * sinf(c_sph[2][1][j] * x) - c_sph[2][2][j] * x * cosf(c_sph[2][3][j] * x) +
                c_sph[2][4][j] * sinf(c_sph[2][5][j] * x)) / x3 * factor;
    r[12 + j] = (c_sph[3][0][j] * x3 * cosf(c_sph[3][1][j] * x) - c_sph[3][2][j] * x2 * sinf(c_sph[3][3][j] * x) -
                 c_sph[3][4][j] * x * cosf(c_sph[3][5][j] * x) + c_sph[3][6][j] * sinf(c_sph[3][7][j] * x)) / x4 * factor;
  }
}

#define SH0 0.28209479177387814f  /* 0.5 sqrt(1/pi) */
#define SH1 0.4886025119029199f   /* sqrt(3/(4 pi)) */
#define SH2 0.31539156525252005f  /* sqrt(5/(16 pi)) */
#define SH3 0.3731763325901154f   /* sqrt(7/(16 pi)) */
#define ANGLE_SHRINK 0.999999f    /* (1 - 1e-6) as float32 */

__global__ void k_angle_basis_fwd(int64_t n_trip, const int32_t* __restrict__ lg, const float* __restrict__ unit,
                                  float factor, float cutoff, float* __restrict__ basis) {
  const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= n_trip) return;
  const int64_t a = lg[5 * t + 2], b = lg[5 * t + 4];
  const float ax = unit[3 * a], ay = unit[3 * a + 1], az = unit[3 * a + 2];
  const float bx = unit[3 * b], by = unit[3 * b + 1], bz = unit[3 * b + 2];
  const float x = (ax * bx + ay * by + az * bz) * ANGLE_SHRINK;
  const float ct = cosf(acosf(x));
  const float nb = sqrtf(bx * bx + by * by + bz * bz);
  float r[16];
  radial16(nb / cutoff, factor, r);
  const float sh[4] = {SH0, SH1 * ct, SH2 * (3.f * ct * ct - 1.f), SH3 * ct * (5.f * ct * ct - 3.f)};
  float4* out = reinterpret_cast<float4*>(basis + 16 * t);
#pragma unroll
  for (int l = 0; l < 4; ++l)
    out[l] = make_float4(r[4 * l] * sh[l], r[4 * l + 1] * sh[l], r[4 * l + 2] * sh[l], r[4 * l + 3] * sh[l]);
}

__global__ void k_angle_basis_bwd(int64_t n_trip, const int32_t* __restrict__ lg, const float* __restrict__ unit,
                                  float factor, float cutoff, const float* __restrict__ dbasis,
                                  float* __restrict__ dunit) {
  const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= n_trip) return;
  const int64_t a = lg[5 * t + 2], b = lg[5 * t + 4];
  const float ax = unit[3 * a], ay = unit[3 * a + 1], az = unit[3 * a + 2];
  const float bx = unit[3 * b], by = unit[3 * b + 1], bz = unit[3 * b + 2];
  const float x = (ax * bx + ay * by + az * bz) * ANGLE_SHRINK;
  const float theta = acosf(x);
  const float ct = cosf(theta);
  const float nb = sqrtf(bx * bx + by * by + bz * bz);
  float r[16];
  radial16(nb / cutoff, factor, r);
  const float dsh[4] = {0.f, SH1, SH2 * 6.f * ct, SH3 * (15.f * ct * ct - 3.f)};
  float dct = 0.f;
#pragma unroll
  for (int k = 4; k < 16; ++k) dct += dbasis[16 * t + k] * r[k] * dsh[k >> 2];
  // d cos(theta)/d theta = -sin(theta); d acos(x)/dx = -1/sqrt(1 - x^2)   (same two steps as autograd)
  const float dtheta = dct * (-sinf(theta));
  const float dx = dtheta * (-rsqrtf(1.f - x * x));
  const float dd = dx * ANGLE_SHRINK;
  atomicAdd(dunit + 3 * a, dd * bx); atomicAdd(dunit + 3 * a + 1, dd * by); atomicAdd(dunit + 3 * a + 2, dd * bz);
  atomicAdd(dunit + 3 * b, dd * ax); atomicAdd(dunit + 3 * b + 1, dd * ay); atomicAdd(dunit + 3 * b + 2, dd * az);
}

// Fourier angle expansion (three_body_expansion = "fourier"; matris/model/basis_function.py:79-113,
// matris/model/feature_embed.py:183-203): theta = acos(x (1 - 1e-6)), basis = [1/sqrt 2, sin(f_k theta), cos(f_k theta)]
// / sqrt(pi) with three frequencies f_k (seven values per triplet).
#define FOURIER_INV_SQRT_PI 0.5641895835477563f
__global__ void k_fourier_fwd(int64_t n_trip, const int32_t* __restrict__ lg, const float* __restrict__ unit,
                              const float* __restrict__ freq, float* __restrict__ basis) {
  const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= n_trip) return;
  const int64_t a = lg[5 * t + 2], b = lg[5 * t + 4];
  const float x = (unit[3 * a] * unit[3 * b] + unit[3 * a + 1] * unit[3 * b + 1] + unit[3 * a + 2] * unit[3 * b + 2]) *
                  ANGLE_SHRINK;
  const float theta = acosf(x);
  float* out = basis + 7 * t;
  out[0] = 0.70710677f * FOURIER_INV_SQRT_PI;
#pragma unroll
  for (int k = 0; k < 3; ++k) {
    const float ang = theta * freq[k];
    out[1 + k] = sinf(ang) * FOURIER_INV_SQRT_PI;
    out[4 + k] = cosf(ang) * FOURIER_INV_SQRT_PI;
  }
}

__global__ void k_fourier_bwd(int64_t n_trip, const int32_t* __restrict__ lg, const float* __restrict__ unit,
                              const float* __restrict__ freq, const float* __restrict__ dbasis,
                              float* __restrict__ dunit) {
  const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= n_trip) return;
  const int64_t a = lg[5 * t + 2], b = lg[5 * t + 4];
  const float ax = unit[3 * a], ay = unit[3 * a + 1], az = unit[3 * a + 2];
  const float bx = unit[3 * b], by = unit[3 * b + 1], bz = unit[3 * b + 2];
  const float x = (ax * bx + ay * by + az * bz) * ANGLE_SHRINK;
  const float theta = acosf(x);
  float dtheta = 0.f;
#pragma unroll
  for (int k = 0; k < 3; ++k) {
    const float f = freq[k], ang = theta * f;
    dtheta += (dbasis[7 * t + 1 + k] * cosf(ang) - dbasis[7 * t + 4 + k] * sinf(ang)) * f;
  }
  dtheta *= FOURIER_INV_SQRT_PI;
  const float dd = dtheta * (-rsqrtf(1.f - x * x)) * ANGLE_SHRINK;
  atomicAdd(dunit + 3 * a, dd * bx); atomicAdd(dunit + 3 * a + 1, dd * by); atomicAdd(dunit + 3 * a + 2, dd * bz);
  atomicAdd(dunit + 3 * b, dd * ax); atomicAdd(dunit + 3 * b + 1, dd * ay); atomicAdd(dunit + 3 * b + 2, dd * az);
}

}  // namespace mb

using namespace mb;
#define STREAM ((cudaStream_t)stream)
#define MB_REQUIRE(cond) do { if (!(cond)) return MB_ERR_INVALID; } while (0)

extern "C" int mb_edge_geometry_fwd(int64_t n_edges, const float* cart, const float* lattice,
                                    const int32_t* atom_struct, const int32_t* center, const int32_t* neighbor,
                                    const int32_t* image, float* vec, float* len, float* unit, void* stream) {
  MB_REQUIRE(n_edges >= 0 && cart && lattice && atom_struct && center && neighbor && image && vec && len && unit);
  if (n_edges == 0) return MB_OK;
  k_edge_geometry_fwd<<<grid1(n_edges), GEO_THREADS, 0, STREAM>>>(n_edges, cart, lattice, atom_struct, center, neighbor,
                                                                image, vec, len, unit);
  MB_LAUNCH_CHECK("k_edge_geometry_fwd");
  return MB_OK;
}

extern "C" int mb_edge_geometry_bwd(int32_t n_atoms, int32_t n_struct, int64_t n_edges, const int32_t* edge_ptr,
                                    const int32_t* atom_ptr, const int32_t* rev, const float* vec, const float* len,
                                    const float* unit, const float* dlen, const float* dunit, float* g_edge,
                                    float* dcart, float* virial_atom, float* dstrain, void* stream) {
  MB_REQUIRE(n_atoms > 0 && n_struct > 0 && n_edges > 0 && edge_ptr && atom_ptr && rev && vec && len && unit && dlen &&
             dunit && g_edge && dcart && virial_atom && dstrain);
  k_edge_grad<<<grid1(n_edges), GEO_THREADS, 0, STREAM>>>(n_edges, len, unit, dlen, dunit, g_edge);
  k_atom_grad<<<grid1((int64_t)n_atoms * 32), GEO_THREADS, 0, STREAM>>>(n_atoms, edge_ptr, rev, vec, g_edge, dcart,
                                                                       virial_atom);
  k_struct_virial<<<grid1((int64_t)n_struct * 32), GEO_THREADS, 0, STREAM>>>(n_struct, atom_ptr, virial_atom, dstrain);
  MB_LAUNCH_CHECK("mb_edge_geometry_bwd");
  return MB_OK;
}

// ------------------------------------------------------------------ allocation-free force / virial reduction
// Scratch for mb_edge_geometry_bwd_static: the per-edge gradient (3 floats per directed edge) followed by the
// per-atom virial partials (9 floats per atom).  It is part of the library image, so every GPU that loads the
// library holds these bytes until the process exits.
static __device__ __align__(256) float g_static_scratch[3 * MB_STATIC_MAX_EDGES + 9 * MB_STATIC_MAX_ATOMS];

// Host code must not hand `g_static_scratch` itself to a kernel: in host code that name is only a stand-in for
// the symbol.  The device address is looked up once per device, with that device current.
static float* static_scratch_address(int* status) {
  constexpr int MAX_DEVICES = 64;
  static float* address[MAX_DEVICES] = {nullptr};
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) {
    mb::set_cuda_error(e != cudaSuccess ? e : cudaErrorInvalidDevice, "cudaGetDevice (static scratch)");
    *status = MB_ERR_CUDA;
    return nullptr;
  }
  if (!address[dev]) {
    float* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_static_scratch);
    if (e != cudaSuccess || !p) {
      mb::set_cuda_error(e != cudaSuccess ? e : cudaErrorInvalidSymbol, "cudaGetSymbolAddress(g_static_scratch)");
      *status = MB_ERR_CUDA;
      return nullptr;
    }
    address[dev] = p;
  }
  *status = MB_OK;
  return address[dev];
}

extern "C" int mb_edge_geometry_bwd_static(int32_t n_atoms, int32_t n_struct, int64_t n_edges, const int32_t* edge_ptr,
                                           const int32_t* atom_ptr, const int32_t* rev, const float* vec,
                                           const float* len, const float* unit, const float* dlen, const float* dunit,
                                           float* dcart, float* dstrain, void* stream) {
  MB_REQUIRE(n_atoms > 0 && n_struct > 0 && n_edges > 0 && edge_ptr && atom_ptr && rev && vec && len && unit && dlen &&
             dunit && dcart && dstrain);
  if (n_edges > MB_STATIC_MAX_EDGES || n_atoms > MB_STATIC_MAX_ATOMS) return MB_ERR_TOO_LARGE;
  int status = MB_OK;
  float* scratch = static_scratch_address(&status);
  if (!scratch) return status;
  float* g_edge = scratch;                                  // [n_edges,3]  written in full by k_edge_grad before it is read
  float* virial_atom = scratch + 3 * MB_STATIC_MAX_EDGES;   // [n_atoms,9]  written in full by k_atom_grad before it is read
  k_edge_grad<<<grid1(n_edges), GEO_THREADS, 0, STREAM>>>(n_edges, len, unit, dlen, dunit, g_edge);
  k_atom_grad<<<grid1((int64_t)n_atoms * 32), GEO_THREADS, 0, STREAM>>>(n_atoms, edge_ptr, rev, vec, g_edge, dcart,
                                                                       virial_atom);
  k_struct_virial<<<grid1((int64_t)n_struct * 32), GEO_THREADS, 0, STREAM>>>(n_struct, atom_ptr, virial_atom, dstrain);
  MB_LAUNCH_CHECK("mb_edge_geometry_bwd_static");
  return MB_OK;
}

extern "C" int mb_bessel_fwd(int32_t n_bonds, const int32_t* u2d, const float* len, const float* freq_a, float cut_a,
                             const float* freq_b, float cut_b, int32_t p, float* rbf_a, float* rbf_b, void* stream) {
  MB_REQUIRE(n_bonds >= 0 && u2d && len && freq_a && freq_b && rbf_a && rbf_b && p >= 1 && cut_a > 0 && cut_b > 0);
  if (n_bonds == 0) return MB_OK;
  k_bessel_fwd<<<grid1(n_bonds), GEO_THREADS, 0, STREAM>>>(n_bonds, u2d, len, freq_a, cut_a, freq_b, cut_b, p, rbf_a,
                                                         rbf_b);
  MB_LAUNCH_CHECK("k_bessel_fwd");
  return MB_OK;
}

extern "C" int mb_bessel_bwd(int32_t n_bonds, const int32_t* u2d, const float* len, const float* freq_a, float cut_a,
                             const float* freq_b, float cut_b, int32_t p, const float* drbf_a, const float* drbf_b,
                             float* dlen, void* stream) {
  MB_REQUIRE(n_bonds >= 0 && u2d && len && freq_a && freq_b && drbf_a && drbf_b && dlen && p >= 1);
  if (n_bonds == 0) return MB_OK;
  k_bessel_bwd<<<grid1(n_bonds), GEO_THREADS, 0, STREAM>>>(n_bonds, u2d, len, freq_a, cut_a, freq_b, cut_b, p, drbf_a,
                                                         drbf_b, dlen);
  MB_LAUNCH_CHECK("k_bessel_bwd");
  return MB_OK;
}

extern "C" int mb_gaussian_fwd(int32_t n_bonds, const int32_t* u2d, const float* len, const float* off_a, float coeff_a,
                               const float* off_b, float coeff_b, float* rbf_a, float* rbf_b, void* stream) {
  MB_REQUIRE(n_bonds >= 0 && u2d && len && off_a && off_b && rbf_a && rbf_b);
  if (n_bonds == 0) return MB_OK;
  k_gaussian_fwd<<<grid1(n_bonds), GEO_THREADS, 0, STREAM>>>(n_bonds, u2d, len, off_a, coeff_a, off_b, coeff_b, rbf_a,
                                                           rbf_b);
  MB_LAUNCH_CHECK("k_gaussian_fwd");
  return MB_OK;
}

extern "C" int mb_gaussian_bwd(int32_t n_bonds, const int32_t* u2d, const float* len, const float* off_a, float coeff_a,
                               const float* off_b, float coeff_b, const float* drbf_a, const float* drbf_b,
                               float* dlen, void* stream) {
  MB_REQUIRE(n_bonds >= 0 && u2d && len && off_a && off_b && drbf_a && drbf_b && dlen);
  if (n_bonds == 0) return MB_OK;
  k_gaussian_bwd<<<grid1(n_bonds), GEO_THREADS, 0, STREAM>>>(n_bonds, u2d, len, off_a, coeff_a, off_b, coeff_b, drbf_a,
                                                           drbf_b, dlen);
  MB_LAUNCH_CHECK("k_gaussian_bwd");
  return MB_OK;
}

extern "C" int mb_fourier_basis_fwd(int64_t n_trip, const int32_t* line_graph, const float* unit, const float* freq,
                                    float* basis, void* stream) {
  MB_REQUIRE(n_trip >= 0 && line_graph && unit && freq && basis);
  if (n_trip == 0) return MB_OK;
  k_fourier_fwd<<<grid1(n_trip), GEO_THREADS, 0, STREAM>>>(n_trip, line_graph, unit, freq, basis);
  MB_LAUNCH_CHECK("k_fourier_fwd");
  return MB_OK;
}

extern "C" int mb_fourier_basis_bwd(int64_t n_trip, const int32_t* line_graph, const float* unit, const float* freq,
                                    const float* dbasis, float* dunit, void* stream) {
  MB_REQUIRE(n_trip >= 0 && line_graph && unit && freq && dbasis && dunit);
  if (n_trip == 0) return MB_OK;
  k_fourier_bwd<<<grid1(n_trip), GEO_THREADS, 0, STREAM>>>(n_trip, line_graph, unit, freq, dbasis, dunit);
  MB_LAUNCH_CHECK("k_fourier_bwd");
  return MB_OK;
}

extern "C" int mb_angle_basis_fwd(int64_t n_trip, const int32_t* line_graph, const float* unit, float factor,
                                  float cutoff, float* basis, void* stream) {
  MB_REQUIRE(n_trip >= 0 && line_graph && unit && basis && cutoff > 0);
  if (n_trip == 0) return MB_OK;
  k_angle_basis_fwd<<<grid1(n_trip), GEO_THREADS, 0, STREAM>>>(n_trip, line_graph, unit, factor, cutoff, basis);
  MB_LAUNCH_CHECK("k_angle_basis_fwd");
  return MB_OK;
}

extern "C" int mb_angle_basis_bwd(int64_t n_trip, const int32_t* line_graph, const float* unit, float factor,
                                  float cutoff, const float* dbasis, float* dunit, void* stream) {
  MB_REQUIRE(n_trip >= 0 && line_graph && unit && dbasis && dunit && cutoff > 0);
  if (n_trip == 0) return MB_OK;
  k_angle_basis_bwd<<<grid1(n_trip), GEO_THREADS, 0, STREAM>>>(n_trip, line_graph, unit, factor, cutoff, dbasis, dunit);
  MB_LAUNCH_CHECK("k_angle_basis_bwd");
  return MB_OK;
}
