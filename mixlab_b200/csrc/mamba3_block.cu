// Element-wise stages of mixlab's canonical Mamba-3 block around the scan
// (mamba3_canonical_block_impl, gpu/ir.cpp:2034-2105):
//   conv  x_branch = causal depthwise conv of x_proj, weight [D, K], tap k multiplies x[t-k]   (:1397-1425)
//   bc    b = RMSNorm(b_proj rows of N, b_norm_scale, eps) + b_bias, same for c                 (:2089-2094)
//   post  out = RMSNorm(y rows of D, post_norm, eps) z sigmoid(z)                               (:2099-2102)
// and their backward passes: HBM streams in 16-byte pieces.  A thread owns 8 consecutive channels.  Sums over
// (batch, step) - the weight, scale and bias gradients - go through per-CTA partial rows in the workspace and a
// fixed-order second pass (no atomics).
#include "common.cuh"

namespace mxb {
namespace m3b {

using bf16 = __nv_bfloat16;
constexpr int kRun = 16;     // steps per lane for the convolution
constexpr int kMaxK = 4;     // taps

struct BlkP {
  int B, T, D, N, G, K;
  float eps;
};

template <typename IO>
__device__ __forceinline__ void load8(const IO* p, float (&e)[8]);
template <>
__device__ __forceinline__ void load8<float>(const float* p, float (&e)[8]) {
  const float4 a = __ldg(reinterpret_cast<const float4*>(p)), b = __ldg(reinterpret_cast<const float4*>(p) + 1);
  e[0] = a.x; e[1] = a.y; e[2] = a.z; e[3] = a.w; e[4] = b.x; e[5] = b.y; e[6] = b.z; e[7] = b.w;
}
template <>
__device__ __forceinline__ void load8<bf16>(const bf16* p, float (&e)[8]) {
  const uint4 v = __ldg(reinterpret_cast<const uint4*>(p));
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) { e[2 * i] = __low2float(h[i]); e[2 * i + 1] = __high2float(h[i]); }
}
template <typename IO>
__device__ __forceinline__ void store8(IO* p, const float (&e)[8]);
template <>
__device__ __forceinline__ void store8<float>(float* p, const float (&e)[8]) {
  reinterpret_cast<float4*>(p)[0] = make_float4(e[0], e[1], e[2], e[3]);
  reinterpret_cast<float4*>(p)[1] = make_float4(e[4], e[5], e[6], e[7]);
}
template <>
__device__ __forceinline__ void store8<bf16>(bf16* p, const float (&e)[8]) {
  uint4 v;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(e[2 * i], e[2 * i + 1]);
  *reinterpret_cast<uint4*>(p) = v;
}
__device__ __forceinline__ float sigmoid_f(float x) { return __fdividef(1.f, 1.f + __expf(-x)); }

// ------------------------------------------------------------------ depthwise convolution
// grid (ceil(D/8 / 128), ceil(T / kRun), B) x 128: thread = 8 channels, kRun steps; weights w[d][k], k < K <= 4.
template <typename IO>
__global__ void __launch_bounds__(128) m3b_conv_fwd_kernel(BlkP p, const IO* __restrict__ x, const float* __restrict__ w,
                                                           IO* __restrict__ y) {
  const int cg = blockIdx.x * 128 + threadIdx.x, ch = cg * 8;
  if (ch >= p.D) return;
  const int t0 = blockIdx.y * kRun, b = blockIdx.z;
  float wk[kMaxK][8];
#pragma unroll
  for (int k = 0; k < kMaxK; ++k)
#pragma unroll
    for (int c = 0; c < 8; ++c) wk[k][c] = k < p.K ? w[(size_t)(ch + c) * p.K + k] : 0.f;
  const IO* __restrict__ xb = x + (size_t)b * p.T * p.D + ch;
  IO* __restrict__ yb = y + (size_t)b * p.T * p.D + ch;
  float x1[8], x2[8], x3[8];
#pragma unroll
  for (int c = 0; c < 8; ++c) x1[c] = x2[c] = x3[c] = 0.f;
  if (t0 - 1 >= 0) load8<IO>(xb + (size_t)(t0 - 1) * p.D, x1);
  if (t0 - 2 >= 0) load8<IO>(xb + (size_t)(t0 - 2) * p.D, x2);
  if (t0 - 3 >= 0) load8<IO>(xb + (size_t)(t0 - 3) * p.D, x3);
#pragma unroll
  for (int r = 0; r < kRun; ++r) {
    const int t = t0 + r;
    const bool in = t < p.T;
    float x0[8], o[8];
    load8<IO>(xb + (size_t)(in ? t : t0) * p.D, x0);  // clamped address: the loads of the run can all be in flight
#pragma unroll
    for (int c = 0; c < 8; ++c) o[c] = wk[0][c] * x0[c] + wk[1][c] * x1[c] + wk[2][c] * x2[c] + wk[3][c] * x3[c];
    if (in) store8<IO>(yb + (size_t)t * p.D, o);
#pragma unroll
    for (int c = 0; c < 8; ++c) { x3[c] = x2[c]; x2[c] = x1[c]; x1[c] = x0[c]; }
  }
}
// dx[t] = sum_k w[k] dy[t+k];  dw[d][k] partial = sum over this run of x[t-k] dy[t]  -> dwp[(b, run)][k][D]
template <typename IO>
__global__ void __launch_bounds__(128) m3b_conv_bwd_kernel(BlkP p, const IO* __restrict__ x, const float* __restrict__ w,
                                                           const IO* __restrict__ dy, IO* __restrict__ dx,
                                                           float* __restrict__ dwp) {
  const int cg = blockIdx.x * 128 + threadIdx.x, ch = cg * 8;
  if (ch >= p.D) return;
  const int t0 = blockIdx.y * kRun, b = blockIdx.z;
  float wk[kMaxK][8], dw[kMaxK][8];
#pragma unroll
  for (int k = 0; k < kMaxK; ++k)
#pragma unroll
    for (int c = 0; c < 8; ++c) { wk[k][c] = k < p.K ? w[(size_t)(ch + c) * p.K + k] : 0.f; dw[k][c] = 0.f; }
  const IO* __restrict__ xb = x + (size_t)b * p.T * p.D + ch;
  const IO* __restrict__ gb = dy + (size_t)b * p.T * p.D + ch;
  IO* __restrict__ ob = dx + (size_t)b * p.T * p.D + ch;
  float x1[8], x2[8], x3[8], g1[8], g2[8], g3[8];  // previous inputs; previous three dy
#pragma unroll
  for (int c = 0; c < 8; ++c) x1[c] = x2[c] = x3[c] = g1[c] = g2[c] = g3[c] = 0.f;
  if (t0 - 1 >= 0) load8<IO>(xb + (size_t)(t0 - 1) * p.D, x1);
  if (t0 - 2 >= 0) load8<IO>(xb + (size_t)(t0 - 2) * p.D, x2);
  if (t0 - 3 >= 0) load8<IO>(xb + (size_t)(t0 - 3) * p.D, x3);
#pragma unroll
  for (int r = 0; r < kRun + 3; ++r) {
    const int t = t0 + r;
    const bool in = t < p.T;
    float x0[8], g0[8];
    load8<IO>(gb + (size_t)(in ? t : t0) * p.D, g0);  // clamped addresses, masked below
    if (r < kRun) load8<IO>(xb + (size_t)(in ? t : t0) * p.D, x0);
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      g0[c] = in ? g0[c] : 0.f;
      x0[c] = (in && r < kRun) ? x0[c] : 0.f;
    }
    if (r < kRun) {
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        dw[0][c] = fmaf(x0[c], g0[c], dw[0][c]);
        dw[1][c] = fmaf(x1[c], g0[c], dw[1][c]);
        dw[2][c] = fmaf(x2[c], g0[c], dw[2][c]);
        dw[3][c] = fmaf(x3[c], g0[c], dw[3][c]);
      }
    }
    if (r >= 3 && t - 3 < p.T) {  // dx[t-3] = w0 dy[t-3] + w1 dy[t-2] + w2 dy[t-1] + w3 dy[t]
      float o[8];
#pragma unroll
      for (int c = 0; c < 8; ++c) o[c] = wk[0][c] * g3[c] + wk[1][c] * g2[c] + wk[2][c] * g1[c] + wk[3][c] * g0[c];
      store8<IO>(ob + (size_t)(t - 3) * p.D, o);
    }
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      x3[c] = x2[c]; x2[c] = x1[c]; x1[c] = x0[c];
      g3[c] = g2[c]; g2[c] = g1[c]; g1[c] = g0[c];
    }
  }
  float* dst = dwp + ((size_t)(b * gridDim.y + blockIdx.y) * kMaxK) * p.D + ch;
#pragma unroll
  for (int k = 0; k < kMaxK; ++k) store8<float>(dst + (size_t)k * p.D, dw[k]);
}
// dw[d][k] = sum over rows of dwp[row][k][d]  (fixed order); one thread per (d, k)
__global__ void __launch_bounds__(256) m3b_conv_dw_kernel(BlkP p, const float* __restrict__ dwp, int rows,
                                                          float* __restrict__ dw) {
  const int i = blockIdx.x * 256 + threadIdx.x;
  if (i >= p.D * p.K) return;
  const int d = i / p.K, k = i % p.K;
  float s = 0.f;
  for (int r = 0; r < rows; ++r) s += dwp[((size_t)r * kMaxK + k) * p.D + d];
  dw[i] = s;
}
// out[f(j)] = sum over rows of part[row][j] in a fixed order: a CTA owns 32 columns, its 8 warps take every 8th row,
// then the 8 slices are added in order.  K > 0: columns are [k][d] and the result is stored as [d][K] (k < K only).
__global__ void __launch_bounds__(256) m3b_colsum_kernel(const float* __restrict__ part, int rows, int n,
                                                         float* __restrict__ out, int D, int K) {
  __shared__ float red[8][32];
  const int j = blockIdx.x * 32 + (threadIdx.x & 31), slice = threadIdx.x >> 5;
  float s = 0.f;
  if (j < n)
    for (int r = slice; r < rows; r += 8) s += part[(size_t)r * n + j];
  red[slice][threadIdx.x & 31] = s;
  __syncthreads();
  if (threadIdx.x < 32 && j < n) {
    float t = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) t += red[k][threadIdx.x];
    if (K > 0) {
      const int k = j / D, d = j % D;
      if (k < K) out[(size_t)d * K + k] = t;
    } else {
      out[j] = t;
    }
  }
}

// sum over the 16 lanes of a group; the mask names only the caller's half of the warp (the two lane groups of a
// warp may run different numbers of loop iterations)
__device__ __forceinline__ float group_sum(float v) {
  const unsigned mask = 0xffffu << (threadIdx.x & 16);
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(mask, v, o);
  return v;
}

// ------------------------------------------------------------------ B / C: RMSNorm over N + bias
// grid (ctas, G, 2) x 128: blockIdx.z selects b or c, blockIdx.y the group; 8 lane groups of 16 lanes, a lane group
// per row (b, t).  N <= 128, N % 8 == 0.
template <typename IO>
struct BcArgs {
  const IO* x[2];
  const float* scale[2];
  const float* bias[2];
  IO* y[2];
  const IO* dy[2];
  IO* dx[2];
  float* part[2];  // [ctas][G][2][N]: dscale, dbias partial rows
};
template <typename IO>
__global__ void __launch_bounds__(128) m3b_bc_fwd_kernel(BlkP p, BcArgs<IO> a) {
  const int which = blockIdx.z, g = blockIdx.y, lane16 = threadIdx.x & 15, grp = threadIdx.x >> 4;
  const bool act = lane16 * 8 < p.N;
  float sc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, bi[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (act) { load8<float>(a.scale[which] + lane16 * 8, sc); load8<float>(a.bias[which] + g * p.N + lane16 * 8, bi); }
  const size_t nbt = (size_t)p.B * p.T;
  for (size_t bt = (size_t)blockIdx.x * 8 + grp; bt < nbt; bt += (size_t)gridDim.x * 8) {
    const size_t off = (bt * p.G + g) * p.N + lane16 * 8;
    float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (act) load8<IO>(a.x[which] + off, v);
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < 8; ++c) ss = fmaf(v[c], v[c], ss);
    ss = group_sum(ss);
    const float rn = rsqrtf(ss / (float)p.N + p.eps);
#pragma unroll
    for (int c = 0; c < 8; ++c) v[c] = fmaf(v[c] * rn, sc[c], bi[c]);
    if (act) store8<IO>(a.y[which] + off, v);
  }
}
template <typename IO>
__global__ void __launch_bounds__(128) m3b_bc_bwd_kernel(BlkP p, BcArgs<IO> a) {
  __shared__ float red[8][2][128];
  const int which = blockIdx.z, g = blockIdx.y, lane16 = threadIdx.x & 15, grp = threadIdx.x >> 4;
  const bool act = lane16 * 8 < p.N;
  float sc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  float ds[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, db[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (act) load8<float>(a.scale[which] + lane16 * 8, sc);
  const size_t nbt = (size_t)p.B * p.T;
  for (size_t bt = (size_t)blockIdx.x * 8 + grp; bt < nbt; bt += (size_t)gridDim.x * 8) {
    const size_t off = (bt * p.G + g) * p.N + lane16 * 8;
    float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, gy[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (act) { load8<IO>(a.x[which] + off, v); load8<IO>(a.dy[which] + off, gy); }
    float ss = 0.f, dot = 0.f;
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      ss = fmaf(v[c], v[c], ss);
      dot = fmaf(v[c], gy[c] * sc[c], dot);
    }
    ss = group_sum(ss);
    dot = group_sum(dot);
    const float rn = rsqrtf(ss / (float)p.N + p.eps);
    const float k2 = rn * rn * dot / (float)p.N;
    float o[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      ds[c] = fmaf(gy[c], v[c] * rn, ds[c]);
      db[c] += gy[c];
      o[c] = rn * (gy[c] * sc[c] - v[c] * k2);
    }
    if (act) store8<IO>(a.dx[which] + off, o);
  }
#pragma unroll
  for (int c = 0; c < 8; ++c) { red[grp][0][lane16 * 8 + c] = ds[c]; red[grp][1][lane16 * 8 + c] = db[c]; }
  __syncthreads();
  float* dst = a.part[which] + ((size_t)(blockIdx.x * p.G + g) * 2) * p.N;
  for (int i = threadIdx.x; i < 2 * p.N; i += 128) {
    const int kind = i / p.N, c = i % p.N;
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) s += red[k][kind][c];
    dst[(size_t)kind * p.N + c] = s;
  }
}
// from the column sums tab[g][kind][c] over the CTAs: dbias[g][c] = tab[g][1][c], dscale[c] = sum over g of tab[g][0][c]
__global__ void __launch_bounds__(128) m3b_bc_final_kernel(BlkP p, const float* __restrict__ tab,
                                                           float* __restrict__ dscale, float* __restrict__ dbias) {
  const int c = threadIdx.x;
  if (c >= p.N) return;
  float s = 0.f;
  for (int g = 0; g < p.G; ++g) {
    s += tab[((size_t)g * 2 + 0) * p.N + c];
    dbias[g * p.N + c] = tab[((size_t)g * 2 + 1) * p.N + c];
  }
  dscale[c] = s;
}

// ------------------------------------------------------------------ post: RMSNorm over D x SiLU gate
// a CTA of 256 threads per token row (D <= 2048, D % 8 == 0), grid-stride over the B*T rows
__device__ __forceinline__ float cta_sum(float v, float* red) {
  v = warp_sum(v);
  __syncthreads();  // red may still be read from the previous use
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float s = 0.f;
#pragma unroll
  for (int k = 0; k < 8; ++k) s += red[k];
  return s;
}
template <typename IO>
__global__ void __launch_bounds__(256) m3b_post_fwd_kernel(BlkP p, const IO* __restrict__ y, const IO* __restrict__ z,
                                                           const float* __restrict__ wn, IO* __restrict__ out) {
  __shared__ float red[8];
  const int ch = threadIdx.x * 8;
  const bool act = ch < p.D;
  float w[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (act) load8<float>(wn + ch, w);
  const size_t rows = (size_t)p.B * p.T;
  for (size_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const size_t off = row * p.D + ch;
    float yv[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, zv[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (act) { load8<IO>(y + off, yv); load8<IO>(z + off, zv); }
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < 8; ++c) ss = fmaf(yv[c], yv[c], ss);
    ss = cta_sum(ss, red);
    const float rn = rsqrtf(ss / (float)p.D + p.eps);
#pragma unroll
    for (int c = 0; c < 8; ++c) yv[c] = yv[c] * rn * w[c] * zv[c] * sigmoid_f(zv[c]);
    if (act) store8<IO>(out + off, yv);
  }
}
template <typename IO>
__global__ void __launch_bounds__(256) m3b_post_bwd_kernel(BlkP p, const IO* __restrict__ y, const IO* __restrict__ z,
                                                           const float* __restrict__ wn, const IO* __restrict__ dout,
                                                           IO* __restrict__ dy, IO* __restrict__ dz,
                                                           float* __restrict__ dwp) {
  __shared__ float red[8];
  const int ch = threadIdx.x * 8;
  const bool act = ch < p.D;
  float w[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, dw[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (act) load8<float>(wn + ch, w);
  const size_t rows = (size_t)p.B * p.T;
  for (size_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const size_t off = row * p.D + ch;
    float yv[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, zv[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    float gv[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (act) { load8<IO>(y + off, yv); load8<IO>(z + off, zv); load8<IO>(dout + off, gv); }
    float ss = 0.f, dot = 0.f, g[8], sz[8], dsz[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      const float sg = sigmoid_f(zv[c]);
      sz[c] = zv[c] * sg;
      dsz[c] = fmaf(sz[c], 1.f - sg, sg);
      g[c] = gv[c] * sz[c] * w[c];
      ss = fmaf(yv[c], yv[c], ss);
      dot = fmaf(yv[c], g[c], dot);
    }
    ss = cta_sum(ss, red);
    dot = cta_sum(dot, red);
    const float rn = rsqrtf(ss / (float)p.D + p.eps);
    const float k2 = rn * rn * dot / (float)p.D;
    float dzv[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      const float yn = yv[c] * rn;
      dw[c] = fmaf(gv[c] * sz[c], yn, dw[c]);
      dzv[c] = gv[c] * w[c] * yn * dsz[c];
      g[c] = rn * (g[c] - yv[c] * k2);
    }
    if (act) { store8<IO>(dy + off, g); store8<IO>(dz + off, dzv); }
  }
  if (act) store8<float>(dwp + (size_t)blockIdx.x * p.D + ch, dw);
}

}  // namespace m3b

// ------------------------------------------------------------------ host
using m3b::BlkP;

static BlkP make_m3b(const mxb_mamba3_desc* d, int K, float eps) {
  BlkP p{};
  p.B = d->B; p.T = d->T; p.D = d->D; p.N = d->N; p.G = d->G; p.K = K; p.eps = eps;
  return p;
}
bool mamba3_block_supported(const mxb_mamba3_desc* d) {
  return d->D % 8 == 0 && d->D <= 2048 && d->N % 8 == 0 && d->N <= 128 && d->G > 0;
}
static int m3b_runs(const mxb_mamba3_desc* d) { return (d->T + m3b::kRun - 1) / m3b::kRun; }
static int m3b_bc_ctas(const mxb_mamba3_desc* d) {
  const size_t want = ((size_t)d->B * d->T + 7) / 8;
  return (int)(want < 148 * 4 ? want : 148 * 4);
}
static int m3b_post_ctas(const mxb_mamba3_desc* d) {
  const size_t rows = (size_t)d->B * d->T;
  return (int)(rows < 148 * 8 ? rows : 148 * 8);
}
size_t mamba3_block_workspace_bytes(const mxb_mamba3_desc* d) {
  const size_t conv = (size_t)d->B * m3b_runs(d) * m3b::kMaxK * d->D * sizeof(float);
  const size_t bc = 2 * ((size_t)m3b_bc_ctas(d) + 1) * d->G * 2 * d->N * sizeof(float);
  const size_t post = (size_t)m3b_post_ctas(d) * d->D * sizeof(float);
  size_t m = conv > bc ? conv : bc;
  m = m > post ? m : post;
  return m + 256;
}

template <typename IO>
static mxb_status m3b_conv(const mxb_mamba3_desc* d, int K, const void* x, const float* w, void* y, const void* dy,
                           void* dx, float* dw, void* ws, cudaStream_t st) {
  BlkP p = make_m3b(d, K, 0.f);
  const dim3 grid((d->D / 8 + 127) / 128, m3b_runs(d), d->B);
  if (!dy) {
    MXB_LAUNCH("m3b_conv_fwd_kernel", st,
               (m3b::m3b_conv_fwd_kernel<IO><<<grid, 128, 0, st>>>(p, static_cast<const IO*>(x), w, static_cast<IO*>(y))));
    return check_launch("m3b_conv_fwd");
  }
  float* part = reinterpret_cast<float*>(static_cast<char*>(ws) + 256);
  MXB_LAUNCH("m3b_conv_bwd_kernel", st,
             (m3b::m3b_conv_bwd_kernel<IO><<<grid, 128, 0, st>>>(p, static_cast<const IO*>(x), w, static_cast<const IO*>(dy),
                                                                 static_cast<IO*>(dx), part)));
  const int rows = d->B * m3b_runs(d), n = m3b::kMaxK * d->D;
  MXB_LAUNCH("m3b_colsum_kernel", st, (m3b::m3b_colsum_kernel<<<(n + 31) / 32, 256, 0, st>>>(part, rows, n, dw, d->D, K)));
  return check_launch("m3b_conv_bwd");
}
mxb_status mamba3_block_conv(const mxb_mamba3_desc* d, int K, const void* x, const float* w, void* y, const void* dy,
                             void* dx, float* dw, void* ws, cudaStream_t st) {
  return d->io_dtype == MXB_F32 ? m3b_conv<float>(d, K, x, w, y, dy, dx, dw, ws, st)
                                : m3b_conv<m3b::bf16>(d, K, x, w, y, dy, dx, dw, ws, st);
}

template <typename IO>
static mxb_status m3b_bc(const mxb_mamba3_desc* d, float eps, const void* bp, const void* cp, const float* bs,
                         const float* cs, const float* bb, const float* cb, void* b, void* c, const void* db,
                         const void* dc, void* dbp, void* dcp, float* dbs, float* dcs, float* dbb, float* dcb, void* ws,
                         cudaStream_t st) {
  BlkP p = make_m3b(d, 0, eps);
  m3b::BcArgs<IO> a{};
  a.x[0] = static_cast<const IO*>(bp); a.x[1] = static_cast<const IO*>(cp);
  a.scale[0] = bs; a.scale[1] = cs; a.bias[0] = bb; a.bias[1] = cb;
  const int ctas = m3b_bc_ctas(d);
  if (!db) {
    a.y[0] = static_cast<IO*>(b); a.y[1] = static_cast<IO*>(c);
    MXB_LAUNCH("m3b_bc_fwd_kernel", st, (m3b::m3b_bc_fwd_kernel<IO><<<dim3(ctas, d->G, 2), 128, 0, st>>>(p, a)));
    return check_launch("m3b_bc_fwd");
  }
  a.dy[0] = static_cast<const IO*>(db); a.dy[1] = static_cast<const IO*>(dc);
  a.dx[0] = static_cast<IO*>(dbp); a.dx[1] = static_cast<IO*>(dcp);
  float* base = reinterpret_cast<float*>(static_cast<char*>(ws) + 256);
  const size_t per = (size_t)ctas * d->G * 2 * d->N;
  a.part[0] = base; a.part[1] = base + per;
  MXB_LAUNCH("m3b_bc_bwd_kernel", st, (m3b::m3b_bc_bwd_kernel<IO><<<dim3(ctas, d->G, 2), 128, 0, st>>>(p, a)));
  const int n = d->G * 2 * d->N;
  float* tab = base + 2 * per;  // [2][G][2][N]
  float* outs[2][2] = {{dbs, dbb}, {dcs, dcb}};
  for (int w = 0; w < 2; ++w) {
    MXB_LAUNCH("m3b_colsum_kernel", st,
               (m3b::m3b_colsum_kernel<<<(n + 31) / 32, 256, 0, st>>>(a.part[w], ctas, n, tab + (size_t)w * n, n, 0)));
    MXB_LAUNCH("m3b_bc_final_kernel", st,
               (m3b::m3b_bc_final_kernel<<<1, 128, 0, st>>>(p, tab + (size_t)w * n, outs[w][0], outs[w][1])));
  }
  return check_launch("m3b_bc_bwd");
}
mxb_status mamba3_block_bc(const mxb_mamba3_desc* d, float eps, const void* bp, const void* cp, const float* bs,
                           const float* cs, const float* bb, const float* cb, void* b, void* c, const void* db,
                           const void* dc, void* dbp, void* dcp, float* dbs, float* dcs, float* dbb, float* dcb, void* ws,
                           cudaStream_t st) {
  return d->io_dtype == MXB_F32
             ? m3b_bc<float>(d, eps, bp, cp, bs, cs, bb, cb, b, c, db, dc, dbp, dcp, dbs, dcs, dbb, dcb, ws, st)
             : m3b_bc<m3b::bf16>(d, eps, bp, cp, bs, cs, bb, cb, b, c, db, dc, dbp, dcp, dbs, dcs, dbb, dcb, ws, st);
}

template <typename IO>
static mxb_status m3b_post(const mxb_mamba3_desc* d, float eps, const void* y, const void* z, const float* wn, void* out,
                           const void* dout, void* dy, void* dz, float* dwn, void* ws, cudaStream_t st) {
  BlkP p = make_m3b(d, 0, eps);
  const int ctas = m3b_post_ctas(d);
  if (!dout) {
    MXB_LAUNCH("m3b_post_fwd_kernel", st,
               (m3b::m3b_post_fwd_kernel<IO><<<ctas, 256, 0, st>>>(p, static_cast<const IO*>(y), static_cast<const IO*>(z),
                                                                   wn, static_cast<IO*>(out))));
    return check_launch("m3b_post_fwd");
  }
  float* part = reinterpret_cast<float*>(static_cast<char*>(ws) + 256);
  MXB_LAUNCH("m3b_post_bwd_kernel", st,
             (m3b::m3b_post_bwd_kernel<IO><<<ctas, 256, 0, st>>>(p, static_cast<const IO*>(y), static_cast<const IO*>(z), wn,
                                                                 static_cast<const IO*>(dout), static_cast<IO*>(dy),
                                                                 static_cast<IO*>(dz), part)));
  MXB_LAUNCH("m3b_colsum_kernel", st,
             (m3b::m3b_colsum_kernel<<<(d->D + 31) / 32, 256, 0, st>>>(part, ctas, d->D, dwn, d->D, 0)));
  return check_launch("m3b_post_bwd");
}
mxb_status mamba3_block_post(const mxb_mamba3_desc* d, float eps, const void* y, const void* z, const float* wn, void* out,
                             const void* dout, void* dy, void* dz, float* dwn, void* ws, cudaStream_t st) {
  return d->io_dtype == MXB_F32 ? m3b_post<float>(d, eps, y, z, wn, out, dout, dy, dz, dwn, ws, st)
                                : m3b_post<m3b::bf16>(d, eps, y, z, wn, out, dout, dy, dz, dwn, ws, st);
}

}  // namespace mxb
