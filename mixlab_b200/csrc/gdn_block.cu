// Element-wise stages of mixlab's gated_deltanet block around the scan
// (emitGatedDeltaNetDeltaIR, arch/blocks_gated_deltanet.go:207-343; short convolution :345-368):
//   pre   q_seq = SiLU(conv4(q_proj)), k_seq = SiLU(conv4(k_proj)), v = SiLU(conv4(v_proj))      causal, 4 taps
//         q = q_seq rsqrt(mean(q_seq^2) + 1e-6) / dk,  k = k_seq rsqrt(mean(k_seq^2) + 1e-6) / sqrt(dk)
//         gate = exp(-softplus(a_raw + dt_bias) exp(A_log)),  beta = sigmoid(b_raw)
//   post  y = o rsqrt(mean(o^2) + 1e-5) o_norm SiLU(z)
// and their backward passes.  All of it is an HBM stream: every element is read once (plus a 3-step halo of the
// convolution) and written once, in 16-byte pieces.
//
// Work split: a row is one (batch, step, head) vector of D <= 128 channels; a thread owns 8 consecutive channels
// (one 16-byte bf16 unit), so 16 lanes cover a row and the row reductions are 4 shuffles.  For the convolution a
// lane group walks kRun consecutive steps of one (batch, head) with the previous three inputs in registers.
// Sums over (batch, step) - convolution weight, norm weight, A_log, dt_bias gradients - go through per-CTA partial
// rows in the workspace and a fixed-order second pass (no atomics).
#include "common.cuh"

namespace mxb {
namespace blk {

using bf16 = __nv_bfloat16;
constexpr int kRun = 16;      // steps per lane group (3 more are recomputed as halo in the backward)
constexpr int kGroups = 8;    // lane groups per CTA (128 threads)
constexpr int kTile = kRun * kGroups;

struct BlockP {
  int B, T, H, Dk, Dv, gate_is_log;
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
// sum over the 16 lanes of a group.  The mask names only the caller's half of the warp: the two lane groups of a
// warp may run different numbers of loop iterations, so neither may wait for the other.
__device__ __forceinline__ float group_sum(float v) {
  const unsigned mask = 0xffffu << (threadIdx.x & 16);
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(mask, v, o);
  return v;
}
__device__ __forceinline__ float sigmoid_f(float x) { return __fdividef(1.f, 1.f + __expf(-x)); }
// sigmoid for the streams: bf16 I/O takes tanh.approx (one MUFU op, relative error ~5e-4, far below the rounding
// of the stored result); fp32 I/O takes exp + reciprocal (a few ulp)
template <typename IO>
__device__ __forceinline__ float sigmoid_io(float x) {
  return sigmoid_f(x);
}
template <>
__device__ __forceinline__ float sigmoid_io<__nv_bfloat16>(float x) {
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.5f * x));
  return fmaf(0.5f, t, 0.5f);
}
__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(__expf(x)); }

// which of the three streams (q, k, v) a CTA works on
template <typename IO>
struct PreArgs {
  const IO* x[3];        // q_proj, k_proj, v_proj   [B,T,H*D]
  const float* w[3];     // conv weights             [4, H*D]
  IO* y[3];              // q, k, v
  const IO* dy[3];       // backward: dq, dk, dv
  IO* dx[3];             // backward: dq_proj, dk_proj, dv_proj
  float* dwp[3];         // backward: per-CTA partial rows [B*ntiles][4][H*D]
};

// ------------------------------------------------------------------ pre: forward
// grid (3 * ntiles, H, B) x 128.  blockIdx.x / ntiles selects q, k or v.
template <typename IO>
__global__ void __launch_bounds__(128) gdn_block_pre_fwd_kernel(BlockP p, PreArgs<IO> a, int ntiles) {
  const int which = blockIdx.x / ntiles, tile = blockIdx.x % ntiles;
  const int h = blockIdx.y, b = blockIdx.z;
  const int D = which == 2 ? p.Dv : p.Dk, C = p.H * D;
  const int lane16 = threadIdx.x & 15, grp = threadIdx.x >> 4;
  const bool act = lane16 * 8 < D;
  const int ch = h * D + lane16 * 8;  // first of this thread's 8 channels
  const int t0 = tile * kTile + grp * kRun;
  const IO* x = a.x[which] + (size_t)b * p.T * C + ch;
  IO* y = a.y[which] + (size_t)b * p.T * C + ch;
  float w[4][8];  // zero for the lanes beyond D: their zero results take part in the row sums
#pragma unroll
  for (int tap = 0; tap < 4; ++tap)
#pragma unroll
    for (int c = 0; c < 8; ++c) w[tap][c] = 0.f;
  if (act) {
#pragma unroll
    for (int tap = 0; tap < 4; ++tap) load8<float>(a.w[which] + tap * C + ch, w[tap]);
  }
  const float scale = which == 0 ? 1.f / (float)D : rsqrtf((float)D);  // q: 1/dk, k: 1/sqrt(dk)
  float x1[8], x2[8], x3[8];  // inputs of the previous three steps
#pragma unroll
  for (int c = 0; c < 8; ++c) x1[c] = x2[c] = x3[c] = 0.f;
  if (act) {
    if (t0 - 1 >= 0 && t0 - 1 < p.T) load8<IO>(x + (size_t)(t0 - 1) * C, x1);
    if (t0 - 2 >= 0 && t0 - 2 < p.T) load8<IO>(x + (size_t)(t0 - 2) * C, x2);
    if (t0 - 3 >= 0 && t0 - 3 < p.T) load8<IO>(x + (size_t)(t0 - 3) * C, x3);
  }
#pragma unroll
  for (int r = 0; r < kRun; ++r) {
    const int t = t0 + r;
    const bool in = act && t < p.T;  // t < T is uniform over the 16 lanes of a group
    float x0[8], s[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) x0[c] = 0.f;
    if (in) load8<IO>(x + (size_t)t * C, x0);
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      const float acc = w[0][c] * x0[c] + w[1][c] * x1[c] + w[2][c] * x2[c] + w[3][c] * x3[c];
      s[c] = acc * sigmoid_io<IO>(acc);  // rows past T are computed on zero-filled inputs and not stored
      ss = fmaf(s[c], s[c], ss);
    }
    if (which < 2) {
      ss = group_sum(ss);
      const float rn = rsqrtf(ss / (float)D + 1e-6f) * scale;
#pragma unroll
      for (int c = 0; c < 8; ++c) s[c] *= rn;
    }
    if (in) store8<IO>(y + (size_t)t * C, s);
#pragma unroll
    for (int c = 0; c < 8; ++c) { x3[c] = x2[c]; x2[c] = x1[c]; x1[c] = x0[c]; }
  }
}

// gate = exp(-softplus(a_raw + dt_bias) exp(A_log)) (or its log), beta = sigmoid(b_raw): one thread per (b, t, h)
__global__ void __launch_bounds__(256) gdn_block_gate_fwd_kernel(BlockP p, const float* __restrict__ a_raw,
                                                                 const float* __restrict__ b_raw,
                                                                 const float* __restrict__ a_log,
                                                                 const float* __restrict__ dt_bias,
                                                                 float* __restrict__ beta, float* __restrict__ gate) {
  const size_t n = (size_t)p.B * p.T * p.H;
  for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < n; i += (size_t)gridDim.x * 256) {
    const int h = (int)(i % p.H);
    const float lg = -softplus_f(a_raw[i] + dt_bias[h]) * expf(a_log[h]);
    gate[i] = p.gate_is_log ? lg : expf(lg);
    beta[i] = sigmoid_f(b_raw[i]);
  }
}

// ------------------------------------------------------------------ pre: backward
// Same split as the forward.  A lane group recomputes the convolution of its run and of the three steps after it
// (their ds feeds dx of the run), keeps the last four ds in registers and emits dx three steps behind.
// The backward keeps 4 channels per thread (a warp covers a row): its per-thread state - weights, weight-gradient
// accumulators, three previous inputs and three previous ds per channel - would otherwise take ~180 registers and
// leave two CTAs per SM.
constexpr int kBwdGroups = 4;                   // warps per CTA, one run each
constexpr int kBwdTile = kRun * kBwdGroups;
template <typename IO>
__device__ __forceinline__ void load4(const IO* p, float (&e)[4]);
template <>
__device__ __forceinline__ void load4<float>(const float* p, float (&e)[4]) {
  const float4 a = __ldg(reinterpret_cast<const float4*>(p));
  e[0] = a.x; e[1] = a.y; e[2] = a.z; e[3] = a.w;
}
template <>
__device__ __forceinline__ void load4<bf16>(const bf16* p, float (&e)[4]) {
  const uint2 v = __ldg(reinterpret_cast<const uint2*>(p));
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
  e[0] = __low2float(h[0]); e[1] = __high2float(h[0]); e[2] = __low2float(h[1]); e[3] = __high2float(h[1]);
}
template <typename IO>
__device__ __forceinline__ void store4(IO* p, const float (&e)[4]);
template <>
__device__ __forceinline__ void store4<float>(float* p, const float (&e)[4]) {
  *reinterpret_cast<float4*>(p) = make_float4(e[0], e[1], e[2], e[3]);
}
template <>
__device__ __forceinline__ void store4<bf16>(bf16* p, const float (&e)[4]) {
  uint2 v;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
  h[0] = __floats2bfloat162_rn(e[0], e[1]);
  h[1] = __floats2bfloat162_rn(e[2], e[3]);
  *reinterpret_cast<uint2*>(p) = v;
}

template <typename IO>
__global__ void __launch_bounds__(128) gdn_block_pre_bwd_kernel(BlockP p, PreArgs<IO> a, int ntiles) {
  __shared__ float red[kBwdGroups][4][128];
  const int which = blockIdx.x / ntiles, tile = blockIdx.x % ntiles;
  const int h = blockIdx.y, b = blockIdx.z;
  const int D = which == 2 ? p.Dv : p.Dk, C = p.H * D;
  const int lane32 = threadIdx.x & 31, grp = threadIdx.x >> 5;
  const bool act = lane32 * 4 < D;
  const int ch = h * D + lane32 * 4;
  const int t0 = tile * kBwdTile + grp * kRun;
  const IO* x = a.x[which] + (size_t)b * p.T * C + ch;
  const IO* dy = a.dy[which] + (size_t)b * p.T * C + ch;
  IO* dx = a.dx[which] + (size_t)b * p.T * C + ch;
  float w[4][4], dw[4][4];
#pragma unroll
  for (int tap = 0; tap < 4; ++tap)
#pragma unroll
    for (int c = 0; c < 4; ++c) { w[tap][c] = 0.f; dw[tap][c] = 0.f; }
  if (act) {
#pragma unroll
    for (int tap = 0; tap < 4; ++tap) load4<float>(a.w[which] + tap * C + ch, w[tap]);
  }
  const float scale = which == 0 ? 1.f / (float)D : rsqrtf((float)D);
  float x1[4], x2[4], x3[4], d1[4], d2[4], d3[4];  // previous inputs; previous three ds
#pragma unroll
  for (int c = 0; c < 4; ++c) x1[c] = x2[c] = x3[c] = d1[c] = d2[c] = d3[c] = 0.f;
  if (act) {
    if (t0 - 1 >= 0 && t0 - 1 < p.T) load4<IO>(x + (size_t)(t0 - 1) * C, x1);
    if (t0 - 2 >= 0 && t0 - 2 < p.T) load4<IO>(x + (size_t)(t0 - 2) * C, x2);
    if (t0 - 3 >= 0 && t0 - 3 < p.T) load4<IO>(x + (size_t)(t0 - 3) * C, x3);
  }
#pragma unroll
  for (int r = 0; r < kRun + 3; ++r) {
    const int t = t0 + r;
    const bool in = act && t < p.T;
    float x0[4], g[4], ds[4];
#pragma unroll
    for (int c = 0; c < 4; ++c) { x0[c] = 0.f; g[c] = 0.f; }
    if (in) { load4<IO>(x + (size_t)t * C, x0); load4<IO>(dy + (size_t)t * C, g); }
    // one sigmoid per element gives SiLU and its derivative; rows past T have zero dy, hence zero ds
    float sv[4], dsl[4], ss = 0.f, dot = 0.f;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const float acc = w[0][c] * x0[c] + w[1][c] * x1[c] + w[2][c] * x2[c] + w[3][c] * x3[c];
      const float sg = sigmoid_io<IO>(acc);
      sv[c] = acc * sg;
      dsl[c] = fmaf(sv[c], 1.f - sg, sg);  // sg (1 + acc (1 - sg))
      ss = fmaf(sv[c], sv[c], ss);
      dot = fmaf(sv[c], g[c], dot);
    }
    if (which < 2) {  // y = s rn scale: ds_c = scale rn (g_c - s_c rn^2 dot / D)
      ss = warp_sum(ss);
      dot = warp_sum(dot);
      const float rn = rsqrtf(ss / (float)D + 1e-6f);
      const float k2 = rn * rn * dot / (float)D;
#pragma unroll
      for (int c = 0; c < 4; ++c) g[c] = scale * rn * (g[c] - sv[c] * k2);
    }
#pragma unroll
    for (int c = 0; c < 4; ++c) ds[c] = g[c] * dsl[c];
    if (r < kRun) {  // this step belongs to the run: its share of the weight gradient
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        dw[0][c] = fmaf(x0[c], ds[c], dw[0][c]);
        dw[1][c] = fmaf(x1[c], ds[c], dw[1][c]);
        dw[2][c] = fmaf(x2[c], ds[c], dw[2][c]);
        dw[3][c] = fmaf(x3[c], ds[c], dw[3][c]);
      }
    }
    if (r >= 3) {  // dx of step t-3 is complete: w0 ds[t-3] + w1 ds[t-2] + w2 ds[t-1] + w3 ds[t]
      const int to = t - 3;
      if (act && to < p.T) {
        float o[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) o[c] = w[0][c] * d3[c] + w[1][c] * d2[c] + w[2][c] * d1[c] + w[3][c] * ds[c];
        store4<IO>(dx + (size_t)to * C, o);
      }
    }
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      x3[c] = x2[c]; x2[c] = x1[c]; x1[c] = x0[c];
      d3[c] = d2[c]; d2[c] = d1[c]; d1[c] = ds[c];
    }
  }
  // weight-gradient partial of this CTA: sum over its lane groups in a fixed order
#pragma unroll
  for (int tap = 0; tap < 4; ++tap)
#pragma unroll
    for (int c = 0; c < 4; ++c) red[grp][tap][lane32 * 4 + c] = dw[tap][c];
  __syncthreads();
  float* dst = a.dwp[which] + ((size_t)(b * ntiles + tile) * 4) * C + h * D;
  for (int i = threadIdx.x; i < 4 * D; i += 128) {
    const int tap = i / D, c = i % D;
    float s = 0.f;
#pragma unroll
    for (int g2 = 0; g2 < kBwdGroups; ++g2) s += red[g2][tap][c];
    dst[(size_t)tap * C + c] = s;
  }
}

// out[j] = sum over rows of part[row][j] in a fixed order: a CTA owns 32 columns, its 8 warps take every 8th row
// (coalesced 128-byte reads, 8 loads in flight per column), then the 8 slices are added in order.  grid ceil(n / 32)
__global__ void __launch_bounds__(256) gdn_block_colsum_kernel(const float* __restrict__ part, int rows, int n,
                                                               float* __restrict__ out) {
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
    out[j] = t;
  }
}

// gate / beta backward: one CTA per head walks all (b, t); the two per-head sums (A_log, dt_bias) in a fixed order
__global__ void __launch_bounds__(256) gdn_block_gate_bwd_kernel(BlockP p, const float* __restrict__ a_raw,
                                                                 const float* __restrict__ b_raw,
                                                                 const float* __restrict__ a_log,
                                                                 const float* __restrict__ dt_bias,
                                                                 const float* __restrict__ dbeta,
                                                                 const float* __restrict__ dgate,
                                                                 float* __restrict__ da_raw, float* __restrict__ db_raw,
                                                                 float* __restrict__ da_log, float* __restrict__ ddt_bias) {
  __shared__ float red[2][8];
  const int h = blockIdx.x, tid = threadIdx.x;
  const float A = expf(a_log[h]), bias = dt_bias[h];
  float s_alog = 0.f, s_bias = 0.f;
  const int n = p.B * p.T;
  for (int i = tid; i < n; i += 256) {
    const size_t idx = (size_t)i * p.H + h;
    const float z = a_raw[idx] + bias;
    const float lg = -softplus_f(z) * A;
    const float dlg = p.gate_is_log ? dgate[idx] : dgate[idx] * expf(lg);
    const float da = -A * dlg * sigmoid_f(z);
    da_raw[idx] = da;
    s_bias += da;
    s_alog = fmaf(dlg, lg, s_alog);  // d lg / d A_log = lg
    const float bt = sigmoid_f(b_raw[idx]);
    db_raw[idx] = dbeta[idx] * bt * (1.f - bt);
  }
  s_alog = warp_sum(s_alog);
  s_bias = warp_sum(s_bias);
  if ((tid & 31) == 0) { red[0][tid >> 5] = s_alog; red[1][tid >> 5] = s_bias; }
  __syncthreads();
  if (tid == 0) {
    float x = 0.f, y = 0.f;
    for (int w = 0; w < 8; ++w) { x += red[0][w]; y += red[1][w]; }
    da_log[h] = x;
    ddt_bias[h] = y;
  }
}

// The same with every (b, t, h) element on its own thread, coalesced, for head counts that divide 256: a thread's
// head is then tid % H for every element it touches.  Per-CTA partial sums [2][G][H] -> fixed-order second pass.
constexpr int kGatePerCta = 256 * 16;
__global__ void __launch_bounds__(256) gdn_block_gate_bwd_flat_kernel(BlockP p, const float* __restrict__ a_raw,
                                                                      const float* __restrict__ b_raw,
                                                                      const float* __restrict__ a_log,
                                                                      const float* __restrict__ dt_bias,
                                                                      const float* __restrict__ dbeta,
                                                                      const float* __restrict__ dgate,
                                                                      float* __restrict__ da_raw,
                                                                      float* __restrict__ db_raw,
                                                                      float* __restrict__ part) {
  __shared__ float red[2][256];
  const int tid = threadIdx.x, h = tid % p.H;
  const float A = expf(a_log[h]), bias = dt_bias[h];
  const size_t n = (size_t)p.B * p.T * p.H, base = (size_t)blockIdx.x * kGatePerCta;
  const size_t end = base + kGatePerCta < n ? base + kGatePerCta : n;
  float s_alog = 0.f, s_bias = 0.f;
  for (size_t idx = base + tid; idx < end; idx += 256) {
    const float z = a_raw[idx] + bias;
    const float lg = -softplus_f(z) * A;
    const float dlg = p.gate_is_log ? dgate[idx] : dgate[idx] * expf(lg);
    const float da = -A * dlg * sigmoid_f(z);
    da_raw[idx] = da;
    s_bias += da;
    s_alog = fmaf(dlg, lg, s_alog);
    const float bt = sigmoid_f(b_raw[idx]);
    db_raw[idx] = dbeta[idx] * bt * (1.f - bt);
  }
  red[0][tid] = s_alog;
  red[1][tid] = s_bias;
  __syncthreads();
  if (tid < p.H) {
    float x = 0.f, y = 0.f;
    for (int j = tid; j < 256; j += p.H) { x += red[0][j]; y += red[1][j]; }
    part[(size_t)blockIdx.x * p.H + tid] = x;
    part[((size_t)gridDim.x + blockIdx.x) * p.H + tid] = y;
  }
}

// ------------------------------------------------------------------ post
// y = o rsqrt(mean(o^2) + 1e-5) o_norm SiLU(z); rows = (b, t, h), D = Dv; 8 rows per CTA pass
template <typename IO>
__global__ void __launch_bounds__(128) gdn_block_post_fwd_kernel(BlockP p, const IO* __restrict__ o,
                                                                 const IO* __restrict__ z,
                                                                 const float* __restrict__ wn, IO* __restrict__ y) {
  const int D = p.Dv, lane16 = threadIdx.x & 15, grp = threadIdx.x >> 4;
  const bool act = lane16 * 8 < D;
  const size_t rows = (size_t)p.B * p.T * p.H;
  float w[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (act) load8<float>(wn + lane16 * 8, w);
  for (size_t row = (size_t)blockIdx.x * kGroups + grp; row < rows; row += (size_t)gridDim.x * kGroups) {
    const size_t off = row * D + lane16 * 8;
    float ov[8], zv[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) ov[c] = zv[c] = 0.f;
    if (act) { load8<IO>(o + off, ov); load8<IO>(z + off, zv); }
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < 8; ++c) ss = fmaf(ov[c], ov[c], ss);
    ss = group_sum(ss);
    const float rn = rsqrtf(ss / (float)D + 1e-5f);
#pragma unroll
    for (int c = 0; c < 8; ++c) ov[c] = ov[c] * rn * w[c] * zv[c] * sigmoid_io<IO>(zv[c]);
    if (act) store8<IO>(y + off, ov);
  }
}

template <typename IO>
__global__ void __launch_bounds__(128) gdn_block_post_bwd_kernel(BlockP p, const IO* __restrict__ o,
                                                                 const IO* __restrict__ z,
                                                                 const float* __restrict__ wn,
                                                                 const IO* __restrict__ dy, IO* __restrict__ d_o,
                                                                 IO* __restrict__ dz, float* __restrict__ dwp) {
  __shared__ float red[kGroups][128];
  const int D = p.Dv, lane16 = threadIdx.x & 15, grp = threadIdx.x >> 4;
  const bool act = lane16 * 8 < D;
  const size_t rows = (size_t)p.B * p.T * p.H;
  float w[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, dw[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (act) load8<float>(wn + lane16 * 8, w);
  for (size_t row = (size_t)blockIdx.x * kGroups + grp; row < rows; row += (size_t)gridDim.x * kGroups) {
    const size_t off = row * D + lane16 * 8;
    float ov[8], zv[8], gv[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) ov[c] = zv[c] = gv[c] = 0.f;
    if (act) { load8<IO>(o + off, ov); load8<IO>(z + off, zv); load8<IO>(dy + off, gv); }
    float ss = 0.f, dot = 0.f, g[8], sz[8], dsz[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      const float sg = sigmoid_io<IO>(zv[c]);
      sz[c] = zv[c] * sg;
      dsz[c] = fmaf(sz[c], 1.f - sg, sg);
      g[c] = gv[c] * sz[c] * w[c];  // gradient at o rn
      ss = fmaf(ov[c], ov[c], ss);
      dot = fmaf(ov[c], g[c], dot);
    }
    ss = group_sum(ss);
    dot = group_sum(dot);
    const float rn = rsqrtf(ss / (float)D + 1e-5f);
    const float k2 = rn * rn * dot / (float)D;
    float dzv[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      const float on = ov[c] * rn;
      dw[c] = fmaf(gv[c] * sz[c], on, dw[c]);
      dzv[c] = gv[c] * w[c] * on * dsz[c];
      g[c] = rn * (g[c] - ov[c] * k2);
    }
    if (act) { store8<IO>(d_o + off, g); store8<IO>(dz + off, dzv); }
  }
#pragma unroll
  for (int c = 0; c < 8; ++c) red[grp][lane16 * 8 + c] = dw[c];
  __syncthreads();
  for (int c = threadIdx.x; c < D; c += 128) {
    float s = 0.f;
#pragma unroll
    for (int g2 = 0; g2 < kGroups; ++g2) s += red[g2][c];
    dwp[(size_t)blockIdx.x * D + c] = s;
  }
}

}  // namespace blk

// ------------------------------------------------------------------ host
using blk::BlockP;

static BlockP make_blk(const mxb_gdn_desc* d) {
  BlockP p{};
  p.B = d->B; p.T = d->T; p.H = d->H; p.Dk = d->Dk; p.Dv = d->Dv; p.gate_is_log = d->gate_is_log;
  return p;
}
bool gdn_block_supported(const mxb_gdn_desc* d) {
  return d->Dk % 8 == 0 && d->Dv % 8 == 0 && d->Dk <= 128 && d->Dv <= 128 && d->Dk > 0 && d->Dv > 0;
}
static int blk_tiles(const mxb_gdn_desc* d) { return (d->T + blk::kTile - 1) / blk::kTile; }
static int blk_bwd_tiles(const mxb_gdn_desc* d) { return (d->T + blk::kBwdTile - 1) / blk::kBwdTile; }
static int blk_post_ctas(const mxb_gdn_desc* d) {
  const size_t rows = (size_t)d->B * d->T * d->H;
  const size_t want = (rows + blk::kGroups - 1) / blk::kGroups;
  return (int)(want < 148 * 16 ? want : 148 * 16);
}
static int blk_gate_ctas(const mxb_gdn_desc* d) {
  const size_t n = (size_t)d->B * d->T * d->H;
  return (int)((n + blk::kGatePerCta - 1) / blk::kGatePerCta);
}
// backward partial rows: conv weights of q, k, v and the per-head gate sums; or the norm weight
size_t gdn_block_workspace_bytes(const mxb_gdn_desc* d) {
  const size_t rows = (size_t)d->B * blk_bwd_tiles(d);
  const size_t pre = rows * 4 * ((size_t)2 * d->H * d->Dk + (size_t)d->H * d->Dv) * sizeof(float);
  const size_t post = (size_t)blk_post_ctas(d) * d->Dv * sizeof(float);
  const size_t gate = 2 * (size_t)blk_gate_ctas(d) * d->H * sizeof(float);
  return (pre + gate > post ? pre + gate : post) + 256;
}

template <typename IO>
static mxb_status blk_pre_fwd(const mxb_gdn_desc* d, const void* qp, const void* kp, const void* vp, const float* cq,
                              const float* ck, const float* cv, const float* a_raw, const float* b_raw,
                              const float* a_log, const float* dt_bias, void* q, void* k, void* v, float* beta,
                              float* gate, cudaStream_t st) {
  BlockP p = make_blk(d);
  blk::PreArgs<IO> a{};
  a.x[0] = static_cast<const IO*>(qp); a.x[1] = static_cast<const IO*>(kp); a.x[2] = static_cast<const IO*>(vp);
  a.w[0] = cq; a.w[1] = ck; a.w[2] = cv;
  a.y[0] = static_cast<IO*>(q); a.y[1] = static_cast<IO*>(k); a.y[2] = static_cast<IO*>(v);
  const int nt = blk_tiles(d);
  MXB_LAUNCH("gdn_block_pre_fwd_kernel", st,
             (blk::gdn_block_pre_fwd_kernel<IO><<<dim3(3 * nt, d->H, d->B), 128, 0, st>>>(p, a, nt)));
  const size_t n = (size_t)d->B * d->T * d->H;
  const int gb = (int)((n + 255) / 256 < 148 * 8 ? (n + 255) / 256 : 148 * 8);
  MXB_LAUNCH("gdn_block_gate_fwd_kernel", st,
             (blk::gdn_block_gate_fwd_kernel<<<gb, 256, 0, st>>>(p, a_raw, b_raw, a_log, dt_bias, beta, gate)));
  return check_launch("gdn_block_pre_fwd");
}
mxb_status gdn_block_pre_fwd(const mxb_gdn_desc* d, const void* qp, const void* kp, const void* vp, const float* cq,
                             const float* ck, const float* cv, const float* a_raw, const float* b_raw,
                             const float* a_log, const float* dt_bias, void* q, void* k, void* v, float* beta,
                             float* gate, cudaStream_t st) {
  return d->io_dtype == MXB_F32
             ? blk_pre_fwd<float>(d, qp, kp, vp, cq, ck, cv, a_raw, b_raw, a_log, dt_bias, q, k, v, beta, gate, st)
             : blk_pre_fwd<blk::bf16>(d, qp, kp, vp, cq, ck, cv, a_raw, b_raw, a_log, dt_bias, q, k, v, beta, gate, st);
}

template <typename IO>
static mxb_status blk_pre_bwd(const mxb_gdn_desc* d, const void* qp, const void* kp, const void* vp, const float* cq,
                              const float* ck, const float* cv, const float* a_raw, const float* b_raw,
                              const float* a_log, const float* dt_bias, const void* dq, const void* dk, const void* dv,
                              const float* dbeta, const float* dgate, void* dqp, void* dkp, void* dvp, float* dcq,
                              float* dck, float* dcv, float* da_raw, float* db_raw, float* da_log, float* ddt_bias,
                              void* ws, cudaStream_t st) {
  BlockP p = make_blk(d);
  blk::PreArgs<IO> a{};
  a.x[0] = static_cast<const IO*>(qp); a.x[1] = static_cast<const IO*>(kp); a.x[2] = static_cast<const IO*>(vp);
  a.w[0] = cq; a.w[1] = ck; a.w[2] = cv;
  a.dy[0] = static_cast<const IO*>(dq); a.dy[1] = static_cast<const IO*>(dk); a.dy[2] = static_cast<const IO*>(dv);
  a.dx[0] = static_cast<IO*>(dqp); a.dx[1] = static_cast<IO*>(dkp); a.dx[2] = static_cast<IO*>(dvp);
  const int nt = blk_bwd_tiles(d);
  const size_t rows = (size_t)d->B * nt, Ck = (size_t)d->H * d->Dk, Cv = (size_t)d->H * d->Dv;
  float* base = reinterpret_cast<float*>(static_cast<char*>(ws) + 256);
  a.dwp[0] = base; a.dwp[1] = base + rows * 4 * Ck; a.dwp[2] = base + rows * 8 * Ck;
  MXB_LAUNCH("gdn_block_pre_bwd_kernel", st,
             (blk::gdn_block_pre_bwd_kernel<IO><<<dim3(3 * nt, d->H, d->B), 128, 0, st>>>(p, a, nt)));
  float* outs[3] = {dcq, dck, dcv};
  for (int w = 0; w < 3; ++w) {
    const int n = (int)(4 * (w == 2 ? Cv : Ck));
    MXB_LAUNCH("gdn_block_colsum_kernel", st,
               (blk::gdn_block_colsum_kernel<<<(n + 31) / 32, 256, 0, st>>>(a.dwp[w], (int)rows, n, outs[w])));
  }
  if (256 % d->H == 0) {
    const int gc = blk_gate_ctas(d);
    float* gpart = base + rows * 4 * (2 * Ck + Cv);
    MXB_LAUNCH("gdn_block_gate_bwd_flat_kernel", st,
               (blk::gdn_block_gate_bwd_flat_kernel<<<gc, 256, 0, st>>>(p, a_raw, b_raw, a_log, dt_bias, dbeta, dgate,
                                                                       da_raw, db_raw, gpart)));
    MXB_LAUNCH("gdn_block_colsum_kernel", st,
               (blk::gdn_block_colsum_kernel<<<(d->H + 31) / 32, 256, 0, st>>>(gpart, gc, d->H, da_log)));
    MXB_LAUNCH("gdn_block_colsum_kernel", st,
               (blk::gdn_block_colsum_kernel<<<(d->H + 31) / 32, 256, 0, st>>>(gpart + (size_t)gc * d->H, gc, d->H,
                                                                                 ddt_bias)));
  } else {
    MXB_LAUNCH("gdn_block_gate_bwd_kernel", st,
               (blk::gdn_block_gate_bwd_kernel<<<d->H, 256, 0, st>>>(p, a_raw, b_raw, a_log, dt_bias, dbeta, dgate,
                                                                      da_raw, db_raw, da_log, ddt_bias)));
  }
  return check_launch("gdn_block_pre_bwd");
}
mxb_status gdn_block_pre_bwd(const mxb_gdn_desc* d, const void* qp, const void* kp, const void* vp, const float* cq,
                             const float* ck, const float* cv, const float* a_raw, const float* b_raw,
                             const float* a_log, const float* dt_bias, const void* dq, const void* dk, const void* dv,
                             const float* dbeta, const float* dgate, void* dqp, void* dkp, void* dvp, float* dcq,
                             float* dck, float* dcv, float* da_raw, float* db_raw, float* da_log, float* ddt_bias,
                             void* ws, cudaStream_t st) {
  return d->io_dtype == MXB_F32
             ? blk_pre_bwd<float>(d, qp, kp, vp, cq, ck, cv, a_raw, b_raw, a_log, dt_bias, dq, dk, dv, dbeta, dgate, dqp,
                                  dkp, dvp, dcq, dck, dcv, da_raw, db_raw, da_log, ddt_bias, ws, st)
             : blk_pre_bwd<blk::bf16>(d, qp, kp, vp, cq, ck, cv, a_raw, b_raw, a_log, dt_bias, dq, dk, dv, dbeta, dgate,
                                      dqp, dkp, dvp, dcq, dck, dcv, da_raw, db_raw, da_log, ddt_bias, ws, st);
}

template <typename IO>
static mxb_status blk_post(const mxb_gdn_desc* d, const void* o, const void* z, const float* wn, void* y,
                           const void* dy, void* d_o, void* dz, float* dwn, void* ws, cudaStream_t st) {
  BlockP p = make_blk(d);
  const int ctas = blk_post_ctas(d);
  if (!dy) {
    MXB_LAUNCH("gdn_block_post_fwd_kernel", st,
               (blk::gdn_block_post_fwd_kernel<IO><<<ctas, 128, 0, st>>>(p, static_cast<const IO*>(o),
                                                                         static_cast<const IO*>(z), wn,
                                                                         static_cast<IO*>(y))));
    return check_launch("gdn_block_post_fwd");
  }
  float* part = reinterpret_cast<float*>(static_cast<char*>(ws) + 256);
  MXB_LAUNCH("gdn_block_post_bwd_kernel", st,
             (blk::gdn_block_post_bwd_kernel<IO><<<ctas, 128, 0, st>>>(p, static_cast<const IO*>(o),
                                                                       static_cast<const IO*>(z), wn,
                                                                       static_cast<const IO*>(dy), static_cast<IO*>(d_o),
                                                                       static_cast<IO*>(dz), part)));
  MXB_LAUNCH("gdn_block_colsum_kernel", st,
             (blk::gdn_block_colsum_kernel<<<(d->Dv + 31) / 32, 256, 0, st>>>(part, ctas, d->Dv, dwn)));
  return check_launch("gdn_block_post_bwd");
}
mxb_status gdn_block_post(const mxb_gdn_desc* d, const void* o, const void* z, const float* wn, void* y, const void* dy,
                          void* d_o, void* dz, float* dwn, void* ws, cudaStream_t st) {
  return d->io_dtype == MXB_F32 ? blk_post<float>(d, o, z, wn, y, dy, d_o, dz, dwn, ws, st)
                                : blk_post<blk::bf16>(d, o, z, wn, y, dy, d_o, dz, dwn, ws, st);
}

}  // namespace mxb
