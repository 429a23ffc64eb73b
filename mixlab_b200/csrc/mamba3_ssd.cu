// Mamba-3 selective scan in chunked dual ("SSD") form on tensor cores - head-broadcast
// layout (dt, lambda, theta per (b,t,head), A per head), head dim 64, d_state 128, bf16 I/O.
//
// With scalar decay per (step, head) the exponential-trapezoidal recurrence
//     h_t = alpha_t h_{t-1} + gamma_t Brot_t x_t^T + beta_t Brot_{t-1} x_{t-1}^T ,  y_t = Crot_t^T h_t
// (reference: gpu/cuda_kernels/mamba3_selective_scan_fwd_v2_emit.cu:65-115) has the closed form
//     y_t = sum_{s<=t} (Crot_t . Brot_s) exp(Lam_t - Lam_s) w_ts x_s ,   Lam = cumsum(dt A),
//     w_ts = e_s = gamma_s + (1-lambda_{s+1}) dt_{s+1}  for s < t,   w_tt = gamma_t,
// because beta_{s+1} exp(Lam_t - Lam_{s+1}) = (1-lambda_{s+1}) dt_{s+1} exp(Lam_t - Lam_s).  Per chunk of
// 64 steps (M_ts = exp(Lam_t-Lam_s) w_ts [s<=t], r_s = exp(Lam_end - Lam_s), L = exp(Lam_end)):
//     Y  = (Crot Brot^T * M) X + diag(exp(Lam)) Crot H0          H1 = L H0 + Brot^T diag(r e) X
// so the only sequential part is the elementwise chunk scan H1 = L H0 + Hc.  The backward is the
// hand-derived adjoint of these two lines (checked against float64 autograd of the recurrence
// before it was written); its sequential part is the mirrored scan dH0 = L dH1 + Dc.
//
//   m3s_scalars_kernel      per (b, head): dt, lambda, wrapped cumulative angle (fp64 prefix sum)
//   m3s_chunk_scalars_kernel per chunk: decay sums, trapezoid weights, rotation sines/cosines (one record)
//   m3s_state_pass_kernel   per (b, head), sequential over the chunks, forward or reverse: the chunk contribution
//                           Brot^T diag(r e) X (or Crot^T diag(exp(Lam)) dY) folded into the running state
//   m3s_chunk_out_kernel    per chunk: Y
//   m3s_chunk_grad_kernel   per chunk: dx, rotated-row gradients -> dB, dC partials, per-token scalars
//   m3s_final_kernel        per (b, head): suffix sum of the angle gradient, ddt, dlambda, dtheta, da_log
#include <cuda.h>

#include <cstring>

#include "common.cuh"
#include "umma_tiles.cuh"

namespace mxb {
namespace m3s {

constexpr int Q = 64;    // chunk
constexpr int P = 64;    // head dim
constexpr int N = 128;   // d_state
using bf16 = __nv_bfloat16;

struct SsdP {
  int B, T, D, G, NH, n;   // n = chunks
  int no_tma;              // stage operands with cp.async even where tensor maps can be made
  const bf16 *x, *b, *c, *dy;
  const float *dt_raw, *lam_raw, *theta, *a_log;
  bf16 *y, *dx;
  float *ddt, *dlam, *dtheta, *da_log;
  int* status;
  // workspace
  float *dt, *lam, *phi;        // [B,NH,T]
  bf16 *H0, *dH1;               // [B,NH,n,N,P] state at chunk start / state gradient at chunk end
  float *dphi, *da, *de, *dgam; // [B,NH,T] per-token scalar gradients
  float* dal_part;              // [B,NH] per-batch shares of da_log
  float* cs;                    // [B,NH,n] ChunkScal records
  bf16 *pb, *pc;                // [B,NH,T,N] per-head partial dB, dC (summed in fp32 by the reduce kernel)
};

__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : (x < -20.f ? expf(x) : log1pf(expf(x))); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + expf(-x)); }
__device__ __forceinline__ uint4 ldg16(const void* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }
__device__ __forceinline__ void sts16(uint8_t* base, uint32_t off, uint4 v) { *reinterpret_cast<uint4*>(base + off) = v; }
__device__ __forceinline__ void unpack8(uint4 v, float (&e)[8]) {
  tc::unpack_bf16(v.x, e[0], e[1]); tc::unpack_bf16(v.y, e[2], e[3]);
  tc::unpack_bf16(v.z, e[4], e[5]); tc::unpack_bf16(v.w, e[6], e[7]);
}
__device__ __forceinline__ uint4 pack8(const float* e) {
  return make_uint4(tc::pack_bf16(e[0], e[1]), tc::pack_bf16(e[2], e[3]), tc::pack_bf16(e[4], e[5]),
                    tc::pack_bf16(e[6], e[7]));
}
__device__ __forceinline__ void ld_acc32(uint32_t taddr, int warp, int c0, float (&f)[32]) {
  uint32_t r[32];
  tc::tmem_ld_32x32b_x32(taddr + ((uint32_t)(32 * (warp & 3)) << 16) + (uint32_t)c0, r);
  tc::tmem_ld_wait();
#pragma unroll
  for (int i = 0; i < 32; ++i) f[i] = __uint_as_float(r[i]);
}

__device__ __forceinline__ void ld_acc16(uint32_t taddr, int warp, int c0, float (&f)[16]) {
  uint32_t r[16];
  tc::tmem_ld_32x32b_x16(taddr + ((uint32_t)(32 * (warp & 3)) << 16) + (uint32_t)c0, r);
  tc::tmem_ld_wait();
#pragma unroll
  for (int i = 0; i < 16; ++i) f[i] = __uint_as_float(r[i]);
}

// Per-chunk scalars: computed once per (batch, head, chunk) by m3s_chunk_scalars_kernel into a workspace record
// and fetched by every chunk kernel with its operand tiles (the record is a whole number of 16-byte units).
struct ChunkScal {
  float Lam[Q];   // in-chunk inclusive cumulative sum of dt A
  float gam[Q];   // lambda dt
  float e[Q];     // gam_s + (1 - lambda_{s+1}) dt_{s+1}
  float sn[Q], cs[Q];  // sine / cosine of the cumulative rotation angle
  float dexp[Q];  // exp(Lam)
  float r[Q];     // exp(Lam_last - Lam)
  float re[Q];    // r e
  float L, A, pad[2];
};
static_assert(sizeof(ChunkScal) % 16 == 0, "record moves in 16-byte units");
constexpr int kScalUnits = sizeof(ChunkScal) / 16;

__global__ void __launch_bounds__(64) m3s_chunk_scalars_kernel(SsdP p) {
  __shared__ __align__(16) ChunkScal s;
  __shared__ float sdt[Q];
  const int tid = threadIdx.x, c = blockIdx.x, head = blockIdx.y, b = blockIdx.z, t0 = c * Q;
  const size_t base = ((size_t)b * p.NH + head) * p.T;
  const size_t ci = ((size_t)b * p.NH + head) * p.n + c;
  const float A = -expf(p.a_log[head]);
  {
    const int t = t0 + tid;
    const bool ok = t < p.T;
    const float dt = ok ? p.dt[base + t] : 0.f, lam = ok ? p.lam[base + t] : 0.f;
    const float nxt = (t + 1 < p.T) ? (1.f - p.lam[base + t + 1]) * p.dt[base + t + 1] : 0.f;
    sdt[tid] = dt;
    s.gam[tid] = lam * dt;
    s.e[tid] = lam * dt + nxt;
    float sn = 0.f, cs = 1.f;
    if (ok) sincosf(p.phi[base + t], &sn, &cs);
    s.sn[tid] = sn; s.cs[tid] = cs;
  }
  __syncthreads();
  if (tid < 32) {  // inclusive in-chunk cumulative sum of a = dt A, two per lane
    const float a0 = sdt[2 * tid] * A, a1 = sdt[2 * tid + 1] * A;
    float v = a0 + a1;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float t = __shfl_up_sync(0xffffffffu, v, o);
      if (tid >= o) v += t;
    }
    s.Lam[2 * tid] = v - a1;
    s.Lam[2 * tid + 1] = v;
  }
  __syncthreads();
  {
    const float last = s.Lam[Q - 1];
    const float r = __expf(last - s.Lam[tid]);
    s.dexp[tid] = __expf(s.Lam[tid]);
    s.r[tid] = r;
    s.re[tid] = r * s.e[tid];
    if (tid == 0) { s.L = __expf(last); s.A = A; s.pad[0] = s.pad[1] = 0.f; }
  }
  __syncthreads();
  uint4* dst = reinterpret_cast<uint4*>(p.cs + ci * (sizeof(ChunkScal) / 4));
  for (int u = tid; u < kScalUnits; u += 64) dst[u] = reinterpret_cast<const uint4*>(&s)[u];
}
// cp.async of the record of chunk ci into shared memory (part of the caller's current cp.async group)
__device__ __forceinline__ void issue_chunk_scalars(const SsdP& p, size_t ci, ChunkScal& s) {
  const uint32_t sd = tc::smem_u32(&s);
  const float* src = p.cs + ci * (sizeof(ChunkScal) / 4);
  for (int u = threadIdx.x; u < kScalUnits; u += blockDim.x) tc::cp_async16(sd + 16 * u, src + 4 * u);
}

// ---- asynchronous staging: raw cp.async copies into the blocked layout, then in-place fix-ups ----
// With t = 8 (u / 128) + u % 8 and c8 = (u / 8) % 16 the unit of a [64][128] tile sits at byte 16 u, and
// likewise for [.][64] tiles with t = 8 (u / 64) + u % 8, c8 = (u / 8) % 8: eight consecutive lanes fill one
// 128-byte row group (no bank conflicts) and read 64-byte pieces of a row.
__device__ __forceinline__ void issue_rows_tile(uint8_t* dst, const bf16* src, const SsdP& p, int b, int g, int t0) {
  const uint32_t sd = tc::smem_u32(dst);
  for (int u = threadIdx.x; u < Q * 16; u += blockDim.x) {
    const int t = ((u >> 7) << 3) | (u & 7), c8 = (u >> 3) & 15;
    const bool ok = t0 + t < p.T;
    tc::cp_async16(sd + 16 * u, ok ? src + (((size_t)b * p.T + t0 + t) * p.G + g) * N + c8 * 8 : src, ok);
  }
}
__device__ __forceinline__ void issue_x_tile(uint8_t* dst, const bf16* src, const SsdP& p, int b, int d0, int t0) {
  const uint32_t sd = tc::smem_u32(dst);
  for (int u = threadIdx.x; u < Q * 8; u += blockDim.x) {
    const int t = ((u >> 6) << 3) | (u & 7), c8 = (u >> 3) & 7;
    const bool ok = t0 + t < p.T;
    tc::cp_async16(sd + 16 * u, ok ? src + ((size_t)b * p.T + t0 + t) * p.D + d0 + c8 * 8 : src, ok);
  }
}
// [128 n][64 p] bf16 state saved by the state pass as the byte image of the blocked tile
__device__ __forceinline__ void issue_state_tile(uint8_t* dst, const bf16* src) {
  const uint32_t sd = tc::smem_u32(dst);
  for (int u = threadIdx.x; u < N * 8; u += blockDim.x) tc::cp_async16(sd + 16 * u, src + 8 * u);
}
// Rotates the (even, odd) pairs of every row of a landed [64][128] tile in place.
__device__ __forceinline__ void rotate_tile(uint8_t* tile, const float* sn, const float* cs) {
  for (int u = threadIdx.x; u < Q * 16; u += blockDim.x) {
    const int t = ((u >> 7) << 3) | (u & 7);
    float e[8];
    unpack8(*reinterpret_cast<const uint4*>(tile + 16 * u), e);
    const float s_ = sn[t], c_ = cs[t];
#pragma unroll
    for (int k = 0; k < 8; k += 2) {
      const float ev = e[k], od = e[k + 1];
      e[k] = c_ * ev + s_ * od;
      e[k + 1] = -s_ * ev + c_ * od;
    }
    *reinterpret_cast<uint4*>(tile + 16 * u) = pack8(e);
  }
}
// dst = diag(rowscale) src for [64][64] tiles (dst may be src).
__device__ __forceinline__ void scale_x_tile(uint8_t* dst, const uint8_t* src, const float* rowscale) {
  for (int u = threadIdx.x; u < Q * 8; u += blockDim.x) {
    const int t = ((u >> 6) << 3) | (u & 7);
    *reinterpret_cast<uint4*>(dst + 16 * u) =
        tc::scale_bf16x8(*reinterpret_cast<const uint4*>(src + 16 * u), rowscale[t]);
  }
}

// ---- the same fix-ups and views for tiles that the copy engine wrote with 128-byte swizzle (SW = true) ----
template <bool SW>
__device__ __forceinline__ uint32_t in_unit(int t, int c8, int W) {
  return SW ? tc::sw128_unit(t, c8) : tc::kmajor_unit(t, c8, W);
}
template <bool SW>
__device__ __forceinline__ tc::Tile in_kmajor(const void* ptr, int W) {
  return SW ? tc::kmajor_sw128_tile(ptr, 8192) : tc::kmajor_tile(ptr, W);
}
template <bool SW>
__device__ __forceinline__ tc::Tile in_mnmajor(const void* ptr, int W) {
  return SW ? tc::mnmajor_sw128_tile(ptr, 8192) : tc::mnmajor_tile(ptr, W);
}
template <bool SW>
__device__ __forceinline__ void rotate_in_tile(uint8_t* tile, const float* sn, const float* cs) {
  if (!SW) { rotate_tile(tile, sn, cs); return; }
  // four units per pass, all loads before the first store (a store in between would pin the order of the
  // loads that follow it); unit w of a slab belongs to row w / 8
  const int nt = blockDim.x;
  for (int w0 = threadIdx.x; w0 < Q * 16; w0 += 4 * nt) {
    uint4 raw[4];
    float sv[4], cv[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int w = w0 + q * nt, t = (w >> 3) & 63;
      raw[q] = *reinterpret_cast<const uint4*>(tile + 16 * w);
      sv[q] = sn[t]; cv[q] = cs[t];
    }
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      float e[8];
      unpack8(raw[q], e);
#pragma unroll
      for (int k = 0; k < 8; k += 2) {
        const float ev = e[k], od = e[k + 1];
        e[k] = cv[q] * ev + sv[q] * od;
        e[k + 1] = -sv[q] * ev + cv[q] * od;
      }
      raw[q] = pack8(e);
    }
#pragma unroll
    for (int q = 0; q < 4; ++q) *reinterpret_cast<uint4*>(tile + 16 * (w0 + q * nt)) = raw[q];
  }
}
template <bool SW>
__device__ __forceinline__ void scale_in_tile(uint8_t* dst, const uint8_t* src, const float* rowscale) {
  if (!SW) { scale_x_tile(dst, src, rowscale); return; }
  for (int w = threadIdx.x; w < Q * 8; w += blockDim.x)
    *reinterpret_cast<uint4*>(dst + 16 * w) =
        tc::scale_bf16x8(*reinterpret_cast<const uint4*>(src + 16 * w), rowscale[w >> 3]);
}
struct ChunkMaps {
  CUtensorMap b, c;   // [B,T,G,128] viewed as (N, G, T, B), boxes of 64 columns x 64 steps, 128-byte swizzle
  CUtensorMap x, dy;  // [B,T,heads,64] viewed as (P, heads, T, B)
};

// Threads of the two per-(batch, head) scalar kernels: they are chains of dependent fp64 operations behind strided
// loads, so many short chains (4 steps per thread at T = 4096) hide the latencies that few long ones expose.
constexpr int kScalThreads = 1024;
// Inclusive prefix sum of one double per thread over a kScalThreads-thread CTA (warp scans + the warp totals, a fixed
// order); wtot is kScalThreads / 32 doubles of shared memory.  Also returns the CTA total.
__device__ __forceinline__ double cta_scan(double v, double* wtot, double& total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const double t = __shfl_up_sync(0xffffffffu, v, o);
    if (lane >= o) v += t;
  }
  if (lane == 31) wtot[warp] = v;
  __syncthreads();
  double off = 0.0, tot = 0.0;
#pragma unroll
  for (int w = 0; w < kScalThreads / 32; ++w) {
    const double x = wtot[w];
    if (w < warp) off += x;
    tot += x;
  }
  total = tot;
  return v + off;
}

// ------------------------------------------------------------ per-(b,head) scalars
constexpr int kScalBatch = 4;
__global__ void __launch_bounds__(kScalThreads) m3s_scalars_kernel(SsdP p) {
  __shared__ double wtot[kScalThreads / 32];
  const int head = blockIdx.x, b = blockIdx.y, tid = threadIdx.x;
  const size_t base = ((size_t)b * p.NH + head) * p.T;
  const int per = (p.T + kScalThreads - 1) / kScalThreads, lo = tid * per, hi = min(p.T, lo + per);
  // Batches of kScalBatch steps: all loads of a batch are issued before its first store (a store in between would
  // pin the order, since the compiler cannot prove the arrays distinct, and every step would pay a full memory latency).
  double acc = 0.0;
  for (int t0 = lo; t0 < hi; t0 += kScalBatch) {
    float draw[kScalBatch], lraw[kScalBatch], th[kScalBatch];
#pragma unroll
    for (int x = 0; x < kScalBatch; ++x) {
      const int t = min(t0 + x, hi - 1);
      const size_t r = ((size_t)b * p.T + t) * p.NH + head;
      draw[x] = __ldg(p.dt_raw + r);
      lraw[x] = __ldg(p.lam_raw + r);
      th[x] = __ldg(p.theta + r);
    }
#pragma unroll
    for (int x = 0; x < kScalBatch; ++x) {
      if (t0 + x < hi) {
        const float dt = softplus_f(draw[x]);
        p.dt[base + t0 + x] = dt;
        p.lam[base + t0 + x] = sigmoid_f(lraw[x]);
        acc += (double)dt * (double)th[x];
      }
    }
  }
  double total;
  double phi = cta_scan(acc, wtot, total) - acc;  // angle at the start of this thread's steps
  const double two_pi = 6.283185307179586476925, inv_two_pi = 1.0 / two_pi;
  for (int t0 = lo; t0 < hi; t0 += kScalBatch) {
    float dtv[kScalBatch], th[kScalBatch];
#pragma unroll
    for (int x = 0; x < kScalBatch; ++x) {
      const int t = min(t0 + x, hi - 1);
      dtv[x] = p.dt[base + t];
      th[x] = __ldg(p.theta + ((size_t)b * p.T + t) * p.NH + head);
    }
#pragma unroll
    for (int x = 0; x < kScalBatch; ++x) {
      if (t0 + x < hi) {
        phi += (double)dtv[x] * (double)th[x];
        p.phi[base + t0 + x] = (float)(phi - two_pi * rint(phi * inv_two_pi));  // wrapped to [-pi, pi]
      }
    }
  }
}

// ------------------------------------------------------------ state pass
// One CTA per (batch, head) walks the chunks in order (mode 0) or in reverse (mode 1) and keeps the running
// state in registers (thread = state row n and 32 of its 64 fp32 columns):
//   mode 0: H0_c = H;  H = L_c H + Brot_c^T diag(r e) X_c          (states at chunk start, for y and the backward)
//   mode 1: dH1_c = dH; dH = L_c dH + Crot_c^T diag(exp(Lam)) dY_c  (state gradients at chunk end)
// The chunk contribution is one M=128 tcgen05 tile that never leaves the SM; the operands of the next chunks are
// in flight in a ring of kPassStages buffers (a chunk takes ~1.5 us here and a copy up to ~2 us, so with two
// buffers every chunk waited ~0.9 k cycles for its tiles) while the current one is rotated, multiplied and folded
// in.  The saved state leaves as the byte image of the [128][64] operand tile (one bulk copy per chunk).
constexpr int kPassStages = 3;
constexpr int kPassStoreThread = 64;   // issues the state-image stores (its own bulk-group queue)
constexpr int kPassSmem = kPassStages * (16384 + 8192) + kPassStages * sizeof(ChunkScal) + 2 * 16384 + 64 + 1024;

struct PassMaps {
  CUtensorMap r;  // b or c: [B,T,G,128] viewed as (N, G, T, B), boxes of 64 columns x 64 steps, 128-byte swizzle
  CUtensorMap x;  // x or dy: [B,T,heads,64] viewed as (P, heads, T, B)
};

// TMA = true: the three operand boxes of a chunk and its scalar record arrive by the copy engine on one mbarrier
// per buffer (tiles in the 128-byte-swizzled layout); TMA = false: cp.async staging into the un-swizzled layout.
template <bool TMA>
__global__ void __launch_bounds__(256) m3s_state_pass_kernel(SsdP p, int mode, const __grid_constant__ PassMaps maps) {
  extern __shared__ uint8_t raw[];
  uint8_t* sm = raw + ((1024u - (tc::smem_u32(raw) & 1023u)) & 1023u);
  uint8_t* Himg = sm + kPassStages * (16384 + 8192);  // 2 x [128 n][64 p] bf16 images of the state on their way out
  uint8_t* scal = Himg + 2 * 16384;
  uint64_t* mbar = reinterpret_cast<uint64_t*>(scal + kPassStages * sizeof(ChunkScal));  // [0] MMA, [1 + stage] stage full
  uint32_t* tslot = reinterpret_cast<uint32_t*>(mbar + 1 + kPassStages);
  const int tid = threadIdx.x, warp = tid >> 5;
  const int nrow = tid & 127, half = tid >> 7;  // thread = state row n, 32 of its 64 columns
  const int head = blockIdx.x, b = blockIdx.y;
  const int d0 = head * P, g = d0 / (p.D / p.G);
  const size_t cbase = ((size_t)b * p.NH + head) * p.n;
  auto Rt = [&](int buf) { return sm + buf * 16384; };             // [64 s][128 n] B or C rows, rotated in place
  auto Xt = [&](int buf) { return sm + kPassStages * 16384 + buf * 8192; };  // [64 s][64 p]  x or dy, scaled in place
  auto Sc = [&](int buf) -> ChunkScal& { return *reinterpret_cast<ChunkScal*>(scal + buf * sizeof(ChunkScal)); };
  auto chunk_at = [&](int it) { return mode == 0 ? it : p.n - 1 - it; };
  auto issue = [&](int it) {
    if (it < p.n) {
      const int c = chunk_at(it), buf = it % kPassStages;
      if (TMA) {
        // two threads of two other warps than the one that issues the MMAs share the copies; the barrier's single
        // arrival is the expect_tx, so the phase cannot complete before every byte announced there has landed
        if (tid == 32) {
          tc::mbar_expect_tx(&mbar[1 + buf], 16384 + 8192 + (uint32_t)sizeof(ChunkScal));
          tc::tma_load_4d(tc::smem_u32(Rt(buf)), &maps.r, 0, g, c * Q, b, &mbar[1 + buf]);
          tc::tma_load_4d(tc::smem_u32(Rt(buf)) + 8192, &maps.r, 64, g, c * Q, b, &mbar[1 + buf]);
        }
        if (tid == 96) {
          tc::tma_load_4d(tc::smem_u32(Xt(buf)), &maps.x, 0, head, c * Q, b, &mbar[1 + buf]);
          tc::bulk_load(tc::smem_u32(&Sc(buf)), p.cs + (cbase + c) * (sizeof(ChunkScal) / 4), (uint32_t)sizeof(ChunkScal),
                        &mbar[1 + buf]);
        }
      } else {
        issue_rows_tile(Rt(buf), mode == 0 ? p.b : p.c, p, b, g, c * Q);
        issue_x_tile(Xt(buf), mode == 0 ? p.x : p.dy, p, b, d0, c * Q);
        issue_chunk_scalars(p, cbase + c, Sc(buf));
      }
    }
    if (!TMA) tc::cp_async_commit();
  };
  // rows of the landed tiles: rotate B/C pairs, scale x/dy (16-byte units; a unit never straddles a pair)
  auto fix_tiles = [&](int buf) {
    const ChunkScal& s = Sc(buf);
    const float* rowscale = mode == 0 ? s.re : s.dexp;
    if (TMA) {  // swizzled slabs of [64 rows][128 bytes]: unit w of a slab belongs to row w / 8
      rotate_in_tile<true>(Rt(buf), s.sn, s.cs);
      {  // both units of this thread: loads first, then the stores
        const uint4 a = *reinterpret_cast<const uint4*>(Xt(buf) + 16 * tid);
        const uint4 c2 = *reinterpret_cast<const uint4*>(Xt(buf) + 16 * (tid + 256));
        const float ra = rowscale[tid >> 3], rc = rowscale[(tid + 256) >> 3];
        *reinterpret_cast<uint4*>(Xt(buf) + 16 * tid) = tc::scale_bf16x8(a, ra);
        *reinterpret_cast<uint4*>(Xt(buf) + 16 * (tid + 256)) = tc::scale_bf16x8(c2, rc);
      }
    } else {
      rotate_tile(Rt(buf), s.sn, s.cs);
      scale_x_tile(Xt(buf), Xt(buf), rowscale);
    }
  };
  if (warp == 0) { tc::tmem_alloc(tslot, 64); tc::tmem_relinquish(); }
  if (tid == 0) {
    for (int m = 0; m < 1 + kPassStages; ++m) tc::mbar_init(&mbar[m], 1);
    tc::mbar_fence_init();
  }
  __syncthreads();  // barriers initialised before the copies can complete on them
  for (int it = 0; it < kPassStages; ++it) issue(it);
  float H[32];
#pragma unroll
  for (int x = 0; x < 32; ++x) H[x] = 0.f;
  bool ok = true;
  if (TMA) ok = tc::mbar_wait(&mbar[1], 0);
  else tc::cp_async_wait<kPassStages - 1>();  // operands of the first chunk
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t taddr = *tslot;
  bf16* out = mode == 0 ? p.H0 : p.dH1;
  uint32_t ph = 0;
  fix_tiles(0);
  for (int it = 0; it < p.n; ++it) {
    const int c = chunk_at(it), buf = it % kPassStages, nbuf = (it + 1) % kPassStages;
    const float L = Sc(buf).L;
    uint8_t* Hi = Himg + (it & 1) * 16384;  // the image written two chunks ago has left this tile (checked below)
#pragma unroll
    for (int x = 0; x < 4; ++x) sts16(Hi, tc::kmajor_unit(nrow, 4 * half + x, P), pack8(&H[8 * x]));
    tc::fence_async_smem();
    tc::fence_before_sync();
    // tiles of this chunk rotated and scaled (during the previous chunk's MMA), image staged
    ok = __syncthreads_and(ok);  // the barrier also makes the verdict of the bounded waits uniform, so that all
    if (!ok) break;              // threads leave the loop together
    tc::fence_after_sync();
    if (tid == 0) {  // [128 n x 64 p] = R^T X, both contracted over their rows
      if (TMA)
        tc::issue_gemm(taddr, tc::mnmajor_sw128_tile(Rt(buf), 8192), tc::mnmajor_sw128_tile(Xt(buf), 8192), 128, P, Q, false);
      else
        tc::issue_gemm(taddr, tc::mnmajor_tile(Rt(buf), N), tc::mnmajor_tile(Xt(buf), P), 128, P, Q, false);
      tc::mma_commit(mbar);
    }
    if (tid == kPassStoreThread) {  // the state image leaves from another warp than the one issuing the MMAs
      tc::bulk_store(out + (cbase + c) * (N * P), tc::smem_u32(Hi), 16384);
      tc::bulk_commit();
      tc::bulk_wait_read<1>();  // all but the copy just issued have been read out of shared memory
    }
    if (it + 1 < p.n) {  // while the tensor core works: the next chunk's tiles
      if (TMA) { if (ok) ok = tc::mbar_wait(&mbar[1 + nbuf], ((it + 1) / kPassStages) & 1); }
      else tc::cp_async_wait<kPassStages - 2>();
      __syncthreads();
      fix_tiles(nbuf);
    }
    if (ok) ok = tc::mbar_wait(mbar, ph);
    ph ^= 1;
    tc::fence_after_sync();
    issue(it + kPassStages);  // this buffer is free: the MMA has read the tiles, every thread has read L
    if (ok) {
      float f[32];
      ld_acc32(taddr, warp, 32 * half, f);
#pragma unroll
      for (int jj = 0; jj < 32; ++jj) H[jj] = fmaf(L, H[jj], f[jj]);
    }
    tc::fence_before_sync();
  }
  if (!TMA) tc::cp_async_wait<0>();
  if (tid == kPassStoreThread) tc::bulk_wait_read<0>();  // shared memory must outlive the copies
  if (!ok && tid == 0) atomicExch(p.status, 11);
  tc::fence_before_sync();
  __syncthreads();
  if (warp == 0) tc::tmem_dealloc(taddr, 64);
}

// ------------------------------------------------------------ chunk output
// A CTA is a chain of dependent steps, so the kernel is sized for FOUR CTAs per SM: 128 TMEM columns and 51 KB of
// shared memory.  The chunk state H0 lands in the Brot tile once G = Crot Brot^T has been formed (its copy hides
// behind the mask epilogue), and Crot H0 joins the second MMA batch.
constexpr int kOutSmem = 16384 * 2 + 8192 * 2 + sizeof(ChunkScal) + 64 + 1024;

template <bool TMA>
__global__ void __launch_bounds__(128, 4) m3s_chunk_out_kernel(SsdP p, const __grid_constant__ ChunkMaps maps) {
  extern __shared__ uint8_t raw[];
  uint8_t* sm = raw + ((1024u - (tc::smem_u32(raw) & 1023u)) & 1023u);
  uint8_t* Bt = sm;               // [64][128] Brot, then [128][64] H0
  uint8_t* Ct = Bt + 16384;       // [64][128] Crot
  uint8_t* Ht = Bt;
  uint8_t* Xt = Ct + 16384;       // [64][64]  x
  uint8_t* Gm = Xt + 8192;        // [64][64]  (Crot Brot^T) * M
  ChunkScal& s = *reinterpret_cast<ChunkScal*>(Gm + 8192);
  uint64_t* mbar = reinterpret_cast<uint64_t*>(&s + 1);  // [0] MMA completion, [1] token tiles landed, [2] H0 landed
  uint32_t* tslot = reinterpret_cast<uint32_t*>(mbar + 3);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int c = blockIdx.x, head = blockIdx.y, b = blockIdx.z, t0 = c * Q;
  const int d0 = head * P, g = d0 / (p.D / p.G);
  const size_t ci = ((size_t)b * p.NH + head) * p.n + c;

  if (warp == 0) { tc::tmem_alloc(tslot, 128); tc::tmem_relinquish(); }
  // the thread that initialises the barriers also issues the copies, on another warp than the TMEM allocation
  if (tid == 32) {
    for (int m = 0; m < 3; ++m) tc::mbar_init(mbar + m, 1);
    tc::mbar_fence_init();
  }
  bool ok = true;
  if (TMA) {  // every operand by the copy engine
    if (tid == 32) {
      tc::mbar_expect_tx(mbar + 1, 2 * 16384 + 8192 + (uint32_t)sizeof(ChunkScal));
      for (int sl = 0; sl < 2; ++sl) {
        tc::tma_load_4d(tc::smem_u32(Bt) + 8192 * sl, &maps.b, 64 * sl, g, t0, b, mbar + 1);
        tc::tma_load_4d(tc::smem_u32(Ct) + 8192 * sl, &maps.c, 64 * sl, g, t0, b, mbar + 1);
      }
      tc::tma_load_4d(tc::smem_u32(Xt), &maps.x, 0, head, t0, b, mbar + 1);
      tc::bulk_load(tc::smem_u32(&s), p.cs + ci * (sizeof(ChunkScal) / 4), (uint32_t)sizeof(ChunkScal), mbar + 1);
    }
    __syncthreads();  // barriers initialised before anyone waits on them
    ok = tc::mbar_wait(mbar + 1, 0);
  } else {
    issue_rows_tile(Bt, p.b, p, b, g, t0);
    issue_rows_tile(Ct, p.c, p, b, g, t0);
    issue_x_tile(Xt, p.x, p, b, d0, t0);
    issue_chunk_scalars(p, ci, s);
    tc::cp_async_commit();
    tc::cp_async_wait<0>();
  }
  __syncthreads();
  rotate_in_tile<TMA>(Bt, s.sn, s.cs);
  rotate_in_tile<TMA>(Ct, s.sn, s.cs);
  tc::fence_async_smem();
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t taddr = *tslot;
  if (tid == 0) {
    tc::issue_gemm(taddr, in_kmajor<TMA>(Ct, N), in_kmajor<TMA>(Bt, N), 64, Q, N, false);           // G = Crot Brot^T
    tc::mma_commit(mbar);
  }
  if (ok) ok = tc::mbar_wait(mbar, 0);
  tc::fence_after_sync();
  // Brot is dead: the chunk state takes its place while the mask is applied
  if (TMA) {
    if (tid == 32) {
      tc::mbar_expect_tx(mbar + 2, 16384);
      tc::bulk_load(tc::smem_u32(Ht), p.H0 + ci * (N * P), 16384, mbar + 2);
    }
  } else {
    issue_state_tile(Ht, p.H0 + ci * (N * P));
    tc::cp_async_commit();
  }
  const int t = 16 * warp + (lane & 15);
  const bool own = lane < 16;
  if (ok) {
    // Lanes 16-31 hold no accumulator rows: they take over columns 32..63 of the row of lane - 16, so all 32
    // lanes share the mask arithmetic (branch-free, so the exponentials of different columns overlap).
    const float lt = s.Lam[t], gt = s.gam[t];
    const int hx = lane >> 4;
    float f[32];
    {
      float fa[32], fb[32];
      ld_acc32(taddr, warp, 0, fa);
      ld_acc32(taddr, warp, 32, fb);
#pragma unroll
      for (int q = 0; q < 32; ++q) {
        const float up = __shfl_sync(0xffffffffu, fb[q], lane & 15);
        f[q] = hx ? up : fa[q];
      }
    }
#pragma unroll
    for (int jj = 0; jj < 32; ++jj) {
      const int sx = 32 * hx + jj;
      const float mv = __expf(fminf(lt - s.Lam[sx], 0.f)) * (sx < t ? s.e[sx] : gt);
      f[jj] = (sx <= t) ? f[jj] * mv : 0.f;
    }
#pragma unroll
    for (int x = 0; x < 4; ++x) sts16(Gm, tc::kmajor_unit(t, 4 * hx + x, Q), pack8(&f[8 * x]));
  }
  if (TMA) { if (ok) ok = tc::mbar_wait(mbar + 2, 0); }  // H0
  else tc::cp_async_wait<0>();
  tc::fence_async_smem();
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  if (ok && tid == 0) {
    tc::issue_gemm(taddr, tc::kmajor_tile(Gm, Q), in_mnmajor<TMA>(Xt, P), 64, P, Q, false);  // (G*M) X, over the consumed G
    tc::issue_gemm(taddr + 64, in_kmajor<TMA>(Ct, N), tc::mnmajor_tile(Ht, P), 64, P, N, false);    // Crot H0
    tc::mma_commit(mbar);
  }
  if (ok) ok = tc::mbar_wait(mbar, 1);
  tc::fence_after_sync();
  if (ok) {  // y = (G*M) X + exp(Lam) Crot H0, assembled over the x tile (dead) and written out in full rows
    const float de = s.dexp[t];
    for (int c0 = 0; c0 < P; c0 += 32) {
      float f[32], f2[32];
      ld_acc32(taddr, warp, c0, f);
      ld_acc32(taddr + 64, warp, c0, f2);
      if (own) {
#pragma unroll
        for (int jj = 0; jj < 32; ++jj) f[jj] = fmaf(de, f2[jj], f[jj]);
#pragma unroll
        for (int x = 0; x < 4; ++x) sts16(Xt, tc::kmajor_unit(t, (c0 >> 3) + x, P), pack8(&f[8 * x]));
      }
    }
  } else if (tid == 0) {
    atomicExch(p.status, 12);
  }
  tc::fence_before_sync();
  __syncthreads();
  if (ok) {
    for (int u = tid; u < Q * 8; u += 128) {  // 64-byte row pieces, conflict-free shared-memory reads
      const int r = ((u >> 6) << 3) | (u & 7), c8 = (u >> 3) & 7;
      if (t0 + r < p.T)
        *reinterpret_cast<uint4*>(p.y + ((size_t)b * p.T + t0 + r) * p.D + d0 + c8 * 8) =
            *reinterpret_cast<const uint4*>(Xt + 16 * u);
    }
  }
  if (warp == 0) tc::tmem_dealloc(taddr, 128);
}

// ------------------------------------------------------------ chunk gradients
// 256 TMEM columns and < 113 KB of shared memory, so two CTAs share an SM:
//   phase 1: G [0,64), dY X^T [64,128), Crot H0 [128,192), Brot dH1 [192,256)
//   phase 2: dx [0,64), dCrot [64,192)           (Brot dH1 still live in [192,256))
//   phase 3: dBrot [0,128)
// All accumulators are M=64: row i of every result is in TMEM lane (i%16)+32*(i/16); warps 0-3 take the
// first half of the columns, warps 4-7 the second.  The G*M tile reuses the x tile once x is dead.
constexpr int kGradSmem = 16384 * 4 + 8192 * 5 + sizeof(ChunkScal) + (4 * Q + 4 * Q + 8 * Q + 32) * 4 + 64 + 1024;

template <bool SW>
__device__ __forceinline__ float row_dot32_64(const uint8_t* tile, int r, int c0, const float (&f)[32]) {
  // sum_k tile[r][c0 + k] f[k] for a [.][64] tile: four independent chains
  uint4 raw[4];
#pragma unroll
  for (int x = 0; x < 4; ++x) raw[x] = *reinterpret_cast<const uint4*>(tile + in_unit<SW>(r, (c0 >> 3) + x, P));
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int x = 0; x < 4; ++x) {
    float e[8];
    unpack8(raw[x], e);
#pragma unroll
    for (int y = 0; y < 8; ++y) acc[x] = fmaf(e[y], f[8 * x + y], acc[x]);
  }
  return (acc[0] + acc[1]) + (acc[2] + acc[3]);
}

template <bool TMA>
__global__ void __launch_bounds__(256) m3s_chunk_grad_kernel(SsdP p, const __grid_constant__ ChunkMaps maps) {
  extern __shared__ uint8_t raw[];
  uint8_t* sm = raw + ((1024u - (tc::smem_u32(raw) & 1023u)) & 1023u);
  uint8_t* Bt = sm;                // [64][128] Brot
  uint8_t* Ct = Bt + 16384;        // [64][128] Crot
  uint8_t* Ht = Ct + 16384;        // [128][64] H0
  uint8_t* Dt = Ht + 16384;        // [128][64] dH1
  uint8_t* Xt = Dt + 16384;        // [64][64]  x
  uint8_t* Yt = Xt + 8192;         // [64][64]  dY
  uint8_t* Xs = Yt + 8192;         // [64][64]  r e x
  uint8_t* Ys = Xs + 8192;         // [64][64]  exp(Lam) dY
  uint8_t* GMt = Xt;               // [64][64]  G*M  (written after the last read of x)
  uint8_t* dGt = Ys + 8192;        // [64][64]  dG
  ChunkScal& s = *reinterpret_cast<ChunkScal*>(dGt + 8192);
  float* csw_e = reinterpret_cast<float*>(&s + 1);  // [4][Q] per-warp column sums for de
  float* csw_l = csw_e + 4 * Q;                     // [4][Q] per-warp column sums for dLam
  float* part = csw_l + 4 * Q;                      // [2][4][Q]: per half: dLam, de, dgam, dphi row partials
  float* red = part + 8 * Q;                        // [32]
  uint64_t* mbar = reinterpret_cast<uint64_t*>(red + 32);  // [0] MMA completion, [1] token tiles, [2] state images
  uint32_t* tslot = reinterpret_cast<uint32_t*>(mbar + 4);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int c = blockIdx.x, head = blockIdx.y, b = blockIdx.z, t0 = c * Q;
  const int d0 = head * P, g = d0 / (p.D / p.G);
  const size_t ci = ((size_t)b * p.NH + head) * p.n + c;
  const bool own = lane < 16;
  const int t = 16 * (warp & 3) + (lane & 15), hc = warp >> 2;

  if (warp == 0) { tc::tmem_alloc(tslot, 256); tc::tmem_relinquish(); }
  // the thread that initialises the barriers also issues the copies, on another warp than the TMEM allocation
  if (tid == 32) {
    for (int m = 0; m < 3; ++m) tc::mbar_init(mbar + m, 1);
    tc::mbar_fence_init();
  }
  bool ok = true;
  if (TMA) {  // every operand by the copy engine: token tiles on one barrier, the state images on another
    if (tid == 32) {
      tc::mbar_expect_tx(mbar + 1, 2 * 16384 + 2 * 8192 + (uint32_t)sizeof(ChunkScal));
      for (int sl = 0; sl < 2; ++sl) {
        tc::tma_load_4d(tc::smem_u32(Bt) + 8192 * sl, &maps.b, 64 * sl, g, t0, b, mbar + 1);
        tc::tma_load_4d(tc::smem_u32(Ct) + 8192 * sl, &maps.c, 64 * sl, g, t0, b, mbar + 1);
      }
      tc::tma_load_4d(tc::smem_u32(Xt), &maps.x, 0, head, t0, b, mbar + 1);
      tc::tma_load_4d(tc::smem_u32(Yt), &maps.dy, 0, head, t0, b, mbar + 1);
      tc::bulk_load(tc::smem_u32(&s), p.cs + ci * (sizeof(ChunkScal) / 4), (uint32_t)sizeof(ChunkScal), mbar + 1);
      tc::mbar_expect_tx(mbar + 2, 2 * 16384);
      tc::bulk_load(tc::smem_u32(Ht), p.H0 + ci * (N * P), 16384, mbar + 2);
      tc::bulk_load(tc::smem_u32(Dt), p.dH1 + ci * (N * P), 16384, mbar + 2);
    }
  } else {
    issue_rows_tile(Bt, p.b, p, b, g, t0);
    issue_rows_tile(Ct, p.c, p, b, g, t0);
    issue_x_tile(Xt, p.x, p, b, d0, t0);
    issue_x_tile(Yt, p.dy, p, b, d0, t0);
    issue_chunk_scalars(p, ci, s);
    tc::cp_async_commit();
    issue_state_tile(Ht, p.H0 + ci * (N * P));
    issue_state_tile(Dt, p.dH1 + ci * (N * P));
    tc::cp_async_commit();
  }
  for (int u = tid; u < 8 * Q; u += 256) { csw_e[u] = 0.f; }  // csw_e and csw_l are contiguous
  if (TMA) __syncthreads();  // barriers initialised before anyone waits on them
  if (TMA) ok = tc::mbar_wait(mbar + 1, 0);
  else tc::cp_async_wait<1>();
  __syncthreads();
  rotate_in_tile<TMA>(Bt, s.sn, s.cs);
  rotate_in_tile<TMA>(Ct, s.sn, s.cs);
  scale_in_tile<TMA>(Xs, Xt, s.re);
  scale_in_tile<TMA>(Ys, Yt, s.dexp);
  if (TMA) { if (ok) ok = tc::mbar_wait(mbar + 2, 0); }
  else tc::cp_async_wait<0>();
  tc::fence_async_smem();
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t taddr = *tslot;
  if (tid == 0) {
    tc::issue_gemm(taddr + 0, in_kmajor<TMA>(Ct, N), in_kmajor<TMA>(Bt, N), 64, Q, N, false);         // G
    tc::issue_gemm(taddr + 64, in_kmajor<TMA>(Yt, P), in_kmajor<TMA>(Xt, P), 64, Q, P, false);        // dY X^T
    tc::issue_gemm(taddr + 128, in_kmajor<TMA>(Ct, N), tc::mnmajor_tile(Ht, P), 64, P, N, false);     // Crot H0
    tc::issue_gemm(taddr + 192, in_kmajor<TMA>(Bt, N), tc::mnmajor_tile(Dt, P), 64, P, N, false);     // Brot dH1
    tc::mma_commit(mbar);
  }
  {  // <dH1, H0> while the tensor core works
    float acc = 0.f;
    for (int u = tid; u < N * 8; u += 256) {
      float a[8], d[8];
      unpack8(*reinterpret_cast<const uint4*>(Ht + u * 16), a);
      unpack8(*reinterpret_cast<const uint4*>(Dt + u * 16), d);
#pragma unroll
      for (int y = 0; y < 8; ++y) acc = fmaf(a[y], d[y], acc);
    }
    acc = warp_sum(acc);
    if (lane == 0) red[warp] = acc;
  }
  if (ok) ok = tc::mbar_wait(mbar, 0);
  tc::fence_after_sync();
  float dl_own = 0.f, de_own = 0.f, dg_own = 0.f, zsum = 0.f;
  const float lt = s.Lam[t], gt = s.gam[t], et = s.e[t], rt = s.r[t], dxt = s.dexp[t];
  if (ok) {
    {  // kappa_t = exp(Lam_t) dY_t . (Crot H0)_t   and   zeta_s = (Brot dH1)_s . x_s   (32 channels per half)
      const int c0 = 32 * hc;
      float f[32];
      ld_acc32(taddr + 128, warp, c0, f);
      if (own) dl_own += dxt * row_dot32_64<TMA>(Yt, t, c0, f);
      ld_acc32(taddr + 192, warp, c0, f);
      if (own) {
        const float zeta = row_dot32_64<TMA>(Xt, t, c0, f);
        de_own += rt * zeta;
        dl_own -= rt * et * zeta;
        zsum = rt * et * zeta;
      }
    }
  }
  __syncthreads();  // every read of the x tile is done: G*M may overwrite it
  if (ok) {
    {  // G and dY X^T: 32 columns per half.  Lanes 16-31 hold no accumulator rows; they take over columns
       // 16..31 of the row of lane - 16, so all 32 lanes share the mask arithmetic.
      const int c0 = 32 * hc, hx = lane >> 4;
      float fg[16], fd[16];
      {
        float fa[32];
        ld_acc32(taddr + 0, warp, c0, fa);
#pragma unroll
        for (int q = 0; q < 16; ++q) {
          const float up = __shfl_sync(0xffffffffu, fa[16 + q], lane & 15);
          fg[q] = hx ? up : fa[q];
        }
        ld_acc32(taddr + 64, warp, c0, fa);
#pragma unroll
        for (int q = 0; q < 16; ++q) {
          const float up = __shfl_sync(0xffffffffu, fa[16 + q], lane & 15);
          fd[q] = hx ? up : fa[q];
        }
      }
      float rs = 0.f, dgc = 0.f;
      float gm[16], dg[16], ce[16], cl[16];
#pragma unroll
      for (int q = 0; q < 16; ++q) {
        const int sx = c0 + 16 * hx + q;
        // branch-free so that the exponentials of different columns overlap
        const bool in = sx <= t;
        const float Dv = in ? __expf(fminf(lt - s.Lam[sx], 0.f)) : 0.f;
        const float Mv = Dv * (sx < t ? s.e[sx] : gt);
        const float dGM = in ? fd[q] : 0.f;
        const float gv = in ? fg[q] : 0.f;
        gm[q] = gv * Mv;                 // (G*M)_ts
        dg[q] = dGM * Mv;                // dG_ts
        const float dM = dGM * gv;
        const float dw = dM * Dv;
        const float ml = dM * Mv;
        rs += ml;
        dgc += (sx == t) ? dw : 0.f;
        ce[q] = (sx < t) ? dw : 0.f;     // de_s and dLam_s: column sums over the 16 rows of this warp
        cl[q] = ml;
      }
#pragma unroll
      for (int x = 0; x < 2; ++x) {
        sts16(GMt, tc::kmajor_unit(t, (c0 >> 3) + 2 * hx + x, Q), pack8(&gm[8 * x]));
        sts16(dGt, tc::kmajor_unit(t, (c0 >> 3) + 2 * hx + x, Q), pack8(&dg[8 * x]));
      }
      colsum16(ce, lane);  // the two 16-lane halves reduce their own 16 columns side by side
      colsum16(cl, lane);
      {
        const int sx = c0 + 16 * hx + (lane & 15);
        csw_e[(warp & 3) * Q + sx] += ce[0];
        csw_l[(warp & 3) * Q + sx] -= cl[0];
      }
      rs += __shfl_xor_sync(0xffffffffu, rs, 16);
      dgc += __shfl_xor_sync(0xffffffffu, dgc, 16);
      dl_own += rs;
      dg_own += dgc;
    }
  }
  {
    const float tot = warp_sum(own ? zsum : 0.f);
    if (lane == 0) red[8 + warp] = tot;
  }
  tc::fence_async_smem();
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  if (ok && tid == 0) {
    tc::issue_gemm(taddr + 0, tc::mnmajor_tile(GMt, Q), in_mnmajor<TMA>(Yt, P), 64, P, Q, false);     // (G*M)^T dY
    tc::issue_gemm(taddr + 64, in_kmajor<TMA>(Ys, P), tc::kmajor_tile(Ht, P), 64, N, P, false);       // (e^Lam dY) H0^T
    tc::issue_gemm(taddr + 64, tc::kmajor_tile(dGt, Q), in_mnmajor<TMA>(Bt, N), 64, N, Q, true);      // + dG Brot
    tc::mma_commit(mbar);
  }
  if (ok) ok = tc::mbar_wait(mbar, 1);
  tc::fence_after_sync();
  float dphi_own = 0.f;
  if (ok) {
    {  // dx_s = (G*M)^T dY + r e (Brot dH1)
      const int c0 = 32 * hc;
      float f[32], f2[32];
      ld_acc32(taddr + 0, warp, c0, f);
      ld_acc32(taddr + 192, warp, c0, f2);
      if (own && t0 + t < p.T) {
        const float sc = rt * et;
#pragma unroll
        for (int jj = 0; jj < 32; ++jj) f[jj] = fmaf(sc, f2[jj], f[jj]);
        uint4* dst = reinterpret_cast<uint4*>(p.dx + ((size_t)b * p.T + t0 + t) * p.D + d0 + c0);
#pragma unroll
        for (int x = 0; x < 4; ++x) dst[x] = pack8(&f[8 * x]);
      }
    }
    // dCrot rows: un-rotate into the per-head partial rows of dC, and their share of the angle gradient
    const float sn = s.sn[t], cs = s.cs[t];
    for (int c0 = 64 * hc; c0 < 64 * hc + 64; c0 += 32) {
      float gc[32];
      ld_acc32(taddr + 64, warp, c0, gc);
      if (own && t0 + t < p.T) {
        bf16* pcr = p.pc + ((((size_t)b * p.NH + head) * p.T) + t0 + t) * N + c0;
#pragma unroll
        for (int x = 0; x < 4; ++x) {
          float cr[8], oc[8];
          unpack8(*reinterpret_cast<const uint4*>(Ct + in_unit<TMA>(t, (c0 >> 3) + x, N)), cr);
#pragma unroll
          for (int k = 0; k < 8; k += 2) {
            const float c0v = gc[8 * x + k], c1v = gc[8 * x + k + 1];
            oc[k] = cs * c0v - sn * c1v; oc[k + 1] = sn * c0v + cs * c1v;
            dphi_own += cr[k + 1] * c0v - cr[k] * c1v;
          }
          *reinterpret_cast<uint4*>(pcr + 8 * x) = pack8(oc);
        }
      }
    }
  }
  tc::fence_before_sync();
  __syncthreads();  // columns [0,192) are free again
  tc::fence_after_sync();
  if (ok && tid == 0) {
    tc::issue_gemm(taddr + 0, in_kmajor<TMA>(Xs, P), tc::kmajor_tile(Dt, P), 64, N, P, false);        // (r e x) dH1^T
    tc::issue_gemm(taddr + 0, tc::mnmajor_tile(dGt, Q), in_mnmajor<TMA>(Ct, N), 64, N, Q, true);      // + dG^T Crot
    tc::mma_commit(mbar);
  }
  if (ok) ok = tc::mbar_wait(mbar, 0);
  tc::fence_after_sync();
  if (ok) {
    const float sn = s.sn[t], cs = s.cs[t];
    for (int c0 = 64 * hc; c0 < 64 * hc + 64; c0 += 32) {
      float gb[32];
      ld_acc32(taddr + 0, warp, c0, gb);
      if (own && t0 + t < p.T) {
        bf16* pbr = p.pb + ((((size_t)b * p.NH + head) * p.T) + t0 + t) * N + c0;
#pragma unroll
        for (int x = 0; x < 4; ++x) {
          float br[8], ob[8];
          unpack8(*reinterpret_cast<const uint4*>(Bt + in_unit<TMA>(t, (c0 >> 3) + x, N)), br);
#pragma unroll
          for (int k = 0; k < 8; k += 2) {
            const float b0 = gb[8 * x + k], b1 = gb[8 * x + k + 1];
            ob[k] = cs * b0 - sn * b1; ob[k + 1] = sn * b0 + cs * b1;
            dphi_own += br[k + 1] * b0 - br[k] * b1;
          }
          *reinterpret_cast<uint4*>(pbr + 8 * x) = pack8(ob);
        }
      }
    }
  }
  if (own) {
    part[(hc * 4 + 0) * Q + t] = dl_own;
    part[(hc * 4 + 1) * Q + t] = de_own;
    part[(hc * 4 + 2) * Q + t] = dg_own;
    part[(hc * 4 + 3) * Q + t] = dphi_own;
  }
  tc::fence_before_sync();
  __syncthreads();
  if (tid < 32) {  // dLam -> da: reverse in-chunk cumulative sum (one warp, two rows per lane, fixed order)
    float zs = 0.f, hh = 0.f;
    for (int wv = 0; wv < 8; ++wv) { zs += red[8 + wv]; hh += red[wv]; }
    const float base = zs + s.L * hh;  // d/dLam_end
    const int ra = Q - 1 - 2 * tid, rb = ra - 1;
    float a = part[0 * Q + ra] + part[4 * Q + ra] + csw_l[ra] + csw_l[Q + ra] + csw_l[2 * Q + ra] + csw_l[3 * Q + ra];
    float bq = part[0 * Q + rb] + part[4 * Q + rb] + csw_l[rb] + csw_l[Q + rb] + csw_l[2 * Q + rb] + csw_l[3 * Q + rb];
    warp_rcumsum64(a, bq, tid);
    s.Lam[ra] = base + a;  // Lam is dead by now: reuse for da
    s.Lam[rb] = base + bq;
  }
  __syncthreads();
  if (!ok && tid == 0) atomicExch(p.status, 13);
  if (ok && tid < Q && t0 + tid < p.T) {
    const size_t o = ((size_t)b * p.NH + head) * p.T + t0 + tid;
    p.da[o] = s.Lam[tid];
    p.de[o] = part[1 * Q + tid] + part[5 * Q + tid] + csw_e[tid] + csw_e[Q + tid] + csw_e[2 * Q + tid] + csw_e[3 * Q + tid];
    p.dgam[o] = part[2 * Q + tid] + part[6 * Q + tid];
    p.dphi[o] = part[3 * Q + tid] + part[7 * Q + tid];
  }
  if (warp == 0) tc::tmem_dealloc(taddr, 256);
}


// ------------------------------------------------------------ final per-token scalars
__global__ void __launch_bounds__(kScalThreads) m3s_final_kernel(SsdP p) {
  __shared__ double wtot[kScalThreads / 32];
  __shared__ float wsum[kScalThreads / 32];
  const int head = blockIdx.x, b = blockIdx.y, tid = threadIdx.x;
  const size_t base = ((size_t)b * p.NH + head) * p.T;
  const float A = -expf(p.a_log[head]);
  const int per = (p.T + kScalThreads - 1) / kScalThreads, lo = tid * per, hi = min(p.T, lo + per);
  double acc = 0.0;
  for (int t0 = lo; t0 < hi; t0 += kScalBatch) {
    float v[kScalBatch];
#pragma unroll
    for (int x = 0; x < kScalBatch; ++x) v[x] = t0 + x < hi ? p.dphi[base + t0 + x] : 0.f;
#pragma unroll
    for (int x = 0; x < kScalBatch; ++x) acc += (double)v[x];
  }
  double total;
  const double incl = cta_scan(acc, wtot, total);
  double suf = total - incl;  // sum over the threads after this one (exclusive suffix; exact enough in fp64)
  float dal = 0.f;
  // backwards over this thread's steps, kFinalBatch at a time with the loads of a batch ahead of its stores
  constexpr int kFinalBatch = 4;
  for (int t1 = hi - 1; t1 >= lo; t1 -= kFinalBatch) {
    float dph[kFinalBatch], dtv[kFinalBatch], lamv[kFinalBatch], thv[kFinalBatch], dgv[kFinalBatch], dev[kFinalBatch],
        dnv[kFinalBatch], dav[kFinalBatch], drw[kFinalBatch];
#pragma unroll
    for (int x = 0; x < kFinalBatch; ++x) {
      const int t = max(t1 - x, lo);
      const size_t r = ((size_t)b * p.T + t) * p.NH + head;
      dph[x] = p.dphi[base + t];
      dtv[x] = p.dt[base + t];
      lamv[x] = p.lam[base + t];
      thv[x] = __ldg(p.theta + r);
      drw[x] = __ldg(p.dt_raw + r);
      dgv[x] = p.dgam[base + t];
      dev[x] = p.de[base + t];
      dnv[x] = t > 0 ? p.de[base + t - 1] : 0.f;
      dav[x] = p.da[base + t];
    }
#pragma unroll
    for (int x = 0; x < kFinalBatch; ++x) {
      const int t = t1 - x;
      if (t >= lo) {
        suf += (double)dph[x];
        const float dinc = (float)suf;
        const size_t r = ((size_t)b * p.T + t) * p.NH + head;
        const float dt = dtv[x], lam = lamv[x];
        const float dgam = dgv[x] + dev[x], dnxt = dnv[x], da = dav[x];
        const float ddelta = A * da + lam * dgam + (1.f - lam) * dnxt + thv[x] * dinc;
        p.ddt[r] = ddelta * sigmoid_f(drw[x]);
        p.dlam[r] = dt * (dgam - dnxt) * lam * (1.f - lam);
        p.dtheta[r] = dt * dinc;
        dal = fmaf(dt, da, dal);
      }
    }
  }
  dal = warp_sum(dal);
  if ((tid & 31) == 0) wsum[tid >> 5] = dal;
  __syncthreads();
  if (tid == 0) {
    float tot = 0.f;
    for (int i = 0; i < kScalThreads / 32; ++i) tot += wsum[i];
    p.dal_part[b * p.NH + head] = A * tot;  // summed over the batch in a fixed order by m3s_dalog_kernel
  }
}
__global__ void m3s_dalog_kernel(SsdP p) {
  const int head = blockIdx.x * blockDim.x + threadIdx.x;
  if (head >= p.NH) return;
  float s = 0.f;
  for (int b = 0; b < p.B; ++b) s += p.dal_part[b * p.NH + head];
  p.da_log[head] = s;
}

// dB[b,t,g,:] = sum over the heads of group g of the per-head partial rows (fp32, fixed order).
// One warp per (b, t, g): a lane owns 4 consecutive states.
__global__ void __launch_bounds__(128) m3s_reduce_kernel(const bf16* __restrict__ pb, const bf16* __restrict__ pc,
                                                         bf16* __restrict__ db, bf16* __restrict__ dc, int T, int G, int NH) {
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * 4 + (threadIdx.x >> 5), g = blockIdx.y, b = blockIdx.z, per = NH / G;
  if (t >= T) return;
  float sb[4] = {0.f, 0.f, 0.f, 0.f}, sc[4] = {0.f, 0.f, 0.f, 0.f};
  for (int h = g * per; h < (g + 1) * per; ++h) {
    const size_t pi = (((size_t)b * NH + h) * T + t) * N + 4 * lane;
    const uint2 vb = __ldg(reinterpret_cast<const uint2*>(pb + pi));
    const uint2 vc = __ldg(reinterpret_cast<const uint2*>(pc + pi));
    float a0, a1;
    tc::unpack_bf16(vb.x, a0, a1); sb[0] += a0; sb[1] += a1;
    tc::unpack_bf16(vb.y, a0, a1); sb[2] += a0; sb[3] += a1;
    tc::unpack_bf16(vc.x, a0, a1); sc[0] += a0; sc[1] += a1;
    tc::unpack_bf16(vc.y, a0, a1); sc[2] += a0; sc[3] += a1;
  }
  const size_t gi = (((size_t)b * T + t) * G + g) * N + 4 * lane;
  *reinterpret_cast<uint2*>(db + gi) = make_uint2(tc::pack_bf16(sb[0], sb[1]), tc::pack_bf16(sb[2], sb[3]));
  *reinterpret_cast<uint2*>(dc + gi) = make_uint2(tc::pack_bf16(sc[0], sc[1]), tc::pack_bf16(sc[2], sc[3]));
}

}  // namespace m3s

// ------------------------------------------------------------------ host
using m3s::SsdP;

bool mamba3_ssd_supported(const mxb_mamba3_desc* d) {
  if (d->io_dtype != MXB_BF16 || d->nheads <= 0 || d->D % d->nheads) return false;
  if (d->D / d->nheads != m3s::P || d->N != m3s::N) return false;
  if ((d->D / d->G) % m3s::P || d->nheads % d->G) return false;
  return true;
}

static size_t carve_ssd(SsdP& p, void* ws, bool bwd) {
  Carver cv(ws);
  const size_t bh = (size_t)p.B * p.NH, nst = bh * p.n * m3s::N * m3s::P;
  p.status = cv.take<int>(64);
  p.dt = cv.take<float>(bh * p.T);
  p.lam = cv.take<float>(bh * p.T);
  p.phi = cv.take<float>(bh * p.T);
  p.cs = cv.take<float>(bh * p.n * (sizeof(m3s::ChunkScal) / 4));
  p.H0 = cv.take<m3s::bf16>(nst);
  if (bwd) {
    p.dH1 = cv.take<m3s::bf16>(nst);
    p.dphi = cv.take<float>(bh * p.T);
    p.da = cv.take<float>(bh * p.T);
    p.de = cv.take<float>(bh * p.T);
    p.dgam = cv.take<float>(bh * p.T);
    p.dal_part = cv.take<float>(bh);
    p.pb = cv.take<m3s::bf16>(bh * p.T * m3s::N);
    p.pc = cv.take<m3s::bf16>(bh * p.T * m3s::N);
  }
  return cv.bytes();
}

static SsdP make_ssd(const mxb_mamba3_desc* d) {
  SsdP p{};
  p.B = d->B; p.T = d->T; p.D = d->D; p.G = d->G; p.NH = d->nheads;
  p.n = (d->T + m3s::Q - 1) / m3s::Q;
  p.no_tma = (d->flags & MXB_MAMBA3_NO_TMA) ? 1 : 0;
  return p;
}

size_t mamba3_ssd_workspace_bytes(const mxb_mamba3_desc* d, bool bwd) {
  SsdP p = make_ssd(d);
  return carve_ssd(p, nullptr, bwd);
}

template <typename KernelT>
static mxb_status ssd_smem(KernelT k, size_t bytes) {
  cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
  if (e != cudaSuccess) { set_last_cuda_error((int)e); return MXB_ERR_CUDA; }
  return MXB_OK;
}

bool make_tma_map_bthd(CUtensorMap* m, const void* base, int B, int T, int H, int D);

// Tensor maps for the token-indexed operands of the chunk kernels (dy only in the backward); false when one
// cannot be made (no tensor-map entry point in the driver): the kernels then stage with cp.async.  Either way
// the operand bases are 16-byte aligned: the dispatcher refuses other pointers.
static bool ssd_chunk_maps(const SsdP& p, m3s::ChunkMaps& maps) {
  std::memset(&maps, 0, sizeof maps);
  if (p.no_tma) return false;
  bool ok = make_tma_map_bthd(&maps.b, p.b, p.B, p.T, p.G, m3s::N) && make_tma_map_bthd(&maps.c, p.c, p.B, p.T, p.G, m3s::N) &&
            make_tma_map_bthd(&maps.x, p.x, p.B, p.T, p.NH, m3s::P);
  if (ok && p.dy) ok = make_tma_map_bthd(&maps.dy, p.dy, p.B, p.T, p.NH, m3s::P);
  return ok;
}

// Sequential pass over the chunks (mode 0: forward states, mode 1: reverse state gradients); the copy engine
// feeds it when tensor maps can be made for the operands, cp.async otherwise.
static mxb_status ssd_state_pass(SsdP& p, int mode, cudaStream_t st) {
  m3s::PassMaps maps;
  std::memset(&maps, 0, sizeof maps);
  const bool tma = !p.no_tma && make_tma_map_bthd(&maps.r, mode == 0 ? p.b : p.c, p.B, p.T, p.G, m3s::N) &&
                   make_tma_map_bthd(&maps.x, mode == 0 ? p.x : p.dy, p.B, p.T, p.NH, m3s::P);
  if (tma) {
    if (ssd_smem(m3s::m3s_state_pass_kernel<true>, m3s::kPassSmem) != MXB_OK) return MXB_ERR_CUDA;
    MXB_LAUNCH("m3s_state_pass_kernel", st,
               (m3s::m3s_state_pass_kernel<true><<<dim3(p.NH, p.B), 256, m3s::kPassSmem, st>>>(p, mode, maps)));
  } else {
    if (ssd_smem(m3s::m3s_state_pass_kernel<false>, m3s::kPassSmem) != MXB_OK) return MXB_ERR_CUDA;
    MXB_LAUNCH("m3s_state_pass_kernel", st,
               (m3s::m3s_state_pass_kernel<false><<<dim3(p.NH, p.B), 256, m3s::kPassSmem, st>>>(p, mode, maps)));
  }
  return check_launch("m3s_state_pass_kernel");
}

static mxb_status ssd_forward(SsdP& p, cudaStream_t st) {
  const dim3 gc(p.n, p.NH, p.B);
  if (cudaMemsetAsync(p.status, 0, 256, st) != cudaSuccess) return MXB_ERR_CUDA;
  MXB_LAUNCH("m3s_scalars_kernel", st, (m3s::m3s_scalars_kernel<<<dim3(p.NH, p.B), m3s::kScalThreads, 0, st>>>(p)));
  MXB_LAUNCH("m3s_chunk_scalars_kernel", st, (m3s::m3s_chunk_scalars_kernel<<<gc, 64, 0, st>>>(p)));
  mxb_status ps = ssd_state_pass(p, 0, st);
  if (ps != MXB_OK) return ps;
  if (p.y) {
    m3s::ChunkMaps maps;
    if (ssd_chunk_maps(p, maps)) {
      if (ssd_smem(m3s::m3s_chunk_out_kernel<true>, m3s::kOutSmem) != MXB_OK) return MXB_ERR_CUDA;
      MXB_LAUNCH("m3s_chunk_out_kernel", st, (m3s::m3s_chunk_out_kernel<true><<<gc, 128, m3s::kOutSmem, st>>>(p, maps)));
    } else {
      if (ssd_smem(m3s::m3s_chunk_out_kernel<false>, m3s::kOutSmem) != MXB_OK) return MXB_ERR_CUDA;
      MXB_LAUNCH("m3s_chunk_out_kernel", st, (m3s::m3s_chunk_out_kernel<false><<<gc, 128, m3s::kOutSmem, st>>>(p, maps)));
    }
  }
  return check_launch("mamba3 ssd forward");
}

mxb_status mamba3_ssd_fwd(const mxb_mamba3_desc* d, const void* x, const float* dt, const float* lam,
                          const float* theta, const float* a_log, const void* b, const void* c, void* y, void* ws,
                          cudaStream_t st) {
  SsdP p = make_ssd(d);
  p.x = static_cast<const m3s::bf16*>(x); p.b = static_cast<const m3s::bf16*>(b); p.c = static_cast<const m3s::bf16*>(c);
  p.dt_raw = dt; p.lam_raw = lam; p.theta = theta; p.a_log = a_log; p.y = static_cast<m3s::bf16*>(y);
  carve_ssd(p, ws, false);
  return ssd_forward(p, st);
}

mxb_status mamba3_ssd_bwd(const mxb_mamba3_desc* d, const void* x, const float* dt, const float* lam,
                          const float* theta, const float* a_log, const void* b, const void* c, const void* dy,
                          void* dx, float* ddt, float* dlam, float* dtheta, float* da_log, void* db, void* dc, void* ws,
                          cudaStream_t st) {
  SsdP p = make_ssd(d);
  p.x = static_cast<const m3s::bf16*>(x); p.b = static_cast<const m3s::bf16*>(b); p.c = static_cast<const m3s::bf16*>(c);
  p.dy = static_cast<const m3s::bf16*>(dy); p.dx = static_cast<m3s::bf16*>(dx);
  p.dt_raw = dt; p.lam_raw = lam; p.theta = theta; p.a_log = a_log;
  p.ddt = ddt; p.dlam = dlam; p.dtheta = dtheta; p.da_log = da_log;
  carve_ssd(p, ws, true);
  p.y = nullptr;  // the forward recompute stops at the chunk states
  if (d->flags & MXB_MAMBA3_BWD_USE_SAVED) {  // dt, lambda, phi, the chunk decays and H0 are still in place
    if (cudaMemsetAsync(p.status, 0, 256, st) != cudaSuccess) return MXB_ERR_CUDA;
  } else {
    mxb_status s = ssd_forward(p, st);
    if (s != MXB_OK) return s;
  }
  const dim3 gc(p.n, p.NH, p.B);
  mxb_status ps = ssd_state_pass(p, 1, st);
  if (ps != MXB_OK) return ps;
  m3s::ChunkMaps maps;
  if (ssd_chunk_maps(p, maps)) {
    if (ssd_smem(m3s::m3s_chunk_grad_kernel<true>, m3s::kGradSmem) != MXB_OK) return MXB_ERR_CUDA;
    MXB_LAUNCH("m3s_chunk_grad_kernel", st, (m3s::m3s_chunk_grad_kernel<true><<<gc, 256, m3s::kGradSmem, st>>>(p, maps)));
  } else {
    if (ssd_smem(m3s::m3s_chunk_grad_kernel<false>, m3s::kGradSmem) != MXB_OK) return MXB_ERR_CUDA;
    MXB_LAUNCH("m3s_chunk_grad_kernel", st, (m3s::m3s_chunk_grad_kernel<false><<<gc, 256, m3s::kGradSmem, st>>>(p, maps)));
  }
  MXB_LAUNCH("m3s_final_kernel", st, (m3s::m3s_final_kernel<<<dim3(p.NH, p.B), m3s::kScalThreads, 0, st>>>(p)));
  MXB_LAUNCH("m3s_dalog_kernel", st, (m3s::m3s_dalog_kernel<<<(p.NH + 127) / 128, 128, 0, st>>>(p)));
  MXB_LAUNCH("m3s_reduce_kernel", st,
             (m3s::m3s_reduce_kernel<<<dim3((p.T + 3) / 4, p.G, p.B), 128, 0, st>>>(p.pb, p.pc, static_cast<m3s::bf16*>(db),
                                                                            static_cast<m3s::bf16*>(dc), p.T, p.G, p.NH)));
  return check_launch("mamba3 ssd backward");
}

}  // namespace mxb
