// Mamba-3 selective scan, head-broadcast layout (dt, lambda, theta per (b,t,head), A per
// head) - one CTA per (head, batch) instead of one warp per channel.
//
// In this layout the cumulative angle, the decay alpha = exp(dt A), the trapezoid
// weights and therefore the rotated B and C rows are the same for every channel of a head,
// so they are computed once per (step, head) into shared memory (blocks of 16 steps) and
// every warp then advances its channels with plain FMAs:
//     h[ch][n] = alpha h[ch][n] + (gamma x_t[ch]) Brot_t[n] + (beta x_{t-1}[ch]) Brot_{t-1}[n]
//     y_t[ch]  = sum_n h[ch][n] Crot_t[n]
// Lane l owns states SPL*l .. SPL*l+SPL-1 (whole pairs) of CPW channels; the CPW partial
// sums of a step are reduced across the warp together (a halving butterfly), and the
// outputs of a block are written back coalesced.  Same recurrence as mamba3.cu (reference:
// gpu/cuda_kernels/mamba3_selective_scan_fwd_v2_emit.cu:65-115).
#include "common.cuh"

namespace mxb {

constexpr int kHB = 8;   // steps per block (= checkpoint window of the backward)

struct M3H {
  int B, T, D, N, G, NH, P, nW;
  const void *x, *b, *c;
  const float *dt, *lam, *theta, *a_log;
  void* y;
  float *ck_h, *ck_phi;  // checkpoints [B,nW,D,N], [B,nW,NH]
};

__device__ __forceinline__ float m3h_softplus(float x) {
  if (x > 20.f) return x;
  if (x < -20.f) return expf(x);
  return log1pf(expf(x));
}
__device__ __forceinline__ float m3h_sigmoid(float x) { return 1.f / (1.f + expf(-x)); }
__device__ __forceinline__ float m3h_wrap(float phi) {
  const float k = rintf(phi * 0.15915494309189535f);
  phi = fmaf(-k, 6.28125f, phi);
  return fmaf(-k, 1.9353071795864769e-3f, phi);
}

// Sums CPW per-channel partials over the 32 lanes; on return lane l holds the total of
// channel (l % CPW) (CPW a power of two <= 8).
template <int CPW>
__device__ __forceinline__ float reduce_channels(float (&v)[CPW], int lane) {
  // halving butterfly: after the round with offset o, lanes differing in bit o share work
  int n = CPW;
#pragma unroll
  for (int o = 16; o >= 1; o >>= 1) {
    if (n > 1) {
      const bool upper = (lane & o) != 0;
      n >>= 1;
#pragma unroll
      for (int i = 0; i < CPW / 2; ++i) {
        if (i < n) {
          const float send = upper ? v[i] : v[i + n];
          const float keep = upper ? v[i + n] : v[i];
          v[i] = keep + __shfl_xor_sync(0xffffffffu, send, o);
        }
      }
    } else {
      v[0] += __shfl_xor_sync(0xffffffffu, v[0], o);
    }
  }
  return v[0];
}
// Which channel (0..CPW-1) lane `lane` holds after reduce_channels.
template <int CPW>
__device__ __forceinline__ int reduced_channel(int lane) {
  int ch = 0, n = CPW;
#pragma unroll
  for (int o = 16; o >= 1; o >>= 1) {
    if (n > 1) {
      n >>= 1;
      if (lane & o) ch += n;
    }
  }
  return ch;
}

template <typename IO, int SPL, int CPW>
__global__ void __launch_bounds__(256) mamba3_head_fwd_kernel(M3H p) {
  constexpr int NW = 8;            // warps
  const int N = SPL * 32, P = CPW * NW;
  __shared__ __align__(16) float s_brot[(kHB + 1) * SPL * 32];  // row 0 = last step of the previous block
  __shared__ __align__(16) float s_crot[kHB * SPL * 32];
  __shared__ float s_x[(kHB + 1) * CPW * NW];                   // row 0 = x of the previous step
  __shared__ float s_y[kHB * CPW * NW];
  __shared__ float s_al[kHB], s_ga[kHB], s_be[kHB], s_sin[kHB], s_cos[kHB];
  __shared__ float s_phi;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int head = blockIdx.x, b = blockIdx.y;
  const int d0 = head * P;                    // first channel of the head
  const int g = d0 / (p.D / p.G);
  const float A = -expf(p.a_log[head]);
  const IO* X = static_cast<const IO*>(p.x);
  const IO* Bp = static_cast<const IO*>(p.b);
  const IO* Cp = static_cast<const IO*>(p.c);
  IO* Y = static_cast<IO*>(p.y);

  float h[CPW][SPL];
#pragma unroll
  for (int c = 0; c < CPW; ++c)
#pragma unroll
    for (int j = 0; j < SPL; ++j) h[c][j] = 0.f;
  if (tid == 0) s_phi = 0.f;
  for (int i = tid; i < N; i += 256) s_brot[i] = 0.f;
  for (int i = tid; i < P; i += 256) s_x[i] = 0.f;
  __syncthreads();

  for (int t0 = 0; t0 < p.T; t0 += kHB) {
    const int nt = min(kHB, p.T - t0);
    // ---- per-step scalars of the head (one thread per step, then a serial angle prefix) ----
    if (tid < nt) {
      const size_t r = ((size_t)b * p.T + t0 + tid) * p.NH + head;
      const float dt = m3h_softplus(p.dt[r]), lam = m3h_sigmoid(p.lam[r]);
      const float al = expf(dt * A);
      s_al[tid] = al;
      s_ga[tid] = lam * dt;
      s_be[tid] = (1.f - lam) * dt * al;
      s_sin[tid] = dt * p.theta[r];  // angle increment, turned into sin/cos below
    }
    __syncthreads();
    if (tid == 0) {
      float phi = s_phi;
      if (p.ck_phi) p.ck_phi[((size_t)b * p.nW + t0 / kHB) * p.NH + head] = phi;
      for (int s = 0; s < nt; ++s) {
        phi = m3h_wrap(phi + s_sin[s]);
        float sn, cs;
        sincosf(phi, &sn, &cs);
        s_sin[s] = sn;
        s_cos[s] = cs;
      }
      s_phi = phi;
    }
    if (p.ck_h) {  // state at the start of the block
      const size_t wrow = ((size_t)b * p.nW + t0 / kHB) * p.D;
#pragma unroll
      for (int c = 0; c < CPW; ++c)
#pragma unroll
        for (int j = 0; j < SPL; ++j) p.ck_h[(wrow + d0 + warp * CPW + c) * N + SPL * lane + j] = h[c][j];
    }
    __syncthreads();
    // ---- rotated B, C rows and x of the block ----
    for (int u = tid; u < nt * (N / 2); u += 256) {
      const int s = u / (N / 2), kp = u - s * (N / 2);
      const size_t gi = (((size_t)b * p.T + t0 + s) * p.G + g) * N + 2 * kp;
      const float be = to_f32(Bp[gi]), bo = to_f32(Bp[gi + 1]), ce = to_f32(Cp[gi]), co = to_f32(Cp[gi + 1]);
      const float sn = s_sin[s], cs = s_cos[s];
      s_brot[(s + 1) * N + 2 * kp] = cs * be + sn * bo;
      s_brot[(s + 1) * N + 2 * kp + 1] = -sn * be + cs * bo;
      s_crot[s * N + 2 * kp] = cs * ce + sn * co;
      s_crot[s * N + 2 * kp + 1] = -sn * ce + cs * co;
    }
    for (int u = tid; u < nt * P; u += 256) {
      const int s = u / P, ch = u - s * P;
      s_x[(s + 1) * P + ch] = to_f32(X[((size_t)b * p.T + t0 + s) * p.D + d0 + ch]);
    }
    __syncthreads();
    // ---- recurrence: each warp advances its CPW channels through the block ----
    const int mych = reduced_channel<CPW>(lane);
    for (int s = 0; s < nt; ++s) {
      const float al = s_al[s], ga = s_ga[s], be = s_be[s];
      float br[SPL], bp[SPL], cr[SPL];
#pragma unroll
      for (int j = 0; j < SPL; ++j) {
        br[j] = s_brot[(s + 1) * N + SPL * lane + j];
        bp[j] = s_brot[s * N + SPL * lane + j];
        cr[j] = s_crot[s * N + SPL * lane + j];
      }
      float part[CPW];
#pragma unroll
      for (int c = 0; c < CPW; ++c) {
        const float gx = ga * s_x[(s + 1) * P + warp * CPW + c];
        const float bx = be * s_x[s * P + warp * CPW + c];
        float acc = 0.f;
#pragma unroll
        for (int j = 0; j < SPL; ++j) {
          h[c][j] = fmaf(al, h[c][j], fmaf(gx, br[j], bx * bp[j]));
          acc = fmaf(h[c][j], cr[j], acc);
        }
        part[c] = acc;
      }
      const float tot = reduce_channels<CPW>(part, lane);
      s_y[s * P + warp * CPW + mych] = tot;  // lanes holding the same channel write the same value
    }
    __syncthreads();
    if (Y) {
      for (int u = tid; u < nt * P; u += 256) {
        const int s = u / P, ch = u - s * P;
        Y[((size_t)b * p.T + t0 + s) * p.D + d0 + ch] = from_f32<IO>(s_y[u]);
      }
    }
    // carry the last step's Brot and x into row 0
    for (int i = tid; i < N; i += 256) s_brot[i] = s_brot[nt * N + i];
    for (int i = tid; i < P; i += 256) s_x[i] = s_x[nt * P + i];
    __syncthreads();
  }
}

// ----------------------------------------------------------------- backward
// One CTA per (16 channels of a head, batch): 8 warps x 2 channels, lane = SPL states of both.
// Windows of kHB steps are walked backwards: the window is replayed forward from its
// checkpoint into a per-thread history in shared memory, then the closed-form adjoint
// (gpu/ir.cpp:1526-1623) is applied step by step.  Gradients of the rotated B and C rows are
// summed over the CTA's channels in shared memory and un-rotated once per window.
struct M3HB {
  M3H f;
  const void* dy;
  void* dx;
  float *ddt, *dlam, *dtheta, *da_log;
  float *pb, *pc;  // per-CTA partial gradients of B and C: [B][D/16][T][N]
  float* hpart;    // per-CTA shares of the head-broadcast gradients: 3 x [B][T][D/16] (dtheta, ddt, dlambda)
  float* dalpart;  // per-warp shares of da_log: [B][D/16][8]
  void *db, *dc;   // final gradients (io dtype), written by the reduction kernel
};

template <typename IO, int SPW>
__global__ void __launch_bounds__(256) mamba3_head_bwd_kernel(M3HB q) {
  // SPW states per warp (N = 8 SPW); a warp holds all CH = 16 channels of the CTA for its states:
  // lane = (channel group cg, state st), CPT channels per thread.
  constexpr int CH = 16, W = kHB, CG = 32 / SPW, CPT = CH / CG, N = 8 * SPW;
  const M3H& p = q.f;
  extern __shared__ float hist[];  // [W][CPT][256]  h after each step of the window
  __shared__ __align__(16) float s_brot[(W + 1) * N], s_crot[W * N];
  __shared__ __align__(16) float s_gb[(W + 1) * N], s_gc[W * N], s_carry[N];
  __shared__ float s_x[(W + 1) * CH], s_dy[W * CH];
  __shared__ float s_pdx[8 * W * CH], s_psc[8 * W * 2];  // per-warp partials of dx and of (dlam, ddelta)
  __shared__ float s_al[W], s_ga[W], s_be[W], s_lam[W], s_dt[W], s_dtraw[W], s_th[W], s_sin[W + 1], s_cos[W + 1];
  __shared__ float s_gphi[W], s_gphi_p[W * 4];  // angle gradient per step; its per-warp shares (N / 64 of them)
  __shared__ float s_phicarry;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int st = lane % SPW, cg = lane / SPW, n = warp * SPW + st, c0 = cg * CPT;
  const int d0 = blockIdx.x * CH, b = blockIdx.y;
  const int head = d0 / p.P, g = d0 / (p.D / p.G);
  const float A = -expf(p.a_log[head]);
  const IO* X = static_cast<const IO*>(p.x);
  const IO* Bp = static_cast<const IO*>(p.b);
  const IO* Cp = static_cast<const IO*>(p.c);
  const IO* DY = static_cast<const IO*>(q.dy);
  IO* DX = static_cast<IO*>(q.dx);
  auto H = [&](int s_, int c) -> float& { return hist[(s_ * CPT + c) * 256 + tid]; };

  float dh[CPT], pend[CPT], dal = 0.f;
#pragma unroll
  for (int c = 0; c < CPT; ++c) dh[c] = pend[c] = 0.f;
  for (int i = tid; i < N; i += 256) s_carry[i] = 0.f;
  if (tid == 0) s_phicarry = 0.f;
  __syncthreads();

  for (int w = p.nW - 1; w >= 0; --w) {
    const int ts = w * W, nt = min(W, p.T - ts);
    // ---- A: per-step scalars, angles ----
    if (tid < nt) {
      const size_t r = ((size_t)b * p.T + ts + tid) * p.NH + head;
      const float raw = p.dt[r];
      const float dt = m3h_softplus(raw), lam = m3h_sigmoid(p.lam[r]), al = expf(dt * A), th = p.theta[r];
      s_dtraw[tid] = raw; s_dt[tid] = dt; s_lam[tid] = lam; s_al[tid] = al; s_th[tid] = th;
      s_ga[tid] = lam * dt;
      s_be[tid] = (1.f - lam) * dt * al;
    }
    __syncthreads();
    if (tid == 0) {
      float phi = p.ck_phi[((size_t)b * p.nW + w) * p.NH + head];
      sincosf(phi, &s_sin[0], &s_cos[0]);  // angle of step ts-1
      for (int s_ = 0; s_ < nt; ++s_) {
        phi = m3h_wrap(fmaf(s_dt[s_], s_th[s_], phi));
        sincosf(phi, &s_sin[s_ + 1], &s_cos[s_ + 1]);
      }
    }
    __syncthreads();
    // ---- B: rotated rows (row 0 = step ts-1), x, dy; reset accumulators ----
    for (int u = tid; u < (nt + 1) * (N / 2); u += 256) {
      const int r = u / (N / 2), kp = u - r * (N / 2);  // r = 0 is step ts-1
      const int t = ts + r - 1;
      float b0 = 0.f, b1 = 0.f, cc0 = 0.f, cc1 = 0.f;
      if (t >= 0) {
        const size_t gi = (((size_t)b * p.T + t) * p.G + g) * N + 2 * kp;
        const float be = to_f32(Bp[gi]), bo = to_f32(Bp[gi + 1]);
        const float sn = s_sin[r], cs = s_cos[r];
        b0 = cs * be + sn * bo; b1 = -sn * be + cs * bo;
        if (r > 0) {
          const float ce = to_f32(Cp[gi]), co = to_f32(Cp[gi + 1]);
          cc0 = cs * ce + sn * co; cc1 = -sn * ce + cs * co;
        }
      }
      s_brot[r * N + 2 * kp] = b0; s_brot[r * N + 2 * kp + 1] = b1;
      if (r > 0) { s_crot[(r - 1) * N + 2 * kp] = cc0; s_crot[(r - 1) * N + 2 * kp + 1] = cc1; }
    }
    for (int u = tid; u < (nt + 1) * N; u += 256) s_gb[u] = (u >= nt * N) ? s_carry[u - nt * N] : 0.f;
    for (int u = tid; u < (nt + 1) * CH; u += 256) {
      const int r = u / CH, ch = u - r * CH, t = ts + r - 1;
      s_x[u] = t >= 0 ? to_f32(X[((size_t)b * p.T + t) * p.D + d0 + ch]) : 0.f;
      if (r > 0) s_dy[(r - 1) * CH + ch] = to_f32(DY[((size_t)b * p.T + t) * p.D + d0 + ch]);
    }
    // ---- C: replay the window from its checkpoint ----
    float ck[CPT], h[CPT];
    {
      const size_t wrow = ((size_t)b * p.nW + w) * p.D;
#pragma unroll
      for (int c = 0; c < CPT; ++c) ck[c] = h[c] = p.ck_h[(wrow + d0 + c0 + c) * N + n];
    }
    __syncthreads();
    for (int s_ = 0; s_ < nt; ++s_) {
      const float al = s_al[s_], ga = s_ga[s_], be = s_be[s_];
      const float br = s_brot[(s_ + 1) * N + n], bp = s_brot[s_ * N + n];
#pragma unroll
      for (int c = 0; c < CPT; ++c) {
        h[c] = fmaf(al, h[c], fmaf(ga * s_x[(s_ + 1) * CH + c0 + c], br, be * s_x[s_ * CH + c0 + c] * bp));
        H(s_, c) = h[c];
      }
    }
    // ---- D: reverse over the window ----
    for (int s_ = nt - 1; s_ >= 0; --s_) {
      const float al = s_al[s_], lam = s_lam[s_], dt = s_dt[s_];
      const float bni = (1.f - lam) * dt * al;
      const float br = s_brot[(s_ + 1) * N + n], bp = s_brot[s_ * N + n], cr = s_crot[s_ * N + n];
      float pdx[CPT], sdl = 0.f, sdd = 0.f, gbc = 0.f, gbp = 0.f, gcc = 0.f;
#pragma unroll
      for (int c = 0; c < CPT; ++c) {
        const float x = s_x[(s_ + 1) * CH + c0 + c], xp = s_x[s_ * CH + c0 + c], dy = s_dy[s_ * CH + c0 + c];
        const float ha = H(s_, c);
        const float hb = s_ > 0 ? H(s_ - 1, c) : ck[c];
        const float up = fmaf(dy, cr, dh[c]);
        const float pin = bp * xp;
        pdx[c] = fmaf(lam * dt * br, up, pend[c]);
        pend[c] = bni * bp * up;
        gbc = fmaf(x, up, gbc);
        gbp = fmaf(xp, up, gbp);
        gcc = fmaf(dy, ha, gcc);
        sdl = fmaf(dt * (br * x - al * pin), up, sdl);
        sdd = fmaf(A * al * hb + (1.f - lam) * (al + dt * A * al) * pin + lam * br * x, up, sdd);
        dal = fmaf(dt * al * A * (hb + (1.f - lam) * dt * pin), up, dal);
        dh[c] = al * up;
      }
      // sums over the channel groups of this warp (same state n): lanes st, st+SPW, ...
#pragma unroll
      for (int o = SPW; o < 32; o <<= 1) {
        gbc += __shfl_xor_sync(0xffffffffu, gbc, o);
        gbp += __shfl_xor_sync(0xffffffffu, gbp, o);
        gcc += __shfl_xor_sync(0xffffffffu, gcc, o);
      }
      if (cg == 0) {  // one owner per (step, state): plain read-modify-write
        s_gb[(s_ + 1) * N + n] += lam * dt * gbc;
        s_gb[s_ * N + n] += bni * gbp;
        s_gc[s_ * N + n] = gcc;
      }
      // dx partial of this warp: sum over its SPW states, per channel (halving butterfly over the state lanes)
      {
        int m = CPT;
#pragma unroll
        for (int o = SPW / 2; o >= 1; o >>= 1) {
          if (m > 1) {
            const bool upper = (st & o) != 0;
            m >>= 1;
#pragma unroll
            for (int i = 0; i < CPT / 2; ++i)
              if (i < m) {
                const float send = upper ? pdx[i] : pdx[i + m];
                const float keep = upper ? pdx[i + m] : pdx[i];
                pdx[i] = keep + __shfl_xor_sync(0xffffffffu, send, o);
              }
          } else {
            pdx[0] += __shfl_xor_sync(0xffffffffu, pdx[0], o);
          }
        }
        int chl = 0, mm = CPT;
#pragma unroll
        for (int o = SPW / 2; o >= 1; o >>= 1)
          if (mm > 1) { mm >>= 1; if (st & o) chl += mm; }
        s_pdx[(warp * W + s_) * CH + c0 + chl] = pdx[0];
      }
      sdl = warp_sum(sdl);
      sdd = warp_sum(sdd);
      if (lane == 0) {
        s_psc[(warp * W + s_) * 2] = sdl;
        s_psc[(warp * W + s_) * 2 + 1] = sdd;
      }
    }
    __syncthreads();
    // ---- E: un-rotate the summed row gradients, angle gradient, per-step head scalars ----
    for (int u = tid; u < nt * (N / 2); u += 256) {
      const int s_ = u / (N / 2), kp = u - s_ * (N / 2);
      const float sn = s_sin[s_ + 1], cs = s_cos[s_ + 1];
      const float gb0 = s_gb[(s_ + 1) * N + 2 * kp], gb1 = s_gb[(s_ + 1) * N + 2 * kp + 1];
      const float gc0 = s_gc[s_ * N + 2 * kp], gc1 = s_gc[s_ * N + 2 * kp + 1];
      const size_t pi = (((size_t)b * gridDim.x + blockIdx.x) * p.T + ts + s_) * N + 2 * kp;
      *reinterpret_cast<float2*>(q.pb + pi) = make_float2(cs * gb0 - sn * gb1, sn * gb0 + cs * gb1);
      *reinterpret_cast<float2*>(q.pc + pi) = make_float2(cs * gc0 - sn * gc1, sn * gc0 + cs * gc1);
      const float b0 = s_brot[(s_ + 1) * N + 2 * kp], b1 = s_brot[(s_ + 1) * N + 2 * kp + 1];
      const float cc0 = s_crot[s_ * N + 2 * kp], cc1 = s_crot[s_ * N + 2 * kp + 1];
      float gph = b1 * gb0 - b0 * gb1 + cc1 * gc0 - cc0 * gc1;
      // N/2 >= 32 pairs per step and 32 | N/2: a warp's items all belong to one step
      gph = warp_sum(gph);
      if (lane == 0) s_gphi_p[s_ * 4 + (kp >> 5)] = gph;  // added in a fixed order below
    }
    for (int u = tid; u < nt * CH; u += 256) {
      const int s_ = u / CH, ch = u - s_ * CH;
      float tot = 0.f;
#pragma unroll
      for (int wv = 0; wv < 8; ++wv) tot += s_pdx[(wv * W + s_) * CH + ch];
      DX[((size_t)b * p.T + ts + s_) * p.D + d0 + ch] = from_f32<IO>(tot);
    }
    __syncthreads();
    if (tid == 0) {
      float carry = s_phicarry;
      for (int s_ = nt - 1; s_ >= 0; --s_) {
        for (int j = 0; j < N / 64; ++j) carry += s_gphi_p[s_ * 4 + j];
        s_gphi[s_] = carry;  // suffix sum of the angle gradient
      }
      s_phicarry = carry;
    }
    for (int i = tid; i < N; i += 256) s_carry[i] = s_gb[i];  // pending gradient of Brot at step ts-1
    __syncthreads();
    if (tid < nt) {
      const size_t r = ((size_t)b * p.T + ts + tid) * p.NH + head;
      const float lam = s_lam[tid], carry = s_gphi[tid];
      float sdl = 0.f, sdd = 0.f;
#pragma unroll
      for (int wv = 0; wv < 8; ++wv) { sdl += s_psc[(wv * W + tid) * 2]; sdd += s_psc[(wv * W + tid) * 2 + 1]; }
      // this CTA's share; the CTAs of a head are added in slice order by m3h_head_sum_kernel
      const size_t plane = (size_t)p.B * p.T * gridDim.x;
      const size_t hp = ((size_t)b * p.T + ts + tid) * gridDim.x + blockIdx.x;
      q.hpart[hp] = carry * s_dt[tid];
      q.hpart[plane + hp] = (sdd + carry * s_th[tid]) * m3h_sigmoid(s_dtraw[tid]);
      q.hpart[2 * plane + hp] = sdl * lam * (1.f - lam);
    }
    __syncthreads();
  }
  dal = warp_sum(dal);
  if (lane == 0) q.dalpart[((size_t)b * gridDim.x + blockIdx.x) * 8 + warp] = dal;
}

// dtheta, ddt, dlambda [B,T,NH] = the shares of the CTAs of each head, added in slice order.
__global__ void __launch_bounds__(256) m3h_head_sum_kernel(const float* __restrict__ hpart, float* __restrict__ dtheta,
                                                           float* __restrict__ ddt, float* __restrict__ dlam, size_t rows,
                                                           int nslice, int NH) {
  const int per = nslice / NH;
  const size_t plane = rows * nslice;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < rows * NH; i += (size_t)gridDim.x * blockDim.x) {
    const size_t r = i / NH;
    const int h = (int)(i - r * NH);
    float a = 0.f, d = 0.f, l = 0.f;
    for (int s = 0; s < per; ++s) {
      const size_t j = r * nslice + (size_t)h * per + s;
      a += hpart[j];
      d += hpart[plane + j];
      l += hpart[2 * plane + j];
    }
    dtheta[i] = a;
    ddt[i] = d;
    dlam[i] = l;
  }
}

// da_log [NH] = the per-warp shares over the batch, the CTAs of the head and their warps, in that order.
__global__ void __launch_bounds__(128) m3h_dalog_sum_kernel(const float* __restrict__ part, float* __restrict__ da_log, int B,
                                                            int nslice, int NH) {
  const int h = blockIdx.x * blockDim.x + threadIdx.x;
  if (h >= NH) return;
  const int per = nslice / NH;
  float s = 0.f;
  for (int b = 0; b < B; ++b)
    for (int c = 0; c < per; ++c)
      for (int w = 0; w < 8; ++w) s += part[((size_t)b * nslice + h * per + c) * 8 + w];
  da_log[h] = s;
}

bool mamba3_head_supported(const mxb_mamba3_desc* d) {
  if (d->nheads <= 0 || d->D % d->nheads) return false;
  const int P = d->D / d->nheads;
  if (!(P == 64 || P == 32 || P == 16 || P == 8)) return false;
  if (!(d->N == 128 || d->N == 64)) return false;
  if ((d->D / d->G) % P) return false;  // a head must lie inside one B/C group
  return true;
}

template <typename IO, int SPL, int CPW>
static mxb_status m3h_launch(const M3H& p, cudaStream_t st) {
  MXB_LAUNCH("mamba3_head_fwd_kernel", st, (mamba3_head_fwd_kernel<IO, SPL, CPW><<<dim3(p.NH, p.B), 256, 0, st>>>(p)));
  return check_launch("mamba3_head_fwd_kernel");
}
template <typename IO, int SPL>
static mxb_status m3h_cpw(const M3H& p, cudaStream_t st) {
  switch (p.P) {
    case 64: return m3h_launch<IO, SPL, 8>(p, st);
    case 32: return m3h_launch<IO, SPL, 4>(p, st);
    case 16: return m3h_launch<IO, SPL, 2>(p, st);
    default: return m3h_launch<IO, SPL, 1>(p, st);
  }
}

// y == nullptr with checkpoints = the checkpoint pass of the backward.
mxb_status mamba3_head_fwd(const mxb_mamba3_desc* d, const void* x, const float* dt, const float* lam,
                           const float* theta, const float* a_log, const void* b, const void* c, void* y,
                           float* ck_h, float* ck_phi, cudaStream_t st) {
  M3H p{};
  p.B = d->B; p.T = d->T; p.D = d->D; p.N = d->N; p.G = d->G; p.NH = d->nheads; p.P = d->D / d->nheads;
  p.nW = (d->T + kHB - 1) / kHB;
  p.x = x; p.dt = dt; p.lam = lam; p.theta = theta; p.a_log = a_log; p.b = b; p.c = c; p.y = y;
  p.ck_h = ck_h; p.ck_phi = ck_phi;
  const bool f32 = d->io_dtype == MXB_F32;
  if (d->N == 128) return f32 ? m3h_cpw<float, 4>(p, st) : m3h_cpw<__nv_bfloat16, 4>(p, st);
  return f32 ? m3h_cpw<float, 2>(p, st) : m3h_cpw<__nv_bfloat16, 2>(p, st);
}

// dB[b,t,g,:] = sum of the partial rows of the CTAs whose channels lie in group g (fixed order).
template <typename IO>
__global__ void __launch_bounds__(128) m3h_reduce_kernel(const float* __restrict__ pb, const float* __restrict__ pc,
                                                         IO* __restrict__ db, IO* __restrict__ dc, int T, int N, int G,
                                                         int nchunks) {
  const int t = blockIdx.x, g = blockIdx.y, b = blockIdx.z, per = nchunks / G;
  for (int n = threadIdx.x; n < N; n += blockDim.x) {
    float sb = 0.f, sc = 0.f;
    for (int ch = g * per; ch < (g + 1) * per; ++ch) {
      const size_t pi = (((size_t)b * nchunks + ch) * T + t) * N + n;
      sb += pb[pi];
      sc += pc[pi];
    }
    const size_t gi = (((size_t)b * T + t) * G + g) * N + n;
    db[gi] = from_f32<IO>(sb);
    dc[gi] = from_f32<IO>(sc);
  }
}

template <typename IO, int SPW>
static mxb_status m3hb_launch(const M3HB& q, cudaStream_t st) {
  const size_t sm = sizeof(float) * kHB * (16 / (32 / SPW)) * 256;
  cudaError_t e = cudaFuncSetAttribute(mamba3_head_bwd_kernel<IO, SPW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);
  if (e != cudaSuccess) { set_last_cuda_error((int)e); return MXB_ERR_CUDA; }
  MXB_LAUNCH("mamba3_head_bwd_kernel", st,
             (mamba3_head_bwd_kernel<IO, SPW><<<dim3(q.f.D / 16, q.f.B), 256, sm, st>>>(q)));
  mxb_status s = check_launch("mamba3_head_bwd_kernel");
  if (s != MXB_OK) return s;
  const int nchunks = q.f.D / 16;
  MXB_LAUNCH("m3h_reduce_kernel", st,
             (m3h_reduce_kernel<IO><<<dim3(q.f.T, q.f.G, q.f.B), 128, 0, st>>>(q.pb, q.pc, static_cast<IO*>(q.db),
                                                                            static_cast<IO*>(q.dc), q.f.T, q.f.N,
                                                                            q.f.G, nchunks)));
  const size_t rows = (size_t)q.f.B * q.f.T;
  const int hb = (int)((rows * q.f.NH + 255) / 256 < 1184 ? (rows * q.f.NH + 255) / 256 : 1184);
  MXB_LAUNCH("m3h_head_sum_kernel", st,
             (m3h_head_sum_kernel<<<hb, 256, 0, st>>>(q.hpart, q.dtheta, q.ddt, q.dlam, rows, nchunks, q.f.NH)));
  MXB_LAUNCH("m3h_dalog_sum_kernel", st,
             (m3h_dalog_sum_kernel<<<(q.f.NH + 127) / 128, 128, 0, st>>>(q.dalpart, q.da_log, q.f.B, nchunks, q.f.NH)));
  return check_launch("m3h_reduce_kernel");
}

int mamba3_head_window() { return kHB; }

size_t mamba3_head_partial_floats(const mxb_mamba3_desc* d) {
  return (size_t)d->B * (d->D / 16) * d->T * d->N;
}

bool mamba3_head_bwd_supported(const mxb_mamba3_desc* d) {
  return mamba3_head_supported(d) && (d->D / d->nheads) % 16 == 0;
}

size_t mamba3_head_scalar_floats(const mxb_mamba3_desc* d) {  // hpart + dalpart
  return 3 * (size_t)d->B * d->T * (d->D / 16) + (size_t)d->B * (d->D / 16) * 8;
}

// Reverse pass; the caller has run the checkpoint pass.  hscal: mamba3_head_scalar_floats() floats of scratch.
mxb_status mamba3_head_bwd(const mxb_mamba3_desc* d, const void* x, const float* dt, const float* lam,
                           const float* theta, const float* a_log, const void* b, const void* c, const void* dy,
                           void* dx, float* ddt, float* dlam, float* dtheta, float* da_log, void* db, void* dc,
                           float* pb, float* pc, float* hscal, float* ck_h, float* ck_phi, cudaStream_t st) {
  M3HB q{};
  M3H& p = q.f;
  p.B = d->B; p.T = d->T; p.D = d->D; p.N = d->N; p.G = d->G; p.NH = d->nheads; p.P = d->D / d->nheads;
  p.nW = (d->T + kHB - 1) / kHB;
  p.x = x; p.dt = dt; p.lam = lam; p.theta = theta; p.a_log = a_log; p.b = b; p.c = c;
  p.ck_h = ck_h; p.ck_phi = ck_phi;
  q.dy = dy; q.dx = dx; q.ddt = ddt; q.dlam = dlam; q.dtheta = dtheta; q.da_log = da_log; q.db = db; q.dc = dc; q.pb = pb; q.pc = pc;
  q.hpart = hscal;
  q.dalpart = hscal + 3 * (size_t)d->B * d->T * (d->D / 16);
  const bool f32 = d->io_dtype == MXB_F32;
  if (d->N == 128) return f32 ? m3hb_launch<float, 16>(q, st) : m3hb_launch<__nv_bfloat16, 16>(q, st);
  return f32 ? m3hb_launch<float, 8>(q, st) : m3hb_launch<__nv_bfloat16, 8>(q, st);
}

}  // namespace mxb
