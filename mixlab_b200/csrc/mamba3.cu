// Mamba-3 exponential-trapezoidal selective scan with rotated state pairs,
// forward and backward - recurrent form.
//
// Recurrence (reference: gpu/cuda_kernels/mamba3_selective_scan_fwd_v2_emit.cu:65-115,
// closed-form VJP gpu/ir.cpp:1526-1623, float64 oracle
// train/gpu_trainer_mamba3_test.go:612-808):
//     dt = softplus(dt_raw); lam = sigmoid(lambda_raw); A = -exp(a_log)
//     phi_t = phi_{t-1} + dt_t theta_t
//     Brot = R^T(phi) B ; Crot = R^T(phi) C   (even' = c e + s o ; odd' = -s e + c o)
//     alpha = exp(dt A); beta = (1-lam) dt alpha; gamma = lam dt
//     h_t = alpha h_{t-1} + gamma Brot_t x_t + [t>0] beta Brot_{t-1} x_{t-1}
//     y_t = sum_n h_t[n] Crot_t[n]
//
// Mapping: LPC lanes per (batch, channel): a whole warp, whose lanes own state pairs lane, lane+32, ... (PR of
// them), so d_state up to 256 is covered (the reference's kernels stop at 64, gpu/mamba3_cuda_primitive.cpp:22);
// for d_state <= 32 / <= 16 a half / a quarter of a warp, so that two / four channels share a warp and no lane is
// without a state pair at the sizes the reference runs (d_state 16).  The cumulative angle is kept wrapped
// to [-pi, pi] so fp32 keeps its resolution over thousands of steps.
//
// Short problems (few batch x channel pairs) would leave most of the GPU idle behind T-long walks, so the
// kernels also run window-parallel: one warp per (batch, channel, window of kM3Window steps).  Every carried
// quantity is linear in what crosses a window boundary, which turns the walk into local walks plus short scans
// over the windows:
//   forward   window sums of dt theta -> scan: angle at each window start
//             local walks from a zero state -> scan with exp(A sum dt): state at each window start
//             walks from the true start states write y
//   backward  (after the same two scans) local reverse walks of dh from zero -> reverse scan: dh entering each
//             window and the `up` value of its first step, from which the window before takes the trapezoid's
//             look-back terms; true reverse walks with window-local angle-gradient sums; reverse scan of those
//             sums; one pass adds the later windows' sums to ddt and dtheta.
// The walks cost about twice the serial arithmetic, so the serial kernels stay for shapes whose (batch, channel)
// pairs fill the GPU by themselves.
//
// Two parameter layouts share the kernels through index helpers: the
// reference's per-channel one, and a head-broadcast one where dt, lambda, theta
// and a_log carry one value per (b,t,head) / per head.
//
// Backward: a checkpointing forward pass stores (h, phi) every W steps; the
// reverse pass walks the windows backwards, replays each window into shared
// memory and applies the closed-form adjoint step by step.  Every sum over
// channels or over the batch has a fixed order, so the same inputs give the same
// bits: the warps of a CTA are channels of one group and add their dB, dC rows
// through shared memory once per step; CTAs that share a group write partial
// rows that a second kernel adds in slice order; head-broadcast gradients and
// da_log go through per-channel / per-batch partials in the same way.
#include <algorithm>

#include "common.cuh"

namespace mxb {

constexpr int kM3Window = 16;

struct M3P {
  int B, T, D, N, G, NH, Kp, nW;
  int LPC;  // lanes per channel: 32, or 16 / 8 where d_state <= 32 / 16 would leave most lanes of a warp without a state pair
  const void *x, *b, *c;
  const float *dt, *lam, *theta, *a_log;
  void* y;
  float *ck_h, *ck_phi;  // checkpoints [B,nW,D,N], [B,nW,D,Kp]
  const void* dy;
  void* dx;
  float *ddt, *dlam, *dtheta, *da_log;
  // channel kernels: CW channels (warps) per CTA, S = channels per group / CW slices per group
  int CW, S;
  float *pb32, *pc32;  // [B,T,G,S,N] rows summed over the CW channels of a CTA
  float* hd;           // head-broadcast layout only: per-channel ddt, dlam, dtheta, 3 x [B,T,D]
  float* dal_part;     // per-batch (window-parallel: per batch and window) da_log: [.,D,N], or [.,D] head-broadcast
  // window-parallel kernels
  float* dtsum;        // [B,nW,D] sum of dt over the window
  float *dhk, *upk;    // [B,nW,D,N]: dh entering the window from later steps; `up` of the window's first step
  float* ang;          // [B,nW,D,Kp]: angle-gradient sum of the window, then of all later windows
};

__device__ __forceinline__ float m3_softplus(float x) {
  if (x > 20.f) return x;
  if (x < -20.f) return expf(x);
  return log1pf(expf(x));
}
__device__ __forceinline__ float m3_sigmoid(float x) { return 1.f / (1.f + expf(-x)); }
__device__ __forceinline__ float m3_wrap(float phi) {
  // Cody-Waite reduction by 2 pi = 6.28125 + 1.9353071795864769e-3
  const float k = rintf(phi * 0.15915494309189535f);
  phi = fmaf(-k, 6.28125f, phi);
  return fmaf(-k, 1.9353071795864769e-3f, phi);
}

// Sum over the LPC lanes that share a channel (LPC = 32: the whole warp); every lane of the group gets the sum.
template <int LPC>
__device__ __forceinline__ float group_sum(float v) {
#pragma unroll
  for (int o = LPC / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

struct M3Idx {
  int D, N, G, NH, Kp, cpg, cph;
  __device__ M3Idx(const M3P& p)
      : D(p.D), N(p.N), G(p.G), NH(p.NH), Kp(p.Kp), cpg(p.D / p.G), cph(p.NH > 0 ? p.D / p.NH : 1) {}
  __device__ size_t chan(size_t row, int d) const { return NH > 0 ? row * NH + d / cph : row * D + d; }
  __device__ size_t theta(size_t row, int d, int kp) const {
    return NH > 0 ? row * NH + d / cph : (row * D + d) * Kp + kp;
  }
  __device__ size_t alog(int d, int n) const { return NH > 0 ? (size_t)(d / cph) : (size_t)d * N + n; }
  __device__ size_t grp(size_t row, int d, int n) const { return (row * G + d / cpg) * N + n; }
};

// ------------------------------------------------------------------ forward
// Also the checkpoint pass of the backward (y == nullptr, ck_h != nullptr).
// MODE 0: the whole sequence (also the checkpoint pass of the serial backward: y == nullptr, ck_h != nullptr).
// MODE 1: one window from a zero state and the window's start angle; leaves the local end state in ck_h.
// MODE 2: one window from the true start state in ck_h; writes y.
template <typename IO, int PR, int LPC, int MODE>
__global__ void __launch_bounds__(256) mamba3_fwd_kernel(M3P p) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  constexpr int CPW = 32 / LPC;  // channels per warp
  const int sl = lane % LPC, d_raw = (blockIdx.x * 8 + warp) * CPW + lane / LPC;
  const int b = MODE == 0 ? blockIdx.y : blockIdx.z;
  if ((blockIdx.x * 8 + warp) * CPW >= p.D) return;
  const bool live = d_raw < p.D;       // lanes past the last channel walk a copy of it and store nothing
  const int d = live ? d_raw : p.D - 1;
  const M3Idx ix(p);
  const IO* X = static_cast<const IO*>(p.x);
  const IO* Bp = static_cast<const IO*>(p.b);
  const IO* Cp = static_cast<const IO*>(p.c);
  IO* Y = static_cast<IO*>(p.y);
  float A0[PR], A1[PR], h0[PR], h1[PR], phi[PR], pb0[PR], pb1[PR];
#pragma unroll
  for (int r = 0; r < PR; ++r) {
    const int kp = sl + LPC * r;
    const bool act = kp < p.Kp;
    A0[r] = act ? -expf(p.a_log[ix.alog(d, 2 * kp)]) : 0.f;
    A1[r] = act ? -expf(p.a_log[ix.alog(d, 2 * kp + 1)]) : 0.f;
    h0[r] = h1[r] = phi[r] = pb0[r] = pb1[r] = 0.f;
  }
  const int ts = MODE == 0 ? 0 : (int)blockIdx.y * kM3Window;
  const int te = MODE == 0 ? p.T : min(p.T, ts + kM3Window);
  const size_t wrow_w = MODE == 0 ? 0 : ((size_t)b * p.nW + blockIdx.y) * p.D + d;
  float px = 0.f;
  if (MODE != 0) {
#pragma unroll
    for (int r = 0; r < PR; ++r) {
      const int kp = sl + LPC * r;
      if (kp < p.Kp) {
        phi[r] = p.ck_phi[wrow_w * p.Kp + kp];
        if (MODE == 2) {
          h0[r] = p.ck_h[wrow_w * p.N + 2 * kp];
          h1[r] = p.ck_h[wrow_w * p.N + 2 * kp + 1];
        }
        if (ts > 0) {  // rotated B of the step before the window, at the window's start angle
          float s, c;
          sincosf(phi[r], &s, &c);
          const size_t gi = ix.grp((size_t)b * p.T + ts - 1, d, 2 * kp);
          const float be = to_f32(Bp[gi]), bo = to_f32(Bp[gi + 1]);
          pb0[r] = c * be + s * bo;
          pb1[r] = -s * be + c * bo;
        }
      }
    }
    if (ts > 0) px = to_f32(X[((size_t)b * p.T + ts - 1) * p.D + d]);
  }
  for (int t = ts; t < te; ++t) {
    const size_t row = (size_t)b * p.T + t;
    if (MODE == 0 && p.ck_h && (t % kM3Window) == 0) {
      const size_t wrow = ((size_t)b * p.nW + t / kM3Window) * p.D + d;
#pragma unroll
      for (int r = 0; r < PR; ++r) {
        const int kp = sl + LPC * r;
        if (kp < p.Kp && live) {
          p.ck_h[wrow * p.N + 2 * kp] = h0[r];
          p.ck_h[wrow * p.N + 2 * kp + 1] = h1[r];
          p.ck_phi[wrow * p.Kp + kp] = phi[r];
        }
      }
    }
    const float x = to_f32(X[row * p.D + d]);
    const float dt = m3_softplus(p.dt[ix.chan(row, d)]);
    const float lam = m3_sigmoid(p.lam[ix.chan(row, d)]);
    const float gamma = lam * dt, bfac = (1.f - lam) * dt;
    float part = 0.f;
#pragma unroll
    for (int r = 0; r < PR; ++r) {
      const int kp = sl + LPC * r;
      if (kp < p.Kp) {
        phi[r] = m3_wrap(fmaf(dt, p.theta[ix.theta(row, d, kp)], phi[r]));
        float s, c;
        sincosf(phi[r], &s, &c);
        const size_t gi = ix.grp(row, d, 2 * kp);
        const float be = to_f32(Bp[gi]), bo = to_f32(Bp[gi + 1]);
        const float b0 = c * be + s * bo, b1 = -s * be + c * bo;
        const float al0 = expf(dt * A0[r]), al1 = expf(dt * A1[r]);
        h0[r] = al0 * h0[r] + gamma * b0 * x + bfac * al0 * pb0[r] * px;
        h1[r] = al1 * h1[r] + gamma * b1 * x + bfac * al1 * pb1[r] * px;
        if (MODE != 1) {
          const float ce = to_f32(Cp[gi]), co = to_f32(Cp[gi + 1]);
          const float c0 = c * ce + s * co, c1 = -s * ce + c * co;
          part += h0[r] * c0 + h1[r] * c1;
        }
        pb0[r] = b0;
        pb1[r] = b1;
      }
    }
    px = x;  // t = 0 uses px = 0, which realises the [t>0] factor
    if (MODE != 1 && Y) {
      part = group_sum<LPC>(part);
      if (sl == 0 && live) Y[row * p.D + d] = from_f32<IO>(part);
    }
  }
  if (MODE == 1) {
#pragma unroll
    for (int r = 0; r < PR; ++r) {
      const int kp = sl + LPC * r;
      if (kp < p.Kp && live) {
        p.ck_h[wrow_w * p.N + 2 * kp] = h0[r];
        p.ck_h[wrow_w * p.N + 2 * kp + 1] = h1[r];
      }
    }
  }
}

// ------------------------------------------------- window-parallel: sums and scans
// Sum of dt theta (per state pair) and of dt over each window.
template <int PR, int LPC>
__global__ void __launch_bounds__(256) m3w_phase_kernel(M3P p) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  constexpr int CPW = 32 / LPC;
  const int sl = lane % LPC, d_raw = (blockIdx.x * 8 + warp) * CPW + lane / LPC, w = blockIdx.y, b = blockIdx.z;
  if ((blockIdx.x * 8 + warp) * CPW >= p.D) return;
  const bool live = d_raw < p.D;
  const int d = live ? d_raw : p.D - 1;
  const M3Idx ix(p);
  const int ts = w * kM3Window, te = min(p.T, ts + kM3Window);
  float ph[PR], dts = 0.f;
#pragma unroll
  for (int r = 0; r < PR; ++r) ph[r] = 0.f;
  for (int t = ts; t < te; ++t) {
    const size_t row = (size_t)b * p.T + t;
    const float dt = m3_softplus(p.dt[ix.chan(row, d)]);
    dts += dt;
#pragma unroll
    for (int r = 0; r < PR; ++r) {
      const int kp = sl + LPC * r;
      if (kp < p.Kp) ph[r] = fmaf(dt, p.theta[ix.theta(row, d, kp)], ph[r]);
    }
  }
  const size_t wrow = ((size_t)b * p.nW + w) * p.D + d;
#pragma unroll
  for (int r = 0; r < PR; ++r) {
    const int kp = sl + LPC * r;
    if (kp < p.Kp && live) p.ck_phi[wrow * p.Kp + kp] = ph[r];
  }
  if (sl == 0 && live) p.dtsum[wrow] = dts;
}

constexpr int kScanBatch = 8;

// ck_phi: window sums -> wrapped angle at each window start (exclusive scan over the windows).
__global__ void __launch_bounds__(256) m3w_phase_scan_kernel(M3P p) {
  const size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
  if (i >= (size_t)p.B * p.D * p.Kp) return;
  const size_t per = (size_t)p.D * p.Kp, b = i / per, rem = i - b * per;
  float run = 0.f;
  // kScanBatch windows at a time, every load of a batch before its first store: a store in between would pin the
  // order (the compiler must assume the arrays overlap) and each window would pay a full memory latency
  for (int w0 = 0; w0 < p.nW; w0 += kScanBatch) {
    float loc[kScanBatch];
#pragma unroll
    for (int x = 0; x < kScanBatch; ++x) loc[x] = w0 + x < p.nW ? p.ck_phi[(b * p.nW + w0 + x) * per + rem] : 0.f;
#pragma unroll
    for (int x = 0; x < kScanBatch; ++x) {
      if (w0 + x < p.nW) {
        p.ck_phi[(b * p.nW + w0 + x) * per + rem] = run;
        run = m3_wrap(run + loc[x]);
      }
    }
  }
}

// ck_h: local end states -> true state at each window start:  H <- exp(A sum dt) H + local.
__global__ void __launch_bounds__(256) m3w_state_scan_kernel(M3P p) {
  const size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
  if (i >= (size_t)p.B * p.D * p.N) return;
  const M3Idx ix(p);
  const size_t per = (size_t)p.D * p.N, b = i / per, rem = i - b * per;
  const int d = (int)(rem / p.N), n = (int)(rem - (size_t)d * p.N);
  const float A = -expf(p.a_log[ix.alog(d, n)]);
  float H = 0.f;
  for (int w0 = 0; w0 < p.nW; w0 += kScanBatch) {
    float loc[kScanBatch], dec[kScanBatch];
#pragma unroll
    for (int x = 0; x < kScanBatch; ++x) {
      const bool in = w0 + x < p.nW;
      loc[x] = in ? p.ck_h[(b * p.nW + w0 + x) * per + rem] : 0.f;
      dec[x] = in ? p.dtsum[(b * p.nW + w0 + x) * p.D + d] : 0.f;
    }
#pragma unroll
    for (int x = 0; x < kScanBatch; ++x) {
      if (w0 + x < p.nW) {
        p.ck_h[(b * p.nW + w0 + x) * per + rem] = H;
        H = fmaf(expf(A * dec[x]), H, loc[x]);
      }
    }
  }
}

// Reverse walk of dh alone through one window, from zero:  up_t = dh_t + dy_t Crot_t,  dh_{t-1} = alpha_t up_t.
// Leaves the local dh that leaves the window at its start (dhk) and the local up of its first step (upk).
template <typename IO, int PR, int LPC>
__global__ void __launch_bounds__(256) m3w_dh_local_kernel(M3P p) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  constexpr int CPW = 32 / LPC;
  const int sl = lane % LPC, d_raw = (blockIdx.x * 8 + warp) * CPW + lane / LPC, w = blockIdx.y, b = blockIdx.z;
  if ((blockIdx.x * 8 + warp) * CPW >= p.D) return;
  const bool live = d_raw < p.D;
  const int d = live ? d_raw : p.D - 1;
  const M3Idx ix(p);
  const IO* Cp = static_cast<const IO*>(p.c);
  const IO* DY = static_cast<const IO*>(p.dy);
  const int ts = w * kM3Window, te = min(p.T, ts + kM3Window);
  const size_t wrow = ((size_t)b * p.nW + w) * p.D + d;
  float A0[PR], A1[PR], phi[PR], dh0[PR], dh1[PR], u0[PR], u1[PR];
#pragma unroll
  for (int r = 0; r < PR; ++r) {
    const int kp = sl + LPC * r;
    const bool act = kp < p.Kp;
    A0[r] = act ? -expf(p.a_log[ix.alog(d, 2 * kp)]) : 0.f;
    A1[r] = act ? -expf(p.a_log[ix.alog(d, 2 * kp + 1)]) : 0.f;
    phi[r] = act ? p.ck_phi[wrow * p.Kp + kp] : 0.f;
    dh0[r] = dh1[r] = u0[r] = u1[r] = 0.f;
  }
  for (int t = ts; t < te; ++t) {  // the angle of the window's last step
    const size_t row = (size_t)b * p.T + t;
    const float dt = m3_softplus(p.dt[ix.chan(row, d)]);
#pragma unroll
    for (int r = 0; r < PR; ++r) {
      const int kp = sl + LPC * r;
      if (kp < p.Kp) phi[r] = m3_wrap(fmaf(dt, p.theta[ix.theta(row, d, kp)], phi[r]));
    }
  }
  for (int t = te - 1; t >= ts; --t) {
    const size_t row = (size_t)b * p.T + t;
    const float dt = m3_softplus(p.dt[ix.chan(row, d)]);
    const float dy = to_f32(DY[row * p.D + d]);
#pragma unroll
    for (int r = 0; r < PR; ++r) {
      const int kp = sl + LPC * r;
      if (kp < p.Kp) {
        float s, c;
        sincosf(phi[r], &s, &c);
        const size_t gi = ix.grp(row, d, 2 * kp);
        const float ce = to_f32(Cp[gi]), co = to_f32(Cp[gi + 1]);
        u0[r] = fmaf(dy, c * ce + s * co, dh0[r]);
        u1[r] = fmaf(dy, -s * ce + c * co, dh1[r]);
        dh0[r] = expf(dt * A0[r]) * u0[r];
        dh1[r] = expf(dt * A1[r]) * u1[r];
        phi[r] = m3_wrap(fmaf(-dt, p.theta[ix.theta(row, d, kp)], phi[r]));  // back to the step before
      }
    }
  }
#pragma unroll
  for (int r = 0; r < PR; ++r) {
    const int kp = sl + LPC * r;
    if (kp < p.Kp && live) {
      p.dhk[wrow * p.N + 2 * kp] = dh0[r];
      p.dhk[wrow * p.N + 2 * kp + 1] = dh1[r];
      p.upk[wrow * p.N + 2 * kp] = u0[r];
      p.upk[wrow * p.N + 2 * kp + 1] = u1[r];
    }
  }
}

// Reverse scan over the windows: dhk <- dh entering the window from later steps (DH); upk <- true up of the
// window's first step = (decay over the window's other steps) DH + local;  DH <- (decay over the window) DH + local.
__global__ void __launch_bounds__(256) m3w_dh_scan_kernel(M3P p) {
  const size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
  if (i >= (size_t)p.B * p.D * p.N) return;
  const M3Idx ix(p);
  const size_t per = (size_t)p.D * p.N, b = i / per, rem = i - b * per;
  const int d = (int)(rem / p.N), n = (int)(rem - (size_t)d * p.N);
  const float A = -expf(p.a_log[ix.alog(d, n)]);
  float DH = 0.f;
  for (int w0 = p.nW - 1; w0 >= 0; w0 -= kScanBatch) {
    float ldh[kScanBatch], lup[kScanBatch], dts[kScanBatch], dt0[kScanBatch];
#pragma unroll
    for (int x = 0; x < kScanBatch; ++x) {
      const int w = w0 - x;
      const bool in = w >= 0;
      const size_t idx = (b * p.nW + (in ? w : 0)) * per + rem;
      ldh[x] = in ? p.dhk[idx] : 0.f;
      lup[x] = in ? p.upk[idx] : 0.f;
      dts[x] = in ? p.dtsum[(b * p.nW + w) * p.D + d] : 0.f;
      dt0[x] = in ? p.dt[ix.chan(b * p.T + (size_t)w * kM3Window, d)] : 0.f;
    }
#pragma unroll
    for (int x = 0; x < kScanBatch; ++x) {
      const int w = w0 - x;
      if (w >= 0) {
        const size_t idx = (b * p.nW + w) * per + rem;
        p.dhk[idx] = DH;
        p.upk[idx] = fmaf(expf(A * (dts[x] - m3_softplus(dt0[x]))), DH, lup[x]);
        DH = fmaf(expf(A * dts[x]), DH, ldh[x]);
      }
    }
  }
}

// ang: per-window sums -> sum over all later windows (exclusive reverse scan).
__global__ void __launch_bounds__(256) m3w_ang_scan_kernel(M3P p) {
  const size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
  if (i >= (size_t)p.B * p.D * p.Kp) return;
  const size_t per = (size_t)p.D * p.Kp, b = i / per, rem = i - b * per;
  float run = 0.f;
  for (int w0 = p.nW - 1; w0 >= 0; w0 -= kScanBatch) {
    float tot[kScanBatch];
#pragma unroll
    for (int x = 0; x < kScanBatch; ++x) tot[x] = w0 - x >= 0 ? p.ang[(b * p.nW + w0 - x) * per + rem] : 0.f;
#pragma unroll
    for (int x = 0; x < kScanBatch; ++x) {
      if (w0 - x >= 0) {
        p.ang[(b * p.nW + w0 - x) * per + rem] = run;
        run += tot[x];
      }
    }
  }
}

// The angle gradient reaches every earlier step: add the later windows' sums to ddt and dtheta of each step
// (the walks used only the sums inside their own window).  One warp per (batch, step, channel).
__global__ void __launch_bounds__(256) m3w_fix_kernel(M3P p) {
  const int lane = threadIdx.x & 31;
  const size_t wi = blockIdx.x * (size_t)(blockDim.x >> 5) + (threadIdx.x >> 5);
  if (wi >= (size_t)p.B * p.T * p.D) return;
  const M3Idx ix(p);
  const size_t row = wi / p.D;
  const int d = (int)(wi - row * p.D);
  const size_t b = row / p.T;
  const int w = (int)(row - b * p.T) / kM3Window;
  if (w == p.nW - 1) return;  // nothing comes after the last window
  const float dt_raw = p.dt[ix.chan(row, d)], dt = m3_softplus(dt_raw);
  const float* off = p.ang + ((b * p.nW + w) * p.D + d) * p.Kp;
  const bool per_head = p.NH > 0;
  float s_th = 0.f, s_off = 0.f;
  for (int kp = lane; kp < p.Kp; kp += 32) {
    const float o = off[kp];
    s_th = fmaf(o, p.theta[ix.theta(row, d, kp)], s_th);
    if (per_head) s_off += o;
    else p.dtheta[ix.theta(row, d, kp)] += o * dt;
  }
  s_th = warp_sum(s_th);
  if (per_head) s_off = warp_sum(s_off);
  if (lane == 0) {
    if (per_head) {
      const size_t btd = (size_t)p.B * p.T * p.D;
      p.hd[row * p.D + d] += s_th * m3_sigmoid(dt_raw);
      p.hd[2 * btd + row * p.D + d] += s_off * dt;
    } else {
      p.ddt[row * p.D + d] += s_th * m3_sigmoid(dt_raw);
    }
  }
}

// The same for few state pairs per channel (Kp <= 16), where a warp per channel would leave most lanes idle: one
// thread per (batch, step, channel) walks its pairs.
__global__ void __launch_bounds__(256) m3w_fix_small_kernel(M3P p) {
  const size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
  if (i >= (size_t)p.B * p.T * p.D) return;
  const M3Idx ix(p);
  const size_t row = i / p.D;
  const int d = (int)(i - row * p.D);
  const size_t b = row / p.T;
  const int w = (int)(row - b * p.T) / kM3Window;
  if (w == p.nW - 1) return;  // nothing comes after the last window
  const float dt_raw = p.dt[ix.chan(row, d)], dt = m3_softplus(dt_raw);
  const float* off = p.ang + ((b * p.nW + w) * p.D + d) * p.Kp;
  const bool per_head = p.NH > 0;
  float s_th = 0.f, s_off = 0.f;
  for (int kp = 0; kp < p.Kp; ++kp) {
    const float o = off[kp];
    s_th = fmaf(o, p.theta[ix.theta(row, d, kp)], s_th);
    if (per_head) s_off += o;
    else p.dtheta[ix.theta(row, d, kp)] += o * dt;
  }
  if (per_head) {
    const size_t btd = (size_t)p.B * p.T * p.D;
    p.hd[row * p.D + d] += s_th * m3_sigmoid(dt_raw);
    p.hd[2 * btd + row * p.D + d] += s_off * dt;
  } else {
    p.ddt[row * p.D + d] += s_th * m3_sigmoid(dt_raw);
  }
}

// ----------------------------------------------------------------- backward
// WIN false: a warp walks all windows of its channel in reverse, carrying dh, the trapezoid's look-back terms and
// the angle-gradient sum.  WIN true: a warp has one window (blockIdx.y); what enters it from later steps comes from
// dhk / upk, and its angle-gradient sum and da_log share leave as per-window partials.
template <typename IO, int PR, int LPC, bool WIN>
__global__ void __launch_bounds__(256) mamba3_bwd_kernel(M3P p) {
  extern __shared__ float smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  constexpr int CPW = 32 / LPC;  // channels per warp
  const int CW = p.CW;  // channels per CTA = CPW * warps; divides the channels of a group, so every lane has a channel
  const int sl = lane % LPC, wc = warp * CPW + lane / LPC;  // lane within its channel, channel within the CTA
  const int d = blockIdx.x * CW + wc, b = WIN ? blockIdx.z : blockIdx.y;
  const int cpg = p.D / p.G, g = d / cpg, slice = (d % cpg) / CW;
  // per warp: [W][PR][3][32]  (h0_after, h1_after, phi)
  float* buf = smem + (size_t)warp * kM3Window * PR * 3 * 32;
  // [2 (step parity)][2 (dB, dC)][CW][N]: the rows of one step, added over the warps by the first 2N threads
  // while the warps already fill the other half with the next step (one barrier per step)
  float* red = smem + (size_t)(blockDim.x >> 5) * kM3Window * PR * 3 * 32;
  auto slot = [&](int s, int r, int which) -> float& { return buf[((s * PR + r) * 3 + which) * 32 + lane]; };
  const M3Idx ix(p);
  const IO* X = static_cast<const IO*>(p.x);
  const IO* Bp = static_cast<const IO*>(p.b);
  const IO* Cp = static_cast<const IO*>(p.c);
  const IO* DY = static_cast<const IO*>(p.dy);
  IO* DX = static_cast<IO*>(p.dx);
  const bool per_head = p.NH > 0;

  float A0[PR], A1[PR], dh0[PR], dh1[PR], carry[PR], pgb0[PR], pgb1[PR], dal0[PR], dal1[PR];
#pragma unroll
  for (int r = 0; r < PR; ++r) {
    const int kp = sl + LPC * r;
    const bool act = kp < p.Kp;
    A0[r] = act ? -expf(p.a_log[ix.alog(d, 2 * kp)]) : 0.f;
    A1[r] = act ? -expf(p.a_log[ix.alog(d, 2 * kp + 1)]) : 0.f;
    dh0[r] = dh1[r] = carry[r] = pgb0[r] = pgb1[r] = dal0[r] = dal1[r] = 0.f;
  }
  float pend_dx = 0.f;  // contribution of step t+1 to dx_t (lane partial)
  const int w_hi = WIN ? (int)blockIdx.y : p.nW - 1, w_lo = WIN ? (int)blockIdx.y : 0;
  if (WIN) {
    const size_t wrow = ((size_t)b * p.nW + w_hi) * p.D + d;
#pragma unroll
    for (int r = 0; r < PR; ++r) {
      const int kp = sl + LPC * r;
      if (kp < p.Kp) {
        dh0[r] = p.dhk[wrow * p.N + 2 * kp];
        dh1[r] = p.dhk[wrow * p.N + 2 * kp + 1];
      }
    }
  }

  for (int w = w_hi; w >= w_lo; --w) {
    const int ts = w * kM3Window, te = min(p.T, ts + kM3Window);
    const size_t wrow = ((size_t)b * p.nW + w) * p.D + d;
    // ---- replay the window forward, keeping h_after and phi per step ----
    float h0[PR], h1[PR], phi[PR], pb0[PR], pb1[PR], ck0[PR], ck1[PR], ckphi[PR];
    float px = ts > 0 ? to_f32(X[((size_t)b * p.T + ts - 1) * p.D + d]) : 0.f;
#pragma unroll
    for (int r = 0; r < PR; ++r) {
      const int kp = sl + LPC * r;
      const bool act = kp < p.Kp;
      ck0[r] = h0[r] = act ? p.ck_h[wrow * p.N + 2 * kp] : 0.f;
      ck1[r] = h1[r] = act ? p.ck_h[wrow * p.N + 2 * kp + 1] : 0.f;
      ckphi[r] = phi[r] = act ? p.ck_phi[wrow * p.Kp + kp] : 0.f;
      pb0[r] = pb1[r] = 0.f;
      if (act && ts > 0) {  // rotated B of step ts-1 uses the checkpointed angle
        float s, c;
        sincosf(phi[r], &s, &c);
        const size_t gi = ix.grp((size_t)b * p.T + ts - 1, d, 2 * kp);
        const float be = to_f32(Bp[gi]), bo = to_f32(Bp[gi + 1]);
        pb0[r] = c * be + s * bo;
        pb1[r] = -s * be + c * bo;
      }
    }
    for (int t = ts; t < te; ++t) {
      const size_t row = (size_t)b * p.T + t;
      const float x = to_f32(X[row * p.D + d]);
      const float dt = m3_softplus(p.dt[ix.chan(row, d)]);
      const float lam = m3_sigmoid(p.lam[ix.chan(row, d)]);
      const float gamma = lam * dt, bfac = (1.f - lam) * dt;
#pragma unroll
      for (int r = 0; r < PR; ++r) {
        const int kp = sl + LPC * r;
        if (kp < p.Kp) {
          phi[r] = m3_wrap(fmaf(dt, p.theta[ix.theta(row, d, kp)], phi[r]));
          float s, c;
          sincosf(phi[r], &s, &c);
          const size_t gi = ix.grp(row, d, 2 * kp);
          const float be = to_f32(Bp[gi]), bo = to_f32(Bp[gi + 1]);
          const float b0 = c * be + s * bo, b1 = -s * be + c * bo;
          const float al0 = expf(dt * A0[r]), al1 = expf(dt * A1[r]);
          h0[r] = al0 * h0[r] + gamma * b0 * x + bfac * al0 * pb0[r] * px;
          h1[r] = al1 * h1[r] + gamma * b1 * x + bfac * al1 * pb1[r] * px;
          pb0[r] = b0;
          pb1[r] = b1;
          slot(t - ts, r, 0) = h0[r];
          slot(t - ts, r, 1) = h1[r];
          slot(t - ts, r, 2) = phi[r];
        }
      }
      px = x;
    }
    if (WIN && te < p.T) {
      // what the first step of the next window sends back to this window's last step: px and pb are x and the
      // rotated B of step te-1 now, upk holds that step's `up`
      const size_t row_e = (size_t)b * p.T + te;
      const float dt_e = m3_softplus(p.dt[ix.chan(row_e, d)]);
      const float bf_e = (1.f - m3_sigmoid(p.lam[ix.chan(row_e, d)])) * dt_e;
      const size_t wnext = wrow + p.D;
      float acc = 0.f;
#pragma unroll
      for (int r = 0; r < PR; ++r) {
        const int kp = sl + LPC * r;
        if (kp < p.Kp) {
          const float bni0 = bf_e * expf(dt_e * A0[r]), bni1 = bf_e * expf(dt_e * A1[r]);
          const float up0 = p.upk[wnext * p.N + 2 * kp], up1 = p.upk[wnext * p.N + 2 * kp + 1];
          pgb0[r] = bni0 * px * up0;
          pgb1[r] = bni1 * px * up1;
          acc += bni0 * pb0[r] * up0 + bni1 * pb1[r] * up1;
        }
      }
      pend_dx = acc;
    }
    // ---- reverse over the window ----
    for (int t = te - 1; t >= ts; --t) {
      const size_t row = (size_t)b * p.T + t;
      const float x = to_f32(X[row * p.D + d]);
      const float xprev = t > 0 ? to_f32(X[(row - 1) * p.D + d]) : 0.f;
      const float dt_raw = p.dt[ix.chan(row, d)];
      const float dt = m3_softplus(dt_raw);
      const float lam = m3_sigmoid(p.lam[ix.chan(row, d)]);
      const float dy = to_f32(DY[row * p.D + d]);
      float s_dx = pend_dx, s_pdx = 0.f, s_dlam = 0.f, s_ddelta = 0.f, s_dtheta = 0.f;
#pragma unroll
      for (int r = 0; r < PR; ++r) {
        const int kp = sl + LPC * r;
        if (kp < p.Kp) {
          const float ha0 = slot(t - ts, r, 0), ha1 = slot(t - ts, r, 1), ph = slot(t - ts, r, 2);
          const float hb0 = (t == ts) ? ck0[r] : slot(t - ts - 1, r, 0);
          const float hb1 = (t == ts) ? ck1[r] : slot(t - ts - 1, r, 1);
          const float php = (t == ts) ? ckphi[r] : slot(t - ts - 1, r, 2);
          float s, c, sp, cp;
          sincosf(ph, &s, &c);
          sincosf(php, &sp, &cp);
          const size_t gi = ix.grp(row, d, 2 * kp);
          const float be = to_f32(Bp[gi]), bo = to_f32(Bp[gi + 1]);
          const float ce = to_f32(Cp[gi]), co = to_f32(Cp[gi + 1]);
          const float b0 = c * be + s * bo, b1 = -s * be + c * bo;
          const float c0 = c * ce + s * co, c1 = -s * ce + c * co;
          float q0 = 0.f, q1 = 0.f;  // rotated B of step t-1
          if (t > 0) {
            const size_t gp = ix.grp(row - 1, d, 2 * kp);
            const float pe = to_f32(Bp[gp]), po = to_f32(Bp[gp + 1]);
            q0 = cp * pe + sp * po;
            q1 = -sp * pe + cp * po;
          }
          const float al0 = expf(dt * A0[r]), al1 = expf(dt * A1[r]);
          const float up0 = dh0[r] + dy * c0, up1 = dh1[r] + dy * c1;
          s_dx += lam * dt * (b0 * up0 + b1 * up1);
          const float gb0 = lam * dt * x * up0 + pgb0[r];
          const float gb1 = lam * dt * x * up1 + pgb1[r];
          const float gc0 = dy * ha0, gc1 = dy * ha1;
          const float pin0 = q0 * xprev, pin1 = q1 * xprev;
          const float bni0 = (1.f - lam) * dt * al0, bni1 = (1.f - lam) * dt * al1;
          s_pdx += bni0 * q0 * up0 + bni1 * q1 * up1;
          pgb0[r] = bni0 * xprev * up0;
          pgb1[r] = bni1 * xprev * up1;
          s_dlam += (-dt * al0 * pin0 + dt * b0 * x) * up0 + (-dt * al1 * pin1 + dt * b1 * x) * up1;
          const float dterm0 = A0[r] * al0 * hb0 + (1.f - lam) * (al0 + dt * A0[r] * al0) * pin0 + lam * b0 * x;
          const float dterm1 = A1[r] * al1 * hb1 + (1.f - lam) * (al1 + dt * A1[r] * al1) * pin1 + lam * b1 * x;
          s_ddelta += dterm0 * up0 + dterm1 * up1;
          dal0[r] += (dt * al0 * A0[r] * hb0 + (1.f - lam) * dt * dt * al0 * A0[r] * pin0) * up0;
          dal1[r] += (dt * al1 * A1[r] * hb1 + (1.f - lam) * dt * dt * al1 * A1[r] * pin1) * up1;
          dh0[r] = al0 * up0;
          dh1[r] = al1 * up1;
          // rotation adjoint
          float* rb = red + (size_t)(((t & 1) * 2 + 0) * CW + wc) * p.N + 2 * kp;
          float* rc = red + (size_t)(((t & 1) * 2 + 1) * CW + wc) * p.N + 2 * kp;
          *reinterpret_cast<float2*>(rb) = make_float2(c * gb0 - s * gb1, s * gb0 + c * gb1);
          *reinterpret_cast<float2*>(rc) = make_float2(c * gc0 - s * gc1, s * gc0 + c * gc1);
          carry[r] += b1 * gb0 - b0 * gb1 + c1 * gc0 - c0 * gc1;
          const float th = p.theta[ix.theta(row, d, kp)];
          s_ddelta += carry[r] * th;
          if (per_head) s_dtheta += carry[r] * dt;
          else p.dtheta[ix.theta(row, d, kp)] = carry[r] * dt;
        }
      }
      s_dx = group_sum<LPC>(s_dx);
      s_dlam = group_sum<LPC>(s_dlam) * lam * (1.f - lam);
      s_ddelta = group_sum<LPC>(s_ddelta) * m3_sigmoid(dt_raw);
      if (per_head) s_dtheta = group_sum<LPC>(s_dtheta);
      pend_dx = s_pdx;
      if (sl == 0) {
        DX[row * p.D + d] = from_f32<IO>(s_dx);
        if (per_head) {  // per channel; m3_head_sum_kernel adds the channels of a head
          const size_t btd = (size_t)p.B * p.T * p.D;
          p.hd[row * p.D + d] = s_ddelta;
          p.hd[btd + row * p.D + d] = s_dlam;
          p.hd[2 * btd + row * p.D + d] = s_dtheta;
        } else {
          p.ddt[row * p.D + d] = s_ddelta;
          p.dlam[row * p.D + d] = s_dlam;
        }
      }
      __syncthreads();
      for (int i = threadIdx.x; i < 2 * p.N; i += blockDim.x) {
        const int which = i >= p.N, n = i - which * p.N;
        const float* src = red + (size_t)(((t & 1) * 2 + which) * CW) * p.N + n;
        float acc = 0.f;
        for (int w2 = 0; w2 < CW; ++w2) acc += src[(size_t)w2 * p.N];
        (which ? p.pc32 : p.pb32)[((row * p.G + g) * p.S + slice) * p.N + n] = acc;
      }
    }
  }
  // da_log: d/d a_log = d/dA * A  (A = -exp(a_log)); the closed form above already carries A.
  const size_t bw = WIN ? (size_t)b * p.nW + w_hi : (size_t)b;  // which partial of da_log this warp fills
  if (WIN) {
#pragma unroll
    for (int r = 0; r < PR; ++r) {
      const int kp = sl + LPC * r;
      if (kp < p.Kp) p.ang[(bw * p.D + d) * p.Kp + kp] = carry[r];
    }
  }
  if (per_head) {
    float s = 0.f;
#pragma unroll
    for (int r = 0; r < PR; ++r) s += dal0[r] + dal1[r];
    s = group_sum<LPC>(s);
    if (sl == 0) p.dal_part[bw * p.D + d] = s;
  } else {
#pragma unroll
    for (int r = 0; r < PR; ++r) {
      const int kp = sl + LPC * r;
      if (kp < p.Kp) {
        p.dal_part[(bw * p.D + d) * p.N + 2 * kp] = dal0[r];
        p.dal_part[(bw * p.D + d) * p.N + 2 * kp + 1] = dal1[r];
      }
    }
  }
}

// dB[b,t,g,:] = the S slice rows of the group added in slice order, in the tensors' dtype.
template <typename IO>
__global__ void __launch_bounds__(256) m3_bc_sum_kernel(const float* __restrict__ pb, const float* __restrict__ pc,
                                                        IO* __restrict__ db, IO* __restrict__ dc, size_t rows, int S, int N) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < rows * N; i += (size_t)gridDim.x * blockDim.x) {
    const size_t r = i / N;
    const int n = (int)(i - r * N);
    float sb = 0.f, sc = 0.f;
    for (int s = 0; s < S; ++s) {
      sb += pb[(r * S + s) * N + n];
      sc += pc[(r * S + s) * N + n];
    }
    db[i] = from_f32<IO>(sb);
    dc[i] = from_f32<IO>(sc);
  }
}

// Head-broadcast layout: ddt, dlam, dtheta [B,T,NH] = the per-channel values of a head added in channel order.
__global__ void __launch_bounds__(256) m3_head_sum_kernel(const float* __restrict__ hd, float* __restrict__ ddt,
                                                          float* __restrict__ dlam, float* __restrict__ dtheta,
                                                          size_t rows, int D, int NH) {
  const int cph = D / NH;
  const size_t btd = rows * D;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < rows * NH; i += (size_t)gridDim.x * blockDim.x) {
    const size_t r = i / NH;
    const int h = (int)(i - r * NH);
    float a = 0.f, l = 0.f, th = 0.f;
    for (int c = 0; c < cph; ++c) {
      const size_t j = r * D + (size_t)h * cph + c;
      a += hd[j];
      l += hd[btd + j];
      th += hd[2 * btd + j];
    }
    ddt[i] = a;
    dlam[i] = l;
    dtheta[i] = th;
  }
}

// da_log = the per-batch partials added in batch order ([D,N]), and over the channels of a head ([NH]).
__global__ void __launch_bounds__(256) m3_dalog_sum_kernel(const float* __restrict__ part, float* __restrict__ out, int B,
                                                           int D, int N, int NH) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (NH > 0) {
    if (i >= NH) return;
    const int cph = D / NH;
    float s = 0.f;
    for (int b = 0; b < B; ++b)
      for (int c = 0; c < cph; ++c) s += part[(size_t)b * D + i * cph + c];
    out[i] = s;
  } else {
    if (i >= D * N) return;
    float s = 0.f;
    for (int b = 0; b < B; ++b) s += part[(size_t)b * D * N + i];
    out[i] = s;
  }
}

// --------------------------------------------------------------------- host
bool mamba3_head_supported(const mxb_mamba3_desc* d);
bool mamba3_head_bwd_supported(const mxb_mamba3_desc* d);
size_t mamba3_head_partial_floats(const mxb_mamba3_desc* d);
size_t mamba3_head_scalar_floats(const mxb_mamba3_desc* d);
bool mamba3_ssd_supported(const mxb_mamba3_desc* d);
size_t mamba3_ssd_workspace_bytes(const mxb_mamba3_desc* d, bool bwd);
mxb_status mamba3_ssd_fwd(const mxb_mamba3_desc*, const void*, const float*, const float*, const float*, const float*,
                          const void*, const void*, void*, void*, cudaStream_t);
mxb_status mamba3_ssd_bwd(const mxb_mamba3_desc*, const void*, const float*, const float*, const float*, const float*,
                          const void*, const void*, const void*, void*, float*, float*, float*, float*, void*, void*,
                          void*, cudaStream_t);
static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
static bool use_ssd(const mxb_mamba3_desc* d) {
  return !(d->flags & (MXB_MAMBA3_CHANNEL_KERNELS | MXB_MAMBA3_RECURRENT_KERNELS)) && mamba3_ssd_supported(d);
}
int mamba3_head_window();
mxb_status mamba3_head_bwd(const mxb_mamba3_desc*, const void*, const float*, const float*, const float*, const float*,
                           const void*, const void*, const void*, void*, float*, float*, float*, float*, void*, void*,
                           float*, float*, float*, float*, float*, cudaStream_t);
static M3P make_m3(const mxb_mamba3_desc* d) {
  M3P p{};
  p.B = d->B; p.T = d->T; p.D = d->D; p.N = d->N; p.G = d->G; p.NH = d->nheads;
  p.Kp = d->N / 2;
  p.nW = (d->T + kM3Window - 1) / kM3Window;
  // channels that share a warp must share a group (the backward adds their dB, dC rows inside the CTA)
  p.LPC = p.Kp <= 8 ? 8 : p.Kp <= 16 ? 16 : 32;
  if (d->G >= 1 && d->D % d->G == 0 && (d->D / d->G) % (32 / p.LPC) != 0) p.LPC = 32;
  return p;
}

bool mamba3_supported(const mxb_mamba3_desc* d) {
  if (d->N < 2 || d->N % 2 || d->N > 256) return false;
  if (d->G < 1 || d->D % d->G) return false;
  if (d->nheads < 0 || (d->nheads > 0 && d->D % d->nheads)) return false;
  return true;
}

// Channels per CTA of the channel backward: 32 / LPC per warp times the largest number of warps (up to 8; 4 where a
// lane owns four state pairs and the replay buffers are that much larger) that divides the warps of a group.
static int m3_channel_warps(const M3P& p) {
  const int cpw = 32 / p.LPC, wpg = p.D / p.G / cpw, cap = p.Kp > 64 ? 4 : 8;
  int w = 1;
  for (int c = 1; c <= cap; ++c)
    if (wpg % c == 0) w = c;
  return w * cpw;
}

// Window-parallel channel kernels: where the (batch, channel) pairs alone leave half of the GPU's warp slots empty,
// unless a flag asks for one of the two forms.
static bool m3_use_windows(const mxb_mamba3_desc* d) {
  if (d->flags & MXB_MAMBA3_SERIAL_WALK) return false;
  if (d->flags & MXB_MAMBA3_WINDOW_PARALLEL) return true;
  return (size_t)d->B * d->D * 2 <= (size_t)148 * 64 && d->T > kM3Window;
}

static size_t carve_m3(M3P& p, void* ws, bool io_f32, size_t partial_floats = 0, float** pb = nullptr,
                       float** pc = nullptr, bool windows = false, bool bwd = true, size_t head_scalar_floats = 0,
                       float** hscal = nullptr) {
  Carver cv(ws);
  if (partial_floats) {  // head-broadcast kernels
    float* a = cv.take<float>(partial_floats);
    float* b2 = cv.take<float>(partial_floats);
    float* h3 = cv.take<float>(head_scalar_floats);
    if (pb) *pb = a;
    if (pc) *pc = b2;
    if (hscal) *hscal = h3;
  }
  p.ck_h = cv.take<float>((size_t)p.B * p.nW * p.D * p.N);
  p.ck_phi = cv.take<float>((size_t)p.B * p.nW * p.D * p.Kp);
  if (partial_floats) return cv.bytes();
  if (windows) p.dtsum = cv.take<float>((size_t)p.B * p.nW * p.D);
  if (!bwd) return cv.bytes();
  p.CW = m3_channel_warps(p);
  p.S = p.D / p.G / p.CW;
  const size_t rows = (size_t)p.B * p.T * p.G * p.S * p.N;
  p.pb32 = cv.take<float>(rows);
  p.pc32 = cv.take<float>(rows);
  if (p.NH > 0) p.hd = cv.take<float>(3 * (size_t)p.B * p.T * p.D);
  const size_t parts = windows ? (size_t)p.B * p.nW : (size_t)p.B;
  p.dal_part = cv.take<float>(p.NH > 0 ? parts * p.D : parts * p.D * p.N);
  if (windows) {
    p.dhk = cv.take<float>((size_t)p.B * p.nW * p.D * p.N);
    p.upk = cv.take<float>((size_t)p.B * p.nW * p.D * p.N);
    p.ang = cv.take<float>((size_t)p.B * p.nW * p.D * p.Kp);
  }
  return cv.bytes();
}

size_t mamba3_workspace_bytes(const mxb_mamba3_desc* d, bool bwd) {
  if (use_ssd(d)) return mamba3_ssd_workspace_bytes(d, bwd || (d->flags & MXB_MAMBA3_SAVE_FOR_BWD));
  M3P p = make_m3(d);
  if (!bwd) {  // only the window-parallel channel kernels need scratch in the forward
    const bool head = !(d->flags & MXB_MAMBA3_CHANNEL_KERNELS) && mamba3_head_supported(d);
    if (head || !m3_use_windows(d)) return 0;
    return carve_m3(p, nullptr, d->io_dtype == MXB_F32, 0, nullptr, nullptr, true, false);
  }
  const bool head = !(d->flags & MXB_MAMBA3_CHANNEL_KERNELS) && mamba3_head_bwd_supported(d);
  if (head) p.nW = (d->T + mamba3_head_window() - 1) / mamba3_head_window();  // checkpoint spacing of the head kernels
  return carve_m3(p, nullptr, d->io_dtype == MXB_F32, head ? mamba3_head_partial_floats(d) : 0, nullptr, nullptr,
                  !head && m3_use_windows(d), true, head ? mamba3_head_scalar_floats(d) : 0);
}

// PRV state pairs per lane, LPCV lanes per channel
#define M3_PR_DISPATCH(p, call)                                                   \
  do {                                                                           \
    if ((p).LPC == 8) { constexpr int PRV = 1, LPCV = 8; call; }                 \
    else if ((p).LPC == 16) { constexpr int PRV = 1, LPCV = 16; call; }          \
    else if ((p).Kp <= 32) { constexpr int PRV = 1, LPCV = 32; call; }           \
    else if ((p).Kp <= 64) { constexpr int PRV = 2, LPCV = 32; call; }           \
    else { constexpr int PRV = 4, LPCV = 32; call; }                             \
  } while (0)

static dim3 m3_walk_grid(const M3P& p, int ny, int nz) {
  const int per_cta = 8 * (32 / p.LPC);  // channels per 256-thread CTA
  return dim3((p.D + per_cta - 1) / per_cta, ny, nz);
}

static int m3_blocks(size_t n) { return (int)((n + 255) / 256); }

// Serial walk: y, or the checkpoints of the serial backward (p.y == nullptr).
template <typename IO>
static mxb_status m3_fwd_serial(const M3P& p, cudaStream_t st) {
  M3_PR_DISPATCH(p, MXB_LAUNCH("mamba3_fwd_kernel", st,
                               (mamba3_fwd_kernel<IO, PRV, LPCV, 0><<<m3_walk_grid(p, p.B, 1), 256, 0, st>>>(p))));
  return check_launch("mamba3_fwd_kernel");
}

// Window-parallel: angle and state at every window start (ck_phi, ck_h), then y if asked for.
template <typename IO>
static mxb_status m3_fwd_windows(const M3P& p, bool write_y, cudaStream_t st) {
  const dim3 grid = m3_walk_grid(p, p.nW, p.B);
  M3_PR_DISPATCH(p, MXB_LAUNCH("m3w_phase_kernel", st, (m3w_phase_kernel<PRV, LPCV><<<grid, 256, 0, st>>>(p))));
  MXB_LAUNCH("m3w_phase_scan_kernel", st,
             (m3w_phase_scan_kernel<<<m3_blocks((size_t)p.B * p.D * p.Kp), 256, 0, st>>>(p)));
  M3_PR_DISPATCH(p, MXB_LAUNCH("mamba3_fwd_kernel", st, (mamba3_fwd_kernel<IO, PRV, LPCV, 1><<<grid, 256, 0, st>>>(p))));
  MXB_LAUNCH("m3w_state_scan_kernel", st,
             (m3w_state_scan_kernel<<<m3_blocks((size_t)p.B * p.D * p.N), 256, 0, st>>>(p)));
  if (write_y)
    M3_PR_DISPATCH(p, MXB_LAUNCH("mamba3_fwd_kernel", st, (mamba3_fwd_kernel<IO, PRV, LPCV, 2><<<grid, 256, 0, st>>>(p))));
  return check_launch("mamba3 window-parallel forward");
}

template <typename IO, int PR, int LPC, bool WIN>
static mxb_status m3_bwd_launch(const M3P& p, cudaStream_t st) {
  const int warps = p.CW / (32 / LPC);
  const size_t sm = sizeof(float) * ((size_t)warps * kM3Window * PR * 3 * 32 + 4 * (size_t)p.CW * p.N);
  if (sm > 48 * 1024) {
    cudaError_t e =
        cudaFuncSetAttribute(mamba3_bwd_kernel<IO, PR, LPC, WIN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);
    if (e != cudaSuccess) { set_last_cuda_error((int)e); return MXB_ERR_CUDA; }
  }
  const dim3 grid = WIN ? dim3(p.D / p.CW, p.nW, p.B) : dim3(p.D / p.CW, p.B);
  MXB_LAUNCH("mamba3_bwd_kernel", st, (mamba3_bwd_kernel<IO, PR, LPC, WIN><<<grid, 32 * warps, sm, st>>>(p)));
  return check_launch("mamba3_bwd_kernel");
}
template <typename IO, bool WIN>
static mxb_status m3_bwd_pr(const M3P& p, cudaStream_t st) {
  mxb_status s = MXB_OK;
  M3_PR_DISPATCH(p, (s = m3_bwd_launch<IO, PRV, LPCV, WIN>(p, st)));
  return s;
}

// Window-parallel backward after m3_fwd_windows: dh at the window boundaries, the true walks, the angle fix-up.
template <typename IO>
static mxb_status m3_bwd_windows(const M3P& p, cudaStream_t st) {
  const dim3 grid = m3_walk_grid(p, p.nW, p.B);
  M3_PR_DISPATCH(p, MXB_LAUNCH("m3w_dh_local_kernel", st, (m3w_dh_local_kernel<IO, PRV, LPCV><<<grid, 256, 0, st>>>(p))));
  MXB_LAUNCH("m3w_dh_scan_kernel", st, (m3w_dh_scan_kernel<<<m3_blocks((size_t)p.B * p.D * p.N), 256, 0, st>>>(p)));
  mxb_status s = check_launch("mamba3 window-parallel dh");
  if (s != MXB_OK) return s;
  s = m3_bwd_pr<IO, true>(p, st);
  if (s != MXB_OK) return s;
  MXB_LAUNCH("m3w_ang_scan_kernel", st, (m3w_ang_scan_kernel<<<m3_blocks((size_t)p.B * p.D * p.Kp), 256, 0, st>>>(p)));
  if (p.Kp <= 16)
    MXB_LAUNCH("m3w_fix_small_kernel", st, (m3w_fix_small_kernel<<<m3_blocks((size_t)p.B * p.T * p.D), 256, 0, st>>>(p)));
  else
    MXB_LAUNCH("m3w_fix_kernel", st, (m3w_fix_kernel<<<m3_blocks((size_t)p.B * p.T * p.D * 32), 256, 0, st>>>(p)));
  return check_launch("mamba3 window-parallel angle fix-up");
}


mxb_status mamba3_head_fwd(const mxb_mamba3_desc*, const void*, const float*, const float*, const float*, const float*,
                           const void*, const void*, void*, float*, float*, cudaStream_t);

mxb_status mamba3_fwd(const mxb_mamba3_desc* d, const void* x, const float* dt, const float* lam,
                      const float* theta, const float* a_log, const void* b, const void* c, void* y, void* ws,
                      cudaStream_t st) {
  if (use_ssd(d)) {  // the chunked kernels move whole 16-byte units, by TMA or by cp.async
    if (!aligned16(x) || !aligned16(b) || !aligned16(c) || !aligned16(y) || !aligned16(ws)) return MXB_ERR_ALIGNMENT;
    return mamba3_ssd_fwd(d, x, dt, lam, theta, a_log, b, c, y, ws, st);
  }
  if (!(d->flags & MXB_MAMBA3_CHANNEL_KERNELS) && mamba3_head_supported(d))
    return mamba3_head_fwd(d, x, dt, lam, theta, a_log, b, c, y, nullptr, nullptr, st);
  M3P p = make_m3(d);
  p.x = x; p.dt = dt; p.lam = lam; p.theta = theta; p.a_log = a_log; p.b = b; p.c = c; p.y = y;
  const bool f32 = d->io_dtype == MXB_F32;
  if (m3_use_windows(d)) {
    carve_m3(p, ws, f32, 0, nullptr, nullptr, true, false);
    return f32 ? m3_fwd_windows<float>(p, true, st) : m3_fwd_windows<__nv_bfloat16>(p, true, st);
  }
  return f32 ? m3_fwd_serial<float>(p, st) : m3_fwd_serial<__nv_bfloat16>(p, st);
}

mxb_status mamba3_bwd(const mxb_mamba3_desc* d, const void* x, const float* dt, const float* lam,
                      const float* theta, const float* a_log, const void* b, const void* c,
                      const void* dy, void* dx, float* ddt, float* dlam, float* dtheta, float* da_log,
                      void* db, void* dc, void* ws, cudaStream_t st) {
  if (use_ssd(d)) {
    if (!aligned16(x) || !aligned16(b) || !aligned16(c) || !aligned16(dy) || !aligned16(dx) || !aligned16(db) ||
        !aligned16(dc) || !aligned16(ws))
      return MXB_ERR_ALIGNMENT;
    return mamba3_ssd_bwd(d, x, dt, lam, theta, a_log, b, c, dy, dx, ddt, dlam, dtheta, da_log, db, dc, ws, st);
  }
  M3P p = make_m3(d);
  const bool f32 = d->io_dtype == MXB_F32;
  p.x = x; p.dt = dt; p.lam = lam; p.theta = theta; p.a_log = a_log; p.b = b; p.c = c;
  p.dy = dy; p.dx = dx; p.ddt = ddt; p.dlam = dlam; p.dtheta = dtheta; p.da_log = da_log;
  const bool head_bwd = !(d->flags & MXB_MAMBA3_CHANNEL_KERNELS) && mamba3_head_bwd_supported(d);
  float *pb = nullptr, *pc = nullptr, *hscal = nullptr;
  if (head_bwd) p.nW = (d->T + mamba3_head_window() - 1) / mamba3_head_window();
  const bool windows = !head_bwd && m3_use_windows(d);
  carve_m3(p, ws, f32, head_bwd ? mamba3_head_partial_floats(d) : 0, &pb, &pc, windows, true,
           head_bwd ? mamba3_head_scalar_floats(d) : 0, &hscal);
  mxb_status s;
  if (head_bwd) {
    // CTA-per-head kernels: checkpoint pass (y == nullptr), reverse pass, fixed-order sums of the per-CTA shares
    s = mamba3_head_fwd(d, x, dt, lam, theta, a_log, b, c, nullptr, p.ck_h, p.ck_phi, st);
    if (s != MXB_OK) return s;
    return mamba3_head_bwd(d, x, dt, lam, theta, a_log, b, c, dy, dx, ddt, dlam, dtheta, da_log, db, dc, pb, pc, hscal,
                           p.ck_h, p.ck_phi, st);
  }
  // warp-per-channel kernels: checkpoints (no y), reverse pass, fixed-order sums of the partials
  if (windows) {
    s = f32 ? m3_fwd_windows<float>(p, false, st) : m3_fwd_windows<__nv_bfloat16>(p, false, st);
    if (s != MXB_OK) return s;
    s = f32 ? m3_bwd_windows<float>(p, st) : m3_bwd_windows<__nv_bfloat16>(p, st);
  } else {
    s = f32 ? m3_fwd_serial<float>(p, st) : m3_fwd_serial<__nv_bfloat16>(p, st);
    if (s != MXB_OK) return s;
    s = f32 ? m3_bwd_pr<float, false>(p, st) : m3_bwd_pr<__nv_bfloat16, false>(p, st);
  }
  if (s != MXB_OK) return s;
  const size_t rows = (size_t)p.B * p.T * p.G;
  const int grid = (int)std::min<size_t>((rows * p.N + 255) / 256, 148 * 8);
  if (f32)
    MXB_LAUNCH("m3_bc_sum_kernel", st, (m3_bc_sum_kernel<float><<<grid, 256, 0, st>>>(
        p.pb32, p.pc32, static_cast<float*>(db), static_cast<float*>(dc), rows, p.S, p.N)));
  else
    MXB_LAUNCH("m3_bc_sum_kernel", st, (m3_bc_sum_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(
        p.pb32, p.pc32, static_cast<__nv_bfloat16*>(db), static_cast<__nv_bfloat16*>(dc), rows, p.S, p.N)));
  if (p.NH > 0) {
    const size_t bt = (size_t)p.B * p.T;
    const int gh = (int)std::min<size_t>((bt * p.NH + 255) / 256, 148 * 8);
    MXB_LAUNCH("m3_head_sum_kernel", st, (m3_head_sum_kernel<<<gh, 256, 0, st>>>(p.hd, ddt, dlam, dtheta, bt, p.D, p.NH)));
  }
  const int nal = p.NH > 0 ? p.NH : p.D * p.N;
  MXB_LAUNCH("m3_dalog_sum_kernel", st, (m3_dalog_sum_kernel<<<(nal + 255) / 256, 256, 0, st>>>(p.dal_part, da_log, windows ? p.B * p.nW : p.B, p.D, p.N, p.NH)));
  return check_launch("mamba3 channel backward sums");
}

}  // namespace mxb
