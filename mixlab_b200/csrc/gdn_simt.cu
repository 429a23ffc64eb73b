// Gated delta rule, chunked WY/UT form, forward and backward - full-fp32
// CUDA-core path.  Serves fp32 I/O (parity to 1e-4 cannot be met through
// bf16/tf32 tensor-core operands) and any shape the tensor-core path does not
// cover (ragged Dk/Dv, chunk != 64).  Math follows the reference's
// gated_delta_scan_chunked (gpu/ir.cpp:2352-2550):
//
//   gam = cumsum_C(log max(gate,1e-30));  E(x) = exp(clamp(x,-80,0))
//   A   = -(k beta . k^T) * E(gam_i-gam_j) * [i>j];   T = (I-A)^-1
//   u   = T (v beta);  w = T (k beta E(gam));  P = (q k^T) * E(gam_i-gam_j) * [i>=j]
//   per chunk:  v_new = u - w S;  o = (q E(gam)) S + P v_new
//               S <- S E(gam_last) + (k E(gam_last-gam))^T v_new
//
// The backward is hand-derived (the reference differentiates the forward with
// MLX autograd; only the solve has a VJP, tril(T^T dT T^T,-1),
// gpu/gated_delta_cuda_primitive.cpp:104-132, which appears below as dA).
//
// Kernels:
//   gdn_prep_kernel        one CTA per (chunk, b*H+h): gam, T, w, u, P -> workspace
//   gdn_state_fwd_kernel   one CTA per (32-column slab of Dv, b*H+h), sequential over
//                          chunks: v_new, out, state (columns of Dv are independent)
//   gdn_state_bwd_kernel   same mapping, reverse over chunks: dv_new, dS
//   gdn_chunk_bwd_kernel   one CTA per chunk: dq, dk, dv, dbeta, dgate
//   gdn_recurrent_fwd_kernel  token-by-token recurrence (chunk <= 1,
//                          gated_delta_scan_naive, gpu/ir.cpp:2314-2350)
#include "common.cuh"

namespace mxb {

struct GdnP {
  int B, T, H, K, V, C, n, gate_is_log, save;
  const void *q, *k, *v;
  const float *beta, *gate, *h0;
  void* out;
  float* hT;
  const void* dO;
  const float* dhT_in;
  void *dq, *dk, *dv;
  float *dbeta, *dgate, *dh0;
  // workspace, all fp32, indexed by ci = (b*H+h)*n + chunk
  float *gam;   // [C]
  float *Tm;    // [C,C]
  float *w;     // [C,K]
  float *u;     // [C,V]
  float *P;     // [C,C]
  float *hs;    // [V,K]  state at chunk start, transposed
  float *vn;    // [C,V]
  float *dhs;   // [V,K]  dS at chunk end, transposed
  float *dvn;   // [C,V]
  float *dqi, *dw, *dkt;  // [C,K]
};

// out(i,j, sum_{kk in [lo(i,j), hi(i,j))} a(i,kk) b(kk,j)); consecutive threads walk j.
template <typename FA, typename FB, typename FL, typename FH, typename FO>
__device__ __forceinline__ void cta_gemm_r(int M, int N, FA a, FB b, FL lo, FH hi, FO out) {
  for (int idx = threadIdx.x; idx < M * N; idx += blockDim.x) {
    const int i = idx / N, j = idx - i * N;
    float acc = 0.f;
    const int h = hi(i, j);
    for (int kk = lo(i, j); kk < h; ++kk) acc = fmaf(a(i, kk), b(kk, j), acc);
    out(i, j, acc);
  }
}
template <typename FA, typename FB, typename FO>
__device__ __forceinline__ void cta_gemm(int M, int N, int Kd, FA a, FB b, FO out) {
  cta_gemm_r(M, N, a, b, [](int, int) { return 0; }, [Kd](int, int) { return Kd; }, out);
}
// Row-mapped variant: warp w owns rows w, w+nw, ...; lanes walk j.  elem(i,j,acc)
// returns a value that is summed over the row and handed to row(i,sum) by lane 0.
template <typename FA, typename FB, typename FL, typename FH, typename FE, typename FR>
__device__ __forceinline__ void cta_gemm_rows(int M, int N, FA a, FB b, FL lo, FH hi, FE elem, FR row) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  for (int i = warp; i < M; i += nw) {
    float part = 0.f;
    for (int j = lane; j < N; j += 32) {
      float acc = 0.f;
      const int h = hi(i, j);
      for (int kk = lo(i, j); kk < h; ++kk) acc = fmaf(a(i, kk), b(kk, j), acc);
      part += elem(i, j, acc);
    }
    part = warp_sum(part);
    if (lane == 0) row(i, part);
  }
}

__device__ __forceinline__ float log_gate(float g, int gate_is_log) {
  return gate_is_log ? fmaxf(g, kLogGateFloor) : logf(fmaxf(g, kGateFloor));
}

// ------------------------------------------------------------------ prep
template <typename IO>
__global__ void __launch_bounds__(256) gdn_prep_kernel(GdnP p) {
  extern __shared__ float smem[];
  const int C = p.C, K = p.K, V = p.V, ldk = K + 1, ldc = C + 1;
  float* ks = smem;            // [C][ldk]
  float* Am = ks + C * ldk;    // [C][ldc]
  float* Tm = Am + C * ldc;    // [C][ldc]
  float* gam = Tm + C * ldc;   // [C]
  float* bet = gam + C;        // [C]
  float* bd = bet + C;         // [C] beta * E(gam)
  const int tid = threadIdx.x, c = blockIdx.x, bh = blockIdx.y;
  const int b = bh / p.H, h = bh % p.H, t0 = c * C;
  const size_t ci = (size_t)bh * p.n + c;
  const IO* q = static_cast<const IO*>(p.q);
  const IO* k = static_cast<const IO*>(p.k);
  const IO* v = static_cast<const IO*>(p.v);
  auto row = [&](int i) { return ((size_t)(b * p.T + t0 + i) * p.H + h); };

  if (tid < C) {
    const bool ok = t0 + tid < p.T;
    bet[tid] = ok ? p.beta[row(tid)] : 0.f;
    gam[tid] = ok ? log_gate(p.gate[row(tid)], p.gate_is_log) : 0.f;
  }
  for (int idx = tid; idx < C * K; idx += blockDim.x) {
    const int i = idx / K, kk = idx - i * K;
    ks[i * ldk + kk] = (t0 + i < p.T) ? to_f32(k[row(i) * K + kk]) : 0.f;
  }
  __syncthreads();
  if (tid == 0) {
    float acc = 0.f;
    for (int i = 0; i < C; ++i) { acc += gam[i]; gam[i] = acc; }
  }
  __syncthreads();
  if (tid < C) {
    bd[tid] = bet[tid] * exp_nonpos_precise(gam[tid]);
    p.gam[ci * C + tid] = gam[tid];
  }
  cta_gemm(C, C, K, [&](int i, int kk) { return ks[i * ldk + kk]; },
           [&](int kk, int j) { return ks[j * ldk + kk]; },
           [&](int i, int j, float acc) {
             Am[i * ldc + j] = (i > j) ? -bet[i] * acc * exp_nonpos_precise(gam[i] - gam[j]) : 0.f;
           });
  __syncthreads();
  // T = (I - A)^-1, one thread per column, forward substitution over rows.
  if (tid < C) {
    const int col = tid;
    for (int i = 0; i < C; ++i) {
      float s = (i == col) ? 1.f : 0.f;
      for (int j = col; j < i; ++j) s = fmaf(Am[i * ldc + j], Tm[j * ldc + col], s);
      Tm[i * ldc + col] = (i < col) ? 0.f : s;
    }
  }
  __syncthreads();
  for (int idx = tid; idx < C * C; idx += blockDim.x) {
    const int i = idx / C, j = idx - i * C;
    p.Tm[ci * C * C + idx] = Tm[i * ldc + j];
  }
  auto lo0 = [](int, int) { return 0; };
  auto hi_i = [](int i, int) { return i + 1; };
  // u = T (v beta)
  cta_gemm_r(C, V, [&](int i, int m) { return Tm[i * ldc + m]; },
             [&](int m, int j) { return (t0 + m < p.T) ? to_f32(v[row(m) * V + j]) * bet[m] : 0.f; },
             lo0, hi_i, [&](int i, int j, float acc) { p.u[(ci * C + i) * V + j] = acc; });
  // w = T (k beta E(gam))
  cta_gemm_r(C, K, [&](int i, int m) { return Tm[i * ldc + m]; },
             [&](int m, int kk) { return ks[m * ldk + kk] * bd[m]; },
             lo0, hi_i, [&](int i, int kk, float acc) { p.w[(ci * C + i) * K + kk] = acc; });
  // P = (q k^T) * Gamma * [i>=j]
  cta_gemm(C, C, K,
           [&](int i, int kk) { return (t0 + i < p.T) ? to_f32(q[row(i) * K + kk]) : 0.f; },
           [&](int kk, int j) { return ks[j * ldk + kk]; },
           [&](int i, int j, float acc) {
             p.P[ci * C * C + i * C + j] = (i >= j) ? acc * exp_nonpos_precise(gam[i] - gam[j]) : 0.f;
           });
}

// ------------------------------------------------------------ state forward
template <typename IO>
__global__ void __launch_bounds__(256) gdn_state_fwd_kernel(GdnP p) {
  extern __shared__ float smem[];
  const int C = p.C, K = p.K, V = p.V;
  float* S = smem;            // [K][33]
  float* vn = S + K * 33;     // [C][32]
  float* vr = vn + C * 32;    // [C][32]  r_i * v_new
  float* dd = vr + C * 32;    // [C] E(gam)
  float* rr = dd + C;         // [C] E(gam_last - gam)
  const int tid = threadIdx.x, j = tid & 31, rg = tid >> 5;
  const int bh = blockIdx.y, b = bh / p.H, h = bh % p.H;
  const int jv = blockIdx.x * 32 + j;
  const bool jok = jv < V;
  const IO* q = static_cast<const IO*>(p.q);
  const IO* k = static_cast<const IO*>(p.k);
  IO* out = static_cast<IO*>(p.out);

  for (int kk = rg; kk < K; kk += 8)
    S[kk * 33 + j] = (p.h0 && jok) ? p.h0[((size_t)bh * K + kk) * V + jv] : 0.f;
  __syncthreads();

  for (int c = 0; c < p.n; ++c) {
    const size_t ci = (size_t)bh * p.n + c;
    const int t0 = c * C;
    auto row = [&](int i) { return ((size_t)(b * p.T + t0 + i) * p.H + h); };
    const float* gam = p.gam + ci * C;
    const float glast = gam[C - 1];
    if (tid < C) {
      dd[tid] = exp_nonpos_precise(gam[tid]);
      rr[tid] = exp_nonpos_precise(glast - gam[tid]);
    }
    if (p.save) {  // state at chunk start, transposed [V][K]
      for (int idx = tid; idx < 32 * K; idx += blockDim.x) {
        const int jj = idx / K, kk = idx - jj * K;
        const int col = blockIdx.x * 32 + jj;
        if (col < V) p.hs[(ci * V + col) * K + kk] = S[kk * 33 + jj];
      }
    }
    __syncthreads();
    // v_new = u - w S
    const float* w = p.w + ci * C * K;
    for (int i = rg; i < C; i += 8) {
      float acc = 0.f;
      for (int kk = 0; kk < K; ++kk) acc = fmaf(w[i * K + kk], S[kk * 33 + j], acc);
      const float val = jok ? p.u[(ci * C + i) * V + jv] - acc : 0.f;
      vn[i * 32 + j] = val;
      vr[i * 32 + j] = val * rr[i];
      if (p.save && jok) p.vn[(ci * C + i) * V + jv] = val;
    }
    __syncthreads();
    // o = E(gam) (q S) + P v_new
    const float* P = p.P + ci * C * C;
    for (int i = rg; i < C; i += 8) {
      if (t0 + i >= p.T) continue;
      float acc = 0.f;
      const IO* qi = q + row(i) * K;
      for (int kk = 0; kk < K; ++kk) acc = fmaf(to_f32(qi[kk]), S[kk * 33 + j], acc);
      acc *= dd[i];
      for (int m = 0; m <= i; ++m) acc = fmaf(P[i * C + m], vn[m * 32 + j], acc);
      if (jok) out[row(i) * V + jv] = from_f32<IO>(acc);
    }
    __syncthreads();
    // S <- S E(gam_last) + (k r)^T v_new
    const float L = exp_nonpos_precise(glast);
    const int imax = min(C, p.T - t0);
    for (int kk = rg; kk < K; kk += 8) {
      float acc = S[kk * 33 + j] * L;
      for (int i = 0; i < imax; ++i) acc = fmaf(to_f32(k[row(i) * K + kk]), vr[i * 32 + j], acc);
      S[kk * 33 + j] = acc;
    }
    __syncthreads();
  }
  if (p.hT && jok)
    for (int kk = rg; kk < K; kk += 8) p.hT[((size_t)bh * K + kk) * V + jv] = S[kk * 33 + j];
}

// ----------------------------------------------------------- state backward
template <typename IO>
__global__ void __launch_bounds__(256) gdn_state_bwd_kernel(GdnP p) {
  extern __shared__ float smem[];
  const int C = p.C, K = p.K, V = p.V;
  float* dS = smem;            // [K][33]
  float* dOs = dS + K * 33;    // [C][32]
  float* dOd = dOs + C * 32;   // [C][32]  E(gam_i) dO
  float* dvs = dOd + C * 32;   // [C][32]  dv_new
  float* dd = dvs + C * 32;
  float* rr = dd + C;
  const int tid = threadIdx.x, j = tid & 31, rg = tid >> 5;
  const int bh = blockIdx.y, b = bh / p.H, h = bh % p.H;
  const int jv = blockIdx.x * 32 + j;
  const bool jok = jv < V;
  const IO* q = static_cast<const IO*>(p.q);
  const IO* k = static_cast<const IO*>(p.k);
  const IO* dO = static_cast<const IO*>(p.dO);

  for (int kk = rg; kk < K; kk += 8)
    dS[kk * 33 + j] = (p.dhT_in && jok) ? p.dhT_in[((size_t)bh * K + kk) * V + jv] : 0.f;
  __syncthreads();

  for (int c = p.n - 1; c >= 0; --c) {
    const size_t ci = (size_t)bh * p.n + c;
    const int t0 = c * C;
    auto row = [&](int i) { return ((size_t)(b * p.T + t0 + i) * p.H + h); };
    const float* gam = p.gam + ci * C;
    const float glast = gam[C - 1];
    const int imax = min(C, p.T - t0);
    if (tid < C) {
      dd[tid] = exp_nonpos_precise(gam[tid]);
      rr[tid] = exp_nonpos_precise(glast - gam[tid]);
    }
    for (int idx = tid; idx < 32 * K; idx += blockDim.x) {  // dS at chunk end, transposed
      const int jj = idx / K, kk = idx - jj * K;
      const int col = blockIdx.x * 32 + jj;
      if (col < V) p.dhs[(ci * V + col) * K + kk] = dS[kk * 33 + jj];
    }
    __syncthreads();
    for (int i = rg; i < C; i += 8) {
      const float x = (i < imax && jok) ? to_f32(dO[row(i) * V + jv]) : 0.f;
      dOs[i * 32 + j] = x;
      dOd[i * 32 + j] = x * dd[i];
    }
    __syncthreads();
    // dv_new = P^T dO + (k r) dS
    const float* P = p.P + ci * C * C;
    for (int i = rg; i < C; i += 8) {
      float acc = 0.f;
      if (i < imax) {
        const IO* ki = k + row(i) * K;
        for (int kk = 0; kk < K; ++kk) acc = fmaf(to_f32(ki[kk]), dS[kk * 33 + j], acc);
        acc *= rr[i];
      }
      for (int m = i; m < C; ++m) acc = fmaf(P[m * C + i], dOs[m * 32 + j], acc);
      dvs[i * 32 + j] = acc;
      if (jok) p.dvn[(ci * C + i) * V + jv] = acc;
    }
    __syncthreads();
    // dS <- E(gam_last) dS + (q E(gam))^T dO - w^T dv_new
    const float L = exp_nonpos_precise(glast);
    const float* w = p.w + ci * C * K;
    for (int kk = rg; kk < K; kk += 8) {
      float acc = dS[kk * 33 + j] * L;
      for (int i = 0; i < imax; ++i) acc = fmaf(to_f32(q[row(i) * K + kk]), dOd[i * 32 + j], acc);
      for (int i = 0; i < C; ++i) acc = fmaf(-w[i * K + kk], dvs[i * 32 + j], acc);
      dS[kk * 33 + j] = acc;
    }
    __syncthreads();
  }
  if (p.dh0 && jok)
    for (int kk = rg; kk < K; kk += 8) p.dh0[((size_t)bh * K + kk) * V + jv] = dS[kk * 33 + j];
}

// ----------------------------------------------------------- chunk backward
template <typename IO>
__global__ void __launch_bounds__(256) gdn_chunk_bwd_kernel(GdnP p) {
  extern __shared__ float smem[];
  const int C = p.C, K = p.K, V = p.V, ldc = C + 1;
  const int lds = (K > V ? K : V) + 1;
  float* stage = smem;             // [C][lds]
  float* Tm = stage + C * lds;     // [C][ldc]
  float* G = Tm + C * ldc;         // Gamma (lower incl.)
  float* X1 = G + C * ldc;         // dP*Gamma
  float* X2 = X1 + C * ldc;        // scratch / dT / dA
  float* X3 = X2 + C * ldc;        // k k^T
  float* X4 = X3 + C * ldc;        // scratch / T^T dT / symmetric M
  float* gam = X4 + C * ldc;
  float* bet = gam + C;
  float* dd = bet + C;
  float* rr = dd + C;
  float* dgam = rr + C;
  float* dbet = dgam + C;
  float* rs1 = dbet + C;          // [C] per-row scratch sums
  float* rs2 = rs1 + C;
  float* red = rs2 + C;           // [32]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int c = blockIdx.x, bh = blockIdx.y, b = bh / p.H, h = bh % p.H, t0 = c * C;
  const size_t ci = (size_t)bh * p.n + c;
  const int imax = min(C, p.T - t0);
  const IO* q = static_cast<const IO*>(p.q);
  const IO* k = static_cast<const IO*>(p.k);
  const IO* v = static_cast<const IO*>(p.v);
  const IO* dO = static_cast<const IO*>(p.dO);
  auto row = [&](int i) { return ((size_t)(b * p.T + t0 + i) * p.H + h); };
  auto ldq = [&](int i, int kk) { return i < imax ? to_f32(q[row(i) * K + kk]) : 0.f; };
  auto ldk = [&](int i, int kk) { return i < imax ? to_f32(k[row(i) * K + kk]) : 0.f; };
  auto ldv = [&](int i, int jj) { return i < imax ? to_f32(v[row(i) * V + jj]) : 0.f; };
  auto lddo = [&](int i, int jj) { return i < imax ? to_f32(dO[row(i) * V + jj]) : 0.f; };
  const float* hs = p.hs + ci * V * K;
  const float* dhs = p.dhs + ci * V * K;
  const float* vn = p.vn + ci * C * V;
  const float* dvn = p.dvn + ci * C * V;
  float* dqi = p.dqi + ci * C * K;
  float* dw = p.dw + ci * C * K;
  float* dkt = p.dkt + ci * C * K;
  auto lo0 = [](int, int) { return 0; };

  if (tid < C) {
    gam[tid] = p.gam[ci * C + tid];
    bet[tid] = (tid < imax) ? p.beta[row(tid)] : 0.f;
    dgam[tid] = 0.f;
    dbet[tid] = 0.f;
  }
  __syncthreads();
  const float glast = gam[C - 1];
  const float L = exp_nonpos_precise(glast);
  if (tid < C) {
    dd[tid] = exp_nonpos_precise(gam[tid]);
    rr[tid] = exp_nonpos_precise(glast - gam[tid]);
  }
  for (int idx = tid; idx < C * C; idx += blockDim.x) {
    const int i = idx / C, j = idx - i * C;
    Tm[i * ldc + j] = p.Tm[ci * C * C + idx];
    G[i * ldc + j] = (i >= j) ? exp_nonpos_precise(gam[i] - gam[j]) : 0.f;
  }
  // ---- A: contractions with the two states (operands straight from global) ----
  cta_gemm(C, K, V, [&](int i, int jj) { return lddo(i, jj); },
           [&](int jj, int kk) { return hs[jj * K + kk]; },
           [&](int i, int kk, float acc) { dqi[i * K + kk] = acc; });
  cta_gemm(C, K, V, [&](int i, int jj) { return dvn[i * V + jj]; },
           [&](int jj, int kk) { return hs[jj * K + kk]; },
           [&](int i, int kk, float acc) { dw[i * K + kk] = -acc; });
  cta_gemm(C, K, V, [&](int i, int jj) { return vn[i * V + jj]; },
           [&](int jj, int kk) { return dhs[jj * K + kk]; },
           [&](int i, int kk, float acc) { dkt[i * K + kk] = acc; });
  {  // L <dS_end, S_start>
    float part = 0.f;
    for (int idx = tid; idx < V * K; idx += blockDim.x) part = fmaf(hs[idx], dhs[idx], part);
    part = warp_sum(part);
    if (lane == 0) red[warp] = part;
  }
  // stage <- v_new
  for (int idx = tid; idx < C * V; idx += blockDim.x) {
    const int i = idx / V, jj = idx - i * V;
    stage[i * lds + jj] = vn[idx];
  }
  __syncthreads();
  if (tid == 0) {
    float s = 0.f;
    for (int wv = 0; wv < (int)(blockDim.x >> 5); ++wv) s += red[wv];
    dgam[C - 1] += L * s;
  }
  // ---- B: dP * Gamma ----
  cta_gemm_r(C, C, [&](int i, int jj) { return lddo(i, jj); },
             [&](int jj, int j) { return stage[j * lds + jj]; }, lo0,
             [&](int i, int j) { return (i >= j) ? V : 0; },
             [&](int i, int j, float acc) { X1[i * ldc + j] = acc * G[i * ldc + j]; });
  __syncthreads();
  // ---- C: stage <- k ; q k^T, k k^T, dq, partial dk ----
  for (int idx = tid; idx < C * K; idx += blockDim.x) {
    const int i = idx / K, kk = idx - i * K;
    stage[i * lds + kk] = ldk(i, kk);
  }
  __syncthreads();
  cta_gemm_r(C, C, [&](int i, int kk) { return ldq(i, kk); },
             [&](int kk, int j) { return stage[j * lds + kk]; }, lo0,
             [&](int i, int j) { return (i >= j) ? K : 0; },
             [&](int i, int j, float acc) { X2[i * ldc + j] = acc * X1[i * ldc + j]; });
  cta_gemm_r(C, C, [&](int i, int kk) { return stage[i * lds + kk]; },
             [&](int kk, int j) { return stage[j * lds + kk]; }, lo0,
             [&](int i, int j) { return (i > j) ? K : 0; },
             [&](int i, int j, float acc) { X3[i * ldc + j] = acc; });
  // row reductions that read dqi / dkt before dkt is overwritten
  for (int i = warp; i < C; i += (blockDim.x >> 5)) {
    float s1 = 0.f, s2 = 0.f;
    for (int kk = lane; kk < K; kk += 32) {
      s1 = fmaf(ldq(i, kk), dqi[i * K + kk], s1);
      s2 = fmaf(stage[i * lds + kk], dkt[i * K + kk], s2);
    }
    s1 = warp_sum(s1);
    s2 = warp_sum(s2);
    if (lane == 0) {
      rs1[i] = dd[i] * s1;  // dgam_i contribution from (q E(gam)) S
      rs2[i] = rr[i] * s2;  // rho_i
    }
  }
  __syncthreads();
  if (tid < C) {
    float s = 0.f;
    for (int j = 0; j <= tid; ++j) s += X2[tid * ldc + j];
    for (int m = tid; m < C; ++m) s -= X2[m * ldc + tid];
    dgam[tid] += s + rs1[tid] - rs2[tid];
  }
  __syncthreads();
  if (tid == 0) {
    float s = 0.f;
    for (int i = 0; i < C; ++i) s += rs2[i];
    dgam[C - 1] += s;
  }
  __syncthreads();
  // dq = E(gam) dqi + (dP Gamma) k      (final)
  {
    IO* dq = static_cast<IO*>(p.dq);
    cta_gemm_r(C, K, [&](int i, int j) { return X1[i * ldc + j]; },
               [&](int j, int kk) { return stage[j * lds + kk]; }, lo0,
               [&](int i, int) { return i + 1; },
               [&](int i, int kk, float acc) {
                 if (i < imax) dq[row(i) * K + kk] = from_f32<IO>(fmaf(dd[i], dqi[i * K + kk], acc));
               });
  }
  // dk partial = (dP Gamma)^T q + r dkt     (kept in dkt)
  cta_gemm_r(C, K, [&](int i, int m) { return X1[m * ldc + i]; },
             [&](int m, int kk) { return ldq(m, kk); },
             [](int i, int) { return i; }, [C](int, int) { return C; },
             [&](int i, int kk, float acc) { dkt[i * K + kk] = fmaf(rr[i], dkt[i * K + kk], acc); });
  __syncthreads();
  // ---- D: dT = du (v beta)^T + dw (k beta E(gam))^T  (strictly lower part is all that is used)
  for (int idx = tid; idx < C * V; idx += blockDim.x) {
    const int i = idx / V, jj = idx - i * V;
    stage[i * lds + jj] = ldv(i, jj) * bet[i];
  }
  __syncthreads();
  cta_gemm(C, C, V, [&](int i, int jj) { return dvn[i * V + jj]; },
           [&](int jj, int j) { return stage[j * lds + jj]; },
           [&](int i, int j, float acc) { X2[i * ldc + j] = acc; });
  __syncthreads();
  for (int idx = tid; idx < C * K; idx += blockDim.x) {
    const int i = idx / K, kk = idx - i * K;
    stage[i * lds + kk] = ldk(i, kk) * bet[i] * dd[i];
  }
  __syncthreads();
  cta_gemm(C, C, K, [&](int i, int kk) { return dw[i * K + kk]; },
           [&](int kk, int j) { return stage[j * lds + kk]; },
           [&](int i, int j, float acc) { X2[i * ldc + j] += acc; });
  __syncthreads();
  // X4 = T^T dT ;  dA = (X4 T^T) strictly lower -> X2
  cta_gemm_r(C, C, [&](int i, int m) { return Tm[m * ldc + i]; },
             [&](int m, int j) { return X2[m * ldc + j]; },
             [](int i, int) { return i; }, [C](int, int) { return C; },
             [&](int i, int j, float acc) { X4[i * ldc + j] = acc; });
  __syncthreads();
  cta_gemm_r(C, C, [&](int i, int m) { return X4[i * ldc + m]; },
             [&](int m, int j) { return Tm[j * ldc + m]; }, lo0,
             [&](int i, int j) { return (i > j) ? j + 1 : 0; },
             [&](int i, int j, float acc) { X2[i * ldc + j] = (i > j) ? acc : 0.f; });
  // stage <- k again (X2 is not read until after the next barrier)
  for (int idx = tid; idx < C * K; idx += blockDim.x) {
    const int i = idx / K, kk = idx - i * K;
    stage[i * lds + kk] = ldk(i, kk);
  }
  __syncthreads();
  // ---- E: M = -dA Gamma ; Mb = beta_i M ; dbeta, dgam from A ; X4 <- Mb + Mb^T
  for (int idx = tid; idx < C * C; idx += blockDim.x) {
    const int i = idx / C, j = idx - i * C;
    if (i > j) {
      const float M = -X2[i * ldc + j] * G[i * ldc + j];
      X2[i * ldc + j] = M * X3[i * ldc + j];  // M * (k_i.k_j)
      const float mb = M * bet[i];
      X4[i * ldc + j] = mb;
      X4[j * ldc + i] = mb;
    } else if (i == j) {
      X2[i * ldc + i] = 0.f;
      X4[i * ldc + i] = 0.f;
    }
  }
  __syncthreads();
  if (tid < C) {
    float rs = 0.f, cs = 0.f;
    for (int j = 0; j < tid; ++j) rs += X2[tid * ldc + j];
    for (int m = tid + 1; m < C; ++m) cs += bet[m] * X2[m * ldc + tid];
    dbet[tid] += rs;
    dgam[tid] += bet[tid] * rs - cs;
  }
  // dv = beta (T^T du) ; dbeta += v . (T^T du)
  {
    IO* dv = static_cast<IO*>(p.dv);
    cta_gemm_rows(C, V, [&](int i, int m) { return Tm[m * ldc + i]; },
                  [&](int m, int jj) { return dvn[m * V + jj]; },
                  [](int i, int) { return i; }, [C](int, int) { return C; },
                  [&](int i, int jj, float acc) {
                    if (i < imax) dv[row(i) * V + jj] = from_f32<IO>(bet[i] * acc);
                    return ldv(i, jj) * acc;
                  },
                  [&](int i, float s) { rs1[i] = s; });
  }
  // z = T^T dw ; dk = partial + beta E(gam) z + (Mb + Mb^T) k ; k.z row sums
  {
    IO* dk = static_cast<IO*>(p.dk);
    const int nw = blockDim.x >> 5;
    for (int i = warp; i < C; i += nw) {
      float part = 0.f;
      for (int kk = lane; kk < K; kk += 32) {
        float z = 0.f;
        for (int m = i; m < C; ++m) z = fmaf(Tm[m * ldc + i], dw[m * K + kk], z);
        float acc = 0.f;
        for (int jx = 0; jx < C; ++jx) acc = fmaf(X4[i * ldc + jx], stage[jx * lds + kk], acc);
        if (i < imax) dk[row(i) * K + kk] = from_f32<IO>(dkt[i * K + kk] + bet[i] * dd[i] * z + acc);
        part = fmaf(stage[i * lds + kk], z, part);
      }
      part = warp_sum(part);
      if (lane == 0) rs2[i] = part;  // k_i . z_i
    }
  }
  __syncthreads();
  if (tid < C) {
    const float vdu = rs1[tid];
    const float kz = rs2[tid];
    dbet[tid] += vdu + dd[tid] * kz;
    dgam[tid] += bet[tid] * dd[tid] * kz;
  }
  __syncthreads();
  if (tid == 0) {  // dg = reverse cumulative sum of dgam within the chunk
    float acc = 0.f;
    for (int i = C - 1; i >= 0; --i) { acc += dgam[i]; dgam[i] = acc; }
  }
  __syncthreads();
  if (tid < imax) {
    p.dbeta[row(tid)] = dbet[tid];
    float dg = dgam[tid];
    const float gin = p.gate[row(tid)];
    if (p.gate_is_log) {
      if (gin < kLogGateFloor) dg = 0.f;
    } else {
      dg = (gin > kGateFloor) ? dg / gin : 0.f;
    }
    p.dgate[row(tid)] = dg;
  }
}

// --------------------------------------------------- token-by-token forward
template <typename IO>
__global__ void __launch_bounds__(256) gdn_recurrent_fwd_kernel(GdnP p) {
  extern __shared__ float smem[];
  const int K = p.K, V = p.V;
  float* S = smem;           // [K][33]
  float* sk = S + K * 33;    // [K]
  float* sq = sk + K;        // [K]
  float* red = sq + K;       // [2][8][32]
  const int tid = threadIdx.x, j = tid & 31, rg = tid >> 5;
  const int bh = blockIdx.y, b = bh / p.H, h = bh % p.H;
  const int jv = blockIdx.x * 32 + j;
  const bool jok = jv < V;
  const IO* q = static_cast<const IO*>(p.q);
  const IO* k = static_cast<const IO*>(p.k);
  const IO* v = static_cast<const IO*>(p.v);
  IO* out = static_cast<IO*>(p.out);
  for (int kk = rg; kk < K; kk += 8)
    S[kk * 33 + j] = (p.h0 && jok) ? p.h0[((size_t)bh * K + kk) * V + jv] : 0.f;
  for (int t = 0; t < p.T; ++t) {
    const size_t r = (size_t)(b * p.T + t) * p.H + h;
    __syncthreads();
    for (int i = tid; i < K; i += blockDim.x) {
      sk[i] = to_f32(k[r * K + i]);
      sq[i] = to_f32(q[r * K + i]);
    }
    __syncthreads();
    const float gv = p.gate[r];
    const float a = p.gate_is_log ? expf(gv) : gv;
    float pk = 0.f, pq = 0.f, qk = 0.f;
    for (int kk = rg; kk < K; kk += 8) {
      const float s = S[kk * 33 + j];
      pk = fmaf(sk[kk], s, pk);
      pq = fmaf(sq[kk], s, pq);
    }
    for (int kk = 0; kk < K; ++kk) qk = fmaf(sq[kk], sk[kk], qk);
    red[rg * 32 + j] = pk;
    red[256 + rg * 32 + j] = pq;
    __syncthreads();
    pk = 0.f; pq = 0.f;
    for (int wv = 0; wv < 8; ++wv) { pk += red[wv * 32 + j]; pq += red[256 + wv * 32 + j]; }
    const float vv = jok ? to_f32(v[r * V + jv]) : 0.f;
    const float e = p.beta[r] * (vv - a * pk);
    for (int kk = rg; kk < K; kk += 8) S[kk * 33 + j] = fmaf(sk[kk], e, a * S[kk * 33 + j]);
    if (rg == 0 && jok) out[r * V + jv] = from_f32<IO>(fmaf(qk, e, a * pq));
  }
  __syncthreads();
  if (p.hT && jok)
    for (int kk = rg; kk < K; kk += 8) p.hT[((size_t)bh * K + kk) * V + jv] = S[kk * 33 + j];
}

// ------------------------------------------------------------------ host
static size_t carve(GdnP& p, void* ws, bool bwd) {
  Carver cv(ws);
  const size_t nc = (size_t)p.B * p.H * p.n, C = p.C, K = p.K, V = p.V;
  cv.take<int>(64);  // device status header (always zero on this path)
  p.gam = cv.take<float>(nc * C);
  p.Tm = cv.take<float>(nc * C * C);
  p.w = cv.take<float>(nc * C * K);
  p.u = cv.take<float>(nc * C * V);
  p.P = cv.take<float>(nc * C * C);
  if (bwd) {
    p.hs = cv.take<float>(nc * V * K);
    p.vn = cv.take<float>(nc * C * V);
    p.dhs = cv.take<float>(nc * V * K);
    p.dvn = cv.take<float>(nc * C * V);
    p.dqi = cv.take<float>(nc * C * K);
    p.dw = cv.take<float>(nc * C * K);
    p.dkt = cv.take<float>(nc * C * K);
  }
  return cv.bytes();
}

static GdnP make_params(const mxb_gdn_desc* d) {
  GdnP p{};
  p.B = d->B; p.T = d->T; p.H = d->H; p.K = d->Dk; p.V = d->Dv;
  p.C = d->chunk > 64 ? 64 : d->chunk;
  if (p.C < 2) p.C = 64;  // the backward of the token recurrence runs in chunked form
  p.n = (d->T + p.C - 1) / p.C;
  p.gate_is_log = d->gate_is_log;
  return p;
}

size_t gdn_simt_workspace_bytes(const mxb_gdn_desc* d, bool bwd) {
  if (!bwd && d->chunk <= 1) return 0;
  GdnP p = make_params(d);
  return carve(p, nullptr, bwd);
}

// Any chunk size is accepted: the result does not depend on it, and sizes above 64 are computed
// with chunks of 64 (make_params), as the reference allows larger scan_chunk_size overrides
// (arch/blocks_gated_deltanet.go:11-17).  Dv up to 256 covers the reference default Dv = 2 Dk.
bool gdn_simt_supported(const mxb_gdn_desc* d) {
  return d->Dk >= 1 && d->Dv >= 1 && d->Dk <= 128 && d->Dv <= 256;
}

template <typename KernelT>
static mxb_status set_smem(KernelT kern, size_t bytes) {
  if (bytes > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e != cudaSuccess) { set_last_cuda_error((int)e); return MXB_ERR_CUDA; }
  }
  return MXB_OK;
}

template <typename IO>
static mxb_status run_fwd(GdnP& p, bool chunked, cudaStream_t st) {
  const int C = p.C, K = p.K, V = p.V;
  dim3 gslab((V + 31) / 32, p.B * p.H);
  if (!chunked) {
    size_t sm = sizeof(float) * (K * 33 + 2 * K + 512);
    if (set_smem(gdn_recurrent_fwd_kernel<IO>, sm) != MXB_OK) return MXB_ERR_CUDA;
    MXB_LAUNCH("gdn_recurrent_fwd_kernel", st, (gdn_recurrent_fwd_kernel<IO><<<gslab, 256, sm, st>>>(p)));
    return check_launch("gdn_recurrent_fwd_kernel");
  }
  size_t sm1 = sizeof(float) * (C * (K + 1) + 2 * C * (C + 1) + 3 * C);
  if (set_smem(gdn_prep_kernel<IO>, sm1) != MXB_OK) return MXB_ERR_CUDA;
  MXB_LAUNCH("gdn_prep_kernel", st, (gdn_prep_kernel<IO><<<dim3(p.n, p.B * p.H), 256, sm1, st>>>(p)));
  mxb_status s = check_launch("gdn_prep_kernel");
  if (s != MXB_OK) return s;
  size_t sm2 = sizeof(float) * (K * 33 + 2 * C * 32 + 2 * C);
  if (set_smem(gdn_state_fwd_kernel<IO>, sm2) != MXB_OK) return MXB_ERR_CUDA;
  MXB_LAUNCH("gdn_state_fwd_kernel", st, (gdn_state_fwd_kernel<IO><<<gslab, 256, sm2, st>>>(p)));
  return check_launch("gdn_state_fwd_kernel");
}

template <typename IO>
static mxb_status run_bwd(GdnP& p, bool recompute, cudaStream_t st) {
  const int C = p.C, K = p.K, V = p.V;
  p.save = 1;
  mxb_status s = MXB_OK;
  if (recompute) {
    // forward recompute into the workspace; out is not needed -> write into dv (overwritten later)
    void* keep_out = p.out;
    float* keep_hT = p.hT;
    p.out = p.dv;
    p.hT = nullptr;
    s = run_fwd<IO>(p, true, st);
    p.out = keep_out;
    p.hT = keep_hT;
    if (s != MXB_OK) return s;
  }
  dim3 gslab((V + 31) / 32, p.B * p.H);
  size_t sm3 = sizeof(float) * (K * 33 + 3 * C * 32 + 2 * C);
  if (set_smem(gdn_state_bwd_kernel<IO>, sm3) != MXB_OK) return MXB_ERR_CUDA;
  MXB_LAUNCH("gdn_state_bwd_kernel", st, (gdn_state_bwd_kernel<IO><<<gslab, 256, sm3, st>>>(p)));
  s = check_launch("gdn_state_bwd_kernel");
  if (s != MXB_OK) return s;
  const int lds = (K > V ? K : V) + 1;
  size_t sm4 = sizeof(float) * (C * lds + 6 * C * (C + 1) + 8 * C + 32);
  if (set_smem(gdn_chunk_bwd_kernel<IO>, sm4) != MXB_OK) return MXB_ERR_CUDA;
  MXB_LAUNCH("gdn_chunk_bwd_kernel", st, (gdn_chunk_bwd_kernel<IO><<<dim3(p.n, p.B * p.H), 256, sm4, st>>>(p)));
  return check_launch("gdn_chunk_bwd_kernel");
}

mxb_status gdn_simt_fwd(const mxb_gdn_desc* d, const void* q, const void* k, const void* v,
                        const float* beta, const float* gate, const float* h0, void* out, float* hT,
                        void* ws, cudaStream_t st) {
  GdnP p = make_params(d);
  p.q = q; p.k = k; p.v = v; p.beta = beta; p.gate = gate; p.h0 = h0; p.out = out; p.hT = hT;
  const bool chunked = d->chunk > 1;
  if (chunked) {
    p.save = (d->flags & MXB_GDN_SAVE_FOR_BWD) ? 1 : 0;
    carve(p, ws, p.save != 0);
    if (cudaMemsetAsync(ws, 0, 256, st) != cudaSuccess) return MXB_ERR_CUDA;
  }
  return d->io_dtype == MXB_F32 ? run_fwd<float>(p, chunked, st) : run_fwd<__nv_bfloat16>(p, chunked, st);
}

mxb_status gdn_simt_bwd(const mxb_gdn_desc* d, const void* q, const void* k, const void* v,
                        const float* beta, const float* gate, const float* h0, const void* dO,
                        const float* dhT, void* dq, void* dk, void* dv, float* dbeta, float* dgate,
                        float* dh0, void* ws, cudaStream_t st) {
  GdnP p = make_params(d);
  p.q = q; p.k = k; p.v = v; p.beta = beta; p.gate = gate; p.h0 = h0;
  p.dO = dO; p.dhT_in = dhT; p.dq = dq; p.dk = dk; p.dv = dv; p.dbeta = dbeta; p.dgate = dgate; p.dh0 = dh0;
  carve(p, ws, true);
  if (cudaMemsetAsync(ws, 0, 256, st) != cudaSuccess) return MXB_ERR_CUDA;
  // saved intermediates exist only for the chunked forward
  const bool recompute = !(d->flags & MXB_GDN_BWD_USE_SAVED) || d->chunk <= 1;
  return d->io_dtype == MXB_F32 ? run_bwd<float>(p, recompute, st) : run_bwd<__nv_bfloat16>(p, recompute, st);
}

}  // namespace mxb
