// Gated delta rule - single-token recurrent decode step (HBM-bound stream).
//
// Semantics: the loop body of the reference's gated_delta_scan_naive
// (gpu/ir.cpp:2334-2345) applied once to a persistent fp32 state [N,H,Dk,Dv]:
//     S <- a S ; pred = k^T S ; S <- S + k (x) beta (v - pred) ; o = q^T S
//
// The state is read once and written once.  Both contractions over Dk are taken
// from the SAME pass over the loaded state:
//     pred = a (k^T S_old)         o = a (q^T S_old) + (q.k) beta (v - pred)
// so there is a single cross-warp reduction between the load and the store.
//
// Mapping: one CTA per (sequence, head, 128-column block); a warp reads whole
// 512-byte rows with 128-bit loads (lane = 4 columns), warp w owns rows
// w, w+8, ...; each thread keeps its ROWS float4 pieces of the state in
// registers between the load and the store.
#include "common.cuh"

namespace mxb {

template <typename IO, int ROWS>
__global__ void __launch_bounds__(256, (ROWS <= 16 ? 2 : 1))
gdn_decode_kernel(float* __restrict__ state, const IO* __restrict__ q, const IO* __restrict__ k,
                  const IO* __restrict__ v, const float* __restrict__ beta,
                  const float* __restrict__ gate, IO* __restrict__ out, int Dk, int Dv,
                  int gate_is_log) {
  __shared__ float s_k[8 * ROWS];
  __shared__ float s_q[8 * ROWS];
  __shared__ __align__(16) float s_red[2][8][128];

  const int tid = threadIdx.x;
  const int cg = tid & 31, rg = tid >> 5;
  const int sh = blockIdx.y;
  const int c0 = blockIdx.x * 128 + 4 * cg;
  const bool col_ok = c0 < Dv;

  for (int i = tid; i < 8 * ROWS; i += 256) {
    s_k[i] = i < Dk ? to_f32(k[(size_t)sh * Dk + i]) : 0.0f;
    s_q[i] = i < Dk ? to_f32(q[(size_t)sh * Dk + i]) : 0.0f;
  }
  float* sp = state + (size_t)sh * Dk * Dv;
  float4 S[ROWS];
#pragma unroll
  for (int r = 0; r < ROWS; ++r) {
    const int row = rg + 8 * r;
    if (col_ok && row < Dk) S[r] = __ldcs(reinterpret_cast<const float4*>(sp + (size_t)row * Dv + c0));
    else S[r] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  const float gv = gate[sh];
  const float a = gate_is_log ? expf(gv) : gv;
  const float bt = beta[sh];
  __syncthreads();

  float4 pk = make_float4(0.f, 0.f, 0.f, 0.f), pq = pk;
#pragma unroll
  for (int r = 0; r < ROWS; ++r) {
    const float kr = s_k[rg + 8 * r], qr = s_q[rg + 8 * r];
    pk.x = fmaf(kr, S[r].x, pk.x); pk.y = fmaf(kr, S[r].y, pk.y);
    pk.z = fmaf(kr, S[r].z, pk.z); pk.w = fmaf(kr, S[r].w, pk.w);
    pq.x = fmaf(qr, S[r].x, pq.x); pq.y = fmaf(qr, S[r].y, pq.y);
    pq.z = fmaf(qr, S[r].z, pq.z); pq.w = fmaf(qr, S[r].w, pq.w);
  }
  *reinterpret_cast<float4*>(&s_red[0][rg][4 * cg]) = pk;
  *reinterpret_cast<float4*>(&s_red[1][rg][4 * cg]) = pq;
  float qk = 0.f;
  for (int i = cg; i < Dk; i += 32) qk = fmaf(s_q[i], s_k[i], qk);
  qk = warp_sum(qk);
  __syncthreads();

  pk = make_float4(0.f, 0.f, 0.f, 0.f); pq = pk;
#pragma unroll
  for (int w = 0; w < 8; ++w) {
    const float4 x = *reinterpret_cast<const float4*>(&s_red[0][w][4 * cg]);
    const float4 y = *reinterpret_cast<const float4*>(&s_red[1][w][4 * cg]);
    pk.x += x.x; pk.y += x.y; pk.z += x.z; pk.w += x.w;
    pq.x += y.x; pq.y += y.y; pq.z += y.z; pq.w += y.w;
  }
  if (!col_ok) return;
  float4 vv;
  const IO* vp = v + (size_t)sh * Dv + c0;
  vv.x = to_f32(vp[0]); vv.y = to_f32(vp[1]); vv.z = to_f32(vp[2]); vv.w = to_f32(vp[3]);
  float4 e;
  e.x = bt * (vv.x - a * pk.x); e.y = bt * (vv.y - a * pk.y);
  e.z = bt * (vv.z - a * pk.z); e.w = bt * (vv.w - a * pk.w);
#pragma unroll
  for (int r = 0; r < ROWS; ++r) {
    const int row = rg + 8 * r;
    if (row < Dk) {
      const float kr = s_k[row];
      float4 n;
      n.x = fmaf(kr, e.x, a * S[r].x); n.y = fmaf(kr, e.y, a * S[r].y);
      n.z = fmaf(kr, e.z, a * S[r].z); n.w = fmaf(kr, e.w, a * S[r].w);
      __stcs(reinterpret_cast<float4*>(sp + (size_t)row * Dv + c0), n);
    }
  }
  if (rg == 0) {
    IO* op = out + (size_t)sh * Dv + c0;
    op[0] = from_f32<IO>(fmaf(qk, e.x, a * pq.x));
    op[1] = from_f32<IO>(fmaf(qk, e.y, a * pq.y));
    op[2] = from_f32<IO>(fmaf(qk, e.z, a * pq.z));
    op[3] = from_f32<IO>(fmaf(qk, e.w, a * pq.w));
  }
}

template <typename IO>
static mxb_status launch_decode(const mxb_gdn_desc* d, float* state, const void* q, const void* k,
                                const void* v, const float* beta, const float* gate, void* out,
                                cudaStream_t st) {
  dim3 grid((d->Dv + 127) / 128, d->B * d->H);
  auto Q = static_cast<const IO*>(q);
  auto K = static_cast<const IO*>(k);
  auto V = static_cast<const IO*>(v);
  auto O = static_cast<IO*>(out);
  if (d->Dk <= 64)
    MXB_LAUNCH("gdn_decode_kernel", st, (gdn_decode_kernel<IO, 8><<<grid, 256, 0, st>>>(state, Q, K, V, beta, gate, O, d->Dk, d->Dv, d->gate_is_log)));
  else if (d->Dk <= 128)
    MXB_LAUNCH("gdn_decode_kernel", st, (gdn_decode_kernel<IO, 16><<<grid, 256, 0, st>>>(state, Q, K, V, beta, gate, O, d->Dk, d->Dv, d->gate_is_log)));
  else
    MXB_LAUNCH("gdn_decode_kernel", st, (gdn_decode_kernel<IO, 32><<<grid, 256, 0, st>>>(state, Q, K, V, beta, gate, O, d->Dk, d->Dv, d->gate_is_log)));
  return check_launch("gdn_decode_kernel");
}

bool gdn_decode_bulk_supported(const mxb_gdn_desc* d);
mxb_status gdn_decode_bulk_dispatch(const mxb_gdn_desc*, float*, const void*, const void*, const void*, const float*,
                                    const float*, void*, cudaStream_t);

mxb_status gdn_decode_dispatch(const mxb_gdn_desc* d, float* state, const void* q, const void* k,
                               const void* v, const float* beta, const float* gate, void* out,
                               cudaStream_t st) {
  if (d->Dv % 4 != 0 || d->Dk > 256) return MXB_ERR_UNSUPPORTED;
  if (!(d->flags & MXB_GDN_DECODE_REGISTER_KERNEL) && gdn_decode_bulk_supported(d))
    return gdn_decode_bulk_dispatch(d, state, q, k, v, beta, gate, out, st);
  if (d->io_dtype == MXB_F32) return launch_decode<float>(d, state, q, k, v, beta, gate, out, st);
  return launch_decode<__nv_bfloat16>(d, state, q, k, v, beta, gate, out, st);
}

}  // namespace mxb
