// float32 tensors through the tensor-core gated delta rule (opt-in: MXB_GDN_F32_IO_BF16_OPERANDS).
//
// The reference computes this op in float32 only (gpu/ir.cpp:2352-2550); a caller that keeps float32 tensors
// gets the full-fp32 CUDA-core kernels by default.  With the flag it accepts bf16 rounding of q, k, v and of
// the results and gets the tensor-core kernels instead: one streaming pass narrows the operands into the
// workspace, the bf16 kernels run on those copies, one pass widens the results.  beta, gate and every state
// are float32 in both paths and are passed through untouched.
//
// Workspace = [the tensor-core kernels' own workspace | q16 k16 v16 o16 | dq16 dk16 dv16 (backward only)];
// o16 holds out in the forward and d_out in the backward.  A forward with MXB_GDN_SAVE_FOR_BWD leaves q16, k16,
// v16 in place, and the backward with MXB_GDN_BWD_USE_SAVED does not narrow them again.
#include <cuda_bf16.h>

#include "common.cuh"

namespace mxb {

bool gdn_tc_supported(const mxb_gdn_desc*);
size_t gdn_tc_workspace_bytes(const mxb_gdn_desc*, bool bwd);
mxb_status gdn_tc_fwd(const mxb_gdn_desc*, const void*, const void*, const void*, const float*, const float*,
                      const float*, void*, float*, void*, cudaStream_t);
mxb_status gdn_tc_bwd(const mxb_gdn_desc*, const void*, const void*, const void*, const float*, const float*,
                      const float*, const void*, const float*, void*, void*, void*, float*, float*, float*, void*,
                      cudaStream_t);

namespace f32io {

constexpr int kThreads = 256;
constexpr int kMaxSeg = 4;
constexpr int kCtasPerSeg = 148 * 4;

// Up to four tensors per launch (blockIdx.y picks one); every count is a multiple of 8 because the head
// widths are, and every pointer is 16-byte aligned (checked at the C boundary / carved at 256 bytes).
struct Segs {
  const void* src[kMaxSeg];
  void* dst[kMaxSeg];
  size_t n[kMaxSeg];
};

__global__ void __launch_bounds__(kThreads) narrow_kernel(Segs sg) {
  const int s = blockIdx.y;
  const float4* src = static_cast<const float4*>(sg.src[s]);
  uint4* dst = static_cast<uint4*>(sg.dst[s]);
  const size_t units = sg.n[s] / 8;
  for (size_t u = (size_t)blockIdx.x * kThreads + threadIdx.x; u < units; u += (size_t)gridDim.x * kThreads) {
    const float4 a = __ldg(src + 2 * u), b = __ldg(src + 2 * u + 1);
    __nv_bfloat162 p0 = __floats2bfloat162_rn(a.x, a.y), p1 = __floats2bfloat162_rn(a.z, a.w);
    __nv_bfloat162 p2 = __floats2bfloat162_rn(b.x, b.y), p3 = __floats2bfloat162_rn(b.z, b.w);
    uint4 o;
    o.x = *reinterpret_cast<uint32_t*>(&p0); o.y = *reinterpret_cast<uint32_t*>(&p1);
    o.z = *reinterpret_cast<uint32_t*>(&p2); o.w = *reinterpret_cast<uint32_t*>(&p3);
    dst[u] = o;
  }
}

__global__ void __launch_bounds__(kThreads) widen_kernel(Segs sg) {
  const int s = blockIdx.y;
  const uint4* src = static_cast<const uint4*>(sg.src[s]);
  float4* dst = static_cast<float4*>(sg.dst[s]);
  const size_t units = sg.n[s] / 8;
  for (size_t u = (size_t)blockIdx.x * kThreads + threadIdx.x; u < units; u += (size_t)gridDim.x * kThreads) {
    const uint4 r = __ldg(src + u);
    // a bf16 is the upper half of the float with the same value
    dst[2 * u] = make_float4(__uint_as_float(r.x << 16), __uint_as_float(r.x & 0xffff0000u),
                             __uint_as_float(r.y << 16), __uint_as_float(r.y & 0xffff0000u));
    dst[2 * u + 1] = make_float4(__uint_as_float(r.z << 16), __uint_as_float(r.z & 0xffff0000u),
                                 __uint_as_float(r.w << 16), __uint_as_float(r.w & 0xffff0000u));
  }
}

struct Stage {
  void* inner;
  __nv_bfloat16 *q, *k, *v, *o, *dq, *dk, *dv;
  size_t nk, nv, bytes;
};

static mxb_gdn_desc narrow_desc(const mxb_gdn_desc* d) {
  mxb_gdn_desc n = *d;
  n.io_dtype = MXB_BF16;
  n.flags &= ~MXB_GDN_F32_IO_BF16_OPERANDS;
  return n;
}

static Stage carve(const mxb_gdn_desc* d, void* ws, bool bwd, bool inner_bwd) {
  const mxb_gdn_desc n = narrow_desc(d);
  Stage s{};
  s.nk = (size_t)d->B * d->T * d->H * d->Dk;
  s.nv = (size_t)d->B * d->T * d->H * d->Dv;
  Carver cv(ws);
  s.inner = cv.take<char>(gdn_tc_workspace_bytes(&n, inner_bwd));
  s.q = cv.take<__nv_bfloat16>(s.nk);
  s.k = cv.take<__nv_bfloat16>(s.nk);
  s.v = cv.take<__nv_bfloat16>(s.nv);
  s.o = cv.take<__nv_bfloat16>(s.nv);
  if (bwd) {
    s.dq = cv.take<__nv_bfloat16>(s.nk);
    s.dk = cv.take<__nv_bfloat16>(s.nk);
    s.dv = cv.take<__nv_bfloat16>(s.nv);
  }
  s.bytes = cv.bytes();
  return s;
}

static mxb_status run(bool narrow, const Segs& sg, int nseg, cudaStream_t st) {
  if (nseg == 0) return MXB_OK;
  const dim3 grid(kCtasPerSeg, nseg);
  if (narrow) MXB_LAUNCH("gdn_f32io_narrow_kernel", st, (narrow_kernel<<<grid, kThreads, 0, st>>>(sg)));
  else MXB_LAUNCH("gdn_f32io_widen_kernel", st, (widen_kernel<<<grid, kThreads, 0, st>>>(sg)));
  return check_launch(narrow ? "gdn_f32io_narrow_kernel" : "gdn_f32io_widen_kernel");
}

}  // namespace f32io

bool gdn_f32io_wanted(const mxb_gdn_desc* d) {
  if (d->io_dtype != MXB_F32 || !(d->flags & MXB_GDN_F32_IO_BF16_OPERANDS) || (d->flags & MXB_GDN_FORCE_FP32_PATH))
    return false;
  const mxb_gdn_desc n = f32io::narrow_desc(d);
  return gdn_tc_supported(&n);
}

// The saving forward and the backward must agree on where q16, k16, v16 live, so both carve around the
// BACKWARD size of the inner workspace; a saving forward asks for the whole backward size, as the plain
// entry does, so that one buffer serves both calls.
size_t gdn_f32io_workspace_bytes(const mxb_gdn_desc* d, bool bwd) {
  const bool save = bwd || (d->flags & MXB_GDN_SAVE_FOR_BWD);
  return f32io::carve(d, nullptr, save, save).bytes;
}

mxb_status gdn_f32io_fwd(const mxb_gdn_desc* d, const void* q, const void* k, const void* v, const float* beta,
                         const float* gate, const float* h0, void* out, float* hT, void* ws, cudaStream_t st) {
  const bool save = (d->flags & MXB_GDN_SAVE_FOR_BWD) != 0;
  const f32io::Stage s = f32io::carve(d, ws, false, save);
  const mxb_gdn_desc n = f32io::narrow_desc(d);
  f32io::Segs in{{q, k, v, nullptr}, {s.q, s.k, s.v, nullptr}, {s.nk, s.nk, s.nv, 0}};
  mxb_status r = f32io::run(true, in, 3, st);
  if (r != MXB_OK) return r;
  r = gdn_tc_fwd(&n, s.q, s.k, s.v, beta, gate, h0, s.o, hT, s.inner, st);
  if (r != MXB_OK) return r;
  f32io::Segs o{{s.o, nullptr, nullptr, nullptr}, {out, nullptr, nullptr, nullptr}, {s.nv, 0, 0, 0}};
  return f32io::run(false, o, 1, st);
}

mxb_status gdn_f32io_bwd(const mxb_gdn_desc* d, const void* q, const void* k, const void* v, const float* beta,
                         const float* gate, const float* h0, const void* dO, const float* dhT, void* dq, void* dk,
                         void* dv, float* dbeta, float* dgate, float* dh0, void* ws, cudaStream_t st) {
  const f32io::Stage s = f32io::carve(d, ws, true, true);
  const mxb_gdn_desc n = f32io::narrow_desc(d);
  mxb_status r;
  if (d->flags & MXB_GDN_BWD_USE_SAVED) {
    f32io::Segs in{{dO, nullptr, nullptr, nullptr}, {s.o, nullptr, nullptr, nullptr}, {s.nv, 0, 0, 0}};
    r = f32io::run(true, in, 1, st);
  } else {
    f32io::Segs in{{q, k, v, dO}, {s.q, s.k, s.v, s.o}, {s.nk, s.nk, s.nv, s.nv}};
    r = f32io::run(true, in, 4, st);
  }
  if (r != MXB_OK) return r;
  r = gdn_tc_bwd(&n, s.q, s.k, s.v, beta, gate, h0, s.o, dhT, s.dq, s.dk, s.dv, dbeta, dgate, dh0, s.inner, st);
  if (r != MXB_OK) return r;
  f32io::Segs o{{s.dq, s.dk, s.dv, nullptr}, {dq, dk, dv, nullptr}, {s.nk, s.nk, s.nv, 0}};
  return f32io::run(false, o, 3, st);
}

}  // namespace mxb
