// Element-wise passes of the data-parallel gradient exchange over flat fp32 buckets.
//
// The reference does these steps with one MLX op after another per weight
// (gpu/distributed_step.cpp:140-152: isfinite / where / multiply before the sums, :231-240 and
// gpu/optimizer_step_guard.cpp:76-104: divide, isfinite / where, square-sum, scale after them).  Over a gigabyte
// of gradients that is a dozen trips through HBM; here each side of the all-reduce is one fused streaming pass
// per bucket, plus one pass that applies the clipping scale:
//
//   dp_sanitize_kernel   x <- finite(x) ? x * scale : 0, flag <- any non-finite          (before the sums)
//   dp_finalize_kernel   x <- x * inv_denominator, non-finite -> 0 and counted, sum of squares  (after the sums)
//   dp_reduce_kernel     per-CTA partial sums -> totals, in a fixed order (no floating-point atomics)
//   dp_scale_kernel      x <- x * clip scale computed on the device from the totals          (no host round trip)
//
// All passes are 128-bit vectorised grid-stride streams sized to the SM count: they are bound by HBM bandwidth.
#include "common.cuh"

namespace mxb {

constexpr int kDpThreads = 256;
constexpr int kDpMaxCtas = 148 * 8;

__device__ __forceinline__ bool finite_f(float v) { return fabsf(v) <= 3.402823466e38f; }  // false for NaN and Inf

// Head and tail elements that do not fill a 16-byte unit are handled by plain loops of CTA 0.
struct Span {
  size_t head, units, tail_begin, n;
};
__device__ __forceinline__ Span make_span(const float* x, size_t n) {
  const size_t mis = (reinterpret_cast<uintptr_t>(x) & 15) / 4;
  size_t head = mis ? 4 - mis : 0;
  if (head > n) head = n;
  const size_t units = (n - head) / 4;
  return Span{head, units, head + 4 * units, n};
}

__global__ void __launch_bounds__(kDpThreads) dp_sanitize_kernel(float* x, size_t n, float scale, float* flag) {
  const Span sp = make_span(x, n);
  bool bad = false;
  float4* v = reinterpret_cast<float4*>(x + sp.head);
  for (size_t u = (size_t)blockIdx.x * blockDim.x + threadIdx.x; u < sp.units; u += (size_t)gridDim.x * blockDim.x) {
    float4 t = v[u];
    float e[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const bool f = finite_f(e[k]);
      bad |= !f;
      e[k] = f ? e[k] * scale : 0.f;
    }
    v[u] = make_float4(e[0], e[1], e[2], e[3]);
  }
  if (blockIdx.x == 0) {
    for (size_t i = threadIdx.x; i < sp.head + (sp.n - sp.tail_begin); i += blockDim.x) {
      const size_t j = i < sp.head ? i : sp.tail_begin + (i - sp.head);
      const bool f = finite_f(x[j]);
      bad |= !f;
      x[j] = f ? x[j] * scale : 0.f;
    }
  }
  if (__syncthreads_or(bad) && threadIdx.x == 0) *flag = 1.0f;  // every writer stores the same value: no race to resolve
}

// partial[2 * blockIdx.x] = sum of squares, partial[2 * blockIdx.x + 1] = number of non-finite entries.
// With den_dev the divisor is read from device memory (the all-reduced loss denominator, which then never has to
// visit the host between the sums and this pass); a zero, negative or non-finite one leaves the values as they are
// (the host reads it afterwards and skips or rejects the step).
__global__ void __launch_bounds__(kDpThreads) dp_finalize_kernel(float* x, size_t n, float inv_denominator,
                                                                 const float* den_dev, float* partial) {
  __shared__ float red[2][kDpThreads / 32];
  if (den_dev) {
    const float den = *den_dev;
    inv_denominator = (den > 0.f && finite_f(den)) ? 1.f / den : 1.f;
  }
  const Span sp = make_span(x, n);
  float sq = 0.f, cnt = 0.f;
  float4* v = reinterpret_cast<float4*>(x + sp.head);
  for (size_t u = (size_t)blockIdx.x * blockDim.x + threadIdx.x; u < sp.units; u += (size_t)gridDim.x * blockDim.x) {
    float4 t = v[u];
    float e[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float y = e[k] * inv_denominator;
      const bool f = finite_f(y);
      cnt += f ? 0.f : 1.f;
      e[k] = f ? y : 0.f;
      sq = fmaf(e[k], e[k], sq);
    }
    v[u] = make_float4(e[0], e[1], e[2], e[3]);
  }
  if (blockIdx.x == 0) {
    for (size_t i = threadIdx.x; i < sp.head + (sp.n - sp.tail_begin); i += blockDim.x) {
      const size_t j = i < sp.head ? i : sp.tail_begin + (i - sp.head);
      const float y = x[j] * inv_denominator;
      const bool f = finite_f(y);
      cnt += f ? 0.f : 1.f;
      x[j] = f ? y : 0.f;
      sq = fmaf(x[j], x[j], sq);
    }
  }
  sq = warp_sum(sq);
  cnt = warp_sum(cnt);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) { red[0][warp] = sq; red[1][warp] = cnt; }
  __syncthreads();
  if (threadIdx.x == 0) {
    float a = 0.f, b = 0.f;
    for (int wv = 0; wv < kDpThreads / 32; ++wv) { a += red[0][wv]; b += red[1][wv]; }
    partial[2 * blockIdx.x] = a;
    partial[2 * blockIdx.x + 1] = b;
  }
}

// totals[0] += sum of the squares, totals[1] += non-finite count over `nparts` partial pairs, in index order (one
// warp, fixed order: the same inputs give the same bits); totals[2] = clip scale from the running totals:
// min(1, max_norm / (sqrt(totals[0]) + 1e-6)), or 0 if anything was non-finite, or 1 if max_norm <= 0.
__global__ void __launch_bounds__(32) dp_reduce_kernel(const float* partial, int nparts, float max_norm, float* totals) {
  float a = 0.f, b = 0.f;
  for (int i = threadIdx.x; i < nparts; i += 32) {
    a += partial[2 * i];
    b += partial[2 * i + 1];
  }
  a = warp_sum(a);
  b = warp_sum(b);
  if (threadIdx.x == 0) {
    const float sq = totals[0] + a, cnt = totals[1] + b;
    totals[0] = sq;
    totals[1] = cnt;
    const float norm = sqrtf(sq);
    float scale = 1.f;
    if (max_norm > 0.f) {
      scale = fminf(1.f, max_norm / (norm + 1e-6f));
      if (cnt != 0.f || !finite_f(norm)) scale = 0.f;
    }
    totals[2] = scale;
  }
}

__global__ void __launch_bounds__(kDpThreads) dp_scale_kernel(float* x, size_t n, const float* scale_dev) {
  const float s = *scale_dev;
  if (s == 1.f) return;
  const Span sp = make_span(x, n);
  float4* v = reinterpret_cast<float4*>(x + sp.head);
  for (size_t u = (size_t)blockIdx.x * blockDim.x + threadIdx.x; u < sp.units; u += (size_t)gridDim.x * blockDim.x) {
    float4 t = v[u];
    v[u] = make_float4(t.x * s, t.y * s, t.z * s, t.w * s);
  }
  if (blockIdx.x == 0)
    for (size_t i = threadIdx.x; i < sp.head + (sp.n - sp.tail_begin); i += blockDim.x) {
      const size_t j = i < sp.head ? i : sp.tail_begin + (i - sp.head);
      x[j] *= s;
    }
}

static int dp_grid(size_t n) {
  const size_t want = (n / 4 + kDpThreads - 1) / kDpThreads;
  return (int)(want < 1 ? 1 : (want > (size_t)kDpMaxCtas ? (size_t)kDpMaxCtas : want));
}

}  // namespace mxb

using namespace mxb;

extern "C" {

size_t mxb_dp_partial_floats(void) { return 2 * (size_t)kDpMaxCtas; }

mxb_status mxb_dp_sanitize(float* x, size_t n, float scale, float* flag, void* stream) {
  if (!x || !flag) return MXB_ERR_INVALID_ARGUMENT;
  if (n == 0) return MXB_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  MXB_LAUNCH("dp_sanitize_kernel", st, (dp_sanitize_kernel<<<dp_grid(n), kDpThreads, 0, st>>>(x, n, scale, flag)));
  return check_launch("dp_sanitize_kernel");
}

static mxb_status dp_finalize_run(float* x, size_t n, float inv_denominator, const float* den_dev, float max_norm,
                                  float* partial, float* totals, void* stream) {
  if (!x || !partial || !totals) return MXB_ERR_INVALID_ARGUMENT;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int grid = dp_grid(n);
  if (n > 0) {
    MXB_LAUNCH("dp_finalize_kernel", st,
               (dp_finalize_kernel<<<grid, kDpThreads, 0, st>>>(x, n, inv_denominator, den_dev, partial)));
    mxb_status s = check_launch("dp_finalize_kernel");
    if (s != MXB_OK) return s;
  }
  MXB_LAUNCH("dp_reduce_kernel", st, (dp_reduce_kernel<<<1, 32, 0, st>>>(partial, n > 0 ? grid : 0, max_norm, totals)));
  return check_launch("dp_reduce_kernel");
}

mxb_status mxb_dp_finalize(float* x, size_t n, float inv_denominator, float max_norm, float* partial, float* totals,
                           void* stream) {
  return dp_finalize_run(x, n, inv_denominator, nullptr, max_norm, partial, totals, stream);
}

mxb_status mxb_dp_finalize_dev(float* x, size_t n, const float* denominator_dev, float max_norm, float* partial,
                               float* totals, void* stream) {
  if (!denominator_dev) return MXB_ERR_INVALID_ARGUMENT;
  return dp_finalize_run(x, n, 1.f, denominator_dev, max_norm, partial, totals, stream);
}

mxb_status mxb_dp_scale(float* x, size_t n, const float* scale_dev, void* stream) {
  if (!x || !scale_dev) return MXB_ERR_INVALID_ARGUMENT;
  if (n == 0) return MXB_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  MXB_LAUNCH("dp_scale_kernel", st, (dp_scale_kernel<<<dp_grid(n), kDpThreads, 0, st>>>(x, n, scale_dev)));
  return check_launch("dp_scale_kernel");
}

}  // extern "C"
