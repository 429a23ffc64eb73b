// Shared device/host helpers for the mixlab_b200 kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/mixlab_b200.h"

namespace mxb {

// Numeric guards of the reference's chunked scan (gpu/ir.cpp:35-37).
constexpr float kGateFloor = 1e-30f;
constexpr float kLogGateFloor = -69.07755278982137f;  // log(1e-30)
constexpr float kExpClampMin = -80.0f;

// exp(clamp(x, -80, 0)) - stable_exp_nonpos, gpu/ir.cpp:903-905.
__device__ __forceinline__ float exp_nonpos(float x) {
  return __expf(fminf(fmaxf(x, kExpClampMin), 0.0f));
}
// Full-precision variant for the fp32 parity path.
__device__ __forceinline__ float exp_nonpos_precise(float x) {
  return expf(fminf(fmaxf(x, kExpClampMin), 0.0f));
}

template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Column sums over the 16 rows that lanes 0-15 of a warp hold (lanes 16-31 must pass zeros): v[c] is this
// lane's value for column c.  Recursive halving: 30 shuffles instead of 32 x 4.  On return lane l holds in
// v[0], v[1] the sums of columns colsum16_col(l) and colsum16_col(l) + 1.
template <int M, int N, int W>
__device__ __forceinline__ void colsum16_step(float (&v)[W], int lane) {
  const bool up = (lane & M) != 0;
#pragma unroll
  for (int k = 0; k < N; ++k) {
    const float send = up ? v[k] : v[k + N];
    const float keep = up ? v[k + N] : v[k];
    v[k] = keep + __shfl_xor_sync(0xffffffffu, send, M);
  }
}
__device__ __forceinline__ void colsum16(float (&v)[32], int lane) {
  colsum16_step<8, 16, 32>(v, lane);
  colsum16_step<4, 8, 32>(v, lane);
  colsum16_step<2, 4, 32>(v, lane);
  colsum16_step<1, 2, 32>(v, lane);
}
__device__ __forceinline__ int colsum16_col(int lane) { return 2 * (lane & 15); }

// Same for 16 columns: on return lane l holds in v[0] the sum of column (l & 15).  15 shuffles.
__device__ __forceinline__ void colsum16(float (&v)[16], int lane) {
  colsum16_step<8, 8, 16>(v, lane);
  colsum16_step<4, 4, 16>(v, lane);
  colsum16_step<2, 2, 16>(v, lane);
  colsum16_step<1, 1, 16>(v, lane);
}

// Reverse inclusive cumulative sum over 64 values by one warp, two per lane: call with a = x[63 - 2 lane],
// b = x[62 - 2 lane]; returns in a, b the sums x[63] + ... + x[63 - 2 lane] and ... + x[62 - 2 lane].  A fixed order.
__device__ __forceinline__ void warp_rcumsum64(float& a, float& b, int lane) {
  float v = a + b;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float t = __shfl_up_sync(0xffffffffu, v, o);
    if (lane >= o) v += t;
  }
  a = v - b;
  b = v;
}

// ---- host side ----------------------------------------------------------
void note_launch(int n = 1);           // bumps mxb_launch_count()
mxb_status check_launch(const char* what);  // cudaGetLastError -> status
void set_last_cuda_error(int e);
// Optional per-launch CUDA-event tracing (mxb_trace_enable); no-ops when off.
void trace_begin(const char* name, cudaStream_t st);
void trace_end(cudaStream_t st);

// Launch wrapper: counts the launch and, when tracing is on, brackets it with events.
#define MXB_LAUNCH(name, st, ...)   \
  do {                              \
    ::mxb::trace_begin(name, st);   \
    __VA_ARGS__;                    \
    ::mxb::trace_end(st);           \
    ::mxb::note_launch();           \
  } while (0)

inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// Carves a caller-provided workspace into 256-byte aligned pieces.
struct Carver {
  char* base;
  size_t off = 0;
  explicit Carver(void* p) : base(static_cast<char*>(p)) {}
  template <typename T>
  T* take(size_t count) {
    off = align_up(off, 256);
    T* r = base ? reinterpret_cast<T*>(base + off) : nullptr;
    off += count * sizeof(T);
    return r;
  }
  size_t bytes() const { return align_up(off, 256); }
};

}  // namespace mxb
