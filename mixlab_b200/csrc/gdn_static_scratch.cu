// Allocation-free forward of the gated delta rule.
//
// mxb_gdn_fwd needs a caller-provided workspace.  Some hosts cannot supply one: a
// program embedded in a runtime that has already reserved the whole device for its
// own memory pool (mixlab's trainer sits on MLX's allocator), or a latency-critical
// loop in which any call into an allocator, which may block or synchronise the
// device, is off limits.  For those callers this file carries its own scratch: a
// fixed array in device global memory that exists once per GPU for as long as the
// library is loaded.  The entry point runs the full-fp32 CUDA-core forward
// (gdn_simt.cu) with that array as its workspace and never calls cudaMalloc,
// cudaFree or any allocating routine.
//
// Consequences of sharing one array:
//   * problems whose workspace exceeds MXB_GDN_STATIC_SCRATCH_BYTES are rejected;
//   * the array keeps whatever the previous call left in it.  The kernels write every
//     scratch element before reading it and the 256-byte status header is cleared on
//     each call, so a call never depends on old contents;
//   * two calls that overlap on the GPU (different streams, or different host threads)
//     would race on the array: callers must serialise them.
//
// In host code the array's name is only a handle, not a device address, so its address
// is obtained with cudaGetSymbolAddress the first time the entry point runs on a
// device (with that device current) and cached per device.  That first call therefore
// does a little one-off set-up work; make it before starting any stream capture.
// The array's memory is reserved by the CUDA runtime when this library's device code is
// loaded on a GPU, which with lazy loading is that same first call: on a device with
// less than the array's size free it fails with MXB_ERR_CUDA.  The cached address
// belongs to the context it was looked up in: it does not survive cudaDeviceReset, and
// the caller's stream must belong to the device that is current during the call.
#include <cstdio>
#include <mutex>

#include "common.cuh"

namespace mxb {

constexpr size_t kStaticScratchBytes = MXB_GDN_STATIC_SCRATCH_BYTES;
constexpr int kMaxDevices = 64;

static __device__ __align__(256) unsigned char g_gdn_scratch[kStaticScratchBytes];

static std::mutex g_scratch_mu;
static void* g_scratch_ptr[kMaxDevices] = {nullptr};

size_t gdn_simt_workspace_bytes(const mxb_gdn_desc*, bool bwd);
bool gdn_simt_supported(const mxb_gdn_desc*);
mxb_status gdn_simt_fwd(const mxb_gdn_desc*, const void*, const void*, const void*, const float*,
                        const float*, const float*, void*, float*, void*, cudaStream_t);

// Device address of the scratch array on the current device (set up once per device).
static mxb_status scratch_address(void** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) { set_last_cuda_error((int)e); return MXB_ERR_CUDA; }
  if (dev < 0 || dev >= kMaxDevices) return MXB_ERR_UNSUPPORTED;
  std::lock_guard<std::mutex> lk(g_scratch_mu);
  if (!g_scratch_ptr[dev]) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_gdn_scratch);
    if (e != cudaSuccess || ptr == nullptr) {
      set_last_cuda_error((int)e);
      std::fprintf(stderr, "[mixlab_b200] cudaGetSymbolAddress(static scratch) failed: %s\n", cudaGetErrorString(e));
      return MXB_ERR_CUDA;
    }
    g_scratch_ptr[dev] = ptr;
  }
  *out = g_scratch_ptr[dev];
  return MXB_OK;
}

}  // namespace mxb

using namespace mxb;

extern "C" {

size_t mxb_gdn_static_scratch_bytes(void) { return kStaticScratchBytes; }

mxb_status mxb_gdn_fwd_static_scratch(const mxb_gdn_desc* d, const void* q, const void* k, const void* v,
                                      const float* beta, const float* gate, const float* h0, void* out,
                                      float* hT, void* stream) {
  if (!d || !q || !k || !v || !beta || !gate || !out) return MXB_ERR_INVALID_ARGUMENT;
  if (d->B <= 0 || d->T <= 0 || d->H <= 0 || d->Dk <= 0 || d->Dv <= 0) return MXB_ERR_INVALID_ARGUMENT;
  if (d->io_dtype != MXB_F32 && d->io_dtype != MXB_BF16) return MXB_ERR_INVALID_ARGUMENT;
  if (d->gate_is_log != 0 && d->gate_is_log != 1) return MXB_ERR_INVALID_ARGUMENT;
  if (!gdn_simt_supported(d)) return MXB_ERR_UNSUPPORTED;
  // Only the forward-sized scratch is checked against the array, so the flags that would make the kernels keep
  // more in it (MXB_GDN_SAVE_FOR_BWD: the saved tiles could not be handed to a backward anyway, the array's
  // address is private) or pick other kernels are dropped from a private copy of the descriptor.
  mxb_gdn_desc own = *d;
  own.flags = MXB_GDN_FORCE_FP32_PATH;
  d = &own;
  const size_t need = gdn_simt_workspace_bytes(d, false);
  if (need > kStaticScratchBytes) {
    std::fprintf(stderr,
                 "[mixlab_b200] mxb_gdn_fwd_static_scratch: this problem needs %zu bytes of scratch, the built-in "
                 "array holds %zu; use mxb_gdn_fwd with a caller-provided workspace\n",
                 need, kStaticScratchBytes);
    return MXB_ERR_WORKSPACE;
  }
  void* ws = nullptr;
  if (need > 0) {
    mxb_status s = scratch_address(&ws);
    if (s != MXB_OK) return s;
  }
  return gdn_simt_fwd(d, q, k, v, beta, gate, h0, out, hT, ws, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
