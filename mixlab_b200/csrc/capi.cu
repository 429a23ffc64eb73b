// C ABI of libmixlab_b200: argument validation, path selection, host-buffer
// context.  Declarations and the reference interfaces they replace are in
// include/mixlab_b200.h.
#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <new>
#include <string>
#include <vector>

#include "common.cuh"

namespace mxb {

static std::atomic<uint64_t> g_launches{0};
static thread_local int g_last_cuda_error = 0;

void note_launch(int n) { g_launches.fetch_add((uint64_t)n, std::memory_order_relaxed); }
void set_last_cuda_error(int e) { g_last_cuda_error = e; }
mxb_status check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) return MXB_OK;
  g_last_cuda_error = (int)e;
  std::fprintf(stderr, "[mixlab_b200] %s: %s\n", what, cudaGetErrorString(e));
  return MXB_ERR_CUDA;
}

// ---- per-launch event tracing -------------------------------------------
struct TraceRec { const char* name; cudaEvent_t e0, e1; };
static std::atomic<bool> g_trace_on{false};
static std::mutex g_trace_mu;
static std::vector<TraceRec> g_trace;
static thread_local cudaEvent_t g_open_e0 = nullptr;
static thread_local const char* g_open_name = nullptr;

void trace_begin(const char* name, cudaStream_t st) {
  if (!g_trace_on.load(std::memory_order_relaxed)) return;
  cudaEvent_t e = nullptr;
  if (cudaEventCreate(&e) != cudaSuccess) return;
  cudaEventRecord(e, st);
  g_open_e0 = e;
  g_open_name = name;
}
void trace_end(cudaStream_t st) {
  if (!g_open_e0) return;
  cudaEvent_t e = nullptr;
  if (cudaEventCreate(&e) == cudaSuccess) {
    cudaEventRecord(e, st);
    std::lock_guard<std::mutex> lk(g_trace_mu);
    g_trace.push_back({g_open_name, g_open_e0, e});
  } else {
    cudaEventDestroy(g_open_e0);
  }
  g_open_e0 = nullptr;
}
static void trace_clear() {
  std::lock_guard<std::mutex> lk(g_trace_mu);
  for (auto& r : g_trace) { cudaEventDestroy(r.e0); cudaEventDestroy(r.e1); }
  g_trace.clear();
}

// kernels (other translation units)
mxb_status gdn_decode_dispatch(const mxb_gdn_desc*, float*, const void*, const void*, const void*,
                               const float*, const float*, void*, cudaStream_t);
size_t gdn_simt_workspace_bytes(const mxb_gdn_desc*, bool bwd);
bool gdn_simt_supported(const mxb_gdn_desc*);
mxb_status gdn_simt_fwd(const mxb_gdn_desc*, const void*, const void*, const void*, const float*,
                        const float*, const float*, void*, float*, void*, cudaStream_t);
mxb_status gdn_simt_bwd(const mxb_gdn_desc*, const void*, const void*, const void*, const float*,
                        const float*, const float*, const void*, const float*, void*, void*, void*,
                        float*, float*, float*, void*, cudaStream_t);
bool gdn_tc_supported(const mxb_gdn_desc*);
bool gdn_f32io_wanted(const mxb_gdn_desc*);
size_t gdn_f32io_workspace_bytes(const mxb_gdn_desc*, bool bwd);
mxb_status gdn_f32io_fwd(const mxb_gdn_desc*, const void*, const void*, const void*, const float*, const float*,
                         const float*, void*, float*, void*, cudaStream_t);
mxb_status gdn_f32io_bwd(const mxb_gdn_desc*, const void*, const void*, const void*, const float*, const float*,
                         const float*, const void*, const float*, void*, void*, void*, float*, float*, float*, void*,
                         cudaStream_t);
size_t gdn_tc_workspace_bytes(const mxb_gdn_desc*, bool bwd);
mxb_status gdn_tc_fwd(const mxb_gdn_desc*, const void*, const void*, const void*, const float*,
                      const float*, const float*, void*, float*, void*, cudaStream_t);
mxb_status gdn_tc_bwd(const mxb_gdn_desc*, const void*, const void*, const void*, const float*,
                      const float*, const float*, const void*, const float*, void*, void*, void*,
                      float*, float*, float*, void*, cudaStream_t);
mxb_status umma_selftest(const void*, uint32_t, const void*, uint32_t, const uint32_t*, float*, int*, cudaStream_t);
mxb_status wait_timeout_selftest(void*, uint32_t, cudaStream_t);
bool gdn_block_supported(const mxb_gdn_desc*);
size_t gdn_block_workspace_bytes(const mxb_gdn_desc*);
mxb_status gdn_block_pre_fwd(const mxb_gdn_desc*, const void*, const void*, const void*, const float*, const float*,
                             const float*, const float*, const float*, const float*, const float*, void*, void*, void*,
                             float*, float*, cudaStream_t);
mxb_status gdn_block_pre_bwd(const mxb_gdn_desc*, const void*, const void*, const void*, const float*, const float*,
                             const float*, const float*, const float*, const float*, const float*, const void*,
                             const void*, const void*, const float*, const float*, void*, void*, void*, float*, float*,
                             float*, float*, float*, float*, float*, void*, cudaStream_t);
mxb_status gdn_block_post(const mxb_gdn_desc*, const void*, const void*, const float*, void*, const void*, void*, void*,
                          float*, void*, cudaStream_t);
bool mamba3_block_supported(const mxb_mamba3_desc*);
size_t mamba3_block_workspace_bytes(const mxb_mamba3_desc*);
mxb_status mamba3_block_conv(const mxb_mamba3_desc*, int, const void*, const float*, void*, const void*, void*, float*,
                             void*, cudaStream_t);
mxb_status mamba3_block_bc(const mxb_mamba3_desc*, float, const void*, const void*, const float*, const float*,
                           const float*, const float*, void*, void*, const void*, const void*, void*, void*, float*,
                           float*, float*, float*, void*, cudaStream_t);
mxb_status mamba3_block_post(const mxb_mamba3_desc*, float, const void*, const void*, const float*, void*, const void*,
                             void*, void*, float*, void*, cudaStream_t);
bool mamba3_supported(const mxb_mamba3_desc*);
size_t mamba3_workspace_bytes(const mxb_mamba3_desc*, bool bwd);
mxb_status mamba3_fwd(const mxb_mamba3_desc*, const void*, const float*, const float*, const float*,
                      const float*, const void*, const void*, void*, void*, cudaStream_t);
mxb_status mamba3_bwd(const mxb_mamba3_desc*, const void*, const float*, const float*, const float*,
                      const float*, const void*, const void*, const void*, void*, float*, float*,
                      float*, float*, void*, void*, void*, cudaStream_t);

static mxb_status check_gdn_desc(const mxb_gdn_desc* d, bool need_T) {
  if (!d) return MXB_ERR_INVALID_ARGUMENT;
  if (d->B <= 0 || d->H <= 0 || d->Dk <= 0 || d->Dv <= 0) return MXB_ERR_INVALID_ARGUMENT;
  if (need_T && d->T <= 0) return MXB_ERR_INVALID_ARGUMENT;
  if (d->io_dtype != MXB_F32 && d->io_dtype != MXB_BF16) return MXB_ERR_INVALID_ARGUMENT;
  if (d->gate_is_log != 0 && d->gate_is_log != 1) return MXB_ERR_INVALID_ARGUMENT;
  return MXB_OK;
}

static bool use_tc(const mxb_gdn_desc* d) {
  return !(d->flags & MXB_GDN_FORCE_FP32_PATH) && gdn_tc_supported(d);
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace mxb

using namespace mxb;

extern "C" {

const char* mxb_status_string(mxb_status s) {
  switch (s) {
    case MXB_OK: return "ok";
    case MXB_ERR_INVALID_ARGUMENT: return "invalid argument";
    case MXB_ERR_UNSUPPORTED: return "unsupported shape or dtype";
    case MXB_ERR_WORKSPACE: return "workspace missing or too small";
    case MXB_ERR_CUDA: return "CUDA runtime error";
    case MXB_ERR_ALIGNMENT: return "pointer not sufficiently aligned";
    case MXB_ERR_NO_DEVICE: return "no sm_100 CUDA device (there is no CPU fallback)";
    default: return "unknown status";
  }
}

int mxb_version(void) { return 100; }
int mxb_last_cuda_error(void) { return g_last_cuda_error; }
uint64_t mxb_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

void mxb_trace_enable(int on) {
  trace_clear();
  g_trace_on.store(on != 0);
}

size_t mxb_trace_summary(char* buf, size_t cap) {
  // one line per kernel name: "<name> <launches> <total_ms>\n"; waits for the recorded events.
  std::lock_guard<std::mutex> lk(g_trace_mu);
  std::vector<std::string> names;
  std::vector<int> counts;
  std::vector<double> totals;
  for (auto& r : g_trace) {
    if (cudaEventSynchronize(r.e1) != cudaSuccess) continue;
    float ms = 0.f;
    if (cudaEventElapsedTime(&ms, r.e0, r.e1) != cudaSuccess) continue;
    size_t i = 0;
    for (; i < names.size(); ++i) if (names[i] == r.name) break;
    if (i == names.size()) { names.push_back(r.name); counts.push_back(0); totals.push_back(0.0); }
    counts[i] += 1;
    totals[i] += ms;
  }
  std::string out;
  for (size_t i = 0; i < names.size(); ++i) {
    char line[256];
    std::snprintf(line, sizeof line, "%s %d %.6f\n", names[i].c_str(), counts[i], totals[i]);
    out += line;
  }
  if (buf && cap > 0) {
    const size_t n = out.size() < cap - 1 ? out.size() : cap - 1;
    std::memcpy(buf, out.data(), n);
    buf[n] = 0;
  }
  return out.size();
}

size_t mxb_gdn_fwd_workspace_bytes(const mxb_gdn_desc* d) {
  if (check_gdn_desc(d, true) != MXB_OK) return 0;
  const bool save = (d->flags & MXB_GDN_SAVE_FOR_BWD) != 0;
  if (gdn_f32io_wanted(d)) return gdn_f32io_workspace_bytes(d, false);
  if (use_tc(d)) return gdn_tc_workspace_bytes(d, save);
  return gdn_simt_workspace_bytes(d, save);
}

size_t mxb_gdn_bwd_workspace_bytes(const mxb_gdn_desc* d) {
  if (check_gdn_desc(d, true) != MXB_OK) return 0;
  if (gdn_f32io_wanted(d)) return gdn_f32io_workspace_bytes(d, true);
  if (use_tc(d)) return gdn_tc_workspace_bytes(d, true);
  return gdn_simt_workspace_bytes(d, true);
}

mxb_status mxb_gdn_fwd(const mxb_gdn_desc* d, const void* q, const void* k, const void* v,
                       const float* beta, const float* gate, const float* h0, void* out, float* hT,
                       void* workspace, size_t workspace_bytes, void* stream) {
  mxb_status s = check_gdn_desc(d, true);
  if (s != MXB_OK) return s;
  if (!q || !k || !v || !beta || !gate || !out) return MXB_ERR_INVALID_ARGUMENT;
  const size_t need = mxb_gdn_fwd_workspace_bytes(d);
  if (need > 0 && (!workspace || workspace_bytes < need)) return MXB_ERR_WORKSPACE;
  if (need > 0 && !aligned16(workspace)) return MXB_ERR_ALIGNMENT;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool f32io = gdn_f32io_wanted(d);
  if (f32io || use_tc(d)) {  // these kernels move whole 16-byte units (TMA tiles, bulk copies, 128-bit loads)
    if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(out) || !aligned16(h0) || !aligned16(hT))
      return MXB_ERR_ALIGNMENT;
    if (f32io) return gdn_f32io_fwd(d, q, k, v, beta, gate, h0, out, hT, workspace, st);
    return gdn_tc_fwd(d, q, k, v, beta, gate, h0, out, hT, workspace, st);
  }
  if (!gdn_simt_supported(d)) return MXB_ERR_UNSUPPORTED;
  return gdn_simt_fwd(d, q, k, v, beta, gate, h0, out, hT, workspace, st);
}

mxb_status mxb_gdn_bwd(const mxb_gdn_desc* d, const void* q, const void* k, const void* v,
                       const float* beta, const float* gate, const float* h0, const void* d_out,
                       const float* d_hT, void* dq, void* dk, void* dv, float* dbeta, float* dgate,
                       float* dh0, void* workspace, size_t workspace_bytes, void* stream) {
  mxb_status s = check_gdn_desc(d, true);
  if (s != MXB_OK) return s;
  if (!q || !k || !v || !beta || !gate || !d_out || !dq || !dk || !dv || !dbeta || !dgate)
    return MXB_ERR_INVALID_ARGUMENT;
  const size_t need = mxb_gdn_bwd_workspace_bytes(d);
  if (!workspace || workspace_bytes < need) return MXB_ERR_WORKSPACE;
  if (!aligned16(workspace)) return MXB_ERR_ALIGNMENT;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool f32io = gdn_f32io_wanted(d);
  if (f32io || use_tc(d)) {
    if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(d_out) || !aligned16(dq) || !aligned16(dk) ||
        !aligned16(dv) || !aligned16(h0) || !aligned16(d_hT) || !aligned16(dh0))
      return MXB_ERR_ALIGNMENT;
    if (f32io)
      return gdn_f32io_bwd(d, q, k, v, beta, gate, h0, d_out, d_hT, dq, dk, dv, dbeta, dgate, dh0, workspace, st);
    return gdn_tc_bwd(d, q, k, v, beta, gate, h0, d_out, d_hT, dq, dk, dv, dbeta, dgate, dh0, workspace, st);
  }
  if (!gdn_simt_supported(d)) return MXB_ERR_UNSUPPORTED;
  return gdn_simt_bwd(d, q, k, v, beta, gate, h0, d_out, d_hT, dq, dk, dv, dbeta, dgate, dh0, workspace, st);
}

mxb_status mxb_gdn_device_status(const void* workspace, int32_t* out) {
  if (!workspace || !out) return MXB_ERR_INVALID_ARGUMENT;
  cudaError_t e = cudaMemcpy(out, workspace, sizeof(int32_t), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) { g_last_cuda_error = (int)e; return MXB_ERR_CUDA; }
  return MXB_OK;
}

mxb_status mxb_gdn_decode_step(const mxb_gdn_desc* d, float* state, const void* q, const void* k,
                               const void* v, const float* beta, const float* gate, void* out,
                               void* stream) {
  mxb_status s = check_gdn_desc(d, false);
  if (s != MXB_OK) return s;
  if (!state || !q || !k || !v || !beta || !gate || !out) return MXB_ERR_INVALID_ARGUMENT;
  if (!aligned16(state)) return MXB_ERR_ALIGNMENT;
  return gdn_decode_dispatch(d, state, q, k, v, beta, gate, out, static_cast<cudaStream_t>(stream));
}

// ---------------------------------------------------------------- gated_deltanet block stages
static mxb_status check_block_desc(const mxb_gdn_desc* d) {
  if (!d) return MXB_ERR_INVALID_ARGUMENT;
  if (d->B <= 0 || d->T <= 0 || d->H <= 0 || d->Dk <= 0 || d->Dv <= 0) return MXB_ERR_INVALID_ARGUMENT;
  if (d->io_dtype != MXB_F32 && d->io_dtype != MXB_BF16) return MXB_ERR_INVALID_ARGUMENT;
  if (!gdn_block_supported(d)) return MXB_ERR_UNSUPPORTED;
  return MXB_OK;
}
size_t mxb_gdn_block_workspace_bytes(const mxb_gdn_desc* d) {
  return check_block_desc(d) == MXB_OK ? gdn_block_workspace_bytes(d) : 0;
}
mxb_status mxb_gdn_block_pre_fwd(const mxb_gdn_desc* d, const void* q_proj, const void* k_proj, const void* v_proj,
                                 const float* conv_q, const float* conv_k, const float* conv_v, const float* a_raw,
                                 const float* b_raw, const float* a_log, const float* dt_bias, void* q, void* k,
                                 void* v, float* beta, float* gate, void* stream) {
  mxb_status s = check_block_desc(d);
  if (s != MXB_OK) return s;
  if (!q_proj || !k_proj || !v_proj || !conv_q || !conv_k || !conv_v || !a_raw || !b_raw || !a_log || !dt_bias || !q ||
      !k || !v || !beta || !gate)
    return MXB_ERR_INVALID_ARGUMENT;
  if (!aligned16(q_proj) || !aligned16(k_proj) || !aligned16(v_proj) || !aligned16(q) || !aligned16(k) || !aligned16(v) ||
      !aligned16(conv_q) || !aligned16(conv_k) || !aligned16(conv_v))
    return MXB_ERR_ALIGNMENT;
  return gdn_block_pre_fwd(d, q_proj, k_proj, v_proj, conv_q, conv_k, conv_v, a_raw, b_raw, a_log, dt_bias, q, k, v, beta,
                           gate, static_cast<cudaStream_t>(stream));
}
mxb_status mxb_gdn_block_pre_bwd(const mxb_gdn_desc* d, const void* q_proj, const void* k_proj, const void* v_proj,
                                 const float* conv_q, const float* conv_k, const float* conv_v, const float* a_raw,
                                 const float* b_raw, const float* a_log, const float* dt_bias, const void* dq,
                                 const void* dk, const void* dv, const float* dbeta, const float* dgate, void* dq_proj,
                                 void* dk_proj, void* dv_proj, float* dconv_q, float* dconv_k, float* dconv_v,
                                 float* da_raw, float* db_raw, float* da_log, float* ddt_bias, void* workspace,
                                 size_t workspace_bytes, void* stream) {
  mxb_status s = check_block_desc(d);
  if (s != MXB_OK) return s;
  if (!q_proj || !k_proj || !v_proj || !conv_q || !conv_k || !conv_v || !a_raw || !b_raw || !a_log || !dt_bias || !dq ||
      !dk || !dv || !dbeta || !dgate || !dq_proj || !dk_proj || !dv_proj || !dconv_q || !dconv_k || !dconv_v || !da_raw ||
      !db_raw || !da_log || !ddt_bias || !workspace)
    return MXB_ERR_INVALID_ARGUMENT;
  if (!aligned16(q_proj) || !aligned16(k_proj) || !aligned16(v_proj) || !aligned16(dq) || !aligned16(dk) || !aligned16(dv) ||
      !aligned16(dq_proj) || !aligned16(dk_proj) || !aligned16(dv_proj) || !aligned16(conv_q) || !aligned16(conv_k) ||
      !aligned16(conv_v) || !aligned16(workspace))
    return MXB_ERR_ALIGNMENT;
  if (workspace_bytes < gdn_block_workspace_bytes(d)) return MXB_ERR_WORKSPACE;
  return gdn_block_pre_bwd(d, q_proj, k_proj, v_proj, conv_q, conv_k, conv_v, a_raw, b_raw, a_log, dt_bias, dq, dk, dv, dbeta,
                           dgate, dq_proj, dk_proj, dv_proj, dconv_q, dconv_k, dconv_v, da_raw, db_raw, da_log, ddt_bias,
                           workspace, static_cast<cudaStream_t>(stream));
}
mxb_status mxb_gdn_block_post_fwd(const mxb_gdn_desc* d, const void* o, const void* z, const float* o_norm, void* y,
                                  void* stream) {
  mxb_status s = check_block_desc(d);
  if (s != MXB_OK) return s;
  if (!o || !z || !o_norm || !y) return MXB_ERR_INVALID_ARGUMENT;
  if (!aligned16(o) || !aligned16(z) || !aligned16(y) || !aligned16(o_norm)) return MXB_ERR_ALIGNMENT;
  return gdn_block_post(d, o, z, o_norm, y, nullptr, nullptr, nullptr, nullptr, nullptr, static_cast<cudaStream_t>(stream));
}
mxb_status mxb_gdn_block_post_bwd(const mxb_gdn_desc* d, const void* o, const void* z, const float* o_norm,
                                  const void* dy, void* d_o, void* dz, float* do_norm, void* workspace,
                                  size_t workspace_bytes, void* stream) {
  mxb_status s = check_block_desc(d);
  if (s != MXB_OK) return s;
  if (!o || !z || !o_norm || !dy || !d_o || !dz || !do_norm || !workspace) return MXB_ERR_INVALID_ARGUMENT;
  if (!aligned16(o) || !aligned16(z) || !aligned16(dy) || !aligned16(d_o) || !aligned16(dz) || !aligned16(o_norm) ||
      !aligned16(workspace))
    return MXB_ERR_ALIGNMENT;
  if (workspace_bytes < gdn_block_workspace_bytes(d)) return MXB_ERR_WORKSPACE;
  return gdn_block_post(d, o, z, o_norm, nullptr, dy, d_o, dz, do_norm, workspace, static_cast<cudaStream_t>(stream));
}

static mxb_status check_m3_desc(const mxb_mamba3_desc* d) {
  if (!d) return MXB_ERR_INVALID_ARGUMENT;
  if (d->B <= 0 || d->T <= 0 || d->D <= 0 || d->N <= 0 || d->G <= 0) return MXB_ERR_INVALID_ARGUMENT;
  if (d->io_dtype != MXB_F32 && d->io_dtype != MXB_BF16) return MXB_ERR_INVALID_ARGUMENT;
  if (!mamba3_supported(d)) return MXB_ERR_UNSUPPORTED;
  return MXB_OK;
}

size_t mxb_mamba3_fwd_workspace_bytes(const mxb_mamba3_desc* d) {
  return check_m3_desc(d) == MXB_OK ? mamba3_workspace_bytes(d, false) : 0;
}
size_t mxb_mamba3_bwd_workspace_bytes(const mxb_mamba3_desc* d) {
  return check_m3_desc(d) == MXB_OK ? mamba3_workspace_bytes(d, true) : 0;
}

mxb_status mxb_mamba3_fwd(const mxb_mamba3_desc* d, const void* x, const float* dt, const float* lambda,
                          const float* theta, const float* a_log, const void* b, const void* c, void* y,
                          void* workspace, size_t workspace_bytes, void* stream) {
  mxb_status s = check_m3_desc(d);
  if (s != MXB_OK) return s;
  if (!x || !dt || !lambda || !theta || !a_log || !b || !c || !y) return MXB_ERR_INVALID_ARGUMENT;
  const size_t need = mamba3_workspace_bytes(d, false);
  if (need > 0 && (!workspace || workspace_bytes < need)) return MXB_ERR_WORKSPACE;
  return mamba3_fwd(d, x, dt, lambda, theta, a_log, b, c, y, workspace, static_cast<cudaStream_t>(stream));
}

mxb_status mxb_mamba3_bwd(const mxb_mamba3_desc* d, const void* x, const float* dt, const float* lambda,
                          const float* theta, const float* a_log, const void* b, const void* c,
                          const void* dy, void* dx, float* ddt, float* dlambda, float* dtheta,
                          float* da_log, void* db, void* dc, void* workspace, size_t workspace_bytes,
                          void* stream) {
  mxb_status s = check_m3_desc(d);
  if (s != MXB_OK) return s;
  if (!x || !dt || !lambda || !theta || !a_log || !b || !c || !dy || !dx || !ddt || !dlambda ||
      !dtheta || !da_log || !db || !dc)
    return MXB_ERR_INVALID_ARGUMENT;
  const size_t need = mamba3_workspace_bytes(d, true);
  if (!workspace || workspace_bytes < need) return MXB_ERR_WORKSPACE;
  return mamba3_bwd(d, x, dt, lambda, theta, a_log, b, c, dy, dx, ddt, dlambda, dtheta, da_log, db, dc,
                    workspace, static_cast<cudaStream_t>(stream));
}

// ---------------------------------------------------------------- IR op records
static mxb_status ir_op_to_gdn(const mxb_ir_op* op, mxb_gdn_desc* d) {
  if (op->n_inputs < 5 || op->n_outputs < 1 || op->n_int_params < 5 || !op->inputs || !op->outputs || !op->int_params)
    return MXB_ERR_INVALID_ARGUMENT;  // "OP_GATED_DELTA_SCAN requires B,T,H,Dk,Dv"
  const int32_t* ip = op->int_params;
  *d = mxb_gdn_desc{ip[0], ip[1], ip[2], ip[3], ip[4], op->n_int_params >= 6 ? ip[5] : 0, op->io_dtype, 0, 0};
  if (d->chunk < 0) d->chunk = 0;
  // The record has no room for kernel-selection bits: a deployment that accepts bf16 operand rounding for its float32
  // tensors says so once per process (MXB_IR_GDN_FLAGS=64 is MXB_GDN_F32_IO_BF16_OPERANDS), and its unchanged op
  // records then reach the tensor-core kernels.
  static const int32_t env_flags = [] {
    const char* e = std::getenv("MXB_IR_GDN_FLAGS");
    return e ? (int32_t)std::atoi(e) : 0;
  }();
  d->flags = env_flags & (MXB_GDN_F32_IO_BF16_OPERANDS | MXB_GDN_FORCE_FP32_PATH | MXB_GDN_NO_TMA);
  return MXB_OK;
}
static mxb_status ir_op_to_m3(const mxb_ir_op* op, mxb_mamba3_desc* d) {
  if (op->n_inputs < 7 || op->n_outputs < 1 || op->n_int_params < 5 || !op->inputs || !op->outputs || !op->int_params)
    return MXB_ERR_INVALID_ARGUMENT;  // "OP_MAMBA3_SELECTIVE_SCAN requires 7 inputs and B,T,D,N,G params"
  const int32_t* ip = op->int_params;
  *d = mxb_mamba3_desc{ip[0], ip[1], ip[2], ip[3], ip[4], 0, op->io_dtype, 0};
  return MXB_OK;
}

size_t mxb_ir_op_workspace_bytes(const mxb_ir_op* op) {
  if (!op) return 0;
  if (op->op_type == MXB_OP_GATED_DELTA_SCAN) {
    mxb_gdn_desc d;
    return ir_op_to_gdn(op, &d) == MXB_OK ? mxb_gdn_fwd_workspace_bytes(&d) : 0;
  }
  if (op->op_type == MXB_OP_MAMBA3_SELECTIVE_SCAN) {
    mxb_mamba3_desc d;
    return ir_op_to_m3(op, &d) == MXB_OK ? mxb_mamba3_fwd_workspace_bytes(&d) : 0;
  }
  return 0;
}

mxb_status mxb_ir_op_forward(const mxb_ir_op* op, void* workspace, size_t workspace_bytes, void* stream) {
  if (!op) return MXB_ERR_INVALID_ARGUMENT;
  if (op->op_type == MXB_OP_GATED_DELTA_SCAN) {
    mxb_gdn_desc d;
    mxb_status s = ir_op_to_gdn(op, &d);
    if (s != MXB_OK) return s;
    const void* const* in = op->inputs;
    return mxb_gdn_fwd(&d, in[0], in[1], in[2], static_cast<const float*>(in[3]), static_cast<const float*>(in[4]), nullptr,
                       op->outputs[0], nullptr, workspace, workspace_bytes, stream);
  }
  if (op->op_type == MXB_OP_MAMBA3_SELECTIVE_SCAN) {
    mxb_mamba3_desc d;
    mxb_status s = ir_op_to_m3(op, &d);
    if (s != MXB_OK) return s;
    const void* const* in = op->inputs;
    return mxb_mamba3_fwd(&d, in[0], static_cast<const float*>(in[1]), static_cast<const float*>(in[2]),
                          static_cast<const float*>(in[3]), static_cast<const float*>(in[4]), in[5], in[6], op->outputs[0],
                          workspace, workspace_bytes, stream);
  }
  return MXB_ERR_UNSUPPORTED;
}

mxb_status mxb_selftest_umma(const void* a_img, uint32_t a_bytes, const void* b_img, uint32_t b_bytes,
                             const uint32_t* fields, float* d_out, int* status, void* stream) {
  if (!a_img || !b_img || !fields || !d_out || !status) return MXB_ERR_INVALID_ARGUMENT;
  return umma_selftest(a_img, a_bytes, b_img, b_bytes, fields, d_out, status, static_cast<cudaStream_t>(stream));
}

mxb_status mxb_selftest_wait_timeout(void* workspace, size_t workspace_bytes, uint32_t poll_limit, void* stream) {
  if (!workspace || workspace_bytes < 256) return MXB_ERR_WORKSPACE;
  if (!aligned16(workspace)) return MXB_ERR_ALIGNMENT;
  return wait_timeout_selftest(workspace, poll_limit, static_cast<cudaStream_t>(stream));
}

// ---------------------------------------------------------------- Mamba-3 block stages
static mxb_status check_m3_block_desc(const mxb_mamba3_desc* d) {
  if (!d) return MXB_ERR_INVALID_ARGUMENT;
  if (d->B <= 0 || d->T <= 0 || d->D <= 0 || d->N <= 0 || d->G <= 0) return MXB_ERR_INVALID_ARGUMENT;
  if (d->io_dtype != MXB_F32 && d->io_dtype != MXB_BF16) return MXB_ERR_INVALID_ARGUMENT;
  if (!mamba3_block_supported(d)) return MXB_ERR_UNSUPPORTED;
  return MXB_OK;
}
size_t mxb_mamba3_block_workspace_bytes(const mxb_mamba3_desc* d) {
  return check_m3_block_desc(d) == MXB_OK ? mamba3_block_workspace_bytes(d) : 0;
}
mxb_status mxb_mamba3_block_conv_fwd(const mxb_mamba3_desc* d, int32_t K, const void* x, const float* w, void* y,
                                     void* stream) {
  mxb_status s = check_m3_block_desc(d);
  if (s != MXB_OK) return s;
  if (K < 1 || K > 4) return MXB_ERR_UNSUPPORTED;
  if (!x || !w || !y) return MXB_ERR_INVALID_ARGUMENT;
  if (!aligned16(x) || !aligned16(y)) return MXB_ERR_ALIGNMENT;
  return mamba3_block_conv(d, K, x, w, y, nullptr, nullptr, nullptr, nullptr, static_cast<cudaStream_t>(stream));
}
mxb_status mxb_mamba3_block_conv_bwd(const mxb_mamba3_desc* d, int32_t K, const void* x, const float* w, const void* dy,
                                     void* dx, float* dw, void* workspace, size_t workspace_bytes, void* stream) {
  mxb_status s = check_m3_block_desc(d);
  if (s != MXB_OK) return s;
  if (K < 1 || K > 4) return MXB_ERR_UNSUPPORTED;
  if (!x || !w || !dy || !dx || !dw || !workspace) return MXB_ERR_INVALID_ARGUMENT;
  if (!aligned16(x) || !aligned16(dy) || !aligned16(dx) || !aligned16(workspace)) return MXB_ERR_ALIGNMENT;
  if (workspace_bytes < mamba3_block_workspace_bytes(d)) return MXB_ERR_WORKSPACE;
  return mamba3_block_conv(d, K, x, w, nullptr, dy, dx, dw, workspace, static_cast<cudaStream_t>(stream));
}
mxb_status mxb_mamba3_block_bc_fwd(const mxb_mamba3_desc* d, float eps, const void* b_proj, const void* c_proj,
                                   const float* b_scale, const float* c_scale, const float* b_bias, const float* c_bias,
                                   void* b, void* c, void* stream) {
  mxb_status s = check_m3_block_desc(d);
  if (s != MXB_OK) return s;
  if (!b_proj || !c_proj || !b_scale || !c_scale || !b_bias || !c_bias || !b || !c) return MXB_ERR_INVALID_ARGUMENT;
  if (!aligned16(b_proj) || !aligned16(c_proj) || !aligned16(b) || !aligned16(c) || !aligned16(b_scale) ||
      !aligned16(c_scale) || !aligned16(b_bias) || !aligned16(c_bias))
    return MXB_ERR_ALIGNMENT;
  return mamba3_block_bc(d, eps, b_proj, c_proj, b_scale, c_scale, b_bias, c_bias, b, c, nullptr, nullptr, nullptr, nullptr,
                         nullptr, nullptr, nullptr, nullptr, nullptr, static_cast<cudaStream_t>(stream));
}
mxb_status mxb_mamba3_block_bc_bwd(const mxb_mamba3_desc* d, float eps, const void* b_proj, const void* c_proj,
                                   const float* b_scale, const float* c_scale, const void* db, const void* dc,
                                   void* db_proj, void* dc_proj, float* db_scale, float* dc_scale, float* db_bias,
                                   float* dc_bias, void* workspace, size_t workspace_bytes, void* stream) {
  mxb_status s = check_m3_block_desc(d);
  if (s != MXB_OK) return s;
  if (!b_proj || !c_proj || !b_scale || !c_scale || !db || !dc || !db_proj || !dc_proj || !db_scale || !dc_scale ||
      !db_bias || !dc_bias || !workspace)
    return MXB_ERR_INVALID_ARGUMENT;
  if (!aligned16(b_proj) || !aligned16(c_proj) || !aligned16(db) || !aligned16(dc) || !aligned16(db_proj) ||
      !aligned16(dc_proj) || !aligned16(b_scale) || !aligned16(c_scale) || !aligned16(workspace))
    return MXB_ERR_ALIGNMENT;
  if (workspace_bytes < mamba3_block_workspace_bytes(d)) return MXB_ERR_WORKSPACE;
  return mamba3_block_bc(d, eps, b_proj, c_proj, b_scale, c_scale, nullptr, nullptr, nullptr, nullptr, db, dc, db_proj,
                         dc_proj, db_scale, dc_scale, db_bias, dc_bias, workspace, static_cast<cudaStream_t>(stream));
}
mxb_status mxb_mamba3_block_post_fwd(const mxb_mamba3_desc* d, float eps, const void* y, const void* z,
                                     const float* post_norm, void* out, void* stream) {
  mxb_status s = check_m3_block_desc(d);
  if (s != MXB_OK) return s;
  if (!y || !z || !post_norm || !out) return MXB_ERR_INVALID_ARGUMENT;
  if (!aligned16(y) || !aligned16(z) || !aligned16(out) || !aligned16(post_norm)) return MXB_ERR_ALIGNMENT;
  return mamba3_block_post(d, eps, y, z, post_norm, out, nullptr, nullptr, nullptr, nullptr, nullptr,
                           static_cast<cudaStream_t>(stream));
}
mxb_status mxb_mamba3_block_post_bwd(const mxb_mamba3_desc* d, float eps, const void* y, const void* z,
                                     const float* post_norm, const void* dout, void* dy, void* dz, float* dpost_norm,
                                     void* workspace, size_t workspace_bytes, void* stream) {
  mxb_status s = check_m3_block_desc(d);
  if (s != MXB_OK) return s;
  if (!y || !z || !post_norm || !dout || !dy || !dz || !dpost_norm || !workspace) return MXB_ERR_INVALID_ARGUMENT;
  if (!aligned16(y) || !aligned16(z) || !aligned16(dout) || !aligned16(dy) || !aligned16(dz) || !aligned16(post_norm) ||
      !aligned16(workspace))
    return MXB_ERR_ALIGNMENT;
  if (workspace_bytes < mamba3_block_workspace_bytes(d)) return MXB_ERR_WORKSPACE;
  return mamba3_block_post(d, eps, y, z, post_norm, nullptr, dout, dy, dz, dpost_norm, workspace,
                           static_cast<cudaStream_t>(stream));
}

// ---------------------------------------------------------------- host ctx
struct mxb_host_ctx {
  int device;
  char* arena;
  size_t arena_bytes;
  cudaStream_t stream;           // kernels of the even slices
  cudaStream_t stream2;          // kernels of the odd slices (small slices do not fill the GPU: let two overlap)
  cudaStream_t s_h2d, s_d2h;     // copy engines, one per direction
  cudaEvent_t h2d_done[2], comp_done[2], d2h_done[2];
  cudaEvent_t do_done[2], fwd_done[2];  // dO uploaded / forward finished: the forward need not wait for dO, nor out for the backward
  cudaEvent_t bg_up;                    // beta and gate of the whole batch uploaded
};

#define MXB_CUDA_TRY(expr)                          \
  do {                                              \
    cudaError_t e__ = (expr);                       \
    if (e__ != cudaSuccess) {                       \
      g_last_cuda_error = (int)e__;                 \
      return MXB_ERR_CUDA;                          \
    }                                               \
  } while (0)

mxb_status mxb_host_ctx_create(int device, size_t arena_bytes, mxb_host_ctx** out) {
  if (!out || arena_bytes == 0) return MXB_ERR_INVALID_ARGUMENT;
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess || device < 0 || device >= n) return MXB_ERR_NO_DEVICE;
  MXB_CUDA_TRY(cudaSetDevice(device));
  mxb_host_ctx* c = new (std::nothrow) mxb_host_ctx{};
  if (!c) return MXB_ERR_INVALID_ARGUMENT;
  c->device = device;
  c->arena_bytes = arena_bytes;
  cudaError_t e = cudaMalloc(reinterpret_cast<void**>(&c->arena), arena_bytes);
  if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking);
  if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&c->stream2, cudaStreamNonBlocking);
  if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&c->s_h2d, cudaStreamNonBlocking);
  if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&c->s_d2h, cudaStreamNonBlocking);
  for (int i = 0; i < 2 && e == cudaSuccess; ++i) {
    e = cudaEventCreateWithFlags(&c->h2d_done[i], cudaEventDisableTiming);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&c->comp_done[i], cudaEventDisableTiming);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&c->d2h_done[i], cudaEventDisableTiming);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&c->do_done[i], cudaEventDisableTiming);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&c->fwd_done[i], cudaEventDisableTiming);
  }
  if (e == cudaSuccess) e = cudaEventCreateWithFlags(&c->bg_up, cudaEventDisableTiming);
  if (e != cudaSuccess) {
    g_last_cuda_error = (int)e;
    mxb_host_ctx_destroy(c);
    return MXB_ERR_CUDA;
  }
  *out = c;
  return MXB_OK;
}

void mxb_host_ctx_destroy(mxb_host_ctx* c) {
  if (!c) return;
  cudaSetDevice(c->device);
  cudaDeviceSynchronize();
  for (int i = 0; i < 2; ++i) {
    if (c->h2d_done[i]) cudaEventDestroy(c->h2d_done[i]);
    if (c->comp_done[i]) cudaEventDestroy(c->comp_done[i]);
    if (c->d2h_done[i]) cudaEventDestroy(c->d2h_done[i]);
    if (c->do_done[i]) cudaEventDestroy(c->do_done[i]);
    if (c->fwd_done[i]) cudaEventDestroy(c->fwd_done[i]);
  }
  if (c->bg_up) cudaEventDestroy(c->bg_up);
  if (c->stream) cudaStreamDestroy(c->stream);
  if (c->stream2) cudaStreamDestroy(c->stream2);
  if (c->s_h2d) cudaStreamDestroy(c->s_h2d);
  if (c->s_d2h) cudaStreamDestroy(c->s_d2h);
  if (c->arena) cudaFree(c->arena);
  delete c;
}

// Per-head scalars of a head group: compact[r][j] = full[r][h0 + j] (gather) and back (scatter).
__global__ void __launch_bounds__(256) head_gather_kernel(const float* __restrict__ full, float* __restrict__ compact,
                                                          size_t rows, int H, int h0, int Hs) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < rows * Hs; i += (size_t)gridDim.x * blockDim.x)
    compact[i] = full[(i / Hs) * H + h0 + (i % Hs)];
}
__global__ void __launch_bounds__(256) head_scatter_kernel(const float* __restrict__ compact, float* __restrict__ full,
                                                           size_t rows, int H, int h0, int Hs) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < rows * Hs; i += (size_t)gridDim.x * blockDim.x)
    full[(i / Hs) * H + h0 + (i % Hs)] = compact[i];
}

// The batch is cut into slices; slice i+1 is uploaded and slice i-1 downloaded while slice i computes (two device
// slots per tensor, two copy streams, two kernel streams, events between them).  A slice is one sequence, or - when
// the batch has few sequences - a group of heads of one sequence, moved by strided copies: the first upload and the
// last download are the part of the traffic nothing overlaps, so slices are kept to about a sixteenth of the batch.
// beta and gate (and their gradients) are small: they cross once for the whole batch.
static mxb_status host_gdn_pipeline(mxb_host_ctx* c, const mxb_gdn_desc* d, const void* q, const void* k,
                                    const void* v, const float* beta, const float* gate, void* out,
                                    const void* d_out, void* dq, void* dk, void* dv, float* dbeta, float* dgate) {
  if (!c) return MXB_ERR_INVALID_ARGUMENT;
  mxb_status s = check_gdn_desc(d, true);
  if (s != MXB_OK) return s;
  if (!q || !k || !v || !beta || !gate || !out) return MXB_ERR_INVALID_ARGUMENT;
  const bool bwd = d_out != nullptr;
  if (bwd && (!dq || !dk || !dv || !dbeta || !dgate)) return MXB_ERR_INVALID_ARGUMENT;
  MXB_CUDA_TRY(cudaSetDevice(c->device));
  const size_t es = d->io_dtype == MXB_F32 ? 4 : 2;
  // sequences per slice (MXB_HOST_SLICE_SEQS overrides the default of 1) and head groups per sequence
  // (MXB_HOST_HEAD_SPLIT overrides; by default doubled until there are 16 slices, while a group's rows stay >= 1 KB)
  int per = 1, nsplit = 1;
  bool per_set = false;
  if (const char* ev = std::getenv("MXB_HOST_SLICE_SEQS")) { per = std::atoi(ev); per_set = true; }
  if (per < 1) per = 1;
  if (per > d->B) per = d->B;
  if (const char* ev = std::getenv("MXB_HOST_HEAD_SPLIT")) {
    nsplit = std::atoi(ev);
    if (nsplit < 1 || d->H % nsplit) nsplit = 1;
  } else if (!per_set) {
    const size_t dmin = (size_t)(d->Dk < d->Dv ? d->Dk : d->Dv) * es;
    while (d->B * nsplit < 16 && d->H % (2 * nsplit) == 0 && (size_t)(d->H / (2 * nsplit)) * dmin >= 1024) nsplit *= 2;
  }
  if (nsplit > 1) per = 1;
  const int Hs = d->H / nsplit;  // heads of the largest slice
  struct Slice { int b0, nb, h0, hs; };
  std::vector<Slice> slices;
  if (nsplit > 1) {
    // equal head groups: cutting the last group finer (to shorten the download that overlaps nothing) was slower,
    // every extra slice pays the latency of the sequential state passes once more
    for (int b0 = 0; b0 < d->B; ++b0)
      for (int g = 0; g < nsplit; ++g) slices.push_back({b0, 1, g * Hs, Hs});
  } else {
    for (int b0 = 0; b0 < d->B; b0 += per) slices.push_back({b0, b0 + per <= d->B ? per : d->B - b0, 0, d->H});
  }
  const int nslices = (int)slices.size();
  // per-sequence element counts of a slice's tensors
  const size_t sk = (size_t)d->T * Hs * d->Dk, sv = (size_t)d->T * Hs * d->Dv, ss = (size_t)d->T * Hs;
  mxb_gdn_desc d1 = *d;
  d1.B = per;
  d1.H = Hs;
  mxb_gdn_desc df = d1, db = d1;
  // The slices' kernels stage their operands with per-thread copies where they have such a variant: this call is
  // bound by the two PCIe copy streams, which ran slower beside kernels fed by the tensor-copy engine.
  df.flags |= MXB_GDN_NO_TMA;
  db.flags |= MXB_GDN_NO_TMA;
  if (bwd) {  // keep the forward intermediates in the arena for the backward that follows
    df.flags |= MXB_GDN_SAVE_FOR_BWD;
    db.flags |= MXB_GDN_BWD_USE_SAVED;
  }
  const size_t ws_f = mxb_gdn_fwd_workspace_bytes(&df), ws_b = bwd ? mxb_gdn_bwd_workspace_bytes(&db) : 0;
  const size_t ws_bytes = ws_f > ws_b ? ws_f : ws_b;
  const size_t nk = sk * per, nv = sv * per, ns = ss * per;  // slot capacities
  const size_t nfull = (size_t)d->B * d->T * d->H;           // beta, gate and their gradients, whole batch
  Carver cv(c->arena);
  char *i_q[2], *i_k[2], *i_v[2], *i_do[2], *o_out[2], *o_q[2], *o_k[2], *o_v[2];
  float *i_b[2], *i_g[2], *o_b[2], *o_g[2];
  float* f_beta = cv.take<float>(nfull);
  float* f_gate = cv.take<float>(nfull);
  float* f_dbeta = bwd ? cv.take<float>(nfull) : nullptr;
  float* f_dgate = bwd ? cv.take<float>(nfull) : nullptr;
  for (int sl = 0; sl < 2; ++sl) {
    i_q[sl] = cv.take<char>(nk * es); i_k[sl] = cv.take<char>(nk * es); i_v[sl] = cv.take<char>(nv * es);
    o_out[sl] = cv.take<char>(nv * es);
    i_b[sl] = i_g[sl] = o_b[sl] = o_g[sl] = nullptr;
    if (nsplit > 1) { i_b[sl] = cv.take<float>(ns); i_g[sl] = cv.take<float>(ns); }
    i_do[sl] = o_q[sl] = o_k[sl] = o_v[sl] = nullptr;
    if (bwd) {
      i_do[sl] = cv.take<char>(nv * es);
      o_q[sl] = cv.take<char>(nk * es); o_k[sl] = cv.take<char>(nk * es); o_v[sl] = cv.take<char>(nv * es);
      if (nsplit > 1) { o_b[sl] = cv.take<float>(ns); o_g[sl] = cv.take<float>(ns); }
    }
  }
  char* wss[2] = {cv.take<char>(ws_bytes), cv.take<char>(ws_bytes)};  // one workspace per slot
  if (cv.bytes() > c->arena_bytes) return MXB_ERR_WORKSPACE;
  auto hp = [](const void* base, size_t off) { return static_cast<const char*>(base) + off; };
  auto hpw = [](void* base, size_t off) { return static_cast<char*>(base) + off; };
  const cudaMemcpyKind H2D = cudaMemcpyHostToDevice, D2H = cudaMemcpyDeviceToHost;
  // a [rows][Hs][D] slice of a [.][H][D] tensor: one contiguous block, or rows of Hs*D elements at a pitch of H*D
  auto up = [&](char* dst, const void* src, size_t off_bytes, size_t bytes, int D, int hs) -> cudaError_t {
    if (nsplit == 1) return cudaMemcpyAsync(dst, hp(src, off_bytes), bytes, H2D, c->s_h2d);
    const size_t w = (size_t)hs * D * es;
    return cudaMemcpy2DAsync(dst, w, hp(src, off_bytes), (size_t)d->H * D * es, w, (size_t)d->T, H2D, c->s_h2d);
  };
  auto down = [&](void* dst, size_t off_bytes, const char* src, size_t bytes, int D, int hs) -> cudaError_t {
    if (nsplit == 1) return cudaMemcpyAsync(hpw(dst, off_bytes), src, bytes, D2H, c->s_d2h);
    const size_t w = (size_t)hs * D * es;
    return cudaMemcpy2DAsync(hpw(dst, off_bytes), (size_t)d->H * D * es, src, w, w, (size_t)d->T, D2H, c->s_d2h);
  };
  MXB_CUDA_TRY(cudaMemcpyAsync(f_beta, beta, nfull * 4, H2D, c->s_h2d));
  MXB_CUDA_TRY(cudaMemcpyAsync(f_gate, gate, nfull * 4, H2D, c->s_h2d));
  MXB_CUDA_TRY(cudaEventRecord(c->bg_up, c->s_h2d));
  for (int bi = 0; bi < nslices; ++bi) {
    const int sl = bi & 1;
    const int b0 = slices[bi].b0, nb = slices[bi].nb, h0 = slices[bi].h0, hs = slices[bi].hs;
    const size_t ck = sk * nb * es, cvb = sv * nb * es;   // bytes of this slice (contiguous slices only)
    // element offsets of the slice's first row in the full tensors
    const size_t ok_ = ((size_t)b0 * d->T * d->H + h0) * d->Dk * es, ov_ = ((size_t)b0 * d->T * d->H + h0) * d->Dv * es;
    const size_t os_ = (size_t)b0 * d->T * d->H;
    df.B = db.B = nb;
    df.H = db.H = hs;
    if (bi >= 2) MXB_CUDA_TRY(cudaStreamWaitEvent(c->s_h2d, c->comp_done[sl], 0));  // slot inputs consumed
    MXB_CUDA_TRY(up(i_q[sl], q, ok_, ck, d->Dk, hs));
    MXB_CUDA_TRY(up(i_k[sl], k, ok_, ck, d->Dk, hs));
    MXB_CUDA_TRY(up(i_v[sl], v, ov_, cvb, d->Dv, hs));
    MXB_CUDA_TRY(cudaEventRecord(c->h2d_done[sl], c->s_h2d));
    if (bwd) {
      MXB_CUDA_TRY(up(i_do[sl], d_out, ov_, cvb, d->Dv, hs));
      MXB_CUDA_TRY(cudaEventRecord(c->do_done[sl], c->s_h2d));
    }
    cudaStream_t kst = sl ? c->stream2 : c->stream;
    char* ws = wss[sl];
    MXB_CUDA_TRY(cudaStreamWaitEvent(kst, c->h2d_done[sl], 0));
    if (bi < 2) MXB_CUDA_TRY(cudaStreamWaitEvent(kst, c->bg_up, 0));
    if (bi >= 2) MXB_CUDA_TRY(cudaStreamWaitEvent(kst, c->d2h_done[sl], 0));  // slot outputs drained
    const float *sb = f_beta + os_, *sg = f_gate + os_;
    float *sdb = bwd ? f_dbeta + os_ : nullptr, *sdg = bwd ? f_dgate + os_ : nullptr;
    const size_t rows = (size_t)nb * d->T;
    const int gblocks = (int)((rows * hs + 255) / 256 < 592 ? (rows * hs + 255) / 256 : 592);
    if (nsplit > 1) {
      MXB_LAUNCH("head_gather_kernel", kst, (head_gather_kernel<<<gblocks, 256, 0, kst>>>(sb, i_b[sl], rows, d->H, h0, hs)));
      MXB_LAUNCH("head_gather_kernel", kst, (head_gather_kernel<<<gblocks, 256, 0, kst>>>(sg, i_g[sl], rows, d->H, h0, hs)));
      sb = i_b[sl]; sg = i_g[sl];
      sdb = o_b[sl]; sdg = o_g[sl];
    }
    s = mxb_gdn_fwd(&df, i_q[sl], i_k[sl], i_v[sl], sb, sg, nullptr, o_out[sl], nullptr, ws, ws_bytes, kst);
    if (s != MXB_OK) return s;
    MXB_CUDA_TRY(cudaEventRecord(c->fwd_done[sl], kst));
    if (bwd) {
      MXB_CUDA_TRY(cudaStreamWaitEvent(kst, c->do_done[sl], 0));
      s = mxb_gdn_bwd(&db, i_q[sl], i_k[sl], i_v[sl], sb, sg, nullptr, i_do[sl], nullptr, o_q[sl], o_k[sl], o_v[sl], sdb,
                      sdg, nullptr, ws, ws_bytes, kst);
      if (s != MXB_OK) return s;
      if (nsplit > 1) {
        MXB_LAUNCH("head_scatter_kernel", kst,
                   (head_scatter_kernel<<<gblocks, 256, 0, kst>>>(o_b[sl], f_dbeta + os_, rows, d->H, h0, hs)));
        MXB_LAUNCH("head_scatter_kernel", kst,
                   (head_scatter_kernel<<<gblocks, 256, 0, kst>>>(o_g[sl], f_dgate + os_, rows, d->H, h0, hs)));
      }
    }
    MXB_CUDA_TRY(cudaEventRecord(c->comp_done[sl], kst));
    MXB_CUDA_TRY(cudaStreamWaitEvent(c->s_d2h, c->fwd_done[sl], 0));
    MXB_CUDA_TRY(down(out, ov_, o_out[sl], cvb, d->Dv, hs));
    if (bwd) {
      MXB_CUDA_TRY(cudaStreamWaitEvent(c->s_d2h, c->comp_done[sl], 0));
      MXB_CUDA_TRY(down(dq, ok_, o_q[sl], ck, d->Dk, hs));
      MXB_CUDA_TRY(down(dk, ok_, o_k[sl], ck, d->Dk, hs));
      MXB_CUDA_TRY(down(dv, ov_, o_v[sl], cvb, d->Dv, hs));
    }
    MXB_CUDA_TRY(cudaEventRecord(c->d2h_done[sl], c->s_d2h));
  }
  if (bwd) {  // the per-head gradients of the whole batch, once every slice has computed
    MXB_CUDA_TRY(cudaStreamWaitEvent(c->s_d2h, c->comp_done[0], 0));
    if (nslices > 1) MXB_CUDA_TRY(cudaStreamWaitEvent(c->s_d2h, c->comp_done[1], 0));
    MXB_CUDA_TRY(cudaMemcpyAsync(dbeta, f_dbeta, nfull * 4, D2H, c->s_d2h));
    MXB_CUDA_TRY(cudaMemcpyAsync(dgate, f_dgate, nfull * 4, D2H, c->s_d2h));
  }
  MXB_CUDA_TRY(cudaStreamSynchronize(c->s_d2h));
  MXB_CUDA_TRY(cudaStreamSynchronize(c->stream));
  MXB_CUDA_TRY(cudaStreamSynchronize(c->stream2));
  return MXB_OK;
}

mxb_status mxb_host_gdn(mxb_host_ctx* c, const mxb_gdn_desc* d, const void* q, const void* k,
                        const void* v, const float* beta, const float* gate, void* out,
                        const void* d_out, void* dq, void* dk, void* dv, float* dbeta, float* dgate) {
  const mxb_status s = host_gdn_pipeline(c, d, q, k, v, beta, gate, out, d_out, dq, dk, dv, dbeta, dgate);
  if (s != MXB_OK && c) {
    // The call is blocking also when it fails: copies of earlier slices may still be reading or writing the
    // caller's host buffers and the arena slots, so all four streams are drained (errors ignored) before returning.
    const int keep = g_last_cuda_error;
    cudaStreamSynchronize(c->s_h2d);
    cudaStreamSynchronize(c->s_d2h);
    cudaStreamSynchronize(c->stream);
    cudaStreamSynchronize(c->stream2);
    g_last_cuda_error = keep;
  }
  return s;
}

}  // extern "C"
