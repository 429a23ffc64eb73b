/*
 * mixlab_b200 - C ABI of the B200 (sm_100a) sequence-mixing primitives.
 *
 * Drop-in boundary for the operators mixlab's IR lowers `gated_deltanet` and
 * `mamba3-canonical` blocks to.  Plain C: pointers, sizes, a stream handle.
 * No exceptions cross this boundary and the compute entry points never
 * allocate, free or synchronise: every buffer (inputs, outputs, workspace)
 * is a caller-owned DEVICE pointer and work is enqueued on the caller's
 * stream.  The `mxb_host_*` entry points are the exception by design: they
 * take HOST buffers like the reference bridge does (mlx_tensor_input,
 * gpu/mlx_bridge.h:92-99) and own a device arena created up front.
 *
 * Reference interfaces replaced (paths inside the mixlab checkout):
 *   OP_GATED_DELTA_SCAN        arch/ir.go:586-603, gpu/ir.cpp:4633-4654
 *     gated_delta_scan_naive   gpu/ir.cpp:2314-2350
 *     gated_delta_scan_chunked gpu/ir.cpp:2352-2550
 *     solve_strictly_lower_cuda_primitive  gpu/gated_delta_cuda_primitive.h:8-11
 *   OP_MAMBA3_SELECTIVE_SCAN   arch/ir.go:528-553, gpu/ir.cpp:4837-4853
 *     mamba3_selective_scan_cuda_forward / _vjp  gpu/mamba3_cuda_primitive.h:12-33
 *
 * Tensor layouts are the reference operator's (row-major, innermost last):
 *   q,k [B,T,H,Dk]  v,out [B,T,H,Dv]  beta,gate [B,T,H]  state [B,H,Dk,Dv]
 *   x,dt,lambda,y [B,T,D]  theta [B,T,D,N/2]  a_log [D,N]  b,c [B,T,G,N]
 */
#ifndef MIXLAB_B200_H
#define MIXLAB_B200_H

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define MXB_API __attribute__((visibility("default")))
#else
#define MXB_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

typedef int32_t mxb_status;
enum {
  MXB_OK = 0,
  MXB_ERR_INVALID_ARGUMENT = -1, /* null pointer, non-positive extent, bad enum */
  MXB_ERR_UNSUPPORTED = -2,      /* shape / dtype combination no kernel covers */
  MXB_ERR_WORKSPACE = -3,        /* workspace missing or smaller than *_workspace_bytes */
  MXB_ERR_CUDA = -4,             /* a CUDA runtime call failed (see mxb_last_cuda_error) */
  MXB_ERR_ALIGNMENT = -5,        /* pointer not aligned as the entry point requires */
  MXB_ERR_NO_DEVICE = -6         /* no sm_100 device; there is no CPU fallback */
};

/* Element types.  1 = float32 matches the reference's mlx_tensor_input.dtype
 * (gpu/mlx_bridge.h:94); bf16 is new (the reference computes this path in
 * fp32 only, gpu/ir.cpp:2372-2376). */
enum { MXB_F32 = 1, MXB_BF16 = 2 };

/* Operator codes, identical to the reference IR (arch/ir.go:53,56). */
enum { MXB_OP_GATED_DELTA_SCAN = 60, MXB_OP_MAMBA3_SELECTIVE_SCAN = 63 };

MXB_API const char* mxb_status_string(mxb_status s);
MXB_API int mxb_version(void);
/* cudaError_t (as int) of the most recent failing CUDA call on this thread. */
MXB_API int mxb_last_cuda_error(void);
/* Number of kernels this library has launched in this process (all threads). */
MXB_API uint64_t mxb_launch_count(void);
/* Per-launch tracing with CUDA events on the launching stream (the reference has
 * only compiled-out section timers for this path, gpu/ir.cpp:2426-2431).
 * enable(1) clears earlier records and starts recording; enable(0) stops.
 * summary() waits for the recorded events and writes one line per kernel,
 * "<name> <launches> <total_ms>\n", returning the untruncated length. */
MXB_API void mxb_trace_enable(int on);
MXB_API size_t mxb_trace_summary(char* buf, size_t capacity);

/* ------------------------------------------------------------------------
 * Gated delta rule.  IntParams of OP_GATED_DELTA_SCAN are [B,T,H,Dk,Dv,chunk]
 * (arch/ir.go:600-602); chunk <= 1 selects the token-by-token recurrence
 * (gpu/ir.cpp:4648-4652), chunk >= 2 the chunked WY/UT form.  The result does not
 * depend on the chunk size; sizes above 64 (which the reference accepts,
 * arch/blocks_gated_deltanet.go:11-17) are computed with chunks of 64.
 *
 * Numeric guards: the chunked form floors the gate at 1e-30 and clamps every decay
 * exponent to [-80, 0] (gpu/ir.cpp:35-37, :2396, :893-905); the recurrence applies
 * neither (gpu/ir.cpp:2334).  mxb_gdn_fwd follows the reference in both forms.
 * mxb_gdn_bwd always differentiates the chunked form (chunks of 64), also for
 * chunk <= 1: the gradient with respect to a gate below the floor is then zero,
 * where differentiating the unguarded recurrence would give a (tiny) nonzero value.
 * ---------------------------------------------------------------------- */
typedef struct {
  int32_t B, T, H, Dk, Dv, chunk;
  int32_t io_dtype;    /* MXB_F32 | MXB_BF16: q,k,v,out,d_out,dq,dk,dv.  beta, gate,
                          dbeta, dgate and every state are always float32. */
  int32_t gate_is_log; /* 0: 5th input is the multiplicative gate in (0,1] (reference
                          convention, arch/ir.go:593); 1: it is the log decay g <= 0
                          and dgate is the gradient with respect to g. */
  int32_t flags;       /* MXB_GDN_* bits */
} mxb_gdn_desc;

enum {
  MXB_GDN_FORCE_FP32_PATH = 1, /* use the full-fp32 CUDA-core kernels even where a
                                  tensor-core path exists for the shape */
  MXB_GDN_BWD_FP32_KERNELS = 2, /* tensor-core forward, but backward through the fp32
                                   CUDA-core kernels (a cross-check of the two backwards) */
  MXB_GDN_SAVE_FOR_BWD = 4,     /* forward: also keep the per-chunk states and v_new in the
                                   workspace, which must then have the BACKWARD size */
  MXB_GDN_DECODE_REGISTER_KERNEL = 16, /* decode step: use the register-resident kernel even where
                                          the bulk-copy pipelined kernel covers the shape */
  MXB_GDN_NO_TMA = 32,          /* tensor-core path: stage k, q, v of the prep kernel with cp.async instead
                                   of TMA tensor copies (a cross-check of the two staging paths) */
  MXB_GDN_F32_IO_BF16_OPERANDS = 64, /* io_dtype MXB_F32 only: round q, k, v (and d_out) to bf16, run the
                                        tensor-core kernels on the copies and widen the results back to
                                        float32.  Results then carry bf16 rounding (relative 2^-9), which the
                                        reference's float32 evaluation does not; without the flag float32
                                        tensors take the full-fp32 kernels.  Needs the larger workspace the
                                        size queries report for this flag; ignored where the tensor-core
                                        kernels do not cover the shape or MXB_GDN_FORCE_FP32_PATH is set. */
  MXB_GDN_BWD_USE_SAVED = 8     /* backward: the workspace still holds what a forward with
                                   MXB_GDN_SAVE_FOR_BWD on the same inputs left there, so the
                                   forward recompute is skipped (the reference keeps its forward
                                   intermediates alive through MLX autograd in the same way) */
};

MXB_API size_t mxb_gdn_fwd_workspace_bytes(const mxb_gdn_desc* d);
MXB_API size_t mxb_gdn_bwd_workspace_bytes(const mxb_gdn_desc* d);

/* out [B,T,H,Dv]; h0 (optional) initial state, hT (optional) final state,
 * both [B,H,Dk,Dv] fp32.  Replaces gated_delta_scan_{naive,chunked}
 * (gpu/ir.cpp:2314-2550), which start from a zero state and return only out. */
MXB_API mxb_status mxb_gdn_fwd(const mxb_gdn_desc* d, const void* q, const void* k, const void* v,
                       const float* beta, const float* gate, const float* h0, void* out,
                       float* hT, void* workspace, size_t workspace_bytes, void* stream);

/* All gradients of (out, hT) with respect to (q,k,v,beta,gate,h0).  The
 * reference obtains these by MLX autograd through gpu/ir.cpp:2352-2550 with the
 * solve VJP of gpu/gated_delta_cuda_primitive.cpp:104-132; this is a
 * hand-written backward.  d_hT, dh0 may be NULL. */
MXB_API mxb_status mxb_gdn_bwd(const mxb_gdn_desc* d, const void* q, const void* k, const void* v,
                       const float* beta, const float* gate, const float* h0,
                       const void* d_out, const float* d_hT, void* dq, void* dk, void* dv,
                       float* dbeta, float* dgate, float* dh0, void* workspace,
                       size_t workspace_bytes, void* stream);

/* Forward without a workspace argument, for hosts that cannot allocate device
 * memory: programs living inside a runtime that has reserved the whole GPU for its
 * own pool, or loops where a call into an allocator (which may block or synchronise)
 * is not acceptable.  No counterpart in the reference.  The scratch is a fixed array
 * of MXB_GDN_STATIC_SCRATCH_BYTES inside the library (present once per GPU while the
 * library is loaded); problems whose workspace (mxb_gdn_fwd_workspace_bytes with
 * flags = MXB_GDN_FORCE_FP32_PATH) is larger return MXB_ERR_WORKSPACE before anything
 * is launched.  Always runs the full-fp32 CUDA-core kernels; same arguments and
 * results as mxb_gdn_fwd with that flag.  desc.flags is ignored: in particular
 * MXB_GDN_SAVE_FOR_BWD saves nothing (the array is private to this entry point).
 * Calls no cudaMalloc/cudaFree.  All calls on a GPU share the one array: do not let
 * two of them overlap on the device.  The first call on each device looks up the
 * array's address; make that call before any stream capture begins.  The array's
 * memory is reserved when the CUDA runtime loads this library's device code on that
 * GPU (at the latest during that first call), so on a device without 16 MiB free the
 * first call returns MXB_ERR_CUDA.  The stream must belong to the device that is
 * current during the call, and the cached address does not survive cudaDeviceReset. */
#define MXB_GDN_STATIC_SCRATCH_BYTES (16u << 20)
MXB_API size_t mxb_gdn_static_scratch_bytes(void);
MXB_API mxb_status mxb_gdn_fwd_static_scratch(const mxb_gdn_desc* d, const void* q, const void* k,
                                      const void* v, const float* beta, const float* gate,
                                      const float* h0, void* out, float* hT, void* stream);

/* The tensor-core kernels bound every wait on an mbarrier; a wait that gives up
 * makes the kernel leave in an orderly way and write a nonzero code into the first
 * word of the workspace.  This BLOCKING call copies that word to *out (0 = no
 * device-side error).  Workspaces of the fp32 path never set it. */
MXB_API mxb_status mxb_gdn_device_status(const void* workspace, int32_t* out);

/* One token of the recurrence on a persistent state: the loop body of
 * gated_delta_scan_naive (gpu/ir.cpp:2334-2345).  desc.T is ignored, desc.B is
 * the number of sequences.  state [B,H,Dk,Dv] fp32 is updated in place;
 * q,k [B,H,Dk], v,out [B,H,Dv] in io_dtype; beta,gate [B,H] fp32. */
MXB_API mxb_status mxb_gdn_decode_step(const mxb_gdn_desc* d, float* state, const void* q,
                               const void* k, const void* v, const float* beta,
                               const float* gate, void* out, void* stream);

/* ------------------------------------------------------------------------
 * Element-wise stages of the gated_deltanet block on either side of the scan
 * (emitGatedDeltaNetDeltaIR, arch/blocks_gated_deltanet.go:207-343; the 4-tap
 * causal convolution is emitGatedDeltaNetShortConv1D, :345-368).  They replace
 * the chain of MatMul-free IR ops between the projections and the scan (Full /
 * Slice / Concat / Mul / Add / SiLU, RMSNorm, ScalarMul, Softplus, Exp, Sigmoid)
 * and between the scan and the output projection (RMSNorm, SiLU, Mul).  The
 * projections themselves are matrix products and stay with the caller.
 *
 * desc: B, T, H, Dk, Dv (multiples of 8, <= 128), io_dtype (q_proj .. v, o, z, y
 * and their gradients), gate_is_log (gate is produced / its gradient taken as
 * log gate, the form mxb_gdn_fwd accepts with the same bit).  chunk and flags are
 * ignored.  Convolution weights [4, C] (tap j multiplies x[t-j]), a_raw, b_raw,
 * beta, gate [B,T,H], A_log, dt_bias [H], o_norm [Dv] are float32.
 *   pre   q = RMSNorm(SiLU(conv(q_proj)), 1, 1e-6) / Dk          [B,T,H,Dk]
 *         k = RMSNorm(SiLU(conv(k_proj)), 1, 1e-6) / sqrt(Dk)    [B,T,H,Dk]
 *         v = SiLU(conv(v_proj))                                 [B,T,H,Dv]
 *         gate = exp(-softplus(a_raw + dt_bias) exp(A_log)), beta = sigmoid(b_raw)
 *   post  y = RMSNorm(o, o_norm, 1e-5) SiLU(z)                   [B,T,H*Dv]
 * The backward entry points return every gradient; sums over (batch, step) go
 * through partial rows in the workspace in a fixed order.
 * ---------------------------------------------------------------------- */
MXB_API size_t mxb_gdn_block_workspace_bytes(const mxb_gdn_desc* d);
MXB_API mxb_status mxb_gdn_block_pre_fwd(const mxb_gdn_desc* d, const void* q_proj, const void* k_proj,
                                 const void* v_proj, const float* conv_q, const float* conv_k,
                                 const float* conv_v, const float* a_raw, const float* b_raw,
                                 const float* a_log, const float* dt_bias, void* q, void* k, void* v,
                                 float* beta, float* gate, void* stream);
MXB_API mxb_status mxb_gdn_block_pre_bwd(const mxb_gdn_desc* d, const void* q_proj, const void* k_proj,
                                 const void* v_proj, const float* conv_q, const float* conv_k,
                                 const float* conv_v, const float* a_raw, const float* b_raw,
                                 const float* a_log, const float* dt_bias, const void* dq, const void* dk,
                                 const void* dv, const float* dbeta, const float* dgate, void* dq_proj,
                                 void* dk_proj, void* dv_proj, float* dconv_q, float* dconv_k,
                                 float* dconv_v, float* da_raw, float* db_raw, float* da_log,
                                 float* ddt_bias, void* workspace, size_t workspace_bytes, void* stream);
MXB_API mxb_status mxb_gdn_block_post_fwd(const mxb_gdn_desc* d, const void* o, const void* z,
                                  const float* o_norm, void* y, void* stream);
MXB_API mxb_status mxb_gdn_block_post_bwd(const mxb_gdn_desc* d, const void* o, const void* z,
                                  const float* o_norm, const void* dy, void* d_o, void* dz,
                                  float* do_norm, void* workspace, size_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------------
 * Mamba-3 exponential-trapezoidal selective scan.  IntParams of
 * OP_MAMBA3_SELECTIVE_SCAN are [B,T,D,N,G(,chunk)] (arch/ir.go:541-553).
 * ---------------------------------------------------------------------- */
typedef struct {
  int32_t B, T, D, N, G;
  int32_t nheads;   /* 0: reference per-channel layout - dt,lambda [B,T,D], theta
                       [B,T,D,N/2], a_log [D,N].  >0: head-broadcast layout - dt,
                       lambda, theta [B,T,nheads], a_log [nheads]; D % nheads == 0 and
                       every channel and state pair of a head shares the value. */
  int32_t io_dtype; /* x, b, c, y, dy, dx, db, dc.  dt, lambda, theta, a_log and
                       their gradients are always float32. */
  int32_t flags;
} mxb_mamba3_desc;

enum {
  MXB_MAMBA3_CHANNEL_KERNELS = 1,  /* head-broadcast layout: use the warp-per-channel kernels even
                                      where the CTA-per-head kernels cover the shape */
  MXB_MAMBA3_RECURRENT_KERNELS = 2,/* use the recurrent (CTA-per-head) kernels even where the chunked
                                      tensor-core kernels cover the shape */
  MXB_MAMBA3_SAVE_FOR_BWD = 4,     /* forward: mxb_mamba3_fwd_workspace_bytes returns the backward size and
                                      the chunk states and per-token scalars stay in the workspace */
  MXB_MAMBA3_NO_TMA = 16,          /* chunked kernels: stage the operand tiles with cp.async instead of
                                      the copy engine (the path taken anyway when the driver offers no
                                      tensor-map entry point).  Both stagings need x, b, c, y, dy, dx, db,
                                      dc 16-byte aligned: other pointers return MXB_ERR_ALIGNMENT */
  MXB_MAMBA3_SERIAL_WALK = 32,     /* warp-per-channel kernels: one warp walks the whole sequence of its
                                      (batch, channel) pair, also where there are too few pairs to fill the GPU */
  MXB_MAMBA3_WINDOW_PARALLEL = 64, /* warp-per-channel kernels: one warp per (batch, channel, window of 16
                                      steps) with scans over the windows in between, also where the pairs alone
                                      would fill the GPU (the window form does about twice the arithmetic; by
                                      default it is taken when 2 B D <= 148 x 64 warps).  The forward then needs
                                      the workspace mxb_mamba3_fwd_workspace_bytes reports. */
  MXB_MAMBA3_BWD_USE_SAVED = 8     /* backward: the workspace is the one a forward call with
                                      MXB_MAMBA3_SAVE_FOR_BWD just filled for the same inputs; the forward
                                      recompute is skipped.  Honoured by the chunked tensor-core kernels;
                                      the other kernel families recompute as always. */
};

MXB_API size_t mxb_mamba3_fwd_workspace_bytes(const mxb_mamba3_desc* d);
MXB_API size_t mxb_mamba3_bwd_workspace_bytes(const mxb_mamba3_desc* d);

/* Replaces mamba3_selective_scan_cuda_forward (gpu/mamba3_cuda_primitive.h:12-24). */
MXB_API mxb_status mxb_mamba3_fwd(const mxb_mamba3_desc* d, const void* x, const float* dt,
                          const float* lambda, const float* theta, const float* a_log,
                          const void* b, const void* c, void* y, void* workspace,
                          size_t workspace_bytes, void* stream);

/* Replaces mamba3_selective_scan_cuda_vjp (gpu/mamba3_cuda_primitive.h:26-33):
 * gradients in the argument order x, dt, lambda, theta, a_log, b, c. */
MXB_API mxb_status mxb_mamba3_bwd(const mxb_mamba3_desc* d, const void* x, const float* dt,
                          const float* lambda, const float* theta, const float* a_log,
                          const void* b, const void* c, const void* dy, void* dx,
                          float* ddt, float* dlambda, float* dtheta, float* da_log,
                          void* db, void* dc, void* workspace, size_t workspace_bytes,
                          void* stream);

/* ------------------------------------------------------------------------
 * Element-wise stages of the canonical Mamba-3 block on either side of the scan
 * (mamba3_canonical_block_impl / _vjp, gpu/ir.cpp:2034-2105, :2107-2288).  The
 * projections are matrix products and stay with the caller.  desc: B, T, D (the
 * inner width, multiple of 8, <= 2048), N (multiple of 8, <= 128), G, io_dtype;
 * nheads and flags are ignored.  Weights, scales and biases are float32.
 *   conv  y = causal depthwise convolution of x [B,T,D] with w [D,K], K <= 4; tap k
 *         multiplies x[t-k] (causal_depthwise_conv1d, gpu/ir.cpp:1397-1425)
 *   bc    b = RMSNorm(b_proj rows of N, b_scale [N], eps) + b_bias [G*N], same for c;
 *         b_proj, c_proj, b, c are [B,T,G*N]
 *   post  out = RMSNorm(y rows of D, post_norm [D], eps) z sigmoid(z); y, z [B,T,D]
 * Each backward entry point returns every gradient; sums over (batch, step) go
 * through partial rows in the workspace in a fixed order.
 * ---------------------------------------------------------------------- */
MXB_API size_t mxb_mamba3_block_workspace_bytes(const mxb_mamba3_desc* d);
MXB_API mxb_status mxb_mamba3_block_conv_fwd(const mxb_mamba3_desc* d, int32_t K, const void* x, const float* w,
                                     void* y, void* stream);
MXB_API mxb_status mxb_mamba3_block_conv_bwd(const mxb_mamba3_desc* d, int32_t K, const void* x, const float* w,
                                     const void* dy, void* dx, float* dw, void* workspace,
                                     size_t workspace_bytes, void* stream);
MXB_API mxb_status mxb_mamba3_block_bc_fwd(const mxb_mamba3_desc* d, float eps, const void* b_proj,
                                   const void* c_proj, const float* b_scale, const float* c_scale,
                                   const float* b_bias, const float* c_bias, void* b, void* c,
                                   void* stream);
MXB_API mxb_status mxb_mamba3_block_bc_bwd(const mxb_mamba3_desc* d, float eps, const void* b_proj,
                                   const void* c_proj, const float* b_scale, const float* c_scale,
                                   const void* db, const void* dc, void* db_proj, void* dc_proj,
                                   float* db_scale, float* dc_scale, float* db_bias, float* dc_bias,
                                   void* workspace, size_t workspace_bytes, void* stream);
MXB_API mxb_status mxb_mamba3_block_post_fwd(const mxb_mamba3_desc* d, float eps, const void* y, const void* z,
                                     const float* post_norm, void* out, void* stream);
MXB_API mxb_status mxb_mamba3_block_post_bwd(const mxb_mamba3_desc* d, float eps, const void* y, const void* z,
                                     const float* post_norm, const void* dout, void* dy, void* dz,
                                     float* dpost_norm, void* workspace, size_t workspace_bytes,
                                     void* stream);

/* ------------------------------------------------------------------------
 * Data-parallel gradient exchange: the element-wise passes on either side of the
 * per-bucket all-reduce, over flat float32 buckets on the device (the collective
 * itself is the caller's: NCCL).  They fuse what the reference does op by op per
 * weight: non-finite entries zeroed and gradients turned into numerators before
 * the sums (gpu/distributed_step.cpp:140-152); division by the global
 * denominator, non-finite count, global norm and clipping after them
 * (gpu/distributed_step.cpp:231-240, gpu/optimizer_step_guard.cpp:76-104).
 *   sanitize  x <- finite(x) ? x * scale : 0; *flag = 1 if anything was non-finite
 *             (flag is only ever set, clear it before the first bucket)
 *   finalize  x <- x * inv_denominator with non-finite results zeroed and counted;
 *             totals[0] += sum of squares, totals[1] += count (zero totals before the
 *             first bucket), totals[2] = clip scale so far: min(1, max_norm /
 *             (sqrt(totals[0]) + 1e-6)), 0 if totals[1] != 0, 1 if max_norm <= 0.
 *             partial: scratch of mxb_dp_partial_floats() floats.  Sums run in a fixed
 *             order (no floating-point atomics): same inputs, same bits.
 *   scale     x <- x * *scale_dev (a device scalar, e.g. totals + 2 after the last
 *             finalize: no host round trip between norm and clipping)
 * ---------------------------------------------------------------------- */
MXB_API size_t mxb_dp_partial_floats(void);
MXB_API mxb_status mxb_dp_sanitize(float* x, size_t n, float scale, float* flag, void* stream);
MXB_API mxb_status mxb_dp_finalize(float* x, size_t n, float inv_denominator, float max_norm,
                           float* partial, float* totals, void* stream);
/* finalize with the divisor read from device memory (the all-reduced loss denominator where the sums left it), so
 * that a bucket can be finalized as soon as its own sum has arrived, while later buckets are still in flight and
 * without a host read in between.  A zero, negative or non-finite divisor leaves the values undivided; the host
 * checks it after the step. */
MXB_API mxb_status mxb_dp_finalize_dev(float* x, size_t n, const float* denominator_dev, float max_norm,
                               float* partial, float* totals, void* stream);
MXB_API mxb_status mxb_dp_scale(float* x, size_t n, const float* scale_dev, void* stream);

/* ------------------------------------------------------------------------
 * IR op records.  The reference's Go side hands every op to the interpreter as
 * one record (mlx_ir_program_add_op, gpu/mlx_bridge.h:83-89): op type, input and
 * output names, float params, int params; the interpreter resolves the names to
 * arrays and switches on the op type (gpu/ir.cpp:4633-4654 for op 60,
 * :4837-4853 for op 63).  mxb_ir_op is that record after name resolution:
 * device pointers instead of names, everything else unchanged, so a cgo shim
 * can forward the records of these two ops as they are.  Rules taken over from
 * the interpreter: op 60 needs 5 inputs (q, k, v, beta, gate), 1 output and
 * IntParams [B,T,H,Dk,Dv(,chunk)] with a missing or non-positive chunk meaning
 * the token recurrence; op 63 needs 7 inputs (x, dt, lambda, theta, a_log,
 * B_proj, C_proj), 1 output and IntParams [B,T,D,N,G(,chunk)] (the chunk size
 * does not change the result and is ignored).  Anything else is
 * MXB_ERR_INVALID_ARGUMENT, other op types MXB_ERR_UNSUPPORTED.  The gate of op
 * 60 is the multiplicative decay (reference convention).
 * ---------------------------------------------------------------------- */
typedef struct {
  int32_t op_type;              /* MXB_OP_GATED_DELTA_SCAN | MXB_OP_MAMBA3_SELECTIVE_SCAN */
  const void* const* inputs;    /* device pointers, in the order of the record's input names */
  int32_t n_inputs;
  void* const* outputs;
  int32_t n_outputs;
  const float* float_params;    /* unused by these two ops */
  int32_t n_float_params;
  const int32_t* int_params;
  int32_t n_int_params;
  int32_t io_dtype;             /* MXB_F32 (the reference's only dtype) | MXB_BF16 */
} mxb_ir_op;

/* Kernel-selection bits for gated-delta records come from the environment variable MXB_IR_GDN_FLAGS (read once per
 * process; only MXB_GDN_F32_IO_BF16_OPERANDS, MXB_GDN_FORCE_FP32_PATH and MXB_GDN_NO_TMA are honoured): the record
 * itself is the reference's and has no field for them. */
MXB_API size_t mxb_ir_op_workspace_bytes(const mxb_ir_op* op);
MXB_API mxb_status mxb_ir_op_forward(const mxb_ir_op* op, void* workspace, size_t workspace_bytes,
                             void* stream);

/* ------------------------------------------------------------------------
 * Diagnostics (no counterpart in the reference).  One tcgen05.mma tile
 * D[128 x ncols] = A * B^T from caller-built shared-memory images (device
 * pointers, multiples of 16 bytes) and raw descriptor fields:
 *   fields[0..2] = A leading-byte-offset, stride-byte-offset, swizzle mode
 *   fields[3..5] = the same for B
 *   fields[6] = instruction descriptor, [7] = number of K steps,
 *   fields[8], [9] = byte advance of A / B per K step, [10] = ncols (N)
 * d_out receives the 128 TMEM lanes x ncols fp32 columns; *status is set to 1
 * if the completion wait gave up.  Used by the tests to pin the operand
 * layouts the production kernels rely on.
 * ---------------------------------------------------------------------- */
MXB_API mxb_status mxb_selftest_umma(const void* a_img, uint32_t a_bytes, const void* b_img,
                             uint32_t b_bytes, const uint32_t* fields, float* d_out,
                             int* status, void* stream);

/* Runs the give-up path of the bounded device-side waits on purpose, without a
 * fault: a small kernel polls a barrier that nothing arrives on poll_limit times
 * (1 .. 65536), leaves normally and writes code 9 into the status word that leads
 * `workspace` (>= 256 bytes, cleared first), where mxb_gdn_device_status reads it
 * like the status of a production kernel whose copy or MMA never completed. */
MXB_API mxb_status mxb_selftest_wait_timeout(void* workspace, size_t workspace_bytes,
                                     uint32_t poll_limit, void* stream);

/* ------------------------------------------------------------------------
 * Host-buffer evaluation, the shape of the reference bridge's
 * mlx_ir_eval_program_named_for_output / _grads_named_for_output
 * (gpu/mlx_bridge.h:163-203): caller-owned HOST tensors in, HOST tensors out,
 * one blocking call.  A context owns a device arena and a stream; it is
 * created once (the only place this library allocates device memory).
 * ---------------------------------------------------------------------- */
typedef struct mxb_host_ctx mxb_host_ctx;

MXB_API mxb_status mxb_host_ctx_create(int device, size_t arena_bytes, mxb_host_ctx** out);
MXB_API void mxb_host_ctx_destroy(mxb_host_ctx* ctx);

/* Forward (+ backward when d_out != NULL) of OP_GATED_DELTA_SCAN on host
 * buffers: H2D of the inputs, the kernels, D2H of the results, then a stream
 * synchronise.  Gradient pointers are ignored when d_out is NULL.  The batch is
 * cut into slices (a sequence, or a group of heads of a sequence moved by strided
 * copies) that are uploaded, computed and downloaded overlapped; beta, gate and
 * their gradients cross once for the whole batch.  Pinned host buffers make the
 * copies asynchronous.  The arena must hold 4 (8 with a backward) [B,T,H] float
 * arrays, two slots of every slice tensor and two slice workspaces:
 * MXB_ERR_WORKSPACE otherwise.  Environment: MXB_HOST_SLICE_SEQS (sequences per
 * slice), MXB_HOST_HEAD_SPLIT (head groups per sequence) override the slicing. */
MXB_API mxb_status mxb_host_gdn(mxb_host_ctx* ctx, const mxb_gdn_desc* d, const void* q,
                        const void* k, const void* v, const float* beta, const float* gate,
                        void* out, const void* d_out, void* dq, void* dk, void* dv,
                        float* dbeta, float* dgate);

#ifdef __cplusplus
}
#endif
#endif /* MIXLAB_B200_H */
