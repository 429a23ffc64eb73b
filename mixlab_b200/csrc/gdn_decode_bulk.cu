// Gated delta rule - recurrent decode step, bulk-copy pipelined variant.
//
// Same update as gdn_decode.cu (loop body of gated_delta_scan_naive, gpu/ir.cpp:2334-2345),
// for states whose per-(sequence, head) tile [Dk, Dv] fp32 is one contiguous block of at
// most 64 KB (Dk = Dv = 128 in the benchmark).  Persistent CTAs, one per SM, stream the
// tiles through a three-stage shared-memory ring:
//     cp.async.bulk global -> shared (mbarrier complete_tx)   tile n+2
//     update in place in shared memory                        tile n
//     cp.async.bulk shared -> global (bulk group)             tile n-1 draining
// so the copy engine always has a load and a store in flight while the SM computes.  Every
// wait on an mbarrier is bounded; a wait that gives up raises a device flag and the CTA
// stops issuing work (no trap).
#include "common.cuh"
#include "tcgen05.cuh"

namespace mxb {

static __device__ int g_decode_bulk_status = 0;

namespace {
constexpr int kStages = 3;
constexpr int kMaxTileBytes = 65536;

__device__ __forceinline__ void bulk_load(uint32_t dst_smem, const void* src, uint32_t bytes, uint64_t* mbar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst_smem),
               "l"(src), "r"(bytes), "r"(tc::smem_u32(mbar))
               : "memory");
}
__device__ __forceinline__ void bulk_store(void* dst, uint32_t src_smem, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(src_smem), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void bulk_wait_all() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}
}  // namespace

// Dk <= 128 rows, Dv == 128 columns (one warp reads a whole 512-byte row), 256 threads.
template <typename IO>
__global__ void __launch_bounds__(256, 1)
gdn_decode_bulk_kernel(float* __restrict__ state, const IO* __restrict__ q, const IO* __restrict__ k,
                       const IO* __restrict__ v, const float* __restrict__ beta, const float* __restrict__ gate,
                       IO* __restrict__ out, int ntiles, int Dk, int gate_is_log) {
  extern __shared__ uint8_t raw[];
  uint8_t* sm = raw + ((128u - (tc::smem_u32(raw) & 127u)) & 127u);
  float* tiles = reinterpret_cast<float*>(sm);  // [kStages][Dk*128]
  float* s_k = tiles + kStages * (kMaxTileBytes / 4);   // [2][128]
  float* s_q = s_k + 256;                                // [2][128]
  float* s_red = s_q + 256;                              // [2][8][128]
  uint64_t* full = reinterpret_cast<uint64_t*>(s_red + 2048);

  constexpr int Dv = 128;
  const int tid = threadIdx.x, cg = tid & 31, rg = tid >> 5;
  const uint32_t tile_bytes = (uint32_t)Dk * Dv * 4u;
  const int first = blockIdx.x, stride = gridDim.x;
  const int my_tiles = first < ntiles ? (ntiles - first + stride - 1) / stride : 0;

  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) tc::mbar_init(&full[s], 1);
    tc::mbar_fence_init();
  }
  __syncthreads();
  if (tid == 0) {
    for (int it = 0; it < 2 && it < my_tiles; ++it) {
      const size_t t = (size_t)first + (size_t)it * stride;
      tc::mbar_expect_tx(&full[it], tile_bytes);
      bulk_load(tc::smem_u32(tiles + it * (kMaxTileBytes / 4)), state + t * Dk * Dv, tile_bytes, &full[it]);
    }
  }
  // per-tile small inputs, prefetched one tile ahead into registers
  float pre_kq = 0.f, pre_beta = 0.f, pre_gate = 0.f;
  float4 pre_v = make_float4(0.f, 0.f, 0.f, 0.f);
  auto prefetch = [&](int it) {
    if (it < my_tiles) {
      const size_t t = (size_t)first + (size_t)it * stride;
      const int r = tid & 127;
      pre_kq = r < Dk ? to_f32((tid < 128 ? k : q)[t * Dk + r]) : 0.f;
      const IO* vp = v + t * Dv + 4 * cg;
      pre_v = make_float4(to_f32(vp[0]), to_f32(vp[1]), to_f32(vp[2]), to_f32(vp[3]));
      pre_beta = beta[t];
      pre_gate = gate[t];
    }
  };
  prefetch(0);
  bool ok = true;

  for (int it = 0; it < my_tiles; ++it) {
    const int s = it % kStages, par = (it / kStages) & 1, buf = it & 1;
    const size_t t = (size_t)first + (size_t)it * stride;
    float* S = tiles + s * (kMaxTileBytes / 4);
    // publish this tile's k, q (prefetched last iteration) and fetch the next tile's
    (tid < 128 ? s_k : s_q)[buf * 128 + (tid & 127)] = pre_kq;
    const float4 vv = pre_v;
    const float bt = pre_beta;
    const float a = gate_is_log ? expf(pre_gate) : pre_gate;
    prefetch(it + 1);
    if (ok) ok = tc::mbar_wait(&full[s], par);
    // k, q visible; tile landed for everybody
    ok = __syncthreads_and(ok);  // the barrier also makes the verdict of the bounded waits uniform, so that all
    if (!ok) break;              // threads leave the loop together
    const float* sk = s_k + buf * 128;
    const float* sq = s_q + buf * 128;
    float4 pk = make_float4(0.f, 0.f, 0.f, 0.f), pq = pk;
    if (ok) {
      for (int row = rg; row < Dk; row += 8) {
        const float4 x = *reinterpret_cast<const float4*>(S + row * Dv + 4 * cg);
        const float kr = sk[row], qr = sq[row];
        pk.x = fmaf(kr, x.x, pk.x); pk.y = fmaf(kr, x.y, pk.y); pk.z = fmaf(kr, x.z, pk.z); pk.w = fmaf(kr, x.w, pk.w);
        pq.x = fmaf(qr, x.x, pq.x); pq.y = fmaf(qr, x.y, pq.y); pq.z = fmaf(qr, x.z, pq.z); pq.w = fmaf(qr, x.w, pq.w);
      }
    }
    *reinterpret_cast<float4*>(&s_red[(0 * 8 + rg) * 128 + 4 * cg]) = pk;
    *reinterpret_cast<float4*>(&s_red[(1 * 8 + rg) * 128 + 4 * cg]) = pq;
    float qk = 0.f;
    for (int i = cg; i < Dk; i += 32) qk = fmaf(sq[i], sk[i], qk);
    qk = warp_sum(qk);
    __syncthreads();
    pk = make_float4(0.f, 0.f, 0.f, 0.f); pq = pk;
#pragma unroll
    for (int w = 0; w < 8; ++w) {
      const float4 x = *reinterpret_cast<const float4*>(&s_red[(0 * 8 + w) * 128 + 4 * cg]);
      const float4 y = *reinterpret_cast<const float4*>(&s_red[(1 * 8 + w) * 128 + 4 * cg]);
      pk.x += x.x; pk.y += x.y; pk.z += x.z; pk.w += x.w;
      pq.x += y.x; pq.y += y.y; pq.z += y.z; pq.w += y.w;
    }
    float4 e;
    e.x = bt * (vv.x - a * pk.x); e.y = bt * (vv.y - a * pk.y);
    e.z = bt * (vv.z - a * pk.z); e.w = bt * (vv.w - a * pk.w);
    if (ok) {
      for (int row = rg; row < Dk; row += 8) {
        float4* px = reinterpret_cast<float4*>(S + row * Dv + 4 * cg);
        const float4 x = *px;
        const float kr = sk[row];
        *px = make_float4(fmaf(kr, e.x, a * x.x), fmaf(kr, e.y, a * x.y), fmaf(kr, e.z, a * x.z), fmaf(kr, e.w, a * x.w));
      }
      if (rg == 0) {
        IO* op = out + t * Dv + 4 * cg;
        op[0] = from_f32<IO>(fmaf(qk, e.x, a * pq.x));
        op[1] = from_f32<IO>(fmaf(qk, e.y, a * pq.y));
        op[2] = from_f32<IO>(fmaf(qk, e.z, a * pq.z));
        op[3] = from_f32<IO>(fmaf(qk, e.w, a * pq.w));
      }
    }
    tc::fence_async_smem();  // updated tile -> visible to the bulk store
    __syncthreads();
    if (tid == 0 && ok) {
      bulk_store(state + t * Dk * Dv, tc::smem_u32(S), tile_bytes);
      bulk_commit();
      if (it + 2 < my_tiles) {
        bulk_wait_read<1>();  // the store issued one tile ago has drained its stage
        const int s2 = (it + 2) % kStages;
        const size_t t2 = (size_t)first + (size_t)(it + 2) * stride;
        tc::mbar_expect_tx(&full[s2], tile_bytes);
        bulk_load(tc::smem_u32(tiles + s2 * (kMaxTileBytes / 4)), state + t2 * Dk * Dv, tile_bytes, &full[s2]);
      }
    }
  }
  if (tid == 0) {
    bulk_wait_all<0>();
    if (!ok) atomicExch(&g_decode_bulk_status, 1);
  }
}

constexpr int kDecodeBulkSmem = kStages * kMaxTileBytes + (256 + 256 + 2048) * 4 + 64 + 128;

bool gdn_decode_bulk_supported(const mxb_gdn_desc* d) {
  return d->Dv == 128 && d->Dk <= 128 && d->Dk % 4 == 0 && d->Dk >= 8;
}

template <typename IO>
static mxb_status launch_bulk(const mxb_gdn_desc* d, float* state, const void* q, const void* k, const void* v,
                              const float* beta, const float* gate, void* out, cudaStream_t st) {
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 148;
  }
  cudaError_t e = cudaFuncSetAttribute(gdn_decode_bulk_kernel<IO>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       kDecodeBulkSmem);
  if (e != cudaSuccess) { set_last_cuda_error((int)e); return MXB_ERR_CUDA; }
  const int ntiles = d->B * d->H;
  const int grid = ntiles < sms ? ntiles : sms;
  MXB_LAUNCH("gdn_decode_bulk_kernel", st,
             (gdn_decode_bulk_kernel<IO><<<grid, 256, kDecodeBulkSmem, st>>>(
                 state, static_cast<const IO*>(q), static_cast<const IO*>(k), static_cast<const IO*>(v), beta, gate,
                 static_cast<IO*>(out), ntiles, d->Dk, d->gate_is_log)));
  return check_launch("gdn_decode_bulk_kernel");
}

mxb_status gdn_decode_bulk_dispatch(const mxb_gdn_desc* d, float* state, const void* q, const void* k, const void* v,
                                    const float* beta, const float* gate, void* out, cudaStream_t st) {
  if (d->io_dtype == MXB_F32) return launch_bulk<float>(d, state, q, k, v, beta, gate, out, st);
  return launch_bulk<__nv_bfloat16>(d, state, q, k, v, beta, gate, out, st);
}

int gdn_decode_bulk_status() {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_decode_bulk_status, sizeof(int)) != cudaSuccess) return -1;
  return v;
}

}  // namespace mxb
