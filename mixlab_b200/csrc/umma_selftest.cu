// Hardware self-test of the tcgen05 plumbing: runs one D = A * B^T tile through
// tcgen05.mma from caller-provided shared-memory images and descriptor fields and
// dumps the 128 TMEM lanes.  The host side lays the operands out; this kernel only
// copies the images into shared memory, builds the descriptors and issues the MMAs.
// It lets the layout conventions used by the production kernels (K-major / MN-major,
// swizzle modes, M=64 lane mapping) be checked against a plain matrix product.
#include "common.cuh"
#include "tcgen05.cuh"

namespace mxb {

struct UmmaTestP {
  const uint8_t* a_img;
  const uint8_t* b_img;
  uint32_t a_bytes, b_bytes;
  uint32_t a_lbo, a_sbo, a_swz, b_lbo, b_sbo, b_swz;
  uint32_t idesc, ksteps, a_kstep_bytes, b_kstep_bytes, ncols;
  float* d_out;  // [128][ncols]
  int* status;   // 0 ok, 1 mbarrier wait gave up
};

__global__ void __launch_bounds__(128) umma_selftest_kernel(UmmaTestP p) {
  extern __shared__ uint8_t raw[];
  __shared__ uint64_t mbar;
  __shared__ uint32_t tmem_slot;
  const uint32_t base = (tc::smem_u32(raw) + 1023u) & ~1023u;
  uint8_t* sa = raw + (base - tc::smem_u32(raw));
  uint8_t* sb = sa + ((p.a_bytes + 1023u) & ~1023u);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  for (uint32_t i = tid * 16; i < p.a_bytes; i += 128 * 16)
    *reinterpret_cast<uint4*>(sa + i) = *reinterpret_cast<const uint4*>(p.a_img + i);
  for (uint32_t i = tid * 16; i < p.b_bytes; i += 128 * 16)
    *reinterpret_cast<uint4*>(sb + i) = *reinterpret_cast<const uint4*>(p.b_img + i);
  tc::fence_async_smem();
  uint32_t tcols = 32;
  while (tcols < p.ncols) tcols <<= 1;
  if (warp == 0) {
    tc::tmem_alloc(&tmem_slot, tcols);
    tc::tmem_relinquish();
  }
  if (tid == 0) {
    tc::mbar_init(&mbar, 1);
    tc::mbar_fence_init();
  }
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t taddr = tmem_slot;
  if (tid == 0) {
    const uint64_t da = tc::make_smem_desc(tc::smem_u32(sa), p.a_lbo, p.a_sbo, p.a_swz);
    const uint64_t db = tc::make_smem_desc(tc::smem_u32(sb), p.b_lbo, p.b_sbo, p.b_swz);
    for (uint32_t ks = 0; ks < p.ksteps; ++ks)
      tc::mma_ss(taddr, da + ((ks * p.a_kstep_bytes) >> 4), db + ((ks * p.b_kstep_bytes) >> 4), p.idesc, ks > 0);
    tc::mma_commit(&mbar);
  }
  const bool ok = tc::mbar_wait(&mbar, 0);
  tc::fence_after_sync();
  if (ok) {
    for (uint32_t c0 = 0; c0 < p.ncols; c0 += 16) {
      uint32_t r[16];
      tc::tmem_ld_32x32b_x16(taddr + ((uint32_t)(32 * warp) << 16) + c0, r);
      tc::tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 16; ++i)
        if (c0 + i < p.ncols) p.d_out[(size_t)(32 * warp + lane) * p.ncols + c0 + i] = __uint_as_float(r[i]);
    }
  } else if (tid == 0) {
    *p.status = 1;
  }
  tc::fence_before_sync();
  __syncthreads();
  if (warp == 0) tc::tmem_dealloc(taddr, tcols);
}

mxb_status umma_selftest(const void* a_img, uint32_t a_bytes, const void* b_img, uint32_t b_bytes,
                         const uint32_t* f, float* d_out, int* status, cudaStream_t st) {
  UmmaTestP p{};
  p.a_img = static_cast<const uint8_t*>(a_img);
  p.b_img = static_cast<const uint8_t*>(b_img);
  p.a_bytes = a_bytes; p.b_bytes = b_bytes;
  p.a_lbo = f[0]; p.a_sbo = f[1]; p.a_swz = f[2];
  p.b_lbo = f[3]; p.b_sbo = f[4]; p.b_swz = f[5];
  p.idesc = f[6]; p.ksteps = f[7]; p.a_kstep_bytes = f[8]; p.b_kstep_bytes = f[9]; p.ncols = f[10];
  p.d_out = d_out; p.status = status;
  if (a_bytes % 16 || b_bytes % 16 || p.ncols < 8 || p.ncols > 256) return MXB_ERR_INVALID_ARGUMENT;
  const size_t sm = ((a_bytes + 1023u) & ~1023u) + ((b_bytes + 1023u) & ~1023u) + 1024;
  if (sm > 200 * 1024) return MXB_ERR_UNSUPPORTED;
  cudaError_t e = cudaFuncSetAttribute(umma_selftest_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);
  if (e != cudaSuccess) { set_last_cuda_error((int)e); return MXB_ERR_CUDA; }
  MXB_LAUNCH("umma_selftest_kernel", st, (umma_selftest_kernel<<<1, 128, sm, st>>>(p)));
  return check_launch("umma_selftest_kernel");
}

// A wait that runs out on purpose: one barrier that nothing ever arrives on, polled `limit` times by every
// thread through the same bounded wait the production kernels use.  The kernel then leaves normally and
// records code 9 in the status word, exactly like a production kernel whose copy or MMA never completed.
__global__ void __launch_bounds__(64) wait_timeout_selftest_kernel(int* status, uint32_t limit) {
  __shared__ uint64_t mbar;
  if (threadIdx.x == 0) {
    tc::mbar_init(&mbar, 1);
    tc::mbar_fence_init();
  }
  __syncthreads();
  const bool ok = tc::mbar_wait(&mbar, 0, limit);
  if (!__syncthreads_and(ok) && threadIdx.x == 0) atomicExch(status, 9);
}

mxb_status wait_timeout_selftest(void* workspace, uint32_t limit, cudaStream_t st) {
  if (limit == 0 || limit > (1u << 16)) return MXB_ERR_INVALID_ARGUMENT;  // keeps the polling short
  cudaError_t e = cudaMemsetAsync(workspace, 0, 256, st);
  if (e != cudaSuccess) { set_last_cuda_error((int)e); return MXB_ERR_CUDA; }
  MXB_LAUNCH("wait_timeout_selftest_kernel", st,
             (wait_timeout_selftest_kernel<<<1, 64, 0, st>>>(static_cast<int*>(workspace), limit)));
  return check_launch("wait_timeout_selftest_kernel");
}

}  // namespace mxb
