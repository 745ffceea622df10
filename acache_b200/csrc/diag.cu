// Diagnostic kernel: the rate at which one thread's stream of tcgen05.mma instructions on
// resident shared-memory operands is retired, as a function of the product's width N, the CTA
// group (1 or 2), the number of TMEM accumulators the stream alternates between, the number of
// products between two tcgen05.commit and the number of k steps per loop iteration.  No operand
// is loaded (shared memory is zeroed) and nothing is written back: the number isolates the
// tensor pipe and its issue path from the memory system.  Used by `microbench --mma-rate`.
#include "common.cuh"
#include "tcgen05.cuh"

namespace acache {
namespace diag {

using namespace tc;

struct Cfg { int n, nacc, commit_every, iters, stages, kper; };

__device__ __forceinline__ void mma_pair(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t acc) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
               ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(acc) : "memory");
}
__device__ __forceinline__ void commit_pair(uint32_t bar) {
  const uint16_t both = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(bar), "h"(both) : "memory");
}
__device__ __forceinline__ uint64_t global_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

template <int CG>
__global__ void __launch_bounds__(128, 1) mma_rate_kernel(Cfg c, long long* out) {
  extern __shared__ __align__(1024) uint8_t smem[];
  __shared__ uint64_t bars[2];
  __shared__ uint32_t tslot;
  const int tid = threadIdx.x, warp = tid >> 5;
  uint32_t rank = 0;
  if (CG == 2) asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
  const int brows = CG == 2 ? c.n / 2 : c.n;
  const int stage_bytes = 16384 + brows * 128;
  for (int i = tid; i < c.stages * stage_bytes / 16; i += blockDim.x) reinterpret_cast<uint4*>(smem)[i] = make_uint4(0, 0, 0, 0);
  if (tid == 0) {
    mbar_init(smem_u32(&bars[0]), 1);
    mbar_init(smem_u32(&bars[1]), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tslot)), "r"(512) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  fence_proxy_async();
  tc_fence_before();
  __syncthreads();
  if (CG == 2) asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
  tc_fence_after();
  const uint32_t tmem = tslot;
  if (tid == 0 && rank == 0) {
    const uint32_t idesc = make_idesc(1, 0, (uint32_t)c.n, CG == 2 ? 256 : 128);
    const int acc_cols = (c.n + 31) & ~31;
    const long long t0 = clock64();
    const uint64_t n0 = global_ns();
    long long issued = 0;
    for (int it = 0; it < c.iters; ++it) {
      const int s = it % c.stages;
      const uint32_t a = smem_u32(smem) + s * stage_bytes, b = a + 16384;
      for (int ks = 0; ks < c.kper; ++ks) {
        for (int r = 0; r < c.nacc; ++r, ++issued) {
          const uint32_t d = tmem + (uint32_t)(r * acc_cols);
          const uint64_t ad = make_desc(a + (ks & 3) * 32, 16, 1024), bd = make_desc(b + (ks & 3) * 32, 16, 1024);
          if (CG == 2) mma_pair(d, ad, bd, idesc, it > 0 || ks > 0);
          else mma_ss(d, ad, bd, idesc, it > 0 || ks > 0);
        }
      }
      if (c.commit_every && (it % c.commit_every) == c.commit_every - 1) {
        if (CG == 2) commit_pair(smem_u32(&bars[1]));
        else mma_commit(smem_u32(&bars[1]));
      }
    }
    if (CG == 2) commit_pair(smem_u32(&bars[0]));
    else mma_commit(smem_u32(&bars[0]));
    const bool done = mbar_wait(smem_u32(&bars[0]), 0);
    const long long t1 = clock64();
    const uint64_t n1 = global_ns();
    if (blockIdx.x == 0) {
      out[0] = t1 - t0;
      out[1] = (long long)(n1 - n0);
      out[2] = issued;
      out[3] = done ? 1 : 0;
    }
  } else if (tid == 0 && CG == 2) {
    mbar_wait(smem_u32(&bars[0]), 0);   // the leader's last commit also arrives here
  }
  tc_fence_before();
  __syncthreads();
  if (CG == 2) asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
  if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory");
}

}  // namespace diag
}  // namespace acache

using namespace acache;

extern "C" int acache_diag_mma_rate(int cta_group, int n, int n_accumulators, int commit_every, int k_steps, int iters,
                                    long long* result4, void* stream) {
  if ((cta_group != 1 && cta_group != 2) || n < 16 || n > 256 || n % 16 != 0 || n_accumulators < 1 || commit_every < 0 ||
      k_steps < 1 || iters < 1 || !result4)
    return ACACHE_EINVAL;
  if (n_accumulators * ((n + 31) & ~31) > 512) return ACACHE_EINVAL;
  diag::Cfg c{n, n_accumulators, commit_every, iters, 2, k_steps};
  const int brows = cta_group == 2 ? n / 2 : n;
  const size_t smem = (size_t)c.stages * (16384 + brows * 128) + 1024;
  cudaStream_t st = (cudaStream_t)stream;
  if (cta_group == 1) {
    ACACHE_CUDA_CHECK(cudaFuncSetAttribute(diag::mma_rate_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    diag::mma_rate_kernel<1><<<kNumSMs, 128, smem, st>>>(c, result4);
  } else {
    ACACHE_CUDA_CHECK(cudaFuncSetAttribute(diag::mma_rate_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3(kNumSMs);
    lc.blockDim = dim3(128);
    lc.dynamicSmemBytes = smem;
    lc.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = 2;
    at[0].val.clusterDim.y = 1;
    at[0].val.clusterDim.z = 1;
    lc.attrs = at;
    lc.numAttrs = 1;
    ACACHE_CUDA_CHECK(cudaLaunchKernelEx(&lc, diag::mma_rate_kernel<2>, c, result4));
  }
  ACACHE_LAUNCH_CHECK();
  return ACACHE_OK;
}
