// Calibration probe for the tile model of the tt.dot kernels: what one thread's tcgen05 instruction stream costs.
//
// One CTA pair per two SMs issues cta_group::2 MMAs (M 256, K 16, bf16) back to back on resident shared memory;
// nothing is loaded and nothing waits on another CTA, so the cycles per block of MMAs (clock64 of the issuing
// thread, start to the completion of a final commit) are the cost of the instruction stream itself: the tensor pipe
// when the stream is lean, the issuing thread when it is not. The shapes differ only in the code around the MMAs.
// With N = 256 an MMA occupies the pipe for 128 cycles; with N = 64 for 32, which exposes the issue cost.
//
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -o tcgen05_issue_probe tcgen05_issue_probe.cu && ./tcgen05_issue_probe
//
// Every wait is bounded; the probe allocates 64 bytes of device memory and runs for a few milliseconds.
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <cstdlib>

namespace {

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile("{\n.reg .pred P;\nelect.sync _|P, 0xffffffff;\nselp.u32 %0, 1, 0, P;\n}\n" : "=r"(pred));
  return pred != 0;
}
__device__ __forceinline__ void mma(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}" ::"r"(d), "l"(a),
               "l"(b), "r"(idesc), "r"(accumulate)
               : "memory");
}
__device__ __forceinline__ void mma_acc(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc) {
  asm volatile("{\n.reg .pred p;\nsetp.eq.b32 p, 0, 0;\ntcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}" ::"r"(d), "l"(a),
               "l"(b), "r"(idesc)
               : "memory");
}
__device__ __forceinline__ void commit_both(uint32_t bar) {  // one commit, delivered to both CTAs of the pair
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
               "h"(static_cast<uint16_t>(3))
               : "memory");
}
__device__ __forceinline__ bool test_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n.reg .pred p;\nmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
               : "=r"(ok)
               : "r"(bar), "r"(parity)
               : "memory");
  return ok != 0;
}

struct Params {
  uint32_t n;          // MMA N
  uint32_t desc_hi;    // shared-memory descriptor, upper word (SWIZZLE_128B, stride 1024 bytes)
  uint32_t kstep;      // start-address step per MMA, 16-byte units
  uint32_t work;       // SHAPE 5: cycles of other work the issuing thread does per block
};

enum Shape {
  kLean = 0,            // 4 MMAs per block, descriptors from two multiply-adds, nothing else
  kCommit = 1,          // + one multicast commit per block
  kCommitAndProbe = 2,  // + a test_wait of the next stage's barrier and a warp vote between the MMAs (the library kernel's block)
  kEightPerCommit = 3,  // 8 MMAs and one commit per block
  kBranchPerMma = 4,    // every MMA in a divergent region of its own
  kOtherWork = 5,       // kLean + `work` cycles of unrelated work per block by the issuing thread
  kTwoAccumulators = 6  // 4 MMAs into one accumulator, 4 into the other, one commit (the wide tile's block)
};

template <int SHAPE>
__global__ void __launch_bounds__(128, 1) probe_kernel(Params p, int blocks, long long *out) {
  extern __shared__ uint8_t raw[];
  __shared__ uint32_t tmem_base_s;
  __shared__ unsigned long long done_bar, stage_bar[8];
  uint32_t rank;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
  const uint32_t base = (smem_u32(raw) + 1023u) & ~1023u;
  for (uint32_t i = threadIdx.x; i < 192 * 1024 / 4; i += blockDim.x)
    reinterpret_cast<uint32_t *>(raw + (base - smem_u32(raw)))[i] = 0x3F003F00u;  // bf16 0.5 everywhere
  if (threadIdx.x == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&done_bar)));
    for (int q = 0; q < 8; ++q) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&stage_bar[q])));
    asm volatile("fence.mbarrier_init.release.cluster;");
  }
  if (threadIdx.x < 32) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(smem_u32(&tmem_base_s)));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
  }
  asm volatile("fence.proxy.async.shared::cta;");
  asm volatile("tcgen05.fence::before_thread_sync;");
  __syncthreads();
  asm volatile("barrier.cluster.arrive.release.aligned;");
  asm volatile("barrier.cluster.wait.acquire.aligned;");
  asm volatile("tcgen05.fence::after_thread_sync;");
  const uint32_t tmem = tmem_base_s;
  const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((p.n >> 3) << 17) | ((256u >> 4) << 24);
  if (threadIdx.x < 32 && rank == 0) {
    const long long t0 = clock64();
    const bool issuer = elect_one();
    const uint32_t hi = p.desc_hi, ks = p.kstep;
    const uint32_t lo_base = (1u << 16) | ((base & 0x3FFFFu) >> 4);
    auto desc = [](uint32_t h, uint32_t l) { return (static_cast<uint64_t>(h) << 32) | static_cast<uint64_t>(l); };
    uint32_t stage = 0, accumulate = 0;
    for (int it = 0; it < blocks; ++it) {
      const uint32_t alo = lo_base + stage * 2048u, blo = alo + 1024u;  // 32 KiB stages: A at +0, B at +16 KiB
      const uint32_t next = stage == 3 ? 0u : stage + 1u;
      if (SHAPE == kCommitAndProbe) {
        if (issuer) mma(tmem, desc(hi, alo), desc(hi, blo), idesc, accumulate);
        const bool peek = test_wait(smem_u32(&stage_bar[4 + next]), 1u);  // a fresh barrier: the phase before the first is complete
        if (issuer) {
          mma_acc(tmem, desc(hi, alo + ks), desc(hi, blo + ks), idesc);
          mma_acc(tmem, desc(hi, alo + 2 * ks), desc(hi, blo + 2 * ks), idesc);
        }
        const bool all = __all_sync(0xffffffffu, peek);
        if (issuer) {
          mma_acc(tmem, desc(hi, alo + 3 * ks), desc(hi, blo + 3 * ks), idesc);
          commit_both(smem_u32(&stage_bar[stage]));
        }
        if (!all) break;
      } else if (SHAPE == kBranchPerMma) {
        if (issuer) mma(tmem, desc(hi, alo), desc(hi, blo), idesc, accumulate);
        __syncwarp();
        if (issuer) mma_acc(tmem, desc(hi, alo + ks), desc(hi, blo + ks), idesc);
        __syncwarp();
        if (issuer) mma_acc(tmem, desc(hi, alo + 2 * ks), desc(hi, blo + 2 * ks), idesc);
        __syncwarp();
        if (issuer) mma_acc(tmem, desc(hi, alo + 3 * ks), desc(hi, blo + 3 * ks), idesc);
      } else if (issuer) {
        const uint32_t d0 = tmem, d1 = tmem + 256u;
        mma(d0, desc(hi, alo), desc(hi, blo), idesc, accumulate);
#pragma unroll
        for (int j = 1; j < 4; ++j) mma_acc(d0, desc(hi, alo + j * ks), desc(hi, blo + j * ks), idesc);
        if (SHAPE == kEightPerCommit) {
#pragma unroll
          for (int j = 0; j < 4; ++j) mma_acc(d0, desc(hi, alo + 512u + j * ks), desc(hi, blo + 512u + j * ks), idesc);
        }
        if (SHAPE == kTwoAccumulators) {
          mma(d1, desc(hi, alo), desc(hi, blo + 512u), idesc, accumulate);
#pragma unroll
          for (int j = 1; j < 4; ++j) mma_acc(d1, desc(hi, alo + j * ks), desc(hi, blo + 512u + j * ks), idesc);
        }
        if (SHAPE == kCommit || SHAPE == kEightPerCommit || SHAPE == kTwoAccumulators) commit_both(smem_u32(&stage_bar[stage]));
        if (SHAPE == kOtherWork) {
          const long long g0 = clock64();
          while (clock64() - g0 < static_cast<long long>(p.work)) {
          }
        }
      }
      accumulate = 1;
      __syncwarp();
      stage = next;
    }
    if (issuer) {
      uint32_t leader_bar;
      asm volatile("mapa.shared::cluster.u32 %0, %1, 0;" : "=r"(leader_bar) : "r"(smem_u32(&done_bar)));
      asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(leader_bar) : "memory");
      uint32_t ok = 0;
      for (int spin = 0; spin < (1 << 20) && !ok; ++spin)
        asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], 0;\nselp.u32 %0, 1, 0, p;\n}"
                     : "=r"(ok)
                     : "r"(smem_u32(&done_bar))
                     : "memory");
      if (blockIdx.x == 0) {
        out[0] = clock64() - t0;
        out[1] = ok;
      }
    }
    __syncwarp();
  }
  asm volatile("tcgen05.fence::before_thread_sync;");
  __syncthreads();
  asm volatile("barrier.cluster.arrive.release.aligned;");
  asm volatile("barrier.cluster.wait.acquire.aligned;");
  if (threadIdx.x < 32) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem));
}

template <int SHAPE>
void run(const char *what, uint32_t n, uint32_t work, int mmas_per_block, long long *out) {
  const int smem = 193 * 1024 + 1024;
  cudaFuncSetAttribute(probe_kernel<SHAPE>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  Params p;
  p.n = n;
  p.desc_hi = ((1024u >> 4) & 0x3FFFu) | (1u << 14) | (2u << 29);
  p.kstep = 2;
  p.work = work;
  cudaLaunchConfig_t lc = {};
  lc.gridDim = dim3(148);
  lc.blockDim = dim3(128);
  lc.dynamicSmemBytes = smem;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  lc.attrs = attr;
  lc.numAttrs = 1;
  const int blocks = 4096;
  for (int rep = 0; rep < 2; ++rep) {
    cudaLaunchKernelEx(&lc, probe_kernel<SHAPE>, p, blocks, out);
    const cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) {
      printf("%s: CUDA error %s\n", what, cudaGetErrorString(e));
      exit(1);
    }
  }
  long long h[2];
  cudaMemcpy(h, out, sizeof h, cudaMemcpyDeviceToHost);
  const double per_block = static_cast<double>(h[0]) / blocks;
  printf("N=%3u  %-72s %7.1f cycles per block, %6.1f per MMA%s\n", n, what, per_block, per_block / mmas_per_block,
         h[1] ? "" : "  (final wait ran out)");
  fflush(stdout);
}

}  // namespace

int main() {
  long long *out = nullptr;
  if (cudaMalloc(&out, 64) != cudaSuccess) {
    printf("no CUDA device\n");
    return 1;
  }
  for (uint32_t n : {256u, 64u}) {
    run<kLean>("4 MMAs per block, lean", n, 0, 4, out);
    run<kCommit>("4 MMAs + one multicast commit", n, 0, 4, out);
    run<kCommitAndProbe>("4 MMAs + commit + barrier probe and warp vote between the MMAs", n, 0, 4, out);
    run<kEightPerCommit>("8 MMAs + one commit", n, 0, 8, out);
    run<kBranchPerMma>("4 MMAs, each in a divergent region of its own", n, 0, 4, out);
    run<kTwoAccumulators>("4 MMAs into one accumulator, 4 into the other, one commit", n, 0, 8, out);
    run<kOtherWork>("4 MMAs + 100 cycles of other work by the issuing thread", n, 100, 4, out);
    run<kOtherWork>("4 MMAs + 300 cycles of other work by the issuing thread", n, 300, 4, out);
  }
  cudaFree(out);
  return 0;
}
