// Microbenchmark: issue rate of tcgen05.mma kind::f8f6f4 from shared-memory operands, with nothing else going on.
// One CTA per SM; one thread issues a long run of M = 128, K = 32 MMAs over a ring of four K-major, 128-byte-swizzled
// stages (A 128 x 128 bytes, B N x 128 bytes), with one tcgen05.commit per `PER_COMMIT` MMAs, and waits (bounded) only
// at the very end.  The operands are zero bytes: the cycle count, not the clock, is the result.
//
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 --expt-relaxed-constexpr -I msamp/ops/csrc \
//        benchmarks/mma_fp8_shapes.cu -o mma_fp8_shapes && ./mma_fp8_shapes
//
// The nominal rate (4.5 PFLOP/s dense over 148 SMs at 1.965 GHz) would be 8192 multiply-adds per cycle and SM, i.e.
// 128 cycles for a 128 x 256 x 32 MMA.
//
// Result on B200 (cycles per MMA): N = 256: 128.0 with a commit per 1, 4, 16 or 128 MMAs and with a tcgen05 fence per four;
// N = 128: 72.8; N = 64: 68.3 (issue-bound); CTA pair 256 x 256 x 32: 128.1; A and B MN-major: 149.1 for N = 256 and N = 128.
// A blocking wait on a completed mbarrier phase per four MMAs: 264; a non-blocking test: 187; a busy delay of nominally
// 64 / 128 / 256 / 512 cycles per four MMAs: 163 / 179 / 212 / 270.  The pipe buffers next to nothing: whatever the issuing
// thread does between two MMAs beyond about 60 cycles is lost, which is why the GEMM's main loop probes the next stage's
// barrier before the last MMA of a K block instead of waiting on it between K blocks.
#include <cstdio>
#include "tcgen05.cuh"
using namespace tc5;

// EXTRA, done by the issuing thread after every fourth MMA (a K block of the GEMM main loop): 0 nothing, 1 a tcgen05 fence,
// 2 a wait on an mbarrier whose phase is already complete plus the fence (what the main loop does when its data is there),
// 3 the same with the non-blocking test_wait, 4 the wait without the fence, 5 wait + fence after the second MMA of the K block
// instead, 6 / 7 a chain of 16 / 64 dependent integer multiply-adds, >= 16 a busy delay of EXTRA cycles on clock64.
template <int N, int PER_COMMIT, int EXTRA>
__global__ void __launch_bounds__(128, 1) k(long long* out, int n_mma, int mn) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  __shared__ uint32_t holder;
  __shared__ uint64_t barmem[3];
  __shared__ int abort_flag;
  const uint32_t bar = smem_u32(&barmem[0]);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int STAGE = 128 * 128 + N * 128;
  for (int i = threadIdx.x; i < (4 * STAGE) / 4; i += 128) reinterpret_cast<uint32_t*>(smem_raw + (base - raw))[i] = 0;
  if (threadIdx.x == 0) {
    mbar_init(bar, 1);
    mbar_init(bar + 8, 1);
    mbar_init(bar + 16, 1);
    mbar_arrive(bar + 16);    // phase 0 of this one is complete from the start
    abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(&holder), 512);
    tmem_relinquish();
  }
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tm = holder;
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  if (warp == 1 && lane == 0) {
    // mn: both operands MN-major (the layout of the weight-gradient GEMM: [k rows][128 bytes of M or N] panels)
    const uint32_t idesc = idesc_f8(128, N, 0, 0, mn, mn);
    const long long t0 = clock64();
    for (int j = 0; j < n_mma; ++j) {
      const uint32_t sa = base + (uint32_t)((j >> 2) & 3) * STAGE;
      const uint64_t da = mn ? smem_desc_mn_sw128(sa, 128 * 128) + (uint64_t)(32 * 128 / 16) * (j & 3) : smem_desc_k_sw128(sa) + 2ull * (j & 3);
      const uint64_t db = mn ? smem_desc_mn_sw128(sa + 128 * 128, 128 * 128) + (uint64_t)(32 * 128 / 16) * (j & 3)
                             : smem_desc_k_sw128(sa + 128 * 128) + 2ull * (j & 3);
      mma_f8f6f4(tm + (uint32_t)(((j >> 7) & 1) * N), da, db, idesc, (j & 127) ? 1u : 0u);
      if ((j % PER_COMMIT) == PER_COMMIT - 1) mma_commit(bar + 8);    // arrivals nobody waits for
      if ((j & 3) == 1 && EXTRA == 5) {    // the same wait, but in the middle of the K block
        mbar_wait(bar + 16, 0, &abort_flag, nullptr, 0);
        fence_after_sync();
      }
      if ((j & 3) == 3) {
        if (EXTRA == 3) {
          while (!mbar_test(bar + 16, 0)) {}
          fence_after_sync();
        }
        if (EXTRA == 4) mbar_wait(bar + 16, 0, &abort_flag, nullptr, 0);
        if (EXTRA == 6 || EXTRA == 7) {
          uint32_t x = (uint32_t)j;
#pragma unroll 1
          for (int i = 0; i < (EXTRA == 6 ? 16 : 64); ++i) asm volatile("mad.lo.u32 %0, %0, %0, %0;" : "+r"(x));
          if (x == 0x12345u) out[0] = 1;
        }
        if (EXTRA == 1) fence_after_sync();
        if (EXTRA == 2) {
          mbar_wait(bar + 16, 0, &abort_flag, nullptr, 0);
          fence_after_sync();
        }
        if (EXTRA >= 16) {
          const long long until = clock64() + EXTRA;
          while (clock64() < until) {}
        }
      }
    }
    mma_commit(bar);
    const long long t1 = clock64();
    mbar_wait(bar, 0, &abort_flag, nullptr, 0);
    const long long t2 = clock64();
    out[2 * blockIdx.x] = t1 - t0;
    out[2 * blockIdx.x + 1] = t2 - t0;
  }
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  if (warp == 0) tmem_dealloc(tm, 512);
}

// The same run for a CTA pair: one thread of the even CTA issues 256 x 256 x 32 MMAs (cta_group::2; A 128 rows and B 128
// rows from each CTA's shared memory), one multicast commit per four MMAs.
__global__ void __launch_bounds__(128, 1) k_pair(long long* out, int n_mma) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  __shared__ uint32_t holder;
  __shared__ uint64_t barmem[2];
  __shared__ int abort_flag;
  const uint32_t bar = smem_u32(&barmem[0]);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  constexpr int STAGE = 128 * 128 + 128 * 128;
  for (int i = threadIdx.x; i < (6 * STAGE) / 4; i += 128) reinterpret_cast<uint32_t*>(smem_raw + (base - raw))[i] = 0;
  if (threadIdx.x == 0) {
    mbar_init(bar, 1);
    mbar_init(bar + 8, 1);
    abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 0) {
    tmem_alloc_pair(smem_u32(&holder), 512);
    tmem_relinquish_pair();
  }
  fence_before_sync();
  __syncthreads();
  cluster_sync();
  fence_after_sync();
  const uint32_t tm = holder;
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  if (warp == 1 && lane == 0 && rank == 0) {
    const uint32_t idesc = idesc_f8(256, 256, 0, 0, 0, 0);
    const long long t0 = clock64();
    for (int j = 0; j < n_mma; ++j) {
      const uint32_t sa = base + (uint32_t)((j >> 2) % 6) * STAGE;
      const uint64_t da = smem_desc_k_sw128(sa) + 2ull * (j & 3);
      const uint64_t db = smem_desc_k_sw128(sa + 128 * 128) + 2ull * (j & 3);
      mma_f8f6f4_pair(tm + (uint32_t)(((j >> 7) & 1) * 256), da, db, idesc, (j & 127) ? 1u : 0u);
      if ((j & 3) == 3) mma_commit_pair_mc(bar + 8, (uint16_t)3);    // arrivals nobody waits for
    }
    mma_commit_pair(bar);
    const long long t1 = clock64();
    mbar_wait(bar, 0, &abort_flag, nullptr, 0);
    const long long t2 = clock64();
    out[2 * (blockIdx.x / 2)] = t1 - t0;
    out[2 * (blockIdx.x / 2) + 1] = t2 - t0;
  }
  fence_before_sync();
  __syncthreads();
  cluster_sync();
  fence_after_sync();
  if (warp == 0) tmem_dealloc_pair(tm, 512);
}

void run_pair(long long* d, int n_mma) {
  constexpr int SMEM = 6 * (128 * 128 + 128 * 128) + 2048;
  cudaFuncSetAttribute(k_pair, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(148);
  cfg.blockDim = dim3(128);
  cfg.dynamicSmemBytes = SMEM;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaSuccess;
  for (int rep = 0; rep < 2 && e == cudaSuccess; ++rep) e = cudaLaunchKernelEx(&cfg, k_pair, d, n_mma);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  long long h[2 * 74];
  cudaMemcpy(h, d, sizeof(h), cudaMemcpyDeviceToHost);
  double issue = 0, total = 0;
  for (int i = 0; i < 74; ++i) {
    issue += (double)h[2 * i] / 74;
    total += (double)h[2 * i + 1] / 74;
  }
  printf("CTA pair 256 x 256 x 32 e4m3, commit every 4 MMAs: err=%d, %.1f cycles per MMA until all issued, %.1f until all complete; %.0f multiply-adds per cycle and SM\n",
         (int)e, issue / n_mma, total / n_mma, 128.0 * 256 * 32 * n_mma / total);
}

template <int N, int PER_COMMIT, int EXTRA = 0>
void run(long long* d, int n_mma, int mn = 0) {
  constexpr int SMEM = 4 * (128 * 128 + N * 128) + 2048;
  cudaFuncSetAttribute(k<N, PER_COMMIT, EXTRA>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
  for (int rep = 0; rep < 2; ++rep) k<N, PER_COMMIT, EXTRA><<<148, 128, SMEM>>>(d, n_mma, mn);
  cudaError_t e = cudaDeviceSynchronize();
  long long h[2 * 148];
  cudaMemcpy(h, d, sizeof(h), cudaMemcpyDeviceToHost);
  double issue = 0, total = 0;
  for (int i = 0; i < 148; ++i) {
    issue += (double)h[2 * i] / 148;
    total += (double)h[2 * i + 1] / 148;
  }
  printf("128 x %3d x 32 e4m3%s, commit every %3d MMAs, extra %3d: err=%d, %.1f cycles per MMA until all issued, %.1f until all complete; %.0f multiply-adds per cycle\n",
         N, mn ? " (A, B MN-major)" : "", PER_COMMIT, EXTRA, (int)e, issue / n_mma, total / n_mma, 128.0 * N * 32 * n_mma / total);
}

int main() {
  long long* d;
  cudaMalloc(&d, 2 * 148 * sizeof(long long));
  const int n = 4096;
  run<64, 4>(d, n);
  run<128, 4>(d, n);
  run<256, 4>(d, n);
  run<256, 1>(d, n);
  run<256, 16>(d, n);
  run<256, 128>(d, n);
  run<256, 4>(d, n, 1);
  run<128, 4>(d, n, 1);
  run_pair(d, n);
  run<256, 4, 1>(d, n);
  run<256, 4, 2>(d, n);
  run<256, 4, 3>(d, n);
  run<256, 4, 4>(d, n);
  run<256, 4, 5>(d, n);
  run<256, 4, 6>(d, n);
  run<256, 4, 7>(d, n);
  run<256, 4, 64>(d, n);
  run<256, 4, 128>(d, n);
  run<256, 4, 256>(d, n);
  run<256, 4, 384>(d, n);
  run<256, 4, 512>(d, n);
  return 0;
}
