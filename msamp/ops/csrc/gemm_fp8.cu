// FP8 GEMM for sm_100a:  D[M,N] = (sa_inv * sb_inv) * A[M,K] * B[N,K]^T  (+ bias[N]) (+ D)
//
// A and B hold e4m3 or e5m2 bytes with K contiguous ("TN" layout); the per-tensor scale_inv
// factors are read from device memory so that no host synchronisation is needed.  The kernel is
// persistent (one CTA per SM) and warp specialised:
//   warp 0        TMA producer: 128-byte-swizzled A/B tiles into a ring of shared-memory stages
//   warp 1        allocates TMEM and issues tcgen05.mma (kind::f8f6f4, 128 x BN x 32 per instruction)
//   warps 2..5    epilogue: tcgen05.ld the fp32 accumulator, scale, add bias / previous D, convert,
//                 store, and optionally reduce max|D| for the next quantisation
// Two accumulator buffers in TMEM let the epilogue of tile i overlap the main loop of tile i+1.
// Every wait on an mbarrier is bounded; when one gives up the CTA sets the device status word,
// lets its outstanding copies land, frees its TMEM and returns.
//
// Replaces the cuBLASLt call behind the reference's Gemm.fp8_gemm (msamp/operators/gemm/gemm.py:121-144).
#include "gemm_common.cuh"

namespace {
using namespace gemm;

// Tile index -> (m tile, n tile).  Tiles are walked in groups of group_m row tiles: inside a group the row
// index runs fastest, so the CTAs of one wave share a few A tiles and a few B tiles that stay in L2
// (with a plain column-major walk a wave touches every A tile once and large-K problems stream A
// from HBM once per column of tiles).  The host picks group_m so that a group's slab of A stays well
// inside the 126 MB L2; when all of A fits, one group covers every row tile and B is streamed exactly once.
__device__ __forceinline__ void tile_to_mn(int tile, int num_m, int num_n, int group_m, int& mi, int& ni) {
  const int per_group = group_m * num_n;
  const int g = tile / per_group;
  const int first = g * group_m;
  const int gsize = (num_m - first) < group_m ? (num_m - first) : group_m;
  const int r = tile - g * per_group;
  mi = first + r % gsize;
  ni = r / gsize;
}

template <int BN, typename OutT>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_fp8_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b, const GemmParams p) {
  using C = Cfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  // 128B-swizzled tiles need 1024-byte alignment.
  const uint32_t raw_addr = tc5::smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw_addr);

  const uint32_t bars = base + C::TILE_BYTES;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (C::STAGES + s); };
  auto tfull_bar = [&](int b) { return bars + 8u * (2 * C::STAGES + b); };
  auto tempty_bar = [&](int b) { return bars + 8u * (2 * C::STAGES + 2 + b); };
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(smem + C::TILE_BYTES + 8 * (2 * C::STAGES + 4));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const int num_m = (p.M + BM - 1) / BM;
  const int num_n = (p.N + BN - 1) / BN;
  const int num_tiles = num_m * num_n;
  const int num_kb = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; ++s) {
      tc5::mbar_init(full_bar(s), 1);
      tc5::mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      tc5::mbar_init(tfull_bar(b), 1);
      tc5::mbar_init(tempty_bar(b), 4);
    }
    *abort_flag = 0;
    tc5::mbar_fence_init();
    tc5::tma_prefetch_desc(&tma_a);
    tc5::tma_prefetch_desc(&tma_b);
  }
  if (warp == 1) {
    tc5::tmem_alloc(tc5::smem_u32(tmem_holder), C::TMEM_COLS);
    tc5::tmem_relinquish();
  }
  tc5::fence_before_sync();
  __syncthreads();
  tc5::fence_after_sync();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t it = 0;
      for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
        int mi, ni;
        tile_to_mn(tile, num_m, num_n, p.group_m, mi, ni);
        const int m0 = mi * BM;
        const int n0 = ni * BN;
        bool ok = true;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % C::STAGES;
          const uint32_t ph = (it / C::STAGES) & 1;
          if (!tc5::mbar_wait(empty_bar(s), ph ^ 1, abort_flag, p.status, 1u)) { ok = false; break; }
          tc5::mbar_arrive_expect_tx(full_bar(s), C::STAGE_BYTES);
          const uint32_t sa = base + s * C::STAGE_BYTES;
          tc5::tma_load_2d(sa, &tma_a, kb * BK, m0, full_bar(s));
          tc5::tma_load_2d(sa + C::A_BYTES, &tma_b, kb * BK, n0, full_bar(s));
        }
        if (!ok) break;
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = tc5::idesc_f8(BM, BN, p.a_fmt, p.b_fmt);
      uint32_t it = 0;
      uint32_t lt = 0;
      for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++lt) {
        const int buf = lt & 1;
        const uint32_t aph = (lt >> 1) & 1;
        if (!tc5::mbar_wait(tempty_bar(buf), aph ^ 1, abort_flag, p.status, 1u)) break;
        tc5::fence_after_sync();
        const uint32_t tmem_d = tmem_base + (uint32_t)(buf * BN);
        bool ok = true;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % C::STAGES;
          const uint32_t ph = (it / C::STAGES) & 1;
          if (!tc5::mbar_wait(full_bar(s), ph, abort_flag, p.status, 1u)) { ok = false; break; }
          tc5::fence_after_sync();
          const uint32_t sa = base + s * C::STAGE_BYTES;
          const uint64_t da = tc5::smem_desc_k_sw128(sa);
          const uint64_t db = tc5::smem_desc_k_sw128(sa + C::A_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            // +2 in the start-address field == +32 bytes along K inside the swizzle atom
            tc5::mma_f8f6f4(tmem_d, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc, (kb | k) ? 1u : 0u);
          }
          tc5::mma_commit(empty_bar(s));    // frees the stage once these MMAs have read it
        }
        if (!ok) break;
        tc5::mma_commit(tfull_bar(buf));    // accumulator complete
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (4 warps)
    const int q = warp & 3;    // TMEM lane quarter this warp may access
    const float alpha = (*p.scale_inv_a) * (*p.scale_inv_b);
    OutT* D = reinterpret_cast<OutT*>(p.d);
    const bool vec_ok = ((reinterpret_cast<uintptr_t>(D) & 15) == 0) && ((p.ldd * sizeof(OutT)) % 16 == 0);
    float amax = 0.0f;
    uint32_t lt = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++lt) {
      int mi, ni;
      tile_to_mn(tile, num_m, num_n, p.group_m, mi, ni);
      const int m0 = mi * BM;
      const int n0 = ni * BN;
      const int buf = lt & 1;
      const uint32_t aph = (lt >> 1) & 1;
      if (!tc5::mbar_wait(tfull_bar(buf), aph, abort_flag, p.status, 1u)) break;
      tc5::fence_after_sync();
      const int row = m0 + q * 32 + lane;
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * BN);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tc5::tmem_ld32(taddr + (uint32_t)(c * 32), r);
        tc5::tmem_ld_wait();
        const int col = n0 + c * 32;
        int valid = p.N - col;
        valid = valid > 32 ? 32 : valid;
        if (row < p.M && valid > 0) {
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) * alpha;
          if (p.bias != nullptr) {
            if (p.bias_dtype == DT_F32) {
              const float* b = reinterpret_cast<const float*>(p.bias) + col;
#pragma unroll
              for (int j = 0; j < 32; ++j) if (j < valid) v[j] += __ldg(b + j);
            } else if (p.bias_dtype == DT_BF16) {
              const __nv_bfloat16* b = reinterpret_cast<const __nv_bfloat16*>(p.bias) + col;
#pragma unroll
              for (int j = 0; j < 32; ++j) if (j < valid) v[j] += __bfloat162float(b[j]);
            } else {
              const __half* b = reinterpret_cast<const __half*>(p.bias) + col;
#pragma unroll
              for (int j = 0; j < 32; ++j) if (j < valid) v[j] += __half2float(b[j]);
            }
          }
          OutT* dst = D + (int64_t)row * p.ldd + col;
          if (p.accumulate) {
            float old[32];
            load_chunk<OutT>(dst, old, vec_ok, valid);
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] += old[j];
          }
          if (p.amax_out != nullptr) {
#pragma unroll
            for (int j = 0; j < 32; ++j) if (j < valid) amax = fmaxf(amax, abs_nan_to_inf(v[j]));
          }
          store_chunk<OutT>(dst, v, vec_ok, valid);
        }
      }
      tc5::fence_before_sync();
      __syncwarp();
      if (lane == 0) tc5::mbar_arrive(tempty_bar(buf));
    }
    if (p.amax_out != nullptr) {
      amax = warp_max(amax);
      if (lane == 0) atomic_max_nonneg(p.amax_out, amax);
    }
  }

  // ---------------------------------------------------------------------- tear-down
  __syncwarp();
  if (*abort_flag) __nanosleep(200000);    // let copies / MMAs in flight finish before smem and TMEM go away
  tc5::fence_before_sync();
  __syncthreads();
  tc5::fence_after_sync();
  if (warp == 1) tc5::tmem_dealloc(tmem_base, C::TMEM_COLS);
}

template <int BN, typename OutT>
int launch(const CUtensorMap& ma, const CUtensorMap& mb, const GemmParams& p, int max_ctas, cudaStream_t stream) {
  using C = Cfg<BN>;
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!configured[dev & 63]) {
    cudaError_t e = cudaFuncSetAttribute(gemm_fp8_kernel<BN, OutT>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
    if (e != cudaSuccess) {
      msamp_set_error("cudaFuncSetAttribute: %s", cudaGetErrorString(e));
      return MSAMP_ELAUNCH;
    }
    configured[dev & 63] = true;
  }
  const int num_tiles = ((p.M + BM - 1) / BM) * ((p.N + BN - 1) / BN);
  int grid = msamp_sm_count();
  if (max_ctas > 0 && max_ctas < grid) grid = max_ctas;
  if (num_tiles < grid) grid = num_tiles;
  gemm_fp8_kernel<BN, OutT><<<grid, kGemmThreads, C::SMEM_BYTES, stream>>>(ma, mb, p);
  return msamp_check_launch("gemm_fp8_kernel");
}

}    // namespace

// A: [M, K] fp8 bytes with row pitch lda (bytes), B: [N, K] with pitch ldb, D: [M, N] of out_dtype
// with row pitch ldd (elements).  K, lda, ldb must be multiples of 16 and A, B 16-byte aligned
// (TMA rules).  bias may be null; amax_out (nullable) must be zeroed by the caller and receives
// max|D|.  max_ctas > 0 caps the number of persistent CTAs (to leave SMs to a concurrent kernel).
MSAMP_API int msamp_gemm_fp8(const void* A, const void* B, void* D, int M, int N, int K, int64_t lda, int64_t ldb, int64_t ldd,
                             int a_fmt, int b_fmt, int out_dtype, const float* scale_inv_a, const float* scale_inv_b,
                             const void* bias, int bias_dtype, int accumulate, float* amax_out, int max_ctas, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  MSAMP_REQUIRE(M > 0 && N > 0 && K > 0, "msamp_gemm_fp8: empty problem M=%d N=%d K=%d", M, N, K);
  MSAMP_REQUIRE(K % 16 == 0 && lda % 16 == 0 && ldb % 16 == 0, "msamp_gemm_fp8: K and the row pitches must be multiples of 16");
  MSAMP_REQUIRE((reinterpret_cast<uintptr_t>(A) & 15) == 0 && (reinterpret_cast<uintptr_t>(B) & 15) == 0,
                "msamp_gemm_fp8: operands must be 16-byte aligned");
  MSAMP_REQUIRE(scale_inv_a && scale_inv_b && D, "msamp_gemm_fp8: null pointer");
  const int bn = (N > 128 && (int64_t)((M + BM - 1) / BM) * ((N + 255) / 256) >= msamp_sm_count()) ? 256 : 128;
  CUtensorMap ma, mb;
  int rc = make_map(A, M, K, lda, BM, &ma);
  if (rc) return rc;
  rc = make_map(B, N, K, ldb, bn, &mb);
  if (rc) return rc;
  GemmParams p;
  p.d = D; p.bias = bias; p.scale_inv_a = scale_inv_a; p.scale_inv_b = scale_inv_b; p.amax_out = amax_out;
  p.status = msamp_device_status_ptr();
  p.M = M; p.N = N; p.K = K; p.ldd = ldd; p.out_dtype = out_dtype; p.bias_dtype = bias_dtype; p.accumulate = accumulate;
  p.a_fmt = a_fmt; p.b_fmt = b_fmt;
  {
    const int num_m = (M + BM - 1) / BM;
    int64_t g = (48ll << 20) / ((int64_t)BM * K);    // row tiles whose A slab is about 48 MB
    if (g < 8) g = 8;
    p.group_m = g >= num_m ? num_m : (int)g;
  }
  MSAMP_DISPATCH_HP(out_dtype, T, {
    if (bn == 256) return launch<256, T>(ma, mb, p, max_ctas, stream);
    return launch<128, T>(ma, mb, p, max_ctas, stream);
  });
  return MSAMP_OK;
}
