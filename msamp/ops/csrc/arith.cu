// FP8 accumulate (in place  fp8 <- quantise(dequantise(fp8) + other)  with a fresh per-tensor
// scale) and reductions over FP8 payloads.
//
// The reference does the accumulate in one kernel around a software grid barrier that spins
// without limit and assumes all blocks are co-resident (msamp/operators/arithmetic/
// vectorized_pointwise.h:184-301).  Here the two passes are two ordinary launches (amax, then
// requantise) followed by a one-thread publish of the new meta, so there is nothing to wait on.
#include "common.cuh"

namespace {

constexpr int kThreads = 256;

template <typename T, int FMT>
__global__ void __launch_bounds__(kThreads) add_amax_kernel(const uint8_t* __restrict__ q, const T* __restrict__ other, int64_t n,
                                                             const float* __restrict__ scale_inv, float* amax_tmp) {
  __shared__ float red[32];
  const float si = *scale_inv;
  float m = 0.0f;
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) m = fmaxf(m, abs_nan_to_inf(fp8_to_f32<FMT>(q[i]) * si + to_f32<T>(other[i])));
  m = block_max(m, red);
  if (threadIdx.x == 0) atomic_max_nonneg(amax_tmp, m);
}

template <typename T, int FMT>
__global__ void __launch_bounds__(kThreads) add_requant_kernel(uint8_t* __restrict__ q, const T* __restrict__ other, int64_t n,
                                                                const float* __restrict__ scale, const float* __restrict__ scale_inv,
                                                                const float* __restrict__ amax_tmp) {
  const float si = *scale_inv;
  const float sf = msamp_compute_scale(*amax_tmp, *scale, fp8_max(FMT), 0);
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) q[i] = f32_to_fp8<FMT>((fp8_to_f32<FMT>(q[i]) * si + to_f32<T>(other[i])) * sf);
}

__global__ void add_publish_kernel(float* scale, float* scale_inv, float* amax, const float* amax_tmp, float fp_max) {
  float a = *amax_tmp;
  float sf = msamp_compute_scale(a, *scale, fp_max, 0);
  *scale = sf;
  *scale_inv = __frcp_rn(sf);
  *amax = a;
}

template <int FMT>
__global__ void __launch_bounds__(kThreads) fp8_sumsq_kernel(const uint8_t* __restrict__ q, int64_t n, float* out) {
  __shared__ float red[32];
  float s = 0.0f;
  int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const bool vec = (reinterpret_cast<uintptr_t>(q) & 15) == 0;
  int64_t done = 0;
  if (vec) {
    int64_t nv = n / 16;
    for (int64_t i = tid; i < nv; i += stride) {
      Bytes16 r = reinterpret_cast<const Bytes16*>(q)[i];
      const uint8_t* b = reinterpret_cast<const uint8_t*>(&r);
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        float v = fp8_to_f32<FMT>(b[j]);
        s += v * v;
      }
    }
    done = nv * 16;
  }
  for (int64_t i = done + tid; i < n; i += stride) {
    float v = fp8_to_f32<FMT>(q[i]);
    s += v * v;
  }
  s = block_sum(s, red);
  if (threadIdx.x == 0) atomicAdd(out, s);
}

}    // namespace

// amax_tmp: one float of scratch owned by the caller (any value on entry).
MSAMP_API int msamp_add_to_fp8(void* fp8, int64_t n, int fmt, float* scale, float* scale_inv, float* amax, const void* other,
                               int other_dtype, float* amax_tmp, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  MSAMP_REQUIRE(fp8 && scale && scale_inv && amax && other && amax_tmp && n >= 0, "msamp_add_to_fp8: bad arguments");
  if (n == 0) return MSAMP_OK;
  cudaMemsetAsync(amax_tmp, 0, sizeof(float), stream);
  int grid = msamp_grid_for(n, kThreads, 8);
  MSAMP_DISPATCH_HP(other_dtype, T, {
    MSAMP_DISPATCH_FP8(fmt, F, {
      add_amax_kernel<T, F><<<grid, kThreads, 0, stream>>>((const uint8_t*)fp8, (const T*)other, n, scale_inv, amax_tmp);
      add_requant_kernel<T, F><<<grid, kThreads, 0, stream>>>((uint8_t*)fp8, (const T*)other, n, scale, scale_inv, amax_tmp);
      add_publish_kernel<<<1, 1, 0, stream>>>(scale, scale_inv, amax, amax_tmp, fp8_max(F));
    });
  });
  return msamp_check_launch("msamp_add_to_fp8");
}

// *out += sum of squares of the raw FP8 numbers.
MSAMP_API int msamp_fp8_sumsq(const void* q, int64_t n, int fmt, float* out, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  if (n <= 0) return MSAMP_OK;
  int grid = msamp_grid_for((n + 15) / 16, kThreads, 4);
  MSAMP_DISPATCH_FP8(fmt, F, { fp8_sumsq_kernel<F><<<grid, kThreads, 0, stream>>>((const uint8_t*)q, n, out); });
  return msamp_check_launch("msamp_fp8_sumsq");
}
