// Simulated FP4 (e2m1) in bf16 and the derivative used by the differentiable gradient estimator.
// Same value set and interval rules as the reference kernels (msamp/operators/fp4_quantize/quantize.cu:16-119).
#include "common.cuh"

namespace {

__constant__ float kGrid[15] = {-6.0f, -4.0f, -3.0f, -2.0f, -1.5f, -1.0f, -0.5f, 0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};

// Nearest representable value; a value exactly half-way between two neighbours goes to the upper one.
__device__ __forceinline__ float nearest_e2m1(float x) {
  float best = kGrid[14];
#pragma unroll
  for (int i = 13; i >= 0; --i) {
    float mid = 0.5f * (kGrid[i] + kGrid[i + 1]);
    if (x < mid) best = kGrid[i];
  }
  return best;
}

__global__ void fp4_quantize_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ out, int64_t n) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) out[i] = __float2bfloat16(nearest_e2m1(__bfloat162float(x[i])));
}

// d/dx of the smooth surrogate on the interval [a, a + delta): min(|2 (x - a) / delta - 1|^(1/k - 1) / k, clamp).
__device__ __forceinline__ float dge(float x, float a, float delta, float k, float clamp_max) {
  float t = fabsf(2.0f * (x - a) / delta - 1.0f);
  return fminf(powf(t, 1.0f / k - 1.0f) / k, clamp_max);
}

__global__ void fp4_dge_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ out, float k, float clamp_max,
                               int64_t n) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) {
    float v = __bfloat162float(x[i]);
    float dy = 0.0f;
    if (v < -4.0f) {
      dy = dge(v, -6.0f, 2.0f, k, clamp_max);    // also used below -6, as the reference does
    } else if (v <= 6.0f) {
      int j = 1;
#pragma unroll
      for (int q = 2; q < 14; ++q)
        if (v >= kGrid[q]) j = q;
      dy = dge(v, kGrid[j], kGrid[j + 1] - kGrid[j], k, clamp_max);
    }
    out[i] = __float2bfloat16(dy);
  }
}

}    // namespace

MSAMP_API int msamp_fp4_quantize_bf16(const void* x, void* out, int64_t n, void* stream_) {
  if (n <= 0) return MSAMP_OK;
  int grid = msamp_grid_for(n, 256, 8);
  fp4_quantize_kernel<<<grid, 256, 0, (cudaStream_t)stream_>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)out, n);
  return msamp_check_launch("msamp_fp4_quantize_bf16");
}

MSAMP_API int msamp_fp4_dge_bf16(const void* x, void* out, float k, float clamp_max, int64_t n, void* stream_) {
  if (n <= 0) return MSAMP_OK;
  int grid = msamp_grid_for(n, 256, 8);
  fp4_dge_kernel<<<grid, 256, 0, (cudaStream_t)stream_>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)out, k, clamp_max, n);
  return msamp_check_launch("msamp_fp4_dge_bf16");
}
