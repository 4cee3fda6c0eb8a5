// Shared declarations for the sm_100a kernel library: status codes, dtype tags, the power-of-two
// scale rule, float atomics and the device-side error word.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define MSAMP_API extern "C" __attribute__((visibility("default")))

enum MsampStatus {
  MSAMP_OK = 0,
  MSAMP_EINVAL = 1,
  MSAMP_EDTYPE = 2,
  MSAMP_ELAUNCH = 3,
  MSAMP_ETIMEOUT = 4,
  MSAMP_ETMAP = 5,
  MSAMP_ECAPACITY = 6,
  MSAMP_EARCH = 7,
};

enum MsampDtype { DT_F32 = 0, DT_F16 = 1, DT_BF16 = 2 };
enum MsampFp8 { FMT_E4M3 = 0, FMT_E5M2 = 1 };

// Host side: remember a message for msamp_last_error().
void msamp_set_error(const char* fmt, ...);
int msamp_check_launch(const char* what);
// Device error word (host-mapped). Kernels OR a code into it when a bounded wait gives up.
unsigned int* msamp_device_status_ptr();
// Number of SMs of the current device (cached).
int msamp_sm_count();

#define MSAMP_REQUIRE(cond, ...)   \
  do {                             \
    if (!(cond)) {                 \
      msamp_set_error(__VA_ARGS__); \
      return MSAMP_EINVAL;         \
    }                              \
  } while (0)

// ---------------------------------------------------------------------------------------------
// dtype helpers
// ---------------------------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

template <int FMT>
__device__ __forceinline__ uint8_t f32_to_fp8(float v) {
  return (uint8_t)__nv_cvt_float_to_fp8(v, __NV_SATFINITE, FMT == FMT_E4M3 ? __NV_E4M3 : __NV_E5M2);
}
template <int FMT>
__device__ __forceinline__ uint16_t f32x2_to_fp8x2(float a, float b) {
  return (uint16_t)__nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, FMT == FMT_E4M3 ? __NV_E4M3 : __NV_E5M2);
}
template <int FMT>
__device__ __forceinline__ float fp8_to_f32(uint8_t v) {
  __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)v, FMT == FMT_E4M3 ? __NV_E4M3 : __NV_E5M2);
  return __half2float(__half(h));
}

#define MSAMP_DISPATCH_HP(code, T, ...)                 \
  switch (code) {                                       \
    case DT_F32: { using T = float; __VA_ARGS__; break; }         \
    case DT_F16: { using T = __half; __VA_ARGS__; break; }        \
    case DT_BF16: { using T = __nv_bfloat16; __VA_ARGS__; break; } \
    default: msamp_set_error("unsupported dtype code %d", (int)(code)); return MSAMP_EDTYPE; \
  }

#define MSAMP_DISPATCH_FP8(code, F, ...)                \
  switch (code) {                                       \
    case FMT_E4M3: { constexpr int F = FMT_E4M3; __VA_ARGS__; break; } \
    case FMT_E5M2: { constexpr int F = FMT_E5M2; __VA_ARGS__; break; } \
    default: msamp_set_error("unsupported fp8 format %d", (int)(code)); return MSAMP_EDTYPE; \
  }

__host__ __device__ __forceinline__ float fp8_max(int fmt) { return fmt == FMT_E4M3 ? 448.0f : 57344.0f; }

// ---------------------------------------------------------------------------------------------
// Scale rule: exp = floor(log2(fp_max / amax)) - margin; sf = 2^|exp|; sf = 1/sf when exp < 0;
// the previous scale is kept when amax is zero, negative or not finite.  The exponent is clamped
// so that the scale itself stays finite and normal.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float msamp_compute_scale(float amax, float old_scale, float fp_max, int margin) {
  if (!(amax > 0.0f) || isinf(amax) || isnan(amax)) return old_scale;
  float ratio = __fdiv_rn(fp_max, amax);
  float e = floorf(log2f(ratio)) - (float)margin;
  e = fminf(fmaxf(e, -126.0f), 126.0f);
  return exp2f(e);    // exact for integral e
}

// amax values are non-negative or +inf, for which the IEEE bit pattern is monotone as an integer.
__device__ __forceinline__ void atomic_max_nonneg(float* addr, float v) {
  atomicMax(reinterpret_cast<int*>(addr), __float_as_int(v));
}
// |v| with NaN mapped to +inf so that a single max reduction reports any non-finite input.
__device__ __forceinline__ float abs_nan_to_inf(float v) {
  float a = fabsf(v);
  return (a != a) ? __int_as_float(0x7f800000) : a;
}

// GeLU, tanh form, and its derivative, written with the logistic function: 0.5 (1 + tanh(u)) == 1 / (1 + exp(-2u)).
// One exponential and one approximate division per element keep it cheap enough for a GEMM epilogue.  One definition
// for the elementwise kernels and the GEMM epilogues, so that a fused path produces the bits of the separate kernels.
__device__ __forceinline__ float gelu_sigmoid_2u(float x) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  const float u = k0 * (x + k1 * x * x * x);
  return __fdividef(1.0f, 1.0f + __expf(-2.0f * u));
}
__device__ __forceinline__ float gelu_f(float x) { return x * gelu_sigmoid_2u(x); }
__device__ __forceinline__ float gelu_grad_f(float x) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  const float s = gelu_sigmoid_2u(x);
  // d/dx [x s(2u)] = s + x * 2 s (1 - s) * du/dx
  return s + 2.0f * x * s * (1.0f - s) * k0 * (1.0f + 3.0f * k1 * x * x);
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Block-wide max of non-negative values; result valid in thread 0. `red` holds >= 32 floats.
__device__ __forceinline__ float block_max(float v, float* red) {
  v = warp_max(v);
  int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  if (lane == 0) red[w] = v;
  __syncthreads();
  int nw = (blockDim.x + 31) >> 5;
  v = (threadIdx.x < nw) ? red[threadIdx.x] : 0.0f;
  if (w == 0) v = warp_max(v);
  __syncthreads();
  return v;
}
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  if (lane == 0) red[w] = v;
  __syncthreads();
  int nw = (blockDim.x + 31) >> 5;
  v = (threadIdx.x < nw) ? red[threadIdx.x] : 0.0f;
  if (w == 0) v = warp_sum(v);
  __syncthreads();
  return v;
}

// Grid size for a grid-stride elementwise kernel: enough CTAs to fill every SM a few times over,
// never more than the work needs.
static inline int msamp_grid_for(int64_t work_items, int threads, int ctas_per_sm = 8) {
  int64_t need = (work_items + threads - 1) / threads;
  int64_t cap = (int64_t)msamp_sm_count() * ctas_per_sm;
  if (need < 1) need = 1;
  return (int)(need < cap ? need : cap);
}

struct alignas(16) Bytes16 { uint32_t w[4]; };
struct alignas(8) Bytes8 { uint32_t w[2]; };
