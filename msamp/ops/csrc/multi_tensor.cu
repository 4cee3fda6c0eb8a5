// Multi-tensor gradient statistics and clipping: ONE launch computes the squared 2-norm over any mix of
// high-precision (fp32 / fp16 / bf16) and FP8 (e4m3 / e5m2, per-tensor scale_inv) gradient tensors and
// raises a flag when any value is not finite; ONE launch applies the clip coefficient (high-precision
// tensors are multiplied, FP8 tensors only have their scale_inv multiplied - their bytes are not
// touched).  Nothing is read back to the host.
//
// Replaces the per-tensor loops of the reference: apex multi_tensor_l2norm / multi_tensor_scale in
// msamp/megatron/optimizer/clip_grads.py:79-107, the ScalingTensor branch of
// torch._amp_foreach_non_finite_check_and_unscale_ in msamp/common/tensor/tensor.py:798-844 and the
// stack of norms in msamp/nn/clip_grad.py:45-88.
#include "common.cuh"

namespace {

constexpr int kThreads = 256;
constexpr int kChunk = 65536;    // elements per work item

struct NormTensor {
  const void* data;
  float* scale_inv;    // FP8 tensors: dequantisation factor (also what clipping multiplies); null otherwise
  int64_t n;
  int code;            // 0 fp32, 1 fp16, 2 bf16, 3 e4m3, 4 e5m2
  int pad;
};

template <typename T>
__device__ __forceinline__ float sumsq_hp(const T* p, int64_t begin, int64_t end) {
  float s = 0.0f;
  constexpr int N = 16 / sizeof(T);
  const bool vec = (reinterpret_cast<uintptr_t>(p + begin) & 15) == 0;
  int64_t i = begin;
  if (vec) {
    const int64_t nv = (end - begin) / N;
    const Bytes16* v = reinterpret_cast<const Bytes16*>(p + begin);
    for (int64_t k = threadIdx.x; k < nv; k += kThreads) {
      Bytes16 x = v[k];
      const T* e = reinterpret_cast<const T*>(&x);
#pragma unroll
      for (int j = 0; j < N; ++j) {
        float f = to_f32<T>(e[j]);
        s += f * f;
      }
    }
    i = begin + nv * N;
  }
  for (int64_t k = i + threadIdx.x; k < end; k += kThreads) {
    float f = to_f32<T>(p[k]);
    s += f * f;
  }
  return s;
}

template <int FMT>
__device__ __forceinline__ float sumsq_fp8(const uint8_t* p, int64_t begin, int64_t end) {
  float s = 0.0f;
  const bool vec = (reinterpret_cast<uintptr_t>(p + begin) & 15) == 0;
  int64_t i = begin;
  if (vec) {
    const int64_t nv = (end - begin) / 16;
    const Bytes16* v = reinterpret_cast<const Bytes16*>(p + begin);
    for (int64_t k = threadIdx.x; k < nv; k += kThreads) {
      Bytes16 x = v[k];
      const uint8_t* e = reinterpret_cast<const uint8_t*>(&x);
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        float f = fp8_to_f32<FMT>(e[j]);
        s += f * f;
      }
    }
    i = begin + nv * 16;
  }
  for (int64_t k = i + threadIdx.x; k < end; k += kThreads) {
    float f = fp8_to_f32<FMT>(p[k]);
    s += f * f;
  }
  return s;
}

// work: (tensor, chunk) pairs.  out[0] += sum of squares of the dequantised values; out[1] = 1 if anything is not finite.
__global__ void __launch_bounds__(kThreads) multi_sumsq_kernel(const NormTensor* __restrict__ tensors, const int* __restrict__ work, int n_work,
                                                                float* out) {
  __shared__ float red[32];
  float total = 0.0f;
  for (int w = blockIdx.x; w < n_work; w += gridDim.x) {
    const NormTensor t = tensors[work[2 * w]];
    const int64_t begin = (int64_t)work[2 * w + 1] * kChunk;
    const int64_t end = begin + kChunk < t.n ? begin + kChunk : t.n;
    float s;
    switch (t.code) {
      case 0: s = sumsq_hp<float>((const float*)t.data, begin, end); break;
      case 1: s = sumsq_hp<__half>((const __half*)t.data, begin, end); break;
      case 2: s = sumsq_hp<__nv_bfloat16>((const __nv_bfloat16*)t.data, begin, end); break;
      case 3: s = sumsq_fp8<FMT_E4M3>((const uint8_t*)t.data, begin, end); break;
      default: s = sumsq_fp8<FMT_E5M2>((const uint8_t*)t.data, begin, end); break;
    }
    if (t.scale_inv != nullptr) {
      const float si = *t.scale_inv;
      s *= si * si;
    }
    total += s;
  }
  total = block_sum(total, red);
  if (threadIdx.x == 0) {
    atomicAdd(out, total);
    if (!(fabsf(total) <= 3.0e38f)) out[1] = 1.0f;    // inf or NaN anywhere in this CTA's share
  }
}

// coef = min(1, max_norm / (sqrt(sumsq) + eps)); high-precision tensors are scaled in place, FP8 tensors through scale_inv.
__global__ void __launch_bounds__(kThreads) multi_clip_kernel(const NormTensor* __restrict__ tensors, const int* __restrict__ work, int n_work,
                                                               const float* __restrict__ sumsq, float max_norm, float eps) {
  const float coef = fminf(1.0f, max_norm / (sqrtf(*sumsq) + eps));
  if (coef >= 1.0f) return;
  for (int w = blockIdx.x; w < n_work; w += gridDim.x) {
    const NormTensor t = tensors[work[2 * w]];
    const int chunk = work[2 * w + 1];
    if (t.scale_inv != nullptr || t.code >= 3) {    // scaled tensors are clipped through their dequantisation factor
      if (chunk == 0 && threadIdx.x == 0 && t.scale_inv != nullptr) *t.scale_inv *= coef;
      continue;
    }
    const int64_t begin = (int64_t)chunk * kChunk;
    const int64_t end = begin + kChunk < t.n ? begin + kChunk : t.n;
    for (int64_t k = begin + threadIdx.x; k < end; k += kThreads) {
      if (t.code == 0) {
        float* p = (float*)t.data;
        p[k] *= coef;
      } else if (t.code == 1) {
        __half* p = (__half*)t.data;
        p[k] = __float2half_rn(__half2float(p[k]) * coef);
      } else {
        __nv_bfloat16* p = (__nv_bfloat16*)t.data;
        p[k] = __float2bfloat16_rn(__bfloat162float(p[k]) * coef);
      }
    }
  }
}

// ---- multi-tensor quantisation ---------------------------------------------------------------------------------
// One launch casts any number of high-precision tensors to FP8, each with its own scale: either the scale stored for
// the tensor (delayed scaling; max|x| is recorded) or the scale that a given amax implies (in-time scaling from an
// amax the producer already reduced, e.g. the wgrad GEMM epilogue).  Replaces one cast launch per tensor
// (msamp/common/tensor/cast.py:17-65 called per gradient in msamp/nn/distributed.py:160-176).
struct CastTensor {
  const void* src;
  uint8_t* dst;
  float* scale;            // read; rewritten when amax_in is given
  float* scale_inv;        // receives 1 / scale (nullable)
  const float* amax_in;    // nullable: max|x|, from which the scale is derived by the power-of-two rule
  float* amax_out;         // nullable: receives max|x| (zeroed by the caller)
  int64_t n;
  int code;                // 0 fp32, 1 fp16, 2 bf16
  int fmt;                 // FMT_E4M3 / FMT_E5M2
};

template <typename T, int FMT>
__device__ __forceinline__ float cast_chunk(const T* src, uint8_t* dst, int64_t begin, int64_t end, float scale) {
  float m = 0.0f;
  constexpr int N = 16 / sizeof(T);
  const bool vec = ((reinterpret_cast<uintptr_t>(src + begin) & 15) == 0) && ((reinterpret_cast<uintptr_t>(dst + begin) & (N - 1)) == 0);
  int64_t i = begin;
  if (vec) {
    const int64_t nv = (end - begin) / N;
    const Bytes16* v = reinterpret_cast<const Bytes16*>(src + begin);
    for (int64_t k = threadIdx.x; k < nv; k += kThreads) {
      Bytes16 x = v[k];
      const T* e = reinterpret_cast<const T*>(&x);
      uint16_t o[N / 2];
#pragma unroll
      for (int j = 0; j < N; j += 2) {
        const float a = to_f32<T>(e[j]), b = to_f32<T>(e[j + 1]);
        m = fmaxf(m, fmaxf(abs_nan_to_inf(a), abs_nan_to_inf(b)));
        o[j / 2] = f32x2_to_fp8x2<FMT>(a * scale, b * scale);
      }
      if (N == 8) *reinterpret_cast<Bytes8*>(dst + begin + k * N) = *reinterpret_cast<Bytes8*>(o);
      else        *reinterpret_cast<uint32_t*>(dst + begin + k * N) = *reinterpret_cast<uint32_t*>(o);
    }
    i = begin + nv * N;
  }
  for (int64_t k = i + threadIdx.x; k < end; k += kThreads) {
    const float a = to_f32<T>(src[k]);
    m = fmaxf(m, abs_nan_to_inf(a));
    dst[k] = f32_to_fp8<FMT>(a * scale);
  }
  return m;
}

__global__ void __launch_bounds__(kThreads) multi_cast_kernel(const CastTensor* __restrict__ tensors, const int* __restrict__ work, int n_work) {
  __shared__ float red[32];
  for (int w = blockIdx.x; w < n_work; w += gridDim.x) {
    const CastTensor t = tensors[work[2 * w]];
    const int chunk = work[2 * w + 1];
    const int64_t begin = (int64_t)chunk * kChunk;
    const int64_t end = begin + kChunk < t.n ? begin + kChunk : t.n;
    float scale = *t.scale;
    if (t.amax_in != nullptr) {
      const float a = *t.amax_in;
      if ((a > 0.0f) && !isinf(a) && !isnan(a)) scale = msamp_compute_scale(a, scale, fp8_max(t.fmt), 0);
    }
    __syncthreads();    // every thread has read the old scale before one of them may replace it
    if (chunk == 0 && threadIdx.x == 0) {
      if (t.amax_in != nullptr) *t.scale = scale;
      if (t.scale_inv != nullptr) *t.scale_inv = __frcp_rn(scale);
    }
    float m;
    if (t.fmt == FMT_E4M3) {
      if (t.code == 0) m = cast_chunk<float, FMT_E4M3>((const float*)t.src, t.dst, begin, end, scale);
      else if (t.code == 1) m = cast_chunk<__half, FMT_E4M3>((const __half*)t.src, t.dst, begin, end, scale);
      else m = cast_chunk<__nv_bfloat16, FMT_E4M3>((const __nv_bfloat16*)t.src, t.dst, begin, end, scale);
    } else {
      if (t.code == 0) m = cast_chunk<float, FMT_E5M2>((const float*)t.src, t.dst, begin, end, scale);
      else if (t.code == 1) m = cast_chunk<__half, FMT_E5M2>((const __half*)t.src, t.dst, begin, end, scale);
      else m = cast_chunk<__nv_bfloat16, FMT_E5M2>((const __nv_bfloat16*)t.src, t.dst, begin, end, scale);
    }
    if (t.amax_out != nullptr) {
      m = block_max(m, red);
      if (threadIdx.x == 0) atomic_max_nonneg(t.amax_out, m);
    }
  }
}

}    // namespace

MSAMP_API int msamp_multi_tensor_cast_desc_bytes() { return (int)sizeof(CastTensor); }

// tensors: device array of CastTensor; work: n_work (tensor, chunk) pairs with chunks of msamp_multi_tensor_chunk() elements.
// A tensor with several chunks must not change its scale while the launch runs: with amax_in the new scale depends on the
// amax only (or stays the old one when the amax is unusable), so every chunk derives the same value.
MSAMP_API int msamp_multi_tensor_cast(const void* tensors, const int* work, int n_work, void* stream_) {
  if (n_work <= 0) return MSAMP_OK;
  MSAMP_REQUIRE(tensors && work, "multi_tensor_cast: null pointer");
  int grid = msamp_sm_count() * 4;
  if (n_work < grid) grid = n_work;
  multi_cast_kernel<<<grid, kThreads, 0, (cudaStream_t)stream_>>>((const CastTensor*)tensors, work, n_work);
  return msamp_check_launch("msamp_multi_tensor_cast");
}

MSAMP_API int msamp_multi_tensor_desc_bytes() { return (int)sizeof(NormTensor); }
MSAMP_API int msamp_multi_tensor_chunk() { return kChunk; }

// tensors / work: device arrays (see NormTensor; work holds n_work (tensor, chunk) pairs).  out: two floats, zeroed by
// the caller: out[0] accumulates the squared norm, out[1] becomes 1 when a non-finite value was seen.
MSAMP_API int msamp_multi_tensor_sumsq(const void* tensors, const int* work, int n_work, float* out, void* stream_) {
  if (n_work <= 0) return MSAMP_OK;
  MSAMP_REQUIRE(tensors && work && out, "multi_tensor_sumsq: null pointer");
  int grid = msamp_sm_count() * 4;
  if (n_work < grid) grid = n_work;
  multi_sumsq_kernel<<<grid, kThreads, 0, (cudaStream_t)stream_>>>((const NormTensor*)tensors, work, n_work, out);
  return msamp_check_launch("msamp_multi_tensor_sumsq");
}

// Scales every tensor by min(1, max_norm / (sqrt(*sumsq) + eps)); sumsq is a device scalar (e.g. out[0] of the call above,
// after any cross-rank all-reduce).
MSAMP_API int msamp_multi_tensor_clip(const void* tensors, const int* work, int n_work, const float* sumsq, float max_norm, float eps,
                                      void* stream_) {
  if (n_work <= 0) return MSAMP_OK;
  MSAMP_REQUIRE(tensors && work && sumsq, "multi_tensor_clip: null pointer");
  int grid = msamp_sm_count() * 4;
  if (n_work < grid) grid = n_work;
  multi_clip_kernel<<<grid, kThreads, 0, (cudaStream_t)stream_>>>((const NormTensor*)tensors, work, n_work, sumsq, max_norm, eps);
  return msamp_check_launch("msamp_multi_tensor_clip");
}
