// Multi-tensor low-bit Adam / AdamW.
//
// One launch per stage covers every parameter of the optimizer (the reference launches two kernels
// per parameter from a Python loop and synchronises with the host twice per step,
// msamp/optim/adamw.py:148-199, msamp/optim/adamw.cu:30-153).
//
//   stage 1  reads p, g, m, v; computes the new moments and the new parameter in fp32 and reduces
//            max|p_new|, max|m_new|, max|v_new| per tensor.
//   stage 2  derives the new per-tensor scales from those maxima on the device, recomputes the same
//            values and stores them in their storage formats (scaled fp16 / e4m3 / e5m2 / plain),
//            then block 0 of each tensor publishes scale, scale_inv and amax into the metas.
//
// The update itself always uses the unquantised new moments, exactly like the reference kernels.
#include "common.cuh"

namespace {

// storage codes: 0 f32, 1 f16, 2 bf16, 3 e4m3, 4 e5m2
enum { ST_F32 = 0, ST_F16 = 1, ST_BF16 = 2, ST_E4M3 = 3, ST_E5M2 = 4 };

struct AdamTensor {
  void* p;
  const void* g;
  void* m;
  void* v;
  float* p_scale;    // null when the parameter is unscaled
  float* p_scale_inv;
  float* p_amax;
  const float* g_scale_inv;    // null: gradient is plain high precision
  float* m_scale;
  float* m_scale_inv;
  float* m_amax;
  float* v_scale;
  float* v_scale_inv;
  float* v_amax;
  uint8_t* w8;            // optional: e4m3 copy of the NEW parameter (scaled-fp16 parameters only), written by stage 2
  float* w8_scale_inv;    // 1 / scale of that copy (written when the metas are published)
  int64_t n;
  int p_st, g_st, m_st, v_st;
  float lr_wd_factor;    // 1 - lr * wd (decoupled) or 1
  float l2;              // wd for L2 mode, else 0
  float beta1, beta2, eps, step_size, inv_sqrt_bc2, gsign;
  int tensor_scale;
  int g_index;           // fused reduce-scatter: index of this tensor in the ranks' symmetric gradient buffers, else -1
  float red[4];          // stage-1 results: max|p|, max|m|, max|v|
};

// Symmetric FP8 gradient buffers of the data-parallel group (see symm.cu): with them stage 1 pulls every rank's
// e4m3 bytes of a tensor this rank owns, dequantises each with that rank's scale, averages in fp32, rounds the
// mean to e4m3 once (stored locally for stage 2) and feeds the rounded value straight into the Adam arithmetic -
// the reduce-scatter and the first optimizer pass are one kernel, and the averaged gradient is never read back.
constexpr int kMaxPeers = 8;
struct PeerGrads {
  const uint8_t* data[kMaxPeers];    // flat e4m3 gradient buffer of every rank (same layout everywhere)
  float* meta[kMaxPeers];            // [3][n_tensors] per rank: scale_inv | amax | result scale_inv
  int world, rank, n_tensors;
};

constexpr int kChunk = 32768;    // elements per block
constexpr int kAdamThreads = 256;

__device__ __forceinline__ float st_max(int st) {
  switch (st) {
    case ST_F16: return 65504.0f;
    case ST_E4M3: return 448.0f;
    case ST_E5M2: return 57344.0f;
    default: return 3.0e38f;
  }
}

__device__ __forceinline__ void load8(const void* base, int st, int64_t i, float (&o)[8]) {
  switch (st) {
    case ST_F32: {
      const float4* p = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(base) + i);
      float4 a = p[0], b = p[1];
      o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w; o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
      break;
    }
    case ST_F16: {
      Bytes16 r = *reinterpret_cast<const Bytes16*>(reinterpret_cast<const __half*>(base) + i);
      const __half* e = reinterpret_cast<const __half*>(&r);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = __half2float(e[j]);
      break;
    }
    case ST_BF16: {
      Bytes16 r = *reinterpret_cast<const Bytes16*>(reinterpret_cast<const __nv_bfloat16*>(base) + i);
      const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&r);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = __bfloat162float(e[j]);
      break;
    }
    case ST_E4M3: {
      Bytes8 r = *reinterpret_cast<const Bytes8*>(reinterpret_cast<const uint8_t*>(base) + i);
      const uint16_t* e = reinterpret_cast<const uint16_t*>(&r);
#pragma unroll
      for (int j = 0; j < 4; ++j) {    // two elements per hardware conversion
        __half2_raw h = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)e[j], __NV_E4M3);
        float2 f = __half22float2(__half2(h));
        o[2 * j] = f.x;
        o[2 * j + 1] = f.y;
      }
      break;
    }
    default: {
      Bytes8 r = *reinterpret_cast<const Bytes8*>(reinterpret_cast<const uint8_t*>(base) + i);
      const uint16_t* e = reinterpret_cast<const uint16_t*>(&r);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        __half2_raw h = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)e[j], __NV_E5M2);
        float2 f = __half22float2(__half2(h));
        o[2 * j] = f.x;
        o[2 * j + 1] = f.y;
      }
      break;
    }
  }
}

__device__ __forceinline__ float load1(const void* base, int st, int64_t i) {
  switch (st) {
    case ST_F32: return reinterpret_cast<const float*>(base)[i];
    case ST_F16: return __half2float(reinterpret_cast<const __half*>(base)[i]);
    case ST_BF16: return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(base)[i]);
    case ST_E4M3: return fp8_to_f32<FMT_E4M3>(reinterpret_cast<const uint8_t*>(base)[i]);
    default: return fp8_to_f32<FMT_E5M2>(reinterpret_cast<const uint8_t*>(base)[i]);
  }
}

__device__ __forceinline__ float sat(float x, float mx) { return (x != x) ? x : fminf(fmaxf(x, -mx), mx); }

__device__ __forceinline__ void store8(void* base, int st, int64_t i, const float (&o)[8]) {
  switch (st) {
    case ST_F32: {
      float4* p = reinterpret_cast<float4*>(reinterpret_cast<float*>(base) + i);
      p[0] = make_float4(o[0], o[1], o[2], o[3]);
      p[1] = make_float4(o[4], o[5], o[6], o[7]);
      break;
    }
    case ST_F16: {
      Bytes16 r;
      __half* e = reinterpret_cast<__half*>(&r);
#pragma unroll
      for (int j = 0; j < 8; ++j) e[j] = __float2half_rn(sat(o[j], 65504.0f));
      *reinterpret_cast<Bytes16*>(reinterpret_cast<__half*>(base) + i) = r;
      break;
    }
    case ST_BF16: {
      Bytes16 r;
      __nv_bfloat16* e = reinterpret_cast<__nv_bfloat16*>(&r);
#pragma unroll
      for (int j = 0; j < 8; ++j) e[j] = __float2bfloat16_rn(o[j]);
      *reinterpret_cast<Bytes16*>(reinterpret_cast<__nv_bfloat16*>(base) + i) = r;
      break;
    }
    case ST_E4M3: {
      Bytes8 r;
      uint16_t* e = reinterpret_cast<uint16_t*>(&r);
#pragma unroll
      for (int j = 0; j < 8; j += 2) e[j / 2] = f32x2_to_fp8x2<FMT_E4M3>(o[j], o[j + 1]);
      *reinterpret_cast<Bytes8*>(reinterpret_cast<uint8_t*>(base) + i) = r;
      break;
    }
    default: {
      Bytes8 r;
      uint16_t* e = reinterpret_cast<uint16_t*>(&r);
#pragma unroll
      for (int j = 0; j < 8; j += 2) e[j / 2] = f32x2_to_fp8x2<FMT_E5M2>(o[j], o[j + 1]);
      *reinterpret_cast<Bytes8*>(reinterpret_cast<uint8_t*>(base) + i) = r;
      break;
    }
  }
}

__device__ __forceinline__ void store1(void* base, int st, int64_t i, float x) {
  switch (st) {
    case ST_F32: reinterpret_cast<float*>(base)[i] = x; break;
    case ST_F16: reinterpret_cast<__half*>(base)[i] = __float2half_rn(sat(x, 65504.0f)); break;
    case ST_BF16: reinterpret_cast<__nv_bfloat16*>(base)[i] = __float2bfloat16_rn(x); break;
    case ST_E4M3: reinterpret_cast<uint8_t*>(base)[i] = f32_to_fp8<FMT_E4M3>(x); break;
    default: reinterpret_cast<uint8_t*>(base)[i] = f32_to_fp8<FMT_E5M2>(x); break;
  }
}

struct Elem {
  float p, m, v;
};

__device__ __forceinline__ Elem adam_elem(const AdamTensor& t, float p, float g, float m, float v, float psi, float gsi, float msi,
                                          float vsi) {
  p *= psi;
  g = g * gsi * t.gsign;
  g += t.l2 * p;
  p *= t.lr_wd_factor;
  Elem e;
  e.m = t.beta1 * (m * msi) + (1.0f - t.beta1) * g;
  e.v = t.beta2 * (v * vsi) + (1.0f - t.beta2) * (g * g);
  // sqrt and the division use the hardware approximations (about 1 ulp): the kernel is otherwise bound by
  // instruction issue, not by memory, and Adam is insensitive to errors of that size
  float root;
  asm("sqrt.approx.ftz.f32 %0, %1;" : "=f"(root) : "f"(e.v));
  float denom = root * t.inv_sqrt_bc2 + t.eps;
  e.p = p - t.step_size * __fdividef(e.m, denom);
  return e;
}

// Work of one block on elements [begin, end) of tensor t.  The storage codes are template
// parameters for the combinations that dominate real models (the switches in load8/store8 then
// fold away and the four loads of an iteration are issued back to back); -1 means "read the code
// from the descriptor at run time".
template <int STAGE, int PS, int GS, int MS, int VS>
__device__ __forceinline__ void adam_block(AdamTensor& t, int64_t begin, int64_t end, float* red) {
  const int p_st = PS >= 0 ? PS : t.p_st, g_st = GS >= 0 ? GS : t.g_st, m_st = MS >= 0 ? MS : t.m_st, v_st = VS >= 0 ? VS : t.v_st;
  const float psi = t.p_scale_inv ? *t.p_scale_inv : 1.0f;
  const float gsi = t.g_scale_inv ? *t.g_scale_inv : 1.0f;
  const float msi = t.m_scale_inv ? *t.m_scale_inv : 1.0f;
  const float vsi = t.v_scale_inv ? *t.v_scale_inv : 1.0f;

  float ps = 1.0f, ms = 1.0f, vs = 1.0f;
  if (STAGE == 2) {
    if (t.p_scale) ps = msamp_compute_scale(t.red[0], *t.p_scale, st_max(p_st), 0);
    if (t.m_scale) ms = t.tensor_scale ? msamp_compute_scale(t.red[1], 1.0f, st_max(m_st), 0) : 1.0f;
    if (t.v_scale) vs = t.tensor_scale ? msamp_compute_scale(t.red[2], 1.0f, st_max(v_st), 0) : 1.0f;
  }

  // e4m3 copy of the new parameter: scale from the power-of-two rule on max|p| (stage 1), applied to the payload that is
  // stored with scale ps, i.e. payload * (s8 / ps) - the arithmetic of re-quantising the stored tensor
  uint8_t* w8 = (STAGE == 2 && p_st == ST_F16 && t.p_scale) ? t.w8 : nullptr;
  const float w8_factor = w8 ? msamp_compute_scale(t.red[0], 1.0f, 448.0f, 0) * __frcp_rn(ps) : 0.0f;
  const bool vec = ((reinterpret_cast<uintptr_t>(t.p) | reinterpret_cast<uintptr_t>(t.g) | reinterpret_cast<uintptr_t>(t.m) |
                     reinterpret_cast<uintptr_t>(t.v) | reinterpret_cast<uintptr_t>(w8)) & 15) == 0;
  float ap = 0.0f, am = 0.0f, av = 0.0f;
  if (vec) {
#pragma unroll 2
    for (int64_t i = begin + (int64_t)threadIdx.x * 8; i + 8 <= end; i += (int64_t)kAdamThreads * 8) {
      float p[8], g[8], m[8], v[8];
      load8(t.p, p_st, i, p);
      load8(t.g, g_st, i, g);
      load8(t.m, m_st, i, m);
      load8(t.v, v_st, i, v);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        Elem e = adam_elem(t, p[j], g[j], m[j], v[j], psi, gsi, msi, vsi);
        if (STAGE == 1) {
          ap = fmaxf(ap, abs_nan_to_inf(e.p));
          am = fmaxf(am, abs_nan_to_inf(e.m));
          av = fmaxf(av, abs_nan_to_inf(e.v));
        } else {
          p[j] = e.p * ps;
          m[j] = e.m * ms;
          v[j] = e.v * vs;
        }
      }
      if (STAGE == 2) {
        store8(t.p, p_st, i, p);
        store8(t.m, m_st, i, m);
        store8(t.v, v_st, i, v);
        if (w8 != nullptr) {
          // the e4m3 copy is taken from the parameter AS STORED (rounded to fp16), with the factor a separate cast of the
          // stored tensor would use, so it equals that cast bit for bit
          uint16_t o8[4];
#pragma unroll
          for (int j = 0; j < 8; j += 2) {
            const float a = __half2float(__float2half_rn(sat(p[j], 65504.0f))), b = __half2float(__float2half_rn(sat(p[j + 1], 65504.0f)));
            o8[j / 2] = f32x2_to_fp8x2<FMT_E4M3>(a * w8_factor, b * w8_factor);
          }
          *reinterpret_cast<uint2*>(w8 + i) = *reinterpret_cast<const uint2*>(o8);
        }
      }
    }
  }
  {
    // tail of the chunk (or the whole chunk when the pointers are not 16-byte aligned)
    int64_t tail = vec ? begin + ((end - begin) / 8) * 8 : begin;
    for (int64_t i = tail + threadIdx.x; i < end; i += kAdamThreads) {
      Elem e = adam_elem(t, load1(t.p, p_st, i), load1(t.g, g_st, i), load1(t.m, m_st, i), load1(t.v, v_st, i), psi, gsi, msi, vsi);
      if (STAGE == 1) {
        ap = fmaxf(ap, abs_nan_to_inf(e.p));
        am = fmaxf(am, abs_nan_to_inf(e.m));
        av = fmaxf(av, abs_nan_to_inf(e.v));
      } else {
        store1(t.p, p_st, i, e.p * ps);
        store1(t.m, m_st, i, e.m * ms);
        store1(t.v, v_st, i, e.v * vs);
        if (w8 != nullptr) w8[i] = f32_to_fp8<FMT_E4M3>(__half2float(__float2half_rn(sat(e.p * ps, 65504.0f))) * w8_factor);
      }
    }
  }
  if (STAGE == 1) {
    ap = block_max(ap, red);
    am = block_max(am, red);
    av = block_max(av, red);
    if (threadIdx.x == 0) {
      atomic_max_nonneg(&t.red[0], ap);
      atomic_max_nonneg(&t.red[1], am);
      atomic_max_nonneg(&t.red[2], av);
    }
  }
}

// Stage 1 of a tensor whose gradient still lies, unreduced, in the ranks' symmetric buffers.
__device__ __forceinline__ void adam_block_reduce(AdamTensor& t, const PeerGrads& pg, int64_t begin, int64_t end, bool first_chunk, float* red) {
  const float psi = t.p_scale_inv ? *t.p_scale_inv : 1.0f;
  const float msi = t.m_scale_inv ? *t.m_scale_inv : 1.0f;
  const float vsi = t.v_scale_inv ? *t.v_scale_inv : 1.0f;
  const int64_t goff = reinterpret_cast<const uint8_t*>(t.g) - pg.data[pg.rank];    // same offset in every rank's buffer
  float sinv[kMaxPeers];
  float amax = 0.0f;
  const float inv_world = 1.0f / (float)pg.world;
#pragma unroll
  for (int r = 0; r < kMaxPeers; ++r) {
    if (r < pg.world) {
      sinv[r] = pg.meta[r][t.g_index] * inv_world;
      amax = fmaxf(amax, abs_nan_to_inf(pg.meta[r][pg.n_tensors + t.g_index]));
    }
  }
  // same rule and the same summation order as the stand-alone reduce kernel, so both paths produce the same bytes
  const float new_scale = msamp_compute_scale(amax, 1.0f, 448.0f, 0);
  const float gsi = __frcp_rn(new_scale);
  if (first_chunk && threadIdx.x == 0) pg.meta[pg.rank][2 * pg.n_tensors + t.g_index] = gsi;
  uint8_t* gq = reinterpret_cast<uint8_t*>(const_cast<void*>(t.g));
  float ap = 0.0f, am = 0.0f, av = 0.0f;
  const bool vec = ((reinterpret_cast<uintptr_t>(t.p) | reinterpret_cast<uintptr_t>(t.g) | reinterpret_cast<uintptr_t>(t.m) |
                     reinterpret_cast<uintptr_t>(t.v)) & 15) == 0;
  int64_t done = begin;
  if (vec) {
#pragma unroll 2
    for (int64_t i = begin + (int64_t)threadIdx.x * 8; i + 8 <= end; i += (int64_t)kAdamThreads * 8) {
      float acc[8], p[8], m[8], v[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.0f;
#pragma unroll
      for (int r = 0; r < kMaxPeers; ++r) {
        if (r < pg.world) {
          const int src = (pg.rank + r) % pg.world;    // stagger peers so that the ranks do not all hit one GPU at once
          const Bytes8 b = *reinterpret_cast<const Bytes8*>(pg.data[src] + goff + i);
          const uint8_t* e = reinterpret_cast<const uint8_t*>(&b);
          const float sc = sinv[src];
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[j] += fp8_to_f32<FMT_E4M3>(e[j]) * sc;
        }
      }
      load8(t.p, t.p_st, i, p);
      load8(t.m, t.m_st, i, m);
      load8(t.v, t.v_st, i, v);
      Bytes8 q;
      uint16_t* qe = reinterpret_cast<uint16_t*>(&q);
#pragma unroll
      for (int j = 0; j < 8; j += 2) qe[j / 2] = f32x2_to_fp8x2<FMT_E4M3>(acc[j] * new_scale, acc[j + 1] * new_scale);
      *reinterpret_cast<Bytes8*>(gq + i) = q;    // the reduced gradient, for stage 2
      const uint8_t* qb = reinterpret_cast<const uint8_t*>(&q);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        Elem e = adam_elem(t, p[j], fp8_to_f32<FMT_E4M3>(qb[j]), m[j], v[j], psi, gsi, msi, vsi);
        ap = fmaxf(ap, abs_nan_to_inf(e.p));
        am = fmaxf(am, abs_nan_to_inf(e.m));
        av = fmaxf(av, abs_nan_to_inf(e.v));
      }
    }
    done = begin + ((end - begin) / 8) * 8;
  }
  for (int64_t i = done + threadIdx.x; i < end; i += kAdamThreads) {
    float acc = 0.0f;
    for (int r = 0; r < pg.world; ++r) {
      const int src = (pg.rank + r) % pg.world;
      acc += fp8_to_f32<FMT_E4M3>(pg.data[src][goff + i]) * sinv[src];
    }
    const uint8_t q = f32_to_fp8<FMT_E4M3>(acc * new_scale);
    gq[i] = q;
    Elem e = adam_elem(t, load1(t.p, t.p_st, i), fp8_to_f32<FMT_E4M3>(q), load1(t.m, t.m_st, i), load1(t.v, t.v_st, i), psi, gsi, msi, vsi);
    ap = fmaxf(ap, abs_nan_to_inf(e.p));
    am = fmaxf(am, abs_nan_to_inf(e.m));
    av = fmaxf(av, abs_nan_to_inf(e.v));
  }
  ap = block_max(ap, red);
  am = block_max(am, red);
  av = block_max(av, red);
  if (threadIdx.x == 0) {
    atomic_max_nonneg(&t.red[0], ap);
    atomic_max_nonneg(&t.red[1], am);
    atomic_max_nonneg(&t.red[2], av);
  }
}

__global__ void __launch_bounds__(kAdamThreads) lbadam_reduce_stage1_kernel(AdamTensor* tensors, const int* __restrict__ work, const PeerGrads pg) {
  __shared__ float red[32];
  AdamTensor& t = tensors[work[2 * blockIdx.x]];
  const int chunk = work[2 * blockIdx.x + 1];
  const int64_t begin = (int64_t)chunk * kChunk;
  const int64_t end = (begin + kChunk < t.n) ? begin + kChunk : t.n;
  if (t.g_index >= 0 && t.g_st == ST_E4M3) {
    adam_block_reduce(t, pg, begin, end, chunk == 0, red);
  } else {
    adam_block<1, -1, -1, -1, -1>(t, begin, end, red);    // gradients that were reduced elsewhere (high-precision parameters)
  }
}

// block -> (tensor, chunk) map: work[2*b] = tensor index, work[2*b+1] = chunk index
template <int STAGE>
__global__ void __launch_bounds__(kAdamThreads) lbadam_kernel(AdamTensor* tensors, const int* __restrict__ work) {
  __shared__ float red[32];
  AdamTensor& t = tensors[work[2 * blockIdx.x]];
  const int chunk = work[2 * blockIdx.x + 1];
  const int64_t begin = (int64_t)chunk * kChunk;
  const int64_t end = (begin + kChunk < t.n) ? begin + kChunk : t.n;
  const int combo = (t.p_st << 9) | (t.g_st << 6) | (t.m_st << 3) | t.v_st;
#define MSAMP_COMBO(P, G, M, V) \
  case ((P << 9) | (G << 6) | (M << 3) | V): adam_block<STAGE, P, G, M, V>(t, begin, end, red); break;
  switch (combo) {
    MSAMP_COMBO(ST_F16, ST_E4M3, ST_E4M3, ST_F16)      // FP8-linear weights at O2
    MSAMP_COMBO(ST_F32, ST_F32, ST_E4M3, ST_F16)       // biases / LayerNorm at O2
    MSAMP_COMBO(ST_BF16, ST_BF16, ST_E4M3, ST_F16)     // bf16 embeddings at O2
    MSAMP_COMBO(ST_F16, ST_E4M3, ST_F32, ST_F32)       // the same three at O1
    MSAMP_COMBO(ST_F32, ST_F32, ST_F32, ST_F32)
    MSAMP_COMBO(ST_BF16, ST_BF16, ST_F32, ST_F32)
    default: adam_block<STAGE, -1, -1, -1, -1>(t, begin, end, red); break;
  }
#undef MSAMP_COMBO
}

// After stage 2 has consumed the old inverse scales everywhere: publish the new metas.
__global__ void lbadam_finalize_kernel(AdamTensor* tensors, int n) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  AdamTensor& t = tensors[i];
  if (t.p_scale) {
    float s = msamp_compute_scale(t.red[0], *t.p_scale, st_max(t.p_st), 0);
    *t.p_scale = s;
    *t.p_scale_inv = __frcp_rn(s);
    if (t.p_amax) *t.p_amax = t.red[0];
    if (t.w8 && t.w8_scale_inv && t.p_st == ST_F16) *t.w8_scale_inv = __frcp_rn(msamp_compute_scale(t.red[0], 1.0f, 448.0f, 0));
  }
  if (t.m_scale) {
    float s = t.tensor_scale ? msamp_compute_scale(t.red[1], 1.0f, st_max(t.m_st), 0) : 1.0f;
    *t.m_scale = s;
    *t.m_scale_inv = __frcp_rn(s);
    if (t.m_amax) *t.m_amax = t.red[1];
  }
  if (t.v_scale) {
    float s = t.tensor_scale ? msamp_compute_scale(t.red[2], 1.0f, st_max(t.v_st), 0) : 1.0f;
    *t.v_scale = s;
    *t.v_scale_inv = __frcp_rn(s);
    if (t.v_amax) *t.v_amax = t.red[2];
  }
}

}    // namespace

MSAMP_API int msamp_lbadam_tensor_bytes() { return (int)sizeof(AdamTensor); }
MSAMP_API int msamp_lbadam_chunk() { return kChunk; }

// `tensors`: device array of n_tensors descriptors (layout of AdamTensor; `red` must be zero on
// entry); `work`: device array of 2 * n_blocks ints mapping each block to (tensor, chunk).
MSAMP_API int msamp_lbadam_step(void* tensors, int n_tensors, const int* work, int n_blocks, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  if (n_tensors <= 0 || n_blocks <= 0) return MSAMP_OK;
  lbadam_kernel<1><<<n_blocks, kAdamThreads, 0, stream>>>((AdamTensor*)tensors, work);
  lbadam_kernel<2><<<n_blocks, kAdamThreads, 0, stream>>>((AdamTensor*)tensors, work);
  lbadam_finalize_kernel<<<(n_tensors + 127) / 128, 128, 0, stream>>>((AdamTensor*)tensors, n_tensors);
  return msamp_check_launch("msamp_lbadam_step");
}

// Same step with the FP8 gradient reduce-scatter folded into stage 1.  data / meta: `world` device pointers to the
// ranks' symmetric gradient and meta buffers (this rank's own at index `rank`); descriptors with g_index >= 0 must
// have `g` pointing into this rank's buffer and `g_scale_inv` at meta row 2 of that tensor.  The caller has made sure
// (cross-rank barrier on the stream) that every rank finished writing its gradients and metas.
MSAMP_API int msamp_lbadam_step_reduce(void* tensors, int n_tensors, const int* work, int n_blocks, void* const* data, void* const* meta,
                                       int world, int rank, int n_sym_tensors, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  if (n_tensors <= 0 || n_blocks <= 0) return MSAMP_OK;
  MSAMP_REQUIRE(world >= 1 && world <= kMaxPeers && rank >= 0 && rank < world, "lbadam_step_reduce: bad world=%d rank=%d", world, rank);
  PeerGrads pg;
  for (int r = 0; r < kMaxPeers; ++r) {
    pg.data[r] = r < world ? (const uint8_t*)data[r] : nullptr;
    pg.meta[r] = r < world ? (float*)meta[r] : nullptr;
  }
  pg.world = world; pg.rank = rank; pg.n_tensors = n_sym_tensors;
  lbadam_reduce_stage1_kernel<<<n_blocks, kAdamThreads, 0, stream>>>((AdamTensor*)tensors, work, pg);
  lbadam_kernel<2><<<n_blocks, kAdamThreads, 0, stream>>>((AdamTensor*)tensors, work);
  lbadam_finalize_kernel<<<(n_tensors + 127) / 128, 128, 0, stream>>>((AdamTensor*)tensors, n_tensors);
  return msamp_check_launch("msamp_lbadam_step_reduce");
}
