// Non-GEMM kernels of the transformer block: LayerNorm forward/backward, GeLU forward/backward
// (tanh form), and fused softmax cross-entropy (loss + in-place logit gradient).  All are
// HBM-bandwidth bound: one pass over the data with 16-byte accesses, statistics in fp32.
#include <atomic>
#include <type_traits>

#include "common.cuh"
#include "msamp_noalloc.h"
#include "tcgen05.cuh"

namespace {

// ------------------------------------------------------------------------------------------------
// LayerNorm.  One CTA per row; the row is held in registers between the statistics and the
// normalisation (up to LN_VPT 16-byte vectors per thread), so x is read once.
// ------------------------------------------------------------------------------------------------
constexpr int LN_THREADS = 256;    // widest CTA; rows that fit use 128 threads so that more rows are in flight per SM
constexpr int LN_VPT = 4;          // vectors per thread -> rows up to 256 * 4 * 8 = 8192 elements of 16-bit data

// N consecutive affine parameters (gamma or beta) starting at column c, as floats, with 16-byte loads.
template <typename P, int N>
__device__ __forceinline__ void ld_params(const void* p, int c, float (&o)[N]) {
  const P* src = reinterpret_cast<const P*>(p) + c;
  if constexpr (sizeof(P) == 4) {
#pragma unroll
    for (int j = 0; j < N; j += 4) {
      float4 v = __ldg(reinterpret_cast<const float4*>(src + j));
      o[j] = v.x; o[j + 1] = v.y; o[j + 2] = v.z; o[j + 3] = v.w;
    }
  } else {
#pragma unroll
    for (int j = 0; j < N; j += 8) {
      Bytes16 v = *reinterpret_cast<const Bytes16*>(src + j);
      const P* e = reinterpret_cast<const P*>(&v);
#pragma unroll
      for (int q = 0; q < 8 && j + q < N; ++q) o[j + q] = to_f32<P>(e[q]);
    }
  }
}

// Optional quantised output of the forward kernel (all pointers may be null).
struct LnQuant {
  uint8_t* y8;             // [rows, cols] e4m3 copy of the output
  float* scale;            // quantisation scale (read; rewritten from amax_in when that is given)
  const float* amax_in;    // max|y| from an earlier pass: the scale is derived from it by the power-of-two rule
  float* amax_out;         // receives max|y| (zeroed by the host wrapper)
  float* scale_inv_out;    // receives 1 / scale
};

template <typename T, typename P, int THREADS>
__global__ void __launch_bounds__(THREADS) layernorm_fwd_kernel(const T* __restrict__ x, const void* __restrict__ gamma,
                                                                 const void* __restrict__ beta, T* __restrict__ y,
                                                                 float* __restrict__ mean_out, float* __restrict__ rstd_out, int rows,
                                                                 int cols, float eps, LnQuant q) {
  __shared__ float red[32];
  __shared__ float stat[2];
  constexpr int N = 16 / sizeof(T);
  const int nvec = cols / N;
  // Optional e4m3 copy of the output (quantised from the values as rounded to T, i.e. the bits a separate
  // cast of y would produce) and / or max|y|.
  float q_scale = 1.0f;
  if (q.scale != nullptr) {
    q_scale = *q.scale;
    if (q.amax_in != nullptr) {
      const float a = *q.amax_in;
      if ((a > 0.0f) && !isinf(a) && !isnan(a)) q_scale = msamp_compute_scale(a, q_scale, 448.0f, 0);
      if (blockIdx.x == 0 && threadIdx.x == 0) *q.scale = q_scale;
    }
    if (q.scale_inv_out != nullptr && blockIdx.x == 0 && threadIdx.x == 0) *q.scale_inv_out = __frcp_rn(q_scale);
  }
  float amax = 0.0f;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* xr = x + (int64_t)row * cols;
    Bytes16 v[LN_VPT];
    float sum = 0.0f;
#pragma unroll
    for (int k = 0; k < LN_VPT; ++k) {
      int i = threadIdx.x + k * THREADS;
      if (i < nvec) {
        v[k] = reinterpret_cast<const Bytes16*>(xr)[i];
        const T* e = reinterpret_cast<const T*>(&v[k]);
#pragma unroll
        for (int j = 0; j < N; ++j) sum += to_f32<T>(e[j]);
      }
    }
    sum = block_sum(sum, red);
    if (threadIdx.x == 0) stat[0] = sum / cols;
    __syncthreads();
    const float mean = stat[0];
    float sq = 0.0f;
#pragma unroll
    for (int k = 0; k < LN_VPT; ++k) {
      int i = threadIdx.x + k * THREADS;
      if (i < nvec) {
        const T* e = reinterpret_cast<const T*>(&v[k]);
#pragma unroll
        for (int j = 0; j < N; ++j) {
          float d = to_f32<T>(e[j]) - mean;
          sq += d * d;
        }
      }
    }
    sq = block_sum(sq, red);
    if (threadIdx.x == 0) stat[1] = rsqrtf(sq / cols + eps);
    __syncthreads();
    const float rstd = stat[1];
    if (threadIdx.x == 0) {
      mean_out[row] = mean;
      rstd_out[row] = rstd;
    }
    T* yr = y + (int64_t)row * cols;
    uint8_t* y8r = q.y8 + (int64_t)row * cols;
#pragma unroll
    for (int k = 0; k < LN_VPT; ++k) {
      int i = threadIdx.x + k * THREADS;
      if (i < nvec) {
        const T* e = reinterpret_cast<const T*>(&v[k]);
        float g[N], b[N];
        ld_params<P, N>(gamma, i * N, g);
        if (beta) {
          ld_params<P, N>(beta, i * N, b);
        } else {
#pragma unroll
          for (int j = 0; j < N; ++j) b[j] = 0.0f;
        }
        Bytes16 o;
        T* oe = reinterpret_cast<T*>(&o);
#pragma unroll
        for (int j = 0; j < N; ++j) oe[j] = from_f32<T>((to_f32<T>(e[j]) - mean) * rstd * g[j] + b[j]);
        if (y != nullptr) reinterpret_cast<Bytes16*>(yr)[i] = o;
        if (q.amax_out != nullptr || q.y8 != nullptr) {
          uint16_t o8[N / 2];
#pragma unroll
          for (int j = 0; j < N; j += 2) {
            const float a0 = to_f32<T>(oe[j]), a1 = to_f32<T>(oe[j + 1]);
            amax = fmaxf(amax, fmaxf(abs_nan_to_inf(a0), abs_nan_to_inf(a1)));
            o8[j / 2] = f32x2_to_fp8x2<FMT_E4M3>(a0 * q_scale, a1 * q_scale);
          }
          if (q.y8 != nullptr) {
            if (N == 8) reinterpret_cast<Bytes8*>(y8r)[i] = *reinterpret_cast<Bytes8*>(o8);
            else        reinterpret_cast<uint32_t*>(y8r)[i] = *reinterpret_cast<uint32_t*>(o8);
          }
        }
      }
    }
    __syncthreads();
  }
  if (q.amax_out != nullptr) {
    amax = block_max(amax, red);
    if (threadIdx.x == 0) atomic_max_nonneg(q.amax_out, amax);
  }
}

// Block-wide sums of two values at once (one round of barriers); results valid in every thread.
__device__ __forceinline__ float2 block_sum2(float a, float b, float2* red) {
  a = warp_sum(a);
  b = warp_sum(b);
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  if (lane == 0) red[w] = make_float2(a, b);
  __syncthreads();
  const int nw = (blockDim.x + 31) >> 5;
  float2 v = (lane < nw) ? red[lane] : make_float2(0.0f, 0.0f);
  v.x = warp_sum(v.x);
  v.y = warp_sum(v.y);
  __syncthreads();
  return v;
}

// Backward: dx per row (+ the skip-connection gradient dres, + max|dx|); dgamma / dbeta partial sums per CTA (each
// thread owns fixed columns, whose gamma it keeps in registers for all rows), written to part[gridDim.x][2][cols] and
// reduced by a second kernel.  A CTA of 256 threads owns one row at a time and loads the next row's x, dy and dres
// while it works on the current one, so that two rows per CTA are in flight.
constexpr int LN_BWD_THREADS = 256;
template <typename T, typename P, int VPT>
__global__ void __launch_bounds__(LN_BWD_THREADS, (VPT <= 2 ? 2 : 1)) layernorm_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x,
                                                                          const void* __restrict__ gamma, const float* __restrict__ mean,
                                                                          const float* __restrict__ rstd, T* __restrict__ dx,
                                                                          float* __restrict__ part, int rows, int cols,
                                                                          const T* __restrict__ dres, float* amax_out) {
  __shared__ float2 red2[32];
  __shared__ float red[32];
  constexpr int N = 16 / sizeof(T);
  constexpr int THREADS = LN_BWD_THREADS;
  const int nvec = cols / N;
  float amax = 0.0f;
  float dg[VPT][N], db[VPT][N], gm[VPT][N];
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    int i = threadIdx.x + k * THREADS;
#pragma unroll
    for (int j = 0; j < N; ++j) dg[k][j] = db[k][j] = gm[k][j] = 0.0f;
    if (i < nvec) ld_params<P, N>(gamma, i * N, gm[k]);
  }
  Bytes16 vx[VPT], vd[VPT], vr[VPT], nx[VPT], nd[VPT], nr[VPT];
  float mu = 0.0f, rs = 0.0f, nmu = 0.0f, nrs = 0.0f;
  auto load_row = [&](int row, Bytes16 (&ox)[VPT], Bytes16 (&od)[VPT], Bytes16 (&orr)[VPT], float& omu, float& ors) {
    const Bytes16* xr = reinterpret_cast<const Bytes16*>(x + (int64_t)row * cols);
    const Bytes16* dyr = reinterpret_cast<const Bytes16*>(dy + (int64_t)row * cols);
    const Bytes16* rr = reinterpret_cast<const Bytes16*>(dres + (int64_t)row * cols);
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      int i = threadIdx.x + k * THREADS;
      if (i < nvec) {
        ox[k] = xr[i];
        od[k] = dyr[i];
        if (dres != nullptr) orr[k] = rr[i];
      }
    }
    omu = mean[row];
    ors = rstd[row];
  };
  int row = blockIdx.x;
  if (row < rows) load_row(row, vx, vd, vr, mu, rs);
  for (; row < rows; row += gridDim.x) {
    const int next = row + gridDim.x;
    if (next < rows) load_row(next, nx, nd, nr, nmu, nrs);
    float s1 = 0.0f, s2 = 0.0f;    // sum(g*dy), sum(g*dy*xhat)
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      int i = threadIdx.x + k * THREADS;
      if (i < nvec) {
        const T* ex = reinterpret_cast<const T*>(&vx[k]);
        const T* ed = reinterpret_cast<const T*>(&vd[k]);
#pragma unroll
        for (int j = 0; j < N; ++j) {
          float xh = (to_f32<T>(ex[j]) - mu) * rs;
          float d = to_f32<T>(ed[j]);
          float gd = d * gm[k][j];
          s1 += gd;
          s2 += gd * xh;
          dg[k][j] += d * xh;
          db[k][j] += d;
        }
      }
    }
    const float2 tot = block_sum2(s1, s2, red2);
    const float m1 = tot.x / cols, m2 = tot.y / cols;
    T* dxr = dx + (int64_t)row * cols;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      int i = threadIdx.x + k * THREADS;
      if (i < nvec) {
        const T* ex = reinterpret_cast<const T*>(&vx[k]);
        const T* ed = reinterpret_cast<const T*>(&vd[k]);
        const T* er = reinterpret_cast<const T*>(&vr[k]);
        Bytes16 o;
        T* oe = reinterpret_cast<T*>(&o);
#pragma unroll
        for (int j = 0; j < N; ++j) {
          float xh = (to_f32<T>(ex[j]) - mu) * rs;
          float gd = to_f32<T>(ed[j]) * gm[k][j];
          float r = rs * (gd - m1 - xh * m2);
          if (dres != nullptr) r += to_f32<T>(er[j]);    // gradient of the skip connection around the LayerNorm branch
          oe[j] = from_f32<T>(r);
          if (amax_out != nullptr) amax = fmaxf(amax, abs_nan_to_inf(to_f32<T>(oe[j])));
        }
        reinterpret_cast<Bytes16*>(dxr)[i] = o;
      }
    }
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      vx[k] = nx[k];
      vd[k] = nd[k];
      vr[k] = nr[k];
    }
    mu = nmu;
    rs = nrs;
  }
  if (amax_out != nullptr) {
    amax = block_max(amax, red);
    if (threadIdx.x == 0) atomic_max_nonneg(amax_out, amax);
  }
  float* pg = part + (int64_t)blockIdx.x * 2 * cols;
  float* pb = pg + cols;
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    int i = threadIdx.x + k * THREADS;
    if (i < nvec) {
#pragma unroll
      for (int j = 0; j < N; ++j) {
        pg[i * N + j] = dg[k][j];
        pb[i * N + j] = db[k][j];
      }
    }
  }
}

// LayerNorm backward for 16-bit rows, fed by bulk copies (cp.async.bulk, global -> shared, completion on an mbarrier).
// The register-prefetching kernel above keeps one row per CTA in flight beyond the current one, which at two resident
// CTAs per SM is about a third of the bytes HBM needs in flight (it ran at 2.1-2.8 TB/s); here one thread keeps
// LN_BULK_STAGES - 1 rows (x, dy and the skip-connection gradient) of every CTA on their way while the CTA works on the
// current one.  Each CTA takes a contiguous block of rows, whose mean / rstd it reads into shared memory once.
// Same arithmetic and outputs as layernorm_bwd_kernel.  A wait that gives up sets bit 16 of the device status word.
constexpr int LN_BULK_STAGES = 4;
constexpr int LN_BULK_MAX_ROWS = 512;    // rows per CTA whose statistics fit the static shared arrays
template <typename T, typename P, int VPT>
__global__ void __launch_bounds__(LN_BWD_THREADS, 2)
layernorm_bwd_bulk_kernel(const T* __restrict__ dy, const T* __restrict__ x, const void* __restrict__ gamma, const float* __restrict__ mean,
                          const float* __restrict__ rstd, T* __restrict__ dx, float* __restrict__ part, int rows, int cols,
                          const T* __restrict__ dres, float* amax_out, int rows_per_cta, unsigned int* status) {
  extern __shared__ __align__(128) uint8_t ln_ring[];
  __shared__ float2 red2[32];
  __shared__ float red[32];
  __shared__ float s_mean[LN_BULK_MAX_ROWS], s_rstd[LN_BULK_MAX_ROWS];
  __shared__ __align__(8) uint64_t bar_mem[LN_BULK_STAGES];
  __shared__ int abort_word;
  constexpr int N = 16 / sizeof(T);
  constexpr int THREADS = LN_BWD_THREADS;
  const int nvec = cols / N;
  const uint32_t row_bytes = (uint32_t)cols * (uint32_t)sizeof(T);
  const uint32_t stage_bytes = 3u * row_bytes;    // x | dy | dres
  const uint32_t ring = tc5::smem_u32(ln_ring);
  const uint32_t bars = tc5::smem_u32(bar_mem);
  volatile int* abort_flag = &abort_word;
  const int r0 = blockIdx.x * rows_per_cta;
  const int n = min(rows - r0, rows_per_cta);    // >= 1: the grid is sized from rows_per_cta
  if (threadIdx.x == 0) {
    for (int s = 0; s < LN_BULK_STAGES; ++s) tc5::mbar_init(bars + 8u * s, 1);
    abort_word = 0;
    tc5::mbar_fence_init();
  }
  for (int i = threadIdx.x; i < n; i += THREADS) {
    s_mean[i] = mean[r0 + i];
    s_rstd[i] = rstd[r0 + i];
  }
  __syncthreads();
  auto issue = [&](int j) {    // thread 0: bring row r0 + j into stage j % LN_BULK_STAGES
    const uint32_t b = bars + 8u * (uint32_t)(j % LN_BULK_STAGES);
    const uint32_t dst = ring + (uint32_t)(j % LN_BULK_STAGES) * stage_bytes;
    const int64_t off = (int64_t)(r0 + j) * cols;
    tc5::mbar_arrive_expect_tx(b, (dres != nullptr ? 3u : 2u) * row_bytes);
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(x + off),
                 "r"(row_bytes), "r"(b)
                 : "memory");
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst + row_bytes),
                 "l"(dy + off), "r"(row_bytes), "r"(b)
                 : "memory");
    if (dres != nullptr)
      asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst + 2u * row_bytes),
                   "l"(dres + off), "r"(row_bytes), "r"(b)
                   : "memory");
  };
  if (threadIdx.x == 0)
    for (int j = 0; j < LN_BULK_STAGES - 1 && j < n; ++j) issue(j);
  float amax = 0.0f;
  float dg[VPT][N], db[VPT][N], gm[VPT][N];
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    int i = threadIdx.x + k * THREADS;
#pragma unroll
    for (int j = 0; j < N; ++j) dg[k][j] = db[k][j] = gm[k][j] = 0.0f;
    if (i < nvec) ld_params<P, N>(gamma, i * N, gm[k]);
  }
  bool ok = true;
  for (int it = 0; it < n; ++it) {
    // every thread has finished row it - 1: its stage takes row it + LN_BULK_STAGES - 1.  Also the place where the CTA
    // agrees to stop after a wait that gave up.
    if (__syncthreads_or(!ok)) break;
    if (threadIdx.x == 0 && it + LN_BULK_STAGES - 1 < n) issue(it + LN_BULK_STAGES - 1);
    const int st = it % LN_BULK_STAGES;
    ok = tc5::mbar_wait(bars + 8u * (uint32_t)st, (uint32_t)(it / LN_BULK_STAGES) & 1u, abort_flag, status, 16u);
    const uint8_t* sx = ln_ring + (size_t)st * stage_bytes;
    const Bytes16* xs = reinterpret_cast<const Bytes16*>(sx);
    const Bytes16* ds = reinterpret_cast<const Bytes16*>(sx + row_bytes);
    const Bytes16* rs_ = reinterpret_cast<const Bytes16*>(sx + 2u * row_bytes);
    const float mu = s_mean[it], rs = s_rstd[it];
    Bytes16 vx[VPT], vd[VPT], vr[VPT];
    float s1 = 0.0f, s2 = 0.0f;    // sum(g*dy), sum(g*dy*xhat)
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      int i = threadIdx.x + k * THREADS;
      if (i < nvec) {
        vx[k] = xs[i];
        vd[k] = ds[i];
        if (dres != nullptr) vr[k] = rs_[i];
        const T* ex = reinterpret_cast<const T*>(&vx[k]);
        const T* ed = reinterpret_cast<const T*>(&vd[k]);
#pragma unroll
        for (int j = 0; j < N; ++j) {
          float xh = (to_f32<T>(ex[j]) - mu) * rs;
          float d = to_f32<T>(ed[j]);
          float gd = d * gm[k][j];
          s1 += gd;
          s2 += gd * xh;
          dg[k][j] += d * xh;
          db[k][j] += d;
        }
      }
    }
    const float2 tot = block_sum2(s1, s2, red2);
    const float m1 = tot.x / cols, m2 = tot.y / cols;
    T* dxr = dx + (int64_t)(r0 + it) * cols;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      int i = threadIdx.x + k * THREADS;
      if (i < nvec) {
        const T* ex = reinterpret_cast<const T*>(&vx[k]);
        const T* ed = reinterpret_cast<const T*>(&vd[k]);
        const T* er = reinterpret_cast<const T*>(&vr[k]);
        Bytes16 o;
        T* oe = reinterpret_cast<T*>(&o);
#pragma unroll
        for (int j = 0; j < N; ++j) {
          float xh = (to_f32<T>(ex[j]) - mu) * rs;
          float gd = to_f32<T>(ed[j]) * gm[k][j];
          float r = rs * (gd - m1 - xh * m2);
          if (dres != nullptr) r += to_f32<T>(er[j]);
          oe[j] = from_f32<T>(r);
          if (amax_out != nullptr) amax = fmaxf(amax, abs_nan_to_inf(to_f32<T>(oe[j])));
        }
        reinterpret_cast<Bytes16*>(dxr)[i] = o;
      }
    }
  }
  if (amax_out != nullptr) {
    amax = block_max(amax, red);
    if (threadIdx.x == 0) atomic_max_nonneg(amax_out, amax);
  }
  float* pg = part + (int64_t)blockIdx.x * 2 * cols;
  float* pb = pg + cols;
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    int i = threadIdx.x + k * THREADS;
    if (i < nvec) {
#pragma unroll
      for (int j = 0; j < N; ++j) {
        pg[i * N + j] = dg[k][j];
        pb[i * N + j] = db[k][j];
      }
    }
  }
}

template <typename T, typename P>
void launch_ln_bwd(int grid, cudaStream_t stream, const void* dy, const void* x, const void* gamma, const float* mean, const float* rstd,
                   void* dx, float* part, int rows, int cols, const void* dres, float* amax_out) {
  const int nvec = cols / (16 / (int)sizeof(T));
  const int vpt = (nvec + LN_BWD_THREADS - 1) / LN_BWD_THREADS;
  if (vpt <= 1)
    layernorm_bwd_kernel<T, P, 1><<<grid, LN_BWD_THREADS, 0, stream>>>((const T*)dy, (const T*)x, gamma, mean, rstd, (T*)dx, part, rows, cols, (const T*)dres, amax_out);
  else if (vpt == 2)
    layernorm_bwd_kernel<T, P, 2><<<grid, LN_BWD_THREADS, 0, stream>>>((const T*)dy, (const T*)x, gamma, mean, rstd, (T*)dx, part, rows, cols, (const T*)dres, amax_out);
  else
    layernorm_bwd_kernel<T, P, 4><<<grid, LN_BWD_THREADS, 0, stream>>>((const T*)dy, (const T*)x, gamma, mean, rstd, (T*)dx, part, rows, cols, (const T*)dres, amax_out);
}

// Column sums of the per-CTA partials: a block of 32 x 8 threads owns 32 columns; the 8 thread rows
// stride over the partials (coalesced 128-byte reads) and are combined through shared memory.
__global__ void __launch_bounds__(256) layernorm_reduce_kernel(const float* __restrict__ part, int nparts, int cols, void* dgamma,
                                                                void* dbeta, int pdtype) {
  __shared__ float sg[8][33], sb[8][33];
  const int cx = threadIdx.x & 31, ry = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + cx;
  float g = 0.0f, b = 0.0f;
  if (c < cols) {
    for (int i = ry; i < nparts; i += 8) {
      g += part[(int64_t)i * 2 * cols + c];
      b += part[(int64_t)i * 2 * cols + cols + c];
    }
  }
  sg[ry][cx] = g;
  sb[ry][cx] = b;
  __syncthreads();
  if (ry == 0 && c < cols) {
#pragma unroll
    for (int k = 1; k < 8; ++k) {
      g += sg[k][cx];
      b += sb[k][cx];
    }
    if (pdtype == DT_F32) {
      reinterpret_cast<float*>(dgamma)[c] = g;
      if (dbeta) reinterpret_cast<float*>(dbeta)[c] = b;
    } else if (pdtype == DT_BF16) {
      reinterpret_cast<__nv_bfloat16*>(dgamma)[c] = __float2bfloat16_rn(g);
      if (dbeta) reinterpret_cast<__nv_bfloat16*>(dbeta)[c] = __float2bfloat16_rn(b);
    } else {
      reinterpret_cast<__half*>(dgamma)[c] = __float2half_rn(g);
      if (dbeta) reinterpret_cast<__half*>(dbeta)[c] = __float2half_rn(b);
    }
  }
}

// ------------------------------------------------------------------------------------------------
// GeLU, tanh form: 0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3)))
// ------------------------------------------------------------------------------------------------
template <typename T, bool BWD>
__global__ void __launch_bounds__(256) gelu_kernel(const T* __restrict__ x, const T* __restrict__ dy, T* __restrict__ out, int64_t n) {
  constexpr int N = 16 / sizeof(T);
  int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  int64_t nv = n / N;
  for (int64_t i = tid; i < nv; i += stride) {
    Bytes16 vx = reinterpret_cast<const Bytes16*>(x)[i];
    Bytes16 vd;
    if (BWD) vd = reinterpret_cast<const Bytes16*>(dy)[i];
    const T* ex = reinterpret_cast<const T*>(&vx);
    const T* ed = reinterpret_cast<const T*>(&vd);
    Bytes16 o;
    T* oe = reinterpret_cast<T*>(&o);
#pragma unroll
    for (int j = 0; j < N; ++j) {
      float xv = to_f32<T>(ex[j]);
      oe[j] = from_f32<T>(BWD ? to_f32<T>(ed[j]) * gelu_grad_f(xv) : gelu_f(xv));
    }
    reinterpret_cast<Bytes16*>(out)[i] = o;
  }
  for (int64_t i = nv * N + tid; i < n; i += stride) {
    float xv = to_f32<T>(x[i]);
    out[i] = from_f32<T>(BWD ? to_f32<T>(dy[i]) * gelu_grad_f(xv) : gelu_f(xv));
  }
}

// ------------------------------------------------------------------------------------------------
// Softmax cross-entropy over [rows, vocab] logits, one CTA per row.
// Forward pass: loss[row] = logsumexp(logits) - logits[target]; lse saved.
// Backward pass (in place): logits <- (softmax(logits) - onehot(target)) * gscale[0] * (target valid).
// Rows whose target equals ignore_index contribute zero loss and zero gradient.
// ------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(512) xent_fwd_kernel(const T* __restrict__ logits, const int64_t* __restrict__ target,
                                                        float* __restrict__ loss, float* __restrict__ lse_out, int vocab,
                                                        int64_t row_stride, int64_t ignore_index) {
  __shared__ float red[32];
  constexpr int N = 16 / sizeof(T);
  const int row = blockIdx.x;
  const T* lr = logits + (int64_t)row * row_stride;
  const int nv = vocab / N;
  // online max / sum
  float m = -INFINITY, s = 0.0f;
  for (int i = threadIdx.x; i < nv; i += blockDim.x) {
    Bytes16 v = reinterpret_cast<const Bytes16*>(lr)[i];
    const T* e = reinterpret_cast<const T*>(&v);
    float lm = -INFINITY;
#pragma unroll
    for (int j = 0; j < N; ++j) lm = fmaxf(lm, to_f32<T>(e[j]));
    if (lm > m) {
      s *= __expf(m - lm);
      m = lm;
    }
#pragma unroll
    for (int j = 0; j < N; ++j) s += __expf(to_f32<T>(e[j]) - m);
  }
  for (int i = nv * N + threadIdx.x; i < vocab; i += blockDim.x) {
    float v = to_f32<T>(lr[i]);
    if (v > m) {
      s *= __expf(m - v);
      m = v;
    }
    s += __expf(v - m);
  }
  // combine (m, s) across the block: first the exact max, then the rescaled sums
  float mm = m;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mm = fmaxf(mm, __shfl_xor_sync(0xffffffffu, mm, o));
  __shared__ float wmax[32];
  if ((threadIdx.x & 31) == 0) wmax[threadIdx.x >> 5] = mm;
  __syncthreads();
  float bm = -INFINITY;
  for (int w = 0; w < (int)(blockDim.x >> 5); ++w) bm = fmaxf(bm, wmax[w]);
  float contrib = (m == -INFINITY) ? 0.0f : s * __expf(m - bm);
  float total = block_sum(contrib, red);
  if (threadIdx.x == 0) {
    float lse = bm + logf(total);
    lse_out[row] = lse;
    int64_t t = target[row];
    loss[row] = (t == ignore_index || t < 0 || t >= vocab) ? 0.0f : lse - to_f32<T>(lr[t]);
  }
}

template <typename T>
__global__ void __launch_bounds__(512) xent_bwd_kernel(T* __restrict__ logits, const int64_t* __restrict__ target,
                                                        const float* __restrict__ lse_in, const float* __restrict__ gscale, int vocab,
                                                        int64_t row_stride, int64_t ignore_index) {
  constexpr int N = 16 / sizeof(T);
  const int row = blockIdx.x;
  T* lr = logits + (int64_t)row * row_stride;
  const int64_t t = target[row];
  const bool valid = !(t == ignore_index || t < 0 || t >= vocab);
  const float gs = valid ? *gscale : 0.0f;
  const float lse = lse_in[row];
  const int nv = vocab / N;
  for (int i = threadIdx.x; i < nv; i += blockDim.x) {
    Bytes16 v = reinterpret_cast<const Bytes16*>(lr)[i];
    T* e = reinterpret_cast<T*>(&v);
#pragma unroll
    for (int j = 0; j < N; ++j) {
      int c = i * N + j;
      float pr = __expf(to_f32<T>(e[j]) - lse);
      e[j] = from_f32<T>((pr - ((valid && c == t) ? 1.0f : 0.0f)) * gs);
    }
    reinterpret_cast<Bytes16*>(lr)[i] = v;
  }
  for (int c = nv * N + threadIdx.x; c < vocab; c += blockDim.x) {
    float pr = __expf(to_f32<T>(lr[c]) - lse);
    lr[c] = from_f32<T>((pr - ((valid && c == t) ? 1.0f : 0.0f)) * gs);
  }
}

}    // namespace

// Launch `kernel<T, P, THREADS>` for the (activation dtype, parameter dtype) pair; parameters are either fp32 or of the
// activation dtype.
#define MSAMP_LN_DISPATCH(dtype, pdtype, T, P, ...)                                   \
  MSAMP_DISPATCH_HP(dtype, T, {                                                       \
    if ((pdtype) == DT_F32) { using P = float; __VA_ARGS__; }                          \
    else if ((pdtype) == (dtype)) { using P = T; __VA_ARGS__; }                        \
    else { msamp_set_error("layernorm: parameters must be fp32 or match the activation dtype"); return MSAMP_EDTYPE; } \
  })

template <typename T, typename P>
int launch_ln_bwd_bulk_p(int grid, size_t ring_bytes, cudaStream_t stream, const void* dy, const void* x, const void* gamma, const float* mean,
                         const float* rstd, void* dx, float* part, int rows, int cols, const void* dres, float* amax_out, int rpc) {
  const int vpt = (cols / 8 + LN_BWD_THREADS - 1) / LN_BWD_THREADS;
  unsigned int* status = msamp_device_status_ptr();
#define MSAMP_LN_BULK(VPT_)                                                                                                              \
  {                                                                                                                                      \
    auto kern = layernorm_bwd_bulk_kernel<T, P, VPT_>;                                                                                   \
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ring_bytes) != cudaSuccess) {                       \
      msamp_set_error("layernorm_bwd: cannot reserve %zu bytes of shared memory", ring_bytes);                                           \
      return MSAMP_ELAUNCH;                                                                                                              \
    }                                                                                                                                    \
    kern<<<grid, LN_BWD_THREADS, ring_bytes, stream>>>((const T*)dy, (const T*)x, gamma, mean, rstd, (T*)dx, part, rows, cols, (const T*)dres, \
                                                        amax_out, rpc, status);                                                          \
  }
  if (vpt <= 1) MSAMP_LN_BULK(1) else MSAMP_LN_BULK(2)
#undef MSAMP_LN_BULK
  return MSAMP_OK;
}
template <typename T>
int launch_ln_bwd_bulk(int pdtype, int grid, size_t ring_bytes, cudaStream_t stream, const void* dy, const void* x, const void* gamma,
                       const float* mean, const float* rstd, void* dx, float* part, int rows, int cols, const void* dres, float* amax_out,
                       int rpc) {
  const int own = sizeof(T) == 2 && std::is_same<T, __half>::value ? DT_F16 : DT_BF16;
  if (pdtype == DT_F32) return launch_ln_bwd_bulk_p<T, float>(grid, ring_bytes, stream, dy, x, gamma, mean, rstd, dx, part, rows, cols, dres, amax_out, rpc);
  if (pdtype == own) return launch_ln_bwd_bulk_p<T, T>(grid, ring_bytes, stream, dy, x, gamma, mean, rstd, dx, part, rows, cols, dres, amax_out, rpc);
  msamp_set_error("layernorm: parameters must be fp32 or match the activation dtype");
  return MSAMP_EDTYPE;
}

MSAMP_API int msamp_layernorm_max_cols(int dtype) { return LN_THREADS * LN_VPT * (dtype == DT_F32 ? 4 : 8); }

#define MSAMP_LN_ALIGNED(ptr) ((reinterpret_cast<uintptr_t>(ptr) & 15) == 0)

// y (may be null) receives LayerNorm(x) in the activation dtype.  y8 (may be null) receives its e4m3 copy,
// quantised with *q_scale; with amax_in non-null the scale is first derived from *amax_in by the
// power-of-two rule and stored to *q_scale; amax_out (nullable, cleared here) receives max|y|;
// scale_inv_out (nullable) receives 1 / scale.  With y and y8 both null the launch only produces the
// row statistics and max|y| (the first pass of in-time scaling).
MSAMP_API int msamp_layernorm_fwd_q(const void* x, const void* gamma, const void* beta, int dtype, int pdtype, void* y, float* mean,
                                    float* rstd, int rows, int cols, float eps, void* y8, float* q_scale, const float* amax_in,
                                    float* amax_out, float* scale_inv_out, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  MSAMP_REQUIRE(rows >= 0 && cols > 0, "layernorm: bad shape");
  MSAMP_REQUIRE(cols <= msamp_layernorm_max_cols(dtype) && cols % (dtype == DT_F32 ? 4 : 8) == 0,
                "layernorm: cols=%d must be a multiple of the 16-byte vector and at most %d", cols, msamp_layernorm_max_cols(dtype));
  MSAMP_REQUIRE(MSAMP_LN_ALIGNED(x) && MSAMP_LN_ALIGNED(y) && MSAMP_LN_ALIGNED(gamma) && MSAMP_LN_ALIGNED(beta) && MSAMP_LN_ALIGNED(y8),
                "layernorm: x, y, y8, gamma and beta must be 16-byte aligned");
  MSAMP_REQUIRE(y8 == nullptr || q_scale != nullptr, "layernorm: a quantised output needs its scale");
  if (amax_out) cudaMemsetAsync(amax_out, 0, sizeof(float), stream);
  if (rows == 0) return MSAMP_OK;
  LnQuant q;
  q.y8 = (uint8_t*)y8; q.scale = q_scale; q.amax_in = amax_in; q.amax_out = amax_out; q.scale_inv_out = scale_inv_out;
  const bool narrow = cols <= 128 * LN_VPT * (dtype == DT_F32 ? 4 : 8);
  int cap = msamp_sm_count() * (narrow ? 16 : 8);
  int grid = rows < cap ? rows : cap;
  MSAMP_LN_DISPATCH(dtype, pdtype, T, P, {
    if (narrow)
      layernorm_fwd_kernel<T, P, 128><<<grid, 128, 0, stream>>>((const T*)x, gamma, beta, (T*)y, mean, rstd, rows, cols, eps, q);
    else
      layernorm_fwd_kernel<T, P, 256><<<grid, 256, 0, stream>>>((const T*)x, gamma, beta, (T*)y, mean, rstd, rows, cols, eps, q);
  });
  return msamp_check_launch("msamp_layernorm_fwd");
}

MSAMP_API int msamp_layernorm_fwd(const void* x, const void* gamma, const void* beta, int dtype, int pdtype, void* y, float* mean,
                                  float* rstd, int rows, int cols, float eps, void* stream_) {
  return msamp_layernorm_fwd_q(x, gamma, beta, dtype, pdtype, y, mean, rstd, rows, cols, eps, nullptr, nullptr, nullptr, nullptr, nullptr,
                               stream_);
}

// part: scratch of msamp_layernorm_bwd_parts() * 2 * cols floats owned by the caller.
MSAMP_API int msamp_layernorm_bwd_parts() { return msamp_sm_count() * 4; }

// dres (nullable, [rows, cols] of the activation dtype) is added to dx: the gradient that reaches x through the skip
// connection around the LayerNorm branch.  amax_out (nullable, cleared here) receives max|dx| of the stored values.
MSAMP_API int msamp_layernorm_bwd_ex(const void* dy, const void* x, const void* gamma, int dtype, int pdtype, const float* mean,
                                     const float* rstd, void* dx, void* dgamma, void* dbeta, float* part, int rows, int cols,
                                     const void* dres, float* amax_out, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  MSAMP_REQUIRE(rows > 0 && cols > 0, "layernorm_bwd: bad shape");
  MSAMP_REQUIRE(cols <= msamp_layernorm_max_cols(dtype) && cols % (dtype == DT_F32 ? 4 : 8) == 0, "layernorm_bwd: unsupported cols=%d", cols);
  MSAMP_REQUIRE(MSAMP_LN_ALIGNED(dy) && MSAMP_LN_ALIGNED(x) && MSAMP_LN_ALIGNED(dx) && MSAMP_LN_ALIGNED(gamma) && MSAMP_LN_ALIGNED(dres),
                "layernorm_bwd: dy, x, dx, dres and gamma must be 16-byte aligned");
  if (amax_out) cudaMemsetAsync(amax_out, 0, sizeof(float), stream);
  int nparts = msamp_sm_count() * 2;    // two CTAs of 256 threads are resident per SM; never more than msamp_layernorm_bwd_parts()
  int grid = rows < nparts ? rows : nparts;
  // the bulk-copy kernel: 16-bit data, one or two vectors per thread, enough rows per CTA to fill its ring, statistics that
  // fit its shared arrays
  {
    const int rpc = (rows + nparts - 1) / nparts;
    const int nvec16 = cols / 8;
    const size_t ring_bytes = (size_t)LN_BULK_STAGES * 3 * cols * 2;
    if (dtype != DT_F32 && nvec16 <= 2 * LN_BWD_THREADS && rpc >= LN_BULK_STAGES && rpc <= LN_BULK_MAX_ROWS && ring_bytes <= 100 * 1024 &&
        (cols * 2) % 16 == 0) {
      const int grid_b = (rows + rpc - 1) / rpc;
      int rc = MSAMP_OK;
      if (dtype == DT_BF16) rc = launch_ln_bwd_bulk<__nv_bfloat16>(pdtype, grid_b, ring_bytes, stream, dy, x, gamma, mean, rstd, dx, part, rows, cols, dres, amax_out, rpc);
      else                  rc = launch_ln_bwd_bulk<__half>(pdtype, grid_b, ring_bytes, stream, dy, x, gamma, mean, rstd, dx, part, rows, cols, dres, amax_out, rpc);
      if (rc) return rc;
      layernorm_reduce_kernel<<<(cols + 31) / 32, 256, 0, stream>>>(part, grid_b, cols, dgamma, dbeta, pdtype);
      return msamp_check_launch("msamp_layernorm_bwd (bulk)");
    }
  }
  MSAMP_LN_DISPATCH(dtype, pdtype, T, P, { launch_ln_bwd<T, P>(grid, stream, dy, x, gamma, mean, rstd, dx, part, rows, cols, dres, amax_out); });
  layernorm_reduce_kernel<<<(cols + 31) / 32, 256, 0, stream>>>(part, grid, cols, dgamma, dbeta, pdtype);
  return msamp_check_launch("msamp_layernorm_bwd");
}

MSAMP_API int msamp_layernorm_bwd(const void* dy, const void* x, const void* gamma, int dtype, int pdtype, const float* mean,
                                  const float* rstd, void* dx, void* dgamma, void* dbeta, float* part, int rows, int cols,
                                  void* stream_) {
  return msamp_layernorm_bwd_ex(dy, x, gamma, dtype, pdtype, mean, rstd, dx, dgamma, dbeta, part, rows, cols, nullptr, nullptr, stream_);
}

// ---- allocation-free LayerNorm backward ---------------------------------------------------------
// Scratch for the per-CTA partial sums of dgamma / dbeta lives in this file-scope array instead of
// caller-provided memory.  Every device that loads the library holds these 4 MiB until exit.
static __device__ __align__(256) float g_ln_static_part[MSAMP_LN_STATIC_PARTS * 2 * MSAMP_LN_STATIC_MAX_COLS];

MSAMP_API int msamp_layernorm_bwd_static(const void* dy, const void* x, const void* gamma, int dtype, int pdtype, const float* mean,
                                         const float* rstd, void* dx, void* dgamma, void* dbeta, int rows, int cols, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  MSAMP_REQUIRE(rows > 0 && cols > 0, "layernorm_bwd_static: bad shape");
  if (cols > MSAMP_LN_STATIC_MAX_COLS) {
    msamp_set_error("layernorm_bwd_static: cols=%d exceeds the static scratch capacity of %d columns; use msamp_layernorm_bwd "
                    "with caller-provided scratch", cols, MSAMP_LN_STATIC_MAX_COLS);
    return MSAMP_ECAPACITY;
  }
  MSAMP_REQUIRE(cols <= msamp_layernorm_max_cols(dtype) && cols % (dtype == DT_F32 ? 4 : 8) == 0,
                "layernorm_bwd_static: unsupported cols=%d", cols);
  MSAMP_REQUIRE(MSAMP_LN_ALIGNED(dy) && MSAMP_LN_ALIGNED(x) && MSAMP_LN_ALIGNED(dx) && MSAMP_LN_ALIGNED(gamma),
                "layernorm_bwd_static: dy, x, dx and gamma must be 16-byte aligned");
  // In host code the array's name is only a handle; the device address has to be asked for, once
  // per device, with that device current.
  static std::atomic<float*> scratch_of_device[64];    // zero-initialised; two threads racing here store the same address
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    msamp_set_error("layernorm_bwd_static: cannot identify the current device");
    return MSAMP_EINVAL;
  }
  if (scratch_of_device[dev].load(std::memory_order_acquire) == nullptr) {
    float* ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress((void**)&ptr, g_ln_static_part);
    if (e != cudaSuccess || ptr == nullptr) {
      msamp_set_error("layernorm_bwd_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
      return MSAMP_ELAUNCH;
    }
    scratch_of_device[dev].store(ptr, std::memory_order_release);
  }
  float* part = scratch_of_device[dev].load(std::memory_order_acquire);
  const int grid = rows < MSAMP_LN_STATIC_PARTS ? rows : MSAMP_LN_STATIC_PARTS;
  // Each of the `grid` CTAs overwrites its whole slice of the scratch and the reduction reads
  // exactly those slices, so leftovers of an earlier call never need clearing.
  MSAMP_LN_DISPATCH(dtype, pdtype, T, P, { launch_ln_bwd<T, P>(grid, stream, dy, x, gamma, mean, rstd, dx, part, rows, cols, nullptr, nullptr); });
  layernorm_reduce_kernel<<<(cols + 31) / 32, 256, 0, stream>>>(part, grid, cols, dgamma, dbeta, pdtype);
  return msamp_check_launch("msamp_layernorm_bwd_static");
}

MSAMP_API int msamp_gelu_fwd(const void* x, void* y, int64_t n, int dtype, void* stream_) {
  if (n <= 0) return MSAMP_OK;
  MSAMP_REQUIRE(((uintptr_t)x & 15) == 0 && ((uintptr_t)y & 15) == 0, "gelu: pointers must be 16-byte aligned");
  int grid = msamp_grid_for((n + 7) / 8, 256, 8);
  MSAMP_DISPATCH_HP(dtype, T, { gelu_kernel<T, false><<<grid, 256, 0, (cudaStream_t)stream_>>>((const T*)x, nullptr, (T*)y, n); });
  return msamp_check_launch("msamp_gelu_fwd");
}

MSAMP_API int msamp_gelu_bwd(const void* x, const void* dy, void* dx, int64_t n, int dtype, void* stream_) {
  if (n <= 0) return MSAMP_OK;
  MSAMP_REQUIRE(((uintptr_t)x & 15) == 0 && ((uintptr_t)dy & 15) == 0 && ((uintptr_t)dx & 15) == 0, "gelu: pointers must be 16-byte aligned");
  int grid = msamp_grid_for((n + 7) / 8, 256, 8);
  MSAMP_DISPATCH_HP(dtype, T, { gelu_kernel<T, true><<<grid, 256, 0, (cudaStream_t)stream_>>>((const T*)x, (const T*)dy, (T*)dx, n); });
  return msamp_check_launch("msamp_gelu_bwd");
}

MSAMP_API int msamp_xent_fwd(const void* logits, const int64_t* target, float* loss, float* lse, int rows, int vocab, int64_t row_stride,
                             int64_t ignore_index, int dtype, void* stream_) {
  if (rows <= 0) return MSAMP_OK;
  MSAMP_REQUIRE(((uintptr_t)logits & 15) == 0 && (row_stride * (dtype == DT_F32 ? 4 : 2)) % 16 == 0, "xent: rows must be 16-byte aligned");
  MSAMP_DISPATCH_HP(dtype, T, {
    xent_fwd_kernel<T><<<rows, 512, 0, (cudaStream_t)stream_>>>((const T*)logits, target, loss, lse, vocab, row_stride, ignore_index);
  });
  return msamp_check_launch("msamp_xent_fwd");
}

MSAMP_API int msamp_xent_bwd(void* logits, const int64_t* target, const float* lse, const float* gscale, int rows, int vocab,
                             int64_t row_stride, int64_t ignore_index, int dtype, void* stream_) {
  if (rows <= 0) return MSAMP_OK;
  MSAMP_REQUIRE(((uintptr_t)logits & 15) == 0 && (row_stride * (dtype == DT_F32 ? 4 : 2)) % 16 == 0, "xent: rows must be 16-byte aligned");
  MSAMP_DISPATCH_HP(dtype, T, {
    xent_bwd_kernel<T><<<rows, 512, 0, (cudaStream_t)stream_>>>((T*)logits, target, lse, gscale, vocab, row_stride, ignore_index);
  });
  return msamp_check_launch("msamp_xent_bwd");
}
