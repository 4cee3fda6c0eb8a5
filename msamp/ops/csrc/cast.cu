// Cast family: amax, high precision -> FP8 (optionally with a transposed copy), FP8 -> high
// precision, byte transpose and the vectorised scale update.  All kernels are bandwidth bound;
// they use 16-byte accesses when the pointers allow it and a grid sized from the SM count.
#include "common.cuh"

namespace {

constexpr int kThreads = 256;

template <typename T>
struct VecOf {
  static constexpr int N = 16 / sizeof(T);
};

// ---- amax (+ optional scale update by the last block to finish) -------------------------------
template <typename T, bool VEC>
__global__ void __launch_bounds__(kThreads) amax_kernel(const T* __restrict__ x, int64_t n, float* amax, float* scale,
                                                         float* scale_inv, float fp_max, int margin, float prescale,
                                                         unsigned int* counter) {
  __shared__ float red[32];
  float m = 0.0f;
  int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  if (VEC) {
    constexpr int N = VecOf<T>::N;
    int64_t nv = n / N;
    const Bytes16* xv = reinterpret_cast<const Bytes16*>(x);
    // four independent 16-byte loads per thread and iteration keep enough bytes in flight for HBM3e
    for (int64_t i = tid; i < nv; i += 4 * stride) {
      Bytes16 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (i + u * stride < nv) v[u] = xv[i + u * stride];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (i + u * stride < nv) {
          const T* e = reinterpret_cast<const T*>(&v[u]);
#pragma unroll
          for (int j = 0; j < N; ++j) m = fmaxf(m, abs_nan_to_inf(to_f32<T>(e[j])));
        }
      }
    }
    for (int64_t i = nv * N + tid; i < n; i += stride) m = fmaxf(m, abs_nan_to_inf(to_f32<T>(x[i])));
  } else {
    for (int64_t i = tid; i < n; i += stride) m = fmaxf(m, abs_nan_to_inf(to_f32<T>(x[i])));
  }
  m = block_max(m, red);
  if (threadIdx.x == 0) {
    atomic_max_nonneg(amax, m);
    if (counter != nullptr) {
      __threadfence();
      unsigned int done = atomicAdd(counter, 1u);
      if (done == gridDim.x - 1) {
        // Every other block has published its maximum: derive the scale once.
        __threadfence();
        float a = *(volatile float*)amax;
        float s = msamp_compute_scale(a, *scale, fp_max, margin) * prescale;
        *scale = s;
        *scale_inv = __frcp_rn(s);
        *counter = 0;    // ready for the next launch on this stream
      }
    }
  }
}

// ---- high precision -> fp8 ------------------------------------------------------------------------
// ACT == 1 quantises gelu(x) (rounded to T first, i.e. the bits a separate GeLU kernel would have stored)
// instead of x; amax then refers to gelu(x) as well.
template <typename T, int ACT>
__device__ __forceinline__ float cast_pre(T e) {
  float a = to_f32<T>(e);
  if (ACT == 1) a = to_f32<T>(from_f32<T>(gelu_f(a)));
  return a;
}

template <typename T, int FMT, bool VEC, int ACT>
__global__ void __launch_bounds__(kThreads) cast_to_fp8_kernel(const T* __restrict__ x, uint8_t* __restrict__ out, int64_t n,
                                                                float* scale_ptr, float* amax, float* scale_inv_out,
                                                                const float* amax_in, float fp_max, float prescale, int rescale) {
  __shared__ float red[32];
  float scale = *scale_ptr;
  float logical_scale = scale;
  if (amax_in != nullptr && rescale) {
    // Re-quantisation of a tensor that is stored as x * s_old: *scale_ptr holds 1 / s_old and *amax_in
    // holds max|x|.  The payload is multiplied by s_new / s_old where s_new follows the power-of-two
    // rule; scale_inv_out receives 1 / s_new and *scale_ptr is left alone.
    logical_scale = msamp_compute_scale(*amax_in, 1.0f, fp_max, 0);
    scale = logical_scale * scale;
  } else if (amax_in != nullptr) {
    // In-time scaling from an amax that an earlier kernel produced (e.g. a GEMM epilogue): every
    // thread derives the same scale; one thread publishes it. When amax is unusable the old
    // scale is kept, so the concurrent read of *scale_ptr by other blocks sees a value that the
    // write does not change.
    float a = *amax_in;
    if ((a > 0.0f) && !isinf(a) && !isnan(a)) scale = msamp_compute_scale(a, scale, fp_max, 0) * prescale;
    logical_scale = scale;
    if (blockIdx.x == 0 && threadIdx.x == 0) *scale_ptr = scale;
  }
  if (scale_inv_out != nullptr && blockIdx.x == 0 && threadIdx.x == 0) *scale_inv_out = __frcp_rn(logical_scale);
  float m = 0.0f;
  int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  if (VEC) {
    constexpr int N = VecOf<T>::N;    // 8 (16-bit) or 4 (fp32) inputs -> N bytes out
    int64_t nv = n / N;
    const Bytes16* xv = reinterpret_cast<const Bytes16*>(x);
    for (int64_t i = tid; i < nv; i += 4 * stride) {
      Bytes16 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (i + u * stride < nv) v[u] = xv[i + u * stride];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (i + u * stride < nv) {
          const T* e = reinterpret_cast<const T*>(&v[u]);
          uint16_t o[N / 2];
#pragma unroll
          for (int j = 0; j < N; j += 2) {
            float a = cast_pre<T, ACT>(e[j]), b = cast_pre<T, ACT>(e[j + 1]);
            m = fmaxf(m, fmaxf(abs_nan_to_inf(a), abs_nan_to_inf(b)));
            o[j / 2] = f32x2_to_fp8x2<FMT>(a * scale, b * scale);
          }
          if (N == 8) {
            reinterpret_cast<Bytes8*>(out)[i + u * stride] = *reinterpret_cast<Bytes8*>(o);
          } else {
            reinterpret_cast<uint32_t*>(out)[i + u * stride] = *reinterpret_cast<uint32_t*>(o);
          }
        }
      }
    }
    for (int64_t i = nv * N + tid; i < n; i += stride) {
      float a = cast_pre<T, ACT>(x[i]);
      m = fmaxf(m, abs_nan_to_inf(a));
      out[i] = f32_to_fp8<FMT>(a * scale);
    }
  } else {
    for (int64_t i = tid; i < n; i += stride) {
      float a = cast_pre<T, ACT>(x[i]);
      m = fmaxf(m, abs_nan_to_inf(a));
      out[i] = f32_to_fp8<FMT>(a * scale);
    }
  }
  if (amax != nullptr) {
    m = block_max(m, red);
    if (threadIdx.x == 0) atomic_max_nonneg(amax, m);
  }
}

// ---- high precision [rows, cols] -> fp8 with the column sums of the input -------------------------
// Used for the output gradient of a linear layer: the bias gradient falls out of the pass that
// quantises dy.  A CTA owns a slab of 256 16-byte column vectors and walks down the rows, four rows in
// flight per thread; every thread keeps the partial sums of its own columns in registers and adds
// them to colsum (fp32, zeroed by the caller) once at the end.  cols must be a multiple of 16 bytes.
constexpr int kColsumRows = 6;    // rows in flight per thread
template <typename T, int FMT>
__global__ void __launch_bounds__(kThreads, 4) cast_rows_colsum_kernel(const T* __restrict__ x, uint8_t* __restrict__ out, int rows, int cols,
                                                                        float* scale_ptr, float* amax, float* scale_inv_out,
                                                                        float* __restrict__ colsum, const float* amax_in, float fp_max) {
  __shared__ float red[32];
  constexpr int N = VecOf<T>::N;
  constexpr int U = kColsumRows;
  float scale = *scale_ptr;
  if (amax_in != nullptr) {    // in-time scaling from an amax that the producer of x already reduced
    const float a = *amax_in;
    if ((a > 0.0f) && !isinf(a) && !isnan(a)) scale = msamp_compute_scale(a, scale, fp_max, 0);
    if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) *scale_ptr = scale;
  }
  if (scale_inv_out != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) *scale_inv_out = __frcp_rn(scale);
  const int cv = cols / N;                                   // vectors per row
  const int vec = blockIdx.y * kThreads + threadIdx.x;       // this thread's column vector
  const int gx = (int)gridDim.x;
  float m = 0.0f;
  float cs[N];
#pragma unroll
  for (int j = 0; j < N; ++j) cs[j] = 0.0f;
  if (vec < cv) {
    const Bytes16* xv = reinterpret_cast<const Bytes16*>(x);
    for (int r = blockIdx.x; r < rows; r += U * gx) {
      Bytes16 v[U];
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (r + u * gx < rows) v[u] = xv[(int64_t)(r + u * gx) * cv + vec];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int rr = r + u * gx;
        if (rr < rows) {
          const T* e = reinterpret_cast<const T*>(&v[u]);
          uint16_t o[N / 2];
#pragma unroll
          for (int j = 0; j < N; j += 2) {
            float a = to_f32<T>(e[j]), b = to_f32<T>(e[j + 1]);
            m = fmaxf(m, fmaxf(abs_nan_to_inf(a), abs_nan_to_inf(b)));
            cs[j] += a;
            cs[j + 1] += b;
            o[j / 2] = f32x2_to_fp8x2<FMT>(a * scale, b * scale);
          }
          if (N == 8) {
            reinterpret_cast<Bytes8*>(out)[(int64_t)rr * cv + vec] = *reinterpret_cast<Bytes8*>(o);
          } else {
            reinterpret_cast<uint32_t*>(out)[(int64_t)rr * cv + vec] = *reinterpret_cast<uint32_t*>(o);
          }
        }
      }
    }
#pragma unroll
    for (int j = 0; j < N; ++j) atomicAdd(colsum + (int64_t)vec * N + j, cs[j]);
  }
  if (amax != nullptr) {
    m = block_max(m, red);
    if (threadIdx.x == 0) atomic_max_nonneg(amax, m);
  }
}

// ---- fp8 -> high precision ------------------------------------------------------------------------
template <typename T, int FMT, bool VEC>
__global__ void __launch_bounds__(kThreads) cast_from_fp8_kernel(const uint8_t* __restrict__ in, T* __restrict__ out, int64_t n,
                                                                  const float* __restrict__ scale_inv_ptr) {
  const float si = *scale_inv_ptr;
  int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  if (VEC) {
    constexpr int N = VecOf<T>::N;
    int64_t nv = n / N;
    for (int64_t i = tid; i < nv; i += stride) {
      uint8_t b[N];
      if (N == 8) {
        *reinterpret_cast<Bytes8*>(b) = reinterpret_cast<const Bytes8*>(in)[i];
      } else {
        *reinterpret_cast<uint32_t*>(b) = reinterpret_cast<const uint32_t*>(in)[i];
      }
      Bytes16 o;
      T* e = reinterpret_cast<T*>(&o);
#pragma unroll
      for (int j = 0; j < N; ++j) e[j] = from_f32<T>(fp8_to_f32<FMT>(b[j]) * si);
      reinterpret_cast<Bytes16*>(out)[i] = o;
    }
    for (int64_t i = nv * N + tid; i < n; i += stride) out[i] = from_f32<T>(fp8_to_f32<FMT>(in[i]) * si);
  } else {
    for (int64_t i = tid; i < n; i += stride) out[i] = from_f32<T>(fp8_to_f32<FMT>(in[i]) * si);
  }
}

// ---- cast + transpose -----------------------------------------------------------------------------
// One CTA converts a tile of 128 rows x 64 columns.  The row-major copy is written straight from
// registers (64-byte runs); the transposed copy goes through shared memory and leaves in 128-byte
// runs.  The shared tile is stored transposed with a row stride of 33 words, which makes the
// word reads of the second phase conflict free.
constexpr int kTileR = 128;
constexpr int kTileC = 64;
constexpr int kCtStride = 132;    // bytes per transposed row in shared memory

template <typename T, int FMT, bool WRITE_ROWMAJOR>
__global__ void __launch_bounds__(kThreads) cast_transpose_kernel(const T* __restrict__ x, uint8_t* __restrict__ out,
                                                                   uint8_t* __restrict__ out_t, int rows, int cols,
                                                                   const float* __restrict__ scale_ptr, float* amax,
                                                                   float* scale_inv_out, const float* __restrict__ amax_in,
                                                                   float fp_max, bool aligned, float* __restrict__ colsum) {
  __shared__ __align__(16) uint8_t tile_t[kTileC * kCtStride];    // [c][r]
  __shared__ float red[32];
  __shared__ float colred[kThreads / 32][kTileC];    // per-warp column sums of the tile (only with colsum)
  float scale = *scale_ptr;
  float logical_scale = scale;
  if (amax_in != nullptr) {
    // Re-quantisation of a tensor that is stored as x * s_old: *scale_ptr holds 1 / s_old and
    // *amax_in holds max|x|.  The payload is multiplied by s_new / s_old where s_new follows the
    // power-of-two rule; scale_inv_out receives 1 / s_new.
    logical_scale = msamp_compute_scale(*amax_in, 1.0f, fp_max, 0);
    scale = logical_scale * scale;
  }
  if (scale_inv_out != nullptr && blockIdx.x == 0 && threadIdx.x == 0) *scale_inv_out = __frcp_rn(logical_scale);
  const int tiles_c = (cols + kTileC - 1) / kTileC;
  const int tiles_r = (rows + kTileR - 1) / kTileR;
  const int64_t ntiles = (int64_t)tiles_c * tiles_r;
  float m = 0.0f;
  for (int64_t t = blockIdx.x; t < ntiles; t += gridDim.x) {
    const int r0 = (int)(t / tiles_c) * kTileR;
    const int c0 = (int)(t % tiles_c) * kTileC;
    const bool full = aligned && (r0 + kTileR <= rows) && (c0 + kTileC <= cols);
    if (full) {
      // 8 threads cover the 64 columns (8 each); a thread converts 4 consecutive rows and transposes its
      // 4 x 8 bytes in registers, so the shared tile is written with 32-bit stores.
      const int rg = threadIdx.x >> 3, cc = (threadIdx.x & 7) * 8;
      uint32_t w[4][2];
      float cs[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int r = rg * 4 + i;
        const T* src = x + (int64_t)(r0 + r) * cols + c0 + cc;
        T e[8];
        if constexpr (sizeof(T) == 2) {
          *reinterpret_cast<Bytes16*>(e) = *reinterpret_cast<const Bytes16*>(src);
        } else {
          *reinterpret_cast<Bytes16*>(e) = *reinterpret_cast<const Bytes16*>(src);
          *reinterpret_cast<Bytes16*>(e + 4) = *reinterpret_cast<const Bytes16*>(src + 4);
        }
        uint16_t q[4];
#pragma unroll
        for (int j = 0; j < 8; j += 2) {
          float a0 = to_f32<T>(e[j]), a1 = to_f32<T>(e[j + 1]);
          m = fmaxf(m, fmaxf(abs_nan_to_inf(a0), abs_nan_to_inf(a1)));
          cs[j] += a0;
          cs[j + 1] += a1;
          q[j / 2] = f32x2_to_fp8x2<FMT>(a0 * scale, a1 * scale);
        }
        w[i][0] = (uint32_t)q[0] | ((uint32_t)q[1] << 16);
        w[i][1] = (uint32_t)q[2] | ((uint32_t)q[3] << 16);
        if (WRITE_ROWMAJOR) {
          Bytes8 o;
          o.w[0] = w[i][0];
          o.w[1] = w[i][1];
          *reinterpret_cast<Bytes8*>(out + (int64_t)(r0 + r) * cols + c0 + cc) = o;
        }
      }
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        // 4 x 4 byte transpose: column word j holds rows 4*rg .. 4*rg+3 of column cc + 4*h + j
        const uint32_t a = __byte_perm(w[0][h], w[1][h], 0x5140), b2 = __byte_perm(w[2][h], w[3][h], 0x5140);
        const uint32_t c = __byte_perm(w[0][h], w[1][h], 0x7362), d = __byte_perm(w[2][h], w[3][h], 0x7362);
        uint32_t* base = reinterpret_cast<uint32_t*>(tile_t);
        base[(cc + 4 * h + 0) * (kCtStride / 4) + rg] = __byte_perm(a, b2, 0x5410);
        base[(cc + 4 * h + 1) * (kCtStride / 4) + rg] = __byte_perm(a, b2, 0x7632);
        base[(cc + 4 * h + 2) * (kCtStride / 4) + rg] = __byte_perm(c, d, 0x5410);
        base[(cc + 4 * h + 3) * (kCtStride / 4) + rg] = __byte_perm(c, d, 0x7632);
      }
      if (colsum != nullptr) {
        // lanes l, l+8, l+16, l+24 hold the same eight columns for different rows
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          cs[j] += __shfl_xor_sync(0xffffffffu, cs[j], 8);
          cs[j] += __shfl_xor_sync(0xffffffffu, cs[j], 16);
        }
        if ((threadIdx.x & 31) < 8) {
#pragma unroll
          for (int j = 0; j < 8; ++j) colred[threadIdx.x >> 5][cc + j] = cs[j];
        }
      }
      __syncthreads();
      if (colsum != nullptr && threadIdx.x < kTileC) {
        float acc = 0.0f;
#pragma unroll
        for (int wv = 0; wv < kThreads / 32; ++wv) acc += colred[wv][threadIdx.x];
        atomicAdd(colsum + c0 + threadIdx.x, acc);
      }
      {
        // 4 threads cover one transposed row of 128 bytes (32 each)
        const int c = threadIdx.x >> 2, rr = (threadIdx.x & 3) * 32;
        Bytes16 o0, o1;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          o0.w[j] = *reinterpret_cast<const uint32_t*>(&tile_t[c * kCtStride + rr + 4 * j]);
          o1.w[j] = *reinterpret_cast<const uint32_t*>(&tile_t[c * kCtStride + rr + 16 + 4 * j]);
        }
        uint8_t* dst = out_t + (int64_t)(c0 + c) * rows + r0 + rr;
        *reinterpret_cast<Bytes16*>(dst) = o0;
        *reinterpret_cast<Bytes16*>(dst + 16) = o1;
      }
      __syncthreads();
    } else {
      for (int i = threadIdx.x; i < kTileR * kTileC; i += blockDim.x) {
        const int r = i / kTileC, c = i % kTileC;
        uint8_t q = 0;
        if (r0 + r < rows && c0 + c < cols) {
          float a = to_f32<T>(x[(int64_t)(r0 + r) * cols + c0 + c]);
          m = fmaxf(m, abs_nan_to_inf(a));
          if (colsum != nullptr) atomicAdd(colsum + c0 + c, a);
          q = f32_to_fp8<FMT>(a * scale);
          if (WRITE_ROWMAJOR) out[(int64_t)(r0 + r) * cols + c0 + c] = q;
        }
        tile_t[c * kCtStride + r] = q;
      }
      __syncthreads();
      for (int i = threadIdx.x; i < kTileR * kTileC; i += blockDim.x) {
        const int c = i / kTileR, r = i % kTileR;
        if (r0 + r < rows && c0 + c < cols) out_t[(int64_t)(c0 + c) * rows + r0 + r] = tile_t[c * kCtStride + r];
      }
      __syncthreads();
    }
  }
  if (amax != nullptr) {
    m = block_max(m, red);
    if (threadIdx.x == 0) atomic_max_nonneg(amax, m);
  }
}

// ---- byte transpose ---------------------------------------------------------------------------------
constexpr int kTile = 64;
constexpr int kTStride = kTile + 4;    // bytes; keeps 4-byte alignment and spreads banks
__global__ void __launch_bounds__(kThreads) transpose_bytes_kernel(const uint8_t* __restrict__ in, uint8_t* __restrict__ out,
                                                                    int rows, int cols, bool aligned) {
  __shared__ __align__(16) uint8_t tile_t[kTile * kTStride];
  const int tiles_c = (cols + kTile - 1) / kTile;
  const int tiles_r = (rows + kTile - 1) / kTile;
  const int64_t ntiles = (int64_t)tiles_c * tiles_r;
  for (int64_t t = blockIdx.x; t < ntiles; t += gridDim.x) {
    const int r0 = (int)(t / tiles_c) * kTile;
    const int c0 = (int)(t % tiles_c) * kTile;
    const bool full = aligned && (r0 + kTile <= rows) && (c0 + kTile <= cols);
    if (full) {
      // 4 threads cover a 64-byte row (16 bytes each); 64 rows in one pass.
      const int r = threadIdx.x >> 2, cc = (threadIdx.x & 3) * 16;
      Bytes16 v = *reinterpret_cast<const Bytes16*>(in + (int64_t)(r0 + r) * cols + c0 + cc);
      const uint8_t* b = reinterpret_cast<const uint8_t*>(&v);
#pragma unroll
      for (int j = 0; j < 16; ++j) tile_t[(cc + j) * kTStride + r] = b[j];
      __syncthreads();
      Bytes16 o;
#pragma unroll
      for (int j = 0; j < 4; ++j) o.w[j] = *reinterpret_cast<const uint32_t*>(&tile_t[r * kTStride + cc + 4 * j]);
      *reinterpret_cast<Bytes16*>(out + (int64_t)(c0 + r) * rows + r0 + cc) = o;
      __syncthreads();
    } else {
      for (int i = threadIdx.x; i < kTile * kTile; i += blockDim.x) {
        const int r = i / kTile, c = i % kTile;
        tile_t[c * kTStride + r] = (r0 + r < rows && c0 + c < cols) ? in[(int64_t)(r0 + r) * cols + c0 + c] : 0;
      }
      __syncthreads();
      for (int i = threadIdx.x; i < kTile * kTile; i += blockDim.x) {
        const int c = i / kTile, r = i % kTile;
        if (r0 + r < rows && c0 + c < cols) out[(int64_t)(c0 + c) * rows + r0 + r] = tile_t[c * kTStride + r];
      }
      __syncthreads();
    }
  }
}

// ---- vectorised scale update ------------------------------------------------------------------------
__global__ void update_scales_kernel(const float* __restrict__ amax, int64_t amax_stride, float* scale, float* scale_inv,
                                     int n, float fp_max, int margin) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) {
    float s = msamp_compute_scale(amax[(int64_t)i * amax_stride], scale[i], fp_max, margin);
    scale[i] = s;
    scale_inv[i] = __frcp_rn(s);
  }
}

// Delayed-scaling bookkeeping for n metas that share flat buffers (one launch for all layers),
// amax is [n, window]: a non-finite newest entry is dropped, the scale is recomputed from the
// window maximum and the window moves by one slot with slot 0 cleared.  `bad[i]` (optional) is set
// to 1 when meta i saw a non-finite entry, so that the host can restart its warm-up counter later
// without synchronising now.  scale_inv is left alone: it belongs to the tensors that were
// quantised with the old scale and is refreshed by the next cast.
__global__ void roll_windows_kernel(float* amax, float* scale, int* bad, int n, int window, float fp_max, int margin) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float* a = amax + (int64_t)i * window;
  const bool finite = !(isinf(a[0]) || isnan(a[0]));
  if (!finite) a[0] = 0.0f;
  float mx = 0.0f;
  for (int j = 0; j < window; ++j) mx = fmaxf(mx, a[j]);
  scale[i] = msamp_compute_scale(mx, scale[i], fp_max, margin);
  for (int j = window - 1; j > 0; --j) a[j] = a[j - 1];
  a[0] = 0.0f;
  if (bad != nullptr) bad[i] = finite ? 0 : 1;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
inline bool aligned8(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 7) == 0; }

}    // namespace

// amax[0] = max|x| (NaN counts as +inf). With `counter` non-null the last block also writes
// scale = rule(amax) * prescale and scale_inv = 1/scale; `counter` is a zero-initialised word
// of scratch that the kernel leaves at zero again.
MSAMP_API int msamp_amax(const void* x, int64_t n, int dtype, float* amax, float* scale, float* scale_inv, float fp_max,
                         int margin, float prescale, unsigned int* counter, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  MSAMP_REQUIRE(n >= 0 && amax != nullptr, "msamp_amax: bad arguments");
  cudaMemsetAsync(amax, 0, sizeof(float), stream);
  int grid = msamp_grid_for((n + 31) / 32, kThreads, 6);
  if (n == 0) grid = 1;
  MSAMP_DISPATCH_HP(dtype, T, {
    if (aligned16(x))
      amax_kernel<T, true><<<grid, kThreads, 0, stream>>>((const T*)x, n, amax, scale, scale_inv, fp_max, margin, prescale, counter);
    else
      amax_kernel<T, false><<<grid, kThreads, 0, stream>>>((const T*)x, n, amax, scale, scale_inv, fp_max, margin, prescale, counter);
  });
  return msamp_check_launch("msamp_amax");
}

// out = saturate_fp8(act(x) * scale). With `amax` non-null it receives max|act(x)| (it is cleared first);
// with `scale_inv_out` non-null it receives 1 / scale. With `amax_in` non-null (amax and amax_in must
// differ) the scale is first derived from it:
//   rescale == 0: scale = rule(*amax_in) * prescale, stored to *scale (in-time scaling from a producer's amax);
//   rescale == 1: x is a scaled tensor (x0 * s_old), *scale holds 1 / s_old and *amax_in max|x0|; the
//                 effective factor is rule(amax) / s_old, scale_inv_out receives 1 / rule(amax), *scale is not written.
// act: 0 = identity, 1 = GeLU (tanh form), applied and rounded to the input type before quantising.
MSAMP_API int msamp_cast_to_fp8_ex(const void* x, int64_t n, int dtype, void* out, int fmt, float* scale, float* amax,
                                   float* scale_inv_out, const float* amax_in, float prescale, int rescale, int act, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  MSAMP_REQUIRE(n >= 0 && scale != nullptr, "msamp_cast_to_fp8: bad arguments");
  MSAMP_REQUIRE(act == 0 || act == 1, "msamp_cast_to_fp8: unknown activation %d", act);
  if (amax) cudaMemsetAsync(amax, 0, sizeof(float), stream);
  if (n == 0) return MSAMP_OK;
  int grid = msamp_grid_for((n + 31) / 32, kThreads, 6);
  const bool vec = aligned16(x) && aligned8(out);
#define MSAMP_CAST_LAUNCH(V, A) \
  cast_to_fp8_kernel<T, F, V, A><<<grid, kThreads, 0, stream>>>((const T*)x, (uint8_t*)out, n, scale, amax, scale_inv_out, amax_in, fp8_max(F), prescale, rescale)
  MSAMP_DISPATCH_HP(dtype, T, {
    MSAMP_DISPATCH_FP8(fmt, F, {
      if (vec && act == 0) MSAMP_CAST_LAUNCH(true, 0);
      else if (vec) MSAMP_CAST_LAUNCH(true, 1);
      else if (act == 0) MSAMP_CAST_LAUNCH(false, 0);
      else MSAMP_CAST_LAUNCH(false, 1);
    });
  });
#undef MSAMP_CAST_LAUNCH
  return msamp_check_launch("msamp_cast_to_fp8");
}

MSAMP_API int msamp_cast_to_fp8(const void* x, int64_t n, int dtype, void* out, int fmt, float* scale, float* amax,
                                float* scale_inv_out, const float* amax_in, float prescale, void* stream_) {
  return msamp_cast_to_fp8_ex(x, n, dtype, out, fmt, scale, amax, scale_inv_out, amax_in, prescale, 0, 0, stream_);
}

// x is [rows, cols] row-major, out its FP8 copy; the column sums of x are ADDED to colsum (fp32 [cols],
// zeroed by the caller).  cols * sizeof(element) must be a multiple of 16 and x, out 16- / 8-byte aligned.
// With amax_in non-null (it must differ from amax) the scale is first derived from it by the power-of-two rule and stored to *scale.
MSAMP_API int msamp_cast_to_fp8_colsum(const void* x, int rows, int cols, int dtype, void* out, int fmt, float* scale,
                                       float* amax, float* scale_inv_out, float* colsum, const float* amax_in, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  MSAMP_REQUIRE(rows >= 0 && cols >= 0 && scale != nullptr && colsum != nullptr && out != nullptr, "msamp_cast_to_fp8_colsum: bad arguments");
  const int esize = dtype == DT_F32 ? 4 : 2;
  MSAMP_REQUIRE(((int64_t)cols * esize) % 16 == 0 && aligned16(x) && aligned8(out), "msamp_cast_to_fp8_colsum: rows must be 16-byte multiples and aligned");
  if (amax) cudaMemsetAsync(amax, 0, sizeof(float), stream);
  if ((int64_t)rows * cols == 0) return MSAMP_OK;
  const int cv = cols * esize / 16;
  const int slabs = (cv + kThreads - 1) / kThreads;
  int per_slab = msamp_sm_count() * 4 / slabs;    // four CTAs are resident per SM (64 registers per thread)
  if (per_slab < 1) per_slab = 1;
  int gx = (rows + kColsumRows - 1) / kColsumRows;
  if (gx > per_slab) gx = per_slab;
  if (gx < 1) gx = 1;
  dim3 grid((unsigned)gx, (unsigned)slabs, 1);
  MSAMP_DISPATCH_HP(dtype, T, {
    MSAMP_DISPATCH_FP8(fmt, F, {
      cast_rows_colsum_kernel<T, F><<<grid, kThreads, 0, stream>>>((const T*)x, (uint8_t*)out, rows, cols, scale, amax, scale_inv_out, colsum, amax_in, fp8_max(F));
    });
  });
  return msamp_check_launch("msamp_cast_to_fp8_colsum");
}

MSAMP_API int msamp_cast_from_fp8(const void* in, int64_t n, int fmt, const float* scale_inv, void* out, int out_dtype,
                                  void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  MSAMP_REQUIRE(n >= 0 && scale_inv != nullptr, "msamp_cast_from_fp8: bad arguments");
  if (n == 0) return MSAMP_OK;
  int grid = msamp_grid_for((n + 7) / 8, kThreads, 4);
  const bool vec = aligned16(out) && aligned8(in);
  MSAMP_DISPATCH_HP(out_dtype, T, {
    MSAMP_DISPATCH_FP8(fmt, F, {
      if (vec)
        cast_from_fp8_kernel<T, F, true><<<grid, kThreads, 0, stream>>>((const uint8_t*)in, (T*)out, n, scale_inv);
      else
        cast_from_fp8_kernel<T, F, false><<<grid, kThreads, 0, stream>>>((const uint8_t*)in, (T*)out, n, scale_inv);
    });
  });
  return msamp_check_launch("msamp_cast_from_fp8");
}

// x is [rows, cols] row-major. out (may be null) is the row-major FP8 copy, out_t the [cols, rows] one.
// With amax_in non-null the input is a scaled tensor (x * s_old): `scale` must then point to
// 1 / s_old, amax_in to max|x|, and the effective factor becomes rule(amax) / s_old.
// colsum (may be null): fp32 [cols]; the column sums of x are ADDED to it (the bias gradient of a
// linear layer when x is the output gradient), so the caller zeroes it first.
static int cast_transpose_impl(const void* x, int rows, int cols, int dtype, void* out, void* out_t, int fmt, const float* scale,
                               float* amax, float* scale_inv_out, const float* amax_in, float* colsum, cudaStream_t stream) {
  MSAMP_REQUIRE(rows >= 0 && cols >= 0 && out_t != nullptr && scale != nullptr, "msamp_cast_transpose_fp8: bad arguments");
  if (amax) cudaMemsetAsync(amax, 0, sizeof(float), stream);
  if ((int64_t)rows * cols == 0) return MSAMP_OK;
  int64_t ntiles = (int64_t)((rows + kTileR - 1) / kTileR) * ((cols + kTileC - 1) / kTileC);
  int cap = msamp_sm_count() * 8;
  int grid = (int)(ntiles < cap ? ntiles : cap);
  const bool aligned = aligned16(x) && aligned16(out_t) && (out == nullptr || aligned8(out)) && (cols % 8 == 0) && (rows % 16 == 0);
  MSAMP_DISPATCH_HP(dtype, T, {
    MSAMP_DISPATCH_FP8(fmt, F, {
      if (out)
        cast_transpose_kernel<T, F, true><<<grid, kThreads, 0, stream>>>((const T*)x, (uint8_t*)out, (uint8_t*)out_t, rows, cols, scale, amax, scale_inv_out, amax_in, fp8_max(F), aligned, colsum);
      else
        cast_transpose_kernel<T, F, false><<<grid, kThreads, 0, stream>>>((const T*)x, nullptr, (uint8_t*)out_t, rows, cols, scale, amax, scale_inv_out, amax_in, fp8_max(F), aligned, colsum);
    });
  });
  return msamp_check_launch("msamp_cast_transpose_fp8");
}

MSAMP_API int msamp_cast_transpose_fp8(const void* x, int rows, int cols, int dtype, void* out, void* out_t, int fmt,
                                       const float* scale, float* amax, float* scale_inv_out, const float* amax_in, void* stream_) {
  return cast_transpose_impl(x, rows, cols, dtype, out, out_t, fmt, scale, amax, scale_inv_out, amax_in, nullptr, (cudaStream_t)stream_);
}

MSAMP_API int msamp_cast_transpose_fp8_colsum(const void* x, int rows, int cols, int dtype, void* out, void* out_t, int fmt,
                                              const float* scale, float* amax, float* scale_inv_out, const float* amax_in,
                                              float* colsum, void* stream_) {
  return cast_transpose_impl(x, rows, cols, dtype, out, out_t, fmt, scale, amax, scale_inv_out, amax_in, colsum, (cudaStream_t)stream_);
}

MSAMP_API int msamp_transpose_fp8(const void* in, int rows, int cols, void* out, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  MSAMP_REQUIRE(rows >= 0 && cols >= 0, "msamp_transpose_fp8: bad arguments");
  if ((int64_t)rows * cols == 0) return MSAMP_OK;
  int64_t ntiles = (int64_t)((rows + kTile - 1) / kTile) * ((cols + kTile - 1) / kTile);
  int cap = msamp_sm_count() * 8;
  int grid = (int)(ntiles < cap ? ntiles : cap);
  const bool aligned = aligned16(in) && aligned16(out) && (cols % 16 == 0) && (rows % 16 == 0);
  transpose_bytes_kernel<<<grid, kThreads, 0, stream>>>((const uint8_t*)in, (uint8_t*)out, rows, cols, aligned);
  return msamp_check_launch("msamp_transpose_fp8");
}

// scale[i] = rule(amax[i * amax_stride]); scale_inv[i] = 1 / scale[i].
MSAMP_API int msamp_update_scales(const float* amax, int64_t amax_stride, float* scale, float* scale_inv, int n, float fp_max,
                                  int margin, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  if (n <= 0) return MSAMP_OK;
  update_scales_kernel<<<(n + 127) / 128, 128, 0, stream>>>(amax, amax_stride, scale, scale_inv, n, fp_max, margin);
  return msamp_check_launch("msamp_update_scales");
}

MSAMP_API int msamp_roll_windows(float* amax, float* scale, int* bad, int n, int window, float fp_max, int margin,
                                 void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  if (n <= 0) return MSAMP_OK;
  roll_windows_kernel<<<(n + 127) / 128, 128, 0, stream>>>(amax, scale, bad, n, window, fp_max, margin);
  return msamp_check_launch("msamp_roll_windows");
}
