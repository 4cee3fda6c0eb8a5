// Pieces shared by the plain and the fused (compute + collective) FP8 GEMM kernels: tile
// configuration, epilogue load/store helpers and the cached tensor-map builder.
#pragma once
#include <mutex>
#include <unordered_map>

#include "tcgen05.cuh"

namespace gemm {


constexpr int BM = 128;
constexpr int BK = 128;    // bytes == fp8 elements per stage along K (one 128B swizzle atom)
constexpr int UMMA_K = 32;
constexpr int kGemmThreads = 192;

template <int BN>
struct Cfg {
  static constexpr int STAGES = (BN == 256) ? 4 : 6;
  static constexpr int A_BYTES = BM * BK;
  static constexpr int B_BYTES = BN * BK;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int TILE_BYTES = STAGES * STAGE_BYTES;
  static constexpr int BAR_BYTES = 256;
  static constexpr int SMEM_BYTES = TILE_BYTES + BAR_BYTES + 1024;    // +1024: manual alignment slack
  static constexpr int TMEM_COLS = 2 * BN;                            // two accumulator buffers (512 or 256)
};

struct GemmParams {
  void* d;
  const void* bias;
  const float* scale_inv_a;
  const float* scale_inv_b;
  float* amax_out;
  unsigned int* status;
  int M, N, K;
  int64_t ldd;    // elements
  int out_dtype;
  int bias_dtype;
  int accumulate;
  int a_fmt, b_fmt;
  int group_m;    // row tiles per rasterisation group (see tile_to_mn); 0 means all of them
};

template <typename OutT>
__device__ __forceinline__ void store_chunk(OutT* dst, const float (&v)[32], bool vec_ok, int valid) {
  if (vec_ok && valid == 32) {
    if constexpr (sizeof(OutT) == 4) {
#pragma unroll
      for (int j = 0; j < 32; j += 4) *reinterpret_cast<float4*>(dst + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
    } else {
#pragma unroll
      for (int j = 0; j < 32; j += 8) {
        Bytes16 o;
        OutT* e = reinterpret_cast<OutT*>(&o);
#pragma unroll
        for (int q = 0; q < 8; ++q) e[q] = from_f32<OutT>(v[j + q]);
        *reinterpret_cast<Bytes16*>(dst + j) = o;
      }
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (j < valid) dst[j] = from_f32<OutT>(v[j]);
  }
}

template <typename OutT>
__device__ __forceinline__ void load_chunk(const OutT* src, float (&v)[32], bool vec_ok, int valid) {
  if (vec_ok && valid == 32) {
    if constexpr (sizeof(OutT) == 4) {
#pragma unroll
      for (int j = 0; j < 32; j += 4) {
        float4 t = *reinterpret_cast<const float4*>(src + j);
        v[j] = t.x; v[j + 1] = t.y; v[j + 2] = t.z; v[j + 3] = t.w;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; j += 8) {
        Bytes16 o = *reinterpret_cast<const Bytes16*>(src + j);
        const OutT* e = reinterpret_cast<const OutT*>(&o);
#pragma unroll
        for (int q = 0; q < 8; ++q) v[j + q] = to_f32<OutT>(e[q]);
      }
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = (j < valid) ? to_f32<OutT>(src[j]) : 0.0f;
  }
}


// ---- host side -----------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(sym);
    }
  });
  return fn;
}

struct MapKey {
  const void* ptr;
  int64_t rows, cols, pitch;
  int box_rows;
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && rows == o.rows && cols == o.cols && pitch == o.pitch && box_rows == o.box_rows;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    size_t h = reinterpret_cast<size_t>(k.ptr);
    h ^= (size_t)k.rows * 0x9e3779b97f4a7c15ull + (h << 6) + (h >> 2);
    h ^= (size_t)k.cols * 0xc2b2ae3d27d4eb4full + (h << 6) + (h >> 2);
    h ^= (size_t)k.pitch * 0x165667b19e3779f9ull + (h << 6) + (h >> 2);
    h ^= (size_t)k.box_rows + (h << 6) + (h >> 2);
    return h;
  }
};

inline std::unordered_map<MapKey, CUtensorMap, MapKeyHash>& maps_cache() {
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> m;
  return m;
}
inline std::mutex& maps_mutex() {
  static std::mutex m;
  return m;
}

// Tensor map over a [rows, cols] byte matrix with row pitch `pitch` bytes; box = [box_rows, 128].
inline int make_map(const void* ptr, int64_t rows, int64_t cols, int64_t pitch, int box_rows, CUtensorMap* out) {
  MapKey key{ptr, rows, cols, pitch, box_rows};
  {
    std::lock_guard<std::mutex> lk(maps_mutex());
    auto it = maps_cache().find(key);
    if (it != maps_cache().end()) {
      *out = it->second;
      return MSAMP_OK;
    }
  }
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) {
    msamp_set_error("cuTensorMapEncodeTiled is not available from the driver");
    return MSAMP_ETMAP;
  }
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)pitch};
  cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    msamp_set_error("cuTensorMapEncodeTiled failed with %d (ptr=%p rows=%lld cols=%lld pitch=%lld)", (int)r, ptr,
                    (long long)rows, (long long)cols, (long long)pitch);
    return MSAMP_ETMAP;
  }
  std::lock_guard<std::mutex> lk(maps_mutex());
  if (maps_cache().size() > 8192) maps_cache().clear();
  maps_cache()[key] = *out;
  return MSAMP_OK;
}


}    // namespace gemm
