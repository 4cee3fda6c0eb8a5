// Symmetric memory over NVLink and the fused communication kernels built on it.
//
// Every rank (one process per GPU) allocates the same set of buffers, exports them as CUDA IPC
// handles and maps its peers' buffers, so each kernel holds a table of W base pointers and moves data
// with ordinary 16-byte loads and stores that travel over NVLink / NVSwitch.  Cross-rank ordering
// uses per-rank flag words: a writer publishes `epoch` with st.release.sys after a system fence, a
// reader polls its local copy with ld.acquire.sys.  Every wait is bounded: when it gives up it sets
// bit 1 of the device status word and the kernel returns, leaving the context usable.
//
// No TMA multicast and no library kernel ever sees a peer pointer here.
//
// Fused paths in this file
//   msamp_symm_grad_reduce   FP8 weight-gradient reduce-scatter / all-reduce: each owner pulls its
//                            tensors' e4m3 bytes from all peers, dequantises each with that peer's own
//                            per-tensor scale, averages in fp32, agrees on the result scale from
//                            the MAX of the peers' amax values and rounds once (the reference rounds at
//                            every hop of an NCCL ring, msamp/operators/dist_op/dist.cpp:39-104, after a
//                            separate amax all-reduce, msamp/nn/distributed.py:136-193).
//   msamp_symm_cast_bcast    ZeRO weight publish: scaled-fp16 master -> e4m3 with a fresh scale, stored
//                            straight into every peer's weight buffer together with its scale_inv
//                            (replaces cast + all-gather + scale_inv all-gather,
//                            msamp/deepspeed/runtime/zero/fp8_stage_1_and_2.py:760-853).
#include <string.h>

#include "common.cuh"

namespace {

constexpr int kMaxRanks = 8;
constexpr int kFlagSlots = 8;    // independent barrier slots per buffer set

struct PeerTable {
  uint8_t* data[kMaxRanks];     // flat byte buffers (gradients or weights)
  float* meta[kMaxRanks];       // per-tensor fp32 arrays: [3][n_tensors] = scale_inv, amax, spare
  uint32_t* flags[kMaxRanks];   // [kFlagSlots][kMaxRanks]
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint64_t gtimer() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Announce `epoch` in slot `slot` to every rank (one CTA does it), then wait until every rank has
// announced it.  Returns false after `limit_ns` without success.
__device__ bool symm_barrier(const PeerTable& pt, int rank, int world, int slot, uint32_t epoch, bool announce, uint64_t limit_ns,
                             unsigned int* status) {
  __shared__ int ok_flag;
  if (announce) {
    __threadfence_system();    // this rank's earlier writes (any memory) become visible before the flag
    if (threadIdx.x < world) st_release_sys(pt.flags[threadIdx.x] + slot * kMaxRanks + rank, epoch);
  }
  if (threadIdx.x == 0) ok_flag = 1;
  __syncthreads();
  if (threadIdx.x < world) {
    const uint32_t* f = pt.flags[rank] + slot * kMaxRanks + threadIdx.x;
    const uint64_t t0 = gtimer();
    uint32_t spins = 0;
    // epochs only grow; compare with wrap-around tolerance
    uint32_t seen;
    while ((int32_t)((seen = ld_acquire_sys(f)) - epoch) < 0) {
      if ((++spins & 0xff) == 0) {
        if (gtimer() - t0 > limit_ns) {
          ok_flag = 0;
          if (status) atomicOr(status, 2u);
          break;
        }
        __nanosleep(200);
      }
    }
    // A peer can never be ahead of this rank on the same slot when all ranks issue the same sequence of calls
    // (it cannot leave the call before this rank has arrived).  If it is, this rank skipped a call: report it
    // instead of letting the flags run out of step silently.
    if ((int32_t)(seen - epoch) > 0) {
      ok_flag = 0;
      if (status) atomicOr(status, 8u);
    }
  }
  __syncthreads();
  return ok_flag != 0;
}

// ---- barrier-only kernel (also used by tests of the timeout path) -------------------------------
__global__ void symm_barrier_kernel(PeerTable pt, int rank, int world, int slot, uint32_t epoch, uint64_t limit_ns, unsigned int* status,
                                    int announce) {
  symm_barrier(pt, rank, world, slot, epoch, announce != 0 && blockIdx.x == 0, limit_ns, status);
}

// ---- FP8 gradient reduce ---------------------------------------------------------------------------
struct ReduceArgs {
  PeerTable grads;              // data = flat e4m3 gradients, meta = [scale_inv | amax | -] per tensor
  const int64_t* offsets;       // [n_tensors + 1] byte offsets of the tensors in the flat buffer (multiples of 16)
  const int* work;              // (tensor, chunk) pairs this rank has to reduce
  int n_work;
  int n_tensors;
  int rank, world;
  uint32_t epoch;
  int broadcast;                // 1: write the result to every rank (all-reduce); 0: only locally (reduce-scatter)
  uint64_t limit_ns;
  unsigned int* status;
};

constexpr int kReduceThreads = 256;
constexpr int kReduceChunk = 16384;    // bytes per work item

__global__ void __launch_bounds__(kReduceThreads) symm_grad_reduce_kernel(const ReduceArgs a) {
  // (1) wait until every rank has finished writing its gradients and metas.  A CTA whose wait gave up skips the
  // work but still takes part in the completion count below, so that the shared counter returns to zero.
  const bool ready = symm_barrier(a.grads, a.rank, a.world, 0, a.epoch, blockIdx.x == 0, a.limit_ns, a.status);

  const float inv_world = 1.0f / (float)a.world;
  for (int w = blockIdx.x; ready && w < a.n_work; w += gridDim.x) {
    const int t = a.work[2 * w];
    const int64_t begin = a.offsets[t] + (int64_t)a.work[2 * w + 1] * kReduceChunk;
    int64_t end = begin + kReduceChunk;
    if (end > a.offsets[t + 1]) end = a.offsets[t + 1];

    float sinv[kMaxRanks];
    float amax = 0.0f;
#pragma unroll
    for (int r = 0; r < kMaxRanks; ++r) {
      if (r < a.world) {
        sinv[r] = a.grads.meta[r][t] * inv_world;
        amax = fmaxf(amax, abs_nan_to_inf(a.grads.meta[r][a.n_tensors + t]));
      }
    }
    // The mean is bounded by the largest per-rank amax, so a scale derived from it cannot overflow.
    const float new_scale = msamp_compute_scale(amax, 1.0f, 448.0f, 0);

    for (int64_t i = begin + (int64_t)threadIdx.x * 16; i < end; i += (int64_t)kReduceThreads * 16) {
      float acc[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) acc[j] = 0.0f;
#pragma unroll
      for (int r = 0; r < kMaxRanks; ++r) {
        if (r < a.world) {
          const int src = (a.rank + r) % a.world;    // stagger peers so that ranks do not all hit one GPU at once
          Bytes16 v = *reinterpret_cast<const Bytes16*>(a.grads.data[src] + i);
          const uint8_t* b = reinterpret_cast<const uint8_t*>(&v);
          const float s = sinv[src];
#pragma unroll
          for (int j = 0; j < 16; ++j) acc[j] += fp8_to_f32<FMT_E4M3>(b[j]) * s;
        }
      }
      Bytes16 o;
      uint16_t* e = reinterpret_cast<uint16_t*>(&o);
#pragma unroll
      for (int j = 0; j < 16; j += 2) e[j / 2] = f32x2_to_fp8x2<FMT_E4M3>(acc[j] * new_scale, acc[j + 1] * new_scale);
      if (a.broadcast) {
#pragma unroll
        for (int r = 0; r < kMaxRanks; ++r)
          if (r < a.world) *reinterpret_cast<Bytes16*>(a.grads.data[(a.rank + r) % a.world] + i) = o;
      } else {
        *reinterpret_cast<Bytes16*>(a.grads.data[a.rank] + i) = o;
      }
    }
    // the first chunk of each tensor publishes the result's meta into the third meta row
    if (a.work[2 * w + 1] == 0 && threadIdx.x == 0) {
      const float si = __frcp_rn(new_scale);
      if (a.broadcast) {
        for (int r = 0; r < a.world; ++r) {
          a.grads.meta[r][2 * a.n_tensors + t] = si;
        }
      } else {
        a.grads.meta[a.rank][2 * a.n_tensors + t] = si;
      }
    }
  }
  // (2) nobody may reuse the buffers (or read broadcast results) before every rank is done
  __syncthreads();
  // all CTAs of this rank must be finished before the announcement: count them in (low half: arrivals, high half:
  // CTAs that gave up).  Only a complete reduction is announced; after a give-up the peers' waits run out as well
  // and every rank reports the failure through the status word.
  __shared__ unsigned int announce;
  if (threadIdx.x == 0) {
    __threadfence_system();
    unsigned int* counter = reinterpret_cast<unsigned int*>(a.grads.flags[a.rank] + (kFlagSlots - 1) * kMaxRanks);
    const unsigned int before = atomicAdd(counter, ready ? 1u : 0x10001u);
    const bool is_last = (before & 0xffffu) == gridDim.x - 1;
    announce = (is_last && ready && (before >> 16) == 0u) ? 1u : 0u;
    if (is_last) *counter = 0u;
  }
  __syncthreads();
  if (!ready) return;
  symm_barrier(a.grads, a.rank, a.world, 1, a.epoch, announce != 0, a.limit_ns, a.status);
}

// After the reduce: scale_inv <- agreed value (row 2 -> row 0), for the tensors listed.
__global__ void symm_commit_meta_kernel(float* meta, int n_tensors, const int* tensors, int n) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) {
    int t = tensors[i];
    meta[t] = meta[2 * n_tensors + t];
  }
}

// ---- master -> e4m3 cast with broadcast --------------------------------------------------------------
struct CastBcastArgs {
  PeerTable weights;            // data = flat e4m3 weights, meta row 0 = scale_inv per tensor
  const int64_t* offsets;       // [n_tensors + 1] byte offsets
  const int* work;              // (tensor, chunk) pairs owned by this rank
  const void* const* master;    // [n_tensors] pointers to the scaled-fp16 master values (null if not owned)
  const float* const* master_sinv;    // [n_tensors] pointers to their scale_inv
  const float* const* master_amax;    // [n_tensors] pointers to max|w|
  int n_work, n_tensors, rank, world;
  uint32_t epoch;
  uint64_t limit_ns;
  unsigned int* status;
};

__global__ void __launch_bounds__(kReduceThreads) symm_cast_bcast_kernel(const CastBcastArgs a) {
  for (int w = blockIdx.x; w < a.n_work; w += gridDim.x) {
    const int t = a.work[2 * w];
    const int64_t tbeg = a.offsets[t];
    const int64_t begin = tbeg + (int64_t)a.work[2 * w + 1] * kReduceChunk;
    int64_t end = begin + kReduceChunk;
    const int64_t tend = a.offsets[t + 1];
    if (end > tend) end = tend;
    const __half* src = reinterpret_cast<const __half*>(a.master[t]);
    const float new_scale = msamp_compute_scale(*a.master_amax[t], 1.0f, 448.0f, 0);
    const float factor = new_scale * (*a.master_sinv[t]);
    for (int64_t i = begin + (int64_t)threadIdx.x * 16; i < end; i += (int64_t)kReduceThreads * 16) {
      const int64_t e0 = i - tbeg;    // element index inside the tensor (1 byte per element)
      Bytes16 h0 = *reinterpret_cast<const Bytes16*>(src + e0);
      Bytes16 h1 = *reinterpret_cast<const Bytes16*>(src + e0 + 8);
      const __half* x0 = reinterpret_cast<const __half*>(&h0);
      const __half* x1 = reinterpret_cast<const __half*>(&h1);
      Bytes16 o;
      uint16_t* e = reinterpret_cast<uint16_t*>(&o);
#pragma unroll
      for (int j = 0; j < 8; j += 2) {
        e[j / 2] = f32x2_to_fp8x2<FMT_E4M3>(__half2float(x0[j]) * factor, __half2float(x0[j + 1]) * factor);
        e[4 + j / 2] = f32x2_to_fp8x2<FMT_E4M3>(__half2float(x1[j]) * factor, __half2float(x1[j + 1]) * factor);
      }
#pragma unroll
      for (int r = 0; r < kMaxRanks; ++r)
        if (r < a.world) *reinterpret_cast<Bytes16*>(a.weights.data[(a.rank + r) % a.world] + i) = o;
    }
    if (a.work[2 * w + 1] == 0 && threadIdx.x == 0) {
      const float si = __frcp_rn(new_scale);
      for (int r = 0; r < a.world; ++r) {
        a.weights.meta[r][t] = si;
        a.weights.meta[r][a.n_tensors + t] = *a.master_amax[t];
      }
    }
  }
  __syncthreads();
  __shared__ unsigned int last;
  if (threadIdx.x == 0) {
    __threadfence_system();
    unsigned int* counter = reinterpret_cast<unsigned int*>(a.weights.flags[a.rank] + (kFlagSlots - 1) * kMaxRanks);
    last = (atomicAdd(counter, 1u) == gridDim.x - 1) ? 1u : 0u;
    if (last) *counter = 0u;
  }
  __syncthreads();
  symm_barrier(a.weights, a.rank, a.world, 2, a.epoch, last != 0, a.limit_ns, a.status);
}

int fill_table(PeerTable& pt, void* const* data, void* const* meta, void* const* flags, int world) {
  if (world < 1 || world > kMaxRanks) {
    msamp_set_error("symmetric kernels support 1..%d ranks, got %d", kMaxRanks, world);
    return MSAMP_EINVAL;
  }
  for (int r = 0; r < kMaxRanks; ++r) {
    pt.data[r] = r < world ? (uint8_t*)data[r] : nullptr;
    pt.meta[r] = r < world ? (float*)meta[r] : nullptr;
    pt.flags[r] = r < world ? (uint32_t*)flags[r] : nullptr;
  }
  return MSAMP_OK;
}

}    // namespace

MSAMP_API int msamp_symm_max_ranks() { return kMaxRanks; }
MSAMP_API int msamp_symm_flag_words() { return kFlagSlots * kMaxRanks; }
MSAMP_API int msamp_symm_chunk_bytes() { return kReduceChunk; }

// Allocate `bytes` of zeroed device memory that can be shared with other processes; `handle` receives
// the 64-byte IPC handle.
MSAMP_API int msamp_symm_alloc(size_t bytes, void** ptr, void* handle) {
  cudaError_t e = cudaMalloc(ptr, bytes);
  if (e != cudaSuccess) {
    msamp_set_error("symm_alloc(%zu): %s", bytes, cudaGetErrorString(e));
    return MSAMP_ELAUNCH;
  }
  cudaMemset(*ptr, 0, bytes);
  e = cudaIpcGetMemHandle((cudaIpcMemHandle_t*)handle, *ptr);
  if (e != cudaSuccess) {
    msamp_set_error("cudaIpcGetMemHandle: %s", cudaGetErrorString(e));
    cudaFree(*ptr);
    return MSAMP_ELAUNCH;
  }
  return MSAMP_OK;
}

MSAMP_API int msamp_symm_open(const void* handle, void** ptr) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  cudaError_t e = cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) {
    msamp_set_error("cudaIpcOpenMemHandle: %s", cudaGetErrorString(e));
    return MSAMP_ELAUNCH;
  }
  return MSAMP_OK;
}

MSAMP_API int msamp_symm_close(void* ptr) { return cudaIpcCloseMemHandle(ptr) == cudaSuccess ? MSAMP_OK : MSAMP_ELAUNCH; }
MSAMP_API int msamp_symm_free(void* ptr) { return cudaFree(ptr) == cudaSuccess ? MSAMP_OK : MSAMP_ELAUNCH; }

// Cross-rank barrier on slot `slot` (3..6 are free for callers). announce = 0 only waits: with no
// peer announcing it exercises the bounded-wait path.
MSAMP_API int msamp_symm_barrier(void* const* flags, int rank, int world, int slot, unsigned int epoch, double limit_seconds,
                                 int announce, void* stream_) {
  PeerTable pt;
  void* dummy[kMaxRanks] = {nullptr};
  int rc = fill_table(pt, dummy, dummy, flags, world);
  if (rc) return rc;
  MSAMP_REQUIRE(slot >= 0 && slot < kFlagSlots - 1, "symm_barrier: bad slot %d", slot);
  symm_barrier_kernel<<<1, 32, 0, (cudaStream_t)stream_>>>(pt, rank, world, slot, epoch, (uint64_t)(limit_seconds * 1e9),
                                                           msamp_device_status_ptr(), announce);
  return msamp_check_launch("msamp_symm_barrier");
}

// data/meta/flags: arrays of `world` device pointers (this rank's own buffers at index `rank`).
// offsets, work: device arrays.  The result replaces this rank's copy of the tensors it owns (and
// everybody's copy with broadcast = 1); the agreed scale_inv lands in meta row 2.
MSAMP_API int msamp_symm_grad_reduce(void* const* data, void* const* meta, void* const* flags, const int64_t* offsets, const int* work,
                                     int n_work, int n_tensors, int rank, int world, unsigned int epoch, int broadcast,
                                     double limit_seconds, int max_ctas, void* stream_) {
  ReduceArgs a;
  int rc = fill_table(a.grads, data, meta, flags, world);
  if (rc) return rc;
  a.offsets = offsets; a.work = work; a.n_work = n_work; a.n_tensors = n_tensors; a.rank = rank; a.world = world; a.epoch = epoch;
  a.broadcast = broadcast; a.limit_ns = (uint64_t)(limit_seconds * 1e9); a.status = msamp_device_status_ptr();
  int grid = msamp_sm_count() * 2;
  if (max_ctas > 0 && max_ctas < grid) grid = max_ctas;
  // every CTA takes part in the barriers, so the grid must be co-resident: at most 2 CTAs of 256 threads per SM
  symm_grad_reduce_kernel<<<grid, kReduceThreads, 0, (cudaStream_t)stream_>>>(a);
  return msamp_check_launch("msamp_symm_grad_reduce");
}

MSAMP_API int msamp_symm_commit_meta(float* meta, int n_tensors, const int* tensors, int n, void* stream_) {
  if (n <= 0) return MSAMP_OK;
  symm_commit_meta_kernel<<<(n + 127) / 128, 128, 0, (cudaStream_t)stream_>>>(meta, n_tensors, tensors, n);
  return msamp_check_launch("msamp_symm_commit_meta");
}

MSAMP_API int msamp_symm_cast_bcast(void* const* data, void* const* meta, void* const* flags, const int64_t* offsets, const int* work,
                                    int n_work, int n_tensors, const void* const* master, const float* const* master_sinv,
                                    const float* const* master_amax, int rank, int world, unsigned int epoch, double limit_seconds,
                                    void* stream_) {
  CastBcastArgs a;
  int rc = fill_table(a.weights, data, meta, flags, world);
  if (rc) return rc;
  a.offsets = offsets; a.work = work; a.n_work = n_work; a.n_tensors = n_tensors; a.master = master; a.master_sinv = master_sinv;
  a.master_amax = master_amax; a.rank = rank; a.world = world; a.epoch = epoch; a.limit_ns = (uint64_t)(limit_seconds * 1e9);
  a.status = msamp_device_status_ptr();
  int grid = msamp_sm_count() * 2;
  symm_cast_bcast_kernel<<<grid, kReduceThreads, 0, (cudaStream_t)stream_>>>(a);
  return msamp_check_launch("msamp_symm_cast_bcast");
}
