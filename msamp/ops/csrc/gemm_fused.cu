// FP8 GEMM fused with a collective over NVLink peer memory (one kernel does both).
//
//   gather + GEMM     One operand is sharded over the W ranks of a group (Megatron sequence-parallel
//                     all-gather -> GEMM, ZeRO-3/FSDP parameter all-gather -> GEMM).  A few CTAs of the
//                     persistent grid act as copy engines: they pull the peers' shards with bulk async
//                     copies (global -> shared -> global, never multicast) chunk by chunk into local
//                     buffers and publish a flag per chunk; the remaining CTAs run the tcgen05 main
//                     loop, starting with the tiles that need only the local shard and waiting
//                     (bounded) on the flag of a remote chunk right before its first TMA load.
//                     Shards can be concatenated along the rows of A or B, or along K.
//   GEMM + reduce-scatter   Row-parallel linear / sequence-parallel dgrad: every rank computes a partial
//                     D; the epilogue stores each tile straight into the owning rank's staging slot
//                     over NVLink (rows owned by other ranks are computed first), then, after a
//                     cross-rank barrier inside the kernel, each rank sums its W slots.
//
// Replaces the separate NCCL all_gather_base / reduce_scatter_base calls around te_gemm in the
// reference (msamp/megatron/layers.py:94-112, 138-203).  Every wait is bounded and reports through
// the device status word (bit 0 pipeline, bit 1 peer flag, bit 2 grid barrier).
#include "gemm_common.cuh"

namespace {
using namespace gemm;

constexpr int kMaxRanks = 8;
constexpr int kPiece = 32768;    // bytes moved per bulk copy by a copy warp
constexpr int kRsStageBytes = 4 * 8192;    // reduce-scatter epilogue: 32 rows x 256 bytes per epilogue warp

enum GatherMode { G_NONE = 0, G_A_ROWS = 1, G_B_ROWS = 2, G_B_K = 3, G_A_K = 4 };

struct FusedMaps {
  CUtensorMap a[kMaxRanks];
  CUtensorMap b[kMaxRanks];
};

struct FusedArgs {
  int gather;
  int world, rank;
  const uint8_t* peer[kMaxRanks];    // peers' shard buffers (peer[rank] unused)
  uint8_t* local[kMaxRanks];         // local copies of the peers' shards (local[rank] = own shard)
  int64_t chunk_bytes;               // contiguous bytes per flag chunk (chunk_rows * row pitch)
  int chunks_per_shard;
  int chunk_rows;
  int shard_tiles;                   // tiles (BM or BN rows) per shard for row gathers; k-blocks per shard for K gathers
  uint32_t* chunk_flags;             // [world][chunks_per_shard], local memory, holds epochs
  uint32_t* sym_flags[kMaxRanks];    // cross-rank flag words [slots][kMaxRanks]
  uint32_t epoch;
  int n_comm;
  uint64_t limit_ns;
  int rs;
  uint8_t* stage[kMaxRanks];         // peers' staging buffers [world][rows_per_rank][N] of OutT
  int rows_per_rank;
  void* rs_out;
  int64_t rs_ldo;
  unsigned int* counters;            // local scratch words, all left at zero: [0] comm CTAs done, [1] compute CTAs done,
                                     // [2 + world * chunks_per_shard] pieces landed per gathered chunk
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu(uint32_t* p, uint32_t v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async;" ::: "memory"); }

__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src), "r"(bytes),
               "r"(bar)
               : "memory");
}
__device__ __forceinline__ void bulk_s2g(void* dst, uint32_t src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// Bounded wait for a 32-bit flag to reach `epoch` (monotone counters, wrap tolerant).
template <bool SYS>
__device__ __forceinline__ bool wait_flag(const uint32_t* f, uint32_t epoch, uint64_t limit_ns, volatile int* abort_flag,
                                          unsigned int* status, unsigned int bit) {
  uint64_t t0 = 0;
  for (uint32_t spin = 0;; ++spin) {
    uint32_t v = SYS ? ld_acquire_sys(f) : ld_acquire_gpu(f);
    if ((int32_t)(v - epoch) >= 0) return true;
    if ((spin & 0x3f) == 0x3f) {
      if (*abort_flag) return false;
      uint64_t now = tc5::globaltimer_ns();
      if (t0 == 0) {
        t0 = now;
      } else if (now - t0 > limit_ns) {
        *abort_flag = 1;
        if (status) atomicOr(status, bit);
        return false;
      }
      __nanosleep(100);
    }
  }
}

// Tile index -> (m tile, n tile).  Gathers walk the sharded dimension slowly, starting with the
// local shard; reduce-scatter walks rows slowly, ending with the rows this rank owns.
__device__ __forceinline__ void tile_coords(int t, int num_m, int num_n, const FusedArgs& f, int& mi, int& ni) {
  if (f.gather == G_A_ROWS) {
    mi = ((t / num_n) + f.rank * f.shard_tiles) % num_m;
    ni = t % num_n;
  } else if (f.gather == G_B_ROWS) {
    ni = ((t / num_m) + f.rank * f.shard_tiles) % num_n;
    mi = t % num_m;
  } else if (f.rs) {
    const int per_rank = num_m / f.world;
    mi = ((t / num_n) + (f.rank + 1) * per_rank) % num_m;
    ni = t % num_n;
  } else {
    mi = t % num_m;
    ni = t / num_m;
  }
}

template <int BN, typename OutT>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_fused_kernel(const __grid_constant__ FusedMaps maps, const GemmParams p, const FusedArgs f) {
  using C = Cfg<BN>;
  extern __shared__ uint8_t smem_raw[];
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
  int* role_flag = reinterpret_cast<int*>(tmem_holder + 10);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_m = (p.M + BM - 1) / BM;
  const int num_n = (p.N + BN - 1) / BN;
  const int num_tiles = num_m * num_n;
  const int num_kb = (p.K + BK - 1) / BK;
  const int n_comm = f.gather ? f.n_comm : 0;
  const bool is_comm = (int)blockIdx.x < n_comm;
  const int cta = (int)blockIdx.x - n_comm;
  const int ncta = (int)gridDim.x - n_comm;

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
    *role_flag = 0;
    tc5::mbar_fence_init();
  }
  if (warp == 1 && !is_comm) {
    tc5::tmem_alloc(tc5::smem_u32(tmem_holder), C::TMEM_COLS);
    tc5::tmem_relinquish();
  }
  tc5::fence_before_sync();
  __syncthreads();
  tc5::fence_after_sync();
  const uint32_t tmem_base = *tmem_holder;

  if (is_comm) {
    // ================================================================== copy engine CTA
    // Peers' shards must be complete before anything is read from them: one cross-rank barrier.
    if (warp == 0 && lane < f.world) {
      if (blockIdx.x == 0) {
        __threadfence_system();
        st_release_sys(f.sym_flags[lane] + 0 * kMaxRanks + f.rank, f.epoch);
      }
      wait_flag<true>(f.sym_flags[f.rank] + 0 * kMaxRanks + lane, f.epoch, f.limit_ns, abort_flag, p.status, 2u);
    }
    __syncthreads();
    if (!*abort_flag && lane == 0) {
      // Each of the six warps owns one 32 KiB slot of shared memory and moves every sixth piece.
      constexpr int kWarps = kGemmThreads / 32;
      const int pieces_per_chunk = (int)((f.chunk_bytes + kPiece - 1) / kPiece);
      const int remote_chunks = (f.world - 1) * f.chunks_per_shard;
      const uint32_t slot = base + warp * kPiece;
      const uint32_t bar = full_bar(warp % C::STAGES) + ((warp >= C::STAGES) ? 8u * C::STAGES : 0u);    // one private barrier per warp
      uint32_t phase = 0;
      int it = 0;
      for (int c = (int)blockIdx.x; c < remote_chunks; c += n_comm, ++it) {
        const int src = (f.rank + 1 + c / f.chunks_per_shard) % f.world;
        const int ch = c % f.chunks_per_shard;
        const uint8_t* from = f.peer[src] + (int64_t)ch * f.chunk_bytes;
        uint8_t* to = f.local[src] + (int64_t)ch * f.chunk_bytes;
        bool ok = true;
        for (int q = warp; q < pieces_per_chunk; q += kWarps) {
          const int64_t off = (int64_t)q * kPiece;
          const uint32_t bytes = (uint32_t)((f.chunk_bytes - off) < kPiece ? (f.chunk_bytes - off) : kPiece);
          tc5::mbar_arrive_expect_tx(bar, bytes);
          bulk_g2s(slot, from + off, bytes, bar);
          if (!tc5::mbar_wait(bar, phase, abort_flag, p.status, 2u)) { ok = false; break; }
          phase ^= 1;
          bulk_s2g(to + off, slot, bytes);
          bulk_commit();
          bulk_wait_all();    // the piece is in local memory and the slot is free again
        }
        if (!ok) break;
        // publish the chunk once all of its pieces (spread over the warps) have landed
        fence_proxy_async();
        __threadfence();
        const int mine = (pieces_per_chunk - warp + kWarps - 1) / kWarps;
        if (mine > 0) {
          // one counter per chunk (not a small ring shared by chunks): the six warps never synchronise with each
          // other, so any reuse of a counter could mix the pieces of two chunks
          unsigned int* cnt = f.counters + 2 + src * f.chunks_per_shard + ch;
          unsigned int done = atomicAdd(cnt, (unsigned int)mine) + mine;
          if (done == (unsigned int)pieces_per_chunk) {
            *cnt = 0;
            st_release_gpu(f.chunk_flags + src * f.chunks_per_shard + ch, f.epoch);
          }
        }
      }
    }
    __syncthreads();
    // Tell the peers that this rank no longer reads their shards, and stay until they have said the same.
    if (threadIdx.x == 0) {
      __threadfence_system();
      unsigned int n = atomicAdd(&f.counters[0], 1u);
      *role_flag = (n == (unsigned int)n_comm - 1) ? 1 : 0;
      if (*role_flag) f.counters[0] = 0;
    }
    __syncthreads();
    if (*role_flag && warp == 0 && lane < f.world) {
      st_release_sys(f.sym_flags[lane] + 1 * kMaxRanks + f.rank, f.epoch);
      wait_flag<true>(f.sym_flags[f.rank] + 1 * kMaxRanks + lane, f.epoch, f.limit_ns, abort_flag, p.status, 2u);
    }
  } else if (warp == 0) {
    // ================================================================== TMA producer
    if (lane == 0) {
      uint32_t it = 0;
      for (int tile = cta; tile < num_tiles; tile += ncta) {
        int mi, ni;
        tile_coords(tile, num_m, num_n, f, mi, ni);
        const int m0 = mi * BM, n0 = ni * BN;
        const CUtensorMap* map_a = &maps.a[0];
        const CUtensorMap* map_b = &maps.b[0];
        int a_row = m0, b_row = n0;
        bool ok = true;
        if (f.gather == G_A_ROWS) {
          const int src = mi / f.shard_tiles;
          a_row = (mi % f.shard_tiles) * BM;
          map_a = &maps.a[src];
          if (src != f.rank) {
            ok = wait_flag<false>(f.chunk_flags + src * f.chunks_per_shard + a_row / f.chunk_rows, f.epoch, f.limit_ns, abort_flag, p.status, 2u);
            fence_proxy_async();
          }
        } else if (f.gather == G_B_ROWS) {
          const int src = ni / f.shard_tiles;
          b_row = (ni % f.shard_tiles) * BN;
          map_b = &maps.b[src];
          if (src != f.rank) {
            ok = wait_flag<false>(f.chunk_flags + src * f.chunks_per_shard + b_row / f.chunk_rows, f.epoch, f.limit_ns, abort_flag, p.status, 2u);
            fence_proxy_async();
          }
        }
        if (!ok) break;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          int ka = kb * BK, kbb = kb * BK;
          if (f.gather == G_B_K || f.gather == G_A_K) {
            // k-blocks are visited shard by shard, local shard first
            const int src = (f.rank + kb / f.shard_tiles) % f.world;
            const int koff = (kb % f.shard_tiles) * BK;
            const int kfull = src * f.shard_tiles * BK + koff;
            if (f.gather == G_B_K) {
              map_b = &maps.b[src];
              kbb = koff;
              ka = kfull;
            } else {
              map_a = &maps.a[src];
              ka = koff;
              kbb = kfull;
            }
            if (src != f.rank && (kb % f.shard_tiles) == 0) {
              const int row = (f.gather == G_B_K) ? n0 : m0;
              const int tile_rows = (f.gather == G_B_K) ? BN : BM;
              // a tile may straddle two flag chunks when the chunk is smaller than the tile
              for (int r = row; r < row + tile_rows && ok; r += f.chunk_rows) {
                const int ch = r / f.chunk_rows;
                if (ch < f.chunks_per_shard)
                  ok = wait_flag<false>(f.chunk_flags + src * f.chunks_per_shard + ch, f.epoch, f.limit_ns, abort_flag, p.status, 2u);
              }
              fence_proxy_async();
              if (!ok) break;
            }
          }
          const int s = it % C::STAGES;
          const uint32_t ph = (it / C::STAGES) & 1;
          if (!tc5::mbar_wait(empty_bar(s), ph ^ 1, abort_flag, p.status, 1u)) { ok = false; break; }
          tc5::mbar_arrive_expect_tx(full_bar(s), C::STAGE_BYTES);
          const uint32_t sa = base + s * C::STAGE_BYTES;
          tc5::tma_load_2d(sa, map_a, ka, a_row, full_bar(s));
          tc5::tma_load_2d(sa + C::A_BYTES, map_b, kbb, b_row, full_bar(s));
        }
        if (!ok) break;
      }
    }
  } else if (warp == 1) {
    // ================================================================== MMA issuer
    if (lane == 0) {
      const uint32_t idesc = tc5::idesc_f8(BM, BN, p.a_fmt, p.b_fmt);
      uint32_t lt = 0;
      // As in gemm_fp8.cu: the tensor pipe idles for whatever this thread does between two MMAs, and a blocking wait on
      // a stage barrier costs 100-140 cycles even when the data is there.  The barrier of the next stage is probed
      // without blocking before the last MMA of a K block; the blocking wait runs only when the probe failed.
      const uint64_t da0 = tc5::smem_desc_k_sw128(base);
      const uint64_t db0 = tc5::smem_desc_k_sw128(base + C::A_BYTES);
      int s = 0;
      uint32_t ph = 0;
      bool pre_ok = false;
      for (int tile = cta; tile < num_tiles; tile += ncta, ++lt) {
        const int buf = lt & 1;
        const uint32_t aph = (lt >> 1) & 1;
        if (!tc5::mbar_wait(tempty_bar(buf), aph ^ 1, abort_flag, p.status, 1u)) break;
        tc5::fence_after_sync();
        const uint32_t tmem_d = tmem_base + (uint32_t)(buf * BN);
        bool ok = true;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!pre_ok && !tc5::mbar_wait(full_bar(s), ph, abort_flag, p.status, 1u)) { ok = false; break; }
          tc5::fence_after_sync();
          const uint64_t da = da0 + (uint64_t)(s * (C::STAGE_BYTES >> 4));
          const uint64_t db = db0 + (uint64_t)(s * (C::STAGE_BYTES >> 4));
          int sn = s + 1;
          uint32_t phn = ph;
          if (sn == C::STAGES) { sn = 0; phn ^= 1u; }
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            if (k == BK / UMMA_K - 1) pre_ok = tc5::mbar_test(full_bar(sn), phn);
            tc5::mma_f8f6f4(tmem_d, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc, (kb | k) ? 1u : 0u);
          }
          tc5::mma_commit(empty_bar(s));
          s = sn;
          ph = phn;
        }
        if (!ok) break;
        tc5::mma_commit(tfull_bar(buf));
      }
    }
  } else {
    // ================================================================== epilogue (4 warps)
    const int q = warp & 3;
    const float alpha = (*p.scale_inv_a) * (*p.scale_inv_b);
    OutT* D = reinterpret_cast<OutT*>(p.d);
    const bool vec_ok = f.rs ? ((p.N * sizeof(OutT)) % 16 == 0)
                             : (((reinterpret_cast<uintptr_t>(D) & 15) == 0) && ((p.ldd * sizeof(OutT)) % 16 == 0));
    float amax = 0.0f;
    uint32_t lt = 0;
    for (int tile = cta; tile < num_tiles; tile += ncta, ++lt) {
      int mi, ni;
      tile_coords(tile, num_m, num_n, f, mi, ni);
      const int m0 = mi * BM, n0 = ni * BN;
      const int buf = lt & 1;
      const uint32_t aph = (lt >> 1) & 1;
      if (!tc5::mbar_wait(tfull_bar(buf), aph, abort_flag, p.status, 1u)) break;
      tc5::fence_after_sync();
      const int row = m0 + q * 32 + lane;
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * BN);
      OutT* row_ptr = D + (int64_t)row * p.ldd;
      if (f.rs) {
        // The 128 rows of a tile belong to one rank (`owner`); they land in the slot reserved for this rank in
        // the owner's staging buffer.  A thread holds one row of the accumulator, so direct stores would hit the
        // peer with scattered 64-byte pieces; instead each warp turns 32 rows x 256 bytes around in shared memory
        // (16-byte chunks XOR-swizzled by the row) and writes whole 256-byte row segments, two rows per store.
        const int owner = m0 / f.rows_per_rank;
        OutT* tile_ptr = reinterpret_cast<OutT*>(f.stage[owner < f.world ? owner : 0]) +
                         ((int64_t)f.rank * f.rows_per_rank + (m0 % f.rows_per_rank) + q * 32) * (int64_t)p.N;
        constexpr int kColsPerPass = 256 / (int)sizeof(OutT);    // columns in 256 bytes
        constexpr int kChunksPerPass = kColsPerPass / 32;        // tcgen05.ld pieces per pass
        const uint32_t wbase = base + C::TILE_BYTES + C::BAR_BYTES + (uint32_t)q * 8192u;
#pragma unroll 1
        for (int pass = 0; pass < BN / kColsPerPass; ++pass) {
#pragma unroll
          for (int cc = 0; cc < kChunksPerPass; ++cc) {
            uint32_t r[32];
            tc5::tmem_ld32(taddr + (uint32_t)(pass * kColsPerPass + cc * 32), r);
            tc5::tmem_ld_wait();
            alignas(16) OutT o[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) o[j] = from_f32<OutT>(__uint_as_float(r[j]) * alpha);
            const Bytes16* o16 = reinterpret_cast<const Bytes16*>(o);
            constexpr int kPieces = 32 * (int)sizeof(OutT) / 16;    // 16-byte pieces of this 32-column chunk
#pragma unroll
            for (int j = 0; j < kPieces; ++j) {
              const uint32_t ch = (uint32_t)(cc * kPieces + j);
              const uint32_t addr = wbase + (uint32_t)lane * 256u + ((ch ^ ((uint32_t)lane & 15u)) << 4);
              asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(o16[j].w[0]), "r"(o16[j].w[1]), "r"(o16[j].w[2]), "r"(o16[j].w[3])
                           : "memory");
            }
          }
          __syncwarp();
          const int col_b = (n0 + pass * kColsPerPass) * (int)sizeof(OutT) + (lane & 15) * 16;    // byte offset inside the row
#pragma unroll 4
          for (int i = 0; i < 16; ++i) {
            const int rr = 2 * i + (lane >> 4);
            const uint32_t addr = wbase + (uint32_t)rr * 256u + ((((uint32_t)lane & 15u) ^ ((uint32_t)rr & 15u)) << 4);
            uint4 v;
            asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
            if (m0 + q * 32 + rr < p.M && col_b < p.N * (int)sizeof(OutT))
              *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(tile_ptr + (int64_t)rr * p.N) + col_b) = v;
          }
          __syncwarp();
        }
        tc5::fence_before_sync();
        __syncwarp();
        if (lane == 0) tc5::mbar_arrive(tempty_bar(buf));
        continue;
      }
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
          if (p.bias != nullptr && p.bias_dtype == DT_F32) {
            const float* b = reinterpret_cast<const float*>(p.bias) + col;
#pragma unroll
            for (int j = 0; j < 32; ++j) if (j < valid) v[j] += __ldg(b + j);
          }
          OutT* dst = row_ptr + col;
          if (p.accumulate && !f.rs) {
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
    if (f.rs) __threadfence_system();    // pushed tiles are visible to their owners before this CTA reports in
  }

  // ---------------------------------------------------------------------- reduce-scatter tail
  if (f.rs && !is_comm) {
    __syncthreads();
    if (threadIdx.x == 0) {
      unsigned int n = atomicAdd(&f.counters[1], 1u);
      *role_flag = (n == (unsigned int)ncta - 1) ? 1 : 0;
      if (*role_flag) f.counters[1] = 0;
    }
    __syncthreads();
    if (warp == 0 && lane < f.world) {
      if (*role_flag) {
        __threadfence_system();
        st_release_sys(f.sym_flags[lane] + 2 * kMaxRanks + f.rank, f.epoch);    // every tile of this rank has been pushed
      }
      wait_flag<true>(f.sym_flags[f.rank] + 2 * kMaxRanks + lane, f.epoch, f.limit_ns, abort_flag, p.status, 2u);
    }
    __syncthreads();
    if (!*abort_flag) {
      // out[r, :] = sum over source ranks of stage[src][r, :]
      const OutT* st = reinterpret_cast<const OutT*>(f.stage[f.rank]);
      OutT* out = reinterpret_cast<OutT*>(f.rs_out);
      constexpr int V = 16 / sizeof(OutT);
      const int64_t slot_elems = (int64_t)f.rows_per_rank * p.N;
      const int vec_per_row = p.N / V;
      const int64_t total = (int64_t)f.rows_per_rank * vec_per_row;
      for (int64_t i = (int64_t)cta * kGemmThreads + threadIdx.x; i < total; i += (int64_t)ncta * kGemmThreads) {
        const int r = (int)(i / vec_per_row), cv = (int)(i % vec_per_row);
        float acc[V];
#pragma unroll
        for (int j = 0; j < V; ++j) acc[j] = 0.0f;
        for (int s = 0; s < f.world; ++s) {
          Bytes16 v = *reinterpret_cast<const Bytes16*>(st + s * slot_elems + (int64_t)r * p.N + cv * V);
          const OutT* e = reinterpret_cast<const OutT*>(&v);
#pragma unroll
          for (int j = 0; j < V; ++j) acc[j] += to_f32<OutT>(e[j]);
        }
        Bytes16 o;
        OutT* oe = reinterpret_cast<OutT*>(&o);
#pragma unroll
        for (int j = 0; j < V; ++j) oe[j] = from_f32<OutT>(acc[j]);
        *reinterpret_cast<Bytes16*>(out + (int64_t)r * f.rs_ldo + cv * V) = o;
      }
    }
  }

  // ---------------------------------------------------------------------- tear-down
  __syncwarp();
  if (*abort_flag) __nanosleep(200000);
  tc5::fence_before_sync();
  __syncthreads();
  tc5::fence_after_sync();
  if (warp == 1 && !is_comm) tc5::tmem_dealloc(tmem_base, C::TMEM_COLS);
}

template <int BN, typename OutT>
int launch_fused(const FusedMaps& maps, const GemmParams& p, const FusedArgs& f, cudaStream_t stream) {
  using C = Cfg<BN>;
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!configured[dev & 63]) {
    cudaError_t e = cudaFuncSetAttribute(gemm_fused_kernel<BN, OutT>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES + kRsStageBytes);
    if (e != cudaSuccess) {
      msamp_set_error("cudaFuncSetAttribute(fused): %s", cudaGetErrorString(e));
      return MSAMP_ELAUNCH;
    }
    configured[dev & 63] = true;
  }
  // All CTAs take part in flag waits, so the grid must be co-resident: one CTA per SM at most.
  int grid = msamp_sm_count();
  gemm_fused_kernel<BN, OutT><<<grid, kGemmThreads, C::SMEM_BYTES + kRsStageBytes, stream>>>(maps, p, f);
  return msamp_check_launch("gemm_fused_kernel");
}

}    // namespace

// Descriptor passed from Python (all pointers as 64-bit integers).
struct MsampFusedDesc {
  // GEMM
  uint64_t a[kMaxRanks];       // A operand: one pointer, or one per source shard for gather modes on A
  uint64_t b[kMaxRanks];       // B operand: likewise
  uint64_t d;                  // output (ignored with rs)
  uint64_t scale_inv_a, scale_inv_b, bias, amax_out;
  int32_t M, N, K;
  int32_t a_fmt, b_fmt, out_dtype, bias_dtype, accumulate;
  int64_t lda, ldb, ldd;       // row pitches: bytes for a/b, elements for d
  // gather
  int32_t gather, world, rank, n_comm;
  uint64_t peer[kMaxRanks];    // peers' shard buffers
  int64_t shard_rows;          // rows of one shard (row gathers) / columns of K in one shard (K gathers)
  int64_t shard_pitch;         // row pitch of a shard buffer in bytes
  int64_t shard_nrows;         // number of rows in a shard buffer
  uint64_t chunk_flags;
  uint64_t sym_flags[kMaxRanks];
  uint32_t epoch;
  int32_t rs;
  uint64_t stage[kMaxRanks];
  int32_t rows_per_rank, pad;
  uint64_t rs_out;
  int64_t rs_ldo;
  uint64_t counters;
  double limit_seconds;
};

MSAMP_API int msamp_fused_desc_bytes() { return (int)sizeof(MsampFusedDesc); }

MSAMP_API int msamp_gemm_fused(const MsampFusedDesc* d, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  MSAMP_REQUIRE(d->M > 0 && d->N > 0 && d->K > 0 && d->K % 16 == 0, "gemm_fused: bad problem M=%d N=%d K=%d", d->M, d->N, d->K);
  MSAMP_REQUIRE(d->world >= 1 && d->world <= kMaxRanks, "gemm_fused: world=%d not supported", d->world);
  // 128 x 256 tiles, except that a row gather of B whose shards are a multiple of 128 but not of 256 rows (e.g. 7168 / 8
  // = 896 or 21504 / 8 = 2688) uses 128 x 128 tiles: a tile must not straddle two ranks' shards.
  int bn = (d->N >= 256) ? 256 : 128;
  if (d->gather == G_B_ROWS && d->shard_rows % 256 != 0) bn = 128;
  FusedMaps maps;
  FusedArgs f = {};
  GemmParams p;
  p.d = (void*)d->d; p.bias = (const void*)d->bias; p.scale_inv_a = (const float*)d->scale_inv_a; p.scale_inv_b = (const float*)d->scale_inv_b;
  p.amax_out = (float*)d->amax_out; p.status = msamp_device_status_ptr();
  p.M = d->M; p.N = d->N; p.K = d->K; p.ldd = d->ldd; p.out_dtype = d->out_dtype; p.bias_dtype = d->bias_dtype; p.accumulate = d->accumulate;
  p.a_fmt = d->a_fmt; p.b_fmt = d->b_fmt; p.group_m = 0;
  f.gather = d->gather; f.world = d->world; f.rank = d->rank; f.epoch = d->epoch; f.n_comm = d->n_comm;
  f.limit_ns = (uint64_t)(d->limit_seconds * 1e9);
  f.rs = d->rs; f.rows_per_rank = d->rows_per_rank; f.rs_out = (void*)d->rs_out; f.rs_ldo = d->rs_ldo;
  f.counters = (unsigned int*)d->counters;
  f.chunk_flags = (uint32_t*)d->chunk_flags;
  for (int r = 0; r < kMaxRanks; ++r) {
    f.peer[r] = (const uint8_t*)d->peer[r];
    f.sym_flags[r] = (uint32_t*)d->sym_flags[r];
    f.stage[r] = (uint8_t*)d->stage[r];
    f.local[r] = nullptr;
  }
  int rc;
  const int W = d->world;
  if (d->gather == G_A_ROWS) {
    MSAMP_REQUIRE(d->shard_rows % BM == 0 && d->M == d->shard_rows * W, "gemm_fused: A row shards must be multiples of %d rows", BM);
    for (int r = 0; r < W; ++r) {
      rc = make_map((const void*)d->a[r], d->shard_rows, d->K, d->lda, BM, &maps.a[r]);
      if (rc) return rc;
      f.local[r] = (uint8_t*)d->a[r];
    }
    rc = make_map((const void*)d->b[0], d->N, d->K, d->ldb, bn, &maps.b[0]);
    if (rc) return rc;
    f.shard_tiles = (int)(d->shard_rows / BM);
    f.chunk_rows = BM;
    f.chunk_bytes = (int64_t)BM * d->lda;
    f.chunks_per_shard = f.shard_tiles;
  } else if (d->gather == G_B_ROWS) {
    MSAMP_REQUIRE(d->shard_rows % bn == 0 && d->N == d->shard_rows * W, "gemm_fused: B row shards must be multiples of %d rows", bn);
    for (int r = 0; r < W; ++r) {
      rc = make_map((const void*)d->b[r], d->shard_rows, d->K, d->ldb, bn, &maps.b[r]);
      if (rc) return rc;
      f.local[r] = (uint8_t*)d->b[r];
    }
    rc = make_map((const void*)d->a[0], d->M, d->K, d->lda, BM, &maps.a[0]);
    if (rc) return rc;
    f.shard_tiles = (int)(d->shard_rows / bn);
    f.chunk_rows = bn;
    f.chunk_bytes = (int64_t)bn * d->ldb;
    f.chunks_per_shard = f.shard_tiles;
  } else if (d->gather == G_B_K || d->gather == G_A_K) {
    // shard buffers are [shard_nrows, shard_rows(K part)] with pitch shard_pitch; the other operand is local and complete
    MSAMP_REQUIRE(d->shard_rows % BK == 0 && d->K == d->shard_rows * W, "gemm_fused: K shards must be multiples of %d", BK);
    const bool on_b = d->gather == G_B_K;
    const int tile_rows = on_b ? bn : BM;
    for (int r = 0; r < W; ++r) {
      const void* ptr = (const void*)(on_b ? d->b[r] : d->a[r]);
      rc = make_map(ptr, d->shard_nrows, d->shard_rows, d->shard_pitch, tile_rows, on_b ? &maps.b[r] : &maps.a[r]);
      if (rc) return rc;
      f.local[r] = (uint8_t*)ptr;
    }
    rc = on_b ? make_map((const void*)d->a[0], d->M, d->K, d->lda, BM, &maps.a[0]) : make_map((const void*)d->b[0], d->N, d->K, d->ldb, bn, &maps.b[0]);
    if (rc) return rc;
    f.shard_tiles = (int)(d->shard_rows / BK);
    f.chunk_rows = tile_rows;
    f.chunk_bytes = (int64_t)tile_rows * d->shard_pitch;
    f.chunks_per_shard = (int)((d->shard_nrows + tile_rows - 1) / tile_rows);
    // the last chunk of a shard may be short: it is still copied as a whole chunk, so the shard buffers
    // must be allocated with their row count rounded up to the tile height
  } else {
    rc = make_map((const void*)d->a[0], d->M, d->K, d->lda, BM, &maps.a[0]);
    if (rc) return rc;
    rc = make_map((const void*)d->b[0], d->N, d->K, d->ldb, bn, &maps.b[0]);
    if (rc) return rc;
  }
  if (d->rs) {
    MSAMP_REQUIRE(d->rows_per_rank % BM == 0 && d->M == d->rows_per_rank * W, "gemm_fused: reduce-scatter needs M = world * rows_per_rank, multiple of %d", BM);
    MSAMP_REQUIRE((d->N * (d->out_dtype == DT_F32 ? 4 : 2)) % 16 == 0, "gemm_fused: reduce-scatter needs 16-byte rows");
  }
  if (f.gather && f.n_comm <= 0) f.n_comm = 12;
  MSAMP_DISPATCH_HP(d->out_dtype, T, {
    if (bn == 256) return launch_fused<256, T>(maps, p, f, stream);
    return launch_fused<128, T>(maps, p, f, stream);
  });
  return MSAMP_OK;
}
