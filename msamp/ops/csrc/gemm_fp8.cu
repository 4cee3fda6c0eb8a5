// FP8 GEMM for sm_100a:  D[M,N] = epilogue( (sa_inv * sb_inv) * A[M,K] * B[N,K]^T )
//
// A and B hold e4m3 or e5m2 bytes.  Either operand may be stored K-major ([M,K] resp. [N,K] with K
// contiguous) or MN-major ([K,M] resp. [K,N] with the M / N index contiguous): the tensor core reads
// both layouts from 128-byte-swizzled shared memory, so forward, dgrad and wgrad of a linear layer
// all read x, W and dy in the one layout they were quantised in and no transposed FP8 copy is ever
// written.  The per-tensor scale_inv factors are read from device memory (no host synchronisation).
//
// Two persistent, warp-specialised kernels share the code below:
//   * CTA-pair kernel (default when the problem fills the device): a cluster of two CTAs on the two SMs of a
//     TPC computes a 256 x 256 tile with tcgen05.mma.cta_group::2.  Each CTA loads its own 128 rows of A
//     and its own 128 rows of B with its own TMA (no multicast), i.e. 32 KB per 128-byte K block instead
//     of the 48 KB a single CTA needs for 128 x 256.  The even CTA issues the MMAs for both.
//   * single-CTA kernel (smaller problems, and calls that cap their CTAs): 128 x 256 tiles, or 128 x 128
//     when those would not fill the device.
// Roles:  warp 0 TMA producer (ring of shared-memory stages), warp 1 TMEM allocation + MMA issue,
// warps 2..9 epilogue (tcgen05.ld the fp32 accumulator, scale, bias / residual / GeLU derivative,
// convert, store, optional max|D| and optional quantised copy).  Two accumulator buffers in TMEM
// let the epilogue of tile i overlap the main loop of tile i+1.  Every wait on an mbarrier is
// bounded; when one gives up the CTA sets the device status word, lets its outstanding copies land,
// frees its TMEM and returns.
//
// Replaces the cuBLASLt call behind the reference's Gemm.fp8_gemm (msamp/operators/gemm/gemm.py:121-144)
// and the fp8 transposes around it (msamp/nn/functional.py:81-103).
#include "gemm_common.cuh"

namespace {
using namespace gemm;

// warp 0: TMA producer, warp 1: MMA issuer, warps 2..9: epilogue.  Two epilogue warps share each TMEM lane quarter
// (a warp may only touch the lanes 32 * (warp % 4) ...) and split the columns of the tile between them: with GeLU,
// its derivative, the skip connection or the quantised copy in the epilogue, four warps alone need longer for a tile
// than the tensor core needs for the next one.
constexpr int kThreadsEpi8 = 320;

struct GemmArgs {
  void* d;                    // [M,N] out_dtype, row pitch ldd elements
  const void* bias;           // [N] or null
  const void* residual;       // [M,N] out_dtype with pitch ldr, added to the product (may alias d), or null
  const void* gelu_src;       // [M,N] out_dtype with pitch ldg: the product is multiplied by gelu'(gelu_src), or null
  const float* scale_inv_a;
  const float* scale_inv_b;
  float* amax_out;            // max|D| (or max|gelu(D)| with act == 1); zeroed by the caller
  uint8_t* d8;                // optional FP8 copy of act(D) * (*d8_scale), row pitch ld8 bytes
  const float* d8_scale;
  float* d8_scale_inv_out;    // optional: receives 1 / *d8_scale
  unsigned int* status;
  unsigned long long* stats;  // optional [4 * gridDim.x] cycle counters for tuning: producer wait, MMA wait for data, MMA wait for TMEM, total
  int64_t ldd, ldr, ldg, ld8;
  int M, N, K;
  int bias_dtype;
  int a_fmt, b_fmt, d8_fmt;
  int a_mn, b_mn;             // 1: that operand is stored [K, M] / [K, N]
  int act;                    // 0: identity, 1: amax_out and d8 refer to gelu(D)
  int group_m;                // row tiles per rasterisation group (see tile_to_mn); 0 means all of them
  int tma_store;              // 1: tma_d describes D and full 16-bit tiles are stored through it
  float* colsum;              // optional [N] fp32: += column sums of D as stored (a bias gradient); zeroed by the caller
  int no_d;                   // 1: D itself is not written (only amax_out / d8 / colsum are wanted)
};

template <int BN, bool PAIR, int NSTAGES = 0>
struct Tile {
  static constexpr int TILE_M = PAIR ? 256 : 128;
  static constexpr int B_ROWS = PAIR ? BN / 2 : BN;    // rows of B this CTA keeps in shared memory
  static constexpr int A_BYTES = BM * BK;
  static constexpr int B_BYTES = B_ROWS * BK;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = NSTAGES ? NSTAGES : (PAIR ? 6 : ((BN == 256) ? 4 : 6));
  static constexpr int TILE_BYTES = STAGES * STAGE_BYTES;
  static constexpr int STAGING_OFF = TILE_BYTES + 1024;         // after the barriers, 1024-byte aligned: 4 KB per epilogue warp
  static constexpr int SMEM_BYTES = STAGING_OFF + 8 * 4096 + 1024;    // + manual alignment slack
  static_assert(SMEM_BYTES <= 227 * 1024, "GEMM shared memory");
  static constexpr int TMEM_COLS = 2 * BN;                       // two accumulator buffers
  static constexpr uint32_t TX_BYTES = PAIR ? 2 * STAGE_BYTES : STAGE_BYTES;
};

// Tile index -> (m tile, n tile).  Tiles are walked in groups of group_m row tiles: inside a group the row
// index runs fastest, so the CTAs of one wave share a few A tiles and a few B tiles that stay in L2
// (with a plain column-major walk a wave touches every A tile once and large-K problems stream A
// from HBM once per column of tiles).  The host picks group_m so that a group's slab of A stays well
// inside the 126 MB L2; when all of A fits, one group covers every row tile and B is streamed exactly once.
__device__ __forceinline__ void tile_to_mn(int tile, int num_m, int num_n, int group_m, int& mi, int& ni) {
  const int per_group = group_m * num_n;
  const int g = tile / per_group;
  const int first = g * group_m;
  const int gsize = (num_m - first) < group_m ? (num_m - first) : group_m;
  const int r = tile - g * per_group;
  mi = first + r % gsize;
  ni = r / gsize;
}

template <int FMT>
__device__ __forceinline__ void store_fp8_chunk(uint8_t* dst, const float (&w)[32], float scale, bool vec_ok, int valid) {
  if (vec_ok && valid == 32) {
#pragma unroll
    for (int j = 0; j < 32; j += 16) {
      Bytes16 o;
      uint16_t* e = reinterpret_cast<uint16_t*>(&o);
#pragma unroll
      for (int q = 0; q < 8; ++q) e[q] = f32x2_to_fp8x2<FMT>(w[j + 2 * q] * scale, w[j + 2 * q + 1] * scale);
      *reinterpret_cast<Bytes16*>(dst + j) = o;
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (j < valid) dst[j] = f32_to_fp8<FMT>(w[j] * scale);
  }
}

// Ragged tiles and fp32 outputs: every thread adds its row's values (as rounded to the output type) to the column sums.
template <typename OutT>
__device__ __forceinline__ void colsum_chunk(float* cs, const float (&v)[32], int valid) {
#pragma unroll
  for (int j = 0; j < 32; ++j)
    if (j < valid) atomicAdd(cs + j, to_f32<OutT>(from_f32<OutT>(v[j])));
}

template <int BN, bool PAIR, typename OutT, int NSTAGES = 0>
__global__ void __launch_bounds__(kThreadsEpi8, 1)
gemm_fp8_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                const __grid_constant__ CUtensorMap tma_d, const GemmArgs p) {
  using C = Tile<BN, PAIR, NSTAGES>;
  extern __shared__ uint8_t smem_raw[];
  // 128B-swizzled tiles need 1024-byte alignment (the offset is the same in both CTAs of a pair).
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

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = PAIR ? tc5::cluster_ctarank() : 0u;    // 0: the CTA that issues the MMAs
  const int first_tile = PAIR ? (int)tc5::cluster_id_x() : (int)blockIdx.x;
  const int tile_step = PAIR ? (int)tc5::cluster_count_x() : (int)gridDim.x;

  const int num_m = (p.M + C::TILE_M - 1) / C::TILE_M;
  const int num_n = (p.N + BN - 1) / BN;
  const int num_tiles = num_m * num_n;
  const int num_kb = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; ++s) {
      tc5::mbar_init(full_bar(s), 1);     // the producer of the issuing CTA arrives; bytes of both CTAs are counted
      tc5::mbar_init(empty_bar(s), 1);    // one tcgen05.commit
    }
    for (int b = 0; b < 2; ++b) {
      tc5::mbar_init(tfull_bar(b), 1);
      tc5::mbar_init(tempty_bar(b), PAIR ? 16 : 8);    // the epilogue warps of every CTA that reads this accumulator
    }
    *abort_flag = 0;
    tc5::mbar_fence_init();
    tc5::tma_prefetch_desc(&tma_a);
    tc5::tma_prefetch_desc(&tma_b);
  }
  if (warp == 1) {
    if (PAIR) {
      tc5::tmem_alloc_pair(tc5::smem_u32(tmem_holder), C::TMEM_COLS);
      tc5::tmem_relinquish_pair();
    } else {
      tc5::tmem_alloc(tc5::smem_u32(tmem_holder), C::TMEM_COLS);
      tc5::tmem_relinquish();
    }
  }
  tc5::fence_before_sync();
  __syncthreads();
  if (PAIR) tc5::cluster_sync();    // the partner's barriers exist before anything may signal them
  tc5::fence_after_sync();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (every CTA loads its own halves)
    if (lane == 0) {
      uint32_t it = 0;
      long long st_wait = 0;
      for (int tile = first_tile; tile < num_tiles; tile += tile_step) {
        int mi, ni;
        tile_to_mn(tile, num_m, num_n, p.group_m, mi, ni);
        const int m0 = mi * C::TILE_M + (int)rank * BM;
        const int n0 = ni * BN + (int)rank * C::B_ROWS;
        bool ok = true;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % C::STAGES;
          const uint32_t ph = (it / C::STAGES) & 1;
          const long long t0 = p.stats ? clock64() : 0;
          if (!tc5::mbar_wait(empty_bar(s), ph ^ 1, abort_flag, p.status, 1u)) { ok = false; break; }
          if (p.stats) st_wait += clock64() - t0;
          const uint32_t sa = base + s * C::STAGE_BYTES;
          const uint32_t sb = sa + C::A_BYTES;
          if (PAIR) {
            if (rank == 0) tc5::mbar_arrive_expect_tx(full_bar(s), C::TX_BYTES);
            const uint32_t fb = tc5::map_to_cta(full_bar(s), 0);
            if (p.a_mn) tc5::tma_load_2d_pair(sa, &tma_a, m0, kb * BK, fb);
            else        tc5::tma_load_2d_pair(sa, &tma_a, kb * BK, m0, fb);
            if (p.b_mn) tc5::tma_load_2d_pair(sb, &tma_b, n0, kb * BK, fb);
            else        tc5::tma_load_2d_pair(sb, &tma_b, kb * BK, n0, fb);
          } else {
            tc5::mbar_arrive_expect_tx(full_bar(s), C::TX_BYTES);
            if (p.a_mn) tc5::tma_load_2d(sa, &tma_a, m0, kb * BK, full_bar(s));
            else        tc5::tma_load_2d(sa, &tma_a, kb * BK, m0, full_bar(s));
            if (p.b_mn) {
              // one panel of 128 columns x BK rows per load (the swizzle atom is 128 bytes wide)
#pragma unroll
              for (int pn = 0; pn < C::B_ROWS / 128; ++pn) tc5::tma_load_2d(sb + pn * (128 * BK), &tma_b, n0 + pn * 128, kb * BK, full_bar(s));
            } else {
              tc5::tma_load_2d(sb, &tma_b, kb * BK, n0, full_bar(s));
            }
          }
        }
        if (!ok) break;
      }
      if (p.stats) {
        unsigned int smid;
        asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
        p.stats[4 * blockIdx.x + 0] = (unsigned long long)st_wait | ((unsigned long long)smid << 48);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (one thread per CTA pair)
    if (lane == 0 && rank == 0) {
      const uint32_t idesc = tc5::idesc_f8(C::TILE_M, BN, p.a_fmt, p.b_fmt, p.a_mn, p.b_mn);
      // Descriptor step per 32-element K slice: 32 bytes inside the swizzle atom for a K-major tile,
      // 32 rows of 128 bytes for an MN-major tile (encoded in units of 16 bytes).
      const uint64_t a_step = p.a_mn ? (uint64_t)(32 * 128 / 16) : 2ull;
      const uint64_t b_step = p.b_mn ? (uint64_t)(32 * 128 / 16) : 2ull;
      uint32_t lt = 0;
      long long w_data = 0, w_tmem = 0;
      const long long t_begin = p.stats ? clock64() : 0;
      // The tensor pipe buffers next to nothing.  An M = 128, N = 256, K = 32 MMA runs for 128 cycles, and whatever
      // the issuing thread does between two MMAs beyond about 60 cycles leaves the pipe idle for as long
      // (benchmarks/mma_fp8_shapes.cu: a delay of X cycles per K block costs X cycles per K block; commits and
      // fences are free).  A blocking wait on a stage's barrier between two K blocks costs 100-140 cycles even when
      // the data arrived long ago, which held this loop at 155 cycles per MMA with no loads and no epilogue at all.
      // So the barrier of the NEXT stage is probed, without blocking, before the last MMA of the current K block is
      // issued: the probe's latency overlaps with that issue, and the blocking wait is taken only when the probe
      // failed (133 cycles per MMA in the same experiment).  Polling in a loop instead (here or in the producer)
      // is much worse than the suspending wait: it measured 185-200 cycles per MMA.
      // Stage index, parity and descriptors advance by additions.
      const uint64_t da0 = p.a_mn ? tc5::smem_desc_mn_sw128(base, 128 * BK) : tc5::smem_desc_k_sw128(base);
      const uint64_t db0 = p.b_mn ? tc5::smem_desc_mn_sw128(base + C::A_BYTES, 128 * BK) : tc5::smem_desc_k_sw128(base + C::A_BYTES);
      int s = 0;
      uint32_t ph = 0;
      bool pre_ok = false;
      for (int tile = first_tile; tile < num_tiles; tile += tile_step, ++lt) {
        const int buf = lt & 1;
        const uint32_t aph = (lt >> 1) & 1;
        long long t0 = p.stats ? clock64() : 0;
        if (!tc5::mbar_wait(tempty_bar(buf), aph ^ 1, abort_flag, p.status, 1u)) break;
        if (p.stats) w_tmem += clock64() - t0;
        tc5::fence_after_sync();
        const uint32_t tmem_d = tmem_base + (uint32_t)(buf * BN);
        bool ok = true;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!pre_ok) {
            t0 = p.stats ? clock64() : 0;
            if (!tc5::mbar_wait(full_bar(s), ph, abort_flag, p.status, 1u)) { ok = false; break; }
            if (p.stats) w_data += clock64() - t0;
          }
          tc5::fence_after_sync();
          const uint64_t da = da0 + (uint64_t)(s * (C::STAGE_BYTES >> 4));
          const uint64_t db = db0 + (uint64_t)(s * (C::STAGE_BYTES >> 4));
          int sn = s + 1;
          uint32_t phn = ph;
          if (sn == C::STAGES) { sn = 0; phn ^= 1u; }
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            if (k == BK / UMMA_K - 1) pre_ok = tc5::mbar_test(full_bar(sn), phn);
            if (PAIR) {
              tc5::mma_f8f6f4_pair(tmem_d, da + a_step * k, db + b_step * k, idesc, (kb | k) ? 1u : 0u);
            } else {
              tc5::mma_f8f6f4(tmem_d, da + a_step * k, db + b_step * k, idesc, (kb | k) ? 1u : 0u);
            }
          }
          // frees the stage (in both CTAs: one multicast commit) once these MMAs have read it
          if (PAIR) tc5::mma_commit_pair_mc(empty_bar(s), (uint16_t)3);
          else      tc5::mma_commit(empty_bar(s));
          s = sn;
          ph = phn;
        }
        if (!ok) break;
        if (PAIR) tc5::mma_commit_pair_mc(tfull_bar(buf), (uint16_t)3);    // accumulator complete, in both CTAs' TMEM
        else      tc5::mma_commit(tfull_bar(buf));
      }
      if (p.stats) {
        p.stats[4 * blockIdx.x + 1] = (unsigned long long)w_data;
        p.stats[4 * blockIdx.x + 2] = (unsigned long long)w_tmem;
        p.stats[4 * blockIdx.x + 3] = (unsigned long long)(clock64() - t_begin);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (4 warps per CTA)
    const int q = warp & 3;             // TMEM lane quarter this warp may access
    const int chalf = (warp - 2) >> 2;    // which half of the tile's columns this warp handles
    const float alpha = (*p.scale_inv_a) * (*p.scale_inv_b);
    const float q_scale = p.d8 ? *p.d8_scale : 1.0f;
    if (p.d8_scale_inv_out != nullptr && blockIdx.x == 0 && threadIdx.x == 64) *p.d8_scale_inv_out = __frcp_rn(q_scale);
    OutT* D = reinterpret_cast<OutT*>(p.d);
    const OutT* R = reinterpret_cast<const OutT*>(p.residual);
    const OutT* G = reinterpret_cast<const OutT*>(p.gelu_src);
    const bool vec_ok = ((reinterpret_cast<uintptr_t>(D) & 15) == 0) && ((p.ldd * sizeof(OutT)) % 16 == 0);
    const bool vec_r = R && ((reinterpret_cast<uintptr_t>(R) & 15) == 0) && ((p.ldr * sizeof(OutT)) % 16 == 0);
    const bool vec_g = G && ((reinterpret_cast<uintptr_t>(G) & 15) == 0) && ((p.ldg * sizeof(OutT)) % 16 == 0);
    const bool vec_8 = p.d8 && ((reinterpret_cast<uintptr_t>(p.d8) & 15) == 0) && (p.ld8 % 16 == 0);
    const uint32_t tempty_remote = PAIR ? tc5::map_to_cta(tempty_bar(0), 0) : 0u;
    // 16-bit outputs of full tiles go through a per-warp staging buffer of 32 rows x 128 bytes: the thread that owns a
    // row writes its 64 converted columns there (16-byte pieces XOR-swizzled by row), then the warp writes the rows out
    // with every store instruction covering four complete 128-byte lines.  Storing straight from the row-per-thread
    // layout touches 32 different lines with 16 bytes each per instruction, which cost 11 % of the GEMM on N >= 12288.
    const uint32_t stage = base + (uint32_t)C::STAGING_OFF + (uint32_t)(warp - 2) * 4096u;
    const bool staged_ok = sizeof(OutT) == 2 && ((vec_ok && p.tma_store != 0) || p.no_d != 0);
    float amax = 0.0f;
    uint32_t lt = 0;
    for (int tile = first_tile; tile < num_tiles; tile += tile_step, ++lt) {
      int mi, ni;
      tile_to_mn(tile, num_m, num_n, p.group_m, mi, ni);
      const int m0 = mi * C::TILE_M + (int)rank * BM;
      const int n0 = ni * BN;
      const int buf = lt & 1;
      const uint32_t aph = (lt >> 1) & 1;
      const int row = m0 + q * 32 + lane;
      const bool full_tile = staged_ok && (m0 + q * 32 + 32 <= p.M) && (n0 + BN <= p.N);    // uniform over the warp
      if ((R != nullptr || G != nullptr) && row < p.M) {
        // While the main loop of this tile is still running, pull this thread's slice of the residual / GeLU
        // source into L2, so that the loads below do not wait for HBM one chunk at a time.
        const OutT* src = R != nullptr ? R + (int64_t)row * p.ldr + n0 : G + (int64_t)row * p.ldg + n0;
        const int cols_here = (p.N - n0) < BN ? (p.N - n0) : BN;
        for (int b = 0; b < cols_here * (int)sizeof(OutT); b += 128)
          asm volatile("prefetch.global.L2 [%0];" ::"l"(reinterpret_cast<const char*>(src) + b));
      }
      if (!tc5::mbar_wait(tfull_bar(buf), aph, abort_flag, p.status, 1u)) break;
      tc5::fence_after_sync();
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * BN);
#pragma unroll 1
      for (int c = chalf * (BN / 64); c < (chalf + 1) * (BN / 64); ++c) {
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
          if (p.bias != nullptr) {
            if (p.bias_dtype == DT_F32) {
              const float* b = reinterpret_cast<const float*>(p.bias) + col;
              if (valid == 32 && (reinterpret_cast<uintptr_t>(b) & 15) == 0) {
#pragma unroll
                for (int j = 0; j < 32; j += 4) {
                  const float4 t = __ldg(reinterpret_cast<const float4*>(b + j));
                  v[j] += t.x; v[j + 1] += t.y; v[j + 2] += t.z; v[j + 3] += t.w;
                }
              } else {
#pragma unroll
                for (int j = 0; j < 32; ++j) if (j < valid) v[j] += __ldg(b + j);
              }
            } else if (p.bias_dtype == DT_BF16) {
              const __nv_bfloat16* b = reinterpret_cast<const __nv_bfloat16*>(p.bias) + col;
#pragma unroll
              for (int j = 0; j < 32; ++j) if (j < valid) v[j] += __bfloat162float(b[j]);
            } else {
              const __half* b = reinterpret_cast<const __half*>(p.bias) + col;
#pragma unroll
              for (int j = 0; j < 32; ++j) if (j < valid) v[j] += __half2float(b[j]);
            }
          }
          if (R != nullptr) {
            float old[32];
            load_chunk<OutT>(R + (int64_t)row * p.ldr + col, old, vec_r, valid);
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] += old[j];
          }
          if (G != nullptr) {
            float h[32];
            load_chunk<OutT>(G + (int64_t)row * p.ldg + col, h, vec_g, valid);
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] *= gelu_grad_f(h[j]);
          }
          OutT* dst = D + (int64_t)row * p.ldd + col;
          if constexpr (sizeof(OutT) == 2) {
            if (full_tile) {
              const uint32_t srow = stage + (uint32_t)lane * 128u;
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                Bytes16 o;
                OutT* e = reinterpret_cast<OutT*>(&o);
#pragma unroll
                for (int t = 0; t < 8; ++t) e[t] = from_f32<OutT>(v[8 * j + t]);
                const uint32_t piece = (uint32_t)((c & 1) * 4 + j);
                const uint4 u = *reinterpret_cast<const uint4*>(&o);
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(srow + ((piece ^ (uint32_t)(lane & 7)) << 4)), "r"(u.x),
                             "r"(u.y), "r"(u.z), "r"(u.w)
                             : "memory");
              }
              if (c & 1) {
                // the staging rows are laid out exactly as a 128-byte-swizzled TMA box of 32 rows x 128 bytes: one thread
                // hands them to the TMA unit, which writes complete lines without occupying the load/store path
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0 && !p.no_d) {
                  tc5::tma_store_2d(&tma_d, stage, (col - 32) * (int)sizeof(OutT), m0 + q * 32);
                  tc5::bulk_commit_group();
                }
                if (p.colsum != nullptr) {
                  // column sums of the 32 staged rows: lane L owns columns 2L and 2L + 1 of the 64-column group and walks
                  // down the rows (one 4-byte word per row; a row's 32 words are a permutation of its 128 bytes, so the
                  // reads of a warp are conflict free)
                  float s0 = 0.0f, s1 = 0.0f;
                  const uint32_t piece = (uint32_t)lane >> 2, word = ((uint32_t)lane & 3u) * 4u;
#pragma unroll 8
                  for (uint32_t r = 0; r < 32; ++r) {
                    uint32_t wv;
                    asm volatile("ld.shared.b32 %0, [%1];" : "=r"(wv) : "r"(stage + r * 128u + ((piece ^ (r & 7u)) << 4) + word));
                    const OutT* e2 = reinterpret_cast<const OutT*>(&wv);
                    s0 += to_f32<OutT>(e2[0]);
                    s1 += to_f32<OutT>(e2[1]);
                  }
                  atomicAdd(p.colsum + (col - 32) + 2 * lane, s0);
                  atomicAdd(p.colsum + (col - 32) + 2 * lane + 1, s1);
                }
                if (lane == 0 && !p.no_d) tc5::bulk_wait_read<0>();    // the buffer is rewritten by the next 64 columns
                __syncwarp();
              }
            } else {
              if (!p.no_d) store_chunk<OutT>(dst, v, vec_ok, valid);
              if (p.colsum != nullptr) colsum_chunk<OutT>(p.colsum + col, v, valid);
            }
          } else {
            if (!p.no_d) store_chunk<OutT>(dst, v, vec_ok, valid);
            if (p.colsum != nullptr) colsum_chunk<OutT>(p.colsum + col, v, valid);
          }
          if (p.amax_out != nullptr || p.d8 != nullptr) {
            // statistics and the quantised copy are taken from the values as stored (rounded to the
            // output type), so that they equal what a separate pass over D would produce
            float w[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              float t = to_f32<OutT>(from_f32<OutT>(v[j]));
              w[j] = p.act ? to_f32<OutT>(from_f32<OutT>(gelu_f(t))) : t;
            }
            if (p.amax_out != nullptr) {
#pragma unroll
              for (int j = 0; j < 32; ++j) if (j < valid) amax = fmaxf(amax, abs_nan_to_inf(w[j]));
            }
            if (p.d8 != nullptr) {
              uint8_t* d8 = p.d8 + (int64_t)row * p.ld8 + col;
              if (p.d8_fmt == FMT_E4M3) store_fp8_chunk<FMT_E4M3>(d8, w, q_scale, vec_8, valid);
              else                      store_fp8_chunk<FMT_E5M2>(d8, w, q_scale, vec_8, valid);
            }
          }
        }
      }
      tc5::fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        if (PAIR) tc5::mbar_arrive_cluster(tempty_remote + 8u * buf);
        else      tc5::mbar_arrive(tempty_bar(buf));
      }
    }
    if (lane == 0) tc5::bulk_wait_all<0>();    // TMA stores of this warp have landed before the CTA goes away
    if (p.amax_out != nullptr) {
      amax = warp_max(amax);
      if (lane == 0) atomic_max_nonneg(p.amax_out, amax);
    }
  }

  // ---------------------------------------------------------------------- tear-down
  __syncwarp();
  if (*abort_flag) __nanosleep(200000);    // let copies / MMAs in flight finish before smem and TMEM go away
  tc5::fence_before_sync();
  __syncthreads();
  if (PAIR) tc5::cluster_sync();    // the partner may still read this CTA's operands or signal its barriers
  tc5::fence_after_sync();
  if (warp == 1) {
    if (PAIR) tc5::tmem_dealloc_pair(tmem_base, C::TMEM_COLS);
    else      tc5::tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

// Co-resident CTA pairs the device can hold for the pair kernel (one CTA per SM, clusters of two).
template <int BN, typename OutT, int NSTAGES>
int max_pairs(int smem_bytes) {
  static int cached[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  dev &= 63;
  if (cached[dev] == 0) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * (unsigned)msamp_sm_count(), 1, 1);
    cfg.blockDim = dim3(kThreadsEpi8, 1, 1);
    cfg.dynamicSmemBytes = (size_t)smem_bytes;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, gemm_fp8_kernel<BN, true, OutT, NSTAGES>, &cfg) != cudaSuccess || n <= 0) {
      cudaGetLastError();
      n = msamp_sm_count() / 2;
    }
    cached[dev] = n;
  }
  return cached[dev];
}

template <int BN, bool PAIR, typename OutT, int NSTAGES = 0>
int launch(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& md, const GemmArgs& p, int max_ctas, cudaStream_t stream) {
  using C = Tile<BN, PAIR, NSTAGES>;
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!configured[dev & 63]) {
    cudaError_t e = cudaFuncSetAttribute(gemm_fp8_kernel<BN, PAIR, OutT, NSTAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
    if (e != cudaSuccess) {
      msamp_set_error("cudaFuncSetAttribute: %s", cudaGetErrorString(e));
      return MSAMP_ELAUNCH;
    }
    configured[dev & 63] = true;
  }
  const int num_tiles = ((p.M + C::TILE_M - 1) / C::TILE_M) * ((p.N + BN - 1) / BN);
  if (PAIR) {
    int pairs = max_pairs<BN, OutT, NSTAGES>(C::SMEM_BYTES);
    if (max_ctas > 0 && max_ctas / 2 < pairs) pairs = max_ctas / 2 > 0 ? max_ctas / 2 : 1;
    if (num_tiles < pairs) pairs = num_tiles;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * (unsigned)pairs, 1, 1);
    cfg.blockDim = dim3(kThreadsEpi8, 1, 1);
    cfg.dynamicSmemBytes = C::SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_fp8_kernel<BN, PAIR, OutT, NSTAGES>, ma, mb, md, p);
    if (e != cudaSuccess) {
      msamp_set_error("gemm_fp8 pair kernel launch: %s", cudaGetErrorString(e));
      cudaGetLastError();
      return MSAMP_ELAUNCH;
    }
    return msamp_check_launch("gemm_fp8_kernel(pair)");
  }
  int grid = msamp_sm_count();
  if (max_ctas > 0 && max_ctas < grid) grid = max_ctas;
  if (num_tiles < grid) grid = num_tiles;
  gemm_fp8_kernel<BN, PAIR, OutT, NSTAGES><<<grid, kThreadsEpi8, C::SMEM_BYTES, stream>>>(ma, mb, md, p);
  return msamp_check_launch("gemm_fp8_kernel");
}

}    // namespace

// Full description of one GEMM call (see the fields of GemmArgs above for the epilogue options).
//   a: [M,K] bytes with row pitch lda when a_mn == 0, else [K,M] with row pitch lda
//   b: [N,K] with row pitch ldb when b_mn == 0, else [K,N]
// The contiguous dimension of each operand, its pitch and its base address must be multiples of 16 bytes
// (TMA rules).  tile: 0 = choose, 1 = CTA-pair 256x256, 2 = single CTA.
struct MsampGemmDesc {
  const void* a;
  const void* b;
  void* d;
  const void* bias;
  const void* residual;
  const void* gelu_src;
  const float* scale_inv_a;
  const float* scale_inv_b;
  float* amax_out;
  void* d8;
  const float* d8_scale;
  float* d8_scale_inv_out;
  int64_t lda, ldb, ldd, ldr, ldg, ld8;
  int M, N, K;
  int a_fmt, b_fmt, d8_fmt;
  int a_mn, b_mn;
  int out_dtype, bias_dtype;
  int act;
  int max_ctas;
  int tile;
  unsigned long long* stats;    // optional tuning counters, 4 per CTA (see GemmArgs)
  float* colsum;                // optional [N] fp32, += column sums of D as stored; zeroed by the caller
};

MSAMP_API int msamp_gemm_fp8_ex(const MsampGemmDesc* g, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  const int M = g->M, N = g->N, K = g->K;
  MSAMP_REQUIRE(M > 0 && N > 0 && K > 0, "msamp_gemm_fp8: empty problem M=%d N=%d K=%d", M, N, K);
  MSAMP_REQUIRE(g->lda % 16 == 0 && g->ldb % 16 == 0, "msamp_gemm_fp8: the row pitches must be multiples of 16");
  MSAMP_REQUIRE((g->a_mn ? M : K) % 16 == 0 && (g->b_mn ? N : K) % 16 == 0,
                "msamp_gemm_fp8: the contiguous dimension of each operand must be a multiple of 16");
  MSAMP_REQUIRE((reinterpret_cast<uintptr_t>(g->a) & 15) == 0 && (reinterpret_cast<uintptr_t>(g->b) & 15) == 0,
                "msamp_gemm_fp8: operands must be 16-byte aligned");
  MSAMP_REQUIRE(g->scale_inv_a && g->scale_inv_b, "msamp_gemm_fp8: null pointer");
  MSAMP_REQUIRE(g->d != nullptr || g->d8 != nullptr || g->amax_out != nullptr || g->colsum != nullptr,
                "msamp_gemm_fp8: no output requested");
  MSAMP_REQUIRE(g->d != nullptr || (g->residual == nullptr), "msamp_gemm_fp8: a residual needs the output it is added to");
  MSAMP_REQUIRE(g->d8 == nullptr || g->d8_scale != nullptr, "msamp_gemm_fp8: a quantised copy needs its scale");
  const int sms = msamp_sm_count();
  // Tile choice.  Problems that fill the device with 256-wide tiles run on the CTA-pair kernel (256x256 tiles over two
  // SMs): it moves a third less data per FLOP through L2 and shared memory, and since the MMA issue loop stopped
  // leaving the tensor pipe idle between K blocks that is what counts: under the 1 kW power cap a GPT-7B step measured
  // 235.6 ms with it, 239.5 ms with single-CTA 128x256 tiles and 237.2 ms with the pair kernel everywhere but in the
  // weight-gradient layout (same GPU, same run).  Calls that cap their CTAs to share the GPU with a communication
  // kernel, and smaller problems, use single-CTA 128x256 or 128x128 tiles.
  const int64_t tiles_256 = (int64_t)((M + BM - 1) / BM) * ((N + 255) / 256);
  int tile = g->tile;
  if (tile == 0) tile = (N > 128 && tiles_256 >= 2 * sms && g->max_ctas <= 0) ? 1 : 2;
  const bool pair = tile == 1;
  const int bn = pair ? 256 : ((N > 128 && tiles_256 >= sms) ? 256 : 128);
  CUtensorMap ma, mb;
  int rc;
  if (g->a_mn) rc = make_map(g->a, K, M, g->lda, BK, &ma);
  else         rc = make_map(g->a, M, K, g->lda, BM, &ma);
  if (rc) return rc;
  if (g->b_mn) rc = make_map(g->b, K, N, g->ldb, BK, &mb);
  else         rc = make_map(g->b, N, K, g->ldb, pair ? bn / 2 : bn, &mb);
  if (rc) return rc;
  // 16-bit outputs of full tiles are written by TMA from the epilogue's staging buffers: a byte view of D with boxes of
  // 32 rows x 128 bytes.  Without it (fp32 output, unaligned D) the map argument is a placeholder that is never used.
  CUtensorMap md = ma;
  int tma_store = 0;
  {
    const int esize = g->out_dtype == DT_F32 ? 4 : 2;
    if (g->d != nullptr && esize == 2 && (reinterpret_cast<uintptr_t>(g->d) & 15) == 0 && (g->ldd * esize) % 16 == 0 && N >= 128 &&
        make_map(g->d, M, (int64_t)N * esize, g->ldd * esize, 32, &md) == MSAMP_OK)
      tma_store = 1;
    else
      md = ma;
  }
  GemmArgs p;
  p.tma_store = tma_store;
  p.colsum = g->colsum;
  p.no_d = g->d == nullptr ? 1 : 0;
  p.d = g->d; p.bias = g->bias; p.residual = g->residual; p.gelu_src = g->gelu_src;
  p.scale_inv_a = g->scale_inv_a; p.scale_inv_b = g->scale_inv_b; p.amax_out = g->amax_out;
  p.d8 = (uint8_t*)g->d8; p.d8_scale = g->d8_scale; p.d8_scale_inv_out = g->d8 ? g->d8_scale_inv_out : nullptr;
  p.status = msamp_device_status_ptr();
  p.stats = g->stats;
  p.ldd = g->ldd; p.ldr = g->ldr; p.ldg = g->ldg; p.ld8 = g->ld8;
  p.M = M; p.N = N; p.K = K; p.bias_dtype = g->bias_dtype;
  p.a_fmt = g->a_fmt; p.b_fmt = g->b_fmt; p.d8_fmt = g->d8_fmt; p.a_mn = g->a_mn ? 1 : 0; p.b_mn = g->b_mn ? 1 : 0; p.act = g->act;
  {
    const int tile_m = pair ? 256 : BM;
    const int num_m = (M + tile_m - 1) / tile_m;
    int64_t grp = (48ll << 20) / ((int64_t)tile_m * K);    // row tiles whose A slab is about 48 MB
    if (grp < 4) grp = 4;
    p.group_m = grp >= num_m ? num_m : (int)grp;
  }
  MSAMP_DISPATCH_HP(g->out_dtype, T, {
    if (pair) return launch<256, true, T>(ma, mb, md, p, g->max_ctas, stream);
    if (bn == 256) return launch<256, false, T>(ma, mb, md, p, g->max_ctas, stream);
    return launch<128, false, T>(ma, mb, md, p, g->max_ctas, stream);
  });
  return MSAMP_OK;
}

// A: [M, K] fp8 bytes with row pitch lda (bytes), B: [N, K] with pitch ldb, D: [M, N] of out_dtype
// with row pitch ldd (elements).  K, lda, ldb must be multiples of 16 and A, B 16-byte aligned
// (TMA rules).  bias may be null; amax_out (nullable) must be zeroed by the caller and receives
// max|D|.  max_ctas > 0 caps the number of persistent CTAs (to leave SMs to a concurrent kernel).
MSAMP_API int msamp_gemm_fp8(const void* A, const void* B, void* D, int M, int N, int K, int64_t lda, int64_t ldb, int64_t ldd,
                             int a_fmt, int b_fmt, int out_dtype, const float* scale_inv_a, const float* scale_inv_b,
                             const void* bias, int bias_dtype, int accumulate, float* amax_out, int max_ctas, void* stream_) {
  MsampGemmDesc g = {};
  g.a = A; g.b = B; g.d = D; g.bias = bias; g.residual = accumulate ? D : nullptr; g.ldr = ldd;
  g.scale_inv_a = scale_inv_a; g.scale_inv_b = scale_inv_b; g.amax_out = amax_out;
  g.lda = lda; g.ldb = ldb; g.ldd = ldd; g.M = M; g.N = N; g.K = K; g.a_fmt = a_fmt; g.b_fmt = b_fmt;
  g.out_dtype = out_dtype; g.bias_dtype = bias_dtype; g.max_ctas = max_ctas;
  return msamp_gemm_fp8_ex(&g, stream_);
}
