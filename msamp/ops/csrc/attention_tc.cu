// Softmax attention for bf16, head size 128, on the sm_100a tensor path (tcgen05 + TMEM + TMA).
//
// Three warp-specialised kernels share one structure: warp 0 streams operand tiles with TMA
// (4-D tensor maps over the strided [batch, seq, head, 128] views, 128-byte swizzle), warp 1 issues
// tcgen05.mma (kind::f16) into TMEM, and warps 2..9 (one thread per accumulator row) read the scores
// back with tcgen05.ld, do the softmax arithmetic and write the bf16 probability operand into
// swizzled shared memory for the next MMA.
//
//   forward   CTA = 128 query rows, key tiles of 64:  S = Q K^T  ->  P = exp2(S - m)  ->  O += P V.
//             Two groups of softmax warps take alternating key tiles; K, V, S and P live in rings
//             four tiles deep, so scores are ready ahead of the group that needs them; O
//             accumulates in TMEM (one accumulator per group) and is rescaled lazily.
//   dK/dV     CTA = 128 key rows, query tiles of 64:  S^T = K Q^T, dP^T = V dO^T,
//             dV += P^T dO, dK += dS^T Q, both accumulated in TMEM over the whole loop.
//   dQ        CTA = 128 query rows, key tiles of 64:  S = Q K^T, dP = dO V^T, dQ += dS K in TMEM.
//
// V, dO, Q and K enter the second kind of product with the reduction index as rows of the tile, so
// the same shared-memory tile is described once K-major and once MN-major; nothing is transposed.
// The backward pass is deterministic (no atomics).  Every mbarrier wait is bounded; when one gives
// up, bit 2 (value 4) of the device status word is set and the CTA frees its TMEM and returns.
//
// Same arithmetic as the mma.sync kernels in attention.cu, which remain the path for head size 64.
#include <cstdlib>
#include <mutex>
#include <unordered_map>

#include "tcgen05.cuh"

namespace {

constexpr int kTcThreads = 320;    // warp 0: TMA, warp 1: MMA, warps 2-5 and 6-9: the two softmax groups
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr unsigned int kStatusBit = 4u;

struct TcParams {
  __nv_bfloat16* o;
  float* lse;             // [b, h, s] natural-log sum-exp of the scaled scores
  const float* delta;     // [b, h, s] rowsum(dO * O)
  __nv_bfloat16* dq;
  __nv_bfloat16* dk;
  __nv_bfloat16* dv;
  int64_t o_sb, o_ss, o_sh;    // element strides: batch, sequence, head
  int64_t dq_sb, dq_ss, dq_sh;
  int64_t dk_sb, dk_ss, dk_sh;
  int64_t dv_sb, dv_ss, dv_sh;
  int batch, heads, seqlen, causal;
  float scale;
  unsigned int* status;
};

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 t = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&t);
}
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
// Makes this thread's ordinary shared-memory writes visible to the async proxy (the MMA reads them).
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// 128 fp32 values of one row -> bf16 -> 256 contiguous bytes in global memory.
__device__ __forceinline__ void st_row32(__nv_bfloat16* dst, const float (&v)[32]) {
  uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    uint4 u;
    u.x = pack_bf16(v[8 * t], v[8 * t + 1]);
    u.y = pack_bf16(v[8 * t + 2], v[8 * t + 3]);
    u.z = pack_bf16(v[8 * t + 4], v[8 * t + 5]);
    u.w = pack_bf16(v[8 * t + 6], v[8 * t + 7]);
    d4[t] = u;
  }
}

#define TC_WAIT(bar_, ph_) \
  if (!tc5::mbar_wait((bar_), (ph_), abort_flag, p.status, kStatusBit)) break

// ============================================================================================ forward
namespace fwd {
constexpr int NB = 4;                         // ring depth of the K, V, S and P buffers (key tile j uses slot j & 3)
constexpr uint32_t PANEL_Q = 128 * 128;       // [128 query rows][64 bf16]
constexpr uint32_t TILE_Q = 2 * PANEL_Q;
constexpr uint32_t PANEL_KV = 64 * 128;       // [64 key rows][64 bf16]
constexpr uint32_t TILE_KV = 2 * PANEL_KV;    // 16 KB
constexpr uint32_t TILE_P = 128 * 128;        // [128 query rows][64 keys] bf16
constexpr uint32_t OFF_Q = 0, OFF_K = TILE_Q, OFF_V = OFF_K + NB * TILE_KV, OFF_P = OFF_V + NB * TILE_KV, OFF_BAR = OFF_P + NB * TILE_P;
enum { B_Q = 0, B_KF = 1, B_KE = B_KF + NB, B_VF = B_KE + NB, B_VE = B_VF + NB, B_SF = B_VE + NB, B_SE = B_SF + NB, B_PF = B_SE + NB,
       B_PE = B_PF + NB, B_OF = B_PE + NB, B_ACC = B_OF + 2, NBAR = B_ACC + 1 };
constexpr int SMEM = OFF_BAR + NBAR * 8 + 16 + 1024;
constexpr uint32_t TM_S = 0, TM_O = 256, TM_COLS = 512;    // four 64-column score buffers, two 128-column outputs
constexpr float kRescaleStep = 8.0f;    // the reference maximum may lag the true one by 2^8
}    // namespace fwd

// The two softmax groups work on alternating key tiles (64 keys each) and never exchange anything
// inside the loop: group g owns the score and probability slots of its tiles and its own output
// accumulator O_g in TMEM with its own reference maximum m_g and row sum l_g, i.e. each group computes
// attention over its half of the key tiles and the halves are merged once at the end.  Scores are
// computed up to four tiles ahead, so a group finds its next S ready when it has finished a tile.
// O_g stays in TMEM and is accumulated by the MMA itself; it is only read back and rescaled when a
// row's maximum grew by more than kRescaleStep since the last rescale (probabilities then stay
// below 2^8, far inside bf16/fp32 range).
__global__ void __launch_bounds__(kTcThreads, 1)
attn_fwd_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                   const __grid_constant__ CUtensorMap map_v, const TcParams p) {
  using namespace fwd;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = tc5::smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw_addr);
  const uint32_t bars = base + OFF_BAR;
  auto bar = [&](int i) { return bars + 8u * (uint32_t)i; };
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(smem + OFF_BAR + NBAR * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
  // Wait used by full warps that go on to warp-collective TMEM accesses: the outcome is made uniform.
  auto wait_warp = [&](uint32_t br, uint32_t ph) {
    return __all_sync(0xffffffffu, tc5::mbar_wait(br, ph, abort_flag, p.status, kStatusBit)) != 0;
  };

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int qt = (int)gridDim.x - 1 - (int)blockIdx.x;    // long rows first
  const int bh = blockIdx.y;
  const int b = bh / p.heads;
  const int h = bh - b * p.heads;
  const int q0 = qt * 128;
  const int n_all = (p.seqlen + 63) / 64;
  const int n_kv = p.causal ? min(2 * qt + 2, n_all) : n_all;

  if (threadIdx.x == 0) {
    tc5::mbar_init(bar(B_Q), 1);
    for (int s = 0; s < NB; ++s) {
      tc5::mbar_init(bar(B_KF + s), 1);
      tc5::mbar_init(bar(B_KE + s), 1);
      tc5::mbar_init(bar(B_VF + s), 1);
      tc5::mbar_init(bar(B_VE + s), 1);
      tc5::mbar_init(bar(B_SF + s), 1);
      tc5::mbar_init(bar(B_SE + s), 4);
      tc5::mbar_init(bar(B_PF + s), 4);
      tc5::mbar_init(bar(B_PE + s), 1);
    }
    tc5::mbar_init(bar(B_OF + 0), 1);
    tc5::mbar_init(bar(B_OF + 1), 1);
    tc5::mbar_init(bar(B_ACC), 1);
    *abort_flag = 0;
    tc5::mbar_fence_init();
    tc5::tma_prefetch_desc(&map_q);
    tc5::tma_prefetch_desc(&map_k);
    tc5::tma_prefetch_desc(&map_v);
  }
  if (warp == 1) {
    tc5::tmem_alloc(tc5::smem_u32(tmem_holder), TM_COLS);
    tc5::tmem_relinquish();
  }
  tc5::fence_before_sync();
  __syncthreads();
  tc5::fence_after_sync();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tc5::mbar_arrive_expect_tx(bar(B_Q), TILE_Q);
      tc5::tma_load_4d(base + OFF_Q, &map_q, 0, h, q0, b, bar(B_Q));
      tc5::tma_load_4d(base + OFF_Q + PANEL_Q, &map_q, 64, h, q0, b, bar(B_Q));
      for (int j = 0; j < n_kv; ++j) {
        const int s = j & (NB - 1);
        const uint32_t ph = (uint32_t)(j / NB) & 1u;
        TC_WAIT(bar(B_KE + s), ph ^ 1u);
        tc5::mbar_arrive_expect_tx(bar(B_KF + s), TILE_KV);
        tc5::tma_load_4d(base + OFF_K + s * TILE_KV, &map_k, 0, h, j * 64, b, bar(B_KF + s));
        tc5::tma_load_4d(base + OFF_K + s * TILE_KV + PANEL_KV, &map_k, 64, h, j * 64, b, bar(B_KF + s));
        TC_WAIT(bar(B_VE + s), ph ^ 1u);
        tc5::mbar_arrive_expect_tx(bar(B_VF + s), TILE_KV);
        tc5::tma_load_4d(base + OFF_V + s * TILE_KV, &map_v, 0, h, j * 64, b, bar(B_VF + s));
        tc5::tma_load_4d(base + OFF_V + s * TILE_KV + PANEL_KV, &map_v, 64, h, j * 64, b, bar(B_VF + s));
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc_s = tc5::idesc_bf16(128, 64, 0, 0);
      const uint32_t idesc_o = tc5::idesc_bf16(128, 128, 0, 1);
      // S[j&3] = Q K_j^T
      auto issue_s = [&](int j) -> bool {
        const int s = j & (NB - 1);
        const uint32_t ph = (uint32_t)(j / NB) & 1u;
        if (!tc5::mbar_wait(bar(B_SE + s), ph ^ 1u, abort_flag, p.status, kStatusBit)) return false;
        if (!tc5::mbar_wait(bar(B_KF + s), ph, abort_flag, p.status, kStatusBit)) return false;
        tc5::fence_after_sync();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t offa = (uint32_t)(kk >> 2) * PANEL_Q + (uint32_t)(kk & 3) * 32u;
          const uint32_t offb = (uint32_t)(kk >> 2) * PANEL_KV + (uint32_t)(kk & 3) * 32u;
          tc5::mma_f16(tmem_base + TM_S + (uint32_t)s * 64u, tc5::smem_desc_k_sw128(base + OFF_Q + offa),
                       tc5::smem_desc_k_sw128(base + OFF_K + s * TILE_KV + offb), idesc_s, kk ? 1u : 0u);
        }
        tc5::mma_commit(bar(B_KE + s));
        tc5::mma_commit(bar(B_SF + s));
        return true;
      };
      do {
        TC_WAIT(bar(B_Q), 0u);
        bool ok = true;
        for (int j = 0; j < NB && j < n_kv; ++j)
          if (!issue_s(j)) { ok = false; break; }
        if (!ok) break;
        for (int j = 0; j < n_kv; ++j) {
          const int s = j & (NB - 1);
          const uint32_t ph = (uint32_t)(j / NB) & 1u;
          if (!tc5::mbar_wait(bar(B_PF + s), ph, abort_flag, p.status, kStatusBit)) { ok = false; break; }
          if (!tc5::mbar_wait(bar(B_VF + s), ph, abort_flag, p.status, kStatusBit)) { ok = false; break; }
          tc5::fence_after_sync();
          // O[j&1] (+)= P_j V_j : A = P (K-major), B = V with the key index as rows (MN-major)
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            tc5::mma_f16(tmem_base + TM_O + (uint32_t)(j & 1) * 128u, tc5::smem_desc_k_sw128(base + OFF_P + s * TILE_P + (uint32_t)kk * 32u),
                         tc5::smem_desc_mn_sw128(base + OFF_V + s * TILE_KV + (uint32_t)kk * 2048u, PANEL_KV), idesc_o,
                         (j >= 2 || kk) ? 1u : 0u);
          }
          tc5::mma_commit(bar(B_VE + s));
          tc5::mma_commit(bar(B_PE + s));
          tc5::mma_commit(bar(B_OF + (j & 1)));
          if (j + NB < n_kv && !issue_s(j + NB)) { ok = false; break; }
        }
        if (ok) tc5::mma_commit(bar(B_ACC));
      } while (false);
    }
  } else {
    // ------------------------------------------------------------------ softmax: one thread per query row and group
    const int qd = warp & 3;           // TMEM lane quarter this warp may access
    const int wg = (warp - 2) >> 2;    // group 0: even key tiles, group 1: odd key tiles
    const int row = qd * 32 + lane;
    const int grow = q0 + row;
    const uint32_t tlane = tmem_base + ((uint32_t)(qd * 32) << 16);
    const uint32_t to = tlane + TM_O + (uint32_t)wg * 128u;
    const float sl = p.scale * kLog2e;
    const int lim = p.causal ? min(grow, p.seqlen - 1) : p.seqlen - 1;    // last visible column
    const uint32_t swz = (uint32_t)(row & 7);
    float m = -INFINITY, l = 0.0f;    // reference maximum (log2 units) and row sum of this group
    bool ok = true;

    for (int j = wg; j < n_kv; j += 2) {
      const int s = j & (NB - 1);
      const uint32_t ph = (uint32_t)(j / NB) & 1u;
      const int k = j >> 1;    // index of this tile within the group
      if (!wait_warp(bar(B_SF + s), ph)) { ok = false; break; }
      tc5::fence_after_sync();
      uint32_t r[2][32];
      tc5::tmem_ld32(tlane + TM_S + (uint32_t)s * 64u, r[0]);
      tc5::tmem_ld32(tlane + TM_S + (uint32_t)s * 64u + 32u, r[1]);
      tc5::tmem_ld_wait();
      tc5::fence_before_sync();
      __syncwarp();
      if (lane == 0) tc5::mbar_arrive(bar(B_SE + s));    // the slot may take the scores of tile j + 4
      const int col0 = j * 64;
      const bool need_mask = (p.causal && col0 + 63 > q0) || (col0 + 64 > p.seqlen);
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
      if (need_mask) {
#pragma unroll
        for (int i = 0; i < 64; ++i)
          if (col0 + i <= lim) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(r[i >> 5][i & 31]));
      } else {
#pragma unroll
        for (int i = 0; i < 64; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(r[i >> 5][i & 31]));
      }
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * sl;    // sl > 0
      const bool grow_m = mx > m + kRescaleStep || (m == -INFINITY && mx > -INFINITY);
      if (__any_sync(0xffffffffu, grow_m)) {
        const float m_new = grow_m ? mx : m;
        const float corr = (m == -INFINITY) ? 0.0f : ex2(m - m_new);
        if (k > 0) {
          // every earlier product of this group must have landed in O before it is rescaled
          if (!wait_warp(bar(B_OF + wg), (uint32_t)(k - 1) & 1u)) { ok = false; break; }
          tc5::fence_after_sync();
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            uint32_t x[32];
            tc5::tmem_ld32(to + (uint32_t)c * 32u, x);
            tc5::tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) x[i] = __float_as_uint(__uint_as_float(x[i]) * corr);
            tc5::tmem_st32(to + (uint32_t)c * 32u, x);
          }
          tc5::tmem_st_wait();
        }
        l *= corr;
        m = m_new;
      }
      if (!wait_warp(bar(B_PE + s), ph ^ 1u)) { ok = false; break; }
      const float m_use = (m == -INFINITY) ? 0.0f : m;
      float sum4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
      const uint32_t prow = base + OFF_P + s * TILE_P + (uint32_t)row * 128u;
#pragma unroll
      for (int g = 0; g < 8; ++g) {    // 16-byte chunk g = columns 8g .. 8g+7
        float e[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          e[i] = ex2(fmaf(__uint_as_float(r[g >> 2][(g & 3) * 8 + i]), sl, -m_use));
          if (need_mask && col0 + g * 8 + i > lim) e[i] = 0.0f;
          sum4[i & 3] += e[i];
        }
        st_shared_v4(prow + ((((uint32_t)g) ^ swz) << 4), pack_bf16(e[0], e[1]), pack_bf16(e[2], e[3]), pack_bf16(e[4], e[5]),
                     pack_bf16(e[6], e[7]));
      }
      l += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
      tc5::fence_before_sync();
      fence_async_smem();
      __syncwarp();
      if (lane == 0) tc5::mbar_arrive(bar(B_PF + s));
    }
    ok = ok && wait_warp(bar(B_ACC), 0u);
    tc5::fence_after_sync();
    // merge the two groups: both halves of every row meet through shared memory (the Q tile is dead by now)
    float* xm = reinterpret_cast<float*>(smem + OFF_Q);    // [2][128] maxima, then [2][128] sums
    float* xl = xm + 256;
    xm[wg * 128 + row] = m;
    xl[wg * 128 + row] = l;
    asm volatile("bar.sync 1, 256;" ::: "memory");    // reached by all eight softmax warps, also after a failed wait
    if (ok) {
      const float m0 = xm[row], m1 = xm[128 + row], l0 = xl[row], l1 = xl[128 + row];
      const float mm = fmaxf(m0, m1);
      const float f0 = (m0 == -INFINITY) ? 0.0f : ex2(m0 - mm);
      const float f1 = (m1 == -INFINITY) ? 0.0f : ex2(m1 - mm);
      const float lt = l0 * f0 + l1 * f1;
      const float inv = lt > 0.0f ? 1.0f / lt : 0.0f;
      const float g0 = f0 * inv, g1 = f1 * inv;
      const bool two = n_kv > 1;    // with one key tile group 1 never wrote its accumulator
      __nv_bfloat16* dst = p.o + (int64_t)b * p.o_sb + (int64_t)grow * p.o_ss + (int64_t)h * p.o_sh + wg * 64;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t a0[32], a1[32];
        float v[32];
        tc5::tmem_ld32(tlane + TM_O + (uint32_t)wg * 64u + (uint32_t)c * 32u, a0);
        if (two) tc5::tmem_ld32(tlane + TM_O + 128u + (uint32_t)wg * 64u + (uint32_t)c * 32u, a1);
        tc5::tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(a0[i]) * g0;
        if (two) {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = fmaf(__uint_as_float(a1[i]), g1, v[i]);
        }
        if (grow < p.seqlen) st_row32(dst + c * 32, v);
      }
      if (wg == 0 && grow < p.seqlen) p.lse[(int64_t)bh * p.seqlen + grow] = lt > 0.0f ? mm * kLn2 + logf(lt) : -INFINITY;
    }
  }

  // ---------------------------------------------------------------------- tear-down
  __syncwarp();
  if (*abort_flag) __nanosleep(200000);    // let copies / MMAs in flight finish before smem and TMEM go away
  tc5::fence_before_sync();
  __syncthreads();
  tc5::fence_after_sync();
  if (warp == 1) tc5::tmem_dealloc(tmem_base, TM_COLS);
}

// ====================================================================== forward, 128-key score tiles, P in tensor memory
namespace fwd2 {
constexpr int NK = 3;                         // ring depth of the K tiles (128 keys each)
constexpr int NV = 5;                         // ring depth of the V sub-tiles (64 keys each)
constexpr uint32_t PANEL_Q = 128 * 128;       // [128 query rows][64 bf16]
constexpr uint32_t TILE_Q = 2 * PANEL_Q;      // 32 KB
constexpr uint32_t PANEL_K = 128 * 128;       // [128 key rows][64 bf16]
constexpr uint32_t TILE_K = 2 * PANEL_K;      // 32 KB
constexpr uint32_t PANEL_V = 64 * 128;        // [64 key rows][64 bf16]
constexpr uint32_t TILE_V = 2 * PANEL_V;      // 16 KB
constexpr uint32_t OFF_Q = 0, OFF_K = TILE_Q, OFF_V = OFF_K + NK * TILE_K, OFF_X = OFF_V + NV * TILE_V, OFF_BAR = OFF_X + 2048;
enum { B_Q = 0, B_KF = 1, B_KE = B_KF + NK, B_VF = B_KE + NK, B_VE = B_VF + NV, B_SF = B_VE + NV, B_PF = B_SF + 2, B_OF = B_PF + 4,
       B_ACC = B_OF + 2, NBAR = B_ACC + 1 };
constexpr int SMEM = OFF_BAR + NBAR * 8 + 16 + 1024;
constexpr uint32_t TM_S = 0, TM_O = 256, TM_COLS = 512;    // two 128-column score slots, two 128-column outputs
constexpr float kRescaleStep = 8.0f;
}    // namespace fwd2

// Measured on this part: a 128 x N x 16 bf16 tcgen05.mma costs about 70 cycles for N = 64 as well as for N = 128 (the
// A operand, 4 KB, is fed at 64 B/clk whatever N is), wherever A comes from.  S = Q K^T is therefore issued over 128
// keys at a time (8 MMAs per 128 keys instead of 16).  The two softmax groups split every 128-key score tile by
// columns: group g owns keys [128 J + 64 g, 128 J + 64 g + 64) of tile J, with its own output accumulator O_g,
// reference maximum and row sum, exactly as if the groups took alternating 64-key tiles; the halves are merged once
// at the end.  Probabilities are packed to bf16 and stored with tcgen05.st over the first 32 columns of the 64-column
// half they were computed from, and O_g += P V reads them from tensor memory (no shared-memory round trip for P).
// The tensor pipe executes MMAs in issue order, so slot J & 1 may take the scores of tile J + 2 as soon as that MMA is
// issued after both PV products of tile J: no "slot free" barriers are needed.
__global__ void __launch_bounds__(kTcThreads, 1)
attn_fwd_tm_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                   const __grid_constant__ CUtensorMap map_v, const TcParams p) {
  using namespace fwd2;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = tc5::smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw_addr);
  const uint32_t bars = base + OFF_BAR;
  auto bar = [&](int i) { return bars + 8u * (uint32_t)i; };
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(smem + OFF_BAR + NBAR * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
  auto wait_warp = [&](uint32_t br, uint32_t ph) {
    return __all_sync(0xffffffffu, tc5::mbar_wait(br, ph, abort_flag, p.status, kStatusBit)) != 0;
  };

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int qt = (int)gridDim.x - 1 - (int)blockIdx.x;    // long rows first
  const int bh = blockIdx.y;
  const int b = bh / p.heads;
  const int h = bh - b * p.heads;
  const int q0 = qt * 128;
  const int n_all = (p.seqlen + 63) / 64;
  const int n_kv = p.causal ? min(2 * qt + 2, n_all) : n_all;    // 64-key sub-tiles with a visible key
  const int n_t = (n_kv + 1) >> 1;                               // 128-key tiles; a trailing odd sub-tile is fully masked

  if (threadIdx.x == 0) {
    tc5::mbar_init(bar(B_Q), 1);
    for (int s = 0; s < NK; ++s) {
      tc5::mbar_init(bar(B_KF + s), 1);
      tc5::mbar_init(bar(B_KE + s), 1);
    }
    for (int s = 0; s < NV; ++s) {
      tc5::mbar_init(bar(B_VF + s), 1);
      tc5::mbar_init(bar(B_VE + s), 1);
    }
    tc5::mbar_init(bar(B_SF + 0), 1);
    tc5::mbar_init(bar(B_SF + 1), 1);
    for (int s = 0; s < 4; ++s) tc5::mbar_init(bar(B_PF + s), 4);
    tc5::mbar_init(bar(B_OF + 0), 1);
    tc5::mbar_init(bar(B_OF + 1), 1);
    tc5::mbar_init(bar(B_ACC), 1);
    *abort_flag = 0;
    tc5::mbar_fence_init();
    tc5::tma_prefetch_desc(&map_q);
    tc5::tma_prefetch_desc(&map_k);
    tc5::tma_prefetch_desc(&map_v);
  }
  if (warp == 1) {
    tc5::tmem_alloc(tc5::smem_u32(tmem_holder), TM_COLS);
    tc5::tmem_relinquish();
  }
  tc5::fence_before_sync();
  __syncthreads();
  tc5::fence_after_sync();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tc5::mbar_arrive_expect_tx(bar(B_Q), TILE_Q);
      tc5::tma_load_4d(base + OFF_Q, &map_q, 0, h, q0, b, bar(B_Q));
      tc5::tma_load_4d(base + OFF_Q + PANEL_Q, &map_q, 64, h, q0, b, bar(B_Q));
      bool ok = true;
      for (int t = 0; t < n_t && ok; ++t) {
        const int ks = t % NK;
        TC_WAIT(bar(B_KE + ks), ((uint32_t)(t / NK) & 1u) ^ 1u);
        tc5::mbar_arrive_expect_tx(bar(B_KF + ks), TILE_K);
        tc5::tma_load_4d(base + OFF_K + ks * TILE_K, &map_k, 0, h, t * 128, b, bar(B_KF + ks));
        tc5::tma_load_4d(base + OFF_K + ks * TILE_K + PANEL_K, &map_k, 64, h, t * 128, b, bar(B_KF + ks));
        for (int g = 0; g < 2; ++g) {
          const int j = 2 * t + g;
          const int vs = j % NV;
          if (!tc5::mbar_wait(bar(B_VE + vs), ((uint32_t)(j / NV) & 1u) ^ 1u, abort_flag, p.status, kStatusBit)) { ok = false; break; }
          tc5::mbar_arrive_expect_tx(bar(B_VF + vs), TILE_V);
          tc5::tma_load_4d(base + OFF_V + vs * TILE_V, &map_v, 0, h, j * 64, b, bar(B_VF + vs));
          tc5::tma_load_4d(base + OFF_V + vs * TILE_V + PANEL_V, &map_v, 64, h, j * 64, b, bar(B_VF + vs));
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc_s = tc5::idesc_bf16(128, 128, 0, 0);
      const uint32_t idesc_o = tc5::idesc_bf16(128, 128, 0, 1);
      // S[t & 1] = Q K_t^T over 128 keys
      auto issue_s = [&](int t) -> bool {
        const int ks = t % NK;
        if (!tc5::mbar_wait(bar(B_KF + ks), (uint32_t)(t / NK) & 1u, abort_flag, p.status, kStatusBit)) return false;
        tc5::fence_after_sync();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t off = (uint32_t)(kk >> 2) * PANEL_Q + (uint32_t)(kk & 3) * 32u;    // PANEL_K == PANEL_Q
          tc5::mma_f16(tmem_base + TM_S + (uint32_t)(t & 1) * 128u, tc5::smem_desc_k_sw128(base + OFF_Q + off),
                       tc5::smem_desc_k_sw128(base + OFF_K + ks * TILE_K + off), idesc_s, kk ? 1u : 0u);
        }
        tc5::mma_commit(bar(B_KE + ks));
        tc5::mma_commit(bar(B_SF + (t & 1)));
        return true;
      };
      do {
        TC_WAIT(bar(B_Q), 0u);
        bool ok = true;
        for (int t = 0; t < 2 && t < n_t; ++t)
          if (!issue_s(t)) { ok = false; break; }
        if (!ok) break;
        for (int t = 0; t < n_t && ok; ++t) {
          for (int g = 0; g < 2; ++g) {
            const int j = 2 * t + g;
            const int vs = j % NV;
            if (!tc5::mbar_wait(bar(B_PF + (t & 1) * 2 + g), (uint32_t)(t >> 1) & 1u, abort_flag, p.status, kStatusBit)) { ok = false; break; }
            if (!tc5::mbar_wait(bar(B_VF + vs), (uint32_t)(j / NV) & 1u, abort_flag, p.status, kStatusBit)) { ok = false; break; }
            tc5::fence_after_sync();
            // O_g (+)= P V : A = P from the first 32 columns of its half of the score slot, B = V with the key index as rows
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
              tc5::mma_f16_ta(tmem_base + TM_O + (uint32_t)g * 128u,
                              tmem_base + TM_S + (uint32_t)(t & 1) * 128u + (uint32_t)g * 64u + (uint32_t)kk * 8u,
                              tc5::smem_desc_mn_sw128(base + OFF_V + vs * TILE_V + (uint32_t)kk * 2048u, PANEL_V), idesc_o,
                              (t > 0 || kk) ? 1u : 0u);
            }
            tc5::mma_commit(bar(B_VE + vs));
            tc5::mma_commit(bar(B_OF + g));
          }
          if (ok && t + 2 < n_t && !issue_s(t + 2)) ok = false;
        }
        if (ok) tc5::mma_commit(bar(B_ACC));
      } while (false);
    }
  } else {
    // ------------------------------------------------------------------ softmax: one thread per query row and group
    const int qd = warp & 3;           // TMEM lane quarter this warp may access
    const int wg = (warp - 2) >> 2;    // group g: second index of the 64-key halves it owns
    const int row = qd * 32 + lane;
    const int grow = q0 + row;
    const uint32_t tlane = tmem_base + ((uint32_t)(qd * 32) << 16);
    const uint32_t to = tlane + TM_O + (uint32_t)wg * 128u;
    const float sl = p.scale * kLog2e;
    const int lim = p.causal ? min(grow, p.seqlen - 1) : p.seqlen - 1;    // last visible column
    float m = -INFINITY, l = 0.0f;    // reference maximum (log2 units) and row sum of this group
    bool ok = true;

    for (int t = 0; t < n_t; ++t) {
      const uint32_t ts = tlane + TM_S + (uint32_t)(t & 1) * 128u + (uint32_t)wg * 64u;
      if (!wait_warp(bar(B_SF + (t & 1)), (uint32_t)(t >> 1) & 1u)) { ok = false; break; }
      tc5::fence_after_sync();
      uint32_t r[2][32];
      tc5::tmem_ld32(ts, r[0]);
      tc5::tmem_ld32(ts + 32u, r[1]);
      tc5::tmem_ld_wait();
      const int col0 = (2 * t + wg) * 64;
      const bool need_mask = (p.causal && col0 + 63 > q0) || (col0 + 64 > p.seqlen);
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
      if (need_mask) {
#pragma unroll
        for (int i = 0; i < 64; ++i)
          if (col0 + i <= lim) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(r[i >> 5][i & 31]));
      } else {
#pragma unroll
        for (int i = 0; i < 64; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(r[i >> 5][i & 31]));
      }
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * sl;    // sl > 0
      const bool grow_m = mx > m + kRescaleStep || (m == -INFINITY && mx > -INFINITY);
      if (__any_sync(0xffffffffu, grow_m)) {
        const float m_new = grow_m ? mx : m;
        const float corr = (m == -INFINITY) ? 0.0f : ex2(m - m_new);
        if (t > 0) {
          // every earlier product of this group must have landed in O before it is rescaled
          if (!wait_warp(bar(B_OF + wg), (uint32_t)(t - 1) & 1u)) { ok = false; break; }
          tc5::fence_after_sync();
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            uint32_t x[32];
            tc5::tmem_ld32(to + (uint32_t)c * 32u, x);
            tc5::tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) x[i] = __float_as_uint(__uint_as_float(x[i]) * corr);
            tc5::tmem_st32(to + (uint32_t)c * 32u, x);
          }
        }
        l *= corr;
        m = m_new;
      }
      const float m_use = (m == -INFINITY) ? 0.0f : m;
      float sum4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
      uint32_t pk[32];
#pragma unroll
      for (int g = 0; g < 8; ++g) {    // columns 8g .. 8g+7 -> packed columns 4g .. 4g+3
        float e[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          e[i] = ex2(fmaf(__uint_as_float(r[g >> 2][(g & 3) * 8 + i]), sl, -m_use));
          if (need_mask && col0 + g * 8 + i > lim) e[i] = 0.0f;
          sum4[i & 3] += e[i];
        }
        pk[4 * g] = pack_bf16(e[0], e[1]);
        pk[4 * g + 1] = pack_bf16(e[2], e[3]);
        pk[4 * g + 2] = pack_bf16(e[4], e[5]);
        pk[4 * g + 3] = pack_bf16(e[6], e[7]);
      }
      l += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
      tc5::tmem_st32(ts, pk);
      tc5::tmem_st_wait();    // also covers the rescaled accumulator
      tc5::fence_before_sync();
      __syncwarp();
      if (lane == 0) tc5::mbar_arrive(bar(B_PF + (t & 1) * 2 + wg));
    }
    ok = ok && wait_warp(bar(B_ACC), 0u);
    tc5::fence_after_sync();
    // merge the two groups: both halves of every row meet through shared memory
    float* xm = reinterpret_cast<float*>(smem + OFF_X);    // [2][128] maxima, then [2][128] sums
    float* xl = xm + 256;
    xm[wg * 128 + row] = m;
    xl[wg * 128 + row] = l;
    asm volatile("bar.sync 1, 256;" ::: "memory");    // reached by all eight softmax warps, also after a failed wait
    if (ok) {
      const float m0 = xm[row], m1 = xm[128 + row], l0 = xl[row], l1 = xl[128 + row];
      const float mm = fmaxf(m0, m1);
      const float f0 = (m0 == -INFINITY) ? 0.0f : ex2(m0 - mm);
      const float f1 = (m1 == -INFINITY) ? 0.0f : ex2(m1 - mm);
      const float lt = l0 * f0 + l1 * f1;
      const float inv = lt > 0.0f ? 1.0f / lt : 0.0f;
      const float g0 = f0 * inv, g1 = f1 * inv;
      // both accumulators were written (a group whose keys are all masked accumulated zeros)
      __nv_bfloat16* dst = p.o + (int64_t)b * p.o_sb + (int64_t)grow * p.o_ss + (int64_t)h * p.o_sh + wg * 64;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t a0[32], a1[32];
        float v[32];
        tc5::tmem_ld32(tlane + TM_O + (uint32_t)wg * 64u + (uint32_t)c * 32u, a0);
        tc5::tmem_ld32(tlane + TM_O + 128u + (uint32_t)wg * 64u + (uint32_t)c * 32u, a1);
        tc5::tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = fmaf(__uint_as_float(a1[i]), g1, __uint_as_float(a0[i]) * g0);
        if (grow < p.seqlen) st_row32(dst + c * 32, v);
      }
      if (wg == 0 && grow < p.seqlen) p.lse[(int64_t)bh * p.seqlen + grow] = lt > 0.0f ? mm * kLn2 + logf(lt) : -INFINITY;
    }
  }

  // ---------------------------------------------------------------------- tear-down
  __syncwarp();
  if (*abort_flag) __nanosleep(200000);    // let copies / MMAs in flight finish before smem and TMEM go away
  tc5::fence_before_sync();
  __syncthreads();
  tc5::fence_after_sync();
  if (warp == 1) tc5::tmem_dealloc(tmem_base, TM_COLS);
}

// ================================================================= forward, persistent CTAs over (query tile, batch, head)
namespace fwd3 {
using namespace fwd2;    // same tiles, rings and tensor-memory layout
constexpr uint32_t OFF_X3 = OFF_V + NV * TILE_V;          // two merge buffers of 2 KB (alternating work items)
constexpr uint32_t OFF_BAR3 = OFF_X3 + 4096;
enum { B3_QE = NBAR, B3_OE = NBAR + 1, B3_X = NBAR + 2, NBAR3 = NBAR + 3 };
constexpr int SMEM3 = OFF_BAR3 + NBAR3 * 8 + 16 + 1024;
}    // namespace fwd3

// The schedule of attn_fwd_tm_kernel with one CTA per SM that walks a list of work items (query tile, batch * head),
// grouped by head and by falling length (see item_qt below).  Every ring (K, V, score slots) and every barrier keeps
// running across items, so the TMA warp loads Q, K and V of the next item while the softmax warps are still in the
// epilogue of the current one, and the MMA warp has the first two score tiles of the next item ready when they return:
// the ~8 k cycles of prologue and epilogue per item (of ~23 k on average for sequence 2048) are hidden.  Two extra
// barriers order the reuse: B3_QE (all score MMAs of an item issued and complete: the Q tile may be overwritten) and
// B3_OE (the softmax warps have read both output accumulators: the first PV product of the next item may overwrite them);
// B3_X is where the eight softmax warps meet before the two groups' partial results are merged.
__global__ void __launch_bounds__(kTcThreads, 1)
attn_fwd_ps_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                   const __grid_constant__ CUtensorMap map_v, const TcParams p, int n_qt, int n_items) {
  using namespace fwd3;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = tc5::smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw_addr);
  const uint32_t bars = base + OFF_BAR3;
  auto bar = [&](int i) { return bars + 8u * (uint32_t)i; };
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(smem + OFF_BAR3 + NBAR3 * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
  auto wait_warp = [&](uint32_t br, uint32_t ph) {
    return __all_sync(0xffffffffu, tc5::mbar_wait(br, ph, abort_flag, p.status, kStatusBit)) != 0;
  };
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int bh_total = p.batch * p.heads;
  const int n_all = (p.seqlen + 63) / 64;
  // work item -> (query tile, batch * head) and its number of 128-key tiles
  // Items are ordered in groups of G (batch, head) pairs, inside a group by falling query tile (= falling length), so
  // that the CTAs of a few consecutive waves work on the same heads: a head's K and V (1 MB at sequence 2048) are read
  // from HBM by its longest rows and found in L2 by the others (with all heads of one query-tile level in a wave the
  // kernel read K / V 3.9 times).  G * n_qt is about four waves, which the snake walk below balances exactly.
  const int G = max(1, (4 * (int)gridDim.x) / n_qt);
  auto item_qt = [&](int item) {
    const int g = item / (G * n_qt);
    const int hg = min(G, bh_total - g * G);
    return n_qt - 1 - (item - g * G * n_qt) / hg;
  };
  auto item_bh = [&](int item) {
    const int g = item / (G * n_qt);
    const int hg = min(G, bh_total - g * G);
    return g * G + (item - g * G * n_qt) % hg;
  };
  // items are sorted by falling length; CTA c takes one item per wave of gridDim.x items, walking even waves upwards
  // and odd waves downwards, so that the per-CTA sums stay within about one tile of each other
  const int n_waves = (n_items + (int)gridDim.x - 1) / (int)gridDim.x;
  auto item_at = [&](int w) {
    const int c = (w & 1) ? (int)gridDim.x - 1 - (int)blockIdx.x : (int)blockIdx.x;
    return w * (int)gridDim.x + c;
  };
  auto item_tiles = [&](int qt) {
    const int n_kv = p.causal ? min(2 * qt + 2, n_all) : n_all;
    return (n_kv + 1) >> 1;
  };

  if (threadIdx.x == 0) {
    tc5::mbar_init(bar(B_Q), 1);
    for (int s = 0; s < NK; ++s) {
      tc5::mbar_init(bar(B_KF + s), 1);
      tc5::mbar_init(bar(B_KE + s), 1);
    }
    for (int s = 0; s < NV; ++s) {
      tc5::mbar_init(bar(B_VF + s), 1);
      tc5::mbar_init(bar(B_VE + s), 1);
    }
    tc5::mbar_init(bar(B_SF + 0), 1);
    tc5::mbar_init(bar(B_SF + 1), 1);
    for (int s = 0; s < 4; ++s) tc5::mbar_init(bar(B_PF + s), 4);
    tc5::mbar_init(bar(B_OF + 0), 1);
    tc5::mbar_init(bar(B_OF + 1), 1);
    tc5::mbar_init(bar(B_ACC), 1);
    tc5::mbar_init(bar(B3_QE), 1);
    tc5::mbar_init(bar(B3_OE), 8);
    tc5::mbar_init(bar(B3_X), 8);
    *abort_flag = 0;
    tc5::mbar_fence_init();
    tc5::tma_prefetch_desc(&map_q);
    tc5::tma_prefetch_desc(&map_k);
    tc5::tma_prefetch_desc(&map_v);
  }
  if (warp == 1) {
    tc5::tmem_alloc(tc5::smem_u32(tmem_holder), TM_COLS);
    tc5::tmem_relinquish();
  }
  tc5::fence_before_sync();
  __syncthreads();
  tc5::fence_after_sync();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int gt = 0;    // 128-key tiles loaded so far (all items)
      bool ok = true;
      int it = 0;
      for (int w = 0; w < n_waves && ok; ++w) {
        const int item = item_at(w);
        if (item >= n_items) continue;
        const int qt = item_qt(item);
        const int bh = item_bh(item);
        const int b = bh / p.heads, h = bh - b * p.heads;
        const int n_t = item_tiles(qt);
        if (it > 0 && !tc5::mbar_wait(bar(B3_QE), (uint32_t)(it - 1) & 1u, abort_flag, p.status, kStatusBit)) break;
        tc5::mbar_arrive_expect_tx(bar(B_Q), TILE_Q);
        tc5::tma_load_4d(base + OFF_Q, &map_q, 0, h, qt * 128, b, bar(B_Q));
        tc5::tma_load_4d(base + OFF_Q + PANEL_Q, &map_q, 64, h, qt * 128, b, bar(B_Q));
        for (int t = 0; t < n_t && ok; ++t, ++gt) {
          const int ks = gt % NK;
          if (!tc5::mbar_wait(bar(B_KE + ks), ((uint32_t)(gt / NK) & 1u) ^ 1u, abort_flag, p.status, kStatusBit)) { ok = false; break; }
          tc5::mbar_arrive_expect_tx(bar(B_KF + ks), TILE_K);
          tc5::tma_load_4d(base + OFF_K + ks * TILE_K, &map_k, 0, h, t * 128, b, bar(B_KF + ks));
          tc5::tma_load_4d(base + OFF_K + ks * TILE_K + PANEL_K, &map_k, 64, h, t * 128, b, bar(B_KF + ks));
          for (int g = 0; g < 2; ++g) {
            const int gj = 2 * gt + g;    // 64-key sub-tiles loaded so far
            const int vs = gj % NV;
            if (!tc5::mbar_wait(bar(B_VE + vs), ((uint32_t)(gj / NV) & 1u) ^ 1u, abort_flag, p.status, kStatusBit)) { ok = false; break; }
            tc5::mbar_arrive_expect_tx(bar(B_VF + vs), TILE_V);
            tc5::tma_load_4d(base + OFF_V + vs * TILE_V, &map_v, 0, h, (2 * t + g) * 64, b, bar(B_VF + vs));
            tc5::tma_load_4d(base + OFF_V + vs * TILE_V + PANEL_V, &map_v, 64, h, (2 * t + g) * 64, b, bar(B_VF + vs));
          }
        }
        ++it;
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc_s = tc5::idesc_bf16(128, 128, 0, 0);
      const uint32_t idesc_o = tc5::idesc_bf16(128, 128, 0, 1);
      auto issue_s = [&](int gs) -> bool {    // S[gs & 1] = Q K^T for the gs-th tile of this CTA
        const int ks = gs % NK;
        if (!tc5::mbar_wait(bar(B_KF + ks), (uint32_t)(gs / NK) & 1u, abort_flag, p.status, kStatusBit)) return false;
        tc5::fence_after_sync();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t off = (uint32_t)(kk >> 2) * PANEL_Q + (uint32_t)(kk & 3) * 32u;
          tc5::mma_f16(tmem_base + TM_S + (uint32_t)(gs & 1) * 128u, tc5::smem_desc_k_sw128(base + OFF_Q + off),
                       tc5::smem_desc_k_sw128(base + OFF_K + ks * TILE_K + off), idesc_s, kk ? 1u : 0u);
        }
        tc5::mma_commit(bar(B_KE + ks));
        tc5::mma_commit(bar(B_SF + (gs & 1)));
        return true;
      };
      int g0 = 0;    // tiles of earlier items
      bool ok = true;
      int it = 0;
      for (int w = 0; w < n_waves && ok; ++w) {
        const int item = item_at(w);
        if (item >= n_items) continue;
        const int n_t = item_tiles(item_qt(item));
        if (!tc5::mbar_wait(bar(B_Q), (uint32_t)it & 1u, abort_flag, p.status, kStatusBit)) { ok = false; break; }
        for (int t = 0; t < 2 && t < n_t; ++t)
          if (!issue_s(g0 + t)) { ok = false; break; }
        if (!ok) break;
        if (n_t <= 2) tc5::mma_commit(bar(B3_QE));    // every score product of this item has been issued
        // the softmax warps must have read the previous item's accumulators before they are overwritten
        if (it > 0 && !tc5::mbar_wait(bar(B3_OE), (uint32_t)(it - 1) & 1u, abort_flag, p.status, kStatusBit)) { ok = false; break; }
        for (int t = 0; t < n_t && ok; ++t) {
          const int gs = g0 + t;
          for (int g = 0; g < 2; ++g) {
            const int gj = 2 * gs + g;
            const int vs = gj % NV;
            // the data barrier first: a wait costs 100+ cycles even when its phase completed long ago, and this one
            // then passes while the softmax warps are still at work on P
            if (!tc5::mbar_wait(bar(B_VF + vs), (uint32_t)(gj / NV) & 1u, abort_flag, p.status, kStatusBit)) { ok = false; break; }
            if (!tc5::mbar_wait(bar(B_PF + (gs & 1) * 2 + g), (uint32_t)(gs >> 1) & 1u, abort_flag, p.status, kStatusBit)) { ok = false; break; }
            tc5::fence_after_sync();
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
              tc5::mma_f16_ta(tmem_base + TM_O + (uint32_t)g * 128u,
                              tmem_base + TM_S + (uint32_t)(gs & 1) * 128u + (uint32_t)g * 64u + (uint32_t)kk * 8u,
                              tc5::smem_desc_mn_sw128(base + OFF_V + vs * TILE_V + (uint32_t)kk * 2048u, PANEL_V), idesc_o,
                              (t > 0 || kk) ? 1u : 0u);
            }
            tc5::mma_commit(bar(B_VE + vs));
            tc5::mma_commit(bar(B_OF + g));
          }
          if (ok && t + 2 < n_t) {
            if (!issue_s(gs + 2)) { ok = false; break; }
            if (t + 3 == n_t) tc5::mma_commit(bar(B3_QE));
          }
        }
        if (ok) tc5::mma_commit(bar(B_ACC));
        g0 += n_t;
        ++it;
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax: one thread per query row and group
    const int qd = warp & 3;           // TMEM lane quarter this warp may access
    const int wg = (warp - 2) >> 2;    // group g: second index of the 64-key halves it owns
    const int row = qd * 32 + lane;
    const uint32_t tlane = tmem_base + ((uint32_t)(qd * 32) << 16);
    const uint32_t to = tlane + TM_O + (uint32_t)wg * 128u;
    const float sl = p.scale * kLog2e;
    int g0 = 0;
    bool ok = true;
    int it = 0;
    for (int w = 0; w < n_waves; ++w) {
      const int item = item_at(w);
      if (item >= n_items) continue;
      const int qt = item_qt(item);
      const int bh = item_bh(item);
      const int b = bh / p.heads, h = bh - b * p.heads;
      const int n_t = item_tiles(qt);
      const int q0 = qt * 128;
      const int grow = q0 + row;
      const int lim = p.causal ? min(grow, p.seqlen - 1) : p.seqlen - 1;    // last visible column
      float m = -INFINITY, l = 0.0f;    // reference maximum (log2 units) and row sum of this group
      for (int t = 0; t < n_t; ++t) {
        const int gs = g0 + t;
        const uint32_t ts = tlane + TM_S + (uint32_t)(gs & 1) * 128u + (uint32_t)wg * 64u;
        if (!wait_warp(bar(B_SF + (gs & 1)), (uint32_t)(gs >> 1) & 1u)) { ok = false; break; }
        tc5::fence_after_sync();
        uint32_t r[2][32];
        tc5::tmem_ld32(ts, r[0]);
        tc5::tmem_ld32(ts + 32u, r[1]);
        tc5::tmem_ld_wait();
        const int col0 = (2 * t + wg) * 64;
        const bool need_mask = (p.causal && col0 + 63 > q0) || (col0 + 64 > p.seqlen);
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
        if (need_mask) {
#pragma unroll
          for (int i = 0; i < 64; ++i)
            if (col0 + i <= lim) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(r[i >> 5][i & 31]));
        } else {
#pragma unroll
          for (int i = 0; i < 64; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(r[i >> 5][i & 31]));
        }
        const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * sl;    // sl > 0
        const bool grow_m = mx > m + kRescaleStep || (m == -INFINITY && mx > -INFINITY);
        if (__any_sync(0xffffffffu, grow_m)) {
          const float m_new = grow_m ? mx : m;
          const float corr = (m == -INFINITY) ? 0.0f : ex2(m - m_new);
          if (t > 0) {
            // every earlier product of this group and item must have landed in O before it is rescaled
            if (!wait_warp(bar(B_OF + wg), (uint32_t)(gs - 1) & 1u)) { ok = false; break; }
            tc5::fence_after_sync();
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
              uint32_t x[32];
              tc5::tmem_ld32(to + (uint32_t)c * 32u, x);
              tc5::tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < 32; ++i) x[i] = __float_as_uint(__uint_as_float(x[i]) * corr);
              tc5::tmem_st32(to + (uint32_t)c * 32u, x);
            }
          }
          l *= corr;
          m = m_new;
        }
        const float m_use = (m == -INFINITY) ? 0.0f : m;
        float sum4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        uint32_t pk[32];
#pragma unroll
        for (int g = 0; g < 8; ++g) {    // columns 8g .. 8g+7 -> packed columns 4g .. 4g+3
          float e[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            e[i] = ex2(fmaf(__uint_as_float(r[g >> 2][(g & 3) * 8 + i]), sl, -m_use));
            if (need_mask && col0 + g * 8 + i > lim) e[i] = 0.0f;
            sum4[i & 3] += e[i];
          }
          pk[4 * g] = pack_bf16(e[0], e[1]);
          pk[4 * g + 1] = pack_bf16(e[2], e[3]);
          pk[4 * g + 2] = pack_bf16(e[4], e[5]);
          pk[4 * g + 3] = pack_bf16(e[6], e[7]);
        }
        l += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
        tc5::tmem_st32(ts, pk);
        tc5::tmem_st_wait();    // also covers the rescaled accumulator
        tc5::fence_before_sync();
        __syncwarp();
        if (lane == 0) tc5::mbar_arrive(bar(B_PF + (gs & 1) * 2 + wg));
      }
      ok = ok && wait_warp(bar(B_ACC), (uint32_t)it & 1u);
      tc5::fence_after_sync();
      // merge the two groups through shared memory (two buffers, alternating items: a warp that is already in the next
      // item's merge cannot overwrite values another warp still reads)
      float* xm = reinterpret_cast<float*>(smem + OFF_X3 + (uint32_t)(it & 1) * 2048u);    // [2][128] maxima, then [2][128] sums
      float* xl = xm + 256;
      if (!ok) break;
      xm[wg * 128 + row] = m;
      xl[wg * 128 + row] = l;
      // the eight warps meet on an mbarrier (bounded wait) rather than on a named barrier: a warp that gave up on an
      // earlier wait leaves without arriving, and the others then give up here instead of waiting for it for ever
      __syncwarp();
      if (lane == 0) tc5::mbar_arrive(bar(B3_X));
      if (!wait_warp(bar(B3_X), (uint32_t)it & 1u)) { ok = false; break; }
      const float m0 = xm[row], m1 = xm[128 + row], l0 = xl[row], l1 = xl[128 + row];
      const float mm = fmaxf(m0, m1);
      const float f0 = (m0 == -INFINITY) ? 0.0f : ex2(m0 - mm);
      const float f1 = (m1 == -INFINITY) ? 0.0f : ex2(m1 - mm);
      const float lt = l0 * f0 + l1 * f1;
      const float inv = lt > 0.0f ? 1.0f / lt : 0.0f;
      const float gg0 = f0 * inv, gg1 = f1 * inv;
      uint32_t a0[2][32], a1[2][32];
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        tc5::tmem_ld32(tlane + TM_O + (uint32_t)wg * 64u + (uint32_t)c * 32u, a0[c]);
        tc5::tmem_ld32(tlane + TM_O + 128u + (uint32_t)wg * 64u + (uint32_t)c * 32u, a1[c]);
      }
      tc5::tmem_ld_wait();
      tc5::fence_before_sync();
      __syncwarp();
      if (lane == 0) tc5::mbar_arrive(bar(B3_OE));    // the accumulators may take the next item
      __nv_bfloat16* dst = p.o + (int64_t)b * p.o_sb + (int64_t)grow * p.o_ss + (int64_t)h * p.o_sh + wg * 64;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        float v[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = fmaf(__uint_as_float(a1[c][i]), gg1, __uint_as_float(a0[c][i]) * gg0);
        if (grow < p.seqlen) st_row32(dst + c * 32, v);
      }
      if (wg == 0 && grow < p.seqlen) p.lse[(int64_t)bh * p.seqlen + grow] = lt > 0.0f ? mm * kLn2 + logf(lt) : -INFINITY;
      g0 += n_t;
      ++it;
    }
  }

  // ---------------------------------------------------------------------- tear-down
  __syncwarp();
  if (*abort_flag) __nanosleep(200000);    // let copies / MMAs in flight finish before smem and TMEM go away
  tc5::fence_before_sync();
  __syncthreads();
  tc5::fence_after_sync();
  if (warp == 1) tc5::tmem_dealloc(tmem_base, TM_COLS);
}

// ===================================================================================== delta = rowsum(dO * O)
struct DeltaParams {
  const __nv_bfloat16* o;
  const __nv_bfloat16* d_o;
  float* delta;
  int64_t o_sb, o_ss, o_sh, do_sb, do_ss, do_sh;
  int batch, heads, seqlen;
};

__global__ void attn_delta_tc_kernel(const DeltaParams p) {
  const int64_t gw = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const int64_t total = (int64_t)p.batch * p.heads * p.seqlen;
  if (gw >= total) return;
  const int s = (int)(gw % p.seqlen);
  const int bh = (int)(gw / p.seqlen);
  const int b = bh / p.heads;
  const int h = bh - b * p.heads;
  const uint2 a = *reinterpret_cast<const uint2*>(p.o + (int64_t)b * p.o_sb + (int64_t)s * p.o_ss + (int64_t)h * p.o_sh + lane * 4);
  const uint2 g = *reinterpret_cast<const uint2*>(p.d_o + (int64_t)b * p.do_sb + (int64_t)s * p.do_ss + (int64_t)h * p.do_sh + lane * 4);
  const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&a);
  const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&g);
  float acc = 0.0f;
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const float2 x = __bfloat1622float2(a2[i]);
    const float2 y = __bfloat1622float2(g2[i]);
    acc = fmaf(x.x, y.x, fmaf(x.y, y.y, acc));
  }
  acc = warp_sum(acc);
  if (lane == 0) p.delta[gw] = acc;
}

// ============================================================================================ dK / dV
namespace dkv {
constexpr uint32_t PANEL_KV = 128 * 128;    // [128 key rows][64 bf16]
constexpr uint32_t TILE_KV = 2 * PANEL_KV;
constexpr uint32_t PANEL_Q = 64 * 128;      // [64 query rows][64 bf16]
constexpr uint32_t TILE_Q = 2 * PANEL_Q;    // 16 KB
constexpr uint32_t TILE_P = 128 * 128;      // [128 key rows][64 queries] bf16
constexpr int NSQ = 3;    // ring of Q/dO stages: a stage is read by the first and by the last MMA of its tile
constexpr uint32_t OFF_K = 0, OFF_V = TILE_KV, OFF_Q = 2 * TILE_KV, OFF_DO = OFF_Q + NSQ * TILE_Q, OFF_PT = OFF_DO + NSQ * TILE_Q,
                   OFF_DST = OFF_PT + 2 * TILE_P, OFF_LSE = OFF_DST + 2 * TILE_P, OFF_BAR = OFF_LSE + NSQ * 2 * 64 * 4;
enum { B_KV = 0, B_QF = 1, B_QE = B_QF + NSQ, B_SF = B_QE + NSQ, B_SE = B_SF + 2, B_PF = B_SE + 2, B_PE = B_PF + 2, B_ACC = B_PE + 2,
       NBAR = B_ACC + 1 };
constexpr int SMEM = OFF_BAR + NBAR * 8 + 16 + 1024;
constexpr uint32_t TM_ST = 0, TM_DPT = 128, TM_DV = 256, TM_DK = 384, TM_COLS = 512;
}    // namespace dkv

__global__ void __launch_bounds__(kTcThreads, 1)
attn_bwd_dkdv_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                        const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do, const TcParams p) {
  using namespace dkv;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = tc5::smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw_addr);
  const uint32_t bars = base + OFF_BAR;
  auto bar = [&](int i) { return bars + 8u * (uint32_t)i; };
  float* s_lse = reinterpret_cast<float*>(smem + OFF_LSE);    // [NSQ][64] log2-scaled lse, then [NSQ][64] delta
  float* s_delta = s_lse + NSQ * 64;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(smem + OFF_BAR + NBAR * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
  // Wait used by full warps that go on to warp-collective TMEM accesses: the outcome is made uniform.
  auto wait_warp = [&](uint32_t br, uint32_t ph) {
    return __all_sync(0xffffffffu, tc5::mbar_wait(br, ph, abort_flag, p.status, kStatusBit)) != 0;
  };

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int kt = blockIdx.x;    // key tile 0 has the most query tiles under a causal mask and starts first
  const int bh = blockIdx.y;
  const int b = bh / p.heads;
  const int h = bh - b * p.heads;
  const int k0 = kt * 128;
  const int nq_all = (p.seqlen + 63) / 64;
  const int t_first = p.causal ? 2 * kt : 0;
  const int n_q = nq_all - t_first;    // >= 1 because k0 < seqlen

  if (threadIdx.x == 0) {
    tc5::mbar_init(bar(B_KV), 1);
    for (int s = 0; s < NSQ; ++s) {
      tc5::mbar_init(bar(B_QF + s), 2);    // TMA bytes + the lse/delta rows written by warp 0
      tc5::mbar_init(bar(B_QE + s), 5);    // last MMA that reads the stage + four softmax warps
    }
    for (int s = 0; s < 2; ++s) {
      tc5::mbar_init(bar(B_SF + s), 1);
      tc5::mbar_init(bar(B_SE + s), 4);
      tc5::mbar_init(bar(B_PF + s), 4);
      tc5::mbar_init(bar(B_PE + s), 1);
    }
    tc5::mbar_init(bar(B_ACC), 1);
    *abort_flag = 0;
    tc5::mbar_fence_init();
    tc5::tma_prefetch_desc(&map_q);
    tc5::tma_prefetch_desc(&map_k);
    tc5::tma_prefetch_desc(&map_v);
    tc5::tma_prefetch_desc(&map_do);
  }
  if (warp == 1) {
    tc5::tmem_alloc(tc5::smem_u32(tmem_holder), TM_COLS);
    tc5::tmem_relinquish();
  }
  tc5::fence_before_sync();
  __syncthreads();
  tc5::fence_after_sync();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    // ------------------------------------------------------------------ producer (whole warp: lane 0 issues TMA)
    if (lane == 0) {
      tc5::mbar_arrive_expect_tx(bar(B_KV), 2 * TILE_KV);
      tc5::tma_load_4d(base + OFF_K, &map_k, 0, h, k0, b, bar(B_KV));
      tc5::tma_load_4d(base + OFF_K + PANEL_KV, &map_k, 64, h, k0, b, bar(B_KV));
      tc5::tma_load_4d(base + OFF_V, &map_v, 0, h, k0, b, bar(B_KV));
      tc5::tma_load_4d(base + OFF_V + PANEL_KV, &map_v, 64, h, k0, b, bar(B_KV));
    }
    const float* glse = p.lse + (int64_t)bh * p.seqlen;
    const float* gdelta = p.delta + (int64_t)bh * p.seqlen;
    for (int t = 0; t < n_q; ++t) {
      const int s = t % NSQ;
      const uint32_t ph = (uint32_t)(t / NSQ) & 1u;
      const int qrow0 = (t_first + t) * 64;
      TC_WAIT(bar(B_QE + s), ph ^ 1u);
      if (lane == 0) {
        tc5::mbar_arrive_expect_tx(bar(B_QF + s), 2 * TILE_Q);
        tc5::tma_load_4d(base + OFF_Q + s * TILE_Q, &map_q, 0, h, qrow0, b, bar(B_QF + s));
        tc5::tma_load_4d(base + OFF_Q + s * TILE_Q + PANEL_Q, &map_q, 64, h, qrow0, b, bar(B_QF + s));
        tc5::tma_load_4d(base + OFF_DO + s * TILE_Q, &map_do, 0, h, qrow0, b, bar(B_QF + s));
        tc5::tma_load_4d(base + OFF_DO + s * TILE_Q + PANEL_Q, &map_do, 64, h, qrow0, b, bar(B_QF + s));
      }
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int r = lane + 32 * i;
        const bool in = qrow0 + r < p.seqlen;
        s_lse[s * 64 + r] = in ? glse[qrow0 + r] * kLog2e : INFINITY;    // +inf makes the probability exactly zero
        s_delta[s * 64 + r] = in ? gdelta[qrow0 + r] : 0.0f;
      }
      __syncwarp();
      if (lane == 0) tc5::mbar_arrive(bar(B_QF + s));
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc_s = tc5::idesc_bf16(128, 64, 0, 0);
      const uint32_t idesc_acc = tc5::idesc_bf16(128, 128, 0, 1);
      // S^T = K Q_t^T and dP^T = V dO_t^T into buffer t&1
      auto issue_s = [&](int t) -> bool {
        const int s = t & 1;
        const uint32_t ph = (uint32_t)(t >> 1) & 1u;
        const int st = t % NSQ;
        if (!tc5::mbar_wait(bar(B_SE + s), ph ^ 1u, abort_flag, p.status, kStatusBit)) return false;
        if (!tc5::mbar_wait(bar(B_QF + st), (uint32_t)(t / NSQ) & 1u, abort_flag, p.status, kStatusBit)) return false;
        tc5::fence_after_sync();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t offa = (uint32_t)(kk >> 2) * PANEL_KV + (uint32_t)(kk & 3) * 32u;
          const uint32_t offb = (uint32_t)(kk >> 2) * PANEL_Q + (uint32_t)(kk & 3) * 32u;
          tc5::mma_f16(tmem_base + TM_ST + (uint32_t)s * 64u, tc5::smem_desc_k_sw128(base + OFF_K + offa),
                       tc5::smem_desc_k_sw128(base + OFF_Q + st * TILE_Q + offb), idesc_s, kk ? 1u : 0u);
        }
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t offa = (uint32_t)(kk >> 2) * PANEL_KV + (uint32_t)(kk & 3) * 32u;
          const uint32_t offb = (uint32_t)(kk >> 2) * PANEL_Q + (uint32_t)(kk & 3) * 32u;
          tc5::mma_f16(tmem_base + TM_DPT + (uint32_t)s * 64u, tc5::smem_desc_k_sw128(base + OFF_V + offa),
                       tc5::smem_desc_k_sw128(base + OFF_DO + st * TILE_Q + offb), idesc_s, kk ? 1u : 0u);
        }
        tc5::mma_commit(bar(B_SF + s));
        return true;
      };
      do {
        TC_WAIT(bar(B_KV), 0u);
        if (!issue_s(0)) break;
        if (n_q > 1 && !issue_s(1)) break;
        bool ok = true;
        for (int t = 0; t < n_q; ++t) {
          // the scores two tiles ahead go first: their buffer was released as soon as tile t had been read
          if (t + 2 < n_q && !issue_s(t + 2)) { ok = false; break; }
          const int s = t & 1;
          const int st = t % NSQ;
          const uint32_t ph = (uint32_t)(t >> 1) & 1u;
          if (!tc5::mbar_wait(bar(B_PF + s), ph, abort_flag, p.status, kStatusBit)) { ok = false; break; }
          tc5::fence_after_sync();
          // dV += P^T dO_t ; dK += dS^T Q_t : A from the softmax threads (K-major), B = the TMA tile read MN-major
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            tc5::mma_f16(tmem_base + TM_DV, tc5::smem_desc_k_sw128(base + OFF_PT + s * TILE_P + (uint32_t)kk * 32u),
                         tc5::smem_desc_mn_sw128(base + OFF_DO + st * TILE_Q + (uint32_t)kk * 2048u, PANEL_Q), idesc_acc,
                         (t | kk) ? 1u : 0u);
          }
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            tc5::mma_f16(tmem_base + TM_DK, tc5::smem_desc_k_sw128(base + OFF_DST + s * TILE_P + (uint32_t)kk * 32u),
                         tc5::smem_desc_mn_sw128(base + OFF_Q + st * TILE_Q + (uint32_t)kk * 2048u, PANEL_Q), idesc_acc,
                         (t | kk) ? 1u : 0u);
          }
          tc5::mma_commit(bar(B_PE + s));
          tc5::mma_commit(bar(B_QE + st));
        }
        if (ok) tc5::mma_commit(bar(B_ACC));
      } while (false);
    }
  } else {
    // ------------------------------------------------------------------ one thread per key row
    const int qd = warp & 3;
    const int wg = (warp - 2) >> 2;    // group 0 takes the even query tiles (buffer 0), group 1 the odd ones
    const int row = qd * 32 + lane;
    const int grow = k0 + row;
    const uint32_t tlane = tmem_base + ((uint32_t)(qd * 32) << 16);
    const float sl = p.scale * kLog2e;
    bool ok = true;
    for (int t = wg; t < n_q; t += 2) {
      const int s = t & 1;
      const int st = t % NSQ;
      const uint32_t ph = (uint32_t)(t >> 1) & 1u;
      const int qrow0 = (t_first + t) * 64;
      if (!wait_warp(bar(B_QF + st), (uint32_t)(t / NSQ) & 1u)) { ok = false; break; }
      if (!wait_warp(bar(B_SF + s), ph)) { ok = false; break; }
      tc5::fence_after_sync();
      const bool need_mask = p.causal && (qrow0 < k0 + 128);
      const float4* lse2 = reinterpret_cast<const float4*>(s_lse + st * 64);
      const float4* dlt = reinterpret_cast<const float4*>(s_delta + st * 64);
      uint32_t rs[2][32], rd[2][32];
      tc5::tmem_ld32(tlane + TM_ST + (uint32_t)s * 64u, rs[0]);
      tc5::tmem_ld32(tlane + TM_ST + (uint32_t)s * 64u + 32u, rs[1]);
      tc5::tmem_ld32(tlane + TM_DPT + (uint32_t)s * 64u, rd[0]);
      tc5::tmem_ld32(tlane + TM_DPT + (uint32_t)s * 64u + 32u, rd[1]);
      tc5::tmem_ld_wait();
      tc5::fence_before_sync();
      __syncwarp();
      if (lane == 0) tc5::mbar_arrive(bar(B_SE + s));    // the buffer may take tile t + 2
      if (!wait_warp(bar(B_PE + s), ph ^ 1u)) { ok = false; break; }
      const uint32_t prow = base + OFF_PT + s * TILE_P + (uint32_t)row * 128u;
      const uint32_t drow = base + OFF_DST + s * TILE_P + (uint32_t)row * 128u;
      const uint32_t swz = (uint32_t)(row & 7);
#pragma unroll
      for (int g = 0; g < 8; ++g) {    // 16-byte chunk g = queries 8g .. 8g+7 of the tile
        float e[8], ds[8];
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          const float4 l4 = lse2[g * 2 + hh];
          const float4 d4 = dlt[g * 2 + hh];
          const float la[4] = {l4.x, l4.y, l4.z, l4.w};
          const float da[4] = {d4.x, d4.y, d4.z, d4.w};
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int i = hh * 4 + u;
            const int ql = g * 8 + i;
            float ev = ex2(fmaf(__uint_as_float(rs[ql >> 5][ql & 31]), sl, -la[u]));
            if (need_mask && qrow0 + ql < grow) ev = 0.0f;
            e[i] = ev;
            ds[i] = ev * (__uint_as_float(rd[ql >> 5][ql & 31]) - da[u]);
          }
        }
        const uint32_t off = (((uint32_t)g) ^ swz) << 4;
        st_shared_v4(prow + off, pack_bf16(e[0], e[1]), pack_bf16(e[2], e[3]), pack_bf16(e[4], e[5]), pack_bf16(e[6], e[7]));
        st_shared_v4(drow + off, pack_bf16(ds[0], ds[1]), pack_bf16(ds[2], ds[3]), pack_bf16(ds[4], ds[5]), pack_bf16(ds[6], ds[7]));
      }
      tc5::fence_before_sync();
      fence_async_smem();
      __syncwarp();
      if (lane == 0) {
        tc5::mbar_arrive(bar(B_PF + s));
        tc5::mbar_arrive(bar(B_QE + st));
      }
    }
    if (ok && wait_warp(bar(B_ACC), 0u)) {
      tc5::fence_after_sync();
      __nv_bfloat16* dv = p.dv + (int64_t)b * p.dv_sb + (int64_t)grow * p.dv_ss + (int64_t)h * p.dv_sh;
      __nv_bfloat16* dk = p.dk + (int64_t)b * p.dk_sb + (int64_t)grow * p.dk_ss + (int64_t)h * p.dk_sh;
      // group 0 stores dV, group 1 stores dK
      __nv_bfloat16* dst = wg == 0 ? dv : dk;
      const float f = wg == 0 ? 1.0f : p.scale;
      const uint32_t tsrc = tlane + (wg == 0 ? TM_DV : TM_DK);
#pragma unroll
      for (int c = 0; c < 4; c += 2) {
        uint32_t r0[32], r1[32];
        float v[32];
        tc5::tmem_ld32(tsrc + (uint32_t)c * 32u, r0);
        tc5::tmem_ld32(tsrc + (uint32_t)c * 32u + 32u, r1);
        tc5::tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r0[i]) * f;
        if (grow < p.seqlen) st_row32(dst + c * 32, v);
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r1[i]) * f;
        if (grow < p.seqlen) st_row32(dst + c * 32 + 32, v);
      }
    }
  }

  __syncwarp();
  if (*abort_flag) __nanosleep(200000);
  tc5::fence_before_sync();
  __syncthreads();
  tc5::fence_after_sync();
  if (warp == 1) tc5::tmem_dealloc(tmem_base, TM_COLS);
}

// ================================================================================================= dQ
namespace dqk {
constexpr uint32_t PANEL_Q = 128 * 128;     // [128 query rows][64 bf16]
constexpr uint32_t TILE_Q = 2 * PANEL_Q;
constexpr uint32_t PANEL_KV = 64 * 128;     // [64 key rows][64 bf16]
constexpr uint32_t TILE_KV = 2 * PANEL_KV;
constexpr uint32_t TILE_DS = 128 * 128;     // [128 query rows][64 keys] bf16
constexpr int NSK = 4;    // ring of K/V stages: a stage is read by the first and by the last MMA of its tile
constexpr uint32_t OFF_Q = 0, OFF_DO = TILE_Q, OFF_K = 2 * TILE_Q, OFF_V = OFF_K + NSK * TILE_KV, OFF_DS = OFF_V + NSK * TILE_KV,
                   OFF_BAR = OFF_DS + 2 * TILE_DS;
enum { B_Q = 0, B_KF = 1, B_KE = B_KF + NSK, B_SF = B_KE + NSK, B_SE = B_SF + 2, B_PF = B_SE + 2, B_PE = B_PF + 2, B_ACC = B_PE + 2,
       NBAR = B_ACC + 1 };
constexpr int SMEM = OFF_BAR + NBAR * 8 + 16 + 1024;
constexpr uint32_t TM_S = 0, TM_DP = 128, TM_DQ = 256, TM_COLS = 512;
}    // namespace dqk

__global__ void __launch_bounds__(kTcThreads, 1)
attn_bwd_dq_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                      const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do, const TcParams p) {
  using namespace dqk;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = tc5::smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw_addr);
  const uint32_t bars = base + OFF_BAR;
  auto bar = [&](int i) { return bars + 8u * (uint32_t)i; };
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(smem + OFF_BAR + NBAR * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
  // Wait used by full warps that go on to warp-collective TMEM accesses: the outcome is made uniform.
  auto wait_warp = [&](uint32_t br, uint32_t ph) {
    return __all_sync(0xffffffffu, tc5::mbar_wait(br, ph, abort_flag, p.status, kStatusBit)) != 0;
  };

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int qt = (int)gridDim.x - 1 - (int)blockIdx.x;
  const int bh = blockIdx.y;
  const int b = bh / p.heads;
  const int h = bh - b * p.heads;
  const int q0 = qt * 128;
  const int nk_all = (p.seqlen + 63) / 64;
  const int n_kv = p.causal ? min(2 * qt + 2, nk_all) : nk_all;

  if (threadIdx.x == 0) {
    tc5::mbar_init(bar(B_Q), 1);
    for (int s = 0; s < NSK; ++s) {
      tc5::mbar_init(bar(B_KF + s), 1);
      tc5::mbar_init(bar(B_KE + s), 1);
    }
    for (int s = 0; s < 2; ++s) {
      tc5::mbar_init(bar(B_SF + s), 1);
      tc5::mbar_init(bar(B_SE + s), 4);
      tc5::mbar_init(bar(B_PF + s), 4);
      tc5::mbar_init(bar(B_PE + s), 1);
    }
    tc5::mbar_init(bar(B_ACC), 1);
    *abort_flag = 0;
    tc5::mbar_fence_init();
    tc5::tma_prefetch_desc(&map_q);
    tc5::tma_prefetch_desc(&map_k);
    tc5::tma_prefetch_desc(&map_v);
    tc5::tma_prefetch_desc(&map_do);
  }
  if (warp == 1) {
    tc5::tmem_alloc(tc5::smem_u32(tmem_holder), TM_COLS);
    tc5::tmem_relinquish();
  }
  tc5::fence_before_sync();
  __syncthreads();
  tc5::fence_after_sync();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    if (lane == 0) {
      tc5::mbar_arrive_expect_tx(bar(B_Q), 2 * TILE_Q);
      tc5::tma_load_4d(base + OFF_Q, &map_q, 0, h, q0, b, bar(B_Q));
      tc5::tma_load_4d(base + OFF_Q + PANEL_Q, &map_q, 64, h, q0, b, bar(B_Q));
      tc5::tma_load_4d(base + OFF_DO, &map_do, 0, h, q0, b, bar(B_Q));
      tc5::tma_load_4d(base + OFF_DO + PANEL_Q, &map_do, 64, h, q0, b, bar(B_Q));
      for (int j = 0; j < n_kv; ++j) {
        const int s = j % NSK;
        const uint32_t ph = (uint32_t)(j / NSK) & 1u;
        TC_WAIT(bar(B_KE + s), ph ^ 1u);
        tc5::mbar_arrive_expect_tx(bar(B_KF + s), 2 * TILE_KV);
        tc5::tma_load_4d(base + OFF_K + s * TILE_KV, &map_k, 0, h, j * 64, b, bar(B_KF + s));
        tc5::tma_load_4d(base + OFF_K + s * TILE_KV + PANEL_KV, &map_k, 64, h, j * 64, b, bar(B_KF + s));
        tc5::tma_load_4d(base + OFF_V + s * TILE_KV, &map_v, 0, h, j * 64, b, bar(B_KF + s));
        tc5::tma_load_4d(base + OFF_V + s * TILE_KV + PANEL_KV, &map_v, 64, h, j * 64, b, bar(B_KF + s));
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc_s = tc5::idesc_bf16(128, 64, 0, 0);
      const uint32_t idesc_acc = tc5::idesc_bf16(128, 128, 0, 1);
      auto issue_s = [&](int j) -> bool {
        const int s = j & 1;
        const int st = j % NSK;
        const uint32_t ph = (uint32_t)(j >> 1) & 1u;
        if (!tc5::mbar_wait(bar(B_SE + s), ph ^ 1u, abort_flag, p.status, kStatusBit)) return false;
        if (!tc5::mbar_wait(bar(B_KF + st), (uint32_t)(j / NSK) & 1u, abort_flag, p.status, kStatusBit)) return false;
        tc5::fence_after_sync();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t offa = (uint32_t)(kk >> 2) * PANEL_Q + (uint32_t)(kk & 3) * 32u;
          const uint32_t offb = (uint32_t)(kk >> 2) * PANEL_KV + (uint32_t)(kk & 3) * 32u;
          tc5::mma_f16(tmem_base + TM_S + (uint32_t)s * 64u, tc5::smem_desc_k_sw128(base + OFF_Q + offa),
                       tc5::smem_desc_k_sw128(base + OFF_K + st * TILE_KV + offb), idesc_s, kk ? 1u : 0u);
        }
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t offa = (uint32_t)(kk >> 2) * PANEL_Q + (uint32_t)(kk & 3) * 32u;
          const uint32_t offb = (uint32_t)(kk >> 2) * PANEL_KV + (uint32_t)(kk & 3) * 32u;
          tc5::mma_f16(tmem_base + TM_DP + (uint32_t)s * 64u, tc5::smem_desc_k_sw128(base + OFF_DO + offa),
                       tc5::smem_desc_k_sw128(base + OFF_V + st * TILE_KV + offb), idesc_s, kk ? 1u : 0u);
        }
        tc5::mma_commit(bar(B_SF + s));
        return true;
      };
      do {
        TC_WAIT(bar(B_Q), 0u);
        if (!issue_s(0)) break;
        if (n_kv > 1 && !issue_s(1)) break;
        bool ok = true;
        for (int j = 0; j < n_kv; ++j) {
          // the scores two tiles ahead go first: their buffer was released as soon as tile j had been read
          if (j + 2 < n_kv && !issue_s(j + 2)) { ok = false; break; }
          const int s = j & 1;
          const int st = j % NSK;
          const uint32_t ph = (uint32_t)(j >> 1) & 1u;
          if (!tc5::mbar_wait(bar(B_PF + s), ph, abort_flag, p.status, kStatusBit)) { ok = false; break; }
          tc5::fence_after_sync();
          // dQ += dS K_j : B = the K tile with the key index as rows (MN-major)
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            tc5::mma_f16(tmem_base + TM_DQ, tc5::smem_desc_k_sw128(base + OFF_DS + s * TILE_DS + (uint32_t)kk * 32u),
                         tc5::smem_desc_mn_sw128(base + OFF_K + st * TILE_KV + (uint32_t)kk * 2048u, PANEL_KV), idesc_acc,
                         (j | kk) ? 1u : 0u);
          }
          tc5::mma_commit(bar(B_PE + s));
          tc5::mma_commit(bar(B_KE + st));
        }
        if (ok) tc5::mma_commit(bar(B_ACC));
      } while (false);
    }
  } else {
    const int qd = warp & 3;
    const int wg = (warp - 2) >> 2;    // group 0 takes the even key tiles (buffer 0), group 1 the odd ones
    const int row = qd * 32 + lane;
    const int grow = q0 + row;
    const uint32_t tlane = tmem_base + ((uint32_t)(qd * 32) << 16);
    const float sl = p.scale * kLog2e;
    const bool in = grow < p.seqlen;
    const float lse2 = in ? p.lse[(int64_t)bh * p.seqlen + grow] * kLog2e : INFINITY;
    const float dlt = in ? p.delta[(int64_t)bh * p.seqlen + grow] : 0.0f;
    const int lim = p.causal ? min(grow, p.seqlen - 1) : p.seqlen - 1;
    bool ok = true;
    for (int j = wg; j < n_kv; j += 2) {
      const int s = j & 1;
      const uint32_t ph = (uint32_t)(j >> 1) & 1u;
      const int col0 = j * 64;
      if (!wait_warp(bar(B_SF + s), ph)) { ok = false; break; }
      tc5::fence_after_sync();
      const bool need_mask = (p.causal && col0 + 63 > q0) || (col0 + 64 > p.seqlen);
      uint32_t rs[2][32], rd[2][32];
      tc5::tmem_ld32(tlane + TM_S + (uint32_t)s * 64u, rs[0]);
      tc5::tmem_ld32(tlane + TM_S + (uint32_t)s * 64u + 32u, rs[1]);
      tc5::tmem_ld32(tlane + TM_DP + (uint32_t)s * 64u, rd[0]);
      tc5::tmem_ld32(tlane + TM_DP + (uint32_t)s * 64u + 32u, rd[1]);
      tc5::tmem_ld_wait();
      tc5::fence_before_sync();
      __syncwarp();
      if (lane == 0) tc5::mbar_arrive(bar(B_SE + s));    // the buffer may take tile j + 2
      if (!wait_warp(bar(B_PE + s), ph ^ 1u)) { ok = false; break; }
      const uint32_t drow = base + OFF_DS + s * TILE_DS + (uint32_t)row * 128u;
      const uint32_t swz = (uint32_t)(row & 7);
#pragma unroll
      for (int g = 0; g < 8; ++g) {    // 16-byte chunk g = keys 8g .. 8g+7 of the tile
        float ds[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int c = g * 8 + i;
          float e = ex2(fmaf(__uint_as_float(rs[c >> 5][c & 31]), sl, -lse2));
          if (need_mask && col0 + c > lim) e = 0.0f;
          ds[i] = e * (__uint_as_float(rd[c >> 5][c & 31]) - dlt);
        }
        st_shared_v4(drow + ((((uint32_t)g) ^ swz) << 4), pack_bf16(ds[0], ds[1]), pack_bf16(ds[2], ds[3]), pack_bf16(ds[4], ds[5]),
                     pack_bf16(ds[6], ds[7]));
      }
      tc5::fence_before_sync();
      fence_async_smem();
      __syncwarp();
      if (lane == 0) tc5::mbar_arrive(bar(B_PF + s));
    }
    if (ok && wait_warp(bar(B_ACC), 0u)) {
      tc5::fence_after_sync();
      __nv_bfloat16* dq = p.dq + (int64_t)b * p.dq_sb + (int64_t)grow * p.dq_ss + (int64_t)h * p.dq_sh;
      // each group stores one half of the row
      uint32_t r0[32], r1[32];
      float v[32];
      tc5::tmem_ld32(tlane + TM_DQ + (uint32_t)wg * 64u, r0);
      tc5::tmem_ld32(tlane + TM_DQ + (uint32_t)wg * 64u + 32u, r1);
      tc5::tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r0[i]) * p.scale;
      if (in) st_row32(dq + wg * 64, v);
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r1[i]) * p.scale;
      if (in) st_row32(dq + wg * 64 + 32, v);
    }
  }

  __syncwarp();
  if (*abort_flag) __nanosleep(200000);
  tc5::fence_before_sync();
  __syncthreads();
  tc5::fence_after_sync();
  if (warp == 1) tc5::tmem_dealloc(tmem_base, TM_COLS);
}

// ========================================================================= dK / dV, 128-query tiles, dS^T in tensor memory
namespace dkv2 {
constexpr uint32_t PANEL = 128 * 128;      // [128 rows][64 bf16]
constexpr uint32_t TILE = 2 * PANEL;       // 32 KB: 128 rows x 128 bf16
constexpr int NSQ = 2;                     // Q / dO stages (a stage is read by the first and by the last MMA of its tile)
constexpr uint32_t OFF_K = 0, OFF_V = TILE, OFF_Q = 2 * TILE, OFF_DO = OFF_Q + NSQ * TILE, OFF_PT = OFF_DO + NSQ * TILE,
                   OFF_LSE = OFF_PT + TILE, OFF_BAR = OFF_LSE + NSQ * 2 * 128 * 4;
enum { B_KV = 0, B_QF = 1, B_QE = B_QF + NSQ, B_SF = B_QE + NSQ, B_SE = B_SF + 1, B_DF = B_SE + 1, B_PF = B_DF + 1, B_PE = B_PF + 1,
       B_ACC = B_PE + 1, NBAR = B_ACC + 1 };
// seven 32 KB tiles leave 3 KB of the 227 KB: the dynamic array is declared 128-byte aligned, so rounding its start up to
// 1024 bytes costs at most 896
constexpr int SMEM = OFF_BAR + NBAR * 8 + 16 + 896;
static_assert(SMEM <= 227 * 1024, "dK/dV kernel: shared memory");
constexpr uint32_t TM_ST = 0, TM_DPT = 128, TM_DV = 256, TM_DK = 384, TM_COLS = 512;
}    // namespace dkv2

// dK and dV for 128 key rows; query tiles of 128, so that S^T = K Q^T and dP^T = V dO^T are N = 128 products (an M = 128
// bf16 MMA costs the same for N = 64).  Tensor memory holds exactly S^T, dP^T, dV and dK (4 x 128 columns).  The eight
// softmax warps split a tile by columns (group g: queries 64 g .. 64 g + 63).  S^T is read into registers and released
// at once, so the scores of the next tile are computed during the arithmetic of this one; P^T goes to shared memory (A
// operand of dV += P^T dO); dS^T is packed to bf16 and stored over the dP^T columns it came from (A operand of
// dK += dS^T Q, read from tensor memory).  dP^T of the next tile is issued after dK of this one (in-order tensor pipe).
__global__ void __launch_bounds__(kTcThreads, 1)
attn_bwd_dkdv_tm_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                        const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do, const TcParams p) {
  using namespace dkv2;
  extern __shared__ __align__(128) uint8_t smem_raw128[];
  const uint32_t raw_addr = tc5::smem_u32(smem_raw128);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* smem = smem_raw128 + (base - raw_addr);
  const uint32_t bars = base + OFF_BAR;
  auto bar = [&](int i) { return bars + 8u * (uint32_t)i; };
  float* s_lse = reinterpret_cast<float*>(smem + OFF_LSE);    // [NSQ][128] log2-scaled lse, then [NSQ][128] delta
  float* s_delta = s_lse + NSQ * 128;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(smem + OFF_BAR + NBAR * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
  auto wait_warp = [&](uint32_t br, uint32_t ph) {
    return __all_sync(0xffffffffu, tc5::mbar_wait(br, ph, abort_flag, p.status, kStatusBit)) != 0;
  };

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int kt = blockIdx.x;    // key tile 0 has the most query tiles under a causal mask and starts first
  const int bh = blockIdx.y;
  const int b = bh / p.heads;
  const int h = bh - b * p.heads;
  const int k0 = kt * 128;
  const int nq_all = (p.seqlen + 127) / 128;
  const int t_first = p.causal ? kt : 0;
  const int n_q = nq_all - t_first;    // >= 1 because k0 < seqlen

  if (threadIdx.x == 0) {
    tc5::mbar_init(bar(B_KV), 1);
    for (int s = 0; s < NSQ; ++s) {
      tc5::mbar_init(bar(B_QF + s), 2);    // TMA bytes + the lse/delta rows written by warp 0
      tc5::mbar_init(bar(B_QE + s), 9);    // last MMA that reads the stage + eight softmax warps
    }
    tc5::mbar_init(bar(B_SF), 1);
    tc5::mbar_init(bar(B_SE), 8);
    tc5::mbar_init(bar(B_DF), 1);
    tc5::mbar_init(bar(B_PF), 8);
    tc5::mbar_init(bar(B_PE), 1);
    tc5::mbar_init(bar(B_ACC), 1);
    *abort_flag = 0;
    tc5::mbar_fence_init();
    tc5::tma_prefetch_desc(&map_q);
    tc5::tma_prefetch_desc(&map_k);
    tc5::tma_prefetch_desc(&map_v);
    tc5::tma_prefetch_desc(&map_do);
  }
  if (warp == 1) {
    tc5::tmem_alloc(tc5::smem_u32(tmem_holder), TM_COLS);
    tc5::tmem_relinquish();
  }
  tc5::fence_before_sync();
  __syncthreads();
  tc5::fence_after_sync();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    // ------------------------------------------------------------------ producer (whole warp: lane 0 issues TMA)
    if (lane == 0) {
      tc5::mbar_arrive_expect_tx(bar(B_KV), 2 * TILE);
      tc5::tma_load_4d(base + OFF_K, &map_k, 0, h, k0, b, bar(B_KV));
      tc5::tma_load_4d(base + OFF_K + PANEL, &map_k, 64, h, k0, b, bar(B_KV));
      tc5::tma_load_4d(base + OFF_V, &map_v, 0, h, k0, b, bar(B_KV));
      tc5::tma_load_4d(base + OFF_V + PANEL, &map_v, 64, h, k0, b, bar(B_KV));
    }
    const float* glse = p.lse + (int64_t)bh * p.seqlen;
    const float* gdelta = p.delta + (int64_t)bh * p.seqlen;
    for (int t = 0; t < n_q; ++t) {
      const int s = t % NSQ;
      const uint32_t ph = (uint32_t)(t / NSQ) & 1u;
      const int qrow0 = (t_first + t) * 128;
      TC_WAIT(bar(B_QE + s), ph ^ 1u);
      if (lane == 0) {
        tc5::mbar_arrive_expect_tx(bar(B_QF + s), 2 * TILE);
        tc5::tma_load_4d(base + OFF_Q + s * TILE, &map_q, 0, h, qrow0, b, bar(B_QF + s));
        tc5::tma_load_4d(base + OFF_Q + s * TILE + PANEL, &map_q, 64, h, qrow0, b, bar(B_QF + s));
        tc5::tma_load_4d(base + OFF_DO + s * TILE, &map_do, 0, h, qrow0, b, bar(B_QF + s));
        tc5::tma_load_4d(base + OFF_DO + s * TILE + PANEL, &map_do, 64, h, qrow0, b, bar(B_QF + s));
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int r = lane + 32 * i;
        const bool in = qrow0 + r < p.seqlen;
        s_lse[s * 128 + r] = in ? glse[qrow0 + r] * kLog2e : INFINITY;    // +inf makes the probability exactly zero
        s_delta[s * 128 + r] = in ? gdelta[qrow0 + r] : 0.0f;
      }
      __syncwarp();
      if (lane == 0) tc5::mbar_arrive(bar(B_QF + s));
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc_s = tc5::idesc_bf16(128, 128, 0, 0);
      const uint32_t idesc_acc = tc5::idesc_bf16(128, 128, 0, 1);
      auto issue_st = [&](int t) -> bool {    // S^T = K Q_t^T
        const int st = t % NSQ;
        if (t > 0 && !tc5::mbar_wait(bar(B_SE), (uint32_t)(t - 1) & 1u, abort_flag, p.status, kStatusBit)) return false;
        if (!tc5::mbar_wait(bar(B_QF + st), (uint32_t)(t / NSQ) & 1u, abort_flag, p.status, kStatusBit)) return false;
        tc5::fence_after_sync();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t off = (uint32_t)(kk >> 2) * PANEL + (uint32_t)(kk & 3) * 32u;
          tc5::mma_f16(tmem_base + TM_ST, tc5::smem_desc_k_sw128(base + OFF_K + off), tc5::smem_desc_k_sw128(base + OFF_Q + st * TILE + off),
                       idesc_s, kk ? 1u : 0u);
        }
        tc5::mma_commit(bar(B_SF));
        return true;
      };
      auto issue_dpt = [&](int t) {    // dP^T = V dO_t^T (the stage was waited for by issue_st(t))
        const int st = t % NSQ;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t off = (uint32_t)(kk >> 2) * PANEL + (uint32_t)(kk & 3) * 32u;
          tc5::mma_f16(tmem_base + TM_DPT, tc5::smem_desc_k_sw128(base + OFF_V + off), tc5::smem_desc_k_sw128(base + OFF_DO + st * TILE + off),
                       idesc_s, kk ? 1u : 0u);
        }
        tc5::mma_commit(bar(B_DF));
      };
      do {
        TC_WAIT(bar(B_KV), 0u);
        if (!issue_st(0)) break;
        issue_dpt(0);
        bool ok = true;
        for (int t = 0; t < n_q; ++t) {
          const int st = t % NSQ;
          // the scores of the next tile go first when their operands are already there (the usual case); otherwise they
          // follow dK of this tile, so that a late Q / dO stage does not hold up the products that are ready
          bool pending = t + 1 < n_q;
          if (pending && tc5::mbar_test(bar(B_SE), (uint32_t)t & 1u) &&
              tc5::mbar_test(bar(B_QF + (t + 1) % NSQ), (uint32_t)((t + 1) / NSQ) & 1u)) {
            if (!issue_st(t + 1)) { ok = false; break; }
            pending = false;
          }
          if (!tc5::mbar_wait(bar(B_PF), (uint32_t)t & 1u, abort_flag, p.status, kStatusBit)) { ok = false; break; }
          tc5::fence_after_sync();
          // dV += P^T dO_t : A = P^T from shared memory (K-major over the 128 queries), B = dO read MN-major
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            tc5::mma_f16(tmem_base + TM_DV, tc5::smem_desc_k_sw128(base + OFF_PT + (uint32_t)(kk >> 2) * PANEL + (uint32_t)(kk & 3) * 32u),
                         tc5::smem_desc_mn_sw128(base + OFF_DO + st * TILE + (uint32_t)kk * 2048u, PANEL), idesc_acc, (t | kk) ? 1u : 0u);
          }
          tc5::mma_commit(bar(B_PE));
          // dK += dS^T Q_t : A = dS^T from tensor memory (group g: 32 packed columns at the start of its half), B = Q MN-major
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            tc5::mma_f16_ta(tmem_base + TM_DK, tmem_base + TM_DPT + (uint32_t)(kk >> 2) * 64u + (uint32_t)(kk & 3) * 8u,
                            tc5::smem_desc_mn_sw128(base + OFF_Q + st * TILE + (uint32_t)kk * 2048u, PANEL), idesc_acc, (t | kk) ? 1u : 0u);
          }
          tc5::mma_commit(bar(B_QE + st));
          if (pending && !issue_st(t + 1)) { ok = false; break; }
          if (t + 1 < n_q) issue_dpt(t + 1);
        }
        if (ok) tc5::mma_commit(bar(B_ACC));
      } while (false);
    }
  } else {
    // ------------------------------------------------------------------ one thread per key row and query half
    const int qd = warp & 3;
    const int wg = (warp - 2) >> 2;    // group g: queries 64 g .. 64 g + 63 of every tile
    const int row = qd * 32 + lane;
    const int grow = k0 + row;
    const uint32_t tlane = tmem_base + ((uint32_t)(qd * 32) << 16);
    const float sl = p.scale * kLog2e;
    const uint32_t prow = base + OFF_PT + (uint32_t)wg * PANEL + (uint32_t)row * 128u;
    const uint32_t swz = (uint32_t)(row & 7);
    bool ok = true;
    for (int t = 0; t < n_q; ++t) {
      const int st = t % NSQ;
      const int qrow0 = (t_first + t) * 128 + wg * 64;    // first query of this group's half
      if (!wait_warp(bar(B_QF + st), (uint32_t)(t / NSQ) & 1u)) { ok = false; break; }
      if (!wait_warp(bar(B_SF), (uint32_t)t & 1u)) { ok = false; break; }
      tc5::fence_after_sync();
      const bool need_mask = p.causal && (qrow0 < k0 + 128);
      const float4* lse2 = reinterpret_cast<const float4*>(s_lse + st * 128 + wg * 64);
      const float4* dlt = reinterpret_cast<const float4*>(s_delta + st * 128 + wg * 64);
      uint32_t rs[2][32], rd[2][32];
      tc5::tmem_ld32(tlane + TM_ST + (uint32_t)wg * 64u, rs[0]);
      tc5::tmem_ld32(tlane + TM_ST + (uint32_t)wg * 64u + 32u, rs[1]);
      tc5::tmem_ld_wait();
      tc5::fence_before_sync();
      __syncwarp();
      if (lane == 0) tc5::mbar_arrive(bar(B_SE));    // the score tile may take tile t + 1
      if (!wait_warp(bar(B_DF), (uint32_t)t & 1u)) { ok = false; break; }
      tc5::fence_after_sync();
      tc5::tmem_ld32(tlane + TM_DPT + (uint32_t)wg * 64u, rd[0]);
      tc5::tmem_ld32(tlane + TM_DPT + (uint32_t)wg * 64u + 32u, rd[1]);
      tc5::tmem_ld_wait();
      if (t > 0 && !wait_warp(bar(B_PE), (uint32_t)(t - 1) & 1u)) { ok = false; break; }    // dV of the previous tile has read P^T
      uint32_t pk[32];
#pragma unroll
      for (int g = 0; g < 8; ++g) {    // 16-byte chunk g = queries 8g .. 8g+7 of this half
        float e[8], ds[8];
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          const float4 l4 = lse2[g * 2 + hh];
          const float4 d4 = dlt[g * 2 + hh];
          const float la[4] = {l4.x, l4.y, l4.z, l4.w};
          const float da[4] = {d4.x, d4.y, d4.z, d4.w};
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int i = hh * 4 + u;
            const int ql = g * 8 + i;
            float ev = ex2(fmaf(__uint_as_float(rs[ql >> 5][ql & 31]), sl, -la[u]));
            if (need_mask && qrow0 + ql < grow) ev = 0.0f;
            e[i] = ev;
            ds[i] = ev * (__uint_as_float(rd[ql >> 5][ql & 31]) - da[u]);
          }
        }
        st_shared_v4(prow + ((((uint32_t)g) ^ swz) << 4), pack_bf16(e[0], e[1]), pack_bf16(e[2], e[3]), pack_bf16(e[4], e[5]),
                     pack_bf16(e[6], e[7]));
        pk[4 * g] = pack_bf16(ds[0], ds[1]);
        pk[4 * g + 1] = pack_bf16(ds[2], ds[3]);
        pk[4 * g + 2] = pack_bf16(ds[4], ds[5]);
        pk[4 * g + 3] = pack_bf16(ds[6], ds[7]);
      }
      tc5::tmem_st32(tlane + TM_DPT + (uint32_t)wg * 64u, pk);
      tc5::tmem_st_wait();
      tc5::fence_before_sync();
      fence_async_smem();
      __syncwarp();
      if (lane == 0) {
        tc5::mbar_arrive(bar(B_PF));
        tc5::mbar_arrive(bar(B_QE + st));
      }
    }
    if (ok && wait_warp(bar(B_ACC), 0u)) {
      tc5::fence_after_sync();
      __nv_bfloat16* dv = p.dv + (int64_t)b * p.dv_sb + (int64_t)grow * p.dv_ss + (int64_t)h * p.dv_sh;
      __nv_bfloat16* dk = p.dk + (int64_t)b * p.dk_sb + (int64_t)grow * p.dk_ss + (int64_t)h * p.dk_sh;
      // group 0 stores dV, group 1 stores dK
      __nv_bfloat16* dst = wg == 0 ? dv : dk;
      const float f = wg == 0 ? 1.0f : p.scale;
      const uint32_t tsrc = tlane + (wg == 0 ? TM_DV : TM_DK);
#pragma unroll
      for (int c = 0; c < 4; c += 2) {
        uint32_t r0[32], r1[32];
        float v[32];
        tc5::tmem_ld32(tsrc + (uint32_t)c * 32u, r0);
        tc5::tmem_ld32(tsrc + (uint32_t)c * 32u + 32u, r1);
        tc5::tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r0[i]) * f;
        if (grow < p.seqlen) st_row32(dst + c * 32, v);
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r1[i]) * f;
        if (grow < p.seqlen) st_row32(dst + c * 32 + 32, v);
      }
    }
  }

  __syncwarp();
  if (*abort_flag) __nanosleep(200000);
  tc5::fence_before_sync();
  __syncthreads();
  tc5::fence_after_sync();
  if (warp == 1) tc5::tmem_dealloc(tmem_base, TM_COLS);
}

// ================================================================================ dQ, 128-key tiles, dS in tensor memory
namespace dqk2 {
constexpr uint32_t PANEL = 128 * 128;      // [128 rows][64 bf16]: one 64-wide slice of the head dimension
constexpr uint32_t TILE = 2 * PANEL;       // 32 KB: 128 rows x 128 bf16
constexpr int NK = 3;    // K tiles: read by the first (S) and by the last (dQ) MMA of their step, so three are alive
constexpr int NV = 2;    // V tiles: read by dP only
constexpr uint32_t OFF_Q = 0, OFF_DO = TILE, OFF_K = 2 * TILE, OFF_V = OFF_K + NK * TILE, OFF_BAR = OFF_V + NV * TILE;
enum { B_Q = 0, B_KF = 1, B_KE = B_KF + NK, B_VF = B_KE + NK, B_VE = B_VF + NV, B_SF = B_VE + NV, B_SE = B_SF + 1, B_DF = B_SE + 1,
       B_PF = B_DF + 2, B_ACC = B_PF + 2, NBAR = B_ACC + 1 };
constexpr int SMEM = OFF_BAR + NBAR * 8 + 16 + 1024;
// one 128-column score tile, two 128-column dP tiles (dS is written over the dP tile it came from), dQ
constexpr uint32_t TM_S = 0, TM_DP = 128, TM_DQ = 384, TM_COLS = 512;
}    // namespace dqk2

// dQ for 128 query rows; key tiles of 128 (an M = 128 bf16 MMA costs the same ~70 cycles for N = 64 and N = 128, so the
// two score products S = Q K^T and dP = dO V^T are issued over 128 keys at a time).  The eight softmax warps split every
// tile by columns (group g: keys [128 T + 64 g, + 64)).  S is read into registers and its tile released at once; dS is
// packed to bf16 and stored with tcgen05.st over the dP columns it was computed from (group g: the first 32 columns of
// its 64-column half), from where dQ += dS K reads it as the A operand: no shared-memory round trip, and the two dP tiles
// alternate so that dP of tile T + 1 is computed while dS of tile T is still being consumed.  The tensor pipe executes
// MMAs in issue order, so dP(T + 2) may overwrite tile T & 1 once it is issued after dQ(T).
__global__ void __launch_bounds__(kTcThreads, 1)
attn_bwd_dq_tm_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                      const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do, const TcParams p) {
  using namespace dqk2;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = tc5::smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw_addr);
  const uint32_t bars = base + OFF_BAR;
  auto bar = [&](int i) { return bars + 8u * (uint32_t)i; };
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(smem + OFF_BAR + NBAR * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
  auto wait_warp = [&](uint32_t br, uint32_t ph) {
    return __all_sync(0xffffffffu, tc5::mbar_wait(br, ph, abort_flag, p.status, kStatusBit)) != 0;
  };

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int qt = (int)gridDim.x - 1 - (int)blockIdx.x;
  const int bh = blockIdx.y;
  const int b = bh / p.heads;
  const int h = bh - b * p.heads;
  const int q0 = qt * 128;
  const int nk_all = (p.seqlen + 63) / 64;
  const int n_kv = p.causal ? min(2 * qt + 2, nk_all) : nk_all;    // 64-key halves with a visible key
  const int n_t = (n_kv + 1) >> 1;                                 // 128-key tiles; a trailing odd half is fully masked

  if (threadIdx.x == 0) {
    tc5::mbar_init(bar(B_Q), 1);
    for (int s = 0; s < NK; ++s) {
      tc5::mbar_init(bar(B_KF + s), 1);
      tc5::mbar_init(bar(B_KE + s), 1);
    }
    for (int s = 0; s < NV; ++s) {
      tc5::mbar_init(bar(B_VF + s), 1);
      tc5::mbar_init(bar(B_VE + s), 1);
    }
    tc5::mbar_init(bar(B_SF), 1);
    tc5::mbar_init(bar(B_SE), 8);
    for (int s = 0; s < 2; ++s) {
      tc5::mbar_init(bar(B_DF + s), 1);
      tc5::mbar_init(bar(B_PF + s), 8);
    }
    tc5::mbar_init(bar(B_ACC), 1);
    *abort_flag = 0;
    tc5::mbar_fence_init();
    tc5::tma_prefetch_desc(&map_q);
    tc5::tma_prefetch_desc(&map_k);
    tc5::tma_prefetch_desc(&map_v);
    tc5::tma_prefetch_desc(&map_do);
  }
  if (warp == 1) {
    tc5::tmem_alloc(tc5::smem_u32(tmem_holder), TM_COLS);
    tc5::tmem_relinquish();
  }
  tc5::fence_before_sync();
  __syncthreads();
  tc5::fence_after_sync();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    if (lane == 0) {
      tc5::mbar_arrive_expect_tx(bar(B_Q), 2 * TILE);
      tc5::tma_load_4d(base + OFF_Q, &map_q, 0, h, q0, b, bar(B_Q));
      tc5::tma_load_4d(base + OFF_Q + PANEL, &map_q, 64, h, q0, b, bar(B_Q));
      tc5::tma_load_4d(base + OFF_DO, &map_do, 0, h, q0, b, bar(B_Q));
      tc5::tma_load_4d(base + OFF_DO + PANEL, &map_do, 64, h, q0, b, bar(B_Q));
      for (int t = 0; t < n_t; ++t) {
        const int ks = t % NK, vs = t % NV;
        TC_WAIT(bar(B_KE + ks), ((uint32_t)(t / NK) & 1u) ^ 1u);
        tc5::mbar_arrive_expect_tx(bar(B_KF + ks), TILE);
        tc5::tma_load_4d(base + OFF_K + ks * TILE, &map_k, 0, h, t * 128, b, bar(B_KF + ks));
        tc5::tma_load_4d(base + OFF_K + ks * TILE + PANEL, &map_k, 64, h, t * 128, b, bar(B_KF + ks));
        TC_WAIT(bar(B_VE + vs), ((uint32_t)(t / NV) & 1u) ^ 1u);
        tc5::mbar_arrive_expect_tx(bar(B_VF + vs), TILE);
        tc5::tma_load_4d(base + OFF_V + vs * TILE, &map_v, 0, h, t * 128, b, bar(B_VF + vs));
        tc5::tma_load_4d(base + OFF_V + vs * TILE + PANEL, &map_v, 64, h, t * 128, b, bar(B_VF + vs));
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc_s = tc5::idesc_bf16(128, 128, 0, 0);
      const uint32_t idesc_acc = tc5::idesc_bf16(128, 128, 0, 1);
      // S = Q K_t^T (single tile, released by the softmax warps as soon as they hold it in registers) and
      // dP[t & 1] = dO V_t^T
      auto issue_s = [&](int t) -> bool {
        const int ks = t % NK, vs = t % NV;
        if (t > 0 && !tc5::mbar_wait(bar(B_SE), (uint32_t)(t - 1) & 1u, abort_flag, p.status, kStatusBit)) return false;
        if (!tc5::mbar_wait(bar(B_KF + ks), (uint32_t)(t / NK) & 1u, abort_flag, p.status, kStatusBit)) return false;
        tc5::fence_after_sync();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t off = (uint32_t)(kk >> 2) * PANEL + (uint32_t)(kk & 3) * 32u;
          tc5::mma_f16(tmem_base + TM_S, tc5::smem_desc_k_sw128(base + OFF_Q + off), tc5::smem_desc_k_sw128(base + OFF_K + ks * TILE + off),
                       idesc_s, kk ? 1u : 0u);
        }
        tc5::mma_commit(bar(B_SF));
        if (!tc5::mbar_wait(bar(B_VF + vs), (uint32_t)(t / NV) & 1u, abort_flag, p.status, kStatusBit)) return false;
        tc5::fence_after_sync();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t off = (uint32_t)(kk >> 2) * PANEL + (uint32_t)(kk & 3) * 32u;
          tc5::mma_f16(tmem_base + TM_DP + (uint32_t)(t & 1) * 128u, tc5::smem_desc_k_sw128(base + OFF_DO + off),
                       tc5::smem_desc_k_sw128(base + OFF_V + vs * TILE + off), idesc_s, kk ? 1u : 0u);
        }
        tc5::mma_commit(bar(B_VE + vs));
        tc5::mma_commit(bar(B_DF + (t & 1)));
        return true;
      };
      do {
        TC_WAIT(bar(B_Q), 0u);
        if (!issue_s(0)) break;
        bool ok = true;
        for (int t = 0; t < n_t; ++t) {
          if (t + 1 < n_t && !issue_s(t + 1)) { ok = false; break; }
          const int ks = t % NK;
          if (!tc5::mbar_wait(bar(B_PF + (t & 1)), (uint32_t)(t >> 1) & 1u, abort_flag, p.status, kStatusBit)) { ok = false; break; }
          tc5::fence_after_sync();
          // dQ += dS K_t : A = dS from tensor memory (group g wrote keys 64 g .. 64 g + 63 as 32 packed columns at the start
          // of its half), B = the K tile with the key index as rows (MN-major)
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            tc5::mma_f16_ta(tmem_base + TM_DQ,
                            tmem_base + TM_DP + (uint32_t)(t & 1) * 128u + (uint32_t)(kk >> 2) * 64u + (uint32_t)(kk & 3) * 8u,
                            tc5::smem_desc_mn_sw128(base + OFF_K + ks * TILE + (uint32_t)kk * 2048u, PANEL), idesc_acc, (t | kk) ? 1u : 0u);
          }
          tc5::mma_commit(bar(B_KE + ks));
        }
        if (ok) tc5::mma_commit(bar(B_ACC));
      } while (false);
    }
  } else {
    const int qd = warp & 3;
    const int wg = (warp - 2) >> 2;    // group g: the g-th 64-key half of every tile
    const int row = qd * 32 + lane;
    const int grow = q0 + row;
    const uint32_t tlane = tmem_base + ((uint32_t)(qd * 32) << 16);
    const float sl = p.scale * kLog2e;
    const bool in = grow < p.seqlen;
    const float lse2 = in ? p.lse[(int64_t)bh * p.seqlen + grow] * kLog2e : INFINITY;
    const float dlt = in ? p.delta[(int64_t)bh * p.seqlen + grow] : 0.0f;
    const int lim = p.causal ? min(grow, p.seqlen - 1) : p.seqlen - 1;
    bool ok = true;
    for (int t = 0; t < n_t; ++t) {
      const int col0 = (2 * t + wg) * 64;
      const uint32_t tdp = tlane + TM_DP + (uint32_t)(t & 1) * 128u + (uint32_t)wg * 64u;
      if (!wait_warp(bar(B_SF), (uint32_t)t & 1u)) { ok = false; break; }
      tc5::fence_after_sync();
      const bool need_mask = (p.causal && col0 + 63 > q0) || (col0 + 64 > p.seqlen);
      uint32_t rs[2][32], rd[2][32];
      tc5::tmem_ld32(tlane + TM_S + (uint32_t)wg * 64u, rs[0]);
      tc5::tmem_ld32(tlane + TM_S + (uint32_t)wg * 64u + 32u, rs[1]);
      tc5::tmem_ld_wait();
      tc5::fence_before_sync();
      __syncwarp();
      if (lane == 0) tc5::mbar_arrive(bar(B_SE));    // the score tile may take tile t + 1
      if (!wait_warp(bar(B_DF + (t & 1)), (uint32_t)(t >> 1) & 1u)) { ok = false; break; }
      tc5::fence_after_sync();
      tc5::tmem_ld32(tdp, rd[0]);
      tc5::tmem_ld32(tdp + 32u, rd[1]);
      tc5::tmem_ld_wait();
      uint32_t pk[32];
#pragma unroll
      for (int g = 0; g < 8; ++g) {    // keys 8g .. 8g+7 of this half -> packed columns 4g .. 4g+3
        float ds[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int c = g * 8 + i;
          float e = ex2(fmaf(__uint_as_float(rs[c >> 5][c & 31]), sl, -lse2));
          if (need_mask && col0 + c > lim) e = 0.0f;
          ds[i] = e * (__uint_as_float(rd[c >> 5][c & 31]) - dlt);
        }
        pk[4 * g] = pack_bf16(ds[0], ds[1]);
        pk[4 * g + 1] = pack_bf16(ds[2], ds[3]);
        pk[4 * g + 2] = pack_bf16(ds[4], ds[5]);
        pk[4 * g + 3] = pack_bf16(ds[6], ds[7]);
      }
      tc5::tmem_st32(tdp, pk);
      tc5::tmem_st_wait();
      tc5::fence_before_sync();
      __syncwarp();
      if (lane == 0) tc5::mbar_arrive(bar(B_PF + (t & 1)));
    }
    if (ok && wait_warp(bar(B_ACC), 0u)) {
      tc5::fence_after_sync();
      __nv_bfloat16* dq = p.dq + (int64_t)b * p.dq_sb + (int64_t)grow * p.dq_ss + (int64_t)h * p.dq_sh;
      // each group stores one half of the row
      uint32_t r0[32], r1[32];
      float v[32];
      tc5::tmem_ld32(tlane + TM_DQ + (uint32_t)wg * 64u, r0);
      tc5::tmem_ld32(tlane + TM_DQ + (uint32_t)wg * 64u + 32u, r1);
      tc5::tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r0[i]) * p.scale;
      if (in) st_row32(dq + wg * 64, v);
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r1[i]) * p.scale;
      if (in) st_row32(dq + wg * 64 + 32, v);
    }
  }

  __syncwarp();
  if (*abort_flag) __nanosleep(200000);
  tc5::fence_before_sync();
  __syncthreads();
  tc5::fence_after_sync();
  if (warp == 1) tc5::tmem_dealloc(tmem_base, TM_COLS);
}

// ============================================================================ dQ, persistent CTAs over the work items
namespace dqk3 {
using namespace dqk2;
enum { B3_QE = NBAR, B3_OE = NBAR + 1, NBAR3 = NBAR + 2 };
constexpr int SMEM3 = OFF_BAR + NBAR3 * 8 + 16 + 1024;
}    // namespace dqk3

// Work item -> (level, batch * head) for the persistent attention kernels: groups of G heads, inside a group by rising
// level (level 0 is the longest row), so that consecutive waves work on the same heads (their K / V or Q / dO stay in
// L2) and a walk that alternates direction per wave gives every CTA the same amount of work per group.
struct ItemOrder {
  int n_lv, bh_total, G;
  __device__ __forceinline__ void decode(int item, int& level, int& bh) const {
    const int g = item / (G * n_lv);
    const int hg = min(G, bh_total - g * G);
    const int j = item - g * G * n_lv;
    level = j / hg;
    bh = g * G + j % hg;
  }
};

// attn_bwd_dq_tm_kernel with one CTA per SM walking the (query tile, batch * head) items.  Rings, the score tile and
// the dP tiles keep running across items (one global tile counter), so Q / dO / K / V of the next item are loaded and
// its first score products issued while the softmax warps still store dQ of the current one.  B3_QE: the score products
// of an item are complete, Q and dO may be overwritten; B3_OE: the softmax warps have read dQ, the accumulator may be
// overwritten by the first product of the next item.
__global__ void __launch_bounds__(kTcThreads, 1)
attn_bwd_dq_ps_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                      const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do, const TcParams p, int n_qt,
                      int n_items) {
  using namespace dqk3;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = tc5::smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw_addr);
  const uint32_t bars = base + OFF_BAR;
  auto bar = [&](int i) { return bars + 8u * (uint32_t)i; };
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(smem + OFF_BAR + NBAR3 * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
  auto wait_warp = [&](uint32_t br, uint32_t ph) {
    return __all_sync(0xffffffffu, tc5::mbar_wait(br, ph, abort_flag, p.status, kStatusBit)) != 0;
  };
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int nk_all = (p.seqlen + 63) / 64;
  const ItemOrder order{n_qt, p.batch * p.heads, max(1, (4 * (int)gridDim.x) / n_qt)};
  const int n_waves = (n_items + (int)gridDim.x - 1) / (int)gridDim.x;
  auto item_at = [&](int w) {
    const int c = (w & 1) ? (int)gridDim.x - 1 - (int)blockIdx.x : (int)blockIdx.x;
    return w * (int)gridDim.x + c;
  };
  auto tiles_of = [&](int qt) {
    const int n_kv = p.causal ? min(2 * qt + 2, nk_all) : nk_all;
    return (n_kv + 1) >> 1;
  };

  if (threadIdx.x == 0) {
    tc5::mbar_init(bar(B_Q), 1);
    for (int s = 0; s < NK; ++s) {
      tc5::mbar_init(bar(B_KF + s), 1);
      tc5::mbar_init(bar(B_KE + s), 1);
    }
    for (int s = 0; s < NV; ++s) {
      tc5::mbar_init(bar(B_VF + s), 1);
      tc5::mbar_init(bar(B_VE + s), 1);
    }
    tc5::mbar_init(bar(B_SF), 1);
    tc5::mbar_init(bar(B_SE), 8);
    for (int s = 0; s < 2; ++s) {
      tc5::mbar_init(bar(B_DF + s), 1);
      tc5::mbar_init(bar(B_PF + s), 8);
    }
    tc5::mbar_init(bar(B_ACC), 1);
    tc5::mbar_init(bar(B3_QE), 1);
    tc5::mbar_init(bar(B3_OE), 8);
    *abort_flag = 0;
    tc5::mbar_fence_init();
    tc5::tma_prefetch_desc(&map_q);
    tc5::tma_prefetch_desc(&map_k);
    tc5::tma_prefetch_desc(&map_v);
    tc5::tma_prefetch_desc(&map_do);
  }
  if (warp == 1) {
    tc5::tmem_alloc(tc5::smem_u32(tmem_holder), TM_COLS);
    tc5::tmem_relinquish();
  }
  tc5::fence_before_sync();
  __syncthreads();
  tc5::fence_after_sync();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    if (lane == 0) {
      int gt = 0, it = 0;
      bool ok = true;
      for (int w = 0; w < n_waves && ok; ++w) {
        const int item = item_at(w);
        if (item >= n_items) continue;
        int level, bh;
        order.decode(item, level, bh);
        const int qt = n_qt - 1 - level;
        const int b = bh / p.heads, h = bh - b * p.heads;
        const int n_t = tiles_of(qt);
        if (it > 0 && !tc5::mbar_wait(bar(B3_QE), (uint32_t)(it - 1) & 1u, abort_flag, p.status, kStatusBit)) break;
        tc5::mbar_arrive_expect_tx(bar(B_Q), 2 * TILE);
        tc5::tma_load_4d(base + OFF_Q, &map_q, 0, h, qt * 128, b, bar(B_Q));
        tc5::tma_load_4d(base + OFF_Q + PANEL, &map_q, 64, h, qt * 128, b, bar(B_Q));
        tc5::tma_load_4d(base + OFF_DO, &map_do, 0, h, qt * 128, b, bar(B_Q));
        tc5::tma_load_4d(base + OFF_DO + PANEL, &map_do, 64, h, qt * 128, b, bar(B_Q));
        for (int t = 0; t < n_t; ++t, ++gt) {
          const int ks = gt % NK, vs = gt % NV;
          if (!tc5::mbar_wait(bar(B_KE + ks), ((uint32_t)(gt / NK) & 1u) ^ 1u, abort_flag, p.status, kStatusBit)) { ok = false; break; }
          tc5::mbar_arrive_expect_tx(bar(B_KF + ks), TILE);
          tc5::tma_load_4d(base + OFF_K + ks * TILE, &map_k, 0, h, t * 128, b, bar(B_KF + ks));
          tc5::tma_load_4d(base + OFF_K + ks * TILE + PANEL, &map_k, 64, h, t * 128, b, bar(B_KF + ks));
          if (!tc5::mbar_wait(bar(B_VE + vs), ((uint32_t)(gt / NV) & 1u) ^ 1u, abort_flag, p.status, kStatusBit)) { ok = false; break; }
          tc5::mbar_arrive_expect_tx(bar(B_VF + vs), TILE);
          tc5::tma_load_4d(base + OFF_V + vs * TILE, &map_v, 0, h, t * 128, b, bar(B_VF + vs));
          tc5::tma_load_4d(base + OFF_V + vs * TILE + PANEL, &map_v, 64, h, t * 128, b, bar(B_VF + vs));
        }
        ++it;
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc_s = tc5::idesc_bf16(128, 128, 0, 0);
      const uint32_t idesc_acc = tc5::idesc_bf16(128, 128, 0, 1);
      // S = Q K^T and dP[gt & 1] = dO V^T for the gt-th tile of this CTA
      auto issue_s = [&](int gt) -> bool {
        const int ks = gt % NK, vs = gt % NV;
        // data barriers first (they pass while the softmax warps still hold S), so that the two products are issued back
        // to back once S is free: a wait between them idles the tensor pipe for 100+ cycles even when V is there
        if (!tc5::mbar_wait(bar(B_KF + ks), (uint32_t)(gt / NK) & 1u, abort_flag, p.status, kStatusBit)) return false;
        if (!tc5::mbar_wait(bar(B_VF + vs), (uint32_t)(gt / NV) & 1u, abort_flag, p.status, kStatusBit)) return false;
        if (gt > 0 && !tc5::mbar_wait(bar(B_SE), (uint32_t)(gt - 1) & 1u, abort_flag, p.status, kStatusBit)) return false;
        tc5::fence_after_sync();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t off = (uint32_t)(kk >> 2) * PANEL + (uint32_t)(kk & 3) * 32u;
          tc5::mma_f16(tmem_base + TM_S, tc5::smem_desc_k_sw128(base + OFF_Q + off), tc5::smem_desc_k_sw128(base + OFF_K + ks * TILE + off),
                       idesc_s, kk ? 1u : 0u);
        }
        tc5::mma_commit(bar(B_SF));
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t off = (uint32_t)(kk >> 2) * PANEL + (uint32_t)(kk & 3) * 32u;
          tc5::mma_f16(tmem_base + TM_DP + (uint32_t)(gt & 1) * 128u, tc5::smem_desc_k_sw128(base + OFF_DO + off),
                       tc5::smem_desc_k_sw128(base + OFF_V + vs * TILE + off), idesc_s, kk ? 1u : 0u);
        }
        tc5::mma_commit(bar(B_VE + vs));
        tc5::mma_commit(bar(B_DF + (gt & 1)));
        return true;
      };
      int g0 = 0, it = 0;
      bool ok = true;
      for (int w = 0; w < n_waves && ok; ++w) {
        const int item = item_at(w);
        if (item >= n_items) continue;
        int level, bh;
        order.decode(item, level, bh);
        const int n_t = tiles_of(n_qt - 1 - level);
        if (!tc5::mbar_wait(bar(B_Q), (uint32_t)it & 1u, abort_flag, p.status, kStatusBit)) { ok = false; break; }
        if (!issue_s(g0)) { ok = false; break; }
        if (n_t == 1) tc5::mma_commit(bar(B3_QE));
        if (it > 0 && !tc5::mbar_wait(bar(B3_OE), (uint32_t)(it - 1) & 1u, abort_flag, p.status, kStatusBit)) { ok = false; break; }
        for (int t = 0; t < n_t; ++t) {
          const int gt = g0 + t;
          if (t + 1 < n_t) {
            if (!issue_s(gt + 1)) { ok = false; break; }
            if (t + 2 == n_t) tc5::mma_commit(bar(B3_QE));    // every score product of this item is issued
          }
          const int ks = gt % NK;
          if (!tc5::mbar_wait(bar(B_PF + (gt & 1)), (uint32_t)(gt >> 1) & 1u, abort_flag, p.status, kStatusBit)) { ok = false; break; }
          tc5::fence_after_sync();
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            tc5::mma_f16_ta(tmem_base + TM_DQ,
                            tmem_base + TM_DP + (uint32_t)(gt & 1) * 128u + (uint32_t)(kk >> 2) * 64u + (uint32_t)(kk & 3) * 8u,
                            tc5::smem_desc_mn_sw128(base + OFF_K + ks * TILE + (uint32_t)kk * 2048u, PANEL), idesc_acc, (t | kk) ? 1u : 0u);
          }
          tc5::mma_commit(bar(B_KE + ks));
        }
        if (!ok) break;
        tc5::mma_commit(bar(B_ACC));
        g0 += n_t;
        ++it;
      }
    }
  } else {
    const int qd = warp & 3;
    const int wg = (warp - 2) >> 2;    // group g: the g-th 64-key half of every tile
    const int row = qd * 32 + lane;
    const uint32_t tlane = tmem_base + ((uint32_t)(qd * 32) << 16);
    const float sl = p.scale * kLog2e;
    int g0 = 0, it = 0;
    bool ok = true;
    for (int w = 0; w < n_waves && ok; ++w) {
      const int item = item_at(w);
      if (item >= n_items) continue;
      int level, bh;
      order.decode(item, level, bh);
      const int qt = n_qt - 1 - level;
      const int b = bh / p.heads, h = bh - b * p.heads;
      const int n_t = tiles_of(qt);
      const int q0 = qt * 128;
      const int grow = q0 + row;
      const bool in = grow < p.seqlen;
      const float lse2 = in ? p.lse[(int64_t)bh * p.seqlen + grow] * kLog2e : INFINITY;
      const float dlt = in ? p.delta[(int64_t)bh * p.seqlen + grow] : 0.0f;
      const int lim = p.causal ? min(grow, p.seqlen - 1) : p.seqlen - 1;
      for (int t = 0; t < n_t; ++t) {
        const int gt = g0 + t;
        const int col0 = (2 * t + wg) * 64;
        const uint32_t tdp = tlane + TM_DP + (uint32_t)(gt & 1) * 128u + (uint32_t)wg * 64u;
        if (!wait_warp(bar(B_SF), (uint32_t)gt & 1u)) { ok = false; break; }
        tc5::fence_after_sync();
        const bool need_mask = (p.causal && col0 + 63 > q0) || (col0 + 64 > p.seqlen);
        uint32_t rs[2][32], rd[2][32];
        tc5::tmem_ld32(tlane + TM_S + (uint32_t)wg * 64u, rs[0]);
        tc5::tmem_ld32(tlane + TM_S + (uint32_t)wg * 64u + 32u, rs[1]);
        tc5::tmem_ld_wait();
        tc5::fence_before_sync();
        __syncwarp();
        if (lane == 0) tc5::mbar_arrive(bar(B_SE));    // the score tile may take the next tile
        if (!wait_warp(bar(B_DF + (gt & 1)), (uint32_t)(gt >> 1) & 1u)) { ok = false; break; }
        tc5::fence_after_sync();
        tc5::tmem_ld32(tdp, rd[0]);
        tc5::tmem_ld32(tdp + 32u, rd[1]);
        tc5::tmem_ld_wait();
        uint32_t pk[32];
#pragma unroll
        for (int g = 0; g < 8; ++g) {    // keys 8g .. 8g+7 of this half -> packed columns 4g .. 4g+3
          float ds[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int c = g * 8 + i;
            float e = ex2(fmaf(__uint_as_float(rs[c >> 5][c & 31]), sl, -lse2));
            if (need_mask && col0 + c > lim) e = 0.0f;
            ds[i] = e * (__uint_as_float(rd[c >> 5][c & 31]) - dlt);
          }
          pk[4 * g] = pack_bf16(ds[0], ds[1]);
          pk[4 * g + 1] = pack_bf16(ds[2], ds[3]);
          pk[4 * g + 2] = pack_bf16(ds[4], ds[5]);
          pk[4 * g + 3] = pack_bf16(ds[6], ds[7]);
        }
        tc5::tmem_st32(tdp, pk);
        tc5::tmem_st_wait();
        tc5::fence_before_sync();
        __syncwarp();
        if (lane == 0) tc5::mbar_arrive(bar(B_PF + (gt & 1)));
      }
      if (!ok || !wait_warp(bar(B_ACC), (uint32_t)it & 1u)) { ok = false; break; }
      tc5::fence_after_sync();
      __nv_bfloat16* dq = p.dq + (int64_t)b * p.dq_sb + (int64_t)grow * p.dq_ss + (int64_t)h * p.dq_sh;
      // each group stores one half of the row
      uint32_t r0[32], r1[32];
      float v[32];
      tc5::tmem_ld32(tlane + TM_DQ + (uint32_t)wg * 64u, r0);
      tc5::tmem_ld32(tlane + TM_DQ + (uint32_t)wg * 64u + 32u, r1);
      tc5::tmem_ld_wait();
      tc5::fence_before_sync();
      __syncwarp();
      if (lane == 0) tc5::mbar_arrive(bar(B3_OE));    // the accumulator may take the next item
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r0[i]) * p.scale;
      if (in) st_row32(dq + wg * 64, v);
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r1[i]) * p.scale;
      if (in) st_row32(dq + wg * 64 + 32, v);
      g0 += n_t;
      ++it;
    }
  }

  __syncwarp();
  if (*abort_flag) __nanosleep(200000);
  tc5::fence_before_sync();
  __syncthreads();
  tc5::fence_after_sync();
  if (warp == 1) tc5::tmem_dealloc(tmem_base, TM_COLS);
}

// ====================================================================== dK / dV, persistent CTAs over the work items
namespace dkv3 {
using namespace dkv2;
enum { B3_KVE = NBAR, B3_OE = NBAR + 1, NBAR3 = NBAR + 2 };
constexpr int SMEM3 = OFF_BAR + NBAR3 * 8 + 16 + 896;
static_assert(SMEM3 <= 227 * 1024, "persistent dK/dV kernel: shared memory");
}    // namespace dkv3

// attn_bwd_dkdv_tm_kernel with one CTA per SM walking the (key tile, batch * head) items; the Q / dO stages, the score
// tiles and all barriers keep running across items (one global query-tile counter).  B3_KVE: every S^T / dP^T product of
// an item is complete, K and V may be overwritten by the next item's; B3_OE: the softmax warps have read dV and dK, the
// first products of the next item may overwrite the accumulators.
__global__ void __launch_bounds__(kTcThreads, 1)
attn_bwd_dkdv_ps_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                        const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do, const TcParams p, int n_kt,
                        int n_items) {
  using namespace dkv3;
  extern __shared__ __align__(128) uint8_t smem_raw128[];
  const uint32_t raw_addr = tc5::smem_u32(smem_raw128);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* smem = smem_raw128 + (base - raw_addr);
  const uint32_t bars = base + OFF_BAR;
  auto bar = [&](int i) { return bars + 8u * (uint32_t)i; };
  float* s_lse = reinterpret_cast<float*>(smem + OFF_LSE);    // [NSQ][128] log2-scaled lse, then [NSQ][128] delta
  float* s_delta = s_lse + NSQ * 128;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(smem + OFF_BAR + NBAR3 * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
  auto wait_warp = [&](uint32_t br, uint32_t ph) {
    return __all_sync(0xffffffffu, tc5::mbar_wait(br, ph, abort_flag, p.status, kStatusBit)) != 0;
  };
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int nq_all = (p.seqlen + 127) / 128;
  const ItemOrder order{n_kt, p.batch * p.heads, max(1, (4 * (int)gridDim.x) / n_kt)};
  const int n_waves = (n_items + (int)gridDim.x - 1) / (int)gridDim.x;
  auto item_at = [&](int w) {
    const int c = (w & 1) ? (int)gridDim.x - 1 - (int)blockIdx.x : (int)blockIdx.x;
    return w * (int)gridDim.x + c;
  };

  if (threadIdx.x == 0) {
    tc5::mbar_init(bar(B_KV), 1);
    for (int s = 0; s < NSQ; ++s) {
      tc5::mbar_init(bar(B_QF + s), 2);    // TMA bytes + the lse/delta rows written by warp 0
      tc5::mbar_init(bar(B_QE + s), 9);    // last MMA that reads the stage + eight softmax warps
    }
    tc5::mbar_init(bar(B_SF), 1);
    tc5::mbar_init(bar(B_SE), 8);
    tc5::mbar_init(bar(B_DF), 1);
    tc5::mbar_init(bar(B_PF), 8);
    tc5::mbar_init(bar(B_PE), 1);
    tc5::mbar_init(bar(B_ACC), 1);
    tc5::mbar_init(bar(B3_KVE), 1);
    tc5::mbar_init(bar(B3_OE), 8);
    *abort_flag = 0;
    tc5::mbar_fence_init();
    tc5::tma_prefetch_desc(&map_q);
    tc5::tma_prefetch_desc(&map_k);
    tc5::tma_prefetch_desc(&map_v);
    tc5::tma_prefetch_desc(&map_do);
  }
  if (warp == 1) {
    tc5::tmem_alloc(tc5::smem_u32(tmem_holder), TM_COLS);
    tc5::tmem_relinquish();
  }
  tc5::fence_before_sync();
  __syncthreads();
  tc5::fence_after_sync();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    // ------------------------------------------------------------------ producer (whole warp: lane 0 issues TMA)
    int gq = 0, it = 0;
    bool ok = true;
    for (int w = 0; w < n_waves && ok; ++w) {
      const int item = item_at(w);
      if (item >= n_items) continue;
      int kt, bh;
      order.decode(item, kt, bh);
      const int b = bh / p.heads, h = bh - b * p.heads;
      const int k0 = kt * 128;
      const int t_first = p.causal ? kt : 0;
      const int n_q = nq_all - t_first;
      if (it > 0 && !__all_sync(0xffffffffu, tc5::mbar_wait(bar(B3_KVE), (uint32_t)(it - 1) & 1u, abort_flag, p.status, kStatusBit))) break;
      if (lane == 0) {
        tc5::mbar_arrive_expect_tx(bar(B_KV), 2 * TILE);
        tc5::tma_load_4d(base + OFF_K, &map_k, 0, h, k0, b, bar(B_KV));
        tc5::tma_load_4d(base + OFF_K + PANEL, &map_k, 64, h, k0, b, bar(B_KV));
        tc5::tma_load_4d(base + OFF_V, &map_v, 0, h, k0, b, bar(B_KV));
        tc5::tma_load_4d(base + OFF_V + PANEL, &map_v, 64, h, k0, b, bar(B_KV));
      }
      const float* glse = p.lse + (int64_t)bh * p.seqlen;
      const float* gdelta = p.delta + (int64_t)bh * p.seqlen;
      for (int t = 0; t < n_q; ++t, ++gq) {
        const int s = gq % NSQ;
        const int qrow0 = (t_first + t) * 128;
        if (!__all_sync(0xffffffffu, tc5::mbar_wait(bar(B_QE + s), ((uint32_t)(gq / NSQ) & 1u) ^ 1u, abort_flag, p.status, kStatusBit))) { ok = false; break; }
        if (lane == 0) {
          tc5::mbar_arrive_expect_tx(bar(B_QF + s), 2 * TILE);
          tc5::tma_load_4d(base + OFF_Q + s * TILE, &map_q, 0, h, qrow0, b, bar(B_QF + s));
          tc5::tma_load_4d(base + OFF_Q + s * TILE + PANEL, &map_q, 64, h, qrow0, b, bar(B_QF + s));
          tc5::tma_load_4d(base + OFF_DO + s * TILE, &map_do, 0, h, qrow0, b, bar(B_QF + s));
          tc5::tma_load_4d(base + OFF_DO + s * TILE + PANEL, &map_do, 64, h, qrow0, b, bar(B_QF + s));
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int r = lane + 32 * i;
          const bool in = qrow0 + r < p.seqlen;
          s_lse[s * 128 + r] = in ? glse[qrow0 + r] * kLog2e : INFINITY;    // +inf makes the probability exactly zero
          s_delta[s * 128 + r] = in ? gdelta[qrow0 + r] : 0.0f;
        }
        __syncwarp();
        if (lane == 0) tc5::mbar_arrive(bar(B_QF + s));
      }
      ++it;
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc_s = tc5::idesc_bf16(128, 128, 0, 0);
      const uint32_t idesc_acc = tc5::idesc_bf16(128, 128, 0, 1);
      auto issue_st = [&](int gq) -> bool {    // S^T = K Q^T for the gq-th query tile of this CTA
        const int st = gq % NSQ;
        if (!tc5::mbar_wait(bar(B_QF + st), (uint32_t)(gq / NSQ) & 1u, abort_flag, p.status, kStatusBit)) return false;    // data first
        if (gq > 0 && !tc5::mbar_wait(bar(B_SE), (uint32_t)(gq - 1) & 1u, abort_flag, p.status, kStatusBit)) return false;
        tc5::fence_after_sync();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t off = (uint32_t)(kk >> 2) * PANEL + (uint32_t)(kk & 3) * 32u;
          tc5::mma_f16(tmem_base + TM_ST, tc5::smem_desc_k_sw128(base + OFF_K + off), tc5::smem_desc_k_sw128(base + OFF_Q + st * TILE + off),
                       idesc_s, kk ? 1u : 0u);
        }
        tc5::mma_commit(bar(B_SF));
        return true;
      };
      auto issue_dpt = [&](int gq) {    // dP^T = V dO^T (the stage was waited for by issue_st(gq))
        const int st = gq % NSQ;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t off = (uint32_t)(kk >> 2) * PANEL + (uint32_t)(kk & 3) * 32u;
          tc5::mma_f16(tmem_base + TM_DPT, tc5::smem_desc_k_sw128(base + OFF_V + off), tc5::smem_desc_k_sw128(base + OFF_DO + st * TILE + off),
                       idesc_s, kk ? 1u : 0u);
        }
        tc5::mma_commit(bar(B_DF));
      };
      int g0 = 0, it = 0;
      bool ok = true;
      for (int w = 0; w < n_waves && ok; ++w) {
        const int item = item_at(w);
        if (item >= n_items) continue;
        int kt, bh;
        order.decode(item, kt, bh);
        const int n_q = nq_all - (p.causal ? kt : 0);
        if (!tc5::mbar_wait(bar(B_KV), (uint32_t)it & 1u, abort_flag, p.status, kStatusBit)) { ok = false; break; }
        if (!issue_st(g0)) { ok = false; break; }
        issue_dpt(g0);
        if (n_q == 1) tc5::mma_commit(bar(B3_KVE));
        if (it > 0 && !tc5::mbar_wait(bar(B3_OE), (uint32_t)(it - 1) & 1u, abort_flag, p.status, kStatusBit)) { ok = false; break; }
        for (int t = 0; t < n_q; ++t) {
          const int gq = g0 + t;
          const int st = gq % NSQ;
          bool pending = t + 1 < n_q;
          if (pending && tc5::mbar_test(bar(B_SE), (uint32_t)gq & 1u) &&
              tc5::mbar_test(bar(B_QF + (gq + 1) % NSQ), (uint32_t)((gq + 1) / NSQ) & 1u)) {
            if (!issue_st(gq + 1)) { ok = false; break; }
            pending = false;
          }
          if (!tc5::mbar_wait(bar(B_PF), (uint32_t)gq & 1u, abort_flag, p.status, kStatusBit)) { ok = false; break; }
          tc5::fence_after_sync();
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            tc5::mma_f16(tmem_base + TM_DV, tc5::smem_desc_k_sw128(base + OFF_PT + (uint32_t)(kk >> 2) * PANEL + (uint32_t)(kk & 3) * 32u),
                         tc5::smem_desc_mn_sw128(base + OFF_DO + st * TILE + (uint32_t)kk * 2048u, PANEL), idesc_acc, (t | kk) ? 1u : 0u);
          }
          tc5::mma_commit(bar(B_PE));
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            tc5::mma_f16_ta(tmem_base + TM_DK, tmem_base + TM_DPT + (uint32_t)(kk >> 2) * 64u + (uint32_t)(kk & 3) * 8u,
                            tc5::smem_desc_mn_sw128(base + OFF_Q + st * TILE + (uint32_t)kk * 2048u, PANEL), idesc_acc, (t | kk) ? 1u : 0u);
          }
          tc5::mma_commit(bar(B_QE + st));
          if (pending && !issue_st(gq + 1)) { ok = false; break; }
          if (t + 1 < n_q) {
            issue_dpt(gq + 1);
            if (t + 2 == n_q) tc5::mma_commit(bar(B3_KVE));    // every S^T / dP^T product of this item is issued
          }
        }
        if (!ok) break;
        tc5::mma_commit(bar(B_ACC));
        g0 += n_q;
        ++it;
      }
    }
  } else {
    // ------------------------------------------------------------------ one thread per key row and query half
    const int qd = warp & 3;
    const int wg = (warp - 2) >> 2;    // group g: queries 64 g .. 64 g + 63 of every tile
    const int row = qd * 32 + lane;
    const uint32_t tlane = tmem_base + ((uint32_t)(qd * 32) << 16);
    const float sl = p.scale * kLog2e;
    const uint32_t prow = base + OFF_PT + (uint32_t)wg * PANEL + (uint32_t)row * 128u;
    const uint32_t swz = (uint32_t)(row & 7);
    int g0 = 0, it = 0;
    bool ok = true;
    for (int w = 0; w < n_waves && ok; ++w) {
      const int item = item_at(w);
      if (item >= n_items) continue;
      int kt, bh;
      order.decode(item, kt, bh);
      const int b = bh / p.heads, h = bh - b * p.heads;
      const int k0 = kt * 128;
      const int grow = k0 + row;
      const int t_first = p.causal ? kt : 0;
      const int n_q = nq_all - t_first;
      for (int t = 0; t < n_q; ++t) {
        const int gq = g0 + t;
        const int st = gq % NSQ;
        const int qrow0 = (t_first + t) * 128 + wg * 64;    // first query of this group's half
        if (!wait_warp(bar(B_QF + st), (uint32_t)(gq / NSQ) & 1u)) { ok = false; break; }
        if (!wait_warp(bar(B_SF), (uint32_t)gq & 1u)) { ok = false; break; }
        tc5::fence_after_sync();
        const bool need_mask = p.causal && (qrow0 < k0 + 128);
        const float4* lse2 = reinterpret_cast<const float4*>(s_lse + st * 128 + wg * 64);
        const float4* dlt = reinterpret_cast<const float4*>(s_delta + st * 128 + wg * 64);
        uint32_t rs[2][32], rd[2][32];
        tc5::tmem_ld32(tlane + TM_ST + (uint32_t)wg * 64u, rs[0]);
        tc5::tmem_ld32(tlane + TM_ST + (uint32_t)wg * 64u + 32u, rs[1]);
        tc5::tmem_ld_wait();
        tc5::fence_before_sync();
        __syncwarp();
        if (lane == 0) tc5::mbar_arrive(bar(B_SE));    // the score tile may take the next tile
        if (!wait_warp(bar(B_DF), (uint32_t)gq & 1u)) { ok = false; break; }
        tc5::fence_after_sync();
        tc5::tmem_ld32(tlane + TM_DPT + (uint32_t)wg * 64u, rd[0]);
        tc5::tmem_ld32(tlane + TM_DPT + (uint32_t)wg * 64u + 32u, rd[1]);
        tc5::tmem_ld_wait();
        if (gq > 0 && !wait_warp(bar(B_PE), (uint32_t)(gq - 1) & 1u)) { ok = false; break; }    // dV of the previous tile has read P^T
        uint32_t pk[32];
#pragma unroll
        for (int g = 0; g < 8; ++g) {    // 16-byte chunk g = queries 8g .. 8g+7 of this half
          float e[8], ds[8];
#pragma unroll
          for (int hh = 0; hh < 2; ++hh) {
            const float4 l4 = lse2[g * 2 + hh];
            const float4 d4 = dlt[g * 2 + hh];
            const float la[4] = {l4.x, l4.y, l4.z, l4.w};
            const float da[4] = {d4.x, d4.y, d4.z, d4.w};
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const int i = hh * 4 + u;
              const int ql = g * 8 + i;
              float ev = ex2(fmaf(__uint_as_float(rs[ql >> 5][ql & 31]), sl, -la[u]));
              if (need_mask && qrow0 + ql < grow) ev = 0.0f;
              e[i] = ev;
              ds[i] = ev * (__uint_as_float(rd[ql >> 5][ql & 31]) - da[u]);
            }
          }
          st_shared_v4(prow + ((((uint32_t)g) ^ swz) << 4), pack_bf16(e[0], e[1]), pack_bf16(e[2], e[3]), pack_bf16(e[4], e[5]),
                       pack_bf16(e[6], e[7]));
          pk[4 * g] = pack_bf16(ds[0], ds[1]);
          pk[4 * g + 1] = pack_bf16(ds[2], ds[3]);
          pk[4 * g + 2] = pack_bf16(ds[4], ds[5]);
          pk[4 * g + 3] = pack_bf16(ds[6], ds[7]);
        }
        tc5::tmem_st32(tlane + TM_DPT + (uint32_t)wg * 64u, pk);
        tc5::tmem_st_wait();
        tc5::fence_before_sync();
        fence_async_smem();
        __syncwarp();
        if (lane == 0) {
          tc5::mbar_arrive(bar(B_PF));
          tc5::mbar_arrive(bar(B_QE + st));
        }
      }
      if (!ok || !wait_warp(bar(B_ACC), (uint32_t)it & 1u)) { ok = false; break; }
      tc5::fence_after_sync();
      // group 0 stores dV, group 1 stores dK: read the whole accumulator first, so that it is free for the next item
      __nv_bfloat16* dst = wg == 0 ? p.dv + (int64_t)b * p.dv_sb + (int64_t)grow * p.dv_ss + (int64_t)h * p.dv_sh
                                   : p.dk + (int64_t)b * p.dk_sb + (int64_t)grow * p.dk_ss + (int64_t)h * p.dk_sh;
      const float f = wg == 0 ? 1.0f : p.scale;
      const uint32_t tsrc = tlane + (wg == 0 ? TM_DV : TM_DK);
      uint32_t acc[4][32];
#pragma unroll
      for (int c = 0; c < 4; ++c) tc5::tmem_ld32(tsrc + (uint32_t)c * 32u, acc[c]);
      tc5::tmem_ld_wait();
      tc5::fence_before_sync();
      __syncwarp();
      if (lane == 0) tc5::mbar_arrive(bar(B3_OE));
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        float v[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(acc[c][i]) * f;
        if (grow < p.seqlen) st_row32(dst + c * 32, v);
      }
      g0 += n_q;
      ++it;
    }
  }

  __syncwarp();
  if (*abort_flag) __nanosleep(200000);
  tc5::fence_before_sync();
  __syncthreads();
  tc5::fence_after_sync();
  if (warp == 1) tc5::tmem_dealloc(tmem_base, TM_COLS);
}

// ---- host side -----------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
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

struct Map4Key {
  const void* ptr;
  int64_t sb, ss, sh;
  int batch, heads, seqlen, box_rows;
  bool operator==(const Map4Key& o) const {
    return ptr == o.ptr && sb == o.sb && ss == o.ss && sh == o.sh && batch == o.batch && heads == o.heads && seqlen == o.seqlen &&
           box_rows == o.box_rows;
  }
};
struct Map4Hash {
  size_t operator()(const Map4Key& k) const {
    size_t hsh = reinterpret_cast<size_t>(k.ptr);
    auto mix = [&](size_t v) { hsh ^= v * 0x9e3779b97f4a7c15ull + (hsh << 6) + (hsh >> 2); };
    mix((size_t)k.sb); mix((size_t)k.ss); mix((size_t)k.sh); mix((size_t)k.batch); mix((size_t)k.heads); mix((size_t)k.seqlen);
    mix((size_t)k.box_rows);
    return hsh;
  }
};

// Tensor map over a bf16 [batch, seq, head, 128] view given by element strides; the box is
// [box_rows sequence positions][64 elements] of one head (one 128-byte-swizzled panel).
int make_map4(const void* ptr, int batch, int heads, int seqlen, int64_t sb, int64_t ss, int64_t sh, int box_rows, CUtensorMap* out) {
  static std::unordered_map<Map4Key, CUtensorMap, Map4Hash> cache;
  static std::mutex mu;
  Map4Key key{ptr, sb, ss, sh, batch, heads, seqlen, box_rows};
  {
    std::lock_guard<std::mutex> lk(mu);
    auto it = cache.find(key);
    if (it != cache.end()) {
      *out = it->second;
      return MSAMP_OK;
    }
  }
  EncodeTiledFn fn = encode_fn();
  if (!fn) {
    msamp_set_error("cuTensorMapEncodeTiled is not available from the driver");
    return MSAMP_ETMAP;
  }
  // A dimension of extent 1 still needs a valid (16-byte multiple) stride.
  cuuint64_t dims[4] = {128, (cuuint64_t)heads, (cuuint64_t)seqlen, (cuuint64_t)batch};
  cuuint64_t strides[3] = {(cuuint64_t)sh * 2, (cuuint64_t)ss * 2, (cuuint64_t)sb * 2};
  for (int i = 0; i < 3; ++i)
    if (strides[i] == 0) strides[i] = 256;
  cuuint32_t box[4] = {64, 1, (cuuint32_t)box_rows, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    msamp_set_error("cuTensorMapEncodeTiled (attention) failed with %d (ptr=%p b=%d h=%d s=%d strides=%lld,%lld,%lld)", (int)r, ptr,
                    batch, heads, seqlen, (long long)sb, (long long)ss, (long long)sh);
    return MSAMP_ETMAP;
  }
  std::lock_guard<std::mutex> lk(mu);
  if (cache.size() > 4096) cache.clear();
  cache[key] = *out;
  return MSAMP_OK;
}

template <typename K>
int set_smem(K kernel, int bytes) {
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e != cudaSuccess) {
    msamp_set_error("cudaFuncSetAttribute(%d bytes): %s", bytes, cudaGetErrorString(e));
    return MSAMP_ELAUNCH;
  }
  return MSAMP_OK;
}

}    // namespace

// Same contract as msamp_attention_fwd (attention.cu) for head_dim 128: strides are the (batch, seq, head)
// element strides of q, k, v, o; every pointer 16-byte aligned, every stride a multiple of 8 elements.
MSAMP_API int msamp_attention_tc_fwd(const void* q, const void* k, const void* v, void* o, float* lse, const int64_t* strides, int batch,
                                     int heads, int seqlen, int head_dim, float scale, int causal, void* stream_) {
  MSAMP_REQUIRE(head_dim == 128, "attention (tcgen05): head_dim must be 128 (got %d)", head_dim);
  MSAMP_REQUIRE(batch > 0 && heads > 0 && seqlen > 0, "attention: empty problem");
  for (int i = 0; i < 12; ++i) MSAMP_REQUIRE(strides[i] % 8 == 0, "attention: stride %d is not a multiple of 8 elements", i);
  CUtensorMap mq, mk, mv;
  int rc;
  if ((rc = make_map4(q, batch, heads, seqlen, strides[0], strides[1], strides[2], 128, &mq))) return rc;
  if ((rc = make_map4(k, batch, heads, seqlen, strides[3], strides[4], strides[5], 64, &mk))) return rc;
  if ((rc = make_map4(v, batch, heads, seqlen, strides[6], strides[7], strides[8], 64, &mv))) return rc;
  TcParams p = {};
  p.o = (__nv_bfloat16*)o; p.lse = lse;
  p.o_sb = strides[9]; p.o_ss = strides[10]; p.o_sh = strides[11];
  p.batch = batch; p.heads = heads; p.seqlen = seqlen; p.causal = causal; p.scale = scale;
  p.status = msamp_device_status_ptr();
  dim3 grid((seqlen + 127) / 128, batch * heads);
  // MSAMP_ATTN_FWD_SMEM=1 selects the kernel with 64-key score tiles and P in shared memory (default: 128-key score
  // tiles, P in tensor memory).
  static const bool smem_operands = [] { const char* e = getenv("MSAMP_ATTN_FWD_SMEM"); return e && e[0] == '1'; }();
  if (smem_operands) {
    if ((rc = set_smem(attn_fwd_tc_kernel, fwd::SMEM))) return rc;
    attn_fwd_tc_kernel<<<grid, kTcThreads, fwd::SMEM, (cudaStream_t)stream_>>>(mq, mk, mv, p);
    return msamp_check_launch("attn_fwd_tc_kernel");
  }
  CUtensorMap mk128;
  if ((rc = make_map4(k, batch, heads, seqlen, strides[3], strides[4], strides[5], 128, &mk128))) return rc;
  // MSAMP_ATTN_FWD_PERSIST=0 launches one CTA per (query tile, batch, head) instead of persistent CTAs
  static const bool persistent = [] { const char* e = getenv("MSAMP_ATTN_FWD_PERSIST"); return !(e && e[0] == '0'); }();
  if (!persistent) {
    if ((rc = set_smem(attn_fwd_tm_kernel, fwd2::SMEM))) return rc;
    attn_fwd_tm_kernel<<<grid, kTcThreads, fwd2::SMEM, (cudaStream_t)stream_>>>(mq, mk128, mv, p);
    return msamp_check_launch("attn_fwd_tm_kernel");
  }
  const int n_qt = (seqlen + 127) / 128;
  const int n_items = n_qt * batch * heads;
  const int ctas = n_items < msamp_sm_count() ? n_items : msamp_sm_count();
  if ((rc = set_smem(attn_fwd_ps_kernel, fwd3::SMEM3))) return rc;
  attn_fwd_ps_kernel<<<ctas, kTcThreads, fwd3::SMEM3, (cudaStream_t)stream_>>>(mq, mk128, mv, p, n_qt, n_items);
  return msamp_check_launch("attn_fwd_ps_kernel");
}

// Same contract as msamp_attention_bwd (attention.cu) for head_dim 128.
MSAMP_API int msamp_attention_tc_bwd(const void* q, const void* k, const void* v, const void* o, const float* lse, const void* d_o,
                                     void* dq, void* dk, void* dv, float* delta, const int64_t* strides, int batch, int heads,
                                     int seqlen, int head_dim, float scale, int causal, void* stream_) {
  MSAMP_REQUIRE(head_dim == 128, "attention (tcgen05): head_dim must be 128 (got %d)", head_dim);
  MSAMP_REQUIRE(batch > 0 && heads > 0 && seqlen > 0, "attention: empty problem");
  for (int i = 0; i < 24; ++i) MSAMP_REQUIRE(strides[i] % 8 == 0, "attention: stride %d is not a multiple of 8 elements", i);
  cudaStream_t stream = (cudaStream_t)stream_;
  {
    DeltaParams d = {};
    d.o = (const __nv_bfloat16*)o; d.d_o = (const __nv_bfloat16*)d_o; d.delta = delta;
    d.o_sb = strides[9]; d.o_ss = strides[10]; d.o_sh = strides[11];
    d.do_sb = strides[12]; d.do_ss = strides[13]; d.do_sh = strides[14];
    d.batch = batch; d.heads = heads; d.seqlen = seqlen;
    const int64_t warps = (int64_t)batch * heads * seqlen;
    attn_delta_tc_kernel<<<(unsigned)((warps * 32 + 255) / 256), 256, 0, stream>>>(d);
  }
  TcParams p = {};
  p.lse = const_cast<float*>(lse); p.delta = delta;
  p.dq = (__nv_bfloat16*)dq; p.dk = (__nv_bfloat16*)dk; p.dv = (__nv_bfloat16*)dv;
  p.dq_sb = strides[15]; p.dq_ss = strides[16]; p.dq_sh = strides[17];
  p.dk_sb = strides[18]; p.dk_ss = strides[19]; p.dk_sh = strides[20];
  p.dv_sb = strides[21]; p.dv_ss = strides[22]; p.dv_sh = strides[23];
  p.batch = batch; p.heads = heads; p.seqlen = seqlen; p.causal = causal; p.scale = scale;
  p.status = msamp_device_status_ptr();
  int rc;
  {
    CUtensorMap mq, mk, mv, mdo;
    if ((rc = make_map4(q, batch, heads, seqlen, strides[0], strides[1], strides[2], 64, &mq))) return rc;
    if ((rc = make_map4(k, batch, heads, seqlen, strides[3], strides[4], strides[5], 128, &mk))) return rc;
    if ((rc = make_map4(v, batch, heads, seqlen, strides[6], strides[7], strides[8], 128, &mv))) return rc;
    if ((rc = make_map4(d_o, batch, heads, seqlen, strides[12], strides[13], strides[14], 64, &mdo))) return rc;
    dim3 grid((seqlen + 127) / 128, batch * heads);
    static const bool smem_operands = [] { const char* e = getenv("MSAMP_ATTN_BWD_SMEM"); return e && e[0] == '1'; }();
    if (smem_operands) {
      if ((rc = set_smem(attn_bwd_dkdv_tc_kernel, dkv::SMEM))) return rc;
      attn_bwd_dkdv_tc_kernel<<<grid, kTcThreads, dkv::SMEM, stream>>>(mq, mk, mv, mdo, p);
    } else {
      CUtensorMap mq128, mdo128;
      if ((rc = make_map4(q, batch, heads, seqlen, strides[0], strides[1], strides[2], 128, &mq128))) return rc;
      if ((rc = make_map4(d_o, batch, heads, seqlen, strides[12], strides[13], strides[14], 128, &mdo128))) return rc;
      static const bool persistent = [] { const char* e = getenv("MSAMP_ATTN_BWD_PERSIST"); return !(e && e[0] == '0'); }();
      if (persistent) {
        const int n_kt = (seqlen + 127) / 128;
        const int n_items = n_kt * batch * heads;
        const int ctas = n_items < msamp_sm_count() ? n_items : msamp_sm_count();
        if ((rc = set_smem(attn_bwd_dkdv_ps_kernel, dkv3::SMEM3))) return rc;
        attn_bwd_dkdv_ps_kernel<<<ctas, kTcThreads, dkv3::SMEM3, stream>>>(mq128, mk, mv, mdo128, p, n_kt, n_items);
      } else {
        if ((rc = set_smem(attn_bwd_dkdv_tm_kernel, dkv2::SMEM))) return rc;
        attn_bwd_dkdv_tm_kernel<<<grid, kTcThreads, dkv2::SMEM, stream>>>(mq128, mk, mv, mdo128, p);
      }
    }
  }
  {
    CUtensorMap mq, mk, mv, mdo;
    if ((rc = make_map4(q, batch, heads, seqlen, strides[0], strides[1], strides[2], 128, &mq))) return rc;
    if ((rc = make_map4(k, batch, heads, seqlen, strides[3], strides[4], strides[5], 64, &mk))) return rc;
    if ((rc = make_map4(v, batch, heads, seqlen, strides[6], strides[7], strides[8], 64, &mv))) return rc;
    if ((rc = make_map4(d_o, batch, heads, seqlen, strides[12], strides[13], strides[14], 128, &mdo))) return rc;
    dim3 grid((seqlen + 127) / 128, batch * heads);
    // MSAMP_ATTN_BWD_SMEM=1 selects the kernels with 64-wide score tiles and the second operand in shared memory
    static const bool smem_operands = [] { const char* e = getenv("MSAMP_ATTN_BWD_SMEM"); return e && e[0] == '1'; }();
    if (smem_operands) {
      if ((rc = set_smem(attn_bwd_dq_tc_kernel, dqk::SMEM))) return rc;
      attn_bwd_dq_tc_kernel<<<grid, kTcThreads, dqk::SMEM, stream>>>(mq, mk, mv, mdo, p);
    } else {
      CUtensorMap mk128, mv128;
      if ((rc = make_map4(k, batch, heads, seqlen, strides[3], strides[4], strides[5], 128, &mk128))) return rc;
      if ((rc = make_map4(v, batch, heads, seqlen, strides[6], strides[7], strides[8], 128, &mv128))) return rc;
      // MSAMP_ATTN_BWD_PERSIST=0: one CTA per (tile, batch, head) instead of persistent CTAs over the work items
      static const bool persistent = [] { const char* e = getenv("MSAMP_ATTN_BWD_PERSIST"); return !(e && e[0] == '0'); }();
      if (persistent) {
        const int n_qt = (seqlen + 127) / 128;
        const int n_items = n_qt * batch * heads;
        const int ctas = n_items < msamp_sm_count() ? n_items : msamp_sm_count();
        if ((rc = set_smem(attn_bwd_dq_ps_kernel, dqk3::SMEM3))) return rc;
        attn_bwd_dq_ps_kernel<<<ctas, kTcThreads, dqk3::SMEM3, stream>>>(mq, mk128, mv128, mdo, p, n_qt, n_items);
      } else {
        if ((rc = set_smem(attn_bwd_dq_tm_kernel, dqk2::SMEM))) return rc;
        attn_bwd_dq_tm_kernel<<<grid, kTcThreads, dqk2::SMEM, stream>>>(mq, mk128, mv128, mdo, p);
      }
    }
  }
  return msamp_check_launch("attn_bwd_tc kernels");
}
