// Causal (or full) softmax attention, forward and backward, for bf16 with head size 64 or 128.
//
// Flash-style tiling: a CTA of four warps owns 64 query rows (forward and dQ) or 64 key rows
// (dK/dV); the other operand streams through shared memory in 64- or 32-row tiles with cp.async
// double buffering; scores never touch global memory.  Tiles are stored with a 16-byte-chunk XOR
// swizzle so that ldmatrix is bank-conflict free.  q, k, v, o and their gradients are addressed
// through (batch, sequence, head) strides, so the fused [tokens, 3*hidden] output of a QKV
// projection is consumed, and its gradient produced, in place without any reshuffling copy.
//
// The backward pass is two kernels (dK/dV looping over query tiles, dQ looping over key tiles): it
// recomputes the scores twice but needs no atomics and is deterministic.
#include "common.cuh"

namespace {

constexpr int kAttnThreads = 128;
constexpr float kLog2e = 1.4426950408889634f;

struct AttnParams {
  const __nv_bfloat16* q;
  const __nv_bfloat16* k;
  const __nv_bfloat16* v;
  __nv_bfloat16* o;
  float* lse;    // [b, h, s]
  // backward only
  const __nv_bfloat16* d_o;
  const float* delta;    // [b, h, s] rowsum(dO * O)
  __nv_bfloat16* dq;
  __nv_bfloat16* dk;
  __nv_bfloat16* dv;
  int64_t q_sb, q_ss, q_sh;    // strides in elements: batch, sequence, head
  int64_t k_sb, k_ss, k_sh;
  int64_t v_sb, v_ss, v_sh;
  int64_t o_sb, o_ss, o_sh;
  int64_t do_sb, do_ss, do_sh;
  int64_t dq_sb, dq_ss, dq_sh;
  int64_t dk_sb, dk_ss, dk_sh;
  int64_t dv_sb, dv_ss, dv_sh;
  int batch, heads, seqlen;
  float scale;
  int causal;
};

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  int sz = valid ? 16 : 0;    // src-size 0 => the 16 bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// A tile of ROWS x D bf16 in shared memory; 16-byte chunk c of row r lives at chunk (c ^ (r & 7)).
template <int D>
struct Tile {
  static constexpr int CHUNKS = D / 8;    // 16-byte chunks per row
  static constexpr int ROW_BYTES = D * 2;
  __device__ static __forceinline__ uint32_t offset(int row, int chunk) { return row * ROW_BYTES + ((chunk ^ (row & 7)) << 4); }
};

// Copy `rows` rows (row index r0.. in the sequence, bounded by seqlen) into a swizzled tile.
template <int D, int ROWS>
__device__ __forceinline__ void load_tile(uint32_t smem_base, const __nv_bfloat16* g, int64_t row_stride, int r0, int seqlen) {
  constexpr int CH = Tile<D>::CHUNKS;
  constexpr int TOTAL = ROWS * CH;
  for (int i = threadIdx.x; i < TOTAL; i += kAttnThreads) {
    int r = i / CH, c = i % CH;
    bool ok = (r0 + r) < seqlen;
    const __nv_bfloat16* src = g + (int64_t)(ok ? (r0 + r) : 0) * row_stride + c * 8;
    cp_async16(smem_base + Tile<D>::offset(r, c), src, ok);
  }
}

// ldmatrix address helpers (lane-dependent part)
// A operand, 16x16 block at (row0, k0): row = row0 + (l%8) + 8*((l/8)%2), chunk = k0/8 + l/16
template <int D>
__device__ __forceinline__ uint32_t addr_a(uint32_t base, int row0, int k0, int lane) {
  int row = row0 + (lane & 7) + ((lane >> 3) & 1) * 8;
  int chunk = (k0 >> 3) + (lane >> 4);
  return base + Tile<D>::offset(row, chunk);
}
// B operand from memory [n][k] (non-transposed ldmatrix), two n-tiles (n0..n0+15) x 16 k:
// row(n) = n0 + (l%8) + 8*(l/16), chunk = k0/8 + (l/8)%2  -> regs: (b0,b1) of tile n0, (b0,b1) of tile n0+8
template <int D>
__device__ __forceinline__ uint32_t addr_b(uint32_t base, int n0, int k0, int lane) {
  int row = n0 + (lane & 7) + (lane >> 4) * 8;
  int chunk = (k0 >> 3) + ((lane >> 3) & 1);
  return base + Tile<D>::offset(row, chunk);
}
// B operand from memory [k][n] (transposed ldmatrix), 16 k x two n-tiles (n0..n0+15):
// row(k) = k0 + (l%8) + 8*((l/8)%2), chunk = n0/8 + l/16 -> regs: (b0,b1) of tile n0, (b0,b1) of tile n0+8
template <int D>
__device__ __forceinline__ uint32_t addr_bt(uint32_t base, int k0, int n0, int lane) {
  int row = k0 + (lane & 7) + ((lane >> 3) & 1) * 8;
  int chunk = (n0 >> 3) + (lane >> 4);
  return base + Tile<D>::offset(row, chunk);
}

// ===================================================================================== forward
template <int D>
__global__ void __launch_bounds__(kAttnThreads) attn_fwd_kernel(const AttnParams p) {
  constexpr int BR = 64, BC = 64;
  constexpr int TILE_BYTES = BC * D * 2;
  extern __shared__ __align__(128) uint8_t smem[];
  const uint32_t sQ = smem_addr(smem);
  const uint32_t sK = sQ + BR * D * 2;              // 2 buffers
  const uint32_t sV = sK + 2 * TILE_BYTES;          // 2 buffers

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  // heavy (late) query tiles first for better causal load balance
  const int qblk = gridDim.x - 1 - blockIdx.x;
  const int bh = blockIdx.y;
  const int b = bh / p.heads, h = bh % p.heads;
  const int q0 = qblk * BR;

  const __nv_bfloat16* gq = p.q + b * p.q_sb + h * p.q_sh;
  const __nv_bfloat16* gk = p.k + b * p.k_sb + h * p.k_sh;
  const __nv_bfloat16* gv = p.v + b * p.v_sb + h * p.v_sh;

  int n_kv = (p.seqlen + BC - 1) / BC;
  if (p.causal) {
    int lim = (q0 + BR + BC - 1) / BC;
    n_kv = lim < n_kv ? lim : n_kv;
  }

  load_tile<D, BR>(sQ, gq, p.q_ss, q0, p.seqlen);
  load_tile<D, BC>(sK, gk, p.k_ss, 0, p.seqlen);
  load_tile<D, BC>(sV, gv, p.v_ss, 0, p.seqlen);
  cp_async_commit();

  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.0f, l1 = 0.0f;
  const float sl2 = p.scale * kLog2e;
  const int row_a = q0 + warp * 16 + g;    // this thread's two rows: row_a, row_a + 8

  for (int j = 0; j < n_kv; ++j) {
    const int buf = j & 1;
    if (j + 1 < n_kv) {
      load_tile<D, BC>(sK + (buf ^ 1) * TILE_BYTES, gk, p.k_ss, (j + 1) * BC, p.seqlen);
      load_tile<D, BC>(sV + (buf ^ 1) * TILE_BYTES, gv, p.v_ss, (j + 1) * BC, p.seqlen);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const uint32_t kb = sK + buf * TILE_BYTES, vb = sV + buf * TILE_BYTES;

    float s[BC / 8][4];
#pragma unroll
    for (int i = 0; i < BC / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.0f;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
      uint32_t a0, a1, a2, a3;
      ldmatrix_x4(addr_a<D>(sQ, warp * 16, kk * 16, lane), a0, a1, a2, a3);
#pragma unroll
      for (int nt = 0; nt < BC / 16; ++nt) {
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4(addr_b<D>(kb, nt * 16, kk * 16, lane), b0, b1, b2, b3);
        mma_bf16(s[2 * nt], a0, a1, a2, a3, b0, b1);
        mma_bf16(s[2 * nt + 1], a0, a1, a2, a3, b2, b3);
      }
    }
    // mask
    const int c0 = j * BC;
    const bool need_mask = (p.causal && (c0 + BC - 1 > q0 + warp * 16)) || (c0 + BC > p.seqlen);
    if (need_mask) {
#pragma unroll
      for (int i = 0; i < BC / 8; ++i) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          int col = c0 + i * 8 + 2 * t + (e & 1);
          int row = row_a + ((e >> 1) ? 8 : 0);
          if (col >= p.seqlen || (p.causal && col > row)) s[i][e] = -INFINITY;
        }
      }
    }
    // online softmax
    float mx0 = m0, mx1 = m1;
#pragma unroll
    for (int i = 0; i < BC / 8; ++i) {
      mx0 = fmaxf(mx0, fmaxf(s[i][0], s[i][1]));
      mx1 = fmaxf(mx1, fmaxf(s[i][2], s[i][3]));
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float ms0 = (mx0 == -INFINITY) ? 0.0f : mx0 * sl2;
    const float ms1 = (mx1 == -INFINITY) ? 0.0f : mx1 * sl2;
    const float corr0 = exp2f((m0 == -INFINITY ? -INFINITY : m0 * sl2) - ms0);
    const float corr1 = exp2f((m1 == -INFINITY ? -INFINITY : m1 * sl2) - ms1);
    m0 = mx0;
    m1 = mx1;
    float rs0 = 0.0f, rs1 = 0.0f;
#pragma unroll
    for (int i = 0; i < BC / 8; ++i) {
      s[i][0] = exp2f(s[i][0] * sl2 - ms0);
      s[i][1] = exp2f(s[i][1] * sl2 - ms0);
      s[i][2] = exp2f(s[i][2] * sl2 - ms1);
      s[i][3] = exp2f(s[i][3] * sl2 - ms1);
      rs0 += s[i][0] + s[i][1];
      rs1 += s[i][2] + s[i][3];
    }
    l0 = l0 * corr0 + rs0;
    l1 = l1 * corr1 + rs1;
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      o[i][0] *= corr0; o[i][1] *= corr0; o[i][2] *= corr1; o[i][3] *= corr1;
    }
    // O += P V
#pragma unroll
    for (int kk = 0; kk < BC / 16; ++kk) {
      uint32_t a0 = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
      uint32_t a1 = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
      uint32_t a2 = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      uint32_t a3 = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int nt = 0; nt < D / 16; ++nt) {
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4_trans(addr_bt<D>(vb, kk * 16, nt * 16, lane), b0, b1, b2, b3);
        mma_bf16(o[2 * nt], a0, a1, a2, a3, b0, b1);
        mma_bf16(o[2 * nt + 1], a0, a1, a2, a3, b2, b3);
      }
    }
    __syncthreads();    // everyone is done with this buffer before it is refilled
  }

  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  const float inv0 = l0 > 0.0f ? 1.0f / l0 : 0.0f;
  const float inv1 = l1 > 0.0f ? 1.0f / l1 : 0.0f;
  __nv_bfloat16* go = p.o + b * p.o_sb + h * p.o_sh;
#pragma unroll
  for (int i = 0; i < D / 8; ++i) {
    int col = i * 8 + 2 * t;
    if (row_a < p.seqlen) *reinterpret_cast<uint32_t*>(go + (int64_t)row_a * p.o_ss + col) = pack_bf16(o[i][0] * inv0, o[i][1] * inv0);
    if (row_a + 8 < p.seqlen)
      *reinterpret_cast<uint32_t*>(go + (int64_t)(row_a + 8) * p.o_ss + col) = pack_bf16(o[i][2] * inv1, o[i][3] * inv1);
  }
  if (t == 0) {
    float* lse = p.lse + (int64_t)bh * p.seqlen;
    if (row_a < p.seqlen) lse[row_a] = (l0 > 0.0f) ? m0 * p.scale + logf(l0) : -INFINITY;
    if (row_a + 8 < p.seqlen) lse[row_a + 8] = (l1 > 0.0f) ? m1 * p.scale + logf(l1) : -INFINITY;
  }
}

// ===================================================================================== delta = rowsum(dO * O)
template <int D>
__global__ void attn_delta_kernel(const AttnParams p) {
  // one warp per (b, h, row)
  const int64_t gw = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const int64_t total = (int64_t)p.batch * p.heads * p.seqlen;
  if (gw >= total) return;
  const int r = (int)(gw % p.seqlen);
  const int bh = (int)(gw / p.seqlen);
  const int b = bh / p.heads, h = bh % p.heads;
  const __nv_bfloat16* o = p.o + b * p.o_sb + h * p.o_sh + (int64_t)r * p.o_ss;
  const __nv_bfloat16* d = p.d_o + b * p.do_sb + h * p.do_sh + (int64_t)r * p.do_ss;
  float acc = 0.0f;
  for (int c = lane * 2; c < D; c += 64) {
    __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(o + c);
    __nv_bfloat162 e = *reinterpret_cast<const __nv_bfloat162*>(d + c);
    acc += __bfloat162float(a.x) * __bfloat162float(e.x) + __bfloat162float(a.y) * __bfloat162float(e.y);
  }
  acc = warp_sum(acc);
  if (lane == 0) const_cast<float*>(p.delta)[gw] = acc;
}

// ===================================================================================== dK, dV
// CTA owns 64 key rows (16 per warp); loops over 32-row query tiles.  Everything is computed in the
// transposed frame: S^T = K Q^T, dP^T = V dO^T, dV += P^T dO, dK += dS^T Q.
template <int D>
__global__ void __launch_bounds__(kAttnThreads) attn_bwd_dkdv_kernel(const AttnParams p) {
  constexpr int BC = 64, BR = 32;
  constexpr int KV_BYTES = BC * D * 2, Q_BYTES = BR * D * 2;
  extern __shared__ __align__(128) uint8_t smem[];
  const uint32_t sK = smem_addr(smem);
  const uint32_t sV = sK + KV_BYTES;
  const uint32_t sQ = sV + KV_BYTES;            // 2 buffers
  const uint32_t sDO = sQ + 2 * Q_BYTES;        // 2 buffers
  float* sLse = reinterpret_cast<float*>(smem + 2 * KV_BYTES + 4 * Q_BYTES);    // [2][BR]
  float* sDelta = sLse + 2 * BR;                                                 // [2][BR]

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int kblk = blockIdx.x;
  const int bh = blockIdx.y;
  const int b = bh / p.heads, h = bh % p.heads;
  const int c0 = kblk * BC;

  const __nv_bfloat16* gq = p.q + b * p.q_sb + h * p.q_sh;
  const __nv_bfloat16* gk = p.k + b * p.k_sb + h * p.k_sh;
  const __nv_bfloat16* gv = p.v + b * p.v_sb + h * p.v_sh;
  const __nv_bfloat16* gdo = p.d_o + b * p.do_sb + h * p.do_sh;
  const float* glse = p.lse + (int64_t)bh * p.seqlen;
  const float* gdelta = p.delta + (int64_t)bh * p.seqlen;

  const int n_q = (p.seqlen + BR - 1) / BR;
  const int q_begin = p.causal ? (c0 / BR) : 0;

  auto load_q = [&](int qi, int buf) {
    load_tile<D, BR>(sQ + buf * Q_BYTES, gq, p.q_ss, qi * BR, p.seqlen);
    load_tile<D, BR>(sDO + buf * Q_BYTES, gdo, p.do_ss, qi * BR, p.seqlen);
    if (threadIdx.x < BR) {
      int r = qi * BR + threadIdx.x;
      sLse[buf * BR + threadIdx.x] = r < p.seqlen ? glse[r] : INFINITY;
      sDelta[buf * BR + threadIdx.x] = r < p.seqlen ? gdelta[r] : 0.0f;
    }
  };

  load_tile<D, BC>(sK, gk, p.k_ss, c0, p.seqlen);
  load_tile<D, BC>(sV, gv, p.v_ss, c0, p.seqlen);
  if (q_begin < n_q) load_q(q_begin, 0);
  cp_async_commit();

  float dk[D / 8][4], dv[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) {
    dk[i][0] = dk[i][1] = dk[i][2] = dk[i][3] = 0.0f;
    dv[i][0] = dv[i][1] = dv[i][2] = dv[i][3] = 0.0f;
  }
  const int kv_a = c0 + warp * 16 + g;    // this thread's key rows: kv_a, kv_a + 8

  for (int qi = q_begin; qi < n_q; ++qi) {
    const int buf = (qi - q_begin) & 1;
    if (qi + 1 < n_q) {
      load_q(qi + 1, buf ^ 1);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const uint32_t qb = sQ + buf * Q_BYTES, dob = sDO + buf * Q_BYTES;
    const float* lse = sLse + buf * BR;
    const float* delta = sDelta + buf * BR;
    const int r0 = qi * BR;

    // S^T (16 x BR) and dP^T (16 x BR)
    float st[BR / 8][4], dpt[BR / 8][4];
#pragma unroll
    for (int i = 0; i < BR / 8; ++i) {
      st[i][0] = st[i][1] = st[i][2] = st[i][3] = 0.0f;
      dpt[i][0] = dpt[i][1] = dpt[i][2] = dpt[i][3] = 0.0f;
    }
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
      uint32_t a0, a1, a2, a3, e0, e1, e2, e3;
      ldmatrix_x4(addr_a<D>(sK, warp * 16, kk * 16, lane), a0, a1, a2, a3);
      ldmatrix_x4(addr_a<D>(sV, warp * 16, kk * 16, lane), e0, e1, e2, e3);
#pragma unroll
      for (int nt = 0; nt < BR / 16; ++nt) {
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4(addr_b<D>(qb, nt * 16, kk * 16, lane), b0, b1, b2, b3);
        mma_bf16(st[2 * nt], a0, a1, a2, a3, b0, b1);
        mma_bf16(st[2 * nt + 1], a0, a1, a2, a3, b2, b3);
        ldmatrix_x4(addr_b<D>(dob, nt * 16, kk * 16, lane), b0, b1, b2, b3);
        mma_bf16(dpt[2 * nt], e0, e1, e2, e3, b0, b1);
        mma_bf16(dpt[2 * nt + 1], e0, e1, e2, e3, b2, b3);
      }
    }
    // P^T = exp(S^T * scale - lse[q]);  dS^T = P^T * (dP^T - delta[q]) * scale
#pragma unroll
    for (int i = 0; i < BR / 8; ++i) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        int ql = i * 8 + 2 * t + (e & 1);
        int qrow = r0 + ql;
        int kv = kv_a + ((e >> 1) ? 8 : 0);
        bool masked = (qrow >= p.seqlen) || (kv >= p.seqlen) || (p.causal && kv > qrow);
        float pv = masked ? 0.0f : exp2f((st[i][e] * p.scale - lse[ql]) * kLog2e);
        st[i][e] = pv;
        dpt[i][e] = pv * (dpt[i][e] - delta[ql]) * p.scale;
      }
    }
    // dV += P^T dO ; dK += dS^T Q   (k-dimension = query rows of this tile)
#pragma unroll
    for (int kk = 0; kk < BR / 16; ++kk) {
      uint32_t pa0 = pack_bf16(st[2 * kk][0], st[2 * kk][1]);
      uint32_t pa1 = pack_bf16(st[2 * kk][2], st[2 * kk][3]);
      uint32_t pa2 = pack_bf16(st[2 * kk + 1][0], st[2 * kk + 1][1]);
      uint32_t pa3 = pack_bf16(st[2 * kk + 1][2], st[2 * kk + 1][3]);
      uint32_t sa0 = pack_bf16(dpt[2 * kk][0], dpt[2 * kk][1]);
      uint32_t sa1 = pack_bf16(dpt[2 * kk][2], dpt[2 * kk][3]);
      uint32_t sa2 = pack_bf16(dpt[2 * kk + 1][0], dpt[2 * kk + 1][1]);
      uint32_t sa3 = pack_bf16(dpt[2 * kk + 1][2], dpt[2 * kk + 1][3]);
#pragma unroll
      for (int nt = 0; nt < D / 16; ++nt) {
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4_trans(addr_bt<D>(dob, kk * 16, nt * 16, lane), b0, b1, b2, b3);
        mma_bf16(dv[2 * nt], pa0, pa1, pa2, pa3, b0, b1);
        mma_bf16(dv[2 * nt + 1], pa0, pa1, pa2, pa3, b2, b3);
        ldmatrix_x4_trans(addr_bt<D>(qb, kk * 16, nt * 16, lane), b0, b1, b2, b3);
        mma_bf16(dk[2 * nt], sa0, sa1, sa2, sa3, b0, b1);
        mma_bf16(dk[2 * nt + 1], sa0, sa1, sa2, sa3, b2, b3);
      }
    }
    __syncthreads();
  }

  __nv_bfloat16* gdk = p.dk + b * p.dk_sb + h * p.dk_sh;
  __nv_bfloat16* gdv = p.dv + b * p.dv_sb + h * p.dv_sh;
#pragma unroll
  for (int i = 0; i < D / 8; ++i) {
    int col = i * 8 + 2 * t;
    if (kv_a < p.seqlen) {
      *reinterpret_cast<uint32_t*>(gdk + (int64_t)kv_a * p.dk_ss + col) = pack_bf16(dk[i][0], dk[i][1]);
      *reinterpret_cast<uint32_t*>(gdv + (int64_t)kv_a * p.dv_ss + col) = pack_bf16(dv[i][0], dv[i][1]);
    }
    if (kv_a + 8 < p.seqlen) {
      *reinterpret_cast<uint32_t*>(gdk + (int64_t)(kv_a + 8) * p.dk_ss + col) = pack_bf16(dk[i][2], dk[i][3]);
      *reinterpret_cast<uint32_t*>(gdv + (int64_t)(kv_a + 8) * p.dv_ss + col) = pack_bf16(dv[i][2], dv[i][3]);
    }
  }
}

// ===================================================================================== dQ
// CTA owns 64 query rows (16 per warp); loops over 64-row key tiles.
template <int D>
__global__ void __launch_bounds__(kAttnThreads) attn_bwd_dq_kernel(const AttnParams p) {
  constexpr int BR = 64, BC = 64;
  constexpr int Q_BYTES = BR * D * 2, KV_BYTES = BC * D * 2;
  extern __shared__ __align__(128) uint8_t smem[];
  const uint32_t sQ = smem_addr(smem);
  const uint32_t sDO = sQ + Q_BYTES;
  const uint32_t sK = sDO + Q_BYTES;            // 2 buffers
  const uint32_t sV = sK + 2 * KV_BYTES;        // 2 buffers

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int qblk = gridDim.x - 1 - blockIdx.x;
  const int bh = blockIdx.y;
  const int b = bh / p.heads, h = bh % p.heads;
  const int q0 = qblk * BR;

  const __nv_bfloat16* gq = p.q + b * p.q_sb + h * p.q_sh;
  const __nv_bfloat16* gk = p.k + b * p.k_sb + h * p.k_sh;
  const __nv_bfloat16* gv = p.v + b * p.v_sb + h * p.v_sh;
  const __nv_bfloat16* gdo = p.d_o + b * p.do_sb + h * p.do_sh;

  int n_kv = (p.seqlen + BC - 1) / BC;
  if (p.causal) {
    int lim = (q0 + BR + BC - 1) / BC;
    n_kv = lim < n_kv ? lim : n_kv;
  }
  load_tile<D, BR>(sQ, gq, p.q_ss, q0, p.seqlen);
  load_tile<D, BR>(sDO, gdo, p.do_ss, q0, p.seqlen);
  load_tile<D, BC>(sK, gk, p.k_ss, 0, p.seqlen);
  load_tile<D, BC>(sV, gv, p.v_ss, 0, p.seqlen);
  cp_async_commit();

  const int row_a = q0 + warp * 16 + g;
  const float* glse = p.lse + (int64_t)bh * p.seqlen;
  const float* gdelta = p.delta + (int64_t)bh * p.seqlen;
  const float lse0 = row_a < p.seqlen ? glse[row_a] : INFINITY;
  const float lse1 = row_a + 8 < p.seqlen ? glse[row_a + 8] : INFINITY;
  const float dl0 = row_a < p.seqlen ? gdelta[row_a] : 0.0f;
  const float dl1 = row_a + 8 < p.seqlen ? gdelta[row_a + 8] : 0.0f;

  float dq[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) dq[i][0] = dq[i][1] = dq[i][2] = dq[i][3] = 0.0f;

  for (int j = 0; j < n_kv; ++j) {
    const int buf = j & 1;
    if (j + 1 < n_kv) {
      load_tile<D, BC>(sK + (buf ^ 1) * KV_BYTES, gk, p.k_ss, (j + 1) * BC, p.seqlen);
      load_tile<D, BC>(sV + (buf ^ 1) * KV_BYTES, gv, p.v_ss, (j + 1) * BC, p.seqlen);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const uint32_t kb = sK + buf * KV_BYTES, vb = sV + buf * KV_BYTES;
    const int c0 = j * BC;

    float s[BC / 8][4], dp[BC / 8][4];
#pragma unroll
    for (int i = 0; i < BC / 8; ++i) {
      s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.0f;
      dp[i][0] = dp[i][1] = dp[i][2] = dp[i][3] = 0.0f;
    }
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
      uint32_t a0, a1, a2, a3, e0, e1, e2, e3;
      ldmatrix_x4(addr_a<D>(sQ, warp * 16, kk * 16, lane), a0, a1, a2, a3);
      ldmatrix_x4(addr_a<D>(sDO, warp * 16, kk * 16, lane), e0, e1, e2, e3);
#pragma unroll
      for (int nt = 0; nt < BC / 16; ++nt) {
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4(addr_b<D>(kb, nt * 16, kk * 16, lane), b0, b1, b2, b3);
        mma_bf16(s[2 * nt], a0, a1, a2, a3, b0, b1);
        mma_bf16(s[2 * nt + 1], a0, a1, a2, a3, b2, b3);
        ldmatrix_x4(addr_b<D>(vb, nt * 16, kk * 16, lane), b0, b1, b2, b3);
        mma_bf16(dp[2 * nt], e0, e1, e2, e3, b0, b1);
        mma_bf16(dp[2 * nt + 1], e0, e1, e2, e3, b2, b3);
      }
    }
#pragma unroll
    for (int i = 0; i < BC / 8; ++i) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        int col = c0 + i * 8 + 2 * t + (e & 1);
        bool hi = (e >> 1) != 0;
        int row = row_a + (hi ? 8 : 0);
        bool masked = (col >= p.seqlen) || (row >= p.seqlen) || (p.causal && col > row);
        float pv = masked ? 0.0f : exp2f((s[i][e] * p.scale - (hi ? lse1 : lse0)) * kLog2e);
        s[i][e] = pv * (dp[i][e] - (hi ? dl1 : dl0)) * p.scale;    // dS
      }
    }
    // dQ += dS K
#pragma unroll
    for (int kk = 0; kk < BC / 16; ++kk) {
      uint32_t a0 = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
      uint32_t a1 = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
      uint32_t a2 = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      uint32_t a3 = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int nt = 0; nt < D / 16; ++nt) {
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4_trans(addr_bt<D>(kb, kk * 16, nt * 16, lane), b0, b1, b2, b3);
        mma_bf16(dq[2 * nt], a0, a1, a2, a3, b0, b1);
        mma_bf16(dq[2 * nt + 1], a0, a1, a2, a3, b2, b3);
      }
    }
    __syncthreads();
  }

  __nv_bfloat16* gdq = p.dq + b * p.dq_sb + h * p.dq_sh;
#pragma unroll
  for (int i = 0; i < D / 8; ++i) {
    int col = i * 8 + 2 * t;
    if (row_a < p.seqlen) *reinterpret_cast<uint32_t*>(gdq + (int64_t)row_a * p.dq_ss + col) = pack_bf16(dq[i][0], dq[i][1]);
    if (row_a + 8 < p.seqlen) *reinterpret_cast<uint32_t*>(gdq + (int64_t)(row_a + 8) * p.dq_ss + col) = pack_bf16(dq[i][2], dq[i][3]);
  }
}

template <typename K>
int set_smem(K kernel, int bytes) {
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e != cudaSuccess) {
    msamp_set_error("cudaFuncSetAttribute(attention): %s", cudaGetErrorString(e));
    return MSAMP_ELAUNCH;
  }
  return MSAMP_OK;
}

template <int D>
int run_fwd(const AttnParams& p, cudaStream_t stream) {
  constexpr int SMEM = 64 * D * 2 + 4 * 64 * D * 2;
  int rc = set_smem(attn_fwd_kernel<D>, SMEM);
  if (rc) return rc;
  dim3 grid((p.seqlen + 63) / 64, p.batch * p.heads);
  attn_fwd_kernel<D><<<grid, kAttnThreads, SMEM, stream>>>(p);
  return msamp_check_launch("attn_fwd_kernel");
}

template <int D>
int run_bwd(const AttnParams& p, cudaStream_t stream) {
  {
    int64_t warps = (int64_t)p.batch * p.heads * p.seqlen;
    int blocks = (int)((warps * 32 + 255) / 256);
    attn_delta_kernel<D><<<blocks, 256, 0, stream>>>(p);
  }
  {
    constexpr int SMEM = 2 * 64 * D * 2 + 4 * 32 * D * 2 + 4 * 32 * 4;
    int rc = set_smem(attn_bwd_dkdv_kernel<D>, SMEM);
    if (rc) return rc;
    dim3 grid((p.seqlen + 63) / 64, p.batch * p.heads);
    attn_bwd_dkdv_kernel<D><<<grid, kAttnThreads, SMEM, stream>>>(p);
  }
  {
    constexpr int SMEM = 2 * 64 * D * 2 + 4 * 64 * D * 2;
    int rc = set_smem(attn_bwd_dq_kernel<D>, SMEM);
    if (rc) return rc;
    dim3 grid((p.seqlen + 63) / 64, p.batch * p.heads);
    attn_bwd_dq_kernel<D><<<grid, kAttnThreads, SMEM, stream>>>(p);
  }
  return msamp_check_launch("attn_bwd kernels");
}

}    // namespace

// strides: 24 int64 values = (batch, seq, head) element strides of q, k, v, o, dO, dq, dk, dv in that order.
// Every pointer must be 16-byte aligned and every stride a multiple of 8 elements (16-byte cp.async).
MSAMP_API int msamp_attention_fwd(const void* q, const void* k, const void* v, void* o, float* lse, const int64_t* strides, int batch,
                                  int heads, int seqlen, int head_dim, float scale, int causal, void* stream_) {
  MSAMP_REQUIRE(head_dim == 64 || head_dim == 128, "attention: head_dim must be 64 or 128 (got %d)", head_dim);
  MSAMP_REQUIRE(batch > 0 && heads > 0 && seqlen > 0, "attention: empty problem");
  for (int i = 0; i < 12; ++i) MSAMP_REQUIRE(strides[i] % 8 == 0, "attention: stride %d is not a multiple of 8 elements", i);
  AttnParams p = {};
  p.q = (const __nv_bfloat16*)q; p.k = (const __nv_bfloat16*)k; p.v = (const __nv_bfloat16*)v; p.o = (__nv_bfloat16*)o; p.lse = lse;
  p.q_sb = strides[0]; p.q_ss = strides[1]; p.q_sh = strides[2];
  p.k_sb = strides[3]; p.k_ss = strides[4]; p.k_sh = strides[5];
  p.v_sb = strides[6]; p.v_ss = strides[7]; p.v_sh = strides[8];
  p.o_sb = strides[9]; p.o_ss = strides[10]; p.o_sh = strides[11];
  p.batch = batch; p.heads = heads; p.seqlen = seqlen; p.scale = scale; p.causal = causal;
  return head_dim == 128 ? run_fwd<128>(p, (cudaStream_t)stream_) : run_fwd<64>(p, (cudaStream_t)stream_);
}

// delta: scratch [batch, heads, seqlen] fp32 owned by the caller.
MSAMP_API int msamp_attention_bwd(const void* q, const void* k, const void* v, const void* o, const float* lse, const void* d_o,
                                  void* dq, void* dk, void* dv, float* delta, const int64_t* strides, int batch, int heads, int seqlen,
                                  int head_dim, float scale, int causal, void* stream_) {
  MSAMP_REQUIRE(head_dim == 64 || head_dim == 128, "attention: head_dim must be 64 or 128 (got %d)", head_dim);
  MSAMP_REQUIRE(batch > 0 && heads > 0 && seqlen > 0, "attention: empty problem");
  for (int i = 0; i < 24; ++i) MSAMP_REQUIRE(strides[i] % 8 == 0, "attention: stride %d is not a multiple of 8 elements", i);
  AttnParams p = {};
  p.q = (const __nv_bfloat16*)q; p.k = (const __nv_bfloat16*)k; p.v = (const __nv_bfloat16*)v; p.o = (__nv_bfloat16*)const_cast<void*>(o);
  p.lse = const_cast<float*>(lse); p.d_o = (const __nv_bfloat16*)d_o; p.delta = delta;
  p.dq = (__nv_bfloat16*)dq; p.dk = (__nv_bfloat16*)dk; p.dv = (__nv_bfloat16*)dv;
  p.q_sb = strides[0]; p.q_ss = strides[1]; p.q_sh = strides[2];
  p.k_sb = strides[3]; p.k_ss = strides[4]; p.k_sh = strides[5];
  p.v_sb = strides[6]; p.v_ss = strides[7]; p.v_sh = strides[8];
  p.o_sb = strides[9]; p.o_ss = strides[10]; p.o_sh = strides[11];
  p.do_sb = strides[12]; p.do_ss = strides[13]; p.do_sh = strides[14];
  p.dq_sb = strides[15]; p.dq_ss = strides[16]; p.dq_sh = strides[17];
  p.dk_sb = strides[18]; p.dk_ss = strides[19]; p.dk_sh = strides[20];
  p.dv_sb = strides[21]; p.dv_ss = strides[22]; p.dv_sh = strides[23];
  p.batch = batch; p.heads = heads; p.seqlen = seqlen; p.scale = scale; p.causal = causal;
  return head_dim == 128 ? run_bwd<128>(p, (cudaStream_t)stream_) : run_bwd<64>(p, (cudaStream_t)stream_);
}
