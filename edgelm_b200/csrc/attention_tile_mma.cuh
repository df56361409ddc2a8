// One 64-key tile of decode attention on the tensor cores: scores, running softmax and weighted
// values of up to 16 query rows against a key tile and a value tile in shared memory (bfloat16,
// rows padded by 16 bytes so that ldmatrix reads hit distinct banks).  Pure register arithmetic of
// one warp, no synchronisation beyond the warp's own.
#pragma once
#include <cuda_bf16.h>
#include <math_constants.h>
#include <stdint.h>

namespace edgelm {

__device__ __forceinline__ void dm_mma(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void dm_ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void dm_ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ uint32_t dm_pack(float a, float b) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&v);
}
__device__ __forceinline__ float dm_exp2(float x) {   // 2^x on the special-function unit; 2^-inf = 0
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t dm_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// Rotary encoding of eight dims d .. d + 7 of a head row's first half (`lo`) with their partners in the second
// half (`hi`): (a, b) -> (a cos - b sin, b cos + a sin) in float32, rounded to bfloat16.  cos_row / sin_row: the
// position's row of the tables [head_dim / 2], 16-byte aligned at d.
__device__ __forceinline__ void dm_rotate8_vals(uint4& lo, uint4& hi, const float* cs, const float* sn) {   // cs, sn: 8 values each
  const __nv_bfloat16* pl = reinterpret_cast<const __nv_bfloat16*>(&lo);
  const __nv_bfloat16* ph = reinterpret_cast<const __nv_bfloat16*>(&hi);
  __nv_bfloat16 ol[8], oh[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float av = __bfloat162float(pl[j]), bv = __bfloat162float(ph[j]);
    ol[j] = __float2bfloat16_rn(av * cs[j] - bv * sn[j]);
    oh[j] = __float2bfloat16_rn(bv * cs[j] + av * sn[j]);
  }
  lo = *reinterpret_cast<const uint4*>(ol);
  hi = *reinterpret_cast<const uint4*>(oh);
}
__device__ __forceinline__ void dm_rotate8(uint4& lo, uint4& hi, const float* cos_row, const float* sin_row, int d) {
  const float4 c0 = *reinterpret_cast<const float4*>(cos_row + d), c1 = *reinterpret_cast<const float4*>(cos_row + d + 4);
  const float4 s0 = *reinterpret_cast<const float4*>(sin_row + d), s1 = *reinterpret_cast<const float4*>(sin_row + d + 4);
  const float cs[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w}, sn[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
  dm_rotate8_vals(lo, hi, cs, sn);
}

constexpr int DM_ROWS = 16;       // query heads of a kv head served in one pass (rows of the A operand)
constexpr int DM_TILE_KEYS = 64;  // keys of a tile: one page of the cache

// The query rows [16][HD + 8] in shared memory as the A fragments of the score products.
template <int HDT>
__device__ __forceinline__ void dm_load_queries(const __nv_bfloat16* Qs, uint32_t (&qa)[HDT][4]) {
  constexpr int PITCH = HDT * 16 + 8;
  const int lane = threadIdx.x & 31, mi = lane >> 3;
  // matrices: (rows 0-7, k 0-7), (rows 8-15, k 0-7), (rows 0-7, k 8-15), (rows 8-15, k 8-15)
#pragma unroll
  for (int ks = 0; ks < HDT; ++ks)
    dm_ldmatrix_x4(dm_smem_u32(Qs + ((mi & 1) * 8 + (lane & 7)) * PITCH + ks * 16 + (mi >> 1) * 8), qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3]);
}

// Fold one tile into the warp's running state, in two halves so that a caller can wait for the values while the
// scores are computed: dm_tile_scores needs the key tile only and leaves the tile's weights in `s` (with the running
// maximum, the sum and the rescaled accumulators up to date), dm_tile_values adds the weighted values.  A lane holds
// rows gid = lane / 4 (state mA, lA and o[.][0..1]) and gid + 8 (mB, lB, o[.][2..3]); `valid` >= 1 keys of the tile
// belong to the sequence, the value rows of the others hold zeros.
template <int HDT>
__device__ __forceinline__ void dm_tile_scores(const __nv_bfloat16* Kt, const uint32_t (&qa)[HDT][4], int valid, float scale,
                                               float (&s)[8][4], float (&o)[HDT * 2][4], float& mA, float& mB, float& lA,
                                               float& lB) {
  constexpr int HD = HDT * 16, PITCH = HD + 8;
  const int lane = threadIdx.x & 31, tig = lane & 3, mi = lane >> 3;
  // ---- scores: 8 tiles of 8 keys
#pragma unroll
  for (int nt = 0; nt < 8; ++nt) {
    s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
    for (int ks2 = 0; ks2 < HDT; ks2 += 2) {
      uint32_t b0, b1, b2, b3;
      dm_ldmatrix_x4(dm_smem_u32(Kt + (nt * 8 + (lane & 7)) * PITCH + (ks2 + (mi >> 1)) * 16 + (mi & 1) * 8), b0, b1, b2, b3);
      dm_mma(s[nt], qa[ks2][0], qa[ks2][1], qa[ks2][2], qa[ks2][3], b0, b1);
      dm_mma(s[nt], qa[ks2 + 1][0], qa[ks2 + 1][1], qa[ks2 + 1][2], qa[ks2 + 1][3], b2, b3);
    }
  }
  // the exponentials are 2^x on the special-function unit: p = 2^((s - max) * scale * log2(e)), with the scale
  // folded into one multiply-add per score; the running maximum stays in the units of the scaled scores
  if (valid < DM_TILE_KEYS) {
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      const int key = nt * 8 + tig * 2;
      if (key >= valid) s[nt][0] = s[nt][2] = -CUDART_INF_F;
      if (key + 1 >= valid) s[nt][1] = s[nt][3] = -CUDART_INF_F;
    }
  }
  float mxA = -CUDART_INF_F, mxB = -CUDART_INF_F;
#pragma unroll
  for (int nt = 0; nt < 8; ++nt) {
    mxA = fmaxf(mxA, fmaxf(s[nt][0], s[nt][1]));
    mxB = fmaxf(mxB, fmaxf(s[nt][2], s[nt][3]));
  }
  mxA = fmaxf(mxA, __shfl_xor_sync(0xffffffffu, mxA, 1));
  mxA = fmaxf(mxA, __shfl_xor_sync(0xffffffffu, mxA, 2));
  mxB = fmaxf(mxB, __shfl_xor_sync(0xffffffffu, mxB, 1));
  mxB = fmaxf(mxB, __shfl_xor_sync(0xffffffffu, mxB, 2));
  constexpr float LOG2E = 1.4426950408889634f;
  const float c2 = scale * LOG2E;
  const float nmA = fmaxf(mA, mxA * scale), nmB = fmaxf(mB, mxB * scale);   // finite: valid >= 1, scale > 0
  const float corrA = dm_exp2((mA - nmA) * LOG2E), corrB = dm_exp2((mB - nmB) * LOG2E);
  const float offA = nmA * LOG2E, offB = nmB * LOG2E;
  float sumA = 0.f, sumB = 0.f;
#pragma unroll
  for (int nt = 0; nt < 8; ++nt) {
    s[nt][0] = dm_exp2(fmaf(s[nt][0], c2, -offA));
    s[nt][1] = dm_exp2(fmaf(s[nt][1], c2, -offA));
    s[nt][2] = dm_exp2(fmaf(s[nt][2], c2, -offB));
    s[nt][3] = dm_exp2(fmaf(s[nt][3], c2, -offB));
    sumA += s[nt][0] + s[nt][1];
    sumB += s[nt][2] + s[nt][3];
  }
  sumA += __shfl_xor_sync(0xffffffffu, sumA, 1);
  sumA += __shfl_xor_sync(0xffffffffu, sumA, 2);
  sumB += __shfl_xor_sync(0xffffffffu, sumB, 1);
  sumB += __shfl_xor_sync(0xffffffffu, sumB, 2);
  lA = lA * corrA + sumA;
  lB = lB * corrB + sumB;
  mA = nmA;
  mB = nmB;
#pragma unroll
  for (int i = 0; i < HD / 8; ++i) {
    o[i][0] *= corrA;
    o[i][1] *= corrA;
    o[i][2] *= corrB;
    o[i][3] *= corrB;
  }
}

template <int HDT>
__device__ __forceinline__ void dm_tile_values(const __nv_bfloat16* Vt, const float (&s)[8][4], float (&o)[HDT * 2][4]) {
  constexpr int HD = HDT * 16, PITCH = HD + 8;
  const int lane = threadIdx.x & 31, mi = lane >> 3;
  // ---- values: 4 steps of 16 keys
#pragma unroll
  for (int kt = 0; kt < 4; ++kt) {
    const uint32_t a0 = dm_pack(s[2 * kt][0], s[2 * kt][1]), a1 = dm_pack(s[2 * kt][2], s[2 * kt][3]);
    const uint32_t a2 = dm_pack(s[2 * kt + 1][0], s[2 * kt + 1][1]), a3 = dm_pack(s[2 * kt + 1][2], s[2 * kt + 1][3]);
#pragma unroll
    for (int dt = 0; dt < HD / 8; dt += 2) {
      uint32_t b0, b1, b2, b3;
      dm_ldmatrix_x4_trans(dm_smem_u32(Vt + (kt * 16 + (mi & 1) * 8 + (lane & 7)) * PITCH + (dt + (mi >> 1)) * 8), b0, b1, b2, b3);
      dm_mma(o[dt], a0, a1, a2, a3, b0, b1);
      dm_mma(o[dt + 1], a0, a1, a2, a3, b2, b3);
    }
  }
}

template <int HDT>
__device__ __forceinline__ void dm_tile_update(const __nv_bfloat16* Kt, const __nv_bfloat16* Vt, const uint32_t (&qa)[HDT][4],
                                               int valid, float scale, float (&o)[HDT * 2][4], float& mA, float& mB,
                                               float& lA, float& lB) {
  float s[8][4];
  dm_tile_scores<HDT>(Kt, qa, valid, scale, s, o, mA, mB, lA, lB);
  dm_tile_values<HDT>(Vt, s, o);
}

}  // namespace edgelm

// ---------------------------------------------------------------------------------------------------------------
// The same tile for up to 8 query heads, with the roles of the operands swapped: the keys are the 16-row operand and
// the heads the 8 columns, S^T = K Q^T and O^T = V^T P^T.  No row of a product is padding then (with the heads as
// rows, 8 of the 16 are zeros whenever a kv head serves 8 heads or fewer), a lane holds 16 scores instead of 32,
// and the accumulators are half as many: the tile costs half the tensor-core work and half the exponentials.
namespace edgelm {

__device__ __forceinline__ void dm_mma_b(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  dm_mma(c, a0, a1, a2, a3, b0, b1);
}
__device__ __forceinline__ uint32_t dm_transpose8(uint32_t x) {   // an 8 x 8 matrix of 16-bit values spread over the warp, transposed
  uint32_t y;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(y) : "r"(x));
  return y;
}

constexpr int DM_HEADS_T = 8;   // query heads of a kv head that the swapped form serves in one pass

// Query rows 0..7 of Qs [.][HD + 8] as the B fragments of the score products: qb[ks] = dims ks * 16 .. + 15.
template <int HDT>
__device__ __forceinline__ void dm_load_queries_t(const __nv_bfloat16* Qs, uint32_t (&qb)[HDT][2]) {
  constexpr int PITCH = HDT * 16 + 8;
  const int lane = threadIdx.x & 31, mi = lane >> 3;
  // matrices: (heads, dims 0-7), (heads, dims 8-15) of step ks2, then of step ks2 + 1
#pragma unroll
  for (int ks2 = 0; ks2 < HDT; ks2 += 2)
    dm_ldmatrix_x4(dm_smem_u32(Qs + (lane & 7) * PITCH + (ks2 + (mi >> 1)) * 16 + (mi & 1) * 8), qb[ks2][0], qb[ks2][1], qb[ks2 + 1][0], qb[ks2 + 1][1]);
}

// Fold one tile into the warp's running state.  A lane holds the heads 2 tig (state mA, lA, o[.][0] and o[.][2]) and
// 2 tig + 1 (mB, lB, o[.][1], o[.][3]); o[dt][0..1] is dim dt * 16 + gid, o[dt][2..3] dim dt * 16 + gid + 8.  mA and
// mB are the same in the eight lanes that share a head; lA and lB are the lane's own share of the sum (its keys
// gid, gid + 8, gid + 16, ..): add the eight lanes' shares when the tiles are done (dm_sum_over_keys).
template <int HDT>
__device__ __forceinline__ void dm_tile_scores_t(const __nv_bfloat16* Kt, const uint32_t (&qb)[HDT][2], int valid, float scale,
                                                 float (&s)[4][4], float (&o)[HDT][4], float& mA, float& mB, float& lA, float& lB) {
  constexpr int HD = HDT * 16, PITCH = HD + 8;
  const int lane = threadIdx.x & 31, gid = lane >> 2, mi = lane >> 3;
  // ---- scores: 4 blocks of 16 keys; s[mt][0..1] is key mt * 16 + gid, s[mt][2..3] key mt * 16 + gid + 8
#pragma unroll
  for (int mt = 0; mt < 4; ++mt) {
    s[mt][0] = s[mt][1] = s[mt][2] = s[mt][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < HDT; ++ks) {
      uint32_t a0, a1, a2, a3;
      dm_ldmatrix_x4(dm_smem_u32(Kt + (mt * 16 + (mi & 1) * 8 + (lane & 7)) * PITCH + ks * 16 + (mi >> 1) * 8), a0, a1, a2, a3);
      dm_mma_b(s[mt], a0, a1, a2, a3, qb[ks][0], qb[ks][1]);
    }
  }
  if (valid < DM_TILE_KEYS) {
#pragma unroll
    for (int mt = 0; mt < 4; ++mt) {
      if (mt * 16 + gid >= valid) s[mt][0] = s[mt][1] = -CUDART_INF_F;
      if (mt * 16 + gid + 8 >= valid) s[mt][2] = s[mt][3] = -CUDART_INF_F;
    }
  }
  float mxA = -CUDART_INF_F, mxB = -CUDART_INF_F;
#pragma unroll
  for (int mt = 0; mt < 4; ++mt) {
    mxA = fmaxf(mxA, fmaxf(s[mt][0], s[mt][2]));
    mxB = fmaxf(mxB, fmaxf(s[mt][1], s[mt][3]));
  }
#pragma unroll
  for (int off = 4; off < 32; off <<= 1) {   // over the lanes that hold the other keys of the same heads
    mxA = fmaxf(mxA, __shfl_xor_sync(0xffffffffu, mxA, off));
    mxB = fmaxf(mxB, __shfl_xor_sync(0xffffffffu, mxB, off));
  }
  constexpr float LOG2E = 1.4426950408889634f;
  const float c2 = scale * LOG2E;
  const float nmA = fmaxf(mA, mxA * scale), nmB = fmaxf(mB, mxB * scale);   // finite: valid >= 1, scale > 0
  const float corrA = dm_exp2((mA - nmA) * LOG2E), corrB = dm_exp2((mB - nmB) * LOG2E);
  const float offA = nmA * LOG2E, offB = nmB * LOG2E;
  float sumA = 0.f, sumB = 0.f;
#pragma unroll
  for (int mt = 0; mt < 4; ++mt) {
    s[mt][0] = dm_exp2(fmaf(s[mt][0], c2, -offA));
    s[mt][1] = dm_exp2(fmaf(s[mt][1], c2, -offB));
    s[mt][2] = dm_exp2(fmaf(s[mt][2], c2, -offA));
    s[mt][3] = dm_exp2(fmaf(s[mt][3], c2, -offB));
    sumA += s[mt][0] + s[mt][2];
    sumB += s[mt][1] + s[mt][3];
  }
  lA = lA * corrA + sumA;
  lB = lB * corrB + sumB;
  mA = nmA;
  mB = nmB;
#pragma unroll
  for (int dt = 0; dt < HDT; ++dt) {
    o[dt][0] *= corrA;
    o[dt][1] *= corrB;
    o[dt][2] *= corrA;
    o[dt][3] *= corrB;
  }
}

template <int HDT>
__device__ __forceinline__ void dm_tile_values_t(const __nv_bfloat16* Vt, const float (&s)[4][4], float (&o)[HDT][4]) {
  constexpr int HD = HDT * 16, PITCH = HD + 8;
  const int lane = threadIdx.x & 31, mi = lane >> 3;
  // ---- values: O^T += V^T P^T, 4 steps of 16 keys; the weights of a step, held as (key, two heads) per lane, go
  // through a transpose to (head, two keys), which is how the 8-column operand wants them
#pragma unroll
  for (int kt = 0; kt < 4; ++kt) {
    const uint32_t b0 = dm_transpose8(dm_pack(s[kt][0], s[kt][1])), b1 = dm_transpose8(dm_pack(s[kt][2], s[kt][3]));
#pragma unroll
    for (int dt = 0; dt < HDT; ++dt) {
      uint32_t a0, a1, a2, a3;
      // matrices as stored (8 keys x 8 dims each): (keys 0-7, dims 0-7), (keys 0-7, dims 8-15), (keys 8-15, dims 0-7), (keys 8-15, dims 8-15)
      dm_ldmatrix_x4_trans(dm_smem_u32(Vt + (kt * 16 + (mi >> 1) * 8 + (lane & 7)) * PITCH + dt * 16 + (mi & 1) * 8), a0, a1, a2, a3);
      dm_mma_b(o[dt], a0, a1, a2, a3, b0, b1);
    }
  }
}

template <int HDT>
__device__ __forceinline__ void dm_tile_update_t(const __nv_bfloat16* Kt, const __nv_bfloat16* Vt, const uint32_t (&qb)[HDT][2],
                                                 int valid, float scale, float (&o)[HDT][4], float& mA, float& mB, float& lA,
                                                 float& lB) {
  float s[4][4];
  dm_tile_scores_t<HDT>(Kt, qb, valid, scale, s, o, mA, mB, lA, lB);
  dm_tile_values_t<HDT>(Vt, s, o);
}

// The eight lanes that share a head each hold a share of its sum of weights: all of them get the whole.
__device__ __forceinline__ void dm_sum_over_keys(float& lA, float& lB) {
#pragma unroll
  for (int off = 4; off < 32; off <<= 1) {
    lA += __shfl_xor_sync(0xffffffffu, lA, off);
    lB += __shfl_xor_sync(0xffffffffu, lB, off);
  }
}

}  // namespace edgelm
