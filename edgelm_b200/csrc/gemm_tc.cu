// out = a . W^T in bfloat16 on the fifth-generation tensor cores (tcgen05), float32 accumulation
// in tensor memory, operands staged by TMA, with the same fused epilogues as the CUDA-core kernel.
//
//   a [M, K] bfloat16 (row pitch lda), W [N, K] bfloat16 row-major (out, in): both K-major, which is
//   what tcgen05.mma takes for A and B without a transpose.
//
// One CTA computes a 128 x BN tile.  Six warps, three roles:
//   warp 0    one lane issues TMA loads (cp.async.bulk.tensor.2d, 128-byte swizzle) of a 128 x 64
//             tile of `a` and a BN x 64 tile of W (two for SwiGLU) into a ring of STAGES stages,
//             each guarded by a full/empty mbarrier pair;
//   warp 1    allocates BN (or 2 BN) columns of tensor memory; one lane issues four tcgen05.mma
//             (M 128, N BN, K 16) per stage and commits the stage's release, then the tile's end;
//   warps 2-5 wait for the accumulator, read it with tcgen05.ld (each warp its 32 lanes = rows),
//             apply the epilogue and store.
// M, N and K tails need no special code: TMA fills what lies outside a tensor with zeros, and the
// epilogue stores only rows < M and columns < N.  K must be a multiple of 8 (16-byte row pitch).
//
// Every wait on an mbarrier is bounded (about a second of SM clock): when it runs out the kernel
// sets ERR_WAIT_TIMEOUT in the error word, raises a block-wide abort flag that ends the other
// roles' waits, frees its tensor memory and returns.
#include "attention_tile_mma.cuh"   // dm_rotate8: the rotation, as the separate kernels and the decode attention do it
#include "tc_common.cuh"

namespace edgelm {

enum : int { TC_EPI_STORE = 0, TC_EPI_RESIDUAL = 1, TC_EPI_SWIGLU = 2, TC_EPI_ROPE = 3 };

// What the epilogue of the stacked q, k, v projection of a prompt step needs to finish the job of three kernels
// (TC_EPI_ROPE): each token's position, its sequence's row of the page table, the rotation table, the cache.
// Query heads are rotated and stored to `out`; key heads are rotated and written into their cache page, value heads
// written there as they are; the k and v columns of `out` are not written (attention reads the cache).
struct RopeAppend {
  const int32_t* tok_pos;
  const int32_t* tok_seq;
  const int32_t* seq_slot;
  const int32_t* page_table;
  const float* cos_t;
  const float* sin_t;
  __nv_bfloat16* kcache;
  __nv_bfloat16* vcache;
  int table_stride, n_pages, max_pos, nh, nkv, hd;
};

constexpr int TC_BM = 128;   // rows of `a` per tile = lanes of tensor memory
constexpr int TC_STAGES = 3;   // ring stages of the one-tile kernel when several blocks share an SM (48 KB stages: 144 KB)
constexpr int TC_DEEP_BYTES = 192 * 1024;   // ring of the one-tile kernel when the grid is at most one block an SM
constexpr int TC_THREADS = 192;
// z / (1 + e^-z) with the exponential and the reciprocal on the special-function unit (2^x and 1/x to about 2^-22):
// the result is rounded to bfloat16 right after; an epilogue thread computes 64 to 128 of these while its tile's
// tensor memory is held.  (z < -88: 2^x overflows to infinity, the reciprocal is 0 and the result -0, the limit.)
__device__ __forceinline__ float silu_tc(float z) {
  float e, r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(z * -1.4426950408889634f));
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.0f + e));
  return z * r;
}

template <typename TOut> struct OutVec;
template <> struct OutVec<float> {
  static __device__ __forceinline__ void store8(float* p, const float* v) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
  }
};
template <> struct OutVec<__nv_bfloat16> {
  static __device__ __forceinline__ void store8(__nv_bfloat16* p, const float* v) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
    __nv_bfloat162 c = __floats2bfloat162_rn(v[4], v[5]), d = __floats2bfloat162_rn(v[6], v[7]);
    uint4 u;
    u.x = *reinterpret_cast<uint32_t*>(&a);
    u.y = *reinterpret_cast<uint32_t*>(&b);
    u.z = *reinterpret_cast<uint32_t*>(&c);
    u.w = *reinterpret_cast<uint32_t*>(&d);
    *reinterpret_cast<uint4*>(p) = u;
  }
};

// The epilogue of the 32 columns of one row that a thread holds after tcgen05.ld: 16-byte loads of the
// residual and 16-byte stores where the row allows them, element by element at the ragged edge.  (Going
// through shared memory to make a warp's accesses run along rows was measured: twice as slow, the scalar
// instructions cost more than the scattered vectors.)
// The residual of a piece, fetched ahead of the accumulator it will be added to (it does not depend on the
// MMAs): 32 floats of the thread's row, valid only where the vector path applies.
struct ResidualAhead {
  float4 v[8];
  bool have;
};
__device__ __forceinline__ void fetch_residual(ResidualAhead& ra, const float* residual, int ldo, int row, int col0, int M,
                                               int N, int vec_ok) {
  ra.have = residual != nullptr && vec_ok && row < M && col0 + 32 <= N;
  if (ra.have) {
    const float4* p = reinterpret_cast<const float4*>(residual + (size_t)row * ldo + col0);
#pragma unroll
    for (int i = 0; i < 8; ++i) ra.v[i] = p[i];
  }
}

template <int EPI, typename TOut>
__device__ __forceinline__ void epilogue_piece(const uint32_t* r, const uint32_t* r2, TOut* out, int ldo,
                                               const float* residual, int row, int col0, int M, int N, int vec_ok,
                                               const ResidualAhead* ahead = nullptr) {
  if (row >= M) return;
  const size_t base = (size_t)row * ldo + col0;
  const bool full = vec_ok && (col0 + 32 <= N);
#pragma unroll
  for (int j0 = 0; j0 < 32; j0 += 8) {
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float acc = __uint_as_float(r[j0 + j]);
      if (EPI == TC_EPI_SWIGLU) v[j] = silu_tc(acc) * __uint_as_float(r2[j0 + j]);
      else v[j] = acc;
    }
    if (full) {
      if (EPI == TC_EPI_RESIDUAL) {
        const bool pre = ahead != nullptr && ahead->have;
        const float4 a = pre ? ahead->v[j0 / 4] : *reinterpret_cast<const float4*>(residual + base + j0);
        const float4 b = pre ? ahead->v[j0 / 4 + 1] : *reinterpret_cast<const float4*>(residual + base + j0 + 4);
        v[0] += a.x; v[1] += a.y; v[2] += a.z; v[3] += a.w;
        v[4] += b.x; v[5] += b.y; v[6] += b.z; v[7] += b.w;
      }
      OutVec<TOut>::store8(out + base + j0, v);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (col0 + j0 + j < N) {
          float x = v[j];
          if (EPI == TC_EPI_RESIDUAL) x += residual[base + j0 + j];
          out[base + j0 + j] = from_f32<TOut>(x);
        }
      }
    }
  }
}

// What a row of the rotation epilogue needs besides the sums, fetched while the sums are still being made: the token's
// position, its page (tiles that hold key or value heads), and, at head size 64, the position's row of the rotation
// table in registers (the same for every head of the tile).
struct RopeRow {
  int pos;    // -1: the row takes no part (beyond M, or a position or page out of range, which is reported)
  int page;
  bool have_table;
  float c[32], s[32];
};
__device__ __forceinline__ void rope_row_fetch(RopeRow& rr, const RopeAppend& ra, int row, int M, bool with_page, int* err) {
  rr.pos = rr.page = -1;
  rr.have_table = false;
  if (row >= M) return;
  const int pos = ra.tok_pos[row];
  if (pos < 0 || pos >= ra.max_pos) {
    atomicOr(err, ERR_POSITION_RANGE);
    return;
  }
  if (with_page) {
    const int page = ra.page_table[(size_t)ra.seq_slot[ra.tok_seq[row]] * ra.table_stride + pos / PAGE];
    if (page < 0 || page >= ra.n_pages) {
      atomicOr(err, ERR_PAGE_RANGE);
      return;
    }
    rr.page = page;
  }
  rr.pos = pos;
  if (ra.hd == 64) {
    const float4* c = reinterpret_cast<const float4*>(ra.cos_t + (size_t)pos * 32);
    const float4* sn = reinterpret_cast<const float4*>(ra.sin_t + (size_t)pos * 32);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float4 cv = c[i], sv = sn[i];
      rr.c[4 * i] = cv.x; rr.c[4 * i + 1] = cv.y; rr.c[4 * i + 2] = cv.z; rr.c[4 * i + 3] = cv.w;
      rr.s[4 * i] = sv.x; rr.s[4 * i + 1] = sv.y; rr.s[4 * i + 2] = sv.z; rr.s[4 * i + 3] = sv.w;
    }
    rr.have_table = true;
  }
}

// 32 columns of a head's first half (`lo`, the head's dims d0 .. d0 + 31) and their partners in its second half (`hi`)
// of one token's row.  The sums are rounded to bfloat16 first and rotated then, eight pairs at a time with the
// arithmetic of the separate rotation kernel: a token's cache rows are the same bits whichever way they were made.
__device__ __forceinline__ void epilogue_rope_piece(const uint32_t* lo, const uint32_t* hi, const RopeAppend& ra, const RopeRow& rr,
                                                    __nv_bfloat16* out, int ldo, int row, int head, int d0) {
  if (rr.pos < 0) return;
  const int half = ra.hd >> 1;
  __nv_bfloat16* dst;
  if (head < ra.nh) {
    dst = out + (size_t)row * ldo + (size_t)head * ra.hd;
  } else {
    const bool is_k = head < ra.nh + ra.nkv;
    const int kvh = is_k ? head - ra.nh : head - ra.nh - ra.nkv;
    dst = (is_k ? ra.kcache : ra.vcache) + (((size_t)rr.page * ra.nkv + kvh) * PAGE + rr.pos % PAGE) * ra.hd;
  }
  const bool rotate = head < ra.nh + ra.nkv;
  const float* c = ra.cos_t + (size_t)rr.pos * half;
  const float* sn = ra.sin_t + (size_t)rr.pos * half;
#pragma unroll
  for (int j0 = 0; j0 < 32; j0 += 8) {
    uint4 a, b;
    a.x = dm_pack(__uint_as_float(lo[j0]), __uint_as_float(lo[j0 + 1]));
    a.y = dm_pack(__uint_as_float(lo[j0 + 2]), __uint_as_float(lo[j0 + 3]));
    a.z = dm_pack(__uint_as_float(lo[j0 + 4]), __uint_as_float(lo[j0 + 5]));
    a.w = dm_pack(__uint_as_float(lo[j0 + 6]), __uint_as_float(lo[j0 + 7]));
    b.x = dm_pack(__uint_as_float(hi[j0]), __uint_as_float(hi[j0 + 1]));
    b.y = dm_pack(__uint_as_float(hi[j0 + 2]), __uint_as_float(hi[j0 + 3]));
    b.z = dm_pack(__uint_as_float(hi[j0 + 4]), __uint_as_float(hi[j0 + 5]));
    b.w = dm_pack(__uint_as_float(hi[j0 + 6]), __uint_as_float(hi[j0 + 7]));
    if (rotate) {
      if (rr.have_table) dm_rotate8_vals(a, b, rr.c + j0, rr.s + j0);   // (head size 64: d0 is 0)
      else dm_rotate8(a, b, c, sn, d0 + j0);
    }
    *reinterpret_cast<uint4*>(dst + d0 + j0) = a;
    *reinterpret_cast<uint4*>(dst + half + d0 + j0) = b;
  }
}

// All heads of a tile of BN columns (a multiple of the head size) for the rows of one epilogue warp.
template <int BN>
__device__ __forceinline__ void epilogue_rope_tile(uint32_t taddr, const RopeAppend& ra, const RopeRow& rr, __nv_bfloat16* out,
                                                   int ldo, int row, int n0, int N) {
  const int hd = ra.hd, half = hd >> 1;
#pragma unroll 1
  for (int h0 = 0; h0 < BN; h0 += hd) {
    if (n0 + h0 >= N) break;   // uniform over the block
#pragma unroll 1
    for (int d0 = 0; d0 < half; d0 += 32) {
      uint32_t lo[32], hi[32];
      tmem_ld32(taddr + (uint32_t)(h0 + d0), lo);
      tmem_ld32(taddr + (uint32_t)(h0 + half + d0), hi);
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      epilogue_rope_piece(lo, hi, ra, rr, out, ldo, row, (n0 + h0) / hd, d0);
    }
  }
}

template <int BN, int EPI, typename TOut, int STAGES>
__global__ void __launch_bounds__(TC_THREADS)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               const __grid_constant__ CUtensorMap map_b2, TOut* out, int ldo, const float* residual,
               int M, int N, int K, int vec_ok, int* err, int k_splits, float* partial, const RopeAppend rope) {
  // k_splits > 1: block z of the grid accumulates its share of K only and leaves the raw sums in
  // `partial` [split][weight][M][N] (float32); splitk_reduce_kernel adds the splits in their order and
  // applies the epilogue.  For products of few tiles and long K (decoding 17 to 128 sequences), which
  // would otherwise run on a handful of SMs.
  constexpr int NB = EPI == TC_EPI_SWIGLU ? 2 : 1;
  constexpr int A_BYTES = TC_BM * TC_BK * 2, B_BYTES = BN * TC_BK * 2;
  constexpr int STAGE_BYTES = A_BYTES + NB * B_BYTES;
  constexpr uint32_t TMEM_COLS = NB * BN < 32 ? 32 : NB * BN;  // 64, 128 or 256: powers of two
  static_assert((TMEM_COLS & (TMEM_COLS - 1)) == 0 && TMEM_COLS <= 512, "tensor memory columns: a power of two");
  static_assert(STAGE_BYTES % 1024 == 0, "stages keep the 1024-byte alignment of swizzled tiles");

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + STAGES;
  uint64_t* tmem_full_bar = bars + 2 * STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.y * TC_BM, n0 = blockIdx.x * BN;
  const int n_k_all = (K + TC_BK - 1) / TC_BK;
  const int k_per = (n_k_all + k_splits - 1) / k_splits;
  const int k_first = blockIdx.z * k_per;
  const int n_k = max(0, min(n_k_all, k_first + k_per) - k_first);   // (the host picks splits that all get a share)

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    mbar_init(smem_u32(tmem_full_bar), 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  // The weights' tiles of the first ring of stages are requested ahead of the wait for the kernel before this one
  // (nothing on the stream writes weights): when that kernel is done, only the rows of `a` are still to come.
  const int n_ahead = n_k < STAGES ? n_k : STAGES;
  if (warp == 0 && elect_one()) {
    for (int i = 0; i < n_ahead; ++i) {
      const uint32_t bar = smem_u32(&full_bar[i]);
      const uint32_t sa = smem_u32(smem + i * STAGE_BYTES);
      const int x = (k_first + i) * TC_BK;
      mbar_expect_tx(bar, STAGE_BYTES);
      tma_load_2d(sa + A_BYTES, &map_b, bar, x, n0);
      if (NB == 2) tma_load_2d(sa + A_BYTES + B_BYTES, &map_b2, bar, x, n0);
    }
  }
  __syncwarp();
  pdl_launch_dependents();
  pdl_wait();   // (launched as a programmatic dependent: up to here nothing of the kernel before this one was read)
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  // The two role warps walk their loops whole and wait as warps; one elected lane of each issues.  (With the loop
  // inside `if (lane == 0)` the descriptors and coordinates are computed in a divergent region, out of reach of the
  // uniform datapath that the instructions take them from: an MMA then took some 120 clocks to issue, twice what a
  // 128 x 128 x 16 one runs.)
  if (warp == 0) {
    const bool leader = elect_one();
    for (int i = 0; i < n_k; ++i) {
      const int s = i % STAGES;
      if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&empty_bar[s]), ((i / STAGES) & 1) ^ 1, abort_flag, err))) break;
      const uint32_t bar = smem_u32(&full_bar[s]);
      const uint32_t sa = smem_u32(smem + s * STAGE_BYTES);
      const int x = (k_first + i) * TC_BK;
      if (leader) {
        if (i < n_ahead) {   // (the stage's barrier is armed and its weights are on their way)
          tma_load_2d(sa, &map_a, bar, x, m0);
        } else {
          mbar_expect_tx(bar, STAGE_BYTES);
          tma_load_2d(sa, &map_a, bar, x, m0);
          tma_load_2d(sa + A_BYTES, &map_b, bar, x, n0);
          if (NB == 2) tma_load_2d(sa + A_BYTES + B_BYTES, &map_b2, bar, x, n0);
        }
      }
      __syncwarp();
    }
  } else if (warp == 1) {
    constexpr uint32_t idesc = umma_idesc(TC_BM, BN);
    const bool leader = elect_one();
    bool ok = true;
    for (int i = 0; i < n_k && ok; ++i) {
      const int s = i % STAGES;
      ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&full_bar[s]), (i / STAGES) & 1, abort_flag, err));
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t sa = smem_u32(smem + s * STAGE_BYTES);
      const uint64_t da = umma_desc(sa), db = umma_desc(sa + A_BYTES), db2 = umma_desc(sa + A_BYTES + B_BYTES);
      const uint32_t bar_e = smem_u32(&empty_bar[s]);
      if (leader) {
#pragma unroll
        for (int k = 0; k < TC_BK / 16; ++k) {  // 16 bfloat16 = 32 bytes = 2 descriptor address units per step
          const uint32_t acc = (i | k) != 0;
          umma_f16(tmem_base, da + 2 * k, db + 2 * k, idesc, acc);
          if (NB == 2) umma_f16(tmem_base + BN, da + 2 * k, db2 + 2 * k, idesc, acc);
        }
        umma_commit(bar_e);  // arrives when these MMAs have read the stage
      }
      __syncwarp();
    }
    if (ok && leader) umma_commit(smem_u32(tmem_full_bar));
  } else {
    const int q = warp & 3;  // a warp reads the 32 lanes of tensor memory that its index modulo 4 selects
    ResidualAhead ra[2];
    ra[0].have = ra[1].have = false;
    if (EPI == TC_EPI_RESIDUAL && k_splits == 1) fetch_residual(ra[0], residual, ldo, m0 + q * 32 + lane, n0, M, N, vec_ok);  // while the MMAs run
    RopeRow rr;
    if constexpr (EPI == TC_EPI_ROPE) rope_row_fetch(rr, rope, m0 + q * 32 + lane, M, n0 + BN > rope.nh * rope.hd, err);   // likewise
    const bool ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(tmem_full_bar), 0, abort_flag, err));  // one decision per warp
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (ok && EPI == TC_EPI_ROPE) {
      if constexpr (EPI == TC_EPI_ROPE)
        epilogue_rope_tile<BN>(tmem_base + ((uint32_t)(q * 32) << 16), rope, rr, out, ldo, m0 + q * 32 + lane, n0, N);
    } else if (ok) {
#pragma unroll
      for (int c0 = 0; c0 < BN; c0 += 32) {
        if (n0 + c0 >= N) break;  // uniform over the block
        uint32_t r[32], r2[32];
        const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)c0;
        tmem_ld32(taddr, r);
        if (NB == 2) tmem_ld32(taddr + BN, r2);
        if (EPI == TC_EPI_RESIDUAL && k_splits == 1 && c0 + 32 < BN)   // the next piece's residual is on its way while this one is finished
          fetch_residual(ra[((c0 >> 5) + 1) & 1], residual, ldo, m0 + q * 32 + lane, n0 + c0 + 32, M, N, vec_ok);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (k_splits > 1) {   // raw sums of this share of K
          const int row = m0 + q * 32 + lane;
          if (row < M) {
#pragma unroll
            for (int b = 0; b < NB; ++b) {
              float* dst = partial + (((size_t)blockIdx.z * NB + b) * M + row) * N + n0 + c0;
              const uint32_t* src = b == 0 ? r : r2;
              if (n0 + c0 + 32 <= N && N % 4 == 0) {
#pragma unroll
                for (int j = 0; j < 32; j += 4)
                  *reinterpret_cast<float4*>(dst + j) = make_float4(__uint_as_float(src[j]), __uint_as_float(src[j + 1]), __uint_as_float(src[j + 2]), __uint_as_float(src[j + 3]));
              } else {
#pragma unroll
                for (int j = 0; j < 32; ++j)
                  if (n0 + c0 + j < N) dst[j] = __uint_as_float(src[j]);
              }
            }
          }
          continue;
        }
        epilogue_piece<EPI, TOut>(r, r2, out, ldo, residual, m0 + q * 32 + lane, n0 + c0, M, N, vec_ok, &ra[(c0 >> 5) & 1]);
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// out = epilogue(sum over the splits, in their order, of the raw sums a split-K launch left).
template <int EPI, typename TOut>
__global__ void splitk_reduce_kernel(const float* __restrict__ partial, int splits, TOut* out, int ldo, const float* residual,
                                     int M, int N) {
  constexpr int NB = EPI == TC_EPI_SWIGLU ? 2 : 1;
  const size_t plane = (size_t)M * N;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < plane; i += (size_t)gridDim.x * blockDim.x) {
    float a = 0.f, b = 0.f;
    for (int z = 0; z < splits; ++z) {
      a += partial[(size_t)z * NB * plane + i];
      if (NB == 2) b += partial[((size_t)z * NB + 1) * plane + i];
    }
    const int m = (int)(i / N), n = (int)(i - (size_t)m * N);
    const size_t o = (size_t)m * ldo + n;
    if (EPI == TC_EPI_SWIGLU) out[o] = from_f32<TOut>(silu_tc(a) * b);
    else if (EPI == TC_EPI_RESIDUAL) out[o] = from_f32<TOut>(residual[o] + a);
    else out[o] = from_f32<TOut>(a);
  }
}

// ------------------------------------------------------------------------- persistent form
// One CTA per SM walks the tiles tile = blockIdx.x, blockIdx.x + gridDim.x, ... (row tiles fastest, so
// that the CTAs running together share the weight tiles in L2).  The shared-memory ring runs on across
// tiles, and the accumulator has two stages in tensor memory: while the epilogue warps drain tile i
// (tcgen05.ld, epilogue, stores) the MMA warp already accumulates tile i + 1 into the other stage.
// Barriers: full/empty per ring stage as above, tmem_full/tmem_empty per accumulator stage (the
// epilogue's four warps each arrive once on tmem_empty when their rows are read).
constexpr int TCP_STAGES = 4;

template <int BN, int EPI, typename TOut>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tc_persistent_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                          const __grid_constant__ CUtensorMap map_b2, TOut* out, int ldo, const float* residual,
                          int M, int N, int K, int vec_ok, int* err, const RopeAppend rope) {
  constexpr int NB = EPI == TC_EPI_SWIGLU ? 2 : 1;
  constexpr int A_BYTES = TC_BM * TC_BK * 2, B_BYTES = BN * TC_BK * 2;
  constexpr int STAGE_BYTES = A_BYTES + NB * B_BYTES;
  constexpr uint32_t ACC_COLS = NB * BN;          // columns of one accumulator stage
  constexpr uint32_t TMEM_COLS = 2 * ACC_COLS;    // two stages: 256
  static_assert((TMEM_COLS & (TMEM_COLS - 1)) == 0 && TMEM_COLS <= 512, "tensor memory columns: a power of two");
  static_assert(STAGE_BYTES % 1024 == 0, "stages keep the 1024-byte alignment of swizzled tiles");

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + TCP_STAGES * STAGE_BYTES);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + TCP_STAGES;
  uint64_t* tmem_full_bar = bars + 2 * TCP_STAGES;       // [2]
  uint64_t* tmem_empty_bar = bars + 2 * TCP_STAGES + 2;  // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * TCP_STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (M + TC_BM - 1) / TC_BM, tiles_n = (N + BN - 1) / BN;
  const int n_tiles = tiles_m * tiles_n;
  const int n_k = (K + TC_BK - 1) / TC_BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < TCP_STAGES; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&tmem_full_bar[a]), 1);
      mbar_init(smem_u32(&tmem_empty_bar[a]), 4);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  pdl_launch_dependents();   // (after the allocation: a dependent that allocates too then finds every block of this grid served)
  pdl_wait();                // (launched as a programmatic dependent: up to here nothing of the kernel before this one was read)
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  // (the role warps walk their loops whole, one elected lane issues: see the one-tile kernel)
  if (warp == 0) {
    const bool leader = elect_one();
    int it = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
      const int m0 = (tile % tiles_m) * TC_BM, n0 = (tile / tiles_m) * BN;
      for (int i = 0; i < n_k; ++i, ++it) {
        const int s = it % TCP_STAGES;
        ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&empty_bar[s]), ((it / TCP_STAGES) & 1) ^ 1, abort_flag, err));
        if (!ok) break;
        const uint32_t bar = smem_u32(&full_bar[s]);
        const uint32_t sa = smem_u32(smem + s * STAGE_BYTES);
        if (leader) {
          mbar_expect_tx(bar, STAGE_BYTES);
          tma_load_2d(sa, &map_a, bar, i * TC_BK, m0);
          tma_load_2d(sa + A_BYTES, &map_b, bar, i * TC_BK, n0);
          if (NB == 2) tma_load_2d(sa + A_BYTES + B_BYTES, &map_b2, bar, i * TC_BK, n0);
        }
        __syncwarp();
      }
    }
  } else if (warp == 1) {
    constexpr uint32_t idesc = umma_idesc(TC_BM, BN);
    const bool leader = elect_one();
    int it = 0, ti = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++ti) {
      const int as = ti & 1;
      ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&tmem_empty_bar[as]), ((ti >> 1) & 1) ^ 1, abort_flag, err));  // the epilogue has drained this stage
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t acc_addr = tmem_base + (uint32_t)as * ACC_COLS;
      for (int i = 0; i < n_k; ++i, ++it) {
        const int s = it % TCP_STAGES;
        ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&full_bar[s]), (it / TCP_STAGES) & 1, abort_flag, err));
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t sa = smem_u32(smem + s * STAGE_BYTES);
        const uint64_t da = umma_desc(sa), db = umma_desc(sa + A_BYTES), db2 = umma_desc(sa + A_BYTES + B_BYTES);
        const uint32_t bar_e = smem_u32(&empty_bar[s]);
        if (leader) {
#pragma unroll
          for (int k = 0; k < TC_BK / 16; ++k) {
            const uint32_t acc = (i | k) != 0;
            umma_f16(acc_addr, da + 2 * k, db + 2 * k, idesc, acc);
            if (NB == 2) umma_f16(acc_addr + BN, da + 2 * k, db2 + 2 * k, idesc, acc);
          }
          umma_commit(bar_e);
        }
        __syncwarp();
      }
      if (ok && leader) umma_commit(smem_u32(&tmem_full_bar[as]));
    }
  } else {
    const int q = warp & 3;
    int ti = 0;
    for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++ti) {
      const int as = ti & 1;
      const int m0 = (tile % tiles_m) * TC_BM, n0 = (tile / tiles_m) * BN;
      RopeRow rr;
      if constexpr (EPI == TC_EPI_ROPE) rope_row_fetch(rr, rope, m0 + q * 32 + lane, M, n0 + BN > rope.nh * rope.hd, err);   // while the MMAs run
      const bool ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&tmem_full_bar[as]), (ti >> 1) & 1, abort_flag, err));
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      if (!ok) break;
      const uint32_t acc_addr = tmem_base + (uint32_t)as * ACC_COLS + ((uint32_t)(q * 32) << 16);
      if constexpr (EPI == TC_EPI_ROPE) {
        epilogue_rope_tile<BN>(acc_addr, rope, rr, out, ldo, m0 + q * 32 + lane, n0, N);
      } else {
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 32) {
          if (n0 + c0 >= N) break;
          uint32_t r[32], r2[32];
          tmem_ld32(acc_addr + (uint32_t)c0, r);
          if (NB == 2) tmem_ld32(acc_addr + (uint32_t)c0 + BN, r2);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
          epilogue_piece<EPI, TOut>(r, r2, out, ldo, residual, m0 + q * 32 + lane, n0 + c0, M, N, vec_ok);
        }
      }
      // this warp's rows of the stage are in registers or stored: hand the stage back to the MMA warp
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&tmem_empty_bar[as])) : "memory");
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// ------------------------------------------------------------------------- host side
// Which kernel runs a product: by default (auto) wide outputs with a long K go to the persistent kernel with
// 128 x 256 tiles and two accumulator stages (1.10 to 1.16 PFLOP/s at 2048 x 8192 x 2048 against 0.88 to 0.91
// of the other), everything else to the one-tile-per-CTA kernel with 128 x 128 tiles, two CTAs per SM (the
// persistent kernel with narrow tiles starves on shared-memory bandwidth: 0.68 to 0.78).  Forced for comparisons.
static int g_tc_auto = 1, g_tc_persistent = 1, g_tc_wide = 1, g_tc_narrow = 1, g_tc_deep = 1, g_tc_tiny = 1;

// Scratch for split-K launches (set by the caller once; nothing is allocated here): without it no product is split.
static float* g_splitk_ws = nullptr;
static size_t g_splitk_bytes = 0;
static int g_splitk_on = 1;
static int g_last_launches = 1;   // kernels the last edgelm_gemm_tc call launched (2 when it split K)
// Which kernel the last edgelm_gemm_tc call took: tile columns | persistent << 12 | deep ring << 13 | K splits << 16.
// Tests read it so that a product meant for one kernel cannot pass on another.
static int g_last_kernel = 0;

// Splits of K for a product of `tiles` one-tile blocks and `n_k` K blocks of 64: none unless the tiles would leave
// more than half of the SMs idle and K is at least 1,024 (below that the second kernel costs more than the idle
// SMs: measured at 64 rows, N 960, K 576: 6.1 us whole against 7.7 us split); then enough splits for about one and
// a half blocks an SM, at least four K blocks each, within the scratch.  Measured at 64 rows: N 2048, K 8192:
// 60.9 -> 15.5 us; N 2048, K 2048: 16.9 -> 8.5 us; N 576, K 1536: 12.9 -> 9.2 us.
static int splitk_for(int tiles, int n_k, size_t bytes_per_split) {
  if (!g_splitk_on || g_splitk_ws == nullptr || tiles >= 74 || n_k < 16) return 1;
  int s = (222 + tiles - 1) / tiles;
  if (s > n_k / 4) s = n_k / 4;
  while (s > 1 && (size_t)s * bytes_per_split > g_splitk_bytes) --s;
  if (s < 2) return 1;
  const int k_per = (n_k + s - 1) / s;
  return (n_k + k_per - 1) / k_per;   // every split gets a share
}

template <int BN, int EPI, typename TOut>
static int launch_tc(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mb2, void* out, int ldo,
                     const float* residual, int M, int N, int K, int vec_ok, int* err, cudaStream_t stream, bool persistent,
                     const RopeAppend& rope) {
  constexpr int NB = EPI == TC_EPI_SWIGLU ? 2 : 1;
  if (persistent) {
    constexpr int smem = TCP_STAGES * (TC_BM * TC_BK * 2 + NB * BN * TC_BK * 2) + 1024 + 256;
    auto kern = gemm_tc_persistent_kernel<BN, EPI, TOut>;
    static bool configured = false;
    static int n_sms = 0;
    if (!configured) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
      if (e != cudaSuccess) {
        set_error("gemm_tc: %d bytes of shared memory refused: %s", smem, cudaGetErrorString(e));
        return -2;
      }
      int dev = 0;
      cudaGetDevice(&dev);
      cudaDeviceGetAttribute(&n_sms, cudaDevAttrMultiProcessorCount, dev);
      if (n_sms <= 0) n_sms = 148;
      configured = true;
    }
    const int tiles = ((N + BN - 1) / BN) * ((M + TC_BM - 1) / TC_BM);
    const int grid = tiles < n_sms ? tiles : n_sms;
    g_last_launches = 1;
    g_last_kernel = BN | (1 << 12) | (1 << 16);
    cudaError_t le = launch_pdl(32, kern, dim3(grid), dim3(TC_THREADS), (size_t)smem, stream, ma, mb, mb2, (TOut*)out, ldo, residual, M, N, K,
                                vec_ok, err, rope);
    if (le != cudaSuccess) {
      set_error("gemm_tc: launch failed: %s", cudaGetErrorString(le));
      return -2;
    }
    return 0;
  }
  constexpr int STAGE_BYTES = TC_BM * TC_BK * 2 + NB * BN * TC_BK * 2;
  constexpr int DEEP = TC_DEEP_BYTES / STAGE_BYTES;   // 6 stages of 32 KB, 8 of 24 KB
  dim3 grid((N + BN - 1) / BN, (M + TC_BM - 1) / TC_BM);
  // (the rotation epilogue is not one the reduce kernel of split products knows: such a product stays whole)
  const int splits = EPI == TC_EPI_ROPE ? 1 : splitk_for((int)(grid.x * grid.y), (K + TC_BK - 1) / TC_BK, (size_t)NB * M * N * sizeof(float));
  grid.z = splits;
  g_last_launches = splits > 1 ? 2 : 1;
  // a grid of at most one block an SM has the shared memory to itself: a deeper ring hides more of the loads' latency
  // (a short K is a few loads behind one another: 9 of them at K 576)
  static int n_sms = 0;
  if (n_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n_sms, cudaDevAttrMultiProcessorCount, dev);
  }
  const bool deep = g_tc_deep && (long long)grid.x * grid.y * grid.z <= n_sms;
  g_last_kernel = BN | ((deep ? 1 : 0) << 13) | (splits << 16);
  auto go = [&](auto kern, int smem) -> int {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) {
      set_error("gemm_tc: %d bytes of shared memory refused: %s", smem, cudaGetErrorString(e));
      return -2;
    }
    cudaError_t le = launch_pdl(8, kern, grid, dim3(TC_THREADS), (size_t)smem, stream, ma, mb, mb2, (TOut*)out, ldo, residual, M, N, K,
                                vec_ok, err, splits, g_splitk_ws, rope);
    if (le != cudaSuccess) {
      set_error("gemm_tc: launch failed: %s", cudaGetErrorString(le));
      return -2;
    }
    return 0;
  };
  const int rc = deep ? go(gemm_tc_kernel<BN, EPI, TOut, DEEP>, DEEP * STAGE_BYTES + 1024 + 256)
                      : go(gemm_tc_kernel<BN, EPI, TOut, TC_STAGES>, TC_STAGES * STAGE_BYTES + 1024 + 256);
  if (rc) return rc;
  if (EPI != TC_EPI_ROPE && splits > 1) {
    const size_t plane = (size_t)M * N;
    const int blocks = (int)((plane + 255) / 256 < 1184 ? (plane + 255) / 256 : 1184);
    splitk_reduce_kernel<EPI, TOut><<<blocks, 256, 0, stream>>>(g_splitk_ws, splits, (TOut*)out, ldo, residual, M, N);
  }
  return 0;
}

}  // namespace edgelm

using namespace edgelm;

// Negative: choose per product (default).  Else bit 0: the persistent kernel; bit 1: narrow tiles only.
extern "C" int edgelm_gemm_tc_persistent(int on) {
  if (on < 0) {
    g_tc_auto = 1;
    return 0;
  }
  g_tc_auto = 0;
  g_tc_persistent = on & 1;
  g_tc_wide = (on >> 1) & 1 ? 0 : 1;   // bit 1 set: narrow tiles only
  return 0;
}

// Float32 scratch for split-K launches (raw sums of every split); the library only keeps the pointer.  bytes 0: none.
// `on` 0 switches splitting off (comparisons).
extern "C" int edgelm_gemm_tc_splitk(float* scratch, size_t bytes, int on) {
  g_splitk_ws = bytes ? scratch : nullptr;
  g_splitk_bytes = bytes;
  g_splitk_on = on;
  return 0;
}

// bit 0: 64-column tiles where they apply; bit 1: the deep ring for grids of at most one block an SM (comparisons)
// 1 (default): products whose rows are one tile and whose output is narrow run on tiles of 32 columns; 0: never.
extern "C" int edgelm_gemm_tc_tiny(int on) {
  g_tc_tiny = on & 1;
  return 0;
}

extern "C" int edgelm_gemm_tc_narrow(int on) {
  g_tc_narrow = on & 1;
  g_tc_deep = (on >> 1) & 1;
  return 0;
}

extern "C" int edgelm_gemm_tc_last_launches() { return g_last_launches; }
extern "C" int edgelm_gemm_tc_last_kernel() { return g_last_kernel; }

// 1 if the tensor-core kernel takes these operands (alignment and pitch rules of TMA), else 0.
extern "C" int edgelm_gemm_tc_takes(const void* a, int lda, const void* w, const void* w2, int K) {
  const bool ok = K > 0 && K % 8 == 0 && lda % 8 == 0 && (uintptr_t)a % 16 == 0 && (uintptr_t)w % 16 == 0 &&
                  (w2 == nullptr || (uintptr_t)w2 % 16 == 0);
  return ok ? 1 : 0;
}

static int gemm_tc_run(const void* a, int lda, const void* w, const void* w2, void* out, int ldo, const float* residual,
                       int M, int N, int K, int out_dtype, int epilogue, int* err, cudaStream_t stream, const RopeAppend& rope) {
  if (M == 0) return 0;
  EL_REFUSE(M > 0 && N > 0 && K > 0 && lda >= K && ldo >= N, "gemm_tc: bad sizes M=%d N=%d K=%d lda=%d ldo=%d", M, N, K, lda, ldo);
  EL_REFUSE(edgelm_gemm_tc_takes(a, lda, w, w2, K), "gemm_tc: K=%d and lda=%d must be multiples of 8 and the operands 16-byte aligned", K, lda);
  EL_REFUSE(epilogue != TC_EPI_SWIGLU || w2 != nullptr, "gemm_tc: SwiGLU needs the second weight");
  EL_REFUSE(epilogue != TC_EPI_RESIDUAL || (residual != nullptr && out_dtype == DT_F32), "gemm_tc: residual epilogue needs a float32 residual and output");
  EL_REFUSE(err != nullptr, "gemm_tc: needs the error word");
  EL_REFUSE((M + TC_BM - 1) / TC_BM <= 65535, "gemm_tc: too many rows (%d)", M);
  // wide tiles (128 x 256, or 2 x 128 for SwiGLU) when the output is wide enough to fill the device with
  // them: twice the multiply-adds per byte that comes through shared memory
  const long long wide_tiles = (long long)((M + TC_BM - 1) / TC_BM) * ((N + (epilogue == TC_EPI_SWIGLU ? 127 : 255)) / (epilogue == TC_EPI_SWIGLU ? 128 : 256));
  const bool wide = g_tc_auto ? (wide_tiles >= 120 && N >= 1024 && K >= 1024) : (g_tc_wide && wide_tiles >= 120 && N >= 1024);
  // (with a residual the wide tiles go one to a block: measured at 2,048 rows, N 2048: K 8192 65.9 -> 60.0 us, K 2048
  // 25.3 -> 24.0 us; persistent 69.0 and 31.3 us)
  const bool persistent = g_tc_auto ? (wide && epilogue != TC_EPI_RESIDUAL) : g_tc_persistent != 0;
  // tiles of 64 columns for a single weight when 128-column tiles would not fill one wave of SMs and there are
  // several row tiles to share a weight tile in L2 (measured at 2,048 rows: N 576, K 576: 11.6 -> 8.8 us; N 576,
  // K 1536: 16.1 -> 13.5 us; with 256 tiles of 128 columns and K 8192 the narrow tiles lose: 68 -> 107 us)
  const long long tiles128 = (long long)((M + TC_BM - 1) / TC_BM) * ((N + 127) / 128);
  const bool narrow = !wide && epilogue != TC_EPI_SWIGLU && g_tc_narrow && tiles128 < 148 && M > TC_BM &&
                      (epilogue != TC_EPI_ROPE || rope.hd == 64);   // (a tile holds whole heads)
  // tiles of 32 columns when all rows are one tile (decode steps of 17 to 128 sequences) and the weights are small
  // (under 4 Mi elements): they then stream through four times as many SMs, and an epilogue thread has one piece of
  // 32 columns, whose residual it fetched ahead, instead of four one after the other (64 rows: N 576, K 576 7.3 ->
  // 4.5 us; N 576, K 1536 8.6 -> 6.5; N 960, K 2560 8.1 -> 6.9).  Every block reads all rows of `a`, so with large
  // weights the narrow tiles lose (N 2048, K 2048 7.5 -> 8.5 us; K 8192 14.5 -> 17.8).
  const bool tiny = !wide && M <= TC_BM && (long long)N * K < (4LL << 20) && epilogue != TC_EPI_ROPE && g_tc_tiny;
  const int bn = tiny ? 32 : epilogue == TC_EPI_SWIGLU ? (wide ? 128 : 64) : (wide ? 256 : (narrow ? 64 : 128));
  CUtensorMap ma, mb, mb2;
  if (tensor_map(a, M, K, lda, TC_BM, &ma)) return -1;
  if (tensor_map(w, N, K, K, bn, &mb)) return -1;
  mb2 = mb;
  if (w2 && tensor_map(w2, N, K, K, bn, &mb2)) return -1;
  const size_t esz = out_dtype == DT_F32 ? 4 : 2;
  const int vec_ok = ((uintptr_t)out % 16 == 0) && ((size_t)ldo * esz % 16 == 0) &&
                     (residual == nullptr || (uintptr_t)residual % 16 == 0);
  int rc = 0;
  if (wide) {
    if (epilogue == TC_EPI_STORE && out_dtype == DT_BF16)
      rc = launch_tc<256, TC_EPI_STORE, __nv_bfloat16>(ma, mb, mb2, out, ldo, residual, M, N, K, vec_ok, err, stream, persistent, rope);
    else if (epilogue == TC_EPI_STORE && out_dtype == DT_F32)
      rc = launch_tc<256, TC_EPI_STORE, float>(ma, mb, mb2, out, ldo, residual, M, N, K, vec_ok, err, stream, persistent, rope);
    else if (epilogue == TC_EPI_RESIDUAL)
      rc = launch_tc<256, TC_EPI_RESIDUAL, float>(ma, mb, mb2, out, ldo, residual, M, N, K, vec_ok, err, stream, persistent, rope);
    else if (epilogue == TC_EPI_SWIGLU && out_dtype == DT_BF16)
      rc = launch_tc<128, TC_EPI_SWIGLU, __nv_bfloat16>(ma, mb, mb2, out, ldo, residual, M, N, K, vec_ok, err, stream, persistent, rope);
    else if (epilogue == TC_EPI_ROPE && out_dtype == DT_BF16)
      rc = launch_tc<256, TC_EPI_ROPE, __nv_bfloat16>(ma, mb, mb2, out, ldo, residual, M, N, K, vec_ok, err, stream, persistent, rope);
    else
      EL_REFUSE(false, "gemm_tc: unsupported epilogue %d with output dtype %d", epilogue, out_dtype);
  } else if (tiny && epilogue == TC_EPI_STORE && out_dtype == DT_BF16)
    rc = launch_tc<32, TC_EPI_STORE, __nv_bfloat16>(ma, mb, mb2, out, ldo, residual, M, N, K, vec_ok, err, stream, persistent, rope);
  else if (tiny && epilogue == TC_EPI_STORE && out_dtype == DT_F32)
    rc = launch_tc<32, TC_EPI_STORE, float>(ma, mb, mb2, out, ldo, residual, M, N, K, vec_ok, err, stream, persistent, rope);
  else if (tiny && epilogue == TC_EPI_RESIDUAL)
    rc = launch_tc<32, TC_EPI_RESIDUAL, float>(ma, mb, mb2, out, ldo, residual, M, N, K, vec_ok, err, stream, persistent, rope);
  else if (tiny && epilogue == TC_EPI_SWIGLU && out_dtype == DT_BF16)
    rc = launch_tc<32, TC_EPI_SWIGLU, __nv_bfloat16>(ma, mb, mb2, out, ldo, residual, M, N, K, vec_ok, err, stream, persistent, rope);
  else if (narrow && epilogue == TC_EPI_ROPE && out_dtype == DT_BF16)
    rc = launch_tc<64, TC_EPI_ROPE, __nv_bfloat16>(ma, mb, mb2, out, ldo, residual, M, N, K, vec_ok, err, stream, persistent, rope);
  else if (epilogue == TC_EPI_ROPE && out_dtype == DT_BF16)
    rc = launch_tc<128, TC_EPI_ROPE, __nv_bfloat16>(ma, mb, mb2, out, ldo, residual, M, N, K, vec_ok, err, stream, persistent, rope);
  else if (narrow && epilogue == TC_EPI_STORE && out_dtype == DT_BF16)
    rc = launch_tc<64, TC_EPI_STORE, __nv_bfloat16>(ma, mb, mb2, out, ldo, residual, M, N, K, vec_ok, err, stream, persistent, rope);
  else if (narrow && epilogue == TC_EPI_STORE && out_dtype == DT_F32)
    rc = launch_tc<64, TC_EPI_STORE, float>(ma, mb, mb2, out, ldo, residual, M, N, K, vec_ok, err, stream, persistent, rope);
  else if (narrow && epilogue == TC_EPI_RESIDUAL)
    rc = launch_tc<64, TC_EPI_RESIDUAL, float>(ma, mb, mb2, out, ldo, residual, M, N, K, vec_ok, err, stream, persistent, rope);
  else if (epilogue == TC_EPI_STORE && out_dtype == DT_BF16)
    rc = launch_tc<128, TC_EPI_STORE, __nv_bfloat16>(ma, mb, mb2, out, ldo, residual, M, N, K, vec_ok, err, stream, persistent, rope);
  else if (epilogue == TC_EPI_STORE && out_dtype == DT_F32)
    rc = launch_tc<128, TC_EPI_STORE, float>(ma, mb, mb2, out, ldo, residual, M, N, K, vec_ok, err, stream, persistent, rope);
  else if (epilogue == TC_EPI_RESIDUAL)
    rc = launch_tc<128, TC_EPI_RESIDUAL, float>(ma, mb, mb2, out, ldo, residual, M, N, K, vec_ok, err, stream, persistent, rope);
  else if (epilogue == TC_EPI_SWIGLU && out_dtype == DT_BF16)
    rc = launch_tc<64, TC_EPI_SWIGLU, __nv_bfloat16>(ma, mb, mb2, out, ldo, residual, M, N, K, vec_ok, err, stream, persistent, rope);
  else
    EL_REFUSE(false, "gemm_tc: unsupported epilogue %d with output dtype %d", epilogue, out_dtype);
  if (rc) return rc;
  EL_LAUNCH_CHECK("gemm_tc");
  return 0;
}

extern "C" int edgelm_gemm_tc(const void* a, int lda, const void* w, const void* w2, void* out, int ldo,
                              const float* residual, int M, int N, int K, int out_dtype, int epilogue, int* err,
                              cudaStream_t stream) {
  EL_REFUSE(epilogue >= TC_EPI_STORE && epilogue <= TC_EPI_SWIGLU, "gemm_tc: unknown epilogue %d", epilogue);
  return gemm_tc_run(a, lda, w, w2, out, ldo, residual, M, N, K, out_dtype, epilogue, err, stream, RopeAppend{});
}

// 1 if the stacked q, k, v projection of a prompt step can rotate and append in its epilogue: bfloat16, head size 64
// or 128, and the alignments that its 16-byte stores and table reads need.
extern "C" int edgelm_gemm_tc_rope_takes(const void* a, int lda, const void* w, const void* qkv, int ldo, int K, int hd,
                                         const void* kcache, const void* vcache, const void* cos_t, const void* sin_t) {
  const bool ok = edgelm_gemm_tc_takes(a, lda, w, nullptr, K) && (hd == 64 || hd == 128) && (uintptr_t)qkv % 16 == 0 && ldo % 8 == 0 &&
                  (uintptr_t)kcache % 16 == 0 && (uintptr_t)vcache % 16 == 0 && (uintptr_t)cos_t % 16 == 0 && (uintptr_t)sin_t % 16 == 0;
  return ok ? 1 : 0;
}

// qkv[:, :nh * hd] = rotate(a . W^T) for the query heads; the rotated keys and the values go into the cache pages of
// each token's sequence and position (and nowhere else).  W [(nh + 2 nkv) hd, K] is the three weights stacked.
extern "C" int edgelm_gemm_tc_rope(const void* a, int lda, const void* w, void* qkv, int ldo, int M, int K,
                                   const int32_t* tok_pos, const int32_t* tok_seq, const int32_t* seq_slot,
                                   const int32_t* page_table, int table_stride, int n_pages, const float* cos_t,
                                   const float* sin_t, int max_pos, void* kcache, void* vcache, int nh, int nkv, int hd,
                                   int* err, cudaStream_t stream) {
  EL_REFUSE(nh > 0 && nkv > 0 && table_stride > 0 && n_pages > 0 && max_pos > 0, "gemm_tc_rope: bad sizes");
  EL_REFUSE(edgelm_gemm_tc_rope_takes(a, lda, w, qkv, ldo, K, hd, kcache, vcache, cos_t, sin_t),
            "gemm_tc_rope: head size %d (takes 64 and 128), or an operand that is not 16-byte aligned", hd);
  RopeAppend ra;
  ra.tok_pos = tok_pos; ra.tok_seq = tok_seq; ra.seq_slot = seq_slot; ra.page_table = page_table;
  ra.cos_t = cos_t; ra.sin_t = sin_t;
  ra.kcache = static_cast<__nv_bfloat16*>(kcache); ra.vcache = static_cast<__nv_bfloat16*>(vcache);
  ra.table_stride = table_stride; ra.n_pages = n_pages; ra.max_pos = max_pos; ra.nh = nh; ra.nkv = nkv; ra.hd = hd;
  return gemm_tc_run(a, lda, w, nullptr, qkv, ldo, nullptr, M, (nh + 2 * nkv) * hd, K, DT_BF16, TC_EPI_ROPE, err, stream, ra);
}
