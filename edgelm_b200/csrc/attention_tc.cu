// Causal attention of new tokens over the paged cache on the fifth-generation tensor cores
// (tcgen05): bfloat16, head size 64, any number of heads and groups, any lengths.
//
// One CTA takes a tile of up to 128 consecutive tokens of one sequence and one query head, and walks
// the sequence's keys in blocks of 128 (two pages of the cache) up to the tile's last position:
//
//   S   = Q K^T          tcgen05.mma M128 N128 K16 x 4, accumulator in tensor memory (two S buffers)
//   P   = exp2(S - max)  softmax warps, two threads a row: tcgen05.ld of their halves of the row, float32
//                        maximum and denominator, P rounded to bfloat16 into shared memory in the
//                        128-byte-swizzled K-major layout the next MMA reads
//   O  += P V            tcgen05.mma M128 N64 K16 x 8, accumulating in tensor memory over the blocks; V is
//                        used as it lies in the cache, [key][dim]: the MN-major B operand (rows of 128
//                        bytes = the 64 dims of a key).  The reference maximum of a row moves only when
//                        the running maximum has outgrown it by 2^8; then the softmax threads scale
//                        their rows of O in place (tcgen05.ld, multiply, tcgen05.st)
//
// Roles: warp 0 issues the TMA loads (Q once; K and V of a block as two pages each, four stages: with two, a
// group's next block was only requested when its current one was done, and every block waited out a load),
// warp 1 allocates tensor memory and issues the MMAs, warps 2-9 and 10-17 are two softmax groups.  The
// groups take the key blocks in turn (even, odd), each with an S, a P and an O of its own and its own
// reference maximum and denominator; group 0 merges the two at the end.  In a group two threads share a
// row (64 keys each), so that a row's 128 scores need no more registers than a thread has without
// spilling.  Two blocks are in flight in a CTA: the tensor cores work for one group while the other
// computes exponentials, and an SM sub-partition has four softmax warps to overlap the latencies of
// tcgen05.ld.  384 of 512 columns of tensor memory (S, S, O, O).
// Every wait is bounded as in the matrix-product kernels: a wait that runs out sets ERR_WAIT_TIMEOUT,
// raises the block's abort flag, and all roles leave; tensor memory is freed in any case.
//
// Rows of the tile past its token count compute on whatever the Q box brought (other tokens' rows or
// zeros) and are not stored.  A block's second page may not exist: the first is loaded twice and the
// keys are masked.  Value rows past the tile's last position are zeroed in shared memory in the last
// block, so that a stale NaN cannot meet a zero weight.
#include <math_constants.h>

#include "tc_common.cuh"

namespace edgelm {

constexpr int AT_ROWS = 128;    // tokens of a tile = lanes of tensor memory
constexpr int AT_KEYS = 128;    // keys of a block
constexpr int AT_HD = 64;
constexpr int AT_GROUP_THREADS = 256;   // a softmax group: two threads a row, each with 64 of a block's 128 keys
constexpr int AT_THREADS = 64 + 2 * AT_GROUP_THREADS;   // TMA warp, MMA warp, two softmax groups of eight warps
constexpr int AT_Q_BYTES = AT_ROWS * AT_HD * 2;          // 16 KB
constexpr int AT_KV_BYTES = AT_KEYS * AT_HD * 2;         // 16 KB: two pages
constexpr int AT_STAGES = 4;                             // blocks of K and of V in shared memory: the loads run two blocks a group ahead
constexpr int AT_P_BYTES = AT_ROWS * AT_KEYS * 2;        // 32 KB: two K-major tiles of 128 x 64
constexpr int AT_XCHG_BYTES = 2 * 2 * AT_ROWS * 4;   // the two threads of a row tell each other their half's maximum: [group][half][row]
constexpr int AT_SMEM = AT_Q_BYTES + 2 * AT_STAGES * AT_KV_BYTES + 2 * AT_P_BYTES + AT_XCHG_BYTES + 1024 + 512;
constexpr uint32_t AT_TMEM_COLS = 512;                   // S of group 0, S of group 1 (128 each), O_b of group 0, of group 1 (64 each)

__device__ __forceinline__ float at_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t at_pack(float a, float b) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&v);
}

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]),
        "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]),
        "r"(r[30]), "r"(r[31])
      : "memory");
}

constexpr float AT_LAZY = 8.f;   // the reference maximum follows the running maximum only when that has grown by more than 2^8

// The softmax of one block for half a row (64 of its 128 keys; the other half is the partner thread's, same lane,
// four warps further): the scores come from tensor memory once and stay in registers; the two halves' maxima are
// exchanged through shared memory (`mine`, `theirs`) around a barrier of the group.  MASKED: the block touches the
// diagonal (keys past `pos` do not count).  P = exp2(S scale - m_ref), rounded to bfloat16, goes into the half's
// swizzled K-major tile; returns its sum.  m_ref is the row's reference maximum: the first block's maximum, replaced
// by a later block's only when that exceeds it by more than AT_LAZY (P then stays below 2^8, far inside the range
// of bfloat16 and float32); `rescale` is the factor that replacement puts on what was accumulated before (1 if
// none): softmax does not depend on the reference, only its rounding does.  Both threads of a row decide alike.
template <bool MASKED>
__device__ __forceinline__ float at_softmax_block(uint32_t s_addr, uint8_t* p_tile, int row, int key0, int pos, float scale_log2,
                                                  bool first, float& m_ref, float& rescale, float* mine, const float* theirs,
                                                  int group_barrier) {
  uint32_t r[AT_KEYS / 2];
  tmem_ld32(s_addr, r);
  tmem_ld32(s_addr + 32, r + 32);
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
  float mx = -CUDART_INF_F;
#pragma unroll
  for (int i = 0; i < AT_KEYS / 2; ++i)
    if (!MASKED || key0 + i <= pos) mx = fmaxf(mx, __uint_as_float(r[i]));   // (the scale is positive)
  *mine = mx;
  asm volatile("bar.sync %0, %1;" ::"r"(group_barrier), "r"(AT_GROUP_THREADS) : "memory");
  mx = fmaxf(mx, *theirs) * scale_log2;
  rescale = 1.f;
  if (first) {
    m_ref = mx;
  } else if (mx > m_ref + AT_LAZY) {
    rescale = at_exp2(m_ref - mx);   // (0 if the row has seen no key so far)
    m_ref = mx;
  }
  const float m_use = m_ref == -CUDART_INF_F ? 0.f : m_ref;   // (a row of the tile's unused tail may see no key)
  float lsum = 0.f;
#pragma unroll
  for (int c = 0; c < AT_KEYS / 64; ++c) {
    uint32_t pk[16];
#pragma unroll
    for (int i = 0; i < 32; i += 2) {
      float p0 = at_exp2(fmaf(__uint_as_float(r[c * 32 + i]), scale_log2, -m_use));
      float p1 = at_exp2(fmaf(__uint_as_float(r[c * 32 + i + 1]), scale_log2, -m_use));
      if (MASKED) {
        if (key0 + c * 32 + i > pos) p0 = 0.f;
        if (key0 + c * 32 + i + 1 > pos) p1 = 0.f;
      }
      lsum += p0 + p1;
      pk[i >> 1] = at_pack(p0, p1);
    }
    uint8_t* prow = p_tile + row * 128;
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int ch = c * 4 + u;
      *reinterpret_cast<uint4*>(prow + ((ch ^ (row & 7)) << 4)) = make_uint4(pk[u * 4], pk[u * 4 + 1], pk[u * 4 + 2], pk[u * 4 + 3]);
    }
  }
  return lsum;
}

__global__ void __launch_bounds__(AT_THREADS, 1)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, __nv_bfloat16* __restrict__ out, int ldo,
                       const int32_t* __restrict__ page_table, int table_stride, int n_pages,
                       const int32_t* __restrict__ seq_slot, const int32_t* __restrict__ tile_seq,
                       const int32_t* __restrict__ tile_tok0, const int32_t* __restrict__ tile_ntok,
                       const int32_t* __restrict__ tile_pos0, int n_tiles, int nh, int nkv, float scale_log2, int* err) {
  extern __shared__ uint8_t at_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(at_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* q_s = smem;
  uint8_t* k_s = q_s + AT_Q_BYTES;            // [2][16 KB]
  uint8_t* v_s = k_s + AT_STAGES * AT_KV_BYTES;   // [AT_STAGES][16 KB]
  uint8_t* p_s = v_s + AT_STAGES * AT_KV_BYTES;   // [2 groups][2 tiles][128 rows][128 bytes]
  float* xchg = reinterpret_cast<float*>(p_s + 2 * AT_P_BYTES);   // [group][half][row]
  uint64_t* bars = reinterpret_cast<uint64_t*>(p_s + 2 * AT_P_BYTES + AT_XCHG_BYTES);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;                      // [AT_STAGES]
  uint64_t* v_full = k_full + AT_STAGES;            // [AT_STAGES]
  uint64_t* k_empty = v_full + AT_STAGES;           // [AT_STAGES]
  uint64_t* v_empty = k_empty + AT_STAGES;          // [AT_STAGES]
  uint64_t* s_ready = v_empty + AT_STAGES;          // [2]
  uint64_t* p_ready = s_ready + 2;                  // [2] one arrival per thread of the group
  uint64_t* o_ready = p_ready + 2;                  // [2]
  constexpr int N_BARS = 1 + 4 * AT_STAGES + 6;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + N_BARS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile = n_tiles - 1 - (int)blockIdx.x;   // late tiles (long rows of keys) first
  const int head = blockIdx.y, kvh = head / (nh / nkv);
  const int seq = tile_seq[tile], tok0 = tile_tok0[tile], ntok = tile_ntok[tile], pos0 = tile_pos0[tile];
  const int n_keys = pos0 + ntok;                          // keys 0 .. n_keys - 1 are seen by some row of the tile
  const int n_blk = (n_keys + AT_KEYS - 1) / AT_KEYS;
  const int n_pg = (n_keys + PAGE - 1) / PAGE;

  if (threadIdx.x == 0) {
    for (int i = 0; i < N_BARS; ++i) mbar_init(smem_u32(&bars[i]), (&bars[i] == &p_ready[0] || &bars[i] == &p_ready[1]) ? (uint32_t)AT_GROUP_THREADS : 1u);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(AT_TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_o = tmem_base + 2 * AT_KEYS;   // O_b of group g at + g * AT_HD

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      const int32_t* pages = page_table + (size_t)seq_slot[seq] * table_stride;
      mbar_expect_tx(smem_u32(q_full), AT_Q_BYTES);
      tma_load_2d(smem_u32(q_s), &map_q, smem_u32(q_full), head * AT_HD, tok0);
      for (int j = 0; j < n_blk; ++j) {
        const int s = j % AT_STAGES;
        const uint32_t par = (uint32_t)(j / AT_STAGES) & 1u;
        int p0 = pages[2 * j], p1 = 2 * j + 1 < n_pg ? pages[2 * j + 1] : p0;
        if (p0 < 0 || p0 >= n_pages || p1 < 0 || p1 >= n_pages) {
          atomicOr(err, ERR_PAGE_RANGE);
          p0 = p1 = 0;
        }
        const int y0 = (p0 * nkv + kvh) * PAGE, y1 = (p1 * nkv + kvh) * PAGE;
        if (!mbar_wait(smem_u32(&k_empty[s]), par ^ 1u, abort_flag, err)) break;
        mbar_expect_tx(smem_u32(&k_full[s]), AT_KV_BYTES);
        tma_load_2d(smem_u32(k_s + s * AT_KV_BYTES), &map_k, smem_u32(&k_full[s]), 0, y0);
        tma_load_2d(smem_u32(k_s + s * AT_KV_BYTES + AT_KV_BYTES / 2), &map_k, smem_u32(&k_full[s]), 0, y1);
        if (!mbar_wait(smem_u32(&v_empty[s]), par ^ 1u, abort_flag, err)) break;
        mbar_expect_tx(smem_u32(&v_full[s]), AT_KV_BYTES);
        tma_load_2d(smem_u32(v_s + s * AT_KV_BYTES), &map_v, smem_u32(&v_full[s]), 0, y0);
        tma_load_2d(smem_u32(v_s + s * AT_KV_BYTES + AT_KV_BYTES / 2), &map_v, smem_u32(&v_full[s]), 0, y1);
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    // Block j belongs to softmax group j & 1 and uses that group's S, P and O_b.  Order: the scores of blocks 0
    // and 1, then for every block its P V as soon as its P is there, followed by the scores of block j + 2 into
    // the S buffer that the group has just finished reading.
    if (lane == 0) {
      constexpr uint32_t idesc_qk = umma_idesc(AT_ROWS, AT_KEYS);
      constexpr uint32_t idesc_pv = umma_idesc(AT_ROWS, AT_HD) | (1u << 16);   // B (the values) is MN-major
      const uint64_t dq = umma_desc(smem_u32(q_s));
      bool ok = mbar_wait(smem_u32(q_full), 0, abort_flag, err);
      auto issue_qk = [&](int j) {   // S[j & 1] = Q K_j^T
        const int s = j & 1, st = j % AT_STAGES;
        if (!mbar_wait(smem_u32(&k_full[st]), (uint32_t)(j / AT_STAGES) & 1u, abort_flag, err)) return false;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint64_t dk = umma_desc(smem_u32(k_s + st * AT_KV_BYTES));
#pragma unroll
        for (int k = 0; k < AT_HD / 16; ++k) umma_f16(tmem_base + (uint32_t)s * AT_KEYS, dq + 2 * k, dk + 2 * k, idesc_qk, k != 0);
        umma_commit(smem_u32(&s_ready[s]));
        umma_commit(smem_u32(&k_empty[st]));
        return true;
      };
      if (ok) ok = issue_qk(0);
      if (ok && n_blk > 1) ok = issue_qk(1);
      for (int j = 0; j < n_blk && ok; ++j) {
        const int s = j & 1, st = j % AT_STAGES;
        if (!(ok = mbar_wait(smem_u32(&p_ready[s]), (j >> 1) & 1, abort_flag, err))) break;
        if (!(ok = mbar_wait(smem_u32(&v_full[st]), (uint32_t)(j / AT_STAGES) & 1u, abort_flag, err))) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint64_t dv = umma_desc(smem_u32(v_s + st * AT_KV_BYTES));
#pragma unroll
        for (int k = 0; k < AT_KEYS / 16; ++k) {
          // P: two K-major tiles of 64 keys; V: 16 keys further = 16 rows of 128 bytes further
          const uint64_t dp = umma_desc(smem_u32(p_s + s * AT_P_BYTES + (k >> 2) * (AT_P_BYTES / 2))) + 2 * (k & 3);
          umma_f16(tmem_o + (uint32_t)s * AT_HD, dp, dv + (uint64_t)(k * 16 * 128 >> 4), idesc_pv, (k != 0) || (j >= 2));   // O of the group accumulates over its blocks
        }
        umma_commit(smem_u32(&o_ready[s]));
        umma_commit(smem_u32(&v_empty[st]));
        if (j + 2 < n_blk) ok = issue_qk(j + 2);   // (the group has read S of block j: it has written its P)
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax: two groups of eight warps.  The
    // groups take the blocks in turn, each with a reference maximum, denominator and output of its own; in a group
    // two threads share a row (warps w and w + 4 reach the same 32 lanes of tensor memory): each has 64 of a
    // block's 128 keys and 32 of the output's 64 dims.
    const int sw = warp - 2, g = sw >> 3, half = (sw >> 2) & 1, q4 = warp & 3, row = q4 * 32 + lane, pos = pos0 + row;
    const uint32_t lane_off = (uint32_t)(q4 * 32) << 16;
    const uint32_t s_addr = tmem_base + lane_off + (uint32_t)g * AT_KEYS + (uint32_t)half * (AT_KEYS / 2);
    const uint32_t o_addr = tmem_o + lane_off + (uint32_t)g * AT_HD + (uint32_t)half * (AT_HD / 2);
    uint8_t* p_tile = p_s + g * AT_P_BYTES + half * (AT_P_BYTES / 2);
    float* mine = xchg + (g * 2 + half) * AT_ROWS + row;
    const float* theirs = xchg + (g * 2 + (half ^ 1)) * AT_ROWS + row;
    const int group_barrier = 1 + g;
    float m = -CUDART_INF_F, l = 0.f;   // the row's reference maximum (log2 units) and this half's share of the denominator
    bool ok = true;
    int u = 0;   // blocks this group has done
    for (int j = g; j < n_blk; j += 2, ++u) {
      const int key0 = j * AT_KEYS + half * (AT_KEYS / 2);
      if (!(ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&s_ready[g]), u & 1, abort_flag, err)))) break;
      // the group's block before this one has been through its P V: P and O are free (that product was issued long ago)
      if (u > 0 && !(ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&o_ready[g]), (u - 1) & 1, abort_flag, err)))) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      float rescale;
      const float lsum = j * AT_KEYS + AT_KEYS - 1 > pos0
                             ? at_softmax_block<true>(s_addr, p_tile, row, key0, pos, scale_log2, u == 0, m, rescale, mine, theirs, group_barrier)
                             : at_softmax_block<false>(s_addr, p_tile, row, key0, pos, scale_log2, u == 0, m, rescale, mine, theirs, group_barrier);
      if (__any_sync(0xffffffffu, rescale != 1.f)) {   // rare after the first blocks: the warp's share of O times the rows' factors
        uint32_t r[32];
        tmem_ld32(o_addr, r);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
        for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * rescale);
        tmem_st32(o_addr, r);
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      }
      l = fmaf(l, rescale, lsum);
      if (j == n_blk - 1 && n_keys < j * AT_KEYS + AT_KEYS) {
        // value rows past the tile's last position: every weight on them is zero; make them zero too
        if (!(ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&v_full[j % AT_STAGES]), (uint32_t)(j / AT_STAGES) & 1u, abort_flag, err)))) break;
        const int first = n_keys - j * AT_KEYS;   // 1 .. 127
        for (int i = (sw & 7) * 32 + lane; i < (AT_KEYS - first) * 8; i += AT_GROUP_THREADS) {
          const int r = first + (i >> 3);
          *reinterpret_cast<uint4*>(v_s + (j % AT_STAGES) * AT_KV_BYTES + r * 128 + ((i & 7) << 4)) = make_uint4(0, 0, 0, 0);
        }
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&p_ready[g])) : "memory");
    }
    // ---- the group's output out of tensor memory: this thread's 32 dims of its row
    float o[AT_HD / 2];
#pragma unroll
    for (int i = 0; i < AT_HD / 2; ++i) o[i] = 0.f;
    if (ok && u > 0) {
      ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&o_ready[g]), (u - 1) & 1, abort_flag, err));
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      if (ok) {
        uint32_t r[32];
        tmem_ld32(o_addr, r);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
        for (int i = 0; i < 32; ++i) o[i] = __uint_as_float(r[i]);
      }
    }
    // ---- a row's four threads (two groups, two halves) put their results together: every thread hands over its
    // (m, l) and group 1 its 32 dims, through the P tiles (all P V products are done: both groups have read their O);
    // group 0 merges and stores its own 32 dims
    float* hand_ml = reinterpret_cast<float*>(p_s);                                  // [group][half][row][2]
    float* hand_o = hand_ml + 2 * 2 * AT_ROWS * 2;                                   // [half][row][33] of group 1
    asm volatile("bar.sync 3, 512;" ::: "memory");   // nobody's P tiles are read any more
    hand_ml[((g * 2 + half) * AT_ROWS + row) * 2] = m;
    hand_ml[((g * 2 + half) * AT_ROWS + row) * 2 + 1] = l;
    if (g == 1) {
#pragma unroll
      for (int i = 0; i < AT_HD / 2; ++i) hand_o[(half * AT_ROWS + row) * 33 + i] = o[i];
    }
    asm volatile("bar.sync 3, 512;" ::: "memory");
    if (g == 0 && ok && row < ntok) {
      // (the two halves of a group share m; their l add up)
      const float m0 = m, l0 = l + hand_ml[((0 * 2 + (half ^ 1)) * AT_ROWS + row) * 2 + 1];
      const float m1 = hand_ml[((1 * 2 + 0) * AT_ROWS + row) * 2];
      const float l1 = hand_ml[((1 * 2 + 0) * AT_ROWS + row) * 2 + 1] + hand_ml[((1 * 2 + 1) * AT_ROWS + row) * 2 + 1];
      const float mm = fmaxf(m0, m1);
      const float f0 = at_exp2(m0 - mm), f1 = m1 == -CUDART_INF_F ? 0.f : at_exp2(m1 - mm);
      const float inv = 1.0f / (l0 * f0 + l1 * f1);
      const float* o1 = hand_o + (half * AT_ROWS + row) * 33;
      __nv_bfloat16* dst = out + (size_t)(tok0 + row) * ldo + head * AT_HD + half * (AT_HD / 2);
#pragma unroll
      for (int i = 0; i < AT_HD / 2; i += 8) {
        float v[8];
#pragma unroll
        for (int t = 0; t < 8; ++t) v[t] = (o[i + t] * f0 + o1[i + t] * f1) * inv;
        *reinterpret_cast<uint4*>(dst + i) = make_uint4(at_pack(v[0], v[1]), at_pack(v[2], v[3]), at_pack(v[4], v[5]), at_pack(v[6], v[7]));
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(AT_TMEM_COLS) : "memory");
  }
}

}  // namespace edgelm

using namespace edgelm;

// 1 if the tcgen05 prefill attention takes this head size (bfloat16 is implied), else 0.
extern "C" int edgelm_attn_prefill_tc_takes(int hd) { return hd == AT_HD ? 1 : 0; }

// qkv [T, (nh + 2 nkv) * 64] bfloat16 with the queries already rotated; keys and values already in the cache.
// Tiles of at most 128 tokens.
extern "C" int edgelm_attn_prefill_tc(const void* qkv, int ldq, int n_tokens, void* out, int ldo, const void* kcache,
                                      const void* vcache, int n_pages, const int32_t* page_table, int table_stride,
                                      const int32_t* seq_slot, const int32_t* tile_seq, const int32_t* tile_tok0,
                                      const int32_t* tile_ntok, const int32_t* tile_pos0, int n_tiles, int nh, int nkv, int hd,
                                      float scale, int* err, cudaStream_t stream) {
  if (n_tiles == 0) return 0;
  EL_REFUSE(hd == AT_HD, "attn_prefill_tc: head size %d (takes 64)", hd);
  EL_REFUSE(nh > 0 && nkv > 0 && nh % nkv == 0 && nh <= 65535, "attn_prefill_tc: %d heads over %d kv heads", nh, nkv);
  EL_REFUSE(ldq % 8 == 0 && ldo % 8 == 0 && (uintptr_t)qkv % 16 == 0 && (uintptr_t)out % 16 == 0 && (uintptr_t)kcache % 16 == 0 &&
                (uintptr_t)vcache % 16 == 0,
            "attn_prefill_tc: rows and cache must be 16-byte aligned");
  EL_REFUSE(err != nullptr && n_tokens > 0 && (long long)n_pages * nkv * PAGE < (1LL << 31), "attn_prefill_tc: bad arguments");
  CUtensorMap mq, mk, mv;
  if (tensor_map(qkv, n_tokens, ldq, ldq, AT_ROWS, &mq)) return -1;
  if (tensor_map(kcache, n_pages * nkv * PAGE, AT_HD, AT_HD, PAGE, &mk)) return -1;
  if (tensor_map(vcache, n_pages * nkv * PAGE, AT_HD, AT_HD, PAGE, &mv)) return -1;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, AT_SMEM);
    EL_REFUSE(e == cudaSuccess, "attn_prefill_tc: %d bytes of shared memory refused: %s", AT_SMEM, cudaGetErrorString(e));
    configured = true;
  }
  const float scale_log2 = scale * 1.4426950408889634f;
  attn_prefill_tc_kernel<<<dim3(n_tiles, nh), AT_THREADS, AT_SMEM, stream>>>(
      mq, mk, mv, (__nv_bfloat16*)out, ldo, page_table, table_stride, n_pages, seq_slot, tile_seq, tile_tok0, tile_ntok,
      tile_pos0, n_tiles, nh, nkv, scale_log2, err);
  EL_LAUNCH_CHECK("attn_prefill_tc");
  return 0;
}
