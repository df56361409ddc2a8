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
//   O  += P V            tcgen05.mma M128 N64 K16, four for each half of the block's keys, each half into
//                        an accumulator of its own in tensor memory, over the blocks; V is used as it lies
//                        in the cache, [key][dim]: the MN-major B operand (rows of 128 bytes = the 64 dims
//                        of a key).  The reference maximum of a half row moves only when the running
//                        maximum has outgrown it by 2^8; then its thread scales its row of its O in place
//                        (tcgen05.ld, multiply, tcgen05.st)
//
// Roles: warp 0 loads Q and the keys by TMA (two stages), warp 1 the values (three; each block as two
// pages; one warp for both would hold the keys of the block after next behind a wait for a free value
// stage); warp 2 allocates tensor memory and issues the Q K^T products, warp 3 the P V products (two
// issuers, because which comes next depends on how the groups drift); warps 4-11 and 12-19 are two
// softmax groups.  The groups take the key blocks in turn (even, odd), each with an S of its own, two P
// buffers and its own accumulators.  In a group two threads share a row, 64 keys each, and share nothing
// else: each has its own reference maximum, denominator and O (so no exchange between them in the loop,
// and a row's 128 scores need no more registers than a thread has).  A thread frees its S as soon as the
// scores are in its registers: the group's next Q K^T runs while it computes exponentials; with two P
// buffers the next block's P can be written while the tensor cores still read this one's.  The four
// partial results of a row (two groups, two halves) are put together at the end: all four threads reach
// the same lanes of tensor memory, so each reads its 16 dims of the row from all four accumulators.
// What limits the kernel is the special-function unit (an exp2 per score, 16 a clock per SM: 1,024
// clocks a block); the second group starts half a block behind the first so that one group is at its
// exponentials while the other waits, loads and stores.  (Tried and slower: turns at the exponentials,
// strictly one group at a time, 3,050 clocks for a pair of blocks against 2,650; one group of 16 warps,
// four threads a row, each holding the scores of two blocks in registers, 4,200: a block's waits and
// fences then stand against 32 exponentials a thread instead of 64.)
// All 512 columns of tensor memory (S, S, and four O of 64).
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
constexpr int AT_HALF = AT_KEYS / 2;    // keys of a thread
constexpr int AT_HD = 64;
constexpr int AT_GROUP_WARPS = 8;       // a softmax group: two threads a row, each with 64 of a block's 128 keys
constexpr int AT_GROUP_THREADS = AT_GROUP_WARPS * 32;
constexpr int AT_ROLE_WARPS = 4;        // K loads, V loads, Q K^T issue, P V issue
constexpr int AT_THREADS = AT_ROLE_WARPS * 32 + 2 * AT_GROUP_THREADS;
constexpr int AT_Q_BYTES = AT_ROWS * AT_HD * 2;          // 16 KB
constexpr int AT_KV_BYTES = AT_KEYS * AT_HD * 2;         // 16 KB: two pages
constexpr int AT_STAGES = 2;                             // blocks of K in shared memory: a group's blocks use one of them
constexpr int AT_V_STAGES = 3;                           // blocks of V (a stage is free only when the block that used it has been
                                                         // through its P V; measured no faster than two with the cache in L2)
constexpr int AT_P_BYTES = AT_ROWS * AT_KEYS * 2;        // 32 KB: two K-major tiles of 128 x 64, one per half
constexpr int AT_P_BUFS = 2;                             // P buffers of a group
constexpr int AT_N_BARS = 1 + 2 * AT_STAGES + 2 * AT_V_STAGES + 12;
constexpr int AT_SMEM = AT_Q_BYTES + (AT_STAGES + AT_V_STAGES) * AT_KV_BYTES + 2 * AT_P_BUFS * AT_P_BYTES + 1024 + 512;
static_assert(AT_SMEM <= 227 * 1024, "shared memory");
constexpr uint32_t AT_TMEM_COLS = 512;   // S of group 0, of group 1 (128 each); O of (group, half) at 256 + (2 group + half) 64
constexpr int AT_STAGGER_CLOCKS = 1300;   // half of what a group takes for a block
constexpr int AT_TRACE_BLOCKS = 64;   // blocks of a group that a trace has room for
static_assert(AT_STAGES == 2, "a group's blocks use one K stage (the end's exchange lies there)");

__device__ __forceinline__ float at_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// two float32 in a 64-bit register pair, and the packed instructions on them
__device__ __forceinline__ uint64_t at_pair(float lo, float hi) {
  uint64_t d;
  asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "f"(lo), "f"(hi));
  return d;
}
__device__ __forceinline__ void at_unpair(uint64_t v, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ uint64_t at_fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t at_add2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ float at_max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
// A bounded wait that lets the hardware park the warp (a time hint on try_wait) and looks at the abort flag and the
// clock only now and then: the roles of this kernel wait often and long, and their polling would take issue slots
// from the exponentials.
__device__ __forceinline__ bool at_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* err) {
  if (mbar_try(bar, parity)) return true;
  const long long t0 = clock64();
  while (true) {
#pragma unroll 1
    for (int i = 0; i < 8; ++i) {
      uint32_t ok;
      asm volatile(
          "{\n\t.reg .pred p;\n\t"
          "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
          "selp.u32 %0, 1, 0, p;\n\t}"
          : "=r"(ok)
          : "r"(bar), "r"(parity), "r"(20000u)
          : "memory");
      if (ok) return true;
    }
    if (*abort_flag) return false;
    if (clock64() - t0 > TC_WAIT_CYCLES) {
      *abort_flag = 1;
      atomicOr(err, ERR_WAIT_TIMEOUT);
      return false;
    }
  }
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

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
}

constexpr float AT_LAZY = 8.f;   // the reference maximum follows the running maximum only when that has grown by more than 2^8

// The softmax of one block for half a row (64 of its 128 keys): the scores come from tensor memory once and stay in
// registers; `s_free` gets the warp's arrival as soon as they are there.  MASKED: the block touches the diagonal
// (keys past `pos` do not count).  P = exp2(S scale - m_ref), rounded to bfloat16, goes into the half's swizzled
// K-major tile; returns its sum.  m_ref is the half row's reference maximum: the first block's maximum, replaced
// by a later block's only when that exceeds it by more than AT_LAZY (P then stays below 2^8, far inside the range
// of bfloat16 and float32); `rescale` is the factor that replacement puts on what was accumulated before (1 if
// none): softmax does not depend on the reference, only its rounding does.
template <bool MASKED>
__device__ __forceinline__ float at_softmax_block(uint32_t s_addr, uint32_t s_free, uint8_t* p_tile, int row, int key0, int pos,
                                                  float scale_log2, bool first, float& m_ref, float& rescale) {
  uint32_t r[AT_HALF];
  tmem_ld32(s_addr, r);
  tmem_ld32(s_addr + 32, r + 32);
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncwarp();
  if ((threadIdx.x & 31) == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(s_free) : "memory");
  if (MASKED) {
#pragma unroll
    for (int i = 0; i < AT_HALF; ++i)
      if (key0 + i > pos) r[i] = __float_as_uint(-CUDART_INF_F);   // exp2 makes a zero of it
  }
  float mx0 = -CUDART_INF_F, mx1 = -CUDART_INF_F;
#pragma unroll
  for (int i = 0; i < AT_HALF; i += 4) {
    mx0 = at_max3(mx0, __uint_as_float(r[i]), __uint_as_float(r[i + 1]));
    mx1 = at_max3(mx1, __uint_as_float(r[i + 2]), __uint_as_float(r[i + 3]));
  }
  const float mx = fmaxf(mx0, mx1) * scale_log2;   // (the scale is positive)
  rescale = 1.f;
  if (first) {
    m_ref = mx;
  } else if (mx > m_ref + AT_LAZY) {
    rescale = at_exp2(m_ref - mx);   // (0 if the half row has seen no key so far)
    m_ref = mx;
  }
  const float m_use = m_ref == -CUDART_INF_F ? 0.f : m_ref;   // (a half row may have seen no key yet)
  const uint64_t scale2 = at_pair(scale_log2, scale_log2), minus_m2 = at_pair(-m_use, -m_use);
  uint64_t sum_a = at_pair(0.f, 0.f), sum_b = sum_a;
#pragma unroll
  for (int c = 0; c < AT_HALF / 32; ++c) {
    uint32_t pk[16];
#pragma unroll
    for (int i = 0; i < 32; i += 4) {
      const uint32_t* x = r + c * 32 + i;
      float a0, a1, b0, b1;
      at_unpair(at_fma2(at_pair(__uint_as_float(x[0]), __uint_as_float(x[1])), scale2, minus_m2), a0, a1);
      at_unpair(at_fma2(at_pair(__uint_as_float(x[2]), __uint_as_float(x[3])), scale2, minus_m2), b0, b1);
      a0 = at_exp2(a0), a1 = at_exp2(a1), b0 = at_exp2(b0), b1 = at_exp2(b1);
      sum_a = at_add2(sum_a, at_pair(a0, a1));
      sum_b = at_add2(sum_b, at_pair(b0, b1));
      pk[i >> 1] = at_pack(a0, a1);
      pk[(i >> 1) + 1] = at_pack(b0, b1);
    }
    uint8_t* prow = p_tile + row * 128;
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int ch = c * 4 + u;
      *reinterpret_cast<uint4*>(prow + ((ch ^ (row & 7)) << 4)) = make_uint4(pk[u * 4], pk[u * 4 + 1], pk[u * 4 + 2], pk[u * 4 + 3]);
    }
  }
  float s0, s1, s2, s3;
  at_unpair(sum_a, s0, s1);
  at_unpair(sum_b, s2, s3);
  const float lsum = (s0 + s1) + (s2 + s3);
  return lsum;
}

__global__ void __launch_bounds__(AT_THREADS, 1)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, __nv_bfloat16* __restrict__ out, int ldo,
                       const int32_t* __restrict__ page_table, int table_stride, int n_pages,
                       const int32_t* __restrict__ seq_slot, const int32_t* __restrict__ tile_seq,
                       const int32_t* __restrict__ tile_tok0, const int32_t* __restrict__ tile_ntok,
                       const int32_t* __restrict__ tile_pos0, int n_tiles, int nh, int nkv, float scale_log2, int* err,
                       long long* trace) {
  extern __shared__ uint8_t at_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(at_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* q_s = smem;
  uint8_t* k_s = q_s + AT_Q_BYTES;                // [AT_STAGES][16 KB]
  uint8_t* v_s = k_s + AT_STAGES * AT_KV_BYTES;   // [AT_V_STAGES][16 KB]
  uint8_t* p_s = v_s + AT_V_STAGES * AT_KV_BYTES;   // [2 groups][AT_P_BUFS][2 halves][128 rows][128 bytes]
  uint64_t* bars = reinterpret_cast<uint64_t*>(p_s + 2 * AT_P_BUFS * AT_P_BYTES);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;                      // [AT_STAGES]
  uint64_t* v_full = k_full + AT_STAGES;            // [AT_V_STAGES]
  uint64_t* k_empty = v_full + AT_V_STAGES;         // [AT_STAGES]
  uint64_t* v_empty = k_empty + AT_STAGES;          // [AT_V_STAGES]
  uint64_t* s_ready = v_empty + AT_V_STAGES;         // [2] the group's scores are in tensor memory
  uint64_t* s_free = s_ready + 2;                   // [2] ... and in the group's registers: one arrival per warp
  // The next two come in pairs, for a group's even and odd blocks, so that a waiter may fall a block behind.
  uint64_t* p_ready = s_free + 2;                   // [2][2] the group's P is in shared memory: one arrival per warp
  uint64_t* o_ready = p_ready + 4;                  // [2][2] the group's P V is done
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + AT_N_BARS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // `trace` (may be null): clock stamps of the grid's first block.  [group][block][8] from one warp of each softmax
  // group; after those, eight of the block as a whole (thread AT_ROLE_WARPS * 32: entry, tensor memory there, the
  // kernel before this one done, the key blocks done, accumulator read, row stored, block done)
  const bool tracing = trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0;
  auto block_stamp = [&](int i) {
    if (tracing && threadIdx.x == AT_ROLE_WARPS * 32) trace[2 * AT_TRACE_BLOCKS * 8 + i] = clock64();
  };
  block_stamp(0);
  const int tile = n_tiles - 1 - (int)blockIdx.x;   // late tiles (long rows of keys) first
  const int head = blockIdx.y, kvh = head / (nh / nkv);
  const int seq = tile_seq[tile], tok0 = tile_tok0[tile], ntok = tile_ntok[tile], pos0 = tile_pos0[tile];
  const int n_keys = pos0 + ntok;                          // keys 0 .. n_keys - 1 are seen by some row of the tile
  const int n_blk = (n_keys + AT_KEYS - 1) / AT_KEYS;
  const int n_pg = (n_keys + PAGE - 1) / PAGE;

  if (threadIdx.x == 0) {
    for (int i = 0; i < AT_N_BARS; ++i) {
      const bool by_warps = &bars[i] >= s_free && &bars[i] < o_ready;
      mbar_init(smem_u32(&bars[i]), by_warps ? (uint32_t)AT_GROUP_WARPS : 1u);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 2) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(AT_TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;
  block_stamp(1);
  pdl_launch_dependents();
  pdl_wait();   // (launched as a programmatic dependent: up to here only the step's tables were read)
  const uint32_t tmem_o = tmem_base + 2 * AT_KEYS;   // O of (group g, half h) at + (2 g + h) * AT_HD
  block_stamp(2);

  if (warp < 2) {
    // ---------------------------------------------------------------- TMA producers: warp 0 Q and K, warp 1 V
    if (lane == 0) {
      const int32_t* pages = page_table + (size_t)seq_slot[seq] * table_stride;
      const CUtensorMap* map = warp == 0 ? &map_k : &map_v;
      uint8_t* dst = warp == 0 ? k_s : v_s;
      uint64_t* full = warp == 0 ? k_full : v_full;
      uint64_t* empty = warp == 0 ? k_empty : v_empty;
      if (warp == 0) {
        mbar_expect_tx(smem_u32(q_full), AT_Q_BYTES);
        tma_load_2d(smem_u32(q_s), &map_q, smem_u32(q_full), head * AT_HD, tok0);
      }
      const int n_stages = warp == 0 ? AT_STAGES : AT_V_STAGES;
      for (int j = 0; j < n_blk; ++j) {
        const int s = j % n_stages;
        const uint32_t par = (uint32_t)(j / n_stages) & 1u;
        int p0 = pages[2 * j], p1 = 2 * j + 1 < n_pg ? pages[2 * j + 1] : p0;
        if (p0 < 0 || p0 >= n_pages || p1 < 0 || p1 >= n_pages) {
          atomicOr(err, ERR_PAGE_RANGE);
          p0 = p1 = 0;
        }
        const int y0 = (p0 * nkv + kvh) * PAGE, y1 = (p1 * nkv + kvh) * PAGE;
        if (!at_wait(smem_u32(&empty[s]), par ^ 1u, abort_flag, err)) break;
        mbar_expect_tx(smem_u32(&full[s]), AT_KV_BYTES);
        tma_load_2d(smem_u32(dst + s * AT_KV_BYTES), map, smem_u32(&full[s]), 0, y0);
        tma_load_2d(smem_u32(dst + s * AT_KV_BYTES + AT_KV_BYTES / 2), map, smem_u32(&full[s]), 0, y1);
      }
    }
  } else if (warp == 2) {
    // ---------------------------------------------------------------- Q K^T issuer.  Block j belongs to softmax group
    // j & 1 and goes into that group's S as soon as the group has the scores of block j - 2 in its registers.
    // The whole warp walks the loop and waits; one elected lane issues.  (With the loop inside `if (lane == 0)` the
    // descriptors are computed in a divergent region, out of reach of the uniform datapath that the instruction
    // takes them from, and an issue took some 120 clocks.)
    constexpr uint32_t idesc_qk = umma_idesc(AT_ROWS, AT_KEYS);
    const uint64_t dq = umma_desc(smem_u32(q_s));
    bool ok = __all_sync(0xffffffffu, at_wait(smem_u32(q_full), 0, abort_flag, err));
    for (int j = 0; j < n_blk && ok; ++j) {
      const int g = j & 1, st = j % AT_STAGES;
      if (j >= 2 && !(ok = __all_sync(0xffffffffu, at_wait(smem_u32(&s_free[g]), (uint32_t)((j >> 1) - 1) & 1u, abort_flag, err)))) break;
      if (!(ok = __all_sync(0xffffffffu, at_wait(smem_u32(&k_full[st]), (uint32_t)(j / AT_STAGES) & 1u, abort_flag, err)))) break;
      if (j == 1 && n_blk >= 4) {
        // The second group starts half a block's time behind the first.  Nothing else sets the groups' offset, and it
        // stays where it starts: in step, both groups are at their exponentials together and leave the special-function
        // units idle together afterwards (3,100 to 3,400 clocks for a pair of blocks against 2,650 half a block apart).
        const long long t0 = clock64();
        while (clock64() - t0 < AT_STAGGER_CLOCKS) {}
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint64_t dk = umma_desc(smem_u32(k_s + st * AT_KV_BYTES));
      const uint32_t d_s = tmem_base + (uint32_t)g * AT_KEYS, bar_s = smem_u32(&s_ready[g]), bar_k = smem_u32(&k_empty[st]);
      if (elect_one()) {
#pragma unroll
        for (int k = 0; k < AT_HD / 16; ++k) umma_f16(d_s, dq + 2 * k, dk + 2 * k, idesc_qk, k != 0);
        umma_commit(bar_s);
        umma_commit(bar_k);
      }
      __syncwarp();
    }
  } else if (warp == 3) {
    // ---------------------------------------------------------------- P V issuer: a block's two halves (64 keys each)
    // into the two accumulators of its group, which add up over the group's blocks.
    constexpr uint32_t idesc_pv = umma_idesc(AT_ROWS, AT_HD) | (1u << 16);   // B (the values) is MN-major
    bool ok = true;
    for (int j = 0; j < n_blk && ok; ++j) {
      const int g = j & 1, u = j >> 1, st = j % AT_V_STAGES;
      if (!(ok = __all_sync(0xffffffffu, at_wait(smem_u32(&p_ready[2 * g + (u & 1)]), (uint32_t)(u >> 1) & 1u, abort_flag, err)))) break;
      if (!(ok = __all_sync(0xffffffffu, at_wait(smem_u32(&v_full[st]), (uint32_t)(j / AT_V_STAGES) & 1u, abort_flag, err)))) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      if (tracing && lane == 0 && u < AT_TRACE_BLOCKS) trace[(g * AT_TRACE_BLOCKS + u) * 8 + 6] = clock64();   // (the issuer's view: P and V seen,
      const uint64_t dv = umma_desc(smem_u32(v_s + st * AT_KV_BYTES));
      const uint64_t dp = umma_desc(smem_u32(p_s + (g * AT_P_BUFS + (u % AT_P_BUFS)) * AT_P_BYTES));
      const uint32_t d_o = tmem_o + (uint32_t)(2 * g) * AT_HD, bar_o = smem_u32(&o_ready[2 * g + (u & 1)]), bar_v = smem_u32(&v_empty[st]);
      const uint32_t acc = u > 0;
      if (elect_one()) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
#pragma unroll
          for (int k = 0; k < AT_HALF / 16; ++k) {
            // P: the half's tile, 16 keys = 32 bytes further a step; V: 16 keys = 16 rows of 128 bytes further
            umma_f16(d_o + (uint32_t)h * AT_HD, dp + (uint64_t)(h * (AT_P_BYTES / 2) >> 4) + 2 * k,
                     dv + (uint64_t)((h * AT_HALF + k * 16) * 128 >> 4), idesc_pv, k != 0 ? 1u : acc);
          }
        }
        umma_commit(bar_o);
        umma_commit(bar_v);
      }
      __syncwarp();
      if (tracing && lane == 0 && u < AT_TRACE_BLOCKS) trace[(g * AT_TRACE_BLOCKS + u) * 8 + 7] = clock64();   //  product issued)
    }
  } else {
    // ---------------------------------------------------------------- softmax: two groups of eight warps.  The
    // groups take the blocks in turn; in a group two threads share a row (warps w and w + 4 reach the same 32
    // lanes of tensor memory): each has 64 of a block's 128 keys, and a reference maximum, a denominator and an
    // accumulator of its own.
    const int sw = warp - AT_ROLE_WARPS, g = sw >> 3, half = (sw >> 2) & 1, q4 = warp & 3, row = q4 * 32 + lane, pos = pos0 + row;
    const uint32_t lane_off = (uint32_t)(q4 * 32) << 16;
    const uint32_t s_addr = tmem_base + lane_off + (uint32_t)g * AT_KEYS + (uint32_t)half * AT_HALF;
    const uint32_t o_addr = tmem_o + lane_off + (uint32_t)(2 * g + half) * AT_HD;
    float m = -CUDART_INF_F, l = 0.f;   // the half row's reference maximum (log2 units) and denominator
    const bool stamps = tracing && lane == 0 && (sw & 7) == 0;
    auto stamp = [&](int u, int i) {
      if (stamps && u < AT_TRACE_BLOCKS) trace[(g * AT_TRACE_BLOCKS + u) * 8 + i] = clock64();
    };
    bool ok = true;
    int u = 0;   // blocks this group has done
    for (int j = g; j < n_blk; j += 2, ++u) {
      const int key0 = j * AT_KEYS + half * AT_HALF;
      uint8_t* p_tile = p_s + (g * AT_P_BUFS + (u % AT_P_BUFS)) * AT_P_BYTES + half * (AT_P_BYTES / 2);
      stamp(u, 0);
      if (!(ok = __all_sync(0xffffffffu, at_wait(smem_u32(&s_ready[g]), u & 1, abort_flag, err)))) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      stamp(u, 1);
      float rescale;
      const float lsum = j * AT_KEYS + AT_KEYS - 1 > pos0
                             ? at_softmax_block<true>(s_addr, smem_u32(&s_free[g]), p_tile, row, key0, pos, scale_log2, u == 0, m, rescale)
                             : at_softmax_block<false>(s_addr, smem_u32(&s_free[g]), p_tile, row, key0, pos, scale_log2, u == 0, m, rescale);
      stamp(u, 2);
      // The group's block before this one has been through its P V: its accumulators may be scaled, and the P buffer
      // it read is free for the block after this one.  (The P V of the block before last would do for the buffer,
      // and the scaling is rare; but without this wait the two groups fall into step, are at their exponentials
      // together and leave the special-function units idle together: measured a quarter slower.)
      if (u > 0 && !(ok = __all_sync(0xffffffffu, at_wait(smem_u32(&o_ready[2 * g + ((u - 1) & 1)]), (uint32_t)((u - 1) >> 1) & 1u, abort_flag, err)))) break;
      stamp(u, 3);
      if (__any_sync(0xffffffffu, rescale != 1.f)) {   // rare after the first blocks
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
        for (int c = 0; c < AT_HD / 32; ++c) {
          uint32_t r[32];
          tmem_ld32(o_addr + c * 32, r);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * rescale);
          tmem_st32(o_addr + c * 32, r);
        }
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      }
      stamp(u, 4);
      l = fmaf(l, rescale, lsum);
      if (j == n_blk - 1 && n_keys < j * AT_KEYS + AT_KEYS) {
        // value rows past the tile's last position: every weight on them is zero; make them zero too
        if (!(ok = __all_sync(0xffffffffu, at_wait(smem_u32(&v_full[j % AT_V_STAGES]), (uint32_t)(j / AT_V_STAGES) & 1u, abort_flag, err)))) break;
        const int first = n_keys - j * AT_KEYS;   // 1 .. 127
        for (int i = (sw & 7) * 32 + lane; i < (AT_KEYS - first) * 8; i += AT_GROUP_THREADS) {
          const int r = first + (i >> 3);
          *reinterpret_cast<uint4*>(v_s + (j % AT_V_STAGES) * AT_KV_BYTES + r * 128 + ((i & 7) << 4)) = make_uint4(0, 0, 0, 0);
        }
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&p_ready[2 * g + (u & 1)])) : "memory");
      stamp(u, 5);
    }
    block_stamp(3);
    // ---- a row's four threads (two groups, two halves) put their results together.  All four reach the same lanes
    // of tensor memory, so each reads its 16 dims of the row from all four accumulators; only (m, l) go through
    // shared memory (over this group's K stage: its last Q K^T is long done).
    if (ok && u > 0)
      ok = __all_sync(0xffffffffu, at_wait(smem_u32(&o_ready[2 * g + ((u - 1) & 1)]), (uint32_t)((u - 1) >> 1) & 1u, abort_flag, err));
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    const int q = g * 2 + half;
    float* hand_ml = reinterpret_cast<float*>(k_s + g * AT_KV_BYTES);   // [half][row][2]
    hand_ml[(half * AT_ROWS + row) * 2] = m;
    hand_ml[(half * AT_ROWS + row) * 2 + 1] = l;
    block_stamp(4);
    asm volatile("bar.sync 1, %0;" ::"n"(2 * AT_GROUP_THREADS) : "memory");   // both groups' last P V are done
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (ok && !*abort_flag) {
      float f[4], mm = -CUDART_INF_F, den = 0.f;
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const float* ml = reinterpret_cast<const float*>(k_s + (t >> 1) * AT_KV_BYTES) + ((t & 1) * AT_ROWS + row) * 2;
        mm = fmaxf(mm, f[t] = ml[0]);
      }
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const float* ml = reinterpret_cast<const float*>(k_s + (t >> 1) * AT_KV_BYTES) + ((t & 1) * AT_ROWS + row) * 2;
        f[t] = f[t] == -CUDART_INF_F ? 0.f : at_exp2(f[t] - mm);   // (a thread may have seen no key; the row has seen key 0)
        den = fmaf(ml[1], f[t], den);
      }
      uint32_t r[4][16];
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        if (t < 2 || n_blk > 1) {   // (with one block, group 1's accumulators were never written)
          tmem_ld16(tmem_o + lane_off + (uint32_t)(t * AT_HD + q * 16), r[t]);
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i) r[t][i] = 0u;
        }
      }
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      if (row < ntok) {
        const float inv = 1.0f / den;
        float v[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          v[i] = __uint_as_float(r[0][i]) * f[0];
#pragma unroll
          for (int t = 1; t < 4; ++t) v[i] = fmaf(__uint_as_float(r[t][i]), f[t], v[i]);
          v[i] *= inv;
        }
        __nv_bfloat16* dst = out + (size_t)(tok0 + row) * ldo + head * AT_HD + q * 16;
#pragma unroll
        for (int i = 0; i < 16; i += 8)
          *reinterpret_cast<uint4*>(dst + i) = make_uint4(at_pack(v[i], v[i + 1]), at_pack(v[i + 2], v[i + 3]), at_pack(v[i + 4], v[i + 5]), at_pack(v[i + 6], v[i + 7]));
      }
    }
  }
  block_stamp(5);
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  block_stamp(6);
  if (warp == 2) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(AT_TMEM_COLS) : "memory");
  }
}

}  // namespace edgelm

using namespace edgelm;

static long long* g_at_trace = nullptr;
// A device buffer of 2 x 64 x 8 + 8 clock stamps that the next launches fill (one softmax warp of each group of the
// grid's first block: before and after the wait for the scores, after the exponentials, after the wait for the
// last P V, after a rescaling, after the arrival; then eight of the block as a whole), or null to stop.
extern "C" void edgelm_attn_prefill_tc_trace(void* buffer) { g_at_trace = (long long*)buffer; }

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
  launch_pdl(16, attn_prefill_tc_kernel, dim3(n_tiles, nh), dim3(AT_THREADS), (size_t)AT_SMEM, stream,
      mq, mk, mv, (__nv_bfloat16*)out, ldo, page_table, table_stride, n_pages, seq_slot, tile_seq, tile_tok0, tile_ntok,
      tile_pos0, n_tiles, nh, nkv, scale_log2, err, g_at_trace);
  EL_LAUNCH_CHECK("attn_prefill_tc");
  return 0;
}
