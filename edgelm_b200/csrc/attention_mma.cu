// Causal attention of many new tokens over the paged cache on the tensor cores (bfloat16 operands,
// float32 scores, softmax and accumulation), flash style: no score matrix ever reaches memory.
//
// grid (query tile, query head); a block of 4 warps owns 64 consecutive new tokens of one sequence
// for one head, 16 rows per warp.  Keys and values are visited page by page (64 positions):
//   * all threads copy the page's K rows and V rows of the head's kv head into shared memory with
//     16-byte cp.async into rows padded by 16 bytes (so that fragment loads hit distinct banks);
//     rows past the block's last key are zero-filled; two stages, so the next page is on its way
//     while this one is computed;
//   * S = Q K^T with mma.sync.m16n8k16: Q fragments stay in registers for the whole kernel, K
//     fragments come by ldmatrix; scale, causal mask, running max and sum per row in float32;
//   * O += P V: the probabilities go from accumulator layout straight to A fragments (rounded to
//     bfloat16), V fragments by ldmatrix.trans.
// A page whose first key lies beyond every row of a warp is skipped by that warp.
// Long rows need more warps than four: with NG warp groups per block, group i visits the pages i,
// i + NG, ... with shared-memory stages of its own and a named barrier of its own; at the end the
// groups' partial (max, sum, output) are merged in shared memory in the order of the groups.
// Takes head sizes 32, 64, 96, 128; others run on the CUDA-core kernel of attention.cu.
#include <math_constants.h>

#include "common.cuh"

namespace edgelm {

constexpr int PM_WARPS = 4;
constexpr int PM_ROWS = 16 * PM_WARPS;  // new tokens per block

__device__ __forceinline__ uint32_t pm_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void pm_mma(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void pm_ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void pm_ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void pm_cp16(uint32_t dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ uint32_t pm_pack(float a, float b) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&v);
}

template <int HDT, int NG>  // head size / 16 (even); warp groups that share the pages of a tile
__global__ void __launch_bounds__(PM_WARPS * 32 * NG)
attn_prefill_mma_kernel(const __nv_bfloat16* __restrict__ q, int ldq, __nv_bfloat16* __restrict__ out, int ldo,
                        const __nv_bfloat16* __restrict__ kcache, const __nv_bfloat16* __restrict__ vcache,
                        const int32_t* __restrict__ page_table, int table_stride, const int32_t* __restrict__ seq_slot,
                        const int32_t* __restrict__ tile_seq, const int32_t* __restrict__ tile_tok0,
                        const int32_t* __restrict__ tile_ntok, const int32_t* __restrict__ tile_pos0, int nh, int nkv,
                        float scale) {
  constexpr int HD = HDT * 16;
  constexpr int PITCH = HD + 8;             // elements: 16 bytes of padding per row
  constexpr int CHUNKS = HD / 8;            // 16-byte chunks per row
  extern __shared__ __align__(16) uint8_t pm_raw[];
  constexpr int STAGE = 2 * PAGE * PITCH;
  const int group = threadIdx.x / (PM_WARPS * 32), gtid = threadIdx.x % (PM_WARPS * 32);
  __nv_bfloat16* sm = reinterpret_cast<__nv_bfloat16*>(pm_raw) + (size_t)group * 2 * STAGE;  // this group's [2 stages][K: 64 x PITCH | V: 64 x PITCH]

  const int tile = blockIdx.x, head = blockIdx.y;
  const int g = nh / nkv, kvh = head / g;
  const int lane = threadIdx.x & 31, warp = (threadIdx.x >> 5) % PM_WARPS, gid = lane >> 2, tig = lane & 3;
  const int seq = tile_seq[tile], tok0 = tile_tok0[tile], ntok = tile_ntok[tile], pos0 = tile_pos0[tile];
  const int32_t* pages = page_table + (size_t)seq_slot[seq] * table_stride;
  const int nkeys_block = pos0 + ntok;      // keys 0 .. pos0 + ntok - 1
  const int n_pages = (nkeys_block + PAGE - 1) / PAGE;
  const int rowA = warp * 16 + gid, rowB = rowA + 8;      // this lane's two rows (token index inside the tile)
  const int limA = rowA < ntok ? pos0 + rowA : -1;         // last key a row may see; -1: no such row
  const int limB = rowB < ntok ? pos0 + rowB : -1;
  const int warp_limit = min(ntok - 1, warp * 16 + 15) >= warp * 16 ? pos0 + min(ntok - 1, warp * 16 + 15) : -1;
  const int warp_min_limit = warp * 16 < ntok ? pos0 + warp * 16 : -1;   // what the warp's first row sees: pages up to here need no mask
  const float scale2 = scale * 1.4426950408889634f;                     // scores in units of log 2

  auto load_page = [&](int pg, int stage) {
    const int page = pages[pg];
    const __nv_bfloat16* kp = kcache + ((size_t)page * nkv + kvh) * PAGE * HD;
    const __nv_bfloat16* vp = vcache + ((size_t)page * nkv + kvh) * PAGE * HD;
    const int valid = min(PAGE, nkeys_block - pg * PAGE);
    __nv_bfloat16* ks = sm + stage * STAGE;
    __nv_bfloat16* vs = ks + PAGE * PITCH;
    for (int i = gtid; i < PAGE * CHUNKS; i += PM_WARPS * 32) {
      const int r = i / CHUNKS, c = i - r * CHUNKS;
      const int bytes = r < valid ? 16 : 0;   // rows past the last key: zero fill, nothing is read
      pm_cp16(pm_smem(ks + r * PITCH + c * 8), kp + r * HD + c * 8, bytes);
      pm_cp16(pm_smem(vs + r * PITCH + c * 8), vp + r * HD + c * 8, bytes);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };

  // Q fragments for the whole kernel
  uint32_t qa[HDT][4];
  {
    const __nv_bfloat16* qA = q + (size_t)(tok0 + min(rowA, ntok - 1)) * ldq + head * HD;
    const __nv_bfloat16* qB = q + (size_t)(tok0 + min(rowB, ntok - 1)) * ldq + head * HD;
#pragma unroll
    for (int ks = 0; ks < HDT; ++ks) {
      const int d = ks * 16 + tig * 2;
      qa[ks][0] = rowA < ntok ? *reinterpret_cast<const uint32_t*>(qA + d) : 0u;
      qa[ks][1] = rowB < ntok ? *reinterpret_cast<const uint32_t*>(qB + d) : 0u;
      qa[ks][2] = rowA < ntok ? *reinterpret_cast<const uint32_t*>(qA + d + 8) : 0u;
      qa[ks][3] = rowB < ntok ? *reinterpret_cast<const uint32_t*>(qB + d + 8) : 0u;
    }
  }
  float o[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float mA = -CUDART_INF_F, mB = -CUDART_INF_F, lA = 0.f, lB = 0.f;

  auto group_sync = [&]() {   // the 128 threads of this group (barrier 0 is __syncthreads)
    if (NG == 1) __syncthreads();
    else asm volatile("bar.sync %0, %1;" ::"r"(group + 1), "r"(PM_WARPS * 32) : "memory");
  };
  if (group < n_pages) load_page(group, 0);
  for (int pg = group, it = 0; pg < n_pages; pg += NG, ++it) {
    const int stage = it & 1;
    if (pg + NG < n_pages) {
      load_page(pg + NG, stage ^ 1);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    group_sync();
    if (pg * PAGE <= warp_limit) {   // else: no row of this warp sees this page
      const __nv_bfloat16* ks = sm + stage * STAGE;
      const __nv_bfloat16* vs = ks + PAGE * PITCH;
      // ---- S = Q K^T : 8 tiles of 8 keys
      float s[8][4];
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
        for (int ks2 = 0; ks2 < HDT; ks2 += 2) {
          // four 8x8 matrices: (keys nt*8.., d block ks2*16), (.., +8), (.., (ks2+1)*16), (.., +8)
          const int mi = lane >> 3;
          const uint32_t addr = pm_smem(ks + (nt * 8 + (lane & 7)) * PITCH + (ks2 + (mi >> 1)) * 16 + (mi & 1) * 8);
          uint32_t b0, b1, b2, b3;
          pm_ldmatrix_x4(addr, b0, b1, b2, b3);
          pm_mma(s[nt], qa[ks2][0], qa[ks2][1], qa[ks2][2], qa[ks2][3], b0, b1);
          pm_mma(s[nt], qa[ks2 + 1][0], qa[ks2 + 1][1], qa[ks2 + 1][2], qa[ks2 + 1][3], b2, b3);
        }
      }
      // ---- scale, causal mask, running max and sum (float32).  Scores are kept in units of log 2
      // (scale * log2(e) folded into one multiply), so that the exponentials are bare exp2; a page that
      // every row of the warp sees in full needs no mask.
      const bool masked = pg * PAGE + PAGE - 1 > warp_min_limit;
      float mxA = -CUDART_INF_F, mxB = -CUDART_INF_F;
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        const int key = pg * PAGE + nt * 8 + tig * 2;
        if (masked) {
          s[nt][0] = key <= limA ? s[nt][0] * scale2 : -CUDART_INF_F;
          s[nt][1] = key + 1 <= limA ? s[nt][1] * scale2 : -CUDART_INF_F;
          s[nt][2] = key <= limB ? s[nt][2] * scale2 : -CUDART_INF_F;
          s[nt][3] = key + 1 <= limB ? s[nt][3] * scale2 : -CUDART_INF_F;
        } else {
          s[nt][0] *= scale2;
          s[nt][1] *= scale2;
          s[nt][2] *= scale2;
          s[nt][3] *= scale2;
        }
        mxA = fmaxf(mxA, fmaxf(s[nt][0], s[nt][1]));
        mxB = fmaxf(mxB, fmaxf(s[nt][2], s[nt][3]));
      }
      mxA = fmaxf(mxA, __shfl_xor_sync(0xffffffffu, mxA, 1));
      mxA = fmaxf(mxA, __shfl_xor_sync(0xffffffffu, mxA, 2));
      mxB = fmaxf(mxB, __shfl_xor_sync(0xffffffffu, mxB, 1));
      mxB = fmaxf(mxB, __shfl_xor_sync(0xffffffffu, mxB, 2));
      const float nmA = fmaxf(mA, mxA), nmB = fmaxf(mB, mxB);
      const float refA = nmA == -CUDART_INF_F ? 0.f : nmA, refB = nmB == -CUDART_INF_F ? 0.f : nmB;  // a row that sees no key yet
      const float corrA = exp2f(mA - refA), corrB = exp2f(mB - refB);  // exp2(-inf) = 0 on the first page
      float sumA = 0.f, sumB = 0.f;
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        s[nt][0] = exp2f(s[nt][0] - refA);
        s[nt][1] = exp2f(s[nt][1] - refA);
        s[nt][2] = exp2f(s[nt][2] - refB);
        s[nt][3] = exp2f(s[nt][3] - refB);
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
      if (__any_sync(0xffffffffu, corrA != 1.f || corrB != 1.f)) {   // some row's maximum moved: rescale what is gathered
#pragma unroll
        for (int i = 0; i < HD / 8; ++i) {
          o[i][0] *= corrA;
          o[i][1] *= corrA;
          o[i][2] *= corrB;
          o[i][3] *= corrB;
        }
      }
      // ---- O += P V : 4 steps of 16 keys
#pragma unroll
      for (int kt = 0; kt < 4; ++kt) {
        const uint32_t a0 = pm_pack(s[2 * kt][0], s[2 * kt][1]), a1 = pm_pack(s[2 * kt][2], s[2 * kt][3]);
        const uint32_t a2 = pm_pack(s[2 * kt + 1][0], s[2 * kt + 1][1]), a3 = pm_pack(s[2 * kt + 1][2], s[2 * kt + 1][3]);
#pragma unroll
        for (int dt = 0; dt < HD / 8; dt += 2) {
          // transposed 8x8 matrices: (keys kt*16.., d block dt), (keys +8, dt), (keys kt*16.., dt+1), (keys +8, dt+1)
          const int mi = lane >> 3;
          const uint32_t addr = pm_smem(vs + (kt * 16 + (mi & 1) * 8 + (lane & 7)) * PITCH + (dt + (mi >> 1)) * 8);
          uint32_t b0, b1, b2, b3;
          pm_ldmatrix_x4_trans(addr, b0, b1, b2, b3);
          pm_mma(o[dt], a0, a1, a2, a3, b0, b1);
          pm_mma(o[dt + 1], a0, a1, a2, a3, b2, b3);
        }
      }
    }
    group_sync();  // this stage is free for the page after next
  }
  if (NG > 1) {
    // ---- merge the groups: groups 1.. leave (max, sum, output) in shared memory, group 0 folds them in order
    __syncthreads();
    float* mg = reinterpret_cast<float*>(pm_raw);            // [NG - 1][64 rows][HD + 2]
    constexpr int MP = HD + 2;
    if (group > 0) {
      float* a = mg + ((size_t)(group - 1) * PM_ROWS + rowA) * MP;
      float* b = mg + ((size_t)(group - 1) * PM_ROWS + rowB) * MP;
#pragma unroll
      for (int dt = 0; dt < HD / 8; ++dt) {
        a[dt * 8 + tig * 2] = o[dt][0];
        a[dt * 8 + tig * 2 + 1] = o[dt][1];
        b[dt * 8 + tig * 2] = o[dt][2];
        b[dt * 8 + tig * 2 + 1] = o[dt][3];
      }
      if (tig == 0) {
        a[HD] = mA;
        a[HD + 1] = lA;
        b[HD] = mB;
        b[HD + 1] = lB;
      }
    }
    __syncthreads();
    if (group > 0) return;
    for (int gsrc = 1; gsrc < NG; ++gsrc) {
      const float* a = mg + ((size_t)(gsrc - 1) * PM_ROWS + rowA) * MP;
      const float* b = mg + ((size_t)(gsrc - 1) * PM_ROWS + rowB) * MP;
      const float nmA = fmaxf(mA, a[HD]), nmB = fmaxf(mB, b[HD]);
      const float refA = nmA == -CUDART_INF_F ? 0.f : nmA, refB = nmB == -CUDART_INF_F ? 0.f : nmB;
      const float fA0 = exp2f(mA - refA), fA1 = exp2f(a[HD] - refA), fB0 = exp2f(mB - refB), fB1 = exp2f(b[HD] - refB);
      lA = lA * fA0 + a[HD + 1] * fA1;
      lB = lB * fB0 + b[HD + 1] * fB1;
      mA = nmA;
      mB = nmB;
#pragma unroll
      for (int dt = 0; dt < HD / 8; ++dt) {
        o[dt][0] = o[dt][0] * fA0 + a[dt * 8 + tig * 2] * fA1;
        o[dt][1] = o[dt][1] * fA0 + a[dt * 8 + tig * 2 + 1] * fA1;
        o[dt][2] = o[dt][2] * fB0 + b[dt * 8 + tig * 2] * fB1;
        o[dt][3] = o[dt][3] * fB0 + b[dt * 8 + tig * 2 + 1] * fB1;
      }
    }
  }
  const float invA = 1.0f / lA, invB = 1.0f / lB;
#pragma unroll
  for (int dt = 0; dt < HD / 8; ++dt) {
    const int d = head * HD + dt * 8 + tig * 2;
    if (rowA < ntok) *reinterpret_cast<uint32_t*>(out + (size_t)(tok0 + rowA) * ldo + d) = pm_pack(o[dt][0] * invA, o[dt][1] * invA);
    if (rowB < ntok) *reinterpret_cast<uint32_t*>(out + (size_t)(tok0 + rowB) * ldo + d) = pm_pack(o[dt][2] * invB, o[dt][3] * invB);
  }
}

template <int HDT, int NG>
static int launch_prefill_mma_ng(const void* q, int ldq, void* out, int ldo, const void* kc, const void* vc,
                                 const int32_t* page_table, int table_stride, const int32_t* seq_slot, const int32_t* tile_seq,
                                 const int32_t* tile_tok0, const int32_t* tile_ntok, const int32_t* tile_pos0, int n_tiles,
                                 int nh, int nkv, float scale, cudaStream_t stream) {
  constexpr int HD = HDT * 16;
  const size_t smem = (size_t)NG * 2 * 2 * PAGE * (HD + 8) * 2;
  auto kern = attn_prefill_mma_kernel<HDT, NG>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) {
    set_error("attn_prefill_mma: %zu bytes of shared memory refused: %s", smem, cudaGetErrorString(e));
    return -2;
  }
  dim3 grid(n_tiles, nh);
  kern<<<grid, PM_WARPS * 32 * NG, smem, stream>>>((const __nv_bfloat16*)q, ldq, (__nv_bfloat16*)out, ldo, (const __nv_bfloat16*)kc,
                                                  (const __nv_bfloat16*)vc, page_table, table_stride, seq_slot, tile_seq, tile_tok0,
                                                  tile_ntok, tile_pos0, nh, nkv, scale);
  return 0;
}

// Warp groups per block: one when the grid fills the device by itself or rows are short; two or four when
// few blocks walk many pages each (a single long prompt).
static int prefill_groups(int n_tiles, int nh, int max_keys, int hd, int force) {
  if (force == 1 || force == 2 || force == 4) return (force == 4 && hd > 64) ? 2 : force;
  const long long blocks = (long long)n_tiles * nh;
  const int pages = (max_keys + PAGE - 1) / PAGE;
  if (pages >= 16 && blocks < 2 * 148 * 2 && hd <= 64) return 4;
  if (pages >= 6 && blocks < 4 * 148 * 2) return 2;
  return 1;
}

template <int HDT>
static int launch_prefill_mma(int groups, const void* q, int ldq, void* out, int ldo, const void* kc, const void* vc,
                              const int32_t* page_table, int table_stride, const int32_t* seq_slot, const int32_t* tile_seq,
                              const int32_t* tile_tok0, const int32_t* tile_ntok, const int32_t* tile_pos0, int n_tiles,
                              int nh, int nkv, float scale, cudaStream_t stream) {
#define EL_PM(NG) launch_prefill_mma_ng<HDT, NG>(q, ldq, out, ldo, kc, vc, page_table, table_stride, seq_slot, tile_seq, tile_tok0, tile_ntok, tile_pos0, n_tiles, nh, nkv, scale, stream)
  if (groups == 4) {
    if constexpr (HDT <= 4) return EL_PM(4);
    else return EL_PM(2);
  }
  if (groups == 2) return EL_PM(2);
  return EL_PM(1);
#undef EL_PM
}

}  // namespace edgelm

using namespace edgelm;

// Tokens per tile that the host must cut sequences into for this kernel.
extern "C" int edgelm_attn_prefill_mma_tile_tokens() { return PM_ROWS; }

// 1 if the tensor-core prefill kernel takes this head size, else 0.
extern "C" int edgelm_attn_prefill_mma_takes(int hd) { return (hd == 32 || hd == 64 || hd == 96 || hd == 128) ? 1 : 0; }

// Tiles of at most 64 new tokens of one sequence each (tile_ntok <= 64); bfloat16 only.  q and out rows
// must be 4-byte aligned (even ldq, ldo); the cache as in attention.cu.
extern "C" int edgelm_attn_prefill_mma(const void* q, int ldq, void* out, int ldo, const void* kcache, const void* vcache,
                                       const int32_t* page_table, int table_stride, const int32_t* seq_slot,
                                       const int32_t* tile_seq, const int32_t* tile_tok0, const int32_t* tile_ntok,
                                       const int32_t* tile_pos0, int n_tiles, int nh, int nkv, int hd, float scale,
                                       int max_keys, int force_groups, cudaStream_t stream) {
  // max_keys: the most keys a tile attends over (a hint for how many warp groups share a tile's pages);
  // force_groups: 0 to choose, or 1, 2, 4.
  if (n_tiles == 0) return 0;
  EL_REFUSE(nh > 0 && nkv > 0 && nh % nkv == 0, "attn_prefill_mma: %d query heads are not a multiple of %d key/value heads", nh, nkv);
  EL_REFUSE(edgelm_attn_prefill_mma_takes(hd), "attn_prefill_mma: head size %d (takes 32, 64, 96, 128)", hd);
  EL_REFUSE(ldq % 2 == 0 && ldo % 2 == 0 && (uintptr_t)q % 4 == 0 && (uintptr_t)out % 4 == 0, "attn_prefill_mma: rows must be 4-byte aligned");
  EL_REFUSE(n_tiles > 0 && nh <= 65535, "attn_prefill_mma: bad grid");
  const int groups = prefill_groups(n_tiles, nh, max_keys, hd, force_groups);
  int rc = 0;
  switch (hd / 16) {
    case 2: rc = launch_prefill_mma<2>(groups, q, ldq, out, ldo, kcache, vcache, page_table, table_stride, seq_slot, tile_seq, tile_tok0, tile_ntok, tile_pos0, n_tiles, nh, nkv, scale, stream); break;
    case 4: rc = launch_prefill_mma<4>(groups, q, ldq, out, ldo, kcache, vcache, page_table, table_stride, seq_slot, tile_seq, tile_tok0, tile_ntok, tile_pos0, n_tiles, nh, nkv, scale, stream); break;
    case 6: rc = launch_prefill_mma<6>(groups, q, ldq, out, ldo, kcache, vcache, page_table, table_stride, seq_slot, tile_seq, tile_tok0, tile_ntok, tile_pos0, n_tiles, nh, nkv, scale, stream); break;
    case 8: rc = launch_prefill_mma<8>(groups, q, ldq, out, ldo, kcache, vcache, page_table, table_stride, seq_slot, tile_seq, tile_tok0, tile_ntok, tile_pos0, n_tiles, nh, nkv, scale, stream); break;
  }
  if (rc) return rc;
  EL_LAUNCH_CHECK("attn_prefill_mma");
  return 0;
}
