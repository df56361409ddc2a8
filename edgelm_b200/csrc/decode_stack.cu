// A run of decoder layers for one decode step of a few sequences, as ONE persistent kernel.
//
// With one token per sequence and at most 16 sequences every kernel of a layer is a few
// microseconds of memory latency, and a step of a small model is a chain of some two hundred such
// kernels: what it costs is the launches and the cold start of each, not the bytes.  Here one block
// per SM stays resident for the whole run of layers (a cooperative launch, so that all blocks are
// on the device together) and the layers' phases are separated by barriers across the grid, about
// 1.5 microseconds each, instead of kernel boundaries:
//
//   1. qkv  = RMSNorm(x) Wqkv^T                           few-rows product, 16 output columns a unit
//   2. attention of the new token over the cache          unit = (sequence, kv head, chunk of pages);
//      rotation of q and k and the append of k, v fused; every unit leaves its unnormalised sum,
//      its maximum and its denominator
//   3. x   += att Wo^T, att = the units' results folded (in the order of the chunks) and rounded to
//      bfloat16 while they are staged as the product's input
//   4. mid  = silu(RMSNorm(x) Wg^T) * (RMSNorm(x) Wu^T)
//   5. x   += mid Wd^T
//
// The arithmetic is that of the stand-alone kernels (gemv_mma.cu, attention_decode_mma.cuh): weights
// as the 16-row operand of mma.sync.m16n8k16 loaded straight from global memory, the batch as its
// columns, float32 accumulation, norms and softmax in float32, the residual stream in float32.
// Everything a phase reads that an earlier phase wrote is read through L2 (ld.global.cg) after the
// barrier's acquire; weights and tables, which nothing writes, go through the read-only path.
//
// What separate kernels cannot do and this one does: loads that do not depend on the step's own
// arithmetic start a phase early.  The cache tiles of a layer's attention (all but the new token's row,
// which is patched in from shared memory) are requested as soon as the block's tile buffers are free,
// one layer ahead; the first weights of a block's next matrix product go into a staging buffer in
// shared memory while the block finishes the current phase and waits at the barrier.  After a barrier
// a phase then only waits for the few activations it reads from L2.
//
// Every wait is bounded: a barrier that is not complete after DS_WAIT_CYCLES sets ERR_WAIT_TIMEOUT in
// the error word, which makes every other block leave its barrier too, and the kernel returns.
//
// Layers are described by records (StackLayer) in device memory, so that layers may differ in head
// counts, feed-forward width, eps, tables and cache; the head size and the residual width are the
// launch's.  bfloat16 weights and cache; head size 32, 64, 96 or 128; widths multiples of 8.
#include <math_constants.h>

#include "attention_tile_mma.cuh"
#include "common.cuh"

namespace edgelm {

struct StackLayer {
  const __nv_bfloat16* w_qkv;    // [(nh + 2 nkv) hd, D]
  const __nv_bfloat16* w_o;      // [D, nh hd]
  const __nv_bfloat16* w_gate;   // [inter, D]
  const __nv_bfloat16* w_up;     // [inter, D]
  const __nv_bfloat16* w_down;   // [D, inter]
  const float* norm1_w;          // [D]
  const float* norm2_w;          // [D]
  const float* cos_t;            // [max_pos, hd / 2]
  const float* sin_t;
  __nv_bfloat16* kcache;         // [pages][nkv][64][hd]
  __nv_bfloat16* vcache;
  const int32_t* page_table;     // [slots][table_stride]
  int nh, nkv, inter, table_stride, max_pos, n_pages;
  float eps1, eps2, scale;
  int pad;
};
static_assert(sizeof(StackLayer) == 136, "the host packs records of 136 bytes");

constexpr int DS_WARPS = 8;
constexpr int DS_THREADS = DS_WARPS * 32;
constexpr int DS_COLS = 16;        // output columns of a unit of a matrix product
constexpr int DS_K_CHUNK = 4096;   // columns of the activations in shared memory at a time
constexpr int DS_RESERVED = 256;   // head of shared memory: the mbarriers (warps' tiles, weight stage) and two flags
constexpr long long DS_WAIT_CYCLES = 2000000000LL;
constexpr int DS_MAX_SMEM = 227 * 1024;

enum : int { DS_STORE = 0, DS_RESIDUAL = 1, DS_SWIGLU = 2 };
enum : int { DS_SRC_ACT = 0, DS_SRC_NORM = 1, DS_SRC_FOLD = 2 };   // a product's input: bfloat16 rows, RMSNorm(x), attention partials

__device__ __forceinline__ unsigned ds_ld_acquire(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void ds_red_release(unsigned* p, unsigned v) {
  asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ __nv_bfloat16 ds_ld_bf16(const __nv_bfloat16* p) {   // through L2: another block wrote it
  const unsigned short u = __ldcg(reinterpret_cast<const unsigned short*>(p));
  return __ushort_as_bfloat16(u);
}
__device__ __forceinline__ float ds_silu(float z) { return z / (1.0f + expf(-z)); }

__host__ __device__ inline int ds_round_up(int v, int a) { return (v + a - 1) / a * a; }
// Activation row pitch (elements): pitch * 2 bytes = 64 (mod 128), so that the fragment reads of a
// quarter-warp hit distinct banks.
__host__ __device__ inline int ds_pitch(int kc) {
  int p = ds_round_up(kc, 8);
  while ((p * 2) % 128 != 64) p += 8;
  return p;
}
__host__ __device__ inline int ds_kc(int K) { return K <= DS_K_CHUNK ? ds_round_up(K, 32) : DS_K_CHUNK; }
__host__ __device__ inline size_t ds_gemv_bytes(int K, int NT) {   // partial sums, norm factors, activations
  const size_t b = (size_t)DS_WARPS * 2 * NT * 128 * 4 + 64 + (size_t)8 * NT * ds_pitch(ds_kc(K)) * 2;
  return (b + 127) / 128 * 128;
}
__host__ __device__ inline size_t ds_attn_head_bytes(int hd) {   // queries [16][hd + 8], the new key and value
  return ((size_t)DM_ROWS * (hd + 8) * 2 + 2 * (size_t)hd * 2 + 127) / 128 * 128;
}
__host__ __device__ inline size_t ds_attn_warp_bytes(int hd) { return (size_t)2 * PAGE * (hd + 8) * 2; }

// Shared memory: [reserved | matrix products' scratch | attention head | weight stage | tiles of the attention warps].
struct StackPlan {
  int att_warps;     // warps with a key and a value tile each = pages of an attention unit
  int w_bytes;       // the weight stage
  size_t total;
};
__host__ __device__ inline int ds_w_rows_bytes(int NW, int K) { return NW * DS_COLS * ds_pitch(K) * 2; }
inline StackPlan ds_plan(int hd, int max_k, int NT) {
  StackPlan p = {0, 0, 0};
  const long fixed = DS_RESERVED + (long)ds_gemv_bytes(max_k, NT) + (long)ds_attn_head_bytes(hd);
  const long room = (long)DS_MAX_SMEM - fixed;
  const long warp = (long)ds_attn_warp_bytes(hd);
  if (room < warp) return p;
  // the stage wants a weight's 16 rows over the widest input (which also holds two weights over an input
  // half as wide), at most 64 KB, and leaves six warps their tiles if it can; at least 16 KB
  long want = ds_w_rows_bytes(1, max_k);
  if (want > 64 * 1024) want = 64 * 1024;
  long w = room - 6 * warp;
  if (w > want) w = want;
  if (w < 16 * 1024) w = room - warp >= 16 * 1024 ? 16 * 1024 : 0;
  w = (w + 127) / 128 * 128;
  if (w + warp > room) w = 0;
  long warps = (room - w) / warp;
  if (warps > DS_WARPS) warps = DS_WARPS;
  p.att_warps = (int)warps;
  p.w_bytes = (int)w;
  p.total = (size_t)(fixed + w + warps * warp);
  return p;
}

// Barrier across the grid, in two halves so that a block can issue loads that depend on no other block
// between its arrival and its wait.  `target` counts the arrivals that all barriers so far add up to.
__device__ __forceinline__ void ds_grid_arrive(unsigned* bar, unsigned& target) {
  target += gridDim.x;
  __syncthreads();
  if (threadIdx.x == 0) ds_red_release(bar, 1u);   // (the release orders what the block wrote before its barrier; a
  // fence before it cost 0.3 us a barrier, and four counters instead of one made the wait slower: 2.1 against 1.3 us)
}
// False: the wait ran out, or another block's did.
__device__ __forceinline__ bool ds_grid_wait(unsigned* bar, unsigned target, int* err, volatile int* dead) {
  if (threadIdx.x == 0) {
    const long long t0 = clock64();
    int spins = 0;
    while (ds_ld_acquire(bar) < target) {
      if ((++spins & 255) == 0 && (clock64() - t0 > DS_WAIT_CYCLES || (*reinterpret_cast<volatile int*>(err) & ERR_WAIT_TIMEOUT))) {
        atomicOr(err, ERR_WAIT_TIMEOUT);
        *dead = 1;
        break;
      }
    }
  }
  __syncthreads();   // (the acquire of the last load orders what the block reads from here on)
  return *dead == 0;
}
__device__ __forceinline__ bool ds_grid_barrier(unsigned* bar, unsigned& target, int* err, volatile int* dead) {
  ds_grid_arrive(bar, target);
  return ds_grid_wait(bar, target, err, dead);
}

// ---------------------------------------------------------------- few-rows matrix product, one phase
// A phase's weights: out[M, N] = act[M, K] . W[N, K]^T; W2 is SwiGLU's second weight.
struct GemvW {
  const __nv_bfloat16* W;
  const __nv_bfloat16* W2;   // null: one weight
  int N, K;
};

// The weight stage: the 16 (or 2 x 16) weight rows of a block's first unit of its next matrix product,
// columns [0, kpre), rows padded like the activations.  One mbarrier; `parity` flips with every wait.
struct WStage {
  __nv_bfloat16* buf;
  int bytes;
  uint32_t bar;
  uint32_t parity;
};
__device__ __forceinline__ int ds_w_kpre(int stage_bytes, int NW, int K) {
  if (ds_w_rows_bytes(NW, K) <= stage_bytes) return K;
  int k = stage_bytes / (NW * DS_COLS * 2) - 64;   // the padding adds at most 56 elements a row
  return k < 32 ? 0 : k / 32 * 32;
}
__device__ __forceinline__ bool ds_mbar_try(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool ds_mbar_wait(uint32_t bar, uint32_t parity) {   // bounded; whole warps call it
  const long long t0 = clock64();
  bool done = ds_mbar_try(bar, parity);
  while (!done) {
    done = ds_mbar_try(bar, parity);
    if (!done && clock64() - t0 > DS_WAIT_CYCLES) break;
  }
  return __all_sync(0xffffffffu, done);
}

// One warp requests the rows of unit `blockIdx.x` of the matrix product `g` (nothing if the block has no unit).
__device__ __forceinline__ void ds_w_issue(const WStage& ws, const GemvW& g) {
  const int NW = g.W2 ? 2 : 1;
  const int n_units = (g.N + DS_COLS - 1) / DS_COLS;
  const int kpre = ds_w_kpre(ws.bytes, NW, g.K);
  if ((int)blockIdx.x >= n_units || kpre == 0) return;
  const int lane = threadIdx.x & 31, pitch = ds_pitch(kpre);
  if (lane == 0) {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(ws.bar), "r"((uint32_t)(NW * DS_COLS * kpre * 2)) : "memory");
  }
  __syncwarp();
  const int w = lane >> 4, row = lane & 15;
  if (w < NW) {
    const __nv_bfloat16* src = (w ? g.W2 : g.W) + (size_t)min((int)blockIdx.x * DS_COLS + row, g.N - 1) * g.K;
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dm_smem_u32(ws.buf + (size_t)(w * DS_COLS + row) * pitch)), "l"(src), "r"((uint32_t)(kpre * 2)), "r"(ws.bar) : "memory");
  }
}

// The attention units' results of a step: per (sequence, head, chunk) the unnormalised sum [hd], the maximum and
// the denominator.  A sequence has ceil(pages / chunk_pages) chunks.
struct FoldSrc {
  const float* part_o;
  const float* part_ml;
  const int* s_pos;     // shared memory: the sequences' last positions
  int max_chunks, hd, chunk_pages, table_stride;
};

// out[M, N] = act[M, K] . W[N, K]^T; units of 16 columns over the blocks.  act: bfloat16 rows (DS_SRC_ACT),
// RMSNorm(x) (DS_SRC_NORM) or the attention units' results folded and normalised (DS_SRC_FOLD, K = heads x hd).
// `next`: the block's following matrix product, whose first rows are requested once the stage is free.
template <int EPI, typename TOut, int NT, int SRC>
__device__ __forceinline__ void ds_gemv(uint8_t* work, WStage& ws, const __nv_bfloat16* act, int lda, const float* x,
                                        const float* __restrict__ norm_w, float eps, const FoldSrc* fold, const GemvW g,
                                        TOut* out, int ldo, const float* residual, int M, const GemvW* next, int* err) {
  constexpr bool NORM = SRC == DS_SRC_NORM;
  constexpr int NW = EPI == DS_SWIGLU ? 2 : 1;
  constexpr int ROWS = 8 * NT;
  const __nv_bfloat16* __restrict__ W = g.W;
  const __nv_bfloat16* __restrict__ W2 = g.W2;
  const int N = g.N, K = g.K;
  const int n_units = (N + DS_COLS - 1) / DS_COLS;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, gid = lane >> 2, tig = lane & 3;
  if ((int)blockIdx.x >= n_units) {   // no unit here: only the request for the next product
    if (next != nullptr && warp == 1) ds_w_issue(ws, *next);
    return;
  }
  float* red = reinterpret_cast<float*>(work);                          // [DS_WARPS][2][NT][32][4]
  float* inv = red + DS_WARPS * 2 * NT * 128;                           // [16]
  __nv_bfloat16* As = reinterpret_cast<__nv_bfloat16*>(inv + 16);       // [ROWS][pitch]
  const int kc = ds_kc(K), pitch = ds_pitch(kc);
  const int n_kb = (K + 31) / 32;
  const int kpre = ds_w_kpre(ws.bytes, NW, K), wpitch = ds_pitch(kpre);
  constexpr int ONE_PASS_K = 1024;   // up to here a lane keeps its share of a row in registers between the sum and the scaling

  int staged = -1;
  if (NORM && K <= ONE_PASS_K) {
    // a warp per row: one read of the row, the sum of squares by shuffles, the scaled row into shared memory
    for (int r = warp; r < ROWS; r += DS_WARPS) {
      float4 v[ONE_PASS_K / 128], w4[ONE_PASS_K / 128];
      float ss = 0.f;
#pragma unroll
      for (int j = 0; j < ONE_PASS_K / 128; ++j) {   // the row and the norm's weights in one round of loads
        const int k = lane * 4 + j * 128;
        const bool ok = r < M && k < K;
        v[j] = ok ? __ldcg(reinterpret_cast<const float4*>(x + (size_t)r * K + k)) : make_float4(0.f, 0.f, 0.f, 0.f);
        w4[j] = ok ? *reinterpret_cast<const float4*>(norm_w + k) : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int j = 0; j < ONE_PASS_K / 128; ++j) {
        ss = fmaf(v[j].x, v[j].x, ss); ss = fmaf(v[j].y, v[j].y, ss); ss = fmaf(v[j].z, v[j].z, ss); ss = fmaf(v[j].w, v[j].w, ss);
      }
      ss = warp_sum(ss);
      const float sc = 1.0f / sqrtf(ss / (float)K + eps);
#pragma unroll
      for (int j = 0; j < ONE_PASS_K / 128; ++j) {
        const int k = lane * 4 + j * 128;
        if (k < K) {
          uint2 h = make_uint2(0u, 0u);
          if (r < M) {
            h.x = dm_pack(v[j].x * sc * w4[j].x, v[j].y * sc * w4[j].y);
            h.y = dm_pack(v[j].z * sc * w4[j].z, v[j].w * sc * w4[j].w);
          }
          *reinterpret_cast<uint2*>(As + (size_t)r * pitch + k) = h;
        }
      }
    }
    staged = 0;
    __syncthreads();
  } else if (NORM) {
    for (int r = warp; r < ROWS; r += DS_WARPS) {
      float ss = 0.f;
      if (r < M) {
        const float* xr = x + (size_t)r * K;
        for (int k = lane * 4; k < K; k += 128) {
          const float4 v = __ldcg(reinterpret_cast<const float4*>(xr + k));
          ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
        }
      }
      ss = warp_sum(ss);
      if (lane == 0) inv[r] = 1.0f / sqrtf(ss / (float)K + eps);
    }
  }
  constexpr int UN = 4;  // K blocks whose weight loads are in flight together
  bool first = true;
  for (int u = blockIdx.x; u < n_units; u += gridDim.x) {
    const int n0 = u * DS_COLS;
    const int ra = min(n0 + gid, N - 1), rb = min(n0 + gid + 8, N - 1);   // the two weight rows of this lane (clamped)
    const int kst = first ? kpre : 0;   // columns below this come from the stage
    // this warp's first K block of weights that the stage does not hold: on its way while the activations are staged
    uint4 pa[NW], pb[NW];
    const int kb_first = kst / 32 + warp;
    {
      const int k = kb_first * 32 + tig * 8;
      const bool ok = kb_first < n_kb && k < K && k >= kst;
#pragma unroll
      for (int w = 0; w < NW; ++w) {
        const __nv_bfloat16* Wp = w == 0 ? W : W2;
        pa[w] = ok ? *reinterpret_cast<const uint4*>(Wp + (size_t)ra * K + k) : make_uint4(0, 0, 0, 0);
        pb[w] = ok ? *reinterpret_cast<const uint4*>(Wp + (size_t)rb * K + k) : make_uint4(0, 0, 0, 0);
      }
    }
    float acc[NW][NT][4];
#pragma unroll
    for (int w = 0; w < NW; ++w)
#pragma unroll
      for (int t = 0; t < NT; ++t)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[w][t][j] = 0.f;

    for (int kc0 = 0; kc0 < K; kc0 += kc) {
      const int kn = min(kc, K - kc0);
      if (staged != kc0) {   // (one chunk for the usual sizes: staged once for all of the block's units)
        __syncthreads();     // the norm's factors are there; the chunk staged before is used up
        const int kvec = kn / 8;
        if (SRC == DS_SRC_ACT) {
          // four 16-byte loads of a thread in flight together, then their four stores
          for (int i0 = threadIdx.x; i0 < ROWS * kvec; i0 += DS_THREADS * 4) {
            uint4 v[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int i = i0 + j * DS_THREADS, r = i / kvec, k = kc0 + (i - r * kvec) * 8;
              v[j] = (i < ROWS * kvec && r < M) ? __ldcg(reinterpret_cast<const uint4*>(act + (size_t)r * lda + k)) : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int i = i0 + j * DS_THREADS, r = i / kvec, k = (i - r * kvec) * 8;
              if (i < ROWS * kvec) *reinterpret_cast<uint4*>(As + (size_t)r * pitch + k) = v[j];
            }
          }
        } else {
          for (int i = threadIdx.x; i < ROWS * kvec; i += DS_THREADS) {
            const int r = i / kvec, k = kc0 + (i - r * kvec) * 8;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (r < M) {
              if (NORM) {
                const float s = inv[r];
                const float4 x0 = __ldcg(reinterpret_cast<const float4*>(x + (size_t)r * K + k));
                const float4 x1 = __ldcg(reinterpret_cast<const float4*>(x + (size_t)r * K + k + 4));
                const float4 w0 = *reinterpret_cast<const float4*>(norm_w + k);
                const float4 w1 = *reinterpret_cast<const float4*>(norm_w + k + 4);
                v.x = dm_pack(x0.x * s * w0.x, x0.y * s * w0.y);
                v.y = dm_pack(x0.z * s * w0.z, x0.w * s * w0.w);
                v.z = dm_pack(x1.x * s * w1.x, x1.y * s * w1.y);
                v.w = dm_pack(x1.z * s * w1.z, x1.w * s * w1.w);
              } else {   // DS_SRC_FOLD: the chunks' results, four chunks' loads in flight together, folded in their order
                const int head = k / fold->hd, d = k - head * fold->hd, nh = K / fold->hd;
                const int n_pages = max(1, min((fold->s_pos[r] + PAGE) / PAGE, fold->table_stride));
                const int n_chunks = (n_pages + fold->chunk_pages - 1) / fold->chunk_pages;
                const size_t p0 = ((size_t)r * nh + head) * fold->max_chunks;
                float Mx = -CUDART_INF_F, Ls = 0.f, o[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) o[j] = 0.f;
                for (int c0 = 0; c0 < n_chunks; c0 += 4) {
                  float2 ml[4];
                  float4 a0[4], a1[4];
#pragma unroll
                  for (int j = 0; j < 4; ++j) {
                    const bool ok = c0 + j < n_chunks;
                    const size_t pc = p0 + (ok ? c0 + j : c0);
                    ml[j] = __ldcg(reinterpret_cast<const float2*>(fold->part_ml + pc * 2));
                    a0[j] = __ldcg(reinterpret_cast<const float4*>(fold->part_o + pc * fold->hd + d));
                    a1[j] = __ldcg(reinterpret_cast<const float4*>(fold->part_o + pc * fold->hd + d + 4));
                  }
#pragma unroll
                  for (int j = 0; j < 4; ++j) {
                    if (c0 + j < n_chunks) {
                      const float nm = fmaxf(Mx, ml[j].x);
                      const float fo = expf(Mx - nm), fc = expf(ml[j].x - nm);
                      Ls = Ls * fo + ml[j].y * fc;
                      o[0] = o[0] * fo + a0[j].x * fc; o[1] = o[1] * fo + a0[j].y * fc; o[2] = o[2] * fo + a0[j].z * fc; o[3] = o[3] * fo + a0[j].w * fc;
                      o[4] = o[4] * fo + a1[j].x * fc; o[5] = o[5] * fo + a1[j].y * fc; o[6] = o[6] * fo + a1[j].z * fc; o[7] = o[7] * fo + a1[j].w * fc;
                      Mx = nm;
                    }
                  }
                }
                const float il = 1.0f / Ls;
                v.x = dm_pack(o[0] * il, o[1] * il);
                v.y = dm_pack(o[2] * il, o[3] * il);
                v.z = dm_pack(o[4] * il, o[5] * il);
                v.w = dm_pack(o[6] * il, o[7] * il);
              }
            }
            *reinterpret_cast<uint4*>(As + (size_t)r * pitch + (k - kc0)) = v;
          }
        }
        __syncthreads();
        staged = kc0;
      }
      if (first && kc0 == 0 && kpre > 0) {   // the staged rows have arrived (requested a phase ago)
        if (!ds_mbar_wait(ws.bar, ws.parity) && lane == 0) atomicOr(err, ERR_WAIT_TIMEOUT);
        ws.parity ^= 1;
      }
      const int kb_begin = kc0 / 32, kb_end = (kc0 + kn + 31) / 32;
      // ---- K blocks in the stage (lanes past its end, in a last partial block, feed zeros)
      for (int kb = kb_begin + warp; kb < kb_end && kb * 32 < kst; kb += DS_WARPS) {
        const int k = kb * 32 + tig * 8;
        const bool ok = k < kst;
        uint4 wa[NW], wb[NW];
#pragma unroll
        for (int w = 0; w < NW; ++w) {
          wa[w] = ok ? *reinterpret_cast<const uint4*>(ws.buf + (size_t)(w * DS_COLS + gid) * wpitch + k) : make_uint4(0, 0, 0, 0);
          wb[w] = ok ? *reinterpret_cast<const uint4*>(ws.buf + (size_t)(w * DS_COLS + gid + 8) * wpitch + k) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int t = 0; t < NT; ++t) {
          const uint4 av = ok ? *reinterpret_cast<const uint4*>(As + (size_t)(t * 8 + gid) * pitch + (k - kc0)) : make_uint4(0, 0, 0, 0);
#pragma unroll
          for (int w = 0; w < NW; ++w) {
            dm_mma(acc[w][t], wa[w].x, wb[w].x, wa[w].y, wb[w].y, av.x, av.y);
            dm_mma(acc[w][t], wa[w].z, wb[w].z, wa[w].w, wb[w].w, av.z, av.w);
          }
        }
      }
      // ---- K blocks from global memory
      const int kb_lo = max(kb_begin, kst / 32);
      for (int kb0 = kb_lo + warp; kb0 < kb_end; kb0 += DS_WARPS * UN) {
        uint4 wa[UN][NW], wb[UN][NW];
#pragma unroll
        for (int uu = 0; uu < UN; ++uu) {
          const int kb = kb0 + uu * DS_WARPS;
          const int k = kb * 32 + tig * 8;
          const bool ok = kb < kb_end && k < K && k >= kst;
#pragma unroll
          for (int w = 0; w < NW; ++w) {
            if (uu == 0 && kb0 == kb_first) {
              wa[uu][w] = pa[w];
              wb[uu][w] = pb[w];
            } else {
              const __nv_bfloat16* Wp = w == 0 ? W : W2;
              wa[uu][w] = ok ? *reinterpret_cast<const uint4*>(Wp + (size_t)ra * K + k) : make_uint4(0, 0, 0, 0);
              wb[uu][w] = ok ? *reinterpret_cast<const uint4*>(Wp + (size_t)rb * K + k) : make_uint4(0, 0, 0, 0);
            }
          }
        }
#pragma unroll
        for (int uu = 0; uu < UN; ++uu) {
          const int kb = kb0 + uu * DS_WARPS;
          const int k = kb * 32 + tig * 8;
          const bool ok = kb < kb_end && k < K && k >= kst;
#pragma unroll
          for (int t = 0; t < NT; ++t) {
            const uint4 av = ok ? *reinterpret_cast<const uint4*>(As + (size_t)(t * 8 + gid) * pitch + (k - kc0)) : make_uint4(0, 0, 0, 0);
#pragma unroll
            for (int w = 0; w < NW; ++w) {
              dm_mma(acc[w][t], wa[uu][w].x, wb[uu][w].x, wa[uu][w].y, wb[uu][w].y, av.x, av.y);
              dm_mma(acc[w][t], wa[uu][w].z, wb[uu][w].z, wa[uu][w].w, wb[uu][w].w, av.z, av.w);
            }
          }
        }
      }
    }
    // ---- add the warps' partial tiles (in the order of the warps), then the epilogue by warp 0
    float* mine = red + (size_t)warp * 2 * NT * 128;
#pragma unroll
    for (int w = 0; w < NW; ++w)
#pragma unroll
      for (int t = 0; t < NT; ++t)
        *reinterpret_cast<float4*>(mine + ((w * NT + t) * 32 + lane) * 4) = make_float4(acc[w][t][0], acc[w][t][1], acc[w][t][2], acc[w][t][3]);
    __syncthreads();
    if (first && next != nullptr && warp == 1) ds_w_issue(ws, *next);   // every warp is done with the stage
    if (warp == 0) {
#pragma unroll
      for (int t = 0; t < NT; ++t) {
        float s[NW][4];
#pragma unroll
        for (int w = 0; w < NW; ++w) {
#pragma unroll
          for (int j = 0; j < 4; ++j) s[w][j] = 0.f;
          for (int ww = 0; ww < DS_WARPS; ++ww) {
            const float4 p = *reinterpret_cast<const float4*>(red + ((size_t)ww * 2 * NT + w * NT + t) * 128 + lane * 4);
            s[w][0] += p.x; s[w][1] += p.y; s[w][2] += p.z; s[w][3] += p.w;
          }
        }
        // fragment layout: s[.][0], s[.][1]: column n0 + gid, batch rows 2 tig, 2 tig + 1; s[.][2], s[.][3]: column n0 + gid + 8
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int n = n0 + gid + (j >> 1) * 8;
          const int m = t * 8 + tig * 2 + (j & 1);
          if (n < N && m < M) {
            const size_t idx = (size_t)m * ldo + n;
            if (EPI == DS_STORE) out[idx] = from_f32<TOut>(s[0][j]);
            if (EPI == DS_RESIDUAL) out[idx] = from_f32<TOut>(__ldcg(residual + idx) + s[0][j]);
            if (EPI == DS_SWIGLU) out[idx] = from_f32<TOut>(ds_silu(s[0][j]) * s[NW - 1][j]);
          }
        }
      }
    }
    first = false;
    __syncthreads();   // the sums are read before the next unit's partial tiles land
  }
}

// ---------------------------------------------------------------- attention of the new tokens, one phase
// A unit: the pages [p_begin, p_begin + n_tiles) of one (sequence, kv head), a page per warp.
struct AttnUnit {
  int seq, kvh, chunk, n_chunks, nkeys, p_begin, n_tiles;
  const int32_t* pages;
};

// Unit `u` of a layer's attention, or false if the layer has fewer.  Units are numbered sequence by sequence,
// chunk by chunk, kv head by kv head; a sequence has ceil(pages / CH) chunks.
__device__ __forceinline__ bool ds_attn_unit(const StackLayer& L, const int* seq_slot /* shared memory */,
                                             const int* seq_pos /* shared memory */, int B, int CH, int u, AttnUnit& a) {
  int v = u / L.nkv;
  a.kvh = u - v * L.nkv;
  for (int s = 0; s < B; ++s) {
    const int nkeys = seq_pos[s] + 1;
    const int n_pages = max(1, min((nkeys + PAGE - 1) / PAGE, L.table_stride));
    const int n_chunks = (n_pages + CH - 1) / CH;
    if (v < n_chunks) {
      a.seq = s;
      a.chunk = v;
      a.n_chunks = n_chunks;
      a.nkeys = nkeys;
      a.p_begin = v * CH;
      a.n_tiles = min(n_pages, a.p_begin + CH) - a.p_begin;
      a.pages = L.page_table + (size_t)seq_slot[s] * L.table_stride;
      return true;
    }
    v -= n_chunks;
  }
  return false;
}

// Warp `warp` requests its page of the unit: 16-byte asynchronous copies into rows padded by 16 bytes, each lane's
// share of them arriving on the warp's mbarrier (32 arrivals a phase).  Far fewer, larger requests than a bulk
// copy per row, whose issue rate bounded the kernel.
template <int HDT>
__device__ __forceinline__ void ds_attn_issue(const StackLayer& L, const AttnUnit& a, __nv_bfloat16* Kt, __nv_bfloat16* Vt,
                                              uint32_t bar, int* err) {
  constexpr int HD = HDT * 16, PITCH = HD + 8, VPR = HD / 8;   // 16-byte vectors of a row
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (warp >= a.n_tiles) return;
  int page = a.pages[a.p_begin + warp];
  if (page < 0 || page >= L.n_pages) {
    if (lane == 0) atomicOr(err, ERR_PAGE_RANGE);
    page = 0;
  }
  const size_t src = ((size_t)page * L.nkv + a.kvh) * PAGE * HD;
#pragma unroll
  for (int i = lane; i < PAGE * VPR; i += 32) {
    const int r = i / VPR, c = (i - r * VPR) * 8;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dm_smem_u32(Kt + r * PITCH + c)), "l"(L.kcache + src + (size_t)r * HD + c) : "memory");
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dm_smem_u32(Vt + r * PITCH + c)), "l"(L.vcache + src + (size_t)r * HD + c) : "memory");
  }
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}

// `ahead`: the tiles of the block's first unit were requested already (ds_attn_prefetch).
// Every unit leaves its result in part_o / part_ml.
template <int HDT>
__device__ __forceinline__ void ds_attention(uint8_t* head, uint8_t* tiles, uint64_t* bars, const StackLayer& L,
                                             bool ahead, const __nv_bfloat16* qkv, const int* seq_slot,
                                             const int* seq_pos, int B, float* part_o, float* part_ml, int max_chunks,
                                             int att_warps, int* err, uint32_t& phase) {
  using T = __nv_bfloat16;
  constexpr int HD = HDT * 16, PITCH = HD + 8, WS = HD + 2, TILE = PAGE * PITCH, half = HD / 2;
  static_assert(DM_ROWS * WS * 4 <= TILE * 2, "a warp's partial fits its key tile");
  T* Qs = reinterpret_cast<T*>(head);       // [16][PITCH]
  T* newkv = Qs + DM_ROWS * PITCH;          // [2][HD]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, gid = lane >> 2, tig = lane & 3;
  T* Kt = reinterpret_cast<T*>(tiles) + (size_t)warp * 2 * TILE;   // (only warps < att_warps have tiles)
  T* Vt = Kt + TILE;
  auto partial = [&](int w) { return reinterpret_cast<float*>(tiles) + (size_t)w * TILE; };
  const uint32_t bar = dm_smem_u32(&bars[warp]);
  const int nh = L.nh, nkv = L.nkv, g = nh / nkv, ldq = (nh + 2 * nkv) * HD;
  const int CH = att_warps;   // pages of a chunk: one per warp

  AttnUnit a;
  for (int u = blockIdx.x; ds_attn_unit(L, seq_slot, seq_pos, B, CH, u, a); u += gridDim.x) {
    const int seq = a.seq, kvh = a.kvh, nkeys = a.nkeys, pos = nkeys - 1;
    const int tpos = min(max(pos, 0), L.max_pos - 1);
    const bool owner = (pos / PAGE) / CH == a.chunk;
    if ((pos >= L.max_pos || pos < 0 || pos / PAGE >= L.table_stride) && threadIdx.x == 0) atomicOr(err, ERR_POSITION_RANGE);
    __syncthreads();   // the unit before this one is done with the shared memory
    const bool has_tile = warp < a.n_tiles;   // CH = att_warps: at most one tile a warp
    if (!(ahead && u == (int)blockIdx.x)) ds_attn_issue<HDT>(L, a, Kt, Vt, bar, err);   // on their way while the queries are staged
    int page = 0;
    bool page_ok = false;
    if (owner) {
      page = a.pages[min(pos / PAGE, L.table_stride - 1)];
      page_ok = page >= 0 && page < L.n_pages;
      if (!page_ok && threadIdx.x == 0) atomicOr(err, ERR_PAGE_RANGE);
    }
    // rows 0 .. g - 1: the g <= 16 query heads of the kv head, rotated (rows from g on are zero); rows 16 and 17, in
    // the unit that holds the new token: its rotated key and its value, for the cache and for this unit's own tile.
    // An item is eight dims of the first half of a row with their partners in the second half: one round of loads.
    const T* tok = qkv + (size_t)seq * ldq;
    constexpr int IPR = HD / 16;   // items of a row
    for (int i = threadIdx.x; i < DM_ROWS * (HD / 8); i += DS_THREADS) {   // zero rows
      const int r = i / (HD / 8), c = (i - r * (HD / 8)) * 8;
      if (r >= g) *reinterpret_cast<uint4*>(Qs + r * PITCH + c) = make_uint4(0, 0, 0, 0);
    }
    for (int i = threadIdx.x; i < (g + (owner ? 2 : 0)) * IPR; i += DS_THREADS) {
      const int rr = i / IPR, d = (i - rr * IPR) * 8;
      const int r = rr < g ? rr : DM_ROWS + (rr - g);
      const T* row = r < DM_ROWS ? tok + (size_t)(kvh * g + r) * HD : tok + (size_t)(nh + (r - DM_ROWS) * nkv + kvh) * HD;
      uint4 lo = __ldcg(reinterpret_cast<const uint4*>(row + d)), hi = __ldcg(reinterpret_cast<const uint4*>(row + half + d));
      if (r != DM_ROWS + 1) dm_rotate8(lo, hi, L.cos_t + (size_t)tpos * half, L.sin_t + (size_t)tpos * half, d);
      if (r < DM_ROWS) {
        *reinterpret_cast<uint4*>(Qs + r * PITCH + d) = lo;
        *reinterpret_cast<uint4*>(Qs + r * PITCH + half + d) = hi;
      } else {
        *reinterpret_cast<uint4*>(newkv + (r - DM_ROWS) * HD + d) = lo;
        *reinterpret_cast<uint4*>(newkv + (r - DM_ROWS) * HD + half + d) = hi;
        if (page_ok) {
          T* dst = (r == DM_ROWS ? L.kcache : L.vcache) + (((size_t)page * nkv + kvh) * PAGE + pos % PAGE) * HD;
          *reinterpret_cast<uint4*>(dst + d) = lo;
          *reinterpret_cast<uint4*>(dst + half + d) = hi;
        }
      }
    }
    __syncthreads();
    float mA = -CUDART_INF_F, mB = -CUDART_INF_F, lA = 0.f, lB = 0.f;
    // Waits for the warp's tile and mends it (the new token's row, the rows past the sequence's end); false, with the
    // error word set, if the tile never came.
    auto tile_ready = [&](int key0, int valid) {
      if (!ds_mbar_wait(bar, phase)) {
        if (lane == 0) atomicOr(err, ERR_WAIT_TIMEOUT);
        mA = mB = lA = lB = CUDART_NAN_F;
        return false;
      }
      phase ^= 1;
      if (owner && pos >= key0 && pos < key0 + PAGE) {   // the copy read the row before the append, or while it landed
        for (int d = lane; d < HD; d += 32) {
          Kt[(pos - key0) * PITCH + d] = newkv[d];
          Vt[(pos - key0) * PITCH + d] = newkv[HD + d];
        }
      }
      if (valid < PAGE) {   // rows past the sequence's end are not this sequence's: their scores are masked whatever the
        // keys hold, their weights are exactly zero, and zero values keep a stale NaN from meeting them
        for (int i = lane; i < (PAGE - valid) * (HD / 8); i += 32) {
          const int r = valid + i / (HD / 8), c = i - (i / (HD / 8)) * (HD / 8);
          *reinterpret_cast<uint4*>(Vt + r * PITCH + c * 8) = make_uint4(0, 0, 0, 0);
        }
      }
      __syncwarp();
      return true;
    };
    const int key0 = (a.p_begin + warp) * PAGE;
    const int valid = min(PAGE, nkeys - key0);
    // ---- the warp's tile, then its partial into shared memory: into its own key tile, which it no longer reads
    if (g <= DM_HEADS_T) {
      // up to 8 query heads on the kv head: the keys are the 16-row operand; a lane holds the heads 2 tig and 2 tig + 1
      float o[HDT][4];
#pragma unroll
      for (int i = 0; i < HDT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
      if (has_tile) {
        uint32_t qb[HDT][2];
        dm_load_queries_t<HDT>(Qs, qb);
        if (tile_ready(key0, valid)) {
          dm_tile_update_t<HDT>(Kt, Vt, qb, valid, L.scale, o, mA, mB, lA, lB);
          dm_sum_over_keys(lA, lB);
        }
      }
      __syncwarp();
      if (warp < att_warps) {
        float* wa = partial(warp) + (tig * 2) * WS;
        float* wb = wa + WS;
#pragma unroll
        for (int dt = 0; dt < HDT; ++dt) {
          wa[dt * 16 + gid] = o[dt][0];
          wb[dt * 16 + gid] = o[dt][1];
          wa[dt * 16 + gid + 8] = o[dt][2];
          wb[dt * 16 + gid + 8] = o[dt][3];
        }
        if (gid == 0) {
          wa[HD] = mA;
          wa[HD + 1] = lA;
          wb[HD] = mB;
          wb[HD + 1] = lB;
        }
      }
    } else {
      float o[HD / 8][4];   // rows gid and gid + 8
#pragma unroll
      for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
      if (has_tile) {
        uint32_t qa[HDT][4];
        dm_load_queries<HDT>(Qs, qa);
        if (tile_ready(key0, valid)) dm_tile_update<HDT>(Kt, Vt, qa, valid, L.scale, o, mA, mB, lA, lB);
      }
      __syncwarp();
      if (warp < att_warps) {
        float* wa = partial(warp) + gid * WS;
        float* wb = partial(warp) + (gid + 8) * WS;
#pragma unroll
        for (int dt = 0; dt < HD / 8; ++dt) {
          wa[dt * 8 + tig * 2] = o[dt][0];
          wa[dt * 8 + tig * 2 + 1] = o[dt][1];
          wb[dt * 8 + tig * 2] = o[dt][2];
          wb[dt * 8 + tig * 2 + 1] = o[dt][3];
        }
        if (tig == 0) {
          wa[HD] = mA;
          wa[HD + 1] = lA;
          wb[HD] = mB;
          wb[HD + 1] = lB;
        }
      }
    }
    __syncthreads();
    // ---- fold the warps in their order: threads over (row, pair of dims); the unit's result goes to global memory
    for (int i = threadIdx.x; i < g * (HD / 2); i += DS_THREADS) {
      const int r = i / (HD / 2), d = (i - r * (HD / 2)) * 2;
      float M = -CUDART_INF_F;
      bool bad = false;
      for (int w = 0; w < att_warps; ++w) {
        const float mw = partial(w)[r * WS + HD];
        bad = bad || (mw != mw);
        M = fmaxf(M, mw);
      }
      float Lsum = 0.f, o0 = 0.f, o1 = 0.f;
      if (M != -CUDART_INF_F && !bad) {
        for (int w = 0; w < att_warps; ++w) {
          const float* p = partial(w) + r * WS;
          if (p[HD] == -CUDART_INF_F) continue;
          const float f = expf(p[HD] - M);
          Lsum = fmaf(p[HD + 1], f, Lsum);
          o0 = fmaf(p[d], f, o0);
          o1 = fmaf(p[d + 1], f, o1);
        }
      }
      if (bad) M = Lsum = CUDART_NAN_F;
      const size_t pi = ((size_t)seq * nh + kvh * g + r) * max_chunks + a.chunk;
      *reinterpret_cast<float2*>(part_o + pi * HD + d) = make_float2(o0, o1);
      if (d == 0) *reinterpret_cast<float2*>(part_ml + pi * 2) = make_float2(M, Lsum);
    }
  }
}

// Requests the tiles of the block's first unit of layer L's attention, if it has one (all warps call it, after
// a block-wide barrier that follows the last use of the tiles).
template <int HDT>
__device__ __forceinline__ bool ds_attn_prefetch(uint8_t* tiles, uint64_t* bars, const StackLayer& L, const int* seq_slot,
                                                 const int* seq_pos, int B, int att_warps, int* err) {
  constexpr int TILE = PAGE * (HDT * 16 + 8);
  AttnUnit a;
  if (!ds_attn_unit(L, seq_slot, seq_pos, B, att_warps, blockIdx.x, a)) return false;
  const int warp = threadIdx.x >> 5;
  __nv_bfloat16* Kt = reinterpret_cast<__nv_bfloat16*>(tiles) + (size_t)warp * 2 * TILE;
  ds_attn_issue<HDT>(L, a, Kt, Kt + TILE, dm_smem_u32(&bars[warp]), err);
  return true;
}

// ---------------------------------------------------------------- the kernel
// sync[0]: the grid barrier's arrivals; sync[1]: blocks that have left.  Both zero when the kernel starts
// and, unless a wait ran out, when it ends.
template <int HDT, int NT>
__global__ void __launch_bounds__(DS_THREADS, 1)
decode_stack_kernel(const StackLayer* __restrict__ layers, int n_layers, float* x, int B, int D, int max_k,
                    const int32_t* __restrict__ seq_slot_g, const int32_t* __restrict__ seq_pos_g, __nv_bfloat16* qkv,
                    __nv_bfloat16* mid, float* part_o, float* part_ml, int max_chunks, unsigned* sync, int att_warps,
                    int w_bytes, int* err, unsigned long long* trace) {
  constexpr int HD = HDT * 16;
  extern __shared__ __align__(128) uint8_t ds_smem[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(ds_smem);                 // [DS_WARPS] the warps' tiles, [DS_WARPS]: the weight stage
  volatile int* flags = reinterpret_cast<volatile int*>(ds_smem + 96);   // [0]: a wait ran out
  int* seq_pos = reinterpret_cast<int*>(ds_smem + 128);                  // [16] the step's sequences: last position,
  int* seq_slot = seq_pos + 16;                                          // [16] row of the page tables
  uint8_t* work = ds_smem + DS_RESERVED;
  uint8_t* attn_head = work + ds_gemv_bytes(max_k, NT);
  uint8_t* stage = attn_head + ds_attn_head_bytes(HD);
  uint8_t* tiles = stage + w_bytes;
  const int warp = threadIdx.x >> 5;
  if ((threadIdx.x & 31) == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(dm_smem_u32(&bars[warp])), "r"(32));
    if (warp == 0) asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(dm_smem_u32(&bars[DS_WARPS])), "r"(1));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (threadIdx.x == 0) flags[0] = 0;
  if (threadIdx.x < 16) {
    seq_pos[threadIdx.x] = (int)threadIdx.x < B ? seq_pos_g[threadIdx.x] : 0;
    seq_slot[threadIdx.x] = (int)threadIdx.x < B ? seq_slot_g[threadIdx.x] : 0;
  }
  __syncthreads();
  WStage ws = {reinterpret_cast<__nv_bfloat16*>(stage), w_bytes, dm_smem_u32(&bars[DS_WARPS]), 0u};
  unsigned target = 0;
  uint32_t phase = 0;
  bool alive = true;
  // `trace` (may be null): [layer][10] nanosecond stamps of block 0, before and after each phase's own work
  auto stamp = [&](int l, int i) {
    if (trace != nullptr && blockIdx.x == 0 && threadIdx.x == 0) {
      unsigned long long t;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
      trace[l * 10 + i] = t;
    }
  };
  auto qkv_of = [&](const StackLayer& L) { return GemvW{L.w_qkv, nullptr, (L.nh + 2 * L.nkv) * HD, D}; };
  // ---- requests of the first layer: its first weights, its attention's tiles
  bool ahead = false;
  {
    const StackLayer L0 = layers[0];
    if (warp == 1) ds_w_issue(ws, qkv_of(L0));
    ahead = ds_attn_prefetch<HDT>(tiles, bars, L0, seq_slot, seq_pos, B, att_warps, err);
  }
  for (int l = 0; l < n_layers && alive; ++l) {
    const StackLayer L = layers[l];
    const bool more = l + 1 < n_layers;
    const StackLayer Ln = layers[more ? l + 1 : l];
    const int ldq = (L.nh + 2 * L.nkv) * HD, ldo = L.nh * HD;
    const GemvW g_qkv = qkv_of(L), g_o = {L.w_o, nullptr, D, ldo}, g_gu = {L.w_gate, L.w_up, L.inter, D}, g_down = {L.w_down, nullptr, D, L.inter};
    const GemvW g_next = qkv_of(Ln);
    stamp(l, 0);
    const FoldSrc fold = {part_o, part_ml, seq_pos, max_chunks, HD, att_warps, L.table_stride};
    ds_gemv<DS_STORE, __nv_bfloat16, NT, DS_SRC_NORM>(work, ws, nullptr, 0, x, L.norm1_w, L.eps1, nullptr, g_qkv, qkv, ldq, nullptr, B, &g_o, err);
    stamp(l, 1);
    if (!(alive = ds_grid_barrier(sync, target, err, flags))) break;
    stamp(l, 2);
    ds_attention<HDT>(attn_head, tiles, bars, L, ahead, qkv, seq_slot, seq_pos, B, part_o, part_ml, max_chunks, att_warps, err, phase);
    stamp(l, 3);
    ds_grid_arrive(sync, target);   // (its block-wide barrier: every warp is done with its tile)
    ahead = more && ds_attn_prefetch<HDT>(tiles, bars, Ln, seq_slot, seq_pos, B, att_warps, err);   // the next layer's tiles come meanwhile
    if (!(alive = ds_grid_wait(sync, target, err, flags))) break;
    stamp(l, 4);
    ds_gemv<DS_RESIDUAL, float, NT, DS_SRC_FOLD>(work, ws, nullptr, 0, nullptr, nullptr, 0.f, &fold, g_o, x, D, x, B, &g_gu, err);
    stamp(l, 5);
    if (!(alive = ds_grid_barrier(sync, target, err, flags))) break;
    stamp(l, 6);
    ds_gemv<DS_SWIGLU, __nv_bfloat16, NT, DS_SRC_NORM>(work, ws, nullptr, 0, x, L.norm2_w, L.eps2, nullptr, g_gu, mid, L.inter, nullptr, B, &g_down, err);
    stamp(l, 7);
    if (!(alive = ds_grid_barrier(sync, target, err, flags))) break;
    stamp(l, 8);
    ds_gemv<DS_RESIDUAL, float, NT, DS_SRC_ACT>(work, ws, mid, L.inter, nullptr, nullptr, 0.f, nullptr, g_down, x, D, x, B, more ? &g_next : nullptr, err);
    stamp(l, 9);
    if (more && !(alive = ds_grid_barrier(sync, target, err, flags))) break;
  }
  if (alive && threadIdx.x == 0) {   // the last block to leave puts the words back to zero for the next launch
    __threadfence();
    if (atomicAdd(sync + 1, 1u) == gridDim.x - 1) {
      sync[0] = 0u;
      sync[1] = 0u;
    }
  }
}

}  // namespace edgelm

using namespace edgelm;

static bool ds_head_size_taken(int hd) { return hd == 32 || hd == 64 || hd == 96 || hd == 128; }

// Pages of the cache that one attention unit of the kernel covers (a warp each) for a step of `n_seqs`
// sequences; 0: sizes not taken.  The caller sizes the partial results with it: ceil(pages of the longest
// sequence / this) chunks.
extern "C" int edgelm_decode_stack_chunk_pages(int hd, int max_k, int n_seqs) {
  if (!ds_head_size_taken(hd) || max_k <= 0 || n_seqs < 1 || n_seqs > 16) return 0;
  return ds_plan(hd, max_k, n_seqs <= 8 ? 1 : 2).att_warps;
}

// Bytes of a layer record (StackLayer), for the host that packs them.
extern "C" int edgelm_decode_stack_record_bytes() { return (int)sizeof(StackLayer); }

extern "C" int edgelm_decode_stack(const void* layers, int n_layers, float* x, int B, int D, int hd, int max_k,
                                   const int32_t* seq_slot, const int32_t* seq_pos, void* qkv, void* mid,
                                   float* part_o, float* part_ml, int max_chunks, void* sync, int* err,
                                   unsigned long long* trace, cudaStream_t stream) {
  if (B == 0 || n_layers == 0) return 0;
  EL_REFUSE(B >= 1 && B <= 16, "decode_stack: takes 1 to 16 sequences, not %d", B);
  EL_REFUSE(ds_head_size_taken(hd), "decode_stack: head size %d (takes 32, 64, 96, 128)", hd);
  EL_REFUSE(D > 0 && D % 8 == 0 && max_k >= D && max_k % 8 == 0, "decode_stack: widths must be multiples of 8 (D=%d, widest input %d)", D, max_k);
  EL_REFUSE(max_chunks >= 1 && err != nullptr && sync != nullptr, "decode_stack: bad arguments");
  const int NT = B <= 8 ? 1 : 2;
  const StackPlan plan = ds_plan(hd, max_k, NT);
  EL_REFUSE(plan.att_warps >= 1, "decode_stack: no room in shared memory for a key and a value tile (head size %d, widest input %d)", hd, max_k);
  const size_t smem = plan.total;
  static int n_sms = 0;
  if (n_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n_sms, cudaDevAttrMultiProcessorCount, dev);
  }
  const void* kern = nullptr;
#define EL_DS(HDT_, NT_) kern = (const void*)decode_stack_kernel<HDT_, NT_>
  if (NT == 1) {
    if (hd == 32) EL_DS(2, 1); else if (hd == 64) EL_DS(4, 1); else if (hd == 96) EL_DS(6, 1); else EL_DS(8, 1);
  } else {
    if (hd == 32) EL_DS(2, 2); else if (hd == 64) EL_DS(4, 2); else if (hd == 96) EL_DS(6, 2); else EL_DS(8, 2);
  }
#undef EL_DS
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  EL_REFUSE(e == cudaSuccess, "decode_stack: %zu bytes of shared memory refused: %s", smem, cudaGetErrorString(e));
  int resident = 0;
  e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident, kern, DS_THREADS, smem);
  EL_REFUSE(e == cudaSuccess && resident >= 1, "decode_stack: the kernel does not fit an SM (%s)", cudaGetErrorString(e));
  int max_chunks_ = max_chunks, att_warps_ = plan.att_warps, w_bytes_ = plan.w_bytes;
  void* args[] = {(void*)&layers, (void*)&n_layers, (void*)&x, (void*)&B, (void*)&D, (void*)&max_k, (void*)&seq_slot,
                  (void*)&seq_pos, (void*)&qkv, (void*)&mid, (void*)&part_o, (void*)&part_ml, (void*)&max_chunks_,
                  (void*)&sync, (void*)&att_warps_, (void*)&w_bytes_, (void*)&err, (void*)&trace};
  e = cudaLaunchCooperativeKernel(kern, dim3(n_sms), dim3(DS_THREADS), args, smem, stream);
  if (e != cudaSuccess) {
    set_error("decode_stack: launch failed: %s", cudaGetErrorString(e));
    return -2;
  }
  return 0;
}
