// Causal attention over the paged cache, for query heads that share key/value heads.
//
// The cache of one layer is [page][kv_head][PAGE][hd] for keys and the same for values; a
// sequence's position p lies in page `page_table[slot][p / PAGE]` at row `p % PAGE`.  The new
// tokens' keys and values are in the cache already (rope_kv_append runs first), so a token
// attends to itself through the cache, and prompts cut into several steps need nothing more.
//
// Scores, the running maximum, exponentials, their sum and the weighted sum of values are
// float32; the 1/sqrt(hd) scale is applied to the finished dot product.  Keys are visited page
// by page, so a row's arithmetic depends on its own position alone, not on the batch around it.
//
//   attn_prefill: any number of new tokens per sequence.  One block = up to 32 (token, head)
//                 rows of one kv head; a page of K and V is staged in shared memory once for
//                 all of them; a warp owns 4 rows, lanes own keys (scores) then dims (values).
//   attn_decode:  one new token per sequence.  grid (sequence, kv head, split): the pages of a
//                 sequence are dealt to splits and, inside a block, to warps; partial
//                 (max, sum, weighted values) meet in shared memory and, with more than one
//                 split, in a scratch buffer that attn_decode_combine folds in a fixed order.
#include <math_constants.h>

#include <mutex>

#include "common.cuh"

namespace edgelm {

constexpr int RW = 4;          // rows a warp owns
constexpr int ATT_WARPS = 8;   // warps per block
constexpr int ATT_ROWS = RW * ATT_WARPS;

template <typename T, int NC>  // NC = ceil(hd / 32): value dims a lane owns
__global__ void __launch_bounds__(ATT_WARPS * 32)
attn_prefill_kernel(const T* __restrict__ q, int ldq, T* __restrict__ out, int ldo, const T* __restrict__ kcache,
                    const T* __restrict__ vcache, const int32_t* __restrict__ page_table, int table_stride,
                    const int32_t* __restrict__ seq_slot, const int32_t* __restrict__ tile_seq,
                    const int32_t* __restrict__ tile_tok0, const int32_t* __restrict__ tile_ntok,
                    const int32_t* __restrict__ tile_pos0, int nh, int nkv, int hd, float scale) {
  extern __shared__ float smem[];
  const int ks = hd + 1;                       // padded key row: lanes read different rows
  float* Ks = smem;                            // [PAGE][hd + 1]
  float* Vs = Ks + PAGE * ks;                  // [PAGE][hd]
  float* Qs = Vs + PAGE * hd;                  // [ATT_ROWS][hd]
  float* Ps = Qs + ATT_ROWS * hd;              // [ATT_ROWS][PAGE]

  const int tile = blockIdx.x, kvh = blockIdx.y;
  const int g = nh / nkv;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int seq = tile_seq[tile], tok0 = tile_tok0[tile], ntok = tile_ntok[tile], pos0 = tile_pos0[tile];
  const int32_t* pages = page_table + (size_t)seq_slot[seq] * table_stride;
  const int rows_total = ntok * g;
  const int row_base = blockIdx.z * ATT_ROWS;
  if (row_base >= rows_total) return;
  const int rows_here = min(ATT_ROWS, rows_total - row_base);
  // keys this block can need: up to the position of its last row's token
  const int last_tok = (row_base + rows_here - 1) / g;
  const int nkeys_block = pos0 + last_tok + 1;

  // stage the query rows as float
  for (int i = threadIdx.x; i < rows_here * hd; i += blockDim.x) {
    const int r = i / hd, d = i - r * hd;
    const int rr = row_base + r, tok = rr / g, head = kvh * g + rr % g;
    Qs[r * hd + d] = to_f32(q[(size_t)(tok0 + tok) * ldq + head * hd + d]);
  }

  float m[RW], l[RW], acc[RW][NC];
  int limit[RW];
#pragma unroll
  for (int r = 0; r < RW; ++r) {
    m[r] = -CUDART_INF_F;
    l[r] = 0.f;
    const int rr = row_base + warp * RW + r;
    limit[r] = rr < rows_total ? pos0 + rr / g : -1;  // last key this row may see; -1: no row
#pragma unroll
    for (int c = 0; c < NC; ++c) acc[r][c] = 0.f;
  }
  int warp_limit = -1;
#pragma unroll
  for (int r = 0; r < RW; ++r) warp_limit = max(warp_limit, limit[r]);

  const int n_tiles = (nkeys_block + PAGE - 1) / PAGE;
  for (int kt = 0; kt < n_tiles; ++kt) {
    const int page = pages[kt];
    const T* kp = kcache + ((size_t)page * nkv + kvh) * PAGE * hd;
    const T* vp = vcache + ((size_t)page * nkv + kvh) * PAGE * hd;
    const int valid = min(PAGE, nkeys_block - kt * PAGE);  // rows of the page that hold this block's keys
    __syncthreads();  // the previous page is no longer read
    for (int i = threadIdx.x; i < PAGE * hd; i += blockDim.x) {
      const int j = i / hd, d = i - j * hd;
      const bool ok = j < valid;  // what lies behind is not this sequence's: never let it in, not even times zero
      Ks[j * ks + d] = ok ? to_f32(kp[i]) : 0.f;
      Vs[i] = ok ? to_f32(vp[i]) : 0.f;
    }
    __syncthreads();
    const int j0 = kt * PAGE + lane, j1 = j0 + 32;
    if (kt * PAGE > warp_limit) continue;  // none of this warp's rows sees this page
    float s0[RW] = {}, s1[RW] = {};
    const float* k0 = Ks + lane * ks;
    const float* k1 = Ks + (lane + 32) * ks;
    const float* qw = Qs + warp * RW * hd;
    for (int d = 0; d < hd; ++d) {
      const float a = k0[d], b = k1[d];
#pragma unroll
      for (int r = 0; r < RW; ++r) {
        const float qv = qw[r * hd + d];
        s0[r] = fmaf(qv, a, s0[r]);
        s1[r] = fmaf(qv, b, s1[r]);
      }
    }
    float corr[RW];
#pragma unroll
    for (int r = 0; r < RW; ++r) {
      const float a = j0 <= limit[r] ? s0[r] * scale : -CUDART_INF_F;
      const float b = j1 <= limit[r] ? s1[r] * scale : -CUDART_INF_F;
      const float mx = fmaxf(m[r], warp_max(fmaxf(a, b)));
      float p0 = 0.f, p1 = 0.f;
      corr[r] = 1.f;
      if (mx != -CUDART_INF_F) {  // uniform over the warp
        corr[r] = expf(m[r] - mx);
        p0 = expf(a - mx);
        p1 = expf(b - mx);
        l[r] = l[r] * corr[r] + warp_sum(p0 + p1);
        m[r] = mx;
      }
      Ps[(warp * RW + r) * PAGE + lane] = p0;
      Ps[(warp * RW + r) * PAGE + lane + 32] = p1;
    }
    __syncwarp();
#pragma unroll
    for (int r = 0; r < RW; ++r)
#pragma unroll
      for (int c = 0; c < NC; ++c) acc[r][c] *= corr[r];
    const float* pw = Ps + warp * RW * PAGE;
    for (int j = 0; j < valid; ++j) {
      float v[NC];
#pragma unroll
      for (int c = 0; c < NC; ++c) {
        const int d = lane + 32 * c;
        v[c] = d < hd ? Vs[j * hd + d] : 0.f;
      }
#pragma unroll
      for (int r = 0; r < RW; ++r) {
        const float p = pw[r * PAGE + j];
#pragma unroll
        for (int c = 0; c < NC; ++c) acc[r][c] = fmaf(p, v[c], acc[r][c]);
      }
    }
    __syncwarp();
  }
#pragma unroll
  for (int r = 0; r < RW; ++r) {
    const int rr = row_base + warp * RW + r;
    if (rr >= rows_total) continue;
    const int tok = rr / g, head = kvh * g + rr % g;
    const float inv = 1.0f / l[r];
#pragma unroll
    for (int c = 0; c < NC; ++c) {
      const int d = lane + 32 * c;
      if (d < hd) out[(size_t)(tok0 + tok) * ldo + head * hd + d] = from_f32<T>(acc[r][c] * inv);
    }
  }
}

// ------------------------------------------------------------------------- decode
template <typename T> struct KVec;
template <> struct KVec<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void load(const float* p, float* o) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
  }
};
template <> struct KVec<__nv_bfloat16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* o) {
    const uint4 v = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      o[2 * i] = __uint_as_float(w[i] << 16);
      o[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
};

// Partial results of one split: part_o [seq][head][split][hd], part_ml [seq][head][split][2].
template <typename T, int NC>
__global__ void __launch_bounds__(ATT_WARPS * 32)
attn_decode_kernel(const T* __restrict__ q, int ldq, T* __restrict__ out, int ldo, const T* __restrict__ kcache,
                   const T* __restrict__ vcache, const int32_t* __restrict__ page_table, int table_stride,
                   const int32_t* __restrict__ seq_slot, const int32_t* __restrict__ seq_pos, int nh, int nkv, int hd,
                   float scale, int n_splits, float* __restrict__ part_o, float* __restrict__ part_ml) {
  extern __shared__ float smem[];
  float* Qs = smem;                        // [RW][hd]   the row chunk's queries
  float* Ws = Qs + RW * hd;                // [ATT_WARPS][RW][hd + 2]   per-warp partials
  const int seq = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
  const int g = nh / nkv;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nkeys = seq_pos[seq] + 1;      // the new token's own key is the last one
  const int32_t* pages = page_table + (size_t)seq_slot[seq] * table_stride;
  const int n_tiles = (nkeys + PAGE - 1) / PAGE;
  const int per_split = (n_tiles + n_splits - 1) / n_splits;
  const int t_begin = split * per_split, t_end = min(n_tiles, t_begin + per_split);
  const int ws = hd + 2;

  for (int h0 = 0; h0 < g; h0 += RW) {     // chunks of RW query heads of this kv head
    const int rows = min(RW, g - h0);
    __syncthreads();
    for (int i = threadIdx.x; i < rows * hd; i += blockDim.x) {
      const int r = i / hd, d = i - r * hd;
      Qs[i] = to_f32(q[(size_t)seq * ldq + (kvh * g + h0 + r) * hd + d]);
    }
    __syncthreads();
    float m[RW], l[RW], acc[RW][NC];
#pragma unroll
    for (int r = 0; r < RW; ++r) {
      m[r] = -CUDART_INF_F;
      l[r] = 0.f;
#pragma unroll
      for (int c = 0; c < NC; ++c) acc[r][c] = 0.f;
    }
    for (int kt = t_begin + warp; kt < t_end; kt += ATT_WARPS) {
      const int page = pages[kt];
      const T* kp = kcache + ((size_t)page * nkv + kvh) * PAGE * hd;
      const T* vp = vcache + ((size_t)page * nkv + kvh) * PAGE * hd;
      const int valid = min(PAGE, nkeys - kt * PAGE);
      float s0[RW] = {}, s1[RW] = {};
      const bool ok0 = lane < valid, ok1 = lane + 32 < valid;
      for (int d = 0; d < hd; d += KVec<T>::N) {
        float a[KVec<T>::N] = {}, b[KVec<T>::N] = {};
        if (ok0) KVec<T>::load(kp + (size_t)lane * hd + d, a);
        if (ok1) KVec<T>::load(kp + (size_t)(lane + 32) * hd + d, b);
#pragma unroll
        for (int v = 0; v < KVec<T>::N; ++v)
#pragma unroll
          for (int r = 0; r < RW; ++r) {
            const float qv = Qs[r * hd + d + v];
            s0[r] = fmaf(qv, a[v], s0[r]);
            s1[r] = fmaf(qv, b[v], s1[r]);
          }
      }
      float p0[RW], p1[RW];
#pragma unroll
      for (int r = 0; r < RW; ++r) {
        const float a = ok0 ? s0[r] * scale : -CUDART_INF_F;
        const float b = ok1 ? s1[r] * scale : -CUDART_INF_F;
        const float mx = fmaxf(m[r], warp_max(fmaxf(a, b)));  // finite: valid >= 1
        const float corr = expf(m[r] - mx);
        p0[r] = expf(a - mx);
        p1[r] = expf(b - mx);
        l[r] = l[r] * corr + warp_sum(p0[r] + p1[r]);
        m[r] = mx;
#pragma unroll
        for (int c = 0; c < NC; ++c) acc[r][c] *= corr;
      }
      for (int j = 0; j < valid; ++j) {
        float v[NC];
#pragma unroll
        for (int c = 0; c < NC; ++c) {
          const int d = lane + 32 * c;
          v[c] = d < hd ? to_f32(vp[(size_t)j * hd + d]) : 0.f;
        }
#pragma unroll
        for (int r = 0; r < RW; ++r) {
          const float p = __shfl_sync(0xffffffffu, j < 32 ? p0[r] : p1[r], j & 31);
#pragma unroll
          for (int c = 0; c < NC; ++c) acc[r][c] = fmaf(p, v[c], acc[r][c]);
        }
      }
    }
    // warps -> shared memory
#pragma unroll
    for (int r = 0; r < RW; ++r) {
      float* w = Ws + (warp * RW + r) * ws;
#pragma unroll
      for (int c = 0; c < NC; ++c) {
        const int d = lane + 32 * c;
        if (d < hd) w[d] = acc[r][c];
      }
      if (lane == 0) {
        w[hd] = m[r];
        w[hd + 1] = l[r];
      }
    }
    __syncthreads();
    // fold the warps in the order 0..7; warp r folds row r
    if (warp < rows) {
      const int r = warp;
      float M = -CUDART_INF_F;
      for (int w = 0; w < ATT_WARPS; ++w) M = fmaxf(M, Ws[(w * RW + r) * ws + hd]);
      float L = 0.f, o[NC];
#pragma unroll
      for (int c = 0; c < NC; ++c) o[c] = 0.f;
      if (M != -CUDART_INF_F) {
        for (int w = 0; w < ATT_WARPS; ++w) {
          const float* p = Ws + (w * RW + r) * ws;
          if (p[hd] == -CUDART_INF_F) continue;
          const float f = expf(p[hd] - M);
          L = fmaf(p[hd + 1], f, L);
#pragma unroll
          for (int c = 0; c < NC; ++c) {
            const int d = lane + 32 * c;
            if (d < hd) o[c] = fmaf(p[d], f, o[c]);
          }
        }
      }
      const int head = kvh * g + h0 + r;
      if (n_splits == 1) {
        const float inv = 1.0f / L;
#pragma unroll
        for (int c = 0; c < NC; ++c) {
          const int d = lane + 32 * c;
          if (d < hd) out[(size_t)seq * ldo + head * hd + d] = from_f32<T>(o[c] * inv);
        }
      } else {
        const size_t pi = ((size_t)seq * nh + head) * n_splits + split;
#pragma unroll
        for (int c = 0; c < NC; ++c) {
          const int d = lane + 32 * c;
          if (d < hd) part_o[pi * hd + d] = o[c];
        }
        if (lane == 0) {
          part_ml[pi * 2] = M;
          part_ml[pi * 2 + 1] = L;
        }
      }
    }
  }
}

template <typename T>
__global__ void attn_decode_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                           T* __restrict__ out, int ldo, int nh, int hd, int n_splits) {
  const int seq = blockIdx.x, head = blockIdx.y;
  const size_t base = ((size_t)seq * nh + head) * n_splits;
  float M = -CUDART_INF_F;
  for (int s = 0; s < n_splits; ++s) M = fmaxf(M, part_ml[(base + s) * 2]);
  for (int d = threadIdx.x; d < hd; d += blockDim.x) {
    float L = 0.f, o = 0.f;
    for (int s = 0; s < n_splits; ++s) {
      const float ms = part_ml[(base + s) * 2];
      if (ms == -CUDART_INF_F) continue;  // a split that held no page
      const float f = expf(ms - M);
      L = fmaf(part_ml[(base + s) * 2 + 1], f, L);
      o = fmaf(part_o[(base + s) * hd + d], f, o);
    }
    out[(size_t)seq * ldo + head * hd + d] = from_f32<T>(o / L);
  }
}

template <typename T, int NC>
int launch_prefill(const void* q, int ldq, void* out, int ldo, const void* kc, const void* vc, const int32_t* page_table,
                   int table_stride, const int32_t* seq_slot, const int32_t* tile_seq, const int32_t* tile_tok0,
                   const int32_t* tile_ntok, const int32_t* tile_pos0, int n_tiles, int max_tile_tokens, int nh, int nkv,
                   int hd, float scale, cudaStream_t stream) {
  const int g = nh / nkv;
  const size_t smem = sizeof(float) * ((size_t)PAGE * (hd + 1) + (size_t)PAGE * hd + (size_t)ATT_ROWS * hd + (size_t)ATT_ROWS * PAGE);
  auto kern = attn_prefill_kernel<T, NC>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) {
    set_error("attn_prefill: %zu bytes of shared memory refused: %s", smem, cudaGetErrorString(e));
    return -2;
  }
  dim3 grid(n_tiles, nkv, (max_tile_tokens * g + ATT_ROWS - 1) / ATT_ROWS);
  kern<<<grid, ATT_WARPS * 32, smem, stream>>>((const T*)q, ldq, (T*)out, ldo, (const T*)kc, (const T*)vc, page_table,
                                              table_stride, seq_slot, tile_seq, tile_tok0, tile_ntok, tile_pos0, nh, nkv,
                                              hd, scale);
  return 0;
}

template <typename T, int NC>
int launch_decode(const void* q, int ldq, void* out, int ldo, const void* kc, const void* vc, const int32_t* page_table,
                  int table_stride, const int32_t* seq_slot, const int32_t* seq_pos, int n_seqs, int nh, int nkv, int hd,
                  float scale, int n_splits, float* part_o, float* part_ml, cudaStream_t stream) {
  const size_t smem = sizeof(float) * ((size_t)RW * hd + (size_t)ATT_WARPS * RW * (hd + 2));
  auto kern = attn_decode_kernel<T, NC>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) {
      set_error("attn_decode: %zu bytes of shared memory refused: %s", smem, cudaGetErrorString(e));
      return -2;
    }
  }
  dim3 grid(n_seqs, nkv, n_splits);
  kern<<<grid, ATT_WARPS * 32, smem, stream>>>((const T*)q, ldq, (T*)out, ldo, (const T*)kc, (const T*)vc, page_table,
                                              table_stride, seq_slot, seq_pos, nh, nkv, hd, scale, n_splits, part_o, part_ml);
  if (n_splits > 1) {
    dim3 cgrid(n_seqs, nh);
    attn_decode_combine_kernel<T><<<cgrid, 64, 0, stream>>>(part_o, part_ml, (T*)out, ldo, nh, hd, n_splits);
  }
  return 0;
}

static int check_heads(const char* who, int nh, int nkv, int hd) {
  EL_REFUSE(nh > 0 && nkv > 0 && nh % nkv == 0, "%s: %d query heads are not a multiple of %d key/value heads", who, nh, nkv);
  EL_REFUSE(hd >= 16 && hd <= 256 && hd % 16 == 0, "%s: head size %d (takes 16..256 in steps of 16)", who, hd);
  return 0;
}

}  // namespace edgelm

using namespace edgelm;

#define EL_ATT_DISPATCH(FN, ...)                                       \
  do {                                                                 \
    const int nc = (hd + 31) / 32;                                     \
    int rc = 0;                                                        \
    if (dtype == DT_F32) {                                             \
      if (nc <= 1) rc = FN<float, 1>(__VA_ARGS__);                     \
      else if (nc <= 2) rc = FN<float, 2>(__VA_ARGS__);                \
      else if (nc <= 4) rc = FN<float, 4>(__VA_ARGS__);                \
      else rc = FN<float, 8>(__VA_ARGS__);                             \
    } else if (dtype == DT_BF16) {                                     \
      if (nc <= 1) rc = FN<__nv_bfloat16, 1>(__VA_ARGS__);             \
      else if (nc <= 2) rc = FN<__nv_bfloat16, 2>(__VA_ARGS__);        \
      else if (nc <= 4) rc = FN<__nv_bfloat16, 4>(__VA_ARGS__);        \
      else rc = FN<__nv_bfloat16, 8>(__VA_ARGS__);                     \
    } else {                                                           \
      EL_REFUSE(false, "attention: unknown dtype code %d", dtype);     \
    }                                                                  \
    if (rc) return rc;                                                 \
  } while (0)

// Tiles: the host cuts each sequence's new tokens into tiles of at most `max_tile_tokens`
// tokens (so that tokens * heads-per-kv-head fits one or a few blocks of 32 rows).
extern "C" int edgelm_attn_prefill(const void* q, int ldq, void* out, int ldo, const void* kcache, const void* vcache,
                                   int dtype, const int32_t* page_table, int table_stride, const int32_t* seq_slot,
                                   const int32_t* tile_seq, const int32_t* tile_tok0, const int32_t* tile_ntok,
                                   const int32_t* tile_pos0, int n_tiles, int max_tile_tokens, int nh, int nkv, int hd,
                                   float scale, cudaStream_t stream) {
  if (n_tiles == 0) return 0;
  if (check_heads("attn_prefill", nh, nkv, hd)) return -1;
  EL_REFUSE(n_tiles > 0 && max_tile_tokens > 0, "attn_prefill: bad tile counts");
  EL_REFUSE(nkv <= 65535 && (max_tile_tokens * (nh / nkv) + ATT_ROWS - 1) / ATT_ROWS <= 65535, "attn_prefill: grid too large");
  EL_ATT_DISPATCH(launch_prefill, q, ldq, out, ldo, kcache, vcache, page_table, table_stride, seq_slot, tile_seq, tile_tok0,
                  tile_ntok, tile_pos0, n_tiles, max_tile_tokens, nh, nkv, hd, scale, stream);
  EL_LAUNCH_CHECK("attn_prefill");
  return 0;
}

// Scratch: part_o holds n_seqs*nh*n_splits*hd floats, part_ml n_seqs*nh*n_splits*2 (unused when n_splits == 1).
extern "C" int edgelm_attn_decode(const void* q, int ldq, void* out, int ldo, const void* kcache, const void* vcache,
                                  int dtype, const int32_t* page_table, int table_stride, const int32_t* seq_slot,
                                  const int32_t* seq_pos, int n_seqs, int nh, int nkv, int hd, float scale, int n_splits,
                                  float* part_o, float* part_ml, cudaStream_t stream) {
  if (n_seqs == 0) return 0;
  if (check_heads("attn_decode", nh, nkv, hd)) return -1;
  EL_REFUSE(n_splits >= 1 && n_splits <= 65535 && nkv <= 65535, "attn_decode: bad split count %d", n_splits);
  EL_REFUSE(n_splits == 1 || (part_o && part_ml), "attn_decode: %d splits need the scratch buffers", n_splits);
  EL_ATT_DISPATCH(launch_decode, q, ldq, out, ldo, kcache, vcache, page_table, table_stride, seq_slot, seq_pos, n_seqs, nh,
                  nkv, hd, scale, n_splits, part_o, part_ml, stream);
  EL_LAUNCH_CHECK("attn_decode");
  return 0;
}

// ------------------------------------------------------------------------- no-allocation variant
// See no_alloc.h for who this is for and for its rules.  The split partials live in this
// file-scope device array instead of caller-provided buffers.  In host code the array's name is
// only a handle; its device address comes from cudaGetSymbolAddress, looked up once per device
// with that device current.
#include "no_alloc.h"

static __device__ __align__(256) float g_noalloc_scratch[EDGELM_NOALLOC_SCRATCH_FLOATS];

namespace edgelm {
constexpr int NOALLOC_MAX_DEVICES = 64;
static float* g_noalloc_ptr[NOALLOC_MAX_DEVICES] = {};
static std::mutex g_noalloc_mu;

// Device address of the scratch array on the current device (first call per device: set-up).
static int noalloc_scratch(float** ptr) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= NOALLOC_MAX_DEVICES) {
    set_error("attn_decode_noalloc: cannot tell the current device (%s)", e == cudaSuccess ? "index out of range" : cudaGetErrorString(e));
    return -2;
  }
  std::lock_guard<std::mutex> lock(g_noalloc_mu);
  if (g_noalloc_ptr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess || p == nullptr) {
      set_error("attn_decode_noalloc: cudaGetSymbolAddress failed on device %d: %s", dev, cudaGetErrorString(e));
      return -2;
    }
    g_noalloc_ptr[dev] = static_cast<float*>(p);
  }
  *ptr = g_noalloc_ptr[dev];
  return 0;
}
}  // namespace edgelm

extern "C" int edgelm_attn_decode_noalloc(const void* q, int ldq, void* out, int ldo, const void* kcache,
                                          const void* vcache, int dtype, const int32_t* page_table, int table_stride,
                                          const int32_t* seq_slot, const int32_t* seq_pos, int n_seqs, int nh, int nkv,
                                          int hd, float scale, int n_splits, cudaStream_t stream) {
  if (n_seqs == 0) return 0;
  if (check_heads("attn_decode_noalloc", nh, nkv, hd)) return -1;
  EL_REFUSE(n_seqs > 0 && n_splits >= 1 && n_splits <= 65535 && nkv <= 65535, "attn_decode_noalloc: bad counts (%d sequences, %d splits)", n_seqs, n_splits);
  float* part_o = nullptr;
  float* part_ml = nullptr;
  if (n_splits > 1) {
    const long long cells = (long long)n_seqs * nh * n_splits;
    const long long need = cells * (hd + 2);
    EL_REFUSE(need <= (long long)EDGELM_NOALLOC_SCRATCH_FLOATS,
              "attn_decode_noalloc: %d sequences x %d heads x %d splits x (%d + 2) = %lld floats of scratch; the built-in array holds %d",
              n_seqs, nh, n_splits, hd, need, (int)EDGELM_NOALLOC_SCRATCH_FLOATS);
    float* base = nullptr;
    if (noalloc_scratch(&base)) return -2;
    part_o = base;                 // [cells][hd]
    part_ml = base + cells * hd;   // [cells][2]
  }
  EL_ATT_DISPATCH(launch_decode, q, ldq, out, ldo, kcache, vcache, page_table, table_stride, seq_slot, seq_pos, n_seqs, nh,
                  nkv, hd, scale, n_splits, part_o, part_ml, stream);
  EL_LAUNCH_CHECK("attn_decode_noalloc");
  return 0;
}
