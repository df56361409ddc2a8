// Embedding gather, RMSNorm (with optional row gather) and RoPE + cache append.
//
// The residual stream is float32 in both precisions; `T` below is the storage type of
// weights, of normalised activations and of the cache (float or bfloat16).
#include "attention_tile_mma.cuh"
#include "common.cuh"

namespace edgelm {

// ---------------------------------------------------------------- embedding: x[t,:] = E[id_t,:]
template <typename TW>
__global__ void embed_gather_kernel(const int32_t* __restrict__ ids, const TW* __restrict__ table,
                                    float* __restrict__ x, int dim, int vocab, int* __restrict__ err) {
  const int t = blockIdx.x;
  const int id = ids[t];
  if (id < 0 || id >= vocab) {  // the host checks ids that it has seen; ids sampled on the device are checked here
    if (threadIdx.x == 0) atomicOr(err, ERR_TOKEN_RANGE);
    for (int i = threadIdx.x; i < dim; i += blockDim.x) x[(size_t)t * dim + i] = 0.f;
    return;
  }
  const TW* row = table + (size_t)id * dim;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) x[(size_t)t * dim + i] = to_f32(row[i]);
}

// ---------------------------------------------------------------- RMSNorm
// y[r,:] = x[src(r),:] * (1 / sqrt(mean(x^2) + eps)) * w, statistics in float32.
// `rows_idx` (may be null) picks the source row of each output row: the gather of the
// wanted positions before the final norm.
template <typename TOut> struct NormStore;
template <> struct NormStore<float> {
  static __device__ __forceinline__ void store4(float* p, float a, float b, float c, float d) {
    *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
  }
};
template <> struct NormStore<__nv_bfloat16> {
  static __device__ __forceinline__ void store4(__nv_bfloat16* p, float a, float b, float c, float d) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    uint2 u;
    u.x = *reinterpret_cast<uint32_t*>(&lo);
    u.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(p) = u;
  }
};

// VEC: rows are read and written four elements at a time (dim a multiple of 4, 16-byte aligned rows).
template <typename TOut, bool VEC>
__global__ void rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ w, TOut* __restrict__ y,
                               const int32_t* __restrict__ rows_idx, int dim, float eps) {
  __shared__ float red[33];
  pdl_launch_dependents();
  pdl_wait();   // (launched as a programmatic dependent: the rows are the kernel before this one's)
  const int r = blockIdx.x;
  const float* xr = x + (size_t)(rows_idx ? rows_idx[r] : r) * dim;
  float ss = 0.f;
  if (VEC) {
    for (int i = threadIdx.x * 4; i < dim; i += blockDim.x * 4) {
      const float4 v = *reinterpret_cast<const float4*>(xr + i);
      ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
    }
  } else {
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {
      const float v = xr[i];
      ss = fmaf(v, v, ss);
    }
  }
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)dim + eps);
  if (VEC) {
    for (int i = threadIdx.x * 4; i < dim; i += blockDim.x * 4) {
      const float4 v = *reinterpret_cast<const float4*>(xr + i);
      const float4 g = *reinterpret_cast<const float4*>(w + i);
      NormStore<TOut>::store4(y + (size_t)r * dim + i, v.x * inv * g.x, v.y * inv * g.y, v.z * inv * g.z, v.w * inv * g.w);
    }
  } else {
    for (int i = threadIdx.x; i < dim; i += blockDim.x) y[(size_t)r * dim + i] = from_f32<TOut>(xr[i] * inv * w[i]);
  }
}

// The same for rows of up to MAXV * 128 values that are read four at a time: a warp a row, the row in registers
// between the sum of squares and the scaling (one pass over memory, no block-wide barrier).
constexpr int NORM_ROW_WARPS = 4;
template <typename TOut, int MAXV>
__global__ void __launch_bounds__(NORM_ROW_WARPS * 32)
rmsnorm_row_kernel(const float* __restrict__ x, const float* __restrict__ w, TOut* __restrict__ y,
                   const int32_t* __restrict__ rows_idx, int rows, int dim, float eps) {
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31;
  const int r = blockIdx.x * NORM_ROW_WARPS + (threadIdx.x >> 5);
  float4 g[MAXV];   // the weights: nothing on the stream writes them, so they are read ahead of the wait
#pragma unroll
  for (int j = 0; j < MAXV; ++j) {
    const int i = lane * 4 + j * 128;
    g[j] = i < dim ? *reinterpret_cast<const float4*>(w + i) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  pdl_wait();   // (launched as a programmatic dependent: the rows are the kernel before this one's)
  if (r >= rows) return;
  const float* xr = x + (size_t)(rows_idx ? rows_idx[r] : r) * dim;
  float4 v[MAXV];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < MAXV; ++j) {
    const int i = lane * 4 + j * 128;
    v[j] = i < dim ? *reinterpret_cast<const float4*>(xr + i) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
#pragma unroll
  for (int j = 0; j < MAXV; ++j) {
    ss = fmaf(v[j].x, v[j].x, ss); ss = fmaf(v[j].y, v[j].y, ss); ss = fmaf(v[j].z, v[j].z, ss); ss = fmaf(v[j].w, v[j].w, ss);
  }
  ss = warp_sum(ss);
  const float inv = 1.0f / sqrtf(ss / (float)dim + eps);
#pragma unroll
  for (int j = 0; j < MAXV; ++j) {
    const int i = lane * 4 + j * 128;
    if (i < dim) NormStore<TOut>::store4(y + (size_t)r * dim + i, v[j].x * inv * g[j].x, v[j].y * inv * g[j].y, v[j].z * inv * g[j].z, v[j].w * inv * g[j].w);
  }
}

// ---------------------------------------------------------------- RoPE + cache append
// qkv: [tokens, (nh + 2 nkv) * hd], the fused projection's output.  For every token: rotate
// the nh query heads in place, rotate the nkv key heads and write them, with the raw value
// heads, into the cache page that holds the token's position.  Rotation in float32 with the
// half-split pairing (i, i + hd/2); cos/sin come from a table [max_pos, hd/2] that the host
// computed in float64.
template <typename T>
__global__ void rope_kv_append_kernel(T* __restrict__ qkv, const int32_t* __restrict__ tok_pos,
                                      const int32_t* __restrict__ tok_seq, const int32_t* __restrict__ seq_slot,
                                      const int32_t* __restrict__ page_table, int table_stride, int n_pages,
                                      const float* __restrict__ cos_t, const float* __restrict__ sin_t, int max_pos,
                                      T* __restrict__ kcache, T* __restrict__ vcache, int nh, int nkv, int hd,
                                      int* __restrict__ err) {
  const int t = blockIdx.x;
  const int pos = tok_pos[t];
  const int half = hd >> 1;
  if (pos < 0 || pos >= max_pos) {
    if (threadIdx.x == 0) atomicOr(err, ERR_POSITION_RANGE);
    return;
  }
  const int slot = seq_slot[tok_seq[t]];
  const int page = page_table[(size_t)slot * table_stride + pos / PAGE];
  if (page < 0 || page >= n_pages) {
    if (threadIdx.x == 0) atomicOr(err, ERR_PAGE_RANGE);
    return;
  }
  const int in_page = pos % PAGE;
  const float* c = cos_t + (size_t)pos * half;
  const float* s = sin_t + (size_t)pos * half;
  T* row = qkv + (size_t)t * (nh + 2 * nkv) * hd;
  // queries, in place
  for (int i = threadIdx.x; i < nh * half; i += blockDim.x) {
    const int h = i / half, j = i - h * half;
    T* p = row + h * hd;
    const float a = to_f32(p[j]), b = to_f32(p[j + half]);
    p[j] = from_f32<T>(a * c[j] - b * s[j]);
    p[j + half] = from_f32<T>(b * c[j] + a * s[j]);
  }
  // keys (rotated) and values (raw) into the page
  const T* krow = row + (size_t)nh * hd;
  const T* vrow = krow + (size_t)nkv * hd;
  for (int i = threadIdx.x; i < nkv * half; i += blockDim.x) {
    const int h = i / half, j = i - h * half;
    const float a = to_f32(krow[h * hd + j]), b = to_f32(krow[h * hd + j + half]);
    T* dst = kcache + (((size_t)page * nkv + h) * PAGE + in_page) * hd;
    dst[j] = from_f32<T>(a * c[j] - b * s[j]);
    dst[j + half] = from_f32<T>(b * c[j] + a * s[j]);
  }
  for (int i = threadIdx.x; i < nkv * hd; i += blockDim.x) {
    const int h = i / hd, j = i - h * hd;
    vcache[(((size_t)page * nkv + h) * PAGE + in_page) * hd + j] = vrow[i];
  }
}

// The same for bfloat16 with head sizes that are multiples of 16, eight elements (16 bytes) at a time: a work item is
// eight rotation pairs of a query or key head (elements j .. j + 7 and their partners half a head further), or eight
// elements of a value head; a block takes `tokens_per_block` tokens.  Same arithmetic as the kernel above and as
// the rotation fused into the decode attention (dm_rotate8).
__global__ void rope_kv_append_vec_kernel(__nv_bfloat16* __restrict__ qkv, const int32_t* __restrict__ tok_pos,
                                          const int32_t* __restrict__ tok_seq, const int32_t* __restrict__ seq_slot,
                                          const int32_t* __restrict__ page_table, int table_stride, int n_pages,
                                          const float* __restrict__ cos_t, const float* __restrict__ sin_t, int max_pos,
                                          __nv_bfloat16* __restrict__ kcache, __nv_bfloat16* __restrict__ vcache, int nh, int nkv,
                                          int hd, int n_tokens, int tokens_per_block, int* __restrict__ err) {
  pdl_launch_dependents();
  pdl_wait();   // (launched as a programmatic dependent: the projections are the kernel before this one's)
  const int half = hd >> 1, per_head = half >> 3;
  const int rot_items = (nh + nkv) * per_head, items = rot_items + nkv * (hd >> 3);
  for (int w = threadIdx.x; w < tokens_per_block * items; w += blockDim.x) {
    const int tl = w / items, it = w - tl * items, t = blockIdx.x * tokens_per_block + tl;
    if (t >= n_tokens) break;
    const int pos = tok_pos[t];
    if (pos < 0 || pos >= max_pos) {
      if (it == 0) atomicOr(err, ERR_POSITION_RANGE);
      continue;
    }
    const int page = page_table[(size_t)seq_slot[tok_seq[t]] * table_stride + pos / PAGE];
    if (page < 0 || page >= n_pages) {
      if (it == 0) atomicOr(err, ERR_PAGE_RANGE);
      continue;
    }
    const int in_page = pos % PAGE;
    __nv_bfloat16* row = qkv + (size_t)t * (nh + 2 * nkv) * hd;
    if (it < rot_items) {
      const int h = it / per_head, j = (it - h * per_head) << 3;   // heads 0 .. nh - 1: queries; then the keys
      __nv_bfloat16* src = row + h * hd + j;
      uint4 lo = *reinterpret_cast<const uint4*>(src), hi = *reinterpret_cast<const uint4*>(src + half);
      dm_rotate8(lo, hi, cos_t + (size_t)pos * half, sin_t + (size_t)pos * half, j);
      __nv_bfloat16* dst = h < nh ? src : kcache + (((size_t)page * nkv + (h - nh)) * PAGE + in_page) * hd + j;
      *reinterpret_cast<uint4*>(dst) = lo;
      *reinterpret_cast<uint4*>(dst + half) = hi;
    } else {
      const int e = (it - rot_items) << 3, h = e / hd, j = e - h * hd;
      *reinterpret_cast<uint4*>(vcache + (((size_t)page * nkv + h) * PAGE + in_page) * hd + j) =
          *reinterpret_cast<const uint4*>(row + (size_t)(nh + nkv) * hd + e);
    }
  }
}

}  // namespace edgelm

using namespace edgelm;

extern "C" int edgelm_embed_gather(const int32_t* ids, const void* table, int table_dtype, float* x, int n_tokens,
                                   int dim, int vocab, int* err, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  EL_REFUSE(n_tokens > 0 && dim > 0 && vocab > 0, "embed_gather: bad sizes tokens=%d dim=%d vocab=%d", n_tokens, dim, vocab);
  const int threads = dim >= 256 ? 256 : 128;
  if (table_dtype == DT_F32)
    embed_gather_kernel<float><<<n_tokens, threads, 0, stream>>>(ids, (const float*)table, x, dim, vocab, err);
  else if (table_dtype == DT_BF16)
    embed_gather_kernel<__nv_bfloat16><<<n_tokens, threads, 0, stream>>>(ids, (const __nv_bfloat16*)table, x, dim, vocab, err);
  else
    EL_REFUSE(false, "embed_gather: unknown dtype code %d", table_dtype);
  EL_LAUNCH_CHECK("embed_gather");
  return 0;
}

extern "C" int edgelm_rmsnorm(const float* x, const float* w, void* y, int out_dtype, const int32_t* rows_idx,
                              int rows, int dim, float eps, cudaStream_t stream) {
  if (rows == 0) return 0;
  EL_REFUSE(rows > 0 && dim > 0, "rmsnorm: bad sizes rows=%d dim=%d", rows, dim);
  const int threads = dim >= 1024 ? 256 : 128;
  const bool vec = dim % 4 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)w % 16 == 0 && (uintptr_t)y % 16 == 0;
  if (vec && dim <= 2048 && (out_dtype == DT_F32 || out_dtype == DT_BF16)) {   // a warp a row, the row in registers
    const dim3 grid((rows + NORM_ROW_WARPS - 1) / NORM_ROW_WARPS), block(NORM_ROW_WARPS * 32);
    if (out_dtype == DT_F32) {
      if (dim <= 640) launch_pdl(32, rmsnorm_row_kernel<float, 5>, grid, block, (size_t)0, stream, x, w, (float*)y, rows_idx, rows, dim, eps);
      else launch_pdl(32, rmsnorm_row_kernel<float, 16>, grid, block, (size_t)0, stream, x, w, (float*)y, rows_idx, rows, dim, eps);
    } else {
      if (dim <= 640) launch_pdl(32, rmsnorm_row_kernel<__nv_bfloat16, 5>, grid, block, (size_t)0, stream, x, w, (__nv_bfloat16*)y, rows_idx, rows, dim, eps);
      else launch_pdl(32, rmsnorm_row_kernel<__nv_bfloat16, 16>, grid, block, (size_t)0, stream, x, w, (__nv_bfloat16*)y, rows_idx, rows, dim, eps);
    }
    EL_LAUNCH_CHECK("rmsnorm");
    return 0;
  }
  if (out_dtype == DT_F32) {
    if (vec) launch_pdl(32, rmsnorm_kernel<float, true>, dim3(rows), dim3(threads), (size_t)0, stream, x, w, (float*)y, rows_idx, dim, eps);
    else launch_pdl(32, rmsnorm_kernel<float, false>, dim3(rows), dim3(threads), (size_t)0, stream, x, w, (float*)y, rows_idx, dim, eps);
  } else if (out_dtype == DT_BF16) {
    if (vec) launch_pdl(32, rmsnorm_kernel<__nv_bfloat16, true>, dim3(rows), dim3(threads), (size_t)0, stream, x, w, (__nv_bfloat16*)y, rows_idx, dim, eps);
    else launch_pdl(32, rmsnorm_kernel<__nv_bfloat16, false>, dim3(rows), dim3(threads), (size_t)0, stream, x, w, (__nv_bfloat16*)y, rows_idx, dim, eps);
  } else
    EL_REFUSE(false, "rmsnorm: unknown dtype code %d", out_dtype);
  EL_LAUNCH_CHECK("rmsnorm");
  return 0;
}

extern "C" int edgelm_rope_kv_append(void* qkv, int dtype, const int32_t* tok_pos, const int32_t* tok_seq,
                                     const int32_t* seq_slot, const int32_t* page_table, int table_stride, int n_pages,
                                     const float* cos_t, const float* sin_t, int max_pos, void* kcache, void* vcache,
                                     int n_tokens, int nh, int nkv, int hd, int* err, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  EL_REFUSE(hd > 0 && hd % 2 == 0, "rope_kv_append: head size %d is not even", hd);
  EL_REFUSE(nh > 0 && nkv > 0 && n_tokens > 0, "rope_kv_append: bad sizes");
  const int threads = 128;
  if (dtype == DT_F32)
    rope_kv_append_kernel<float><<<n_tokens, threads, 0, stream>>>((float*)qkv, tok_pos, tok_seq, seq_slot, page_table,
                                                                    table_stride, n_pages, cos_t, sin_t, max_pos,
                                                                    (float*)kcache, (float*)vcache, nh, nkv, hd, err);
  else if (dtype == DT_BF16 && hd % 16 == 0 && (uintptr_t)qkv % 16 == 0 && (uintptr_t)kcache % 16 == 0 && (uintptr_t)vcache % 16 == 0 &&
           (uintptr_t)cos_t % 16 == 0 && (uintptr_t)sin_t % 16 == 0) {
    const int items = (nh + nkv) * (hd / 16) + nkv * (hd / 8);
    const int per_block = items >= 256 ? 1 : 256 / items;
    launch_pdl(32, rope_kv_append_vec_kernel, dim3((n_tokens + per_block - 1) / per_block), dim3(256), (size_t)0, stream,
               (__nv_bfloat16*)qkv, tok_pos, tok_seq, seq_slot, page_table, table_stride, n_pages, cos_t, sin_t, max_pos,
               (__nv_bfloat16*)kcache, (__nv_bfloat16*)vcache, nh, nkv, hd, n_tokens, per_block, err);
  } else if (dtype == DT_BF16)
    rope_kv_append_kernel<__nv_bfloat16><<<n_tokens, threads, 0, stream>>>(
        (__nv_bfloat16*)qkv, tok_pos, tok_seq, seq_slot, page_table, table_stride, n_pages, cos_t, sin_t, max_pos,
        (__nv_bfloat16*)kcache, (__nv_bfloat16*)vcache, nh, nkv, hd, err);
  else
    EL_REFUSE(false, "rope_kv_append: unknown dtype code %d", dtype);
  EL_LAUNCH_CHECK("rope_kv_append");
  return 0;
}
