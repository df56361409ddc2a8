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
#include <type_traits>

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
                    const int32_t* __restrict__ tile_pos0, int nh, int nkv, int hd, float scale, int window) {
  // window > 0: a token at position p sees the keys p - window + 1 .. p only (0: every key up to p)
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
  int limit[RW], first[RW];
#pragma unroll
  for (int r = 0; r < RW; ++r) {
    m[r] = -CUDART_INF_F;
    l[r] = 0.f;
    const int rr = row_base + warp * RW + r;
    limit[r] = rr < rows_total ? pos0 + rr / g : -1;  // last key this row may see; -1: no row
    first[r] = window > 0 ? max(0, limit[r] - window + 1) : 0;   // first key it may see
#pragma unroll
    for (int c = 0; c < NC; ++c) acc[r][c] = 0.f;
  }
  int warp_limit = -1;
#pragma unroll
  for (int r = 0; r < RW; ++r) warp_limit = max(warp_limit, limit[r]);

  const int n_tiles = (nkeys_block + PAGE - 1) / PAGE;
  // pages before the first key of the block's first row are seen by none of its rows (and may no longer be held)
  const int kt_begin = window > 0 ? max(0, pos0 + row_base / g - window + 1) / PAGE : 0;
  for (int kt = kt_begin; kt < n_tiles; ++kt) {
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
      const float a = j0 <= limit[r] && j0 >= first[r] ? s0[r] * scale : -CUDART_INF_F;
      const float b = j1 <= limit[r] && j1 >= first[r] ? s1[r] * scale : -CUDART_INF_F;
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

// (KVec: 16-byte vector loads of a key row)
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

// ------------------------------------------------------------------------- decode
// One new token per sequence.  grid (sequence, kv head, split), 4 warps per block.  The pages of
// the sequence that fall to this split are cut into tiles of `tk` keys (a tile of K and of V is
// at most 8 KB); tiles are dealt to the block's warps.  For each tile a warp
//   1. has one lane issue two bulk async copies (cp.async.bulk, completion on the warp's
//      mbarrier) that bring the K rows and the V rows, contiguous in the page, into the warp's
//      own shared memory, and waits for them (bounded);
//   2. scores: a lane owns one or two keys and walks its key's 16-byte chunks in an order
//      rotated by the key index, so that the lanes of a quarter-warp read different banks;
//   3. softmax bookkeeping in float32 (running max, sum), probabilities to shared memory;
//   4. values: a lane owns pairs of dims and walks the keys.
// Other warps and blocks of the SM compute while a warp waits for its copy.  Partial results
// meet in shared memory (warps, folded in the order 0..3) and, with more than one split, in the
// scratch that attn_decode_combine_kernel folds in the order of the splits.
constexpr int DEC_WARPS = 4;
constexpr int DEC_TILE_BYTES = 8192;
constexpr long long DEC_WAIT_CYCLES = 2000000000LL;

// Bytes of the decode kernel's shared memory before the per-warp tiles: queries (padded rows), probabilities,
// per-warp partials, the new token's key and value (as floats' worth of room), the warps' mbarriers.
// Floats per staged query row: the head, 4 floats of padding after every 32, rounded to whole 16-byte pieces.
__host__ __device__ inline int decode_query_pitch(int hd) { return (hd + hd / 8 + 3) / 4 * 4; }

__host__ __device__ inline size_t decode_head_bytes(int hd) {
  const size_t floats = (size_t)RW * decode_query_pitch(hd) + (size_t)DEC_WARPS * RW * 64 + (size_t)DEC_WARPS * RW * (hd + 2) + 2 * (size_t)hd;
  return (floats * 4 + DEC_WARPS * 8 + 127) / 128 * 128;
}

__device__ __forceinline__ uint32_t dec_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ bool dec_mbar_try(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}

template <typename T> struct Pair;  // two neighbouring dims of a value row
template <> struct Pair<float> {
  static __device__ __forceinline__ float2 load(const float* p) { return *reinterpret_cast<const float2*>(p); }
  static __device__ __forceinline__ void store(float* p, float a, float b) { *reinterpret_cast<float2*>(p) = make_float2(a, b); }
};
template <> struct Pair<__nv_bfloat16> {
  static __device__ __forceinline__ float2 load(const __nv_bfloat16* p) {
    const uint32_t u = *reinterpret_cast<const uint32_t*>(p);
    return make_float2(__uint_as_float(u << 16), __uint_as_float(u & 0xffff0000u));
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, float a, float b) {
    *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b);
  }
};

// Partial results of one split: part_o [seq][head][split][hd], part_ml [seq][head][split][2].
template <typename T, int NP>  // NP = ceil(hd / 64): pairs of value dims a lane owns
__global__ void __launch_bounds__(DEC_WARPS * 32)
attn_decode_kernel(const T* __restrict__ q, int ldq, T* __restrict__ out, int ldo, T* kcache, T* vcache,
                   const int32_t* __restrict__ page_table, int table_stride, const int32_t* __restrict__ seq_slot,
                   const int32_t* __restrict__ seq_pos, int nh, int nkv, int hd, float scale, int n_splits, int tk,
                   float* __restrict__ part_o, float* __restrict__ part_ml, int* err,
                   const float* __restrict__ cos_t, const float* __restrict__ sin_t, int max_pos, int window) {
  // window > 0: the token sees the last `window` keys only (its own included); the pages before them are not touched.
  // cos_t given: q, k, v are the raw projections of the new token; this kernel rotates q and k at
  // the token's position (float32, half-split pairing, rounded to T as the stand-alone kernel
  // stores them) and the block that owns the token's page appends k and v to the cache.
  constexpr int VEC = KVec<T>::N;
  extern __shared__ __align__(128) uint8_t dec_smem[];
  const int ws = hd + 2;
  const int qp = decode_query_pitch(hd);                          // query row pitch (see qoff)
  float* Qs = reinterpret_cast<float*>(dec_smem);                 // [RW][qp]
  float* Ps = Qs + RW * qp;                                       // [DEC_WARPS][RW][64]
  float* Wp = Ps + DEC_WARPS * RW * 64;                           // [DEC_WARPS][RW][hd + 2]
  T* newkv = reinterpret_cast<T*>(Wp + DEC_WARPS * RW * ws);      // [2][hd]: the new token's rotated key and its value
  uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<float*>(newkv) + 2 * hd);  // [DEC_WARPS]; newkv has room for 2 hd floats
  const size_t head_bytes = decode_head_bytes(hd);
  const int tile_elems = tk * hd;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  T* Kt = reinterpret_cast<T*>(dec_smem + head_bytes) + (size_t)warp * 2 * tile_elems;  // this warp's K tile, then its V tile
  T* Vt = Kt + tile_elems;

  const int seq = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
  const int g = nh / nkv;
  const int nkeys = seq_pos[seq] + 1;      // the new token's own key is the last one
  const int32_t* pages = page_table + (size_t)seq_slot[seq] * table_stride;
  const int first_key = window > 0 ? max(0, nkeys - window) : 0;
  const int page0 = first_key / PAGE;                       // the first page that holds a key the token sees
  const int n_pages = (nkeys + PAGE - 1) / PAGE - page0;
  const int per_split = (n_pages + n_splits - 1) / n_splits;
  const int p_begin = page0 + split * per_split, p_end = min(page0 + n_pages, p_begin + per_split);
  const int tiles_per_page = PAGE / tk;
  const int n_tiles = max(0, p_end - p_begin) * tiles_per_page;
  const int cpr = hd / VEC;                // 16-byte chunks per key row
  const uint32_t bar = dec_smem_u32(&bars[warp]);
  if (lane == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(1));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();
  pdl_launch_dependents();
  pdl_wait();  // everything below reads what earlier kernels of the step wrote
  uint32_t phase = 0;
  bool failed = false;
  // Query floats are read in 16-byte pieces at a per-key rotated chunk; with 8-float chunks (bfloat16
  // keys) chunks four apart would share banks, so every 32 floats are followed by 4 of padding.
  auto qoff = [&](int d) { return VEC == 8 ? d + ((d >> 5) << 2) : d; };
  const int pos = nkeys - 1;
  const int half = hd >> 1;
  const bool fused = cos_t != nullptr;
  const int tpos = min(pos, max_pos - 1);
  const bool owner = fused && (pos / PAGE - page0) / per_split == split;   // this block's pages include the new token's
  if (fused && pos >= max_pos && threadIdx.x == 0 && err) atomicOr(err, ERR_POSITION_RANGE);
  auto rotated = [&](const T* row, int d) {   // element d of the rotated head `row`
    const int j = d < half ? d : d - half;
    const float c = cos_t[(size_t)tpos * half + j], sn = sin_t[(size_t)tpos * half + j];
    const float self = to_f32(row[d]), other = to_f32(row[d < half ? d + half : d - half]);
    const float y = d < half ? self * c - other * sn : self * c + other * sn;
    return to_f32(from_f32<T>(y));
  };
  if (owner) {
    const int page = pages[pos / PAGE];
    const T* krow = q + (size_t)seq * ldq + (size_t)(nh + kvh) * hd;
    const T* vrow = q + (size_t)seq * ldq + (size_t)(nh + nkv + kvh) * hd;
    if (page < 0) {
      if (threadIdx.x == 0 && err) atomicOr(err, ERR_PAGE_RANGE);
    }
    for (int d = threadIdx.x; d < hd; d += blockDim.x) {
      const T kd = from_f32<T>(rotated(krow, d));
      newkv[d] = kd;
      newkv[hd + d] = vrow[d];
      if (page >= 0) {
        const size_t dst = (((size_t)page * nkv + kvh) * PAGE + pos % PAGE) * hd + d;
        kcache[dst] = kd;
        vcache[dst] = vrow[d];
      }
    }
  }
  auto issue_tile = [&](int t) {   // lane 0: start the two bulk copies of tile t into this warp's buffers
    const int pg = p_begin + t / tiles_per_page, sub = t - (t / tiles_per_page) * tiles_per_page;
    const size_t src = (((size_t)pages[pg] * nkv + kvh) * PAGE + (size_t)sub * tk) * hd;
    const uint32_t bytes = (uint32_t)(tile_elems * sizeof(T));
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // earlier reads of the buffers are done
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(2 * bytes) : "memory");
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dec_smem_u32(Kt)), "l"(kcache + src), "r"(bytes), "r"(bar) : "memory");
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dec_smem_u32(Vt)), "l"(vcache + src), "r"(bytes), "r"(bar) : "memory");
  };
  // a tile takes part if it holds a key of the sequence that the token sees (tiles ascend; the first ones of the
  // window's first page may lie before the window)
  auto tile_key0 = [&](int t) { return (p_begin + t / tiles_per_page) * PAGE + (t - (t / tiles_per_page) * tiles_per_page) * tk; };
  bool pre_issued = false;
  if (warp < n_tiles && tile_key0(warp) < nkeys && tile_key0(warp) + tk > first_key) {   // the first tile is on its way while the queries are staged
    if (lane == 0) issue_tile(warp);
    pre_issued = true;
  }

  for (int h0 = 0; h0 < g; h0 += RW) {     // chunks of RW query heads of this kv head
    const int rows = min(RW, g - h0);
    __syncthreads();
    for (int i = threadIdx.x; i < rows * hd; i += blockDim.x) {
      const int r = i / hd, d = i - r * hd;
      const T* qrow = q + (size_t)seq * ldq + (size_t)(kvh * g + h0 + r) * hd;
      Qs[r * qp + qoff(d)] = fused ? rotated(qrow, d) : to_f32(qrow[d]);
    }
    __syncthreads();
    float m[RW], l[RW], acc[RW][NP][2];
#pragma unroll
    for (int r = 0; r < RW; ++r) {
      m[r] = -CUDART_INF_F;
      l[r] = 0.f;
#pragma unroll
      for (int c = 0; c < NP; ++c) acc[r][c][0] = acc[r][c][1] = 0.f;
    }
    for (int t = warp; t < n_tiles && !failed; t += DEC_WARPS) {
      const int pg = p_begin + t / tiles_per_page, sub = t - (t / tiles_per_page) * tiles_per_page;
      const int key0 = pg * PAGE + sub * tk;
      if (key0 >= nkeys) break;            // later tiles of the last page hold no key (tiles ascend)
      if (key0 + tk <= first_key) continue;   // wholly before the window
      const int valid = min(tk, nkeys - key0);
      if (pre_issued) pre_issued = false;   // this tile's copies were started before the queries were staged
      else if (lane == 0) issue_tile(t);
      {  // bounded wait for the two copies
        const long long t0 = clock64();
        bool done = dec_mbar_try(bar, phase);
        while (!done) {
          done = dec_mbar_try(bar, phase);
          if (!done && clock64() - t0 > DEC_WAIT_CYCLES) break;
        }
        failed = !__all_sync(0xffffffffu, done);
        if (failed) break;
        phase ^= 1;
      }
      if (owner && pos >= key0 && pos < key0 + tk) {   // the copy may have read the row before the append landed: put it in by hand
        for (int d = lane; d < hd; d += 32) {
          Kt[(size_t)(pos - key0) * hd + d] = newkv[d];
          Vt[(size_t)(pos - key0) * hd + d] = newkv[hd + d];
        }
        __syncwarp();
      }
      // scores
      float s[2][RW];
#pragma unroll
      for (int kk2 = 0; kk2 < 2; ++kk2) {
        const int kk = lane + 32 * kk2;
#pragma unroll
        for (int r = 0; r < RW; ++r) s[kk2][r] = 0.f;
        if (kk < valid) {
          const T* krow = Kt + (size_t)kk * hd;
          for (int c = 0; c < cpr; ++c) {
            int cc = c + kk;
            cc -= (cc / cpr) * cpr;          // rotated chunk order: neighbouring keys start at different banks
            float kf[VEC];
            KVec<T>::load(krow + cc * VEC, kf);
#pragma unroll
            for (int r = 0; r < RW; ++r) {
              if (r < rows) {
                const float* qr = Qs + r * qp + qoff(cc * VEC);
#pragma unroll
                for (int v = 0; v < VEC; v += 4) {
                  const float4 qv = *reinterpret_cast<const float4*>(qr + v);
                  s[kk2][r] = fmaf(qv.x, kf[v], s[kk2][r]);
                  s[kk2][r] = fmaf(qv.y, kf[v + 1], s[kk2][r]);
                  s[kk2][r] = fmaf(qv.z, kf[v + 2], s[kk2][r]);
                  s[kk2][r] = fmaf(qv.w, kf[v + 3], s[kk2][r]);
                }
              }
            }
          }
        }
      }
      float* pw = Ps + warp * RW * 64;
#pragma unroll
      for (int r = 0; r < RW; ++r) {
        if (r < rows) {
          const float a = lane < valid && key0 + lane >= first_key ? s[0][r] * scale : -CUDART_INF_F;
          const float b = lane + 32 < valid && key0 + lane + 32 >= first_key ? s[1][r] * scale : -CUDART_INF_F;
          const float mx = fmaxf(m[r], warp_max(fmaxf(a, b)));  // finite: the tile holds a key that the token sees
          const float corr = expf(m[r] - mx);
          const float p0 = expf(a - mx), p1 = expf(b - mx);
          l[r] = l[r] * corr + warp_sum(p0 + p1);
          m[r] = mx;
          pw[r * 64 + lane] = p0;
          pw[r * 64 + lane + 32] = p1;
#pragma unroll
          for (int c = 0; c < NP; ++c) {
            acc[r][c][0] *= corr;
            acc[r][c][1] *= corr;
          }
        }
      }
      __syncwarp();
      // values
      for (int j = 0; j < valid; ++j) {
        float2 v[NP];
#pragma unroll
        for (int c = 0; c < NP; ++c) {
          const int d = 2 * lane + 64 * c;
          v[c] = d < hd ? Pair<T>::load(Vt + (size_t)j * hd + d) : make_float2(0.f, 0.f);
        }
#pragma unroll
        for (int r = 0; r < RW; ++r) {
          if (r < rows) {
            const float p = pw[r * 64 + j];
#pragma unroll
            for (int c = 0; c < NP; ++c) {
              acc[r][c][0] = fmaf(p, v[c].x, acc[r][c][0]);
              acc[r][c][1] = fmaf(p, v[c].y, acc[r][c][1]);
            }
          }
        }
      }
      __syncwarp();
    }
    if (failed) {  // a copy did not arrive: report, and make the rows unmistakably wrong
      if (lane == 0 && err) atomicOr(err, ERR_WAIT_TIMEOUT);
#pragma unroll
      for (int r = 0; r < RW; ++r) m[r] = l[r] = CUDART_NAN_F;
    }
    // warps -> shared memory
#pragma unroll
    for (int r = 0; r < RW; ++r) {
      float* w = Wp + (warp * RW + r) * ws;
#pragma unroll
      for (int c = 0; c < NP; ++c) {
        const int d = 2 * lane + 64 * c;
        if (d < hd) {
          w[d] = acc[r][c][0];
          w[d + 1] = acc[r][c][1];
        }
      }
      if (lane == 0) {
        w[hd] = m[r];
        w[hd + 1] = l[r];
      }
    }
    __syncthreads();
    // fold the warps in the order 0..3; warp r folds row r
    if (warp < rows) {
      const int r = warp;
      float M = -CUDART_INF_F;
      for (int w = 0; w < DEC_WARPS; ++w) M = fmaxf(M, Wp[(w * RW + r) * ws + hd]);
      if (M != M) M = CUDART_NAN_F;
      float L = 0.f, o[NP][2];
#pragma unroll
      for (int c = 0; c < NP; ++c) o[c][0] = o[c][1] = 0.f;
      bool bad = false;
      for (int w = 0; w < DEC_WARPS; ++w) bad = bad || (Wp[(w * RW + r) * ws + hd] != Wp[(w * RW + r) * ws + hd]);
      if (M != -CUDART_INF_F && !bad) {
        for (int w = 0; w < DEC_WARPS; ++w) {
          const float* p = Wp + (w * RW + r) * ws;
          if (p[hd] == -CUDART_INF_F) continue;
          const float f = expf(p[hd] - M);
          L = fmaf(p[hd + 1], f, L);
#pragma unroll
          for (int c = 0; c < NP; ++c) {
            const int d = 2 * lane + 64 * c;
            if (d < hd) {
              o[c][0] = fmaf(p[d], f, o[c][0]);
              o[c][1] = fmaf(p[d + 1], f, o[c][1]);
            }
          }
        }
      }
      if (bad) {
        M = 0.f;
        L = CUDART_NAN_F;
      }
      const int head = kvh * g + h0 + r;
      if (n_splits == 1) {
        const float inv = 1.0f / L;
#pragma unroll
        for (int c = 0; c < NP; ++c) {
          const int d = 2 * lane + 64 * c;
          if (d < hd) Pair<T>::store(out + (size_t)seq * ldo + head * hd + d, o[c][0] * inv, o[c][1] * inv);
        }
      } else {
        const size_t pi = ((size_t)seq * nh + head) * n_splits + split;
#pragma unroll
        for (int c = 0; c < NP; ++c) {
          const int d = 2 * lane + 64 * c;
          if (d < hd) {
            part_o[pi * hd + d] = o[c][0];
            part_o[pi * hd + d + 1] = o[c][1];
          }
        }
        if (lane == 0) {
          part_ml[pi * 2] = M;
          part_ml[pi * 2 + 1] = L;
        }
      }
    }
  }
}

}  // namespace edgelm
#include "attention_decode_mma.cuh"
namespace edgelm {

// The fold of up to Q splits whose values a thread holds all at once (see the kernel below): `ml` are the lane's
// maxima and sums (split c * 32 + lane), `dst` the head's row of the output.
template <typename T, int CHUNKS, int DPT, int Q>
__device__ __forceinline__ void fold_eager(const float* __restrict__ part_o, const float2 (&ml)[CHUNKS], size_t base, int n_splits,
                                           int hd, T* __restrict__ dst) {
  float v[Q][DPT];
#pragma unroll
  for (int q = 0; q < Q; ++q)
#pragma unroll
    for (int i = 0; i < DPT; ++i) {
      const int d = threadIdx.x + i * blockDim.x;
      v[q][i] = q < n_splits && d < hd ? part_o[(base + q) * hd + d] : 0.f;
    }
  float M = -CUDART_INF_F;
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) M = fmaxf(M, ml[c].x);
#pragma unroll
  for (int o = 16; o; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
  float f[CHUNKS];
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) f[c] = ml[c].x == -CUDART_INF_F ? 0.f : expf(ml[c].x - M);
  float L = 0.f, acc[DPT];
#pragma unroll
  for (int i = 0; i < DPT; ++i) acc[i] = 0.f;
#pragma unroll
  for (int q = 0; q < Q; ++q) {
    constexpr int LAST = CHUNKS - 1;
    const int c = (q >> 5) < LAST ? (q >> 5) : LAST;
    const float mq = __shfl_sync(0xffffffffu, ml[c].x, q & 31), fq = __shfl_sync(0xffffffffu, f[c], q & 31);
    const float lq = __shfl_sync(0xffffffffu, ml[c].y, q & 31);
    if (q < n_splits && mq != -CUDART_INF_F) {
      L = fmaf(lq, fq, L);
#pragma unroll
      for (int i = 0; i < DPT; ++i) acc[i] = fmaf(v[q][i], fq, acc[i]);
    }
  }
#pragma unroll
  for (int i = 0; i < DPT; ++i) {
    const int d = threadIdx.x + i * blockDim.x;
    if (d < hd) dst[d] = from_f32<T>(acc[i] / L);
  }
}

// One (sequence, head) a block; every warp of the block holds the splits' maxima and sums (a lane a split, up to
// CHUNKS x 32 of them, read once), finds the overall maximum and each split's weight, and walks the splits that hold
// anything, in their order, handing a split's weight and sum round by shuffle: a split that got no page (most of
// them when a short sequence is dealt to many) costs nothing, the exponentials are one per split, not one per split
// and dim, and the splits' weighted values are requested eight at a time, before the maximum is known (which
// splits hold anything shows in the first read): two round trips to memory in all.
template <typename T, int CHUNKS, int DPT>   // DPT: dims a thread of the 64 holds (head size / 64, rounded up)
__global__ void attn_decode_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                           T* __restrict__ out, int ldo, int nh, int hd, int n_splits) {
  const int seq = blockIdx.x, head = blockIdx.y, lane = threadIdx.x & 31;
  const size_t base = ((size_t)seq * nh + head) * n_splits;
  pdl_launch_dependents();
  pdl_wait();  // the partials are the previous kernel's
  float2 ml[CHUNKS];
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
    const int s = c * 32 + lane;
    ml[c] = s < n_splits ? *reinterpret_cast<const float2*>(part_ml + (base + s) * 2) : make_float2(-CUDART_INF_F, 0.f);
  }
  float L = 0.f, acc[DPT];   // dims threadIdx.x, + blockDim.x, ..
#pragma unroll
  for (int i = 0; i < DPT; ++i) acc[i] = 0.f;
  float M = -CUDART_INF_F;
  if (CHUNKS == 1 && n_splits <= 16) {
    // few splits: every split's values are requested at once, beside the maxima and sums, whether the split holds
    // anything or not (one round trip to memory in all); what an empty split's scratch holds is never used.  (With
    // more splits than that most are empty when it matters, and walking the live ones is cheaper.)
    fold_eager<T, CHUNKS, DPT, 16>(part_o, ml, base, n_splits, hd, out + (size_t)seq * ldo + head * hd);
    return;
  }
  bool have_m = false;
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
    unsigned live = __ballot_sync(0xffffffffu, ml[c].x != -CUDART_INF_F);
    float f = 0.f;
    while (live) {   // eight splits at a time: their sums are requested together and added in the splits' order
      int js[8];
      float v[8][DPT];
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        js[q] = live ? __ffs(live) - 1 : -1;
        live &= live - 1;   // (0 stays 0)
        if (js[q] >= 0) {
          const float* po = part_o + (base + c * 32 + js[q]) * hd;
#pragma unroll
          for (int i = 0; i < DPT; ++i) {
            const int d = threadIdx.x + i * blockDim.x;
            v[q][i] = d < hd ? po[d] : 0.f;
          }
        }
      }
      if (!have_m) {   // (once, while the first requests are on their way)
#pragma unroll
        for (int cc = 0; cc < CHUNKS; ++cc) M = fmaxf(M, ml[cc].x);
#pragma unroll
        for (int o = 16; o; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
        have_m = true;
      }
      if (f == 0.f) f = ml[c].x == -CUDART_INF_F ? 0.f : expf(ml[c].x - M);   // (a split that held no page: -inf)
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        if (js[q] >= 0) {
          const float fj = __shfl_sync(0xffffffffu, f, js[q]), lj = __shfl_sync(0xffffffffu, ml[c].y, js[q]);
          L = fmaf(lj, fj, L);
#pragma unroll
          for (int i = 0; i < DPT; ++i) acc[i] = fmaf(v[q][i], fj, acc[i]);
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < DPT; ++i) {
    const int d = threadIdx.x + i * blockDim.x;
    if (d < hd) out[(size_t)seq * ldo + head * hd + d] = from_f32<T>(acc[i] / L);
  }
}

// The fold for any number of splits, one thread a dim, the splits one after the other.
template <typename T>
__global__ void attn_decode_combine_many_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                                T* __restrict__ out, int ldo, int nh, int hd, int n_splits) {
  const int seq = blockIdx.x, head = blockIdx.y;
  const size_t base = ((size_t)seq * nh + head) * n_splits;
  pdl_launch_dependents();
  pdl_wait();  // the partials are the previous kernel's
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
                   int hd, float scale, int window, cudaStream_t stream) {
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
                                              hd, scale, window);
  return 0;
}

// Device error word that decode attention reports a copy that never arrived to when its caller names none (the
// entry point without allocations); may stay null: the affected rows are then NaN, which no caller can overlook.
static int* g_attn_err = nullptr;
static int g_decode_cuda_cores = 0;  // 1: decode attention on the CUDA-core kernel even where the tensor-core one applies
static int g_decode_last_launches = 1;

// Keys per tile: the largest power of two up to 64 whose K rows fit DEC_TILE_BYTES.
static int decode_tile_keys(int hd, size_t elem) {
  int tk = PAGE;
  while (tk > 1 && (size_t)tk * hd * elem > (size_t)DEC_TILE_BYTES) tk >>= 1;
  return tk;
}

template <typename T, int NC>
int launch_decode(const void* q, int ldq, void* out, int ldo, const void* kc, const void* vc, const int32_t* page_table,
                  int table_stride, const int32_t* seq_slot, const int32_t* seq_pos, int n_seqs, int nh, int nkv, int hd,
                  float scale, int n_splits, float* part_o, float* part_ml, int* err, cudaStream_t stream,
                  const float* cos_t = nullptr, const float* sin_t = nullptr, int max_pos = 0, int window = 0, int meta_ready = 0) {
  constexpr int NP = NC <= 2 ? 1 : NC / 2;  // pairs of dims per lane: ceil(hd / 64)
  dim3 grid(n_seqs, nkv, n_splits);
  cudaError_t le = cudaSuccess;
  bool on_mma = false;
  if (err == nullptr) err = g_attn_err;
  if constexpr (sizeof(T) == 2) {
    // bfloat16 with a head size the MMAs tile (32, 64, 96, 128): the tensor-core kernel, whatever the number of
    // query heads a kv head (with one, 15 of the 16 rows are zero, but the kernel is bound by the cache's bytes:
    // measured at 32/32 heads, 1,500 keys, batch 64: 136 us against the CUDA-core kernel's 210 us).
    const bool aligned = ldq % 8 == 0 && (uintptr_t)q % 16 == 0;   // it reads the query rows 16 bytes at a time
    if ((hd == 32 || hd == 64 || hd == 96 || hd == 128) && !g_decode_cuda_cores && aligned && window <= 0) {   // (a window: the CUDA-core kernel)
      on_mma = true;
      const size_t smem = decode_mma_head_bytes(hd) + (size_t)DEC_WARPS * 2 * PAGE * (hd + 8) * 2;
      auto go = [&](auto kern) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = grid;
        cfg.blockDim = dim3(DEC_WARPS * 32);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        int n_attr = 0;
        if (pdl_enabled() & 2) {
          attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
          attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
          ++n_attr;
        }
        cfg.attrs = attr;
        cfg.numAttrs = n_attr;
        return cudaLaunchKernelEx(&cfg, kern, (const __nv_bfloat16*)q, ldq, (__nv_bfloat16*)out, ldo,
                                  (__nv_bfloat16*)const_cast<void*>(kc), (__nv_bfloat16*)const_cast<void*>(vc), page_table, table_stride,
                                  seq_slot, seq_pos, nh, nkv, scale, n_splits, part_o, part_ml, err, cos_t, sin_t, max_pos, meta_ready);
      };
      switch (hd / 16) {
        case 2: le = go(attn_decode_mma_kernel<2>); break;
        case 4: le = go(attn_decode_mma_kernel<4>); break;
        case 6: le = go(attn_decode_mma_kernel<6>); break;
        default: le = go(attn_decode_mma_kernel<8>); break;
      }
    }
  }
  if (!on_mma) {
    const int tk = decode_tile_keys(hd, sizeof(T));
    const size_t smem = decode_head_bytes(hd) + (size_t)DEC_WARPS * 2 * tk * hd * sizeof(T);
    auto kern = attn_decode_kernel<T, NP>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) {
      set_error("attn_decode: %zu bytes of shared memory refused: %s", smem, cudaGetErrorString(e));
      return -2;
    }
    // both kernels are programmatic dependent launches when that is switched on
    le = launch_pdl(2, kern, grid, dim3(DEC_WARPS * 32), smem, stream, (const T*)q, ldq, (T*)out, ldo,
                    (T*)const_cast<void*>(kc), (T*)const_cast<void*>(vc), page_table, table_stride, seq_slot, seq_pos,
                    nh, nkv, hd, scale, n_splits, tk, part_o, part_ml, err, cos_t, sin_t, max_pos, window);
  }
  g_decode_last_launches = n_splits > 1 ? 2 : 1;
  if (le == cudaSuccess && n_splits > 1) {
    dim3 cgrid(n_seqs, nh);
    auto fold = [&](auto kern) {
      return launch_pdl(2, kern, cgrid, dim3(64), 0, stream, (const float*)part_o, (const float*)part_ml, (T*)out, ldo, nh, hd, n_splits);
    };
    // (a lane holds one split of every 32: 1 or 2 of them in registers)
    auto chunks = [&](auto dpt) {
      constexpr int D = decltype(dpt)::value;
      return n_splits <= 32 ? fold(attn_decode_combine_kernel<T, 1, D>) : fold(attn_decode_combine_kernel<T, 2, D>);
    };
    // (more than 64 splits: no step of the engine asks for them; a plain kernel folds those)
    le = n_splits > 64 ? fold(attn_decode_combine_many_kernel<T>)
         : hd <= 64 ? chunks(std::integral_constant<int, 1>{}) : hd <= 128 ? chunks(std::integral_constant<int, 2>{})
         : chunks(std::integral_constant<int, 4>{});
  }
  if (le != cudaSuccess) {
    set_error("attn_decode: launch failed: %s", cudaGetErrorString(le));
    return -2;
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
                                   float scale, int window, cudaStream_t stream) {
  if (n_tiles == 0) return 0;
  if (check_heads("attn_prefill", nh, nkv, hd)) return -1;
  EL_REFUSE(n_tiles > 0 && max_tile_tokens > 0, "attn_prefill: bad tile counts");
  EL_REFUSE(nkv <= 65535 && (max_tile_tokens * (nh / nkv) + ATT_ROWS - 1) / ATT_ROWS <= 65535, "attn_prefill: grid too large");
  EL_ATT_DISPATCH(launch_prefill, q, ldq, out, ldo, kcache, vcache, page_table, table_stride, seq_slot, tile_seq, tile_tok0,
                  tile_ntok, tile_pos0, n_tiles, max_tile_tokens, nh, nkv, hd, scale, window, stream);
  EL_LAUNCH_CHECK("attn_prefill");
  return 0;
}

// 1: decode attention runs on the CUDA-core kernel for every dtype and head size (for comparisons); 0: default.
extern "C" int edgelm_attn_decode_on_cuda_cores(int on) {
  g_decode_cuda_cores = on ? 1 : 0;
  return 0;
}

// Kernels that the last decode attention call of this process launched (1, or 2 with the combine kernel).
extern "C" int edgelm_attn_decode_last_launches() { return g_decode_last_launches; }

// The device error word (one int32) that decode attention ORs ERR_WAIT_TIMEOUT into when a call names none; null: none.
extern "C" int edgelm_attn_set_error_word(int* err) {
  g_attn_err = err;
  return 0;
}

// Scratch: part_o holds n_seqs*nh*n_splits*hd floats, part_ml n_seqs*nh*n_splits*2 (unused when n_splits == 1).
// meta_ready != 0: the caller vouches that seq_pos, seq_slot and page_table were complete before the kernel that
// precedes this call on the stream started; the tensor-core kernel then reads them ahead of its wait for that kernel.
extern "C" int edgelm_attn_decode(const void* q, int ldq, void* out, int ldo, const void* kcache, const void* vcache,
                                  int dtype, const int32_t* page_table, int table_stride, const int32_t* seq_slot,
                                  const int32_t* seq_pos, int n_seqs, int nh, int nkv, int hd, float scale, int n_splits,
                                  float* part_o, float* part_ml, int window, int meta_ready, int* err, cudaStream_t stream) {
  if (n_seqs == 0) return 0;
  if (check_heads("attn_decode", nh, nkv, hd)) return -1;
  EL_REFUSE(n_splits >= 1 && n_splits <= 2048 && nkv <= 65535, "attn_decode: bad split count %d (takes 1 to 2,048)", n_splits);
  EL_REFUSE(n_splits == 1 || (part_o && part_ml), "attn_decode: %d splits need the scratch buffers", n_splits);
  EL_ATT_DISPATCH(launch_decode, q, ldq, out, ldo, kcache, vcache, page_table, table_stride, seq_slot, seq_pos, n_seqs, nh,
                  nkv, hd, scale, n_splits, part_o, part_ml, err, stream, (const float*)nullptr, (const float*)nullptr, 0, window, meta_ready);
  EL_LAUNCH_CHECK("attn_decode");
  return 0;
}

// Decode attention with rotary positions and the cache append fused in: qkv holds the raw q, k, v
// projections of each sequence's new token ([n_seqs, (nh + 2 nkv) hd]); the kernel rotates q and k at
// the token's position with the cos/sin table [max_pos, hd / 2], appends the rotated k and v to the
// cache (kcache, vcache are written) and attends over the cache including the new token.
extern "C" int edgelm_attn_decode_rope(const void* qkv, int ldq, void* out, int ldo, void* kcache, void* vcache, int dtype,
                                       const int32_t* page_table, int table_stride, const int32_t* seq_slot,
                                       const int32_t* seq_pos, const float* cos_t, const float* sin_t, int max_pos,
                                       int n_seqs, int nh, int nkv, int hd, float scale, int n_splits, float* part_o,
                                       float* part_ml, int window, int meta_ready, int* err, cudaStream_t stream) {
  if (n_seqs == 0) return 0;
  if (check_heads("attn_decode_rope", nh, nkv, hd)) return -1;
  EL_REFUSE(n_splits >= 1 && n_splits <= 2048 && nkv <= 65535, "attn_decode_rope: bad split count %d (takes 1 to 2,048)", n_splits);
  EL_REFUSE(n_splits == 1 || (part_o && part_ml), "attn_decode_rope: %d splits need the scratch buffers", n_splits);
  EL_REFUSE(cos_t && sin_t && max_pos > 0, "attn_decode_rope: needs the position table");
  EL_ATT_DISPATCH(launch_decode, qkv, ldq, out, ldo, kcache, vcache, page_table, table_stride, seq_slot, seq_pos, n_seqs, nh,
                  nkv, hd, scale, n_splits, part_o, part_ml, err, stream, cos_t, sin_t, max_pos, window, meta_ready);
  EL_LAUNCH_CHECK("attn_decode_rope");
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
  EL_REFUSE(n_seqs > 0 && n_splits >= 1 && n_splits <= 2048 && nkv <= 65535, "attn_decode_noalloc: bad counts (%d sequences, %d splits)", n_seqs, n_splits);
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
                  nkv, hd, scale, n_splits, part_o, part_ml, (int*)nullptr, stream);
  EL_LAUNCH_CHECK("attn_decode_noalloc");
  return 0;
}
