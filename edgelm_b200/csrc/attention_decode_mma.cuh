// Decode attention on the tensor cores (bfloat16 cache): the variant of attn_decode_kernel whose
// scores and weighted values are mma.sync.m16n8k16 products.  Included by attention.cu, which owns
// the entry points, the split bookkeeping and the combine kernel.
//
// Same decomposition as the CUDA-core kernel: grid (sequence, kv head, split), 4 warps, a warp per
// 64-key tile, partials folded in shared memory and, across splits, by the combine kernel.  What
// differs is inside a tile.  With up to 8 query heads on the kv head the keys are the 16-row operand
// and the heads the 8 columns (S^T = K Q^T, O^T = V^T P^T: dm_tile_update_t), so no row of a product is
// padding; with more, the heads are the rows of a 16-row A operand (rows from g on are zero).  Either
// way one tile costs a few dozen MMAs instead of thousands of multiply-adds: at batch 64 the CUDA-core
// kernel was bound by instruction issue, not by memory.  Key and value rows come by 16-byte cp.async into rows padded by
// 16 bytes (each lane's share arriving on the warp's mbarrier), so that ldmatrix reads hit distinct
// banks; a bulk copy per row, 128 small requests a tile, was bound by their issue.  Value rows of the
// last tile that lie past the sequence's end are zeroed in shared memory before use.
#pragma once
#include "attention_tile_mma.cuh"

namespace edgelm {

// Shared memory before the per-warp tiles: queries [16][hd + 8] bfloat16, the new token's key and value,
// the warps' mbarriers.  (A warp's partial result [16][hd + 2] float goes into its own key tile when its
// tiles are done: 3 blocks of 4 warps then fit an SM at head size 64.)
__host__ __device__ inline size_t decode_mma_head_bytes(int hd) {
  const size_t b = (size_t)DM_ROWS * (hd + 8) * 2 + 2 * (size_t)hd * 2 + DEC_WARPS * 8;
  return (b + 127) / 128 * 128;
}

template <int HDT>  // head size / 16 (2, 4, 6, 8: the MMAs pair up K steps and value columns); up to head size 64
                    // three blocks share an SM's shared memory, so they have to share its registers too
__global__ void __launch_bounds__(DEC_WARPS * 32, HDT <= 4 ? 3 : 1)
attn_decode_mma_kernel(const __nv_bfloat16* __restrict__ q, int ldq, __nv_bfloat16* __restrict__ out, int ldo,
                       __nv_bfloat16* kcache, __nv_bfloat16* vcache, const int32_t* __restrict__ page_table,
                       int table_stride, const int32_t* __restrict__ seq_slot, const int32_t* __restrict__ seq_pos, int nh,
                       int nkv, float scale, int n_splits, float* __restrict__ part_o, float* __restrict__ part_ml, int* err,
                       const float* __restrict__ cos_t, const float* __restrict__ sin_t, int max_pos, int meta_ready) {
  // meta_ready != 0: the lengths, slots and page tables were complete before the kernel that precedes this one on the
  // stream started (a step's metadata, copied at its start).  The block then reads them, down to the page of its first
  // tile, before it waits for that kernel: two round trips to memory that would otherwise follow the wait.
  using T = __nv_bfloat16;
  constexpr int HD = HDT * 16;
  constexpr int PITCH = HD + 8;          // elements per padded row
  constexpr int WS = HD + 2;
  constexpr int TILE = PAGE * PITCH;     // elements of a K (or V) tile in shared memory
  extern __shared__ __align__(128) uint8_t dm_raw[];
  T* Qs = reinterpret_cast<T*>(dm_raw);                                        // [16][PITCH]
  T* newkv = Qs + DM_ROWS * PITCH;                                             // [2][HD]
  uint64_t* bars = reinterpret_cast<uint64_t*>(newkv + 2 * HD);                // [DEC_WARPS]
  static_assert(DM_ROWS * WS * 4 <= TILE * 2, "a warp's partial fits its key tile");
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, gid = lane >> 2, tig = lane & 3;
  T* Kt = reinterpret_cast<T*>(dm_raw + decode_mma_head_bytes(HD)) + (size_t)warp * 2 * TILE;
  T* Vt = Kt + TILE;

  const int seq = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
  const int g = nh / nkv;
  const uint32_t bar = dec_smem_u32(&bars[warp]);
  if (lane == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(32));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();
  pdl_launch_dependents();
  if (!meta_ready) pdl_wait();
  const int nkeys = seq_pos[seq] + 1;
  const int32_t* pages = page_table + (size_t)seq_slot[seq] * table_stride;
  const int n_pages = (nkeys + PAGE - 1) / PAGE;
  const int per_split = (n_pages + n_splits - 1) / n_splits;
  const int p_begin = split * per_split, p_end = min(n_pages, p_begin + per_split);
  const int n_tiles = max(0, p_end - p_begin);   // a tile is a whole page here
  uint32_t phase = 0;
  bool failed = false;

  const int pos = nkeys - 1, half = HD >> 1;
  const bool fused = cos_t != nullptr;
  const int tpos = min(pos, max_pos - 1);
  const bool owner = fused && (pos / PAGE) / per_split == split;
  if (fused && pos >= max_pos && threadIdx.x == 0 && err) atomicOr(err, ERR_POSITION_RANGE);
  int new_page = -1;
  if (owner) {
    new_page = pages[pos / PAGE];
    if (new_page < 0 && threadIdx.x == 0 && err) atomicOr(err, ERR_PAGE_RANGE);
  }
  const int first_page = warp < n_tiles ? pages[p_begin + warp] : 0;
  if (meta_ready) pdl_wait();   // the queries, the new key and value and the cache rows of the step before are the earlier kernels'
  auto issue_tile = [&](int t, int page) {   // whole warp: 16-byte asynchronous copies into padded rows, a lane's share arriving on the warp's mbarrier
    const size_t src = ((size_t)page * nkv + kvh) * PAGE * HD;
#pragma unroll
    for (int i = lane; i < PAGE * (HD / 8); i += 32) {
      const int r = i / (HD / 8), c = (i - r * (HD / 8)) * 8;
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dec_smem_u32(Kt + r * PITCH + c)), "l"(kcache + src + (size_t)r * HD + c) : "memory");
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dec_smem_u32(Vt + r * PITCH + c)), "l"(vcache + src + (size_t)r * HD + c) : "memory");
    }
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
  };
  bool pre_issued = false;
  if (warp < n_tiles) {   // the first tile is on its way while the queries are staged
    issue_tile(warp, first_page);
    pre_issued = true;
  }

  for (int h0 = 0; h0 < g; h0 += DM_ROWS) {   // passes of 16 query heads (one pass unless a kv head serves more)
    const int rows = min(DM_ROWS, g - h0);
    __syncthreads();
    // rows 0 .. rows - 1: the query heads of this pass (rotated when fused; rows from there on are zero); rows 16 and
    // 17, in the block that holds the new token and on the first pass: its rotated key and its value, for the cache
    // and for this block's own tile.  An item is eight dims of a row's first half with their partners in the second.
    for (int i = threadIdx.x; i < DM_ROWS * (HD / 8); i += blockDim.x) {
      const int r = i / (HD / 8), c = (i - r * (HD / 8)) * 8;
      if (r >= rows) *reinterpret_cast<uint4*>(Qs + r * PITCH + c) = make_uint4(0, 0, 0, 0);
    }
    const T* tok = q + (size_t)seq * ldq;
    for (int i = threadIdx.x; i < (rows + (owner && h0 == 0 ? 2 : 0)) * (HD / 16); i += blockDim.x) {
      const int rr = i / (HD / 16), d = (i - rr * (HD / 16)) * 8;
      const int r = rr < rows ? rr : DM_ROWS + (rr - rows);
      const T* row = r < DM_ROWS ? tok + (size_t)(kvh * g + h0 + r) * HD : tok + (size_t)(nh + (r - DM_ROWS) * nkv + kvh) * HD;
      uint4 lo = *reinterpret_cast<const uint4*>(row + d), hi = *reinterpret_cast<const uint4*>(row + half + d);
      if (fused && r != DM_ROWS + 1) dm_rotate8(lo, hi, cos_t + (size_t)tpos * half, sin_t + (size_t)tpos * half, d);
      if (r < DM_ROWS) {
        *reinterpret_cast<uint4*>(Qs + r * PITCH + d) = lo;
        *reinterpret_cast<uint4*>(Qs + r * PITCH + half + d) = hi;
      } else {
        *reinterpret_cast<uint4*>(newkv + (r - DM_ROWS) * HD + d) = lo;
        *reinterpret_cast<uint4*>(newkv + (r - DM_ROWS) * HD + half + d) = hi;
        if (new_page >= 0) {
          T* dst = (r == DM_ROWS ? kcache : vcache) + (((size_t)new_page * nkv + kvh) * PAGE + pos % PAGE) * HD;
          *reinterpret_cast<uint4*>(dst + d) = lo;
          *reinterpret_cast<uint4*>(dst + half + d) = hi;
        }
      }
    }
    __syncthreads();
    auto partial = [&](int w) { return reinterpret_cast<float*>(dm_raw + decode_mma_head_bytes(HD)) + (size_t)w * 2 * TILE / 2; };
    // The warp's tiles one after the other: wait for the copy, mend the tile, `fold(valid)` it into the running state.
    auto each_tile = [&](auto&& fold) {
      for (int t = warp; t < n_tiles && !failed; t += DEC_WARPS) {
        const int key0 = (p_begin + t) * PAGE;
        const int valid = min(PAGE, nkeys - key0);
        if (pre_issued) pre_issued = false;
        else issue_tile(t, pages[p_begin + t]);
        {
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
        if (owner && pos >= key0 && pos < key0 + PAGE) {   // the copy may have read the row before the append landed
          for (int d = lane; d < HD; d += 32) {
            Kt[(pos - key0) * PITCH + d] = newkv[d];
            Vt[(pos - key0) * PITCH + d] = newkv[HD + d];
          }
        }
        if (valid < PAGE) {   // rows past the sequence's end are not this sequence's: their scores are masked whatever the
          // keys hold and their weights are exactly zero; zero values keep a stale NaN from meeting them
          for (int i = lane; i < (PAGE - valid) * (HD / 8); i += 32) {
            const int r = valid + i / (HD / 8), c = i - (i / (HD / 8)) * (HD / 8);
            *reinterpret_cast<uint4*>(Vt + r * PITCH + c * 8) = make_uint4(0, 0, 0, 0);
          }
        }
        __syncwarp();
        fold(valid);
        __syncwarp();
      }
    };
    float mA = -CUDART_INF_F, mB = -CUDART_INF_F, lA = 0.f, lB = 0.f;
    if (g <= DM_HEADS_T) {
      // up to 8 query heads on the kv head: the keys are the 16-row operand (dm_tile_update_t); a lane holds the
      // heads 2 tig and 2 tig + 1, and of each the dims gid and gid + 8 of every block of 16
      uint32_t qb[HDT][2];
      dm_load_queries_t<HDT>(Qs, qb);
      float o[HDT][4];
#pragma unroll
      for (int i = 0; i < HDT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
      each_tile([&](int valid) { dm_tile_update_t<HDT>(Kt, Vt, qb, valid, scale, o, mA, mB, lA, lB); });
      dm_sum_over_keys(lA, lB);
      if (failed) {
        if (lane == 0 && err) atomicOr(err, ERR_WAIT_TIMEOUT);
        mA = mB = lA = lB = CUDART_NAN_F;
      }
      __syncwarp();
      float* wa = partial(warp) + (tig * 2) * WS;      // rows of the partial are heads
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
    } else {
      uint32_t qa[HDT][4];
      dm_load_queries<HDT>(Qs, qa);
      float o[HD / 8][4];
#pragma unroll
      for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
      each_tile([&](int valid) { dm_tile_update<HDT>(Kt, Vt, qa, valid, scale, o, mA, mB, lA, lB); });   // rows gid and gid + 8
      if (failed) {
        if (lane == 0 && err) atomicOr(err, ERR_WAIT_TIMEOUT);
        mA = mB = lA = lB = CUDART_NAN_F;
      }
      // ---- warps -> shared memory (each into its own key tile, which it no longer reads): rows gid and gid + 8
      __syncwarp();
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
    __syncthreads();
    // ---- fold the warps in the order 0..3: threads over (row, pair of dims)
    for (int i = threadIdx.x; i < rows * (HD / 2); i += blockDim.x) {
      const int r = i / (HD / 2), d = (i - r * (HD / 2)) * 2;
      float M = -CUDART_INF_F;
      bool bad = false;
      for (int w = 0; w < DEC_WARPS; ++w) {
        const float mw = partial(w)[r * WS + HD];
        bad = bad || (mw != mw);
        M = fmaxf(M, mw);
      }
      float L = 0.f, o0 = 0.f, o1 = 0.f;
      if (M != -CUDART_INF_F && !bad) {
        for (int w = 0; w < DEC_WARPS; ++w) {
          const float* p = partial(w) + r * WS;
          if (p[HD] == -CUDART_INF_F) continue;
          const float f = expf(p[HD] - M);
          L = fmaf(p[HD + 1], f, L);
          o0 = fmaf(p[d], f, o0);
          o1 = fmaf(p[d + 1], f, o1);
        }
      }
      if (bad) {
        M = 0.f;
        L = CUDART_NAN_F;
      }
      const int head = kvh * g + h0 + r;
      if (n_splits == 1) {
        const float inv = 1.0f / L;
        *reinterpret_cast<__nv_bfloat162*>(out + (size_t)seq * ldo + head * HD + d) = __floats2bfloat162_rn(o0 * inv, o1 * inv);
      } else {
        const size_t pi = ((size_t)seq * nh + head) * n_splits + split;
        part_o[pi * HD + d] = o0;
        part_o[pi * HD + d + 1] = o1;
        if (d == 0) {
          part_ml[pi * 2] = M;
          part_ml[pi * 2 + 1] = L;
        }
      }
    }
  }
}

}  // namespace edgelm
