// Few-rows bfloat16 matrix products for decoding on the tensor cores:
// out[M, N] = act[M, K] . W[N, K]^T for M <= 16, float32 accumulation.
//
// With a handful of rows the work is reading W once; what the CUDA-core kernel (gemv.cu) adds on
// top, eight multiply-adds and eight shared-memory reads per weight and row, is what limits it
// from 4 rows up.  Here the weights are the 16-row operand of mma.sync.m16n8k16 and the batch is
// its 8 columns, so the arithmetic disappears behind the loads:
//   * a block owns 16 output columns (16 rows of W); its warps (4 to 16: more when the output is
//     narrow, so that one round of loads covers K) take the 32-wide K blocks in turn and their
//     partial 16 x 8 tiles are added in shared memory at the end, in the order of the warps;
//   * a lane loads 16 bytes (8 consecutive k) of two weight rows per K block straight from global
//     memory and uses them as the A fragments of two MMAs; the K index inside a block is permuted
//     (the same permutation on both operands leaves the sum unchanged) so that those 16 bytes are
//     exactly the lane's fragment: no shuffles, no staging of W;
//   * the activations of all rows sit in shared memory (pitch chosen so that the fragment reads
//     hit distinct banks), optionally produced here as RMSNorm(x) from the float32 residual
//     stream, rounded to bfloat16 as the stand-alone norm kernel rounds;
//   * epilogues: store (bfloat16 or float32), += residual (float32), SwiGLU of two weights.
// K must be a multiple of 8 with 16-byte aligned rows; M <= 16.  Launched as a programmatic dependent
// launch: the first weight loads are issued before the wait for the previous kernel.
// A launch can be told the weights that the step reads next (`edgelm_gemv_mma_prefetch_next`): its blocks then ask
// the L2 cache for a slice of them each (cp.async.bulk.prefetch.L2) once their own first loads are out, so that the
// next product's transfer from memory runs under this one's waits, staging and epilogue instead of after them.
#include "common.cuh"

namespace edgelm {

enum : int { GM_STORE = 0, GM_RESIDUAL = 1, GM_SWIGLU = 2 };
constexpr int GM_MAX_WARPS = 16;
constexpr int GM_COLS = 16;  // output columns per block
constexpr int GM_K_CHUNK = 4096;  // columns of the activations in shared memory at a time

__device__ __forceinline__ void mma_bf16_16x8x16(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                                 uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ float gm_silu(float z) { return z / (1.0f + expf(-z)); }

// This block's share of `bytes` at `p` (16-byte aligned, a multiple of 16 bytes) into the L2 cache; one thread calls it.
__device__ __forceinline__ void gm_prefetch_slice(const uint8_t* p, unsigned long long bytes) {
  if (p == nullptr || bytes == 0) return;
  const unsigned long long per = ((bytes + gridDim.x - 1) / gridDim.x + 127ull) & ~127ull;
  unsigned long long off = (unsigned long long)blockIdx.x * per;
  if (off >= bytes) return;
  unsigned long long left = (bytes - off < per ? bytes - off : per) & ~15ull;
  while (left) {
    const unsigned int n = left < 16384ull ? (unsigned int)left : 16384u;
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p + off), "r"(n) : "memory");
    off += n;
    left -= n;
  }
}

// NT: 8-row tiles of the batch (1: M <= 8, 2: M <= 16).  NORM: activations = RMSNorm(x).
// MAXW: the most warps a block is launched with.  UN: K blocks whose weight loads a warp has in flight together
// (4, or 8 for long rows of a single weight: 64 registers of weights either way).
template <int EPI, typename TOut, int NT, bool NORM, int MAXW, int UN>
__global__ void __launch_bounds__(MAXW * 32)
gemv_mma_kernel(const __nv_bfloat16* __restrict__ act, int lda, const float* __restrict__ x,
                const float* __restrict__ norm_w, float eps, const __nv_bfloat16* __restrict__ W,
                const __nv_bfloat16* __restrict__ W2, TOut* out, int ldo, const float* residual, int M, int N, int K,
                int pitch /* bfloat16 elements per activation row in shared memory */,
                int kc /* columns of the activations staged at a time: a multiple of 32 */,
                const uint8_t* next0, unsigned long long next0_bytes, const uint8_t* next1, unsigned long long next1_bytes) {
  constexpr int NW = EPI == GM_SWIGLU ? 2 : 1;
  constexpr int ROWS = 8 * NT;
  const int GM_WARPS = blockDim.x >> 5;  // the block's warps share the K blocks
  extern __shared__ __align__(16) uint8_t gm_smem[];
  __nv_bfloat16* As = reinterpret_cast<__nv_bfloat16*>(gm_smem);                       // [ROWS][pitch]
  float* red = reinterpret_cast<float*>(gm_smem + (size_t)ROWS * pitch * 2);           // [GM_WARPS][NW][NT][32][4]
  float* inv = red + GM_WARPS * NW * NT * 128;                                         // [ROWS]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int gid = lane >> 2, tig = lane & 3;
  const int n0 = blockIdx.x * GM_COLS;
  const int ra = min(n0 + gid, N - 1), rb = min(n0 + gid + 8, N - 1);  // the two weight rows of this lane (clamped)
  const int n_kb = (K + 31) / 32;

  // Weights on their way while the activations are staged.  With one weight: the warp's whole first round of every
  // chunk, loaded into the registers the MMAs read (ea, eb: no second copy).  With two weights a round is 64 registers
  // held across the staging, which cost those kernels more than the loads gained (17.8 -> 21.5 us at N 8192, K 2048):
  // there only the first K block is ahead (pa, pb).
  constexpr bool EARLY = NW == 1;
  uint4 ea[EARLY ? UN : 1], eb[EARLY ? UN : 1];
  auto load_round = [&](int kb0, int kb_end) {
#pragma unroll
    for (int u = 0; u < (EARLY ? UN : 0); ++u) {
      const int kb = kb0 + u * GM_WARPS;
      const int k = kb * 32 + tig * 8;
      const bool ok = kb < kb_end && k < K;
      ea[u] = ok ? *reinterpret_cast<const uint4*>(W + (size_t)ra * K + k) : make_uint4(0, 0, 0, 0);
      eb[u] = ok ? *reinterpret_cast<const uint4*>(W + (size_t)rb * K + k) : make_uint4(0, 0, 0, 0);
    }
  };
  if (EARLY) load_round(warp, (min(kc, K) + 31) / 32);
  uint4 pa[NW], pb[NW];
  if (!EARLY) {
    const int k = warp * 32 + tig * 8;
    const bool ok = warp < n_kb && k < K;
#pragma unroll
    for (int w = 0; w < NW; ++w) {
      const __nv_bfloat16* Wp = w == 0 ? W : W2;
      pa[w] = ok ? *reinterpret_cast<const uint4*>(Wp + (size_t)ra * K + k) : make_uint4(0, 0, 0, 0);
      pb[w] = ok ? *reinterpret_cast<const uint4*>(Wp + (size_t)rb * K + k) : make_uint4(0, 0, 0, 0);
    }
  }

  if (threadIdx.x == 0) {   // (weights: nothing on the stream writes them)
    gm_prefetch_slice(next0, next0_bytes);
    gm_prefetch_slice(next1, next1_bytes);
  }
  pdl_launch_dependents();
  pdl_wait();  // from here on: activations that the kernel before this one wrote
  // the residual values that the epilogue adds to, requested now by the warp that will run it: a round trip to
  // memory less at the end of the block's life (out may be the residual itself: nobody else writes these elements)
  float res_ahead[NT][4];
  if (EPI == GM_RESIDUAL && warp == 0) {
#pragma unroll
    for (int t = 0; t < NT; ++t)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int n = n0 + gid + (j >> 1) * 8, m = t * 8 + tig * 2 + (j & 1);
        res_ahead[t][j] = n < N && m < M ? residual[(size_t)m * ldo + n] : 0.f;
      }
  }
  // ---- activations into shared memory (rows >= M are zero)
  // A normalised row of up to 1,024 values in one chunk: a warp takes a row, keeps it in registers between the sum of
  // squares and the scaling and writes it out rounded: one pass over x, with the norm's weights requested beside it.
  const bool one_pass = NORM && K <= 1024 && K <= kc;
  if (NORM && one_pass) {
    float4 g[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int k = lane * 4 + j * 128;
      g[j] = k < K ? *reinterpret_cast<const float4*>(norm_w + k) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    for (int r = warp; r < ROWS; r += GM_WARPS) {
      float4 v[8];
      float ss = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int k = lane * 4 + j * 128;
        v[j] = r < M && k < K ? *reinterpret_cast<const float4*>(x + (size_t)r * K + k) : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        ss = fmaf(v[j].x, v[j].x, ss); ss = fmaf(v[j].y, v[j].y, ss); ss = fmaf(v[j].z, v[j].z, ss); ss = fmaf(v[j].w, v[j].w, ss);
      }
      ss = warp_sum(ss);
      const float sc = r < M ? 1.0f / sqrtf(ss / (float)K + eps) : 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int k = lane * 4 + j * 128;
        if (k < K) {
          __nv_bfloat162 h0 = __floats2bfloat162_rn(v[j].x * sc * g[j].x, v[j].y * sc * g[j].y);
          __nv_bfloat162 h1 = __floats2bfloat162_rn(v[j].z * sc * g[j].z, v[j].w * sc * g[j].w);
          uint2 u;
          u.x = *reinterpret_cast<uint32_t*>(&h0);
          u.y = *reinterpret_cast<uint32_t*>(&h1);
          *reinterpret_cast<uint2*>(As + (size_t)r * pitch + k) = u;
        }
      }
    }
  } else if (NORM) {
    for (int r = warp; r < ROWS; r += GM_WARPS) {
      float ss = 0.f;
      if (r < M) {
        const float* xr = x + (size_t)r * K;
#pragma unroll 4
        for (int k = lane * 4; k < K; k += 128) {
          const float4 v = *reinterpret_cast<const float4*>(xr + k);
          ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
        }
      }
      ss = warp_sum(ss);
      if (lane == 0) inv[r] = 1.0f / sqrtf(ss / (float)K + eps);
    }
    __syncthreads();
  }
  float acc[NW][NT][4];
#pragma unroll
  for (int w = 0; w < NW; ++w)
#pragma unroll
    for (int t = 0; t < NT; ++t)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[w][t][j] = 0.f;

  for (int kc0 = 0; kc0 < K; kc0 += kc) {   // K in chunks whose activations fit shared memory (one chunk for the usual sizes)
    const int kn = min(kc, K - kc0);
    if (kc0) {
      if (EARLY) load_round(kc0 / 32 + warp, (kc0 + kn + 31) / 32);
      __syncthreads();                      // the previous chunk's activations are used up
    }
    const int kvec = kn / 8;
    if (!NORM) {
      // 16-byte asynchronous copies: all of a thread's pieces are in flight together (one load at a time, a
      // round trip each, was most of a block's life at K = 2048 and beyond); through L1, where the blocks that
      // follow on the same SM find them
      for (int i = threadIdx.x; i < ROWS * kvec; i += blockDim.x) {
        const int r = i / kvec, k = kc0 + (i - r * kvec) * 8;
        __nv_bfloat16* dst = As + (size_t)r * pitch + (k - kc0);
        if (r < M)
          asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(act + (size_t)r * lda + k) : "memory");
        else
          *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
      }
      asm volatile("cp.async.wait_all;" ::: "memory");
    } else if (!one_pass) {
      for (int i0 = threadIdx.x; i0 < ROWS * kvec; i0 += blockDim.x * 2) {   // two pieces' loads in flight together
        float4 x0[2], x1[2], w0[2], w1[2];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const int i = i0 + j * blockDim.x, r = i / kvec, k = kc0 + (i - r * kvec) * 8;
          const bool ok = i < ROWS * kvec && r < M;
          x0[j] = ok ? *reinterpret_cast<const float4*>(x + (size_t)r * K + k) : make_float4(0.f, 0.f, 0.f, 0.f);
          x1[j] = ok ? *reinterpret_cast<const float4*>(x + (size_t)r * K + k + 4) : make_float4(0.f, 0.f, 0.f, 0.f);
          w0[j] = ok ? *reinterpret_cast<const float4*>(norm_w + k) : make_float4(0.f, 0.f, 0.f, 0.f);
          w1[j] = ok ? *reinterpret_cast<const float4*>(norm_w + k + 4) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const int i = i0 + j * blockDim.x, r = i / kvec, k = (i - r * kvec) * 8;
          if (i < ROWS * kvec) {
            const float s = r < M ? inv[r] : 0.f;
            __nv_bfloat162 h0 = __floats2bfloat162_rn(x0[j].x * s * w0[j].x, x0[j].y * s * w0[j].y);
            __nv_bfloat162 h1 = __floats2bfloat162_rn(x0[j].z * s * w0[j].z, x0[j].w * s * w0[j].w);
            __nv_bfloat162 h2 = __floats2bfloat162_rn(x1[j].x * s * w1[j].x, x1[j].y * s * w1[j].y);
            __nv_bfloat162 h3 = __floats2bfloat162_rn(x1[j].z * s * w1[j].z, x1[j].w * s * w1[j].w);
            uint4 v;
            v.x = *reinterpret_cast<uint32_t*>(&h0);
            v.y = *reinterpret_cast<uint32_t*>(&h1);
            v.z = *reinterpret_cast<uint32_t*>(&h2);
            v.w = *reinterpret_cast<uint32_t*>(&h3);
            *reinterpret_cast<uint4*>(As + (size_t)r * pitch + k) = v;
          }
        }
      }
    }
    __syncthreads();

    const int kb_begin = kc0 / 32, kb_end = (kc0 + kn + 31) / 32;
    if constexpr (EARLY) {
      for (int kb0 = kb_begin + warp; kb0 < kb_end; kb0 += GM_WARPS * UN) {
        if (kb0 != kb_begin + warp) load_round(kb0, kb_end);
#pragma unroll
        for (int u = 0; u < UN; ++u) {
          const int kb = kb0 + u * GM_WARPS;
          const int k = kb * 32 + tig * 8;
          const bool ok = kb < kb_end && k < K;
#pragma unroll
          for (int t = 0; t < NT; ++t) {
            const uint4 av = ok ? *reinterpret_cast<const uint4*>(As + (size_t)(t * 8 + gid) * pitch + (k - kc0)) : make_uint4(0, 0, 0, 0);
            mma_bf16_16x8x16(acc[0][t], ea[u].x, eb[u].x, ea[u].y, eb[u].y, av.x, av.y);
            mma_bf16_16x8x16(acc[0][t], ea[u].z, eb[u].z, ea[u].w, eb[u].w, av.z, av.w);
          }
        }
      }
    } else
    for (int kb0 = kb_begin + warp; kb0 < kb_end; kb0 += GM_WARPS * UN) {
      uint4 wa[UN][NW], wb[UN][NW];
#pragma unroll
      for (int u = 0; u < UN; ++u) {
        const int kb = kb0 + u * GM_WARPS;
        const int k = kb * 32 + tig * 8;
        const bool ok = kb < kb_end && k < K;
#pragma unroll
        for (int w = 0; w < NW; ++w) {
          if (u == 0 && kb0 == warp) {
            wa[u][w] = pa[w];
            wb[u][w] = pb[w];
          } else {
            const __nv_bfloat16* Wp = w == 0 ? W : W2;
            wa[u][w] = ok ? *reinterpret_cast<const uint4*>(Wp + (size_t)ra * K + k) : make_uint4(0, 0, 0, 0);
            wb[u][w] = ok ? *reinterpret_cast<const uint4*>(Wp + (size_t)rb * K + k) : make_uint4(0, 0, 0, 0);
          }
        }
      }
#pragma unroll
      for (int u = 0; u < UN; ++u) {
        const int kb = kb0 + u * GM_WARPS;
        const int k = kb * 32 + tig * 8;
        const bool ok = kb < kb_end && k < K;
#pragma unroll
        for (int t = 0; t < NT; ++t) {
          const uint4 av = ok ? *reinterpret_cast<const uint4*>(As + (size_t)(t * 8 + gid) * pitch + (k - kc0)) : make_uint4(0, 0, 0, 0);
#pragma unroll
          for (int w = 0; w < NW; ++w) {
            mma_bf16_16x8x16(acc[w][t], wa[u][w].x, wb[u][w].x, wa[u][w].y, wb[u][w].y, av.x, av.y);
            mma_bf16_16x8x16(acc[w][t], wa[u][w].z, wb[u][w].z, wa[u][w].w, wb[u][w].w, av.z, av.w);
          }
        }
      }
    }
  }

  // ---- add the warps' partial tiles (in the order of the warps), then the epilogue by warp 0
  float* mine = red + (size_t)warp * NW * NT * 128;
#pragma unroll
  for (int w = 0; w < NW; ++w)
#pragma unroll
    for (int t = 0; t < NT; ++t)
      *reinterpret_cast<float4*>(mine + ((w * NT + t) * 32 + lane) * 4) = make_float4(acc[w][t][0], acc[w][t][1], acc[w][t][2], acc[w][t][3]);
  __syncthreads();
  if (warp != 0) return;
#pragma unroll
  for (int t = 0; t < NT; ++t) {
    float s[NW][4];
#pragma unroll
    for (int w = 0; w < NW; ++w) {
#pragma unroll
      for (int j = 0; j < 4; ++j) s[w][j] = 0.f;
      for (int ww = 0; ww < GM_WARPS; ++ww) {
        const float4 p = *reinterpret_cast<const float4*>(red + (((size_t)ww * NW + w) * NT + t) * 128 + lane * 4);
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
        if (EPI == GM_STORE) out[idx] = from_f32<TOut>(s[0][j]);
        if (EPI == GM_RESIDUAL) out[idx] = from_f32<TOut>(res_ahead[t][j] + s[0][j]);
        if (EPI == GM_SWIGLU) out[idx] = from_f32<TOut>(gm_silu(s[0][j]) * s[NW - 1][j]);
      }
    }
  }
}

// The same product for outputs so wide that every SM would get several blocks of 16 columns one after the other
// (the vocabulary, the projections of a wide model): a fixed number of blocks, 16 warps' worth an SM, each of which
// stages the activations once and walks the groups of 16 columns blockIdx.x, blockIdx.x + gridDim.x, ...; the first
// weights of a block's next group are on their way while the warps' partial tiles of this one are added up and
// stored.  (One block a group: 384 to 3,072 blocks came in one and a half to seven waves, each block staged all
// activations again, and nothing streamed while a block staged, reduced and stored.)  All of K in one chunk of
// activations; no norm prologue, no residual epilogue (none of the wide products has them).
template <int EPI, typename TOut, int NT, int MAXW, int UN>
__global__ void __launch_bounds__(MAXW * 32, GM_MAX_WARPS / MAXW)
gemv_mma_walk_kernel(const __nv_bfloat16* __restrict__ act, int lda, const __nv_bfloat16* __restrict__ W,
                     const __nv_bfloat16* __restrict__ W2, TOut* out, int ldo, int M, int N, int K,
                     int pitch /* bfloat16 elements per activation row in shared memory */, int n_groups,
                     const uint8_t* next0, unsigned long long next0_bytes, const uint8_t* next1, unsigned long long next1_bytes) {
  constexpr int NW = EPI == GM_SWIGLU ? 2 : 1;
  constexpr int ROWS = 8 * NT;
  const int GM_WARPS = blockDim.x >> 5;
  extern __shared__ __align__(16) uint8_t gm_smem[];
  __nv_bfloat16* As = reinterpret_cast<__nv_bfloat16*>(gm_smem);                       // [ROWS][pitch]
  float* red = reinterpret_cast<float*>(gm_smem + (size_t)ROWS * pitch * 2);           // [2][GM_WARPS][NW][NT][32][4]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int gid = lane >> 2, tig = lane & 3;
  const int n_kb = (K + 31) / 32;
  int grp = blockIdx.x;
  int ra = min(grp * GM_COLS + gid, N - 1), rb = min(grp * GM_COLS + gid + 8, N - 1);  // the two weight rows of this lane (clamped)

  constexpr bool EARLY = NW == 1;   // (as in the kernel above: a whole round ahead with one weight, a K block with two)
  uint4 ea[EARLY ? UN : 1], eb[EARLY ? UN : 1];
  auto load_round = [&](int kb0) {
#pragma unroll
    for (int u = 0; u < (EARLY ? UN : 0); ++u) {
      const int kb = kb0 + u * GM_WARPS;
      const int k = kb * 32 + tig * 8;
      const bool ok = kb < n_kb && k < K;
      ea[u] = ok ? *reinterpret_cast<const uint4*>(W + (size_t)ra * K + k) : make_uint4(0, 0, 0, 0);
      eb[u] = ok ? *reinterpret_cast<const uint4*>(W + (size_t)rb * K + k) : make_uint4(0, 0, 0, 0);
    }
  };
  uint4 pa[NW], pb[NW];
  auto load_first = [&]() {
    const int k = warp * 32 + tig * 8;
    const bool ok = warp < n_kb && k < K;
#pragma unroll
    for (int w = 0; w < NW; ++w) {
      const __nv_bfloat16* Wp = w == 0 ? W : W2;
      pa[w] = ok ? *reinterpret_cast<const uint4*>(Wp + (size_t)ra * K + k) : make_uint4(0, 0, 0, 0);
      pb[w] = ok ? *reinterpret_cast<const uint4*>(Wp + (size_t)rb * K + k) : make_uint4(0, 0, 0, 0);
    }
  };
  if (EARLY) load_round(warp);
  else load_first();
  if (threadIdx.x == 0) {
    gm_prefetch_slice(next0, next0_bytes);
    gm_prefetch_slice(next1, next1_bytes);
  }
  pdl_launch_dependents();
  pdl_wait();  // from here on: activations that the kernel before this one wrote
  // ---- activations into shared memory, once (rows >= M are zero)
  {
    const int kvec = K / 8;
    for (int i = threadIdx.x; i < ROWS * kvec; i += blockDim.x) {
      const int r = i / kvec, k = (i - r * kvec) * 8;
      __nv_bfloat16* dst = As + (size_t)r * pitch + k;
      if (r < M)
        asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(act + (size_t)r * lda + k) : "memory");
      else
        *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
    }
    asm volatile("cp.async.wait_all;" ::: "memory");
  }
  __syncthreads();

  for (int it = 0; grp < n_groups; ++it) {
    float acc[NW][NT][4];
#pragma unroll
    for (int w = 0; w < NW; ++w)
#pragma unroll
      for (int t = 0; t < NT; ++t)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[w][t][j] = 0.f;
    if constexpr (EARLY) {
      for (int kb0 = warp; kb0 < n_kb; kb0 += GM_WARPS * UN) {
        if (kb0 != warp) load_round(kb0);
#pragma unroll
        for (int u = 0; u < UN; ++u) {
          const int kb = kb0 + u * GM_WARPS;
          const int k = kb * 32 + tig * 8;
          const bool ok = kb < n_kb && k < K;
#pragma unroll
          for (int t = 0; t < NT; ++t) {
            const uint4 av = ok ? *reinterpret_cast<const uint4*>(As + (size_t)(t * 8 + gid) * pitch + k) : make_uint4(0, 0, 0, 0);
            mma_bf16_16x8x16(acc[0][t], ea[u].x, eb[u].x, ea[u].y, eb[u].y, av.x, av.y);
            mma_bf16_16x8x16(acc[0][t], ea[u].z, eb[u].z, ea[u].w, eb[u].w, av.z, av.w);
          }
        }
      }
    } else {
      for (int kb0 = warp; kb0 < n_kb; kb0 += GM_WARPS * UN) {
        uint4 wa[UN][NW], wb[UN][NW];
#pragma unroll
        for (int u = 0; u < UN; ++u) {
          const int kb = kb0 + u * GM_WARPS;
          const int k = kb * 32 + tig * 8;
          const bool ok = kb < n_kb && k < K;
#pragma unroll
          for (int w = 0; w < NW; ++w) {
            if (u == 0 && kb0 == warp) {
              wa[u][w] = pa[w];
              wb[u][w] = pb[w];
            } else {
              const __nv_bfloat16* Wp = w == 0 ? W : W2;
              wa[u][w] = ok ? *reinterpret_cast<const uint4*>(Wp + (size_t)ra * K + k) : make_uint4(0, 0, 0, 0);
              wb[u][w] = ok ? *reinterpret_cast<const uint4*>(Wp + (size_t)rb * K + k) : make_uint4(0, 0, 0, 0);
            }
          }
        }
#pragma unroll
        for (int u = 0; u < UN; ++u) {
          const int kb = kb0 + u * GM_WARPS;
          const int k = kb * 32 + tig * 8;
          const bool ok = kb < n_kb && k < K;
#pragma unroll
          for (int t = 0; t < NT; ++t) {
            const uint4 av = ok ? *reinterpret_cast<const uint4*>(As + (size_t)(t * 8 + gid) * pitch + k) : make_uint4(0, 0, 0, 0);
#pragma unroll
            for (int w = 0; w < NW; ++w) {
              mma_bf16_16x8x16(acc[w][t], wa[u][w].x, wb[u][w].x, wa[u][w].y, wb[u][w].y, av.x, av.y);
              mma_bf16_16x8x16(acc[w][t], wa[u][w].z, wb[u][w].z, wa[u][w].w, wb[u][w].w, av.z, av.w);
            }
          }
        }
      }
    }
    // ---- the next group's first weights set out; then the warps' partial tiles are added (in the order of the
    // warps) and stored by warp 0, out of the half of `red` that belongs to this turn
    const int n0 = grp * GM_COLS;
    grp += gridDim.x;
    if (grp < n_groups) {
      ra = min(grp * GM_COLS + gid, N - 1), rb = min(grp * GM_COLS + gid + 8, N - 1);
      if (EARLY) load_round(warp);
      else load_first();
    }
    float* turn = red + (size_t)(it & 1) * GM_WARPS * NW * NT * 128;
    float* mine = turn + (size_t)warp * NW * NT * 128;
#pragma unroll
    for (int w = 0; w < NW; ++w)
#pragma unroll
      for (int t = 0; t < NT; ++t)
        *reinterpret_cast<float4*>(mine + ((w * NT + t) * 32 + lane) * 4) = make_float4(acc[w][t][0], acc[w][t][1], acc[w][t][2], acc[w][t][3]);
    __syncthreads();
    if (warp != 0) continue;
#pragma unroll
    for (int t = 0; t < NT; ++t) {
      float s[NW][4];
#pragma unroll
      for (int w = 0; w < NW; ++w) {
#pragma unroll
        for (int j = 0; j < 4; ++j) s[w][j] = 0.f;
        for (int ww = 0; ww < GM_WARPS; ++ww) {
          const float4 p = *reinterpret_cast<const float4*>(turn + (((size_t)ww * NW + w) * NT + t) * 128 + lane * 4);
          s[w][0] += p.x; s[w][1] += p.y; s[w][2] += p.z; s[w][3] += p.w;
        }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int n = n0 + gid + (j >> 1) * 8;
        const int m = t * 8 + tig * 2 + (j & 1);
        if (n < N && m < M) {
          const size_t idx = (size_t)m * ldo + n;
          if (EPI == GM_STORE) out[idx] = from_f32<TOut>(s[0][j]);
          if (EPI == GM_SWIGLU) out[idx] = from_f32<TOut>(gm_silu(s[0][j]) * s[NW - 1][j]);
        }
      }
    }
  }
}

// What the next launch from this thread prefetches (set by edgelm_gemv_mma_prefetch_next, cleared by the launch).
struct NextWeights {
  const uint8_t* p;
  unsigned long long bytes;
};
static thread_local NextWeights g_next[2] = {{nullptr, 0}, {nullptr, 0}};
static int g_walk = 1;   // 0: wide outputs also go to the kernel of one block a column group (comparisons)

// Activation row pitch in shared memory: K rounded up so that pitch * 2 bytes = 64 (mod 128); then
// the fragment reads of a quarter-warp (two rows, four 16-byte chunks each) hit distinct banks.
static int act_pitch(int K) {
  int p = (K + 7) / 8 * 8;
  while ((p * 2) % 128 != 64) p += 8;
  return p;
}

template <int EPI, typename TOut, int NT, bool NORM>
static int launch_gemv_mma(const void* act, int lda, const float* x, const float* norm_w, float eps, const void* W,
                           const void* W2, void* out, int ldo, const float* residual, int M, int N, int K,
                           cudaStream_t stream) {
  constexpr int NW = EPI == GM_SWIGLU ? 2 : 1;
  const int kc = K <= GM_K_CHUNK ? (K + 31) / 32 * 32 : GM_K_CHUNK;
  const int pitch = act_pitch(kc);
  // warps per block: wide outputs fill the device with blocks and want few warps; narrow ones get up to
  // 16 warps, about two K blocks each, so that a single round of loads is in flight per warp
  const int n_kb = (K + 31) / 32, blocks = (N + GM_COLS - 1) / GM_COLS;
  // warps per block: as many (up to 16) as it takes to have all of K in flight in one round of loads, unless the
  // output is so wide that the device is full of blocks anyway (the vocabulary product); a narrow output gets at
  // least about two K blocks a warp
  const bool deep = NW == 1 && n_kb >= 64;   // rows of 2,048 and more of one weight: eight K blocks in flight per warp
  const int un = deep ? 8 : 4;
  int GM_WARPS = 4;
  if (blocks < 2 * 148) {
    while (GM_WARPS < GM_MAX_WARPS && GM_WARPS * 2 <= (n_kb + 1) / 2) GM_WARPS *= 2;
  } else if (blocks < 8 * 148) {
    while (GM_WARPS < GM_MAX_WARPS && n_kb > GM_WARPS * un) GM_WARPS *= 2;
  }
  if constexpr (!NORM && EPI != GM_RESIDUAL) {
    // outputs of at least two blocks of 16 columns for every SM, all of K in one chunk: the walking kernel, 16 warps'
    // worth of blocks an SM, a block's warps as many as it takes to have all of K in flight in one round
    // (measured at 8 rows: N 6144, K 2048: 8.6 -> 7.4 us; N 2 x 8192, K 2048: 16.5 -> 15.5; N 49152, K 2048: 41.0 -> 34.3;
    // a short K loses a little, N 49152, K 576: 10.5 -> 11.0 us, and keeps the other kernel)
    if (g_walk && blocks >= 2 * 148 && K <= GM_K_CHUNK && K >= 1024) {
      int ww = 4;
      while (ww < GM_MAX_WARPS && ww * un < n_kb) ww *= 2;
      static int n_sms = 0;
      if (n_sms == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&n_sms, cudaDevAttrMultiProcessorCount, dev);
        if (n_sms <= 0) n_sms = 148;
      }
      const int grid = blocks < n_sms * (GM_MAX_WARPS / ww) ? blocks : n_sms * (GM_MAX_WARPS / ww);
      const size_t wsmem = (size_t)8 * NT * pitch * 2 + (size_t)2 * ww * NW * NT * 128 * 4;
      auto walk = [&](auto kern) -> int {
        if (wsmem > 48 * 1024) {
          cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)wsmem);
          if (e != cudaSuccess) {
            set_error("gemv_mma: %zu bytes of shared memory refused (K = %d): %s", wsmem, K, cudaGetErrorString(e));
            return -2;
          }
        }
        cudaError_t le = launch_pdl(1, kern, dim3(grid), dim3(ww * 32), wsmem, stream, (const __nv_bfloat16*)act, lda,
                                    (const __nv_bfloat16*)W, (const __nv_bfloat16*)W2, (TOut*)out, ldo, M, N, K, pitch, blocks,
                                    g_next[0].p, g_next[0].bytes, g_next[1].p, g_next[1].bytes);
        if (le != cudaSuccess) {
          set_error("gemv_mma: launch failed: %s", cudaGetErrorString(le));
          return -2;
        }
        return 0;
      };
      if constexpr (NW == 1) {
        if (deep) {
          if (ww <= 4) return walk(gemv_mma_walk_kernel<EPI, TOut, NT, 4, 8>);
          if (ww <= 8) return walk(gemv_mma_walk_kernel<EPI, TOut, NT, 8, 8>);
          return walk(gemv_mma_walk_kernel<EPI, TOut, NT, 16, 8>);
        }
      }
      if (ww <= 4) return walk(gemv_mma_walk_kernel<EPI, TOut, NT, 4, 4>);
      if (ww <= 8) return walk(gemv_mma_walk_kernel<EPI, TOut, NT, 8, 4>);
      return walk(gemv_mma_walk_kernel<EPI, TOut, NT, 16, 4>);
    }
  }
  const size_t smem = (size_t)8 * NT * pitch * 2 + (size_t)GM_WARPS * NW * NT * 128 * 4 + 8 * NT * 4;
  auto go = [&](auto kern) -> int {
    if (smem > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) {
        set_error("gemv_mma: %zu bytes of shared memory refused (K = %d): %s", smem, K, cudaGetErrorString(e));
        return -2;
      }
    }
    cudaError_t le = launch_pdl(1, kern, dim3((N + GM_COLS - 1) / GM_COLS), dim3(GM_WARPS * 32), smem, stream,
                                (const __nv_bfloat16*)act, lda, x, norm_w, eps, (const __nv_bfloat16*)W, (const __nv_bfloat16*)W2,
                                (TOut*)out, ldo, residual, M, N, K, pitch, kc, g_next[0].p, g_next[0].bytes, g_next[1].p, g_next[1].bytes);
    if (le != cudaSuccess) {
      set_error("gemv_mma: launch failed: %s", cudaGetErrorString(le));
      return -2;
    }
    return 0;
  };
  if constexpr (NW == 1) {
    if (deep) {
      if (GM_WARPS <= 4) return go(gemv_mma_kernel<EPI, TOut, NT, NORM, 4, 8>);
      if (GM_WARPS <= 8) return go(gemv_mma_kernel<EPI, TOut, NT, NORM, 8, 8>);
      return go(gemv_mma_kernel<EPI, TOut, NT, NORM, 16, 8>);
    }
  }
  if (GM_WARPS <= 4) return go(gemv_mma_kernel<EPI, TOut, NT, NORM, 4, 4>);
  if (GM_WARPS <= 8) return go(gemv_mma_kernel<EPI, TOut, NT, NORM, 8, 4>);
  return go(gemv_mma_kernel<EPI, TOut, NT, NORM, 16, 4>);
}

}  // namespace edgelm

using namespace edgelm;

// 1 if the kernel takes these operands, else 0: bfloat16, M <= 16, K a multiple of 8, 16-byte aligned rows.
extern "C" int edgelm_gemv_mma_takes(const void* act, int lda, const void* w, const void* w2, int M, int K, int normed) {
  bool ok = M >= 1 && M <= 16 && K > 0 && K % 8 == 0 && (uintptr_t)w % 16 == 0 &&
            (w2 == nullptr || (uintptr_t)w2 % 16 == 0) && (uintptr_t)act % 16 == 0;
  if (!normed) ok = ok && lda % 8 == 0;
  return ok ? 1 : 0;
}

extern "C" int edgelm_gemv_mma(const void* act, int lda, const float* norm_w, float eps, const void* w, const void* w2,
                               void* out, int ldo, const float* residual, int M, int N, int K, int out_dtype, int epilogue,
                               cudaStream_t stream) {
  if (M == 0) return 0;
  const bool normed = norm_w != nullptr;
  EL_REFUSE(N > 0 && ldo >= N && (normed || lda >= K), "gemv_mma: bad sizes M=%d N=%d K=%d lda=%d ldo=%d", M, N, K, lda, ldo);
  EL_REFUSE(edgelm_gemv_mma_takes(act, lda, w, w2, M, K, normed ? 1 : 0), "gemv_mma: takes M <= 16, K a multiple of 8, 16-byte aligned rows (M=%d K=%d)", M, K);
  EL_REFUSE(epilogue != GM_SWIGLU || w2 != nullptr, "gemv_mma: SwiGLU needs the second weight");
  EL_REFUSE(epilogue != GM_RESIDUAL || (residual != nullptr && out_dtype == DT_F32), "gemv_mma: residual epilogue needs a float32 residual and output");
  const float* x = normed ? (const float*)act : nullptr;
  int rc = 0;
#define EL_GM(EPI, TOUT)                                                                                                 \
  do {                                                                                                                   \
    if (M <= 8) rc = normed ? launch_gemv_mma<EPI, TOUT, 1, true>(nullptr, 0, x, norm_w, eps, w, w2, out, ldo, residual, M, N, K, stream)  \
                            : launch_gemv_mma<EPI, TOUT, 1, false>(act, lda, nullptr, nullptr, 0.f, w, w2, out, ldo, residual, M, N, K, stream); \
    else rc = normed ? launch_gemv_mma<EPI, TOUT, 2, true>(nullptr, 0, x, norm_w, eps, w, w2, out, ldo, residual, M, N, K, stream)         \
                     : launch_gemv_mma<EPI, TOUT, 2, false>(act, lda, nullptr, nullptr, 0.f, w, w2, out, ldo, residual, M, N, K, stream);  \
  } while (0)
  if (epilogue == GM_STORE && out_dtype == DT_BF16) EL_GM(GM_STORE, __nv_bfloat16);
  else if (epilogue == GM_STORE && out_dtype == DT_F32) EL_GM(GM_STORE, float);
  else if (epilogue == GM_RESIDUAL) EL_GM(GM_RESIDUAL, float);
  else if (epilogue == GM_SWIGLU && out_dtype == DT_BF16) EL_GM(GM_SWIGLU, __nv_bfloat16);
  else EL_REFUSE(false, "gemv_mma: unsupported epilogue %d with output dtype %d", epilogue, out_dtype);
#undef EL_GM
  g_next[0] = g_next[1] = NextWeights{nullptr, 0};
  if (rc) return rc;
  EL_LAUNCH_CHECK("gemv_mma");
  return 0;
}

// 1 (default): wide outputs (at least 296 groups of 16 columns, K from 1,024 to 4,096) go to the walking kernel; 0: never.
extern "C" int edgelm_gemv_mma_walk(int on) {
  g_walk = on ? 1 : 0;
  return 0;
}

// Up to two regions of weights that the step reads after the next few-rows product launched from this thread: that
// launch prefetches them into L2.  Null or 0 bytes: none.  Pointers 16-byte aligned (refused otherwise); the bytes
// are rounded down to whole 16.
extern "C" int edgelm_gemv_mma_prefetch_next(const void* p0, unsigned long long bytes0, const void* p1, unsigned long long bytes1) {
  EL_REFUSE((uintptr_t)p0 % 16 == 0 && (uintptr_t)p1 % 16 == 0, "gemv_mma_prefetch_next: regions must be 16-byte aligned");
  g_next[0] = NextWeights{(const uint8_t*)p0, p0 ? bytes0 : 0};
  g_next[1] = NextWeights{(const uint8_t*)p1, p1 ? bytes1 : 0};
  return 0;
}
