// Next-token choice on the device: first-maximum argmax, and temperature + top-k sampling
// with one xorshift64 stream per sequence.
//
// The sampling rule is: keep the k largest logits (equal logits: lower index first),
// p_i = exp((l_i - l_max) / temperature) in float32, draw u in [0,1) from the sequence's
// xorshift64 state, walk the kept tokens in descending order and return the first whose
// cumulative p reaches u * sum(p).  The row is copied into shared memory once (a vocabulary of up
// to 49,152); a radix select over the logits' bit patterns finds the k-th largest logit; up to
// 1,024 kept tokens are then listed, ranked in the order of the walk and summed with a block-wide
// scan, more (top_k 0: the whole vocabulary) go through a radix descent over their cumulative p.
// The sums are kept in 2^-40 fixed point (integer adds), so the choice does not depend on the
// order in which threads add.
#include <math_constants.h>

#include "common.cuh"

namespace edgelm {

constexpr int SAMPLE_THREADS = 512;

// float -> unsigned key with the same order (larger float, larger key)
__device__ __forceinline__ uint32_t order_key(float x) {
  const uint32_t u = __float_as_uint(x);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
argmax_rows_kernel(const float* __restrict__ logits, int ld, int vocab, int32_t* __restrict__ out) {
  __shared__ float bv[SAMPLE_THREADS / 32];
  __shared__ int bi[SAMPLE_THREADS / 32];
  const float* row = logits + (size_t)blockIdx.x * ld;
  float best = -CUDART_INF_F;
  int idx = 0x7fffffff;
  auto take = [&](float v, int i) {  // strict >: the first maximum among this thread's ascending indices
    if (v > best || (idx == 0x7fffffff && !(v != v))) {
      best = v;
      idx = i;
    }
  };
  if (((uintptr_t)row & 15) == 0) {
    // 16-byte loads, four in flight per thread: the row is read at memory speed, not at one latency per element
    const int n4 = vocab >> 2;
    const float4* row4 = reinterpret_cast<const float4*>(row);
    int i = threadIdx.x;
    for (; i + 3 * (int)blockDim.x < n4; i += 4 * blockDim.x) {
      float4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) v[u] = row4[i + u * blockDim.x];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int b = (i + u * blockDim.x) * 4;
        take(v[u].x, b);
        take(v[u].y, b + 1);
        take(v[u].z, b + 2);
        take(v[u].w, b + 3);
      }
    }
    for (; i < n4; i += blockDim.x) {
      const float4 v = row4[i];
      take(v.x, i * 4);
      take(v.y, i * 4 + 1);
      take(v.z, i * 4 + 2);
      take(v.w, i * 4 + 3);
    }
    for (int j = (n4 << 2) + threadIdx.x; j < vocab; j += blockDim.x) take(row[j], j);
  } else {
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) take(row[i], i);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
    if (ov > best || (ov == best && oi < idx)) {
      best = ov;
      idx = oi;
    }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) {
    bv[warp] = best;
    bi[warp] = idx;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < SAMPLE_THREADS / 32; ++w)
      if (bv[w] > best || (bv[w] == best && bi[w] < idx)) {
        best = bv[w];
        idx = bi[w];
      }
    out[blockIdx.x] = idx == 0x7fffffff ? 0 : idx;
  }
}

// ------------------------------------------------------------------------- temperature + top-k
constexpr int ST = 1024;            // threads of the sampling kernel: one block a row
constexpr int SK_LIST = 1024;       // up to this many kept tokens are put in a list and ranked; more: a weighted radix descent
constexpr int ST_ROW_BYTES = 192 * 1024;   // a row of at most this many bytes is copied into shared memory first

struct SampleShared {
  unsigned int hist[256];
  unsigned long long whist[256];
  unsigned int warp_cnt[ST / 32];
  unsigned int prefix, remaining, found_idx, n_kept;
  unsigned long long target;
  float red[ST / 32];
  // the kept tokens (top-k <= SK_LIST): key, index, 2^-40 fixed-point p; after ranking, in the order of the walk
  uint32_t kkey[SK_LIST];
  int kidx[SK_LIST];
  unsigned long long kp[SK_LIST];
};

// Adds `amount` to hist[bucket] for the lanes with `take`: lanes of a warp that share a bucket add once (logits crowd
// into a few buckets of the high bytes, and one atomic per lane would serialise).
__device__ __forceinline__ void hist_add(unsigned int* hist, bool take, uint32_t bucket) {
  const unsigned int peers = __match_any_sync(0xffffffffu, take ? bucket : 0xffffffffu);
  if (take && (threadIdx.x & 31) == __ffs(peers) - 1) atomicAdd(&hist[bucket], (unsigned int)__popc(peers));
}

// The same for 64-bit amounts (at most 2^40 each): the lanes of a warp that share a bucket add their amounts up first
// (two 32-bit warp reductions of the low and the high 20 bits) and one of them adds the sum.  Integer adds: the
// histogram does not depend on the grouping.  Whole warps call it.
__device__ __forceinline__ void whist_add(unsigned long long* whist, bool take, uint32_t bucket, unsigned long long amount) {
  const int lane = threadIdx.x & 31;
  unsigned int todo = __ballot_sync(0xffffffffu, take);
  while (todo) {
    const int leader = __ffs(todo) - 1;
    const uint32_t b = __shfl_sync(0xffffffffu, bucket, leader);
    const bool mine = take && bucket == b;
    const unsigned int lo = __reduce_add_sync(0xffffffffu, mine ? (unsigned int)(amount & 0xfffffull) : 0u);
    const unsigned int hi = __reduce_add_sync(0xffffffffu, mine ? (unsigned int)(amount >> 20) : 0u);
    if (lane == leader) atomicAdd(&whist[b], (unsigned long long)lo + ((unsigned long long)hi << 20));
    todo &= ~__ballot_sync(0xffffffffu, mine);
  }
}

// Index of the n-th (0-based) element, in index order, whose key equals `key`; vocab if fewer.  A thread counts the
// matches of its own run of consecutive elements (an odd run length keeps the reads off each other's banks), the
// counts are scanned over the block, and the thread whose run holds the n-th match walks it again.
__device__ int nth_equal_index(const float* src, int vocab, uint32_t key, unsigned int n, SampleShared& sh) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int run = ((vocab + ST - 1) / ST) | 1;
  const int lo = min(vocab, (int)threadIdx.x * run), hi = min(vocab, lo + run);
  unsigned int mine = 0;
  for (int i = lo; i < hi; ++i) mine += order_key(src[i]) == key;
  unsigned int incl = mine;   // inclusive scan over the warp, then over the warps
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const unsigned int v = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += v;
  }
  if (threadIdx.x == 0) sh.found_idx = (unsigned int)vocab;
  if (lane == 31) sh.warp_cnt[warp] = incl;
  __syncthreads();
  unsigned int before = incl - mine;
  for (int w = 0; w < warp; ++w) before += sh.warp_cnt[w];
  if (n >= before && n < before + mine) {
    unsigned int seen = before;
    for (int i = lo; i < hi; ++i)
      if (order_key(src[i]) == key && seen++ == n) sh.found_idx = (unsigned int)i;
  }
  __syncthreads();
  const int found = (int)sh.found_idx;
  __syncthreads();
  return found;
}

__device__ __forceinline__ unsigned long long fixed_p(float logit, float lmax, float temperature) {
  const float p = expf((logit - lmax) / temperature);
  return (unsigned long long)((double)p * 1099511627776.0);  // 2^40
}

// One xorshift64 step of the row's stream and the draw's target in [1, total].
__device__ __forceinline__ unsigned long long draw_target(unsigned long long* rng_state, const int32_t* state_index, unsigned long long total) {
  const int si = state_index ? state_index[blockIdx.x] : (int)blockIdx.x;
  unsigned long long s = rng_state[si];
  s ^= s << 13;
  s ^= s >> 7;
  s ^= s << 17;
  rng_state[si] = s;
  const double u = (double)(s >> 11) * (1.0 / 9007199254740992.0);
  unsigned long long t = (unsigned long long)ceil(u * (double)total);
  if (t < 1) t = 1;
  if (t > total) t = total;
  return t;
}

__global__ void __launch_bounds__(ST)
sample_topk_kernel(const float* __restrict__ logits, int ld, int vocab, float temperature, int top_k,
                   unsigned long long* __restrict__ rng_state, const int32_t* __restrict__ state_index,
                   int32_t* __restrict__ out, int row_in_shared, const int32_t* __restrict__ only_flagged) {
  if (only_flagged != nullptr && only_flagged[blockIdx.x] == 0) return;   // (the small kernel chose for this row)
  __shared__ SampleShared sh;
  extern __shared__ __align__(16) float row_s[];
  const float* row = logits + (size_t)blockIdx.x * ld;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const unsigned int k = (top_k > 0 && top_k < vocab) ? (unsigned int)top_k : (unsigned int)vocab;

  // ---- the row into shared memory (every later pass reads it from there), and its maximum
  const float* src = row;
  float lmax = -CUDART_INF_F;
  if (row_in_shared) {
    if (((uintptr_t)row & 15) == 0) {
      const int n4 = vocab >> 2;
      for (int i = threadIdx.x; i < n4; i += ST) {
        const float4 v = reinterpret_cast<const float4*>(row)[i];
        reinterpret_cast<float4*>(row_s)[i] = v;
        lmax = fmaxf(fmaxf(lmax, fmaxf(v.x, v.y)), fmaxf(v.z, v.w));
      }
      for (int i = (n4 << 2) + threadIdx.x; i < vocab; i += ST) {
        row_s[i] = row[i];
        lmax = fmaxf(lmax, row[i]);
      }
    } else {
      for (int i = threadIdx.x; i < vocab; i += ST) {
        row_s[i] = row[i];
        lmax = fmaxf(lmax, row[i]);
      }
    }
    src = row_s;
  } else {
    for (int i = threadIdx.x; i < vocab; i += ST) lmax = fmaxf(lmax, row[i]);
  }
  lmax = warp_max(lmax);
  if (lane == 0) sh.red[warp] = lmax;
  __syncthreads();
  lmax = sh.red[0];
  for (int w = 1; w < ST / 32; ++w) lmax = fmaxf(lmax, sh.red[w]);

  // ---- the k-th largest key: radix select, most significant byte first
  uint32_t prefix = 0;            // the decided high bits of the k-th largest key
  unsigned int remaining = k;     // its rank (1-based, descending) among keys that share those bits
  const bool keep_all = k >= (unsigned int)vocab;   // (top_k 0: nothing to select; every key is at or above 0)
  for (int shift = 24; shift >= 0 && !keep_all; shift -= 8) {
    for (int i = threadIdx.x; i < 256; i += ST) sh.hist[i] = 0;
    __syncthreads();
    const uint32_t mask = shift == 24 ? 0u : (0xffffffffu << (shift + 8));
    for (int base = 0; base < vocab; base += ST) {   // (whole warps, for the warp-wide vote inside hist_add)
      const int i = base + threadIdx.x;
      const uint32_t key = i < vocab ? order_key(src[i]) : 0u;
      hist_add(sh.hist, i < vocab && (key & mask) == prefix, (key >> shift) & 255u);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      unsigned int cum = 0;
      int d = 255;
      for (; d > 0; --d) {
        const unsigned int c = sh.hist[d];
        if (cum + c >= remaining) break;
        cum += c;
      }
      sh.prefix = prefix | ((uint32_t)d << shift);
      sh.remaining = remaining - cum;
    }
    __syncthreads();
    prefix = sh.prefix;
    remaining = sh.remaining;
    __syncthreads();
  }
  const uint32_t kth = prefix;            // key of the k-th largest logit
  // of the tokens whose key equals kth, the first `remaining` by index are kept
  const int tie_end = keep_all ? vocab : nth_equal_index(src, vocab, kth, remaining - 1, sh) + 1;  // keep equal keys with index < tie_end

  if (k <= (unsigned int)SK_LIST) {
    // ---- few kept tokens: list them, rank them in the order of the walk (key descending, index ascending), add up
    if (threadIdx.x == 0) sh.n_kept = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < vocab; i += ST) {
      const float v = src[i];
      const uint32_t key = order_key(v);
      if (key > kth || (key == kth && i < tie_end)) {
        const unsigned int slot = atomicAdd(&sh.n_kept, 1u);
        if (slot < (unsigned int)SK_LIST) {
          sh.kkey[slot] = key;
          sh.kidx[slot] = i;
          sh.kp[slot] = fixed_p(v, lmax, temperature);
        }
      }
    }
    __syncthreads();
    const int n = min((int)sh.n_kept, SK_LIST);
    uint32_t my_key = 0;
    int my_idx = 0, rank = 0;
    unsigned long long my_p = 0;
    if ((int)threadIdx.x < n) {
      my_key = sh.kkey[threadIdx.x];
      my_idx = sh.kidx[threadIdx.x];
      my_p = sh.kp[threadIdx.x];
      for (int j = 0; j < n; ++j) {
        const uint32_t kj = sh.kkey[j];
        rank += kj > my_key || (kj == my_key && sh.kidx[j] < my_idx);
      }
    }
    __syncthreads();
    if ((int)threadIdx.x < n) {
      sh.kidx[rank] = my_idx;
      sh.kp[rank] = my_p;
    }
    __syncthreads();
    // inclusive sums in the order of the walk (thread t: position t)
    unsigned long long incl = (int)threadIdx.x < n ? sh.kp[threadIdx.x] : 0ull;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const unsigned long long v = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += v;
    }
    if (lane == 31) sh.whist[warp] = incl;
    __syncthreads();
    unsigned long long before = 0;
    for (int w = 0; w < warp; ++w) before += sh.whist[w];
    incl += before;
    if (threadIdx.x == 0) {
      unsigned long long total = 0;
      for (int w = 0; w < ST / 32; ++w) total += sh.whist[w];
      sh.target = draw_target(rng_state, state_index, total);
    }
    __syncthreads();
    const unsigned long long target = sh.target;
    const unsigned long long mine = (int)threadIdx.x < n ? sh.kp[threadIdx.x] : 0ull;
    if ((int)threadIdx.x < n && incl >= target && incl - mine < target) out[blockIdx.x] = sh.kidx[threadIdx.x];
    return;
  }

  // ---- many kept tokens: radix descent over their cumulative p
  uint32_t dprefix = 0;
  unsigned long long target = 0;
  for (int level = 0; level < 4; ++level) {
    const int shift = 24 - 8 * level;
    for (int i = threadIdx.x; i < 256; i += ST) sh.whist[i] = 0;
    __syncthreads();
    const uint32_t mask = shift == 24 ? 0u : (0xffffffffu << (shift + 8));
    for (int base = 0; base < vocab; base += ST) {   // (whole warps, for the votes inside whist_add)
      const int i = base + threadIdx.x;
      const float v = i < vocab ? src[i] : 0.f;
      const uint32_t key = order_key(v);
      const bool kept = i < vocab && (key > kth || (key == kth && i < tie_end));
      const bool take = kept && (key & mask) == dprefix;
      whist_add(sh.whist, take, (key >> shift) & 255u, take ? fixed_p(v, lmax, temperature) : 0ull);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      if (level == 0) {
        unsigned long long total = 0;
        for (int d = 0; d < 256; ++d) total += sh.whist[d];
        sh.target = draw_target(rng_state, state_index, total);
      }
      unsigned long long t = sh.target, cum = 0;
      int d = 255;
      for (; d > 0; --d) {
        if (cum + sh.whist[d] >= t) break;
        cum += sh.whist[d];
      }
      sh.target = t - cum;
      sh.prefix = dprefix | ((uint32_t)d << shift);
    }
    __syncthreads();
    dprefix = sh.prefix;
    target = sh.target;
    __syncthreads();
  }
  // dprefix is the key of the chosen logit; equal keys carry equal p: pick by index
  const uint32_t u = (dprefix & 0x80000000u) ? (dprefix & 0x7fffffffu) : ~dprefix;
  const unsigned long long q = fixed_p(__uint_as_float(u), lmax, temperature);
  unsigned int n = q > 0 ? (unsigned int)((target + q - 1) / q) - 1u : 0u;
  int idx = nth_equal_index(src, vocab, dprefix, n, sh);
  if (idx >= vocab || (dprefix == kth && idx >= tie_end)) {
    // rounding put the target past the last kept token of this value: take the last kept one
    int last = -1;
    if (threadIdx.x == 0) {
      for (int i = 0; i < vocab; ++i)
        if (order_key(src[i]) == dprefix && (dprefix != kth || i < tie_end)) {
          last = i;
        }
      sh.found_idx = (unsigned int)(last < 0 ? 0 : last);
    }
    __syncthreads();
    idx = (int)sh.found_idx;
  }
  if (threadIdx.x == 0) out[blockIdx.x] = idx;
}

// ------------------------------------------------------------------------- few kept tokens, the row in registers
// top_k <= SK_LIST and a vocabulary of at most ST * EPT: a thread keeps EPT keys of the row in registers (element
// t + j * ST), the high 16 bits of the k-th largest key are found bit by bit from the top (a block-wide count per
// bit: no histogram, no atomics), the tokens at or above that bound are listed and ranked in the order of the walk,
// and the first k of them are the kept ones.  Returns through `fallback` (1) without choosing if more than SK_LIST
// tokens lie at or above the bound; the caller then runs the general kernel (the stream has not been advanced).
__device__ __forceinline__ unsigned int block_sum_u32(unsigned int v, unsigned int* scratch /* [ST / 32] */) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = __reduce_add_sync(0xffffffffu, v);
  __syncthreads();   // the scratch of the call before this one has been read
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  unsigned int t = scratch[lane];   // ST / 32 == 32 partial sums: one per lane
  return __reduce_add_sync(0xffffffffu, t);
}

template <int EPT>
__global__ void __launch_bounds__(ST)
sample_topk_small_kernel(const float* __restrict__ logits, int ld, int vocab, float temperature, int top_k,
                         unsigned long long* __restrict__ rng_state, const int32_t* __restrict__ state_index,
                         int32_t* __restrict__ out, int32_t* __restrict__ fallback) {
  static_assert(ST == 1024, "a warp reads the 32 warps' partial sums");
  __shared__ SampleShared sh;
  const float* row = logits + (size_t)blockIdx.x * ld;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const unsigned int k = (top_k > 0 && top_k < vocab) ? (unsigned int)top_k : (unsigned int)vocab;
  uint32_t keys[EPT];   // 0 for the slots past the vocabulary: below every real key
  float lmax = -CUDART_INF_F;
#pragma unroll
  for (int j = 0; j < EPT; ++j) {
    const int i = (int)threadIdx.x + j * ST;
    const float v = i < vocab ? row[i] : 0.f;
    keys[j] = i < vocab ? order_key(v) : 0u;
    if (i < vocab) lmax = fmaxf(lmax, v);
  }
  lmax = warp_max(lmax);
  if (lane == 0) sh.red[warp] = lmax;
  __syncthreads();
  lmax = sh.red[lane];
  lmax = warp_max(lmax);
  // ---- the high half of the k-th largest key, a bit at a time (sign, exponent, seven bits of mantissa): the tokens
  // at or above that bound are the k largest and the few that share the bound's high half with the k-th
  uint32_t kth = 0;
  unsigned int remaining = k;   // rank of the wanted key among the keys that share the decided bits
  for (int bit = 31; bit >= 16; --bit) {
    const uint32_t cand = kth | (1u << bit), mask = ~((1u << bit) - 1u);
    unsigned int c = 0;
#pragma unroll
    for (int j = 0; j < EPT; ++j) c += (keys[j] & mask) == cand;
    const unsigned int total = block_sum_u32(c, sh.warp_cnt);
    if (total >= remaining) kth = cand;
    else remaining -= total;
  }
  // ---- the tokens at or above it, listed
  if (threadIdx.x == 0) sh.n_kept = 0;
  __syncthreads();
#pragma unroll
  for (int j = 0; j < EPT; ++j) {
    if (keys[j] >= kth && keys[j] != 0u) {
      const unsigned int slot = atomicAdd(&sh.n_kept, 1u);
      if (slot < (unsigned int)SK_LIST) {
        sh.kkey[slot] = keys[j];
        sh.kidx[slot] = (int)threadIdx.x + j * ST;
      }
    }
  }
  __syncthreads();
  if (sh.n_kept > (unsigned int)SK_LIST) {   // (uniform) too many ties for the list
    if (threadIdx.x == 0) fallback[blockIdx.x] = 1;
    return;
  }
  const int n = (int)sh.n_kept;
  uint32_t my_key = 0;
  int my_idx = 0, rank = 0;
  if ((int)threadIdx.x < n) {
    my_key = sh.kkey[threadIdx.x];
    my_idx = sh.kidx[threadIdx.x];
    for (int j = 0; j < n; ++j) {
      const uint32_t kj = sh.kkey[j];
      rank += kj > my_key || (kj == my_key && sh.kidx[j] < my_idx);
    }
  }
  __syncthreads();
  if ((int)threadIdx.x < n) {   // position in the walk; the first k positions are the kept tokens
    const uint32_t u = (my_key & 0x80000000u) ? (my_key & 0x7fffffffu) : ~my_key;
    sh.kidx[rank] = my_idx;
    sh.kp[rank] = rank < (int)k ? fixed_p(__uint_as_float(u), lmax, temperature) : 0ull;
  }
  __syncthreads();
  const int kept = min(n, (int)k);
  unsigned long long incl = (int)threadIdx.x < kept ? sh.kp[threadIdx.x] : 0ull;
  const unsigned long long mine = incl;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const unsigned long long v = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += v;
  }
  if (lane == 31) sh.whist[warp] = incl;
  __syncthreads();
  for (int w = 0; w < warp; ++w) incl += sh.whist[w];
  if (threadIdx.x == 0) {
    unsigned long long total = 0;
    for (int w = 0; w < ST / 32; ++w) total += sh.whist[w];
    sh.target = draw_target(rng_state, state_index, total);
  }
  __syncthreads();
  const unsigned long long target = sh.target;
  if ((int)threadIdx.x < kept && incl >= target && incl - mine < target) out[blockIdx.x] = sh.kidx[threadIdx.x];
}

}  // namespace edgelm

using namespace edgelm;

extern "C" int edgelm_argmax_rows(const float* logits, int ld, int rows, int vocab, int32_t* out, cudaStream_t stream) {
  if (rows == 0) return 0;
  EL_REFUSE(rows > 0 && vocab > 0 && ld >= vocab, "argmax_rows: bad sizes rows=%d vocab=%d ld=%d", rows, vocab, ld);
  argmax_rows_kernel<<<rows, SAMPLE_THREADS, 0, stream>>>(logits, ld, vocab, out);
  EL_LAUNCH_CHECK("argmax_rows");
  return 0;
}

// rng_state: 64-bit xorshift states, advanced by one draw; row r uses state state_index[r]
// (the sequence's slot), or state r when state_index is null.
extern "C" int edgelm_sample_topk(const float* logits, int ld, int rows, int vocab, float temperature, int top_k,
                                  unsigned long long* rng_state, const int32_t* state_index, int32_t* out,
                                  int32_t* fallback /* [rows] scratch, or null */, cudaStream_t stream) {
  if (rows == 0) return 0;
  EL_REFUSE(rows > 0 && vocab > 0 && ld >= vocab, "sample_topk: bad sizes rows=%d vocab=%d ld=%d", rows, vocab, ld);
  EL_REFUSE(temperature > 0.f, "sample_topk: temperature %g is not positive (greedy goes through argmax_rows)", temperature);
  EL_REFUSE(vocab <= (1 << 24), "sample_topk: vocabulary %d too large for the fixed-point sums", vocab);
  const size_t row_bytes = (size_t)vocab * sizeof(float);
  const int in_shared = row_bytes <= (size_t)ST_ROW_BYTES;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(sample_topk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, ST_ROW_BYTES);
    EL_REFUSE(e == cudaSuccess, "sample_topk: %d bytes of shared memory refused: %s", ST_ROW_BYTES, cudaGetErrorString(e));
    configured = true;
  }
  // few kept tokens and a row that fits the block's registers: the small kernel; rows it could not do (more than
  // 1,024 tokens tied at or above the k-th logit) are flagged and done by the general kernel behind it
  const int k = (top_k > 0 && top_k < vocab) ? top_k : vocab;
  const bool small = fallback != nullptr && k <= SK_LIST && vocab <= ST * 48;
  if (small) {
    cudaMemsetAsync(fallback, 0, sizeof(int32_t) * rows, stream);
    if (vocab <= ST * 16)
      sample_topk_small_kernel<16><<<rows, ST, 0, stream>>>(logits, ld, vocab, temperature, top_k, rng_state, state_index, out, fallback);
    else if (vocab <= ST * 32)
      sample_topk_small_kernel<32><<<rows, ST, 0, stream>>>(logits, ld, vocab, temperature, top_k, rng_state, state_index, out, fallback);
    else
      sample_topk_small_kernel<48><<<rows, ST, 0, stream>>>(logits, ld, vocab, temperature, top_k, rng_state, state_index, out, fallback);
  }
  sample_topk_kernel<<<rows, ST, in_shared ? row_bytes : 0, stream>>>(logits, ld, vocab, temperature, top_k, rng_state, state_index, out,
                                                                    in_shared, small ? fallback : nullptr);
  EL_LAUNCH_CHECK("sample_topk");
  return 0;
}
