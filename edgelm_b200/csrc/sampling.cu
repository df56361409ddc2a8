// Next-token choice on the device: first-maximum argmax, and temperature + top-k sampling
// with one xorshift64 stream per sequence.
//
// The sampling rule is: keep the k largest logits (equal logits: lower index first),
// p_i = exp((l_i - l_max) / temperature) in float32, draw u in [0,1) from the sequence's
// xorshift64 state, walk the kept tokens in descending order and return the first whose
// cumulative p reaches u * sum(p).  Nothing is sorted: a radix descent over the logits' bit
// patterns finds first the k-th largest logit and then the token at which the cumulative sum
// crosses the target.  The sums are kept in 2^-40 fixed point (integer adds), so the choice
// does not depend on the order in which threads add.
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

struct SampleShared {
  unsigned long long hist[256];
  unsigned int warp_cnt[SAMPLE_THREADS / 32];
  unsigned int prefix, remaining, found_idx, running;
  unsigned long long target;
  float red[SAMPLE_THREADS / 32];
};

// Index of the n-th (0-based) element, in index order, whose key equals `key`; vocab if fewer.
__device__ int nth_equal_index(const float* row, int vocab, uint32_t key, unsigned int n, SampleShared& sh) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) {
    sh.running = 0;
    sh.found_idx = (unsigned int)vocab;
  }
  __syncthreads();
  for (int base = 0; base < vocab; base += blockDim.x) {
    const int i = base + threadIdx.x;
    const bool f = i < vocab && order_key(row[i]) == key;
    const unsigned int bal = __ballot_sync(0xffffffffu, f);
    if (lane == 0) sh.warp_cnt[warp] = __popc(bal);
    __syncthreads();
    unsigned int before = sh.running;
    for (int w = 0; w < warp; ++w) before += sh.warp_cnt[w];
    before += __popc(bal & ((1u << lane) - 1u));
    if (f && before == n) sh.found_idx = (unsigned int)i;
    __syncthreads();
    if (threadIdx.x == 0) {
      unsigned int t = 0;
      for (int w = 0; w < SAMPLE_THREADS / 32; ++w) t += sh.warp_cnt[w];
      sh.running += t;
    }
    __syncthreads();
    if (sh.found_idx != (unsigned int)vocab) break;  // uniform: read after the barrier
  }
  __syncthreads();
  return (int)sh.found_idx;
}

__device__ __forceinline__ unsigned long long fixed_p(float logit, float lmax, float temperature) {
  const float p = expf((logit - lmax) / temperature);
  return (unsigned long long)((double)p * 1099511627776.0);  // 2^40
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_topk_kernel(const float* __restrict__ logits, int ld, int vocab, float temperature, int top_k,
                   unsigned long long* __restrict__ rng_state, const int32_t* __restrict__ state_index,
                   int32_t* __restrict__ out) {
  __shared__ SampleShared sh;
  const float* row = logits + (size_t)blockIdx.x * ld;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const unsigned int k = (top_k > 0 && top_k < vocab) ? (unsigned int)top_k : (unsigned int)vocab;

  // ---- the k-th largest key: radix select, most significant byte first
  uint32_t prefix = 0;            // the decided high bits of the k-th largest key
  unsigned int remaining = k;     // its rank (1-based, descending) among keys that share those bits
  for (int shift = 24; shift >= 0; shift -= 8) {
    for (int i = threadIdx.x; i < 256; i += blockDim.x) sh.hist[i] = 0;
    __syncthreads();
    const uint32_t mask = shift == 24 ? 0u : (0xffffffffu << (shift + 8));
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
      const uint32_t key = order_key(row[i]);
      if ((key & mask) == prefix) atomicAdd(&sh.hist[(key >> shift) & 255u], 1ull);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      unsigned int cum = 0;
      int d = 255;
      for (; d > 0; --d) {
        const unsigned int c = (unsigned int)sh.hist[d];
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
  const int tie_end = nth_equal_index(row, vocab, kth, remaining - 1, sh) + 1;  // keep equal keys with index < tie_end

  // ---- maximum logit
  float lmax = -CUDART_INF_F;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) lmax = fmaxf(lmax, row[i]);
  lmax = warp_max(lmax);
  if (lane == 0) sh.red[warp] = lmax;
  __syncthreads();
  lmax = sh.red[0];
  for (int w = 1; w < SAMPLE_THREADS / 32; ++w) lmax = fmaxf(lmax, sh.red[w]);
  __syncthreads();

  // ---- radix descent over the kept tokens' cumulative p
  uint32_t dprefix = 0;
  unsigned long long target = 0;
  for (int level = 0; level < 4; ++level) {
    const int shift = 24 - 8 * level;
    for (int i = threadIdx.x; i < 256; i += blockDim.x) sh.hist[i] = 0;
    __syncthreads();
    const uint32_t mask = shift == 24 ? 0u : (0xffffffffu << (shift + 8));
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
      const float v = row[i];
      const uint32_t key = order_key(v);
      const bool kept = key > kth || (key == kth && i < tie_end);
      if (kept && (key & mask) == dprefix) atomicAdd(&sh.hist[(key >> shift) & 255u], fixed_p(v, lmax, temperature));
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      if (level == 0) {
        unsigned long long total = 0;
        for (int d = 0; d < 256; ++d) total += sh.hist[d];
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
        sh.target = t;
      }
      unsigned long long t = sh.target, cum = 0;
      int d = 255;
      for (; d > 0; --d) {
        if (cum + sh.hist[d] >= t) break;
        cum += sh.hist[d];
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
  int idx = nth_equal_index(row, vocab, dprefix, n, sh);
  if (idx >= vocab || (dprefix == kth && idx >= tie_end)) {
    // rounding put the target past the last kept token of this value: take the last kept one
    int last = -1;
    if (threadIdx.x == 0) {
      for (int i = 0; i < vocab; ++i)
        if (order_key(row[i]) == dprefix && (dprefix != kth || i < tie_end)) {
          last = i;
        }
      sh.found_idx = (unsigned int)(last < 0 ? 0 : last);
    }
    __syncthreads();
    idx = (int)sh.found_idx;
  }
  if (threadIdx.x == 0) out[blockIdx.x] = idx;
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
                                  cudaStream_t stream) {
  if (rows == 0) return 0;
  EL_REFUSE(rows > 0 && vocab > 0 && ld >= vocab, "sample_topk: bad sizes rows=%d vocab=%d ld=%d", rows, vocab, ld);
  EL_REFUSE(temperature > 0.f, "sample_topk: temperature %g is not positive (greedy goes through argmax_rows)", temperature);
  EL_REFUSE(vocab <= (1 << 24), "sample_topk: vocabulary %d too large for the fixed-point sums", vocab);
  sample_topk_kernel<<<rows, SAMPLE_THREADS, 0, stream>>>(logits, ld, vocab, temperature, top_k, rng_state, state_index, out);
  EL_LAUNCH_CHECK("sample_topk");
  return 0;
}
