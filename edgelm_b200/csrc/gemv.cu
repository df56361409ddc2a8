// Few-rows matrix products for decoding: out[M, N] = act[M, K] . W[N, K]^T with M <= 8 per pass.
//
// Decoding is bound by reading each weight once and by the latency of many small kernels, so
// this kernel is built around both:
//   * the activations of all M rows are staged once per block in shared memory, in the compute
//     dtype; every warp then streams its own weight rows with 16-byte loads and keeps M
//     accumulators per column, so a weight is read once for the whole batch;
//   * optionally the activations are produced here: act = RMSNorm(x) from the float32 residual
//     stream (statistics in float32, the result rounded to the compute dtype exactly as the
//     stand-alone norm kernel rounds it), which removes a kernel and a round trip per use;
//   * each warp's first weight loads are issued before the prologue, so that memory latency and
//     the prologue overlap;
//   * epilogues as everywhere: store, += residual (float32), SwiGLU of two weights.
// A column's sum is taken in an order that depends on K alone (lane-strided partial sums, then
// a fixed shuffle tree), so a row's result does not depend on the rest of the batch.
// Takes K a multiple of the 16-byte vector (8 bfloat16, 4 float) with aligned rows; other
// sizes go to the scalar kernel in gemm_simt.cu.
#include "common.cuh"

namespace edgelm {

enum : int { GV_STORE = 0, GV_RESIDUAL = 1, GV_SWIGLU = 2 };
constexpr int GV_ROWS = 8;

template <typename T> struct Vec16;
template <> struct Vec16<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void unpack(const uint4& v, float* o) {
    o[0] = __uint_as_float(v.x); o[1] = __uint_as_float(v.y); o[2] = __uint_as_float(v.z); o[3] = __uint_as_float(v.w);
  }
};
template <> struct Vec16<__nv_bfloat16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void unpack(const uint4& v, float* o) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      o[2 * i] = __uint_as_float(w[i] << 16);
      o[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
};

__device__ __forceinline__ float gv_silu(float z) { return z / (1.0f + expf(-z)); }

// CW: columns a warp works on at once.  NORM: activations = RMSNorm(x) computed in the prologue.
template <typename T, int EPI, typename TOut, int CW, bool NORM>
__global__ void __launch_bounds__(256)
gemv_kernel(const T* __restrict__ act, int lda, const float* __restrict__ x, const float* __restrict__ norm_w, float eps,
            const T* __restrict__ W, const T* __restrict__ W2, TOut* out, int ldo, const float* residual, int M, int N,
            int K, int kc) {
  constexpr int V = Vec16<T>::N;
  constexpr int NW = EPI == GV_SWIGLU ? 2 : 1;
  extern __shared__ __align__(16) uint8_t gv_smem[];
  T* As = reinterpret_cast<T*>(gv_smem);                       // [GV_ROWS][kc]
  float* inv = reinterpret_cast<float*>(gv_smem + (size_t)GV_ROWS * kc * sizeof(T));  // [GV_ROWS]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int m0 = blockIdx.y * GV_ROWS;
  const int rows = min(GV_ROWS, M - m0);
  const int col0 = (blockIdx.x * nwarps + warp) * CW;          // this warp's first column

  // UNR steps of K at a time: their weight vectors are requested together and used in order (a lane's sum runs over
  // its k in increasing order whatever UNR is), so a warp waits for memory once per UNR steps instead of once per
  // step.  The first UNR steps of this warp's columns are requested here, ahead of the wait for the kernel before
  // this one and of the prologue (weights: nothing on the stream writes them).
  constexpr int UNR = NW * CW <= 2 ? 4 : 2;
  const int kn0 = min(kc, K);   // the first chunk of K
  uint4 wpre[UNR][NW][CW];
#pragma unroll
  for (int u = 0; u < UNR; ++u) {
    const int k = lane * V + u * 32 * V;
#pragma unroll
    for (int c = 0; c < CW; ++c) {
      const int n = min(col0 + c, N - 1);
      if (k < kn0) {
        wpre[u][0][c] = *reinterpret_cast<const uint4*>(W + (size_t)n * K + k);
        if (NW == 2) wpre[u][1][c] = *reinterpret_cast<const uint4*>(W2 + (size_t)n * K + k);
      } else {
        wpre[u][0][c] = make_uint4(0, 0, 0, 0);
        if (NW == 2) wpre[u][1][c] = make_uint4(0, 0, 0, 0);
      }
    }
  }

  pdl_launch_dependents();
  pdl_wait();   // (launched as a programmatic dependent: from here on, what the kernel before this one wrote)
  // the residual values that the epilogue adds to, one a lane (column c, row r in lane c * 8 + r), requested now: a
  // trip to memory less at the end of the warp's life (out may be the residual itself: nobody else writes these)
  float res_mine = 0.f;
  if (EPI == GV_RESIDUAL) {
    const int c = lane / GV_ROWS, r = lane - c * GV_ROWS;
    if (c < CW && r < rows && col0 + c < N) res_mine = residual[(size_t)(m0 + r) * ldo + col0 + c];
  }
  // A normalised row of up to 1,024 values in one chunk: a warp takes a row, keeps it in registers between the sum of
  // squares and the scaling and writes it out in the compute dtype: one pass over x, the norm's weights beside it.
  const bool one_pass = NORM && K <= 1024 && K <= kc && K % 4 == 0;
  if (NORM && one_pass) {
    float4 g[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int k = lane * 4 + j * 128;
      g[j] = k < K ? *reinterpret_cast<const float4*>(norm_w + k) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    for (int r = warp; r < rows; r += nwarps) {
      float4 v[8];
      float ss = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int k = lane * 4 + j * 128;
        v[j] = k < K ? *reinterpret_cast<const float4*>(x + (size_t)(m0 + r) * K + k) : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        ss = fmaf(v[j].x, v[j].x, ss); ss = fmaf(v[j].y, v[j].y, ss); ss = fmaf(v[j].z, v[j].z, ss); ss = fmaf(v[j].w, v[j].w, ss);
      }
      ss = warp_sum(ss);
      const float sc = 1.0f / sqrtf(ss / (float)K + eps);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int k = lane * 4 + j * 128;
        if (k < K) {
          T* dst = As + r * kc + k;
          dst[0] = from_f32<T>(v[j].x * sc * g[j].x);
          dst[1] = from_f32<T>(v[j].y * sc * g[j].y);
          dst[2] = from_f32<T>(v[j].z * sc * g[j].z);
          dst[3] = from_f32<T>(v[j].w * sc * g[j].w);
        }
      }
    }
  } else if (NORM) {  // 1 / sqrt(mean(x^2) + eps) per row, a warp per row
    for (int r = warp; r < rows; r += nwarps) {
      const float* xr = x + (size_t)(m0 + r) * K;
      float ss = 0.f;
      for (int k = lane * 4; k < K; k += 128) {
        const float4 v = *reinterpret_cast<const float4*>(xr + k);
        ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
      }
      ss = warp_sum(ss);
      if (lane == 0) inv[r] = 1.0f / sqrtf(ss / (float)K + eps);
    }
    __syncthreads();
  }

  float acc[NW][CW][GV_ROWS];
#pragma unroll
  for (int w = 0; w < NW; ++w)
#pragma unroll
    for (int c = 0; c < CW; ++c)
#pragma unroll
      for (int r = 0; r < GV_ROWS; ++r) acc[w][c][r] = 0.f;

  for (int k0 = 0; k0 < K; k0 += kc) {          // K in chunks that fit shared memory (one chunk for the usual sizes)
    const int kn = min(kc, K - k0);
    if (k0) __syncthreads();
    for (int i = threadIdx.x * V; i < (one_pass ? 0 : rows * kn); i += blockDim.x * V) {
      const int r = i / kn, k = i - r * kn;     // kn is a multiple of V: a vector never crosses rows
      if (NORM) {
        const float s = inv[r];
        const float* xr = x + (size_t)(m0 + r) * K + k0 + k;
        const float* wr = norm_w + k0 + k;
#pragma unroll
        for (int v = 0; v < V; ++v) As[r * kc + k + v] = from_f32<T>(xr[v] * s * wr[v]);
      } else {
        *reinterpret_cast<uint4*>(As + r * kc + k) = *reinterpret_cast<const uint4*>(act + (size_t)(m0 + r) * lda + k0 + k);
      }
    }
    __syncthreads();
    if (col0 < N) {
      for (int kb = lane * V; kb < kn; kb += 32 * V * UNR) {
        uint4 wv[UNR][NW][CW];
#pragma unroll
        for (int u = 0; u < UNR; ++u) {
          const int k = kb + u * 32 * V;
#pragma unroll
          for (int c = 0; c < CW; ++c) {
            if (k0 == 0 && kb == lane * V) {
              wv[u][0][c] = wpre[u][0][c];
              if (NW == 2) wv[u][1][c] = wpre[u][1][c];
            } else if (k < kn) {
              const int n = min(col0 + c, N - 1);
              wv[u][0][c] = *reinterpret_cast<const uint4*>(W + (size_t)n * K + k0 + k);
              if (NW == 2) wv[u][1][c] = *reinterpret_cast<const uint4*>(W2 + (size_t)n * K + k0 + k);
            } else {
              wv[u][0][c] = make_uint4(0, 0, 0, 0);
              if (NW == 2) wv[u][1][c] = make_uint4(0, 0, 0, 0);
            }
          }
        }
#pragma unroll
        for (int u = 0; u < UNR; ++u) {
          const int k = kb + u * 32 * V;
          if (k < kn) {
            float wf[NW][CW][V];
#pragma unroll
            for (int w = 0; w < NW; ++w)
#pragma unroll
              for (int c = 0; c < CW; ++c) Vec16<T>::unpack(wv[u][w][c], wf[w][c]);
#pragma unroll
            for (int r = 0; r < GV_ROWS; ++r) {
              if (r < rows) {
                float af[V];
                Vec16<T>::unpack(*reinterpret_cast<const uint4*>(As + r * kc + k), af);
#pragma unroll
                for (int w = 0; w < NW; ++w)
#pragma unroll
                  for (int c = 0; c < CW; ++c)
#pragma unroll
                    for (int v = 0; v < V; ++v) acc[w][c][r] = fmaf(af[v], wf[w][c][v], acc[w][c][r]);
              }
            }
          }
        }
      }
    }
  }
  if (col0 >= N) return;
#pragma unroll
  for (int c = 0; c < CW; ++c) {
    const int n = col0 + c;
#pragma unroll
    for (int r = 0; r < GV_ROWS; ++r) {
      if (r < rows) {  // uniform over the warp
        const float s = warp_sum(acc[0][c][r]);
        const float s2 = NW == 2 ? warp_sum(acc[NW - 1][c][r]) : 0.f;
        const float res = EPI == GV_RESIDUAL ? __shfl_sync(0xffffffffu, res_mine, c * GV_ROWS + r) : 0.f;
        if (lane == 0 && n < N) {
          const size_t idx = (size_t)(m0 + r) * ldo + n;
          if (EPI == GV_STORE) out[idx] = from_f32<TOut>(s);
          if (EPI == GV_RESIDUAL) out[idx] = from_f32<TOut>(res + s);
          if (EPI == GV_SWIGLU) out[idx] = from_f32<TOut>(gv_silu(s) * s2);
        }
      }
    }
  }
}

template <typename T, int EPI, typename TOut, int CW, bool NORM>
static int launch_gemv_cw(const void* act, int lda, const float* x, const float* norm_w, float eps, const void* W,
                          const void* W2, void* out, int ldo, const float* residual, int M, int N, int K, int threads,
                          cudaStream_t stream) {
  constexpr int V = Vec16<T>::N;
  // shared memory: all rows of one K chunk; chunks of at most 32 KB
  int kc = K;
  const int max_kc = (32 * 1024 / (GV_ROWS * (int)sizeof(T))) / V * V;
  if (kc > max_kc) kc = max_kc;
  const size_t smem = (size_t)GV_ROWS * kc * sizeof(T) + GV_ROWS * sizeof(float);
  const int nwarps = threads / 32;
  dim3 grid((N + nwarps * CW - 1) / (nwarps * CW), (M + GV_ROWS - 1) / GV_ROWS);
  // a programmatic dependent launch, like the tensor-core few-rows kernel: the first weight loads run ahead of the wait
  const cudaError_t le = launch_pdl(1, gemv_kernel<T, EPI, TOut, CW, NORM>, grid, dim3(threads), smem, stream, (const T*)act, lda, x, norm_w,
                                    eps, (const T*)W, (const T*)W2, (TOut*)out, ldo, residual, M, N, K, kc);
  if (le != cudaSuccess) {
    set_error("gemv: launch failed: %s", cudaGetErrorString(le));
    return -2;
  }
  return 0;
}

template <typename T, int EPI, typename TOut, bool NORM>
static int launch_gemv(const void* act, int lda, const float* x, const float* norm_w, float eps, const void* W,
                       const void* W2, void* out, int ldo, const float* residual, int M, int N, int K, int n_sms,
                       cudaStream_t stream) {
  // enough blocks to fill the device: few columns per warp and small blocks for narrow outputs
  const long long cols = N;
  if (cols <= 4LL * 2 * n_sms)
    return launch_gemv_cw<T, EPI, TOut, 1, NORM>(act, lda, x, norm_w, eps, W, W2, out, ldo, residual, M, N, K, 128, stream);
  if (cols <= 8LL * 4 * n_sms)
    return launch_gemv_cw<T, EPI, TOut, 1, NORM>(act, lda, x, norm_w, eps, W, W2, out, ldo, residual, M, N, K, 256, stream);
  if (EPI == GV_SWIGLU || cols <= 16LL * 8 * n_sms)
    return launch_gemv_cw<T, EPI, TOut, 2, NORM>(act, lda, x, norm_w, eps, W, W2, out, ldo, residual, M, N, K, 256, stream);
  return launch_gemv_cw<T, EPI, TOut, 4, NORM>(act, lda, x, norm_w, eps, W, W2, out, ldo, residual, M, N, K, 256, stream);
}

}  // namespace edgelm

using namespace edgelm;

// 1 if the vector kernel takes these operands, else 0 (the scalar kernel of gemm_simt.cu takes the rest).
extern "C" int edgelm_gemv_takes(const void* act, int lda, const void* w, const void* w2, int K, int dtype, int normed) {
  const int v = dtype == DT_BF16 ? 8 : 4;
  bool ok = K > 0 && K % v == 0 && (uintptr_t)w % 16 == 0 && (w2 == nullptr || (uintptr_t)w2 % 16 == 0);
  if (normed) ok = ok && K % 4 == 0 && (uintptr_t)act % 16 == 0;   // act is x (float32) here
  else ok = ok && lda % v == 0 && (uintptr_t)act % 16 == 0;
  return ok ? 1 : 0;
}

// act: [M, K] in `dtype` with pitch lda; or, with norm_w given, x: float32 [M, K] contiguous, and the
// activations are RMSNorm(x) * norm_w rounded to `dtype`.  out_dtype as in gemm_simt.
extern "C" int edgelm_gemv(const void* act, int lda, const float* norm_w, float eps, const void* w, const void* w2,
                           void* out, int ldo, const float* residual, int M, int N, int K, int dtype, int out_dtype,
                           int epilogue, int n_sms, cudaStream_t stream) {
  if (M == 0) return 0;
  const bool normed = norm_w != nullptr;
  EL_REFUSE(M > 0 && N > 0 && K > 0 && ldo >= N && (normed || lda >= K), "gemv: bad sizes M=%d N=%d K=%d lda=%d ldo=%d", M, N, K, lda, ldo);
  EL_REFUSE(edgelm_gemv_takes(act, lda, w, w2, K, dtype, normed ? 1 : 0), "gemv: K=%d and the row pitch must be multiples of a 16-byte vector, rows 16-byte aligned", K);
  EL_REFUSE(epilogue != GV_SWIGLU || w2 != nullptr, "gemv: SwiGLU needs the second weight");
  EL_REFUSE(epilogue != GV_RESIDUAL || (residual != nullptr && out_dtype == DT_F32), "gemv: residual epilogue needs a float32 residual and output");
  EL_REFUSE((M + GV_ROWS - 1) / GV_ROWS <= 65535, "gemv: too many rows (%d)", M);
  if (n_sms <= 0) n_sms = 148;
  const float* x = normed ? (const float*)act : nullptr;
#define EL_GV(T, EPI, TOUT)                                                                                             \
  (normed ? launch_gemv<T, EPI, TOUT, true>(nullptr, 0, x, norm_w, eps, w, w2, out, ldo, residual, M, N, K, n_sms, stream) \
          : launch_gemv<T, EPI, TOUT, false>(act, lda, nullptr, nullptr, 0.f, w, w2, out, ldo, residual, M, N, K, n_sms, stream))
  int rc = 0;
  if (dtype == DT_BF16) {
    if (epilogue == GV_STORE && out_dtype == DT_BF16) rc = EL_GV(__nv_bfloat16, GV_STORE, __nv_bfloat16);
    else if (epilogue == GV_STORE && out_dtype == DT_F32) rc = EL_GV(__nv_bfloat16, GV_STORE, float);
    else if (epilogue == GV_RESIDUAL) rc = EL_GV(__nv_bfloat16, GV_RESIDUAL, float);
    else if (epilogue == GV_SWIGLU && out_dtype == DT_BF16) rc = EL_GV(__nv_bfloat16, GV_SWIGLU, __nv_bfloat16);
    else EL_REFUSE(false, "gemv: unsupported epilogue %d with output dtype %d", epilogue, out_dtype);
  } else if (dtype == DT_F32) {
    EL_REFUSE(out_dtype == DT_F32, "gemv: float32 activations give float32 outputs");
    if (epilogue == GV_STORE) rc = EL_GV(float, GV_STORE, float);
    else if (epilogue == GV_RESIDUAL) rc = EL_GV(float, GV_RESIDUAL, float);
    else if (epilogue == GV_SWIGLU) rc = EL_GV(float, GV_SWIGLU, float);
    else EL_REFUSE(false, "gemv: unknown epilogue %d", epilogue);
  } else {
    EL_REFUSE(false, "gemv: unknown dtype code %d", dtype);
  }
#undef EL_GV
  if (rc) return rc;
  EL_LAUNCH_CHECK("gemv");
  return 0;
}
