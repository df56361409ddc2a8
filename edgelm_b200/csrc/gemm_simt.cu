// y = a . W^T with float32 accumulation on the CUDA cores (FFMA): the whole of the true
// 32-bit path, and the any-size fallback of the bfloat16 path.
//
//   a   [M, K]  float or bfloat16, row stride lda
//   W   [N, K]  float or bfloat16, row-major as a checkpoint stores it (out, in)
// Epilogues:
//   EPI_STORE     out[M, N] (float or bfloat16)             = acc
//   EPI_RESIDUAL  out[M, N] (float) = residual[M, N] + acc   (out may be residual itself)
//   EPI_SWIGLU    out[M, N] = silu(acc_gate) * acc_up with a second weight W2 (up) of W's shape
// Two kernels: a 64x64 tile for many rows and a one-warp-per-output-column kernel for a few
// rows (decode), which reads every weight once.  Each output element is summed over k in an
// order that depends on K alone, never on M or on the row's place in the batch.
#include "common.cuh"

namespace edgelm {

enum : int { EPI_STORE = 0, EPI_RESIDUAL = 1, EPI_SWIGLU = 2 };

__device__ __forceinline__ float silu_f32(float z) { return z / (1.0f + expf(-z)); }

template <int EPI, typename TOut>
__device__ __forceinline__ void epilogue_store(TOut* out, const float* residual, size_t idx, float acc, float acc2) {
  if (EPI == EPI_STORE) out[idx] = from_f32<TOut>(acc);
  if (EPI == EPI_RESIDUAL) out[idx] = from_f32<TOut>(residual[idx] + acc);
  if (EPI == EPI_SWIGLU) out[idx] = from_f32<TOut>(silu_f32(acc) * acc2);
}

// ------------------------------------------------------------------ tiled kernel
constexpr int BM = 64, BN = 64, BK = 16, PADT = 4;

template <typename TA, typename TW, int EPI, typename TOut>
__global__ void __launch_bounds__(256)
gemm_tile_kernel(const TA* __restrict__ A, int lda, const TW* __restrict__ W, const TW* __restrict__ W2,
                 TOut* out, int ldo, const float* residual, int M, int N, int K) {
  __shared__ float As[BK][BM + PADT];
  __shared__ float Ws[BK][BN + PADT];
  __shared__ float Ws2[EPI == EPI_SWIGLU ? BK : 1][BN + PADT];
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  float acc[4][4] = {}, acc2[4][4] = {};
  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int e = tid + i * 256, r = e >> 4, k = e & 15;
      const int gk = k0 + k;
      As[k][r] = (m0 + r < M && gk < K) ? to_f32(A[(size_t)(m0 + r) * lda + gk]) : 0.f;
      const bool ok = (n0 + r < N && gk < K);
      Ws[k][r] = ok ? to_f32(W[(size_t)(n0 + r) * K + gk]) : 0.f;
      if (EPI == EPI_SWIGLU) Ws2[k][r] = ok ? to_f32(W2[(size_t)(n0 + r) * K + gk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float a[4], b[4], b2[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[k][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Ws[k][tx * 4 + j];
      if (EPI == EPI_SWIGLU) {
#pragma unroll
        for (int j = 0; j < 4; ++j) b2[j] = Ws2[k][tx * 4 + j];
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
          if (EPI == EPI_SWIGLU) acc2[i][j] = fmaf(a[i], b2[j], acc2[i][j]);
        }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < N) epilogue_store<EPI, TOut>(out, residual, (size_t)m * ldo + n, acc[i][j], acc2[i][j]);
    }
  }
}

// ------------------------------------------------------------------ few-rows kernel
template <typename T, int VEC> struct VecLoad;
template <> struct VecLoad<float, 4> {
  static __device__ __forceinline__ void load(const float* p, float* o) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
  }
};
template <> struct VecLoad<float, 1> {
  static __device__ __forceinline__ void load(const float* p, float* o) { o[0] = *p; }
};
template <> struct VecLoad<__nv_bfloat16, 8> {
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
template <> struct VecLoad<__nv_bfloat16, 1> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* o) { o[0] = __bfloat162float(*p); }
};

constexpr int GEMV_ROWS = 8;  // rows of `a` that one pass over a weight row serves

template <typename TA, typename TW, int EPI, typename TOut, int VA, int VW>
__global__ void __launch_bounds__(256)
gemv_rows_kernel(const TA* __restrict__ A, int lda, const TW* __restrict__ W, const TW* __restrict__ W2,
                 TOut* out, int ldo, const float* residual, int M, int N, int K) {
  static_assert(VA == VW, "one vector width for both operands");
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int n = blockIdx.x * 8 + warp;
  const int m0 = blockIdx.y * GEMV_ROWS;
  if (n >= N) return;
  const int rows = min(GEMV_ROWS, M - m0);
  float acc[GEMV_ROWS] = {}, acc2[GEMV_ROWS] = {};
  const TW* wrow = W + (size_t)n * K;
  const TW* wrow2 = EPI == EPI_SWIGLU ? W2 + (size_t)n * K : nullptr;
  for (int k = lane * VW; k < K; k += 32 * VW) {
    float w[VW], w2[VW];
    VecLoad<TW, VW>::load(wrow + k, w);
    if (EPI == EPI_SWIGLU) VecLoad<TW, VW>::load(wrow2 + k, w2);
#pragma unroll
    for (int r = 0; r < GEMV_ROWS; ++r) {
      if (r < rows) {
        float a[VA];
        VecLoad<TA, VA>::load(A + (size_t)(m0 + r) * lda + k, a);
#pragma unroll
        for (int v = 0; v < VW; ++v) {
          acc[r] = fmaf(a[v], w[v], acc[r]);
          if (EPI == EPI_SWIGLU) acc2[r] = fmaf(a[v], w2[v], acc2[r]);
        }
      }
    }
  }
#pragma unroll
  for (int r = 0; r < GEMV_ROWS; ++r) {
    if (r < rows) {  // uniform over the warp
      const float s = warp_sum(acc[r]);
      const float s2 = EPI == EPI_SWIGLU ? warp_sum(acc2[r]) : 0.f;
      if (lane == 0) epilogue_store<EPI, TOut>(out, residual, (size_t)(m0 + r) * ldo + n, s, s2);
    }
  }
}

template <typename TA, typename TW, int EPI, typename TOut>
int launch_gemm(const void* A, int lda, const void* W, const void* W2, void* out, int ldo, const float* residual,
                int M, int N, int K, int force_kernel, cudaStream_t stream) {
  const TA* a = (const TA*)A;
  const TW* w = (const TW*)W;
  const TW* w2 = (const TW*)W2;
  TOut* o = (TOut*)out;
  const bool few = force_kernel == 1 || (force_kernel == 0 && M <= 2 * GEMV_ROWS);
  if (few) {
    constexpr int VEC = sizeof(TW) == 2 ? 8 : 4;
    const bool same_width = sizeof(TA) == sizeof(TW);
    const bool aligned = same_width && K % VEC == 0 && lda % VEC == 0 && ((uintptr_t)A % 16 == 0) &&
                         ((uintptr_t)W % 16 == 0) && (W2 == nullptr || (uintptr_t)W2 % 16 == 0);
    dim3 grid((N + 7) / 8, (M + GEMV_ROWS - 1) / GEMV_ROWS);
    if (aligned) {
      if constexpr (sizeof(TA) == sizeof(TW))
        gemv_rows_kernel<TA, TW, EPI, TOut, VEC, VEC><<<grid, 256, 0, stream>>>(a, lda, w, w2, o, ldo, residual, M, N, K);
    } else {
      gemv_rows_kernel<TA, TW, EPI, TOut, 1, 1><<<grid, 256, 0, stream>>>(a, lda, w, w2, o, ldo, residual, M, N, K);
    }
  } else {
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    gemm_tile_kernel<TA, TW, EPI, TOut><<<grid, 256, 0, stream>>>(a, lda, w, w2, o, ldo, residual, M, N, K);
  }
  return 0;
}

}  // namespace edgelm

using namespace edgelm;

// a_dtype: dtype of `a` and of both weights; out_dtype: dtype of `out` (EPI_RESIDUAL: float).
// force_kernel: 0 choose by M, 1 the few-rows kernel, 2 the tile kernel (tests call both).
extern "C" int edgelm_gemm_simt(const void* a, int lda, const void* w, const void* w2, void* out, int ldo,
                                const float* residual, int M, int N, int K, int a_dtype, int out_dtype, int epilogue,
                                int force_kernel, cudaStream_t stream) {
  if (M == 0) return 0;
  EL_REFUSE(M > 0 && N > 0 && K > 0 && lda >= K && ldo >= N, "gemm_simt: bad sizes M=%d N=%d K=%d lda=%d ldo=%d", M, N, K, lda, ldo);
  EL_REFUSE(epilogue != EPI_SWIGLU || w2 != nullptr, "gemm_simt: SwiGLU needs the second weight");
  EL_REFUSE(epilogue != EPI_RESIDUAL || (residual != nullptr && out_dtype == DT_F32), "gemm_simt: residual epilogue needs a float32 residual and output");
  EL_REFUSE((M + BM - 1) / BM <= 65535, "gemm_simt: too many rows (%d)", M);
#define EL_GEMM_CASE(TA, TOUT)                                                                                      \
  switch (epilogue) {                                                                                                \
    case EPI_STORE: launch_gemm<TA, TA, EPI_STORE, TOUT>(a, lda, w, w2, out, ldo, residual, M, N, K, force_kernel, stream); break;       \
    case EPI_RESIDUAL: launch_gemm<TA, TA, EPI_RESIDUAL, float>(a, lda, w, w2, out, ldo, residual, M, N, K, force_kernel, stream); break; \
    case EPI_SWIGLU: launch_gemm<TA, TA, EPI_SWIGLU, TOUT>(a, lda, w, w2, out, ldo, residual, M, N, K, force_kernel, stream); break;     \
    default: EL_REFUSE(false, "gemm_simt: unknown epilogue %d", epilogue);                                           \
  }
  if (a_dtype == DT_F32 && out_dtype == DT_F32) {
    EL_GEMM_CASE(float, float)
  } else if (a_dtype == DT_BF16 && out_dtype == DT_BF16) {
    EL_GEMM_CASE(__nv_bfloat16, __nv_bfloat16)
  } else if (a_dtype == DT_BF16 && out_dtype == DT_F32) {
    EL_GEMM_CASE(__nv_bfloat16, float)
  } else {
    EL_REFUSE(false, "gemm_simt: unsupported dtypes a=%d out=%d", a_dtype, out_dtype);
  }
#undef EL_GEMM_CASE
  EL_LAUNCH_CHECK("gemm_simt");
  return 0;
}
