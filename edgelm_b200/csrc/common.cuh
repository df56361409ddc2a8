// Shared device helpers and the C ABI conventions of the kernel library.
//
// Every exported function is `extern "C"`, takes raw device pointers, sizes and a
// cudaStream_t, allocates nothing, launches on the given stream and returns 0 or a negative
// code after storing a message that `edgelm_last_error()` hands out.  Sizes that a kernel
// does not take are refused here, before any launch, never computed wrongly.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdio>

namespace edgelm {

void set_error(const char* fmt, ...);

#define EL_REFUSE(cond, ...)              \
  do {                                    \
    if (!(cond)) {                        \
      ::edgelm::set_error(__VA_ARGS__);   \
      return -1;                          \
    }                                     \
  } while (0)

#define EL_LAUNCH_CHECK(what)                                                        \
  do {                                                                               \
    cudaError_t e__ = cudaGetLastError();                                            \
    if (e__ != cudaSuccess) {                                                        \
      ::edgelm::set_error("%s: launch failed: %s", what, cudaGetErrorString(e__));   \
      return -2;                                                                     \
    }                                                                                \
  } while (0)

// Dtype codes of the C ABI.
enum : int { DT_F32 = 0, DT_BF16 = 1 };

// Bits of the device error word (one int32 that kernels OR into and the host reads).
enum : int { ERR_TOKEN_RANGE = 1, ERR_POSITION_RANGE = 2, ERR_PAGE_RANGE = 4, ERR_WAIT_TIMEOUT = 8 };

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a block in a fixed order (thread partials -> warp shuffles -> first warp), so that
// a row's result does not depend on anything but the row.  `red` holds 33 floats.
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarp ? red[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  return red[32];
}

// Programmatic dependent launch: a kernel launched with `launch_pdl` may start while the kernel before
// it on the stream is still running.  It must call `pdl_wait()` before it reads anything an earlier
// kernel wrote or writes anything an earlier kernel reads; before that point it may only touch what
// no kernel of the stream writes (weights, tables).  `pdl_launch_dependents()` lets the next kernel
// start early in turn.  In a kernel launched the ordinary way both are no-ops.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Bit mask of the kernel families launched as programmatic dependent launches (1: few-rows matrix
// products, 2: decode attention, 4: unused, 8: one-tile tcgen05 matrix products, 16: tcgen05 prefill attention, 32: RMSNorm,
// the vectorised rotation and cache append, the persistent tcgen05 matrix products); 0: ordinary launches everywhere.
int pdl_enabled();

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(int bit, void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = (pdl_enabled() & bit) ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

// The cache keeps keys and values in pages of PAGE tokens: [page][kv_head][PAGE][head_dim].
constexpr int PAGE = 64;

}  // namespace edgelm
