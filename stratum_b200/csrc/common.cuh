// Shared helpers for the sm_100a kernels: element types, status codes, reductions.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

// Launchers return 0 on success, a positive cudaError_t from the launch, or one of these.
#define STRATUM_ERR_DTYPE (-1)   // dtype code is neither 0 (float32) nor 1 (bfloat16)
#define STRATUM_ERR_SHAPE (-2)   // a size the kernel does not take
#define STRATUM_ERR_ALIGN (-3)   // a pointer or stride is not aligned as the kernel needs
#define STRATUM_ERR_LIMIT (-4)   // beyond a stated maximum

#define STRATUM_DT_F32 0
#define STRATUM_DT_BF16 1

#define STRATUM_EXPORT extern "C" __attribute__((visibility("default")))

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(bf16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_float<bf16>(float v) { return __float2bfloat16_rn(v); }

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

// Sum over a block of up to 1024 threads; every thread gets the result.  The order of
// additions depends only on the block size, never on what else runs.
__device__ __forceinline__ float block_sum(float v, float* scratch /* >= 33 floats */) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int n_warps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = (lane < n_warps) ? scratch[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

// ---------------------------------------------------------------- programmatic dependent launch
// A kernel launched with launch_pdl may begin while the kernel before it in the stream is still
// finishing.  Whatever it does before pdl_wait() must not touch memory an earlier kernel writes (it
// may read weights and the step's description, compute addresses, warm up); pdl_wait() returns once
// every earlier kernel has completed and its writes are visible.  pdl_trigger() lets the kernel
// after this one start its own preamble.  Launched the ordinary way, both are no-ops.
//
// Loads of anything an earlier kernel of the same step produced must not use the read-only path
// (ld.global.nc / __ldg, which the compiler also picks by itself for `const T* __restrict__`): with an early
// start that data changes during this kernel's lifetime, and a stale line may be served.  Such loads go
// through ld_fresh (ld.global.cg: served from L2, where the producer's writes are).
__device__ __forceinline__ float ld_fresh(const float* p) { return __ldcg(p); }
__device__ __forceinline__ float4 ld_fresh(const float4* p) { return __ldcg(p); }
__device__ __forceinline__ uint4 ld_fresh(const uint4* p) { return __ldcg(p); }
__device__ __forceinline__ float ld_fresh(const bf16* p) {
  return __bfloat162float(__ushort_as_bfloat16(__ldcg(reinterpret_cast<const unsigned short*>(p))));
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

#include <stdlib.h>
static inline bool pdl_enabled() {
  static int on = -1;
  if (on < 0) {
    const char* e = getenv("STRATUM_PDL");
    on = (e && e[0] == '0') ? 0 : 1;
  }
  return on == 1;
}

template <typename... KArgs, typename... Args>
static inline int launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                             Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return (int)cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

static inline int launch_status() {
  cudaError_t e = cudaGetLastError();
  return (int)e;
}
