// Shared helpers for the multi-LoRA decode kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/mlora.h"

namespace mlora {

typedef __nv_bfloat16 bf16;

// Records a host-side message that mlora_last_error() returns; gives back `code`.
int fail(int code, const char* fmt, ...);

#define MLORA_REQUIRE(cond, ...)                                   \
  do {                                                             \
    if (!(cond)) return ::mlora::fail(MLORA_EINVAL, __VA_ARGS__);  \
  } while (0)

#define MLORA_CHECK_LAUNCH(name)                                                            \
  do {                                                                                      \
    cudaError_t e_ = cudaGetLastError();                                                    \
    if (e_ != cudaSuccess) return ::mlora::fail(MLORA_ECUDA, "%s: %s", name, cudaGetErrorString(e_)); \
  } while (0)

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

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

// 8 bf16 packed in a 128-bit register quad -> 8 floats.
__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __bfloat1622float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}

__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 v;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return v;
}

// Streaming 128-bit load that does not allocate in L1 (weights are read once).
__device__ __forceinline__ uint4 ld_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

__device__ __forceinline__ uint4 ld_cached(const void* p) {
  return __ldg(reinterpret_cast<const uint4*>(p));
}

}  // namespace mlora

namespace mlora {
void count_launch(int n = 1);
bool pdl_enabled();
bool pdl_enabled_gemm();
bool pdl_enabled_shrink();
bool pdl_enabled_attn();
bool pdl_enabled_norm();

// Programmatic dependent launch.  Every kernel of the decode step is launched with the
// "programmatic stream serialization" attribute and begins with pdl_launch_dependents(), so the next
// kernel in the stream may become resident while this one still runs; a kernel calls pdl_wait() before
// it reads anything an earlier kernel wrote and before it writes global memory at all (work that only
// touches constant inputs -- streaming weights into shared memory -- may run ahead of it).
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

template <typename... KArgs, typename... Args>
cudaError_t launch_pdl_if(bool on, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                          Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = on ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

template <typename... KArgs, typename... Args>
cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
  return launch_pdl_if(pdl_enabled(), kernel, grid, block, smem, st, static_cast<KArgs>(args)...);
}

}
