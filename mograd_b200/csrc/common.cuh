// Shared host/device helpers for the mograd_b200 kernel library (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>

#include "../../include/mograd_b200.h"

#define MGB_EXPORT extern "C" __attribute__((visibility("default")))

namespace mgb {

// ---------------------------------------------------------------- host side
// Records a message for mograd_b200_last_error() and returns `code`.
int fail(int code, const char* fmt, ...);

// cudaGetLastError() after a launch; no synchronisation.
int check_launch(const char* what);

int sm_count();             // multiprocessors of the current device (cached per device)
int max_smem_optin();       // opt-in shared memory per block of the current device

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline size_t round_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

#define MGB_REQUIRE(cond, code, ...) \
  do {                               \
    if (!(cond)) return ::mgb::fail((code), __VA_ARGS__); \
  } while (0)

// Launch with programmatic stream serialization: the grid may be scheduled while the kernel before it on the
// stream is still draining, so its set-up (barriers, TMEM, descriptor prefetch) and the launch latency overlap the
// predecessor's tail.  Only for kernels that call pdl_wait() before their first access to global memory.
template <typename... KArgs, typename... Args>
inline void launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;

  cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);  // errors surface in check_launch()
}

// -------------------------------------------------------------- device side
// Programmatic dependent launch: pdl_wait() returns once every kernel before this one on the stream has
// completed and its writes are visible; nothing before it may touch global memory.  pdl_launch_dependents() lets
// the next kernel's blocks be scheduled as soon as every block of this grid has executed it.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename T>
struct Vec;  // elements per 16-byte vector
template <>
struct Vec<float> {
  static constexpr int N = 4;
};
template <>
struct Vec<__nv_bfloat16> {
  static constexpr int N = 8;
};
template <>
struct Vec<__half> {
  static constexpr int N = 8;
};

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float to_f32(__half v) { return __half2float(v); }
template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ float from_f32<float>(float v) {
  return v;
}
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}
template <>
__device__ __forceinline__ __half from_f32<__half>(float v) {
  return __float2half_rn(v);
}

// 16-byte global load / store of Vec<T>::N elements, widened to float.
__device__ __forceinline__ void load_vec(const float* p, float (&out)[4]) {
  const float4 v = *reinterpret_cast<const float4*>(p);
  out[0] = v.x;
  out[1] = v.y;
  out[2] = v.z;
  out[3] = v.w;
}
__device__ __forceinline__ void load_vec(const __nv_bfloat16* p, float (&out)[8]) {
  const uint4 v = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    out[2 * i] = __uint_as_float(w[i] << 16);
    out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
__device__ __forceinline__ void load_vec(const __half* p, float (&out)[8]) {
  const uint4 v = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
    out[2 * i] = f.x;
    out[2 * i + 1] = f.y;
  }
}
__device__ __forceinline__ void store_vec(float* p, const float (&in)[4]) {
  *reinterpret_cast<float4*>(p) = make_float4(in[0], in[1], in[2], in[3]);
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&h);
}
__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi) {
  const __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&h);
}
// Two floats -> one 32-bit word of two 16-bit elements of type T (element 0 in the low half).
template <typename T>
__device__ __forceinline__ uint32_t pack_pair(float lo, float hi);
template <>
__device__ __forceinline__ uint32_t pack_pair<__nv_bfloat16>(float lo, float hi) {
  return pack_bf16x2(lo, hi);
}
template <>
__device__ __forceinline__ uint32_t pack_pair<__half>(float lo, float hi) {
  return pack_f16x2(lo, hi);
}
__device__ __forceinline__ void store_vec(__half* p, const float (&in)[8]) {
  uint4 v;
  v.x = pack_f16x2(in[0], in[1]);
  v.y = pack_f16x2(in[2], in[3]);
  v.z = pack_f16x2(in[4], in[5]);
  v.w = pack_f16x2(in[6], in[7]);
  *reinterpret_cast<uint4*>(p) = v;
}
__device__ __forceinline__ void store_vec(__nv_bfloat16* p, const float (&in)[8]) {
  uint4 v;
  v.x = pack_bf16x2(in[0], in[1]);
  v.y = pack_bf16x2(in[2], in[3]);
  v.z = pack_bf16x2(in[4], in[5]);
  v.w = pack_bf16x2(in[6], in[7]);
  *reinterpret_cast<uint4*>(p) = v;
}

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

}  // namespace mgb
