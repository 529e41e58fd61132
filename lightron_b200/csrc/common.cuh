// Shared helpers for the sm_100a kernels of lightron_b200.
// Every entry point is extern "C", returns 0 or a negative code, and launches on the
// caller's stream.  Nothing here allocates device memory.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

#define LB_OK 0
#define LB_ERR_ARG (-1)
#define LB_ERR_LAUNCH (-2)
#define LB_ERR_SHAPE (-3)
#define LB_ERR_DRIVER (-4)
#define LB_ERR_TMAP (-5)
#define LB_ERR_CAPACITY (-6)

extern int g_lb_last_cuda_error;
// Wall-time limit of every device-side wait on a flag that another GPU or CTA writes
// (lb_set_flag_wait_ns; kernels take it as a launch parameter).
extern unsigned long long g_lb_flag_wait_ns;
// Number of SMs of the current device (queried once per device).
int lb_num_sms();

#define LB_CHECK_LAUNCH()                                   \
  do {                                                      \
    cudaError_t e__ = cudaGetLastError();                   \
    if (e__ != cudaSuccess) {                               \
      g_lb_last_cuda_error = (int)e__;                      \
      return LB_ERR_LAUNCH;                                 \
    }                                                       \
  } while (0)

typedef __nv_bfloat16 bf16;
typedef __nv_bfloat162 bf162;

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

// 8 bf16 <-> 8 floats through one 16-byte vector
struct __align__(16) bf16x8 {
  bf162 v[4];
};
__device__ __forceinline__ void unpack8(const uint4& u, float* f) {
  const bf162* p = reinterpret_cast<const bf162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; i++) {
    float2 t = __bfloat1622float2(p[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float* f) {
  uint4 u;
  bf162* p = reinterpret_cast<bf162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; i++) p[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return u;
}
