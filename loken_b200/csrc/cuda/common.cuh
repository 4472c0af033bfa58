// Small device helpers shared by the SIMT kernels.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace lk {

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

// Block-wide sum through shared memory (blockDim.x a multiple of 32, <= 1024).
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  float t = (lane < nw) ? red[lane] : 0.f;
  t = warp_sum(t);
  return t;
}
__device__ __forceinline__ float block_max(float v, float* red) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  float t = (lane < nw) ? red[lane] : -INFINITY;
  t = warp_max(t);
  return t;
}

__device__ __forceinline__ float bf2f(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ __nv_bfloat16 f2bf(float v) { return __float2bfloat16(v); }

// e4m3 with saturation to +-448 (the finite range), round to nearest even
__device__ __forceinline__ uint8_t f2e4m3(float v) {
  return static_cast<uint8_t>(__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3));
}
__device__ __forceinline__ float e4m32f(uint8_t v) {
  __half_raw h = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>(v), __NV_E4M3);
  return __half2float(*reinterpret_cast<__half*>(&h));
}

// Scale of an e4m3 activation group: the smallest power of two s with amax / s <= 448.  Powers of two
// make the scaling exact and let the block-scaled MMA take the scale as an E8M0 exponent
// (gemm_mx.cu); the per-K-block fold of gemm_tc.cuh accepts any f32 and so these too.
__device__ __forceinline__ float e4m3_group_scale(float amax) {
  if (!(amax > 0.f)) return 1.f;
  const uint32_t bits = __float_as_uint(__fdiv_rn(amax, 448.f));     // IEEE division: the same bits as the host reference
  int ex = (int)((bits >> 23) & 0xFF) + ((bits & 0x7FFFFF) ? 1 : 0);
  ex = ex < 1 ? 1 : ex > 254 ? 254 : ex;
  return __uint_as_float((uint32_t)ex << 23);
}

__device__ __forceinline__ float silu(float x) { return x / (1.f + __expf(-x)); }

// Programmatic dependent launch (see lkh::launch_pdl): `pdl_wait` returns when the preceding kernel
// of the stream has completed and its writes are visible (at once when this kernel was launched
// the ordinary way); `pdl_launch` lets the following kernel be scheduled from now on.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

}  // namespace lk
