// Row kernels of the decoder: embedding gather, residual add + RMSNorm, SwiGLU (plain and the
// clamped gpt-oss form), and the e4m3 activation quantiser with one scale per token per 128
// values (scales stored transposed, [K/128, ld], so the GEMM epilogue reads them as vectors).
// Norm + quantise and activation + quantise are one launch each: the bf16 intermediate never
// goes to memory.
//
// Counterparts in the reference: cuda/fused_norm_f16.cu (fused_rmsnorm, silu_mul_gu),
// cuda/moe/add_rms_norm.cu, cuda/moe/embed_rows_float.cu, swiglu_oai in src/inference/cuda/fused.cu.
#include "common.cuh"
#include "host_common.h"
#include "loken_cuda.h"

using namespace lk;

namespace {

constexpr int ROW_THREADS = 256;
constexpr int MAX_IT = 8;  // 8 * 256 threads * 8 values = 16384 columns at most

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&v)[8]) {
  uint4 q = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    float2 f = __bfloat1622float2(h[e]);
    v[2 * e] = f.x;
    v[2 * e + 1] = f.y;
  }
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&v)[8]) {
  uint4 q;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&q);
#pragma unroll
  for (int e = 0; e < 4; ++e) h[e] = __floats2bfloat162_rn(v[2 * e], v[2 * e + 1]);
  *reinterpret_cast<uint4*>(p) = q;
}
// Quantise 8 values of a 128-group to e4m3: the 16 threads that share the group agree on amax.
__device__ __forceinline__ void quant8(const float (&v)[8], uint8_t* dst, float* scale_slot, bool writer) {
  float amax = 0.f;
#pragma unroll
  for (int e = 0; e < 8; ++e) amax = fmaxf(amax, fabsf(v[e]));
  // a 128-group is one half-warp; groups are whole, so a half-warp is in or out together
  const unsigned hm = 0xFFFFu << (threadIdx.x & 16);
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(hm, amax, o));
  const float scale = e4m3_group_scale(amax);
  const float inv = 1.f / scale;
  uint2 q;
  uint8_t* b = reinterpret_cast<uint8_t*>(&q);
#pragma unroll
  for (int e = 0; e < 8; ++e) b[e] = f2e4m3(v[e] * inv);
  *reinterpret_cast<uint2*>(dst) = q;
  if (writer) *scale_slot = scale;
}

__global__ void embed_bf16_kernel(const int* __restrict__ tok, const __nv_bfloat16* __restrict__ table,
                                  __nv_bfloat16* __restrict__ out, int H, int vocab, float scale) {
  const int t = blockIdx.x;
  int id = tok[t];
  if (id < 0 || id >= vocab) id = 0;
  const __nv_bfloat16* src = table + (long long)id * H;
  __nv_bfloat16* dst = out + (long long)t * H;
  for (int c = threadIdx.x * 8; c < H; c += blockDim.x * 8) {
    if (c + 8 <= H) {
      float v[8];
      load8(src + c, v);
      if (scale != 1.f) {
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] *= scale;
      }
      store8(dst + c, v);
    } else {
      for (int e = c; e < H; ++e) dst[e] = f2bf(bf2f(src[e]) * scale);
    }
  }
}

// x (+= delta) ; h = rmsnorm(x) * w  ->  bf16 and/or e4m3 + scales
__global__ void __launch_bounds__(ROW_THREADS)
add_rmsnorm_kernel(__nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ delta,
                   const float* __restrict__ delta_f32, const float* __restrict__ w, float eps, int H,
                   __nv_bfloat16* __restrict__ out_bf16, uint8_t* __restrict__ out_fp8,
                   float* __restrict__ scales_t, long long scale_ld, int write_x) {
  pdl_launch();      // nothing is written before the wait: the kernel after this one may set up behind it
  pdl_wait();
  __shared__ float red[32];
  const int row = blockIdx.x;
  __nv_bfloat16* xr = x + (long long)row * H;
  float v[MAX_IT][8];
  float ss = 0.f;
  const int nchunk = H >> 3;
#pragma unroll
  for (int it = 0; it < MAX_IT; ++it) {
    const int c = it * ROW_THREADS + threadIdx.x;
    if (c < nchunk) {
      load8(xr + c * 8, v[it]);
      if (delta) {
        float d[8];
        load8(delta + (long long)row * H + c * 8, d);
#pragma unroll
        for (int e = 0; e < 8; ++e) v[it][e] += d[e];
      }
      if (delta_f32) {
        const float4* d4 = reinterpret_cast<const float4*>(delta_f32 + (long long)row * H + c * 8);
        float4 a = d4[0], b = d4[1];
        v[it][0] += a.x; v[it][1] += a.y; v[it][2] += a.z; v[it][3] += a.w;
        v[it][4] += b.x; v[it][5] += b.y; v[it][6] += b.z; v[it][7] += b.w;
      }
      if (delta || delta_f32) {
        // the residual stream is bf16: round once, then normalise what was stored
#pragma unroll
        for (int e = 0; e < 8; ++e) v[it][e] = bf2f(f2bf(v[it][e]));
        if (write_x) store8(xr + c * 8, v[it]);
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) ss += v[it][e] * v[it][e];
    }
  }
  ss = block_sum(ss, red);
  const float rinv = rsqrtf(ss / (float)H + eps);
#pragma unroll
  for (int it = 0; it < MAX_IT; ++it) {
    const int c = it * ROW_THREADS + threadIdx.x;
    if (c < nchunk) {
      const float4* w4 = reinterpret_cast<const float4*>(w + c * 8);
      float4 a = w4[0], b = w4[1];
      float o[8] = {v[it][0] * rinv * a.x, v[it][1] * rinv * a.y, v[it][2] * rinv * a.z, v[it][3] * rinv * a.w,
                    v[it][4] * rinv * b.x, v[it][5] * rinv * b.y, v[it][6] * rinv * b.z, v[it][7] * rinv * b.w};
      if (out_bf16) store8(out_bf16 + (long long)row * H + c * 8, o);
      if (out_fp8) {
        // quantise what a bf16 consumer would have seen
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = bf2f(f2bf(o[e]));
        quant8(o, out_fp8 + (long long)row * H + c * 8, scales_t + (long long)(c >> 4) * scale_ld + row,
               (threadIdx.x & 15) == 0);
      }
    }
  }
}

// gate_up [T, 2*I] (gate in the first I columns, up in the last I) -> act [T, I]
// mode 0: silu(g) * u ; mode 1: gpt-oss clamped form, g' = min(g, limit), u' = clamp(u, -limit, limit),
// out = g' * sigmoid(alpha * g') * (1 + u')
__global__ void __launch_bounds__(ROW_THREADS)
glu_kernel(const __nv_bfloat16* __restrict__ gu, long long ld_in, int I, int mode, float alpha, float limit,
           __nv_bfloat16* __restrict__ out_bf16, uint8_t* __restrict__ out_fp8, float* __restrict__ scales_t,
           long long scale_ld) {
  pdl_launch();      // nothing is written before the wait: the kernel after this one may set up behind it
  pdl_wait();
  const int row = blockIdx.y;
  const int c = blockIdx.x * ROW_THREADS + threadIdx.x;  // chunk of 8
  const int nchunk = I >> 3;
  const bool live = c < nchunk;
  float o[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  if (live) {
    float g[8], u[8];
    load8(gu + (long long)row * ld_in + c * 8, g);
    load8(gu + (long long)row * ld_in + I + c * 8, u);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      if (mode == 0) {
        o[e] = silu(g[e]) * u[e];
      } else {
        const float gg = fminf(g[e], limit);
        const float uu = fminf(fmaxf(u[e], -limit), limit);
        o[e] = gg / (1.f + __expf(-alpha * gg)) * (1.f + uu);
      }
    }
    if (out_bf16) store8(out_bf16 + (long long)row * I + c * 8, o);
  }
  if (out_fp8) {
#pragma unroll
    for (int e = 0; e < 8; ++e) o[e] = bf2f(f2bf(o[e]));
    float amax = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) amax = fmaxf(amax, fabsf(o[e]));
#pragma unroll
    for (int s = 8; s > 0; s >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, s));
    if (live) {
      const float scale = e4m3_group_scale(amax);
      const float inv = 1.f / scale;
      uint2 q;
      uint8_t* b = reinterpret_cast<uint8_t*>(&q);
#pragma unroll
      for (int e = 0; e < 8; ++e) b[e] = f2e4m3(o[e] * inv);
      *reinterpret_cast<uint2*>(out_fp8 + (long long)row * I + c * 8) = q;
      if ((threadIdx.x & 15) == 0) scales_t[(long long)(c >> 4) * scale_ld + row] = scale;
    }
  }
}

__global__ void __launch_bounds__(ROW_THREADS)
quant_fp8_kernel(const __nv_bfloat16* __restrict__ x, long long ld_in, int K, uint8_t* __restrict__ out,
                 float* __restrict__ scales_t, long long scale_ld) {
  pdl_launch();      // nothing is written before the wait: the kernel after this one may set up behind it
  pdl_wait();
  const int row = blockIdx.y;
  const int c = blockIdx.x * ROW_THREADS + threadIdx.x;
  const bool live = c < (K >> 3);
  float v[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  if (live) load8(x + (long long)row * ld_in + c * 8, v);
  float amax = 0.f;
#pragma unroll
  for (int e = 0; e < 8; ++e) amax = fmaxf(amax, fabsf(v[e]));
#pragma unroll
  for (int s = 8; s > 0; s >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, s));
  if (live) {
    const float scale = e4m3_group_scale(amax);
    const float inv = 1.f / scale;
    uint2 q;
    uint8_t* b = reinterpret_cast<uint8_t*>(&q);
#pragma unroll
    for (int e = 0; e < 8; ++e) b[e] = f2e4m3(v[e] * inv);
    *reinterpret_cast<uint2*>(out + (long long)row * K + c * 8) = q;
    if ((threadIdx.x & 15) == 0) scales_t[(long long)(c >> 4) * scale_ld + row] = scale;
  }
}

// out[t, :] = a[t, :] + b[t, :]  (bf16), used where a residual add stands alone
__global__ void add_bf16_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b,
                                __nv_bfloat16* __restrict__ out, long long n8) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n8) {
    float x[8], y[8];
    load8(a + i * 8, x);
    load8(b + i * 8, y);
#pragma unroll
    for (int e = 0; e < 8; ++e) x[e] += y[e];
    store8(out + i * 8, x);
  }
}

}  // namespace

LK_API int lk_embed_bf16(const int* tokens, const void* table, void* out, int T, int H, int vocab, float scale,
                         void* stream) {
  if (T <= 0) return LKH_OK;
  if (H % 8) return LKH_BAD_ARG;
  embed_bf16_kernel<<<T, 128, 0, (cudaStream_t)stream>>>(tokens, (const __nv_bfloat16*)table,
                                                         (__nv_bfloat16*)out, H, vocab, scale);
  lkh::count_launch();
  return lkh::launch_status();
}

LK_API int lk_add_rmsnorm(void* x, const void* delta, const float* delta_f32, const float* w, float eps, int T,
                          int H, void* out_bf16, void* out_fp8, float* scales_t, long long scale_ld, int write_x,
                          void* stream) {
  if (T <= 0) return LKH_OK;
  if (H % 8 || H > ROW_THREADS * 8 * MAX_IT) return LKH_BAD_ARG;
  if (out_fp8 && (H % 128 || !scales_t)) return LKH_BAD_ARG;
  lkh::launch_pdl(add_rmsnorm_kernel, dim3(T), dim3(ROW_THREADS), 0, (cudaStream_t)stream, (__nv_bfloat16*)x,
                  (const __nv_bfloat16*)delta, delta_f32, w, eps, H, (__nv_bfloat16*)out_bf16, (uint8_t*)out_fp8,
                  scales_t, scale_ld, write_x);
  lkh::count_launch();
  return lkh::launch_status();
}

LK_API int lk_glu(const void* gate_up, long long ld_in, int T, int I, int mode, float alpha, float limit,
                  void* out_bf16, void* out_fp8, float* scales_t, long long scale_ld, void* stream) {
  if (T <= 0) return LKH_OK;
  if (I % 8 || (out_fp8 && (I % 128 || !scales_t))) return LKH_BAD_ARG;
  dim3 grid(((I >> 3) + ROW_THREADS - 1) / ROW_THREADS, T);
  lkh::launch_pdl(glu_kernel, grid, dim3(ROW_THREADS), 0, (cudaStream_t)stream, (const __nv_bfloat16*)gate_up, ld_in, I,
                  mode, alpha, limit, (__nv_bfloat16*)out_bf16, (uint8_t*)out_fp8, scales_t, scale_ld);
  lkh::count_launch();
  return lkh::launch_status();
}

LK_API int lk_quant_fp8(const void* x, long long ld_in, int T, int K, void* out, float* scales_t, long long scale_ld,
                        void* stream) {
  if (T <= 0) return LKH_OK;
  if (K % 128) return LKH_BAD_ARG;
  dim3 grid(((K >> 3) + ROW_THREADS - 1) / ROW_THREADS, T);
  lkh::launch_pdl(quant_fp8_kernel, grid, dim3(ROW_THREADS), 0, (cudaStream_t)stream, (const __nv_bfloat16*)x, ld_in, K,
                  (uint8_t*)out, scales_t, scale_ld);
  lkh::count_launch();
  return lkh::launch_status();
}

LK_API int lk_add_bf16(const void* a, const void* b, void* out, long long n, void* stream) {
  if (n <= 0) return LKH_OK;
  if (n % 8) return LKH_BAD_ARG;
  const long long n8 = n / 8;
  add_bf16_kernel<<<(unsigned)((n8 + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)a, (const __nv_bfloat16*)b, (__nv_bfloat16*)out, n8);
  lkh::count_launch();
  return lkh::launch_status();
}
