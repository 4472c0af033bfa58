// Activation quantiser for the block-scaled GEMM (gemm_mx.cu): bf16 rows -> e4m3 values with one
// E8M0 exponent per 32 values (the OCP microscaling layout the tensor core consumes), fused with
// the row movement or activation that precedes an expert GEMM, so no bf16 intermediate is stored:
//
//   mode 0  plain rows:            out[t]           = q(x[t])
//   mode 1  gather (MoE permute):  out[pair_row[p]] = q(x[p / k])        for pairs with pair_row[p] >= 0
//   mode 2  GLU:                   out[t]           = q(glu(x[t, :I], x[t, I:]))   (SwiGLU or the clamped form)
//
// Exponent of a group: the smallest power of two s with amax / s <= 448 (the largest e4m3 value), so
// the scaling itself is exact and the only rounding is the e4m3 conversion.  Eight values per
// thread; the four threads that share a 32-group agree on amax with two shuffles.
//
// The reference quantises activations to q8_1 blocks (int8 + f16 scale per 32) in front of its
// mat-vec kernels (cuda/moe/rms_qmatmul.cu:115-239, src/inference/cuda/mmvq_gguf.cu:805-1000).
#include "common.cuh"
#include "host_common.h"
#include "loken_cuda.h"

using namespace lk;

namespace {

constexpr int QT = 256;

__global__ void __launch_bounds__(QT)
quant_mx8_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, int K, int mode, const int* __restrict__ pair_row,
                 int kdiv, int glu_mode, float alpha, float limit, uint8_t* __restrict__ out, long long ldo,
                 uint8_t* __restrict__ sf, long long sf_ld) {
  pdl_wait();
  pdl_launch();
  const int row_in = blockIdx.y;
  const int c = blockIdx.x * QT + threadIdx.x;      // chunk of 8 values
  const bool live_c = c < (K >> 3);
  int row_out = row_in;
  long long src_row = row_in;
  bool live = live_c;
  if (mode == 1) {
    row_out = pair_row[row_in];
    src_row = row_in / kdiv;
    live = live && row_out >= 0;
  }
  float v[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  if (live) {
    const __nv_bfloat16* xr = x + src_row * ldx;
    uint4 q = *reinterpret_cast<const uint4*>(xr + c * 8);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 f = __bfloat1622float2(h[e]);
      v[2 * e] = f.x;
      v[2 * e + 1] = f.y;
    }
    if (mode == 2) {
      uint4 qu = *reinterpret_cast<const uint4*>(xr + K + c * 8);
      const __nv_bfloat162* hu = reinterpret_cast<const __nv_bfloat162*>(&qu);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 u = __bfloat1622float2(hu[e]);
        const float uu[2] = {u.x, u.y};
#pragma unroll
        for (int z = 0; z < 2; ++z) {
          const float g = v[2 * e + z];
          float o;
          if (glu_mode == 0) {
            o = silu(g) * uu[z];
          } else {
            const float gg = fminf(g, limit);
            const float uc = fminf(fmaxf(uu[z], -limit), limit);
            o = gg / (1.f + __expf(-alpha * gg)) * (1.f + uc);
          }
          v[2 * e + z] = bf2f(f2bf(o));       // what a bf16 consumer would have seen
        }
      }
    }
  }
  float amax = 0.f;
#pragma unroll
  for (int e = 0; e < 8; ++e) amax = fmaxf(amax, fabsf(v[e]));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
  if (!live) return;
  // smallest power of two s with amax / s <= 448
  int ex = 0;
  if (amax > 0.f) {
    const uint32_t bits = __float_as_uint(__fdiv_rn(amax, 448.f));
    ex = (int)((bits >> 23) & 0xFF) - 127 + ((bits & 0x7FFFFF) ? 1 : 0);
    ex = max(-127, min(127, ex));
  }
  // 2^-ex as a float: exact for ex < 127; ex = 127 would need the subnormal 2^-127, written out below
  const float inv = __uint_as_float((uint32_t)(127 - ex) << 23);
  uint2 q8;
  uint8_t* b = reinterpret_cast<uint8_t*>(&q8);
#pragma unroll
  for (int e = 0; e < 8; ++e) b[e] = f2e4m3(ex == 127 ? v[e] * 5.877471754111438e-39f : v[e] * inv);
  *reinterpret_cast<uint2*>(out + (long long)row_out * ldo + c * 8) = q8;
  if ((threadIdx.x & 3) == 0) sf[(long long)row_out * sf_ld + (c >> 2)] = (uint8_t)(ex + 127);
}

}  // namespace

// x bf16 -> out e4m3 [rows, ldo] + E8M0 exponents sf [rows, sf_ld] (one per 32 values; the caller zero-fills
// the pitch beyond K / 32 once).  mode 0: `rows` rows of x; mode 1: `rows` = P pairs, out row pair_row[p]
// takes x row p / kdiv; mode 2: x is [rows, 2K] (gate | up) and the activation is quantised.
LK_API int lk_quant_mx8(const void* x, long long ldx, int rows, int K, int mode, const int* pair_row, int kdiv,
                        int glu_mode, float alpha, float limit, void* out, long long ldo, void* sf,
                        long long sf_ld, void* stream) {
  if (rows <= 0) return LKH_OK;
  if (!x || !out || !sf || (K & 31) || (ldx & 7) || (ldo & 7) || sf_ld < (K >> 5) || mode < 0 || mode > 2 ||
      (mode == 1 && (!pair_row || kdiv < 1)))
    return LKH_BAD_ARG;
  dim3 grid(((K >> 3) + QT - 1) / QT, rows);
  lkh::launch_pdl(quant_mx8_kernel, grid, dim3(QT), 0, (cudaStream_t)stream, (const __nv_bfloat16*)x, ldx, K, mode,
                  pair_row, kdiv, glu_mode, alpha, limit, (uint8_t*)out, ldo, (uint8_t*)sf, sf_ld);
  lkh::count_launch();
  return lkh::launch_status();
}
