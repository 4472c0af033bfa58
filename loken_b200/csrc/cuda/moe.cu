// Mixture-of-experts routing and data movement around the grouped expert GEMM:
//
//   lk_moe_route    router logits -> top-k expert ids and weights, one warp per token
//                   (softmax over the chosen logits as gpt-oss does, full softmax with optional
//                   renormalisation, or sigmoid scores with optional renormalisation)
//   lk_moe_plan     (token, choice) pairs -> per-expert row ranges of the sorted token buffer,
//                   the row each pair lands in, and the list of N tiles the grouped GEMM walks;
//                   pairs whose expert lives on another rank are marked -1 (expert parallel)
//   lk_moe_permute  token rows -> sorted rows
//   lk_moe_combine  sorted expert outputs -> token rows, weighted, summed in choice order in fp32
//
// Counterparts in the reference: cuda/moe/gate_topk.cu (router + top-k + sort), moe_utils.cuh
// (histogram + offsets), moe_mmq.cu (plan / fold in slot order), loken_moe_sum_topk.
#include "common.cuh"
#include "host_common.h"
#include "loken_cuda.h"
#include "tc100.cuh"

using namespace lk;

namespace {

constexpr int MAX_E = 256;
constexpr int MAX_K = 8;

// One warp: scores of E experts (v[j] = score of expert j * 32 + lane, -inf past E) -> the k best ids and
// their weights.  mode 0: softmax over the chosen logits; 1: full softmax first (renorm optional);
// 2: sigmoid scores (renorm optional).  Ties go to the lowest expert id.
__device__ __forceinline__ void route_warp(float (&v)[MAX_E / 32], int lane, int E, int k, int mode, int renorm,
                                           int* __restrict__ ids, float* __restrict__ wts) {
  constexpr int PER = MAX_E / 32;
  if (mode == 1) {            // full softmax first
    float mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < PER; ++j) mx = fmaxf(mx, v[j]);
    mx = warp_max(mx);
    float z = 0.f;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      v[j] = (j * 32 + lane < E) ? __expf(v[j] - mx) : -INFINITY;
      z += (j * 32 + lane < E) ? v[j] : 0.f;
    }
    z = warp_sum(z);
#pragma unroll
    for (int j = 0; j < PER; ++j)
      if (j * 32 + lane < E) v[j] /= z;
  } else if (mode == 2) {     // sigmoid scores
#pragma unroll
    for (int j = 0; j < PER; ++j)
      if (j * 32 + lane < E) v[j] = 1.f / (1.f + __expf(-v[j]));
  }
  float cv[MAX_K];
  int ci[MAX_K];
  for (int r = 0; r < k; ++r) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const int e = j * 32 + lane;
      if (v[j] > bv) {        // strictly greater: lowest index wins inside a lane
        bv = v[j];
        bi = e;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) {
        bv = ov;
        bi = oi;
      }
    }
    cv[r] = bv;
    ci[r] = bi;
#pragma unroll
    for (int j = 0; j < PER; ++j)
      if (j * 32 + lane == bi) v[j] = -INFINITY;
  }
  float wsum = 0.f;
  const float cm = cv[0];
  if (mode == 0) {
    for (int r = 0; r < k; ++r) {
      cv[r] = __expf(cv[r] - cm);
      wsum += cv[r];
    }
    for (int r = 0; r < k; ++r) cv[r] /= wsum;
  } else if (renorm) {
    for (int r = 0; r < k; ++r) wsum += cv[r];
    wsum = fmaxf(wsum, 6.1035156e-5f);
    for (int r = 0; r < k; ++r) cv[r] /= wsum;
  }
  if (lane == 0) {
    for (int r = 0; r < k; ++r) {
      ids[r] = ci[r] < E ? ci[r] : 0;
      wts[r] = cv[r];
    }
  }
}

__global__ void __launch_bounds__(128)
moe_route_kernel(const float* __restrict__ logits, long long ld, int T, int E, int k, int mode, int renorm,
                 int* __restrict__ ids, float* __restrict__ wts) {
  const int t = blockIdx.x * 4 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (t >= T) return;
  constexpr int PER = MAX_E / 32;
  float v[PER];
  const float* x = logits + (long long)t * ld;
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int e = j * 32 + lane;
    v[j] = e < E ? x[e] : -INFINITY;
  }
  route_warp(v, lane, E, k, mode, renorm, ids + (long long)t * k, wts + (long long)t * k);
}

// Router in one launch: logits = W_r h + b_r for one token per CTA (each warp walks a quarter of the
// experts, its lanes striding over the hidden row with 16-byte loads of the bf16 router matrix, which
// stays in L2), then the top-k of `route_warp`.  For the decode-size steps of a mixture layer this
// replaces a GEMM launch whose single output tile cannot occupy the chip, plus the routing launch.
constexpr int RT_WARPS = 8;
constexpr int RT_EG = 4;       // experts a warp works on at once: four independent load streams per lane
// TT tokens per CTA share every load of the router matrix (L2 traffic and time per token fall with TT;
// the number of CTAs falls too, so small steps use TT = 1).
template <int TT>
__global__ void __launch_bounds__(RT_WARPS * 32)
moe_router_kernel(const __nv_bfloat16* __restrict__ h, long long ldh, const __nv_bfloat16* __restrict__ w,
                  const float* __restrict__ bias, int T, int H, int E, int k, int mode, int renorm,
                  int* __restrict__ ids, float* __restrict__ wts, float* __restrict__ logits_out, long long ldl) {
  pdl_wait();
  pdl_launch();
  extern __shared__ __align__(16) uint8_t rt_smem[];
  const size_t row_bytes = ((size_t)H * 2 + 15) & ~size_t(15);
  float* sc = reinterpret_cast<float*>(rt_smem + TT * row_bytes);           // [TT][MAX_E]
  const int t0 = blockIdx.x * TT;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nchunk = H >> 3;
#pragma unroll
  for (int tt = 0; tt < TT; ++tt) {
    uint4* hs = reinterpret_cast<uint4*>(rt_smem + tt * row_bytes);
    const int t = min(t0 + tt, T - 1);
    for (int c = threadIdx.x; c < nchunk; c += RT_WARPS * 32)
      hs[c] = *reinterpret_cast<const uint4*>(h + (long long)t * ldh + c * 8);
  }
  __syncthreads();
  for (int e0 = warp * RT_EG; e0 < E; e0 += RT_WARPS * RT_EG) {
    float acc[RT_EG][TT];
#pragma unroll
    for (int g = 0; g < RT_EG; ++g)
#pragma unroll
      for (int tt = 0; tt < TT; ++tt) acc[g][tt] = 0.f;
    const uint4* wr[RT_EG];
#pragma unroll
    for (int g = 0; g < RT_EG; ++g) wr[g] = reinterpret_cast<const uint4*>(w + (long long)min(e0 + g, E - 1) * H);
#pragma unroll 2
    for (int c = lane; c < nchunk; c += 32) {
      uint4 a[RT_EG];
#pragma unroll
      for (int g = 0; g < RT_EG; ++g) a[g] = __ldg(wr[g] + c);
#pragma unroll
      for (int tt = 0; tt < TT; ++tt) {
        const uint4 b = reinterpret_cast<const uint4*>(rt_smem + tt * row_bytes)[c];
        const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&b);
        float2 y[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) y[q] = __bfloat1622float2(b2[q]);
#pragma unroll
        for (int g = 0; g < RT_EG; ++g) {
          const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&a[g]);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const float2 x = __bfloat1622float2(a2[q]);
            acc[g][tt] = fmaf(x.x, y[q].x, acc[g][tt]);
            acc[g][tt] = fmaf(x.y, y[q].y, acc[g][tt]);
          }
        }
      }
    }
#pragma unroll
    for (int g = 0; g < RT_EG; ++g)
#pragma unroll
      for (int tt = 0; tt < TT; ++tt) {
        const float v = warp_sum(acc[g][tt]);
        if (lane == 0 && e0 + g < E) sc[tt * MAX_E + e0 + g] = v + (bias ? bias[e0 + g] : 0.f);
      }
  }
  __syncthreads();
  if (logits_out)
    for (int i = threadIdx.x; i < TT * E; i += RT_WARPS * 32) {
      const int tt = i / E, e = i % E;
      if (t0 + tt < T) logits_out[(long long)(t0 + tt) * ldl + e] = sc[tt * MAX_E + e];
    }
  if (warp < TT && t0 + warp < T) {
    constexpr int PER = MAX_E / 32;
    float v[PER];
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const int e = j * 32 + lane;
      v[j] = e < E ? sc[warp * MAX_E + e] : -INFINITY;
    }
    route_warp(v, lane, E, k, mode, renorm, ids + (long long)(t0 + warp) * k, wts + (long long)(t0 + warp) * k);
  }
}

__global__ void __launch_bounds__(1024)
moe_plan_kernel(const int* __restrict__ ids, int P, int E_total, int e_lo, int e_cnt, int BN, int max_tiles,
                int* __restrict__ offsets, int* __restrict__ pair_row, int* __restrict__ tile_expert,
                int* __restrict__ tile_row0, int* __restrict__ tile_rows, int* __restrict__ ntiles,
                int* __restrict__ status) {
  __shared__ int cnt[MAX_E], cur[MAX_E], off[MAX_E + 1], tbase[MAX_E + 1];
  for (int e = threadIdx.x; e < MAX_E; e += blockDim.x) {
    cnt[e] = 0;
    cur[e] = 0;
  }
  __syncthreads();
  for (int p = threadIdx.x; p < P; p += blockDim.x) {
    const int id = ids[p];
    if (id == -1) continue;        // an empty slot (expert-parallel receive buffer): no pair
    if (id < 0 || id >= E_total) {
      if (status) atomicCAS(status, 0, LK_ERR_BOUNDS | (5 << 8));
      continue;
    }
    const int le = id - e_lo;
    if (le >= 0 && le < e_cnt) atomicAdd(&cnt[le], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int o = 0, tb = 0;
    for (int e = 0; e < e_cnt; ++e) {
      off[e] = o;
      tbase[e] = tb;
      o += cnt[e];
      tb += (cnt[e] + BN - 1) / BN;
    }
    off[e_cnt] = o;
    tbase[e_cnt] = tb;
    if (tb > max_tiles) {
      if (status) atomicCAS(status, 0, LK_ERR_SIZE | (5 << 8));
      tb = max_tiles;
    }
    *ntiles = tb;
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= e_cnt; e += blockDim.x) offsets[e] = off[e];
  for (int p = threadIdx.x; p < P; p += blockDim.x) {
    const int id = ids[p];
    const int le = id - e_lo;
    int row = -1;
    if (id >= 0 && id < E_total && le >= 0 && le < e_cnt) row = off[le] + atomicAdd(&cur[le], 1);
    pair_row[p] = row;
  }
  for (int e = threadIdx.x; e < e_cnt; e += blockDim.x) {
    const int nt = (cnt[e] + BN - 1) / BN;
    for (int i = 0; i < nt; ++i) {
      const int t = tbase[e] + i;
      if (t >= max_tiles) break;
      tile_expert[t] = e;
      tile_row0[t] = off[e] + i * BN;
      tile_rows[t] = min(BN, cnt[e] - i * BN);
    }
  }
}

__global__ void moe_permute_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, const int* __restrict__ pair_row,
                                   int k, int H, __nv_bfloat16* __restrict__ xs, long long lds) {
  const int p = blockIdx.x;
  const int row = pair_row[p];
  if (row < 0) return;
  const uint4* src = reinterpret_cast<const uint4*>(x + (long long)(p / k) * ldx);
  uint4* dst = reinterpret_cast<uint4*>(xs + (long long)row * lds);
  for (int c = threadIdx.x; c < H / 8; c += blockDim.x) dst[c] = src[c];
}

__global__ void moe_combine_kernel(const __nv_bfloat16* __restrict__ y, long long ldy, const int* __restrict__ pair_row,
                                   const float* __restrict__ wts, int k, int H, __nv_bfloat16* __restrict__ out,
                                   long long ldo, int accumulate) {
  const int t = blockIdx.x;
  for (int c = threadIdx.x; c < H / 8; c += blockDim.x) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (accumulate) {
      const uint4 q = *reinterpret_cast<const uint4*>(out + (long long)t * ldo + c * 8);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(h[e]);
        acc[2 * e] = f.x;
        acc[2 * e + 1] = f.y;
      }
    }
    for (int j = 0; j < k; ++j) {
      const int row = pair_row[(long long)t * k + j];
      if (row < 0) continue;
      const float w = wts[(long long)t * k + j];
      const uint4 q = *reinterpret_cast<const uint4*>(y + (long long)row * ldy + c * 8);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(h[e]);
        acc[2 * e] = fmaf(w, f.x, acc[2 * e]);
        acc[2 * e + 1] = fmaf(w, f.y, acc[2 * e + 1]);
      }
    }
    uint4 o;
    __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int e = 0; e < 4; ++e) oh[e] = __floats2bfloat162_rn(acc[2 * e], acc[2 * e + 1]);
    *reinterpret_cast<uint4*>(out + (long long)t * ldo + c * 8) = o;
  }
}

}  // namespace

LK_API int lk_moe_route(const float* logits, long long ld, int T, int E, int k, int mode, int renorm, int* ids,
                        float* wts, void* stream) {
  if (T <= 0) return LKH_OK;
  if (E > MAX_E || k > MAX_K || k > E || k < 1) return LKH_BAD_ARG;
  moe_route_kernel<<<(T + 3) / 4, 128, 0, (cudaStream_t)stream>>>(logits, ld, T, E, k, mode, renorm, ids, wts);
  lkh::count_launch();
  return lkh::launch_status();
}

// h bf16 [T, ldh], w bf16 [E, H] (router matrix), bias f32 [E] or null -> ids / wts [T, k]; logits_out optional.
LK_API int lk_moe_router(const void* h, long long ldh, const void* w, const float* bias, int T, int H, int E, int k,
                         int mode, int renorm, int* ids, float* wts, float* logits_out, long long ldl, void* stream) {
  if (T <= 0) return LKH_OK;
  if (E > MAX_E || k > MAX_K || k > E || k < 1 || (H & 7) || (ldh & 7)) return LKH_BAD_ARG;
  const size_t row = ((size_t)H * 2 + 15) & ~size_t(15);
  // tokens per CTA: more of them share each load of the router matrix, fewer CTAs result
  int tt = T <= 32 ? 1 : T <= 256 ? 2 : 4;
  while (tt > 1 && tt * (row + MAX_E * sizeof(float)) > 48 * 1024) tt >>= 1;
  const size_t smem = tt * (row + MAX_E * sizeof(float));
  if (smem > 48 * 1024) return LKH_TOO_LARGE;
  const dim3 grid((T + tt - 1) / tt), block(RT_WARPS * 32);
#define LK_ROUTER(TT)                                                                                              \
  lkh::launch_pdl(moe_router_kernel<TT>, grid, block, smem, (cudaStream_t)stream, (const __nv_bfloat16*)h, ldh,    \
                  (const __nv_bfloat16*)w, bias, T, H, E, k, mode, renorm, ids, wts, logits_out, ldl)
  if (tt == 4) LK_ROUTER(4);
  else if (tt == 2) LK_ROUTER(2);
  else LK_ROUTER(1);
#undef LK_ROUTER
  lkh::count_launch();
  return lkh::launch_status();
}

LK_API int lk_moe_plan(const int* ids, int P, int E_total, int e_lo, int e_cnt, int BN, int max_tiles, int* offsets,
                       int* pair_row, int* tile_expert, int* tile_row0, int* tile_rows, int* ntiles, int* status,
                       void* stream) {
  if (P <= 0) return LKH_OK;
  if (e_cnt > MAX_E || e_cnt < 1 || BN < 1) return LKH_BAD_ARG;
  moe_plan_kernel<<<1, 1024, 0, (cudaStream_t)stream>>>(ids, P, E_total, e_lo, e_cnt, BN, max_tiles, offsets, pair_row,
                                                        tile_expert, tile_row0, tile_rows, ntiles, status);
  lkh::count_launch();
  return lkh::launch_status();
}

LK_API int lk_moe_permute(const void* x, long long ldx, const int* pair_row, int P, int k, int H, void* xs,
                          long long lds, void* stream) {
  if (P <= 0) return LKH_OK;
  if (H % 8) return LKH_BAD_ARG;
  moe_permute_kernel<<<P, 128, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, ldx, pair_row, k, H,
                                                         (__nv_bfloat16*)xs, lds);
  lkh::count_launch();
  return lkh::launch_status();
}

LK_API int lk_moe_combine(const void* y, long long ldy, const int* pair_row, const float* wts, int T, int k, int H,
                          void* out, long long ldo, int accumulate, void* stream) {
  if (T <= 0) return LKH_OK;
  if (H % 8) return LKH_BAD_ARG;
  moe_combine_kernel<<<T, 128, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)y, ldy, pair_row, wts, k, H,
                                                         (__nv_bfloat16*)out, ldo, accumulate);
  lkh::count_launch();
  return lkh::launch_status();
}
