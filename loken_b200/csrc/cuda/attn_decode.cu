// Paged flash-decode attention for GQA over a q8 (or bf16) KV cache, split along the keys.
//
// grid = (kv heads, rows, splits), 4 warps per block.  A row is one query token: a decode step
// of a sequence, or one row of a speculative verify window (row_seq maps rows to block-table
// rows, seq_lens[row] is the number of keys the row may see).
//
// Per 32-key tile a warp runs two phases over the same keys:
//   scores: one key per lane.  The query of each of the G heads that share the kv head is
//           quantised once to int8 with one scale per 32 values (as the reference's decode
//           does), so q.k per 32-block is 8 dp4a, then one fma with d_k * d_q.
//   values: four (hd/32) dims per lane.  The lane streams its 4 code bytes of every key of the
//           tile and accumulates p[g][key] * v for all G heads; p comes from shared memory.
// Running (max, sum, out) per head are merged across the block's warps, and across splits by
// whichever block arrives last on the (row, kv head) counter; that block also adds the
// attention sink (a logit that joins the denominator only, unscaled) and writes bf16, or
// e4m3 with one scale per head when hd = 128, ready for the block-scaled o_proj GEMM.
//
// Counterparts in the reference: cuda/flash_decode_f16.cu (paged GQA decode, split + combine),
// cuda/gptoss_flash_decode.cu (sinks), src/inference/cuda/quantized/flash_splitk.cu (Q8 KV).
#include "common.cuh"
#include "host_common.h"
#include "loken_cuda.h"
#include "tc100.cuh"

using namespace lk;

namespace {

struct DecodeParams {
  const __nv_bfloat16* q;   // [rows, n_q, hd]
  const void* k_cache;
  const void* v_cache;
  const __half* k_scale;
  const __half* v_scale;
  const int* block_table;
  const int* row_seq;       // nullable
  const int* seq_lens;
  const float* sinks;       // nullable, [n_q]
  __nv_bfloat16* out;       // [rows, n_q * hd], nullable when out_fp8
  uint8_t* out_fp8;
  float* out_scales_t;      // [n_q, scale_ld]
  long long scale_ld;
  float* ws;
  int* counters;
  int* status;
  long long num_slots;
  int n_q, n_kv, max_blocks, block_size, window;
  float scale_log2;         // softmax scale * log2(e)
  float* parts_out;         // nullable: emit (weighed values, maximum, sum) per head instead of the attention
};

template <int HD, int G, bool Q8>
__global__ void __launch_bounds__(128)
attn_decode_kernel(const DecodeParams p) {
  constexpr int EPL = HD / 32;
  constexpr int NB = HD / 32;         // 32-value blocks per head
  constexpr float LOG2E = 1.4426950408889634f;
  __shared__ __align__(16) int8_t sq[G][HD];        // quantised queries
  __shared__ float sdq[G][NB];                      // their block scales (pre-multiplied by scale_log2)
  __shared__ __align__(16) float sqf[G][HD];        // float queries for a bf16 cache
  __shared__ __align__(16) float sp[4][32][G];      // probabilities of the current tile, per warp
  __shared__ long long sslot[4][32];
  __shared__ float sm_m[4][G], sm_l[4][G];
  __shared__ float sm_o[4][G][HD];
  __shared__ int s_last;

  const int kvh = blockIdx.x, row = blockIdx.y, split = blockIdx.z, nsplit = gridDim.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int seq = p.row_seq ? p.row_seq[row] : row;
  const int len = p.seq_lens[row];
  const int start = (p.window > 0 && len > p.window) ? len - p.window : 0;
  const int n = len - start;
  int chunk = (n + nsplit - 1) / nsplit;
  chunk = (chunk + 31) & ~31;
  const int r0 = start + split * chunk;
  const int r1 = min(len, r0 + chunk);

  // ---- stage the G queries ----
  for (int g = warp; g < G; g += 4) {
    const __nv_bfloat16* qp = p.q + ((long long)row * p.n_q + kvh * G + g) * HD + lane * EPL;
    float v[EPL];
#pragma unroll
    for (int e = 0; e < EPL; ++e) v[e] = bf2f(qp[e]);
    if constexpr (Q8) {
      float amax = 0.f;
#pragma unroll
      for (int e = 0; e < EPL; ++e) amax = fmaxf(amax, fabsf(v[e]));
      constexpr int LPB = 32 / EPL;
#pragma unroll
      for (int o = LPB / 2; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
      const float d = amax * (1.f / 127.f);
      const float id = d > 0.f ? 1.f / d : 0.f;
#pragma unroll
      for (int e = 0; e < EPL; ++e) sq[g][lane * EPL + e] = (int8_t)__float2int_rn(v[e] * id);
      if ((lane % LPB) == 0) sdq[g][lane / LPB] = d * p.scale_log2;
    } else {
#pragma unroll
      for (int e = 0; e < EPL; ++e) sqf[g][lane * EPL + e] = v[e] * p.scale_log2;
    }
  }
  __syncthreads();

  float m[G], l[G], O[G][EPL];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int e = 0; e < EPL; ++e) O[g][e] = 0.f;
  }

  const int ntiles = r1 > r0 ? (r1 - r0 + 31) / 32 : 0;
  for (int tile = warp; tile < ntiles; tile += 4) {
    const int t = r0 + tile * 32 + lane;
    const bool valid = t < r1;
    long long slot = -1;
    if (valid) {
      const long long blk = p.block_table[(long long)seq * p.max_blocks + t / p.block_size];
      slot = blk * p.block_size + t % p.block_size;
      if (slot < 0 || slot >= p.num_slots) {
        if (p.status) atomicCAS(p.status, 0, LK_ERR_BOUNDS | (2 << 8));
        slot = -1;
      }
    }
    sslot[warp][lane] = slot;
    // ---- scores ----
    float s[G];
#pragma unroll
    for (int g = 0; g < G; ++g) s[g] = 0.f;
    if (slot >= 0) {
      const long long base = (slot * p.n_kv + kvh) * HD;
      if constexpr (Q8) {
        const int4* kc = reinterpret_cast<const int4*>(reinterpret_cast<const int8_t*>(p.k_cache) + base);
        const __half* ks = p.k_scale + (slot * p.n_kv + kvh) * NB;
#pragma unroll
        for (int b = 0; b < NB; ++b) {
          const int4 k0 = kc[2 * b], k1 = kc[2 * b + 1];
          const float dk = __half2float(ks[b]);
#pragma unroll
          for (int g = 0; g < G; ++g) {
            const int4 q0 = *reinterpret_cast<const int4*>(&sq[g][b * 32]);
            const int4 q1 = *reinterpret_cast<const int4*>(&sq[g][b * 32 + 16]);
            int acc = 0;
            acc = __dp4a(k0.x, q0.x, acc); acc = __dp4a(k0.y, q0.y, acc);
            acc = __dp4a(k0.z, q0.z, acc); acc = __dp4a(k0.w, q0.w, acc);
            acc = __dp4a(k1.x, q1.x, acc); acc = __dp4a(k1.y, q1.y, acc);
            acc = __dp4a(k1.z, q1.z, acc); acc = __dp4a(k1.w, q1.w, acc);
            s[g] = fmaf((float)acc, dk * sdq[g][b], s[g]);
          }
        }
      } else {
        const uint4* kc = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(p.k_cache) + base);
#pragma unroll 4
        for (int c = 0; c < HD / 8; ++c) {
          const uint4 kv = kc[c];
          const __nv_bfloat162* k2 = reinterpret_cast<const __nv_bfloat162*>(&kv);
          float kf[8];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 f = __bfloat1622float2(k2[e]);
            kf[2 * e] = f.x;
            kf[2 * e + 1] = f.y;
          }
#pragma unroll
          for (int g = 0; g < G; ++g) {
            const float4 a = *reinterpret_cast<const float4*>(&sqf[g][c * 8]);
            const float4 b = *reinterpret_cast<const float4*>(&sqf[g][c * 8 + 4]);
            s[g] += kf[0] * a.x + kf[1] * a.y + kf[2] * a.z + kf[3] * a.w + kf[4] * b.x + kf[5] * b.y +
                    kf[6] * b.z + kf[7] * b.w;
          }
        }
      }
    }
    // ---- online softmax (per head, across the tile's 32 keys) ----
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const float sv = slot >= 0 ? s[g] : -INFINITY;
      const float tmax = warp_max(sv);
      const float mn = fmaxf(m[g], tmax);
      const float pv = (slot >= 0 && mn > -INFINITY) ? exp2f(sv - mn) : 0.f;
      const float ps = warp_sum(pv);
      const float alpha = (mn > -INFINITY) ? exp2f(m[g] - mn) : 1.f;
      l[g] = l[g] * alpha + ps;
      m[g] = mn;
      sp[warp][lane][g] = pv;
#pragma unroll
      for (int e = 0; e < EPL; ++e) O[g][e] *= alpha;
    }
    __syncwarp();
    // ---- values ----
    const int cnt = min(32, r1 - (r0 + tile * 32));
#pragma unroll 4
    for (int j = 0; j < cnt; ++j) {
      const long long sj = sslot[warp][j];
      if (sj < 0) continue;
      float vf[EPL];
      const long long base = (sj * p.n_kv + kvh) * HD + lane * EPL;
      if constexpr (Q8) {
        const float dv = __half2float(p.v_scale[(sj * p.n_kv + kvh) * NB + (lane * EPL) / 32]);
        if constexpr (EPL == 4) {
          const char4 c = *reinterpret_cast<const char4*>(reinterpret_cast<const int8_t*>(p.v_cache) + base);
          vf[0] = c.x * dv; vf[1] = c.y * dv; vf[2] = c.z * dv; vf[3] = c.w * dv;
        } else {
          const int8_t* c = reinterpret_cast<const int8_t*>(p.v_cache) + base;
#pragma unroll
          for (int e = 0; e < EPL; ++e) vf[e] = c[e] * dv;
        }
      } else {
        const __nv_bfloat16* c = reinterpret_cast<const __nv_bfloat16*>(p.v_cache) + base;
#pragma unroll
        for (int e = 0; e < EPL; ++e) vf[e] = bf2f(c[e]);
      }
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const float pj = sp[warp][j][g];
#pragma unroll
        for (int e = 0; e < EPL; ++e) O[g][e] = fmaf(pj, vf[e], O[g][e]);
      }
    }
    __syncwarp();
  }

  // ---- merge the block's four warps ----
#pragma unroll
  for (int g = 0; g < G; ++g) {
    if (lane == 0) {
      sm_m[warp][g] = m[g];
      sm_l[warp][g] = l[g];
    }
#pragma unroll
    for (int e = 0; e < EPL; ++e) sm_o[warp][g][lane * EPL + e] = O[g][e];
  }
  __syncthreads();

  // thread d (< HD) finishes dim d of every head
  const int d = threadIdx.x;
  const int row_kv = row * p.n_kv + kvh;
  float fm[G], fl[G], fo[G];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    float mm = fmaxf(fmaxf(sm_m[0][g], sm_m[1][g]), fmaxf(sm_m[2][g], sm_m[3][g]));
    float ll = 0.f, oo = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float a = (sm_m[w][g] > -INFINITY) ? exp2f(sm_m[w][g] - mm) : 0.f;
      ll += sm_l[w][g] * a;
      if (d < HD) oo += sm_o[w][g][d < HD ? d : 0] * a;
    }
    fm[g] = mm; fl[g] = ll; fo[g] = oo;
  }

  if (nsplit > 1) {
    float* mine = p.ws + ((long long)row_kv * nsplit + split) * (G * (HD + 2));
#pragma unroll
    for (int g = 0; g < G; ++g) {
      if (d < HD) mine[g * (HD + 2) + d] = fo[g];
      if (d == 0) {
        mine[g * (HD + 2) + HD] = fm[g];
        mine[g * (HD + 2) + HD + 1] = fl[g];
      }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence();     // the barrier carried every thread's partial into this fence
      const int prev = atomicAdd(&p.counters[row_kv], 1);
      s_last = (prev == nsplit - 1);
      if (s_last) p.counters[row_kv] = 0;
      __threadfence();
    }
    __syncthreads();
    if (!s_last) return;
    const float* all = p.ws + (long long)row_kv * nsplit * (G * (HD + 2));
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float mm = -INFINITY;
      for (int s = 0; s < nsplit; ++s) mm = fmaxf(mm, __ldcg(&all[(s * G + g) * (HD + 2) + HD]));
      float ll = 0.f, oo = 0.f;
      for (int s = 0; s < nsplit; ++s) {
        const float ms = __ldcg(&all[(s * G + g) * (HD + 2) + HD]);
        const float a = (ms > -INFINITY) ? exp2f(ms - mm) : 0.f;
        ll += __ldcg(&all[(s * G + g) * (HD + 2) + HD + 1]) * a;
        if (d < HD) oo += __ldcg(&all[(s * G + g) * (HD + 2) + (d < HD ? d : 0)]) * a;
      }
      fm[g] = mm; fl[g] = ll; fo[g] = oo;
    }
  }

  if (p.parts_out) {
    // one range of a context held on several GPUs: hand out the part, the caller merges the ranges
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float* dst = p.parts_out + ((long long)row * p.n_q + kvh * G + g) * (HD + 2);
      if (d < HD) dst[d] = fo[g];
      if (d == 0) {
        dst[HD] = fm[g];
        dst[HD + 1] = fl[g];
      }
    }
    return;
  }

  // ---- sink, normalise, write ----
  __shared__ float red[32];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    const int head = kvh * G + g;
    float mm = fm[g], ll = fl[g], oo = fo[g];
    if (p.sinks) {
      const float sk = p.sinks[head] * LOG2E;
      const float mn = fmaxf(mm, sk);
      const float a = (mm > -INFINITY) ? exp2f(mm - mn) : 0.f;
      ll = ll * a + exp2f(sk - mn);
      oo *= a;
    }
    const float val = ll > 0.f ? oo / ll : 0.f;
    if (p.out && d < HD) p.out[(long long)row * p.n_q * HD + head * HD + d] = f2bf(val);
    if (p.out_fp8) {
      // hd == 128: the head is exactly one 128-group of the o_proj input
      const float r = bf2f(f2bf(d < HD ? val : 0.f));
      const float amax = block_max(fabsf(r), red);
      const float sc = e4m3_group_scale(amax);
      if (d < HD) p.out_fp8[(long long)row * p.n_q * HD + head * HD + d] = f2e4m3(r / sc);
      if (d == 0) p.out_scales_t[(long long)head * p.scale_ld + row] = sc;
    }
  }
}

template <int HD, bool Q8>
int launch_g(const DecodeParams& p, int G, dim3 grid, cudaStream_t st) {
  switch (G) {
    case 1: attn_decode_kernel<HD, 1, Q8><<<grid, 128, 0, st>>>(p); break;
    case 2: attn_decode_kernel<HD, 2, Q8><<<grid, 128, 0, st>>>(p); break;
    case 4: attn_decode_kernel<HD, 4, Q8><<<grid, 128, 0, st>>>(p); break;
    case 8: attn_decode_kernel<HD, 8, Q8><<<grid, 128, 0, st>>>(p); break;
    // groups that are not a power of two (Llama-3.2-3B: 3, Qwen2.5-14B / 32B: 5, Qwen2.5-7B: 7) run here;
    // the tensor-core decode kernels are built for 1, 2, 4 and 8
    case 3: attn_decode_kernel<HD, 3, Q8><<<grid, 128, 0, st>>>(p); break;
    case 5: attn_decode_kernel<HD, 5, Q8><<<grid, 128, 0, st>>>(p); break;
    case 6: attn_decode_kernel<HD, 6, Q8><<<grid, 128, 0, st>>>(p); break;
    case 7: attn_decode_kernel<HD, 7, Q8><<<grid, 128, 0, st>>>(p); break;
    default: return LKH_BAD_ARG;
  }
  lkh::count_launch();
  return lkh::launch_status();
}

}  // namespace

LK_API long long lk_attn_decode_ws_floats(int rows, int n_q, int n_kv, int hd, int nsplit) {
  const int G = n_q / n_kv;
  return (long long)rows * n_kv * nsplit * G * (hd + 2);
}

LK_API int lk_attn_decode(const LkDecodeArgs* a, void* stream) {
  if (a->rows <= 0) return LKH_OK;
  if (a->n_kv <= 0 || a->n_q % a->n_kv) return LKH_BAD_ARG;
  const int G = a->n_q / a->n_kv;
  const int nsplit = a->nsplit < 1 ? 1 : a->nsplit;
  if (nsplit > 1) {
    if (!a->ws || !a->counters) return LKH_BAD_ARG;
    if (lk_attn_decode_ws_floats(a->rows, a->n_q, a->n_kv, a->hd, nsplit) > a->ws_floats ||
        (long long)a->rows * a->n_kv > a->n_counters)
      return LKH_TOO_LARGE;
  }
  if (a->out_fp8 && (a->hd != 128 || !a->out_scales_t)) return LKH_BAD_ARG;
  DecodeParams p;
  p.q = (const __nv_bfloat16*)a->q;
  p.k_cache = a->k_cache; p.v_cache = a->v_cache;
  p.k_scale = (const __half*)a->k_scale; p.v_scale = (const __half*)a->v_scale;
  p.block_table = a->block_table; p.row_seq = a->row_seq; p.seq_lens = a->seq_lens;
  p.sinks = a->sinks;
  p.out = (__nv_bfloat16*)a->out; p.out_fp8 = (uint8_t*)a->out_fp8;
  p.out_scales_t = a->out_scales_t; p.scale_ld = a->scale_ld;
  p.ws = a->ws; p.counters = a->counters; p.status = a->status;
  p.num_slots = a->num_slots;
  p.n_q = a->n_q; p.n_kv = a->n_kv; p.max_blocks = a->max_blocks; p.block_size = a->block_size;
  p.window = a->window;
  p.scale_log2 = a->scale * 1.4426950408889634f;
  p.parts_out = a->parts_out;
  dim3 grid(a->n_kv, a->rows, nsplit);
  cudaStream_t st = (cudaStream_t)stream;
  if (a->hd == 128) return a->kv_q8 ? launch_g<128, true>(p, G, grid, st) : launch_g<128, false>(p, G, grid, st);
  if (a->hd == 64) return a->kv_q8 ? launch_g<64, true>(p, G, grid, st) : launch_g<64, false>(p, G, grid, st);
  return LKH_BAD_ARG;
}
